"""What a kernel does when a bounded device-side wait runs out, exercised without faulting or hanging anything:
a test-only kernel waits, with a limit of a few thousand cycles, on an mbarrier nobody arrives on."""
import pytest
import torch

from oracle import chains
from oracle.we_ref import rel_l2, wf_embedding_ref

pytestmark = pytest.mark.gpu


def test_expired_wait_sets_the_status_word_and_the_device_stays_usable():
    from proteusai_b200 import _lib
    from proteusai_b200.utils.model_utils.wf_embedding.isotropic.cuda.wf_embedding import we_forward_rows
    lib = _lib.lib()
    assert torch.cuda.is_available()
    assert lib.pai_device_status(_lib.current_stream()) == 0
    _lib.check(lib.pai_selftest_wait_timeout(_lib.current_stream()), "pai_selftest_wait_timeout")
    assert lib.pai_device_status(_lib.current_stream()) == -8      # PAI_ERR_DEVICE_WAIT_TIMEOUT, reported once ...
    assert lib.pai_device_status(_lib.current_stream()) == 0       # ... and cleared by the read
    with pytest.raises(RuntimeError, match="bounded device-side wait"):
        _lib.check(lib.pai_selftest_wait_timeout(_lib.current_stream()), "launch")
        _lib.device_status()
    # the context is intact: an ordinary call gives the right answer afterwards
    c, m = chains.chain_batch([200], 200, seed=3)
    wn = torch.from_numpy(chains.wavenumbers(64))
    out, _, _ = we_forward_rows(torch.from_numpy(c).cuda(), wn.cuda(), 1, None)
    assert rel_l2(wf_embedding_ref(torch.from_numpy(c), wn, 1, dtype=torch.float64), out.cpu()) < 1e-4
    _lib.device_status()
