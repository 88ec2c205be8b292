"""Re-entrancy: two Python threads, each on its own CUDA stream, call the library at the same time."""
import threading

import pytest
import torch

from oracle import chains

pytestmark = pytest.mark.gpu


def test_two_threads_two_streams_give_the_serial_results():
    from proteusai_b200.utils.model_utils.attn.geometric_attn import geoattn_forward
    from proteusai_b200.utils.model_utils.wf_embedding.isotropic.cuda.wf_embedding import we_forward_rows
    c, m = chains.chain_batch([900, 640], 900, seed=31)
    c, m = torch.from_numpy(c).cuda(), torch.from_numpy(m).cuda()
    wn = torch.from_numpy(chains.wavenumbers(128)).cuda()
    g = torch.Generator().manual_seed(5)
    q, k, v = (torch.randn(2, 4, 900, 64, generator=g).to(torch.bfloat16).cuda() for _ in range(3))
    sig = torch.from_numpy(chains.sigmas(4)).cuda()
    try:
        ref_we = we_forward_rows(c, wn, 1, m)[0].clone()
        ref_o = geoattn_forward(q, k, v, c, sig, m)[0].clone()
        torch.cuda.synchronize()
        results, errors = {}, []

        def worker(name):
            try:
                stream = torch.cuda.Stream()
                with torch.cuda.stream(stream):
                    for _ in range(5):
                        we = we_forward_rows(c, wn, 1, m)[0]
                        o = geoattn_forward(q, k, v, c, sig, m)[0]
                stream.synchronize()
                results[name] = (we, o)
            except Exception as exc:  # noqa: BLE001
                errors.append(exc)

        threads = [threading.Thread(target=worker, args=(i,)) for i in range(2)]
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        assert not errors, errors
        for we, o in results.values():
            # the embedding's partial sums are added in arrival order: equal to rounding; the attention forward is deterministic
            assert float(torch.norm(we - ref_we) / torch.norm(ref_we)) < 1e-5
            assert torch.equal(o, ref_o)
    finally:
        pass
    from proteusai_b200 import _lib
    _lib.device_status()
