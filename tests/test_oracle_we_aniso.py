"""The anisotropic WE oracle against the reference's own function (golden vectors)."""
import os

import numpy as np
import torch

from oracle.we_aniso_ref import grads_from_partials, wf_embedding_aniso_ref
from oracle.we_ref import rel_l2

KEYS = ("coords_a", "coords_b", "cb", "wn", "mask", "d_out", "out", "d_cb", "d_wn")


def _cases(golden_dir):
    g = np.load(os.path.join(golden_dir, "we_aniso_reference.npz"))
    for name in sorted({k.split(".")[0] for k in g.files}):
        yield name, {x: torch.from_numpy(np.asarray(g[f"{name}.{x}"])) for x in KEYS}


def test_golden_bit_exact_and_partials(golden_dir):
    torch.set_num_threads(1)
    n = 0
    for name, t in _cases(golden_dir):
        out, d_cb, d_k = wf_embedding_aniso_ref(t["coords_a"], t["coords_b"], t["cb"], t["wn"], t["mask"], partials=True, chunk=80)
        assert torch.equal(out, t["out"]), name
        g_cb, g_k = grads_from_partials(t["d_out"], d_cb, d_k)  # the O(N) backward against autograd through the reference
        assert rel_l2(t["d_cb"], g_cb) < 1e-5 and rel_l2(t["d_wn"], g_k) < 1e-5, name
        part = wf_embedding_aniso_ref(t["coords_a"], t["coords_b"], t["cb"], t["wn"], t["mask"], rows=(9, 50), chunk=16)
        assert torch.allclose(part, out[:, 9:50], rtol=1e-5, atol=1e-6)
        n += 1
    assert n == 2


def test_zero_cb_magnitude_reduces_to_isotropic():
    from oracle import chains
    from oracle.we_ref import wf_embedding_ref
    c, m = chains.chain_batch([60, 33], 60, seed=2)
    c, m = torch.from_numpy(c), torch.from_numpy(m)
    b = torch.nn.functional.normalize(torch.randn(2, 60, 3, generator=torch.Generator().manual_seed(1)), dim=2)
    wn = torch.from_numpy(chains.wavenumbers(16))
    aniso = wf_embedding_aniso_ref(c, b, torch.zeros(8), wn, m)
    assert rel_l2(wf_embedding_ref(c, wn, 1, m), aniso) < 1e-6
