"""Parity of the CUDA anisotropic Wavefunction Embedding with the reference's function (golden vectors) and the oracle."""
import os

import numpy as np
import pytest
import torch

from oracle import chains
from oracle.we_aniso_ref import grads_from_partials, wf_embedding_aniso_ref
from oracle.we_ref import rel_l2

pytestmark = pytest.mark.gpu
OUT_TOL, GRAD_TOL = 1e-4, 1e-3
KEYS = ("coords_a", "coords_b", "cb", "wn", "mask", "d_out", "out", "d_cb", "d_wn")


@pytest.fixture(scope="module")
def mod():
    from proteusai_b200 import _lib
    from proteusai_b200.utils.model_utils.wf_embedding.anisotropic.cb_scaling.learnable_wavenumbers.cuda import wf_embedding as m
    _lib.lib()
    return m


def test_golden_forward_and_gradients(mod, golden_dir):
    g = np.load(os.path.join(golden_dir, "we_aniso_reference.npz"))
    for name in sorted({k.split(".")[0] for k in g.files}):
        t = {x: torch.from_numpy(np.asarray(g[f"{name}.{x}"])) for x in KEYS}
        cb, wn = t["cb"].cuda().requires_grad_(True), t["wn"].cuda().requires_grad_(True)
        out = mod.wf_embedding(t["coords_a"].cuda(), t["coords_b"].cuda(), cb, wn, t["mask"].cuda())
        assert rel_l2(t["out"], out.detach().cpu()) < OUT_TOL, name
        out.backward(t["d_out"].cuda())
        assert rel_l2(t["d_cb"], cb.grad.cpu()) < GRAD_TOL and rel_l2(t["d_wn"], wn.grad.cpu()) < GRAD_TOL, name
        assert torch.all(out.detach().cpu()[t["mask"]] == 0)


@pytest.mark.parametrize("z,n,k,lengths", [(2, 1024, 128, [1024, 700]), (1, 333, 5, [333]), (3, 65, 40, [65, 1, 30]), (1, 2048, 64, [2048])])
def test_against_oracle(mod, z, n, k, lengths):
    c, m = chains.chain_batch(lengths, n, seed=n + k)
    c, m = torch.from_numpy(c), torch.from_numpy(m)
    g = torch.Generator().manual_seed(k)
    b = torch.nn.functional.normalize(torch.randn(z, n, 3, generator=g), dim=2)
    cb = torch.rand(k, generator=g) * 2
    wn = torch.from_numpy(chains.wavenumbers(2 * k))
    out, d_cb, d_k = mod.we_aniso_forward_rows(c.cuda(), b.cuda(), cb.cuda(), wn.cuda(), m.cuda())
    rows = (0, min(n, 96))
    r_out, r_cb, r_k = wf_embedding_aniso_ref(c, b, cb, wn, m, rows=rows, partials=True, dtype=torch.float64, chunk=32)
    assert rel_l2(r_out, out[:, rows[0]:rows[1]].cpu()) < OUT_TOL
    assert rel_l2(r_cb, d_cb[:, rows[0]:rows[1]].cpu()) < GRAD_TOL and rel_l2(r_k, d_k[:, rows[0]:rows[1]].cpu()) < GRAD_TOL
    d_out = torch.randn(out.shape, generator=g)
    g_cb, g_k = mod.we_aniso_backward(d_out.cuda(), d_cb, d_k)
    e_cb, e_k = grads_from_partials(d_out.double(), d_cb.cpu().double(), d_k.cpu().double())
    assert rel_l2(e_cb, g_cb.cpu()) < 1e-5 and rel_l2(e_k, g_k.cpu()) < 1e-5
    from proteusai_b200 import _lib
    _lib.device_status()


def test_module_anisotropic_branch(mod):
    from proteusai_b200.utils.model_utils.wf_embedding.wf_embedding import WaveFunctionEmbedding
    m = WaveFunctionEmbedding(d_wf=32, anisotropic=True, learn_wl=True, learn_aa=True).cuda()
    c, mask = chains.chain_batch([90, 50], 90, seed=4)
    c, mask = torch.from_numpy(c), torch.from_numpy(mask)
    b = torch.nn.functional.normalize(torch.randn(2, 90, 3, generator=torch.Generator().manual_seed(0)), dim=2)
    out = m(c.cuda(), b.cuda(), key_padding_mask=mask.cuda())
    ref = wf_embedding_aniso_ref(c, b, m.aa_magnitudes.detach().cpu(), m.get_wavenumbers().detach().cpu(), mask)
    assert rel_l2(ref, out.detach().cpu()) < OUT_TOL
    out.square().sum().backward()
    assert torch.isfinite(m.wavenumbers.grad).all() and torch.isfinite(m.aa_magnitudes.grad).all()
