"""The attention oracle against the reference's own function (golden vectors) and closed forms."""
import os

import numpy as np
import torch

from oracle import chains
from oracle.geoattn_ref import geoattn_grads_autograd, geoattn_grads_closed_form, geoattn_ref

KEYS = ("q", "k", "v", "coords", "spreads", "betas", "mask", "min_rbf", "max_rbf", "out",
        "dq", "dk", "dv", "dspreads", "dbetas")


def _cases(golden_dir):
    g = np.load(os.path.join(golden_dir, "geoattn_reference.npz"))
    for name in sorted({k.split(".")[0] for k in g.files}):
        yield name, {x: torch.from_numpy(np.asarray(g[f"{name}.{x}"])) for x in KEYS}


def test_golden_forward_bit_exact(golden_dir):
    torch.set_num_threads(1)
    for name, t in _cases(golden_dir):
        out = geoattn_ref(t["q"], t["k"], t["v"], t["coords"], t["spreads"], t["betas"], t["mask"],
                          float(t["min_rbf"]), float(t["max_rbf"]), variant="beta_abs", zero_padded_rows=False)
        assert torch.equal(torch.isnan(out), torch.isnan(t["out"])), name
        assert torch.equal(torch.nan_to_num(out), torch.nan_to_num(t["out"])), name
        # the only NaNs of the dense form are the rows of padded queries
        assert torch.equal(torch.isnan(t["out"]).any(-1).any(1), t["mask"]), name


def test_golden_gradients(golden_dir):
    torch.set_num_threads(1)
    for name, t in _cases(golden_dir):
        d_out = (~t["mask"])[:, None, :, None].expand_as(t["out"]).float()
        _, grads = geoattn_grads_autograd(t["q"], t["k"], t["v"], t["coords"], t["spreads"], d_out, t["mask"],
                                          "beta_abs", t["betas"], float(t["min_rbf"]), float(t["max_rbf"]))
        for nm, got in zip(("dq", "dk", "dv", "dspreads", "dbetas"), grads):
            ref = t[nm]
            ok = torch.isfinite(ref)  # the dense form's NaN rows poison dV of padded samples
            assert ok.any(), (name, nm)
            assert torch.allclose(got[ok], ref[ok], atol=1e-6, rtol=1e-5), (name, nm)


def test_closed_form_matches_autograd_fp64():
    g = torch.Generator().manual_seed(0)
    z, h, n, d = 2, 3, 40, 16
    q, k, v, d_out = (torch.randn(z, h, n, d, dtype=torch.float64, generator=g) for _ in range(4))
    c, m = chains.chain_batch([40, 25], 40, seed=3)
    c, m = torch.from_numpy(c), torch.from_numpy(m)
    sp = torch.tensor([3.0, 8.0, 15.0], dtype=torch.float64)
    o_a, grads = geoattn_grads_autograd(q, k, v, c, sp, d_out, m, dtype=torch.float64)
    o_c, lse, dq, dk, dv, ds = geoattn_grads_closed_form(q, k, v, c, sp, d_out, m)
    assert (o_a - o_c).abs().max() < 1e-12
    for a, b in zip(grads, (dq, dk, dv, ds)):
        assert (a - b).abs().max() < 1e-12
    assert torch.all(o_c[1, :, 25:] == 0) and torch.all(torch.isinf(lse[1, :, 25:]))


def test_rigid_motion_invariance_and_padding_content_ignored():
    g = torch.Generator().manual_seed(1)
    z, h, n, d = 1, 2, 32, 8
    q, k, v = (torch.randn(z, h, n, d, dtype=torch.float64, generator=g) for _ in range(3))
    c, m = chains.chain_batch([20], 32, seed=9)
    c, m = torch.from_numpy(c).double(), torch.from_numpy(m)
    sp = torch.tensor([3.0, 15.0], dtype=torch.float64)
    base = geoattn_ref(q, k, v, c, sp, mask=m)
    rot, _ = torch.linalg.qr(torch.randn(3, 3, dtype=torch.float64, generator=g))
    assert (base - geoattn_ref(q, k, v, c @ rot.T + 5.0, sp, mask=m)).abs().max() < 1e-10
    k2, v2, c2 = k.clone(), v.clone(), c.clone()
    k2[:, :, 20:] = 99.0
    v2[:, :, 20:] = -99.0
    c2[:, 20:] = 1e3
    assert torch.equal(base, geoattn_ref(q, k2, v2, c2, sp, mask=m))


def _d64_cases(golden_dir):
    g = np.load(os.path.join(golden_dir, "geoattn_reference_d64.npz"))
    bf = lambda a: torch.from_numpy(np.asarray(a)).view(torch.bfloat16).float()
    for name in sorted({k.split(".")[0] for k in g.files}):
        t = {x: torch.from_numpy(np.asarray(g[f"{name}.{x}"])) for x in
             ("coords", "spreads", "betas", "mask", "min_rbf", "max_rbf", "n_valid", "out", "dq", "dk", "dv", "dspreads", "dbetas")}
        t.update({x: bf(g[f"{name}.{x}"]) for x in ("q", "k", "v", "d_out")})
        yield name, t


def test_golden_d64_in_tree_form(golden_dir):
    """Head dimension 64: the oracle's in-tree form against the reference function run on the valid prefix."""
    torch.set_num_threads(1)
    n_cases = 0
    for name, t in _d64_cases(golden_dir):
        nv = int(t["n_valid"])
        o, grads = geoattn_grads_autograd(t["q"], t["k"], t["v"], t["coords"], t["spreads"], t["d_out"], t["mask"], "beta_abs",
                                          t["betas"], float(t["min_rbf"]), float(t["max_rbf"]))
        assert torch.allclose(o[:, :, :nv], t["out"], atol=2e-6, rtol=1e-5), name
        assert torch.all(o[:, :, nv:] == 0)
        for nm, got in zip(("dq", "dk", "dv"), grads[:3]):
            assert torch.allclose(got[:, :, :nv], t[nm], atol=2e-5, rtol=1e-4), (name, nm)
            assert torch.all(got[:, :, nv:] == 0), (name, nm)
        assert torch.allclose(grads[3], t["dspreads"], atol=1e-4, rtol=1e-3), name
        assert torch.allclose(grads[4], t["dbetas"], atol=1e-4, rtol=1e-3), name
        n_cases += 1
    assert n_cases == 2
