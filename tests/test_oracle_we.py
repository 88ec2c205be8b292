"""The WE oracle against the reference's own function (golden vectors) and against itself."""
import os

import numpy as np
import pytest
import torch

from oracle import chains
from oracle.we_ref import dk_analytic, dk_autograd, rel_l2, wf_embedding_ref

torch.set_num_threads(max(1, min(8, os.cpu_count() or 1)))


def _cases(golden_dir):
    g = np.load(os.path.join(golden_dir, "we_reference.npz"))
    for name in sorted({k.split(".")[0] for k in g.files}):
        yield name, {x: torch.from_numpy(np.asarray(g[f"{name}.{x}"])) for x in
                     ("coords", "wn", "mag", "mask", "out", "dk_sum")}


def test_golden_bit_exact(golden_dir):
    torch.set_num_threads(1)
    n = 0
    for name, t in _cases(golden_dir):
        for chunk in (32, 128):
            out = wf_embedding_ref(t["coords"], t["wn"], int(t["mag"]), t["mask"], chunk=chunk)
            assert torch.equal(out, t["out"]), (name, chunk)
        n += 1
    assert n == 5


def test_golden_dk_from_stored_sums(golden_dir):
    # the analytic backward (stored cos/sin sums) against autograd through the reference function
    for name, t in _cases(golden_dir):
        out, cs, sn = wf_embedding_ref(t["coords"], t["wn"], int(t["mag"]), t["mask"], return_sums=True)
        dk = dk_analytic(torch.ones_like(out), cs, sn)
        assert rel_l2(t["dk_sum"], dk) < 1e-5, name


def test_row_slices_match_full():
    c, m = chains.chain_batch([100, 61], 100, seed=3)
    c, m = torch.from_numpy(c), torch.from_numpy(m)
    wn = torch.from_numpy(chains.wavenumbers(32))
    full = wf_embedding_ref(c, wn, 1, m, chunk=100)
    part = wf_embedding_ref(c, wn, 1, m, rows=(17, 83), chunk=16)
    assert torch.equal(full[:, 17:83], part)


def test_fp64_truth_and_autograd_dk():
    c, m = chains.chain_batch([72, 40], 72, seed=4)
    c, m = torch.from_numpy(c), torch.from_numpy(m)
    wn = torch.from_numpy(chains.wavenumbers(16))
    o32, cs, sn = wf_embedding_ref(c, wn, 1, m, return_sums=True)
    o64 = wf_embedding_ref(c, wn, 1, m, dtype=torch.float64)
    assert rel_l2(o64, o32) < 1e-5
    g = torch.Generator().manual_seed(0)
    d_out = torch.randn(o32.shape, generator=g)
    assert rel_l2(dk_autograd(c, wn, d_out, 1, m), dk_analytic(d_out, cs, sn)) < 1e-5


def test_masked_rows_and_single_token_are_zero():
    c, m = chains.chain_batch([1, 5], 8, seed=5)
    c, m = torch.from_numpy(c), torch.from_numpy(m)
    wn = torch.from_numpy(chains.wavenumbers(8))
    out = wf_embedding_ref(c, wn, 1, m)
    assert torch.all(out[0] == 0)  # one valid token: no pair at all
    assert torch.all(out[1, 5:] == 0)


def test_rigid_motion_invariance_and_permutation_equivariance():
    c, _ = chains.chain_batch([64], 64, seed=6)
    c = torch.from_numpy(c).double()
    wn = torch.from_numpy(chains.wavenumbers(16)).double()
    q, _ = torch.linalg.qr(torch.randn(3, 3, dtype=torch.float64, generator=torch.Generator().manual_seed(1)))
    moved = c @ q.T + torch.tensor([10.0, -3.0, 7.0], dtype=torch.float64)
    base = wf_embedding_ref(c, wn)
    assert rel_l2(base, wf_embedding_ref(moved, wn)) < 1e-10
    perm = torch.randperm(64, generator=torch.Generator().manual_seed(2))
    assert rel_l2(base[:, perm], wf_embedding_ref(c[:, perm], wn)) < 1e-10


def test_chain_geometry():
    rng = np.random.default_rng(0)
    r = chains.random_walk_chain(200, rng)
    steps = np.linalg.norm(np.diff(r, axis=0), axis=1)
    assert np.allclose(steps, 3.8, atol=1e-9)
    d2 = np.linalg.norm(r[2:] - r[:-2], axis=1)  # bond angle 90..120 deg -> 5.37..6.58 A
    assert d2.min() > 5.3 and d2.max() < 6.6
    wn = chains.wavenumbers(512)
    assert wn.shape == (256,) and abs(wn[0] - 2 * np.pi / 3.7) < 1e-6 and wn[-1] > 2 * np.pi / 20.0


def test_dropout_hash_restatement():
    """The keep count and an order-dependent checksum of the hashes were produced by compiling the same 32-bit
    arithmetic as a C program (gcc) over the same index grid: z < 2, i < 50, j < 60, k < 16, seed 1234, p = 0.3."""
    from oracle.we_ref import dropout_hash, dropout_keep
    idx = (np.arange(2)[:, None, None, None], np.arange(50)[None, :, None, None],
           np.arange(60)[None, None, :, None], np.arange(16)[None, None, None, :])
    h = dropout_hash(*idx, 1234)
    assert h.dtype == np.uint32 and h.shape == (2, 50, 60, 16)
    x = 0
    for v in h.ravel().tolist():
        x = (x * 31 + v) & 0xFFFFFFFF
    assert x == 4207743621
    keep = dropout_keep(*idx, 1234, 0.3)
    assert int(keep.sum()) == 67135
    assert abs(keep.mean() - 0.7) < 5e-3
    assert dropout_keep(*idx, 1234, 0.0).all()


def test_dropout_forward_and_gradient_are_consistent():
    c, m = chains.chain_batch([48, 31], 48, seed=8)
    c, m = torch.from_numpy(c), torch.from_numpy(m)
    wn = torch.from_numpy(chains.wavenumbers(16))
    base = wf_embedding_ref(c, wn, 1, m)
    o, cs, sn = wf_embedding_ref(c, wn, 1, m, return_sums=True, dropout_p=0.2, seed=99)
    assert rel_l2(base, o) > 1e-2                       # something was dropped
    assert torch.all(o[1, 31:] == 0)                    # padded rows stay zero
    assert torch.equal(o, wf_embedding_ref(c, wn, 1, m, dropout_p=0.2, seed=99, chunk=16))  # index hash: chunking-free
    assert not torch.equal(o, wf_embedding_ref(c, wn, 1, m, dropout_p=0.2, seed=100))
    # averaged over seeds the scaled output is unbiased
    mean = sum(wf_embedding_ref(c, wn, 1, m, dropout_p=0.2, seed=s).double() for s in range(200)) / 200
    assert rel_l2(base, mean) < 5e-2
    d_out = torch.randn(o.shape, generator=torch.Generator().manual_seed(1))
    assert rel_l2(dk_autograd(c, wn, d_out, 1, m, dropout_p=0.2, seed=99), dk_analytic(d_out, cs, sn)) < 1e-5
