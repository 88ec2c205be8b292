"""Parity of the CUDA geometric attention (through the C ABI) with the CPU oracle.

Tolerance is the one the path is specified to: outputs and gradients within 2e-2 absolute of the
reference arithmetic evaluated in fp32 on the same bf16-rounded inputs."""
import pytest
import torch

from oracle import chains
from oracle.geoattn_ref import geoattn_grads_closed_form, geoattn_ref

pytestmark = pytest.mark.gpu
ABS_TOL = 2e-2


@pytest.fixture(scope="module")
def ga():
    from proteusai_b200 import _lib
    from proteusai_b200.utils.model_utils.attn import geometric_attn as mod
    assert torch.cuda.is_available()
    _lib.lib()
    return mod


def _inputs(z, h, n, lengths, seed, d=64, std=None):
    g = torch.Generator().manual_seed(seed)
    std = std if std is not None else 1.0 / d ** 0.5
    q, k, v, d_out = (torch.randn(z, h, n, d, generator=g) * s for s in (std, std, std, 1.0))
    q, k, v, d_out = (t.to(torch.bfloat16) for t in (q, k, v, d_out))
    c, m = chains.chain_batch(lengths, n, seed=seed)
    sig = torch.from_numpy(chains.sigmas(h)) if h > 1 else torch.tensor([5.0])
    return q, k, v, d_out, torch.from_numpy(c), torch.from_numpy(m), sig


@pytest.mark.parametrize("z,h,n,lengths", [
    (1, 1, 128, [128]), (1, 2, 256, [256]), (2, 3, 384, [384, 200]), (2, 2, 200, [200, 77]),
    (1, 1, 64, [50]), (3, 2, 513, [513, 129, 1]), (1, 8, 1024, [700]),
])
def test_forward_matches_oracle(ga, z, h, n, lengths):
    q, k, v, _, c, m, sig = _inputs(z, h, n, lengths, seed=n + h, std=1.0)
    out, lse = ga.geoattn_forward(q.cuda(), k.cuda(), v.cuda(), c.cuda(), sig.cuda(), m.cuda())
    ref, lse_ref, *_ = geoattn_grads_closed_form(q.float(), k.float(), v.float(), c, sig, torch.zeros_like(q).float(), m,
                                                 dtype=torch.float32)
    err = (out.float().cpu() - ref).abs().max().item()
    assert err < ABS_TOL, err
    live = ~m[:, None, :].expand_as(lse_ref)
    assert torch.allclose(lse.cpu()[live], lse_ref[live], atol=2e-3, rtol=1e-4)
    assert torch.all(torch.isinf(lse.cpu()[~live])) and torch.all(out.cpu()[m[:, None].expand(z, h, n)] == 0)
    from proteusai_b200 import _lib
    _lib.device_status()


def test_forward_public_call_and_no_mask(ga):
    q, k, v, _, c, m, sig = _inputs(2, 4, 300, [300, 300], seed=5)
    out = ga.geometric_attn(q.cuda().float(), k.cuda().float(), v.cuda().float(), c.cuda(), sig.cuda(), None)
    assert out.dtype == torch.float32
    ref = geoattn_ref(q.float(), k.float(), v.float(), c, sig)
    assert (out.cpu() - ref).abs().max().item() < ABS_TOL


@pytest.mark.parametrize("z,h,n,lengths", [
    (1, 1, 128, [128]), (1, 2, 256, [256]), (2, 3, 384, [384, 200]), (2, 2, 200, [200, 77]), (3, 2, 513, [513, 129, 1]),
])
def test_backward_matches_oracle(ga, z, h, n, lengths):
    q, k, v, d_out, c, m, sig = _inputs(z, h, n, lengths, seed=7 * n + h, std=1.0)
    qd, kd, vd = (t.cuda().requires_grad_(True) for t in (q, k, v))
    sd = sig.cuda().requires_grad_(True)
    out = ga.geometric_attn(qd, kd, vd, c.cuda(), sd, None, m.cuda())
    out.backward(d_out.cuda())
    _, _, dq, dk, dv, dsig = geoattn_grads_closed_form(q.float(), k.float(), v.float(), c, sig, d_out.float(), m, dtype=torch.float64)
    for name, got, ref in (("dQ", qd.grad, dq), ("dK", kd.grad, dk), ("dV", vd.grad, dv)):
        err = (got.float().cpu().double() - ref).abs().max().item()
        # gradients come back in bf16 (the dtype of Q): allow their rounding on top of the 2e-2 budget
        assert err < ABS_TOL + ref.abs().max().item() * 2 ** -8, (name, err)
    # 2e-2 relative, plus a floor for sums that nearly cancel (P and dS are rounded to bf16)
    assert torch.all((sd.grad.cpu().double() - dsig).abs() <= 2e-2 * dsig.abs() + 5e-3), (sd.grad, dsig)
    pad = m[:, None, :, None].expand(z, h, n, 64)
    assert torch.all(qd.grad.cpu()[pad] == 0) and torch.all(kd.grad.cpu()[pad] == 0) and torch.all(vd.grad.cpu()[pad] == 0)
    from proteusai_b200 import _lib
    _lib.device_status()


def test_config3_forward_backward(ga):
    # B=8, H=8, N=1024, d=64, bf16, lengths uniform in 256..1024, sigma 3..15 A, N(0,1)/sqrt(d) inputs
    lengths = chains.draw_lengths(8, 256, 1024, seed=1003)
    q, k, v, d_out, c, m, sig = _inputs(8, 8, 1024, lengths, seed=1003)
    out, lse = ga.geoattn_forward(q.cuda(), k.cuda(), v.cuda(), c.cuda(), sig.cuda(), m.cuda())
    dq, dk, dv, dsig = ga.geoattn_backward(q.cuda(), k.cuda(), v.cuda(), out, d_out.cuda(), lse, c.cuda(), sig.cuda(), m.cuda())
    for b in range(8):  # oracle one sample at a time (fp32 on the bf16-rounded inputs)
        sl = slice(b, b + 1)
        o_r, _, dq_r, dk_r, dv_r, ds_r = geoattn_grads_closed_form(
            q[sl].float(), k[sl].float(), v[sl].float(), c[sl], sig, d_out[sl].float(), m[sl], dtype=torch.float32)
        assert (out[sl].float().cpu() - o_r).abs().max().item() < ABS_TOL
        for got, ref in ((dq, dq_r), (dk, dk_r), (dv, dv_r)):
            assert (got[sl].cpu() - ref).abs().max().item() < ABS_TOL
        if b == 0:
            ds_tot = ds_r.double()
        else:
            ds_tot += ds_r.double()
    assert torch.all((dsig.cpu().double() - ds_tot).abs() <= 2e-2 * ds_tot.abs() + 1e-5), (dsig, ds_tot)


def test_in_tree_form_matches_reference_golden(ga, golden_dir):
    """The logit form the reference tree implements (S + beta Rn |S| with the [min_rbf, max_rbf] window) against outputs
    and gradients of the reference's own `torch_attn`, at the reference test's tolerance (atol 1e-2, tests/attn/geo_attn.py:39)."""
    import os

    import numpy as np
    g = np.load(os.path.join(golden_dir, "geoattn_reference_d64.npz"))
    bf = lambda a: torch.from_numpy(np.asarray(a)).view(torch.bfloat16)
    prev = ga.set_logit_form("beta_abs")
    try:
        for name in sorted({k.split(".")[0] for k in g.files}):
            t = {x: torch.from_numpy(np.asarray(g[f"{name}.{x}"])) for x in
                 ("coords", "spreads", "betas", "mask", "min_rbf", "max_rbf", "n_valid", "out", "dq", "dk", "dv", "dspreads", "dbetas")}
            nv = int(t["n_valid"])
            q, k, v = (bf(g[f"{name}.{x}"]).cuda().requires_grad_(True) for x in ("q", "k", "v"))
            sp, be = t["spreads"].cuda().requires_grad_(True), t["betas"].cuda().requires_grad_(True)
            out = ga.geometric_attn(q, k, v, t["coords"].cuda(), sp, be, t["mask"].cuda(), float(t["min_rbf"]), float(t["max_rbf"]))
            out.backward(bf(g[f"{name}.d_out"]).cuda())
            assert (out[:, :, :nv].float().cpu() - t["out"]).abs().max().item() < 1e-2, name
            assert torch.all(out[:, :, nv:] == 0)
            for nm, got in (("dq", q.grad), ("dk", k.grad), ("dv", v.grad)):
                ref = t[nm]
                err = (got[:, :, :nv].float().cpu() - ref).abs().max().item()
                assert err < 1e-2 + ref.abs().max().item() * 2 ** -8, (name, nm, err)  # + bf16 rounding of the returned gradient
                assert torch.all(got[:, :, nv:] == 0), (name, nm)
            assert torch.all((sp.grad.cpu() - t["dspreads"]).abs() <= 2e-2 * t["dspreads"].abs() + 5e-3), (name, sp.grad, t["dspreads"])
            assert torch.all((be.grad.cpu() - t["dbetas"]).abs() <= 2e-2 * t["dbetas"].abs() + 5e-3), (name, be.grad, t["dbetas"])
    finally:
        ga.set_logit_form(prev)
    from proteusai_b200 import _lib
    _lib.device_status()


def test_strided_inputs_and_head_major_output(ga):
    """Q, K, V read in place as the [Z,H,N,d] views of a fused projection output [Z,N,3,H,d], O written as [Z,N,H,d]:
    the same kernel on the same values, so the results equal those of the contiguous call bit for bit."""
    z, h, n, d = 2, 3, 200, 64
    g = torch.Generator().manual_seed(31)
    y = (torch.randn(z, n, 3, h, d, generator=g) / 8).to(torch.bfloat16).cuda()
    q, k, v = (y[:, :, i].permute(0, 2, 1, 3) for i in range(3))
    assert not q.is_contiguous()
    c, m = chains.chain_batch([200, 77], n, seed=32)
    c, m = torch.from_numpy(c).cuda(), torch.from_numpy(m).cuda()
    sig = torch.from_numpy(chains.sigmas(h)).cuda()
    o_ref, l_ref = ga.geoattn_forward(q.contiguous(), k.contiguous(), v.contiguous(), c, sig, m)
    o, l = ga.geoattn_forward(q, k, v, c, sig, m, out_layout="znhd")
    assert o.shape == (z, h, n, d) and o.permute(0, 2, 1, 3).is_contiguous()
    assert torch.equal(o, o_ref) and torch.equal(l, l_ref)
    # a shard of the (batch, head) pairs through the strided path
    o2 = torch.zeros_like(o)
    ga.geoattn_forward(q, k, v, c, sig, m, 2, 5, out=o2)
    assert torch.equal(o2.reshape(z * h, n, d)[2:5], o_ref.reshape(z * h, n, d)[2:5])
    assert torch.all(o2.reshape(z * h, n, d)[:2] == 0) and torch.all(o2.reshape(z * h, n, d)[5:] == 0)
    # the public call without gradients takes the strided path and returns the head-major layout
    with torch.no_grad():
        pub = ga.geometric_attn(q, k, v, c, sig, None, mask=m)
    assert torch.equal(pub, o_ref) and pub.permute(0, 2, 1, 3).is_contiguous()
    # rows that are not on 16-byte boundaries are copied, not rejected
    odd = torch.zeros(z, h, n, d + 4, dtype=torch.bfloat16, device="cuda")[..., 2:d + 2]
    odd.copy_(q)
    o3, _ = ga.geoattn_forward(odd, k, v, c, sig, m)
    assert torch.equal(o3, o_ref)


@pytest.mark.parametrize("form", ["beta_abs", "one_plus_rbf"])
def test_reference_test_configuration_with_heads_of_32(ga, form):
    """The reference test's own setup (tests/attn/geo_attn.py:14-31): batch 1, 4 heads, N 128, d_model 128, i.e. heads
    of 32, fp32 N(0,1) inputs, collinear coordinates 50 N(0,1), spreads 3, betas 1, window [0, 1], at its tolerance
    (atol 1e-2, :39) against the oracle on the bf16-rounded inputs.  Heads narrower than 64 run zero-padded."""
    from oracle.geoattn_ref import geoattn_grads_autograd
    g = torch.Generator().manual_seed(41)
    z, h, n, dk = 1, 4, 128, 32
    q, k, v = (torch.randn(z, h, n, dk, generator=g) for _ in range(3))
    coords = (50 * torch.randn(z, n, 1, generator=g)).expand(z, n, 3).contiguous()
    spreads, betas = torch.full((h,), 3.0), torch.full((h,), 1.0)
    mask = torch.zeros(z, n, dtype=torch.bool)
    d_out = torch.randn(z, h, n, dk, generator=g)
    rnd = lambda t: t.to(torch.bfloat16).float()
    o_ref, grads = geoattn_grads_autograd(rnd(q), rnd(k), rnd(v), coords, spreads, rnd(d_out), mask, variant=form, betas=betas,
                                          min_rbf=0.0, max_rbf=1.0)
    prev = ga.set_logit_form(form)
    try:
        leaves = [t.cuda().requires_grad_(True) for t in (q, k, v, spreads, betas)]
        out = ga.geometric_attn(leaves[0], leaves[1], leaves[2], coords.cuda(), leaves[3], leaves[4], mask.cuda(), 0.0, 1.0)
        assert out.shape == (z, h, n, dk) and out.dtype == torch.float32
        out.backward(rnd(d_out).cuda())
    finally:
        ga.set_logit_form(prev)
    assert (out.detach().cpu() - o_ref.detach()).abs().max().item() < 1e-2
    for got, ref, nm in zip(leaves[:3], grads[:3], ("dq", "dk", "dv")):
        assert got.grad.shape == (z, h, n, dk)
        assert (got.grad.cpu() - ref).abs().max().item() < 1e-2 + ref.abs().max().item() * 2 ** -8, nm
    assert torch.all((leaves[3].grad.cpu() - grads[3]).abs() <= 2e-2 * grads[3].abs() + 1e-2)   # atol of the reference's own test
    if form == "beta_abs":
        assert torch.all((leaves[4].grad.cpu() - grads[4]).abs() <= 2e-2 * grads[4].abs() + 1e-2)   # atol of the reference's own test
    with torch.no_grad():  # the copy-free inference path pads and slices too
        o2 = ga.geometric_attn(q.cuda(), k.cuda(), v.cuda(), coords.cuda(), spreads.cuda(), betas.cuda(), mask.cuda(), 0.0, 1.0) \
            if form == "one_plus_rbf" else None
    if o2 is not None:
        assert (o2.cpu() - o_ref.detach()).abs().max().item() < 1e-2
    with pytest.raises(RuntimeError):
        ga.geometric_attn(torch.zeros(1, 1, 8, 128).cuda(), torch.zeros(1, 1, 8, 128).cuda(), torch.zeros(1, 1, 8, 128).cuda(),
                          torch.zeros(1, 8, 3).cuda(), torch.ones(1).cuda(), None)


@pytest.mark.parametrize("n", [1, 5, 127, 129])
def test_tiny_and_odd_lengths_forward_backward(ga, n):
    q, k, v, d_out, c, m, sig = _inputs(2, 2, n, [n, max(1, n // 2)], seed=900 + n, std=1.0)
    qd, kd, vd = (t.cuda().requires_grad_(True) for t in (q, k, v))
    out = ga.geometric_attn(qd, kd, vd, c.cuda(), sig.cuda(), None, m.cuda())
    out.backward(d_out.cuda())
    o_r, _, dq, dk, dv, _ = geoattn_grads_closed_form(q.float(), k.float(), v.float(), c, sig, d_out.float(), m, dtype=torch.float64)
    assert (out.detach().float().cpu().double() - o_r).abs().max().item() < ABS_TOL
    for got, ref in ((qd.grad, dq), (kd.grad, dk), (vd.grad, dv)):
        assert (got.float().cpu().double() - ref).abs().max().item() < ABS_TOL + ref.abs().max().item() * 2 ** -8


def test_masks_with_holes_and_an_empty_sample(ga):
    """Padding masks need not be prefixes: holes inside a chain, and a sample with no valid token at all (zeros out, zero
    gradients, no NaN anywhere)."""
    z, h, n = 3, 2, 300
    q, k, v, d_out, c, m, sig = _inputs(z, h, n, [300, 300, 300], seed=77, std=1.0)
    g = torch.Generator().manual_seed(78)
    m = torch.zeros(z, n, dtype=torch.bool)
    m[0] = torch.rand(n, generator=g) < 0.3          # holes
    m[1, 100:260] = True                             # a gap that swallows a whole key tile
    m[2] = True                                      # nothing valid
    qd, kd, vd = (t.cuda().requires_grad_(True) for t in (q, k, v))
    sd = sig.cuda().requires_grad_(True)
    out = ga.geometric_attn(qd, kd, vd, c.cuda(), sd, None, m.cuda())
    out.backward(d_out.cuda())
    o_r, _, dq, dk, dv, dsig = geoattn_grads_closed_form(q.float(), k.float(), v.float(), c, sig, d_out.float(), m, dtype=torch.float64)
    assert (out.detach().float().cpu().double() - o_r).abs().max().item() < ABS_TOL
    for got, ref in ((qd.grad, dq), (kd.grad, dk), (vd.grad, dv)):
        assert torch.isfinite(got).all()
        assert (got.float().cpu().double() - ref).abs().max().item() < ABS_TOL + ref.abs().max().item() * 2 ** -8
    assert torch.all(out[2] == 0) and torch.all(qd.grad[2] == 0) and torch.all(kd.grad[2] == 0) and torch.all(vd.grad[2] == 0)
    assert torch.all((sd.grad.cpu().double() - dsig).abs() <= 2e-2 * dsig.abs() + 5e-3)
    from proteusai_b200 import _lib
    _lib.device_status()


def test_batch_plan_lists_live_tiles_and_orders_samples(ga):
    """pai_geoattn_plan against the same bookkeeping done in numpy: live 128-token tiles per sample with their hole flags,
    first valid offsets, valid counts, and the samples by decreasing tile count (stable)."""
    import numpy as np
    z, n = 6, 700
    g = torch.Generator().manual_seed(5)
    m = torch.ones(z, n, dtype=torch.bool)
    for b, length in enumerate([700, 1, 300, 129, 0, 512]):
        m[b, :length] = False
    m[2, 130:200] = True   # a hole
    m[5, 0:128] = True     # an empty first tile
    plan = ga.geoattn_plan(m.cuda()).plan.cpu().numpy()
    tiles = (n + 127) // 128
    assert plan[0] == z and plan[1] == n and plan[2] == tiles and plan[3] == 0
    order, count, nvalid = plan[4:4 + z], plan[4 + z:4 + 2 * z], plan[4 + 2 * z:4 + 3 * z]
    lists = plan[4 + 3 * z:4 + 3 * z + z * tiles].reshape(z, tiles)
    info = plan[4 + 3 * z + z * tiles:4 + 3 * z + 2 * z * tiles].reshape(z, tiles)
    valid = ~m.numpy()
    want_count = []
    for b in range(z):
        live = []
        for t in range(tiles):
            seg = valid[b, t * 128:(t + 1) * 128]
            if seg.any():
                hole = 0x8000 if seg.sum() < 128 else 0
                live.append(t | hole)
                assert info[b, t] == (int(np.argmax(seg)) | hole)
            else:
                assert info[b, t] == -1
        assert list(lists[b, :len(live)]) == live and count[b] == len(live) and nvalid[b] == valid[b].sum()
        want_count.append(len(live))
    assert list(order) == sorted(range(z), key=lambda b: (-want_count[b], b))
    assert ga.geoattn_plan(None) is None
    assert ga.geoattn_plan(m.cuda()) is not ga.geoattn_plan(m.cuda())   # different tensors: different plans
    mc = m.cuda()
    assert ga.geoattn_plan(mc) is ga.geoattn_plan(mc)                    # the same tensor: one plan for all layers


def test_balanced_schedule_covers_every_item_once_and_changes_no_result(ga):
    """pai_geoattn_schedule: every live (batch, head, tile) item sits in exactly one CTA's list, the tiles without a valid
    token are all on the dead list, no list is longer than its capacity and the fullest CTA is close to the mean.  The
    persistent-CTA launch that follows the schedule gives the forward of the one-CTA-per-item launch bit for bit (and
    the backward up to the order of the dQ reductions)."""
    import numpy as np
    from proteusai_b200 import _lib
    z, h, n = 6, 4, 900
    lengths = [900, 130, 512, 77, 0, 640]
    q, k, v, d_out, c, m, sig = (t.cuda() for t in _inputs(z, h, n, lengths, seed=91, std=1.0))
    def check_schedule(mask, z, h, n):
        gp = ga.geoattn_plan(mask)
        tiles = (n + 127) // 128
        plan = gp.plan.cpu().numpy()
        count = plan[4 + z:4 + 2 * z]
        info = plan[4 + 3 * z + z * tiles:4 + 3 * z + 2 * z * tiles].reshape(z, tiles)
        want_live = {((b * h + hh) << 10) | t for b in range(z) for hh in range(h) for t in range(tiles) if info[b, t] >= 0}
        want_dead = {((b * h + hh) << 10) | t for b in range(z) for hh in range(h) for t in range(tiles) if info[b, t] < 0}
        for backward in (False, True):
            sched, bins = gp.schedule(h, backward)
            assert sched is not None and bins > 0
            sw = sched.cpu().numpy()
            cap = int(sw[4])
            assert list(sw[:4]) == [bins, h, z, n] and sw[5] == len(want_dead) and sw[6] == len(want_live)
            cnt = sw[8:8 + bins]
            lists = sw[8 + bins:8 + bins + bins * cap].reshape(bins, cap)
            assert cnt.max() <= cap
            got = [int(x) for b in range(bins) for x in lists[b, :cnt[b]]]
            assert len(got) == len(set(got)) and set(got) == want_live
            dead = sw[8 + bins + bins * cap:8 + bins + bins * cap + len(want_dead)]
            assert set(int(x) for x in dead) == want_dead and len(set(dead.tolist())) == len(want_dead)
            load = np.array([sum(count[(int(x) >> 10) // h] for x in lists[b, :cnt[b]]) for b in range(bins)])
            assert load.max() <= max(count.max(), int(np.ceil(load.sum() / bins)) + count.max())
            # the packing itself, restated: first fit, longest first, into bins of capacity C; C bisected to the smallest that fits
            tile_cost, item_cost = 8, (12 if backward else 5)
            nb = bins if backward else bins // 2   # the forward packs per SM and deals each SM's items to two CTAs
            costs = sorted((int(count[b]) * tile_cost + item_cost for b in range(z) for _ in range(int(count[b]) * h) if count[b] > 0), reverse=True)

            def fits(cap_c):
                loads = [0] * nb
                for cst in costs:
                    for i in range(nb):
                        if loads[i] + cst <= cap_c:
                            loads[i] += cst
                            break
                    else:
                        return None
                return loads
            lo = max(max(costs), -(-sum(costs) // nb))
            hi_c = 2 * lo + 1
            while lo < hi_c:
                mid = (lo + hi_c) // 2
                if fits(mid) is None:
                    lo = mid + 1
                else:
                    hi_c = mid
            assert sw[7] == hi_c
            got_cost = np.array([sum(int(count[(int(x) >> 10) // h]) * tile_cost + item_cost for x in lists[b, :cnt[b]]) for b in range(bins)])
            per_bin = got_cost if backward else got_cost[:nb] + got_cost[nb:2 * nb]
            assert sorted(per_bin.tolist()) == sorted(fits(hi_c))
        return gp

    gp = check_schedule(m, z, h, n)
    m8 = torch.ones(8, 1024, dtype=torch.bool)
    for b, length in enumerate([1024, 1000, 900, 770, 650, 512, 400, 300]):
        m8[b, :length] = False
    check_schedule(m8.cuda(), 8, 8, 1024)   # several items per CTA: the packing has work to do
    o_s, l_s = ga.geoattn_forward(q, k, v, c, sig, m)
    grads_s = ga.geoattn_backward(q, k, v, o_s, d_out, l_s, c, sig, m)
    try:
        _lib.tune(ga_no_order=1)   # one CTA per item, natural order
        o_1, l_1 = ga.geoattn_forward(q, k, v, c, sig, m)
        grads_1 = ga.geoattn_backward(q, k, v, o_1, d_out, l_1, c, sig, m)
    finally:
        _lib.tune_reset()
    assert torch.equal(o_s, o_1) and torch.equal(l_s, l_1)
    scale = max(g.abs().max().item() for g in grads_1[:3])
    for a, b in zip(grads_s[:3], grads_1[:3]):
        assert (a - b).abs().max().item() < 1e-4 * scale
    assert torch.allclose(grads_s[3], grads_1[3], rtol=1e-3, atol=1e-4)
    # a schedule made for another head count is not followed: nothing runs, the status word says so, the next call is fine
    q2, k2, v2 = (torch.cat([t, t], dim=1) for t in (q, k, v))
    sig2 = torch.cat([sig, sig])
    gp.schedules[(2 * h, False)] = gp.schedules[(h, False)]
    ga.geoattn_forward(q2, k2, v2, c, sig2, m)
    with pytest.raises(RuntimeError, match="status -2"):
        _lib.device_status()
    del gp.schedules[(2 * h, False)]
    o_2, _ = ga.geoattn_forward(q2, k2, v2, c, sig2, m)
    assert torch.equal(o_2[:, :h], o_s) and torch.equal(o_2[:, h:], o_s)
    # any number of persistent CTAs may follow a schedule: one (no second CTA to pair with) and an odd count
    lib = _lib.lib()
    for bins in (1, 3):
        nbytes = lib.pai_geoattn_schedule_bytes(z, n, h, bins)
        small = torch.empty((nbytes + 3) // 4, dtype=torch.int32, device="cuda")
        _lib.check(lib.pai_geoattn_schedule(_lib.ptr(gp.plan), z, n, h, bins, 0, _lib.ptr(small), nbytes, _lib.current_stream()),
                   "pai_geoattn_schedule")
        sw = small.cpu().numpy()
        cap = int(sw[4])
        assert int(sw[0]) == bins and int(sw[8:8 + bins].sum()) == int(sw[6]) and int(sw[8:8 + bins].max()) <= cap
        keep = gp.schedules[(h, False)]
        gp.schedules[(h, False)] = (small, bins)
        try:
            o_b, l_b = ga.geoattn_forward(q, k, v, c, sig, m)
        finally:
            gp.schedules[(h, False)] = keep
        _lib.device_status()
        assert torch.equal(o_b, o_s) and torch.equal(l_b, l_s)
    # a large batch has many items per CTA slot and runs without a schedule
    big = torch.zeros(64, 1024, dtype=torch.bool, device="cuda")
    assert ga.geoattn_plan(big).schedule(8, False) == (None, 0)
    _lib.device_status()


def test_query_row_ranges_shard_forward_and_backward(ga):
    """Sharding by query blocks: the forward on row ranges reproduces the full call bit for bit; in the backward dQ rows
    come from their own shard and dK, dV, d_sigma are partial sums that add up to the full gradients."""
    z, h, n = 2, 2, 600
    q, k, v, d_out, c, m, sig = (t.cuda() for t in _inputs(z, h, n, [600, 333], seed=61, std=1.0))
    o_full, l_full = ga.geoattn_forward(q, k, v, c, sig, m)
    o = torch.full_like(o_full, float("nan"))
    l = torch.full_like(l_full, float("nan"))
    ranges = ((0, 256), (256, 512), (512, 600))
    for a, b in ranges:
        ga.geoattn_forward(q, k, v, c, sig, m, out=o, lse=l, q_begin=a, q_end=b)
    assert torch.equal(o, o_full) and torch.equal(l, l_full)
    dq_f, dk_f, dv_f, ds_f = ga.geoattn_backward(q, k, v, o_full, d_out, l_full, c, sig, m)
    dq = torch.full_like(dq_f, float("nan"))
    dk, dv, ds = torch.zeros_like(dk_f), torch.zeros_like(dv_f), torch.zeros_like(ds_f)
    for a, b in ranges:
        dq_p, dk_p, dv_p, ds_p = ga.geoattn_backward(q, k, v, o_full, d_out, l_full, c, sig, m, q_begin=a, q_end=b)
        dq[:, :, a:b] = dq_p[:, :, a:b]
        dk += dk_p
        dv += dv_p
        ds += ds_p
    scale = max(dk_f.abs().max().item(), dv_f.abs().max().item(), dq_f.abs().max().item())
    assert (dq - dq_f).abs().max().item() < 1e-4 * scale      # same tiles, fp32 reductions in another order
    assert (dk - dk_f).abs().max().item() < 1e-4 * scale and (dv - dv_f).abs().max().item() < 1e-4 * scale
    assert torch.allclose(ds, ds_f, rtol=1e-3, atol=1e-4)
    from proteusai_b200 import _lib
    _lib.device_status()


def test_far_key_groups_skip_changes_nothing(ga):
    """Key groups farther than 5.9 sigma from a warp's queries skip the RBF arithmetic; there 1 + R == 1 in fp32, so the
    output with the skip switched off (test-only tuning entry) is the same, bit for bit."""
    from proteusai_b200 import _lib
    q, k, v, _, c, m, sig = (t.cuda() for t in _inputs(2, 8, 1024, [1024, 700], seed=71))
    o_skip, l_skip = ga.geoattn_forward(q, k, v, c, sig, m)
    try:
        _lib.tune(ga_no_far_skip=1)
        o_all, l_all = ga.geoattn_forward(q, k, v, c, sig, m)
    finally:
        _lib.tune_reset()
    assert torch.equal(o_skip, o_all) and torch.equal(l_skip, l_all)


def test_padding_may_hold_nan(ga):
    """Rows of padded tokens are never read into the result: NaN in Q and K there changes nothing (V of padded keys
    meets P = 0 in the tensor core, where 0 x NaN is NaN as in the reference's own dot product, so V stays finite)."""
    z, h, n = 2, 2, 300
    q, k, v, d_out, c, m, sig = (t.cuda() for t in _inputs(z, h, n, [300, 150], seed=81, std=1.0))
    o_ref, l_ref = ga.geoattn_forward(q, k, v, c, sig, m)
    pad = m[:, None, :, None].expand(z, h, n, 64)
    qn, kn = q.clone(), k.clone()
    qn[pad] = float("nan")
    kn[pad] = float("inf")
    o, l = ga.geoattn_forward(qn, kn, v, c, sig, m)
    assert torch.isfinite(o).all() and torch.equal(o, o_ref) and torch.equal(l, l_ref)


def test_logit_form_is_an_argument_and_ignored_inputs_warn(ga):
    import warnings
    q, k, v, d_out, c, m, sig = (t.cuda() for t in _inputs(1, 2, 200, [180], seed=91, std=1.0))
    betas = torch.tensor([0.7, 1.3], device="cuda", requires_grad=True)
    with torch.no_grad():
        a = ga.geometric_attn(q, k, v, c, sig, betas, m, 0.001, 1.0, form="beta_abs")
        prev = ga.set_logit_form("beta_abs")
        try:
            b = ga.geometric_attn(q, k, v, c, sig, betas, m, 0.001, 1.0)
        finally:
            ga.set_logit_form(prev)
        one = ga.geometric_attn(q, k, v, c, sig, None, m)
    assert torch.equal(a, b) and not torch.equal(a, one)
    ga._warned_ignored = False
    with warnings.catch_warnings(record=True) as w:
        warnings.simplefilter("always")
        ga.geometric_attn(q, k, v, c, sig, betas, m, 0.001, 1.0, form="one_plus_rbf")
    assert any("one_plus_rbf" in str(x.message) for x in w)
    # gradients flow through the ten-argument call too
    qd = q.clone().requires_grad_(True)
    out = ga.geometric_attn(qd, k, v, c, sig, betas, m, 0.001, 1.0, form="beta_abs")
    out.backward(d_out)
    assert betas.grad is not None and qd.grad is not None
    with pytest.raises(ValueError):
        ga.geometric_attn(q, k, v, c, sig, betas, m, form="nope")
