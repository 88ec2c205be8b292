"""World-size-2 checks of the sharding logic on CPU ranks (gloo), with the oracle standing in for the
kernels: partition, all-gather reassembly, gradient all-reduce, and what the surviving rank sees when
its peer fails before the collective."""
import datetime
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import chains
from oracle.geoattn_ref import geoattn_grads_closed_form
from oracle.we_ref import dk_analytic, wf_embedding_ref
from proteusai_b200 import sharding


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _we_rows_kernel(coords, wn, mag, mask, r0, r1):
    z, n, _ = coords.shape
    k = wn.shape[0]
    out = torch.full((z, n, 2 * k), float("nan"))
    cs, sn = torch.full((z, n, k), float("nan")), torch.full((z, n, k), float("nan"))
    if r1 > r0:
        o, c, s = wf_embedding_ref(coords, wn, mag, mask, rows=(r0, r1), return_sums=True)
        out[:, r0:r1], cs[:, r0:r1], sn[:, r0:r1] = o, c, s
    return out, cs, sn


def _dk_kernel(d_out, cs, sn, r0, r1):
    return dk_analytic(d_out[:, r0:r1], cs[:, r0:r1], sn[:, r0:r1])


def _attn_kernel(Q, K, V, coords, spreads, mask, b, e, qb, qe):
    z, h, n, d = Q.shape
    o, lse, *_ = geoattn_grads_closed_form(Q, K, V, coords, spreads, torch.zeros_like(Q), mask, dtype=torch.float32)
    out, l2 = torch.full_like(o, float("nan")), torch.full_like(lse, float("nan"))
    out.view(z * h, n, d)[b:e, qb:qe] = o.reshape(z * h, n, d)[b:e, qb:qe]
    l2.view(z * h, n)[b:e, qb:qe] = lse.reshape(z * h, n)[b:e, qb:qe]
    return out, l2


def _attn_bwd_kernel(Q, K, V, O, dO, lse, coords, spreads, mask, b, e, qb, qe):
    """Stand-in for the backward kernel: only the (batch, head) pairs [b, e) and the query rows [qb, qe) contribute."""
    z, h, n, d = Q.shape
    d_sel = torch.zeros_like(dO)
    d_sel.view(z * h, n, d)[b:e, qb:qe] = dO.reshape(z * h, n, d)[b:e, qb:qe]
    _, _, dq, dk, dv, dsig = geoattn_grads_closed_form(Q, K, V, coords, spreads, d_sel, mask, dtype=torch.float32)
    nan = float("nan")
    dq_o, dk_o, dv_o = torch.full_like(dq, nan), torch.full_like(dk, nan), torch.full_like(dv, nan)
    dq_o.view(z * h, n, d)[b:e, qb:qe] = dq.reshape(z * h, n, d)[b:e, qb:qe]
    dk_o.view(z * h, n, d)[b:e] = dk.reshape(z * h, n, d)[b:e]
    dv_o.view(z * h, n, d)[b:e] = dv.reshape(z * h, n, d)[b:e]
    return dq_o, dk_o, dv_o, dsig


def _worker(rank, world, port, case, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.set_num_threads(1)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    try:
        if case == "we":
            for z, n in ((1, 64), (2, 37), (1, 33)):
                c, m = chains.chain_batch([n] + [max(1, n - 9)] * (z - 1), n, seed=n)
                c, m = torch.from_numpy(c), torch.from_numpy(m)
                wn = torch.from_numpy(chains.wavenumbers(16))
                out, cs, sn, rows = sharding.we_forward_sharded(c, wn, 1, m, kernel=_we_rows_kernel)
                full, fcs, fsn = wf_embedding_ref(c, wn, 1, m, return_sums=True)
                # the stand-in's reduction order depends on the chunk shape: compare to rounding, not bit for bit
                assert torch.allclose(out, full, rtol=1e-5, atol=1e-6), (z, n)
                d_out = torch.randn(out.shape, generator=torch.Generator().manual_seed(1))
                dk = sharding.we_backward_dk_sharded(d_out, cs, sn, rows, kernel=_dk_kernel)
                assert torch.allclose(dk, dk_analytic(d_out, fcs, fsn), rtol=1e-5, atol=1e-5)
        elif case == "attn":
            for z, h in ((1, 2), (1, 3), (2, 2)):
                g = torch.Generator().manual_seed(z * 10 + h)
                q, k, v = (torch.randn(z, h, 24, 8, generator=g) for _ in range(3))
                c, m = chains.chain_batch([24] + [17] * (z - 1), 24, seed=5)
                c, m = torch.from_numpy(c), torch.from_numpy(m)
                sp = torch.linspace(3, 15, h)
                out, lse, _ = sharding.geoattn_forward_sharded(q, k, v, c, sp, m, kernel=_attn_kernel)
                o_ref, l_ref, *_ = geoattn_grads_closed_form(q, k, v, c, sp, torch.zeros_like(q), m, dtype=torch.float32)
                assert torch.equal(out, o_ref) and torch.equal(lse, l_ref), (z, h)
            # query-block sharding: 300 rows = 3 blocks of 128 over 2 ranks (uneven), gradients summed over the shards
            g = torch.Generator().manual_seed(77)
            z, h, n = 2, 2, 300
            q, k, v, d_o = (torch.randn(z, h, n, 8, generator=g) for _ in range(4))
            c, m = chains.chain_batch([n, 190], n, seed=6)
            c, m = torch.from_numpy(c), torch.from_numpy(m)
            sp = torch.linspace(3, 15, h)
            o_ref, l_ref, dq_r, dk_r, dv_r, ds_r = geoattn_grads_closed_form(q, k, v, c, sp, d_o, m, dtype=torch.float32)
            out, lse, rows = sharding.geoattn_forward_sharded(q, k, v, c, sp, m, kernel=_attn_kernel, by="query")
            assert rows == ((0, 256) if rank == 0 else (256, 300))
            assert torch.equal(out, o_ref) and torch.equal(lse, l_ref)
            for by in ("zh", "query"):
                dq, dk, dv, ds = sharding.geoattn_backward_sharded(q, k, v, out, d_o, lse, c, sp, m, kernel=_attn_bwd_kernel, by=by)
                for got, ref in ((dq, dq_r), (dk, dk_r), (dv, dv_r), (ds, ds_r)):
                    assert torch.allclose(got, ref, rtol=1e-4, atol=1e-5), by
        elif case == "peer_fails":
            if rank == 1:
                raise RuntimeError("injected failure before the collective")
            t = torch.zeros(4, 3)
            try:
                sharding.all_gather_rows(t, 4, 0, 2)
                ret[rank] = "no error"
            except Exception as exc:  # noqa: BLE001  the collective must end with an error, not hang
                ret[rank] = "error: " + type(exc).__name__
            return
        ret[rank] = "ok"
    finally:
        try:
            dist.destroy_process_group()
        except Exception:  # noqa: BLE001
            pass


def _run(case, expect_fail_rank=None):
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, case, ret)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert not p.is_alive(), "a rank hung"
    return dict(ret), [p.exitcode for p in procs]


def test_shard_range_covers_everything():
    for total in (0, 1, 7, 64, 16384):
        for world in (1, 2, 3, 4, 8):
            pieces = [sharding.shard_range(total, world, r) for r in range(world)]
            assert pieces[0][0] == 0 and pieces[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(pieces, pieces[1:]))


def test_we_sharded_matches_unsharded_world2():
    ret, codes = _run("we")
    assert ret == {0: "ok", 1: "ok"} and codes == [0, 0]


def test_attention_sharded_matches_unsharded_world2():
    ret, codes = _run("attn")
    assert ret == {0: "ok", 1: "ok"} and codes == [0, 0]


def test_peer_failure_surfaces_as_an_error_not_a_hang():
    ret, codes = _run("peer_fails")
    assert codes[1] != 0
    assert ret.get(0, "").startswith("error"), ret
