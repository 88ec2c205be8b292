"""Sharding of the two hot paths across the GPUs of one node (one process per GPU).

Both paths partition without any exchange during the computation:

* Wavefunction Embedding: every rank holds all coordinates (a few hundred kB) and computes a contiguous
  range of observer rows; the output is reassembled with one all-gather; the wavenumber gradient is a
  local reduction followed by an all-reduce of ``[K]`` floats.
* Geometric attention: every rank computes a contiguous range of (batch, head) pairs; outputs are
  reassembled with one all-gather, the spread gradient with an all-reduce of ``[H]`` floats.  With few
  (batch, head) pairs and long sequences the ranks split the query blocks of 128 rows instead (the first axis of
  the reference kernel's grid, ``old/old_scripts/attn/geometric_attn.py:582-585``), keys and values replicated;
  then dQ rows are gathered and dK, dV, d_sigma, which every query block contributes to, are all-reduced.

The compute callables are parameters so that the partition / gather logic can be exercised on CPU
ranks (gloo) with a stand-in kernel; on GPUs the defaults are the CUDA entry points.
"""
import torch
import torch.distributed as dist


def shard_range(total, world, rank):
    """Contiguous range ``[begin, end)`` of ``total`` items owned by ``rank`` (sizes differ by at most one block)."""
    per = (total + world - 1) // world
    return min(total, rank * per), min(total, (rank + 1) * per)


def query_shard_range(n, world, rank, block=128):
    """Query rows ``[begin, end)`` of ``rank`` when the blocks of ``block`` rows are dealt out contiguously."""
    blocks = (n + block - 1) // block
    b, e = shard_range(blocks, world, rank)
    return min(n, b * block), min(n, e * block)


def _world(group):
    if not (dist.is_available() and dist.is_initialized()):
        return 1, 0
    return dist.get_world_size(group), dist.get_rank(group)


def all_gather_rows(full, dim_total, begin, end, group=None, range_of=None):
    """``full`` is a contiguous tensor whose leading dimension has ``dim_total`` items of which this rank
    has filled ``[begin, end)``; afterwards every rank holds all of it.  In place when the split is even.
    ``range_of(rank)`` gives every rank's range (default: ``shard_range``)."""
    world, rank = _world(group)
    if world == 1:
        return full
    if range_of is None:
        range_of = lambda r: shard_range(dim_total, world, r)
    ranges = [range_of(r) for r in range(world)]
    assert ranges[rank] == (begin, end), (ranges[rank], begin, end)
    per = max(e - b for b, e in ranges)
    flat = full.view(dim_total, -1)
    if all(e - b == per for b, e in ranges) and per * world == dim_total:
        dist.all_gather_into_tensor(flat, flat[begin:end], group=group)
    else:
        parts = [torch.empty_like(flat[:per]) for _ in range(world)]
        mine = torch.zeros_like(flat[:per])
        mine[:end - begin] = flat[begin:end]
        dist.all_gather(parts, mine, group=group)
        for r, (b, e) in enumerate(ranges):
            flat[b:e] = parts[r][:e - b]
    return full


def we_forward_sharded(coords, wavenumbers, magnitude_type=1, mask=None, group=None, kernel=None):
    """Forward with observer rows sharded over the ranks of ``group``.  Returns ``(out, cos_sums, sin_sums,
    (row_begin, row_end))``: ``out [Z,N,2K]`` complete on every rank, the two sums valid on the rank's own
    rows only (they stay sharded for the backward)."""
    if kernel is None:
        from proteusai_b200.utils.model_utils.wf_embedding.isotropic.cuda.wf_embedding import we_forward_rows as kernel
    world, rank = _world(group)
    z, n, _ = coords.shape
    r0, r1 = shard_range(n, world, rank)
    out, cs, sn = kernel(coords, wavenumbers, magnitude_type, mask, r0, r1)
    if world > 1:
        if z == 1:
            all_gather_rows(out[0], n, r0, r1, group)
        else:  # rows are the second dimension: gather a [N, Z, 2K] view
            t = out.transpose(0, 1).contiguous()
            all_gather_rows(t, n, r0, r1, group)
            out.copy_(t.transpose(0, 1))
    return out, cs, sn, (r0, r1)


def we_backward_dk_sharded(d_out, cos_sums, sin_sums, rows, group=None, kernel=None):
    """Wavenumber gradient: local reduction over the rank's rows, then a sum over ranks."""
    if kernel is None:
        from proteusai_b200.utils.model_utils.wf_embedding.isotropic.cuda.wf_embedding import we_backward_dk as kernel
    world, _ = _world(group)
    dk = kernel(d_out, cos_sums, sin_sums, rows[0], rows[1])
    if world > 1:
        dist.all_reduce(dk, op=dist.ReduceOp.SUM, group=group)
    return dk


def geoattn_forward_sharded(Q, K, V, coords, spreads, mask=None, group=None, kernel=None, by="zh"):
    """Forward sharded over the ranks, ``O`` and ``L`` complete on every rank afterwards.
    ``by="zh"``: contiguous ranges of (batch, head) pairs; returns ``(O, L, (zh_begin, zh_end))``.
    ``by="query"``: contiguous ranges of 128-row query blocks, every rank reading all keys and values; returns
    ``(O, L, (q_begin, q_end))``.  ``kernel(Q, K, V, coords, spreads, mask, zh_begin, zh_end, q_begin, q_end)``."""
    if kernel is None:
        from proteusai_b200.utils.model_utils.attn.geometric_attn import geoattn_forward

        def kernel(Q, K, V, coords, spreads, mask, b, e, qb, qe):
            return geoattn_forward(Q, K, V, coords, spreads, mask, b, e, q_begin=qb, q_end=qe)
    world, rank = _world(group)
    z, h, n = Q.shape[0], Q.shape[1], Q.shape[2]
    if by == "zh":
        b, e = shard_range(z * h, world, rank)
        out, lse = kernel(Q, K, V, coords, spreads, mask, b, e, 0, n)
        if world > 1:
            all_gather_rows(out.view(z * h, -1), z * h, b, e, group)
            all_gather_rows(lse.view(z * h, -1), z * h, b, e, group)
        return out, lse, (b, e)
    if by != "query":
        raise ValueError(f"by must be 'zh' or 'query', not {by!r}")
    qb, qe = query_shard_range(n, world, rank)
    out, lse = kernel(Q, K, V, coords, spreads, mask, 0, z * h, qb, qe)
    if world > 1:
        rng = lambda r: query_shard_range(n, world, r)
        o_t = out.permute(2, 0, 1, 3).contiguous()  # rows first
        all_gather_rows(o_t, n, qb, qe, group, rng)
        out.copy_(o_t.permute(1, 2, 0, 3))
        l_t = lse.permute(2, 0, 1).contiguous()
        all_gather_rows(l_t, n, qb, qe, group, rng)
        lse.copy_(l_t.permute(1, 2, 0))
    return out, lse, (qb, qe)


def geoattn_backward_sharded(Q, K, V, O, dO, lse, coords, spreads, mask=None, group=None, kernel=None, by="zh"):
    """Gradients ``(dQ, dK, dV, d_spreads)`` complete on every rank.  ``by="zh"``: every rank's (batch, head) pairs are
    gathered, ``d_spreads`` all-reduced.  ``by="query"``: a rank's query blocks give its dQ rows (gathered) and partial
    dK, dV, d_spreads (all-reduced).  ``kernel(Q, K, V, O, dO, lse, coords, spreads, mask, zh_begin, zh_end, q_begin,
    q_end)`` returns the four tensors with only its own ranges meaningful."""
    if kernel is None:
        from proteusai_b200.utils.model_utils.attn.geometric_attn import geoattn_backward

        def kernel(Q, K, V, O, dO, lse, coords, spreads, mask, b, e, qb, qe):
            return geoattn_backward(Q, K, V, O, dO, lse, coords, spreads, mask, b, e, q_begin=qb, q_end=qe)
    world, rank = _world(group)
    z, h, n = Q.shape[0], Q.shape[1], Q.shape[2]
    if by == "zh":
        b, e = shard_range(z * h, world, rank)
        dq, dk, dv, dsig = kernel(Q, K, V, O, dO, lse, coords, spreads, mask, b, e, 0, n)
        if world > 1:
            for t in (dq, dk, dv):
                all_gather_rows(t.view(z * h, -1), z * h, b, e, group)
            dist.all_reduce(dsig, op=dist.ReduceOp.SUM, group=group)
        return dq, dk, dv, dsig
    if by != "query":
        raise ValueError(f"by must be 'zh' or 'query', not {by!r}")
    qb, qe = query_shard_range(n, world, rank)
    dq, dk, dv, dsig = kernel(Q, K, V, O, dO, lse, coords, spreads, mask, 0, z * h, qb, qe)
    if world > 1:
        t = dq.permute(2, 0, 1, 3).contiguous()
        all_gather_rows(t, n, qb, qe, group, lambda r: query_shard_range(n, world, r))
        dq.copy_(t.permute(1, 2, 0, 3))
        for g in (dk, dv, dsig):
            dist.all_reduce(g, op=dist.ReduceOp.SUM, group=group)
    return dq, dk, dv, dsig
