"""Sharding of the two hot paths across the GPUs of one node (one process per GPU).

Both paths partition without any exchange during the computation:

* Wavefunction Embedding: every rank holds all coordinates (a few hundred kB) and computes a contiguous
  range of observer rows; the output is reassembled with one all-gather; the wavenumber gradient is a
  local reduction followed by an all-reduce of ``[K]`` floats.
* Geometric attention: every rank computes a contiguous range of (batch, head) pairs; outputs are
  reassembled with one all-gather, the spread gradient with an all-reduce of ``[H]`` floats.

The compute callables are parameters so that the partition / gather logic can be exercised on CPU
ranks (gloo) with a stand-in kernel; on GPUs the defaults are the CUDA entry points.
"""
import torch
import torch.distributed as dist


def shard_range(total, world, rank):
    """Contiguous range ``[begin, end)`` of ``total`` items owned by ``rank`` (sizes differ by at most one block)."""
    per = (total + world - 1) // world
    return min(total, rank * per), min(total, (rank + 1) * per)


def _world(group):
    if not (dist.is_available() and dist.is_initialized()):
        return 1, 0
    return dist.get_world_size(group), dist.get_rank(group)


def all_gather_rows(full, dim_total, begin, end, group=None):
    """``full`` is a contiguous tensor whose leading dimension has ``dim_total`` items of which this rank
    has filled ``[begin, end)``; afterwards every rank holds all of it.  In place when the split is even."""
    world, rank = _world(group)
    if world == 1:
        return full
    per = (dim_total + world - 1) // world
    flat = full.view(dim_total, -1)
    if dim_total % world == 0:
        dist.all_gather_into_tensor(flat, flat[begin:end], group=group)
    else:
        parts = [torch.empty_like(flat[:per]) for _ in range(world)]
        mine = torch.zeros_like(flat[:per])
        mine[:end - begin] = flat[begin:end]
        dist.all_gather(parts, mine, group=group)
        for r in range(world):
            b, e = shard_range(dim_total, world, r)
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


def geoattn_forward_sharded(Q, K, V, coords, spreads, mask=None, group=None, kernel=None):
    """Forward with (batch, head) pairs sharded over the ranks.  Returns ``(O, L, (zh_begin, zh_end))`` with
    ``O`` and ``L`` complete on every rank."""
    if kernel is None:
        from proteusai_b200.utils.model_utils.attn.geometric_attn import geoattn_forward as kernel
    world, rank = _world(group)
    z, h = Q.shape[0], Q.shape[1]
    b, e = shard_range(z * h, world, rank)
    out, lse = kernel(Q, K, V, coords, spreads, mask, b, e)
    if world > 1:
        all_gather_rows(out.view(z * h, -1), z * h, b, e, group)
        all_gather_rows(lse.view(z * h, -1), z * h, b, e, group)
    return out, lse, (b, e)
