"""Rank program of tests/test_sharding_nccl_gpu.py (launched by torch.distributed.run, one rank per GPU, NCCL):
the sharded calls of proteusai_b200.sharding on real kernels against the same calls on one GPU."""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    from oracle import chains
    from proteusai_b200 import _lib, sharding
    from proteusai_b200.utils.model_utils.attn.geometric_attn import geoattn_backward, geoattn_forward
    from proteusai_b200.utils.model_utils.wf_embedding.isotropic.cuda.wf_embedding import we_backward_dk, we_forward_rows
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rel = lambda a, b: (torch.linalg.vector_norm((a - b).double()) / torch.linalg.vector_norm(b.double())).item()

    # Wavefunction Embedding: observer rows sharded, output all-gathered, dk all-reduced
    for z, n, lengths in ((1, 2048, [2048]), (3, 520, [520, 300, 77])):
        c, m = chains.chain_batch(lengths, n, seed=n)
        c, m = torch.from_numpy(c).to(dev), torch.from_numpy(m).to(dev)
        wn = torch.from_numpy(chains.wavenumbers(64)).to(dev)
        out, cs, sn, rows = sharding.we_forward_sharded(c, wn, 1, m)
        full, fcs, fsn = we_forward_rows(c, wn, 1, m)
        assert rel(out, full) < 1e-5, ("we", z, n, rel(out, full))
        d_out = torch.randn(out.shape, generator=torch.Generator().manual_seed(1)).to(dev)
        dk = sharding.we_backward_dk_sharded(d_out, cs, sn, rows)
        assert rel(dk, we_backward_dk(d_out, fcs, fsn)) < 1e-4

    # geometric attention: by (batch, head) pairs and by query blocks
    z, h, n = 2, 3, 700
    g = torch.Generator().manual_seed(11)
    q, k, v, d_o = ((torch.randn(z, h, n, 64, generator=g)).to(torch.bfloat16).to(dev) for _ in range(4))
    c, m = chains.chain_batch([700, 410], n, seed=12)
    c, m = torch.from_numpy(c).to(dev), torch.from_numpy(m).to(dev)
    sig = torch.from_numpy(chains.sigmas(h)).to(dev)
    o_1, l_1 = geoattn_forward(q, k, v, c, sig, m)
    dq_1, dk_1, dv_1, ds_1 = geoattn_backward(q, k, v, o_1, d_o, l_1, c, sig, m)
    live = ~m[:, None, :].expand(z, h, n)
    for by in ("zh", "query"):
        o, l, _ = sharding.geoattn_forward_sharded(q, k, v, c, sig, m, by=by)
        assert torch.equal(o, o_1) and torch.equal(l[live], l_1[live]), by
        dq, dk, dv, ds = sharding.geoattn_backward_sharded(q, k, v, o, d_o, l, c, sig, m, by=by)
        scale = max(t.abs().max().item() for t in (dq_1, dk_1, dv_1))
        for got, ref in ((dq, dq_1), (dk, dk_1), (dv, dv_1)):
            assert (got - ref).abs().max().item() < 1e-4 * scale, by   # fp32 reductions in another order
        assert torch.allclose(ds, ds_1, rtol=1e-3, atol=1e-4), by
    _lib.device_status()
    dist.barrier()
    if rank == 0:
        print("nccl sharded ok", world)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
