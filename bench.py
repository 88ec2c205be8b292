#!/usr/bin/env python
"""Benchmark of the Wavefunction Embedding forward on the long-sequence configuration
(one random-walk chain, N = 16384, d_model = 512, fp32), the configuration the headline
metric "pair.wavenumber evaluations per second" is quoted on.

    python bench.py --gpus 1 --steps 10 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 ... bench.py --gpus 8 ...
    python bench.py --impl reference          # the reference's CPU formulation on the host cores

One step = one forward over all N observers.  With G ranks the observer rows are sharded
(coordinates replicated) and the output is reassembled with one NCCL all-gather, so the total
work is fixed ("strong" scaling).  Rank 0 prints one JSON line.
"""
import argparse
import json
import os
import statistics
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

N_SEQ, D_MODEL, SEED = 16384, 512, 1004
K_WN = D_MODEL // 2
EVALS_PER_STEP = N_SEQ * (N_SEQ - 1) * K_WN  # observer i, source j != i, wavenumber k
H100_PUBLISHED_EVALS_PER_S = 16384 * 16383 * 256 / 0.386  # reference README.md:34, 386 ms on an H100


def set_sequence_length(n):
    """Profiling aid: a shorter chain of the same kind (the headline workload is N = 16384)."""
    global N_SEQ, EVALS_PER_STEP
    N_SEQ = n
    EVALS_PER_STEP = N_SEQ * (N_SEQ - 1) * K_WN

SFU_NOMINAL_PAIRS_PER_CLK_SM = 8.0  # 16 SFU results per clock per SM = 8 sin+cos pairs
# With a share of the evaluations moved to FMA-pipe polynomials both pipes can be busy at once: 8 evaluations per clock
# on the SFU plus what the fp32 pipe has left after the 5 operations every evaluation costs it, about 12.2 per clock per SM.
BALANCED_PIPE_PAIRS_PER_CLK_SM = 12.2
# DRAM bytes per launch of the HBM-bound kernels, from one ncu capture each (dram__bytes_read.sum + dram__bytes_write.sum;
# profiles/edge_rbf_n16384_ncu_full.md, profiles/encoder_row_kernels_dram.md): writes still in L2 when the launch ends are
# not counted by the counter, so traffic sits a little below the algorithmic bytes; no re-reads in any of them.
NCU_TRAFFIC_BYTES = {"edge_rbf_4x4x16_kernel": 445.1e6 + 4.9e6, "add_layernorm_bf16_kernel": 134.2e6 + 40.3e6,
                     "gelu_bf16_kernel": 268.4e6 + 205.7e6}


def hbm_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json, copy bandwidth)"
    except Exception:  # noqa: BLE001
        return 6650.0, "fallback (earlier measurement on this pool)"


def device_ms(fn, steps, warmup=3, flush=None):
    """Mean device time of ``fn`` over ``steps`` calls (CUDA events on the current stream, L2 flushed between calls
    when ``flush`` is given)."""
    for _ in range(warmup):
        fn()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    torch.cuda.synchronize()
    for a, b in evs:
        if flush is not None:
            flush.zero_()
        a.record()
        fn()
        b.record()
    torch.cuda.synchronize()
    return sum(a.elapsed_time(b) for a, b in evs) / steps


def workload():
    from proteusai_b200 import synthetic as chains
    coords, _ = chains.chain_batch([N_SEQ], N_SEQ, seed=SEED)
    return torch.from_numpy(coords), torch.from_numpy(chains.wavenumbers(D_MODEL))


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed region runs."""

    def __init__(self, device_index):
        super().__init__(daemon=True)
        self.samples, self.reasons, self.max_mhz, self._stop_evt = [], set(), None, threading.Event()
        self.err = None
        try:
            import pynvml
            self.nv = pynvml
            pynvml.nvmlInit()
            uuid = str(torch.cuda.get_device_properties(device_index).uuid)
            uuid = uuid if uuid.startswith("GPU-") else "GPU-" + uuid
            self.h = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception as exc:  # noqa: BLE001
            self.err = repr(exc)
            self.nv = None

    def run(self):
        if self.nv is None:
            return
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._stop_evt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    bits = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except AttributeError:
                    bits = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if bits & bit:
                        self.reasons.add(name)
            except Exception as exc:  # noqa: BLE001
                self.err = repr(exc)
                return
            time.sleep(0.02)

    def stop(self):
        self._stop_evt.set()
        self.join(timeout=2.0)
        out = {"sm_mhz": statistics.median(self.samples) if self.samples else None,
               "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}
        if self.err:
            out["error"] = self.err
        return out


GA_Z, GA_H, GA_N, GA_D, GA_SEED = 8, 8, 1024, 64, 1003


def geoattn_workload():
    """Config: B=8, H=8, N=1024, d_head=64, bf16; Q,K,V ~ N(0,1)/sqrt(d); random-walk chains with lengths
    uniform in 256..1024 (key-padding mask); sigma_h linear 3..15 A; upstream gradient N(0,1)."""
    from proteusai_b200 import synthetic as chains
    lengths = chains.draw_lengths(GA_Z, 256, 1024, seed=GA_SEED)
    coords, mask = chains.chain_batch(lengths, GA_N, seed=GA_SEED)
    g = torch.Generator().manual_seed(GA_SEED)
    q, k, v = (torch.randn(GA_Z, GA_H, GA_N, GA_D, generator=g) / GA_D ** 0.5 for _ in range(3))
    d_out = torch.randn(GA_Z, GA_H, GA_N, GA_D, generator=g)
    q, k, v, d_out = (t.to(torch.bfloat16) for t in (q, k, v, d_out))
    return q, k, v, d_out, torch.from_numpy(coords), torch.from_numpy(mask), torch.from_numpy(chains.sigmas(GA_H)), lengths


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            pk = json.load(f)
        return float(pk["bf16_tflops"]), "measured (MEASURED_PEAKS.json, cuBLAS bf16 burst)"
    except Exception:  # noqa: BLE001
        return 1590.0, "fallback (earlier measurement on this pool)"


def geoattn_cpu_baseline(q, k, v, d_out, coords, mask, sig, lengths):
    """The oracle (restated `torch_attn`, fp32, autograd backward) on the host cores, on ONE sample of the batch (the
    dense formulation holds several [H, N, N] fp32 tensors per sample).  Returns a cpu_baseline dict in TFLOP/s on the
    valid pairs of that sample."""
    from oracle.geoattn_ref import geoattn_grads_autograd
    torch.set_num_threads(os.cpu_count() or 1)
    b = int(np.argmax(lengths))
    sl = slice(b, b + 1)
    args = (q[sl].float(), k[sl].float(), v[sl].float(), coords[sl], sig, d_out[sl].float(), mask[sl])
    geoattn_grads_autograd(*args)  # warm-up
    t0 = time.perf_counter()
    reps = 0
    while reps < 3 or time.perf_counter() - t0 < 8.0:
        geoattn_grads_autograd(*args)
        reps += 1
        if time.perf_counter() - t0 > 20.0:
            break
    dt = (time.perf_counter() - t0) / reps
    flop = 14.0 * GA_H * GA_D * float(lengths[b]) ** 2
    return {"value": flop / dt / 1e12, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"sample {b} of the batch (length {int(lengths[b])}, all 8 heads), forward + autograd backward, "
                      f"{reps} repetitions of {dt:.2f} s"}


def bench_geoattn(dev, world, rank, steps, dist, cpu_baseline=False):
    """Geometric attention forward+backward, (batch, head) pairs sharded over the ranks.
    Returns a dict for the JSON line (rank 0) with TFLOP/s on the valid pairs and on the padded shape."""
    from proteusai_b200.utils.model_utils.attn.geometric_attn import geoattn_backward, geoattn_forward
    q, k, v, d_out, coords, mask, sig, lengths = geoattn_workload()
    host = (q, k, v, d_out, coords, mask, sig)
    q, k, v, d_out, coords, mask, sig = (t.to(dev) for t in (q, k, v, d_out, coords, mask, sig))
    from proteusai_b200 import sharding
    z0, z1 = sharding.shard_range(GA_Z * GA_H, world, rank)
    out = torch.empty(GA_Z, GA_H, GA_N, GA_D, dtype=torch.bfloat16, device=dev)
    lse = torch.empty(GA_Z, GA_H, GA_N, dtype=torch.float32, device=dev)

    def step():
        geoattn_forward(q, k, v, coords, sig, mask, z0, z1, out, lse)
        geoattn_backward(q, k, v, out, d_out, lse, coords, sig, mask, z0, z1)

    for _ in range(3):
        step()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    for a, b in evs:
        a.record()
        step()
        b.record()
    torch.cuda.synchronize()
    total = sum(a.elapsed_time(b) for a, b in evs)
    fa, fb = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    fa.record()
    for _ in range(steps):
        geoattn_forward(q, k, v, coords, sig, mask, z0, z1, out, lse)
    fb.record()
    torch.cuda.synchronize()
    fwd_ms = fa.elapsed_time(fb) / steps
    if world > 1:
        t = torch.tensor([total], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total = float(t.item())
    ms = total / steps
    valid_flop = 14.0 * GA_H * GA_D * float((lengths.astype(np.float64) ** 2).sum())
    padded_flop = 14.0 * GA_Z * GA_H * GA_N * GA_N * GA_D
    # Outside the timed region: reassemble O over the ranks once (NCCL all-gather) and check rows that ANOTHER rank
    # computed against the CPU oracle, so that a wrong offset in the gather cannot pass unnoticed.
    gather_check = None
    if world > 1:
        from oracle.geoattn_ref import geoattn_ref
        o_all, _, _ = sharding.geoattn_forward_sharded(q, k, v, coords, sig, mask)
        zh = ((rank + 1) % world) * ((GA_Z * GA_H + world - 1) // world)  # first pair of the next rank's shard
        zc, hc = zh // GA_H, zh % GA_H
        hq, hk, hv, _, hcoords, hmask, hsig = host
        ref = geoattn_ref(hq[zc:zc + 1, hc:hc + 1].float(), hk[zc:zc + 1, hc:hc + 1].float(), hv[zc:zc + 1, hc:hc + 1].float(),
                          hcoords[zc:zc + 1], hsig[hc:hc + 1], mask=hmask[zc:zc + 1])
        err = torch.tensor([(o_all[zc, hc].float().cpu() - ref[0, 0]).abs().max().item()], device=dev, dtype=torch.float64)
        dist.all_reduce(err, op=dist.ReduceOp.MAX)
        gather_check = float(err.item())
    peak, src = measured_peaks()
    res = {"metric": "geo-attn fwd+bwd TFLOP/s (valid pairs)", "value": valid_flop / (ms * 1e-3) / 1e12, "unit": "TFLOP/s",
           "padded_tflops": padded_flop / (ms * 1e-3) / 1e12, "ms_per_step": ms, "fwd_ms": fwd_ms, "dtype": "bf16",
           "config": {"workload": "geometric attention fwd+bwd, B=8, H=8, N=1024, d_head=64, lengths U{256..1024}, seed 1003",
                      "sharding": f"(batch, head) pairs over {world} rank(s)",
                      "launch": ("persistent CTAs on the balanced schedule of the mask (made once, outside the timed region)" if world == 1
                                 else "one CTA per work item, samples longest first (a shard of the pairs runs without a schedule)")},
           "roofline": {"bound": "tensor", "achieved": valid_flop / (ms * 1e-3) / 1e12, "peak": peak, "unit": "TFLOP/s",
                        "frac": valid_flop / (ms * 1e-3) / 1e12 / peak, "peak_source": src, "traffic": None,
                        "note": "compute-bound kernels: DRAM traffic (about 0.1 GB per step) is not the limiter",
                        # every valid pair costs two ex2 in the forward and three in the backward on the SFU (16 results per
                        # clock per SM): the floor of the step if nothing else took time (far key groups skip some of them)
                        "sfu_floor_ms": 5.0 * GA_H * float((lengths.astype(np.float64) ** 2).sum()) /
                                        (16.0 * torch.cuda.get_device_properties(dev).multi_processor_count * 1.965e9) * 1e3 / world,
                        "frac_of_sfu_floor": 5.0 * GA_H * float((lengths.astype(np.float64) ** 2).sum()) /
                                             (16.0 * torch.cuda.get_device_properties(dev).multi_processor_count * 1.965e9) * 1e3 / world / ms},
           "gather_check_max_abs": gather_check,
           "gpu_launches": 3 * steps}
    if cpu_baseline and rank == 0:
        res["cpu_baseline"] = geoattn_cpu_baseline(*host, lengths)
    return res


EN_Z, EN_N, EN_SEED = 64, 1024, 1005


def encoder_cpu_baseline(model, lengths):
    """The oracle composition of the same model (fp32 arithmetic on its weights, CPU restatements of both kernels) on the
    host cores, on a bounded sample: one chain of the batch's median length, unpadded."""
    from oracle.encoder_ref import encoder_forward_ref
    from proteusai_b200 import synthetic as chains
    torch.set_num_threads(os.cpu_count() or 1)
    n = int(np.sort(lengths)[len(lengths) // 2])
    coords, mask = chains.chain_batch([n], n, seed=EN_SEED)
    tokens = torch.randint(0, 33, (1, n), generator=torch.Generator().manual_seed(EN_SEED))
    args = (model, tokens, torch.from_numpy(coords), torch.from_numpy(mask))
    with torch.no_grad():
        encoder_forward_ref(*args)  # warm-up
        t0 = time.perf_counter()
        reps = 0
        while reps < 2 or time.perf_counter() - t0 < 6.0:
            encoder_forward_ref(*args)
            reps += 1
            if time.perf_counter() - t0 > 20.0:
                break
    dt = (time.perf_counter() - t0) / reps
    return {"value": n / dt, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"one chain of {n} residues (the batch's median length), unpadded, {reps} repetitions of {dt:.2f} s"}


def bench_encoder(dev, world, rank, steps, dist, graphed=False, cpu_baseline=False):
    """Encoder inference (bf16, random weights): token embedding (vocabulary 33 -> 512) + wavefunction embedding, 4 post-norm
    layers of geometric attention (H=8, sigma 3..15 A) and a 2048-wide GELU FFN, linear head to 20 logits.  64 chains with
    lengths uniform in 64..1024 padded to 1024, data-parallel: each rank takes a contiguous slice of the batch.  Returns
    tokens/s over valid tokens (rank 0)."""
    from proteusai_b200 import synthetic as chains
    from proteusai_b200 import sharding
    from proteusai_b200.utils.model_utils.base_modules.encoder import ProteusEncoderModel
    lengths = chains.draw_lengths(EN_Z, 64, 1024, seed=EN_SEED)
    b0, b1 = sharding.shard_range(EN_Z, world, rank)
    coords, mask = chains.chain_batch(lengths[b0:b1], EN_N, seed=EN_SEED + 1 + rank)
    g = torch.Generator().manual_seed(EN_SEED)
    tokens = torch.randint(0, 33, (EN_Z, EN_N), generator=g)[b0:b1]
    torch.manual_seed(EN_SEED)
    model = ProteusEncoderModel(d_model=512, heads=8, layers=4, d_hidden=2048).to(dev).eval().to_compute_dtype_(torch.bfloat16)
    coords_p, mask_p, tokens_p = torch.from_numpy(coords).pin_memory(), torch.from_numpy(mask).pin_memory(), tokens.pin_memory()
    out_host = torch.empty(b1 - b0, EN_N, 20, dtype=torch.bfloat16).pin_memory()

    def step():
        c, m, t = (x.to(dev, non_blocking=True) for x in (coords_p, mask_p, tokens_p))
        with torch.no_grad():
            logits = model(t, c, m)
        out_host.copy_(logits, non_blocking=True)

    for _ in range(3):
        step()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    for a, b in evs:
        a.record()
        step()
        b.record()
    torch.cuda.synchronize()
    total = sum(a.elapsed_time(b) for a, b in evs)
    if world > 1:
        t = torch.tensor([total], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total = float(t.item())
    ms = total / steps
    valid_tokens = int(lengths.sum())
    res = {"metric": "encoder inference tokens/s (valid tokens, host inputs and outputs included)", "value": valid_tokens / (ms * 1e-3),
           "unit": "tokens/s", "padded_tokens_per_s": EN_Z * EN_N / (ms * 1e-3), "ms_per_step": ms, "dtype": "bf16",
           "config": {"workload": "4-layer geometric-attention encoder, d_model 512, H 8, FFN 2048, 64 chains of 64..1024 padded to 1024, seed 1005",
                      "sharding": f"batch over {world} rank(s), no collective"},
           "e2e": {"value": valid_tokens / (ms * 1e-3), "unit": "tokens/s",
                   "h2d_bytes_per_step": int(coords_p.numel() * 4 + mask_p.numel() + tokens_p.numel() * 8) * world,
                   "d2h_bytes_per_step": int(out_host.numel() * 2) * world}}
    if world == 1:
        # the two HBM-bound row kernels of the block, timed alone on this batch's shapes, with their ncu DRAM traffic
        from proteusai_b200.utils.model_utils.base_modules import fused_ops
        rows = (b1 - b0) * EN_N
        x = torch.randn(rows, 512, device=dev).to(torch.bfloat16)
        w = torch.ones(512, device=dev, dtype=torch.bfloat16)
        hbuf = torch.randn(rows, 2048, device=dev).to(torch.bfloat16)
        ln_ms = device_ms(lambda: fused_ops.add_layernorm(x, x, w, w, 1e-5), steps)
        ge_ms = device_ms(lambda: fused_ops.gelu(hbuf, inplace=True), steps)
        peak, src = hbm_peak()
        ln_bytes, ge_bytes = rows * 512 * 2 * 3, rows * 2048 * 2 * 2
        res["row_kernels"] = [
            {"kernel": "add_layernorm_bf16_kernel", "ms": ln_ms, "roofline": {
                "bound": "hbm", "achieved": ln_bytes / (ln_ms * 1e-3) / 1e9, "peak": peak, "unit": "GB/s", "peak_source": src,
                "frac": ln_bytes / (ln_ms * 1e-3) / 1e9 / peak, "traffic": NCU_TRAFFIC_BYTES["add_layernorm_bf16_kernel"] * rows / 65536}},
            {"kernel": "gelu_bf16_kernel", "ms": ge_ms, "roofline": {
                "bound": "hbm", "achieved": ge_bytes / (ge_ms * 1e-3) / 1e9, "peak": peak, "unit": "GB/s", "peak_source": src,
                "frac": ge_bytes / (ge_ms * 1e-3) / 1e9 / peak, "traffic": NCU_TRAFFIC_BYTES["gelu_bf16_kernel"] * rows / 65536}}]
    if cpu_baseline and rank == 0:
        res["cpu_baseline"] = encoder_cpu_baseline(model.float().cpu(), lengths)
        model.to(dev).to_compute_dtype_(torch.bfloat16)
    if graphed:
        # The same forward captured once into a CUDA graph and replayed: inputs are copied into static device buffers,
        # the graph runs, the logits are copied out.  Removes the host's per-kernel launch work from the step.
        c_s, m_s, t_s = (x.to(dev) for x in (coords_p, mask_p, tokens_p))
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side), torch.no_grad():
            for _ in range(3):
                model(t_s, c_s, m_s)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph), torch.no_grad():
            logits_s = model(t_s, c_s, m_s)

        def step_graph():
            c_s.copy_(coords_p, non_blocking=True)
            m_s.copy_(mask_p, non_blocking=True)
            t_s.copy_(tokens_p, non_blocking=True)
            graph.replay()
            out_host.copy_(logits_s, non_blocking=True)

        ref_logits = out_host.clone()
        for _ in range(3):
            step_graph()
        torch.cuda.synchronize()
        # (not bit-equal in general: with a padding mask the WE kernel adds its partial sums in a run-dependent order)
        diff = float((ref_logits.float() - out_host.float()).abs().max())
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            step_graph()
        b.record()
        torch.cuda.synchronize()
        res["cuda_graph"] = {"ms_per_step": a.elapsed_time(b) / steps, "max_abs_diff_vs_eager": diff}
    return res


def bench_graph(dev, steps, cpu_baseline):
    """Neighbour graph (K = 30) and radial-basis edge features (4 x 4 atom pairs x 16 centres) of one chain of
    N = 16384 nodes, the step after the WE in the reference's featuriser.  One GPU (rank 0): the reference
    runs this per sample; nothing to shard inside one chain.  The edge-feature kernel is HBM-write bound (1 kB per edge)."""
    from proteusai_b200 import synthetic as chains
    from proteusai_b200.utils.model_utils.gnn.gnn import edge_rbf, knn_neighbors
    n, k = 16384, 30
    c, _ = chains.chain_batch([n], n, seed=SEED)
    rng = np.random.default_rng(SEED)
    off = rng.normal(size=(1, n, 4, 3))
    off /= np.linalg.norm(off, axis=3, keepdims=True)
    off *= np.array([1.46, 0.0, 1.52, 1.53])[None, None, :, None]
    atoms_h = torch.from_numpy((c[:, :, None, :] + off).astype(np.float32))
    atoms = atoms_h.to(dev)
    ca = atoms[:, :, 1].contiguous()
    centers = torch.linspace(2.0, 22.0, 16, device=dev)
    spread = 20.0 / 16

    def timed_ms(fn):
        for _ in range(3):
            fn()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        for _ in range(steps):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / steps

    idx, _ = knn_neighbors(ca, None, k)
    knn_ms = timed_ms(lambda: knn_neighbors(ca, None, k))
    rbf_ms = timed_ms(lambda: edge_rbf(atoms, idx, centers, spread))  # 503 MB written per call: larger than L2
    ln = torch.nn.LayerNorm(256).to(dev)
    rbf_ln_ms = timed_ms(lambda: edge_rbf(atoms, idx, centers, spread, norm=ln))  # with the edge LayerNorm fused in
    edges = n * k
    out_bytes = edges * 256 * 4
    hbm = None
    try:
        hbm = float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["hbm_gbs"])
    except Exception:
        pass
    peak, src = (hbm, "measured (MEASURED_PEAKS.json, copy bandwidth)") if hbm else (6650.0, "fallback")
    res = {"metric": "graph featurisation nodes/s (K nearest + edge RBFs)", "value": n / ((knn_ms + rbf_ms) * 1e-3), "unit": "nodes/s",
           "knn_ms": knn_ms, "edge_rbf_ms": rbf_ms, "edge_rbf_layernorm_ms": rbf_ln_ms, "dtype": "f32",
           "config": {"workload": f"one chain, N={n}, K={k}, 4 atoms per node, 16 RBF centres, seed {SEED}", "sharding": "rank 0 only"},
           "roofline": {"bound": "hbm", "kernel": "edge_rbf_4x4x16_kernel", "achieved": out_bytes / (rbf_ms * 1e-3) / 1e9, "peak": peak,
                        "unit": "GB/s", "frac": out_bytes / (rbf_ms * 1e-3) / 1e9 / peak, "peak_source": src,
                        "traffic": NCU_TRAFFIC_BYTES["edge_rbf_4x4x16_kernel"]},
           "gpu_launches": 2 * steps}
    if cpu_baseline:
        from oracle.gnn_ref import edge_rbf_ref, get_neighbors_ref
        torch.set_num_threads(os.cpu_count() or 1)
        ns = 2048  # the dense formulation needs N^2 memory: a bounded sample of the same chain
        a_s = atoms_h[:, :ns]
        t0 = time.perf_counter()
        i_s, _ = get_neighbors_ref(a_s[:, :, 1], torch.zeros(1, ns, dtype=torch.bool), k)
        edge_rbf_ref(a_s, i_s, centers.cpu(), spread)
        dt = time.perf_counter() - t0
        res["cpu_baseline"] = {"value": ns / dt, "unit": "nodes/s", "cores": torch.get_num_threads(), "kind": "port",
                               "sample": f"first {ns} nodes of the chain as a chain of their own (dense N x N formulation), {dt:.2f} s"}
    return res


def bench_we_aniso(dev, steps, sfu_rate, nominal, flush):
    """Anisotropic WE (per-wavenumber C-beta scaling, the variant the reference's model calls) forward at the headline
    shape: one chain, N = 16384, 256 wavenumbers.  SFU-bound like the isotropic kernel: one sin + one cos per evaluation."""
    from proteusai_b200.utils.model_utils.wf_embedding.anisotropic.cb_scaling.learnable_wavenumbers.cuda.wf_embedding import \
        we_aniso_forward_rows
    coords_h, wn_h = workload()
    g = torch.Generator().manual_seed(SEED)
    cb = torch.randn(coords_h.shape, generator=g)
    cb = (cb / torch.linalg.vector_norm(cb, dim=2, keepdim=True)).to(dev)
    cbm = torch.rand(wn_h.shape, generator=g).to(dev)
    c, wn = coords_h.to(dev), wn_h.to(dev)
    ms = device_ms(lambda: we_aniso_forward_rows(c, cb, cbm, wn, None, 0, N_SEQ), steps, flush=flush)
    achieved = EVALS_PER_STEP / (ms * 1e-3)
    return {"metric": f"anisotropic WE pair*wavenumber evals/s @N={N_SEQ},d=512", "value": achieved, "unit": "evals/s", "ms_per_step": ms,
            "dtype": "f32", "config": {"workload": f"anisotropic (C-beta scaling) WE forward, Z=1, N={N_SEQ}, 256 wavenumbers, seed {SEED}",
                                       "sharding": "rank 0 only"},
            "roofline": {"bound": "sfu", "kernel": "we_aniso_fwd_kernel", "achieved": achieved / 1e9, "peak": nominal / 1e9,
                         "unit": "Geval/s", "frac": achieved / nominal, "peak_source": "nominal: 8 sin+cos pairs per clock per SM at the maximum SM clock",
                         "peak_measured": sfu_rate / 1e9, "frac_of_measured": achieved / sfu_rate, "traffic": None},
            "gpu_launches": steps}


def bench_we_bwd(dev, steps, flush):
    """WE backward (wavenumber gradient from the stored sums) at Z = 8, N = 16384, K = 256: 16 bytes read per (z, n, k),
    537 MB per call, HBM-bound."""
    from proteusai_b200.utils.model_utils.wf_embedding.isotropic.cuda.wf_embedding import we_backward_dk
    z, n, k = 8, 16384, K_WN
    g = torch.Generator(device=dev).manual_seed(SEED)
    d_out = torch.randn(z, n, 2 * k, device=dev, generator=g)
    cs, sn = torch.randn(z, n, k, device=dev, generator=g), torch.randn(z, n, k, device=dev, generator=g)
    ms = device_ms(lambda: we_backward_dk(d_out, cs, sn), steps, flush=flush)
    nbytes = z * n * k * 16
    peak, src = hbm_peak()
    return {"metric": "WE backward (z,n,k) triples/s @Z=8,N=16384,K=256", "value": z * n * k / (ms * 1e-3), "unit": "triples/s",
            "ms_per_step": ms, "dtype": "f32",
            "config": {"workload": "WE backward dk, Z=8, N=16384, K=256, N(0,1) inputs", "sharding": "rank 0 only",
                       "l2": "flushed between timed calls; inputs 537 MB"},
            "roofline": {"bound": "hbm", "kernel": "we_bwd_partial2_kernel + we_bwd_final_kernel", "achieved": nbytes / (ms * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                         "frac": nbytes / (ms * 1e-3) / 1e9 / peak, "peak_source": src, "traffic": None,
                         "note": "through the public call: the two kernels plus the workspace allocation"},
            "gpu_launches": 2 * steps}


def cpu_port_rate(coords, wn, target_s=12.0, chunk=32):
    """Times the oracle (the reference's dense PyTorch formulation, observer-chunked) on the host
    cores on a bounded run of observer rows.  Returns (evals/s, rows used, seconds)."""
    from oracle.we_ref import wf_embedding_ref
    torch.set_num_threads(os.cpu_count() or 1)
    n = coords.shape[1]
    start = n // 2
    wf_embedding_ref(coords, wn, 1, rows=(start, start + chunk), chunk=chunk)  # warm-up
    t0 = time.perf_counter()
    wf_embedding_ref(coords, wn, 1, rows=(start, start + chunk), chunk=chunk)
    per_chunk = time.perf_counter() - t0
    chunks = int(max(1, min(64, target_s / max(per_chunk, 1e-3))))
    rows = chunks * chunk
    t0 = time.perf_counter()
    wf_embedding_ref(coords, wn, 1, rows=(start, start + rows), chunk=chunk)
    dt = time.perf_counter() - t0
    return rows * (n - 1) * wn.shape[0] / dt, rows, dt


def run_reference(args):
    """The reference arm: the reference's own CPU path for this metric is its dense PyTorch
    formulation; its restatement in oracle/ is timed on all host cores.  Each step is a bounded
    run of observer rows of the same workload."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    coords, wn = workload()
    from oracle.we_ref import wf_embedding_ref
    torch.set_num_threads(os.cpu_count() or 1)
    chunk, rows = 32, 64
    start = N_SEQ // 2
    for _ in range(max(1, min(args.warmup, 2))):
        wf_embedding_ref(coords, wn, 1, rows=(start, start + chunk), chunk=chunk)
    times = []
    for _ in range(args.steps):
        t0 = time.perf_counter()
        wf_embedding_ref(coords, wn, 1, rows=(start, start + rows), chunk=chunk)
        times.append(time.perf_counter() - t0)
    evals = rows * (N_SEQ - 1) * K_WN
    value = evals * len(times) / sum(times)
    line = {
        "impl": "reference", "metric": f"WE pair*wavenumber evals/s @N={N_SEQ},d=512", "value": value, "unit": "evals/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * EVALS_PER_STEP / value, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "WE forward, Z=1, N=16384, d_model=512, random-walk chain, seed 1004",
                   "note": "ms_per_step is the full workload extrapolated from the sample"},
        "cpu_baseline": {"value": value, "unit": "evals/s", "cores": torch.get_num_threads(), "kind": "port",
                         "sample": f"{rows} of {N_SEQ} observer rows x all sources x {K_WN} wavenumbers per step"},
        "e2e": {"value": value, "unit": "evals/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--geoattn", action="store_true", help="also run the attention leg when --n-seq is not the default")
    ap.add_argument("--graph-encoder", action="store_true",
                    help="also time the encoder leg with its forward captured in a CUDA graph (off by default)")
    ap.add_argument("--n-seq", type=int, default=N_SEQ, help="sequence length (default: the headline 16384)")
    args = ap.parse_args()
    if args.n_seq != N_SEQ:
        set_sequence_length(args.n_seq)
    if args.impl == "reference":
        return run_reference(args)

    import torch.distributed as dist
    from proteusai_b200 import _lib
    from proteusai_b200.utils.model_utils.wf_embedding.isotropic.cuda.wf_embedding import we_forward_rows, wf_embedding

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    _lib.lib()  # fail loudly if the native library is missing
    warmup = max(args.warmup, 3)

    coords_h, wn_h = workload()
    coords_pin, wn_pin = coords_h.pin_memory(), wn_h.pin_memory()
    coords_d, wn_d = coords_h.to(dev), wn_h.to(dev)
    from proteusai_b200 import sharding
    r0, r1 = sharding.shard_range(N_SEQ, world, rank)
    out = torch.empty(1, N_SEQ, 2 * K_WN, device=dev)
    cs = torch.empty(1, N_SEQ, K_WN, device=dev)
    sn = torch.empty(1, N_SEQ, K_WN, device=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)  # > 126 MB L2
    out_host = torch.empty(max(r1 - r0, 1), 2 * K_WN).pin_memory()

    def step_resident():
        we_forward_rows(coords_d, wn_d, 1, None, r0, r1, out, cs, sn)
        sharding.all_gather_rows(out[0], N_SEQ, r0, r1)

    def step_e2e():
        c = coords_pin.to(dev, non_blocking=True)
        w = wn_pin.to(dev, non_blocking=True)
        if world == 1:
            o = wf_embedding(c, w, 1, 0.0, None)  # the public call
            out_host.copy_(o[0], non_blocking=True)
        else:
            we_forward_rows(c, w, 1, None, r0, r1, out, cs, sn)
            sharding.all_gather_rows(out[0], N_SEQ, r0, r1)
            out_host[:r1 - r0].copy_(out[0, r0:r1], non_blocking=True)
        torch.cuda.current_stream().synchronize()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, use_events=True):
        """Sum of per-step device times (ms); L2 is flushed between steps outside the timed spans."""
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
        barrier()
        wall = 0.0
        for a, b in evs:
            flush.zero_()
            if use_events:
                a.record()
                fn()
                b.record()
            else:
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                fn()
                wall += (time.perf_counter() - t0) * 1e3
        barrier()
        total = sum(a.elapsed_time(b) for a, b in evs) if use_events else wall
        if world > 1:
            t = torch.tensor([total], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            total = float(t.item())
        return total

    for _ in range(warmup):
        step_resident()
    sampler = ClockSampler(local)
    sampler.start()
    total_ms = timed(step_resident, args.steps)
    clocks = sampler.stop()
    _lib.device_status()

    # kernel alone (no collective), for the roofline
    def kernel_only():
        we_forward_rows(coords_d, wn_d, 1, None, r0, r1, out, cs, sn)
    kern_ms = timed(kernel_only, args.steps) / args.steps
    for _ in range(2):
        step_e2e()
    e2e_ms = timed(step_e2e, args.steps, use_events=False)

    # Outside the timed region: rows that ANOTHER rank computed, as they arrived through the all-gather, against the CPU
    # oracle (64 rows from the middle of the next rank's shard); the largest error over the ranks goes into the line.
    gather_check = None
    if world > 1:
        from oracle.we_ref import rel_l2, wf_embedding_ref
        step_resident()
        o0, o1 = sharding.shard_range(N_SEQ, world, (rank + 1) % world)
        a = (o0 + o1) // 2
        ref = wf_embedding_ref(coords_h, wn_h, 1, rows=(a, a + 64), chunk=32)
        err = torch.tensor([rel_l2(ref, out[:, a:a + 64].cpu())], device=dev, dtype=torch.float64)
        dist.all_reduce(err, op=dist.ReduceOp.MAX)
        gather_check = float(err.item())

    value = EVALS_PER_STEP * args.steps / (total_ms * 1e-3)
    e2e_value = EVALS_PER_STEP * args.steps / (e2e_ms * 1e-3)
    line = None
    if rank == 0:
        sfu_rate, _ = _lib.measure_sfu_peak()
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        evals_per_launch = (r1 - r0) * (N_SEQ - 1) * K_WN
        achieved = evals_per_launch / (kern_ms * 1e-3)
        nominal = SFU_NOMINAL_PAIRS_PER_CLK_SM * sms * (clocks["sm_max_mhz"] or 1965) * 1e6
        balanced = BALANCED_PIPE_PAIRS_PER_CLK_SM * sms * (clocks["sm_max_mhz"] or 1965) * 1e6
        line = {
            "metric": f"WE pair*wavenumber evals/s @N={N_SEQ},d=512", "value": value, "unit": "evals/s",
            "n_gpus": world, "steps": args.steps, "warmup": warmup, "ms_per_step": total_ms / args.steps,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": value / H100_PUBLISHED_EVALS_PER_S if N_SEQ == 16384 else None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"WE forward, Z=1, N={N_SEQ}, d_model=512 (256 wavenumbers), random-walk chain, seed 1004",
                       "sharding": f"observer rows over {world} rank(s), coordinates replicated, NCCL all-gather of the output",
                       "l2": "flushed between timed steps (256 MB memset outside the timed spans)"},
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "evals/s",
                    "h2d_bytes_per_step": int(coords_pin.numel() * 4 + wn_pin.numel() * 4) * world,
                    "d2h_bytes_per_step": int(N_SEQ * 2 * K_WN * 4), "ms_per_step": e2e_ms / args.steps},
            "gpu_launches": args.steps,
            "gather_check": gather_check,
            "roofline": {"bound": "sfu", "achieved": achieved / 1e9, "peak": nominal / 1e9, "unit": "Geval/s",
                         "frac": achieved / nominal, "traffic": None,
                         "peak_source": "nominal: 16 SFU results = 8 sin+cos pairs per clock per SM x SMs x the maximum SM clock "
                                        "(MEASURED_PEAKS.json holds no SFU figure; HBM and tensor peaks do not bound this kernel)",
                         "peak_measured": sfu_rate / 1e9, "frac_of_measured": achieved / sfu_rate,
                         "peak_measured_source": "live: register-only sin+cos loop on this GPU (pai_measure_sfu_peak)",
                         "balanced_pipe_peak": balanced / 1e9, "frac_of_balanced": achieved / balanced,
                         "balanced_pipe_note": "bound with SFU and fp32 pipes both busy (12.2 evaluations per clock per SM): applies "
                                               "because two pairs in eight per lane are evaluated by an FMA-pipe polynomial",
                         "kernel": "we_fwd_kernel", "kernel_ms": kern_ms,
                         "evals_per_launch": evals_per_launch},
        }
        line["geoattn"] = None
        if world == 1 and not args.no_cpu_baseline:
            rate, rows, secs = cpu_port_rate(coords_h, wn_h)
            line["cpu_baseline"] = {"value": rate, "unit": "evals/s", "cores": torch.get_num_threads(), "kind": "port",
                                    "sample": f"{rows} of {N_SEQ} observer rows x all sources x {K_WN} wavenumbers, {secs:.1f} s"}
    ga = None
    full = N_SEQ == 16384 or args.geoattn
    want_cpu = world == 1 and not args.no_cpu_baseline
    if full:
        ga = bench_geoattn(dev, world, rank, max(args.steps, 20), dist, cpu_baseline=want_cpu)
    enc = None
    if full:
        enc = bench_encoder(dev, world, rank, args.steps, dist, graphed=args.graph_encoder, cpu_baseline=want_cpu)
    if rank == 0:
        line["geoattn"] = ga
        line["encoder"] = enc
        line["graph"] = bench_graph(dev, args.steps, want_cpu) if full else None
        if N_SEQ == 16384:
            del out, cs, sn
            line["we_aniso"] = bench_we_aniso(dev, args.steps, sfu_rate, nominal, flush)
            line["we_bwd"] = bench_we_bwd(dev, args.steps, flush)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
