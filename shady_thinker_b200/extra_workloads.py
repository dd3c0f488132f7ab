"""Benchmark bodies of BASELINE configs 1 and 5 (``bench.py --workload cfg1|cfg5``).

cfg1: single-layer decode in the reference's own format (fp32 q/k/v/out, batch 1, nh16/nkv2/hd128, context
512) — 1 MiB of KV, latency-bound: the figure is microseconds per append+attend step.
cfg5: full-depth batched decode step, attention only — 36 layers, each with its own fp16 KV cache, 32 sequences
of context 32768 per GPU (256 over 8 GPUs), nh32/nkv8/hd128; per layer one token per sequence is appended with
RoPE, then attended.  Layers are reduced (and reported) if the GPU has less free memory than 36 layers need.
"""
from __future__ import annotations

import json
import os

import numpy as np

SEED = 0x5EED


def _peak():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def _setup(world: int, local_rank: int):
    import torch
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()
    return torch, dist, barrier


def run_cfg1(args, rank: int, world: int, local_rank: int) -> None:
    """Replicas only (nothing to shard): every rank runs the same step; the line reports rank 0's latency."""
    torch, dist, barrier = _setup(world, local_rank)
    from . import ops
    from ._lib import F32
    from .gpu import GpuContext
    from .model import Model, ModelConfig
    L = 512
    stream = torch.cuda.Stream()
    gpu = GpuContext(local_rank, stream=stream.cuda_stream)
    cfg = ModelConfig(num_attention_heads=16, num_key_value_heads=2, head_dim=128, rope_theta=1e6,
                      partial_rotary_factor=1.0)
    with torch.cuda.stream(stream):
        m = Model(gpu, cfg, max_seq_len=L, kv_dtype=F32, num_attn_splits=0)
        nkv, hd, nh = 2, 128, 16
        ops.fill_randn(gpu, m.state.k_cache[0], L * nkv * hd, F32, SEED, 1)
        ops.fill_randn(gpu, m.state.v_cache[0], L * nkv * hd, F32, SEED, 2)
        ops.fill_randn(gpu, m.state.q_out, nh * hd * 2, F32, SEED, 3)
        ops.fill_randn(gpu, m.state.k_out, nkv * hd, F32, SEED, 4)
        ops.fill_randn(gpu, m.state.v_out, nkv * hd, F32, SEED, 5)
        m.seq_len = L - 1                      # the step appends row 511 and attends to 512 rows
        flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
        times = []
        for i in range(args.warmup + args.steps):
            flush.fill_(i & 0xFF)              # evict the 1 MiB cache from L2 between steps
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            m.fused_split_qknorm_kvstore(gpu, 0)
            m.gqa_attention(gpu, 0, fuse_gate=True)
            b.record(stream)
            gpu.synchronize()
            if i >= args.warmup:
                times.append(a.elapsed_time(b) * 1e3)
        # the same two launches replayed from a CUDA graph (captured on the context's stream): what the kernels cost
        # once the CPU's per-launch latency is out of the picture
        graph_us = None
        try:
            gpu.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                m.fused_split_qknorm_kvstore(gpu, 0)
                m.gqa_attention(gpu, 0, fuse_gate=True)
            gt = []
            for i in range(args.warmup + args.steps):
                flush.fill_(i & 0xFF)
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(stream)
                g.replay()
                b.record(stream)
                gpu.synchronize()
                if i >= args.warmup:
                    gt.append(a.elapsed_time(b) * 1e3)
            graph_us = float(np.median(gt))
        except Exception as e:      # capture is optional: the figure is informational
            graph_us = f"unavailable: {type(e).__name__}"
    barrier()
    if rank == 0:
        us = float(np.median(times))
        kv_bytes = 2 * L * nkv * hd * 4
        peak, src = _peak()
        print(json.dumps({
            "metric": "decode_step_latency", "value": us, "unit": "us", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": us / 1e3, "higher_is_better": False, "scaling": "replicas only",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "cfg1: single decode step, fp32 KV, batch 1, nh16/nkv2/hd128, context 512, full rotary",
                       "l2": "256 MB flush write between steps", "p10_us": float(np.percentile(times, 10)),
                       "p90_us": float(np.percentile(times, 90)), "includes": "position/length uploads, append, attend+gate",
                       "graph_replay_us": graph_us},
            "roofline": {"bound": "hbm", "achieved": kv_bytes / (us * 1e-6) / 1e9, "peak": peak, "unit": "GB/s",
                         "frac": kv_bytes / (us * 1e-6) / 1e9 / peak, "traffic": None,
                         "peak_source": f"{src} (copy bandwidth); informational: 1 MiB of KV is latency-bound"},
            "gpu_launches": 2 * args.steps}), flush=True)
    if dist is not None:
        dist.destroy_process_group()
    gpu.close()


def run_cfg5(args, rank: int, world: int, local_rank: int) -> None:
    torch, dist, barrier = _setup(world, local_rank)
    from . import ops
    from ._lib import F16
    from .batch import BatchedDecoder
    from .gpu import GpuContext
    S, Lctx, nh, nkv, hd, want_layers = 32, 32768, 32, 8, 128, 36
    layer_bytes = 2 * S * Lctx * nkv * hd * 2
    free, _total = torch.cuda.mem_get_info()
    layers = int(min(want_layers, (free * 0.92 - (2 << 30)) // layer_bytes))
    if dist is not None:                      # every rank runs the same depth
        t = torch.tensor([layers], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        layers = int(t.item())
    if layers < 1:
        raise SystemExit("cfg5: not enough free GPU memory for one layer")
    stream = torch.cuda.Stream()
    gpu = GpuContext(local_rank, stream=stream.cuda_stream)
    lens = np.full(S, Lctx, np.uint32)
    with torch.cuda.stream(stream):
        dec = BatchedDecoder(gpu, num_seqs=S, capacities=lens, num_heads=nh, num_kv_heads=nkv, head_dim=hd, kv_dtype=F16,
                             rope_theta=1e6, rotary_dim=hd, has_gate=False, num_layers=layers, num_splits=0)
        dec.set_lengths(lens - 1)
        n = dec.layer_bytes // 2
        ops.fill_randn(gpu, dec.k_cache[0], n, F16, SEED, 9000 + rank * 10 + 1)
        ops.fill_randn(gpu, dec.v_cache[0], n, F16, SEED, 9000 + rank * 10 + 2)
        for l in range(1, layers):            # the other layers hold copies of the same random rows in their own memory
            gpu.copy_buffer(dec.k_cache[0], dec.k_cache[l], dec.layer_bytes)
            gpu.copy_buffer(dec.v_cache[0], dec.v_cache[l], dec.layer_bytes)
        ops.fill_randn(gpu, dec.q_in, S * nh * hd, F16, SEED, 9003)
        ops.fill_randn(gpu, dec.k_in, S * nkv * hd, F16, SEED, 9004)
        ops.fill_randn(gpu, dec.v_in, S * nkv * hd, F16, SEED, 9005)
        gpu.synchronize()

        def step():
            for l in range(layers):
                dec.step(l)

        for _ in range(args.warmup):
            step()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        l0 = gpu.launch_count
        e0.record(stream)
        for _ in range(args.steps):
            step()
        e1.record(stream)
        barrier()
        launches = gpu.launch_count - l0
        ms = e0.elapsed_time(e1)
    t = torch.tensor([ms], dtype=torch.float64, device="cuda")
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    if rank == 0:
        step_bytes = float(dec.kv_bytes_per_step())          # this rank, all layers
        peak, src = _peak()
        per_gpu = step_bytes * args.steps / (ms * 1e-3) / 1e9
        print(json.dumps({
            "metric": "decode_attn_kv_bandwidth", "value": per_gpu * world, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": "cfg5: full-depth batched decode step, attention only (append + attend per layer)",
                       "layers": layers, "layers_asked": want_layers, "seqs_per_gpu": S, "context": Lctx, "num_q_heads": nh,
                       "num_kv_heads": nkv, "head_dim": hd, "kv_dtype": "fp16", "kv_gb_per_gpu": layers * layer_bytes / 1e9,
                       "sharding": f"sequences over {world} GPU(s), no collective", "l2": "4.3 GB of KV per layer"},
            "roofline": {"bound": "hbm", "achieved": per_gpu, "peak": peak, "unit": "GB/s", "frac": per_gpu / peak,
                         "traffic": None, "peak_source": f"{src} (copy bandwidth)",
                         "kernel": "whole step (append + decode per layer) on one GPU"},
            "gpu_launches": int(launches)}), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    gpu.close()
