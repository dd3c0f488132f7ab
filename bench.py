#!/usr/bin/env python
"""Benchmark of the attention hot path on B200.

Default workload ("cfg2", BASELINE config 2): batched ragged decode attention, one layer —
32 sequences per GPU with context lengths uniform in [1024, 8192], 32 query heads, 8 KV
heads, head_dim 128, fp16 KV cache (contiguous per sequence) and fp16 Q with RoPE, fp32
accumulation.  One step = append one token per sequence (RoPE + cache store) and attend.
Metric: algorithmic KV bytes read per second (GB/s).  Sequences are sharded over GPUs with
no data-path collective (weak scaling: every GPU holds its own 32 sequences).

Prints ONE JSON line (rank 0).  `--impl reference` times the CPU restatement of the
reference shaders (the oracle port; the WGSL itself cannot run here) on the host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

SEED = 0x5EED
NH, NKV, HD = 32, 8, 128
SEQS_PER_GPU = 32
LMIN, LMAX = 1024, 8192
N_SETS = 3            # rotating cache sets so no step finds its KV rows in L2
# DRAM bytes (read + write, one launch) per algorithmic byte of the headline decode kernel, as ncu counted them on
# this workload, and the commit whose kernel was captured; the ratio is a property of the kernel's access pattern,
# so a launch timed here is credited with its own algorithmic bytes times this figure.
TRAFFIC_PER_ALGO_BYTE = {"fp16": 1.010, "fp8": 1.023, "fp8e5m2": 1.026}   # by cache format, from the captures under profiles/
TRAFFIC_MEASURED_AT = ("8ae8e09 for fp16 (ncu --set full, one launch of decode16_kernel<half,128>: 524.2 MB read + 4.1 MB written for 523.3 MB "
                       "algorithmic), e207074 for the 8-bit caches (fused step; e4m3 262.7 + 5.0, e5m2 262.6 + 5.8 for 261.6)")


def draw_lengths(rank: int) -> np.ndarray:
    """Lengths *including* the token appended in the step."""
    rng = np.random.default_rng(SEED + 7919 * rank)
    return rng.integers(LMIN, LMAX + 1, SEQS_PER_GPU).astype(np.uint32)


def rank_lengths(rank: int, world: int) -> np.ndarray:
    """The job's batch is 32 sequences per GPU; on several GPUs they are dealt to the ranks longest first, each to
    the rank with the fewest rows so far (sharding.shard_sequences), so every rank streams about the same bytes."""
    if world == 1:
        return draw_lengths(0)
    from shady_thinker_b200.sharding import shard_sequences
    all_lens = np.concatenate([draw_lengths(r) for r in range(world)])
    return all_lens[shard_sequences(all_lens, world)[rank]]


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def measured_tensor_peaks():
    """(burst, sustained) dense bf16 TFLOP/s and where they come from."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return float(p["bf16_tflops"]), float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), "measured"
    return 1590.0, 1400.0, "fallback"


def host_threads(O) -> int:
    """Threads for the CPU legs: all host cores, even when the launcher (torchrun) pinned OMP_NUM_THREADS to 1."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    return max(n, O.num_threads())


class ClockSampler(threading.Thread):
    """Polls NVML (read-only) for SM clock and throttle reasons while the timed region runs."""

    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
               0x80: "hw_power_brake_slowdown"}

    def __init__(self, device_index: int):
        super().__init__(daemon=True)
        self.samples = []
        self.stop_flag = False
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            vis = os.environ.get("CUDA_VISIBLE_DEVICES")
            idx = device_index
            if vis:
                try:
                    idx = int(vis.split(",")[device_index])
                except ValueError:
                    idx = device_index
            self.h = pynvml.nvmlDeviceGetHandleByIndex(idx)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
            self.ok = True
        except Exception:
            self.max_mhz = None

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        while not self.stop_flag:
            try:
                mhz = int(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    rs = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.h))
                except Exception:
                    rs = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
                self.samples.append((time.perf_counter(), mhz, rs))
            except Exception:
                pass
            time.sleep(0.005)

    def summary(self, t0: float, t1: float) -> dict:
        inside = [s for s in self.samples if t0 <= s[0] <= t1] or self.samples
        if not inside:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        bits = 0
        for s in inside:
            bits |= s[2]
        return {"sm_mhz": float(np.median([s[1] for s in inside])), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(v for k, v in self.REASONS.items() if bits & k), "samples": len(inside)}


def host_set(O, lens: np.ndarray, row_off: np.ndarray, set_id: int, rank: int, seqs):
    """The fp16-rounded K/V rows and activations of the chosen sequences, regenerated on the host
    from the same counter-based generator the device fill uses."""
    row = NKV * HD
    base = 1000 * rank + 10 * set_id
    ks, vs = [], []
    for s in seqs:
        L = int(lens[s])
        ks.append(O.round_f16(O.randn((L, NKV, HD), SEED, base + 1, first_idx=int(row_off[s]) * row)))
        vs.append(O.round_f16(O.randn((L, NKV, HD), SEED, base + 2, first_idx=int(row_off[s]) * row)))
    return ks, vs


def run_reference(args, rank: int) -> None:
    """CPU arm: the oracle's f32-faithful decode (one task per sequence, all host threads) on a bounded
    sample of the cfg2 batch.  The rows are post-RoPE; the append is O(1) rows and not part of the sample."""
    if rank != 0:
        return
    from oracle import oracle as O
    O.build()
    threads = host_threads(O)
    lens = draw_lengths(0)
    row_off = np.concatenate([[0], np.cumsum((lens.astype(np.int64) + 15) // 16 * 16)])
    # calibrate on one mid-sized sequence, then size the sample so the whole run stays within ~2 minutes
    order = np.argsort(lens)
    probe = int(order[len(order) // 2])
    ks, vs = host_set(O, lens, row_off, 0, 0, [probe])
    q = O.round_f16(O.randn((SEQS_PER_GPU, NH, HD), SEED, 5))
    t0 = time.perf_counter()
    O.gqa_attention_head(q[probe], ks[0], vs[0], int(lens[probe]), threads=threads)
    per_pos = (time.perf_counter() - t0) / int(lens[probe])          # one sequence uses the head-parallel form
    budget = 100.0 / max(args.steps + args.warmup, 1)
    # sequences run in parallel over threads: est. time ~ sum(L)*per_pos*threads_used/threads
    seqs, tot = [], 0
    for s in order[::-1]:
        est = (tot + int(lens[s])) * per_pos
        if seqs and est > budget:
            break
        seqs.append(int(s))
        tot += int(lens[s])
    ks, vs = host_set(O, lens, row_off, 0, 0, seqs)
    use_lens = [int(lens[s]) for s in seqs]
    if len(seqs) == 1 and tot * per_pos > budget:                     # even one sequence is too long: truncate it
        use_lens = [max(LMIN // 4, int(budget / per_pos))]
    qs = q[seqs]
    nbytes = sum(use_lens) * NKV * HD * 2 * 2

    def step():
        if len(seqs) == 1:
            O.gqa_attention_head(qs[0], ks[0], vs[0], use_lens[0], threads=threads)
        else:
            O.batched_decode(qs, ks, vs, use_lens, threads=threads)

    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = time.perf_counter() - t0
    val = nbytes * args.steps / dt / 1e9
    sample = f"{len(seqs)} of {SEQS_PER_GPU} cfg2 sequences ({sum(use_lens)} positions, {nbytes / 1e6:.1f} MB of fp16-rounded KV as f32) per step"
    print(json.dumps({
        "impl": "reference", "metric": "decode_attn_kv_bandwidth", "value": val, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.gpus),
        "cpu_baseline": {"value": val, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "CPU restatement of gqa_attention_head.wgsl (oracle port); the WGSL through wgpu is unavailable on this box",
    }))


def workload_config(n_gpus: int, shape: str = "plain", kv: str = "fp16") -> dict:
    rope = ("full rotary (rotary_dim = head_dim), no QK-norm, no gate" if shape == "plain" else
            "reference-shaped: rotary_dim = head_dim/4 interleaved, QK RMSNorm with bf16 weights, sigmoid gate")
    return {"workload": "cfg2: batched ragged decode attention, one layer, append+attend per step", "rope": rope,
            "seqs_per_gpu": SEQS_PER_GPU, "context": f"uniform[{LMIN},{LMAX}] (seeded)", "num_q_heads": NH,
            "num_kv_heads": NKV, "head_dim": HD, "kv_dtype": kv if kv == "fp16" else ("fp8 e4m3" if kv == "fp8" else "fp8 e5m2") + " (algorithmic bytes count one byte per element)",
            "q_dtype": "fp16", "accumulate": "fp32",
            "rope_theta": 1e6, "sharding": (f"{SEQS_PER_GPU * n_gpus} sequences dealt to {n_gpus} GPU(s) longest first to the rank with the fewest rows, "
                         "no collective"),
            "l2": f"KV per step > L2 and {N_SETS} cache sets rotate between steps"}


def cpu_baseline(rank: int, row_off, lens: np.ndarray) -> dict:
    """Oracle (f32-faithful port) on a bounded sample of the same batch, all host threads."""
    from oracle import oracle as O
    O.build()
    threads = host_threads(O)
    order = np.argsort(lens)[::-1]
    seqs = [int(s) for s in order[:8]]
    ks, vs = host_set(O, lens, row_off, 0, rank, seqs)
    q = O.round_f16(O.randn((8, NH, HD), SEED, 5))
    use = [int(lens[s]) for s in seqs]
    nbytes = sum(use) * NKV * HD * 2 * 2
    best, t_total, reps = None, 0.0, 0
    while t_total < 8.0 and reps < 20:
        t0 = time.perf_counter()
        O.batched_decode(q, ks, vs, use, threads=threads)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
        t_total += dt
        reps += 1
    return {"value": nbytes / best / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
            "sample": f"8 longest of {SEQS_PER_GPU} cfg2 sequences ({sum(use)} positions, {nbytes / 1e6:.1f} MB of KV), best of {reps}"}


def run_ours(args, rank: int, world: int, local_rank: int) -> None:
    import torch

    from shady_thinker_b200._lib import F8E4M3, F8E5M2, F16
    from shady_thinker_b200.batch import BatchedDecoder
    from shady_thinker_b200.gpu import GpuContext
    from shady_thinker_b200 import ops

    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    stream = torch.cuda.Stream()
    gpu = GpuContext(local_rank, stream=stream.cuda_stream)
    lens = rank_lengths(rank, world)
    S = len(lens)
    sets = []
    ref_shape = args.shape == "reference"
    kv_dt = {"fp8": F8E4M3, "fp8e5m2": F8E5M2}.get(args.kv, F16)      # 8-bit cache rows (half the bytes per row), f16 activations
    qrow = NH * HD * (2 if ref_shape else 1)
    d_norm = None
    if ref_shape:       # bf16 q_norm[hd] then k_norm[hd], N(0, 0.02) (the uniform of model.rs:140-168)
        wf = (np.random.default_rng(SEED).standard_normal(2 * HD) * 0.02).astype(np.float32).view(np.uint32)
        wbits = ((wf + 0x7FFF + ((wf >> 16) & 1)) >> 16).astype(np.uint16)
        d_norm = gpu.upload_buffer("qknorm_weights", wbits.tobytes())
    for i in range(N_SETS):
        d = BatchedDecoder(gpu, num_seqs=S, capacities=lens, num_heads=NH, num_kv_heads=NKV, head_dim=HD,
                           kv_dtype=kv_dt, rope_theta=1e6, rotary_dim=HD // 4 if ref_shape else HD, has_gate=ref_shape,
                           num_splits=0, qk_norm_bf16=d_norm)
        d.set_lengths(lens - 1)
        base = 1000 * rank + 10 * i
        n = d.layer_bytes // (2 if kv_dt == F16 else 1)
        ops.fill_randn(gpu, d.k_cache[0], n, kv_dt, SEED, base + 1)
        ops.fill_randn(gpu, d.v_cache[0], n, kv_dt, SEED, base + 2)
        ops.fill_randn(gpu, d.q_in, S * qrow, F16, SEED, base + 3)
        ops.fill_randn(gpu, d.k_in, S * NKV * HD, F16, SEED, base + 4)
        ops.fill_randn(gpu, d.v_in, S * NKV * HD, F16, SEED, base + 5)
        sets.append(d)
    gpu.synchronize()
    step_bytes = sets[0].kv_bytes_per_step()
    row_off0 = sets[0].row_off

    sampler = ClockSampler(local_rank)
    sampler.start()
    with torch.cuda.stream(stream):
        # ---------------- device-resident throughput ----------------
        for i in range(args.warmup):
            sets[i % N_SETS].step()
        # the launch itself is timed on every ev_stride-th step only: an event pair around each launch costs
        # the whole-step figure a few microseconds of gap per step
        ev_stride = 1 if args.steps <= 16 else 8
        ev_a = [torch.cuda.Event(enable_timing=True) for _ in range(0, args.steps, ev_stride)]
        ev_b = [torch.cuda.Event(enable_timing=True) for _ in range(0, args.steps, ev_stride)]
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        launches0 = gpu.launch_count
        t_wall0 = time.perf_counter()
        e0.record(stream)
        for i in range(args.steps):
            d = sets[i % N_SETS]
            timed = i % ev_stride == 0
            if timed:
                ev_a[i // ev_stride].record(stream)
            d.step()            # one fused launch: RoPE + cache append + split-KV decode + merge
            if timed:
                ev_b[i // ev_stride].record(stream)
        e1.record(stream)
        barrier()
        t_wall1 = time.perf_counter()
        launches = gpu.launch_count - launches0
        total_ms = e0.elapsed_time(e1)
        attend_ms = sum(a.elapsed_time(b) for a, b in zip(ev_a, ev_b)) / len(ev_a)

        # ---------------- end to end with host buffers ----------------
        d0 = sets[0]
        asz = 2
        hq = torch.empty(S * qrow, dtype=torch.float16).pin_memory()
        hk = torch.empty(S * NKV * HD, dtype=torch.float16).pin_memory()
        hv = torch.empty(S * NKV * HD, dtype=torch.float16).pin_memory()
        ho = torch.empty(S * NH * HD, dtype=torch.float16).pin_memory()
        hq.normal_(); hk.normal_(); hv.normal_()
        e2e_steps = max(10, min(args.steps, 2000))
        # The public call for host buffers: with the fused launch the kernel itself reads the pinned activations
        # and writes the pinned output over the host link (no copy calls); else explicit H2D / D2H copies.
        def host_step(d):
            (d.step_from_pinned if d.fused else d.step_from_host)(hq.data_ptr(), hk.data_ptr(), hv.data_ptr(), ho.data_ptr())
        for i in range(max(3, args.warmup)):
            host_step(sets[i % N_SETS])
        barrier()
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        f0.record(stream)
        for i in range(e2e_steps):
            host_step(sets[i % N_SETS])
        f1.record(stream)
        barrier()
        e2e_ms = f0.elapsed_time(f1)
        assert torch.isfinite(ho.float()).all(), "e2e output is not finite"
        # ---------------- a longer witness of the same launch: 100 blocks of 20 back-to-back launches ----------------
        long_blocks, long_per = 100, 20
        lb = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(long_blocks)]
        k = 0
        for a_ev, b_ev in lb:
            a_ev.record(stream)
            for _ in range(long_per):
                sets[k % N_SETS].step()
                k += 1
            b_ev.record(stream)
        barrier()
        long_ms = np.array([a_ev.elapsed_time(b_ev) / long_per for a_ev, b_ev in lb])
    sampler.stop_flag = True
    sampler.join(timeout=2)
    headline_clocks = sampler.summary(t_wall0, t_wall1)

    # ---------------- the other half of the metric and the cross-GPU kernel, after the headline ----------------
    extra = {}
    if not args.no_extra:
        for d in sets:
            d.close()
        extra["cfg3"] = measure_cfg3(gpu, stream, rank, world, local_rank, dist, barrier, steps=30, warmup=3)
        set_prefill_shape(256)      # the same batch and length in the gated-attention head shape (16 / 2 heads of 256)
        extra["cfg3_head_dim_256"] = measure_cfg3(gpu, stream, rank, world, local_rank, dist, barrier, steps=20, warmup=3)
        set_prefill_shape(args.prefill_hd)
        extra["cfg4"] = measure_cfg4(gpu, stream, rank, world, local_rank, dist, barrier, steps=500, warmup=20)

    # ---------------- reduce over ranks: max time, sum bytes ----------------
    t = torch.tensor([total_ms, e2e_ms, attend_ms], dtype=torch.float64, device="cuda")
    b = torch.tensor([float(step_bytes)], dtype=torch.float64, device="cuda")
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(b, op=dist.ReduceOp.SUM)
    total_ms, e2e_ms, attend_ms_max = [float(x) for x in t.tolist()]
    all_bytes = float(b.item())

    if rank == 0:
        peak, peak_src = measured_peaks()
        # One launch per step: the event pair around a single launch adds about 2 us of its own to what it brackets,
        # so when the whole back-to-back region divided by its launches is the smaller figure, that is the launch time.
        bracketed_ms = attend_ms
        if launches == args.steps:
            attend_ms = min(attend_ms, total_ms / args.steps)
        achieved = step_bytes / (attend_ms * 1e-3) / 1e9          # this rank's decode op: algorithmic bytes / duration
        line = {
            "metric": "decode_attn_kv_bandwidth", "value": all_bytes * args.steps / (total_ms * 1e-3) / 1e9, "unit": "GB/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": total_ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": workload_config(world, args.shape, args.kv),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": TRAFFIC_PER_ALGO_BYTE[args.kv] * step_bytes,
                         "peak_source": f"{peak_src} (copy bandwidth)",
                         "kernel": ("decode16_kernel<half,128> with the fused append and split merge (the whole step is this one launch)"
                                    if args.kv == "fp16" else
                                    "decode16_kernel<half,128,8-bit cache> with the fused (quantising) append and split merge "
                                    "(the whole step is this one launch)" if d0.fused else
                                    "decode16_kernel<half,128,8-bit cache> (the step is the append launch plus this attend launch)"),
                         "traffic_source": f"algorithmic bytes x {TRAFFIC_PER_ALGO_BYTE[args.kv]}, the DRAM-byte ratio ncu measured at {TRAFFIC_MEASURED_AT}",
                         "algorithmic_bytes_per_launch": step_bytes, "avg_launch_ms": attend_ms,
                         "avg_launch_ms_single_bracketed": bracketed_ms,
                         "avg_launch_ms_long": {"launches": int(long_blocks * long_per), "median": float(np.median(long_ms)),
                                                "p10": float(np.percentile(long_ms, 10)), "p90": float(np.percentile(long_ms, 90)),
                                                "frac_at_median": step_bytes / (float(np.median(long_ms)) * 1e-3) / 1e9 / peak,
                                                "how": "100 event-bracketed blocks of 20 back-to-back launches, per-launch time of each block"}},
            "e2e": {"value": all_bytes * e2e_steps / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s",
                    "h2d_bytes_per_step": d0.in_bytes, "d2h_bytes_per_step": d0.out_bytes, "steps": e2e_steps,
                    "ms_per_step": e2e_ms / e2e_steps,
                    "path": ("BatchedDecoder.step_from_pinned: the launch reads the pinned activations and writes the "
                             "pinned output over the host link itself, then one stream sync") if d0.fused else
                            "BatchedDecoder.step_from_host: H2D copies, launches, D2H copy, one stream sync"},
            "gpu_launches": int(launches),
            "clocks": headline_clocks,
        }
        if extra:
            line["extra"] = extra
        if world == 1 and not args.no_cpu_baseline and args.kv == "fp16":
            line["cpu_baseline"] = cpu_baseline(rank, row_off0, lens)
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    gpu.close()


# ------------------------------------------------------------------------------------------------
# cfg3: causal prefill attention (BASELINE config 3): batch 4, T 4096, 32 query heads, 8 KV heads,
# head_dim 128, bf16 Q/K/V, RoPE theta 1e6, fp32 softmax statistics; the step also writes K/V into
# the cache (append kernel) and then runs the tcgen05 attention kernel over the cache.
# ------------------------------------------------------------------------------------------------
P_B, P_T, P_NH, P_NKV, P_HD = 4, 4096, 32, 8, 128


def prefill_flops(B=None, T=None, nh=None, hd=None) -> float:
    B, T, nh, hd = B or P_B, T or P_T, nh or P_NH, hd or P_HD
    return 4.0 * B * nh * hd * T * (T + 1) / 2


def set_prefill_shape(hd: int) -> None:
    """cfg3 as BASELINE.json states it has head_dim 128; `--prefill-hd 256` runs the same batch and length with the
    head layout of config 4 (16 query heads, 2 KV heads, head_dim 256: the gated-attention layer shape)."""
    global P_NH, P_NKV, P_HD
    P_NH, P_NKV, P_HD = (16, 2, 256) if hd == 256 else (32, 8, 128)


def prefill_config(n_gpus: int) -> dict:
    return {"workload": "cfg3: causal prefill attention, one layer; a step = K/V norm+RoPE+cache write, then attention with Q normed/rotated in the kernel",
            "batch_per_gpu": P_B, "seq_len": P_T, "num_q_heads": P_NH, "num_kv_heads": P_NKV, "head_dim": P_HD,
            "dtype": "bf16", "softmax": "fp32", "rope_theta": 1e6,
            "sharding": f"batch items over {n_gpus} GPU(s), no collective",
            "l2": "Q+K+V+out per step (403 MB) exceed L2"}


def prefill_cpu_sample(O, threads: int, T: int, nh: int, nkv: int):
    q = O.round_bf16(O.randn((T, nh, P_HD), SEED, 31))
    k = O.round_bf16(O.randn((T, nkv, P_HD), SEED, 32))
    v = O.round_bf16(O.randn((T, nkv, P_HD), SEED, 33))
    t0 = time.perf_counter()
    O.causal_prefill(q, k, v, threads=threads)
    dt = time.perf_counter() - t0
    return prefill_flops(1, T, nh) / dt / 1e12, dt


def run_reference_prefill(args, rank: int) -> None:
    if rank != 0:
        return
    from oracle import oracle as O
    O.build()
    threads = host_threads(O)
    # bounded sample: one batch item, one KV group (4 query heads), T sized to the step count
    T = 1024
    val, dt = prefill_cpu_sample(O, threads, T, 4, 1)
    budget = 100.0 / max(args.steps + args.warmup, 1)
    while dt * 4 < budget and T < P_T:
        T *= 2
        val, dt = prefill_cpu_sample(O, threads, T, 4, 1)
    for _ in range(args.warmup):
        prefill_cpu_sample(O, threads, T, 4, 1)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        prefill_cpu_sample(O, threads, T, 4, 1)
    wall = time.perf_counter() - t0
    val = prefill_flops(1, T, 4) * args.steps / wall / 1e12
    sample = f"1 batch item x 4 query heads (1 KV group) x T={T} of cfg3, token loop of gqa_attention_head.wgsl in f32"
    print(json.dumps({
        "impl": "reference", "metric": "prefill_attn_tflops", "value": val, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": wall / args.steps * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": prefill_config(args.gpus),
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "CPU restatement of the reference's per-token prefill loop (oracle port); the WGSL through wgpu is unavailable on this box",
    }))


class _Cfg3:
    """Buffers and the two calls of a cfg3 step (append with RoPE + cache write, then the tcgen05 attention)."""

    def __init__(self, gpu, rank: int):
        from shady_thinker_b200 import ops
        from shady_thinker_b200._lib import BF16
        B, T, nh, nkv, hd = P_B, P_T, P_NH, P_NKV, P_HD
        self.gpu, self.ops, self.BF16 = gpu, ops, BF16
        self.nq, self.nk = B * T * nh * hd, B * T * nkv * hd
        mk = gpu.create_storage_buffer
        self.bufs = {n: mk(n, (self.nq if n in ("q_in", "q_rot", "out") else self.nk) * 2)
                     for n in ("q_in", "k_in", "v_in", "q_rot", "out", "k_cache", "v_cache")}
        self.pos = gpu.upload_buffer("pos", np.zeros(B, np.uint32).tobytes())
        base = 5000 + 10 * rank
        b = self.bufs
        ops.fill_randn(gpu, b["q_in"], self.nq, BF16, SEED, base + 1)
        ops.fill_randn(gpu, b["k_in"], self.nk, BF16, SEED, base + 2)
        ops.fill_randn(gpu, b["v_in"], self.nk, BF16, SEED, base + 3)
        self.view = ops.KvCacheView(BF16, b["k_cache"], b["v_cache"], T * nkv * hd)
        self.ws_n = ops.prefill_workspace_size(head_dim=hd, num_kv_heads=nkv, num_q_heads=nh, num_seqs=B, seq_len=T, dtype=BF16)
        self.ws = mk("prefill_ws", self.ws_n)

    def append(self):
        b = self.bufs
        self.ops.kv_append_rope(self.gpu, q_proj_full=b["q_in"], k_proj=b["k_in"], v_proj=b["v_in"], q_out=b["q_rot"],
                                q_gate=None, cache=self.view, pos_start=self.pos, num_heads=P_NH, num_kv_heads=P_NKV,
                                head_dim=P_HD, rope_theta=1e6, rotary_dim=P_HD, num_seqs=P_B, tokens_per_seq=P_T,
                                in_dtype=self.BF16, q_dtype=self.BF16, has_gate=False, write_k_back=False)

    def attend(self):
        b = self.bufs
        self.ops.attn_prefill(self.gpu, q=b["q_rot"], cache=self.view, out=b["out"], head_dim=P_HD, num_kv_heads=P_NKV,
                              num_q_heads=P_NH, num_seqs=P_B, seq_len=P_T, dtype=self.BF16)

    def step(self):
        """The whole step through the public call: K/V pass (norm, RoPE, cache rows), then the attention kernel that
        takes Q raw from the projection (norm + RoPE per tile in shared memory)."""
        b = self.bufs
        self.ops.attn_prefill_append(self.gpu, q_proj_full=b["q_in"], k_proj=b["k_in"], v_proj=b["v_in"], cache=self.view,
                                     out=b["out"], workspace=self.ws, workspace_bytes=self.ws_n, num_heads=P_NH,
                                     num_kv_heads=P_NKV, head_dim=P_HD, num_seqs=P_B, seq_len=P_T, rope_theta=1e6,
                                     rotary_dim=P_HD, dtype=self.BF16)

    def close(self):
        for b in list(self.bufs.values()) + [self.pos, self.ws]:
            self.gpu.destroy_buffer(b)
        self.bufs = {}


def _time_cfg3(torch, c: "_Cfg3", gpu, stream, barrier, steps: int, warmup: int, local_rank: int):
    """(total_ms, attend_ms, launches, clocks, two_call_ms): `steps` whole steps through shady_attn_prefill_append
    (total_ms), then `steps` steps of the two-call form (append, then the attention kernel on the rotated Q) with the
    attention launch bracketed (attend_ms per launch, two_call_ms per step)."""
    sampler = ClockSampler(local_rank)
    sampler.start()
    for _ in range(warmup):
        c.step()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    launches0 = gpu.launch_count
    t_wall0 = time.perf_counter()
    e0.record(stream)
    for i in range(steps):
        c.step()
    e1.record(stream)
    barrier()
    t_wall1 = time.perf_counter()
    launches = gpu.launch_count - launches0
    for _ in range(min(warmup, 3)):
        c.append(); c.attend()
    ev_a = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    ev_b = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    g0.record(stream)
    for i in range(steps):
        c.append()
        ev_a[i].record(stream)
        c.attend()
        ev_b[i].record(stream)
    g1.record(stream)
    barrier()
    gpu.synchronize()   # also surfaces a bounded-wait expiry of the prefill kernel
    sampler.stop_flag = True
    sampler.join(timeout=2)
    attend_ms = sum(x.elapsed_time(y) for x, y in zip(ev_a, ev_b)) / steps
    return e0.elapsed_time(e1), attend_ms, launches, sampler.summary(t_wall0, t_wall1), g0.elapsed_time(g1) / steps


def measure_cfg3(gpu, stream, rank, world, local_rank, dist, barrier, steps: int, warmup: int) -> dict:
    """The prefill half of the metric as a short leg of the default line: attention-launch TFLOP/s and whole-step
    TFLOP/s (append included) against the measured bf16 peak, with its own clock sample.  Frees its memory."""
    import torch
    with torch.cuda.stream(stream):
        c = _Cfg3(gpu, rank)
        gpu.synchronize()
        total_ms, attend_ms, launches, clocks, two_call_ms = _time_cfg3(torch, c, gpu, stream, barrier, steps, warmup, local_rank)
        c.close()
    t = torch.tensor([total_ms, attend_ms, two_call_ms], dtype=torch.float64, device="cuda")
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms, attend_ms, two_call_ms = [float(x) for x in t.tolist()]
    flops = prefill_flops()
    burst, sustained, src = measured_tensor_peaks()
    attn = flops / (attend_ms * 1e-3) / 1e12
    step = flops / (total_ms / steps * 1e-3) / 1e12
    return {"workload": prefill_config(world)["workload"], "metric": "prefill_attn_tflops", "unit": "TFLOP/s",
            "steps": steps, "warmup": warmup, "n_gpus": world, "per_gpu": True,
            "attention_launch": {"tflops": attn, "ms": attend_ms,
                                 "what": ("prefill_kernel" if P_HD == 128 else "rowtile_kernel") + " alone, on Q rotated beforehand"},
            "head_dim": P_HD, "num_q_heads": P_NH, "num_kv_heads": P_NKV,
            "whole_step": {"tflops": step, "ms": total_ms / steps,
                           "includes": ("shady_attn_prefill_append: K/V pass (norm, RoPE, cache rows) + attention kernel that norms/rotates Q itself"
                                        if P_HD == 128 else
                                        "shady_attn_prefill_append: one append pass (Q, K normed and rotated, cache rows) + attention kernel with the gate in its epilogue")},
            "whole_step_two_calls": {"tflops": flops / (two_call_ms * 1e-3) / 1e12, "ms": two_call_ms,
                                     "includes": "shady_kv_append_rope (Q, K, V) + shady_attn_prefill"},
            "roofline": {"bound": "tensor", "achieved": attn, "peak": burst, "unit": "TFLOP/s", "frac": attn / burst,
                         "frac_whole_step": step / burst, "peak_source": f"{src} cuBLAS bf16 burst figure (sustained {sustained})",
                         "algorithmic_flops_per_launch": flops},
            "gpu_launches": int(launches), "clocks": clocks}


def run_prefill(args, rank: int, world: int, local_rank: int) -> None:
    torch, dist, barrier = _dist_setup(world, local_rank)
    from shady_thinker_b200.gpu import GpuContext

    stream = torch.cuda.Stream()
    gpu = GpuContext(local_rank, stream=stream.cuda_stream)
    with torch.cuda.stream(stream):
        c = _Cfg3(gpu, rank)
        nq, nk = c.nq, c.nk
        q_in, k_in, v_in, out = (c.bufs[n] for n in ("q_in", "k_in", "v_in", "out"))
        gpu.synchronize()
        total_ms, attend_ms, launches, clocks, _two = _time_cfg3(torch, c, gpu, stream, barrier, args.steps, args.warmup, local_rank)
        # ---- end to end: host activations in, output back ----
        hq = torch.empty(nq, dtype=torch.bfloat16).pin_memory().normal_()
        hk = torch.empty(nk, dtype=torch.bfloat16).pin_memory().normal_()
        hv = torch.empty(nk, dtype=torch.bfloat16).pin_memory().normal_()
        ho = torch.empty(nq, dtype=torch.bfloat16).pin_memory()
        import ctypes as C
        L = gpu._L

        def e2e_step():
            gpu._check(L.shady_buffer_write(gpu.handle, C.c_void_p(q_in.ptr), 0, C.c_void_p(hq.data_ptr()), nq * 2))
            gpu._check(L.shady_buffer_write(gpu.handle, C.c_void_p(k_in.ptr), 0, C.c_void_p(hk.data_ptr()), nk * 2))
            gpu._check(L.shady_buffer_write(gpu.handle, C.c_void_p(v_in.ptr), 0, C.c_void_p(hv.data_ptr()), nk * 2))
            c.step()
            gpu._check(L.shady_buffer_read(gpu.handle, C.c_void_p(out.ptr), 0, C.c_void_p(ho.data_ptr()), nq * 2))

        e2e_steps = max(3, min(args.steps, 20))
        for _ in range(3):
            e2e_step()
        barrier()
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        f0.record(stream)
        for _ in range(e2e_steps):
            e2e_step()
        f1.record(stream)
        barrier()
        e2e_ms = f0.elapsed_time(f1)
        assert torch.isfinite(ho.float()).all(), "e2e output is not finite"

    t = torch.tensor([total_ms, e2e_ms, attend_ms], dtype=torch.float64, device="cuda")
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms, e2e_ms, _ = [float(x) for x in t.tolist()]
    flops = prefill_flops()
    if rank == 0:
        burst, sustained, src = measured_tensor_peaks()
        long_loop = total_ms > 1000.0
        peak = sustained if long_loop else burst
        achieved = flops / (attend_ms * 1e-3) / 1e12
        line = {
            "metric": "prefill_attn_tflops", "value": flops * world * args.steps / (total_ms * 1e-3) / 1e12,
            "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": total_ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic", "config": prefill_config(world),
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                         "traffic": None,
                         "peak_source": f"{src} cuBLAS bf16, {'sustained' if long_loop else 'burst'} figure "
                                        f"(burst {burst}, sustained {sustained})",
                         "kernel": "prefill kernel alone (head_dim 128: prefill_kernel, 256: rowtile_kernel) on Q rotated beforehand; `value` is the whole step through shady_attn_prefill_append",
                         "algorithmic_flops_per_launch": flops,
                         "avg_launch_ms": attend_ms},
            "e2e": {"value": flops * world * e2e_steps / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                    "h2d_bytes_per_step": (nq + 2 * nk) * 2, "d2h_bytes_per_step": nq * 2, "steps": e2e_steps,
                    "ms_per_step": e2e_ms / e2e_steps},
            "gpu_launches": int(launches),
            "clocks": clocks,
        }
        if world == 1 and not args.no_cpu_baseline:
            from oracle import oracle as O
            O.build()
            val, dt = prefill_cpu_sample(O, host_threads(O), 2048, 8, 2)
            line["cpu_baseline"] = {"value": val, "unit": "TFLOP/s", "cores": host_threads(O), "kind": "port",
                                    "sample": f"1 batch item x 8 query heads (2 KV groups) x T=2048 of cfg3, {dt:.1f} s"}
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    gpu.close()


# ------------------------------------------------------------------------------------------------
# Other configurations of the baseline file (the default line stays cfg2)
# ------------------------------------------------------------------------------------------------
def _dist_setup(world: int, local_rank: int):
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


C4_L, C4_NH, C4_NKV, C4_HD = 131072, 16, 2, 256


def measure_cfg4(gpu, stream, rank, world, local_rank, dist, barrier, steps: int, warmup: int) -> dict:
    """cfg4: one sequence of 131072 rows, nh16/nkv2/hd256, bf16 KV.  One GPU: the whole sequence in one cooperative
    launch (decode, grid barrier, record merge).  Several GPUs: rows cut contiguously over the ranks, every rank runs
    the same launch on its rows and the launch's tail exchanges the merged slices over NVLink peer memory and merges
    across ranks (`ShardCombiner.decode_and_combine`; SHADY_CFG4_COMBINE=p2p / nccl select the older forms for
    comparison).  Before timing, the merged rows are checked against the same sequence decoded by rank 0 alone.
    Returns the figures of the leg (rank 0's view after the max over ranks) and frees its memory."""
    import torch
    from shady_thinker_b200 import ops
    from shady_thinker_b200._lib import BF16
    from shady_thinker_b200.sharding import merge_args, shard_rows
    L, nh, nkv, hd = C4_L, C4_NH, C4_NKV, C4_HD
    lo, hi = shard_rows(L, world, rank)
    rows = hi - lo
    row_bytes = nkv * hd * 2
    n_sets = max(3, -(-320_000_000 // max(2 * rows * row_bytes, 1)))    # rotate through > 2x L2 of distinct rows
    mode = os.environ.get("SHADY_CFG4_COMBINE", "fused")
    use_nccl = mode == "nccl"
    comb = None
    with torch.cuda.stream(stream):
        ks = [torch.empty((max(rows, 1), nkv, hd), dtype=torch.bfloat16, device="cuda") for _ in range(n_sets)]
        vs = [torch.empty_like(k) for k in ks]
        for i in range(n_sets):
            ops.fill_randn(gpu, ks[i], ks[i].numel(), BF16, SEED, 7000 + 100 * i + 1, first_idx=lo * nkv * hd)
            ops.fill_randn(gpu, vs[i], vs[i].numel(), BF16, SEED, 7000 + 100 * i + 2, first_idx=lo * nkv * hd)
        q = torch.empty((1, nh, hd), dtype=torch.bfloat16, device="cuda")
        ops.fill_randn(gpu, q, q.numel(), BF16, SEED, 7999)
        lens = torch.tensor([rows], dtype=torch.int32, device="cuda")
        rec = torch.zeros((1, nh, hd + 2), device="cuda")
        gathered = torch.zeros((world, 1, nh, hd + 2), device="cuda")
        out = torch.zeros((1, nh, hd), device="cuda")
        ws_n = ops.decode_workspace_size(head_dim=hd, num_kv_heads=nkv, num_q_heads=nh, num_splits=0, num_seqs=1)
        ws = torch.zeros(ws_n, dtype=torch.uint8, device="cuda")
        views = [ops.KvCacheView(BF16, ks[i], vs[i], 0) for i in range(n_sets)]
        ev = []
        if world > 1 and not use_nccl:
            from shady_thinker_b200.p2p import ShardCombiner
            comb = ShardCombiner(gpu, rank=rank, world=world, num_heads=nh, head_dim=hd)

        def step(i, timed=False):
            view = views[i % n_sets]
            # the launch is bracketed on every 8th step only: two event records per step cost ~5 us of a 50 us step
            bracket = timed and i % 8 == 0
            a = b = None
            if bracket:
                a = torch.cuda.Event(enable_timing=True); b = torch.cuda.Event(enable_timing=True)
                a.record(stream)
            if world == 1:
                ops.attn_decode(gpu, q=q, cache=view, seq_lens=lens, out=out, head_dim=hd, num_kv_heads=nkv,
                                num_q_heads=nh, num_splits=0, seq_lens_host=[rows], q_dtype=BF16, workspace=ws,
                                workspace_bytes=ws_n)
            elif comb is not None and mode == "fused":
                comb.decode_and_combine(q=q, cache=view, seq_lens=lens, seq_len_host=rows, records=rec, out=out,
                                        num_kv_heads=nkv, q_dtype=BF16, workspace=ws, workspace_bytes=ws_n)
            else:
                ops.attn_decode_shard(gpu, q=q, cache=view, seq_lens=lens, records=rec, head_dim=hd, num_kv_heads=nkv,
                                      num_q_heads=nh, num_splits=0, seq_lens_host=[rows], q_dtype=BF16, workspace=ws,
                                      workspace_bytes=ws_n)
                if comb is not None:
                    comb.combine(rec, out)
                else:
                    dist.all_gather_into_tensor(gathered.view(-1), rec.view(-1))
                    ops.attn_reduce(gpu, partials=gathered, out=out, **merge_args(1, nh, hd, world))
            if bracket:
                b.record(stream)
                ev.append((a, b))

        # ---- self-check of the merged rows (set 0) against the whole sequence decoded by one rank ----
        check = {"self_check": "ok", "against": "n/a (one GPU: the whole sequence is one rank's)"}
        if world > 1:
            step(0)
            gpu.synchronize()
            merged = out.clone()
            err = torch.zeros(1, dtype=torch.float64, device="cuda")
            if rank == 0:
                fk = torch.empty((L, nkv, hd), dtype=torch.bfloat16, device="cuda")
                fv = torch.empty_like(fk)
                ops.fill_randn(gpu, fk, fk.numel(), BF16, SEED, 7001)
                ops.fill_randn(gpu, fv, fv.numel(), BF16, SEED, 7002)
                whole = torch.zeros((1, nh, hd), device="cuda")
                ops.attn_decode(gpu, q=q, cache=ops.KvCacheView(BF16, fk, fv, 0),
                                seq_lens=torch.tensor([L], dtype=torch.int32, device="cuda"), out=whole, head_dim=hd,
                                num_kv_heads=nkv, num_q_heads=nh, num_splits=0, seq_lens_host=[L], q_dtype=BF16,
                                workspace=ws, workspace_bytes=ws_n)
                gpu.synchronize()
                err[0] = float((merged - whole).abs().max() / whole.abs().max())
                del fk, fv
            dist.all_reduce(err, op=dist.ReduceOp.MAX)
            rel = float(err.item())
            check = {"self_check": "ok" if rel <= 2e-2 and bool(torch.isfinite(merged).all()) else "FAILED",
                     "rel_err_vs_one_rank": rel, "tolerance": 2e-2,
                     "against": "rank 0 decoding all 131072 rows in one launch (same seeded rows and Q)"}

        for i in range(warmup):
            step(i)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        l0 = gpu.launch_count
        sampler = ClockSampler(local_rank)
        sampler.start()
        t_wall0 = time.perf_counter()
        e0.record(stream)
        for i in range(steps):
            step(i, True)
        e1.record(stream)
        barrier()
        t_wall1 = time.perf_counter()
        sampler.stop_flag = True
        sampler.join(timeout=2)
        gpu.synchronize()       # surfaces a bounded wait (grid barrier, peer flag) that ran out
        launches = gpu.launch_count - l0
        total_ms = e0.elapsed_time(e1)
        dec_ms = sum(a.elapsed_time(b) for a, b in ev) / len(ev)
        assert torch.isfinite(out).all()
    t = torch.tensor([total_ms, dec_ms], dtype=torch.float64, device="cuda")
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms, dec_ms = [float(x) for x in t.tolist()]
    if comb is not None:
        comb.close()
    del ks, vs, views
    torch.cuda.empty_cache()
    peak, src = measured_peaks()
    total_bytes = 2.0 * L * row_bytes
    step_ms = total_ms / steps
    # one launch per step: when the back-to-back region divided by its launches is the smaller figure, that is the launch
    launch_ms = min(dec_ms, step_ms) if launches == steps else dec_ms
    ach = 2.0 * rows * row_bytes / (launch_ms * 1e-3) / 1e9
    combine = ("none (one GPU)" if world == 1 else
               "NCCL all-gather of 16.5 KB records + merge kernel" if use_nccl else
               "one cooperative launch per step: decode, grid barrier, rank-local merge + peer stores over NVLink + flags + merge across ranks"
               if mode == "fused" else "one kernel: peer stores of 16.5 KB records over NVLink + flags + merge")
    return {"workload": "cfg4: long-context single-sequence decode, rows split over the GPUs, log-sum-exp merge across ranks",
            "metric": "decode_attn_kv_bandwidth", "unit": "GB/s", "value": total_bytes / (step_ms * 1e-3) / 1e9,
            "scaling": "strong", "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": step_ms,
            "context": L, "num_q_heads": nh, "num_kv_heads": nkv, "head_dim": hd, "kv_dtype": "bf16",
            "rows_per_gpu": rows, "combine": combine, "l2": f"{n_sets} cache sets rotate between steps",
            "roofline": {"bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak, "traffic": None,
                         "peak_source": f"{src} (copy bandwidth)",
                         "kernel": ("decode16_kernel<bf16,256> on this rank's rows with the merge and the NVLink exchange in its tail (the rank's whole step)"
                                    if world > 1 and mode == "fused" and not use_nccl else
                                    "decode16_kernel<bf16,256>, blocks interleaved over all warps, record merge after the grid barrier"),
                         "algorithmic_bytes_per_launch": 2.0 * rows * row_bytes, "avg_launch_ms": launch_ms,
                         "avg_launch_ms_bracketed": dec_ms,
                         "frac_of_whole_job_hbm_time": (total_bytes / world / (peak * 1e9)) / (step_ms * 1e-3)},
            "gpu_launches": int(launches), "clocks": sampler.summary(t_wall0, t_wall1), **check}


def run_cfg4(args, rank: int, world: int, local_rank: int) -> None:
    torch, dist, barrier = _dist_setup(world, local_rank)
    from shady_thinker_b200.gpu import GpuContext
    stream = torch.cuda.Stream()
    gpu = GpuContext(local_rank, stream=stream.cuda_stream)
    m = measure_cfg4(gpu, stream, rank, world, local_rank, dist, barrier, args.steps, args.warmup)
    if rank == 0:
        cfg_keys = ("workload", "context", "num_q_heads", "num_kv_heads", "head_dim", "kv_dtype", "rows_per_gpu", "combine", "l2")
        print(json.dumps({
            "metric": m["metric"], "value": m["value"], "unit": m["unit"], "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": m["ms_per_step"], "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": {k: m[k] for k in cfg_keys},
            "roofline": m["roofline"], "gpu_launches": m["gpu_launches"], "clocks": m["clocks"],
            "self_check": {k: m[k] for k in m if k in ("self_check", "rel_err_vs_one_rank", "tolerance", "against")}}), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    gpu.close()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU leg (profiling runs)")
    ap.add_argument("--kv", default="fp16", choices=["fp16", "fp8", "fp8e5m2"],
                    help="cfg2 only: storage of the KV cache (fp8 = e4m3, fp8e5m2 = e5m2 rows written by the quantising append)")
    ap.add_argument("--prefill-hd", type=int, default=128, choices=[128, 256],
                    help="cfg3 only: 256 = the wide-head kernel on nh16/nkv2/hd256 (same batch and length)")
    ap.add_argument("--no-extra", action="store_true",
                    help="cfg2 only: skip the short cfg3 (prefill) and cfg4 (long context) legs added to the line as `extra`")
    ap.add_argument("--shape", default="plain", choices=["plain", "reference"],
                    help="cfg2 only: plain = full rotary, no norm, no gate; reference = the reference's defaults "
                         "(rotary_dim = head_dim/4, QK RMSNorm, sigmoid gate)")
    ap.add_argument("--workload", default="cfg2", choices=["cfg1", "cfg2", "cfg3", "cfg4", "cfg5"],
                    help="cfg2 = batched ragged decode (default, the headline); cfg3 = causal prefill; "
                         "cfg1/cfg4/cfg5 = the other BASELINE configs")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.steps == 2000:   # the default suits cfg2 (0.1 ms steps); scale it for the others
        args.steps = {"cfg1": 300, "cfg3": 200, "cfg5": 5}.get(args.workload, 2000)
    set_prefill_shape(args.prefill_hd)
    if args.impl == "reference":
        (run_reference_prefill if args.workload == "cfg3" else run_reference)(args, rank)   # decode configs share the cfg2 sample
        return
    if world != args.gpus and world == 1 and args.gpus > 1:
        sys.exit("launch with torch.distributed.run --nproc-per-node N for --gpus N")
    runner = {"cfg2": run_ours, "cfg3": run_prefill, "cfg4": run_cfg4}.get(args.workload)
    if runner is None:
        from shady_thinker_b200 import extra_workloads
        runner = getattr(extra_workloads, "run_" + args.workload)
    runner(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
