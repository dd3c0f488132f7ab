"""The fused exchange+merge kernel (shady_attn_combine_p2p): alone on one GPU (world 1), and across two GPUs as
child processes when the box has them (row-sharded decode of one sequence, merged over peer memory, against the
oracle's unsharded attention)."""
import os
import sys

import numpy as np
import pytest
import torch

from _util import RTOL_16, rel_err, to_dev, to_host
from shady_thinker_b200._lib import BF16, F32

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_world_of_one_is_a_copy_with_gate(gpu_ctx, oracle):
    from shady_thinker_b200.p2p import ShardCombiner
    nh, hd = 16, 256
    rec = oracle.randn((nh, hd + 2), 3, 1)
    gate = oracle.randn((nh, hd), 3, 2)
    comb = ShardCombiner(gpu_ctx, rank=0, world=1, num_heads=nh, head_dim=hd)
    d_out = torch.full((nh, hd), float("nan"), device="cuda")
    for step in range(3):                       # epochs 1..3 reuse the two buffer generations
        comb.combine(to_dev(rec * (step + 1)), d_out, gate=to_dev(gate) if step == 2 else None)
        gpu_ctx.synchronize()
        want = rec[:, :hd] * (step + 1)
        if step == 2:
            want = oracle.sigmoid_mul(want, gate).reshape(nh, hd)
        assert np.abs(to_host(d_out) - want).max() <= 1e-5
    comb.close()


@pytest.fixture()
def knob_ctx(monkeypatch):
    """A context of its own per test: the SHADY_DECODE_* knobs are read once, when a context is created."""
    made = []

    def make(**env):
        from shady_thinker_b200.gpu import GpuContext
        for k, v in env.items():
            monkeypatch.setenv(k, v)
        made.append(GpuContext(0, stream=0x1))
        return made[-1]
    yield make
    for c in made:
        c.close()


@pytest.mark.parametrize("grid_merge,interleave", [("1", "1"), ("1", "0"), ("0", "1")])
@pytest.mark.parametrize("L", [100, 20000])
def test_world_of_one_fused_step_equals_plain_decode(knob_ctx, oracle, L, grid_merge, interleave):
    """decode + (merge, exchange, merge) with a world of one gives what shady_attn_decode gives: a single span (record
    written directly) and many spans (records merged before the exchange), as one cooperative launch (merge and
    exchange in the decode kernel's tail; blocks interleaved over the warps, the default, or in fixed spans) and as two
    launches (SHADY_DECODE_GRID_MERGE=0)."""
    gpu_ctx = knob_ctx(SHADY_DECODE_GRID_MERGE=grid_merge, SHADY_DECODE_INTERLEAVE=interleave)
    from _util import rounded, run_decode
    from shady_thinker_b200 import ops
    from shady_thinker_b200.p2p import ShardCombiner
    nh, nkv, hd = 16, 2, 256
    q = rounded(oracle, oracle.randn((1, nh, hd), 21, 1), BF16)
    k = rounded(oracle, oracle.randn((L, nkv, hd), 21, 2), BF16)
    v = rounded(oracle, oracle.randn((L, nkv, hd), 21, 3), BF16)
    gate = oracle.randn((nh, hd), 21, 4)
    view = ops.KvCacheView(BF16, to_dev(k, BF16), to_dev(v, BF16), 0)
    want = run_decode(gpu_ctx, q, view, [L], nh=nh, nkv=nkv, hd=hd, num_splits=0, q_dt=BF16, gate=to_dev(gate)[None])[0]
    comb = ShardCombiner(gpu_ctx, rank=0, world=1, num_heads=nh, head_dim=hd)
    ws_n = ops.decode_workspace_size(head_dim=hd, num_kv_heads=nkv, num_q_heads=nh, num_splits=0, num_seqs=1)
    ws = torch.zeros(max(ws_n, 4), dtype=torch.uint8, device="cuda")
    rec = torch.zeros((1, nh, hd + 2), device="cuda")
    lens = torch.tensor([L], dtype=torch.int32).cuda()
    n0 = gpu_ctx.launch_count
    for step in range(3):
        d_out = torch.full((nh, hd), float("nan"), device="cuda")
        comb.decode_and_combine(q=to_dev(q, BF16), cache=view, seq_lens=lens, seq_len_host=L, records=rec, out=d_out,
                                num_kv_heads=nkv, q_dtype=BF16, gate=to_dev(gate), workspace=ws, workspace_bytes=ws_n)
        gpu_ctx.synchronize()
        assert np.abs(to_host(d_out) - want).max() <= 2e-6 * max(1.0, float(np.abs(want).max()))
    assert gpu_ctx.launch_count - n0 == (3 if grid_merge == "1" and L > 512 else 6)   # a single span keeps two launches
    comb.close()


def _rank_main(rank, world, port, q_out):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from oracle import oracle as O
    from shady_thinker_b200 import ops
    from shady_thinker_b200.gpu import GpuContext
    from shady_thinker_b200.p2p import ShardCombiner
    from shady_thinker_b200.sharding import shard_rows
    nh, nkv, hd, L = 16, 2, 256, 3000
    gpu = GpuContext(rank, stream=0x1)
    k = O.round_bf16(O.randn((L, nkv, hd), 9, 2))
    v = O.round_bf16(O.randn((L, nkv, hd), 9, 3))
    lo, hi = shard_rows(L, world, rank)
    d_k = torch.from_numpy(k[lo:hi]).cuda().bfloat16()
    d_v = torch.from_numpy(v[lo:hi]).cuda().bfloat16()
    view = ops.KvCacheView(BF16, d_k, d_v, 0)
    lens = torch.tensor([hi - lo], dtype=torch.int32).cuda()
    ws_n = ops.decode_workspace_size(head_dim=hd, num_kv_heads=nkv, num_q_heads=nh, num_splits=0, num_seqs=1)
    ws = torch.zeros(ws_n, dtype=torch.uint8, device="cuda")
    comb = ShardCombiner(gpu, rank=rank, world=world, num_heads=nh, head_dim=hd)
    rec = torch.zeros((1, nh, hd + 2), device="cuda")
    out = torch.zeros((nh, hd), device="cuda")
    worst = 0.0
    for step in range(4):
        q = O.round_bf16(O.randn((1, nh, hd), 9, 100 + step))
        d_q = torch.from_numpy(q).cuda().bfloat16()
        torch.cuda.synchronize()
        ops.attn_decode_shard(gpu, q=d_q, cache=view, seq_lens=lens, records=rec, head_dim=hd, num_kv_heads=nkv,
                              num_q_heads=nh, num_splits=0, seq_lens_host=[hi - lo], q_dtype=BF16, workspace=ws,
                              workspace_bytes=ws_n)
        comb.combine(rec, out)
        gpu.synchronize()
        ref = O.attention_f64(q[0], k, v, L)
        got = out.cpu().numpy()
        worst = max(worst, float(np.abs(got - ref).max() / np.abs(ref).max()))
    comb.close()
    # the same step as decode + fused merge/exchange kernel (its own exchange buffer)
    comb2 = ShardCombiner(gpu, rank=rank, world=world, num_heads=nh, head_dim=hd)
    for step in range(4):
        q = O.round_bf16(O.randn((1, nh, hd), 9, 200 + step))
        d_q = torch.from_numpy(q).cuda().bfloat16()
        out.fill_(float("nan"))
        torch.cuda.synchronize()
        comb2.decode_and_combine(q=d_q, cache=view, seq_lens=lens, seq_len_host=hi - lo, records=rec, out=out,
                                 num_kv_heads=nkv, q_dtype=BF16, workspace=ws, workspace_bytes=ws_n)
        gpu.synchronize()
        ref = O.attention_f64(q[0], k, v, L)
        got = out.cpu().numpy()
        worst = max(worst, float(np.abs(got - ref).max() / np.abs(ref).max()))
    comb2.close()
    if rank == 0:
        q_out.put(worst)
    dist.barrier()
    dist.destroy_process_group()


def test_two_gpus_row_sharded_decode_with_peer_merge(oracle):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q_out = ctx.Queue()
    port = 29700 + os.getpid() % 200
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, q_out)) for r in range(2)]
    for p in procs:
        p.start()
    worst = q_out.get(timeout=180)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert worst <= RTOL_16
