"""The N>1 host logic on CPU: two gloo ranks shard one long sequence by rows, build shard records with the
oracle, all-gather them and merge rank-major — and deal a ragged batch to ranks — exactly as the GPU path does
with NCCL and ``shady_attn_decode_shard`` / ``shady_attn_reduce``."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _rank_main(rank, world, port, L, out_q):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import oracle as O
    from shady_thinker_b200.sharding import merge_args, shard_rows, shard_sequences
    nh, nkv, hd = 8, 2, 64
    q, k, v = O.randn((nh, hd), 5, 1), O.randn((L, nkv, hd), 5, 2), O.randn((L, nkv, hd), 5, 3)
    lo, hi = shard_rows(L, world, rank)
    rec = np.zeros((nh, hd + 2), np.float32)
    if hi > lo:
        part = O.gqa_attention_head(q, k[lo:hi], v[lo:hi], hi - lo, num_splits=2)   # [nh][2][hd+2]
        rec[:, :hd] = O.gqa_reduce(part)
        lse = part[:, :, hd]
        m = lse.max(1)
        rec[:, hd] = m + np.log(np.exp(lse - m[:, None]).sum(1))
    else:
        rec[:, hd] = -np.inf
    mine = torch.from_numpy(rec.reshape(-1))
    gathered = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(gathered, mine)
    allrec = torch.stack(gathered).numpy().reshape(world, nh, hd + 2)
    ma = merge_args(1, nh, hd, world)
    assert ma["split_stride"] == nh * (hd + 2) and ma["head_stride"] == hd + 2
    merged = O.gqa_reduce(np.ascontiguousarray(allrec.transpose(1, 0, 2)), skip_empty=True)   # [nh][world][hd+2]
    ref = O.attention_f64(q, k, v, L)
    err = float(np.abs(merged - ref).max())
    owned = shard_sequences([100, 4000, 50, 3000, 2500, 10], world)
    if rank == 0:
        out_q.put((err, owned, [shard_rows(L, world, r) for r in range(world)]))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("L", [1000, 20])
def test_row_sharded_decode_merges_over_gloo(L):
    from oracle import oracle as O
    O.build()
    ctx = mp.get_context("spawn")
    out_q = ctx.Queue()
    port = 29600 + (os.getpid() + L) % 300
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, L, out_q)) for r in range(2)]
    for p in procs:
        p.start()
    err, owned, ranges = out_q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert err < 5e-6
    assert sorted(owned[0] + owned[1]) == list(range(6)) and not set(owned[0]) & set(owned[1])
    lens = np.array([100, 4000, 50, 3000, 2500, 10])
    assert abs(lens[owned[0]].sum() - lens[owned[1]].sum()) <= 2500      # balanced to within one sequence
    assert ranges[0][0] == 0 and ranges[-1][1] == L and ranges[0][1] == ranges[1][0]
    if L == 20:
        assert ranges[1] == (20, 20) or ranges[1][1] - ranges[1][0] <= 4  # the second shard is (nearly) empty


def test_shard_rows_covers_everything():
    from shady_thinker_b200.sharding import shard_rows
    for L in (0, 1, 15, 16, 17, 131072, 100003):
        for world in (1, 2, 4, 8):
            pos = 0
            for r in range(world):
                lo, hi = shard_rows(L, world, r)
                assert lo == pos and hi >= lo
                pos = hi
            assert pos == L
