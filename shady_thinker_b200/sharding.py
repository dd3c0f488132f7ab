"""How the path is cut across GPUs of one box (one process per GPU).

* Batched decode (cfg 2, cfg 5): sequences are independent, so they are dealt to ranks, longest first,
  each to the rank with the least rows so far; no data-path collective, outputs stay sharded.
* Long-context decode (cfg 4): the rows of one sequence are cut into contiguous ranges, one per rank; every
  rank produces records ``[nh][hd+2]`` (output, log-sum-exp, unused) for its rows, the records are gathered
  rank-major and merged with the ``gqa_reduce`` math (``ops.attn_reduce`` with ``split_stride = nh*(hd+2)``,
  ``head_stride = hd+2``).  The reference has no counterpart: it is single-device, and its split merge
  (src/shaders/gqa_reduce.wgsl) is the math that is reused across ranks.
"""
from __future__ import annotations

import numpy as np


def shard_rows(seq_len: int, world: int, rank: int) -> tuple[int, int]:
    """Contiguous row range [lo, hi) of rank ``rank``; 16-row aligned cuts, trailing ranks may be empty."""
    per = -(-seq_len // world)
    per = -(-per // 16) * 16
    lo = min(rank * per, seq_len)
    return lo, min(lo + per, seq_len)


def shard_sequences(lens, world: int) -> list[list[int]]:
    """Indices of the sequences each rank owns (greedy longest-first balance of total rows)."""
    lens = np.asarray(lens, dtype=np.int64)
    order = np.argsort(-lens, kind="stable")
    load = [0] * world
    owned: list[list[int]] = [[] for _ in range(world)]
    for i in order:
        r = int(np.argmin(load))
        owned[r].append(int(i))
        load[r] += int(lens[i])
    return [sorted(o) for o in owned]


def merge_args(num_seqs: int, num_heads: int, head_dim: int, world: int) -> dict:
    """Arguments of ``ops.attn_reduce`` that merge rank-major gathered records ``[world][num_seqs][nh][hd+2]``
    of ONE sequence (num_seqs == 1) into the final rows."""
    if num_seqs != 1:
        raise ValueError("rank-major merge is defined per sequence")
    return {"head_dim": head_dim, "num_splits": world, "num_heads": num_heads,
            "split_stride": num_seqs * num_heads * (head_dim + 2), "head_stride": head_dim + 2}
