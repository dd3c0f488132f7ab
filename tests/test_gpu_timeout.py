"""The status path of the bounded device-side waits, exercised by a wait that simply runs out.

A combiner of two ranks is built inside one process on one GPU (``loopback``): every entry of its peer table is
its own buffer and rank 1 does not exist, so rank 1's flag never arrives.  With the flag wait limited to a few
thousand polls the kernel gives up after some milliseconds, records its code and returns; nothing faults, nothing
hangs, and the context must be usable afterwards.
"""
import numpy as np
import pytest
import torch

from _util import rounded, run_decode, to_dev, to_host
from shady_thinker_b200 import ops
from shady_thinker_b200._lib import BF16, ERR_TIMEOUT, ShadyError
from shady_thinker_b200.gpu import GpuContext
from shady_thinker_b200.p2p import ShardCombiner

pytestmark = pytest.mark.gpu


@pytest.fixture()
def short_wait_ctx():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    torch.cuda.set_device(0)
    ctx = GpuContext(0, stream=0x1)
    ctx.set_wait_limits(peer_polls=1 << 12)
    yield ctx
    ctx.close()


def test_combine_gives_up_reports_the_rank_and_recovers(short_wait_ctx, oracle):
    gpu = short_wait_ctx
    nh, hd = 8, 128
    rec = oracle.randn((nh, hd + 2), 5, 1)
    d_out = torch.zeros((nh, hd), device="cuda")
    lone = ShardCombiner(gpu, rank=0, world=2, num_heads=nh, head_dim=hd, loopback=True)
    lone.combine(to_dev(rec), d_out)                 # launches; rank 1 never calls
    with pytest.raises(ShadyError) as e:
        gpu.synchronize()
    assert e.value.code == ERR_TIMEOUT and "rank 1" in str(e.value)
    gpu.synchronize()                                # the status was collected: clean again
    lone.close()
    # the context still works: a world of one merges its own record
    solo = ShardCombiner(gpu, rank=0, world=1, num_heads=nh, head_dim=hd)
    solo.combine(to_dev(rec), d_out)
    gpu.synchronize()
    assert np.abs(to_host(d_out) - rec[:, :hd]).max() <= 1e-6
    solo.close()


def test_uncollected_timeout_refuses_the_next_launch(short_wait_ctx, oracle):
    gpu = short_wait_ctx
    nh, hd = 8, 128
    rec = to_dev(oracle.randn((nh, hd + 2), 5, 2))
    d_out = torch.zeros((nh, hd), device="cuda")
    lone = ShardCombiner(gpu, rank=0, world=2, num_heads=nh, head_dim=hd, loopback=True)
    lone.combine(rec, d_out)
    torch.cuda.synchronize()                         # the host waits on its own: the library has not reported yet
    epoch = lone.epoch
    with pytest.raises(ShadyError) as e:
        lone.combine(rec, d_out)                     # refused before anything is launched
    assert e.value.code == ERR_TIMEOUT and "shady_synchronize" in str(e.value)
    assert lone.epoch == epoch                       # a refused call does not count as an exchange
    with pytest.raises(ShadyError):
        gpu.synchronize()                            # collects the status ...
    gpu.synchronize()                                # ... once
    lone.close()


@pytest.mark.parametrize("L", [200, 20000])
def test_fused_shard_step_gives_up_and_the_workspace_stays_usable(short_wait_ctx, oracle, L):
    """The same through the one-launch sharded step: the decode grid passes its barrier, the exchange waits for a
    rank that is not there, gives up, the grid leaves.  Afterwards the same workspace serves a world-of-one step
    whose rows equal the plain decode (the barrier words and counters were left clean)."""
    gpu = short_wait_ctx
    nh, nkv, hd = 16, 2, 256
    q = rounded(oracle, oracle.randn((1, nh, hd), 23, 1), BF16)
    k = rounded(oracle, oracle.randn((L, nkv, hd), 23, 2), BF16)
    v = rounded(oracle, oracle.randn((L, nkv, hd), 23, 3), BF16)
    view = ops.KvCacheView(BF16, to_dev(k, BF16), to_dev(v, BF16), 0)
    ws_n = ops.decode_workspace_size(head_dim=hd, num_kv_heads=nkv, num_q_heads=nh, num_splits=0, num_seqs=1)
    ws = torch.zeros(ws_n, dtype=torch.uint8, device="cuda")
    rec = torch.zeros((1, nh, hd + 2), device="cuda")
    lens = torch.tensor([L], dtype=torch.int32).cuda()
    d_out = torch.zeros((nh, hd), device="cuda")
    args = dict(q=to_dev(q, BF16), cache=view, seq_lens=lens, seq_len_host=L, records=rec, out=d_out, num_kv_heads=nkv,
                q_dtype=BF16, workspace=ws, workspace_bytes=ws_n)
    lone = ShardCombiner(gpu, rank=0, world=2, num_heads=nh, head_dim=hd, loopback=True)
    lone.decode_and_combine(**args)
    with pytest.raises(ShadyError) as e:
        gpu.synchronize()
    assert e.value.code == ERR_TIMEOUT and "rank 1" in str(e.value)
    lone.close()
    want = run_decode(gpu, q, view, [L], nh=nh, nkv=nkv, hd=hd, num_splits=0, q_dt=BF16)[0]
    solo = ShardCombiner(gpu, rank=0, world=1, num_heads=nh, head_dim=hd)
    d_out.fill_(float("nan"))
    solo.decode_and_combine(**args)
    gpu.synchronize()
    assert np.abs(to_host(d_out) - want).max() <= 2e-6 * max(1.0, float(np.abs(want).max()))
    solo.close()
