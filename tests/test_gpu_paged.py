"""Paged KV cache (pages of a shared pool + per-sequence page tables) against the contiguous cache: the same
rows behind a scrambled page table must give the same bytes out of the same kernels, and appends must land
in the rows the table names."""
import numpy as np
import pytest
import torch

from _util import RTOL_16, RaggedCache, rel_err, rounded, run_decode, to_dev, to_host
from shady_thinker_b200 import ops
from shady_thinker_b200._lib import BF16, F16, F32, ShadyError
from shady_thinker_b200.paged import PagedKvCache

pytestmark = pytest.mark.gpu
TDT = {F16: torch.float16, BF16: torch.bfloat16}


def _scrambled(gpu, lens, page_rows, nkv, hd, dt, seed):
    """A pool whose pages are handed out in shuffled order, each sequence sized to its length."""
    S = len(lens)
    need = sum((L + page_rows - 1) // page_rows for L in lens)
    pc = PagedKvCache(gpu, num_seqs=S, num_pages=need + 3, page_rows=page_rows, num_kv_heads=nkv, head_dim=hd,
                      kv_dtype=dt, max_pages_per_seq=max((L + page_rows - 1) // page_rows for L in lens) + 1)
    rng = np.random.default_rng(seed)
    rng.shuffle(pc.free)
    order = list(range(S))
    rng.shuffle(order)
    for s in order:
        pc.ensure(s, lens[s])
    return pc


def _fill_pool(pc, ks, vs, dt):
    kp = torch.zeros(pc.num_pages * pc.page_rows * pc.nkv * pc.hd, dtype=TDT[dt], device="cuda")
    vp = torch.full_like(kp, float("nan"))   # rows no table entry names must never be read into a result
    kp.fill_(float("nan"))
    row = pc.nkv * pc.hd
    for s, (k, v) in enumerate(zip(ks, vs)):
        dk, dv = to_dev(k, dt).reshape(-1), to_dev(v, dt).reshape(-1)
        for r0 in range(0, k.shape[0], pc.page_rows):
            n = min(pc.page_rows, k.shape[0] - r0)
            off = pc.row_offset(s, r0)
            kp[off:off + n * row] = dk[r0 * row:(r0 + n) * row]
            vp[off:off + n * row] = dv[r0 * row:(r0 + n) * row]
    pc.gpu.copy_buffer(kp, pc.k_pool, kp.numel() * 2)
    pc.gpu.copy_buffer(vp, pc.v_pool, vp.numel() * 2)
    pc.gpu.synchronize()


@pytest.mark.parametrize("dt,hd,nh,nkv,page_rows", [(F16, 128, 8, 2, 64), (BF16, 256, 8, 2, 16), (F16, 128, 32, 8, 256)])
def test_paged_decode_equals_contiguous_bit_for_bit(gpu_ctx, oracle, dt, hd, nh, nkv, page_rows):
    lens = [1, 15, 16, 17, 700, 64, 3000, 257]
    S = len(lens)
    q = rounded(oracle, oracle.randn((S, nh, hd), 91, 1), dt)
    ks = [rounded(oracle, oracle.randn((L, nkv, hd), 91, 10 + i), dt) for i, L in enumerate(lens)]
    vs = [rounded(oracle, oracle.randn((L, nkv, hd), 91, 50 + i), dt) for i, L in enumerate(lens)]
    flat = RaggedCache(ks, vs, dt)
    ref = run_decode(gpu_ctx, q, flat.view, lens, nh=nh, nkv=nkv, hd=hd, num_splits=0, q_dt=dt, out_dt=dt)
    pc = _scrambled(gpu_ctx, lens, page_rows, nkv, hd, dt, 5)
    _fill_pool(pc, ks, vs, dt)
    out = run_decode(gpu_ctx, q, pc.view, lens, nh=nh, nkv=nkv, hd=hd, num_splits=0, q_dt=dt, out_dt=dt)
    assert np.array_equal(out, ref)
    one = run_decode(gpu_ctx, q, pc.view, lens, nh=nh, nkv=nkv, hd=hd, num_splits=1, q_dt=dt, out_dt=F32)
    want = oracle.batched_decode(q, ks, vs, lens)
    for i in range(S):
        assert rel_err(one[i], want[i]) <= RTOL_16


def test_paged_append_then_fused_step_match_the_contiguous_cache(gpu_ctx, oracle):
    """Tokens appended one step at a time across page boundaries: the two-call step and the fused step on the paged
    cache give the bytes of the same steps on per-sequence contiguous caches."""
    dt, hd, nh, nkv, page_rows, S = F16, 128, 8, 2, 16, 3
    start = [14, 31, 0]
    steps = 5
    cap = [s + steps for s in start]
    ks = [rounded(oracle, oracle.randn((c, nkv, hd), 93, 10 + i), dt) for i, c in enumerate(cap)]
    vs = [rounded(oracle, oracle.randn((c, nkv, hd), 93, 20 + i), dt) for i, c in enumerate(cap)]
    flat = RaggedCache(ks, vs, dt)
    pc = _scrambled(gpu_ctx, [max(s, 1) for s in start], page_rows, nkv, hd, dt, 9)
    _fill_pool(pc, [k[:max(s, 1)] for k, s in zip(ks, start)], [v[:max(s, 1)] for v, s in zip(vs, start)], dt)
    ws_bytes = ops.decode_workspace_size(head_dim=hd, num_kv_heads=nkv, num_q_heads=nh, num_splits=0, num_seqs=S)
    outs = {}
    for name, view in (("flat", flat.view), ("paged", pc.view)):
        ws = torch.zeros(max(ws_bytes, 4), dtype=torch.uint8, device="cuda")
        ops.decode_workspace_init(gpu_ctx, ws, ws_bytes, head_dim=hd, num_kv_heads=nkv, num_q_heads=nh, num_splits=0, num_seqs=S)
        res = []
        for t in range(steps):
            lens = [s + t + 1 for s in start]
            if name == "paged":
                for s in range(S):
                    pc.ensure(s, lens[s])
            qf = to_dev(rounded(oracle, oracle.randn((S, nh, 2 * hd), 94, t), dt), dt)
            kp = to_dev(rounded(oracle, oracle.randn((S, nkv, hd), 95, t), dt), dt)
            vp = to_dev(rounded(oracle, oracle.randn((S, nkv, hd), 96, t), dt), dt)
            d_lens = torch.tensor(lens, dtype=torch.int32).cuda()
            d_out = torch.empty((S, nh, hd), dtype=TDT[dt], device="cuda")
            if t % 2 == 0:   # fused launch
                ops.attn_decode_append(gpu_ctx, q_proj_full=qf, k_proj=kp, v_proj=vp, cache=view, seq_lens=d_lens, out=d_out,
                                       num_heads=nh, num_kv_heads=nkv, head_dim=hd, rope_theta=1e6, rotary_dim=hd // 4,
                                       num_seqs=S, in_dtype=dt, out_dtype=dt, has_gate=True, seq_lens_host=lens,
                                       workspace=ws, workspace_bytes=ws_bytes)
            else:            # append kernel, then attend with the gate
                d_pos = torch.tensor([l - 1 for l in lens], dtype=torch.int32).cuda()
                q_rot = torch.empty((S, nh, hd), dtype=TDT[dt], device="cuda")
                gate = torch.empty((S, nh, hd), dtype=torch.float32, device="cuda")
                ops.kv_append_rope(gpu_ctx, q_proj_full=qf, k_proj=kp, v_proj=vp, q_out=q_rot, q_gate=gate, cache=view,
                                   pos_start=d_pos, num_heads=nh, num_kv_heads=nkv, head_dim=hd, rope_theta=1e6,
                                   rotary_dim=hd // 4, num_seqs=S, tokens_per_seq=1, in_dtype=dt, q_dtype=dt,
                                   has_gate=True, write_k_back=False)
                ops.attn_decode(gpu_ctx, q=q_rot, cache=view, seq_lens=d_lens, out=d_out, head_dim=hd, num_kv_heads=nkv,
                                num_q_heads=nh, num_seqs=S, num_splits=0, seq_lens_host=lens, q_dtype=dt, out_dtype=dt,
                                gate=gate, workspace=ws, workspace_bytes=ws_bytes)
            gpu_ctx.synchronize()
            res.append(to_host(d_out))
        outs[name] = res
    for t in range(steps):
        assert np.isfinite(outs["flat"][t]).all()
        assert np.array_equal(outs["paged"][t], outs["flat"][t]), t


def test_paged_cache_is_refused_where_it_cannot_work(gpu_ctx):
    d = torch.zeros(4096, dtype=torch.float16, device="cuda")
    tab = torch.zeros(4, dtype=torch.int32, device="cuda")
    lens = torch.ones(1, dtype=torch.int32, device="cuda")
    out = torch.zeros(128, dtype=torch.float16, device="cuda")
    bad_rows = ops.KvCacheView(F16, d, d, 0, None, None, tab, 24, 4)         # not a multiple of 16
    f32_pages = ops.KvCacheView(F32, d, d, 0, None, None, tab, 16, 4)
    split = ops.KvCacheView(F16, d, d, 0, None, None, tab, 16, 4)
    for view, ns, code in ((bad_rows, 0, 1), (f32_pages, 0, 2), (split, 4, 2)):
        with pytest.raises(ShadyError) as e:
            ops.attn_decode(gpu_ctx, q=out, cache=view, seq_lens=lens, out=out, head_dim=128, num_kv_heads=1, num_q_heads=1,
                            num_seqs=1, num_splits=ns, seq_lens_host=[1], q_dtype=F16, out_dtype=F16,
                            workspace=d, workspace_bytes=8192)
        assert e.value.code == code
    with pytest.raises(ShadyError) as e:
        ops.attn_prefill(gpu_ctx, q=d, cache=split, out=d, head_dim=128, num_kv_heads=1, num_q_heads=1, num_seqs=1,
                         seq_len=8, dtype=F16)
    assert e.value.code == 2
