"""The benchmark configurations as they are written down, at parity-test size, against the oracle.

* config 1: 512 tokens pushed through ``shady_kv_append_rope`` (fp32, theta 1e6, positions 0..511) and then
  decoded — Q and K carry RoPE exactly as the append writes it, not as a test pre-rotates it — for full and
  quarter rotary, through the raw ops and through ``Model.attention_step`` (model.rs:723-725);
* config 5 in shape: several layers, each with its own cache holding different rows, one token per sequence
  appended per layer per step;
* the fused append+attend launch directly against the oracle at a position beyond 100,000, QK-norm and gate on.
"""
import numpy as np
import pytest
import torch

from _util import ATOL_F32, RTOL_16, rel_err, to_dev, to_host
from shady_thinker_b200 import ops
from shady_thinker_b200._lib import BF16, F16, F32
from shady_thinker_b200.batch import BatchedDecoder
from shady_thinker_b200.model import Model, ModelConfig

pytestmark = pytest.mark.gpu


def _oracle_token_path(oracle, qf, kp, vp, T, rd, w):
    """fused_split_qknorm_kvstore for tokens 0..T-1 in order, then gqa_attention_head for the last one."""
    nkv, hd = kp.shape[1], kp.shape[2]
    okc, ovc = np.zeros((T, nkv, hd), np.float32), np.zeros((T, nkv, hd), np.float32)
    oq = og = None
    for t in range(T):
        oq, og, _ = oracle.fused_split_qknorm_kvstore(qf[t], kp[t], vp[t], okc, ovc, t, rope_theta=1e6, rotary_dim=rd,
                                                      qk_norm_bf16=w)
    return oq, og, okc, ovc


@pytest.mark.parametrize("rd", [128, 32])
@pytest.mark.parametrize("norm", [False, True])
def test_config1_rows_written_by_the_append_then_decoded(gpu_ctx, oracle, rd, norm):
    nh, nkv, hd, T = 16, 2, 128, 512
    qf = oracle.randn((T, nh, 2, hd), 41, 1)
    kp = oracle.randn((T, nkv, hd), 41, 2)
    vp = oracle.randn((T, nkv, hd), 41, 3)
    w = oracle.bf16_bits(oracle.randn((2 * hd,), 41, 4) * np.float32(0.02)) if norm else None
    d_w = torch.from_numpy(w.view(np.int16)).cuda() if norm else None
    d_kc = torch.zeros((T, nkv, hd), device="cuda")
    d_vc = torch.zeros((T, nkv, hd), device="cuda")
    cache = ops.KvCacheView(F32, d_kc, d_vc, 0)
    d_q = torch.empty((T, nh, hd), device="cuda")
    d_g = torch.empty((T, nh, hd), device="cuda")
    # tokens 0..510 in one batched append, token 511 by the single-token call the decode step makes
    common = dict(cache=cache, num_heads=nh, num_kv_heads=nkv, head_dim=hd, rope_theta=1e6, rotary_dim=rd,
                  qk_norm_bf16=d_w)
    ops.kv_append_rope(gpu_ctx, q_proj_full=to_dev(qf[:T - 1]), k_proj=to_dev(kp[:T - 1]), v_proj=to_dev(vp[:T - 1]),
                       q_out=d_q, q_gate=d_g, pos_start=torch.zeros(1, dtype=torch.int32).cuda(), num_seqs=1,
                       tokens_per_seq=T - 1, **common)
    ops.kv_append_rope(gpu_ctx, q_proj_full=to_dev(qf[T - 1]), k_proj=to_dev(kp[T - 1]), v_proj=to_dev(vp[T - 1]),
                       q_out=d_q[T - 1], q_gate=d_g[T - 1], pos_start=torch.tensor([T - 1], dtype=torch.int32).cuda(),
                       **common)
    oq, og, okc, ovc = _oracle_token_path(oracle, qf, kp, vp, T, rd, w)
    assert np.abs(to_host(d_kc) - okc).max() <= ATOL_F32
    assert np.abs(to_host(d_q[T - 1]) - oq.reshape(nh, hd)).max() <= ATOL_F32
    want = oracle.gqa_attention_head(oq, okc, ovc, T).reshape(nh, hd)
    for ns in (1, 0):
        d_out = torch.full((1, nh, hd), float("nan"), device="cuda")
        ws_n = ops.decode_workspace_size(head_dim=hd, num_kv_heads=nkv, num_q_heads=nh, num_splits=ns, num_seqs=1)
        ws = torch.zeros(max(ws_n, 4), dtype=torch.uint8, device="cuda")
        ops.attn_decode(gpu_ctx, q=d_q[T - 1], cache=cache, seq_lens=torch.tensor([T], dtype=torch.int32).cuda(),
                        out=d_out, head_dim=hd, num_kv_heads=nkv, num_q_heads=nh, num_splits=ns, seq_lens_host=[T],
                        workspace=ws, workspace_bytes=ws_n)
        gpu_ctx.synchronize()
        assert np.abs(to_host(d_out)[0] - want).max() <= ATOL_F32, ns


def test_config1_through_the_model_surface(gpu_ctx, oracle):
    """512 calls of Model.attention_step (append, attend, gate: model.rs:723-725) on one layer, fp32, full rotary."""
    nh, nkv, hd, T = 16, 2, 128, 512
    cfg = ModelConfig(num_attention_heads=nh, num_key_value_heads=nkv, head_dim=hd, rope_theta=1e6,
                      partial_rotary_factor=1.0)
    m = Model(gpu_ctx, cfg, max_seq_len=T, kv_dtype=F32, num_attn_splits=0)
    qf = oracle.randn((T, nh, 2, hd), 43, 1)
    kp = oracle.randn((T, nkv, hd), 43, 2)
    vp = oracle.randn((T, nkv, hd), 43, 3)
    okc, ovc = np.zeros((T, nkv, hd), np.float32), np.zeros((T, nkv, hd), np.float32)
    m.seq_len = 0
    for t in range(T):
        gpu_ctx.write_buffer(m.state.q_out, 0, qf[t].tobytes())
        gpu_ctx.write_buffer(m.state.k_out, 0, kp[t].tobytes())
        gpu_ctx.write_buffer(m.state.v_out, 0, vp[t].tobytes())
        m.attention_step(gpu_ctx, 0)
        oq, og, _ = oracle.fused_split_qknorm_kvstore(qf[t], kp[t], vp[t], okc, ovc, t, rope_theta=1e6, rotary_dim=hd)
        if t % 73 == 0 or t == T - 1:
            got = np.frombuffer(gpu_ctx.read_buffer(m.state.attn_output, nh * hd * 4), np.float32).reshape(nh, hd)
            want = oracle.sigmoid_mul(oracle.gqa_attention_head(oq, okc, ovc, t + 1), og).reshape(nh, hd)
            assert np.abs(got - want).max() <= ATOL_F32, t
        m.seq_len += 1


def _f64_rows(oracle, q, kc, vc, L):
    return oracle.attention_f64(np.ascontiguousarray(q, np.float32), np.ascontiguousarray(kc[:L], np.float32),
                                np.ascontiguousarray(vc[:L], np.float32), L)


def test_config5_shape_layers_keep_their_own_caches(gpu_ctx, oracle):
    """Three layers, four sequences, three steps: every layer's cache starts with different rows and receives its own
    new row per step; each layer's output is checked against f64 attention over a host mirror of that layer."""
    S, nh, nkv, hd, layers, steps = 4, 8, 2, 128, 3, 3
    start = np.array([5, 300, 17, 1024], np.uint32)
    d = BatchedDecoder(gpu_ctx, num_seqs=S, capacities=start + steps, num_heads=nh, num_kv_heads=nkv, head_dim=hd,
                       kv_dtype=F16, rope_theta=1e6, rotary_dim=hd, has_gate=False, num_layers=layers, num_splits=0)
    rows = int(d.row_off[-1])
    hk = [oracle.round_f16(oracle.randn((rows, nkv, hd), 61, 10 + l)) for l in range(layers)]
    hv = [oracle.round_f16(oracle.randn((rows, nkv, hd), 61, 20 + l)) for l in range(layers)]
    for l in range(layers):
        gpu_ctx.write_buffer(d.k_cache[l], 0, hk[l].astype(np.float16).tobytes())
        gpu_ctx.write_buffer(d.v_cache[l], 0, hv[l].astype(np.float16).tobytes())
    worst = 0.0
    for t in range(steps):
        d.set_lengths(start + t)
        for l in range(layers):
            q = oracle.round_f16(oracle.randn((S, nh, hd), 61, 100 + 10 * t + l))
            k = oracle.round_f16(oracle.randn((S, nkv, hd), 61, 200 + 10 * t + l))
            v = oracle.round_f16(oracle.randn((S, nkv, hd), 61, 300 + 10 * t + l))
            gpu_ctx.write_buffer(d.q_in, 0, q.astype(np.float16).tobytes())
            gpu_ctx.write_buffer(d.k_in, 0, k.astype(np.float16).tobytes())
            gpu_ctx.write_buffer(d.v_in, 0, v.astype(np.float16).tobytes())
            d.step(l)
            gpu_ctx.synchronize()
            out = np.frombuffer(gpu_ctx.read_buffer(d.out, d.out_bytes), np.float16).astype(np.float32).reshape(S, nh, hd)
            for s in range(S):
                pos = int(start[s]) + t
                r0 = int(d.row_off[s])
                # host mirror of the append: full rotary, no norm, no gate (q_proj_full rows are [Q] only)
                oq, _, _ = oracle.fused_split_qknorm_kvstore(np.stack([q[s], q[s]], 1), k[s], v[s], hk[l][r0:], hv[l][r0:],
                                                             pos, rope_theta=1e6, rotary_dim=hd)
                hk[l][r0 + pos] = oracle.round_f16(hk[l][r0 + pos])
                ref = _f64_rows(oracle, oracle.round_f16(oq.reshape(nh, hd)), hk[l][r0:], hv[l][r0:], pos + 1)
                worst = max(worst, rel_err(out[s], ref))
    assert worst <= RTOL_16, worst
    # the layers' caches really differ: row `start` of sequence 0 in layer 0 is not the one in layer 1
    kc0 = np.frombuffer(gpu_ctx.read_buffer(d.k_cache[0], 4096), np.float16)
    kc1 = np.frombuffer(gpu_ctx.read_buffer(d.k_cache[1], 4096), np.float16)
    assert not np.array_equal(kc0, kc1)


@pytest.mark.parametrize("dt,hd", [(F16, 128), (BF16, 256)])
def test_fused_append_decode_against_the_oracle_far_out(gpu_ctx, oracle, dt, hd):
    """One fused launch (norm + RoPE + cache store + attend + gate) at position 100,003: RoPE angles of 1e5 radians in
    f32, the new row patched into the tile stream; against the oracle's append followed by f64 attention."""
    nh, nkv, L = 4, 1, 100_004
    rd = hd // 4
    rnd = oracle.round_f16 if dt == F16 else oracle.round_bf16
    tdt = torch.float16 if dt == F16 else torch.bfloat16
    kc = rnd(oracle.randn((L, nkv, hd), 71, 1))
    vc = rnd(oracle.randn((L, nkv, hd), 71, 2))
    kc[L - 1] = 0
    vc[L - 1] = 0
    qf = rnd(oracle.randn((nh, 2, hd), 71, 3))
    kp = rnd(oracle.randn((nkv, hd), 71, 4))
    vp = rnd(oracle.randn((nkv, hd), 71, 5))
    w = oracle.bf16_bits(oracle.randn((2 * hd,), 71, 6) * np.float32(0.02))
    d_kc, d_vc = torch.from_numpy(kc).cuda().to(tdt), torch.from_numpy(vc).cuda().to(tdt)
    d_out = torch.full((1, nh, hd), float("nan"), device="cuda")
    ws_n = ops.decode_workspace_size(head_dim=hd, num_kv_heads=nkv, num_q_heads=nh, num_splits=0, num_seqs=1)
    ws = torch.zeros(ws_n, dtype=torch.uint8, device="cuda")
    ops.attn_decode_append(gpu_ctx, q_proj_full=torch.from_numpy(qf).cuda().to(tdt), k_proj=torch.from_numpy(kp).cuda().to(tdt),
                           v_proj=torch.from_numpy(vp).cuda().to(tdt), cache=ops.KvCacheView(dt, d_kc, d_vc, 0),
                           seq_lens=torch.tensor([L], dtype=torch.int32).cuda(), out=d_out, num_heads=nh,
                           num_kv_heads=nkv, head_dim=hd, rope_theta=1e6, rotary_dim=rd, num_seqs=1,
                           qk_norm_bf16=torch.from_numpy(w.view(np.int16)).cuda(), in_dtype=dt, out_dtype=F32,
                           has_gate=True, seq_lens_host=[L], workspace=ws, workspace_bytes=ws_n)
    gpu_ctx.synchronize()
    oq, og, _ = oracle.fused_split_qknorm_kvstore(qf, kp, vp, kc, vc, L - 1, rope_theta=1e6, rotary_dim=rd, qk_norm_bf16=w)
    # the cache row the launch stored is the oracle's row, rounded to the cache dtype
    got_row = d_kc[L - 1].float().cpu().numpy()
    assert rel_err(got_row, rnd(kc[L - 1])) <= 1e-2
    kc[L - 1] = rnd(kc[L - 1])
    ref = oracle.sigmoid_mul(oracle.attention_f64(rnd(oq.reshape(nh, hd)), kc, vc, L), og).reshape(nh, hd)
    assert rel_err(to_host(d_out)[0], ref) <= RTOL_16
