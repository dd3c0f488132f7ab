"""The reference's call surface end to end: Model.fused_split_qknorm_kvstore -> gqa_attention ->
sigmoid_mul_gate per token (model.rs:723-725), driven like generate_tokens (inference.rs:89-99),
against the oracle's token loop."""
import numpy as np
import pytest

from _util import ATOL_F32, RTOL_16, rel_err
from shady_thinker_b200._lib import BF16, F16, F32
from shady_thinker_b200.model import Model, ModelConfig

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("kv_dt,splits", [(F32, 1), (F32, 0), (F16, 0), (BF16, 2)])
def test_token_loop_matches_oracle(gpu_ctx, oracle, kv_dt, splits):
    cfg = ModelConfig(num_attention_heads=16, num_key_value_heads=2, num_hidden_layers=2, head_dim=128,
                      rope_theta=1e6, partial_rotary_factor=0.25)
    nh, nkv, hd, T = 16, 2, 128, 24
    m = Model(gpu_ctx, cfg, max_seq_len=64, kv_dtype=kv_dt, num_attn_splits=splits)
    w = [oracle.bf16_bits(oracle.randn((2 * hd,), 3, 90 + l) * np.float32(0.02)) for l in range(2)]
    for l in range(2):
        m.init_qknorm_params(gpu_ctx, l, w[l][:hd].tobytes(), w[l][hd:].tobytes())
    okc = [np.zeros((64, nkv, hd), np.float32) for _ in range(2)]
    ovc = [np.zeros((64, nkv, hd), np.float32) for _ in range(2)]
    m.seq_len = 0                                              # inference.rs:89
    for t in range(T):
        for l in range(2):
            qf = oracle.randn((nh, 2, hd), 3, 1000 + 10 * t + l)
            kp = oracle.randn((nkv, hd), 3, 2000 + 10 * t + l)
            vp = oracle.randn((nkv, hd), 3, 3000 + 10 * t + l)
            gpu_ctx.write_buffer(m.state.q_out, 0, qf.tobytes())
            gpu_ctx.write_buffer(m.state.k_out, 0, kp.tobytes())
            gpu_ctx.write_buffer(m.state.v_out, 0, vp.tobytes())
            m.attention_step(gpu_ctx, l)
            got = np.frombuffer(gpu_ctx.read_buffer(m.state.attn_output, nh * hd * 4), np.float32).reshape(nh, hd)
            oq, og, _ = oracle.fused_split_qknorm_kvstore(qf, kp, vp, okc[l], ovc[l], t, rope_theta=1e6,
                                                          rotary_dim=32, qk_norm_bf16=w[l])
            want = oracle.sigmoid_mul(oracle.gqa_attention_head(oq, okc[l], ovc[l], t + 1), og).reshape(nh, hd)
            if kv_dt == F32:
                assert np.abs(got - want).max() <= ATOL_F32, (t, l)
            else:
                assert rel_err(got, want) <= RTOL_16, (t, l)
        m.seq_len += 1                                          # model.rs:837


def test_cache_slot_swap_keeps_two_sequences_apart(gpu_ctx, oracle):
    cfg = ModelConfig(num_attention_heads=4, num_key_value_heads=2, head_dim=64, rope_theta=1e6)
    m = Model(gpu_ctx, cfg, max_seq_len=8, num_attn_splits=1)
    slot = m.alloc_cache_slot(gpu_ctx)
    outs = {}
    for name, seed in (("a", 1), ("b", 2), ("a2", 1)):
        if name == "b":
            m.swap_cache(slot)
        if name == "a2":
            m.swap_cache(slot)                                  # back to sequence a, continue it
        for t in range(2):
            step = t if name != "a2" else t + 2
            gpu_ctx.write_buffer(m.state.q_out, 0, oracle.randn((4, 2, 64), seed, 10 + step).tobytes())
            gpu_ctx.write_buffer(m.state.k_out, 0, oracle.randn((2, 64), seed, 20 + step).tobytes())
            gpu_ctx.write_buffer(m.state.v_out, 0, oracle.randn((2, 64), seed, 30 + step).tobytes())
            m.attention_step(gpu_ctx, 0)
            m.seq_len += 1
        outs[name] = np.frombuffer(gpu_ctx.read_buffer(m.state.attn_output, 4 * 64 * 4), np.float32).copy()
    assert m.seq_len == 4 and slot.seq_len == 2
    # continuing a after b must equal running a's four tokens without interruption
    m2 = Model(gpu_ctx, cfg, max_seq_len=8, num_attn_splits=1)
    for step in range(4):
        gpu_ctx.write_buffer(m2.state.q_out, 0, oracle.randn((4, 2, 64), 1, 10 + step).tobytes())
        gpu_ctx.write_buffer(m2.state.k_out, 0, oracle.randn((2, 64), 1, 20 + step).tobytes())
        gpu_ctx.write_buffer(m2.state.v_out, 0, oracle.randn((2, 64), 1, 30 + step).tobytes())
        m2.attention_step(gpu_ctx, 0)
        m2.seq_len += 1
    ref = np.frombuffer(gpu_ctx.read_buffer(m2.state.attn_output, 4 * 64 * 4), np.float32)
    np.testing.assert_array_equal(outs["a2"], ref)


def test_step_from_pinned_equals_step_from_host(gpu_ctx):
    """The zero-copy step (kernel reads activations from, and writes the output to, page-locked host memory)
    gives the bytes of the copy-based step; pageable memory is refused with a status, not a fault."""
    import torch
    from shady_thinker_b200 import ops
    from shady_thinker_b200._lib import F16, ShadyError
    from shady_thinker_b200.batch import BatchedDecoder
    S, nh, nkv, hd = 5, 8, 2, 128
    lens = np.array([17, 300, 1, 64, 1000], np.uint32)

    def make():
        d = BatchedDecoder(gpu_ctx, num_seqs=S, capacities=lens + 4, num_heads=nh, num_kv_heads=nkv, head_dim=hd,
                           kv_dtype=F16, rope_theta=1e6, rotary_dim=hd // 4, has_gate=True, num_splits=0)
        d.set_lengths(lens - 1)
        n = d.layer_bytes // 2
        ops.fill_randn(gpu_ctx, d.k_cache[0], n, F16, 7, 1)
        ops.fill_randn(gpu_ctx, d.v_cache[0], n, F16, 7, 2)
        return d

    g = torch.Generator().manual_seed(3)
    hq = torch.randn(S * nh * hd * 2, generator=g).half().pin_memory()
    hk = torch.randn(S * nkv * hd, generator=g).half().pin_memory()
    hv = torch.randn(S * nkv * hd, generator=g).half().pin_memory()
    out_a = torch.zeros(S * nh * hd, dtype=torch.float16).pin_memory()
    out_b = torch.zeros(S * nh * hd, dtype=torch.float16).pin_memory()
    make().step_from_host(hq.data_ptr(), hk.data_ptr(), hv.data_ptr(), out_a.data_ptr())
    make().step_from_pinned(hq.data_ptr(), hk.data_ptr(), hv.data_ptr(), out_b.data_ptr())
    assert torch.isfinite(out_a.float()).all() and out_a.abs().sum() > 0
    assert torch.equal(out_a, out_b)
    pageable = torch.zeros(16)
    with pytest.raises(ShadyError) as e:
        gpu_ctx.host_device_ptr(pageable.data_ptr())
    assert e.value.code == 1


def test_batched_decoder_many_steps_reuse_one_workspace(gpu_ctx):
    """Forty fused steps of a ragged batch through one BatchedDecoder (one workspace whose arrival counters reset
    themselves, lengths growing every step): the last step's output equals f64 attention over the cache rows the
    steps wrote, read back from the device."""
    import torch
    from shady_thinker_b200 import ops
    from shady_thinker_b200._lib import F16
    from shady_thinker_b200.batch import BatchedDecoder
    S, nh, nkv, hd, steps = 6, 8, 2, 128, 40
    start = np.array([0, 3, 100, 1000, 15, 2047], np.uint32)
    d = BatchedDecoder(gpu_ctx, num_seqs=S, capacities=start + steps, num_heads=nh, num_kv_heads=nkv, head_dim=hd,
                       kv_dtype=F16, rope_theta=1e6, rotary_dim=hd, has_gate=False, num_splits=0)
    n = d.layer_bytes // 2
    ops.fill_randn(gpu_ctx, d.k_cache[0], n, F16, 11, 1)
    ops.fill_randn(gpu_ctx, d.v_cache[0], n, F16, 11, 2)
    g = torch.Generator().manual_seed(5)
    for t in range(steps):
        d.set_lengths(start + t)
        q = torch.randn(S * nh * hd, generator=g).half().cuda()
        k = torch.randn(S * nkv * hd, generator=g).half().cuda()
        v = torch.randn(S * nkv * hd, generator=g).half().cuda()
        gpu_ctx.copy_buffer(q, d.q_in, q.numel() * 2)
        gpu_ctx.copy_buffer(k, d.k_in, k.numel() * 2)
        gpu_ctx.copy_buffer(v, d.v_in, v.numel() * 2)
        d.step()
    gpu_ctx.synchronize()
    out = np.frombuffer(gpu_ctx.read_buffer(d.out, d.out_bytes), np.float16).astype(np.float64).reshape(S, nh, hd)
    # the rotated q of the last step, recomputed on the host: full rotary, interleaved pairs, position L-1
    kc = np.frombuffer(gpu_ctx.read_buffer(d.k_cache[0], d.layer_bytes), np.float16).astype(np.float64)
    vc = np.frombuffer(gpu_ctx.read_buffer(d.v_cache[0], d.layer_bytes), np.float16).astype(np.float64)
    qh = q.cpu().numpy().astype(np.float64).reshape(S, nh, hd)
    i = np.arange(hd // 2)
    inv = (1.0 / np.power(np.float32(1e6), (2.0 * i / hd).astype(np.float32))).astype(np.float32)
    worst = 0.0
    for s in range(S):
        L = int(start[s]) + steps
        ang = (np.float32(L - 1) * inv).astype(np.float32).astype(np.float64)
        cs, sn = np.cos(ang), np.sin(ang)
        qr = qh[s].copy()
        qr[:, 0::2] = qh[s][:, 0::2] * cs - qh[s][:, 1::2] * sn
        qr[:, 1::2] = qh[s][:, 1::2] * cs + qh[s][:, 0::2] * sn
        qr = qr.astype(np.float16).astype(np.float64)          # the kernel stages Q in the cache dtype
        off = int(d.row_off[s]) * nkv * hd
        kk = kc[off:off + L * nkv * hd].reshape(L, nkv, hd)
        vv = vc[off:off + L * nkv * hd].reshape(L, nkv, hd)
        for h in range(nh):
            sc = kk[:, h // (nh // nkv)] @ qr[h] / np.sqrt(hd)
            pr = np.exp(sc - sc.max())
            ref = (pr[:, None] * vv[:, h // (nh // nkv)]).sum(0) / pr.sum()
            worst = max(worst, float(np.abs(out[s, h] - ref).max() / np.abs(ref).max()))
    assert worst <= RTOL_16, worst
