"""The INT4 (GPTQ) projections that feed the attention path, alone and with the append as their epilogue.

Oracle: ``oracle.gptq_matvec`` (gptq_matvec.wgsl, one f32 chain per column) followed, for the fused launch, by
``oracle.fused_split_qknorm_kvstore`` on the three projected vectors — the reference's four dispatches
(model.rs:698-714, 723).  fp32 outputs within 1e-3 absolute (the split-K sum adds the same terms in another order).
"""
import numpy as np
import pytest
import torch

from _util import ATOL_F32, RTOL_16, rel_err, to_dev, to_host
from shady_thinker_b200 import ops
from shady_thinker_b200._lib import BF16, F8E4M3, F32

pytestmark = pytest.mark.gpu


def _weight(rng, K, N, gs):
    """Random INT4 weight in the reference's layout; scales sized so that a projection of N(0,1) inputs is O(1)."""
    qw = rng.integers(0, 2 ** 32, (K // 8, N), dtype=np.uint64).astype(np.uint32)
    sc = ((rng.random((K // gs, N)) + 0.5) * (1.0 / (4.6 * np.sqrt(K)))).astype(np.float16)
    dev = ops.GptqMatrix(torch.from_numpy(qw.view(np.int32)).cuda(), torch.from_numpy(sc).cuda(), K, N, gs)
    return qw, sc, dev


@pytest.mark.parametrize("K,N,gs,vecs", [(2048, 1536, 128, 1), (1024, 300, 32, 3), (5120, 512, 128, 5), (64, 40, 64, 2)])
def test_gptq_matvec_matches_the_shader_restatement(gpu_ctx, oracle, K, N, gs, vecs):
    rng = np.random.default_rng(K + N)
    qw, sc, w = _weight(rng, K, N, gs)
    x = oracle.randn((vecs, K), 91, 1)
    d_y = torch.full((vecs, N), float("nan"), device="cuda")
    ops.gptq_matvec(gpu_ctx, w, to_dev(x), d_y, vecs)
    gpu_ctx.synchronize()
    for v in range(vecs):
        want = oracle.gptq_matvec(x[v], qw, sc, gs)
        assert np.abs(to_host(d_y)[v] - want).max() <= ATOL_F32, v


@pytest.mark.parametrize("hd,nh,nkv,kv_dt,S,gate", [(128, 16, 2, F32, 1, True), (256, 4, 2, F32, 2, True),
                                                    (128, 8, 4, BF16, 5, False), (128, 4, 2, F8E4M3, 2, True)])
def test_projections_and_append_in_one_launch(gpu_ctx, oracle, hd, nh, nkv, kv_dt, S, gate):
    K, gs, rd = 1024, 128, hd // 4
    rng = np.random.default_rng(hd + nh + S)
    qcols = (2 if gate else 1) * hd
    qw_q, sc_q, wq = _weight(rng, K, nh * qcols, gs)
    qw_k, sc_k, wk = _weight(rng, K, nkv * hd, gs)
    qw_v, sc_v, wv = _weight(rng, K, nkv * hd, gs)
    x = oracle.randn((S, K), 92, 1)
    w = oracle.bf16_bits(oracle.randn((2 * hd,), 92, 2) * np.float32(0.02))
    pos = np.array([7, 100_003, 0, 31, 4095][:S], np.uint32)
    cap = int(pos.max()) + 1
    ks, vs = (0.5, 0.25) if kv_dt == F8E4M3 else (0.0, 0.0)
    tdt = {F32: torch.float32, BF16: torch.bfloat16, F8E4M3: torch.float8_e4m3fn}[kv_dt]
    d_kc = torch.zeros((S, cap, nkv, hd), dtype=tdt, device="cuda")
    d_vc = torch.zeros_like(d_kc)
    d_q = torch.full((S, nh, hd), float("nan"), device="cuda")
    d_g = torch.full((S, nh, hd), float("nan"), device="cuda") if gate else None
    ops.qkv_proj_append(gpu_ctx, wq=wq, wk=wk, wv=wv, x=to_dev(x), q_out=d_q, q_gate=d_g,
                        cache=ops.KvCacheView(kv_dt, d_kc, d_vc, cap * nkv * hd, k_scale=ks, v_scale=vs),
                        pos_start=torch.from_numpy(pos.astype(np.int32)).cuda(), num_heads=nh, num_kv_heads=nkv, head_dim=hd,
                        rope_theta=1e6, rotary_dim=rd, qk_norm_bf16=torch.from_numpy(w.view(np.int16)).cuda(), num_seqs=S,
                        has_gate=gate)
    gpu_ctx.synchronize()
    for s in range(S):
        qf = oracle.gptq_matvec(x[s], qw_q, sc_q, gs).reshape(nh, 2 if gate else 1, hd)
        if not gate:
            qf = np.concatenate([qf, np.zeros_like(qf)], 1)
        kp = oracle.gptq_matvec(x[s], qw_k, sc_k, gs).reshape(nkv, hd)
        vp = oracle.gptq_matvec(x[s], qw_v, sc_v, gs).reshape(nkv, hd)
        okc, ovc = np.zeros((1, nkv, hd), np.float32), np.zeros((1, nkv, hd), np.float32)
        oq, og, _ = oracle.fused_split_qknorm_kvstore(qf, kp, vp, okc, ovc, int(pos[s]), rope_theta=1e6, rotary_dim=rd,
                                                      qk_norm_bf16=w, cache_position=0)
        assert np.abs(to_host(d_q)[s] - oq).max() <= ATOL_F32, s
        if gate:
            assert np.abs(to_host(d_g)[s] - og).max() <= ATOL_F32, s
        got_k = d_kc[s, int(pos[s])].float().cpu().numpy() * np.float32(ks or 1.0)
        got_v = d_vc[s, int(pos[s])].float().cpu().numpy() * np.float32(vs or 1.0)
        if kv_dt == F32:
            assert np.abs(got_k - okc[0]).max() <= ATOL_F32 and np.abs(got_v - ovc[0]).max() <= ATOL_F32
        elif kv_dt == BF16:
            assert rel_err(got_k, okc[0]) <= 2.0 ** -7 and rel_err(got_v, ovc[0]) <= 2.0 ** -7
        else:   # one e4m3 step at most (values that sit on a rounding boundary)
            for got, want, sc in ((got_k, oracle.round_e4m3(okc[0], ks), ks), (got_v, oracle.round_e4m3(ovc[0], vs), vs)):
                assert np.all(np.abs(got - want) <= np.maximum(np.abs(want), sc * 2.0 ** -6) * 0.126)
        # rows other than the position stay untouched
        if int(pos[s]) > 0:
            assert float(d_kc[s, int(pos[s]) - 1].float().abs().max()) == 0.0


def test_a_decode_step_from_the_hidden_state(gpu_ctx, oracle):
    """Projections + append (one launch), attention with the gate in its epilogue (one launch): the self-attention
    block of model.rs:698-725 from the normed hidden state to the gated attention output, fp32 as in the reference."""
    K, gs, nh, nkv, hd, L = 2048, 128, 16, 2, 128, 300
    rng = np.random.default_rng(5)
    qw_q, sc_q, wq = _weight(rng, K, nh * 2 * hd, gs)
    qw_k, sc_k, wk = _weight(rng, K, nkv * hd, gs)
    qw_v, sc_v, wv = _weight(rng, K, nkv * hd, gs)
    x = oracle.randn((K,), 93, 1)
    okc, ovc = np.zeros((L, nkv, hd), np.float32), np.zeros((L, nkv, hd), np.float32)
    okc[:L - 1], ovc[:L - 1] = oracle.randn((L - 1, nkv, hd), 93, 2), oracle.randn((L - 1, nkv, hd), 93, 3)
    d_kc, d_vc = to_dev(okc), to_dev(ovc)
    cache = ops.KvCacheView(F32, d_kc, d_vc, 0)
    d_q, d_g = torch.empty((nh, hd), device="cuda"), torch.empty((nh, hd), device="cuda")
    d_out = torch.empty((1, nh, hd), device="cuda")
    ops.qkv_proj_append(gpu_ctx, wq=wq, wk=wk, wv=wv, x=to_dev(x), q_out=d_q, q_gate=d_g, cache=cache,
                        pos_start=torch.tensor([L - 1], dtype=torch.int32).cuda(), num_heads=nh, num_kv_heads=nkv,
                        head_dim=hd, rope_theta=1e7, rotary_dim=32)
    ws_n = ops.decode_workspace_size(head_dim=hd, num_kv_heads=nkv, num_q_heads=nh, num_splits=0, num_seqs=1)
    ws = torch.zeros(ws_n, dtype=torch.uint8, device="cuda")
    ops.attn_decode(gpu_ctx, q=d_q, cache=cache, seq_lens=torch.tensor([L], dtype=torch.int32).cuda(), out=d_out, head_dim=hd,
                    num_kv_heads=nkv, num_q_heads=nh, num_splits=0, seq_lens_host=[L], gate=d_g, workspace=ws,
                    workspace_bytes=ws_n)
    gpu_ctx.synchronize()
    qf = oracle.gptq_matvec(x, qw_q, sc_q, gs).reshape(nh, 2, hd)
    kp = oracle.gptq_matvec(x, qw_k, sc_k, gs).reshape(nkv, hd)
    vp = oracle.gptq_matvec(x, qw_v, sc_v, gs).reshape(nkv, hd)
    oq, og, _ = oracle.fused_split_qknorm_kvstore(qf, kp, vp, okc, ovc, L - 1, rope_theta=1e7, rotary_dim=32)
    want = oracle.sigmoid_mul(oracle.gqa_attention_head(oq, okc, ovc, L), og).reshape(nh, hd)
    assert np.abs(to_host(d_out)[0] - want).max() <= ATOL_F32
