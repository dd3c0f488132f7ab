// INT4 (GPTQ, symmetric) matrix-vector products of the attention block's q/k/v projections, with the KV append
// (RMSNorm(1+w), (m)RoPE, cache store) as their epilogue.
//
// What it computes: gptq_matvec.wgsl:20-82 — y[n] = sum_k ((nibble(k, n) - 8) * scale(k / group, n)) * x[k] over
// qweight [K/8][N] u32 (eight nibbles along K per word) and scales [K/group][N] f16 — three times (q, k, v:
// model.rs:698-714), followed by fused_split_qknorm_kvstore.wgsl:106-230 on the three results (model.rs:723).  The
// reference runs four dispatches and round-trips q_out / k_out / v_out through memory in f32; here one launch reads
// the weights once and the projected vectors never leave the chip.
//
// Layout of the work (a matvec is weight-bandwidth bound and, at one token, latency bound):
//   * a unit is what one epilogue needs whole: a Q head (its Q and gate columns: (1+gate)*hd adjacent columns of
//     the q weight) or a KV head (hd columns of the k weight and the same hd columns of the v weight);
//   * a unit is served by a thread-block CLUSTER of kSplit CTAs that split the K rows between them (split-K), so
//     a 16-head + 2-kv-head layer still fills 144 SMs; thread t of every CTA owns column t (t + 256, ...) of the
//     unit, so a warp reads 128 contiguous bytes of a weight row;
//   * the CTAs' partial sums meet in the first CTA of the cluster through distributed shared memory, and that CTA
//     runs the epilogue, one warp per head vector.
// Sums are f32; the order of the additions differs from the shader's single chain (as its own 4-thread variant,
// gptq_matvec_4t.wgsl, differs from it).
#include <cooperative_groups.h>

#include "append_core.cuh"

namespace cg = cooperative_groups;

namespace shady {

constexpr uint32_t kGptqThreads = 256;
constexpr uint32_t kGptqSplit = 8;       // CTAs per cluster (portable maximum)
constexpr uint32_t kGptqMaxCols = 512;   // columns of a unit: (1 + gate) * hd <= 512
constexpr uint32_t kGptqMaxSeqs = 4;     // tokens per pass over the weights

struct GptqW {
    const uint32_t *qweight;
    const uint16_t *scales;   // f16 bits, [K/group][N]
    uint32_t N;
};

struct QkvArgs {
    GptqW wq, wk, wv;
    const float *x;           // [num_seqs][K] f32 (the normed hidden state, model.rs:690)
    uint32_t K, group_size, num_seqs;
    // epilogue == 0: plain matvec of wq into y [num_seqs][N] (units are 256-column slices)
    uint32_t fused;
    float *y;
    // epilogue == 1: the append
    void *q_out;              // [num_seqs][nh][hd] in q_dtype
    float *q_gate;            // [num_seqs][nh][hd] f32 or NULL
    KvAddr kv;
    const uint16_t *norm_w;
    const uint32_t *pos_start, *pos_h, *pos_w;
    uint32_t nh, nkv, hd, has_gate, q_dtype, kv_dtype;
    RopeSpec rope;
    float k_inv, v_inv;
    float inv_freq[128];
};

template <int SB>
__global__ void __launch_bounds__(kGptqThreads) qkv_proj_kernel(const QkvArgs a, const uint32_t seq0) {
    cg::cluster_group cluster = cg::this_cluster();
    const uint32_t crank = cluster.block_rank(), csize = cluster.num_blocks();
    const uint32_t unit = blockIdx.x / csize;
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    extern __shared__ float sm[];
    // [SB][k rows of this CTA] inputs, then [SB][ncols] partial sums (read by the cluster's first CTA)
    const uint32_t packed_rows = a.K / 8;
    const uint32_t pr0 = (uint32_t)(((unsigned long long)packed_rows * crank) / csize);
    const uint32_t pr1 = (uint32_t)(((unsigned long long)packed_rows * (crank + 1)) / csize);
    const uint32_t kn = (pr1 - pr0) * 8;
    const uint32_t kmax = ((packed_rows + csize - 1) / csize + 1) * 8;   // same layout in every CTA of the cluster
    float *sm_x = sm;
    float *sm_part = sm + (size_t)SB * kmax;

    // which columns, of which weights
    uint32_t ncols, colbase[2], half_cols;
    const GptqW *w[2];
    if (!a.fused) {
        w[0] = w[1] = &a.wq;
        colbase[0] = unit * kGptqThreads; colbase[1] = 0;
        ncols = min(kGptqThreads, a.wq.N - colbase[0]); half_cols = ncols;
    } else if (unit < a.nh) {   // a Q head: Q columns then gate columns, adjacent in the q weight (wgsl:122-135)
        w[0] = w[1] = &a.wq;
        ncols = (a.has_gate ? 2u : 1u) * a.hd; half_cols = ncols;
        colbase[0] = unit * ncols; colbase[1] = 0;
    } else {                    // a KV head: hd columns of k, then the same hd columns of v
        w[0] = &a.wk; w[1] = &a.wv;
        ncols = 2 * a.hd; half_cols = a.hd;
        colbase[0] = colbase[1] = (unit - a.nh) * a.hd;
    }
    const uint32_t nseq = min((uint32_t)SB, a.num_seqs - seq0);
    for (uint32_t i = tid; i < SB * kn; i += kGptqThreads) {
        const uint32_t s = i / kn, k = i % kn;
        sm_x[s * kmax + k] = s < nseq ? a.x[(size_t)(seq0 + s) * a.K + pr0 * 8 + k] : 0.f;
    }
    __syncthreads();

    for (uint32_t c = tid; c < ncols; c += kGptqThreads) {
        const uint32_t which = c < half_cols ? 0u : 1u;
        const GptqW &W = *w[which];
        const uint32_t col = colbase[which] + (which ? c - half_cols : c);
        float acc[SB];
#pragma unroll
        for (int s = 0; s < SB; ++s) acc[s] = 0.f;
        const uint32_t *qp = W.qweight + (size_t)pr0 * W.N + col;
        uint32_t group = ~0u;
        float scale = 0.f;
        constexpr uint32_t U = 8;   // weight words in flight per thread
        for (uint32_t pr = pr0; pr < pr1; pr += U) {
            uint32_t packed[U];
#pragma unroll
            for (uint32_t u = 0; u < U; ++u) packed[u] = pr + u < pr1 ? __ldg(qp + (size_t)u * W.N) : 0x88888888u;   // nibble 8 = weight 0
            qp += (size_t)U * W.N;
#pragma unroll
            for (uint32_t u = 0; u < U; ++u) {
                const uint32_t g = ((pr + u) * 8u) / a.group_size;
                if (g != group && pr + u < pr1) {
                    group = g;
                    scale = __half2float(__ushort_as_half(W.scales[(size_t)g * W.N + col]));
                }
                const float *xk = sm_x + (pr + u - pr0) * 8;
#pragma unroll
                for (uint32_t nib = 0; nib < 8; ++nib) {
                    const float wv = ((float)((packed[u] >> (4 * nib)) & 0xFu) - 8.0f) * scale;   // wgsl:50
#pragma unroll
                    for (int s = 0; s < SB; ++s) acc[s] = fmaf(wv, pr + u < pr1 ? xk[s * kmax + nib] : 0.f, acc[s]);
                }
            }
        }
#pragma unroll
        for (int s = 0; s < SB; ++s) sm_part[s * kGptqMaxCols + c] = acc[s];
    }
    cluster.sync();   // every CTA's partial sums are in its shared memory
    if (crank == 0) {
        // the first CTA adds the others' partial sums to its own (distributed shared memory reads)
        for (uint32_t i = tid; i < SB * ncols; i += kGptqThreads) {
            const uint32_t s = i / ncols, c = i % ncols;
            float v = sm_part[s * kGptqMaxCols + c];
            for (uint32_t r = 1; r < csize; ++r) v += cluster.map_shared_rank(sm_part, r)[s * kGptqMaxCols + c];
            sm_part[s * kGptqMaxCols + c] = v;
        }
    }
    cluster.sync();   // the others may leave (and release their shared memory) only now
    if (crank != 0) return;

    if (!a.fused) {
        for (uint32_t i = tid; i < nseq * ncols; i += kGptqThreads) {
            const uint32_t s = i / ncols, c = i % ncols;
            a.y[(size_t)(seq0 + s) * a.wq.N + colbase[0] + c] = sm_part[s * kGptqMaxCols + c];
        }
        return;
    }
    // ---- epilogue: fused_split_qknorm_kvstore.wgsl:106-230 on the unit's vectors, one warp per sequence ----
    for (uint32_t s = warp; s < nseq; s += kGptqThreads / 32) {
        const uint32_t seq = seq0 + s, hd = a.hd;
        float *vals = sm_part + s * kGptqMaxCols;            // [0, hd): Q or K, [hd, 2hd): gate or V
        const uint32_t p_t = a.pos_start[seq];
        const uint32_t p_h = a.pos_h ? a.pos_h[seq] : p_t, p_w = a.pos_w ? a.pos_w[seq] : p_t;
        __syncwarp();
        if (unit < a.nh) {
            warp_norm_rope(vals, lane, hd, a.norm_w, a.rope, a.inv_freq, p_t, p_h, p_w);
            const size_t row = ((size_t)seq * a.nh + unit) * hd;
            for (uint32_t d = lane; d < hd; d += 32) {
                store_from_f32(a.q_out, row + d, a.q_dtype, vals[d]);
                if (a.has_gate && a.q_gate) a.q_gate[row + d] = vals[hd + d];
            }
        } else {
            const uint32_t kh = unit - a.nh;
            warp_norm_rope(vals, lane, hd, a.norm_w ? a.norm_w + hd : nullptr, a.rope, a.inv_freq, p_t, p_h, p_w);
            const size_t esz = dtype_size(a.kv_dtype);
            // cache_position == position (model.rs:493-496)
            char *kc = const_cast<char *>(kv_row_ptr(a.kv, false, seq, p_t, (size_t)a.nkv * hd * esz));
            char *vc = const_cast<char *>(kv_row_ptr(a.kv, true, seq, p_t, (size_t)a.nkv * hd * esz));
            const size_t crow = (size_t)kh * hd;
            for (uint32_t d = lane; d < hd; d += 32) {
                store_from_f32(kc, crow + d, a.kv_dtype, vals[d] * a.k_inv);
                store_from_f32(vc, crow + d, a.kv_dtype, vals[hd + d] * a.v_inv);
            }
        }
    }
}

static int check_weight(shady_ctx *ctx, const char *who, const shady_gptq_weight *w, uint32_t K, uint32_t group_size) {
    const std::string n(who);
    SHADY_REQUIRE(ctx, w && w->d_qweight && w->d_scales && w->N, SHADY_ERR_BAD_ARG, n + ": null or empty weight");
    SHADY_REQUIRE(ctx, w->K == K && w->group_size == group_size, SHADY_ERR_BAD_ARG, n + ": the weights disagree on K or group_size");
    return SHADY_OK;
}

static int launch_qkv(shady_ctx *ctx, QkvArgs &a, uint32_t units) {
    const uint32_t packed_rows = a.K / 8;
    uint32_t split = kGptqSplit;
    while (split > 1 && packed_rows < split * 4) split /= 2;   // tiny K: fewer CTAs per unit
    const uint32_t kmax = ((packed_rows + split - 1) / split + 1) * 8;
    for (uint32_t s0 = 0; s0 < a.num_seqs; s0 += kGptqMaxSeqs) {
        const uint32_t nseq = a.num_seqs - s0 < kGptqMaxSeqs ? a.num_seqs - s0 : kGptqMaxSeqs;
        const uint32_t sb = nseq > 2 ? 4u : nseq;
        const size_t smem = ((size_t)sb * kmax + (size_t)sb * kGptqMaxCols) * sizeof(float);
        SHADY_REQUIRE(ctx, smem <= 200 * 1024, SHADY_ERR_UNSUPPORTED, "gptq: K too large for one pass (shared memory)");
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3(units * split);
        cfg.blockDim = dim3(kGptqThreads);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = ctx->stream;
        cudaLaunchAttribute attr{};
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = split; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        auto go = [&](auto kern) -> cudaError_t {
            if (smem > 48 * 1024) {   // only very wide hidden states need more than the default limit
                const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(200 * 1024));
                if (e != cudaSuccess) return e;
            }
            return cudaLaunchKernelEx(&cfg, kern, a, s0);
        };
        cudaError_t e = sb == 1 ? go(qkv_proj_kernel<1>) : (sb == 2 ? go(qkv_proj_kernel<2>) : go(qkv_proj_kernel<4>));
        if (e != cudaSuccess) return fail(ctx, SHADY_ERR_CUDA, std::string("gptq launch: ") + cudaGetErrorString(e));
        ctx->launches++;
    }
    return SHADY_OK;
}

int launch_gptq_matvec(shady_ctx *ctx, const shady_gptq_weight *w, const float *d_x, float *d_y, uint32_t num_vecs) {
    SHADY_REQUIRE(ctx, w && d_x && d_y && num_vecs, SHADY_ERR_BAD_ARG, "gptq_matvec: null or zero argument");
    SHADY_REQUIRE(ctx, w->K && w->K % 8 == 0 && w->group_size && w->group_size % 8 == 0 && w->K % w->group_size == 0,
                  SHADY_ERR_BAD_ARG, "gptq_matvec: K and group_size must be multiples of 8, K a multiple of group_size");
    if (const int st = check_weight(ctx, "gptq_matvec", w, w->K, w->group_size)) return st;
    QkvArgs a{};
    a.wq = GptqW{w->d_qweight, reinterpret_cast<const uint16_t *>(w->d_scales), w->N};
    a.x = d_x; a.y = d_y; a.K = w->K; a.group_size = w->group_size; a.num_seqs = num_vecs; a.fused = 0;
    return launch_qkv(ctx, a, (w->N + kGptqThreads - 1) / kGptqThreads);
}

int launch_qkv_proj_append(shady_ctx *ctx, const shady_append_params *p, const shady_gptq_weight *wq, const shady_gptq_weight *wk,
                           const shady_gptq_weight *wv, const float *d_x, void *d_q_out, float *d_q_gate,
                           const shady_kv_cache *cache, const uint16_t *d_qk_norm_bf16, const uint32_t *d_pos_start,
                           const uint32_t *d_pos_h, const uint32_t *d_pos_w) {
    SHADY_REQUIRE(ctx, p && wq && wk && wv && d_x && d_q_out && cache && d_pos_start, SHADY_ERR_BAD_ARG, "qkv_proj_append: null argument");
    SHADY_REQUIRE(ctx, p->num_heads && p->num_kv_heads && p->head_dim && p->num_seqs, SHADY_ERR_BAD_ARG, "qkv_proj_append: zero-sized problem");
    SHADY_REQUIRE(ctx, p->tokens_per_seq == 1, SHADY_ERR_UNSUPPORTED, "qkv_proj_append: one token per sequence (the decode step)");
    SHADY_REQUIRE(ctx, p->head_dim <= 256 && p->head_dim % 32 == 0, SHADY_ERR_UNSUPPORTED, "qkv_proj_append: head_dim must be a multiple of 32, at most 256");
    SHADY_REQUIRE(ctx, p->rotary_dim <= p->head_dim && (p->rotary_dim % 2) == 0, SHADY_ERR_BAD_ARG,
                  "qkv_proj_append: rotary_dim must be even and <= head_dim");
    SHADY_REQUIRE(ctx, p->q_dtype <= SHADY_BF16, SHADY_ERR_BAD_ARG, "qkv_proj_append: bad q dtype");
    SHADY_REQUIRE(ctx, !p->has_gate || d_q_gate, SHADY_ERR_BAD_ARG, "qkv_proj_append: has_gate needs d_q_gate");
    const uint32_t K = wq->K, gs = wq->group_size;
    SHADY_REQUIRE(ctx, K && K % 8 == 0 && gs && gs % 8 == 0 && K % gs == 0, SHADY_ERR_BAD_ARG,
                  "qkv_proj_append: K and group_size must be multiples of 8, K a multiple of group_size");
    if (const int st = check_weight(ctx, "qkv_proj_append(q)", wq, K, gs)) return st;
    if (const int st = check_weight(ctx, "qkv_proj_append(k)", wk, K, gs)) return st;
    if (const int st = check_weight(ctx, "qkv_proj_append(v)", wv, K, gs)) return st;
    const uint32_t qcols = (p->has_gate ? 2u : 1u) * p->head_dim;
    SHADY_REQUIRE(ctx, wq->N == p->num_heads * qcols && wk->N == p->num_kv_heads * p->head_dim && wv->N == wk->N, SHADY_ERR_BAD_ARG,
                  "qkv_proj_append: weight widths do not match the head counts (q: nh*(1+gate)*hd, k and v: nkv*hd)");
    QkvArgs a{};
    a.wq = GptqW{wq->d_qweight, reinterpret_cast<const uint16_t *>(wq->d_scales), wq->N};
    a.wk = GptqW{wk->d_qweight, reinterpret_cast<const uint16_t *>(wk->d_scales), wk->N};
    a.wv = GptqW{wv->d_qweight, reinterpret_cast<const uint16_t *>(wv->d_scales), wv->N};
    a.x = d_x; a.K = K; a.group_size = gs; a.num_seqs = p->num_seqs; a.fused = 1;
    a.q_out = d_q_out; a.q_gate = d_q_gate;
    if (const int st = fill_kv_addr(ctx, cache, p->num_kv_heads, p->head_dim, "qkv_proj_append", &a.kv)) return st;
    a.norm_w = d_qk_norm_bf16;
    a.pos_start = d_pos_start; a.pos_h = d_pos_h; a.pos_w = d_pos_w;
    a.nh = p->num_heads; a.nkv = p->num_kv_heads; a.hd = p->head_dim; a.has_gate = p->has_gate;
    a.q_dtype = p->q_dtype; a.kv_dtype = cache->dtype;
    a.rope = RopeSpec{p->rotary_dim, p->s1_limit, p->s2_limit, p->interleaved, p->eps};
    a.k_inv = 1.0f / a.kv.k_scale; a.v_inv = 1.0f / a.kv.v_scale;
    for (uint32_t i = 0; i < p->rotary_dim / 2; ++i)   // wgsl:57, the libm call the stand-alone append and the oracle make
        a.inv_freq[i] = 1.0f / powf(p->rope_theta, 2.0f * (float)i / (float)p->rotary_dim);
    return launch_qkv(ctx, a, p->num_heads + p->num_kv_heads);
}

}  // namespace shady
