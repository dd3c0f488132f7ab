/*
 * CPU restatement of the shady-thinker attention hot path (and of the INT4 projection that
 * feeds it).  TEST INFRASTRUCTURE ONLY:
 * this file is the parity checker and the timed CPU baseline; no product code path may
 * call it.
 *
 * PARITY UNPINNED: the reference holds no golden vector, known-answer test or fixture for
 * this path (its only tests are end-to-end text assertions that need model weights and a
 * graphics adapter), and its implementation is WGSL that cannot be executed here.  The
 * restatement is therefore cross-checked only against itself (f32-faithful vs f64, split
 * vs single pass, token loop vs causal) and against an independent softmax-attention
 * formula.
 *
 * Each function cites the reference file:line it restates (paths relative to the
 * reference project root).  "Faithful" functions keep the shader's f32 operation order:
 * the 256-leaf barrier tree reduction, the -3.402823e+38 running-max seed, natural
 * exp/log, and the f32 rounding of the RoPE angle before cos/sin.  Compile with
 * -ffp-contract=off so no multiply-add is fused behind the shader's back.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define WG 256 /* @workgroup_size(256) in all three shaders */

/* ------------------------------------------------------------------------------------ */
/* Shared helpers                                                                        */
/* ------------------------------------------------------------------------------------ */

/* 256-leaf shared-memory tree: strides 128,64,...,1 (gqa_attention_head.wgsl:75-86,
 * fused_split_qknorm_kvstore.wgsl:139-148). Leaves are destroyed. */
static float tree256(float *leaf) {
    for (int stride = WG / 2; stride > 0; stride >>= 1)
        for (int t = 0; t < stride; ++t) leaf[t] = leaf[t] + leaf[t + stride];
    return leaf[0];
}

/* unpack_bf16: bits << 16 (fused_split_qknorm_kvstore.wgsl:37-40) */
static float bf16_bits_to_f32(uint16_t b) {
    uint32_t u = ((uint32_t)b) << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

int oracle_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* ------------------------------------------------------------------------------------ */
/* a-1: gqa_attention_head.wgsl:30-124 — one call runs every workgroup (q_head, split).  */
/* q [nh][hd]; k_cache, v_cache [pos][nkv][hd]; output [nh][hd] (ns==1) or               */
/* [nh][ns][hd+2] with [hd]=log(l)+m, [hd+1]=m.                                          */
/* ------------------------------------------------------------------------------------ */
void oracle_gqa_attention_head_f32(const float *q, const float *k_cache, const float *v_cache,
                                   float *output, uint32_t seq_len, uint32_t head_dim,
                                   uint32_t num_kv_heads, uint32_t num_q_heads,
                                   uint32_t heads_per_kv, uint32_t num_splits, int threads) {
    const float scale = 1.0f / sqrtf((float)head_dim); /* wgsl:43 */
    const uint32_t pps = (seq_len + num_splits - 1u) / num_splits; /* wgsl:46 */
    const int total = (int)(num_q_heads * num_splits);
    (void)threads;
#pragma omp parallel for schedule(dynamic, 1) num_threads(threads > 0 ? threads : 1)
    for (int wg = 0; wg < total; ++wg) {
        const uint32_t q_head = (uint32_t)wg / num_splits;
        const uint32_t split = (uint32_t)wg % num_splits;
        const uint32_t kv_head = q_head / heads_per_kv; /* wgsl:42 */
        const uint32_t start = split * pps;
        uint32_t end = start + pps;
        if (end > seq_len) end = seq_len;
        float acc[WG];
        float leaf[WG];
        for (uint32_t d = 0; d < head_dim; ++d) acc[d] = 0.0f;
        float running_max = -3.402823e+38f; /* wgsl:56 */
        float running_sum = 0.0f;
        const float *qh = q + (size_t)q_head * head_dim;
        for (uint32_t pos = start; pos < end; ++pos) {
            const size_t kv_base = ((size_t)pos * num_kv_heads + kv_head) * head_dim; /* wgsl:64 */
            for (uint32_t t = 0; t < WG; ++t) {
                float local_dot = 0.0f;
                for (uint32_t d = t; d < head_dim; d += WG) local_dot += qh[d] * k_cache[kv_base + d];
                leaf[t] = local_dot;
            }
            const float score = tree256(leaf) * scale; /* wgsl:88 */
            const float new_max = fmaxf(running_max, score);
            const float correction = expf(running_max - new_max);
            const float exp_score = expf(score - new_max);
            running_sum = running_sum * correction + exp_score;
            for (uint32_t d = 0; d < head_dim; ++d)
                acc[d] = acc[d] * correction + exp_score * v_cache[kv_base + d];
            running_max = new_max;
        }
        if (num_splits == 1u) {
            for (uint32_t d = 0; d < head_dim; ++d)
                output[(size_t)q_head * head_dim + d] = acc[d] / running_sum; /* wgsl:107-111 */
        } else {
            const size_t base = ((size_t)q_head * num_splits + split) * (head_dim + 2u);
            for (uint32_t d = 0; d < head_dim; ++d) output[base + d] = acc[d] / running_sum;
            output[base + head_dim] = logf(running_sum) + running_max; /* wgsl:120 */
            output[base + head_dim + 1u] = running_max;
        }
    }
}

/* ------------------------------------------------------------------------------------ */
/* a-2: gqa_reduce.wgsl:20-65.  partials [nh][ns][hd+2] -> output [nh][hd].              */
/* skip_empty != 0 is the batched/sharded extension: a split whose lse is -inf (or NaN,   */
/* which an empty split produces through 0/0) gets weight 0 and its data is not read.     */
/* skip_empty == 0 is the shader verbatim.                                                */
/* ------------------------------------------------------------------------------------ */
void oracle_gqa_reduce_f32(const float *partials, float *output, uint32_t head_dim,
                           uint32_t num_splits, uint32_t num_heads, int skip_empty) {
    const uint32_t stride = head_dim + 2u;
    for (uint32_t head = 0; head < num_heads; ++head) {
        float gmax = -3.402823e+38f; /* wgsl:35 */
        for (uint32_t s = 0; s < num_splits; ++s) {
            const float lse = partials[((size_t)head * num_splits + s) * stride + head_dim];
            if (skip_empty && !(lse > -INFINITY)) continue;
            gmax = fmaxf(gmax, lse);
        }
        for (uint32_t d = 0; d < head_dim; ++d) {
            float acc = 0.0f, wsum = 0.0f;
            for (uint32_t s = 0; s < num_splits; ++s) {
                const size_t base = ((size_t)head * num_splits + s) * stride;
                const float lse = partials[base + head_dim];
                if (skip_empty && !(lse > -INFINITY)) continue;
                const float w = expf(lse - gmax); /* wgsl:56 */
                acc += w * partials[base + d];
                wsum += w;
            }
            output[(size_t)head * head_dim + d] = acc / wsum;
        }
    }
}

/* ------------------------------------------------------------------------------------ */
/* a-3: fused_split_qknorm_kvstore.wgsl:106-230 with the constants that                  */
/* model.rs:32-54 injects (theta, PARTIAL_DIM, section limits, interleaved).             */
/* ------------------------------------------------------------------------------------ */
typedef struct {
    uint32_t num_heads, num_kv_heads, head_dim;
    float eps;
    uint32_t cache_position, position, position_h, position_w; /* wgsl:12-21 */
    float rope_theta;                                          /* ROPE_THETA */
    uint32_t partial_dim;                                      /* PARTIAL_DIM */
    uint32_t s1_limit, s2_limit;                               /* MROPE_S{1,2}_LIMIT */
    uint32_t interleaved;                                      /* MROPE_INTERLEAVED */
    uint32_t has_norm; /* extension: 0 skips the RMSNorm step entirely (plain RoPE append) */
} oracle_qknorm_params;

/* apply_mrope (wgsl:56-73) */
static void mrope_pair(const oracle_qknorm_params *p, float a, float b, uint32_t freq_idx,
                       float *oa, float *ob) {
    const float freq = 1.0f / powf(p->rope_theta, 2.0f * (float)freq_idx / (float)p->partial_dim);
    uint32_t pos = p->position;
    if ((freq_idx % 3u) == 1u && freq_idx < p->s1_limit) pos = p->position_h;
    else if ((freq_idx % 3u) == 2u && freq_idx < p->s2_limit) pos = p->position_w;
    const float angle = (float)pos * freq;
    const float c = cosf(angle), s = sinf(angle);
    *oa = a * c - b * s;
    *ob = b * c + a * s;
}

/* apply_mrope_to_wg (wgsl:76-104) */
static void mrope_vec(const oracle_qknorm_params *p, float *vals) {
    const uint32_t half = p->partial_dim / 2u;
    for (uint32_t d = 0; d < half; ++d) {
        const uint32_t ia = p->interleaved ? 2u * d : d;
        const uint32_t ib = p->interleaved ? 2u * d + 1u : d + half;
        float oa, ob;
        mrope_pair(p, vals[ia], vals[ib], d, &oa, &ob);
        vals[ia] = oa;
        vals[ib] = ob;
    }
}

/* norm + rope of one head vector (wgsl:126-166 for Q, :181-217 for K) */
static void norm_rope_head(const oracle_qknorm_params *p, float *vals, const uint16_t *w_bf16) {
    const uint32_t hd = p->head_dim;
    if (p->has_norm) {
        float leaf[WG];
        for (uint32_t t = 0; t < WG; ++t) {
            float s = 0.0f;
            for (uint32_t d = t; d < hd; d += WG) s += vals[d] * vals[d];
            leaf[t] = s;
        }
        const float rms = 1.0f / sqrtf(tree256(leaf) / (float)hd + p->eps); /* wgsl:150 */
        for (uint32_t d = 0; d < hd; ++d) {
            const float w = bf16_bits_to_f32(w_bf16[d]);
            vals[d] = vals[d] * rms * (1.0f + w); /* wgsl:158 */
        }
    }
    mrope_vec(p, vals);
}

/* One token.  q_proj_full [nh][2][hd] (Q then gate), k_proj [nkv][hd] in/out, v_proj
 * [nkv][hd]; outputs q_proj [nh][hd], q_gate [nh][hd]; cache rows at cache_position in
 * k_cache/v_cache [pos][nkv][hd].  qk_norm_bf16: q weights [hd] then k weights [hd]
 * (model.rs:157-166); may be NULL when has_norm == 0. */
void oracle_fused_split_qknorm_kvstore_f32(const oracle_qknorm_params *p, const float *q_proj_full,
                                           float *k_proj, const float *v_proj, float *q_proj,
                                           float *q_gate, float *k_cache, float *v_cache,
                                           const uint16_t *qk_norm_bf16) {
    const uint32_t hd = p->head_dim;
    float vals[WG];
    for (uint32_t h = 0; h < p->num_heads; ++h) {
        const float *src = q_proj_full + (size_t)h * hd * 2u; /* wgsl:120 */
        for (uint32_t d = 0; d < hd; ++d) {
            vals[d] = src[d];
            q_gate[(size_t)h * hd + d] = src[hd + d];
        }
        norm_rope_head(p, vals, qk_norm_bf16);
        for (uint32_t d = 0; d < hd; ++d) q_proj[(size_t)h * hd + d] = vals[d];
    }
    for (uint32_t kh = 0; kh < p->num_kv_heads; ++kh) {
        for (uint32_t d = 0; d < hd; ++d) vals[d] = k_proj[(size_t)kh * hd + d];
        norm_rope_head(p, vals, qk_norm_bf16 ? qk_norm_bf16 + hd : NULL);
        const size_t cache_off = ((size_t)p->cache_position * p->num_kv_heads + kh) * hd; /* wgsl:220 */
        for (uint32_t d = 0; d < hd; ++d) {
            k_proj[(size_t)kh * hd + d] = vals[d];
            k_cache[cache_off + d] = vals[d];
            v_cache[cache_off + d] = v_proj[(size_t)kh * hd + d];
        }
    }
}

/* f-1 (next row): sigmoid_mul.wgsl:16-23  out[i] = x[i] * 1/(1+exp(-g[i])) */
void oracle_sigmoid_mul_f32(const float *x, const float *gate, float *out, uint32_t n) {
    for (uint32_t i = 0; i < n; ++i) {
        const float sig = 1.0f / (1.0f + expf(-gate[i]));
        out[i] = x[i] * sig;
    }
}

/* f-4 (next row): gptq_matvec.wgsl:20-82 — symmetric INT4 GPTQ matrix-vector product, one output column
 * at a time, terms added in row order in f32:  sum += ((f32(nibble) - 8) * scale) * input[row]   (wgsl:50-57).
 * qweight [K/8][N] u32 (eight nibbles along K per word, lowest row in the low nibble), scales [K/group][N] f16,
 * two per u32 (unpack2x16float, wgsl:44-45).  The 4-thread variant (gptq_matvec_4t.wgsl) adds the same terms in
 * four interleaved chains; both are the same product to f32 rounding. */
static float f16_bits_to_f32(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16, exp = (h >> 10) & 0x1fu, man = h & 0x3ffu;
    uint32_t u;
    if (exp == 0) {
        if (man == 0) u = sign;
        else {   /* subnormal: normalise */
            int e = -1;
            uint32_t m = man;
            do { m <<= 1; ++e; } while (!(m & 0x400u));
            u = sign | ((uint32_t)(127 - 15 - e) << 23) | ((m & 0x3ffu) << 13);
        }
    } else if (exp == 31) u = sign | 0x7f800000u | (man << 13);
    else u = sign | ((exp + 112u) << 23) | (man << 13);
    float f;
    memcpy(&f, &u, 4);
    return f;
}
void oracle_gptq_matvec_f32(const float *input, const uint32_t *qweight, const uint32_t *scales, float *output,
                            uint32_t K, uint32_t N, uint32_t group_size) {
    const uint32_t packed_rows = K / 8u;
    for (uint32_t col = 0; col < N; ++col) {
        float sum = 0.0f;
        for (uint32_t pr = 0; pr < packed_rows; ++pr) {
            const uint32_t group = (pr * 8u) / group_size;
            const uint32_t sf = group * N + col;
            const uint32_t s2 = scales[sf / 2u];
            const float scale = f16_bits_to_f32((uint16_t)((sf & 1u) ? (s2 >> 16) : (s2 & 0xffffu)));
            const uint32_t packed = qweight[pr * N + col];
            for (uint32_t nib = 0; nib < 8u; ++nib) {
                const float w = ((float)((packed >> (4u * nib)) & 0xFu) - 8.0f) * scale;
                sum += w * input[pr * 8u + nib];
            }
        }
        output[col] = sum;
    }
}

/* ------------------------------------------------------------------------------------ */
/* f64 "truth" of a-1 (+a-2): exact two-pass softmax attention of one token over rows    */
/* [0, seq_len) in double.  Used for the error budget, not as the reference order.       */
/* ------------------------------------------------------------------------------------ */
void oracle_attention_f64(const float *q, const float *k_cache, const float *v_cache, double *output,
                          uint32_t seq_len, uint32_t head_dim, uint32_t num_kv_heads,
                          uint32_t num_q_heads, uint32_t heads_per_kv, int threads) {
    const double scale = 1.0 / sqrt((double)head_dim);
    (void)threads;
#pragma omp parallel for schedule(dynamic, 1) num_threads(threads > 0 ? threads : 1)
    for (int h = 0; h < (int)num_q_heads; ++h) {
        const uint32_t kvh = (uint32_t)h / heads_per_kv;
        double *s = (double *)malloc(sizeof(double) * (seq_len ? seq_len : 1));
        double m = -INFINITY;
        for (uint32_t pos = 0; pos < seq_len; ++pos) {
            const size_t base = ((size_t)pos * num_kv_heads + kvh) * head_dim;
            double dot = 0.0;
            for (uint32_t d = 0; d < head_dim; ++d)
                dot += (double)q[(size_t)h * head_dim + d] * (double)k_cache[base + d];
            s[pos] = dot * scale;
            if (s[pos] > m) m = s[pos];
        }
        double l = 0.0;
        for (uint32_t d = 0; d < head_dim; ++d) output[(size_t)h * head_dim + d] = 0.0;
        for (uint32_t pos = 0; pos < seq_len; ++pos) {
            const size_t base = ((size_t)pos * num_kv_heads + kvh) * head_dim;
            const double p = exp(s[pos] - m);
            l += p;
            for (uint32_t d = 0; d < head_dim; ++d)
                output[(size_t)h * head_dim + d] += p * (double)v_cache[base + d];
        }
        for (uint32_t d = 0; d < head_dim; ++d) output[(size_t)h * head_dim + d] /= l;
        free(s);
    }
}

/* ------------------------------------------------------------------------------------ */
/* a-5: prefill == token loop (inference.rs:93-95): out[t] = attend(q_t, K[0..=t]).      */
/* Inputs are already normed/roped.  q [T][nh][hd], k/v [T][nkv][hd] (cache layout),     */
/* out [T][nh][hd].  Faithful f32 single-split order per token.                          */
/* ------------------------------------------------------------------------------------ */
void oracle_causal_prefill_f32(const float *q, const float *k_cache, const float *v_cache, float *out,
                               uint32_t T, uint32_t head_dim, uint32_t num_kv_heads,
                               uint32_t num_q_heads, uint32_t heads_per_kv, int threads) {
    (void)threads;
#pragma omp parallel for schedule(dynamic, 1) num_threads(threads > 0 ? threads : 1)
    for (int t = (int)T - 1; t >= 0; --t) {
        oracle_gqa_attention_head_f32(q + (size_t)t * num_q_heads * head_dim, k_cache, v_cache,
                                      out + (size_t)t * num_q_heads * head_dim, (uint32_t)t + 1u,
                                      head_dim, num_kv_heads, num_q_heads, heads_per_kv, 1u, 1);
    }
}

/* Same in f64 with two-pass softmax (error-budget truth for the prefill kernel). */
void oracle_causal_prefill_f64(const float *q, const float *k_cache, const float *v_cache, double *out,
                               uint32_t T, uint32_t head_dim, uint32_t num_kv_heads,
                               uint32_t num_q_heads, uint32_t heads_per_kv, int threads) {
    (void)threads;
#pragma omp parallel for schedule(dynamic, 1) num_threads(threads > 0 ? threads : 1)
    for (int t = (int)T - 1; t >= 0; --t) {
        oracle_attention_f64(q + (size_t)t * num_q_heads * head_dim, k_cache, v_cache,
                             out + (size_t)t * num_q_heads * head_dim, (uint32_t)t + 1u, head_dim,
                             num_kv_heads, num_q_heads, heads_per_kv, 1);
    }
}

/* ------------------------------------------------------------------------------------ */
/* Batched ragged decode (extension of a-1 to many sequences; the per-sequence math is    */
/* the shader's).  k_ptrs[i]/v_ptrs[i] point at sequence i's [L_i][nkv][hd] f32 rows.     */
/* ------------------------------------------------------------------------------------ */
void oracle_batched_decode_f32(const float *q, const float *const *k_ptrs, const float *const *v_ptrs,
                               const uint32_t *seq_lens, uint32_t num_seqs, float *out,
                               uint32_t head_dim, uint32_t num_kv_heads, uint32_t num_q_heads,
                               uint32_t heads_per_kv, int threads) {
    (void)threads;
#pragma omp parallel for schedule(dynamic, 1) num_threads(threads > 0 ? threads : 1)
    for (int i = 0; i < (int)num_seqs; ++i) {
        oracle_gqa_attention_head_f32(q + (size_t)i * num_q_heads * head_dim, k_ptrs[i], v_ptrs[i],
                                      out + (size_t)i * num_q_heads * head_dim, seq_lens[i], head_dim,
                                      num_kv_heads, num_q_heads, heads_per_kv, 1u, 1);
    }
}

/* ------------------------------------------------------------------------------------ */
/* Counter-based N(0,1) generator shared with the device fill kernel: element idx of      */
/* tensor tensor_id under seed is a pure function of (seed, tensor_id, idx).              */
/* splitmix64 finaliser -> two 24-bit uniforms -> Box-Muller in double -> f32.            */
/* ------------------------------------------------------------------------------------ */
static uint64_t mix64(uint64_t z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

float oracle_randn_at(uint64_t seed, uint64_t tensor_id, uint64_t idx) {
    const uint64_t r = mix64(mix64(seed ^ (tensor_id * 0xD1B54A32D192ED03ull)) + idx);
    const double u1 = ((double)((r >> 40) & 0xFFFFFFull) + 1.0) * (1.0 / 16777216.0); /* (0,1] */
    const double u2 = (double)((r >> 8) & 0xFFFFFFull) * (1.0 / 16777216.0);          /* [0,1) */
    return (float)(sqrt(-2.0 * log(u1)) * cos(6.283185307179586476925 * u2));
}

void oracle_fill_randn(float *dst, uint64_t n, uint64_t seed, uint64_t tensor_id, uint64_t first_idx) {
#pragma omp parallel for schedule(static)
    for (long long i = 0; i < (long long)n; ++i)
        dst[i] = oracle_randn_at(seed, tensor_id, first_idx + (uint64_t)i);
}
