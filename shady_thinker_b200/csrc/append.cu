// KV append: Q/gate split, Q/K RMSNorm with (1+w) bf16 weights, partial (m)RoPE, cache store.
// Results follow fused_split_qknorm_kvstore.wgsl:106-230; the layout of the work does not:
// one warp per (token, head) instead of a 256-thread workgroup with barrier trees, batched
// over tokens and sequences, cache rows written in the cache's storage dtype.
//
// RoPE frequencies are NOT computed on the device: the host evaluates
// 1/powf(theta, 2i/rotary_dim) once (same libm call the CPU oracle makes) and passes the
// table by value.  At position ~1e5 a 1-ulp difference in the frequency moves the angle by
// ~1e-2 rad, so device powf would break parity with any CPU statement of the shader.
// cos/sin use the accurate sincosf (full-range argument reduction), never the fast
// intrinsics: the shader takes cos/sin of up to 131071 radians in f32 (wgsl:66-68).
#include <math.h>
#include <type_traits>

#include "append_core.cuh"

namespace shady {

struct AppendArgs {
    const void *q_in;
    void *k_io;
    const void *v_in;
    void *q_out;
    float *q_gate;
    KvAddr kv;                // where the cache rows go (per-sequence bases, pointer arrays or pages)
    const uint16_t *norm_w;   // bf16 bits: q[hd] then k[hd]; NULL = no norm
    const uint32_t *pos_start, *pos_h, *pos_w;
    uint32_t nh, nkv, hd;
    float eps;
    uint32_t rd, s1, s2, interleaved;
    uint32_t num_seqs, T;
    uint32_t in_dtype, q_dtype, kv_dtype, has_gate, write_k_back;
    uint32_t head_slices;     // vectorised path: warps that share one token's heads (small batches need the parallelism)
    uint32_t skip_q;          // vectorised path: K/V only (Q is normed and rotated by the prefill attention kernel itself)
    float2 *cs_table;         // vectorised path, optional: (cos, sin) of [token j][pair i < hd/2] of sequence 0, (1, 0) past rd/2
    float k_inv, v_inv;       // 8-bit caches: rows are stored as value * (1 / scale); 1 otherwise
    // vectorised path, listed batch: tokens are packed sequence after sequence, sequence s owns tokens
    // [tok_start[s], tok_start[s+1]); T is not used
    const uint32_t *tok_start;
    uint32_t total_tokens, table_seq;
    // staged path: shared-memory bytes of one warp's token, the status words and the poll limit of its bounded wait
    uint32_t stage_bytes, wait_limit;
    StatusRef status;
    float inv_freq[128];      // [rd/2]
};

constexpr int kAppendWarps = 4;

__global__ void __launch_bounds__(kAppendWarps * 32) append_kernel(const AppendArgs a) {
    __shared__ float sm_vals[kAppendWarps][256];
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t heads = a.nh + a.nkv;
    const unsigned long long wid = (unsigned long long)blockIdx.x * kAppendWarps + warp;
    const unsigned long long total = (unsigned long long)a.num_seqs * a.T * heads;
    if (wid >= total) return;
    const uint32_t h = (uint32_t)(wid % heads);
    const unsigned long long tok = wid / heads;
    const uint32_t s = (uint32_t)(tok / a.T), j = (uint32_t)(tok % a.T);
    const uint32_t hd = a.hd;
    float *vals = sm_vals[warp];
    const bool is_q = h < a.nh;
    const uint32_t kh = h - a.nh;

    // ---- load the head vector (and pass the gate through) ----
    if (is_q) {
        const size_t row = (tok * a.nh + h) * (size_t)(a.has_gate ? 2 * hd : hd);
        for (uint32_t d = lane; d < hd; d += 32) {
            vals[d] = load_as_f32(a.q_in, row + d, a.in_dtype);
            if (a.has_gate && a.q_gate)
                a.q_gate[(tok * a.nh + h) * (size_t)hd + d] = load_as_f32(a.q_in, row + hd + d, a.in_dtype);
        }
    } else {
        const size_t row = (tok * a.nkv + kh) * (size_t)hd;
        for (uint32_t d = lane; d < hd; d += 32) vals[d] = load_as_f32(a.k_io, row + d, a.in_dtype);
    }
    __syncwarp();
    // ---- RMSNorm (wgsl:150-160 / :205-212) and (m)RoPE on the first rd dims (wgsl:56-104) ----
    const uint32_t p_t = (a.pos_start ? a.pos_start[s] : 0u) + j;
    const uint32_t p_h = a.pos_h ? a.pos_h[s] + j : p_t;
    const uint32_t p_w = a.pos_w ? a.pos_w[s] + j : p_t;
    const RopeSpec spec{a.rd, a.s1, a.s2, a.interleaved, a.eps};
    warp_norm_rope(vals, lane, hd, a.norm_w ? a.norm_w + (is_q ? 0 : hd) : nullptr, spec, a.inv_freq, p_t, p_h, p_w);
    // ---- stores ----
    if (is_q) {
        const size_t row = (tok * a.nh + h) * (size_t)hd;
        for (uint32_t d = lane; d < hd; d += 32) store_from_f32(a.q_out, row + d, a.q_dtype, vals[d]);
    } else {
        const size_t esz = dtype_size(a.kv_dtype);
        // cache_position == position (model.rs:493-496)
        char *kc = const_cast<char *>(kv_row_ptr(a.kv, false, s, p_t, (size_t)a.nkv * hd * esz));
        char *vc = const_cast<char *>(kv_row_ptr(a.kv, true, s, p_t, (size_t)a.nkv * hd * esz));
        const size_t crow = (size_t)kh * hd;
        const size_t row = (tok * a.nkv + kh) * (size_t)hd;
        for (uint32_t d = lane; d < hd; d += 32) {
            const float kv = vals[d];
            if (a.write_k_back) store_from_f32(a.k_io, row + d, a.in_dtype, kv);
            store_from_f32(kc, crow + d, a.kv_dtype, kv * a.k_inv);
            store_from_f32(vc, crow + d, a.kv_dtype, load_as_f32(a.v_in, row + d, a.in_dtype) * a.v_inv);
        }
    }
}


// ---------------------------------------------------------------------------------------
// Vectorised path (interleaved RoPE pairs, head_dim 128 or 256): one warp per token.
// cos/sin depend only on (position, pair index), so a lane evaluates its four pairs once and
// reuses them for every Q and K head of the token; each lane moves 8 contiguous elements per
// head with 16/32-byte accesses, and a warp covers 32*8/HD heads per iteration.
// ---------------------------------------------------------------------------------------
// ldraw() only requests the bytes, unpack() is their first use: a warp can hold several requests in flight.
template <typename T> struct Vec8 {
    using raw_t = uint4;
    static __device__ __forceinline__ raw_t ldraw(const T *p) { return *reinterpret_cast<const uint4 *>(p); }
    static __device__ __forceinline__ void unpack(const raw_t &u, float (&v)[8]) {
        const T *e = reinterpret_cast<const T *>(&u);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = to_f32<T>(e[i]);
    }
    static __device__ __forceinline__ void load(const T *p, float (&v)[8]) { unpack(ldraw(p), v); }
    static __device__ __forceinline__ void store(T *p, const float (&v)[8]) {
        uint4 u;
        T *e = reinterpret_cast<T *>(&u);
#pragma unroll
        for (int i = 0; i < 8; ++i) e[i] = from_f32<T>(v[i]);
        *reinterpret_cast<uint4 *>(p) = u;
    }
};
template <> struct Vec8<float> {
    struct raw_t { float4 a, b; };
    static __device__ __forceinline__ raw_t ldraw(const float *p) {
        return raw_t{*reinterpret_cast<const float4 *>(p), *reinterpret_cast<const float4 *>(p + 4)};
    }
    static __device__ __forceinline__ void unpack(const raw_t &r, float (&v)[8]) {
        v[0] = r.a.x; v[1] = r.a.y; v[2] = r.a.z; v[3] = r.a.w; v[4] = r.b.x; v[5] = r.b.y; v[6] = r.b.z; v[7] = r.b.w;
    }
    static __device__ __forceinline__ void load(const float *p, float (&v)[8]) { unpack(ldraw(p), v); }
    static __device__ __forceinline__ void store(float *p, const float (&v)[8]) {
        *reinterpret_cast<float4 *>(p) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4 *>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
    }
};

template <typename F8T> struct Vec8F8 {   // eight 1-byte elements: an 8-byte access
    using raw_t = uint2;
    static __device__ __forceinline__ raw_t ldraw(const F8T *p) { return *reinterpret_cast<const uint2 *>(p); }
    static __device__ __forceinline__ void unpack(const raw_t &u, float (&v)[8]) {
        const F8T *e = reinterpret_cast<const F8T *>(&u);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = float(e[i]);
    }
    static __device__ __forceinline__ void load(const F8T *p, float (&v)[8]) { unpack(ldraw(p), v); }
    static __device__ __forceinline__ void store(F8T *p, const float (&v)[8]) {
        uint2 u;
        F8T *e = reinterpret_cast<F8T *>(&u);
#pragma unroll
        for (int i = 0; i < 8; ++i) e[i] = F8T(v[i]);
        *reinterpret_cast<uint2 *>(p) = u;
    }
};
template <> struct Vec8<__nv_fp8_e4m3> : Vec8F8<__nv_fp8_e4m3> {};
template <> struct Vec8<__nv_fp8_e5m2> : Vec8F8<__nv_fp8_e5m2> {};

// Which sequence a packed token belongs to and its index there; false past the last token.
__device__ __forceinline__ bool locate_token(const AppendArgs &a, unsigned long long tok, uint32_t &s, uint32_t &j) {
    if (a.tok_start) {
        if (tok >= a.total_tokens) return false;
        uint32_t lo = 0, hi = a.num_seqs;   // the sequence with tok_start[s] <= tok < tok_start[s + 1]
        while (hi - lo > 1) {
            const uint32_t mid = (lo + hi) >> 1;
            if (__ldg(a.tok_start + mid) <= (uint32_t)tok) lo = mid; else hi = mid;
        }
        s = lo; j = (uint32_t)tok - __ldg(a.tok_start + lo);
    } else {
        if (tok >= (unsigned long long)a.num_seqs * a.T) return false;
        s = (uint32_t)(tok / a.T); j = (uint32_t)(tok % a.T);
    }
    return true;
}

// What a lane keeps for one token: cos/sin of its four pairs (wgsl:56-68), the norm weights of its eight dims.
template <int HD> struct LaneMath {
    static constexpr int LPH = HD / 8;   // lanes per head
    float cs[4], sn[4], wq[8], wk[8], eps;
    bool has_norm;
    uint32_t p_t;                        // the token's position == its cache row (model.rs:493-496)
    __device__ __forceinline__ void init(const AppendArgs &a, uint32_t s, uint32_t j, uint32_t dl, bool writes_table) {
        p_t = (a.pos_start ? a.pos_start[s] : 0u) + j;
        const uint32_t p_h = a.pos_h ? a.pos_h[s] + j : p_t;
        const uint32_t p_w = a.pos_w ? a.pos_w[s] + j : p_t;
        const uint32_t lane = threadIdx.x & 31, pairs = a.rd / 2;
        auto angle = [&](uint32_t i, float &c, float &sv) {
            uint32_t pos = p_t;
            if ((i % 3u) == 1u && i < a.s1) pos = p_h;
            else if ((i % 3u) == 2u && i < a.s2) pos = p_w;
            sincosf((float)pos * a.inv_freq[i], &sv, &c);
        };
#pragma unroll
        for (int k = 0; k < 4; ++k) { cs[k] = 1.f; sn[k] = 0.f; }
        if (pairs <= 64) {
            // Few rotated dims: the warp evaluates each pair once (lane l takes pairs l and l + 32) and hands the
            // values to the lanes that rotate with them.  The accurate sincosf is the longest run of instructions a
            // token costs, and with a quarter of the dims rotated only a quarter of the lanes would be inside it,
            // four times over.
            for (uint32_t base = 0; base < pairs; base += 32) {   // (the same trips for every lane)
                float c = 1.f, sv = 0.f;
                if (base + lane < pairs) angle(base + lane, c, sv);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const uint32_t want = dl * 4 + k;
                    const float ck = __shfl_sync(0xffffffffu, c, want & 31), sk = __shfl_sync(0xffffffffu, sv, want & 31);
                    if (want >= base && want < base + 32 && want < pairs) { cs[k] = ck; sn[k] = sk; }
                }
            }
        } else {
#pragma unroll
            for (int k = 0; k < 4; ++k)
                if (dl * 4 + k < pairs) angle(dl * 4 + k, cs[k], sn[k]);
        }
        if (a.cs_table && s == a.table_seq && writes_table) {   // one group of HD/8 lanes per token writes the token's table row
            float4 *row = reinterpret_cast<float4 *>(a.cs_table + (size_t)j * (HD / 2) + dl * 4);
            row[0] = make_float4(cs[0], sn[0], cs[1], sn[1]);
            row[1] = make_float4(cs[2], sn[2], cs[3], sn[3]);
        }
        has_norm = a.norm_w != nullptr;
        eps = a.eps;
        if (has_norm) {
            uint16_t bq[8], bk[8];   // bf16 bits
            if (((uintptr_t)a.norm_w & 15) == 0) {   // the lane's eight weights in one access each
                *reinterpret_cast<uint4 *>(bq) = *reinterpret_cast<const uint4 *>(a.norm_w + dl * 8);
                *reinterpret_cast<uint4 *>(bk) = *reinterpret_cast<const uint4 *>(a.norm_w + HD + dl * 8);
            } else {
#pragma unroll
                for (int e = 0; e < 8; ++e) { bq[e] = a.norm_w[dl * 8 + e]; bk[e] = a.norm_w[HD + dl * 8 + e]; }
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                wq[e] = 1.0f + __uint_as_float(((uint32_t)bq[e]) << 16);
                wk[e] = 1.0f + __uint_as_float(((uint32_t)bk[e]) << 16);
            }
        }
    }
    // Two heads at once: the same arithmetic as norm_rope on each, written side by side so that one head's shuffles
    // and square root wait under the other's
    __device__ __forceinline__ void norm_rope2(float (&u)[8], float (&v)[8], const float (&w)[8]) const {
        if (has_norm) {
            float su = 0.f, sv = 0.f;
#pragma unroll
            for (int e = 0; e < 8; ++e) { su += u[e] * u[e]; sv += v[e] * v[e]; }
#pragma unroll
            for (int o = LPH / 2; o > 0; o >>= 1) {
                su += __shfl_xor_sync(0xffffffffu, su, o);
                sv += __shfl_xor_sync(0xffffffffu, sv, o);
            }
            const float ru = 1.0f / sqrtf(su / (float)HD + eps), rv = 1.0f / sqrtf(sv / (float)HD + eps);
#pragma unroll
            for (int e = 0; e < 8; ++e) { u[e] = u[e] * ru * w[e]; v[e] = v[e] * rv * w[e]; }
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float xu = u[2 * k], yu = u[2 * k + 1], xv = v[2 * k], yv = v[2 * k + 1];
            u[2 * k] = xu * cs[k] - yu * sn[k];
            u[2 * k + 1] = yu * cs[k] + xu * sn[k];
            v[2 * k] = xv * cs[k] - yv * sn[k];
            v[2 * k + 1] = yv * cs[k] + xv * sn[k];
        }
    }
    // RMSNorm over the head (wgsl:150-160 / :205-212; every lane of the warp calls it), then the rotation
    __device__ __forceinline__ void norm_rope(float (&v)[8], const float (&w)[8]) const {
        if (has_norm) {
            float ssq = 0.f;
#pragma unroll
            for (int e = 0; e < 8; ++e) ssq += v[e] * v[e];
#pragma unroll
            for (int o = LPH / 2; o > 0; o >>= 1) ssq += __shfl_xor_sync(0xffffffffu, ssq, o);
            const float rms = 1.0f / sqrtf(ssq / (float)HD + eps);
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] = v[e] * rms * w[e];
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float x = v[2 * k], y = v[2 * k + 1];
            v[2 * k] = x * cs[k] - y * sn[k];
            v[2 * k + 1] = y * cs[k] + x * sn[k];
        }
    }
};

template <typename TIn, typename TQ, typename TKV, int HD>
__global__ void __launch_bounds__(kAppendWarps * 32, sizeof(TIn) == 4 ? 4 : 6) append_fast_kernel(const AppendArgs a) {
    constexpr int LPH = HD / 8;       // lanes per head
    constexpr int HPI = 32 / LPH;     // heads per warp iteration
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const unsigned long long wid = (unsigned long long)blockIdx.x * kAppendWarps + warp;
    const unsigned long long tok = wid / a.head_slices;
    const uint32_t slice = (uint32_t)(wid % a.head_slices);
    uint32_t s, j;
    if (!locate_token(a, tok, s, j)) return;
    const uint32_t sub = lane / LPH, dl = lane % LPH, d0 = dl * 8;
    // Every lane takes every trip (the norm shuffles are warp-wide).  A trip's rows are requested kPF trips before
    // they are used: with the request and the use in one trip a warp waited a memory round trip per head, and a
    // pass over 16k tokens ran at under half the memory bandwidth.
    using Raw = typename Vec8<TIn>::raw_t;
    constexpr int kPF = 3;
    const uint32_t step = HPI * a.head_slices;
    // ---- K heads (+ V copy): the first trip's rows are requested here, the second's while the first is worked on ----
    TIn *k_io = reinterpret_cast<TIn *>(a.k_io) + tok * a.nkv * (size_t)HD;
    const TIn *v_in = reinterpret_cast<const TIn *>(a.v_in) + tok * a.nkv * (size_t)HD;
    Raw rk = Raw{}, rv = Raw{};
    auto kv_request = [&](uint32_t kh0) {
        const uint32_t kh = kh0 + sub;
        if (kh < a.nkv) { rk = Vec8<TIn>::ldraw(k_io + (size_t)kh * HD + d0); rv = Vec8<TIn>::ldraw(v_in + (size_t)kh * HD + d0); }
    };
    kv_request(slice * HPI);
    // ---- Q heads: the first kPF trips' rows ----
    const uint32_t qrow = a.has_gate ? 2 * HD : HD;
    const TIn *q_in = reinterpret_cast<const TIn *>(a.q_in) + tok * a.nh * (size_t)qrow;
    TQ *q_out = reinterpret_cast<TQ *>(a.q_out) + tok * a.nh * (size_t)HD;
    Raw rq[kPF];
    uint32_t q_next = slice * HPI;   // the next trip to request
    auto q_request = [&](Raw &r) {
        const uint32_t h = q_next + sub;
        r = Raw{};
        if (h < a.nh && !a.skip_q) r = Vec8<TIn>::ldraw(q_in + (size_t)h * qrow + d0);
        q_next += step;
    };
#pragma unroll
    for (int u = 0; u < kPF; ++u) q_request(rq[u]);
    LaneMath<HD> m;
    m.init(a, s, j, dl, slice == 0 && sub == 0);
    TKV *k_row = reinterpret_cast<TKV *>(const_cast<char *>(kv_row_ptr(a.kv, false, s, m.p_t, (size_t)a.nkv * HD * sizeof(TKV))));
    TKV *v_row = reinterpret_cast<TKV *>(const_cast<char *>(kv_row_ptr(a.kv, true, s, m.p_t, (size_t)a.nkv * HD * sizeof(TKV))));
    for (uint32_t kh0 = slice * HPI; kh0 < a.nkv; kh0 += step) {
        const uint32_t kh = kh0 + sub;
        const bool valid = kh < a.nkv;
        float v[8], vv[8];
        Vec8<TIn>::unpack(rk, v);
        Vec8<TIn>::unpack(rv, vv);
        rk = Raw{}; rv = Raw{};
        kv_request(kh0 + step);
        m.norm_rope(v, m.wk);
        if (valid) {
            if (a.write_k_back) Vec8<TIn>::store(k_io + (size_t)kh * HD + d0, v);
            if constexpr (sizeof(TKV) == 1) {   // 8-bit cache: stored = value / scale
#pragma unroll
                for (int e = 0; e < 8; ++e) { v[e] *= a.k_inv; vv[e] *= a.v_inv; }
            }
            Vec8<TKV>::store(k_row + (size_t)kh * HD + d0, v);
            Vec8<TKV>::store(v_row + (size_t)kh * HD + d0, vv);
        }
    }
    // ---- Q heads ----
    for (uint32_t h0 = slice * HPI; h0 < a.nh && !a.skip_q;) {
#pragma unroll
        for (int u = 0; u < kPF; ++u) {
            if (h0 < a.nh) {   // (the same for every lane)
                const uint32_t h = h0 + sub;
                const bool valid = h < a.nh;
                float v[8];
                Vec8<TIn>::unpack(rq[u], v);
                q_request(rq[u]);
                if (valid && a.has_gate && a.q_gate) {
                    float gt[8];
                    Vec8<TIn>::load(q_in + (size_t)h * qrow + HD + d0, gt);
                    Vec8<float>::store(a.q_gate + (tok * a.nh + h) * (size_t)HD + d0, gt);
                }
                m.norm_rope(v, m.wq);
                if (valid) Vec8<TQ>::store(q_out + (size_t)h * HD + d0, v);
                h0 += step;
            }
        }
    }
}

// ---------------------------------------------------------------------------------------
// Staged path (many tokens, 16-bit projections in the cache's dtype): one warp per token.  The token's K, V and Q
// rows come into shared memory as a few bulk copies (each a contiguous run of up to nh * HD elements, so memory sees
// long bursts instead of one 256/512-byte row per trip and the warp waits once, not once per head); K and Q are
// normed and rotated in place; the rows go out as bulk copies from the same bytes (V is never touched by a lane).
// ---------------------------------------------------------------------------------------
namespace stg {
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void bulk_load(void *dst_smem, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst_smem)), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void bulk_store(void *dst, const void *src_smem, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                 ::"l"(dst), "r"(smem_u32(src_smem)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
}   // namespace stg

constexpr int kTimeoutAppendStage = 17;   // status code: a token's bulk copies did not land

template <typename T, int HD>
__global__ void __launch_bounds__(kAppendWarps * 32) append_staged_kernel(const AppendArgs a) {
    constexpr int LPH = HD / 8, HPI = 32 / LPH;
    extern __shared__ __align__(128) unsigned char stage_smem[];
    __shared__ __align__(8) unsigned long long bars[kAppendWarps];
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const unsigned long long tok = (unsigned long long)blockIdx.x * kAppendWarps + warp;
    uint32_t s, j;
    if (!locate_token(a, tok, s, j)) return;   // (nothing below synchronises across warps)
    const uint32_t sub = lane / LPH, dl = lane % LPH, d0 = dl * 8;
    const uint32_t kv_elems = a.nkv * HD, q_elems = a.skip_q ? 0u : a.nh * HD;
    T *sk = reinterpret_cast<T *>(stage_smem + (size_t)warp * a.stage_bytes), *sv = sk + kv_elems, *sq = sv + kv_elems;
    T *k_io = reinterpret_cast<T *>(a.k_io) + tok * (size_t)kv_elems;
    const T *v_in = reinterpret_cast<const T *>(a.v_in) + tok * (size_t)kv_elems;
    const uint32_t qrow = a.has_gate ? 2 * HD : HD;
    const T *q_in = reinterpret_cast<const T *>(a.q_in) + tok * a.nh * (size_t)qrow;
    const uint32_t bar = stg::smem_u32(&bars[warp]);
    if (lane == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"((2 * kv_elems + q_elems) * (uint32_t)sizeof(T)) : "memory");
        stg::bulk_load(sk, k_io, kv_elems * sizeof(T), bar);
        stg::bulk_load(sv, v_in, kv_elems * sizeof(T), bar);
        if (q_elems) {
            if (!a.has_gate) stg::bulk_load(sq, q_in, q_elems * sizeof(T), bar);
            else for (uint32_t h = 0; h < a.nh; ++h) stg::bulk_load(sq + h * HD, q_in + (size_t)h * qrow, HD * sizeof(T), bar);   // the gate halves stay where they are
        }
    }
    __syncwarp();
    LaneMath<HD> m;
    m.init(a, s, j, dl, sub == 0);   // (under the copies)
    // Bounded wait for the copies.  If it runs out the code is latched and the warp waits once more, as long again,
    // before it leaves: the shared memory must not go to another block while a copy may still land in it.
    bool landed = false;
    for (uint32_t round = 0; round < 2 && !landed; ++round) {
        for (uint32_t i = 0; i < a.wait_limit && !landed; ++i) landed = stg::mbar_try(bar, 0);
        if (!landed && round == 0) report_timeout(a.status, kTimeoutAppendStage);
    }
    if (!landed) return;
    // two trips' heads per turn (norm_rope2)
    auto heads_in_place = [&](T *rows, uint32_t n, const float (&w)[8]) {
        for (uint32_t h0 = 0; h0 < n; h0 += 2 * HPI) {
            const uint32_t ha = h0 + sub, hb = h0 + HPI + sub;
            float u[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            if (ha < n) Vec8<T>::load(rows + ha * HD + d0, u);
            if (hb < n) Vec8<T>::load(rows + hb * HD + d0, v);
            m.norm_rope2(u, v, w);
            if (ha < n) Vec8<T>::store(rows + ha * HD + d0, u);
            if (hb < n) Vec8<T>::store(rows + hb * HD + d0, v);
        }
    };
    heads_in_place(sk, a.nkv, m.wk);
    if (q_elems) heads_in_place(sq, a.nh, m.wq);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the lanes' writes, before the bulk copies read them
    __syncwarp();
    if (lane == 0) {
        const size_t row_bytes = (size_t)kv_elems * sizeof(T);
        stg::bulk_store(const_cast<char *>(kv_row_ptr(a.kv, false, s, m.p_t, row_bytes)), sk, (uint32_t)row_bytes);
        stg::bulk_store(const_cast<char *>(kv_row_ptr(a.kv, true, s, m.p_t, row_bytes)), sv, (uint32_t)row_bytes);
        if (a.write_k_back) stg::bulk_store(k_io, sk, (uint32_t)row_bytes);
        if (q_elems) stg::bulk_store(reinterpret_cast<T *>(a.q_out) + tok * (size_t)q_elems, sq, q_elems * sizeof(T));
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // the block's shared memory stays until the copies have read it
    }
    __syncwarp();
}

// The staged kernel takes a pass when every token has a warp's worth of work anyway (no head slices), the three
// tensors share one 16-bit type, nobody wants the gate copied out, and four tokens' rows fit a block's shared memory.
template <typename T>
static bool try_append_staged(shady_ctx *ctx, AppendArgs &a, unsigned long long toks) {
    if (a.has_gate && a.q_gate) return false;
    if (toks < (unsigned long long)ctx->num_sms * 8) return false;
    const size_t stage = ((size_t)(2 * a.nkv + (a.skip_q ? 0 : a.nh)) * a.hd * sizeof(T) + 127) & ~(size_t)127;
    const size_t smem = stage * kAppendWarps;
    if (smem > 96 * 1024) return false;   // (two blocks of four warps per SM at least)
    if (!a.skip_q && (((uintptr_t)a.q_in | (uintptr_t)a.q_out) & 15)) return false;
    if ((((uintptr_t)a.k_io | (uintptr_t)a.v_in | (uintptr_t)a.kv.k_base | (uintptr_t)a.kv.v_base) & 15) || (a.kv.seq_stride_bytes & 15) ||
        (a.kv.page_bytes & 15))
        return false;   // bulk copies start on 16-byte boundaries
    a.head_slices = 1;
    a.stage_bytes = (uint32_t)stage; a.wait_limit = ctx->wait_mbar; a.status = status_ref(ctx);
    const unsigned blocks = (unsigned)((toks + kAppendWarps - 1) / kAppendWarps);
    auto launch = [&](auto kernel) {
        if (smem > 40 * 1024 &&   // (the kernel's static words count against the 48 KB a launch gets unasked)
            cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
            (void)cudaGetLastError();
            return false;
        }
        kernel<<<blocks, kAppendWarps * 32, smem, ctx->stream>>>(a);
        return true;
    };
    return a.hd == 128 ? launch(append_staged_kernel<T, 128>) : launch(append_staged_kernel<T, 256>);
}

template <typename TIn, typename TQ, typename TKV>
static void launch_append_fast(shady_ctx *ctx, AppendArgs &a) {
    const unsigned long long toks = a.tok_start ? a.total_tokens : (unsigned long long)a.num_seqs * a.T;
    if constexpr (std::is_same<TIn, TQ>::value && std::is_same<TIn, TKV>::value && sizeof(TIn) == 2) {
        if (try_append_staged<TIn>(ctx, a, toks)) return;
    }
    // enough warps to fill the GPU: split a token's heads over several warps when there are few tokens
    const uint32_t hpi = 32 / (a.hd / 8);
    const uint32_t max_slices = ((a.skip_q ? a.nkv : a.nh) + hpi - 1) / hpi;
    unsigned long long want = ((unsigned long long)ctx->num_sms * 8 + toks - 1) / toks;
    a.head_slices = (uint32_t)(want < 1 ? 1 : (want > max_slices ? max_slices : want));
    const unsigned blocks = (unsigned)((toks * a.head_slices + kAppendWarps - 1) / kAppendWarps);
    if (a.hd == 128) append_fast_kernel<TIn, TQ, TKV, 128><<<blocks, kAppendWarps * 32, 0, ctx->stream>>>(a);
    else append_fast_kernel<TIn, TQ, TKV, 256><<<blocks, kAppendWarps * 32, 0, ctx->stream>>>(a);
}

// true if a vectorised instantiation covers this call (and launches it)
static bool try_append_fast(shady_ctx *ctx, AppendArgs &a, const void *q_in, const void *k_io, const void *v_in,
                            const void *q_out) {
    if (!(a.hd == 128 || a.hd == 256) || !a.interleaved || (a.rd % 2)) return false;
    if ((unsigned long long)a.num_seqs * a.T > 0x3fffffffull) return false;
    if ((((uintptr_t)q_in | (uintptr_t)k_io | (uintptr_t)v_in | (uintptr_t)q_out | (uintptr_t)a.q_gate | (uintptr_t)a.kv.k_base |
          (uintptr_t)a.kv.v_base) & 15) || (a.kv.seq_stride_bytes & 15) || (a.kv.page_bytes & 15))
        return false;   // 16-byte vector accesses (per-sequence pointers are required to be 16-byte aligned too)
    const uint32_t i = a.in_dtype, q = a.q_dtype, k = a.kv_dtype;
    if (i == SHADY_F32 && q == SHADY_F32 && k == SHADY_F32) launch_append_fast<float, float, float>(ctx, a);
    else if (i == SHADY_F32 && q == SHADY_F32 && k == SHADY_F16) launch_append_fast<float, float, __half>(ctx, a);
    else if (i == SHADY_F32 && q == SHADY_F32 && k == SHADY_BF16) launch_append_fast<float, float, __nv_bfloat16>(ctx, a);
    else if (i == SHADY_F16 && q == SHADY_F16 && k == SHADY_F16) launch_append_fast<__half, __half, __half>(ctx, a);
    else if (i == SHADY_BF16 && q == SHADY_BF16 && k == SHADY_BF16) launch_append_fast<__nv_bfloat16, __nv_bfloat16, __nv_bfloat16>(ctx, a);
    else if (i == SHADY_F32 && q == SHADY_F32 && k == SHADY_F8E4M3) launch_append_fast<float, float, __nv_fp8_e4m3>(ctx, a);
    else if (i == SHADY_F16 && q == SHADY_F16 && k == SHADY_F8E4M3) launch_append_fast<__half, __half, __nv_fp8_e4m3>(ctx, a);
    else if (i == SHADY_F32 && q == SHADY_F32 && k == SHADY_F8E5M2) launch_append_fast<float, float, __nv_fp8_e5m2>(ctx, a);
    else if (i == SHADY_F16 && q == SHADY_F16 && k == SHADY_F8E5M2) launch_append_fast<__half, __half, __nv_fp8_e5m2>(ctx, a);
    else return false;
    return true;
}

int launch_append_kv_table(shady_ctx *ctx, const shady_append_params *p, const void *d_k_proj, const void *d_v_proj,
                           const shady_kv_cache *cache, const uint16_t *d_qk_norm_bf16, float2 *d_cs_table, const AppendRagged *rg) {
    SHADY_REQUIRE(ctx, p->head_dim == 128 && p->in_dtype == cache->dtype && p->in_dtype != SHADY_F32, SHADY_ERR_UNSUPPORTED,
                  "attn_prefill_append: head_dim 128 and 16-bit projections in the cache dtype");
    AppendArgs a{};
    a.k_io = const_cast<void *>(d_k_proj); a.v_in = d_v_proj;
    if (const int st = fill_kv_addr(ctx, cache, p->num_kv_heads, p->head_dim, "attn_prefill_append", &a.kv)) return st;
    a.norm_w = d_qk_norm_bf16;
    a.nh = p->num_heads; a.nkv = p->num_kv_heads; a.hd = p->head_dim; a.eps = p->eps;
    a.rd = p->rotary_dim; a.s1 = p->s1_limit; a.s2 = p->s2_limit; a.interleaved = 1;
    a.num_seqs = p->num_seqs; a.T = p->tokens_per_seq;
    a.in_dtype = a.q_dtype = a.kv_dtype = p->in_dtype;
    a.skip_q = 1; a.cs_table = d_cs_table;
    if (rg) { a.tok_start = rg->d_tok_start; a.total_tokens = rg->total_tokens; a.table_seq = rg->table_seq; }
    a.k_inv = a.v_inv = 1.0f;
    for (uint32_t i = 0; i < p->rotary_dim / 2; ++i)   // wgsl:57, same libm call as everywhere else
        a.inv_freq[i] = 1.0f / powf(p->rope_theta, 2.0f * (float)i / (float)p->rotary_dim);
    SHADY_REQUIRE(ctx, (rg ? (unsigned long long)rg->total_tokens : (unsigned long long)a.num_seqs * a.T) <= 0x3fffffffull, SHADY_ERR_UNSUPPORTED,
                  "attn_prefill_append: too many tokens for one launch");
    SHADY_REQUIRE(ctx, !((((uintptr_t)d_k_proj | (uintptr_t)d_v_proj | (uintptr_t)a.kv.k_base | (uintptr_t)a.kv.v_base) & 15) ||
                         (a.kv.seq_stride_bytes & 15)),
                  SHADY_ERR_BAD_ARG, "attn_prefill_append: buffers must be 16-byte aligned");
    if (p->in_dtype == SHADY_F16) launch_append_fast<__half, __half, __half>(ctx, a);
    else launch_append_fast<__nv_bfloat16, __nv_bfloat16, __nv_bfloat16>(ctx, a);
    ctx->launches++;
    SHADY_CUDA_OK(ctx, cudaGetLastError());
    return SHADY_OK;
}

// `internal`: called by another launcher of this library, which may leave out the gate output and the positions
// (all sequences then start at position 0)
int launch_append_ex(shady_ctx *ctx, const shady_append_params *p, const void *d_q_proj_full, void *d_k_proj,
                     const void *d_v_proj, void *d_q_out, float *d_q_gate, const shady_kv_cache *cache,
                     const uint16_t *d_qk_norm_bf16, const uint32_t *d_pos_start, const uint32_t *d_pos_h,
                     const uint32_t *d_pos_w, bool internal, const AppendRagged *rg) {
    SHADY_REQUIRE(ctx, p && d_q_proj_full && d_k_proj && d_v_proj && d_q_out && cache && (d_pos_start || internal),
                  SHADY_ERR_BAD_ARG, "kv_append_rope: null argument");
    SHADY_REQUIRE(ctx, p->num_heads && p->num_kv_heads && p->head_dim && p->num_seqs && (p->tokens_per_seq || rg),
                  SHADY_ERR_BAD_ARG, "kv_append_rope: zero-sized problem");
    SHADY_REQUIRE(ctx, p->head_dim <= 256, SHADY_ERR_UNSUPPORTED, "kv_append_rope: head_dim > 256 (the reference shader's limit)");
    SHADY_REQUIRE(ctx, p->rotary_dim <= p->head_dim && (p->rotary_dim % 2) == 0, SHADY_ERR_BAD_ARG,
                  "kv_append_rope: rotary_dim must be even and <= head_dim");
    SHADY_REQUIRE(ctx, p->in_dtype <= SHADY_BF16 && p->q_dtype <= SHADY_BF16 && cache->dtype <= SHADY_F8E5M2,
                  SHADY_ERR_BAD_ARG, "kv_append_rope: bad dtype");
    SHADY_REQUIRE(ctx, !p->has_gate || d_q_gate || internal, SHADY_ERR_BAD_ARG, "kv_append_rope: has_gate needs d_q_gate");
    SHADY_REQUIRE(ctx, (cache->d_k_ptrs && cache->d_v_ptrs) || (cache->d_k_base && cache->d_v_base),
                  SHADY_ERR_BAD_ARG, "kv_append_rope: cache has neither base pointers nor pointer arrays");
    AppendArgs a{};
    a.q_in = d_q_proj_full; a.k_io = d_k_proj; a.v_in = d_v_proj; a.q_out = d_q_out; a.q_gate = d_q_gate;
    if (const int st = fill_kv_addr(ctx, cache, p->num_kv_heads, p->head_dim, "kv_append_rope", &a.kv)) return st;
    a.norm_w = d_qk_norm_bf16;
    a.pos_start = d_pos_start; a.pos_h = d_pos_h; a.pos_w = d_pos_w;
    a.nh = p->num_heads; a.nkv = p->num_kv_heads; a.hd = p->head_dim; a.eps = p->eps;
    a.rd = p->rotary_dim; a.s1 = p->s1_limit; a.s2 = p->s2_limit; a.interleaved = p->interleaved;
    a.num_seqs = p->num_seqs; a.T = p->tokens_per_seq;
    a.in_dtype = p->in_dtype; a.q_dtype = p->q_dtype; a.kv_dtype = cache->dtype;
    a.has_gate = p->has_gate; a.write_k_back = p->write_k_back;
    a.k_inv = 1.0f / a.kv.k_scale; a.v_inv = 1.0f / a.kv.v_scale;
    if (rg) { a.tok_start = rg->d_tok_start; a.total_tokens = rg->total_tokens; a.table_seq = rg->table_seq; }
    // apply_mrope: freq = 1.0 / pow(ROPE_THETA, 2.0 * f32(freq_idx) / f32(PARTIAL_DIM))  (wgsl:57)
    for (uint32_t i = 0; i < p->rotary_dim / 2; ++i)
        a.inv_freq[i] = 1.0f / powf(p->rope_theta, 2.0f * (float)i / (float)p->rotary_dim);
    const unsigned long long warps = (unsigned long long)p->num_seqs * p->tokens_per_seq * (p->num_heads + p->num_kv_heads);
    const unsigned long long blocks = (warps + kAppendWarps - 1) / kAppendWarps;
    SHADY_REQUIRE(ctx, blocks <= 0x7fffffffull, SHADY_ERR_UNSUPPORTED, "kv_append_rope: too many tokens for one launch");
    if (!try_append_fast(ctx, a, d_q_proj_full, d_k_proj, d_v_proj, d_q_out)) {
        SHADY_REQUIRE(ctx, !rg, SHADY_ERR_UNSUPPORTED,
                      "kv_append_rope: a listed batch needs interleaved RoPE, head_dim 128 or 256 and 16-byte aligned buffers");
        append_kernel<<<(unsigned)blocks, kAppendWarps * 32, 0, ctx->stream>>>(a);
    }
    ctx->launches++;
    SHADY_CUDA_OK(ctx, cudaGetLastError());
    return SHADY_OK;
}

int launch_append(shady_ctx *ctx, const shady_append_params *p, const void *d_q_proj_full, void *d_k_proj,
                  const void *d_v_proj, void *d_q_out, float *d_q_gate, const shady_kv_cache *cache,
                  const uint16_t *d_qk_norm_bf16, const uint32_t *d_pos_start, const uint32_t *d_pos_h,
                  const uint32_t *d_pos_w) {
    return launch_append_ex(ctx, p, d_q_proj_full, d_k_proj, d_v_proj, d_q_out, d_q_gate, cache, d_qk_norm_bf16, d_pos_start,
                            d_pos_h, d_pos_w, false, nullptr);
}

}  // namespace shady
