// Split-KV GQA decode attention for sm_100a.
//
// What it computes is gqa_attention_head.wgsl:30-124 (one query token per sequence attends
// to rows [0, L) of that sequence's cache with an online softmax) followed by
// gqa_reduce.wgsl:20-65 (log-sum-exp merge of the splits) — but the work is laid out for
// HBM bandwidth instead of one workgroup per (q_head, split):
//   * one CTA owns (sequence, kv_head, position range) and serves ALL query heads of the
//     KV group from one pass over the K/V rows, so each cache byte leaves HBM once;
//   * 16-bit caches: every warp runs a private multi-stage cp.async (16-byte, L2-only)
//     pipeline over 16-position blocks into XOR-swizzled shared memory, feeds
//     mma.sync.m16n8k16 through ldmatrix (query heads on the M axis), keeps the softmax
//     statistics in fp32 with quad shuffles; no block-wide barrier in the main loop;
//   * fp32 caches (the reference's native format): lanes span head_dim with 128-bit
//     loads, warp-shuffle dot products, fp32 FMA;
//   * ranges come either from an explicit num_splits (ceil(L/ns) ranges, wgsl:46-48) or
//     from a length-balanced chunking that every CTA re-derives from the device-side
//     lengths with a warp scan, so no plan has to be uploaded.
#include "common.cuh"

namespace shady {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

struct DecodeArgs {
    const void *q;
    void *out;
    float *lse;
    const float *gate;
    KvAddr kv;
    const uint32_t *seq_lens;
    float *partials;     // workspace: per sequence [nh][ns][hd+2]
    uint2 *seq_info;     // workspace: per sequence {ns, first split index}
    uint32_t num_seqs, nkv, nh, G, hd;
    uint32_t num_splits; // >0 explicit, 0 = chunked
    uint32_t chunk;      // positions per split in chunked mode
    uint32_t q_dtype, out_dtype;
    uint32_t force_partials;  // 1: always write the partial record (shady_attn_decode_partials)
    float scale_log2;         // 1/sqrt(hd) * log2(e)
};

__device__ __forceinline__ uint32_t splits_of(const DecodeArgs &a, uint32_t L) {
    if (a.num_splits) return a.num_splits;
    return L == 0 ? 1u : (L + a.chunk - 1u) / a.chunk;
}

// Map blockIdx.x -> (sequence, split, splits of that sequence, splits before it).
// Executed by warp 0; result broadcast through shared memory by the caller.
__device__ __forceinline__ void resolve_item(const DecodeArgs &a, uint32_t item, uint32_t lane,
                                             uint32_t *res /*[4]*/) {
    if (a.num_splits) {
        if (lane == 0) {
            res[0] = item / a.num_splits;
            res[1] = item % a.num_splits;
            res[2] = a.num_splits;
            res[3] = (item / a.num_splits) * a.num_splits;
        }
        return;
    }
    uint32_t pref = 0;
    bool found = false;
    for (uint32_t base = 0; base < a.num_seqs && !found; base += 32) {
        const uint32_t j = base + lane;
        const uint32_t ns = j < a.num_seqs ? splits_of(a, a.seq_lens[j]) : 0u;
        uint32_t incl = ns;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t n = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= (uint32_t)o) incl += n;
        }
        const uint32_t total = __shfl_sync(0xffffffffu, incl, 31);
        if (item < pref + total) {
            const uint32_t mask = __ballot_sync(0xffffffffu, pref + incl > item);
            const uint32_t f = __ffs(mask) - 1;
            const uint32_t ns_f = __shfl_sync(0xffffffffu, ns, f);
            const uint32_t excl = __shfl_sync(0xffffffffu, incl, f) - ns_f;
            if (lane == 0) {
                res[0] = base + f;
                res[1] = item - pref - excl;
                res[2] = ns_f;
                res[3] = pref + excl;
            }
            found = true;
        }
        pref += total;
    }
    if (!found && lane == 0) res[0] = 0xffffffffu;  // grid larger than the work: idle CTA
}

// Merge the per-warp (m, l, O) states of one CTA and write either the final rows or the
// split's partial record ([hd] = lse, [hd+1] = running max as in wgsl:112-123).
template <int R, int HD, int NW>
__device__ __forceinline__ void finish_cta(const DecodeArgs &a, const float *sm_m, const float *sm_l,
                                           const float *sm_o, uint32_t seq, uint32_t split, uint32_t ns,
                                           uint32_t pref, uint32_t head0, uint32_t rows_valid) {
    const bool direct = (ns == 1u) && !a.force_partials;
    for (uint32_t idx = threadIdx.x; idx < rows_valid * HD; idx += NW * 32) {
        const uint32_t r = idx / HD, d = idx % HD;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < NW; ++w) M = fmaxf(M, sm_m[w * R + r]);
        float L = 0.f, o = 0.f;
#pragma unroll
        for (int w = 0; w < NW; ++w) {
            const float mw = sm_m[w * R + r];
            if (mw > -INFINITY) {
                const float e = exp2f(mw - M);
                L += sm_l[w * R + r] * e;
                o += sm_o[((size_t)w * R + r) * HD + d] * e;
            }
        }
        float val = L > 0.f ? o / L : 0.f;
        const float lse = L > 0.f ? logf(L) + M * kLn2 : -INFINITY;
        const uint32_t head = head0 + r;
        if (direct) {
            const size_t oi = ((size_t)seq * a.nh + head) * HD + d;
            if (a.gate) val *= sigmoidf_ref(a.gate[oi]);
            store_from_f32(a.out, oi, a.out_dtype, val);
            if (d == 0 && a.lse) a.lse[(size_t)seq * a.nh + head] = lse;
        } else {
            float *rec = a.partials + ((size_t)pref * a.nh + (size_t)head * ns + split) * (HD + 2);
            rec[d] = val;
            if (d == 0) {
                rec[HD] = lse;
                rec[HD + 1] = L > 0.f ? M * kLn2 : -INFINITY;
            }
        }
    }
}

// ---------------------------------------------------------------------------------------
// 16-bit cache path
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void cp_async16(uint32_t smem, const void *gptr, bool valid) {
    const int sz = valid ? 16 : 0;  // src-size 0 => 16 bytes of zeros, nothing read
    asm volatile("cp.async.cg.shared.global.L2::128B [%0], [%1], 16, %2;\n" ::"r"(smem), "l"(gptr), "r"(sz));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
template <typename T>
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mma16816<__half>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma16816<__nv_bfloat16>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <typename T> __device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pack2<__half>(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&h);
}
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&h);
}

constexpr int kBlk = 16;  // positions per warp block (one MMA k-step of P·V)

template <int HD, int NW, int STAGES> struct Decode16Smem {
    static constexpr int kRowBytes = HD * 2;
    static constexpr int kTileBytes = kBlk * kRowBytes;          // one K or V block
    static constexpr int kStageBytes = 2 * kTileBytes;           // K + V
    static constexpr int kWarpBytes = STAGES * kStageBytes;
    static constexpr int kQBytes = 16 * kRowBytes;
    static constexpr int kStatBytes = 2 * NW * 16 * 4;           // merge m and l
    static constexpr int kTotal = kQBytes + NW * kWarpBytes + kStatBytes + 16;
    static_assert(kWarpBytes >= 16 * HD * 4, "merge tile must fit in the warp's pipeline memory");
};

template <typename T, int HD, int NW, int STAGES>
__global__ void __launch_bounds__(NW * 32) decode16_kernel(const DecodeArgs a) {
    using S = Decode16Smem<HD, NW, STAGES>;
    constexpr int CH = HD / 8;  // 16-byte chunks per row
    extern __shared__ __align__(128) unsigned char smem[];
    unsigned char *sm_q = smem;
    unsigned char *sm_pipe = smem + S::kQBytes;
    float *sm_m = reinterpret_cast<float *>(smem + S::kQBytes + NW * S::kWarpBytes);
    float *sm_l = sm_m + NW * 16;
    uint32_t *sm_item = reinterpret_cast<uint32_t *>(sm_l + NW * 16);

    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (warp == 0) resolve_item(a, blockIdx.x, lane, sm_item);
    __syncthreads();
    const uint32_t seq = sm_item[0], split = sm_item[1], ns = sm_item[2], pref = sm_item[3];
    if (seq == 0xffffffffu) return;
    const uint32_t kvh = blockIdx.y;
    const uint32_t row0 = blockIdx.z * 16;                         // first head of the group handled here
    const uint32_t rows_valid = min(16u, a.G - row0);
    const uint32_t head0 = kvh * a.G + row0;
    const uint32_t L = a.seq_lens[seq];
    const uint32_t pps = (L + ns - 1u) / ns;                       // wgsl:46
    const uint32_t start = min(split * pps, L);
    const uint32_t end = min(start + pps, L);
    if (split == 0 && kvh == 0 && blockIdx.z == 0 && tid == 0 && a.seq_info) a.seq_info[seq] = make_uint2(ns, pref);

    // ---- stage Q (rows >= rows_valid are zero) as T, swizzled ----
    for (uint32_t idx = tid; idx < 16 * CH; idx += NW * 32) {
        const uint32_t r = idx / CH, c = idx % CH;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < rows_valid) {
            const size_t e0 = ((size_t)seq * a.nh + head0 + r) * HD + c * 8;
            if (a.q_dtype == SHADY_F32) {
                const float4 f0 = *reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(a.q) + e0);
                const float4 f1 = *reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(a.q) + e0 + 4);
                v.x = pack2<T>(f0.x, f0.y); v.y = pack2<T>(f0.z, f0.w);
                v.z = pack2<T>(f1.x, f1.y); v.w = pack2<T>(f1.z, f1.w);
            } else {
                v = *reinterpret_cast<const uint4 *>(reinterpret_cast<const T *>(a.q) + e0);
            }
        }
        *reinterpret_cast<uint4 *>(sm_q + r * S::kRowBytes + ((c ^ (r & 7)) << 4)) = v;
    }
    __syncthreads();

    const uint32_t g = lane >> 2, t = lane & 3;
    const uint32_t mat = lane >> 3, rin = lane & 7;
    const uint32_t sm_q_addr = (uint32_t)__cvta_generic_to_shared(sm_q);
    // Q fragments (A operand), one ldmatrix.x4 per k-step: mats = (rows0-7,c), (rows8-15,c), (rows0-7,c+1), (rows8-15,c+1)
    uint32_t qa[HD / 16][4];
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
        const uint32_t row = (mat & 1) * 8 + rin, chunk = 2 * ks + (mat >> 1);
        ldsm_x4(qa[ks], sm_q_addr + row * S::kRowBytes + ((chunk ^ rin) << 4));
    }

    const char *kbase = kv_seq_ptr(a.kv.k_base, a.kv.k_ptrs, a.kv.seq_stride_bytes, seq) + (size_t)kvh * S::kRowBytes;
    const char *vbase = kv_seq_ptr(a.kv.v_base, a.kv.v_ptrs, a.kv.seq_stride_bytes, seq) + (size_t)kvh * S::kRowBytes;
    const size_t pos_stride = (size_t)a.nkv * S::kRowBytes;

    const uint32_t nblk = (end - start + kBlk - 1) / kBlk;
    const uint32_t my_n = nblk > warp ? (nblk - warp + NW - 1) / NW : 0;
    const uint32_t warp_smem = (uint32_t)__cvta_generic_to_shared(sm_pipe + warp * S::kWarpBytes);

    // per-lane load geometry: a warp instruction copies 512 bytes = 512/kRowBytes rows
    constexpr int RPI = 512 / S::kRowBytes;          // rows per instruction (2 for hd128, 1 for hd256)
    constexpr int NI = kBlk / RPI;                   // instructions per tile
    const uint32_t l_row = lane / CH * (RPI > 1), l_chunk = lane % CH;
    auto issue = [&](uint32_t bi) {
        const uint32_t pos0 = start + (warp + bi * NW) * kBlk;
        const uint32_t st = warp_smem + (bi % STAGES) * S::kStageBytes;
#pragma unroll
        for (int i = 0; i < NI; ++i) {
            const uint32_t r = i * RPI + l_row;
            const bool ok = pos0 + r < end;
            const size_t goff = (size_t)(pos0 + r) * pos_stride + l_chunk * 16;
            const uint32_t soff = r * S::kRowBytes + ((l_chunk ^ (r & 7)) << 4);
            cp_async16(st + soff, kbase + (ok ? goff : 0), ok);
            cp_async16(st + S::kTileBytes + soff, vbase + (ok ? goff : 0), ok);
        }
    };

    float o[HD / 8][4];
#pragma unroll
    for (int j = 0; j < HD / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
        if ((uint32_t)s < my_n) issue(s);
        cp_async_commit();
    }
    for (uint32_t i = 0; i < my_n; ++i) {
        cp_async_wait<STAGES - 2>();
        __syncwarp();
        if (i + STAGES - 1 < my_n) issue(i + STAGES - 1);
        cp_async_commit();

        const uint32_t st = warp_smem + (i % STAGES) * S::kStageBytes;
        const uint32_t pos0 = start + (warp + i * NW) * kBlk;
        // ---- S = Q K^T : heads x 16 positions ----
        float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
            uint32_t kb[4];
            const uint32_t row = (mat >> 1) * 8 + rin, chunk = 2 * ks + (mat & 1);
            ldsm_x4(kb, st + row * S::kRowBytes + ((chunk ^ rin) << 4));
            mma16816<T>(s[0], qa[ks], kb[0], kb[1]);
            mma16816<T>(s[1], qa[ks], kb[2], kb[3]);
        }
        // ---- online softmax (log2 domain), rows g and g+8 ----
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const uint32_t pos = pos0 + 8 * j + 2 * t + (c & 1);
                s[j][c] = pos < end ? s[j][c] * a.scale_log2 : -INFINITY;
                mx[c >> 1] = fmaxf(mx[c >> 1], s[j][c]);
            }
        float corr[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
            const float m_new = fmaxf(m_run[r], mx[r]);   // finite: every block holds >= 1 valid position
            corr[r] = exp2f(m_run[r] - m_new);
            m_run[r] = m_new;
        }
        float psum[2] = {0.f, 0.f};
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                s[j][c] = exp2f(s[j][c] - m_run[c >> 1]);
                psum[c >> 1] += s[j][c];
            }
        l_run[0] = l_run[0] * corr[0] + psum[0];
        l_run[1] = l_run[1] * corr[1] + psum[1];
        uint32_t pa[4];
        pa[0] = pack2<T>(s[0][0], s[0][1]);
        pa[1] = pack2<T>(s[0][2], s[0][3]);
        pa[2] = pack2<T>(s[1][0], s[1][1]);
        pa[3] = pack2<T>(s[1][2], s[1][3]);
        // ---- O = O*corr + P V ----
#pragma unroll
        for (int jn = 0; jn < HD / 8; jn += 2) {
            uint32_t vb[4];
            const uint32_t row = (mat & 1) * 8 + rin, chunk = jn + (mat >> 1);
            ldsm_x4_t(vb, st + S::kTileBytes + row * S::kRowBytes + ((chunk ^ rin) << 4));
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                o[jn + u][0] *= corr[0]; o[jn + u][1] *= corr[0];
                o[jn + u][2] *= corr[1]; o[jn + u][3] *= corr[1];
            }
            mma16816<T>(o[jn], pa, vb[0], vb[1]);
            mma16816<T>(o[jn + 1], pa, vb[2], vb[3]);
        }
    }
    cp_async_wait<0>();
    __syncthreads();  // every warp is done with its pipeline memory: reuse it for the merge

    // ---- per-warp state -> shared ----
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
    float *sm_o = reinterpret_cast<float *>(sm_pipe);  // [NW][16][HD], warp w at w*kWarpBytes
    static_assert(S::kWarpBytes % 4 == 0, "");
    float *my_o = reinterpret_cast<float *>(sm_pipe + warp * S::kWarpBytes);
    if (t == 0) {
        sm_m[warp * 16 + g] = m_run[0];
        sm_m[warp * 16 + g + 8] = m_run[1];
        sm_l[warp * 16 + g] = l_run[0];
        sm_l[warp * 16 + g + 8] = l_run[1];
    }
#pragma unroll
    for (int jn = 0; jn < HD / 8; ++jn) {
        *reinterpret_cast<float2 *>(my_o + g * HD + jn * 8 + 2 * t) = make_float2(o[jn][0], o[jn][1]);
        *reinterpret_cast<float2 *>(my_o + (g + 8) * HD + jn * 8 + 2 * t) = make_float2(o[jn][2], o[jn][3]);
    }
    __syncthreads();
    // finish_cta indexes warp w's tile at sm_o + w*16*HD floats; the tiles sit kWarpBytes apart,
    // so merge through a strided view.
    {
        const bool direct = (ns == 1u) && !a.force_partials;
        constexpr int WSTRIDE = S::kWarpBytes / 4;
        for (uint32_t idx = tid; idx < rows_valid * HD; idx += NW * 32) {
            const uint32_t r = idx / HD, d = idx % HD;
            float M = -INFINITY;
#pragma unroll
            for (int w = 0; w < NW; ++w) M = fmaxf(M, sm_m[w * 16 + r]);
            float Ls = 0.f, acc = 0.f;
#pragma unroll
            for (int w = 0; w < NW; ++w) {
                const float mw = sm_m[w * 16 + r];
                if (mw > -INFINITY) {
                    const float e = exp2f(mw - M);
                    Ls += sm_l[w * 16 + r] * e;
                    acc += sm_o[(size_t)w * WSTRIDE + r * HD + d] * e;
                }
            }
            float val = Ls > 0.f ? acc / Ls : 0.f;
            const float lse = Ls > 0.f ? logf(Ls) + M * kLn2 : -INFINITY;
            const uint32_t head = head0 + r;
            if (direct) {
                const size_t oi = ((size_t)seq * a.nh + head) * HD + d;
                if (a.gate) val *= sigmoidf_ref(a.gate[oi]);
                store_from_f32(a.out, oi, a.out_dtype, val);
                if (d == 0 && a.lse) a.lse[(size_t)seq * a.nh + head] = lse;
            } else {
                float *rec = a.partials + ((size_t)pref * a.nh + (size_t)head * ns + split) * (HD + 2);
                rec[d] = val;
                if (d == 0) {
                    rec[HD] = lse;
                    rec[HD + 1] = Ls > 0.f ? M * kLn2 : -INFINITY;
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------------------
// fp32 cache path (the reference's own cache format)
// ---------------------------------------------------------------------------------------
template <int HD, int GT, int NW>
__global__ void __launch_bounds__(NW * 32) decode32_kernel(const DecodeArgs a) {
    constexpr int EPL = HD / 32;                 // elements per lane
    constexpr int VEC = EPL >= 4 ? 4 : EPL;      // floats per vector load
    constexpr int NV = EPL / VEC;
    constexpr int U = 4;                         // positions in flight per warp
    __shared__ float sm_m[NW * GT], sm_l[NW * GT];
    __shared__ float sm_o[NW * GT * HD];
    __shared__ uint32_t sm_item[4];

    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (warp == 0) resolve_item(a, blockIdx.x, lane, sm_item);
    __syncthreads();
    const uint32_t seq = sm_item[0], split = sm_item[1], ns = sm_item[2], pref = sm_item[3];
    if (seq == 0xffffffffu) return;
    const uint32_t kvh = blockIdx.y;
    const uint32_t row0 = blockIdx.z * GT;
    const uint32_t rows_valid = min((uint32_t)GT, a.G - row0);
    const uint32_t head0 = kvh * a.G + row0;
    const uint32_t L = a.seq_lens[seq];
    const uint32_t pps = (L + ns - 1u) / ns;
    const uint32_t start = min(split * pps, L);
    const uint32_t end = min(start + pps, L);
    if (split == 0 && kvh == 0 && blockIdx.z == 0 && tid == 0 && a.seq_info) a.seq_info[seq] = make_uint2(ns, pref);

    // lane owns dims (i*32 + lane)*VEC + e
    float q[GT][EPL];
#pragma unroll
    for (int h = 0; h < GT; ++h)
#pragma unroll
        for (int i = 0; i < NV; ++i)
#pragma unroll
            for (int e = 0; e < VEC; ++e) {
                const uint32_t d = (i * 32 + lane) * VEC + e;
                q[h][i * VEC + e] = (uint32_t)h < rows_valid
                                        ? load_as_f32(a.q, ((size_t)seq * a.nh + head0 + h) * HD + d, a.q_dtype) * a.scale_log2
                                        : 0.f;
            }
    float acc[GT][EPL];
    float m_run[GT], l_run[GT];
#pragma unroll
    for (int h = 0; h < GT; ++h) {
        m_run[h] = -INFINITY;
        l_run[h] = 0.f;
#pragma unroll
        for (int e = 0; e < EPL; ++e) acc[h][e] = 0.f;
    }
    const float *kbase = reinterpret_cast<const float *>(kv_seq_ptr(a.kv.k_base, a.kv.k_ptrs, a.kv.seq_stride_bytes, seq)) + (size_t)kvh * HD;
    const float *vbase = reinterpret_cast<const float *>(kv_seq_ptr(a.kv.v_base, a.kv.v_ptrs, a.kv.seq_stride_bytes, seq)) + (size_t)kvh * HD;
    const size_t pos_stride = (size_t)a.nkv * HD;

    for (uint32_t p0 = start + warp * U; p0 < end; p0 += NW * U) {
        float kr[U][EPL], vr[U][EPL];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const uint32_t pos = min(p0 + u, end - 1);
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                const size_t off = (size_t)pos * pos_stride + (i * 32 + lane) * VEC;
                if constexpr (VEC == 4) {
                    const float4 kk = __ldcs(reinterpret_cast<const float4 *>(kbase + off));
                    const float4 vv = __ldcs(reinterpret_cast<const float4 *>(vbase + off));
                    kr[u][i * 4 + 0] = kk.x; kr[u][i * 4 + 1] = kk.y; kr[u][i * 4 + 2] = kk.z; kr[u][i * 4 + 3] = kk.w;
                    vr[u][i * 4 + 0] = vv.x; vr[u][i * 4 + 1] = vv.y; vr[u][i * 4 + 2] = vv.z; vr[u][i * 4 + 3] = vv.w;
                } else {
#pragma unroll
                    for (int e = 0; e < VEC; ++e) {
                        kr[u][i * VEC + e] = __ldcs(kbase + off + e);
                        vr[u][i * VEC + e] = __ldcs(vbase + off + e);
                    }
                }
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (p0 + u >= end) break;
#pragma unroll
            for (int h = 0; h < GT; ++h) {
                float dot = 0.f;
#pragma unroll
                for (int e = 0; e < EPL; ++e) dot = fmaf(q[h][e], kr[u][e], dot);
                dot = warp_sum(dot);  // already in log2 units (q carries scale*log2e)
                const float m_new = fmaxf(m_run[h], dot);
                const float corr = exp2f(m_run[h] - m_new);
                const float p = exp2f(dot - m_new);
                l_run[h] = l_run[h] * corr + p;
#pragma unroll
                for (int e = 0; e < EPL; ++e) acc[h][e] = fmaf(p, vr[u][e], acc[h][e] * corr);
                m_run[h] = m_new;
            }
        }
    }
    // ---- merge the warps ----
#pragma unroll
    for (int h = 0; h < GT; ++h) {
        if (lane == 0) {
            sm_m[warp * GT + h] = m_run[h];
            sm_l[warp * GT + h] = l_run[h];
        }
#pragma unroll
        for (int i = 0; i < NV; ++i)
#pragma unroll
            for (int e = 0; e < VEC; ++e)
                sm_o[((size_t)warp * GT + h) * HD + (i * 32 + lane) * VEC + e] = acc[h][i * VEC + e];
    }
    __syncthreads();
    finish_cta<GT, HD, NW>(a, sm_m, sm_l, sm_o, seq, split, ns, pref, head0, rows_valid);
}

// ---------------------------------------------------------------------------------------
// Merge of split records (gqa_reduce.wgsl:20-65), batched and stride-generalised
// ---------------------------------------------------------------------------------------
struct ReduceArgs {
    const float *partials;
    void *out;
    float *lse;
    const float *gate;
    const uint2 *seq_info;   // batched decode: per-sequence {ns, first split}; else NULL
    uint32_t ns, nh, hd;
    unsigned long long split_stride, head_stride, seq_stride;  // floats
    uint32_t out_dtype;
    uint32_t skip_single;    // batched decode: ns == 1 rows were written by the decode kernel itself
};

__global__ void __launch_bounds__(128) reduce_kernel(const ReduceArgs a) {
    const uint32_t head = blockIdx.x, seq = blockIdx.y;
    uint32_t ns = a.ns;
    unsigned long long sstr = a.split_stride, hstr = a.head_stride;
    const float *base = a.partials + (size_t)seq * a.seq_stride;
    if (a.seq_info) {
        const uint2 info = a.seq_info[seq];
        ns = info.x;
        if (ns == 1 && a.skip_single) return;
        base = a.partials + (size_t)info.y * a.nh * (a.hd + 2);
        sstr = a.hd + 2;
        hstr = (unsigned long long)ns * (a.hd + 2);
    }
    const float *hb = base + (size_t)head * hstr;
    // wgsl:33-43 (a thread-0 loop there; every thread repeats it here, it is ns loads)
    float gmax = -INFINITY;
    for (uint32_t s = 0; s < ns; ++s) {
        const float l = hb[(size_t)s * sstr + a.hd];
        if (l > -INFINITY) gmax = fmaxf(gmax, l);  // false for -inf and NaN: empty splits
    }
    for (uint32_t d = threadIdx.x; d < a.hd; d += blockDim.x) {
        float acc = 0.f, wsum = 0.f;
        for (uint32_t s = 0; s < ns; ++s) {
            const float *rec = hb + (size_t)s * sstr;
            const float l = rec[a.hd];
            if (!(l > -INFINITY)) continue;
            const float w = expf(l - gmax);  // wgsl:56
            acc += w * rec[d];
            wsum += w;
        }
        float val = wsum > 0.f ? acc / wsum : 0.f;
        const size_t oi = ((size_t)seq * a.nh + head) * a.hd + d;
        if (a.gate) val *= sigmoidf_ref(a.gate[oi]);
        store_from_f32(a.out, oi, a.out_dtype, val);
        if (d == 0 && a.lse) a.lse[(size_t)seq * a.nh + head] = wsum > 0.f ? gmax + logf(wsum) : -INFINITY;
    }
}

__global__ void sigmoid_mul_kernel(float *x, const float *gate, uint32_t n) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] = x[i] * sigmoidf_ref(gate[i]);  // sigmoid_mul.wgsl:20-22
}

// ---------------------------------------------------------------------------------------
// Host launchers
// ---------------------------------------------------------------------------------------
template <typename T, int HD, int NW, int STAGES>
static int launch16(shady_ctx *ctx, const DecodeArgs &a, dim3 grid) {
    using S = Decode16Smem<HD, NW, STAGES>;
    auto kern = decode16_kernel<T, HD, NW, STAGES>;
    static thread_local int configured_dev = -1;
    if (configured_dev != ctx->device) {
        SHADY_CUDA_OK(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal));
        configured_dev = ctx->device;
    }
    kern<<<grid, NW * 32, S::kTotal, ctx->stream>>>(a);
    ctx->launches++;
    SHADY_CUDA_OK(ctx, cudaGetLastError());
    return SHADY_OK;
}

template <int HD, int NW>
static int launch32(shady_ctx *ctx, const DecodeArgs &a, uint32_t items) {
    const uint32_t G = a.G;
    const uint32_t GT = G >= 8 ? 8 : (G >= 4 ? 4 : (G >= 2 ? 2 : 1));
    dim3 grid(items, a.nkv, (G + GT - 1) / GT);
    switch (GT) {
        case 8: decode32_kernel<HD, 8, NW><<<grid, NW * 32, 0, ctx->stream>>>(a); break;
        case 4: decode32_kernel<HD, 4, NW><<<grid, NW * 32, 0, ctx->stream>>>(a); break;
        case 2: decode32_kernel<HD, 2, NW><<<grid, NW * 32, 0, ctx->stream>>>(a); break;
        default: decode32_kernel<HD, 1, NW><<<grid, NW * 32, 0, ctx->stream>>>(a); break;
    }
    ctx->launches++;
    SHADY_CUDA_OK(ctx, cudaGetLastError());
    return SHADY_OK;
}

// Work-size policy for the chunked mode: aim at `waves` full waves of resident CTAs.
struct DecodePolicy {
    uint32_t min_chunk, ctas_per_sm, waves;
};
static DecodePolicy policy_for(uint32_t kv_dtype, uint32_t hd) {
    if (kv_dtype == SHADY_F32) return {32u, 4u, 2u};
    return hd > 128 ? DecodePolicy{128u, 1u, 4u} : DecodePolicy{128u, 2u, 4u};
}
static uint32_t target_items(const shady_ctx *ctx, const DecodePolicy &pol) {
    return (uint32_t)ctx->num_sms * pol.ctas_per_sm * pol.waves;
}

size_t decode_workspace_bytes(const shady_ctx *ctx, const shady_decode_params *p, uint32_t kv_dtype) {
    const size_t rec = (size_t)p->num_q_heads * (p->head_dim + 2) * sizeof(float);
    const size_t info = (size_t)p->num_seqs * sizeof(uint2);
    size_t splits;
    if (p->num_splits >= 1) {
        if (p->num_splits == 1) return 0;
        splits = (size_t)p->num_seqs * p->num_splits;
    } else {
        // sum_i ceil(L_i/chunk) <= sum(L)/chunk + S and chunk >= sum(L)*nkv*gz/target
        const int sms = ctx ? ctx->num_sms : 148;
        uint32_t worst = 0;
        for (uint32_t dt = 0; dt < 3; ++dt)
            for (uint32_t hd : {128u, 256u}) {
                const DecodePolicy pol = policy_for(dt, hd);
                worst = worst > (uint32_t)sms * pol.ctas_per_sm * pol.waves ? worst : (uint32_t)sms * pol.ctas_per_sm * pol.waves;
            }
        (void)kv_dtype;
        splits = (size_t)worst / (p->num_kv_heads ? p->num_kv_heads : 1) + p->num_seqs + 1;
    }
    return ((info + 255) / 256) * 256 + splits * rec;
}

int launch_decode(shady_ctx *ctx, const shady_decode_params *p, const void *d_q, const shady_kv_cache *cache,
                  const uint32_t *d_seq_lens, const uint32_t *seq_lens_host, void *d_out, float *d_lse,
                  const float *d_gate, void *d_ws, size_t ws_bytes, float *d_force_partials) {
    SHADY_REQUIRE(ctx, p && d_q && cache && d_seq_lens, SHADY_ERR_BAD_ARG, "decode: null argument");
    SHADY_REQUIRE(ctx, d_out || d_force_partials, SHADY_ERR_BAD_ARG, "decode: null output");
    SHADY_REQUIRE(ctx, p->num_seqs > 0 && p->num_kv_heads > 0 && p->heads_per_kv > 0, SHADY_ERR_BAD_ARG,
                  "decode: zero-sized problem");
    SHADY_REQUIRE(ctx, p->num_q_heads == p->num_kv_heads * p->heads_per_kv, SHADY_ERR_BAD_ARG,
                  "decode: num_q_heads != num_kv_heads * heads_per_kv");
    SHADY_REQUIRE(ctx, cache->dtype <= SHADY_BF16, SHADY_ERR_BAD_ARG, "decode: bad cache dtype");
    SHADY_REQUIRE(ctx, (cache->d_k_ptrs && cache->d_v_ptrs) || (cache->d_k_base && cache->d_v_base),
                  SHADY_ERR_BAD_ARG, "decode: cache has neither base pointers nor pointer arrays");
    SHADY_REQUIRE(ctx, p->q_dtype == SHADY_F32 || p->q_dtype == cache->dtype, SHADY_ERR_UNSUPPORTED,
                  "decode: q_dtype must be f32 or the cache dtype");
    SHADY_REQUIRE(ctx, p->out_dtype == SHADY_F32 || p->out_dtype == cache->dtype, SHADY_ERR_UNSUPPORTED,
                  "decode: out_dtype must be f32 or the cache dtype");
    const uint32_t hd = p->head_dim;
    SHADY_REQUIRE(ctx, hd <= 256, SHADY_ERR_UNSUPPORTED, "decode: head_dim > 256 (the reference shader's limit)");
    const bool f32 = cache->dtype == SHADY_F32;
    if (f32) SHADY_REQUIRE(ctx, hd == 64 || hd == 128 || hd == 256, SHADY_ERR_UNSUPPORTED, "decode: f32 cache needs head_dim 64/128/256");
    else SHADY_REQUIRE(ctx, hd == 128 || hd == 256, SHADY_ERR_UNSUPPORTED, "decode: 16-bit cache needs head_dim 128/256");

    DecodeArgs a{};
    a.q = d_q; a.out = d_out; a.lse = d_lse; a.gate = d_gate;
    a.kv.k_base = (const char *)cache->d_k_base; a.kv.v_base = (const char *)cache->d_v_base;
    a.kv.seq_stride_bytes = cache->seq_stride * dtype_size(cache->dtype);
    a.kv.k_ptrs = cache->d_k_ptrs; a.kv.v_ptrs = cache->d_v_ptrs;
    a.seq_lens = d_seq_lens;
    a.num_seqs = p->num_seqs; a.nkv = p->num_kv_heads; a.nh = p->num_q_heads; a.G = p->heads_per_kv; a.hd = hd;
    a.q_dtype = p->q_dtype; a.out_dtype = p->out_dtype;
    a.scale_log2 = (1.0f / sqrtf((float)hd)) * kLog2e;
    a.num_splits = p->num_splits;

    uint32_t items;
    bool need_reduce;
    if (d_force_partials) {
        SHADY_REQUIRE(ctx, p->num_seqs == 1 && p->num_splits >= 2, SHADY_ERR_BAD_ARG,
                      "decode_partials: needs num_seqs == 1 and num_splits >= 2");
        a.force_partials = 1; a.partials = d_force_partials; a.seq_info = nullptr;
        items = p->num_splits; need_reduce = false;
    } else if (p->num_splits >= 1) {
        items = p->num_seqs * p->num_splits;
        need_reduce = p->num_splits > 1;
    } else {
        SHADY_REQUIRE(ctx, seq_lens_host, SHADY_ERR_BAD_ARG, "decode: num_splits == 0 needs seq_lens_host");
        const DecodePolicy pol = policy_for(cache->dtype, hd);
        const uint32_t gz = f32 ? 1u : (p->heads_per_kv + 15u) / 16u;
        unsigned long long total = 0;
        for (uint32_t i = 0; i < p->num_seqs; ++i) total += seq_lens_host[i];
        const unsigned long long tgt = target_items(ctx, pol);
        unsigned long long chunk = (total * p->num_kv_heads * gz + tgt - 1) / tgt;
        if (chunk < pol.min_chunk) chunk = pol.min_chunk;
        chunk = (chunk + 15) / 16 * 16;
        a.chunk = (uint32_t)chunk;
        items = 0; need_reduce = false;
        for (uint32_t i = 0; i < p->num_seqs; ++i) {
            const uint32_t ns = seq_lens_host[i] == 0 ? 1u : (uint32_t)((seq_lens_host[i] + chunk - 1) / chunk);
            items += ns;
            need_reduce |= ns > 1;
        }
    }
    if (!d_force_partials && (need_reduce || p->num_splits == 0)) {
        const size_t need = decode_workspace_bytes(ctx, p, cache->dtype);
        if (need_reduce) {
            SHADY_REQUIRE(ctx, d_ws && ws_bytes >= need, SHADY_ERR_WORKSPACE, "decode: workspace missing or too small");
        }
        if (d_ws && ws_bytes >= need && need > 0) {
            const size_t info = (((size_t)p->num_seqs * sizeof(uint2)) + 255) / 256 * 256;
            a.seq_info = reinterpret_cast<uint2 *>(d_ws);
            a.partials = reinterpret_cast<float *>(reinterpret_cast<char *>(d_ws) + info);
        }
    }

    int rc;
    if (f32) {
        if (hd == 64) rc = launch32<64, 8>(ctx, a, items);
        else if (hd == 128) rc = launch32<128, 8>(ctx, a, items);
        else rc = launch32<256, 4>(ctx, a, items);
    } else {
        dim3 grid(items, p->num_kv_heads, (p->heads_per_kv + 15) / 16);
        const bool h = cache->dtype == SHADY_F16;
        if (hd == 128) rc = h ? launch16<__half, 128, 4, 3>(ctx, a, grid) : launch16<__nv_bfloat16, 128, 4, 3>(ctx, a, grid);
        else rc = h ? launch16<__half, 256, 4, 3>(ctx, a, grid) : launch16<__nv_bfloat16, 256, 4, 3>(ctx, a, grid);
    }
    if (rc != SHADY_OK) return rc;
    if (need_reduce) {
        ReduceArgs r{};
        r.partials = a.partials; r.out = d_out; r.lse = d_lse; r.gate = d_gate;
        r.seq_info = a.seq_info; r.ns = p->num_splits; r.nh = p->num_q_heads; r.hd = hd;
        r.out_dtype = p->out_dtype; r.skip_single = 1;
        reduce_kernel<<<dim3(p->num_q_heads, p->num_seqs), 128, 0, ctx->stream>>>(r);
        ctx->launches++;
        SHADY_CUDA_OK(ctx, cudaGetLastError());
    }
    return SHADY_OK;
}

int launch_reduce(shady_ctx *ctx, uint32_t hd, uint32_t ns, uint32_t nh, uint64_t split_stride, uint64_t head_stride,
                  const float *d_partials, void *d_out, uint32_t out_dtype, const float *d_gate) {
    SHADY_REQUIRE(ctx, d_partials && d_out && hd && ns && nh, SHADY_ERR_BAD_ARG, "reduce: null or zero argument");
    SHADY_REQUIRE(ctx, out_dtype <= SHADY_BF16, SHADY_ERR_BAD_ARG, "reduce: bad out dtype");
    ReduceArgs r{};
    r.partials = d_partials; r.out = d_out; r.gate = d_gate; r.ns = ns; r.nh = nh; r.hd = hd;
    r.split_stride = split_stride; r.head_stride = head_stride; r.seq_stride = 0; r.out_dtype = out_dtype;
    reduce_kernel<<<dim3(nh, 1), 128, 0, ctx->stream>>>(r);
    ctx->launches++;
    SHADY_CUDA_OK(ctx, cudaGetLastError());
    return SHADY_OK;
}

int launch_sigmoid_mul(shady_ctx *ctx, float *d_x, const float *d_gate, uint32_t n) {
    SHADY_REQUIRE(ctx, d_x && d_gate, SHADY_ERR_BAD_ARG, "sigmoid_mul: null argument");
    if (n == 0) return SHADY_OK;
    sigmoid_mul_kernel<<<(n + 255) / 256, 256, 0, ctx->stream>>>(d_x, d_gate, n);
    ctx->launches++;
    SHADY_CUDA_OK(ctx, cudaGetLastError());
    return SHADY_OK;
}

}  // namespace shady
