// Causal prefill attention on the 5th-generation tensor cores (tcgen05 + TMEM) fed by TMA.
//
// What it computes is the reference's prefill loop (src/inference.rs:93-95): for every token t,
// out[t] = attend(q_t, K[0..=t], V[0..=t]) with the math of gqa_attention_head.wgsl:63-111 — as
// one batched causal flash-attention pass over rows [0,T) of each sequence's cache.
//
// Shape of the kernel (head_dim 128, 16-bit Q/K/V/out, fp32 softmax statistics):
//   * persistent CTAs (one per SM) walk a heaviest-first list of work items; an item = 256 query rows
//     of one (sequence, query head): two 128-row tiles that share every K/V tile; K/V tiles of 128
//     rows arrive through non-multicast 4-D TMA (128-byte swizzle) into a 2-stage ring, completion
//     on mbarriers whose phases run on through the items, so loads and MMAs of the next item start
//     while the softmax of the current one drains;
//   * TMEM (512 columns): S0, S1 (fp32 scores of the two tiles) and O0, O1 (fp32 outputs).
//     P overwrites the first 64 columns of its S as packed 16-bit and is the A operand of the
//     second MMA straight from TMEM;
//   * warp roles: warps 0-3 / 4-7 = softmax of tile 0 / 1 (one thread per row = one TMEM lane),
//     warp 8 = TMA producer, warp 9 = single-thread tcgen05.mma issuer and TMEM owner.  The issuer
//     interleaves the two tiles (S0(j), PV1(j-1), S1(j), PV0(j)) so the tensor pipe works on one
//     tile while the other is in its softmax;
//   * online softmax in the log2 domain with lazy rescaling: O is only rescaled when the running
//     maximum grew by more than 2^8, so the TMEM round trip of O is rare;
//   * causal structure: tile i of the item with row base q0 visits kv tiles 0..(q0+128i)/128 and
//     masks only the last (diagonal) one.
// Every mbarrier wait is bounded: on expiry the kernel records an error code, skips the rest of
// its work, releases TMEM and returns (the host reports SHADY_ERR_TIMEOUT).
#include <cuda.h>

#include <type_traits>

#include "common.cuh"

namespace shady {

constexpr int kPM = 128;                 // query rows per tile
constexpr int kPN = 128;                 // kv rows per tile
constexpr int kPD = 128;                 // head_dim
constexpr int kKvStages = 2;
constexpr uint32_t kSlabBytes = 128 * 64 * 2;   // [128 rows][64 elements] 16-bit, 128B-swizzled
constexpr uint32_t kTileBytes = 2 * kSlabBytes; // 128 x 128 elements
constexpr uint32_t kSmemQ = 0;
constexpr uint32_t kSmemK = kSmemQ + 2 * kTileBytes;
constexpr uint32_t kSmemV = kSmemK + kKvStages * kTileBytes;
constexpr uint32_t kSmemBar = kSmemV + kKvStages * kTileBytes;
constexpr uint32_t kPrefillSmem = kSmemBar + 256 + 1024;  // + barriers + slack for 1024-byte alignment
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kSpinLimit = 1u << 20;  // bounded waits: on the order of a second at worst, then give up
constexpr float kRescaleThreshold = 8.0f;  // log2 units

enum { BAR_QFULL = 0, BAR_KVFULL = 2, BAR_KVEMPTY = 4, BAR_SFULL = 6, BAR_PFULL = 8, BAR_OFULL = 10, BAR_QEMPTY = 12,
       BAR_COUNT = 14 };

struct PrefillArgs {
    void *out;
    int *error;          // device word: 0 = ok, else the code of the wait that expired
    uint32_t B, T, nh, nkv, G;
    uint32_t m_tiles;    // ceil(T / 256)
    float scale_log2;
};

// ---- PTX wrappers ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
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
// Bounded wait.  Returns false (and latches `code` into *error and the CTA's abort word) on expiry or
// when another role has already aborted.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t *abort_word, int *error, int code) {
    for (uint32_t i = 0; i < kSpinLimit; ++i) {
        if (mbar_try(bar, parity)) return true;
        // another role of this CTA, or any CTA of the grid, has already given up: stop waiting
        if ((i & 1023u) == 1023u && (*abort_word || *reinterpret_cast<volatile int *>(error))) return false;
    }
    *abort_word = 1;
    atomicCAS(error, 0, code);
    return false;
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1, int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc]
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem desc]
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
          "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
          "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31]) : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptors (128-byte swizzle, descriptor version 1).
// K-major operand (rows of 64 elements = 128 B, 8-row groups 1024 B apart): LBO unused (1), SBO = 1024 B.
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t saddr) {
    return (uint64_t)((saddr >> 4) & 0x3FFF) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// MN-major operand (V: each kv row holds 64 contiguous head dims = 128 B; 8-row groups 1024 B apart along K;
// the second 64-dim slab kSlabBytes further): LBO = slab stride, SBO = 1024 B.
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t saddr) {
    return (uint64_t)((saddr >> 4) & 0x3FFF) | ((uint64_t)(kSlabBytes >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) |
           (1ull << 46) | (2ull << 61);
}
// Instruction descriptor: fp32 accumulate, 16-bit A/B of format fmt (0 = f16, 1 = bf16), M = N = 128.
__device__ __forceinline__ uint32_t make_idesc(uint32_t fmt, bool b_mn_major) {
    return (1u << 4) | (fmt << 7) | (fmt << 10) | ((b_mn_major ? 1u : 0u) << 16) | ((128u >> 3) << 17) | ((128u >> 4) << 24);
}

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// Instruction-count knobs of the softmax loop (each measured on cfg3; see the profile summary).
#ifndef SHADY_PF_MAX3
#define SHADY_PF_MAX3 1      // three-input max for the row maximum
#endif
#ifndef SHADY_PF_FMA2
#define SHADY_PF_FMA2 1      // packed two-lane fp32 FMA/ADD for s*scale-m and the row sum
#endif
#ifndef SHADY_PF_POLY
#define SHADY_PF_POLY 0      // every n-th pair takes 2^x from an FMA-pipe polynomial instead of MUFU (0 = never)
#endif
__device__ __forceinline__ float max3(float a, float b, float c) {
#if SHADY_PF_MAX3
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
#else
    return fmaxf(a, fmaxf(b, c));
#endif
}
__device__ __forceinline__ unsigned long long pack_f32x2(float lo, float hi) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
// (x0, x1) = (a0, a1) * scale2 + add2 in one instruction
__device__ __forceinline__ void fma_f32x2(float &x0, float &x1, float a0, float a1, unsigned long long scale2, unsigned long long add2) {
    unsigned long long d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(pack_f32x2(a0, a1)), "l"(scale2), "l"(add2));
    asm("mov.b64 {%0, %1}, %2;" : "=f"(x0), "=f"(x1) : "l"(d));
}
__device__ __forceinline__ unsigned long long add_f32x2(unsigned long long a, unsigned long long b) {
    unsigned long long d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
// 2^x on the FMA pipe (Cody-Waite split + cubic), relative error ~6e-4 — below the 16-bit rounding of P.
__device__ __forceinline__ float poly_exp2(float x) {
    x = fmaxf(x, -125.0f);
    const float t = x + 12582912.0f;             // 1.5 * 2^23: the integer part lands in the low mantissa bits
    const float f = x - (t - 12582912.0f);       // fraction in [-0.5, 0.5]
    float p = fmaf(f, 0.0555041f, 0.2402265f);
    p = fmaf(p, f, 0.6931472f);
    p = fmaf(p, f, 1.0f);
    return __int_as_float(__float_as_int(p) + (__float_as_int(t) << 23));
}
template <typename T> __device__ __forceinline__ uint32_t pack16(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pack16<__half>(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&h);
}
template <> __device__ __forceinline__ uint32_t pack16<__nv_bfloat16>(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&h);
}

template <typename T>
__global__ void __launch_bounds__(320, 1)
prefill_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
               const __grid_constant__ CUtensorMap map_v, const PrefillArgs a) {
    extern __shared__ unsigned char smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;  // swizzled tiles need 1024-byte alignment
    unsigned char *smem = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t bar0 = smem_base + kSmemBar;
    auto bar = [&](int i) { return bar0 + 8u * i; };
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem + kSmemBar + 8 * BAR_COUNT);
    volatile uint32_t *abort_word = tmem_slot + 1;

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (*reinterpret_cast<volatile int *>(a.error)) return;   // an earlier CTA's wait expired: do not start
    // Persistent CTAs: work items are (256-row block, sequence, query head), ordered heaviest (latest rows) first.
    // The list is dealt out in rounds of gridDim.x items, left to right in even rounds and right to left in odd
    // ones, so the CTA that got the heaviest item of one round gets the lightest of the next (a plain stride left
    // the first CTAs 6 % above the mean on batch 4 x 32 heads x 4096 rows; the serpentine order leaves 1 %).
    // All roles walk the same list with running barrier phases, so the producer and the MMA issuer run ahead into
    // the next item while the softmax warps finish the current one (pipeline fill/drain overlap instead of adding up).
    struct Item {
        uint32_t b, h, kvh, q0, n[2], nkv;
    };
    const uint32_t bh_count = a.B * a.nh;
    const uint32_t total_items = a.m_tiles * bh_count;
    auto get_item = [&](uint32_t w) {
        Item it;
        const uint32_t m = a.m_tiles - 1 - w / bh_count, bh = w % bh_count;
        it.b = bh / a.nh; it.h = bh % a.nh; it.kvh = it.h / a.G; it.q0 = m * 256;
        it.n[0] = 2 * m + 1;                                   // kv tiles of the two 128-row query tiles
        it.n[1] = (it.q0 + kPM < a.T) ? 2 * m + 2 : 0u;
        it.nkv = it.n[1] ? it.n[1] : it.n[0];
        return it;
    };
    auto item_of_round = [&](uint32_t rnd) {
        return rnd * gridDim.x + ((rnd & 1u) ? gridDim.x - 1u - blockIdx.x : blockIdx.x);
    };
    constexpr uint32_t kFmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;

    if (warp == 8 && lane == 0) {
        mbar_init(bar(BAR_QFULL + 0), 1); mbar_init(bar(BAR_QFULL + 1), 1);
        for (int s = 0; s < kKvStages; ++s) {
            mbar_init(bar(BAR_KVFULL + s), 1); mbar_init(bar(BAR_KVEMPTY + s), 1);
        }
        for (int q = 0; q < 2; ++q) {
            mbar_init(bar(BAR_SFULL + q), 1); mbar_init(bar(BAR_PFULL + q), 128); mbar_init(bar(BAR_OFULL + q), 1);
            mbar_init(bar(BAR_QEMPTY + q), 1);
        }
        *abort_word = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 9) {  // TMEM owner
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void *)tmem_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    // columns: S0 [0,128) S1 [128,256) O0 [256,384) O1 [384,512); P_i = first 64 columns of S_i

    if (warp == 8) {
        // =============================== TMA producer ===============================
        if (lane == 0) {
            bool ok = true;
            uint32_t gk = 0, qc[2] = {0, 0};   // K/V tiles and Q tiles requested so far (barrier phases run through the items)
            for (uint32_t rnd = 0; rnd * gridDim.x < total_items && ok; ++rnd) {
                const uint32_t w = item_of_round(rnd);
                if (w >= total_items) continue;
                const Item it = get_item(w);
                for (int q = 0; q < 2 && ok; ++q) {   // Q of this item, once the last QK of the previous user of the buffer is done
                    if (!it.n[q]) continue;
                    if (qc[q] > 0) ok = mbar_wait(bar(BAR_QEMPTY + q), (qc[q] - 1) & 1, abort_word, a.error, 12);
                    if (!ok) break;
                    ++qc[q];
                    mbar_expect_tx(bar(BAR_QFULL + q), kTileBytes);
                    const uint32_t dst = smem_base + kSmemQ + q * kTileBytes;
                    tma_load_4d(dst, &map_q, bar(BAR_QFULL + q), 0, (int)it.h, (int)(it.q0 + q * kPM), (int)it.b);
                    tma_load_4d(dst + kSlabBytes, &map_q, bar(BAR_QFULL + q), 64, (int)it.h, (int)(it.q0 + q * kPM), (int)it.b);
                }
                for (uint32_t j = 0; j < it.nkv && ok; ++j) {   // K and V tile j travel together: one stage, one barrier
                    const uint32_t gi = gk + j;
                    const uint32_t s = gi % kKvStages, ph = (gi / kKvStages) & 1;
                    if (gi >= kKvStages) ok = mbar_wait(bar(BAR_KVEMPTY + s), ph ^ 1, abort_word, a.error, 1);
                    if (!ok) break;
                    mbar_expect_tx(bar(BAR_KVFULL + s), 2 * kTileBytes);
                    const uint32_t kd = smem_base + kSmemK + s * kTileBytes, vd = smem_base + kSmemV + s * kTileBytes;
                    tma_load_4d(kd, &map_k, bar(BAR_KVFULL + s), 0, (int)it.kvh, (int)(j * kPN), (int)it.b);
                    tma_load_4d(kd + kSlabBytes, &map_k, bar(BAR_KVFULL + s), 64, (int)it.kvh, (int)(j * kPN), (int)it.b);
                    tma_load_4d(vd, &map_v, bar(BAR_KVFULL + s), 0, (int)it.kvh, (int)(j * kPN), (int)it.b);
                    tma_load_4d(vd + kSlabBytes, &map_v, bar(BAR_KVFULL + s), 64, (int)it.kvh, (int)(j * kPN), (int)it.b);
                }
                gk += it.nkv;
            }
        }
    } else if (warp == 9) {
        // =============================== MMA issuer ===============================
        if (lane == 0) {
            const uint32_t idesc_qk = make_idesc(kFmt, false), idesc_pv = make_idesc(kFmt, true);
            bool ok = true;
            auto issue_qk = [&](uint32_t q, uint32_t s) {          // S_q = Q_q * K(stage s)^T
                const uint32_t qa = smem_base + kSmemQ + q * kTileBytes, kb = smem_base + kSmemK + s * kTileBytes;
#pragma unroll
                for (uint32_t ks = 0; ks < kPD / 16; ++ks) {
                    const uint32_t off = (ks >> 2) * kSlabBytes + (ks & 3) * 32;
                    mma_ss(tmem + q * 128, desc_kmajor(qa + off), desc_kmajor(kb + off), idesc_qk, ks > 0);
                }
                tc_commit(bar(BAR_SFULL + q));
            };
            auto issue_pv = [&](uint32_t q, uint32_t s, bool first) {   // O_q (+)= P_q * V(stage s)
                const uint32_t vb = smem_base + kSmemV + s * kTileBytes;
#pragma unroll
                for (uint32_t ks = 0; ks < kPN / 16; ++ks)
                    mma_ts(tmem + 256 + q * 128, tmem + q * 128 + ks * 8, desc_mnmajor(vb + ks * 2048), idesc_pv, !first || (ks > 0));
            };
            uint32_t gk = 0, qc[2] = {0, 0}, tc[2] = {0, 0};   // running counts: K/V tiles, Q loads, score tiles per row tile
            for (uint32_t rnd = 0; rnd * gridDim.x < total_items && ok; ++rnd) {
                const uint32_t w = item_of_round(rnd);
                if (w >= total_items) continue;
                const Item it = get_item(w);
                const uint32_t nkv = it.nkv;
                for (int q = 0; q < 2 && ok; ++q)
                    if (it.n[q]) {
                        ok = mbar_wait(bar(BAR_QFULL + q), qc[q] & 1, abort_word, a.error, 3);
                        ++qc[q];
                    }
                // Per K/V tile the issuer stops three times (K/V landed, P1 stored, P0 stored) and commits three
                // times (S0, S1, stage free): every stop drains the short MMA queue, so there are as few as the
                // dependencies allow.  O needs no barrier of its own inside an item: a commit covers every MMA the
                // thread issued before it, so "S(j) complete" already says "PV(j-1) complete".
                for (uint32_t j = 0; j <= nkv && ok; ++j) {
                    const uint32_t gi = gk + j;
                    const uint32_t s = gi % kKvStages, ph = (gi / kKvStages) & 1;
                    if (j < nkv) {
                        ok = mbar_wait(bar(BAR_KVFULL + s), ph, abort_word, a.error, 4);
                        if (!ok) break;
                        tc_fence_after();
                    }
                    if (j < it.n[0]) {
                        issue_qk(0, s);
                        if (j == it.n[0] - 1) tc_commit(bar(BAR_QEMPTY + 0));   // Q0 of this item is no longer needed
                    }
                    if (j >= 1 && j - 1 < it.n[1]) {
                        const uint32_t sp = (gi - 1) % kKvStages;
                        ok = mbar_wait(bar(BAR_PFULL + 1), (tc[1] + j - 1) & 1, abort_word, a.error, 6);
                        if (!ok) break;
                        tc_fence_after();
                        issue_pv(1, sp, j - 1 == 0);
                        tc_commit(bar(BAR_KVEMPTY + sp));   // PV1 is the last reader of that stage
                        if (j == it.n[1]) tc_commit(bar(BAR_OFULL + 1));   // the item's last PV of tile 1
                    }
                    if (j < it.n[1]) {
                        issue_qk(1, s);
                        if (j == it.n[1] - 1) tc_commit(bar(BAR_QEMPTY + 1));
                    }
                    if (j < it.n[0]) {
                        ok = mbar_wait(bar(BAR_PFULL + 0), (tc[0] + j) & 1, abort_word, a.error, 8);
                        if (!ok) break;
                        tc_fence_after();
                        // (the softmax warps read O of the previous item before they arrive on this P barrier,
                        //  so overwriting O here with the first tile of the next item is safe)
                        issue_pv(0, s, j == 0);
                        if (j >= it.n[1]) tc_commit(bar(BAR_KVEMPTY + s));   // no PV1 on this tile will follow
                        if (j == it.n[0] - 1) tc_commit(bar(BAR_OFULL + 0));
                    }
                }
                gk += nkv; tc[0] += it.n[0]; tc[1] += it.n[1];
            }
        }
    } else {
        // =============================== softmax (one thread per query row) ===============================
        const uint32_t q = warp >> 2;                   // which 128-row tile
        const uint32_t r = tid & 127;                   // row in the tile == TMEM lane
        const uint32_t lane_base = ((warp & 3) * 32) << 16;
        const uint32_t t_s = tmem + lane_base + q * 128, t_o = tmem + lane_base + 256 + q * 128;
        bool ok = true;
        uint32_t c0 = 0, oc = 0;                        // score tiles / items of this row tile finished before the current item (barrier phases)
        for (uint32_t rnd = 0; rnd * gridDim.x < total_items && ok; ++rnd) {
        const uint32_t w = item_of_round(rnd);
        if (w >= total_items) continue;
        const Item item = get_item(w);
        const uint32_t nq = item.n[q], h = item.h, b = item.b;
        const uint32_t row = item.q0 + q * kPM + r;     // global query row == its causal limit
        if (!nq) continue;
        float m_ref = -INFINITY, l_sum = 0.f;
        for (uint32_t j = 0; j < nq && ok; ++j) {
            ok = mbar_wait(bar(BAR_SFULL + q), (c0 + j) & 1, abort_word, a.error, 9);
            if (!ok) break;
            tc_fence_after();
            // one tile of the online softmax; the diagonal tile (the last one) is a second instantiation
            auto tile_body = [&](auto diag_c) {
                constexpr bool diag = decltype(diag_c)::value;   // compile-time: the common path carries no mask code
                // columns of this tile a row may see: all 128, or 0..lim on the diagonal tile
                const int lim = diag ? (int)(row - j * kPN) : 127;
                // ---- pass 1: row maximum (two batches of 64 columns, four independent chains) ----
                float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
    #pragma unroll
                for (int hb = 0; hb < 2; ++hb) {
                    uint32_t va[32], vb[32];
                    tmem_ld32(t_s + hb * 64, va);
                    tmem_ld32(t_s + hb * 64 + 32, vb);
                    tmem_wait_ld();
                    if (!diag) {
    #pragma unroll
                        for (int i = 0; i < 32; i += 4) {
                            mx4[0] = max3(mx4[0], __uint_as_float(va[i]), __uint_as_float(va[i + 1]));
                            mx4[1] = max3(mx4[1], __uint_as_float(va[i + 2]), __uint_as_float(va[i + 3]));
                            mx4[2] = max3(mx4[2], __uint_as_float(vb[i]), __uint_as_float(vb[i + 1]));
                            mx4[3] = max3(mx4[3], __uint_as_float(vb[i + 2]), __uint_as_float(vb[i + 3]));
                        }
                    } else {
    #pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            if (hb * 64 + i <= lim) mx4[i & 1] = fmaxf(mx4[i & 1], __uint_as_float(va[i]));
                            if (hb * 64 + 32 + i <= lim) mx4[2 + (i & 1)] = fmaxf(mx4[2 + (i & 1)], __uint_as_float(vb[i]));
                        }
                    }
                }
                const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * a.scale_log2;  // scale > 0
                // ---- lazy rescale of O and l ----
                float corr = 1.f;
                if (j == 0) {
                    m_ref = mx;
                } else if (mx > m_ref + kRescaleThreshold) {
                    corr = exp2f(m_ref - mx);
                    m_ref = mx;
                }
                if (__any_sync(0xffffffffu, corr != 1.f)) {
                    l_sum *= corr;
    #pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        uint32_t v[32];
                        tmem_ld32(t_o + c * 32, v);
                        tmem_wait_ld();
    #pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * corr);
                        tmem_st32(t_o + c * 32, v);
                    }
                }
                // ---- pass 2: P = exp2(s*scale - m_ref), row sum, pack, store over S; next chunk's load in flight ----
                const float neg_m = -m_ref;
                float ls4[4] = {0.f, 0.f, 0.f, 0.f};
    #if SHADY_PF_FMA2
                const unsigned long long scale2 = pack_f32x2(a.scale_log2, a.scale_log2), negm2 = pack_f32x2(neg_m, neg_m);
                unsigned long long ls2[2] = {0ull, 0ull};
    #endif
                uint32_t vbuf[2][32];
                tmem_ld32(t_s, vbuf[0]);
    #pragma unroll
                for (int c = 0; c < 4; ++c) {
                    tmem_wait_ld();
                    if (c < 3) tmem_ld32(t_s + (c + 1) * 32, vbuf[(c + 1) & 1]);
                    const uint32_t(&v)[32] = vbuf[c & 1];
                    uint32_t pk[16];
    #pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        float x0, x1;
    #if SHADY_PF_FMA2
                        fma_f32x2(x0, x1, __uint_as_float(v[i]), __uint_as_float(v[i + 1]), scale2, negm2);
    #else
                        x0 = fmaf(__uint_as_float(v[i]), a.scale_log2, neg_m);
                        x1 = fmaf(__uint_as_float(v[i + 1]), a.scale_log2, neg_m);
    #endif
                        float p0, p1;
                        if (SHADY_PF_POLY > 0 && ((i >> 1) % (SHADY_PF_POLY > 0 ? SHADY_PF_POLY : 1)) == 0) {
                            p0 = poly_exp2(x0);
                            p1 = poly_exp2(x1);
                        } else {
                            p0 = fast_exp2(x0);
                            p1 = fast_exp2(x1);
                        }
                        if (diag) {
                            if (c * 32 + i > lim) p0 = 0.f;
                            if (c * 32 + i + 1 > lim) p1 = 0.f;
                        }
    #if SHADY_PF_FMA2
                        ls2[(i >> 1) & 1] = add_f32x2(ls2[(i >> 1) & 1], pack_f32x2(p0, p1));
    #else
                        ls4[(i >> 1) & 3] += p0 + p1;
    #endif
                        pk[i >> 1] = pack16<T>(p0, p1);
                    }
                    tmem_st16(t_s + c * 16, pk);
                }
    #if SHADY_PF_FMA2
                {
                    float s0, s1, s2, s3;
                    asm("mov.b64 {%0, %1}, %2;" : "=f"(s0), "=f"(s1) : "l"(ls2[0]));
                    asm("mov.b64 {%0, %1}, %2;" : "=f"(s2), "=f"(s3) : "l"(ls2[1]));
                    ls4[0] = s0 + s1;
                    ls4[1] = s2 + s3;
                }
    #endif
                l_sum += (ls4[0] + ls4[1]) + (ls4[2] + ls4[3]);
                tmem_wait_st();
                tc_fence_before();
                mbar_arrive(bar(BAR_PFULL + q));
            };
            if (j == nq - 1) tile_body(std::true_type{});
            else tile_body(std::false_type{});
        }
        // ---- epilogue: O / l -> global ----
        if (nq && ok) ok = mbar_wait(bar(BAR_OFULL + q), oc & 1, abort_word, a.error, 11);
        if (nq && ok) {
            tc_fence_after();
            const float inv = 1.0f / l_sum;
            T *dst = reinterpret_cast<T *>(a.out) + (((size_t)b * a.T + row) * a.nh + h) * kPD;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t v[32];
                tmem_ld32(t_o + c * 32, v);
                tmem_wait_ld();
                if (row < a.T) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        uint4 w;
                        w.x = pack16<T>(__uint_as_float(v[i]) * inv, __uint_as_float(v[i + 1]) * inv);
                        w.y = pack16<T>(__uint_as_float(v[i + 2]) * inv, __uint_as_float(v[i + 3]) * inv);
                        w.z = pack16<T>(__uint_as_float(v[i + 4]) * inv, __uint_as_float(v[i + 5]) * inv);
                        w.w = pack16<T>(__uint_as_float(v[i + 6]) * inv, __uint_as_float(v[i + 7]) * inv);
                        *reinterpret_cast<uint4 *>(dst + c * 32 + i) = w;
                    }
                }
            }
        }
        c0 += nq;
        ++oc;
        }   // items
    }
    // ---- teardown: everyone arrives, TMEM goes back ----
    tc_fence_before();
    __syncthreads();
    if (warp == 8 && lane == 0 && *abort_word) {
        // an aborted CTA may still have copies in flight: give them a bounded time to land before the
        // shared memory is handed back
        for (int s = 0; s < kKvStages; ++s)
            for (uint32_t i = 0; i < (1u << 16); ++i)
                if (mbar_try(bar(BAR_KVFULL + s), 0)) break;
    }
    __syncthreads();
    if (warp == 9) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
    }
}

// ---- host side -----------------------------------------------------------------------------
// cuTensorMapEncodeTiled is a driver API; it is looked up through the runtime so that the library does not link
// against libcuda (and still loads on a machine without a driver, where only the host-side entry points work).
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

static bool make_map_4d(CUtensorMap *map, CUtensorMapDataType dt, const void *base, uint64_t d0, uint64_t d1, uint64_t d2,
                        uint64_t d3, uint64_t s1, uint64_t s2, uint64_t s3) {
    cuuint64_t dims[4] = {d0, d1, d2, d3};
    cuuint64_t strides[3] = {s1, s2, s3};  // bytes, dims 1..3
    cuuint32_t box[4] = {64, 1, 128, 1};   // 64 elements (128 B, the swizzle span) x 128 rows
    cuuint32_t estr[4] = {1, 1, 1, 1};
    EncodeTiledFn encode = encode_tiled_fn();
    if (!encode) return false;
    return encode(map, dt, 4, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Status word of the bounded waits (0 = ok).  A device-resident global, so nothing is allocated for it.
static __device__ int g_prefill_error_word;
static int *g_prefill_error[64] = {};   // its device address, per device

int launch_prefill(shady_ctx *ctx, const shady_prefill_params *p, const void *d_q, const shady_kv_cache *cache, void *d_out) {
    SHADY_REQUIRE(ctx, p && d_q && cache && d_out, SHADY_ERR_BAD_ARG, "attn_prefill: null argument");
    SHADY_REQUIRE(ctx, p->head_dim == 128, SHADY_ERR_UNSUPPORTED, "attn_prefill: head_dim must be 128");
    SHADY_REQUIRE(ctx, p->dtype == SHADY_BF16 || p->dtype == SHADY_F16, SHADY_ERR_UNSUPPORTED, "attn_prefill: dtype must be bf16 or f16");
    SHADY_REQUIRE(ctx, cache->dtype == p->dtype, SHADY_ERR_UNSUPPORTED, "attn_prefill: cache dtype must equal the Q dtype");
    SHADY_REQUIRE(ctx, p->num_seqs && p->seq_len && p->num_kv_heads && p->num_q_heads % p->num_kv_heads == 0, SHADY_ERR_BAD_ARG,
                  "attn_prefill: bad shape");
    SHADY_REQUIRE(ctx, cache->d_k_base && cache->d_v_base && !cache->d_k_ptrs && !cache->d_page_table, SHADY_ERR_UNSUPPORTED,
                  "attn_prefill: needs base + seq_stride cache addressing (TMA tensor maps), not pointer arrays or pages");
    SHADY_REQUIRE(ctx, p->num_seqs == 1 || cache->seq_stride >= (uint64_t)p->seq_len * p->num_kv_heads * 128, SHADY_ERR_BAD_ARG,
                  "attn_prefill: seq_stride smaller than one sequence");
    SHADY_REQUIRE(ctx, ((uintptr_t)d_q | (uintptr_t)cache->d_k_base | (uintptr_t)cache->d_v_base | (uintptr_t)d_out) % 16 == 0 &&
                           (cache->seq_stride * 2) % 16 == 0,
                  SHADY_ERR_BAD_ARG, "attn_prefill: buffers must be 16-byte aligned");
    SHADY_REQUIRE(ctx, ctx->device >= 0 && ctx->device < 64, SHADY_ERR_UNSUPPORTED, "attn_prefill: device ordinal out of range");
    const uint32_t B = p->num_seqs, T = p->seq_len, nh = p->num_q_heads, nkv = p->num_kv_heads;
    const CUtensorMapDataType dt = p->dtype == SHADY_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    CUtensorMap mq, mk, mv;
    const uint64_t seq_stride_b = (B == 1 ? (uint64_t)T * nkv * 128 : cache->seq_stride) * 2;
    const bool maps_ok = make_map_4d(&mq, dt, d_q, 128, nh, T, B, 128 * 2, (uint64_t)nh * 128 * 2, (uint64_t)T * nh * 128 * 2) &&
                         make_map_4d(&mk, dt, cache->d_k_base, 128, nkv, T, B, 128 * 2, (uint64_t)nkv * 128 * 2, seq_stride_b) &&
                         make_map_4d(&mv, dt, cache->d_v_base, 128, nkv, T, B, 128 * 2, (uint64_t)nkv * 128 * 2, seq_stride_b);
    SHADY_REQUIRE(ctx, maps_ok, SHADY_ERR_CUDA, "attn_prefill: cuTensorMapEncodeTiled failed");
    if (!g_prefill_error[ctx->device]) {
        int *w = nullptr;
        SHADY_CUDA_OK(ctx, cudaGetSymbolAddress(reinterpret_cast<void **>(&w), g_prefill_error_word));
        SHADY_CUDA_OK(ctx, cudaMemsetAsync(w, 0, sizeof(int), ctx->stream));
        g_prefill_error[ctx->device] = w;
    }
    PrefillArgs a{};
    a.out = d_out; a.error = g_prefill_error[ctx->device];
    a.B = B; a.T = T; a.nh = nh; a.nkv = nkv; a.G = nh / nkv;
    a.m_tiles = (T + 255) / 256;
    a.scale_log2 = (1.0f / sqrtf(128.0f)) * 1.4426950408889634f;
    const unsigned long long total_items = (unsigned long long)a.m_tiles * B * nh;
    SHADY_REQUIRE(ctx, total_items <= 0x7fffffffull, SHADY_ERR_UNSUPPORTED, "attn_prefill: too many tiles for one launch");
    const unsigned long long blocks = total_items < (unsigned long long)ctx->num_sms ? total_items : (unsigned long long)ctx->num_sms;   // persistent: one CTA per SM
    SHADY_REQUIRE(ctx, blocks <= 0x7fffffffull, SHADY_ERR_UNSUPPORTED, "attn_prefill: too many tiles for one launch");
    static thread_local int configured_dev = -1;
    if (configured_dev != ctx->device) {
        SHADY_CUDA_OK(ctx, cudaFuncSetAttribute(prefill_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPrefillSmem));
        SHADY_CUDA_OK(ctx, cudaFuncSetAttribute(prefill_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPrefillSmem));
        configured_dev = ctx->device;
    }
    if (p->dtype == SHADY_BF16) {
        prefill_kernel<__nv_bfloat16><<<(unsigned)blocks, 320, kPrefillSmem, ctx->stream>>>(mq, mk, mv, a);
    } else {
        prefill_kernel<__half><<<(unsigned)blocks, 320, kPrefillSmem, ctx->stream>>>(mq, mk, mv, a);
    }
    ctx->launches++;
    SHADY_CUDA_OK(ctx, cudaGetLastError());
    return SHADY_OK;
}

// Reads (and clears) the bounded-wait status of the prefill kernel; blocks until the stream is idle.
int prefill_status(shady_ctx *ctx, int *code) {
    *code = 0;
    if (ctx->device < 0 || ctx->device >= 64 || !g_prefill_error[ctx->device]) return SHADY_OK;
    SHADY_CUDA_OK(ctx, cudaMemcpyAsync(code, g_prefill_error[ctx->device], sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
    SHADY_CUDA_OK(ctx, cudaStreamSynchronize(ctx->stream));
    if (*code) {
        SHADY_CUDA_OK(ctx, cudaMemsetAsync(g_prefill_error[ctx->device], 0, sizeof(int), ctx->stream));
        return fail(ctx, SHADY_ERR_TIMEOUT, "attn_prefill: a device-side wait expired (code " + std::to_string(*code) + ")");
    }
    return SHADY_OK;
}

}  // namespace shady
