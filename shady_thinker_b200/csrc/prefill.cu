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
//
// FUSED variant (shady_attn_prefill_append): Q comes straight from the projection (q_proj_full, Q and gate halves
// per head) instead of from a buffer a separate append pass has normed and rotated.  The raw Q tile lands by TMA in
// one of three rotating shared-memory buffers; four extra warps apply RMSNorm(1+w) and RoPE to it in place
// (fused_split_qknorm_kvstore.wgsl:126-166; cos/sin of (position, pair) from a table the K/V pass of the same step
// wrote), make it visible to the tensor core's proxy and only then signal the MMA issuer; the epilogue multiplies
// by sigmoid(gate) (sigmoid_mul.wgsl).  The 2 x 134 MB round trip of the rotated Q of a 16k-token step never
// happens, and with three buffers a tile of the next item is transformed while the current item still computes.
#include <cuda.h>

#include <string.h>

#include <type_traits>
#include <vector>

#include "common.cuh"

namespace shady {

constexpr int kPM = 128;                 // query rows per tile
constexpr int kPN = 128;                 // kv rows per tile
constexpr int kPD = 128;                 // head_dim
constexpr int kKvStages = 2;
constexpr uint32_t kSlabBytes = 128 * 64 * 2;   // [128 rows][64 elements] 16-bit, 128B-swizzled
constexpr uint32_t kTileBytes = 2 * kSlabBytes; // 128 x 128 elements
// shared memory: [Q buffers: nqb tiles][K stages][V stages][barriers]; nqb = 2 (tile q of an item lives in buffer
// q) or, fused, 3 rotating buffers
constexpr uint32_t kSmemQ = 0;
constexpr uint32_t smem_k_off(uint32_t nqb) { return kSmemQ + nqb * kTileBytes; }
constexpr uint32_t smem_v_off(uint32_t nqb) { return smem_k_off(nqb) + kKvStages * kTileBytes; }
constexpr uint32_t smem_bar_off(uint32_t nqb) { return smem_v_off(nqb) + kKvStages * kTileBytes; }
constexpr uint32_t prefill_smem(uint32_t nqb) { return smem_bar_off(nqb) + 256 + 1024; }  // + barriers + slack for 1024-byte alignment
static_assert(prefill_smem(3) <= 232448, "three Q buffers must fit in 227 KB");
constexpr uint32_t kTmemCols = 512;
constexpr float kRescaleThreshold = 8.0f;  // log2 units

enum { BAR_QFULL = 0, BAR_QEMPTY = 3, BAR_QRAW = 6, BAR_KVFULL = 9, BAR_KVEMPTY = 11, BAR_SFULL = 13, BAR_PFULL = 15,
       BAR_OFULL = 17, BAR_COUNT = 19 };
// fused: four more warps (a warpgroup of their own) norm and rotate the raw Q tiles.  16 warps leave 128 registers
// per thread at launch, too few for the softmax warps, so the warpgroups trade registers once the roles are taken:
// the two softmax warpgroups grow to kRegsSoftmax, the producer/issuer warpgroup and the Q warpgroup shrink to
// kRegsOther (2 x 128 x 176 + 2 x 128 x 80 = 65,536).
constexpr uint32_t kQWarps = 4;
constexpr uint32_t kFusedThreads = 512;
constexpr uint32_t kRegsSoftmax = 176, kRegsOther = 80;

// Batches that are not B equal sequences in one base + stride allocation.  The host lists the row blocks of all
// sequences heaviest first; Q and the output are then packed token-major (sequence after sequence), and K/V rows
// come through one tensor map per sequence (extent T_i, so rows past the sequence read as zero) or, for paged
// caches, through the pool's map and the page table.
struct RaggedRef {
    const uint4 *items;           // [entries] {sequence, row block, T of the sequence, first packed token}; NULL = uniform batch
    const CUtensorMap *kv_maps;   // [2 * num_seqs] K and V map of every sequence, in global memory; NULL = map_k / map_v cover the batch (or the pool)
    const uint32_t *page_table;   // paged caches: [num_seqs][max_pages] page of every page_rows rows
    uint32_t entries, max_pages, page_rows, box_rows, oob_page;
};

struct PrefillArgs {
    void *out;
    RaggedRef rg;
    StatusRef status;    // where a wait that ran out is reported (code 1..12 = which barrier)
    uint32_t wait_mbar;  // poll limit of every mbarrier wait
    uint32_t B, T, nh, nkv, G;
    uint32_t m_tiles;    // ceil(T / 256)
    float scale_log2;
    // fused variant: the raw projection rows [B][T][nh][qrow] (Q half first, then the gate half when has_gate)
    const void *q_src;
    const float2 *cs_table;   // [T][64] (cos, sin) of (position, rotary pair); (1, 0) beyond the rotary dims
    const uint16_t *norm_w;   // bf16 bits of the Q RMSNorm weights [128], or NULL
    uint32_t qrow, has_gate;
    float eps;
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
struct WaitCtx {
    volatile uint32_t *abort_word;   // shared memory: a role of this CTA gave up
    StatusRef status;
    uint32_t limit;
};
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const WaitCtx &w, int code) {
    for (uint32_t i = 0; i < w.limit; ++i) {
        if (mbar_try(bar, parity)) return true;
        // another role of this CTA, or any CTA of the grid, has already given up: stop waiting
        if ((i & 1023u) == 1023u && (*w.abort_word || gave_up(w.status))) return false;
    }
    *w.abort_word = 1;
    report_timeout(w.status, code);
    return false;
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1, int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
// a tensor map that lives in global memory (written by a copy that the stream ordered before this kernel): the
// CTA's first use of it goes through this fence
__device__ __forceinline__ void tensormap_acquire(const CUtensorMap *map) {
    asm volatile("fence.proxy.tensormap::generic.acquire.gpu [%0], 128;" ::"l"(map) : "memory");
}
// One K/V tile (ROWS rows x SLABS slabs of 64 elements) of sequence b, kv head kvh, first row row0, into dst (slab
// stride slab_bytes), completing on bar.  Uniform batches: coordinate 3 = sequence.  Per-sequence maps: coordinate 3 = 0.
// Paged caches: the tile is fetched in boxes of rg.box_rows rows (a page, or the whole tile when a page holds
// several), each at (row in page, page); a box that starts past the sequence takes an out-of-range page and so
// reads as zero, which also keeps the lookup inside the table entries the sequence owns.
template <int ROWS, int SLABS>
__device__ __forceinline__ void tma_load_kv_tile(uint32_t dst, uint32_t slab_bytes, const CUtensorMap *map, uint32_t bar, const RaggedRef &rg,
                                                 uint32_t b, uint32_t kvh, uint32_t row0, uint32_t T, bool per_seq) {
    if (rg.page_table) {
        for (uint32_t r = 0; r < (uint32_t)ROWS; r += rg.box_rows) {
            const uint32_t row = row0 + r;
            const uint32_t page = row < T ? __ldg(rg.page_table + (size_t)b * rg.max_pages + row / rg.page_rows) : rg.oob_page;
#pragma unroll
            for (int c = 0; c < SLABS; ++c)
                tma_load_4d(dst + c * slab_bytes + r * 128u, map, bar, 64 * c, (int)kvh, (int)(row % rg.page_rows), (int)page);
        }
    } else {
#pragma unroll
        for (int c = 0; c < SLABS; ++c) tma_load_4d(dst + c * slab_bytes, map, bar, 64 * c, (int)kvh, (int)row0, per_seq ? 0 : (int)b);
    }
}
// one 8-byte shared-memory word read / written as a unit (the {maximum, tile number} pair two warpgroups hand over)
__device__ __forceinline__ uint2 lds_pair(uint32_t saddr) {
    uint2 v;
    asm volatile("ld.volatile.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(saddr) : "memory");
    return v;
}
__device__ __forceinline__ void sts_pair(uint32_t saddr, uint32_t x, uint32_t y) {
    asm volatile("st.volatile.shared.v2.u32 [%0], {%1, %2};" ::"r"(saddr), "r"(x), "r"(y) : "memory");
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
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
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
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t saddr, uint32_t slab_bytes = kSlabBytes) {
    return (uint64_t)((saddr >> 4) & 0x3FFF) | ((uint64_t)(slab_bytes >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) |
           (1ull << 46) | (2ull << 61);
}
// Instruction descriptor: fp32 accumulate, 16-bit A/B of format fmt (0 = f16, 1 = bf16), M = 128, N = n.
__device__ __forceinline__ uint32_t make_idesc(uint32_t fmt, bool b_mn_major, uint32_t n = 128) {
    return (1u << 4) | (fmt << 7) | (fmt << 10) | ((b_mn_major ? 1u : 0u) << 16) | ((n >> 3) << 17) | ((128u >> 4) << 24);
}

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// Instruction savers of the softmax loop: a three-input max for the row maximum, packed two-lane fp32 FMA/ADD for
// s * scale - m and the row sum.  (2^x from an FMA-pipe polynomial for a share of the elements was measured too:
// slower, the issue slots it takes cost more than the exponential unit it relieves.)
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
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
template <typename T> __device__ __forceinline__ uint32_t pack16(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pack16<__half>(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&h);
}
template <> __device__ __forceinline__ uint32_t pack16<__nv_bfloat16>(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&h);
}

template <typename T, bool FUSED>
__global__ void __launch_bounds__(FUSED ? kFusedThreads : 320, 1)
prefill_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
               const __grid_constant__ CUtensorMap map_v, const PrefillArgs a) {
    constexpr uint32_t NQB = FUSED ? 3u : 2u;   // Q buffers; tile number tq of this CTA lives in buffer tq % NQB
    constexpr uint32_t kSmemK = smem_k_off(NQB), kSmemV = smem_v_off(NQB), kSmemBar = smem_bar_off(NQB);
    extern __shared__ unsigned char smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;  // swizzled tiles need 1024-byte alignment
    unsigned char *smem = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t bar0 = smem_base + kSmemBar;
    auto bar = [&](int i) { return bar0 + 8u * i; };
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem + kSmemBar + 8 * BAR_COUNT);
    volatile uint32_t *abort_word = tmem_slot + 1;

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (gave_up(a.status)) return;   // an earlier wait of this context expired: do not start
    const WaitCtx wc{abort_word, a.status, a.wait_mbar};
    // Persistent CTAs: work items are (256-row block, sequence, query head), ordered heaviest (latest rows) first.
    // The list is dealt out in rounds of gridDim.x items, left to right in even rounds and right to left in odd
    // ones, so the CTA that got the heaviest item of one round gets the lightest of the next (a plain stride left
    // the first CTAs 6 % above the mean on batch 4 x 32 heads x 4096 rows; the serpentine order leaves 1 %).
    // All roles walk the same list with running barrier phases, so the producer and the MMA issuer run ahead into
    // the next item while the softmax warps finish the current one (pipeline fill/drain overlap instead of adding up).
    struct Item {
        uint32_t b, h, kvh, q0, n[2], nkv;
        uint32_t len, tok0;     // rows of the sequence; packed row of its first token (Q, output, gate)
        uint32_t qrow, qseq;    // TMA coordinates 2 and 3 of the item's first Q row
    };
    const uint32_t bh_count = a.B * a.nh;
    const uint32_t total_items = a.rg.items ? a.rg.entries * a.nh : a.m_tiles * bh_count;
    auto get_item = [&](uint32_t w) {
        Item it;
        uint32_t m;
        if (a.rg.items) {   // listed row blocks (heaviest first), the heads of a block side by side
            const uint4 e = __ldg(a.rg.items + w / a.nh);
            it.b = e.x; m = e.y; it.len = e.z; it.tok0 = e.w; it.h = w % a.nh;
            it.q0 = m * 256; it.qrow = it.tok0 + it.q0; it.qseq = 0;
        } else {
            const uint32_t bh = w % bh_count;
            m = a.m_tiles - 1 - w / bh_count;
            it.b = bh / a.nh; it.h = bh % a.nh; it.len = a.T; it.tok0 = it.b * a.T;
            it.q0 = m * 256; it.qrow = it.q0; it.qseq = it.b;
        }
        it.kvh = it.h / a.G;
        it.n[0] = 2 * m + 1;                                   // kv tiles of the two 128-row query tiles
        it.n[1] = (it.q0 + kPM < it.len) ? 2 * m + 2 : 0u;
        it.nkv = it.n[1] ? it.n[1] : it.n[0];
        return it;
    };
    auto item_of_round = [&](uint32_t rnd) {
        return rnd * gridDim.x + ((rnd & 1u) ? gridDim.x - 1u - blockIdx.x : blockIdx.x);
    };
    constexpr uint32_t kFmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;

    if (warp == 8 && lane == 0) {
        for (uint32_t b = 0; b < NQB; ++b) {
            // fused: every thread of the Q warps arrives once its part of the tile is transformed and fenced
            mbar_init(bar(BAR_QFULL + b), FUSED ? 32 * kQWarps : 1); mbar_init(bar(BAR_QEMPTY + b), 1);
            mbar_init(bar(BAR_QRAW + b), 1);
        }
        for (int s = 0; s < kKvStages; ++s) {
            mbar_init(bar(BAR_KVFULL + s), 1); mbar_init(bar(BAR_KVEMPTY + s), 1);
        }
        for (int q = 0; q < 2; ++q) {
            mbar_init(bar(BAR_SFULL + q), 1); mbar_init(bar(BAR_PFULL + q), 128); mbar_init(bar(BAR_OFULL + q), 1);
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

    if (warp >= 8) {
    // the producer/issuer warpgroup and the Q warpgroup give registers up, the softmax warpgroups (below) take them
    if constexpr (FUSED) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsOther));
    if (warp == 8) {
        // =============================== TMA producer ===============================
        if (lane == 0) {
            bool ok = true;
            uint32_t gk = 0, tq = 0;   // K/V tiles and Q tiles requested so far (barrier phases run through the items)
            for (uint32_t rnd = 0; rnd * gridDim.x < total_items && ok; ++rnd) {
                const uint32_t w = item_of_round(rnd);
                if (w >= total_items) continue;
                const Item it = get_item(w);
                for (int q = 0; q < 2 && ok; ++q) {   // Q of this item, once the last QK of the previous user of the buffer is done
                    if (!it.n[q]) continue;
                    const uint32_t buf = tq % NQB, use = tq / NQB;
                    if (use > 0) ok = mbar_wait(bar(BAR_QEMPTY + buf), (use - 1) & 1, wc, 12);
                    if (!ok) break;
                    ++tq;
                    // fused: the tile arrives raw (the Q half of the projection rows) and the Q warps pass it on
                    const uint32_t landed = bar((FUSED ? BAR_QRAW : BAR_QFULL) + buf);
                    mbar_expect_tx(landed, kTileBytes);
                    const uint32_t dst = smem_base + kSmemQ + buf * kTileBytes;
                    tma_load_4d(dst, &map_q, landed, 0, (int)it.h, (int)(it.qrow + q * kPM), (int)it.qseq);
                    tma_load_4d(dst + kSlabBytes, &map_q, landed, 64, (int)it.h, (int)(it.qrow + q * kPM), (int)it.qseq);
                }
                const CUtensorMap *mk = &map_k, *mv = &map_v;
                if (a.rg.kv_maps) {
                    mk = a.rg.kv_maps + 2 * it.b; mv = mk + 1;
                    tensormap_acquire(mk); tensormap_acquire(mv);
                }
                for (uint32_t j = 0; j < it.nkv && ok; ++j) {   // K and V tile j travel together: one stage, one barrier
                    const uint32_t gi = gk + j;
                    const uint32_t s = gi % kKvStages, ph = (gi / kKvStages) & 1;
                    if (gi >= kKvStages) ok = mbar_wait(bar(BAR_KVEMPTY + s), ph ^ 1, wc, 1);
                    if (!ok) break;
                    mbar_expect_tx(bar(BAR_KVFULL + s), 2 * kTileBytes);
                    const uint32_t kd = smem_base + kSmemK + s * kTileBytes, vd = smem_base + kSmemV + s * kTileBytes;
                    tma_load_kv_tile<kPN, 2>(kd, kSlabBytes, mk, bar(BAR_KVFULL + s), a.rg, it.b, it.kvh, j * kPN, it.len, a.rg.kv_maps != nullptr);
                    tma_load_kv_tile<kPN, 2>(vd, kSlabBytes, mv, bar(BAR_KVFULL + s), a.rg, it.b, it.kvh, j * kPN, it.len, a.rg.kv_maps != nullptr);
                }
                gk += it.nkv;
            }
        }
    } else if (warp == 9) {
        // =============================== MMA issuer ===============================
        if (lane == 0) {
            const uint32_t idesc_qk = make_idesc(kFmt, false), idesc_pv = make_idesc(kFmt, true);
            bool ok = true;
            uint32_t qbuf[2] = {0, 0};                             // Q buffers of the current item's two tiles
            auto issue_qk = [&](uint32_t q, uint32_t s) {          // S_q = Q_q * K(stage s)^T
                const uint32_t qa = smem_base + kSmemQ + qbuf[q] * kTileBytes, kb = smem_base + kSmemK + s * kTileBytes;
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
            uint32_t gk = 0, tq = 0, tc[2] = {0, 0};   // running counts: K/V tiles, Q tiles, score tiles per row tile
            for (uint32_t rnd = 0; rnd * gridDim.x < total_items && ok; ++rnd) {
                const uint32_t w = item_of_round(rnd);
                if (w >= total_items) continue;
                const Item it = get_item(w);
                const uint32_t nkv = it.nkv;
                uint32_t qpar[2] = {0, 0};
                for (int q = 0; q < 2; ++q)
                    if (it.n[q]) {
                        qbuf[q] = tq % NQB; qpar[q] = (tq / NQB) & 1;
                        ++tq;
                    }
                // tile 0 must be there before anything is issued; tile 1 only ahead of its own first S (fused: it may
                // still be under the Q warps' hands while S0 of the first K/V tile is computed)
                ok = mbar_wait(bar(BAR_QFULL + qbuf[0]), qpar[0], wc, 3);
                // Per K/V tile the issuer stops three times (K/V landed, P1 stored, P0 stored) and commits three
                // times (S0, S1, stage free): every stop drains the short MMA queue, so there are as few as the
                // dependencies allow.  O needs no barrier of its own inside an item: a commit covers every MMA the
                // thread issued before it, so "S(j) complete" already says "PV(j-1) complete".
                for (uint32_t j = 0; j <= nkv && ok; ++j) {
                    const uint32_t gi = gk + j;
                    const uint32_t s = gi % kKvStages, ph = (gi / kKvStages) & 1;
                    if (j < nkv) {
                        ok = mbar_wait(bar(BAR_KVFULL + s), ph, wc, 4);
                        if (!ok) break;
                        tc_fence_after();
                    }
                    if (j < it.n[0]) {
                        issue_qk(0, s);
                        if (j == it.n[0] - 1) tc_commit(bar(BAR_QEMPTY + qbuf[0]));   // Q0 of this item is no longer needed
                    }
                    if (j >= 1 && j - 1 < it.n[1]) {
                        const uint32_t sp = (gi - 1) % kKvStages;
                        ok = mbar_wait(bar(BAR_PFULL + 1), (tc[1] + j - 1) & 1, wc, 6);
                        if (!ok) break;
                        tc_fence_after();
                        issue_pv(1, sp, j - 1 == 0);
                        tc_commit(bar(BAR_KVEMPTY + sp));   // PV1 is the last reader of that stage
                        if (j == it.n[1]) tc_commit(bar(BAR_OFULL + 1));   // the item's last PV of tile 1
                    }
                    if (j < it.n[1]) {
                        if (j == 0) {
                            ok = mbar_wait(bar(BAR_QFULL + qbuf[1]), qpar[1], wc, 2);
                            if (!ok) break;
                            tc_fence_after();
                        }
                        issue_qk(1, s);
                        if (j == it.n[1] - 1) tc_commit(bar(BAR_QEMPTY + qbuf[1]));
                    }
                    if (j < it.n[0]) {
                        ok = mbar_wait(bar(BAR_PFULL + 0), (tc[0] + j) & 1, wc, 8);
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
    } else if (FUSED && warp >= 10 && warp < 12) {
        // (the producer/issuer warpgroup's two spare warps: nothing to do until the teardown barrier)
    } else if (FUSED && warp >= 12) {
        // =============================== Q warps (fused): RMSNorm(1+w) + RoPE of the raw tile, in place ===============================
        // 16 lanes share a row (8 elements = 16 bytes each), two rows per warp instruction, eight per pass of the four
        // warps.  A lane always owns the same 8 head dims, hence the same four rotary pairs and norm weights.
        constexpr uint32_t kRowsPerPass = 2 * kQWarps, kPasses = kPM / kRowsPerPass;
        const uint32_t qt = tid - 384;                      // 0..127
        const uint32_t c = qt & 15, rsub = qt >> 4;         // 16-byte chunk of the row, row within a pass
        float wq[8];
        if (a.norm_w) {
#pragma unroll
            for (int e = 0; e < 8; ++e) wq[e] = 1.0f + __uint_as_float(((uint32_t)a.norm_w[c * 8 + e]) << 16);
        }
        bool ok = true;
        uint32_t tq = 0;
        constexpr int kBatch = 2;                           // rows a thread has in flight (the register budget is 80)
        for (uint32_t rnd = 0; rnd * gridDim.x < total_items && ok; ++rnd) {
            const uint32_t w = item_of_round(rnd);
            if (w >= total_items) continue;
            const Item it = get_item(w);
            for (int q = 0; q < 2 && ok; ++q) {
                if (!it.n[q]) continue;
                const uint32_t buf = tq % NQB, par = (tq / NQB) & 1;
                ++tq;
                const uint32_t row_base = it.q0 + q * kPM;   // position of the tile's first row (prefill starts at position 0)
                // the table rows of the first batch are requested before the wait: they do not depend on the tile
                float4 tab[kBatch][2];
                auto load_tab = [&](uint32_t pass0) {
#pragma unroll
                    for (int u = 0; u < kBatch; ++u) {
                        const uint32_t pos = min(row_base + (pass0 + u) * kRowsPerPass + rsub, it.len - 1);
                        const float4 *tp = reinterpret_cast<const float4 *>(a.cs_table + (size_t)pos * 64 + c * 4);
                        tab[u][0] = __ldg(tp);
                        tab[u][1] = __ldg(tp + 1);
                    }
                };
                load_tab(0);
                ok = mbar_wait(bar(BAR_QRAW + buf), par, wc, 7);
                if (!ok) break;
                unsigned char *tile = smem + kSmemQ + buf * kTileBytes;
                for (uint32_t pass0 = 0; pass0 < kPasses; pass0 += kBatch) {
                    uint4 raw[kBatch];
                    uint32_t off[kBatch];
#pragma unroll
                    for (int u = 0; u < kBatch; ++u) {
                        const uint32_t r = (pass0 + u) * kRowsPerPass + rsub;
                        off[u] = (c >> 3) * kSlabBytes + r * 128 + (((c & 7) ^ (r & 7)) << 4);
                        raw[u] = *reinterpret_cast<const uint4 *>(tile + off[u]);
                    }
                    float4 cur[kBatch][2];
#pragma unroll
                    for (int u = 0; u < kBatch; ++u) { cur[u][0] = tab[u][0]; cur[u][1] = tab[u][1]; }
                    if (pass0 + kBatch < kPasses) load_tab(pass0 + kBatch);   // next batch's table rows travel under this batch's math
#pragma unroll
                    for (int u = 0; u < kBatch; ++u) {
                        float v[8];
                        const T *e = reinterpret_cast<const T *>(&raw[u]);
#pragma unroll
                        for (int k = 0; k < 8; ++k) v[k] = to_f32<T>(e[k]);
                        if (a.norm_w) {
                            float ssq = 0.f;
#pragma unroll
                            for (int k = 0; k < 8; ++k) ssq += v[k] * v[k];
#pragma unroll
                            for (int o = 8; o > 0; o >>= 1) ssq += __shfl_xor_sync(0xffffffffu, ssq, o);
                            const float rms = 1.0f / sqrtf(ssq / (float)kPD + a.eps);
#pragma unroll
                            for (int k = 0; k < 8; ++k) v[k] = v[k] * rms * wq[k];
                        }
                        const float cs[4] = {cur[u][0].x, cur[u][0].z, cur[u][1].x, cur[u][1].z};
                        const float sn[4] = {cur[u][0].y, cur[u][0].w, cur[u][1].y, cur[u][1].w};
                        uint4 o4;
                        uint32_t *ow = reinterpret_cast<uint32_t *>(&o4);
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const float x = v[2 * k], y = v[2 * k + 1];
                            ow[k] = pack16<T>(x * cs[k] - y * sn[k], y * cs[k] + x * sn[k]);
                        }
                        *reinterpret_cast<uint4 *>(tile + off[u]) = o4;
                    }
                }
                // generic-proxy writes to shared memory -> visible to the tensor core's (async) proxy, then signal
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                mbar_arrive(bar(BAR_QFULL + buf));
            }
        }
    }
    } else {
        if constexpr (FUSED) asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsSoftmax));   // the two softmax warpgroups
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
        const uint32_t nq = item.n[q], h = item.h;
        const uint32_t row = item.q0 + q * kPM + r;     // query row within its sequence == its causal limit
        if (!nq) continue;
        float m_ref = -INFINITY, l_sum = 0.f;
        for (uint32_t j = 0; j < nq && ok; ++j) {
            ok = mbar_wait(bar(BAR_SFULL + q), (c0 + j) & 1, wc, 9);
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
                const unsigned long long scale2 = pack_f32x2(a.scale_log2, a.scale_log2), negm2 = pack_f32x2(neg_m, neg_m);
                unsigned long long ls2[2] = {0ull, 0ull};
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
                        fma_f32x2(x0, x1, __uint_as_float(v[i]), __uint_as_float(v[i + 1]), scale2, negm2);
                        float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
                        if (diag) {
                            if (c * 32 + i > lim) p0 = 0.f;
                            if (c * 32 + i + 1 > lim) p1 = 0.f;
                        }
                        ls2[(i >> 1) & 1] = add_f32x2(ls2[(i >> 1) & 1], pack_f32x2(p0, p1));
                        pk[i >> 1] = pack16<T>(p0, p1);
                    }
                    tmem_st16(t_s + c * 16, pk);
                }
                float s0, s1, s2, s3;
                asm("mov.b64 {%0, %1}, %2;" : "=f"(s0), "=f"(s1) : "l"(ls2[0]));
                asm("mov.b64 {%0, %1}, %2;" : "=f"(s2), "=f"(s3) : "l"(ls2[1]));
                l_sum += (s0 + s1) + (s2 + s3);
                tmem_wait_st();
                tc_fence_before();
                mbar_arrive(bar(BAR_PFULL + q));
            };
            if (j == nq - 1) tile_body(std::true_type{});
            else tile_body(std::false_type{});
        }
        // ---- epilogue: O / l -> global ----
        if (nq && ok) ok = mbar_wait(bar(BAR_OFULL + q), oc & 1, wc, 11);
        if (nq && ok) {
            tc_fence_after();
            const float inv = 1.0f / l_sum;
            T *dst = reinterpret_cast<T *>(a.out) + (((size_t)item.tok0 + row) * a.nh + h) * kPD;
            // fused: the gate half of the row's projection (fused_split_qknorm_kvstore.wgsl:122-135) scales the output
            const T *gate = (FUSED && a.has_gate && row < item.len)
                                ? reinterpret_cast<const T *>(a.q_src) + (((size_t)item.tok0 + row) * a.nh + h) * a.qrow + kPD : nullptr;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t v[32];
                tmem_ld32(t_o + c * 32, v);
                tmem_wait_ld();
                if (FUSED && gate) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        const uint4 g4 = *reinterpret_cast<const uint4 *>(gate + c * 32 + i);
                        const T *ge = reinterpret_cast<const T *>(&g4);
#pragma unroll
                        for (int k = 0; k < 8; ++k)
                            v[i + k] = __float_as_uint(__uint_as_float(v[i + k]) * sigmoidf_ref(to_f32<T>(ge[k])));
                    }
                }
                if (row < item.len) {
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


// =====================================================================================================
// Row-tile kernel (head_dim 256, the gated-attention layer shape): one 128-row Q tile per item, K/V tiles of 64 rows.
//
// S + O of two 128-row tiles would need 768 TMEM columns at this head_dim, so an item is ONE row tile and the depth of
// the pipeline comes from the score buffers instead: O takes 256 TMEM columns, the other 256 hold the scores of four
// consecutive K/V tiles (64 columns each).  P overwrites the first half of its own S buffer and is the A operand of
// the PV MMA straight from TMEM, so a buffer goes through S -> softmax -> PV before the next S may land in it; with
// four buffers that chain (about 4,000 clocks) is no longer what the tile rate waits for.
//   * Shared memory: Q (one buffer of 64 KB, TMA), three K tiles and two V tiles of 32 KB in rings of their own — a K
//     slot is free as soon as its S is computed, a V slot only after its PV, so K runs ahead of V.
//   * Three MMA-issuing threads, because one is not enough at this tile shape: a satisfied barrier wait costs a thread
//     ~250 clocks, a commit ~80, an MMA issue that the pipe back-pressures 64 (the N = 64 score MMAs run at half
//     rate), and the waits, commits and issues of one K/V tile add up to about twice the time the tensor pipe needs to
//     execute its MMAs.  Two threads issue the score MMAs (tiles of even / odd running number), one the PV MMAs; each
//     commits its own.  MMAs of different threads are not ordered among themselves, so what must be ordered goes
//     through barriers: S(t) waits for PV(t - 4) (its buffer), the first PV of an item for the epilogue's reads of O.
//   * Softmax: one warpgroup, one thread per row, the 64 scores of a tile in registers (one pass over TMEM).
//   * Four epilogue warps drain O (x 1/l, x sigmoid(gate)) while the softmax warps are already in the next item; the
//     row sum travels through a shared-memory word with the item's number in it.
// Warps 0-3 softmax, 4 TMA producer, 5 score issuer (even tiles; TMEM owner), 6 PV issuer, 7 score issuer (odd tiles),
// 8-11 epilogue.
// The same kernel was also built for head_dim 128 (128-row K/V tiles, three score buffers, two softmax warpgroups on
// alternate tiles with the rows' running maxima handed over through shared memory, two Q buffers); it reached 953
// TFLOP/s at T = 4096 where the two-tile kernel above gives 1,000, so head_dim 128 stays there.
// =====================================================================================================
namespace rt {
constexpr int kM = 128, kD = 256, kN = 64, kNB = 4, kKStages = 3, kVStages = 2, kSlabs = kD / 64;
constexpr uint32_t kKvSlab = kN * 128;          // [64 rows][64 elements] 16-bit
constexpr uint32_t kKvTile = kSlabs * kKvSlab;  // a K or V tile: 32 KB
constexpr uint32_t kQSlab = 128 * 128;          // [128 rows][64 elements]
constexpr uint32_t kQBytes = kSlabs * kQSlab;   // 64 KB
enum { B_QFULL = 0, B_QEMPTY = 1, B_KFULL = 2, B_KEMPTY = 5, B_VFULL = 8, B_VEMPTY = 10, B_SFULL = 12, B_PFULL = 16, B_PVDONE = 20,
       B_OFULL = 24, B_OFREE = 25, B_COUNT = 26 };
constexpr uint32_t kSmemQ0 = 0, kSmemK = kQBytes, kSmemV = kSmemK + kKStages * kKvTile, kSmemBar = kSmemV + kVStages * kKvTile;
// Words the softmax and the epilogue thread of a row hand each other: {row sum of the item, item number + 1} (an
// 8-byte pair written and read as a unit, the number telling the reader what it has) and the number of items whose
// sum the epilogue thread has taken.
constexpr uint32_t kSmemLPair = kSmemBar + 256, kSmemAck = kSmemLPair + 128 * 8;
constexpr uint32_t kSmem = kSmemAck + 128 * 4 + 1024;
constexpr uint32_t kColO = kNB * kN;            // TMEM: S buffers [0, 256), then O [256, 512); P_b = first 32 columns of S_b
constexpr uint32_t kThreads = 384;
static_assert(kColO + kD <= kTmemCols, "the score buffers and O must fit in TMEM");
static_assert(kSmem <= 232448, "Q and the K and V rings must fit in 227 KB");
}  // namespace rt

struct RowTileArgs {
    void *out;
    RaggedRef rg;
    StatusRef status;
    uint32_t wait_mbar;
    uint32_t B, T, nh, nkv, G, m_tiles;   // m_tiles = ceil(T / 128)
    float scale_log2;
    const void *gate_src;   // optional: projection rows [tokens][nh][gate_row] whose elements [head_dim, 2 head_dim) are the gate
    uint32_t gate_row;
};

template <typename T>
__global__ void __launch_bounds__(rt::kThreads, 1)
rowtile_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
               const __grid_constant__ CUtensorMap map_v, const RowTileArgs a) {
    using namespace rt;
    constexpr uint32_t kWProd = 4, kWSEven = 5, kWPv = 6, kWSOdd = 7, kWEpi = 8;
    extern __shared__ unsigned char smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    unsigned char *smem = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t bar0 = smem_base + kSmemBar;
    auto bar = [&](int i) { return bar0 + 8u * i; };
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem + kSmemBar + 8 * B_COUNT);
    volatile uint32_t *abort_word = tmem_slot + 1;
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (gave_up(a.status)) return;
    const WaitCtx wc{abort_word, a.status, a.wait_mbar};

    struct Item { uint32_t b, h, kvh, q0, nkv, len, tok0, qrow, qseq; };   // fields as in the two-tile kernel
    const uint32_t bh_count = a.B * a.nh, total_items = a.rg.items ? a.rg.entries * a.nh : a.m_tiles * bh_count;
    auto get_item = [&](uint32_t w) {   // heaviest (latest rows) first
        Item it;
        uint32_t m;
        if (a.rg.items) {
            const uint4 e = __ldg(a.rg.items + w / a.nh);
            it.b = e.x; m = e.y; it.len = e.z; it.tok0 = e.w; it.h = w % a.nh;
            it.q0 = m * kM; it.qrow = it.tok0 + it.q0; it.qseq = 0;
        } else {
            const uint32_t bh = w % bh_count;
            m = a.m_tiles - 1 - w / bh_count;
            it.b = bh / a.nh; it.h = bh % a.nh; it.len = a.T; it.tok0 = it.b * a.T;
            it.q0 = m * kM; it.qrow = it.q0; it.qseq = it.b;
        }
        it.kvh = it.h / a.G;
        it.nkv = (m + 1) * (kM / kN);   // kv tiles 0 .. (q0 + 127) / kN; rows past T read as zeros and are masked
        return it;
    };
    auto item_of_round = [&](uint32_t rnd) {   // serpentine deal, as in the two-tile kernel
        return rnd * gridDim.x + ((rnd & 1u) ? gridDim.x - 1u - blockIdx.x : blockIdx.x);
    };
    constexpr uint32_t kFmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;

    if (warp == kWProd && lane == 0) {
        mbar_init(bar(B_QFULL), 1); mbar_init(bar(B_QEMPTY), 2); mbar_init(bar(B_OFULL), 1);
        mbar_init(bar(B_OFREE), 128);
        for (int s = 0; s < kKStages; ++s) { mbar_init(bar(B_KFULL + s), 1); mbar_init(bar(B_KEMPTY + s), 1); }
        for (int s = 0; s < kVStages; ++s) { mbar_init(bar(B_VFULL + s), 1); mbar_init(bar(B_VEMPTY + s), 1); }
        for (int b = 0; b < kNB; ++b) { mbar_init(bar(B_SFULL + b), 1); mbar_init(bar(B_PFULL + b), 128); mbar_init(bar(B_PVDONE + b), 1); }
        *abort_word = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (tid < 128) {   // nothing decided, posted or taken yet
        sts_pair(smem_base + kSmemLPair + 8 * tid, 0u, 0u);
        reinterpret_cast<volatile uint32_t *>(smem + kSmemAck)[tid] = 0u;
    }
    if (warp == kWSEven) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void *)tmem_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == kWProd) {
        // =============================== TMA producer ===============================
        // Two cursors walk the item list, one requesting K tiles (and each item's Q ahead of its first K), one V tiles.
        // Neither waits for the other: the thread polls what each needs next (a free slot; for Q, both score issuers
        // done with the previous item) and requests whatever can go, so K runs as far ahead of V as its ring allows —
        // the score MMAs run up to NB tiles ahead of the PV MMAs, which free the V slots.
        if (lane == 0) {
            bool ok = true;
            struct Cursor { uint32_t rnd, j, g; bool have, done; Item it; const CUtensorMap *map; };
            auto advance = [&](Cursor &c) {   // to the next tile of the CTA's list
                if (c.have && ++c.j < c.it.nkv) return;
                c.have = false;
                for (; c.rnd * gridDim.x < total_items; ++c.rnd) {
                    const uint32_t w = item_of_round(c.rnd);
                    if (w >= total_items) continue;
                    c.it = get_item(w); c.j = 0; c.have = true; ++c.rnd;
                    return;
                }
                c.done = true;
            };
            Cursor kc{0, 0, 0, false, false, {}, &map_k}, vc{0, 0, 0, false, false, {}, &map_v};
            advance(kc); advance(vc);
            uint32_t qi = 0;
            auto k_ready = [&]() {
                if (kc.j == 0 && qi > 0 && !mbar_try(bar(B_QEMPTY), (qi - 1) & 1)) return false;
                return kc.g < (uint32_t)kKStages || mbar_try(bar(B_KEMPTY + kc.g % kKStages), ((kc.g / kKStages) & 1) ^ 1);
            };
            auto v_ready = [&]() {
                return vc.g < (uint32_t)kVStages || mbar_try(bar(B_VEMPTY + vc.g % kVStages), ((vc.g / kVStages) & 1) ^ 1);
            };
            auto request_k = [&]() {
                if (kc.j == 0) {   // the item's Q (both score issuers are done with the previous item's)
                    ++qi;
                    mbar_expect_tx(bar(B_QFULL), kQBytes);
                    for (int c = 0; c < kSlabs; ++c)
                        tma_load_4d(smem_base + kSmemQ0 + c * kQSlab, &map_q, bar(B_QFULL), 64 * c, (int)kc.it.h, (int)kc.it.qrow, (int)kc.it.qseq);
                    if (a.rg.kv_maps) { kc.map = a.rg.kv_maps + 2 * kc.it.b; tensormap_acquire(kc.map); }
                }
                const uint32_t s = kc.g % kKStages;
                mbar_expect_tx(bar(B_KFULL + s), kKvTile);
                tma_load_kv_tile<kN, kSlabs>(smem_base + kSmemK + s * kKvTile, kKvSlab, kc.map, bar(B_KFULL + s), a.rg, kc.it.b, kc.it.kvh,
                                             kc.j * kN, kc.it.len, a.rg.kv_maps != nullptr);
                ++kc.g;
                advance(kc);
            };
            auto request_v = [&]() {
                if (vc.j == 0 && a.rg.kv_maps) { vc.map = a.rg.kv_maps + 2 * vc.it.b + 1; tensormap_acquire(vc.map); }
                const uint32_t s = vc.g % kVStages;
                mbar_expect_tx(bar(B_VFULL + s), kKvTile);
                tma_load_kv_tile<kN, kSlabs>(smem_base + kSmemV + s * kKvTile, kKvSlab, vc.map, bar(B_VFULL + s), a.rg, vc.it.b, vc.it.kvh,
                                             vc.j * kN, vc.it.len, a.rg.kv_maps != nullptr);
                ++vc.g;
                advance(vc);
            };
            uint32_t idle = 0;
            while ((!kc.done || !vc.done) && ok) {
                bool did = false;
                if (!kc.done && k_ready()) { request_k(); did = true; }
                if (!vc.done && v_ready()) { request_v(); did = true; }
                if (did) { idle = 0; continue; }
                if ((++idle & 1023u) == 0 && (*wc.abort_word || gave_up(wc.status))) ok = false;
                if (idle >= wc.limit) {   // nothing could be requested for the whole wait limit
                    *wc.abort_word = 1;
                    report_timeout(wc.status, 1);
                    ok = false;
                }
            }
        }
    } else if (warp == kWSEven || warp == kWSOdd) {
        // =============================== score-MMA issuers ===============================
        if (lane == 0) {
            const uint32_t par = warp == kWSEven ? 0u : 1u;      // this thread's tiles: those whose running number has this parity
            const uint32_t idesc_qk = make_idesc(kFmt, false, kN);
            bool ok = true;
            uint32_t gk = 0, qi = 0, sc = 0;   // running counts: K/V tiles, items, score tiles
            for (uint32_t rnd = 0; rnd * gridDim.x < total_items && ok; ++rnd) {
                const uint32_t w = item_of_round(rnd);
                if (w >= total_items) continue;
                const Item it = get_item(w);
                const uint32_t qa = smem_base + kSmemQ0;
                ok = mbar_wait(bar(B_QFULL), qi & 1, wc, 3);
                ++qi;
                const uint32_t j0 = (par ^ sc) & 1u;   // (an item has an even number of tiles, so both threads have some)
                for (uint32_t j = j0; j < it.nkv && ok; j += 2) {
                    const uint32_t g = gk + j, t = sc + j, s = g % kKStages, b = t % kNB;
                    ok = mbar_wait(bar(B_KFULL + s), (g / kKStages) & 1, wc, 4);
                    // S(t) lands where P(t - NB) lived: that PV must be complete
                    if (ok && t >= (uint32_t)kNB) ok = mbar_wait(bar(B_PVDONE + b), ((t / kNB) - 1) & 1, wc, 6);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t kb = smem_base + kSmemK + s * kKvTile;
#pragma unroll
                    for (uint32_t ks = 0; ks < kD / 16; ++ks) {      // S_b = Q * K(slot s)^T
                        const uint32_t so = (ks >> 2), ko = (ks & 3) * 32;
                        mma_ss(tmem + b * kN, desc_kmajor(qa + so * kQSlab + ko), desc_kmajor(kb + so * kKvSlab + ko), idesc_qk, ks > 0);
                    }
                    tc_commit(bar(B_SFULL + b));
                    tc_commit(bar(B_KEMPTY + s));                    // the K slot is free as soon as this S is computed
                    if (j + 2 >= it.nkv) tc_commit(bar(B_QEMPTY));   // this thread's last S of the item (Q is free when both have said so)
                }
                gk += it.nkv; sc += it.nkv;
            }
        }
    } else if (warp == kWPv) {
        // =============================== PV issuer ===============================
        if (lane == 0) {
            const uint32_t idesc_pv = make_idesc(kFmt, true, kD);
            bool ok = true;
            uint32_t gk = 0, sc = 0, n_item = 0;
            for (uint32_t rnd = 0; rnd * gridDim.x < total_items && ok; ++rnd) {
                const uint32_t w = item_of_round(rnd);
                if (w >= total_items) continue;
                const Item it = get_item(w);
                for (uint32_t j = 0; j < it.nkv && ok; ++j) {
                    const uint32_t g = gk + j, t = sc + j, s = g % kVStages, b = t % kNB;
                    ok = mbar_wait(bar(B_VFULL + s), (g / kVStages) & 1, wc, 5);
                    if (ok) ok = mbar_wait(bar(B_PFULL + b), (t / kNB) & 1, wc, 8);
                    // the item's first PV overwrites O: the epilogue must have read the previous item's
                    if (ok && j == 0 && n_item > 0) ok = mbar_wait(bar(B_OFREE), (n_item - 1) & 1, wc, 7);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t vb = smem_base + kSmemV + s * kKvTile;
#pragma unroll
                    for (uint32_t ks = 0; ks < kN / 16; ++ks)      // O (+)= P_b * V(slot s)
                        mma_ts(tmem + kColO, tmem + b * kN + ks * 8, desc_mnmajor(vb + ks * 2048, kKvSlab), idesc_pv, j > 0 || ks > 0);
                    tc_commit(bar(B_VEMPTY + s));
                    tc_commit(bar(B_PVDONE + b));
                    if (j + 1 == it.nkv) tc_commit(bar(B_OFULL));
                }
                gk += it.nkv; sc += it.nkv; ++n_item;
            }
        }
    } else if (warp >= kWEpi) {
        // =============================== epilogue: O / l (x sigmoid(gate)) -> global ===============================
        const uint32_t quarter = warp & 3, r = quarter * 32 + lane;    // row in the tile == TMEM lane
        const uint32_t t_o = tmem + ((quarter * 32) << 16) + kColO;
        bool ok = true;
        uint32_t oc = 0;
        for (uint32_t rnd = 0; rnd * gridDim.x < total_items && ok; ++rnd) {
            const uint32_t w = item_of_round(rnd);
            if (w >= total_items) continue;
            const Item item = get_item(w);
            const uint32_t row = item.q0 + r;
            // the row's sum, as the softmax thread of this row posted it for item number oc (bounded spin)
            float l_total;
            {
                const uint32_t slot = smem_base + kSmemLPair + 8 * r;
                uint2 pr = lds_pair(slot);
                for (uint32_t i = 0; pr.y != oc + 1 && i < wc.limit; ++i) {
                    pr = lds_pair(slot);
                    if ((i & 1023u) == 1023u && (*wc.abort_word || gave_up(wc.status))) break;
                }
                if (pr.y != oc + 1) {
                    *wc.abort_word = 1;
                    report_timeout(wc.status, 15);
                    ok = false;
                }
                l_total = __uint_as_float(pr.x);
            }
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            reinterpret_cast<volatile uint32_t *>(smem + kSmemAck)[r] = oc + 1;   // taken: the slot may be written again
            const float inv = 1.0f / l_total;
            ok = mbar_wait(bar(B_OFULL), oc & 1, wc, 11);
            if (!ok) break;
            tc_fence_after();
            T *dst = reinterpret_cast<T *>(a.out) + (((size_t)item.tok0 + row) * a.nh + item.h) * kD;
            const T *gate = (a.gate_src && row < item.len)
                                ? reinterpret_cast<const T *>(a.gate_src) + (((size_t)item.tok0 + row) * a.nh + item.h) * a.gate_row + kD : nullptr;
            // The row leaves TMEM first, scaled and packed to 16 bits (head_dim / 2 registers), so that O is free for the
            // next item's first PV after a few hundred clocks; the stores (one row per thread: 32 separate lines per
            // warp instruction, slow) follow, under the next item's MMAs.  With a gate, the row is held as fp32 x
            // sigmoid(gate) rounded once, the gate words loaded while this thread waited for the item's last PV.
            uint32_t pk[kD / 2];
#pragma unroll
            for (int c = 0; c < kD / 16; ++c) {   // 16 columns at a time: the packed row and one chunk are what is live
                uint32_t v[16];
                tmem_ld16(t_o + c * 16, v);
                tmem_wait_ld();
                if (c == kD / 16 - 1) {   // O is read: the next item's first PV may overwrite it
                    tc_fence_before();
                    mbar_arrive(bar(B_OFREE));
                }
                if (gate) {
#pragma unroll
                    for (int i = 0; i < 16; i += 8) {
                        const uint4 g4 = __ldg(reinterpret_cast<const uint4 *>(gate + c * 16 + i));
                        const T *ge = reinterpret_cast<const T *>(&g4);
#pragma unroll
                        for (int k = 0; k < 8; k += 2)
                            pk[c * 8 + (i + k) / 2] = pack16<T>(__uint_as_float(v[i + k]) * inv * sigmoidf_ref(to_f32<T>(ge[k])),
                                                                __uint_as_float(v[i + k + 1]) * inv * sigmoidf_ref(to_f32<T>(ge[k + 1])));
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 16; i += 2)
                        pk[c * 8 + i / 2] = pack16<T>(__uint_as_float(v[i]) * inv, __uint_as_float(v[i + 1]) * inv);
                }
            }
            if (row < item.len) {
#pragma unroll
                for (int i = 0; i < kD / 8; ++i)
                    reinterpret_cast<uint4 *>(dst)[i] = make_uint4(pk[4 * i], pk[4 * i + 1], pk[4 * i + 2], pk[4 * i + 3]);
            }
            ++oc;
        }
    } else {
        // =============================== softmax (one thread per query row) ===============================
        const uint32_t r = tid;                         // row in the tile == TMEM lane
        const uint32_t lane_base = (warp * 32) << 16;
        const uint32_t t_o = tmem + lane_base + kColO;
        bool ok = true;
        uint32_t sc = 0, oc = 0;                        // score tiles / items finished before the current item
        for (uint32_t rnd = 0; rnd * gridDim.x < total_items && ok; ++rnd) {
            const uint32_t w = item_of_round(rnd);
            if (w >= total_items) continue;
            const Item item = get_item(w);
            const uint32_t row = item.q0 + r;           // global query row == its causal limit
            float m_ref = -INFINITY, l_sum = 0.f;
            for (uint32_t j = 0; j < item.nkv && ok; ++j) {
                const uint32_t t = sc + j, b = t % kNB;
                const uint32_t t_s = tmem + lane_base + b * kN;
                ok = mbar_wait(bar(B_SFULL + b), (t / kNB) & 1, wc, 9);
                if (!ok) break;
                tc_fence_after();
                // one tile of the online softmax; tiles that touch the diagonal are a second instantiation, so the
                // common path carries no mask code
                auto tile_body = [&](auto diag_c) {
                    constexpr bool diag = decltype(diag_c)::value;
                    const int lim = diag ? (int)row - (int)(j * kN) : kN - 1;   // columns 0..lim of this tile are visible
                    // ---- row maximum; the 64 scores stay in registers for the second pass ----
                    uint32_t va[32], vb[32];
                    tmem_ld32(t_s, va);
                    tmem_ld32(t_s + 32, vb);
                    tmem_wait_ld();
                    float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
                    if (!diag || lim >= kN - 1) {
#pragma unroll
                        for (int i = 0; i < 32; i += 4) {
                            m4[0] = max3(m4[0], __uint_as_float(va[i]), __uint_as_float(va[i + 1]));
                            m4[1] = max3(m4[1], __uint_as_float(va[i + 2]), __uint_as_float(va[i + 3]));
                            m4[2] = max3(m4[2], __uint_as_float(vb[i]), __uint_as_float(vb[i + 1]));
                            m4[3] = max3(m4[3], __uint_as_float(vb[i + 2]), __uint_as_float(vb[i + 3]));
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            if (i <= lim) m4[i & 1] = fmaxf(m4[i & 1], __uint_as_float(va[i]));
                            if (32 + i <= lim) m4[2 + (i & 1)] = fmaxf(m4[2 + (i & 1)], __uint_as_float(vb[i]));
                        }
                    }
                    // scale > 0; -inf stays -inf (a row that sees nothing of this tile)
                    const float mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])) * a.scale_log2;
                    float corr = 1.f;
                    if (j == 0) m_ref = mx;                  // key 0 is visible to every row: finite
                    else if (mx > m_ref + kRescaleThreshold) { corr = exp2f(m_ref - mx); m_ref = mx; }
                    l_sum *= corr;
                    if (__any_sync(0xffffffffu, corr != 1.f)) {
                        // O belongs to PV(t-1) until that MMA has completed; only a rescale has to wait for it (that
                        // barrier completes next for PV(t-1+NB), which needs the P of a tile after this one first)
                        ok = mbar_wait(bar(B_PVDONE + ((t - 1) % kNB)), ((t - 1) / kNB) & 1, wc, 10);
                        if (!ok) return;
                        tc_fence_after();
#pragma unroll
                        for (int c = 0; c < kD / 32; ++c) {
                            uint32_t v[32];
                            tmem_ld32(t_o + c * 32, v);
                            tmem_wait_ld();
#pragma unroll
                            for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * corr);
                            tmem_st32(t_o + c * 32, v);
                        }
                    }
                    // ---- P = exp2(s * scale - m_ref), masked past the diagonal; packed over the first kN/2 columns of S ----
                    const float neg_m = -m_ref;
                    const unsigned long long scale2 = pack_f32x2(a.scale_log2, a.scale_log2), negm2 = pack_f32x2(neg_m, neg_m);
                    unsigned long long ls2[2] = {0ull, 0ull};
                    // 32 columns -> 16 packed words; base = first column of the chunk
                    auto exp_chunk = [&](const uint32_t (&v)[32], uint32_t (&pk)[16], int base) {
#pragma unroll
                        for (int i = 0; i < 32; i += 2) {
                            float x0, x1;
                            fma_f32x2(x0, x1, __uint_as_float(v[i]), __uint_as_float(v[i + 1]), scale2, negm2);
                            float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
                            if (diag) {
                                if (base + i > lim) p0 = 0.f;
                                if (base + i + 1 > lim) p1 = 0.f;
                            }
                            ls2[(i >> 1) & 1] = add_f32x2(ls2[(i >> 1) & 1], pack_f32x2(p0, p1));
                            pk[i >> 1] = pack16<T>(p0, p1);
                        }
                    };
                    uint32_t pa[16], pb[16];
                    exp_chunk(va, pa, 0);
                    exp_chunk(vb, pb, 32);
                    tmem_st16(t_s, pa);
                    tmem_st16(t_s + 16, pb);
                    {
                        float s0, s1, s2, s3;
                        asm("mov.b64 {%0, %1}, %2;" : "=f"(s0), "=f"(s1) : "l"(ls2[0]));
                        asm("mov.b64 {%0, %1}, %2;" : "=f"(s2), "=f"(s3) : "l"(ls2[1]));
                        l_sum += (s0 + s1) + (s2 + s3);
                    }
                    tmem_wait_st();
                    tc_fence_before();
                    mbar_arrive(bar(B_PFULL + b));
                };
                if ((j + 1) * kN - 1 > item.q0) tile_body(std::true_type{});
                else tile_body(std::false_type{});
            }
            // the item's row sum goes to the epilogue warps; this thread is free for the next item
            if (ok) {
                // (the epilogue thread of this row must have taken the previous item's: bounded spin)
                volatile uint32_t *ack = reinterpret_cast<volatile uint32_t *>(smem + kSmemAck) + r;
                uint32_t got = *ack;
                for (uint32_t i = 0; got < oc && i < wc.limit; ++i) {
                    got = *ack;
                    if ((i & 1023u) == 1023u && (*wc.abort_word || gave_up(wc.status))) break;
                }
                if (got < oc) {
                    *wc.abort_word = 1;
                    report_timeout(wc.status, 16);
                    ok = false;
                }
                sts_pair(smem_base + kSmemLPair + 8 * r, __float_as_uint(l_sum), oc + 1);
            }
            sc += item.nkv;
            ++oc;
        }
    }
    // ---- teardown ----
    tc_fence_before();
    __syncthreads();
    if (warp == kWProd && lane == 0 && *abort_word) {
        // an aborted CTA may still have copies in flight: give them a bounded time to land before shared memory is handed back
        for (int s = 0; s < kKStages + kVStages; ++s)
            for (uint32_t i = 0; i < (1u << 16); ++i)
                if (mbar_try(bar(s < kKStages ? B_KFULL + s : B_VFULL + (s - kKStages)), 0)) break;
    }
    __syncthreads();
    if (warp == kWSEven) {
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
                        uint64_t d3, uint64_t s1, uint64_t s2, uint64_t s3, uint32_t box_rows = 128) {
    if (d3 == 1 && s3 >= (1ull << 40)) s3 = 1ull << 39;   // the stride of a dimension of extent 1 is never used, but must encode
    cuuint64_t dims[4] = {d0, d1, d2, d3};
    cuuint64_t strides[3] = {s1, s2, s3};  // bytes, dims 1..3
    cuuint32_t box[4] = {64, 1, box_rows, 1};   // 64 elements (128 B, the swizzle span) x box_rows rows
    cuuint32_t estr[4] = {1, 1, 1, 1};
    EncodeTiledFn encode = encode_tiled_fn();
    if (!encode) return false;
    return encode(map, dt, 4, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// ---- listed (ragged) batches: host tables --------------------------------------------------
// Workspace of a listed batch: [row-block list][first packed token of every sequence][K and V map of every sequence]
// [what the step from the projections needs].  Every part starts on a 128-byte boundary (tensor maps need 64).
struct RaggedLayout {
    size_t items_off, tok_off, maps_off, extra_off, total;
    uint32_t entries, total_tokens, max_len;
};
static size_t up128(size_t v) { return (v + 127) & ~(size_t)127; }
static RaggedLayout ragged_layout(const shady_prefill_params *p, const uint32_t *lens, bool with_append) {
    RaggedLayout L{};
    const uint32_t block_rows = p->head_dim == 256 ? 128u : 256u;
    unsigned long long toks = 0, entries = 0;
    for (uint32_t s = 0; s < p->num_seqs; ++s) {
        toks += lens[s];
        entries += (lens[s] + block_rows - 1) / block_rows;
        if (lens[s] > L.max_len) L.max_len = lens[s];
    }
    L.entries = (uint32_t)(entries > 0xffffffffull ? 0xffffffffull : entries);
    L.total_tokens = (uint32_t)(toks > 0xffffffffull ? 0xffffffffull : toks);
    L.items_off = 0;
    L.tok_off = up128(L.items_off + (size_t)L.entries * sizeof(uint4));
    L.maps_off = up128(L.tok_off + ((size_t)p->num_seqs + 1) * sizeof(uint32_t));
    L.extra_off = up128(L.maps_off + (size_t)p->num_seqs * 2 * sizeof(CUtensorMap));
    size_t extra = 0;
    if (with_append)
        extra = p->head_dim == 256 ? (size_t)L.total_tokens * p->num_q_heads * 256 * 2 : (size_t)L.max_len * 64 * sizeof(float2);
    L.total = up128(L.extra_off + extra);
    return L;
}
size_t prefill_ragged_workspace_bytes(const shady_prefill_params *p, const uint32_t *h_seq_lens, bool with_append) {
    return ragged_layout(p, h_seq_lens, with_append).total;
}

// Small host tables travel through one page-locked staging buffer of the context; the event says when the last
// copy out of it is done.
static int stage_upload(shady_ctx *ctx, const void *src, size_t bytes, void *d_dst) {
    if (ctx->stage_done) SHADY_CUDA_OK(ctx, cudaEventSynchronize(ctx->stage_done));
    else SHADY_CUDA_OK(ctx, cudaEventCreateWithFlags(&ctx->stage_done, cudaEventDisableTiming));
    if (bytes > ctx->stage_bytes) {
        if (ctx->stage) cudaFreeHost(ctx->stage);
        ctx->stage = nullptr; ctx->stage_bytes = 0;
        const size_t want = bytes * 2 > (64u << 10) ? bytes * 2 : (64u << 10);
        SHADY_CUDA_OK(ctx, cudaHostAlloc(&ctx->stage, want, cudaHostAllocDefault));
        ctx->stage_bytes = want;
    }
    memcpy(ctx->stage, src, bytes);
    SHADY_CUDA_OK(ctx, cudaMemcpyAsync(d_dst, ctx->stage, bytes, cudaMemcpyHostToDevice, ctx->stream));
    SHADY_CUDA_OK(ctx, cudaEventRecord(ctx->stage_done, ctx->stream));
    return SHADY_OK;
}

// What a launcher needs to know about a listed batch once its tables are on their way to the device.
struct RaggedSetup {
    RaggedRef rg;
    RaggedLayout lay;
    bool pool_maps;         // paged cache: map_k / map_v cover the page pools
    CUtensorMap mk, mv;     // ... and are these
    const uint32_t *d_tok_start;
};

// Checks the batch, lists its row blocks heaviest first, encodes the K/V maps and sends everything to the workspace.
static int setup_ragged(shady_ctx *ctx, const std::string &w, const shady_prefill_params *p, const shady_prefill_batch *batch,
                        const shady_kv_cache *cache, void *d_ws, size_t ws_bytes, bool with_append, RaggedSetup *out) {
    SHADY_REQUIRE(ctx, p && batch && batch->h_seq_lens && cache, SHADY_ERR_BAD_ARG, w + ": null argument");
    SHADY_REQUIRE(ctx, p->head_dim == 128 || p->head_dim == 256, SHADY_ERR_UNSUPPORTED, w + ": head_dim must be 128 or 256");
    SHADY_REQUIRE(ctx, p->dtype == SHADY_BF16 || p->dtype == SHADY_F16, SHADY_ERR_UNSUPPORTED, w + ": dtype must be bf16 or f16");
    SHADY_REQUIRE(ctx, cache->dtype == p->dtype, SHADY_ERR_UNSUPPORTED, w + ": cache dtype must equal the Q dtype");
    SHADY_REQUIRE(ctx, p->num_seqs && p->num_kv_heads && p->num_q_heads && p->num_q_heads % p->num_kv_heads == 0, SHADY_ERR_BAD_ARG,
                  w + ": bad shape");
    const uint32_t S = p->num_seqs, hd = p->head_dim, nkv = p->num_kv_heads;
    const uint32_t block_rows = hd == 256 ? 128u : 256u, kv_rows = hd == 256 ? 64u : 128u;
    const uint32_t *lens = batch->h_seq_lens;
    for (uint32_t s = 0; s < S; ++s)
        SHADY_REQUIRE(ctx, lens[s] > 0, SHADY_ERR_BAD_ARG, w + ": sequence " + std::to_string(s) + " is empty");
    const RaggedLayout L = ragged_layout(p, lens, with_append);
    SHADY_REQUIRE(ctx, L.entries != 0xffffffffu && L.total_tokens < 0x7fffffffu && (unsigned long long)L.entries * p->num_q_heads <= 0x7fffffffull,
                  SHADY_ERR_UNSUPPORTED, w + ": too many tokens for one launch");
    SHADY_REQUIRE(ctx, d_ws && ((uintptr_t)d_ws % 128) == 0 && ws_bytes >= L.total, SHADY_ERR_WORKSPACE,
                  w + ": workspace missing, not 128-byte aligned or smaller than shady_prefill_ragged_workspace_size says (" +
                      std::to_string(L.total) + " bytes)");
    const bool paged = cache->d_page_table != nullptr, ptrs = cache->d_k_ptrs != nullptr;
    SHADY_REQUIRE(ctx, paged ? (cache->d_k_base && cache->d_v_base && cache->page_rows && cache->max_pages_per_seq)
                             : ptrs ? (cache->d_v_ptrs && batch->h_k_ptrs && batch->h_v_ptrs) : (cache->d_k_base && cache->d_v_base),
                  SHADY_ERR_BAD_ARG,
                  w + ": the cache needs page pools + table, or pointer arrays with their host copies in the batch, or base pointers");
    if (const int st = pending_timeout(ctx, w.c_str())) return st;

    std::vector<unsigned char> host(L.extra_off, 0);
    uint4 *items = reinterpret_cast<uint4 *>(host.data() + L.items_off);
    uint32_t *tok = reinterpret_cast<uint32_t *>(host.data() + L.tok_off);
    CUtensorMap *maps = reinterpret_cast<CUtensorMap *>(host.data() + L.maps_off);
    // row blocks, heaviest (latest rows: most K/V tiles) first; blocks of equal weight keep the sequences' order
    uint32_t t0 = 0, max_blocks = 0;
    for (uint32_t s = 0; s < S; ++s) {
        tok[s] = t0; t0 += lens[s];
        const uint32_t nb = (lens[s] + block_rows - 1) / block_rows;
        if (nb > max_blocks) max_blocks = nb;
    }
    tok[S] = t0;
    uint32_t e = 0;
    for (uint32_t m = max_blocks; m-- > 0;)
        for (uint32_t s = 0; s < S; ++s)
            if ((uint64_t)m * block_rows < lens[s]) items[e++] = make_uint4(s, m, lens[s], tok[s]);

    RaggedSetup rs{};
    rs.lay = L;
    rs.rg.items = reinterpret_cast<const uint4 *>((char *)d_ws + L.items_off);
    rs.rg.entries = L.entries;
    rs.d_tok_start = reinterpret_cast<const uint32_t *>((char *)d_ws + L.tok_off);
    const CUtensorMapDataType dt = p->dtype == SHADY_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    const uint64_t head_b = (uint64_t)hd * 2, row_b = (uint64_t)nkv * hd * 2;
    if (paged) {
        const uint32_t pr = cache->page_rows;
        SHADY_REQUIRE(ctx, (pr % kv_rows) == 0 || (pr < kv_rows && (kv_rows % pr) == 0 && (pr % 8) == 0), SHADY_ERR_UNSUPPORTED,
                      w + ": page_rows must be a multiple of " + std::to_string(kv_rows) + " or one of 8, 16, 32, 64 below it");
        SHADY_REQUIRE(ctx, (((uintptr_t)cache->d_k_base | (uintptr_t)cache->d_v_base) % 16) == 0, SHADY_ERR_BAD_ARG,
                      w + ": page pools must be 16-byte aligned");
        for (uint32_t s = 0; s < S; ++s)
            SHADY_REQUIRE(ctx, (lens[s] + pr - 1) / pr <= cache->max_pages_per_seq, SHADY_ERR_BAD_ARG,
                          w + ": sequence " + std::to_string(s) + " needs more pages than max_pages_per_seq");
        // the pool's size is not part of the cache description: the map's page extent is a bound the table's entries
        // stay below, and the first page number past it is what a box that starts beyond the sequence asks for
        const uint32_t pages_extent = 1u << 24;
        rs.rg.page_table = cache->d_page_table; rs.rg.max_pages = cache->max_pages_per_seq; rs.rg.page_rows = pr;
        rs.rg.box_rows = pr < kv_rows ? pr : kv_rows; rs.rg.oob_page = pages_extent;
        rs.pool_maps = true;
        const bool ok = make_map_4d(&rs.mk, dt, cache->d_k_base, hd, nkv, pr, pages_extent, head_b, row_b, row_b * pr, rs.rg.box_rows) &&
                        make_map_4d(&rs.mv, dt, cache->d_v_base, hd, nkv, pr, pages_extent, head_b, row_b, row_b * pr, rs.rg.box_rows);
        SHADY_REQUIRE(ctx, ok, SHADY_ERR_CUDA, w + ": cuTensorMapEncodeTiled failed (page pools)");
    } else {
        SHADY_REQUIRE(ctx, ptrs || ((cache->seq_stride * 2) % 16 == 0 && (S == 1 || cache->seq_stride >= (uint64_t)L.max_len * nkv * hd)),
                      SHADY_ERR_BAD_ARG, w + ": seq_stride smaller than the longest sequence or not a multiple of 16 bytes");
        for (uint32_t s = 0; s < S; ++s) {
            const char *kb = ptrs ? (const char *)batch->h_k_ptrs[s] : (const char *)cache->d_k_base + (size_t)s * cache->seq_stride * 2;
            const char *vb = ptrs ? (const char *)batch->h_v_ptrs[s] : (const char *)cache->d_v_base + (size_t)s * cache->seq_stride * 2;
            SHADY_REQUIRE(ctx, kb && vb && (((uintptr_t)kb | (uintptr_t)vb) % 16) == 0, SHADY_ERR_BAD_ARG,
                          w + ": cache of sequence " + std::to_string(s) + " is null or not 16-byte aligned");
            // extent = the sequence's own rows: what lies past them reads as zero whatever the memory holds
            const bool ok = make_map_4d(&maps[2 * s], dt, kb, hd, nkv, lens[s], 1, head_b, row_b, row_b * lens[s], kv_rows) &&
                            make_map_4d(&maps[2 * s + 1], dt, vb, hd, nkv, lens[s], 1, head_b, row_b, row_b * lens[s], kv_rows);
            SHADY_REQUIRE(ctx, ok, SHADY_ERR_CUDA, w + ": cuTensorMapEncodeTiled failed (sequence " + std::to_string(s) + ")");
        }
        rs.rg.kv_maps = reinterpret_cast<const CUtensorMap *>((char *)d_ws + L.maps_off);
    }
    if (const int st = stage_upload(ctx, host.data(), host.size(), d_ws)) return st;
    *out = rs;
    return SHADY_OK;
}

// What the two entry points share: argument checks, tensor maps, the launch.  q_base/qrow describe where Q tiles
// are fetched from: [B][T][nh][qrow] elements with the Q half in the first 128 of every head's qrow elements.
// `rs`: a listed batch (set up by setup_ragged): Q and the output are packed token-major.
struct FusedQ {
    const float2 *cs_table;
    const uint16_t *norm_w;
    uint32_t has_gate;
    float eps;
};
static int launch_prefill_impl(shady_ctx *ctx, const char *who, const shady_prefill_params *p, const void *d_q, uint32_t qrow,
                               const shady_kv_cache *cache, void *d_out, const FusedQ *fq, const RaggedSetup *rs = nullptr) {
    const std::string w(who);
    SHADY_REQUIRE(ctx, p && d_q && cache && d_out, SHADY_ERR_BAD_ARG, w + ": null argument");
    SHADY_REQUIRE(ctx, p->head_dim == 128, SHADY_ERR_UNSUPPORTED, w + ": head_dim must be 128 or 256");
    SHADY_REQUIRE(ctx, p->dtype == SHADY_BF16 || p->dtype == SHADY_F16, SHADY_ERR_UNSUPPORTED, w + ": dtype must be bf16 or f16");
    SHADY_REQUIRE(ctx, cache->dtype == p->dtype, SHADY_ERR_UNSUPPORTED, w + ": cache dtype must equal the Q dtype");
    SHADY_REQUIRE(ctx, p->num_seqs && (rs || p->seq_len) && p->num_kv_heads && p->num_q_heads % p->num_kv_heads == 0, SHADY_ERR_BAD_ARG,
                  w + ": bad shape");
    SHADY_REQUIRE(ctx, rs || (cache->d_k_base && cache->d_v_base && !cache->d_k_ptrs && !cache->d_page_table), SHADY_ERR_UNSUPPORTED,
                  w + ": needs base + seq_stride cache addressing; pointer arrays and pages go through shady_attn_prefill_ragged");
    SHADY_REQUIRE(ctx, rs || p->num_seqs == 1 || cache->seq_stride >= (uint64_t)p->seq_len * p->num_kv_heads * 128, SHADY_ERR_BAD_ARG,
                  w + ": seq_stride smaller than one sequence");
    SHADY_REQUIRE(ctx, ((uintptr_t)d_q | (uintptr_t)d_out) % 16 == 0 &&
                           (rs || (((uintptr_t)cache->d_k_base | (uintptr_t)cache->d_v_base) % 16 == 0 && (cache->seq_stride * 2) % 16 == 0)),
                  SHADY_ERR_BAD_ARG, w + ": buffers must be 16-byte aligned");
    if (const int st = pending_timeout(ctx, who)) return st;
    const uint32_t B = p->num_seqs, T = p->seq_len, nh = p->num_q_heads, nkv = p->num_kv_heads;
    const CUtensorMapDataType dt = p->dtype == SHADY_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    CUtensorMap mq, mk, mv;
    bool maps_ok;
    // the Q map sees 128 of the qrow elements of every head: the gate half (if any) is skipped by the head stride
    if (rs) {
        const uint64_t toks = rs->lay.total_tokens;
        maps_ok = make_map_4d(&mq, dt, d_q, 128, nh, toks, 1, (uint64_t)qrow * 2, (uint64_t)nh * qrow * 2, toks * nh * qrow * 2);
        if (rs->pool_maps) { mk = rs->mk; mv = rs->mv; }
        else { mk = mq; mv = mq; }   // unused: every sequence brings its own pair
    } else {
        const uint64_t seq_stride_b = (B == 1 ? (uint64_t)T * nkv * 128 : cache->seq_stride) * 2;
        maps_ok = make_map_4d(&mq, dt, d_q, 128, nh, T, B, (uint64_t)qrow * 2, (uint64_t)nh * qrow * 2, (uint64_t)T * nh * qrow * 2) &&
                  make_map_4d(&mk, dt, cache->d_k_base, 128, nkv, T, B, 128 * 2, (uint64_t)nkv * 128 * 2, seq_stride_b) &&
                  make_map_4d(&mv, dt, cache->d_v_base, 128, nkv, T, B, 128 * 2, (uint64_t)nkv * 128 * 2, seq_stride_b);
    }
    SHADY_REQUIRE(ctx, maps_ok, SHADY_ERR_CUDA, w + ": cuTensorMapEncodeTiled failed");
    PrefillArgs a{};
    a.out = d_out; a.status = status_ref(ctx); a.wait_mbar = ctx->wait_mbar;
    a.B = B; a.T = T; a.nh = nh; a.nkv = nkv; a.G = nh / nkv;
    a.m_tiles = (T + 255) / 256;
    if (rs) a.rg = rs->rg;
    a.scale_log2 = (1.0f / sqrtf(128.0f)) * 1.4426950408889634f;
    a.q_src = d_q; a.qrow = qrow;
    if (fq) { a.cs_table = fq->cs_table; a.norm_w = fq->norm_w; a.has_gate = fq->has_gate; a.eps = fq->eps; }
    const unsigned long long total_items = rs ? (unsigned long long)rs->rg.entries * nh : (unsigned long long)a.m_tiles * B * nh;
    SHADY_REQUIRE(ctx, total_items <= 0x7fffffffull, SHADY_ERR_UNSUPPORTED, w + ": too many tiles for one launch");
    const unsigned blocks = (unsigned)(total_items < (unsigned long long)ctx->num_sms ? total_items : (unsigned long long)ctx->num_sms);   // persistent: one CTA per SM
    static thread_local int configured_dev = -1;
    if (configured_dev != ctx->device) {
        SHADY_CUDA_OK(ctx, cudaFuncSetAttribute(prefill_kernel<__nv_bfloat16, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, prefill_smem(2)));
        SHADY_CUDA_OK(ctx, cudaFuncSetAttribute(prefill_kernel<__half, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, prefill_smem(2)));
        SHADY_CUDA_OK(ctx, cudaFuncSetAttribute(prefill_kernel<__nv_bfloat16, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, prefill_smem(3)));
        SHADY_CUDA_OK(ctx, cudaFuncSetAttribute(prefill_kernel<__half, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, prefill_smem(3)));
        configured_dev = ctx->device;
    }
    const bool bf = p->dtype == SHADY_BF16;
    if (fq) {
        constexpr unsigned threads = kFusedThreads;
        if (bf) prefill_kernel<__nv_bfloat16, true><<<blocks, threads, prefill_smem(3), ctx->stream>>>(mq, mk, mv, a);
        else prefill_kernel<__half, true><<<blocks, threads, prefill_smem(3), ctx->stream>>>(mq, mk, mv, a);
    } else {
        if (bf) prefill_kernel<__nv_bfloat16, false><<<blocks, 320, prefill_smem(2), ctx->stream>>>(mq, mk, mv, a);
        else prefill_kernel<__half, false><<<blocks, 320, prefill_smem(2), ctx->stream>>>(mq, mk, mv, a);
    }
    ctx->launches++;
    SHADY_CUDA_OK(ctx, cudaGetLastError());
    return SHADY_OK;
}

// head_dim 256 (the row-tile kernel): Q [tokens][nh][256] already normed and rotated; gate_src (optional) the
// projection rows whose second half is the gate
static int launch_prefill256(shady_ctx *ctx, const char *who, const shady_prefill_params *p, const void *d_q,
                             const shady_kv_cache *cache, void *d_out, const void *gate_src, uint32_t gate_row,
                             const RaggedSetup *rs = nullptr) {
    const std::string w(who);
    SHADY_REQUIRE(ctx, p && d_q && cache && d_out, SHADY_ERR_BAD_ARG, w + ": null argument");
    SHADY_REQUIRE(ctx, p->dtype == SHADY_BF16 || p->dtype == SHADY_F16, SHADY_ERR_UNSUPPORTED, w + ": dtype must be bf16 or f16");
    SHADY_REQUIRE(ctx, cache->dtype == p->dtype, SHADY_ERR_UNSUPPORTED, w + ": cache dtype must equal the Q dtype");
    SHADY_REQUIRE(ctx, p->num_seqs && (rs || p->seq_len) && p->num_kv_heads && p->num_q_heads % p->num_kv_heads == 0, SHADY_ERR_BAD_ARG,
                  w + ": bad shape");
    SHADY_REQUIRE(ctx, rs || (cache->d_k_base && cache->d_v_base && !cache->d_k_ptrs && !cache->d_page_table), SHADY_ERR_UNSUPPORTED,
                  w + ": needs base + seq_stride cache addressing; pointer arrays and pages go through shady_attn_prefill_ragged");
    const uint32_t hd = 256, kv_rows = rt::kN;
    SHADY_REQUIRE(ctx, rs || p->num_seqs == 1 || cache->seq_stride >= (uint64_t)p->seq_len * p->num_kv_heads * hd, SHADY_ERR_BAD_ARG,
                  w + ": seq_stride smaller than one sequence");
    SHADY_REQUIRE(ctx, ((uintptr_t)d_q | (uintptr_t)d_out | (uintptr_t)gate_src) % 16 == 0 &&
                           (rs || (((uintptr_t)cache->d_k_base | (uintptr_t)cache->d_v_base) % 16 == 0 && (cache->seq_stride * 2) % 16 == 0)),
                  SHADY_ERR_BAD_ARG, w + ": buffers must be 16-byte aligned");
    if (const int st = pending_timeout(ctx, who)) return st;
    const uint32_t B = p->num_seqs, T = p->seq_len, nh = p->num_q_heads, nkv = p->num_kv_heads;
    const CUtensorMapDataType dt = p->dtype == SHADY_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    CUtensorMap mq, mk, mv;
    bool maps_ok;
    if (rs) {
        const uint64_t toks = rs->lay.total_tokens;
        maps_ok = make_map_4d(&mq, dt, d_q, hd, nh, toks, 1, hd * 2, (uint64_t)nh * hd * 2, toks * nh * hd * 2, 128);
        if (rs->pool_maps) { mk = rs->mk; mv = rs->mv; }
        else { mk = mq; mv = mq; }   // unused: every sequence brings its own pair
    } else {
        const uint64_t seq_stride_b = (B == 1 ? (uint64_t)T * nkv * hd : cache->seq_stride) * 2;
        maps_ok = make_map_4d(&mq, dt, d_q, hd, nh, T, B, hd * 2, (uint64_t)nh * hd * 2, (uint64_t)T * nh * hd * 2, 128) &&
                  make_map_4d(&mk, dt, cache->d_k_base, hd, nkv, T, B, hd * 2, (uint64_t)nkv * hd * 2, seq_stride_b, kv_rows) &&
                  make_map_4d(&mv, dt, cache->d_v_base, hd, nkv, T, B, hd * 2, (uint64_t)nkv * hd * 2, seq_stride_b, kv_rows);
    }
    SHADY_REQUIRE(ctx, maps_ok, SHADY_ERR_CUDA, w + ": cuTensorMapEncodeTiled failed");
    RowTileArgs a{};
    a.out = d_out; a.status = status_ref(ctx); a.wait_mbar = ctx->wait_mbar;
    a.B = B; a.T = T; a.nh = nh; a.nkv = nkv; a.G = nh / nkv;
    a.m_tiles = (T + 127) / 128;
    if (rs) a.rg = rs->rg;
    a.scale_log2 = (1.0f / sqrtf((float)hd)) * 1.4426950408889634f;
    a.gate_src = gate_src; a.gate_row = gate_row;
    const unsigned long long total_items = rs ? (unsigned long long)rs->rg.entries * nh : (unsigned long long)a.m_tiles * B * nh;
    SHADY_REQUIRE(ctx, total_items <= 0x7fffffffull, SHADY_ERR_UNSUPPORTED, w + ": too many tiles for one launch");
    const unsigned blocks = (unsigned)(total_items < (unsigned long long)ctx->num_sms ? total_items : (unsigned long long)ctx->num_sms);
    static thread_local int configured_dev = -1;
    if (configured_dev != ctx->device) {
        SHADY_CUDA_OK(ctx, cudaFuncSetAttribute(rowtile_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, rt::kSmem));
        SHADY_CUDA_OK(ctx, cudaFuncSetAttribute(rowtile_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, rt::kSmem));
        configured_dev = ctx->device;
    }
    if (p->dtype == SHADY_BF16) rowtile_kernel<__nv_bfloat16><<<blocks, rt::kThreads, rt::kSmem, ctx->stream>>>(mq, mk, mv, a);
    else rowtile_kernel<__half><<<blocks, rt::kThreads, rt::kSmem, ctx->stream>>>(mq, mk, mv, a);
    ctx->launches++;
    SHADY_CUDA_OK(ctx, cudaGetLastError());
    return SHADY_OK;
}

int launch_prefill(shady_ctx *ctx, const shady_prefill_params *p, const void *d_q, const shady_kv_cache *cache, void *d_out) {
    if (p && p->head_dim == 256) return launch_prefill256(ctx, "attn_prefill", p, d_q, cache, d_out, nullptr, 0);
    return launch_prefill_impl(ctx, "attn_prefill", p, d_q, 128, cache, d_out, nullptr);
}

int launch_append_ex(shady_ctx *, const shady_append_params *, const void *, void *, const void *, void *, float *,
                     const shady_kv_cache *, const uint16_t *, const uint32_t *, const uint32_t *, const uint32_t *, bool,
                     const AppendRagged *);

// K/V half of the append (norm + RoPE of K, cache rows of K and V) plus the cos/sin table of positions [0, T)
// (append.cu); Q is left to the attention kernel.
int launch_append_kv_table(shady_ctx *ctx, const shady_append_params *ap, const void *d_k_proj, const void *d_v_proj,
                           const shady_kv_cache *cache, const uint16_t *d_qk_norm_bf16, float2 *d_cs_table, const AppendRagged *rg);

// head_dim 128: the cos/sin table of the T positions; head_dim 256: the normed and rotated Q of the whole batch
size_t prefill_workspace_bytes(const shady_prefill_params *p) {
    if (p->head_dim == 256) return (size_t)p->num_seqs * p->seq_len * p->num_q_heads * 256 * 2;
    return (size_t)p->seq_len * 64 * sizeof(float2);
}

static int check_prefill_append(shady_ctx *ctx, const shady_append_params *ap, const shady_prefill_params *p, bool listed) {
    SHADY_REQUIRE(ctx, ap->num_heads == p->num_q_heads && ap->num_kv_heads == p->num_kv_heads && ap->head_dim == p->head_dim &&
                           ap->num_seqs == p->num_seqs && (listed || ap->tokens_per_seq == p->seq_len),
                  SHADY_ERR_BAD_ARG, "attn_prefill_append: append and prefill parameters disagree");
    SHADY_REQUIRE(ctx, ap->in_dtype == p->dtype, SHADY_ERR_UNSUPPORTED, "attn_prefill_append: the projections must have the cache dtype (bf16 or f16)");
    SHADY_REQUIRE(ctx, ap->interleaved && ap->rotary_dim <= p->head_dim && (ap->rotary_dim % 2) == 0 &&
                           ap->s1_limit == ap->rotary_dim / 2 && ap->s2_limit == ap->rotary_dim / 2,
                  SHADY_ERR_UNSUPPORTED, "attn_prefill_append: interleaved RoPE with one position per token only");
    return SHADY_OK;
}

// The whole prefill step from the projections: one pass writes K (normed, rotated) and V into rows [0, T) of every
// sequence's cache and the cos/sin table; the attention kernel then takes Q raw, norms and rotates it tile by tile in
// shared memory and applies the gate in its epilogue.
int launch_prefill_append(shady_ctx *ctx, const shady_append_params *ap, const shady_prefill_params *p, const void *d_q_proj_full,
                          const void *d_k_proj, const void *d_v_proj, const uint16_t *d_qk_norm_bf16, const shady_kv_cache *cache,
                          void *d_out, void *d_ws, size_t ws_bytes) {
    SHADY_REQUIRE(ctx, ap && p && d_q_proj_full && d_k_proj && d_v_proj && cache && d_out, SHADY_ERR_BAD_ARG, "attn_prefill_append: null argument");
    if (const int st = check_prefill_append(ctx, ap, p, false)) return st;
    SHADY_REQUIRE(ctx, d_ws && ws_bytes >= prefill_workspace_bytes(p) && ((uintptr_t)d_ws % 16) == 0, SHADY_ERR_WORKSPACE,
                  "attn_prefill_append: workspace missing, too small or not 16-byte aligned");
    if (p->head_dim == 256) {
        // the wide-head kernel takes Q rotated: one append pass writes it into the workspace (and K/V into the cache);
        // the gate is read from the projection rows by the attention epilogue
        shady_append_params ap2 = *ap;
        ap2.q_dtype = p->dtype; ap2.write_k_back = 0;
        if (const int st = launch_append_ex(ctx, &ap2, d_q_proj_full, const_cast<void *>(d_k_proj), d_v_proj, d_ws, nullptr, cache,
                                            d_qk_norm_bf16, nullptr, nullptr, nullptr, true, nullptr))
            return st;
        return launch_prefill256(ctx, "attn_prefill_append", p, d_ws, cache, d_out, ap->has_gate ? d_q_proj_full : nullptr, 512);
    }
    float2 *table = reinterpret_cast<float2 *>(d_ws);
    if (const int st = launch_append_kv_table(ctx, ap, d_k_proj, d_v_proj, cache, d_qk_norm_bf16, table, nullptr)) return st;
    const FusedQ fq{table, d_qk_norm_bf16, ap->has_gate, ap->eps};
    return launch_prefill_impl(ctx, "attn_prefill_append", p, d_q_proj_full, ap->has_gate ? 256u : 128u, cache, d_out, &fq);
}

// ---- listed batches: prompts of different lengths, caches of any addressing ------------------------------------
int launch_prefill_ragged(shady_ctx *ctx, const shady_prefill_params *p, const shady_prefill_batch *batch, const void *d_q,
                          const shady_kv_cache *cache, void *d_out, void *d_ws, size_t ws_bytes) {
    RaggedSetup rs;
    if (const int st = setup_ragged(ctx, "attn_prefill_ragged", p, batch, cache, d_ws, ws_bytes, false, &rs)) return st;
    if (p->head_dim == 256) return launch_prefill256(ctx, "attn_prefill_ragged", p, d_q, cache, d_out, nullptr, 0, &rs);
    return launch_prefill_impl(ctx, "attn_prefill_ragged", p, d_q, 128, cache, d_out, nullptr, &rs);
}

// Paged caches: the rows between the end of a sequence and the end of the K/V box that holds its last row belong to
// the sequence's last page and travel with the box; the step that has just written the rows before them clears them,
// so that whatever an earlier owner of the page left there cannot reach the output (0 x NaN).
__global__ void zero_page_tail_kernel(KvAddr kv, const uint32_t *tok_start, uint32_t box_rows, uint32_t row_bytes) {
    const uint32_t s = blockIdx.x;
    const uint32_t len = tok_start[s + 1] - tok_start[s];
    const uint32_t end = (len + box_rows - 1) / box_rows * box_rows;
    for (uint32_t row = len; row < end; ++row) {
        uint4 *k = reinterpret_cast<uint4 *>(const_cast<char *>(kv_row_ptr(kv, false, s, row, row_bytes)));
        uint4 *v = reinterpret_cast<uint4 *>(const_cast<char *>(kv_row_ptr(kv, true, s, row, row_bytes)));
        for (uint32_t i = threadIdx.x; i < row_bytes / 16; i += blockDim.x) k[i] = v[i] = make_uint4(0, 0, 0, 0);
    }
}

int launch_prefill_append_ragged(shady_ctx *ctx, const shady_append_params *ap, const shady_prefill_params *p,
                                 const shady_prefill_batch *batch, const void *d_q_proj_full, const void *d_k_proj, const void *d_v_proj,
                                 const uint16_t *d_qk_norm_bf16, const shady_kv_cache *cache, void *d_out, void *d_ws, size_t ws_bytes) {
    SHADY_REQUIRE(ctx, ap && p && d_q_proj_full && d_k_proj && d_v_proj && cache && d_out, SHADY_ERR_BAD_ARG, "attn_prefill_append_ragged: null argument");
    if (const int st = check_prefill_append(ctx, ap, p, true)) return st;
    RaggedSetup rs;
    if (const int st = setup_ragged(ctx, "attn_prefill_append_ragged", p, batch, cache, d_ws, ws_bytes, true, &rs)) return st;
    uint32_t longest = 0;
    for (uint32_t s = 1; s < p->num_seqs; ++s)
        if (batch->h_seq_lens[s] > batch->h_seq_lens[longest]) longest = s;
    const AppendRagged ar{rs.d_tok_start, rs.lay.total_tokens, longest};
    void *extra = (char *)d_ws + rs.lay.extra_off;
    int st;
    if (p->head_dim == 256) {
        shady_append_params ap2 = *ap;
        ap2.q_dtype = p->dtype; ap2.write_k_back = 0;
        st = launch_append_ex(ctx, &ap2, d_q_proj_full, const_cast<void *>(d_k_proj), d_v_proj, extra, nullptr, cache, d_qk_norm_bf16,
                              nullptr, nullptr, nullptr, true, &ar);
    } else {
        st = launch_append_kv_table(ctx, ap, d_k_proj, d_v_proj, cache, d_qk_norm_bf16, reinterpret_cast<float2 *>(extra), &ar);
    }
    if (st) return st;
    if (rs.rg.page_table) {
        KvAddr kv;
        if (const int st2 = fill_kv_addr(ctx, cache, p->num_kv_heads, p->head_dim, "attn_prefill_append_ragged", &kv)) return st2;
        zero_page_tail_kernel<<<p->num_seqs, 128, 0, ctx->stream>>>(kv, rs.d_tok_start, rs.rg.box_rows, p->num_kv_heads * p->head_dim * 2);
        ctx->launches++;
        SHADY_CUDA_OK(ctx, cudaGetLastError());
    }
    if (p->head_dim == 256)
        return launch_prefill256(ctx, "attn_prefill_append_ragged", p, extra, cache, d_out, ap->has_gate ? d_q_proj_full : nullptr, 512, &rs);
    const FusedQ fq{reinterpret_cast<const float2 *>(extra), d_qk_norm_bf16, ap->has_gate, ap->eps};
    return launch_prefill_impl(ctx, "attn_prefill_append_ragged", p, d_q_proj_full, ap->has_gate ? 256u : 128u, cache, d_out, &fq, &rs);
}

}  // namespace shady
