// Shared device/host helpers for the sm_100a attention kernels.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

#include "../../include/shady_attn.h"

// Tuning overrides of the decode launcher, read from the environment once, when the context is created
// (0 = the measured default).  They exist for experiments; nothing on the launch path calls getenv.
struct DecodeKnobs {
    uint32_t variant = 0;       // SHADY_DECODE_VARIANT: {warps, tile slots} configuration
    uint32_t ctas_per_sm = 0;   // SHADY_DECODE_CTAS_PER_SM: spans per SM
    uint32_t kpc = 0;           // SHADY_DECODE_KPC: kv heads per CTA
    uint32_t min_span = 0;      // SHADY_DECODE_MIN_SPAN: smallest span in 16-row blocks
    uint32_t grid_merge = 1;    // SHADY_DECODE_GRID_MERGE=0: merge many-span sequences in a second launch
    uint32_t interleave = 1;    // SHADY_DECODE_INTERLEAVE=0: fixed spans for a single long sequence
    uint32_t pad = ~0u;         // SHADY_DECODE_PAD: line units that a sequence boundary costs a span (unset: from the block size)
    uint32_t early_launch = 1;  // SHADY_DECODE_EARLY_LAUNCH=0: plain stream order between a decode launch and the kernel before it
};

struct shady_ctx {
    int device = 0;
    cudaStream_t stream = nullptr;
    bool owns_stream = false;
    int num_sms = 148;
    uint64_t launches = 0;
    std::string err;
    DecodeKnobs knobs;
    // Bounded device-side waits.  A kernel whose wait runs out latches a code into status_dev (which later waits
    // of the same context poll, so that they give up early) and into status_host, one word of page-locked host
    // memory: shady_synchronize reads it after its single stream sync, and every launcher reads it before it
    // launches, without any device round trip.
    int *status_dev = nullptr;       // device memory, zero while all is well
    int *status_host = nullptr;      // the host word ...
    int *status_host_dev = nullptr;  // ... under the address kernels write it through
    uint32_t wait_grid = 1u << 21;   // polls of the decode grid barrier
    uint32_t wait_peer = 1u << 22;   // polls of a peer's NVLink flag
    uint32_t wait_mbar = 1u << 20;   // polls of an mbarrier in the prefill kernel
    bool rezero_workspace = false;   // a wait ran out: the next decode launch clears its workspace's counters first
    // small host tables (row-block lists, tensor maps of a listed prefill batch) go to the device through this
    // page-locked buffer; stage_done = the last copy out of it
    void *stage = nullptr;
    size_t stage_bytes = 0;
    cudaEvent_t stage_done = nullptr;
};

// What a kernel needs to report (and notice) an expired wait.
struct StatusRef {
    int *dev;    // polled by bounded waits: non-zero = somebody already gave up
    int *host;   // page-locked host word (device-side address)
};
__device__ __forceinline__ void report_timeout(const StatusRef &st, int code) {
    if (atomicCAS(st.dev, 0, code) == 0) {
        *reinterpret_cast<volatile int *>(st.host) = code;
        __threadfence_system();
    }
}
__device__ __forceinline__ bool gave_up(const StatusRef &st) { return *reinterpret_cast<volatile int *>(st.dev) != 0; }

namespace shady {

// ---- status plumbing ------------------------------------------------------------------
int fail(shady_ctx *ctx, int code, const std::string &msg);
// SHADY_ERR_TIMEOUT if an earlier launch of this context gave up a bounded wait and the status has not been
// collected by shady_synchronize yet (launchers call it first: results after such a launch are undefined).
int pending_timeout(shady_ctx *ctx, const char *who);
inline StatusRef status_ref(const shady_ctx *ctx) { return StatusRef{ctx->status_dev, ctx->status_host_dev}; }
#define SHADY_CUDA_OK(ctx, expr)                                                             \
    do {                                                                                     \
        cudaError_t e__ = (expr);                                                            \
        if (e__ != cudaSuccess)                                                              \
            return ::shady::fail(ctx, SHADY_ERR_CUDA,                                        \
                                 std::string(#expr) + ": " + cudaGetErrorString(e__));       \
    } while (0)
#define SHADY_REQUIRE(ctx, cond, code, msg)                       \
    do {                                                          \
        if (!(cond)) return ::shady::fail(ctx, code, msg);        \
    } while (0)

__host__ __device__ inline bool is_f8(uint32_t dt) { return dt == SHADY_F8E4M3 || dt == SHADY_F8E5M2; }
__host__ __device__ inline size_t dtype_size(uint32_t dt) { return dt == SHADY_F32 ? 4 : (is_f8(dt) ? 1 : 2); }

// ---- dtype conversion -------------------------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_fp8_e4m3>(__nv_fp8_e4m3 v) { return float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_fp8_e5m2>(__nv_fp8_e5m2 v) { return float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
// round to nearest even, saturating at the largest finite e4m3 value (448); callers divide by the cache scale first
template <> __device__ __forceinline__ __nv_fp8_e4m3 from_f32<__nv_fp8_e4m3>(float v) { return __nv_fp8_e4m3(v); }
template <> __device__ __forceinline__ __nv_fp8_e5m2 from_f32<__nv_fp8_e5m2>(float v) { return __nv_fp8_e5m2(v); }

// Load / store one element of a buffer whose dtype is only known at run time.
__device__ __forceinline__ float load_as_f32(const void *p, size_t i, uint32_t dt) {
    if (dt == SHADY_F32) return reinterpret_cast<const float *>(p)[i];
    if (dt == SHADY_F16) return __half2float(reinterpret_cast<const __half *>(p)[i]);
    if (dt == SHADY_F8E4M3) return float(reinterpret_cast<const __nv_fp8_e4m3 *>(p)[i]);
    if (dt == SHADY_F8E5M2) return float(reinterpret_cast<const __nv_fp8_e5m2 *>(p)[i]);
    return __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(p)[i]);
}
__device__ __forceinline__ void store_from_f32(void *p, size_t i, uint32_t dt, float v) {
    if (dt == SHADY_F32) reinterpret_cast<float *>(p)[i] = v;
    else if (dt == SHADY_F16) reinterpret_cast<__half *>(p)[i] = __float2half_rn(v);
    else if (dt == SHADY_F8E4M3) reinterpret_cast<__nv_fp8_e4m3 *>(p)[i] = __nv_fp8_e4m3(v);
    else if (dt == SHADY_F8E5M2) reinterpret_cast<__nv_fp8_e5m2 *>(p)[i] = __nv_fp8_e5m2(v);
    else reinterpret_cast<__nv_bfloat16 *>(p)[i] = __float2bfloat16_rn(v);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

__device__ __forceinline__ float sigmoidf_ref(float g) { return 1.0f / (1.0f + expf(-g)); }

// Resolve the base pointer of sequence s in a KV cache (see shady_kv_cache).
struct KvAddr {
    const char *k_base;
    const char *v_base;
    unsigned long long seq_stride_bytes;
    const void *const *k_ptrs;
    const void *const *v_ptrs;
    // paged cache: k_base / v_base are page pools, page_table [num_seqs][max_pages], page_bytes = one page of K (or V)
    const uint32_t *page_table;
    unsigned long long page_bytes;
    uint32_t page_rows, max_pages;
    float k_scale, v_scale;   // 8-bit caches: value = stored * scale (1 for the other dtypes)
};
__device__ __forceinline__ const char *kv_seq_ptr(const char *base, const void *const *ptrs,
                                                  unsigned long long stride_bytes, uint32_t s) {
    return ptrs ? reinterpret_cast<const char *>(ptrs[s]) : base + stride_bytes * s;
}
// Address of cache row `pos` (all kv heads, row_bytes = nkv * hd * element size) of sequence s, paged or not.
__device__ __forceinline__ const char *kv_row_ptr(const KvAddr &kv, bool want_v, uint32_t s, uint32_t pos, size_t row_bytes) {
    if (kv.page_table) {
        const uint32_t pg = kv.page_table[(size_t)s * kv.max_pages + pos / kv.page_rows];
        return (want_v ? kv.v_base : kv.k_base) + (size_t)pg * kv.page_bytes + (size_t)(pos % kv.page_rows) * row_bytes;
    }
    return kv_seq_ptr(want_v ? kv.v_base : kv.k_base, want_v ? kv.v_ptrs : kv.k_ptrs, kv.seq_stride_bytes, s) +
           (size_t)pos * row_bytes;
}
// How the append pass finds a token's sequence when the batch is a list of prompts of different lengths, packed
// token-major (prefill of a listed batch).
struct AppendRagged {
    const uint32_t *d_tok_start;   // [num_seqs + 1] first packed token of every sequence
    uint32_t total_tokens;
    uint32_t table_seq;            // the sequence whose tokens write the cos/sin table (the longest one)
};
// Checks a caller's cache description and turns it into the device-side form (defined in api.cu).
int fill_kv_addr(shady_ctx *ctx, const shady_kv_cache *cache, uint32_t nkv, uint32_t hd, const char *who, KvAddr *out);

}  // namespace shady
