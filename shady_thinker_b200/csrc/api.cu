// extern "C" surface of libshady_attn.so: context, buffers and op entry points declared in
// include/shady_attn.h.  No torch types, no exceptions across the boundary.
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include "common.cuh"

namespace shady {

static thread_local std::string g_create_error;

int fail(shady_ctx *ctx, int code, const std::string &msg) {
    if (ctx) ctx->err = msg;
    else g_create_error = msg;
    return code;
}

int pending_timeout(shady_ctx *ctx, const char *who) {
    if (ctx->status_host && *reinterpret_cast<volatile int *>(ctx->status_host))
        return fail(ctx, SHADY_ERR_TIMEOUT, std::string(who) + ": an earlier launch on this context gave up a bounded wait; call "
                                            "shady_synchronize to collect the status before launching again");
    return SHADY_OK;
}

// Text of a wait code: 1..16 = waits of the prefill kernels (mbarriers, shared-memory handshakes), 17 = the bulk copies of the staged
// append pass, 90 = the decode grid barrier, 100 + r = the NVLink flag of rank r.
std::string timeout_message(int code) {
    if (code >= 100)
        return "combine_p2p: the flag of rank " + std::to_string(code - 100) + " did not arrive in time";
    if (code == 90)
        return "decode: the grid barrier before the record merge ran out; the workspace counters are cleared again before the next launch";
    if (code == 17) return "kv_append: a token's bulk copies into shared memory did not land in time";
    return "attn_prefill: a device-side wait expired (code " + std::to_string(code) + ")";
}

static uint32_t env_u32(const char *name, uint32_t dflt) {
    const char *v = getenv(name);
    return v && *v ? (uint32_t)strtoul(v, nullptr, 10) : dflt;
}

int fill_kv_addr(shady_ctx *ctx, const shady_kv_cache *cache, uint32_t nkv, uint32_t hd, const char *who, KvAddr *out) {
    const std::string w(who);
    SHADY_REQUIRE(ctx, cache->dtype <= SHADY_F8E5M2, SHADY_ERR_BAD_ARG, w + ": bad cache dtype");
    KvAddr kv{};
    kv.k_scale = kv.v_scale = 1.0f;
    if (is_f8(cache->dtype)) {
        SHADY_REQUIRE(ctx, cache->k_scale >= 0.f && cache->v_scale >= 0.f && isfinite(cache->k_scale) && isfinite(cache->v_scale),
                      SHADY_ERR_BAD_ARG, w + ": cache scales must be finite and not negative");
        if (cache->k_scale > 0.f) kv.k_scale = cache->k_scale;
        if (cache->v_scale > 0.f) kv.v_scale = cache->v_scale;
    }
    kv.k_base = (const char *)cache->d_k_base; kv.v_base = (const char *)cache->d_v_base;
    kv.seq_stride_bytes = cache->seq_stride * dtype_size(cache->dtype);
    kv.k_ptrs = cache->d_k_ptrs; kv.v_ptrs = cache->d_v_ptrs;
    if (cache->d_page_table) {
        SHADY_REQUIRE(ctx, cache->d_k_base && cache->d_v_base && !cache->d_k_ptrs && !cache->d_v_ptrs, SHADY_ERR_BAD_ARG,
                      w + ": a paged cache takes the two pool bases and no pointer arrays");
        SHADY_REQUIRE(ctx, cache->page_rows && cache->page_rows % 16 == 0 && cache->max_pages_per_seq, SHADY_ERR_BAD_ARG,
                      w + ": page_rows must be a positive multiple of 16 and max_pages_per_seq positive");
        SHADY_REQUIRE(ctx, cache->dtype != SHADY_F32, SHADY_ERR_UNSUPPORTED, w + ": paged caches are 16-bit or 8-bit");
        kv.page_table = cache->d_page_table;
        kv.page_rows = cache->page_rows; kv.max_pages = cache->max_pages_per_seq;
        kv.page_bytes = (unsigned long long)cache->page_rows * nkv * hd * dtype_size(cache->dtype);
    } else {
        SHADY_REQUIRE(ctx, (cache->d_k_ptrs && cache->d_v_ptrs) || (cache->d_k_base && cache->d_v_base), SHADY_ERR_BAD_ARG,
                      w + ": cache needs base pointers or pointer arrays");
    }
    *out = kv;
    return SHADY_OK;
}

// launchers implemented in the kernel translation units
size_t decode_workspace_bytes(const shady_decode_params *p);
int init_decode_workspace(shady_ctx *, const shady_decode_params *, void *, size_t);
int launch_decode(shady_ctx *, const shady_decode_params *, const void *, const shady_kv_cache *, const uint32_t *,
                  const uint32_t *, void *, float *, const float *, void *, size_t, float *, float *, const struct FusedAppendIn *,
                  const struct ShardExchangeIn *);
struct FusedAppendIn {
    const shady_append_params *ap;
    const void *q_full, *k_proj, *v_proj;
    const uint16_t *norm_w;
};
struct ShardExchangeIn {
    uint32_t world, rank, epoch, out_dtype;
    void *const *d_peer_table;
    void *d_out;
    const float *d_gate;
};
int launch_decode_static(shady_ctx *, const shady_decode_params *, const void *, const shady_kv_cache *, const uint32_t *,
                         const uint32_t *, void *, float *, const float *);
int launch_reduce(shady_ctx *, uint32_t, uint32_t, uint32_t, uint64_t, uint64_t, const float *, void *, uint32_t,
                  const float *);
int launch_sigmoid_mul(shady_ctx *, float *, const float *, uint32_t);
int launch_append(shady_ctx *, const shady_append_params *, const void *, void *, const void *, void *, float *,
                  const shady_kv_cache *, const uint16_t *, const uint32_t *, const uint32_t *, const uint32_t *);
int launch_prefill(shady_ctx *, const shady_prefill_params *, const void *, const shady_kv_cache *, void *);
size_t prefill_workspace_bytes(const shady_prefill_params *p);
size_t prefill_ragged_workspace_bytes(const shady_prefill_params *p, const uint32_t *h_seq_lens, bool with_append);
int launch_prefill_ragged(shady_ctx *, const shady_prefill_params *, const shady_prefill_batch *, const void *, const shady_kv_cache *,
                          void *, void *, size_t);
int launch_prefill_append_ragged(shady_ctx *, const shady_append_params *, const shady_prefill_params *, const shady_prefill_batch *,
                                 const void *, const void *, const void *, const uint16_t *, const shady_kv_cache *, void *, void *,
                                 size_t);
int launch_gptq_matvec(shady_ctx *, const shady_gptq_weight *, const float *, float *, uint32_t);
int launch_qkv_proj_append(shady_ctx *, const shady_append_params *, const shady_gptq_weight *, const shady_gptq_weight *,
                           const shady_gptq_weight *, const float *, void *, float *, const shady_kv_cache *, const uint16_t *,
                           const uint32_t *, const uint32_t *, const uint32_t *);
int launch_prefill_append(shady_ctx *, const shady_append_params *, const shady_prefill_params *, const void *, const void *,
                          const void *, const uint16_t *, const shady_kv_cache *, void *, void *, size_t);
unsigned long long p2p_buffer_bytes(uint32_t world, uint32_t nh, uint32_t hd);
int launch_combine_p2p(shady_ctx *, uint32_t, uint32_t, uint32_t, uint32_t, uint32_t, void *const *, const float *, void *,
                       uint32_t, const float *);

// ---- counter-based N(0,1): the device twin of oracle_randn_at ---------------------------
__host__ __device__ inline unsigned long long mix64(unsigned long long z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
__global__ void fill_randn_kernel(void *dst, unsigned long long n, uint32_t dtype, unsigned long long key,
                                  unsigned long long first_idx) {
    const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
    for (unsigned long long i = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const unsigned long long r = mix64(key + first_idx + i);
        const double u1 = ((double)((r >> 40) & 0xFFFFFFull) + 1.0) * (1.0 / 16777216.0);
        const double u2 = (double)((r >> 8) & 0xFFFFFFull) * (1.0 / 16777216.0);
        const float v = (float)(sqrt(-2.0 * log(u1)) * cos(6.283185307179586476925 * u2));
        store_from_f32(dst, i, dtype, v);
    }
}

}  // namespace shady

using namespace shady;

extern "C" {

int shady_ctx_create(int device, void *stream, shady_ctx **out) {
    if (!out) return fail(nullptr, SHADY_ERR_BAD_ARG, "ctx_create: null out pointer");
    *out = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess) return fail(nullptr, SHADY_ERR_CUDA, std::string("cudaGetDeviceCount: ") + cudaGetErrorString(e));
    if (device < 0 || device >= count) return fail(nullptr, SHADY_ERR_BAD_ARG, "ctx_create: no such CUDA device");
    if ((e = cudaSetDevice(device)) != cudaSuccess)
        return fail(nullptr, SHADY_ERR_CUDA, std::string("cudaSetDevice: ") + cudaGetErrorString(e));
    cudaDeviceProp prop{};
    if ((e = cudaGetDeviceProperties(&prop, device)) != cudaSuccess)
        return fail(nullptr, SHADY_ERR_CUDA, std::string("cudaGetDeviceProperties: ") + cudaGetErrorString(e));
    if (prop.major != 10)
        return fail(nullptr, SHADY_ERR_UNSUPPORTED, "ctx_create: this library is built for sm_100a (B200) only");
    shady_ctx *c = new (std::nothrow) shady_ctx();
    if (!c) return fail(nullptr, SHADY_ERR_BAD_ARG, "ctx_create: out of host memory");
    c->device = device;
    c->num_sms = prop.multiProcessorCount;
    if (stream) {
        c->stream = reinterpret_cast<cudaStream_t>(stream);
    } else {
        if ((e = cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking)) != cudaSuccess) {
            delete c;
            return fail(nullptr, SHADY_ERR_CUDA, std::string("cudaStreamCreate: ") + cudaGetErrorString(e));
        }
        c->owns_stream = true;
    }
    // status words of the bounded waits: 4 bytes of device memory and one page-locked host word the kernels can write
    auto drop = [&](const char *what, cudaError_t err) {
        if (c->status_dev) cudaFree(c->status_dev);
        if (c->status_host) cudaFreeHost(c->status_host);
        if (c->owns_stream) cudaStreamDestroy(c->stream);
        delete c;
        return fail(nullptr, SHADY_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(err));
    };
    if ((e = cudaMalloc(reinterpret_cast<void **>(&c->status_dev), 256)) != cudaSuccess) return drop("cudaMalloc(status word)", e);
    if ((e = cudaMemset(c->status_dev, 0, 256)) != cudaSuccess) return drop("cudaMemset(status word)", e);
    if ((e = cudaHostAlloc(reinterpret_cast<void **>(&c->status_host), 64, cudaHostAllocMapped)) != cudaSuccess)
        return drop("cudaHostAlloc(status word)", e);
    *c->status_host = 0;
    if ((e = cudaHostGetDevicePointer(reinterpret_cast<void **>(&c->status_host_dev), c->status_host, 0)) != cudaSuccess)
        return drop("cudaHostGetDevicePointer(status word)", e);
    c->knobs.variant = env_u32("SHADY_DECODE_VARIANT", 0);
    c->knobs.ctas_per_sm = env_u32("SHADY_DECODE_CTAS_PER_SM", 0);
    c->knobs.kpc = env_u32("SHADY_DECODE_KPC", 0);
    c->knobs.min_span = env_u32("SHADY_DECODE_MIN_SPAN", 0);
    c->knobs.grid_merge = env_u32("SHADY_DECODE_GRID_MERGE", 1);
    c->knobs.interleave = env_u32("SHADY_DECODE_INTERLEAVE", 1);
    c->knobs.pad = env_u32("SHADY_DECODE_PAD", ~0u);
    c->knobs.early_launch = env_u32("SHADY_DECODE_EARLY_LAUNCH", 1);
    *out = c;
    return SHADY_OK;
}

int shady_ctx_destroy(shady_ctx *ctx) {
    if (!ctx) return SHADY_ERR_BAD_ARG;
    if (ctx->owns_stream) {
        cudaSetDevice(ctx->device);
        cudaStreamSynchronize(ctx->stream);
        cudaStreamDestroy(ctx->stream);
    } else {
        cudaSetDevice(ctx->device);
    }
    if (ctx->status_dev) cudaFree(ctx->status_dev);
    if (ctx->status_host) cudaFreeHost(ctx->status_host);
    if (ctx->stage_done) cudaEventDestroy(ctx->stage_done);
    if (ctx->stage) cudaFreeHost(ctx->stage);
    delete ctx;
    return SHADY_OK;
}

int shady_ctx_set_wait_limits(shady_ctx *ctx, uint32_t grid_polls, uint32_t peer_polls, uint32_t mbarrier_polls) {
    if (!ctx) return SHADY_ERR_BAD_ARG;
    if (grid_polls) ctx->wait_grid = grid_polls;
    if (peer_polls) ctx->wait_peer = peer_polls;
    if (mbarrier_polls) ctx->wait_mbar = mbarrier_polls;
    return SHADY_OK;
}

const char *shady_last_error(const shady_ctx *ctx) { return ctx ? ctx->err.c_str() : g_create_error.c_str(); }
void *shady_ctx_stream(const shady_ctx *ctx) { return ctx ? (void *)ctx->stream : nullptr; }
uint64_t shady_ctx_launch_count(const shady_ctx *ctx) { return ctx ? ctx->launches : 0; }

#define CTX_ENTER(ctx)                                   \
    if (!(ctx)) return SHADY_ERR_BAD_ARG;                \
    SHADY_CUDA_OK(ctx, cudaSetDevice((ctx)->device))

int shady_buffer_create(shady_ctx *ctx, size_t bytes, void **d_out) {
    CTX_ENTER(ctx);
    SHADY_REQUIRE(ctx, d_out, SHADY_ERR_BAD_ARG, "buffer_create: null out pointer");
    *d_out = nullptr;
    const size_t aligned = (bytes + 3) & ~(size_t)3;  // gpu.rs:86
    SHADY_CUDA_OK(ctx, cudaMalloc(d_out, aligned ? aligned : 4));
    return SHADY_OK;
}
int shady_buffer_free(shady_ctx *ctx, void *d_buf) {
    CTX_ENTER(ctx);
    if (d_buf) SHADY_CUDA_OK(ctx, cudaFree(d_buf));
    return SHADY_OK;
}
int shady_buffer_write(shady_ctx *ctx, void *d_buf, size_t offset, const void *src, size_t bytes) {
    CTX_ENTER(ctx);
    SHADY_REQUIRE(ctx, d_buf && (src || !bytes), SHADY_ERR_BAD_ARG, "buffer_write: null argument");
    if (bytes) SHADY_CUDA_OK(ctx, cudaMemcpyAsync((char *)d_buf + offset, src, bytes, cudaMemcpyHostToDevice, ctx->stream));
    return SHADY_OK;
}
int shady_buffer_read(shady_ctx *ctx, const void *d_buf, size_t offset, void *dst, size_t bytes) {
    CTX_ENTER(ctx);
    SHADY_REQUIRE(ctx, d_buf && (dst || !bytes), SHADY_ERR_BAD_ARG, "buffer_read: null argument");
    if (bytes) SHADY_CUDA_OK(ctx, cudaMemcpyAsync(dst, (const char *)d_buf + offset, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    SHADY_CUDA_OK(ctx, cudaStreamSynchronize(ctx->stream));
    return SHADY_OK;
}
int shady_buffer_copy(shady_ctx *ctx, const void *d_src, void *d_dst, size_t bytes) {
    CTX_ENTER(ctx);
    SHADY_REQUIRE(ctx, d_src && d_dst, SHADY_ERR_BAD_ARG, "buffer_copy: null argument");
    if (bytes) SHADY_CUDA_OK(ctx, cudaMemcpyAsync(d_dst, d_src, bytes, cudaMemcpyDeviceToDevice, ctx->stream));
    return SHADY_OK;
}
int shady_host_device_ptr(shady_ctx *ctx, const void *host_ptr, void **d_ptr) {
    CTX_ENTER(ctx);
    SHADY_REQUIRE(ctx, host_ptr && d_ptr, SHADY_ERR_BAD_ARG, "host_device_ptr: null argument");
    *d_ptr = nullptr;
    cudaPointerAttributes at{};
    SHADY_CUDA_OK(ctx, cudaPointerGetAttributes(&at, host_ptr));
    SHADY_REQUIRE(ctx, at.type == cudaMemoryTypeHost && at.devicePointer, SHADY_ERR_BAD_ARG,
                  "host_device_ptr: not page-locked host memory the device can address");
    *d_ptr = at.devicePointer;
    return SHADY_OK;
}
int shady_flush(shady_ctx *ctx) {
    CTX_ENTER(ctx);
    const cudaError_t e = cudaStreamQuery(ctx->stream);
    if (e != cudaSuccess && e != cudaErrorNotReady)
        return fail(ctx, SHADY_ERR_CUDA, std::string("flush: ") + cudaGetErrorString(e));
    return SHADY_OK;
}
int shady_synchronize(shady_ctx *ctx) {
    CTX_ENTER(ctx);
    SHADY_CUDA_OK(ctx, cudaStreamSynchronize(ctx->stream));
    // a kernel whose bounded wait ran out wrote its code into the page-locked status word before it ended
    const int code = *reinterpret_cast<volatile int *>(ctx->status_host);
    if (code) {
        *ctx->status_host = 0;
        SHADY_CUDA_OK(ctx, cudaMemsetAsync(ctx->status_dev, 0, sizeof(int), ctx->stream));
        SHADY_CUDA_OK(ctx, cudaStreamSynchronize(ctx->stream));
        ctx->rezero_workspace = true;
        return fail(ctx, SHADY_ERR_TIMEOUT, timeout_message(code));
    }
    return SHADY_OK;
}

int shady_kv_append_rope(shady_ctx *ctx, const shady_append_params *p, const void *d_q_proj_full, void *d_k_proj,
                         const void *d_v_proj, void *d_q_out, float *d_q_gate, const shady_kv_cache *cache,
                         const uint16_t *d_qk_norm_bf16, const uint32_t *d_pos_start, const uint32_t *d_pos_h,
                         const uint32_t *d_pos_w) {
    CTX_ENTER(ctx);
    return launch_append(ctx, p, d_q_proj_full, d_k_proj, d_v_proj, d_q_out, d_q_gate, cache, d_qk_norm_bf16,
                         d_pos_start, d_pos_h, d_pos_w);
}

int shady_decode_workspace_size(const shady_decode_params *p, size_t *bytes) {
    if (!p || !bytes) return SHADY_ERR_BAD_ARG;
    *bytes = decode_workspace_bytes(p);
    return SHADY_OK;
}

int shady_decode_workspace_init(shady_ctx *ctx, const shady_decode_params *p, void *d_workspace, size_t workspace_bytes) {
    CTX_ENTER(ctx);
    return init_decode_workspace(ctx, p, d_workspace, workspace_bytes);
}

int shady_attn_decode(shady_ctx *ctx, const shady_decode_params *p, const void *d_q, const shady_kv_cache *cache,
                      const uint32_t *d_seq_lens, const uint32_t *seq_lens_host, void *d_out, float *d_lse,
                      const float *d_gate, void *d_workspace, size_t workspace_bytes) {
    CTX_ENTER(ctx);
    return launch_decode(ctx, p, d_q, cache, d_seq_lens, seq_lens_host, d_out, d_lse, d_gate, d_workspace,
                         workspace_bytes, nullptr, nullptr, nullptr, nullptr);
}

int shady_attn_decode_static(shady_ctx *ctx, const shady_decode_params *p, const void *d_q, const shady_kv_cache *cache,
                             const uint32_t *d_seq_lens, const uint32_t *seq_lens_host, void *d_out, float *d_lse,
                             const float *d_gate) {
    CTX_ENTER(ctx);
    return launch_decode_static(ctx, p, d_q, cache, d_seq_lens, seq_lens_host, d_out, d_lse, d_gate);
}

int shady_attn_decode_append(shady_ctx *ctx, const shady_append_params *ap, const shady_decode_params *p,
                             const void *d_q_proj_full, const void *d_k_proj, const void *d_v_proj,
                             const uint16_t *d_qk_norm_bf16, const shady_kv_cache *cache, const uint32_t *d_seq_lens,
                             const uint32_t *seq_lens_host, void *d_out, float *d_lse, void *d_workspace,
                             size_t workspace_bytes) {
    CTX_ENTER(ctx);
    FusedAppendIn fa{ap, d_q_proj_full, d_k_proj, d_v_proj, d_qk_norm_bf16};
    return launch_decode(ctx, p, nullptr, cache, d_seq_lens, seq_lens_host, d_out, d_lse, nullptr, d_workspace,
                         workspace_bytes, nullptr, nullptr, &fa, nullptr);
}

int shady_attn_decode_shard(shady_ctx *ctx, const shady_decode_params *p, const void *d_q, const shady_kv_cache *cache,
                            const uint32_t *d_seq_lens, const uint32_t *seq_lens_host, float *d_records, void *d_workspace,
                            size_t workspace_bytes) {
    CTX_ENTER(ctx);
    SHADY_REQUIRE(ctx, d_records, SHADY_ERR_BAD_ARG, "decode_shard: null output");
    return launch_decode(ctx, p, d_q, cache, d_seq_lens, seq_lens_host, nullptr, nullptr, nullptr, d_workspace,
                         workspace_bytes, nullptr, d_records, nullptr, nullptr);
}

int shady_attn_decode_shard_p2p(shady_ctx *ctx, const shady_decode_params *p, const void *d_q, const shady_kv_cache *cache,
                                const uint32_t *d_seq_lens, const uint32_t *seq_lens_host, uint32_t world, uint32_t rank,
                                uint32_t epoch, void *const *d_peer_table, float *d_records, void *d_out, uint32_t out_dtype,
                                const float *d_gate, void *d_workspace, size_t workspace_bytes) {
    CTX_ENTER(ctx);
    SHADY_REQUIRE(ctx, d_records && d_out && d_peer_table, SHADY_ERR_BAD_ARG, "decode_shard_p2p: null argument");
    const ShardExchangeIn px{world, rank, epoch, out_dtype, d_peer_table, d_out, d_gate};
    return launch_decode(ctx, p, d_q, cache, d_seq_lens, seq_lens_host, nullptr, nullptr, nullptr, d_workspace,
                         workspace_bytes, nullptr, d_records, nullptr, &px);
}

int shady_attn_decode_partials(shady_ctx *ctx, const shady_decode_params *p, const void *d_q,
                               const shady_kv_cache *cache, const uint32_t *d_seq_lens, float *d_partials) {
    CTX_ENTER(ctx);
    SHADY_REQUIRE(ctx, d_partials, SHADY_ERR_BAD_ARG, "decode_partials: null output");
    return launch_decode(ctx, p, d_q, cache, d_seq_lens, nullptr, nullptr, nullptr, nullptr, nullptr, 0, d_partials, nullptr, nullptr, nullptr);
}

int shady_attn_reduce(shady_ctx *ctx, uint32_t head_dim, uint32_t num_splits, uint32_t num_heads, uint64_t split_stride,
                      uint64_t head_stride, const float *d_partials, void *d_out, uint32_t out_dtype,
                      const float *d_gate) {
    CTX_ENTER(ctx);
    return launch_reduce(ctx, head_dim, num_splits, num_heads, split_stride, head_stride, d_partials, d_out, out_dtype,
                         d_gate);
}

int shady_attn_prefill(shady_ctx *ctx, const shady_prefill_params *p, const void *d_q, const shady_kv_cache *cache,
                       void *d_out) {
    CTX_ENTER(ctx);
    return launch_prefill(ctx, p, d_q, cache, d_out);
}

int shady_prefill_workspace_size(const shady_prefill_params *p, size_t *bytes) {
    if (!p || !bytes) return SHADY_ERR_BAD_ARG;
    *bytes = prefill_workspace_bytes(p);
    return SHADY_OK;
}

int shady_attn_prefill_append(shady_ctx *ctx, const shady_append_params *ap, const shady_prefill_params *p,
                              const void *d_q_proj_full, const void *d_k_proj, const void *d_v_proj,
                              const uint16_t *d_qk_norm_bf16, const shady_kv_cache *cache, void *d_out, void *d_workspace,
                              size_t workspace_bytes) {
    CTX_ENTER(ctx);
    return launch_prefill_append(ctx, ap, p, d_q_proj_full, d_k_proj, d_v_proj, d_qk_norm_bf16, cache, d_out, d_workspace,
                                 workspace_bytes);
}

int shady_prefill_ragged_workspace_size(const shady_prefill_params *p, const uint32_t *h_seq_lens, int with_append, size_t *bytes) {
    if (!p || !h_seq_lens || !bytes || !p->num_seqs) return SHADY_ERR_BAD_ARG;
    *bytes = prefill_ragged_workspace_bytes(p, h_seq_lens, with_append != 0);
    return SHADY_OK;
}

int shady_attn_prefill_ragged(shady_ctx *ctx, const shady_prefill_params *p, const shady_prefill_batch *batch, const void *d_q,
                              const shady_kv_cache *cache, void *d_out, void *d_workspace, size_t workspace_bytes) {
    CTX_ENTER(ctx);
    SHADY_REQUIRE(ctx, d_q && d_out, SHADY_ERR_BAD_ARG, "attn_prefill_ragged: null argument");
    return launch_prefill_ragged(ctx, p, batch, d_q, cache, d_out, d_workspace, workspace_bytes);
}

int shady_attn_prefill_append_ragged(shady_ctx *ctx, const shady_append_params *ap, const shady_prefill_params *p,
                                     const shady_prefill_batch *batch, const void *d_q_proj_full, const void *d_k_proj,
                                     const void *d_v_proj, const uint16_t *d_qk_norm_bf16, const shady_kv_cache *cache, void *d_out,
                                     void *d_workspace, size_t workspace_bytes) {
    CTX_ENTER(ctx);
    return launch_prefill_append_ragged(ctx, ap, p, batch, d_q_proj_full, d_k_proj, d_v_proj, d_qk_norm_bf16, cache, d_out,
                                        d_workspace, workspace_bytes);
}

int shady_ipc_export(shady_ctx *ctx, void *d_buf, unsigned char handle[64]) {
    CTX_ENTER(ctx);
    SHADY_REQUIRE(ctx, d_buf && handle, SHADY_ERR_BAD_ARG, "ipc_export: null argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    cudaIpcMemHandle_t h;
    SHADY_CUDA_OK(ctx, cudaIpcGetMemHandle(&h, d_buf));
    memcpy(handle, &h, 64);
    return SHADY_OK;
}
int shady_ipc_open(shady_ctx *ctx, const unsigned char handle[64], void **d_peer) {
    CTX_ENTER(ctx);
    SHADY_REQUIRE(ctx, handle && d_peer, SHADY_ERR_BAD_ARG, "ipc_open: null argument");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, 64);
    *d_peer = nullptr;
    SHADY_CUDA_OK(ctx, cudaIpcOpenMemHandle(d_peer, h, cudaIpcMemLazyEnablePeerAccess));
    return SHADY_OK;
}
int shady_ipc_close(shady_ctx *ctx, void *d_peer) {
    CTX_ENTER(ctx);
    if (d_peer) SHADY_CUDA_OK(ctx, cudaIpcCloseMemHandle(d_peer));
    return SHADY_OK;
}
int shady_combine_p2p_buffer_size(uint32_t world, uint32_t num_heads, uint32_t head_dim, size_t *bytes) {
    if (!bytes || !world || !num_heads || !head_dim) return SHADY_ERR_BAD_ARG;
    *bytes = (size_t)p2p_buffer_bytes(world, num_heads, head_dim);
    return SHADY_OK;
}
int shady_attn_combine_p2p(shady_ctx *ctx, uint32_t world, uint32_t rank, uint32_t num_heads, uint32_t head_dim,
                           uint32_t epoch, void *const *d_peer_table, const float *d_records, void *d_out,
                           uint32_t out_dtype, const float *d_gate) {
    CTX_ENTER(ctx);
    return launch_combine_p2p(ctx, world, rank, num_heads, head_dim, epoch, d_peer_table, d_records, d_out, out_dtype, d_gate);
}

int shady_gptq_matvec(shady_ctx *ctx, const shady_gptq_weight *w, const float *d_x, float *d_y, uint32_t num_vecs) {
    CTX_ENTER(ctx);
    return launch_gptq_matvec(ctx, w, d_x, d_y, num_vecs);
}

int shady_qkv_proj_append(shady_ctx *ctx, const shady_append_params *p, const shady_gptq_weight *wq, const shady_gptq_weight *wk,
                          const shady_gptq_weight *wv, const float *d_x, void *d_q_out, float *d_q_gate,
                          const shady_kv_cache *cache, const uint16_t *d_qk_norm_bf16, const uint32_t *d_pos_start,
                          const uint32_t *d_pos_h, const uint32_t *d_pos_w) {
    CTX_ENTER(ctx);
    return launch_qkv_proj_append(ctx, p, wq, wk, wv, d_x, d_q_out, d_q_gate, cache, d_qk_norm_bf16, d_pos_start, d_pos_h,
                                  d_pos_w);
}

int shady_sigmoid_mul(shady_ctx *ctx, float *d_x, const float *d_gate, uint32_t n) {
    CTX_ENTER(ctx);
    return launch_sigmoid_mul(ctx, d_x, d_gate, n);
}

int shady_fill_randn(shady_ctx *ctx, void *d_dst, uint64_t n, uint32_t dtype, uint64_t seed, uint64_t tensor_id,
                     uint64_t first_idx) {
    CTX_ENTER(ctx);
    SHADY_REQUIRE(ctx, d_dst || !n, SHADY_ERR_BAD_ARG, "fill_randn: null destination");
    SHADY_REQUIRE(ctx, dtype <= SHADY_F8E5M2, SHADY_ERR_BAD_ARG, "fill_randn: bad dtype");
    if (!n) return SHADY_OK;
    const unsigned long long key = mix64(seed ^ (tensor_id * 0xD1B54A32D192ED03ull));
    const unsigned long long want = (n + 255) / 256;
    const unsigned blocks = (unsigned)(want < (unsigned long long)ctx->num_sms * 16 ? want : (unsigned long long)ctx->num_sms * 16);
    fill_randn_kernel<<<blocks, 256, 0, ctx->stream>>>(d_dst, n, dtype, key, first_idx);
    ctx->launches++;
    SHADY_CUDA_OK(ctx, cudaGetLastError());
    return SHADY_OK;
}

}  // extern "C"
