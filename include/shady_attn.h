/*
 * shady_attn.h — C ABI of the B200 (sm_100a) attention hot path of shady-thinker.
 *
 * Scope: KV-cache append with Q/K RMSNorm + (m)RoPE, single-token GQA decode attention over
 * the KV cache (split-KV + log-sum-exp merge), causal prefill attention, and the sigmoid
 * output gate that directly follows.  These are the entry points a CUDA backend of the
 * reference's `GpuContext` (src/gpu.rs) binds for the three private `Model` helpers
 * `fused_split_qknorm_kvstore`, `gqa_attention` and `sigmoid_mul_gate`
 * (src/model.rs:486-593).  Each declaration cites the reference interface it replaces.
 *
 * Conventions
 *  - Every function returns an int status (SHADY_OK == 0).  Nothing aborts or throws
 *    across this boundary; `shady_last_error` gives the message of the last failure on a
 *    context.  (The reference panics instead: gpu.rs:43,68,271.)
 *  - All launches are asynchronous on the context's stream and stream-ordered, which gives
 *    the pass-to-pass ordering the reference gets from one compute pass per dispatch
 *    (gpu.rs:223-231).  Parameters travel by value, so the reference's "flush before
 *    overwriting the shared uniform" (model.rs:348-353) has no counterpart.
 *  - The caller owns every buffer.  Ops allocate nothing; scratch memory is an explicit
 *    workspace argument whose size `shady_decode_workspace_size` reports.
 *  - A context is not thread-safe: one context per host thread per device.
 *  - Pointers named `d_*` or documented "device" are device pointers; everything else is
 *    host memory.
 */
#ifndef SHADY_ATTN_H
#define SHADY_ATTN_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ---------------------------------------------------------------- */
#define SHADY_OK 0
#define SHADY_ERR_BAD_ARG 1      /* null pointer, zero size, inconsistent parameters        */
#define SHADY_ERR_UNSUPPORTED 2  /* shape/dtype outside what the kernels cover (hd > 256 …) */
#define SHADY_ERR_CUDA 3         /* a CUDA runtime call failed; see shady_last_error        */
#define SHADY_ERR_WORKSPACE 4    /* workspace missing or too small                          */
#define SHADY_ERR_TIMEOUT 5      /* a bounded device-side wait gave up                      */

/* ---- storage dtypes ----------------------------------------------------------------- */
#define SHADY_F32 0
#define SHADY_F16 1
#define SHADY_BF16 2
#define SHADY_F8E4M3 3   /* KV cache only: 8-bit e4m3 (4 exponent bits, 3 mantissa bits, no infinities) */
#define SHADY_F8E5M2 4   /* KV cache only: 8-bit e5m2 (5 exponent bits, 2 mantissa bits: the top byte of an f16) */

typedef struct shady_ctx shady_ctx;

/* ===================================================================================== */
/* Context and buffers — replaces GpuContext (src/gpu.rs:7-297)                          */
/* ===================================================================================== */

/* GpuContext::new (gpu.rs:17).  `device` is the CUDA ordinal.  `stream` may be NULL (the
 * context creates its own non-blocking stream) or an existing cudaStream_t, which is the
 * counterpart of GpuContext::from_device_queue (gpu.rs:24). */
int shady_ctx_create(int device, void *stream, shady_ctx **out);
int shady_ctx_destroy(shady_ctx *ctx);
/* Message of the last non-zero status on this context ("" if none).  With ctx == NULL,
 * the message of the last failed shady_ctx_create on this thread. */
const char *shady_last_error(const shady_ctx *ctx);
/* The cudaStream_t the context launches on. */
void *shady_ctx_stream(const shady_ctx *ctx);
/* Number of kernels this context has launched so far (bookkeeping for benchmarks). */
uint64_t shady_ctx_launch_count(const shady_ctx *ctx);
/* Iteration limits of the bounded device-side waits of this context's later launches (0 keeps a limit as it is):
 * the grid barrier ahead of the in-launch record merge of shady_attn_decode* (default 2^21 polls), a peer's NVLink
 * flag in shady_attn_combine_p2p / shady_attn_decode_shard_p2p (2^22), an mbarrier of shady_attn_prefill or of the
 * many-token pass of shady_kv_append_rope / shady_attn_prefill_append (2^20).
 * A wait that runs out makes its kernel skip the rest of its work and return; the next shady_synchronize then
 * returns SHADY_ERR_TIMEOUT once (the message names the wait), outputs of launches since the previous successful
 * shady_synchronize are undefined, and until the status has been collected every launch on the context is refused
 * with SHADY_ERR_TIMEOUT.  Nothing else is left behind: the workspace counters are clean again when the kernel ends.
 * No reference counterpart (wgpu has no device-side waits; a lost device panics, gpu.rs:43). */
int shady_ctx_set_wait_limits(shady_ctx *ctx, uint32_t grid_polls, uint32_t peer_polls, uint32_t mbarrier_polls);

/* create_storage_buffer (gpu.rs:95); size is rounded up to 4 bytes as in gpu.rs:86. */
int shady_buffer_create(shady_ctx *ctx, size_t bytes, void **d_out);
int shady_buffer_free(shady_ctx *ctx, void *d_buf);
/* write_buffer (gpu.rs:278): host -> device at byte offset, stream-ordered. */
int shady_buffer_write(shady_ctx *ctx, void *d_buf, size_t offset, const void *src, size_t bytes);
/* read_buffer (gpu.rs:252): device -> host, blocks until the data has arrived. */
int shady_buffer_read(shady_ctx *ctx, const void *d_buf, size_t offset, void *dst, size_t bytes);
/* copy_buffer (gpu.rs:245). */
int shady_buffer_copy(shady_ctx *ctx, const void *d_src, void *d_dst, size_t bytes);
/* Zero-copy alternative to write_buffer/read_buffer (gpu.rs:278, 252) for page-locked host memory
 * (cudaHostAlloc, cudaHostRegister, a pinned torch tensor): *d_ptr receives the address under which
 * kernels read and write that memory directly, so the activations and the result of a step cross the
 * host link inside the launch instead of in copies of their own.  SHADY_ERR_BAD_ARG if host_ptr is
 * not page-locked, device-accessible host memory.  The host reads results after shady_synchronize.
 * No reference counterpart: wgpu buffers cannot be mapped while a dispatch uses them. */
int shady_host_device_ptr(shady_ctx *ctx, const void *host_ptr, void **d_ptr);
/* flush (gpu.rs:237): launches are already submitted, so this only reports a pending
 * asynchronous error. */
int shady_flush(shady_ctx *ctx);
/* device.poll(Maintain::Wait) (gpu.rs:116,270). */
int shady_synchronize(shady_ctx *ctx);

/* ===================================================================================== */
/* KV cache addressing shared by the ops                                                 */
/* ===================================================================================== */

/* Each sequence's cache is rows [pos][num_kv_heads][head_dim], contiguous, K and V in
 * separate buffers — the reference layout (gqa_attention_head.wgsl:64,
 * fused_split_qknorm_kvstore.wgsl:220).  Sequence s lives at d_k_ptrs[s] when the pointer
 * arrays are given, else at d_k_base + s * seq_stride elements.
 *
 * Paged cache (no reference counterpart: the reference reserves max_seq_len rows per layer up
 * front, model.rs:241-256): with d_page_table set, d_k_base / d_v_base are pools of pages
 * [page][page_rows][num_kv_heads][head_dim] and row r of sequence s is row r % page_rows of
 * page d_page_table[s * max_pages_per_seq + r / page_rows]; page_rows is a multiple of 16.
 * Sequences then grow a page at a time and share one pool.  Paged 16-bit caches are taken by
 * shady_kv_append_rope, shady_attn_decode / _static / _shard (num_splits 0 or 1) and
 * shady_attn_decode_append; the other entry points return SHADY_ERR_UNSUPPORTED for them.
 *
 * 8-bit cache (no reference counterpart; the reference's cache is f32, model.rs:241-256): with dtype ==
 * SHADY_F8E4M3 or SHADY_F8E5M2 a stored element is the round-to-nearest-even 8-bit float of value / k_scale (K
 * rows) or value / v_scale (V rows), saturated at the format's largest finite value (448 / 57344); the scales are
 * per cache (0 means 1).  e4m3 keeps one more mantissa bit; e5m2 is cheaper to read (it is the top byte of the f16
 * the tensor core takes, whereas e4m3 needs integer work per byte that bounds the decode kernel).
 * shady_kv_append_rope and shady_qkv_proj_append quantise, and shady_attn_decode / _static / _shard read such
 * caches (head_dim 128 or 256, Q and output f16 or f32); the other entry points return SHADY_ERR_UNSUPPORTED.
 * Zero the struct before filling it: fields added later default to "off". */
typedef struct {
    void *d_k_base;
    void *d_v_base;
    uint64_t seq_stride;     /* elements between consecutive sequences (ignored with ptr arrays) */
    void *const *d_k_ptrs;   /* device array [num_seqs] of device pointers, or NULL */
    void *const *d_v_ptrs;
    uint32_t dtype;          /* SHADY_F32 / SHADY_F16 / SHADY_BF16 / SHADY_F8E4M3 / SHADY_F8E5M2 */
    uint32_t page_rows;      /* paged: rows per page (multiple of 16); else 0 */
    const uint32_t *d_page_table;   /* paged: device array [num_seqs][max_pages_per_seq]; else NULL */
    uint32_t max_pages_per_seq;
    float k_scale;           /* 8-bit caches: value = stored * scale; 0 = 1 */
    float v_scale;
    uint32_t _pad;
} shady_kv_cache;

/* ===================================================================================== */
/* KV append: Q/gate split + Q/K RMSNorm(1+w) + partial (m)RoPE + cache store            */
/* replaces Model::fused_split_qknorm_kvstore (model.rs:486-513) and                     */
/* fused_split_qknorm_kvstore.wgsl:106-230                                               */
/* ===================================================================================== */

typedef struct {
    /* header of the reference uniform (fused_split_qknorm_kvstore.wgsl:12-16) */
    uint32_t num_heads;
    uint32_t num_kv_heads;
    uint32_t head_dim;        /* <= 256 as in the shader */
    float eps;
    /* constants model.rs:32-54 bakes into the shader source */
    float rope_theta;
    uint32_t rotary_dim;      /* PARTIAL_DIM; even, <= head_dim; 0 = no rotation */
    uint32_t s1_limit;        /* MROPE_S1_LIMIT (reference: rotary_dim/2) */
    uint32_t s2_limit;        /* MROPE_S2_LIMIT (reference: rotary_dim/2) */
    uint32_t interleaved;     /* MROPE_INTERLEAVED: pairs (2i,2i+1) else (i, i+rotary_dim/2) */
    /* batching (extension: the reference appends one token of one sequence per dispatch) */
    uint32_t num_seqs;
    uint32_t tokens_per_seq;  /* 1 for decode, T for prefill; token (s,j) sits at row s*T+j */
    /* dtypes */
    uint32_t in_dtype;        /* q_proj_full / k_proj / v_proj */
    uint32_t q_dtype;         /* q_out */
    uint32_t has_gate;        /* 1: q_proj_full rows are [Q|gate] (2*head_dim); 0: Q only */
    uint32_t write_k_back;    /* 1: normed+rotated K also overwrites k_proj (wgsl:224) */
    uint32_t _pad;
} shady_append_params;

/* d_q_proj_full [tokens][nh][(1+has_gate)*hd], d_k_proj / d_v_proj [tokens][nkv][hd] in in_dtype.
 * d_q_out [tokens][nh][hd] in q_dtype.  d_q_gate [tokens][nh][hd] f32 (may be NULL when
 * has_gate == 0).  d_qk_norm_bf16: bf16 weights, q [hd] then k [hd] (model.rs:157-166), or
 * NULL to skip the RMSNorm.  d_pos_start [num_seqs] u32: token (s,j) has RoPE position and
 * cache row pos_start[s]+j (model.rs:493-496 writes one value into all four position
 * fields).  d_pos_h / d_pos_w: optional per-sequence start positions of the height/width
 * mRoPE sections; NULL = same as d_pos_start. */
int shady_kv_append_rope(shady_ctx *ctx, const shady_append_params *p, const void *d_q_proj_full,
                         void *d_k_proj, const void *d_v_proj, void *d_q_out, float *d_q_gate,
                         const shady_kv_cache *cache, const uint16_t *d_qk_norm_bf16,
                         const uint32_t *d_pos_start, const uint32_t *d_pos_h,
                         const uint32_t *d_pos_w);

/* ===================================================================================== */
/* Decode attention — replaces Model::gqa_attention (model.rs:516-573),                  */
/* gqa_attention_head.wgsl:30-124 and gqa_reduce.wgsl:20-65                               */
/* ===================================================================================== */

typedef struct {
    /* the reference's Params (gqa_attention_head.wgsl:9-18); seq_len moved to d_seq_lens */
    uint32_t head_dim;
    uint32_t num_kv_heads;
    uint32_t num_q_heads;
    uint32_t heads_per_kv;
    uint32_t num_splits;      /* >=1: every sequence is cut into this many ceil(L/ns) ranges as in
                                 wgsl:46-48.  0: automatic, length-balanced (needs seq_lens_host). */
    /* batching + dtypes (extensions) */
    uint32_t num_seqs;
    uint32_t q_dtype;         /* SHADY_F32 or the cache dtype */
    uint32_t out_dtype;       /* SHADY_F32 or the cache dtype */
} shady_decode_params;

/* Bytes of scratch `shady_attn_decode` needs for these parameters (upper bound over any
 * sequence lengths; 0 when num_splits == 1).  It replaces the reference's `attn_partials`
 * buffer (model.rs:219-224, 236). */
int shady_decode_workspace_size(const shady_decode_params *p, size_t *bytes);
/* The workspace starts with arrival counters that must be zero before its first use: call this
 * once after allocating it (stream-ordered memset).  Every decode call leaves them zero again (also one
 * whose bounded wait ran out), so no further clearing is needed. */
int shady_decode_workspace_init(shady_ctx *ctx, const shady_decode_params *p, void *d_workspace,
                                size_t workspace_bytes);

/* d_q [num_seqs][nh][hd]; d_seq_lens [num_seqs] u32 = rows to attend to, *including* the
 * token just appended (model.rs:521).  d_out [num_seqs][nh][hd].  d_lse: optional
 * [num_seqs][nh] f32 log-sum-exp of each output row (needed to merge shards of one
 * sequence across GPUs); NULL to skip.  d_gate: optional [num_seqs][nh][hd] f32; when given
 * the output is multiplied by sigmoid(gate) (fuses Model::sigmoid_mul_gate, model.rs:576).
 * seq_lens_host: the same lengths in host memory (they must equal the device values): needed to
 * balance the split plan when num_splits == 0, may be NULL otherwise; for batches of up to 32
 * sequences the kernels also take the lengths from it by value instead of loading them.  A sequence of length 0 yields zeros and
 * lse = -inf.  Splits are merged inside the same launch (gqa_reduce.wgsl math): by the last CTA to arrive for a
 * sequence, or — when a 16-bit sequence is cut into more than 12 spans — by the whole grid after a bounded grid
 * barrier (a cooperative launch; see shady_ctx_set_wait_limits).  Calls that share one workspace must not overlap
 * on the GPU. */
int shady_attn_decode(shady_ctx *ctx, const shady_decode_params *p, const void *d_q,
                      const shady_kv_cache *cache, const uint32_t *d_seq_lens,
                      const uint32_t *seq_lens_host, void *d_out, float *d_lse, const float *d_gate,
                      void *d_workspace, size_t workspace_bytes);

/* Append and attend in ONE launch — the three calls of a self-attention layer (model.rs:723-725:
 * fused_split_qknorm_kvstore, gqa_attention, sigmoid_mul_gate) for a batch of sequences with 16-bit or 8-bit
 * caches (8-bit: f16 or f32 projections; the new rows are quantised as shady_kv_append_rope quantises them).
 * Q is normed/rotated while it is staged; the CTA that owns the tail of a sequence norms/rotates the new K row,
 * stores it and the V row at row seq_len-1 of the cache, then streams them with the rest.  `ap` describes the
 * projections as in shady_kv_append_rope (tokens_per_seq must be 1, interleaved RoPE, one position per token:
 * the position is seq_len-1); with ap->has_gate the output is multiplied by sigmoid(gate) from q_proj_full.
 * d_seq_lens counts the new token, as in shady_attn_decode.  Neither q_out nor q_gate nor k_proj is written. */
int shady_attn_decode_append(shady_ctx *ctx, const shady_append_params *ap, const shady_decode_params *p,
                             const void *d_q_proj_full, const void *d_k_proj, const void *d_v_proj,
                             const uint16_t *d_qk_norm_bf16, const shady_kv_cache *cache, const uint32_t *d_seq_lens,
                             const uint32_t *seq_lens_host, void *d_out, float *d_lse, void *d_workspace,
                             size_t workspace_bytes);

/* One shard of a sequence-split decode (rows of one sequence spread over several GPUs): the same
 * kernels as shady_attn_decode, but the result is written as records d_records[seq][nh][hd+2] in the
 * layout of the reference's partials ([hd] = log-sum-exp, gqa_attention_head.wgsl:112-123), ready to be
 * gathered rank-major and merged with shady_attn_reduce(split_stride = num_seqs*nh*(hd+2),
 * head_stride = hd+2) — gqa_reduce.wgsl across GPUs.  d_seq_lens counts this shard's rows only; a shard
 * with no rows yields lse = -inf and gets weight 0 in the merge. */
int shady_attn_decode_shard(shady_ctx *ctx, const shady_decode_params *p, const void *d_q,
                            const shady_kv_cache *cache, const uint32_t *d_seq_lens,
                            const uint32_t *seq_lens_host, float *d_records, void *d_workspace,
                            size_t workspace_bytes);

/* ---- merging the shards of one sequence across GPUs over NVLink peer memory (no reference counterpart:
 * the reference is single-device; the math is gqa_reduce.wgsl:33-64) ---------------------------------- */
/* Share a buffer made with shady_buffer_create with the other processes of the box (CUDA IPC): export a
 * 64-byte handle here, send it by any host channel, open it there.  Close before the owner frees it. */
int shady_ipc_export(shady_ctx *ctx, void *d_buf, unsigned char handle[64]);
int shady_ipc_open(shady_ctx *ctx, const unsigned char handle[64], void **d_peer);
int shady_ipc_close(shady_ctx *ctx, void *d_peer);
/* Size of the per-rank exchange buffer (flags + two generations of `world` records per head).  It must be
 * zero before the first call. */
int shady_combine_p2p_buffer_size(uint32_t world, uint32_t num_heads, uint32_t head_dim, size_t *bytes);
/* One kernel = exchange + merge: every rank calls it with its own records d_records[nh][hd+2] (from
 * shady_attn_decode_shard, num_seqs == 1).  d_peer_table is a device array [world] of the ranks' exchange
 * buffers as mapped into this process (entry `rank` is the local one).  `epoch` starts at 1 and grows by 1
 * per call on every rank.  The kernel stores its records into every peer's buffer, raises per-head flags,
 * waits (bounded) for the other ranks' flags and writes the merged rows to d_out[nh][hd].  If a peer never
 * arrives the wait expires and the next shady_synchronize returns SHADY_ERR_TIMEOUT. */
int shady_attn_combine_p2p(shady_ctx *ctx, uint32_t world, uint32_t rank, uint32_t num_heads, uint32_t head_dim,
                           uint32_t epoch, void *const *d_peer_table, const float *d_records, void *d_out,
                           uint32_t out_dtype, const float *d_gate);
/* The whole sharded step in ONE cooperative launch: the decode kernel streams this rank's rows, its CTAs meet at a
 * bounded grid barrier, and the grid then merges the rank's split records, stores each (head, 64-dim chunk) slice
 * into every peer's exchange buffer with plain NVLink stores, raises a flag per slice, waits (bounded) for the
 * peers' flags and merges across ranks into d_out[nh][hd] — the work of shady_attn_decode_shard +
 * shady_attn_combine_p2p without their two extra launches.  A shard short enough for a single span keeps two
 * launches (decode, then one merge+exchange kernel).  Arguments as in those two calls (one sequence,
 * num_splits == 0; d_records [nh][hd+2] is scratch).  An exchange buffer serves either this call or
 * shady_attn_combine_p2p, not both in turn. */
int shady_attn_decode_shard_p2p(shady_ctx *ctx, const shady_decode_params *p, const void *d_q,
                                const shady_kv_cache *cache, const uint32_t *d_seq_lens,
                                const uint32_t *seq_lens_host, uint32_t world, uint32_t rank, uint32_t epoch,
                                void *const *d_peer_table, float *d_records, void *d_out, uint32_t out_dtype,
                                const float *d_gate, void *d_workspace, size_t workspace_bytes);

/* No counterpart in the reference.  The same decode as shady_attn_decode for callers that cannot
 * hand over a workspace: a server that gave all device memory to its KV-cache arena at start-up, or
 * a decode loop that cannot take the device-wide stall of an allocation.  The arrival counters and
 * split records live in a 4 MiB array built into the library (every GPU that loads the library
 * holds it until the process exits); nothing is allocated or freed, by this call or below it.
 *  - A launch that needs more scratch than 4 MiB returns SHADY_ERR_WORKSPACE and runs nothing; the
 *    message names both sizes.  (cfg-2-sized batches need about 1.2 MiB.)
 *  - The first call on a device looks up the array's device address; make that call before any
 *    stream capture begins on that device.
 *  - Every call on a device shares the one array and clears its counters on the stream first, so two
 *    calls that overlap on the GPU (different streams or contexts) race; keep them stream-ordered.
 *  - Checks, span plan and kernels are those of shady_attn_decode; only the scratch differs. */
int shady_attn_decode_static(shady_ctx *ctx, const shady_decode_params *p, const void *d_q,
                             const shady_kv_cache *cache, const uint32_t *d_seq_lens,
                             const uint32_t *seq_lens_host, void *d_out, float *d_lse, const float *d_gate);

/* Split-level output of the decode kernel without the merge: d_partials receives the
 * reference layout [nh][num_splits][hd+2] ([hd] = lse, [hd+1] = running max) for ONE
 * sequence (gqa_attention_head.wgsl:112-123).  Requires num_seqs == 1, num_splits >= 2. */
int shady_attn_decode_partials(shady_ctx *ctx, const shady_decode_params *p, const void *d_q,
                               const shady_kv_cache *cache, const uint32_t *d_seq_lens,
                               float *d_partials);

/* gqa_reduce.wgsl:20-65 with its Params {head_dim, num_splits, num_heads}.  Generalised by
 * two strides (in floats) so that both the reference layout (split_stride = hd+2,
 * head_stride = ns*(hd+2)) and rank-major gathered shards (split_stride = nh*(hd+2),
 * head_stride = hd+2) merge with the same kernel.  Splits whose lse is -inf or NaN (empty
 * ranges) get weight 0 and are not read.  d_gate as in shady_attn_decode. */
int shady_attn_reduce(shady_ctx *ctx, uint32_t head_dim, uint32_t num_splits, uint32_t num_heads,
                      uint64_t split_stride, uint64_t head_stride, const float *d_partials,
                      void *d_out, uint32_t out_dtype, const float *d_gate);

/* ===================================================================================== */
/* Causal prefill attention — the batched form of the reference's token loop             */
/* (src/inference.rs:93-95: out[t] = attend(q_t, K[0..=t], V[0..=t]))                    */
/* ===================================================================================== */

typedef struct {
    uint32_t head_dim;        /* 128 or 256 */
    uint32_t num_kv_heads;
    uint32_t num_q_heads;
    uint32_t num_seqs;        /* batch */
    uint32_t seq_len;         /* T tokens per sequence, rows [0,T) of each cache */
    uint32_t dtype;           /* SHADY_BF16 or SHADY_F16: Q, cache and output */
} shady_prefill_params;

/* d_q [num_seqs][T][nh][hd] (already normed/rotated by shady_kv_append_rope, which also
 * wrote rows [0,T) of the cache); d_out same shape.  Requires cache.d_k_base addressing with
 * seq_stride (one allocation): one tensor map covers the batch.  Other caches and prompts of
 * different lengths: shady_attn_prefill_ragged below. */
int shady_attn_prefill(shady_ctx *ctx, const shady_prefill_params *p, const void *d_q,
                       const shady_kv_cache *cache, void *d_out);

/* The whole prefill step from the projections, i.e. what T iterations of model.rs:723-725 (fused_split_qknorm_kvstore,
 * gqa_attention, sigmoid_mul_gate) compute for T new tokens of each of num_seqs empty caches (inference.rs:93-95):
 * K is normed and rotated and K/V are stored in cache rows [0, T) (positions 0..T-1) by one small pass; the
 * attention kernel then takes Q straight from d_q_proj_full, applies RMSNorm(1+w) and RoPE to each Q tile in shared
 * memory, attends causally and multiplies by sigmoid(gate) in its epilogue — the rotated Q and the gate never make a
 * round trip through device memory.  `ap` as in shady_kv_append_rope with tokens_per_seq == p->seq_len,
 * in_dtype == p->dtype (bf16 or f16), interleaved RoPE with one position per token; q_out, q_gate and k_proj are not
 * written.  d_q_proj_full [num_seqs][T][nh][(1+has_gate)*hd]; d_k_proj / d_v_proj [num_seqs][T][nkv][hd];
 * d_out [num_seqs][T][nh][hd].  Cache addressing as in shady_attn_prefill.  d_workspace: at least
 * shady_prefill_workspace_size bytes, 16-byte aligned, no initialisation needed (head_dim 128: a cos/sin table of
 * the T positions; head_dim 256: the rotated Q of the batch, which that kernel takes from memory — there the step is
 * one append pass over Q, K and V plus the attention kernel, whose epilogue still applies the gate).  Replaces the
 * prompt loop of src/inference.rs:93-95 for 16-bit caches. */
int shady_prefill_workspace_size(const shady_prefill_params *p, size_t *bytes);
int shady_attn_prefill_append(shady_ctx *ctx, const shady_append_params *ap, const shady_prefill_params *p,
                              const void *d_q_proj_full, const void *d_k_proj, const void *d_v_proj,
                              const uint16_t *d_qk_norm_bf16, const shady_kv_cache *cache, void *d_out,
                              void *d_workspace, size_t workspace_bytes);

/* Prompts of different lengths in one launch, and caches of any addressing (one allocation with seq_stride,
 * per-sequence pointer arrays, page pools + page table) — what a batch built from the reference's cache slots
 * (model.rs:973-1029), each prefilled by its own token loop (inference.rs:93-95), needs.  Sequence i has
 * h_seq_lens[i] > 0 tokens; Q, the output and (for the _append form) the projections are packed token-major,
 * sequence after sequence: [sum T_i][heads][...].  p->seq_len is not read.  The K/V tiles of a sequence come through
 * a tensor map of its own, encoded on the HOST, which therefore needs the per-sequence base addresses: for a
 * pointer-array cache pass host copies of the two arrays in h_k_ptrs / h_v_ptrs (NULL otherwise).  Rows past a
 * sequence's end are never read from memory with those caches.  Paged caches: page_rows a multiple of the K/V tile
 * (128 rows for head_dim 128, 64 for 256) or 8, 16, 32 or 64 below it; the rows between a sequence's end and the
 * end of its last tile lie in the sequence's last page and must hold finite values — the _append form clears them,
 * shady_attn_prefill_ragged expects the caller's pool to be initialised.  d_workspace: at least
 * shady_prefill_ragged_workspace_size bytes (with_append = 1 for the _append form), 128-byte aligned, written by
 * every call (row-block list, tensor maps, and for the _append form the cos/sin table or the rotated Q); the small
 * tables are copied from a page-locked staging buffer of the context, so these two calls are not capturable into a
 * CUDA graph.  No reference counterpart beyond the loop they replace. */
typedef struct {
    const uint32_t *h_seq_lens;      /* HOST [num_seqs] */
    const void *const *h_k_ptrs;     /* HOST [num_seqs] copy of cache.d_k_ptrs, or NULL */
    const void *const *h_v_ptrs;     /* HOST [num_seqs] copy of cache.d_v_ptrs, or NULL */
} shady_prefill_batch;
int shady_prefill_ragged_workspace_size(const shady_prefill_params *p, const uint32_t *h_seq_lens, int with_append,
                                        size_t *bytes);
int shady_attn_prefill_ragged(shady_ctx *ctx, const shady_prefill_params *p, const shady_prefill_batch *batch,
                              const void *d_q, const shady_kv_cache *cache, void *d_out, void *d_workspace,
                              size_t workspace_bytes);
int shady_attn_prefill_append_ragged(shady_ctx *ctx, const shady_append_params *ap, const shady_prefill_params *p,
                                     const shady_prefill_batch *batch, const void *d_q_proj_full,
                                     const void *d_k_proj, const void *d_v_proj, const uint16_t *d_qk_norm_bf16,
                                     const shady_kv_cache *cache, void *d_out, void *d_workspace,
                                     size_t workspace_bytes);

/* ===================================================================================== */
/* Output gate — replaces Model::sigmoid_mul_gate (model.rs:576-593), sigmoid_mul.wgsl    */
/* ===================================================================================== */
/* x[i] *= 1/(1+exp(-gate[i])) in place (the reference needs a temp + copy: model.rs:584-592). */
int shady_sigmoid_mul(shady_ctx *ctx, float *d_x, const float *d_gate, uint32_t n);

/* ===================================================================================== */
/* q/k/v projections (INT4 GPTQ matvec) with the KV append as their epilogue               */
/* replaces Model::gptq_matvec (model.rs:357-381) at its q/k/v call sites (model.rs:698-714) */
/* and the dispatch that follows them (model.rs:723); gptq_matvec.wgsl, gptq_matvec_4t.wgsl */
/* ===================================================================================== */
/* One symmetric INT4 weight matrix in the reference's layout: d_qweight [K/8][N] u32, eight nibbles along K per
 * word, lowest row in the low nibble (gptq_matvec.wgsl:47-57); d_scales [K/group_size][N] f16, two per u32
 * (unpack2x16float, wgsl:44-45); weight(k, n) = (nibble - 8) * scale(k / group_size, n).  K and group_size are
 * multiples of 8 and group_size divides K. */
typedef struct {
    const uint32_t *d_qweight;
    const uint32_t *d_scales;
    uint32_t K;
    uint32_t N;
    uint32_t group_size;
    uint32_t _pad;
} shady_gptq_weight;

/* Model::gptq_matvec (model.rs:357-381): d_y[v][n] = sum_k weight(k, n) * d_x[v][k] for num_vecs input vectors
 * (the reference has one).  f32 in, f32 out. */
int shady_gptq_matvec(shady_ctx *ctx, const shady_gptq_weight *w, const float *d_x, float *d_y, uint32_t num_vecs);

/* The three projections of a self-attention layer and the append in ONE launch: what model.rs:698-714 followed by
 * model.rs:723 compute with four dispatches and three f32 buffers in between (q_out, k_out, v_out, which are not
 * written here).  d_x [num_seqs][K] f32 is the normed hidden state of one token per sequence.  wq has
 * num_heads * (1 + has_gate) * head_dim columns (per head: Q columns, then gate columns — the layout
 * fused_split_qknorm_kvstore.wgsl:122-135 reads), wk and wv num_kv_heads * head_dim each.  Outputs and the remaining
 * arguments are those of shady_kv_append_rope (`p->tokens_per_seq` must be 1, `p->in_dtype` and `p->write_k_back`
 * are ignored): d_q_out, d_q_gate, the cache row of every sequence at its position. */
int shady_qkv_proj_append(shady_ctx *ctx, const shady_append_params *p, const shady_gptq_weight *wq,
                          const shady_gptq_weight *wk, const shady_gptq_weight *wv, const float *d_x, void *d_q_out,
                          float *d_q_gate, const shady_kv_cache *cache, const uint16_t *d_qk_norm_bf16,
                          const uint32_t *d_pos_start, const uint32_t *d_pos_h, const uint32_t *d_pos_w);

/* ===================================================================================== */
/* Synthetic data — counter-based N(0,1) fill used by the benchmark and the tests         */
/* (no reference counterpart: the reference has no benchmark inputs).                     */
/* ===================================================================================== */
/* Element i of d_dst = randn(seed, tensor_id, first_idx + i) rounded to `dtype`. */
int shady_fill_randn(shady_ctx *ctx, void *d_dst, uint64_t n, uint32_t dtype, uint64_t seed,
                     uint64_t tensor_id, uint64_t first_idx);

#ifdef __cplusplus
}
#endif
#endif /* SHADY_ATTN_H */
