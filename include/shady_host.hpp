// C++ host-side mirror of the reference's call surface for the attention path, over the C ABI in
// shady_attn.h.  The reference's host code is Rust (no toolchain for it here), so this header is what a
// compiled host program uses instead: the same type and method names as src/gpu.rs (`GpuContext`) and
// as the attention helpers of src/model.rs (`Model::fused_split_qknorm_kvstore`, `gqa_attention`,
// `sigmoid_mul_gate`, `InferenceState`, `CacheSlot`), the same argument meaning, and the same error
// behaviour: where the reference panics (`expect`/`unwrap`, gpu.rs:43,68,271) this throws.
#pragma once
#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "shady_attn.h"

namespace shady_thinker {

// wgpu::Buffer stand-in: a device allocation owned by whoever created it.
struct Buffer {
    void *ptr = nullptr;
    size_t size = 0;
    std::string label;
};

class GpuContext {
public:
    // GpuContext::new (gpu.rs:17); with a stream: from_device_queue (gpu.rs:24)
    explicit GpuContext(int device = 0, void *stream = nullptr) {
        if (shady_ctx_create(device, stream, &ctx_) != SHADY_OK) throw std::runtime_error(shady_last_error(nullptr));
    }
    ~GpuContext() {
        if (!ctx_) return;
        for (void *p : live_) shady_buffer_free(ctx_, p);
        shady_ctx_destroy(ctx_);
    }
    GpuContext(const GpuContext &) = delete;
    GpuContext &operator=(const GpuContext &) = delete;

    // gpu.rs:95 (size rounded up to 4 bytes as in gpu.rs:86)
    Buffer create_storage_buffer(const std::string &label, size_t size) {
        Buffer b;
        check(shady_buffer_create(ctx_, size, &b.ptr));
        b.size = (size + 3) & ~size_t(3);
        b.label = label;
        live_.push_back(b.ptr);
        return b;
    }
    // gpu.rs:105
    Buffer upload_buffer(const std::string &label, const void *data, size_t bytes) {
        Buffer b = create_storage_buffer(label, bytes);
        write_buffer(b, 0, data, bytes);
        check(shady_synchronize(ctx_));
        return b;
    }
    // gpu.rs:278
    void write_buffer(const Buffer &buf, size_t offset, const void *data, size_t bytes) {
        check(shady_buffer_write(ctx_, buf.ptr, offset, data, bytes));
    }
    // gpu.rs:252 — blocks until the data has arrived
    std::vector<uint8_t> read_buffer(const Buffer &buf, size_t size) {
        std::vector<uint8_t> out(size);
        check(shady_buffer_read(ctx_, buf.ptr, 0, out.data(), size));
        return out;
    }
    // gpu.rs:245
    void copy_buffer(const Buffer &src, const Buffer &dst, size_t size) { check(shady_buffer_copy(ctx_, src.ptr, dst.ptr, size)); }
    // no gpu.rs counterpart: device-side address of page-locked host memory (zero-copy instead of write/read_buffer)
    void *host_device_ptr(const void *pinned_host) {
        void *d = nullptr;
        check(shady_host_device_ptr(ctx_, pinned_host, &d));
        return d;
    }
    // gpu.rs:237
    void flush() { check(shady_flush(ctx_)); }
    void synchronize() { check(shady_synchronize(ctx_)); }

    shady_ctx *raw() const { return ctx_; }
    void check(int status) const {
        if (status != SHADY_OK) throw std::runtime_error(std::string("shady_attn status ") + std::to_string(status) + ": " + shady_last_error(ctx_));
    }

private:
    shady_ctx *ctx_ = nullptr;
    std::vector<void *> live_;
};

// The ModelConfig fields the hot path reads, with the reference defaults (src/weights.rs:93-152).
struct ModelConfig {
    uint32_t num_attention_heads = 0, num_key_value_heads = 0, num_hidden_layers = 1, head_dim = 128;
    float rms_norm_eps = 1e-6f, rope_theta = 1e7f, partial_rotary_factor = 0.25f;
    bool mrope_interleaved = true;
    // model.rs:33: (config.head_dim as f32 * config.partial_rotary_factor) as u32
    uint32_t rotary_dim() const { return static_cast<uint32_t>(static_cast<float>(head_dim) * partial_rotary_factor); }
};

// model.rs:57-86, the buffers the three helpers touch
struct InferenceState {
    Buffer q_out, q_proj, q_gate, k_out, v_out, attn_output, attn_partials, position, seq_len_dev;
    std::vector<Buffer> k_cache, v_cache, qknorm_params;
    size_t partials_bytes = 0;
};

// model.rs:93-99 (KV part)
struct CacheSlot {
    std::vector<Buffer> k_cache, v_cache;
    uint32_t seq_len = 0;
};

// model.rs:89 fixes this at 1 at compile time; here 0 = pick a balanced split at run time
constexpr uint32_t NUM_ATTN_SPLITS = 0;

class Model {
public:
    ModelConfig config;
    InferenceState state;
    uint32_t seq_len = 0;

    Model(GpuContext &gpu, const ModelConfig &cfg, uint32_t max_seq_len, uint32_t kv_dtype = SHADY_F32,
          uint32_t num_attn_splits = NUM_ATTN_SPLITS)
        : config(cfg), max_seq_len_(max_seq_len), kv_dtype_(kv_dtype), splits_(num_attn_splits) {
        const size_t nh = cfg.num_attention_heads, nkv = cfg.num_key_value_heads, hd = cfg.head_dim, f = 4;
        const size_t esz = kv_dtype == SHADY_F32 ? 4 : 2;
        const shady_decode_params dp = decode_params();
        gpu.check(shady_decode_workspace_size(&dp, &state.partials_bytes));
        state.q_out = gpu.create_storage_buffer("q_out", nh * hd * 2 * f);
        state.q_proj = gpu.create_storage_buffer("q_proj", nh * hd * f);
        state.q_gate = gpu.create_storage_buffer("q_gate", nh * hd * f);
        state.k_out = gpu.create_storage_buffer("k_out", nkv * hd * f);
        state.v_out = gpu.create_storage_buffer("v_out", nkv * hd * f);
        state.attn_output = gpu.create_storage_buffer("attn_output", nh * hd * f);
        state.attn_partials = gpu.create_storage_buffer("attn_partials", state.partials_bytes ? state.partials_bytes : 4);
        state.position = gpu.create_storage_buffer("position", 4);
        state.seq_len_dev = gpu.create_storage_buffer("seq_len", 4);
        for (uint32_t i = 0; i < cfg.num_hidden_layers; ++i) {
            state.k_cache.push_back(gpu.create_storage_buffer("k_cache_" + std::to_string(i), max_seq_len * nkv * hd * esz));
            state.v_cache.push_back(gpu.create_storage_buffer("v_cache_" + std::to_string(i), max_seq_len * nkv * hd * esz));
            state.qknorm_params.push_back(Buffer{});
        }
        gpu.check(shady_decode_workspace_init(gpu.raw(), &dp, state.attn_partials.ptr, state.partials_bytes));
    }

    // model.rs:337-346: only the bf16 weights (q then k) are data; the header fields travel by value
    void init_qknorm_params(GpuContext &gpu, size_t layer_idx, const void *q_norm_bytes, const void *k_norm_bytes) {
        const size_t n = config.head_dim * 2;
        std::vector<uint8_t> both(2 * n);
        std::memcpy(both.data(), q_norm_bytes, n);
        std::memcpy(both.data() + n, k_norm_bytes, n);
        state.qknorm_params[layer_idx] = gpu.upload_buffer("qknorm_params_" + std::to_string(layer_idx), both.data(), both.size());
    }

    // model.rs:486-513
    void fused_split_qknorm_kvstore(GpuContext &gpu, size_t layer_idx) {
        if (seq_len >= max_seq_len_) throw std::runtime_error("KV cache is full");
        const uint32_t position = seq_len;
        gpu.write_buffer(state.position, 0, &position, 4);   // model.rs:493-496
        shady_append_params p{};
        p.num_heads = config.num_attention_heads; p.num_kv_heads = config.num_key_value_heads; p.head_dim = config.head_dim;
        p.eps = config.rms_norm_eps; p.rope_theta = config.rope_theta; p.rotary_dim = config.rotary_dim();
        p.s1_limit = p.s2_limit = p.rotary_dim / 2; p.interleaved = config.mrope_interleaved;
        p.num_seqs = 1; p.tokens_per_seq = 1; p.in_dtype = SHADY_F32; p.q_dtype = SHADY_F32; p.has_gate = 1; p.write_k_back = 1;
        const shady_kv_cache c = cache(layer_idx);
        gpu.check(shady_kv_append_rope(gpu.raw(), &p, state.q_out.ptr, state.k_out.ptr, state.v_out.ptr, state.q_proj.ptr,
                                       static_cast<float *>(state.q_gate.ptr), &c,
                                       static_cast<const uint16_t *>(state.qknorm_params[layer_idx].ptr),
                                       static_cast<const uint32_t *>(state.position.ptr), nullptr, nullptr));
    }

    // model.rs:516-573 (seq_len + 1: the token just appended attends to itself)
    void gqa_attention(GpuContext &gpu, size_t layer_idx) {
        const uint32_t len = seq_len + 1;
        gpu.write_buffer(state.seq_len_dev, 0, &len, 4);
        const shady_decode_params p = decode_params();
        const shady_kv_cache c = cache(layer_idx);
        gpu.check(shady_attn_decode(gpu.raw(), &p, state.q_proj.ptr, &c, static_cast<const uint32_t *>(state.seq_len_dev.ptr), &len,
                                    state.attn_output.ptr, nullptr, nullptr, state.attn_partials.ptr, state.partials_bytes));
    }

    // model.rs:576-593 (in place: no temp buffer + copy)
    void sigmoid_mul_gate(GpuContext &gpu) {
        gpu.check(shady_sigmoid_mul(gpu.raw(), static_cast<float *>(state.attn_output.ptr), static_cast<const float *>(state.q_gate.ptr),
                                    config.num_attention_heads * config.head_dim));
    }

    // model.rs:973-1029, KV part
    CacheSlot alloc_cache_slot(GpuContext &gpu) {
        CacheSlot s;
        const size_t n = size_t(max_seq_len_) * config.num_key_value_heads * config.head_dim * (kv_dtype_ == SHADY_F32 ? 4 : 2);
        for (uint32_t i = 0; i < config.num_hidden_layers; ++i) {
            s.k_cache.push_back(gpu.create_storage_buffer("slot_k_" + std::to_string(i), n));
            s.v_cache.push_back(gpu.create_storage_buffer("slot_v_" + std::to_string(i), n));
        }
        return s;
    }
    void swap_cache(CacheSlot &slot) {
        std::swap(state.k_cache, slot.k_cache);
        std::swap(state.v_cache, slot.v_cache);
        std::swap(seq_len, slot.seq_len);
    }

private:
    uint32_t max_seq_len_, kv_dtype_, splits_;
    shady_decode_params decode_params() const {
        shady_decode_params p{};
        p.head_dim = config.head_dim; p.num_kv_heads = config.num_key_value_heads; p.num_q_heads = config.num_attention_heads;
        p.heads_per_kv = config.num_attention_heads / config.num_key_value_heads; p.num_splits = splits_; p.num_seqs = 1;
        p.q_dtype = SHADY_F32; p.out_dtype = SHADY_F32;
        return p;
    }
    shady_kv_cache cache(size_t layer_idx) const {
        shady_kv_cache c{};
        c.d_k_base = state.k_cache[layer_idx].ptr; c.d_v_base = state.v_cache[layer_idx].ptr; c.dtype = kv_dtype_;
        return c;
    }
};

}  // namespace shady_thinker
