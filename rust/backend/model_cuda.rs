//! The three private attention helpers of `Model` (src/model.rs:486-593 of shady-thinker) with CUDA bodies.
//! Names, arguments and the order in `Model::forward` (model.rs:723-725) are unchanged; only "fill the uniform and
//! dispatch a shader" became "call the C ABI".  Fragment of `impl Model` — it uses the surrounding type's fields
//! (`self.state`, `self.config`, `self.seq_len`) exactly as the wgpu version does.
//!
//! Not compiled where it was written (no Rust toolchain there): reviewed source.
use crate::gpu::GpuContext;          // rust/backend/gpu_cuda.rs in place of src/gpu.rs
use shady_attn_sys::*;
use std::ptr::{null, null_mut};

/// model.rs:89 fixes the split count at compile time; 0 asks the library for a length-balanced split.
const NUM_ATTN_SPLITS: u32 = 0;

impl Model {
    fn cache(&self, layer_idx: usize) -> ShadyKvCache {
        ShadyKvCache {
            d_k_base: self.state.k_cache[layer_idx].ptr,
            d_v_base: self.state.v_cache[layer_idx].ptr,
            seq_stride: 0,
            d_k_ptrs: null(),
            d_v_ptrs: null(),
            dtype: SHADY_F32,                       // the reference's cache format (model.rs:241-256)
            page_rows: 0,
            d_page_table: null(),
            max_pages_per_seq: 0,
            _pad: 0,
        }
    }

    /// model.rs:337 — only the bf16 weights (q_norm then k_norm) are data; the header fields of the 5,152-byte
    /// uniform (model.rs:129-179) travel by value in `ShadyAppendParams`.
    pub fn init_qknorm_params(&mut self, gpu: &mut GpuContext, layer_idx: usize, q_norm_bytes: &[u8], k_norm_bytes: &[u8]) {
        let mut data = Vec::with_capacity(q_norm_bytes.len() + k_norm_bytes.len());
        data.extend_from_slice(q_norm_bytes);
        data.extend_from_slice(k_norm_bytes);
        self.state.qknorm_params[layer_idx] = gpu.upload_buffer(&format!("qknorm_params_{layer_idx}"), &data);
    }

    /// model.rs:486
    fn fused_split_qknorm_kvstore(&self, gpu: &mut GpuContext, layer_idx: usize) {
        let cfg = &self.config;
        let (nh, nkv, hd) = (cfg.num_attention_heads as u32, cfg.num_key_value_heads as u32, cfg.head_dim as u32);
        let partial_dim = (cfg.head_dim as f32 * cfg.partial_rotary_factor) as u32;     // model.rs:33
        let position = self.seq_len as u32;
        gpu.write_buffer(&self.state.position, 0, bytemuck::bytes_of(&position));        // was: offset 16 of the uniform
        let p = ShadyAppendParams {
            num_heads: nh, num_kv_heads: nkv, head_dim: hd, eps: cfg.rms_norm_eps as f32,
            rope_theta: cfg.rope_theta as f32, rotary_dim: partial_dim,
            s1_limit: partial_dim / 2, s2_limit: partial_dim / 2,                         // model.rs:36-45
            interleaved: cfg.mrope_interleaved() as u32,
            num_seqs: 1, tokens_per_seq: 1, in_dtype: SHADY_F32, q_dtype: SHADY_F32,
            has_gate: 1, write_k_back: 1, _pad: 0,
        };
        let s = &self.state;
        gpu.check(unsafe {
            shady_kv_append_rope(gpu.cuda, &p, s.q_out.ptr, s.k_out.ptr, s.v_out.ptr, s.q_proj.ptr,
                                 s.q_gate.ptr as *mut f32, &self.cache(layer_idx),
                                 s.qknorm_params[layer_idx].ptr as *const u16, s.position.ptr as *const u32, null(), null())
        });
    }

    /// model.rs:516
    fn gqa_attention(&self, gpu: &mut GpuContext, layer_idx: usize) {
        let cfg = &self.config;
        let (nh, nkv, hd) = (cfg.num_attention_heads as u32, cfg.num_key_value_heads as u32, cfg.head_dim as u32);
        let seq_len = (self.seq_len + 1) as u32;                                          // include current token (model.rs:521)
        gpu.write_buffer(&self.state.seq_len_dev, 0, bytemuck::bytes_of(&seq_len));
        let p = ShadyDecodeParams {                                                       // the fields of `struct P` (model.rs:524-533)
            head_dim: hd, num_kv_heads: nkv, num_q_heads: nh, heads_per_kv: nh / nkv,
            num_splits: NUM_ATTN_SPLITS, num_seqs: 1, q_dtype: SHADY_F32, out_dtype: SHADY_F32,
        };
        let s = &self.state;
        gpu.check(unsafe {
            shady_attn_decode(gpu.cuda, &p, s.q_proj.ptr, &self.cache(layer_idx), s.seq_len_dev.ptr as *const u32,
                              &seq_len, s.attn_output.ptr, null_mut(), null(), s.attn_partials.ptr, s.partials_bytes)
        });
    }

    /// model.rs:576 — in place: no temp buffer, no copy back.
    fn sigmoid_mul_gate(&self, gpu: &mut GpuContext) {
        let n = (self.config.num_attention_heads * self.config.head_dim) as u32;
        let s = &self.state;
        gpu.check(unsafe { shady_sigmoid_mul(gpu.cuda, s.attn_output.ptr as *mut f32, s.q_gate.ptr as *const f32, n) });
    }

    /// `attn_partials` (model.rs:219-224, 236): sized and zeroed once through the library.
    fn alloc_attn_partials(&mut self, gpu: &mut GpuContext) {
        let cfg = &self.config;
        let (nh, nkv, hd) = (cfg.num_attention_heads as u32, cfg.num_key_value_heads as u32, cfg.head_dim as u32);
        let p = ShadyDecodeParams { head_dim: hd, num_kv_heads: nkv, num_q_heads: nh, heads_per_kv: nh / nkv,
                                    num_splits: NUM_ATTN_SPLITS, num_seqs: 1, q_dtype: SHADY_F32, out_dtype: SHADY_F32 };
        let mut bytes: usize = 0;
        gpu.check(unsafe { shady_decode_workspace_size(&p, &mut bytes) });
        self.state.attn_partials = gpu.create_storage_buffer("attn_partials", bytes.max(4) as u64);
        self.state.partials_bytes = bytes;
        gpu.check(unsafe { shady_decode_workspace_init(gpu.cuda, &p, self.state.attn_partials.ptr, bytes) });
    }
}
