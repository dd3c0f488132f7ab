//! `src/gpu.rs` with a CUDA backend for the attention op: the same `GpuContext` method names and argument
//! meaning as the wgpu one (src/gpu.rs:7-297 of shady-thinker), bodies replaced by calls into `shady-attn-sys`.
//!
//! A drop-in for the attention path only: `dispatch` is kept for the shaders that stay on wgpu and is not used
//! by the three attention helpers any more.  Where the wgpu code `expect`s / `unwrap`s (gpu.rs:43, 68, 271) a
//! non-zero status panics with the library's message.
//!
//! Not compiled where it was written (no Rust toolchain there): reviewed source.
use shady_attn_sys::*;
use std::ffi::CStr;
use std::os::raw::c_void;
use std::ptr::{null, null_mut};

/// Stand-in of `wgpu::Buffer` for the CUDA backend: a device allocation the caller owns.
pub struct CudaBuffer {
    pub ptr: *mut c_void,
    pub size: u64,
    pub label: String,
}

pub struct GpuContext {
    pub cuda: *mut ShadyCtx,
    pending_dispatches: u32,
}

impl GpuContext {
    /// gpu.rs:17 — `device` 0, a stream of the library's own.
    pub fn new() -> Self {
        Self::on_device(0, null_mut())
    }

    /// gpu.rs:24 `from_device_queue`: an externally owned queue becomes an externally owned `cudaStream_t`.
    pub fn from_device_queue(device: i32, stream: *mut c_void) -> Self {
        Self::on_device(device, stream)
    }

    fn on_device(device: i32, stream: *mut c_void) -> Self {
        let mut cuda: *mut ShadyCtx = null_mut();
        let st = unsafe { shady_ctx_create(device, stream, &mut cuda) };
        if st != SHADY_OK {
            let msg = unsafe { CStr::from_ptr(shady_last_error(null())) }.to_string_lossy().into_owned();
            panic!("no suitable GPU adapter found: {msg}");                       // gpu.rs:43
        }
        Self { cuda, pending_dispatches: 0 }
    }

    /// Turns a status into the reference's convention (panic with a message).
    pub fn check(&self, status: i32) {
        if status != SHADY_OK {
            let msg = unsafe { CStr::from_ptr(shady_last_error(self.cuda)) }.to_string_lossy().into_owned();
            panic!("shady_attn status {status}: {msg}");
        }
    }

    /// gpu.rs:80 — the usage flags have no CUDA counterpart; size is rounded up to 4 bytes as in gpu.rs:86.
    pub fn create_buffer(&self, label: &str, size: u64) -> CudaBuffer {
        let mut ptr: *mut c_void = null_mut();
        self.check(unsafe { shady_buffer_create(self.cuda, size as usize, &mut ptr) });
        CudaBuffer { ptr, size: (size + 3) & !3, label: label.to_string() }
    }

    /// gpu.rs:95
    pub fn create_storage_buffer(&self, label: &str, size: u64) -> CudaBuffer {
        self.create_buffer(label, size)
    }

    /// gpu.rs:105 — one stream-ordered copy, then wait (the wgpu code chunks at 64 MB and polls).
    pub fn upload_buffer(&self, label: &str, data: &[u8]) -> CudaBuffer {
        let buffer = self.create_storage_buffer(label, data.len() as u64);
        self.write_buffer(&buffer, 0, data);
        self.check(unsafe { shady_synchronize(self.cuda) });
        buffer
    }

    /// gpu.rs:119 — read-backs go through `read_buffer`; a staging buffer is not needed.
    pub fn create_readback_buffer(&self, label: &str, size: u64) -> CudaBuffer {
        self.create_buffer(label, size)
    }

    /// gpu.rs:188 — the attention helpers no longer come here; other shaders stay with the wgpu context.
    pub fn dispatch(&mut self, pipeline_name: &str, _shader_src: &str, _buffers: &[(u32, &CudaBuffer)], _workgroups: (u32, u32, u32)) {
        self.pending_dispatches += 1;
        panic!("{pipeline_name}: WGSL dispatch is not part of the CUDA backend (attention op only)");
    }

    /// gpu.rs:237 — launches are submitted when they are made; this only reports a pending asynchronous error.
    pub fn flush(&mut self) {
        self.check(unsafe { shady_flush(self.cuda) });
        self.pending_dispatches = 0;
    }

    /// gpu.rs:245
    pub fn copy_buffer(&mut self, src: &CudaBuffer, dst: &CudaBuffer, size: u64) {
        self.check(unsafe { shady_buffer_copy(self.cuda, src.ptr, dst.ptr, size as usize) });
    }

    /// gpu.rs:252 — blocks until the bytes have arrived, as `map_async` + `poll(Wait)` does.
    pub fn read_buffer(&mut self, buffer: &CudaBuffer, size: u64) -> Vec<u8> {
        let mut data = vec![0u8; size as usize];
        self.check(unsafe { shady_buffer_read(self.cuda, buffer.ptr, 0, data.as_mut_ptr() as *mut c_void, size as usize) });
        data
    }

    /// gpu.rs:278
    pub fn write_buffer(&self, buffer: &CudaBuffer, offset: u64, data: &[u8]) {
        self.check(unsafe {
            shady_buffer_write(self.cuda, buffer.ptr, offset as usize, data.as_ptr() as *const c_void, data.len())
        });
    }

    /// `device.poll(Maintain::Wait)` (gpu.rs:116, 270); also reports a bounded device-side wait that ran out.
    pub fn synchronize(&self) {
        self.check(unsafe { shady_synchronize(self.cuda) });
    }
}

impl Drop for GpuContext {
    fn drop(&mut self) {
        unsafe { shady_ctx_destroy(self.cuda) };
    }
}

impl Drop for CudaBuffer {
    fn drop(&mut self) {
        // the owner frees through its context (`shady_buffer_free`); a buffer that outlives its context leaks
    }
}
