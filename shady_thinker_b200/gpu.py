"""Host-side mirror of the reference's ``GpuContext`` (src/gpu.rs:7-297) for the CUDA backend.

Same method names and argument meaning as the Rust type, minus what has no CUDA
counterpart (shader source strings, bind groups).  Buffers are raw device allocations owned
by the caller, as ``wgpu::Buffer`` objects are owned by ``InferenceState`` in the reference.
"""
from __future__ import annotations

import ctypes as C

from . import _lib
from ._lib import ShadyError, check  # noqa: F401


class Buffer:
    """A device allocation (``wgpu::Buffer`` stand-in): address + size."""

    __slots__ = ("ptr", "size", "label")

    def __init__(self, ptr: int, size: int, label: str = ""):
        self.ptr, self.size, self.label = ptr, size, label

    def __repr__(self) -> str:
        return f"Buffer({self.label!r}, 0x{self.ptr:x}, {self.size} B)"


def _addr(buf) -> int:
    """Device address of a Buffer, a torch CUDA tensor, an int, or None."""
    if buf is None:
        return 0
    if isinstance(buf, Buffer):
        return buf.ptr
    if isinstance(buf, int):
        return buf
    if hasattr(buf, "data_ptr"):
        if not buf.is_cuda:
            raise ValueError("expected a CUDA tensor")
        if not buf.is_contiguous():
            raise ValueError("expected a contiguous tensor")
        return buf.data_ptr()
    raise TypeError(f"cannot take a device address of {type(buf)}")


class GpuContext:
    """``GpuContext::new()`` (gpu.rs:17) / ``from_device_queue`` (gpu.rs:24, pass ``stream``)."""

    def __init__(self, device: int = 0, stream: int | None = None):
        self._L = _lib.load()
        h = C.c_void_p()
        st = self._L.shady_ctx_create(device, C.c_void_p(stream) if stream else None, C.byref(h))
        if st != _lib.OK:
            raise ShadyError(st, (self._L.shady_last_error(None) or b"").decode())
        self.handle = h
        self.device = device
        self._live: dict[int, Buffer] = {}

    # -- lifetime -------------------------------------------------------------------------
    def close(self) -> None:
        if getattr(self, "handle", None):
            for b in list(self._live.values()):
                self._L.shady_buffer_free(self.handle, C.c_void_p(b.ptr))
            self._live.clear()
            self._L.shady_ctx_destroy(self.handle)
            self.handle = None

    def __del__(self):  # pragma: no cover - best effort
        try:
            self.close()
        except Exception:
            pass

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    @property
    def stream(self) -> int:
        return int(self._L.shady_ctx_stream(self.handle) or 0)

    @property
    def launch_count(self) -> int:
        return int(self._L.shady_ctx_launch_count(self.handle))

    def _check(self, st: int) -> None:
        check(self.handle, st)

    def set_wait_limits(self, grid_polls: int = 0, peer_polls: int = 0, mbarrier_polls: int = 0) -> None:
        """Iteration limits of the bounded device-side waits of later launches (0 keeps a limit)."""
        self._check(self._L.shady_ctx_set_wait_limits(self.handle, grid_polls, peer_polls, mbarrier_polls))

    # -- buffers (gpu.rs:80-124, 245-280) -------------------------------------------------------
    def create_storage_buffer(self, label: str, size: int) -> Buffer:
        p = C.c_void_p()
        self._check(self._L.shady_buffer_create(self.handle, size, C.byref(p)))
        b = Buffer(p.value, (size + 3) & ~3, label)
        self._live[b.ptr] = b
        return b

    create_buffer = create_storage_buffer

    def upload_buffer(self, label: str, data: bytes) -> Buffer:
        b = self.create_storage_buffer(label, len(data))
        self.write_buffer(b, 0, data)
        self.synchronize()  # gpu.rs:115-116 waits for the upload
        return b

    def destroy_buffer(self, buf: Buffer) -> None:
        self._check(self._L.shady_buffer_free(self.handle, C.c_void_p(buf.ptr)))
        self._live.pop(buf.ptr, None)

    def write_buffer(self, buf, offset: int, data) -> None:
        mv = memoryview(data).cast("B")
        n = mv.nbytes
        src = (C.c_char * n).from_buffer_copy(mv) if n else None
        self._check(self._L.shady_buffer_write(self.handle, C.c_void_p(_addr(buf)), offset, src, n))
        # the staging copy above is pageable: the runtime has consumed it when the call returns

    def read_buffer(self, buf, size: int, offset: int = 0) -> bytes:
        dst = (C.c_char * size)()
        self._check(self._L.shady_buffer_read(self.handle, C.c_void_p(_addr(buf)), offset, dst, size))
        return bytes(dst)

    def copy_buffer(self, src, dst, size: int) -> None:
        self._check(self._L.shady_buffer_copy(self.handle, C.c_void_p(_addr(src)), C.c_void_p(_addr(dst)), size))

    def host_device_ptr(self, host_addr: int) -> int:
        """Device-side address of page-locked host memory (zero-copy alternative to write_buffer/read_buffer)."""
        out = C.c_void_p()
        self._check(self._L.shady_host_device_ptr(self.handle, C.c_void_p(host_addr), C.byref(out)))
        return int(out.value)

    def flush(self) -> None:
        self._check(self._L.shady_flush(self.handle))

    def synchronize(self) -> None:
        self._check(self._L.shady_synchronize(self.handle))
