"""B200 (sm_100a) attention hot path of shady-thinker behind a C ABI.

``libshady_attn.so`` (built by ``shady_thinker_b200.build``) is the product; this package is
the host-side mirror of the reference's call surface for that path:

* ``gpu.GpuContext``  — src/gpu.rs
* ``model.Model``     — the attention helpers of src/model.rs
* ``ops``             — one function per C ABI op
* ``inference``       — the prefill/decode driver loops of src/inference.rs
"""
from ._lib import BF16, F16, F32, LIB_PATH, ShadyError  # noqa: F401

__all__ = ["BF16", "F16", "F32", "LIB_PATH", "ShadyError"]
