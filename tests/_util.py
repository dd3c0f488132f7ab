"""Helpers shared by the GPU parity tests (device memory through torch, compute through the C ABI)."""
import numpy as np
import torch

from shady_thinker_b200 import ops
from shady_thinker_b200._lib import BF16, F16, F32

TORCH_DT = {F32: torch.float32, F16: torch.float16, BF16: torch.bfloat16}
ATOL_F32 = 1e-3      # fp32 I/O: max-abs error bound
RTOL_16 = 2e-2       # fp16/bf16 KV: max|x-ref| / max|ref| bound


def rel_err(x, ref):
    x, ref = np.asarray(x, np.float64), np.asarray(ref, np.float64)
    return float(np.abs(x - ref).max() / max(np.abs(ref).max(), 1e-30))


def to_dev(a, dt=F32):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).cuda().to(TORCH_DT[dt]).contiguous()


def to_host(t):
    return t.detach().float().cpu().numpy()


def rounded(oracle, a, dt):
    """What a tensor holds once stored in dtype dt, as f32 (the oracle's input for 16-bit cases)."""
    if dt == F32:
        return np.asarray(a, np.float32)
    return oracle.round_f16(a) if dt == F16 else oracle.round_bf16(a)


class RaggedCache:
    """Per-sequence K/V allocations + device pointer arrays (the cfg-2 'contiguous per-sequence layout')."""

    def __init__(self, ks, vs, dt):
        self.k = [to_dev(k, dt) for k in ks]
        self.v = [to_dev(v, dt) for v in vs]
        self.k_ptrs = torch.tensor([t.data_ptr() for t in self.k], dtype=torch.int64).cuda()
        self.v_ptrs = torch.tensor([t.data_ptr() for t in self.v], dtype=torch.int64).cuda()
        self.view = ops.KvCacheView(dt, k_ptrs=self.k_ptrs, v_ptrs=self.v_ptrs)


def run_decode(gpu, q, cache_view, lens, *, nh, nkv, hd, num_splits, q_dt=F32, out_dt=F32, want_lse=False, gate=None):
    S = len(lens)
    d_q = to_dev(q, q_dt)
    d_lens = torch.tensor(lens, dtype=torch.int32).cuda()
    d_out = torch.full((S, nh, hd), float("nan"), dtype=TORCH_DT[out_dt], device="cuda")
    d_lse = torch.full((S, nh), float("nan"), dtype=torch.float32, device="cuda") if want_lse else None
    ws_bytes = ops.decode_workspace_size(head_dim=hd, num_kv_heads=nkv, num_q_heads=nh, num_splits=num_splits, num_seqs=S)
    ws = torch.full((max(ws_bytes, 4),), 0xAB, dtype=torch.uint8, device="cuda")   # garbage until initialised
    ops.decode_workspace_init(gpu, ws, ws_bytes, head_dim=hd, num_kv_heads=nkv, num_q_heads=nh, num_splits=num_splits,
                              num_seqs=S)
    torch.cuda.synchronize()
    ops.attn_decode(gpu, q=d_q, cache=cache_view, seq_lens=d_lens, out=d_out, head_dim=hd, num_kv_heads=nkv,
                    num_q_heads=nh, num_seqs=S, num_splits=num_splits, seq_lens_host=lens, q_dtype=q_dt,
                    out_dtype=out_dt, lse=d_lse, gate=gate, workspace=ws, workspace_bytes=ws_bytes)
    gpu.synchronize()
    return (to_host(d_out), to_host(d_lse)) if want_lse else to_host(d_out)
