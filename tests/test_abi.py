"""CPU checks of the boundary: the library loads, exports every symbol the header declares,
and the ctypes structs have the header's sizes.  No compute calls (no GPU here)."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from shady_thinker_b200 import _lib, build
    build.build()
    return _lib.load()


def _declared():
    src = open(os.path.join(ROOT, "include", "shady_attn.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(shady_[a-z0-9_]+)\s*\(", src)))


def test_every_declared_symbol_is_exported(lib):
    from shady_thinker_b200 import _lib
    names = _declared()
    assert len(names) >= 20
    for n in names:
        assert hasattr(lib, n), f"{n} declared in shady_attn.h but not exported"
    assert sorted(_lib.EXPORTS) == names


def test_struct_sizes_match_header():
    from shady_thinker_b200 import _lib
    assert C.sizeof(_lib.DecodeParams) == 32      # same size as the reference's 8 x u32 Params
    assert C.sizeof(_lib.AppendParams) == 64
    assert C.sizeof(_lib.PrefillParams) == 24
    assert C.sizeof(_lib.KvCache) == 64


def test_ctx_create_fails_cleanly_without_a_gpu(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    h = C.c_void_p()
    st = lib.shady_ctx_create(0, None, C.byref(h))
    assert st != 0 and not h.value
    assert lib.shady_last_error(None)


def test_workspace_size_is_host_only(lib):
    from shady_thinker_b200 import ops
    assert ops.decode_workspace_size(head_dim=128, num_kv_heads=8, num_q_heads=32, num_splits=1, num_seqs=32) == 0
    n = ops.decode_workspace_size(head_dim=128, num_kv_heads=2, num_q_heads=16, num_splits=4, num_seqs=1)
    assert n >= 16 * 4 * 130 * 4
    assert ops.decode_workspace_size(head_dim=128, num_kv_heads=8, num_q_heads=32, num_splits=0, num_seqs=32) > 0


def test_model_config_rotary_dim():
    from shady_thinker_b200.model import ModelConfig
    assert ModelConfig(16, 2).rotary_dim == 32          # 128 * 0.25 (weights.rs defaults)
    assert ModelConfig(16, 2, head_dim=256).rotary_dim == 64
    assert ModelConfig(16, 2, partial_rotary_factor=1.0).rotary_dim == 128
