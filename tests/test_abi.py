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
    assert C.sizeof(_lib.KvCache) == 72


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


# ---- the Rust binding as files: `rust/shady-attn-sys` must say what the header says -------------------------

def _rust_lib():
    return open(os.path.join(ROOT, "rust", "shady-attn-sys", "src", "lib.rs")).read()


def _header_prototypes():
    """name -> number of parameters, from include/shady_attn.h."""
    src = re.sub(r"/\*.*?\*/", "", open(os.path.join(ROOT, "include", "shady_attn.h")).read(), flags=re.S)
    out = {}
    for name, args in re.findall(r"\b(shady_[a-z0-9_]+)\s*\(([^;{]*?)\)\s*;", src, flags=re.S):
        out[name] = len([a for a in args.split(",") if a.strip() and a.strip() != "void"])
    return out


def _header_structs():
    src = re.sub(r"/\*.*?\*/", "", open(os.path.join(ROOT, "include", "shady_attn.h")).read(), flags=re.S)
    out = {}
    for body, name in re.findall(r"typedef struct\s*\{(.*?)\}\s*(shady_\w+)\s*;", src, flags=re.S):
        out[name] = [re.search(r"(\w+)\s*(?:\[\d+\])?$", f.strip()).group(1) for f in body.split(";") if f.strip()]
    return out


def test_rust_extern_block_declares_every_export_with_the_same_arity():
    block = re.search(r'extern "C" \{(.*?)\n\}', _rust_lib(), flags=re.S).group(1)
    rust = {}
    for name, args in re.findall(r"pub fn (shady_\w+)\((.*?)\) ->", block):
        rust[name] = len([a for a in args.split(",") if a.strip()])
    assert rust == _header_prototypes()
    from shady_thinker_b200 import _lib
    assert sorted(rust) == sorted(_lib.EXPORTS)


def test_rust_repr_c_structs_keep_the_header_field_order():
    from shady_thinker_b200 import _lib
    lib_rs = _rust_lib()
    ctypes_of = {"shady_kv_cache": _lib.KvCache, "shady_append_params": _lib.AppendParams,
                 "shady_decode_params": _lib.DecodeParams, "shady_prefill_params": _lib.PrefillParams}
    structs = _header_structs()
    assert set(ctypes_of) <= set(structs)
    for cname, fields in structs.items():
        rname = "".join(w.capitalize() for w in cname.split("_"))
        body = re.search(r"#\[repr\(C\)\]\s*#\[derive\(Clone, Copy\)\]\s*pub struct %s \{(.*?)\}" % rname, lib_rs, flags=re.S)
        assert body, f"{rname} missing or not #[repr(C)]"
        assert re.findall(r"pub (\w+):", body.group(1)) == fields, cname
        if cname in ctypes_of:
            assert [f[0] for f in ctypes_of[cname]._fields_] == fields, cname


def test_rust_bindings_are_what_the_generator_writes():
    import importlib.util
    spec = importlib.util.spec_from_file_location("gen_bindings", os.path.join(ROOT, "rust", "shady-attn-sys", "gen_bindings.py"))
    gen = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(gen)
    assert _rust_lib() == gen.generate(), "run python rust/shady-attn-sys/gen_bindings.py after changing the header"


def test_rust_crate_files_exist_and_build_script_targets_sm_100a():
    crate = os.path.join(ROOT, "rust", "shady-attn-sys")
    for f in ("Cargo.toml", "build.rs", os.path.join("src", "lib.rs")):
        assert os.path.exists(os.path.join(crate, f)), f
    b = open(os.path.join(crate, "build.rs")).read()
    assert "arch=compute_100a,code=sm_100a" in b
    from shady_thinker_b200 import build
    for src in build.SOURCES:
        assert f'"{src}"' in b, f"build.rs does not compile {src}"


def test_listed_prefill_workspace_is_host_arithmetic():
    """`shady_prefill_ragged_workspace_size` touches no device: row-block list + packed token starts + two tensor maps
    per sequence (+ the cos/sin table or the rotated Q for the step from the projections), every part 128-byte aligned."""
    from shady_thinker_b200 import ops
    from shady_thinker_b200._lib import BF16

    def up(v):
        return (v + 127) // 128 * 128

    lens = [300, 1, 129, 515]
    for hd, block in ((128, 256), (256, 128)):
        entries = sum((L + block - 1) // block for L in lens)
        base = up(up(up(entries * 16) + (len(lens) + 1) * 4) + len(lens) * 2 * 128)
        plain = ops.prefill_ragged_workspace_size(seq_lens=lens, head_dim=hd, num_kv_heads=2, num_q_heads=4, dtype=BF16)
        fused = ops.prefill_ragged_workspace_size(seq_lens=lens, head_dim=hd, num_kv_heads=2, num_q_heads=4, dtype=BF16,
                                                  with_append=True)
        assert plain == base
        extra = sum(lens) * 4 * 256 * 2 if hd == 256 else max(lens) * 64 * 8
        assert fused == up(base + extra)
