"""The C-ABI library loads without a GPU and exports every function the header declares."""
import ctypes
import os
import re

from yaxus_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions(path=os.path.join("include", "yaxus_cuda.h")):
    text = open(os.path.join(ROOT, path)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(yx_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported():
    names = declared_functions()
    assert len(names) >= 30
    lib = ctypes.CDLL(_lib.CUDA_LIB)
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/yaxus_cuda.h but not exported"


def test_bindings_match_the_header():
    assert sorted(_lib.SIGNATURES) == declared_functions()
    assert sorted(_lib.HOOK_SIGNATURES) == declared_functions(os.path.join("yaxus_b200", "csrc", "yx_hooks.h"))
    _lib.cuda_lib()   # binds every signature; raises on a missing symbol


def header_arity(path=os.path.join("include", "yaxus_cuda.h")):
    """name -> number of parameters, for every function the header declares."""
    text = open(os.path.join(ROOT, path)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    out = {}
    for m in re.finditer(r"\b(yx_[a-z0-9_]+)\s*\(([^;{]*?)\)\s*;", text):
        args = m.group(2).strip()
        out[m.group(1)] = 0 if args in ("", "void") else args.count(",") + 1
    return out


def test_rust_ffi_block_matches_the_header():
    # crates/yaxus-backend-cuda/src/ffi.rs (uncompiled: no rustc here) must declare every header
    # entry, with the same number of parameters, and nothing the header lacks.
    text = open(os.path.join(ROOT, "crates", "yaxus-backend-cuda", "src", "ffi.rs")).read()
    text = re.sub(r"//.*", "", text)
    block = text[text.index('extern "C"'):]
    rust = {}
    for m in re.finditer(r"pub fn (yx_[a-z0-9_]+)\s*\(([^;]*?)\)\s*(?:->\s*[^;]+)?;", block, flags=re.S):
        args = m.group(2).strip()
        rust[m.group(1)] = 0 if not args else len([a for a in args.split(",") if a.strip()])
    assert rust == header_arity()
    # the structs passed by pointer have the header's fields, in order
    for c_name, fields in (("yx_tuning", _lib.Tuning._fields_), ("yx_plan_info", _lib.PlanInfo._fields_)):
        body = text[text.index(f"pub struct {c_name}"):]
        body = body[:body.index("}")]
        assert re.findall(r"pub (\w+):", body) == [f[0] for f in fields], c_name


def test_struct_sizes():
    assert ctypes.sizeof(_lib.Rope) == 65 * 4
    assert ctypes.sizeof(_lib.Layer) == 66 * 4
    assert ctypes.sizeof(_lib.Tuning) == 52
    assert ctypes.sizeof(_lib.PlanInfo) == 48


def test_no_device_means_an_error_not_a_fallback():
    import torch
    if torch.cuda.is_available():
        return
    L = _lib.cuda_lib()
    ctx = ctypes.c_void_p()
    assert L.yx_ctx_create(0, None, ctypes.byref(ctx)) != 0
    assert not ctx.value
    # null handles are rejected, not dereferenced
    assert L.yx_sync(None) == _lib.YX_ERR_INVALID
    assert L.yx_attend(None, None, 0, None, 0, 32, 0, None, 0) == _lib.YX_ERR_INVALID


def test_product_does_not_touch_the_oracle():
    # The oracle is test infrastructure: nothing in the package may import, load or link it.
    pkg = os.path.join(ROOT, "yaxus_b200")
    for root, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cpp", ".h", ".hpp")):
                text = open(os.path.join(root, f)).read()
                assert "yx_ref" not in text and "libyx_oracle" not in text and "yxref_" not in text, f
