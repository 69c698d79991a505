"""CPU-side checks of the C-ABI library: it loads, exports every symbol the
public header declares, and refuses to compute without a CUDA device (there is
no CPU fallback) while still honouring the argument checks that come first."""
import ctypes as C
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def S():
    import slhav2_b200 as mod

    if not os.path.exists(mod.LIB_PATH):
        from slhav2_b200 import build

        build.build()
    return mod


def declared_functions():
    text = open(os.path.join(ROOT, "include", "slha_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(slha_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported_and_bound(S):
    lib = S.load_library()
    names = declared_functions()
    assert len(names) >= 50
    for n in names:
        assert hasattr(lib, n), n
    assert sorted(S.SIGNATURES) == names


def test_layout_introspection(S):
    lib = S.load_library()
    assert lib.slha_abi_version() == 1 and lib.slha_tile_size() == 128 and lib.slha_tile_align() == 64
    assert S.TILE_DTYPE.itemsize == 128
    ctx = lib.slha_init()
    assert ctx and lib.slha_shutdown(ctx) == 0 and lib.slha_shutdown(None) == 0
    bogus = (C.c_uint64 * 1)()
    assert lib.slha_shutdown(C.addressof(bogus)) == S.ERR_INVALID_HANDLE


def test_argument_checks_precede_the_device_check(S):
    lib = S.load_library()
    out = np.zeros(1, np.float32)
    assert lib.slha_process_tile(None, None, None, S.ptr(out)) == S.ERR_NULL
    assert b"NULL" in lib.slha_last_error_message()
    forged = (C.c_uint64 * 1)()
    assert lib.slha_model_dim(C.addressof(forged)) == 0
    assert lib.slha_weights_release(C.addressof(forged)) == S.ERR_INVALID_HANDLE
    t = np.zeros(1, S.TILE_DTYPE)
    t["flags"] = 1 << 7
    assert lib.slha_process_tile(S.ptr(t), S.ptr(np.zeros(128, np.float32)), S.ptr(np.zeros(4, np.uint64)), S.ptr(out)) == S.ERR_INVALID_TILE


def test_no_cpu_fallback(S):
    if S.device_count() > 0:
        pytest.skip("a GPU is present")
    t = np.zeros(1, S.TILE_DTYPE)
    with pytest.raises(S.SlhaError) as e:
        S.process_tile(t, np.zeros(128, np.float32), np.zeros(4, np.uint64))
    assert e.value.code == S.ERR_DEVICE


def test_product_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "slhav2_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                assert "oracle" not in open(os.path.join(dirpath, f)).read().lower(), f


def test_rust_ffi_crate_declares_every_header_function_with_the_same_arity():
    """rust/slha-b200-sys cannot be compiled where this runs (no Rust toolchain), so its extern
    block is held to the header textually: the same function names, the same number of arguments."""
    header = open(os.path.join(ROOT, "include", "slha_b200.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    rust = open(os.path.join(ROOT, "rust", "slha-b200-sys", "src", "lib.rs")).read()
    rust = re.sub(r"//[^\n]*", "", rust)

    def arity(args):
        args = args.strip()
        return 0 if args in ("", "void") else args.count(",") + 1

    c_decl = {m.group(1): arity(m.group(2)) for m in re.finditer(r"\b(slha_[a-z0-9_]+)\s*\(([^()]*)\)\s*;", header)}
    r_decl = {m.group(1): arity(m.group(2)) for m in re.finditer(r"pub fn (slha_[a-z0-9_]+)\s*\(([^()]*)\)", rust)}
    assert sorted(c_decl) == declared_functions()
    assert sorted(r_decl) == sorted(c_decl)
    assert {n: a for n, a in r_decl.items() if c_decl[n] != a} == {}
