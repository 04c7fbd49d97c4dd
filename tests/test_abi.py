"""CPU checks of the C-ABI boundary: the library builds for sm_100a, loads, exports every
symbol the header declares, refuses to run without a GPU (no CPU fallback), and maps shape
errors the way the reference's matmul entry points do (hgemm.zig:369-381)."""
import ctypes
import os
import re

import pytest

import __graft_entry__ as entry


def header_symbols():
    inc = os.path.join(entry.ROOT, "include")
    syms = []
    for name in sorted(os.listdir(inc)):
        if name.endswith(".h"):
            text = open(os.path.join(inc, name)).read()
            syms += re.findall(r"^\s*(?:int|const char\*)\s+(md_\w+)\s*\(", text, flags=re.M)
    return syms


def test_build_and_exports(pkg):
    entry.build()
    lib = ctypes.CDLL(pkg.LIB_PATH)
    syms = header_symbols()
    assert len(syms) >= 30
    for s in syms:
        assert hasattr(lib, s), f"{s} declared in include/ but not exported"
    assert os.path.exists(os.path.join(entry.PKG_DIR, "libmoondream_b200.a"))


def test_every_entry_point_cites_the_reference():
    text = open(os.path.join(entry.ROOT, "include", "moondream_b200.h")).read()
    for zig in ("hgemm.zig:362", "hgemm_trans.zig:400", "attention.zig:125", "attention.zig:256",
                "attention.zig:416", "attention.zig:759", "rope.zig:32", "rope.zig:130"):
        assert zig in text, zig


def test_every_option_key_is_documented_in_the_header():
    """md_set_option / md_get_option compare the key against string literals; each of them must appear, quoted, in the
    public header's option list."""
    src = open(os.path.join(entry.PKG_DIR, "csrc", "md_api.cu")).read()
    header = open(os.path.join(entry.ROOT, "include", "moondream_b200.h")).read()
    keys = set()
    for fn in ("int md_set_option(", "int md_get_option("):
        body = src[src.index(fn):]
        body = body[:body.index("\n}\n")]
        keys |= set(re.findall(r'strcmp\(key, "(\w+)"\)', body))
    assert len(keys) >= 20
    undocumented = sorted(k for k in keys if f'"{k}"' not in header)
    assert not undocumented, f"options missing from include/moondream_b200.h: {undocumented}"


def test_no_cpu_fallback_without_gpu(pkg):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(pkg.MdError) as e:
        pkg.Context(0)
    assert e.value.status == 10  # MD_ERR_NO_DEVICE
    assert "no CPU fallback" in str(e.value)


def test_shape_check_error_mapping(pkg):
    lib = pkg.load()

    def check(a, b, t):
        A = (ctypes.c_size_t * len(a))(*a)
        B = (ctypes.c_size_t * len(b))(*b)
        return lib.md_check_matmul_shapes(A, ctypes.c_size_t(len(a)), B, ctypes.c_size_t(len(b)), ctypes.c_int(t))

    assert check((3, 4), (4, 6), 0) == 0
    assert check((3, 4), (5, 6), 0) == 3          # error.IncompatibleTensorShapes (matmul_test.zig:278-290)
    assert check((3, 4), (6, 4), 1) == 0
    assert check((3, 4), (4, 6), 1) == 3
    assert check((3, 4, 1), (4, 6), 0) == 2       # error.InvalidTensorDimension
    assert pkg.ZIG_ERRORS[3] == "error.IncompatibleTensorShapes"
    assert pkg.ZIG_ERRORS[2] == "error.InvalidTensorDimension"
    assert pkg.ZIG_ERRORS[4] == "error.SequenceTooLong"


def test_null_context_is_rejected(pkg):
    lib = pkg.load()
    assert lib.md_sync(ctypes.c_void_p(0)) == 1
    assert lib.md_hgemm_nn(ctypes.c_void_p(0), None, None, None, ctypes.c_size_t(1), ctypes.c_size_t(1),
                           ctypes.c_size_t(1)) == 1
