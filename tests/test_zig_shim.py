"""The Zig shim (moondream-zig_b200/host/zig/) must keep the reference's `pub fn` signatures literally, so that
src/model/*.zig compiles against it unchanged.  No Zig toolchain exists here, so this is a text check: every shim
function's signature equals the one recorded from the reference (tests/golden/reference_signatures.json, written by
tests/golden/make_reference_signatures.py), every extern declaration names a function include/moondream_b200.h
declares with the same number of parameters, and the build patch links what the library needs."""
import importlib.util
import json
import os
import re

import __graft_entry__ as entry

ZIG = os.path.join(entry.PKG_DIR, "host", "zig")
GOLDEN = os.path.join(entry.ROOT, "tests", "golden")

spec = importlib.util.spec_from_file_location("make_reference_signatures",
                                              os.path.join(GOLDEN, "make_reference_signatures.py"))
sigs = importlib.util.module_from_spec(spec)
spec.loader.exec_module(sigs)


def test_every_shim_function_has_the_reference_signature():
    golden = json.load(open(os.path.join(GOLDEN, "reference_signatures.json")))
    checked = 0
    for shim, (ref_path, names) in sigs.SHIM.items():
        found = sigs.signatures(open(os.path.join(ZIG, shim)).read())
        for name in names:
            rec = golden[f"{shim}:{name}"]
            assert rec["reference_file"] == ref_path
            assert name in found, f"{shim} lacks pub fn {name} ({ref_path}:{rec['line']})"
            assert found[name][1] == rec["signature"], f"{shim}:{name} differs from {ref_path}:{rec['line']}"
            checked += 1
        # and nothing else public that the reference does not have under that name
        extra = set(found) - set(names)
        assert not extra, f"{shim} exports {extra}, which are not reference functions"
    assert checked == 14


def test_golden_signatures_match_the_reference_checkout_when_present():
    ref = os.environ.get("MOONDREAM_ZIG_CHECKOUT", "")
    if not os.path.isdir(ref):
        return      # the fixture is the record; set MOONDREAM_ZIG_CHECKOUT to a checkout of the reference to re-check it
    golden = json.load(open(os.path.join(GOLDEN, "reference_signatures.json")))
    for shim, (ref_path, names) in sigs.SHIM.items():
        found = sigs.signatures(open(os.path.join(ref, ref_path)).read())
        for name in names:
            rec = golden[f"{shim}:{name}"]
            assert found[name] == (rec["line"], rec["signature"])


def test_extern_declarations_match_the_header():
    header = open(os.path.join(entry.ROOT, "include", "moondream_b200.h")).read()
    decls = {}
    for m in re.finditer(r"^(?:int|const char\*)\s+(md_\w+)\s*\(([^;]*?)\)\s*;", header, flags=re.M | re.S):
        args = [a for a in m.group(2).split(",") if a.strip() and a.strip() != "void"]
        decls[m.group(1)] = len(args)
    backend = open(os.path.join(ZIG, "cuda_backend.zig")).read()
    externs = re.findall(r"pub extern fn (md_\w+)\((.*?)\) ", backend)
    assert len(externs) >= 19
    for name, params in externs:
        assert name in decls, f"{name} is not declared in include/moondream_b200.h"
        assert len([p for p in params.split(",") if p.strip()]) == decls[name], name
    # every hot-path entry point the shim needs is bound
    for need in ("md_hgemm_nn", "md_hgemm_nt", "md_sdpa_maskless", "md_sdpa_masked", "md_sdpa_single",
                 "md_create_attention_mask", "md_rope_table", "md_rope_apply", "md_layernorm", "md_gelu",
                 "md_bias_add", "md_add", "md_argmax"):
        assert need in dict(externs)


def test_shim_uses_zig_0_13_idiom_and_the_build_patch_links_the_library():
    for name in os.listdir(ZIG):
        text = open(os.path.join(ZIG, name)).read()
        if name.endswith(".zig"):
            # builtins renamed or removed after 0.13 must not appear in their later spelling
            assert "@typeInfo(T) != .float" not in text
            assert "std.Random" not in text
    patch = open(os.path.join(ZIG, "build_cuda.zig.patch")).read()
    for need in ("libmoondream_b200.a", "cudart_static", "linkLibCpp", ".cwd_relative"):
        assert need in patch
