"""Writes tests/golden/reference_signatures.json: the `pub fn` signatures of the reference functions the Zig shim
(moondream-zig_b200/host/zig/) replaces, read from a checkout of snowclipsed/moondream-zig.

    python tests/golden/make_reference_signatures.py /path/to/moondream-zig

Signatures are stored whitespace-normalised (see `normalise`); tests/test_zig_shim.py compares every shim
function's signature with them, so a shim that drifts from the reference's parameter list fails on CPU."""
import json
import os
import re
import sys

# shim file -> (reference file, [function names])
SHIM = {
    "hgemm.zig": ("src/core/hgemm.zig", ["matmul"]),
    "hgemm_trans.zig": ("src/core/hgemm_trans.zig", ["matmul"]),
    "attention.zig": ("src/core/attention.zig", ["multiMasklessSDPA", "createAttentionMask", "multiMaskedSDPA",
                                                 "singleMaskedSDPA", "cleanupThreadPool"]),
    "rope.zig": ("src/core/rope.zig", ["precomputeFreqsCis", "applyRotEmb"]),
    "ops_forwards.zig": ("src/core/ops.zig", ["add", "layerNorm", "gelu", "broadcast_add_simd"]),
    "sampling_forwards.zig": ("src/utils/sampling.zig", ["argmax"]),
}


def normalise(sig: str) -> str:
    """One line, single spaces, no space inside the parentheses' edges, no trailing comma before ')'."""
    s = re.sub(r"\s+", " ", sig).strip()
    s = re.sub(r",\s*\)", ")", s)
    s = re.sub(r"\(\s+", "(", s)
    return s


def signatures(text: str) -> dict:
    """{name: (line number, normalised signature)} of every top-level `pub fn` (text up to the body's brace)."""
    out = {}
    for m in re.finditer(r"^pub fn (\w+)\(", text, flags=re.M):
        end = text.index("{", m.end())
        # the return type may itself contain braces only for error sets, which the functions here do not use
        out.setdefault(m.group(1), (text.count("\n", 0, m.start()) + 1, normalise(text[m.start():end])))
    return out


def main():
    ref = sys.argv[1]
    result = {}
    for shim, (path, names) in SHIM.items():
        found = signatures(open(os.path.join(ref, path)).read())
        for name in names:
            line, sig = found[name]
            result[f"{shim}:{name}"] = {"reference_file": path, "line": line, "signature": sig}
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_signatures.json")
    json.dump(result, open(out, "w"), indent=1, sort_keys=True)
    print(f"{len(result)} signatures -> {out}")


if __name__ == "__main__":
    main()
