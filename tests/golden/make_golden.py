"""Writes the golden fixtures of this folder.

Two kinds of fixture:
  reference_known_answers.json  the known-answer cases the reference's own tests contain, transcribed from their
                                text (src/core/matmul_test.zig, src/core/ops_test.zig): inputs and expected
                                outputs exactly as asserted there.  The reference is Zig 0.13 and cannot be built
                                or run where this script runs, so its tests are the only upstream source of
                                golden values for this path.
  oracle_vectors.npz            small seeded cases of every function of the path, computed by the CPU oracle
                                (oracle/) at the time the fixtures were frozen.  They pin the oracle against
                                drift (tests/test_oracle.py replays them bit for bit) and give the GPU tests a
                                checker that does not depend on the oracle build (tests/test_gpu_golden.py).

Run from the repository root:  python tests/golden/make_golden.py
"""
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))


def f16_normal(rng, shape, scale=1.0):
    return (rng.standard_normal(shape) * scale).astype(np.float16)


def oracle_cases(oracle):
    """name -> dict of arrays (inputs and the oracle's outputs). Seeds are fixed; every case is tiny."""
    out = {}
    rng = np.random.default_rng(20240611)
    a, b = f16_normal(rng, (37, 72)), f16_normal(rng, (72, 53), 0.1)
    out["hgemm_nn"] = dict(a=a, b=b, c=oracle.hgemm_nn(a, b))
    a, bt = f16_normal(rng, (5, 96)), f16_normal(rng, (41, 96), 0.1)
    out["hgemm_nt"] = dict(a=a, bt=bt, c=oracle.hgemm_nt(a, bt))
    a, bt = f16_normal(rng, (1, 512)), f16_normal(rng, (24, 512), 0.05)
    out["gemv"] = dict(a=a, bt=bt, c=oracle.hgemm_nt(a, bt))
    q, k, v = f16_normal(rng, (2, 37, 72)), f16_normal(rng, (2, 53, 72)), f16_normal(rng, (2, 53, 72))
    out["sdpa_maskless"] = dict(q=q, k=k, v=v, o=oracle.sdpa_maskless(q, k, v))
    pos, s = 7, 21
    mask = oracle.create_attention_mask(pos, s)[0].astype(np.uint8)
    q, k, v = f16_normal(rng, (2, s, 64)), f16_normal(rng, (2, pos + s, 64)), f16_normal(rng, (2, pos + s, 64))
    out["sdpa_masked"] = dict(q=q, k=k, v=v, mask=mask, pos=np.int64(pos), o=oracle.sdpa_masked(q, k, v, mask))
    kv = 9
    q, k, v = f16_normal(rng, (32, 1, 64)), f16_normal(rng, (32, kv, 64)), f16_normal(rng, (32, kv, 64))
    m1 = np.ones((1, kv), np.uint8)
    out["sdpa_single"] = dict(q=q, k=k, v=v, mask=m1, o=oracle.sdpa_single(q, k, v, m1))
    table = oracle.rope_table(32, 64)
    x = f16_normal(rng, (4, 9, 64))
    pos_ids = np.arange(5, 14, dtype=np.int64)
    out["rope"] = dict(table=table, x=x, position_ids=pos_ids, o=oracle.rope_apply(x, table, pos_ids, 32))
    x, w, bb = f16_normal(rng, (2, 1152), 2.0), f16_normal(rng, (1152,)), f16_normal(rng, (1152,), 0.1)
    out["layernorm"] = dict(x=x, w=w, b=bb, y=oracle.layernorm(x, w, bb))
    x = np.linspace(-5, 5, 257).astype(np.float16)
    out["gelu"] = dict(x=x, y=oracle.gelu(x))
    a, bb = f16_normal(rng, (5, 40)), f16_normal(rng, (40,))
    out["bias_add"] = dict(a=a, b=bb, y=oracle.bias_add(a, bb))
    x = f16_normal(rng, (300,))
    out["argmax"] = dict(x=x, idx=np.int64(oracle.argmax(x)))
    return out


KNOWN_ANSWERS = {
    "source": "snowclipsed/moondream-zig, transcribed from the test files' text",
    "sgemm_2x2": {"ref": "src/core/matmul_test.zig:371-400", "a": [[1, 2], [3, 4]], "b": [[5, 6], [7, 8]],
                  "expected": [[19, 22], [43, 50]], "atol": 1e-6},
    "hgemm_identity": {"ref": "src/core/matmul_test.zig (identity case): A x I == A", "size": 32},
    "hgemm_constant": {"ref": "src/core/matmul_test.zig (constant matrices): C[i][j] == K * a * b", "size": 64,
                       "values": [0.5, 1.0, 2.0]},
    "layernorm_rows": {"ref": "src/core/ops_test.zig:1773-1824", "x": [[-1, 0, 1], [-1, 0, 1]], "weight": [1, 1, 1],
                       "bias": [0, 0, 0], "eps": 1e-5, "mean_abs_below": 1e-5, "variance_within": 0.01},
    "layernorm_zero_variance": {"ref": "src/core/ops_test.zig:1849-1866", "x": [[1, 1, 1], [1, 1, 1]],
                                "expect": "finite"},
    "broadcast_add_bias": {"ref": "src/core/ops_test.zig:2581-2611", "a_shape": [3, 4], "a": "arange", "b": "2*arange(4)",
                           "expected": [[0, 3, 6, 9], [4, 7, 10, 13], [8, 11, 14, 17]], "rtol": 1e-3},
    "broadcast_add_general": {"ref": "src/core/ops_test.zig:2613-2639", "a_shape": [2, 3], "a": "arange",
                              "b": "2*arange(3)", "expected": [[0, 3, 6], [3, 6, 9]], "rtol": 1e-3},
    "broadcast_add_ones": {"ref": "src/core/ops_test.zig:1886-1912", "a_shape": [2, 3], "a": "arange", "b": "ones(3)",
                           "expected": [[1, 2, 3], [4, 5, 6]], "atol": 1e-6},
}


def main():
    from oracle import oracle
    cases = oracle_cases(oracle)
    flat = {f"{name}/{key}": np.asarray(val) for name, d in cases.items() for key, val in d.items()}
    np.savez_compressed(os.path.join(HERE, "oracle_vectors.npz"), **flat)
    with open(os.path.join(HERE, "reference_known_answers.json"), "w") as f:
        json.dump(KNOWN_ANSWERS, f, indent=1)
    size = os.path.getsize(os.path.join(HERE, "oracle_vectors.npz"))
    print(f"wrote {len(flat)} arrays ({size / 1024:.0f} KB) and {len(KNOWN_ANSWERS) - 1} known-answer cases")


if __name__ == "__main__":
    main()
