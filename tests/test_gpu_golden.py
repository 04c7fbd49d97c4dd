"""GPU parity against the committed golden vectors (tests/golden/oracle_vectors.npz) and the reference's own
known answers (reference_known_answers.json), through the C ABI: this checker does not depend on the oracle
build of the day.  Tolerance: max|gpu - golden| <= 1e-2 * max|golden| per tensor; bit-exact for the index."""
import json
import os

import numpy as np
import pytest

from conftest import assert_close_ref

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.fixture(scope="module")
def g():
    z = np.load(os.path.join(GOLDEN, "oracle_vectors.npz"))
    cases = {}
    for key in z.files:
        name, field = key.split("/")
        cases.setdefault(name, {})[field] = z[key]
    return cases


def test_matmul_vectors(ctx, g):
    c = g["hgemm_nn"]
    M, K = c["a"].shape
    assert_close_ref(ctx.hgemm_nn(c["a"], c["b"], M, c["b"].shape[1], K), c["c"], "hgemm_nn")
    for name in ("hgemm_nt", "gemv"):
        c = g[name]
        M, K = c["a"].shape
        assert_close_ref(ctx.hgemm_nt(c["a"], c["bt"], M, c["bt"].shape[0], K), c["c"], name)


def test_attention_vectors(ctx, g):
    c = g["sdpa_maskless"]
    h, lq, d = c["q"].shape
    assert_close_ref(ctx.sdpa_maskless(c["q"], c["k"], c["v"], h, lq, c["k"].shape[1], d), c["o"], "maskless")
    c = g["sdpa_masked"]
    h, lq, d = c["q"].shape
    mask = ctx.create_attention_mask(int(c["pos"]), lq)
    np.testing.assert_array_equal(mask.astype(np.uint8), c["mask"])
    assert_close_ref(ctx.sdpa_masked(c["q"], c["k"], c["v"], c["mask"], h, lq, c["k"].shape[1], d), c["o"], "masked")
    c = g["sdpa_single"]
    assert_close_ref(ctx.sdpa_single(c["q"], c["k"], c["v"], c["mask"], c["k"].shape[1]), c["o"], "single")


def test_rope_and_glue_vectors(ctx, g):
    c = g["rope"]
    h, s, d = c["x"].shape
    got = ctx.rope_apply(c["x"], c["table"], c["position_ids"].astype(np.uint64), h, s, d, c["table"].shape[1], 32)
    np.testing.assert_array_equal(got, c["o"])
    np.testing.assert_allclose(ctx.rope_table(32, 64), c["table"], atol=2e-6)
    c = g["layernorm"]
    assert_close_ref(ctx.layernorm(c["x"], c["w"], c["b"], *c["x"].shape), c["y"], "layernorm", rel=2e-3)
    c = g["gelu"]
    assert np.abs(ctx.gelu(c["x"].copy(), c["x"].size).astype(np.float32) - c["y"].astype(np.float32)).max() <= 2e-3
    c = g["bias_add"]
    np.testing.assert_array_equal(ctx.bias_add(c["a"].copy(), c["b"], *c["a"].shape), c["y"])
    c = g["argmax"]
    assert ctx.argmax(c["x"], c["x"].size) == int(c["idx"])


def test_reference_known_answers(ctx):
    with open(os.path.join(GOLDEN, "reference_known_answers.json")) as f:
        known = json.load(f)
    n = known["hgemm_identity"]["size"]
    a = np.random.default_rng(0).standard_normal((n, n)).astype(np.float16)
    np.testing.assert_array_equal(ctx.hgemm_nn(a, np.eye(n, dtype=np.float16), n, n, n), a)
    n = known["hgemm_constant"]["size"]
    for val in known["hgemm_constant"]["values"]:
        m = np.full((n, n), val, np.float16)
        np.testing.assert_allclose(ctx.hgemm_nn(m, m, n, n, n).astype(np.float32), n * val * val, rtol=1e-2)
    c = known["broadcast_add_bias"]
    a = np.arange(12, dtype=np.float16).reshape(3, 4)
    np.testing.assert_allclose(ctx.bias_add(a, (2 * np.arange(4)).astype(np.float16), 3, 4).astype(np.float32),
                               c["expected"], rtol=c["rtol"])
