"""CPU side of the golden fixtures (tests/golden): the oracle must reproduce the frozen vectors bit for bit (it is
the checker of every GPU test, so it must not drift) and must satisfy the known answers that the reference's own
tests assert (transcribed into reference_known_answers.json)."""
import json
import os

import numpy as np
import pytest

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.fixture(scope="module")
def vectors():
    z = np.load(os.path.join(GOLDEN, "oracle_vectors.npz"))
    cases = {}
    for key in z.files:
        name, field = key.split("/")
        cases.setdefault(name, {})[field] = z[key]
    return cases


@pytest.fixture(scope="module")
def known():
    with open(os.path.join(GOLDEN, "reference_known_answers.json")) as f:
        return json.load(f)


def test_fixture_generator_is_deterministic(oracle, vectors):
    """Re-running the committed generator gives the committed arrays: same seeds, same oracle."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(GOLDEN, "make_golden.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    fresh = mod.oracle_cases(oracle)
    assert sorted(fresh) == sorted(vectors)
    for name, d in fresh.items():
        for field, val in d.items():
            np.testing.assert_array_equal(np.asarray(val), vectors[name][field], err_msg=f"{name}/{field}")


def test_oracle_meets_the_reference_known_answers(oracle, known):
    c = known["sgemm_2x2"]
    np.testing.assert_allclose(oracle.sgemm(c["a"], c["b"]), c["expected"], atol=c["atol"])
    n = known["hgemm_identity"]["size"]
    a = np.random.default_rng(0).standard_normal((n, n)).astype(np.float16)
    np.testing.assert_array_equal(oracle.hgemm_nn(a, np.eye(n, dtype=np.float16)), a)
    n = known["hgemm_constant"]["size"]
    for val in known["hgemm_constant"]["values"]:
        got = oracle.hgemm_nn(np.full((n, n), val, np.float16), np.full((n, n), val, np.float16)).astype(np.float32)
        np.testing.assert_allclose(got, n * val * val, rtol=1e-2)
    c = known["layernorm_rows"]
    y = oracle.layernorm(np.array(c["x"], np.float16), np.array(c["weight"], np.float16), np.array(c["bias"], np.float16),
                         np.float16(c["eps"])).astype(np.float32)
    assert abs(y[0].mean()) < c["mean_abs_below"]
    assert abs(((y[0] - y[0].mean()) ** 2).mean() - 1.0) < c["variance_within"]
    c = known["layernorm_zero_variance"]
    y = oracle.layernorm(np.array(c["x"], np.float16), np.ones(3, np.float16), np.zeros(3, np.float16), np.float16(1e-5))
    assert np.isfinite(y.astype(np.float32)).all()
    for key, b_of in (("broadcast_add_bias", lambda n: 2 * np.arange(n)), ("broadcast_add_general", lambda n: 2 * np.arange(n)),
                      ("broadcast_add_ones", lambda n: np.ones(n))):
        c = known[key]
        rows, cols = c["a_shape"]
        a = np.arange(rows * cols, dtype=np.float16).reshape(rows, cols)
        got = oracle.bias_add(a, b_of(cols).astype(np.float16)).astype(np.float32)
        np.testing.assert_allclose(got, c["expected"], rtol=c.get("rtol", 0), atol=c.get("atol", 0))
