"""CPU tests of the oracle (the C++ restatement of the reference's kernels).

Pins:  the hgemm cases of src/core/matmul_test.zig:154-367 (against the same naive
f32-accumulate product, with the same comparison rule) and the sgemm known answers
(matmul_test.zig:371-400).  Everything else in the oracle has no reference test; those
functions are checked against float64 restatements of their formulas and against
algebraic properties.
"""
import numpy as np
import pytest

from conftest import assert_close_ref, compare_results_f16, f16_normal


def naive_f16(a, b):
    # matmul_test.zig:83-106 in numpy: f32 accumulate in k order, one f16 rounding
    acc = np.zeros((a.shape[0], b.shape[1]), np.float32)
    af, bf = a.astype(np.float32), b.astype(np.float32)
    for k in range(a.shape[1]):
        acc += np.outer(af[:, k], bf[k, :]).astype(np.float32)
    return acc.astype(np.float16)


def random_pm1(rng, shape, scale=0.01):
    return ((rng.random(shape, np.float32) * 2 - 1).astype(np.float16).astype(np.float32) * scale).astype(np.float16)


# ---------------------------------------------------------------- hgemm: the pinned row

def test_hgemm_basic_sequential(oracle):
    a = (np.arange(12, dtype=np.float32) * 0.01).astype(np.float16).reshape(4, 3)
    b = (np.arange(12, dtype=np.float32) * 0.01).astype(np.float16).reshape(3, 4)
    exp = oracle.naive_matmul_f16(a, b)
    np.testing.assert_array_equal(exp, naive_f16(a, b))
    compare_results_f16(exp, oracle.hgemm_nn(a, b), 0.005)


def test_hgemm_large(oracle):
    rng = np.random.default_rng(42)
    a, b = random_pm1(rng, (2000, 180)), random_pm1(rng, (180, 1600))
    compare_results_f16(oracle.naive_matmul_f16(a, b), oracle.hgemm_nn(a, b), 0.05)


@pytest.mark.parametrize("m,k,n", [(50, 30, 70), (25, 80, 35), (100, 20, 100)])
def test_hgemm_non_square(oracle, m, k, n):
    rng = np.random.default_rng(m)
    a, b = random_pm1(rng, (m, k)), random_pm1(rng, (k, n))
    compare_results_f16(oracle.naive_matmul_f16(a, b), oracle.hgemm_nn(a, b), 0.05)


def test_hgemm_identity(oracle):
    rng = np.random.default_rng(1)
    a = random_pm1(rng, (32, 32))
    compare_results_f16(a, oracle.hgemm_nn(a, np.eye(32, dtype=np.float16)), 0.005)


def test_hgemm_error_cases(oracle):
    a = np.zeros((3, 4), np.float16)
    b = np.zeros((5, 6), np.float16)
    with pytest.raises(oracle.OracleError) as e:
        oracle.hgemm_nn(a, b)
    assert e.value.code == oracle.ORC_ERR_INCOMPATIBLE_SHAPES
    with pytest.raises(oracle.OracleError) as e:
        oracle.hgemm_nn(np.zeros((3, 4, 1), np.float16), b)
    assert e.value.code == oracle.ORC_ERR_INVALID_DIMENSION


@pytest.mark.parametrize("size", [158, 159, 160, 161, 162, 167, 168, 169])
def test_hgemm_tile_boundaries(oracle, size):
    rng = np.random.default_rng(size)
    a, b = random_pm1(rng, (size, size)), random_pm1(rng, (size, size))
    compare_results_f16(oracle.naive_matmul_f16(a, b), oracle.hgemm_nn(a, b), 0.05)


@pytest.mark.parametrize("val", [1e-2, 1.0])
def test_hgemm_constant_matrices(oracle, val):
    a = np.full((32, 32), val, np.float16)
    compare_results_f16(oracle.naive_matmul_f16(a, a), oracle.hgemm_nn(a, a), 0.01)


def test_sgemm_known_answers(oracle):
    c = oracle.sgemm([[1, 2], [3, 4]], [[5, 6], [7, 8]])
    np.testing.assert_allclose(c, [[19, 22], [43, 50]], atol=1e-6)
    np.testing.assert_allclose(oracle.sgemm([[3.0]], [[4.0]]), [[12.0]], atol=1e-6)
    a = np.arange(1, 5, dtype=np.float32).reshape(4, 1)
    b = np.arange(1, 4, dtype=np.float32).reshape(1, 3)
    np.testing.assert_allclose(oracle.sgemm(a, b), a @ b, atol=1e-6)
    np.testing.assert_array_equal(oracle.sgemm(np.zeros((5, 7)), np.zeros((7, 3))), np.zeros((5, 3)))


@pytest.mark.parametrize("m,k,n", [(167, 168, 169), (1, 300, 5), (200, 7, 340)])
def test_sgemm_random(oracle, m, k, n):
    rng = np.random.default_rng(k)
    a, b = rng.standard_normal((m, k)).astype(np.float32), rng.standard_normal((k, n)).astype(np.float32)
    np.testing.assert_allclose(oracle.sgemm(a, b), a.astype(np.float64) @ b.astype(np.float64), atol=1e-4 * k ** 0.5)


# ---------------------------------------------------------------- unpinned rows: float64 restatements

@pytest.mark.parametrize("m,k,n", [(1, 2048, 96), (1, 100, 33), (2, 64, 40), (8, 256, 24), (9, 200, 170), (200, 169, 9)])
def test_hgemm_nt_matches_nn_and_float64(oracle, m, k, n):
    rng = np.random.default_rng(m * 1000 + n)
    a, w = f16_normal(rng, (m, k)), f16_normal(rng, (n, k), 0.02)
    got = oracle.hgemm_nt(a, w)
    ref = a.astype(np.float64) @ w.astype(np.float64).T
    assert_close_ref(got, ref, "hgemm_nt", rel=2e-3)
    assert_close_ref(got, oracle.hgemm_nn(a, np.ascontiguousarray(w.T)), "nt vs nn", rel=2e-3)


def sdpa64(q, k, v, mask=None):
    s = np.einsum("hqd,hkd->hqk", q.astype(np.float64), k.astype(np.float64)) / np.sqrt(q.shape[-1])
    if mask is not None:
        s = np.where(mask, s, -np.inf)
    s = np.exp(s - s.max(-1, keepdims=True))
    s /= s.sum(-1, keepdims=True)
    return np.einsum("hqk,hkd->hqd", s, v.astype(np.float64))


@pytest.mark.parametrize("h,lq,lk,d", [(2, 5, 5, 72), (3, 37, 53, 72), (4, 170, 170, 64), (1, 1, 9, 8)])
def test_sdpa_maskless(oracle, h, lq, lk, d):
    rng = np.random.default_rng(lq)
    q, k, v = f16_normal(rng, (h, lq, d)), f16_normal(rng, (h, lk, d)), f16_normal(rng, (h, lk, d))
    assert_close_ref(oracle.sdpa_maskless(q, k, v), sdpa64(q, k, v), "maskless", rel=2e-3)


@pytest.mark.parametrize("pos,s", [(0, 1), (0, 7), (5, 1), (16, 37), (100, 3)])
def test_attention_mask_and_masked_sdpa(oracle, pos, s):
    m = oracle.create_attention_mask(pos, s)
    assert m.shape == (1, s, pos + s)
    i, j = np.mgrid[0:s, 0:pos + s]
    np.testing.assert_array_equal(m[0], j <= pos + i)
    rng = np.random.default_rng(pos + s)
    q, k, v = f16_normal(rng, (4, s, 64)), f16_normal(rng, (4, pos + s, 64)), f16_normal(rng, (4, pos + s, 64))
    assert_close_ref(oracle.sdpa_masked(q, k, v, m), sdpa64(q, k, v, m), "masked", rel=2e-3)


@pytest.mark.parametrize("kv", [1, 2, 63, 64, 65, 762, 2048])
def test_sdpa_single(oracle, kv):
    rng = np.random.default_rng(kv)
    q, k, v = f16_normal(rng, (32, 1, 64)), f16_normal(rng, (32, kv, 64)), f16_normal(rng, (32, kv, 64))
    got = oracle.sdpa_single(q, k, v, np.ones(kv, bool))
    assert_close_ref(got, sdpa64(q, k, v), "single", rel=2e-3)
    # agrees with the multi-token routine on the same data
    assert_close_ref(got, oracle.sdpa_masked(q, k, v, np.ones((1, kv), bool)), "single vs masked", rel=2e-3)


def test_sdpa_single_sequence_too_long(oracle):
    z = np.zeros((32, 2049, 64), np.float16)
    with pytest.raises(oracle.OracleError) as e:
        oracle.sdpa_single(np.zeros((32, 1, 64), np.float16), z, z, np.ones(2049, bool))
    assert e.value.code == oracle.ORC_ERR_SEQUENCE_TOO_LONG


def test_duplicated_crops_equal_per_crop_attention(oracle):
    """The reference attends over both (identical) crops as one 1458-token sequence
    (vision_model.zig:36-38,308-316); that equals 729-token attention per crop."""
    rng = np.random.default_rng(3)
    q, k, v = f16_normal(rng, (2, 60, 72)), f16_normal(rng, (2, 60, 72)), f16_normal(rng, (2, 60, 72))
    dup = lambda x: np.concatenate([x, x], axis=1)
    joint = oracle.sdpa_maskless(dup(q), dup(k), dup(v))
    single = oracle.sdpa_maskless(q, k, v)
    assert_close_ref(joint[:, :60], single, "dup crops", rel=1e-3)
    assert_close_ref(joint[:, 60:], single, "dup crops", rel=1e-3)


def test_softmax_rows(oracle):
    rng = np.random.default_rng(0)
    x = rng.standard_normal((7, 33)).astype(np.float32) * 5
    y = oracle.softmax_rows(x)
    np.testing.assert_allclose(y.sum(-1), 1.0, rtol=1e-5)
    e = np.exp(x.astype(np.float64) - x.max(-1, keepdims=True))
    np.testing.assert_allclose(y, e / e.sum(-1, keepdims=True), rtol=1e-5, atol=1e-7)
    x[0, :] = [-200.0] * 32 + [0.0]          # below the -88 cutoff -> exactly zero
    assert (oracle.softmax_rows(x)[0, :32] == 0).all()


def test_rope_table_and_apply(oracle):
    t = oracle.rope_table(32, 2048)
    assert t.shape == (2048, 16, 2)
    j = np.arange(16)
    freqs = (1.0 / np.float32(10000.0) ** (2 * j / 32).astype(np.float32)).astype(np.float32)
    ang = (np.arange(2048, dtype=np.float32)[:, None] * freqs[None, :]).astype(np.float64)
    np.testing.assert_allclose(t[..., 0], np.cos(ang), atol=2e-4)
    np.testing.assert_allclose(t[..., 1], np.sin(ang), atol=2e-4)
    rng = np.random.default_rng(5)
    x = f16_normal(rng, (32, 6, 64))
    pos = np.arange(11, 17)
    r = oracle.rope_apply(x, t, pos, 32)
    np.testing.assert_array_equal(r[..., 32:], x[..., 32:])          # pass-through tail
    xr, xi = x[..., :16].astype(np.float64), x[..., 16:32].astype(np.float64)
    c, s = t[pos, :, 0][None].astype(np.float64), t[pos, :, 1][None].astype(np.float64)
    np.testing.assert_allclose(r[..., :16], xr * c - xi * s, atol=2e-3)
    np.testing.assert_allclose(r[..., 16:32], xr * s + xi * c, atol=2e-3)
    # rotation preserves the norm of every pair (up to f16 rounding)
    np.testing.assert_allclose(np.hypot(r[..., :16].astype(float), r[..., 16:32].astype(float)), np.hypot(xr, xi),
                               atol=4e-3)
    with pytest.raises(oracle.OracleError) as e:
        oracle.rope_apply(x, t, pos, 30)
    assert e.value.code == oracle.ORC_ERR_INVALID_ROT_DIM


@pytest.mark.parametrize("rows,cols", [(1, 2048), (5, 1152), (3, 70), (2, 64), (4, 4304)])
def test_layernorm(oracle, rows, cols):
    rng = np.random.default_rng(cols)
    x = f16_normal(rng, (rows, cols), 2.0)
    w, b = f16_normal(rng, (cols,), 1.0), f16_normal(rng, (cols,), 0.1)
    x64 = x.astype(np.float64)
    eps = float(np.float16(1e-5))
    ref = (x64 - x64.mean(-1, keepdims=True)) / np.sqrt(x64.var(-1, keepdims=True) + eps) * w.astype(np.float64) + b
    assert_close_ref(oracle.layernorm(x, w, b), ref, "layernorm", rel=2e-3)


def test_layernorm_reference_cases(oracle):
    """The reference's own LayerNorm tests (ops_test.zig:1773-1824 "layerNorm basic functionality" and
    :1849-1866 "zero variance"): rows [-1, 0, 1] with unit weight and zero bias normalise to mean ~ 0 and
    variance ~ 1 within the test's tolerances; a constant row stays finite thanks to epsilon."""
    x = np.array([[-1, 0, 1], [-1, 0, 1]], np.float16)
    w, b = np.ones(3, np.float16), np.zeros(3, np.float16)
    y = oracle.layernorm(x, w, b, np.float16(1e-5)).astype(np.float32)
    assert y.shape == x.shape
    mean = y[0].mean()
    assert abs(mean) < 1e-5
    assert abs(((y[0] - mean) ** 2).mean() - 1.0) < 0.01
    const = oracle.layernorm(np.ones((2, 3), np.float16), w, b, np.float16(1e-5))
    assert np.isfinite(const.astype(np.float32)).all()


def test_broadcast_add_reference_cases(oracle):
    """ops_test.zig:2547-2640 (broadcast_add_simd: positional-embedding, bias and general case) and :1886-1935
    (broadcast_add basic), with the tests' own expected values; relative tolerance 0.001 as there."""
    a = np.arange(24, dtype=np.float16).reshape(2, 12)            # [2,3,4] + [1,3,4]
    b = (np.arange(12) * 2).astype(np.float16)
    got = oracle.bias_add(a, b).astype(np.float32)
    exp = (np.arange(24, dtype=np.float16).reshape(2, 12) + b[None, :]).astype(np.float32)
    np.testing.assert_allclose(got, exp, rtol=1e-3)
    a = np.arange(12, dtype=np.float16).reshape(3, 4)             # [3,4] + [4]
    b = (np.arange(4) * 2).astype(np.float16)
    np.testing.assert_allclose(oracle.bias_add(a, b).astype(np.float32),
                               [[0, 3, 6, 9], [4, 7, 10, 13], [8, 11, 14, 17]], rtol=1e-3)
    a = np.arange(6, dtype=np.float16).reshape(2, 3)              # [2,3] + [1,3]
    b = (np.arange(3) * 2).astype(np.float16)
    np.testing.assert_allclose(oracle.bias_add(a, b).astype(np.float32), [[0, 3, 6], [3, 6, 9]], rtol=1e-3)
    a = np.arange(6, dtype=np.float16).reshape(2, 3)              # [2,3] + [3] of ones
    np.testing.assert_allclose(oracle.bias_add(a, np.ones(3, np.float16)).astype(np.float32), [[1, 2, 3], [4, 5, 6]],
                               atol=1e-6)


def test_gelu_constants_and_values(oracle):
    x = np.linspace(-6, 6, 2001).astype(np.float16)
    c, a = 0.7978515625, 0.044708251953125            # f16(sqrt(f16(2/pi))), f16(0.044715)
    assert float(np.float16(np.sqrt(np.float32(np.float16(np.float16(2.0) / np.float16(np.pi)))))) == c
    assert float(np.float16(0.044715)) == a
    x64 = x.astype(np.float64)
    ref = 0.5 * x64 * (1 + np.tanh(c * (x64 + a * x64 ** 3)))
    got = oracle.gelu(x)
    np.testing.assert_allclose(got.astype(np.float64), ref, atol=2e-3, rtol=1e-3)
    big = oracle.gelu(f16_normal(np.random.default_rng(0), (70000,)))   # threaded path
    assert np.isfinite(big).all()


def test_bias_add_add_argmax(oracle):
    rng = np.random.default_rng(9)
    a, b = f16_normal(rng, (5, 37)), f16_normal(rng, (37,))
    np.testing.assert_array_equal(oracle.bias_add(a, b), (a.astype(np.float32) + b.astype(np.float32)).astype(np.float16))
    c = f16_normal(rng, (5, 37))
    np.testing.assert_array_equal(oracle.add(a, c), (a.astype(np.float32) + c.astype(np.float32)).astype(np.float16))
    assert oracle.argmax(np.array([1, 3, 3, 2], np.float16)) == 1        # first maximum wins
    assert oracle.argmax(np.array([-5], np.float16)) == 0


def test_kv_cache(oracle):
    rng = np.random.default_rng(2)
    kc, vc = np.zeros((32, 2048, 64), np.float16), np.zeros((32, 2048, 64), np.float16)
    k1, v1 = f16_normal(rng, (32, 5, 64)), f16_normal(rng, (32, 5, 64))
    n = oracle.kv_update(kc, vc, k1, v1, 0)
    k2, v2 = f16_normal(rng, (32, 1, 64)), f16_normal(rng, (32, 1, 64))
    n = oracle.kv_update(kc, vc, k2, v2, n)
    assert n == 6
    k, v = oracle.kv_active(kc, vc, n)
    np.testing.assert_array_equal(k, np.concatenate([k1, k2], 1))
    np.testing.assert_array_equal(v, np.concatenate([v1, v2], 1))
    with pytest.raises(oracle.OracleError) as e:
        oracle.kv_update(kc, vc, np.zeros((32, 3, 64), np.float16), np.zeros((32, 3, 64), np.float16), 2046)
    assert e.value.code == oracle.ORC_ERR_SEQUENCE_TOO_LONG


def test_preprocess_patchify(oracle):
    rng = np.random.default_rng(4)
    img = rng.integers(0, 256, (2, 28, 42, 3), dtype=np.uint8)
    p = oracle.preprocess_patchify(img)
    assert p.shape == (2, 6, 588)
    v = img.astype(np.float16)
    v = (v / np.float16(255)).astype(np.float16)
    v = ((v - np.float16(0.5)).astype(np.float16) / np.float16(0.5)).astype(np.float16)
    # patch (1,2) of crop 1, element (c=2, ph=3, pw=5)
    assert p[1, 1 * 3 + 2, (2 * 14 + 3) * 14 + 5] == v[1, 14 + 3, 28 + 5, 2]
    ref = v.reshape(2, 2, 14, 3, 14, 3).transpose(0, 1, 3, 5, 2, 4).reshape(2, 6, 588)
    np.testing.assert_array_equal(p, ref)
