"""GPU parity of the glue ops (ops.zig), argmax and the vision preprocessing."""
import numpy as np
import pytest

from conftest import assert_close_ref, f16_normal

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,cols", [(1, 2048), (761, 2048), (729, 1152), (3, 70), (2, 4304), (1, 51200 // 4)])
def test_layernorm(ctx, oracle, rows, cols):
    rng = np.random.default_rng(cols)
    x = f16_normal(rng, (rows, cols), 2.0)
    w, b = f16_normal(rng, (cols,)), f16_normal(rng, (cols,), 0.1)
    assert_close_ref(ctx.layernorm(x, w, b, rows, cols), oracle.layernorm(x, w, b), "layernorm", rel=2e-3)


@pytest.mark.parametrize("rows,cols", [(3645, 1152), (9477, 1152), (4000, 2048), (3000, 72)])
def test_layernorm_with_many_rows_takes_the_packed_form_and_gives_the_same_bits(ctx, oracle, rows, cols):
    """From about 3000 rows on (more than the one-warp-per-row kernel keeps resident) the LayerNorm keeps its row as
    the loaded 16-byte vectors and converts in every pass.  Same operations in the same order: the rows of a large
    call must equal, bit for bit, the same rows normalised in a small call (which takes the other kernel), and the
    whole result the oracle's."""
    rng = np.random.default_rng(rows + cols)
    x = f16_normal(rng, (rows, cols), 2.0)
    w, b = f16_normal(rng, (cols,)), f16_normal(rng, (cols,), 0.1)
    big = ctx.layernorm(x, w, b, rows, cols)
    assert_close_ref(big, oracle.layernorm(x, w, b), "layernorm, many rows", rel=2e-3)
    for lo in (0, rows - 500):
        small = ctx.layernorm(np.ascontiguousarray(x[lo:lo + 500]), w, b, 500, cols)
        np.testing.assert_array_equal(big[lo:lo + 500], small)


def test_layernorm_and_broadcast_add_reference_cases(ctx):
    """The reference's own known-answer cases for the glue (ops_test.zig:1773-1824, 1849-1866, 2547-2640),
    through the C ABI."""
    x = np.array([[-1, 0, 1], [-1, 0, 1]], np.float16)
    w, b = np.ones(3, np.float16), np.zeros(3, np.float16)
    y = ctx.layernorm(x, w, b, 2, 3).astype(np.float32)
    mean = y[0].mean()
    assert abs(mean) < 1e-5 and abs(((y[0] - mean) ** 2).mean() - 1.0) < 0.01
    assert np.isfinite(ctx.layernorm(np.ones((2, 3), np.float16), w, b, 2, 3).astype(np.float32)).all()
    a = np.arange(24, dtype=np.float16).reshape(2, 12)
    bb = (np.arange(12) * 2).astype(np.float16)
    np.testing.assert_allclose(ctx.bias_add(a.copy(), bb, 2, 12).astype(np.float32),
                               (a + bb[None, :]).astype(np.float32), rtol=1e-3)
    a = np.arange(12, dtype=np.float16).reshape(3, 4)
    np.testing.assert_allclose(ctx.bias_add(a.copy(), (np.arange(4) * 2).astype(np.float16), 3, 4).astype(np.float32),
                               [[0, 3, 6, 9], [4, 7, 10, 13], [8, 11, 14, 17]], rtol=1e-3)


def test_gelu_bias_add(ctx, oracle):
    rng = np.random.default_rng(0)
    x = f16_normal(rng, (300, 4304), 2.0)
    got = ctx.gelu(x.copy(), x.size)
    ref = oracle.gelu(x)
    assert np.abs(got.astype(np.float32) - ref.astype(np.float32)).max() <= 2e-3
    b = f16_normal(rng, (4304,))
    np.testing.assert_array_equal(ctx.bias_add(x.copy(), b, 300, 4304), oracle.bias_add(x, b))
    y = f16_normal(rng, (300, 4304))
    np.testing.assert_array_equal(ctx.add(x.copy(), y, x.size), oracle.add(x, y))


def test_argmax_first_maximum(ctx, oracle):
    rng = np.random.default_rng(1)
    x = f16_normal(rng, (51200,))
    assert ctx.argmax(x, x.size) == oracle.argmax(x)
    x[[100, 40000, 51199]] = np.float16(9.0)      # ties: the first index wins (sampling.zig:265-270)
    assert ctx.argmax(x, x.size) == 100
    assert ctx.argmax(np.array([-3.0], np.float16), 1) == 0


@pytest.mark.parametrize("n", [8, 2048, 51200, 65536, 7, 51201, 65544])
def test_argmax_vector_and_scalar_forms(ctx, oracle, n):
    """Rows of a multiple of 8 elements (up to 65536) take 16-byte loads, everything else the scalar kernel: same
    answer as the oracle for random rows, for ties inside one 16-byte vector, across threads and across a thread's
    vectors (the first index wins), for a constant row, a row of -inf and the maximum in the last element."""
    rng = np.random.default_rng(n)
    x = f16_normal(rng, (n,))
    assert ctx.argmax(x, n) == oracle.argmax(x)
    for idx in ([n - 1], [0, n - 1], [n // 2, n // 2 + 1], [3, 5], [n - 3, n // 3]):
        y = x.copy()
        y[idx] = np.float16(11.0)
        assert ctx.argmax(y, n) == min(idx) == oracle.argmax(y)
    if n > 9000:
        y = x.copy()
        y[[1024 * 8 + 17, 17]] = np.float16(11.0)   # the same thread's second and first vector
        assert ctx.argmax(y, n) == 17
    assert ctx.argmax(np.full(n, 2.5, np.float16), n) == 0
    assert ctx.argmax(np.full(n, -np.inf, np.float16), n) == 0


@pytest.mark.parametrize("crops", [1, 2])
def test_preprocess_patchify(ctx, oracle, crops):
    rng = np.random.default_rng(4)
    img = rng.integers(0, 256, (crops, 378, 378, 3), dtype=np.uint8)
    ref = oracle.preprocess_patchify(img).reshape(crops * 729, 588)
    np.testing.assert_array_equal(ctx.preprocess_patchify(img, crops, 378, 378), ref)
    padded = ctx.preprocess_patchify(img, crops, 378, 378, out_stride=592)
    np.testing.assert_array_equal(padded[:, :588], ref)
    assert (padded[:, 588:] == 0).all()
