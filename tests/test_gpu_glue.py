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


@pytest.mark.parametrize("crops", [1, 2])
def test_preprocess_patchify(ctx, oracle, crops):
    rng = np.random.default_rng(4)
    img = rng.integers(0, 256, (crops, 378, 378, 3), dtype=np.uint8)
    ref = oracle.preprocess_patchify(img).reshape(crops * 729, 588)
    np.testing.assert_array_equal(ctx.preprocess_patchify(img, crops, 378, 378), ref)
    padded = ctx.preprocess_patchify(img, crops, 378, 378, out_stride=592)
    np.testing.assert_array_equal(padded[:, :588], ref)
    assert (padded[:, 588:] == 0).all()
