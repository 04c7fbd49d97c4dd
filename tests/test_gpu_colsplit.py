"""Single-GPU checks of the column-split GEMM pieces: the strided column-block output of
md_hgemm_colsplit_push (no peers) and the all-gather re-layout md_gather_colblocks."""
import ctypes as C

import numpy as np
import pytest

from conftest import assert_close_ref, f16_normal

pytestmark = pytest.mark.gpu
_sz = C.c_size_t


@pytest.mark.parametrize("layout", [0, 1])
def test_colsplit_blocks_fill_the_full_matrix(ctx, oracle, layout):
    rng = np.random.default_rng(layout)
    M, K, N, world = 300, 256, 512, 4
    a = f16_normal(rng, (M, K))
    b = f16_normal(rng, (K, N) if layout == 0 else (N, K), 0.05)
    ref = oracle.hgemm_nn(a, b) if layout == 0 else oracle.hgemm_nt(a, b)
    da, c = ctx.upload(a), ctx.upload(np.zeros((M, N), np.float16))
    w = N // world
    for r in range(world):
        bs = np.ascontiguousarray(b[:, r * w:(r + 1) * w] if layout == 0 else b[r * w:(r + 1) * w])
        dbs = ctx.upload(bs)
        ctx._check(ctx.lib.md_hgemm_colsplit_push(ctx.h, C.c_void_p(da.ptr), C.c_void_p(dbs.ptr), C.c_void_p(c.ptr),
                                                  _sz(M), _sz(w), _sz(K), C.c_int(layout), _sz(N), _sz(r * w), _sz(0),
                                                  None))
    ctx.sync()
    assert_close_ref(c.numpy(), ref, "column blocks")


def test_colsplit_rejects_bad_blocks(ctx, pkg):
    d = ctx.alloc((64, 64))
    st = ctx.lib.md_hgemm_colsplit_push(ctx.h, C.c_void_p(d.ptr), C.c_void_p(d.ptr), C.c_void_p(d.ptr), _sz(64),
                                        _sz(32), _sz(64), C.c_int(1), _sz(64), _sz(48), _sz(0), None)
    assert st == 3      # MD_ERR_SHAPE: the block would leave C
    st = ctx.lib.md_hgemm_colsplit_push(ctx.h, C.c_void_p(d.ptr), C.c_void_p(d.ptr), C.c_void_p(d.ptr), _sz(64),
                                        _sz(32), _sz(64), C.c_int(1), _sz(64), _sz(4), _sz(0), None)
    assert st == 6      # MD_ERR_UNSUPPORTED: offset not a multiple of 8 columns


def test_gather_colblocks(ctx):
    rng = np.random.default_rng(3)
    world, M, n = 4, 37, 24
    g = f16_normal(rng, (world, M, n))
    dg, dc = ctx.upload(g), ctx.alloc((M, world * n))
    ctx._check(ctx.lib.md_gather_colblocks(ctx.h, C.c_void_p(dg.ptr), C.c_void_p(dc.ptr), _sz(world), _sz(M), _sz(n)))
    ctx.sync()
    np.testing.assert_array_equal(dc.numpy(), g.transpose(1, 0, 2).reshape(M, world * n))
