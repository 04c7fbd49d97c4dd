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


def _push(ctx, a, b_slice, c_full, M, w, K, layout, N, off, peers):
    arr = (C.c_void_p * max(len(peers), 1))(*[p.ptr for p in peers])
    ctx._check(ctx.lib.md_hgemm_colsplit_push(ctx.h, C.c_void_p(a.ptr), C.c_void_p(b_slice.ptr), C.c_void_p(c_full.ptr),
                                              _sz(M), _sz(w), _sz(K), C.c_int(layout), _sz(N), _sz(off), _sz(len(peers)),
                                              arr))


# tile: forced tile of the tcgen05 GEMM (0 = the cost model's choice, 512 = 256 x 256, "pair" = 256 x 256 on a CTA pair)
@pytest.mark.parametrize("tile", [0, 64, 128, 256, 512, "pair"])
@pytest.mark.parametrize("shape", [(4096, 256, 4096, 1), (1000, 520, 2000, 0), (300, 256, 512, 1)])
@pytest.mark.parametrize("push_tma", [0, 1], ids=["push_warps", "tma_stores"])
def test_colsplit_push_fills_the_peers_copies(ctx, oracle, tile, shape, push_tma):
    """The push epilogue with peers, on one GPU: the two "ranks" are two calls and every rank's peer buffer is the
    other rank's C in the same device memory, so the dedicated push warps, the tile read-back and the column
    clipping at the block edge run exactly as they do across GPUs.  Several tiles per CTA in the first shape."""
    M, K, N, layout = shape
    pair = tile == "pair"
    tile = 0 if pair else tile
    rng = np.random.default_rng(M + tile + pair)
    world, w = 2, N // 2
    a = f16_normal(rng, (M, K))
    b = f16_normal(rng, (K, N) if layout == 0 else (N, K), 0.05)
    ref = oracle.hgemm_nn(a, b) if layout == 0 else oracle.hgemm_nt(a, b)
    da = ctx.upload(a)
    cs = [ctx.upload(np.full((M, N), 7.0, np.float16)) for _ in range(world)]
    ctx.set_option("tc_block_n", tile)
    ctx.set_option("push_tma", push_tma)   # 1: the epilogue's staged chunks go to the peers as TMA stores
    ctx.set_option("tc_pair", 1 if pair else 0 if tile else -1)
    try:
        for r in range(world):
            bs = np.ascontiguousarray(b[:, r * w:(r + 1) * w] if layout == 0 else b[r * w:(r + 1) * w])
            _push(ctx, da, ctx.upload(bs), cs[r], M, w, K, layout, N, r * w, [cs[1 - r]])
        ctx.sync()
        if pair:
            assert ctx.get_option("last_tc_tile") == 2256
    finally:
        ctx.set_option("tc_block_n", 0)
        ctx.set_option("tc_pair", -1)
        ctx.set_option("push_tma", 1)
    got = [c.numpy() for c in cs]
    np.testing.assert_array_equal(got[0], got[1])       # both copies hold every block, bit for bit
    assert_close_ref(got[0], ref, f"pushed blocks, tile {tile}")


def test_colsplit_push_tile_choice_with_peers(ctx):
    """With peers the cost model must still search the tiles (it once fell back to 128 x 64 for every shape with
    peers): the 8192^3 product split over 8 or 2 GPUs takes a wide tile."""
    M = K = 8192
    da = ctx.alloc((M, K))
    for world, allowed in ((8, (128, 256, 512)), (2, (256, 512))):
        w = 8192 // world
        db, c, peer = ctx.alloc((w, K)), ctx.alloc((M, 8192)), ctx.alloc((M, 8192))
        _push(ctx, da, db, c, M, w, K, 1, 8192, 0, [peer] * (world - 1))
        ctx.sync()
        assert ctx.get_option("last_tc_tile") in allowed + (2256,), (world, ctx.get_option("last_tc_tile"))
        for buf in (db, c, peer):
            buf.free()
    da.free()


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
