"""GPU parity of the matmul entry points against the oracle, through the C ABI.

Covers the reference's own hgemm test cases (src/core/matmul_test.zig:154-367, same fill
patterns and comparison rule), the benchmark shapes (config 1, the decode GEMV sweep, vision
and prefill GEMMs) with the north-star tolerance max|gpu - ref| <= 1e-2 * max|ref|, edge
shapes around the tile sizes, and size-independent properties at full size."""
import numpy as np
import pytest

from conftest import assert_close_ref, compare_results_f16, f16_normal

pytestmark = pytest.mark.gpu


def random_pm1(rng, shape, scale=0.01):
    return ((rng.random(shape, np.float32) * 2 - 1).astype(np.float16).astype(np.float32) * scale).astype(np.float16)


# ---- the reference's hgemm tests, run against the GPU library (host pointers = drop-in mode)

def test_ref_basic_sequential(ctx, oracle):
    a = (np.arange(12, dtype=np.float32) * 0.01).astype(np.float16).reshape(4, 3)
    b = (np.arange(12, dtype=np.float32) * 0.01).astype(np.float16).reshape(3, 4)
    compare_results_f16(oracle.naive_matmul_f16(a, b), ctx.hgemm_nn(a, b, 4, 4, 3), 0.005)


def test_ref_large(ctx, oracle):
    rng = np.random.default_rng(42)
    a, b = random_pm1(rng, (2000, 180)), random_pm1(rng, (180, 1600))
    compare_results_f16(oracle.naive_matmul_f16(a, b), ctx.hgemm_nn(a, b, 2000, 1600, 180), 0.05)


@pytest.mark.parametrize("m,k,n", [(50, 30, 70), (25, 80, 35), (100, 20, 100)])
def test_ref_non_square(ctx, oracle, m, k, n):
    rng = np.random.default_rng(m)
    a, b = random_pm1(rng, (m, k)), random_pm1(rng, (k, n))
    compare_results_f16(oracle.naive_matmul_f16(a, b), ctx.hgemm_nn(a, b, m, n, k), 0.05)


def test_ref_identity(ctx):
    a = random_pm1(np.random.default_rng(1), (32, 32))
    compare_results_f16(a, ctx.hgemm_nn(a, np.eye(32, dtype=np.float16), 32, 32, 32), 0.005)


def test_ref_error_case(ctx, pkg):
    with pytest.raises(pkg.MdError) as e:
        ctx.check_matmul_shapes((3, 4), (5, 6), False)
    assert e.value.zig_error == "error.IncompatibleTensorShapes"


@pytest.mark.parametrize("size", [158, 159, 160, 161, 162])
def test_ref_tile_boundaries(ctx, oracle, size):
    rng = np.random.default_rng(size)
    a, b = random_pm1(rng, (size, size)), random_pm1(rng, (size, size))
    compare_results_f16(oracle.naive_matmul_f16(a, b), ctx.hgemm_nn(a, b, size, size, size), 0.05)


@pytest.mark.parametrize("val", [1e-2, 1.0])
def test_ref_constant_matrices(ctx, oracle, val):
    a = np.full((32, 32), val, np.float16)
    compare_results_f16(oracle.naive_matmul_f16(a, a), ctx.hgemm_nn(a, a, 32, 32, 32), 0.01)


# ---- oracle parity, every kernel selected explicitly (mode 1 = SIMT, 2 = tcgen05, 0 = auto)

EDGE = [(1, 8, 8), (7, 16, 24), (8, 64, 8), (9, 72, 40), (127, 128, 136), (128, 64, 128), (129, 200, 264),
        (167, 168, 168), (300, 1152, 520), (64, 592, 1152)]


@pytest.mark.parametrize("layout", ["nn", "nt"])
@pytest.mark.parametrize("m,k,n", EDGE)
@pytest.mark.parametrize("mode", [1, 2])
def test_edge_shapes(ctx, oracle, mode, m, k, n, layout):
    rng = np.random.default_rng(m * 7 + k * 3 + n)
    a = f16_normal(rng, (m, k))
    w_kn = f16_normal(rng, (k, n), 0.05)
    ctx.set_gemm_mode(mode)
    try:
        if layout == "nn":
            got, ref = ctx.hgemm_nn(a, w_kn, m, n, k), oracle.hgemm_nn(a, w_kn)
        else:
            w_nk = np.ascontiguousarray(w_kn.T)
            got, ref = ctx.hgemm_nt(a, w_nk, m, n, k), oracle.hgemm_nt(a, w_nk)
    finally:
        ctx.set_gemm_mode(0)
    assert_close_ref(got, ref, f"mode{mode} {layout} {m}x{n}x{k}")


@pytest.mark.parametrize("m,k,n", [(1, 3, 5), (5, 30, 7), (33, 588, 1152), (3, 7, 9)])
def test_unaligned_shapes_take_the_simt_kernel(ctx, oracle, m, k, n):
    rng = np.random.default_rng(k)
    a, w = f16_normal(rng, (m, k)), f16_normal(rng, (k, n), 0.05)
    assert_close_ref(ctx.hgemm_nn(a, w, m, n, k), oracle.hgemm_nn(a, w), "nn")
    wt = np.ascontiguousarray(w.T)
    assert_close_ref(ctx.hgemm_nt(a, wt, m, n, k), oracle.hgemm_nt(a, wt), "nt")


def test_empty_dims(ctx):
    a = np.zeros((4, 0), np.float16)
    b = np.zeros((0, 8), np.float16)
    out = ctx.hgemm_nn(a, b, 4, 8, 0)
    assert (out == 0).all()


def test_config1_prefill_fc1(ctx, oracle):
    """benchmark config 1: A[64,2048] ~N(0,1), W[2048,8192] ~N(0,0.02), both layouts."""
    rng = np.random.default_rng(1000)
    a, w = f16_normal(rng, (64, 2048)), f16_normal(rng, (2048, 8192), 0.02)
    ref = oracle.hgemm_nn(a, w)
    assert_close_ref(ctx.hgemm_nn(a, w, 64, 8192, 2048), ref, "config1 nn")
    wt = np.ascontiguousarray(w.T)
    assert_close_ref(ctx.hgemm_nt(a, wt, 64, 8192, 2048), oracle.hgemm_nt(a, wt), "config1 nt")


GEMV_SHAPES = [(2048, 6144), (2048, 2048), (2048, 8192), (8192, 2048), (2048, 51200)]


@pytest.mark.parametrize("k,n", GEMV_SHAPES)
@pytest.mark.parametrize("m", [1, 2, 4, 8])
def test_config2_decode_gemv(ctx, oracle, m, k, n):
    """benchmark config 2: M in {1,2,4,8} over the Phi-1.5 layer shapes, weights resident."""
    rng = np.random.default_rng(2000 + m)
    w = f16_normal(rng, (n, k), 0.02)
    a = f16_normal(rng, (m, k))
    wd = ctx.upload(w)
    got = ctx.hgemm_nt(a, wd, m, n, k, out=np.empty((m, n), np.float16))
    wd.free()
    assert_close_ref(got, oracle.hgemm_nt(a, w), f"gemv M={m} {k}->{n}")


@pytest.mark.parametrize("variant", [1, 2, 3, 4, 5, 6])
@pytest.mark.parametrize("m", [1, 5, 8])
def test_gemv_fixed_variants(ctx, oracle, variant, m):
    """Every fixed (warps, unroll) configuration of the GEMV kernel, including the two-warp one whose 64 threads
    take two turns over the 128 outputs of a CTA; N not a multiple of 16, K not a multiple of 32."""
    rng = np.random.default_rng(10 * variant + m)
    k, n = 2056, 1000
    a, w = f16_normal(rng, (m, k)), f16_normal(rng, (n, k), 0.05)
    ctx.set_option("gemv_variant", variant)
    try:
        got = ctx.hgemm_nt(a, w, m, n, k)
    finally:
        ctx.set_option("gemv_variant", 0)
    assert_close_ref(got, oracle.hgemm_nt(a, w), f"gemv variant {variant} M={m}")


@pytest.mark.parametrize("ksplit", [1, 2, 4, 8])
@pytest.mark.parametrize("m,k,n", [(1, 8192, 2048), (8, 2048, 2048), (5, 2056, 1000), (3, 40, 17), (2, 96, 50)])
def test_gemv_split_k(ctx, oracle, ksplit, m, k, n):
    """K split over the CTAs of a cluster (sums added through distributed shared memory): every split count, a K tail,
    K shorter than the split count (the count is clipped), with the fused bias + residual epilogue, twice in a row."""
    rng = np.random.default_rng(ksplit * 100 + m + n)
    a, w = f16_normal(rng, (m, k)), f16_normal(rng, (n, k), 0.05)
    bias, res = f16_normal(rng, (n,), 0.5), f16_normal(rng, (m, n))
    ref = oracle.add(oracle.bias_add(oracle.hgemm_nt(a, w), bias), res)
    da, dw, db, dr = ctx.upload(a), ctx.upload(w), ctx.upload(bias), ctx.upload(res)
    out = ctx.alloc((m, n))
    ctx.set_option("gemv_ksplit", ksplit)
    try:
        for _ in range(2):
            ctx.hgemm_fused(da, dw, out, m, n, k, 1, bias=db, residual=dr)
        ctx.sync()
    finally:
        ctx.set_option("gemv_ksplit", 0)
    assert_close_ref(out.numpy(), ref, f"gemv split-K {ksplit} M={m} {k}->{n}")
    for b in (da, dw, db, dr, out):
        b.free()


@pytest.mark.parametrize("m,k,n", [(3, 2048, 100), (8, 40, 17), (1, 8, 1), (5, 8200, 33)])
def test_gemv_edges(ctx, oracle, m, k, n):
    rng = np.random.default_rng(n)
    a, w = f16_normal(rng, (m, k)), f16_normal(rng, (n, k), 0.05)
    assert_close_ref(ctx.hgemm_nt(a, w, m, n, k), oracle.hgemm_nt(a, w), "gemv edge")


@pytest.mark.parametrize("m,k,n,layout", [(729, 1152, 3456, "nn"), (729, 4304, 1152, "nn"), (729, 1152, 4304, "nn"),
                                          (729, 2304, 8192, "nn"), (761, 2048, 6144, "nt"), (761, 8192, 2048, "nt")])
def test_model_gemm_shapes(ctx, oracle, m, k, n, layout):
    rng = np.random.default_rng(3000 + n)
    a = f16_normal(rng, (m, k))
    if layout == "nn":
        w = f16_normal(rng, (k, n), 0.02)
        got, ref = ctx.hgemm_nn(a, w, m, n, k), oracle.hgemm_nn(a, w)
    else:
        w = f16_normal(rng, (n, k), 0.02)
        got, ref = ctx.hgemm_nt(a, w, m, n, k), oracle.hgemm_nt(a, w)
    assert_close_ref(got, ref, f"{layout} {m}x{n}x{k}")


@pytest.mark.parametrize("layout", [0, 1])
@pytest.mark.parametrize("m,k,n", [(4, 2048, 8192), (200, 1152, 4304), (64, 30, 70)])
def test_fused_epilogue_keeps_reference_rounding(ctx, oracle, m, k, n, layout):
    """bias -> GELU -> residual fused into the GEMM equals the reference's op sequence
    (hgemm, broadcast_add_simd, gelu, add) within the parity bar."""
    rng = np.random.default_rng(m + n)
    a = f16_normal(rng, (m, k))
    w_kn = f16_normal(rng, (k, n), 0.05)
    bias, res = f16_normal(rng, (n,), 0.5), f16_normal(rng, (m, n))
    w = w_kn if layout == 0 else np.ascontiguousarray(w_kn.T)
    ref = oracle.hgemm_nn(a, w_kn) if layout == 0 else oracle.hgemm_nt(a, w)
    ref = oracle.add(oracle.gelu(oracle.bias_add(ref, bias)), res)
    da, dw, db, dr = ctx.upload(a), ctx.upload(w), ctx.upload(bias), ctx.upload(res)
    out = ctx.alloc((m, n))
    ctx.hgemm_fused(da, dw, out, m, n, k, layout, bias=db, gelu=True, residual=dr)
    ctx.sync()
    assert_close_ref(out.numpy(), ref, "fused epilogue")
    for b in (da, dw, db, dr, out):
        b.free()


@pytest.mark.parametrize("layout", [0, 1])
@pytest.mark.parametrize("m,k,n", [(300, 256, 512), (513, 384, 776), (1000, 1152, 4304), (256, 64, 256), (129, 8, 8)])
def test_tile_256x256(ctx, oracle, m, k, n, layout):
    """The 256 x 256 tile (two 128-row sub-tiles sharing one B tile, option tc_block_n = 512), forced on shapes
    with ragged M, N and K, with the fused bias / GELU / residual epilogue, against the oracle and against the
    128 x 256 tile."""
    rng = np.random.default_rng(m + n + k)
    a = f16_normal(rng, (m, k))
    w_kn = f16_normal(rng, (k, n), 0.05)
    bias, res = f16_normal(rng, (n,), 0.5), f16_normal(rng, (m, n))
    w = w_kn if layout == 0 else np.ascontiguousarray(w_kn.T)
    ref = oracle.hgemm_nn(a, w_kn) if layout == 0 else oracle.hgemm_nt(a, w)
    ref = oracle.add(oracle.gelu(oracle.bias_add(ref, bias)), res)
    da, dw, db, dr = ctx.upload(a), ctx.upload(w), ctx.upload(bias), ctx.upload(res)
    outs = {}
    for bn in (512, 256):
        ctx.set_option("tc_block_n", bn)
        try:
            out = ctx.alloc((m, n))
            for _ in range(3):      # consecutive launches: the single accumulator buffer is handed back every tile
                ctx.hgemm_fused(da, dw, out, m, n, k, layout, bias=db, gelu=True, residual=dr)
            ctx.sync()
            outs[bn] = out.numpy()
            out.free()
        finally:
            ctx.set_option("tc_block_n", 0)
    assert_close_ref(outs[512], ref, "256 x 256 tile")
    np.testing.assert_array_equal(outs[512], outs[256])   # same k order, same roundings: identical bits
    for b in (da, dw, db, dr):
        b.free()


@pytest.mark.parametrize("layout", [0, 1])
@pytest.mark.parametrize("splits", [0, 1, 3, 16])
@pytest.mark.parametrize("m,k,n", [(64, 2048, 8192), (9, 520, 1000), (33, 8192, 2048), (40, 64, 136)])
def test_skinny_gemm(ctx, oracle, m, k, n, layout, splits):
    """8 < M <= 64 takes the swapped-operand split-K kernel: both weight layouts, ragged N and K, a K of one
    k-block, every split count (0 = automatic; a request for more splits than k-blocks is clipped), with the fused
    bias / GELU / residual epilogue, three launches in a row (the tile tickets must return to zero), against the
    oracle and against the general tcgen05 kernel."""
    rng = np.random.default_rng(m + n + k + splits)
    a = f16_normal(rng, (m, k))
    w_kn = f16_normal(rng, (k, n), 0.05)
    bias, res = f16_normal(rng, (n,), 0.5), f16_normal(rng, (m, n))
    w = w_kn if layout == 0 else np.ascontiguousarray(w_kn.T)
    ref = oracle.hgemm_nn(a, w_kn) if layout == 0 else oracle.hgemm_nt(a, w)
    ref = oracle.add(oracle.gelu(oracle.bias_add(ref, bias)), res)
    da, dw, db, dr = ctx.upload(a), ctx.upload(w), ctx.upload(bias), ctx.upload(res)
    out = ctx.alloc((m, n))
    ctx.set_option("skinny_splits", splits)
    try:
        for _ in range(3):
            ctx.hgemm_fused(da, dw, out, m, n, k, layout, bias=db, gelu=True, residual=dr)
        ctx.sync()
        assert ctx.get_option("last_tc_tile") >= 1000      # the skinny kernel ran (1000 + number of splits)
        if splits == 1:
            assert ctx.get_option("last_tc_tile") == 1001
    finally:
        ctx.set_option("skinny_splits", 0)
    got = out.numpy()
    assert_close_ref(got, ref, f"skinny {m}x{n}x{k} splits {splits}")
    ctx.set_option("skinny", 0)
    try:
        ctx.hgemm_fused(da, dw, out, m, n, k, layout, bias=db, gelu=True, residual=dr)
        ctx.sync()
        assert ctx.get_option("last_tc_tile") < 1000
    finally:
        ctx.set_option("skinny", 1)
    assert_close_ref(got, out.numpy(), "skinny vs general kernel", rel=2e-3)
    for b in (da, dw, db, dr, out):
        b.free()


@pytest.mark.parametrize("layout", [0, 1])
@pytest.mark.parametrize("m,k,n", [(256, 64, 256), (300, 520, 1000), (1024, 1152, 4304), (129, 8, 8), (100, 64, 264),
                                   (2304, 2048, 2048)])
def test_gemm_on_cta_pairs(ctx, oracle, m, k, n, layout):
    """Option tc_pair: 256 x 256 tiles computed by two CTAs of a cluster (tcgen05 cta_group::2), each loading its own
    rows of A and its half of the B tile.  Ragged M, N and K, a second CTA with one row (M = 129) or none (M = 100),
    more tiles than pairs, the fused bias / GELU / residual epilogue,
    three launches in a row; against the oracle, and bit for bit against the single-CTA kernel (same k order)."""
    rng = np.random.default_rng(m + n + k + layout)
    a = f16_normal(rng, (m, k))
    w_kn = f16_normal(rng, (k, n), 0.05)
    bias, res = f16_normal(rng, (n,), 0.5), f16_normal(rng, (m, n))
    w = w_kn if layout == 0 else np.ascontiguousarray(w_kn.T)
    ref = oracle.hgemm_nn(a, w_kn) if layout == 0 else oracle.hgemm_nt(a, w)
    ref = oracle.add(oracle.gelu(oracle.bias_add(ref, bias)), res)
    da, dw, db, dr = ctx.upload(a), ctx.upload(w), ctx.upload(bias), ctx.upload(res)
    outs = {}
    for pair in (1, 0):
        ctx.set_option("tc_pair", pair)
        try:
            out = ctx.alloc((m, n))
            for _ in range(3):
                ctx.hgemm_fused(da, dw, out, m, n, k, layout, bias=db, gelu=True, residual=dr)
            ctx.sync()
            assert (ctx.get_option("last_tc_tile") == 2256) == (pair == 1)
            outs[pair] = out.numpy()
            out.free()
        finally:
            ctx.set_option("tc_pair", -1)
    assert_close_ref(outs[1], ref, "CTA-pair GEMM")
    np.testing.assert_array_equal(outs[1], outs[0])
    for b in (da, dw, db, dr):
        b.free()


@pytest.mark.parametrize("layout", [0, 1])
@pytest.mark.parametrize("m,k,n,splits", [(761, 8192, 2048, 3), (729, 4304, 1152, 4), (300, 1024, 264, 2),
                                          (129, 2048, 8, 4), (761, 8192, 2048, -1), (2304, 1024, 2048, 2)])
def test_gemm_with_k_split_over_ctas(ctx, oracle, m, k, n, splits, layout):
    """Option tc_splitk: S CTAs per 128 x 256 tile take a range of k-blocks each, leave f32 partial tiles in global
    memory, and the CTA that arrives last at the tile's ticket adds them up in their order and runs the fused
    epilogue.  Ragged M, N and K (a last range shorter than the others), more units than SMs (the last shape), the
    cost model's own choice (-1: it must split the 761 x 2048 x 8192 product), twice in a row with the same bits
    (tickets back at zero, fixed summation order); against the oracle, and close to the unsplit kernel."""
    rng = np.random.default_rng(m + n + k + layout)
    a = f16_normal(rng, (m, k))
    w_kn = f16_normal(rng, (k, n), 0.05)
    bias, res = f16_normal(rng, (n,), 0.5), f16_normal(rng, (m, n))
    w = w_kn if layout == 0 else np.ascontiguousarray(w_kn.T)
    ref = oracle.hgemm_nn(a, w_kn) if layout == 0 else oracle.hgemm_nt(a, w)
    ref = oracle.add(oracle.gelu(oracle.bias_add(ref, bias)), res)
    da, dw, db, dr = ctx.upload(a), ctx.upload(w), ctx.upload(bias), ctx.upload(res)
    outs = {}
    for mode in (splits, 0):
        ctx.set_option("tc_splitk", mode)
        try:
            runs = []
            for _ in range(2):
                out = ctx.alloc((m, n))
                ctx.hgemm_fused(da, dw, out, m, n, k, layout, bias=db, gelu=True, residual=dr)
                ctx.sync()
                runs.append(out.numpy())
                out.free()
            tile = ctx.get_option("last_tc_tile")
            if mode == 0:
                assert tile < 10000
            elif mode > 0:
                assert tile == 10000 * mode + 256, tile
            else:
                assert tile >= 20000 and tile % 10000 == 256, tile
            np.testing.assert_array_equal(runs[0], runs[1])
            outs[mode] = runs[0]
        finally:
            ctx.set_option("tc_splitk", 0)
    assert_close_ref(outs[splits], ref, "split-K GEMM")
    assert_close_ref(outs[splits], outs[0], "split against unsplit", rel=2e-3)
    for b in (da, dw, db, dr):
        b.free()


def test_linearity_at_full_size(ctx):
    """Size-independent property at the lm_head size: (a1 + a2) W == a1 W + a2 W up to rounding,
    and a one-hot activation selects a weight column exactly."""
    rng = np.random.default_rng(5)
    k, n = 2048, 51200
    w = f16_normal(rng, (n, k), 0.02)
    wd = ctx.upload(w)
    onehot = np.zeros((1, k), np.float16)
    onehot[0, 77] = 1.0
    got = ctx.hgemm_nt(onehot, wd, 1, n, k, out=np.empty((1, n), np.float16))
    np.testing.assert_array_equal(got[0], w[:, 77])
    a1, a2 = f16_normal(rng, (1, k), 0.5), f16_normal(rng, (1, k), 0.5)
    s = (a1.astype(np.float32) + a2.astype(np.float32)).astype(np.float16)
    y1 = ctx.hgemm_nt(a1, wd, 1, n, k, out=np.empty((1, n), np.float16)).astype(np.float32)
    y2 = ctx.hgemm_nt(a2, wd, 1, n, k, out=np.empty((1, n), np.float16)).astype(np.float32)
    ys = ctx.hgemm_nt(s, wd, 1, n, k, out=np.empty((1, n), np.float16)).astype(np.float32)
    assert np.abs(ys - (y1 + y2)).max() <= 1e-2 * np.abs(ys).max() + 2e-3
    wd.free()


@pytest.mark.parametrize("m,k,n", [(1, 2048, 6144), (8, 2048, 2048), (8, 8192, 2048), (64, 2048, 512), (3, 2040, 136)])
def test_pinned_host_operands_equal_pageable_ones(ctx, oracle, m, k, n):
    """A caller's buffers in pinned, mapped host memory take two short cuts: a small input (up to 64 KB, a multiple
    of 16 bytes, 16-byte aligned) is fetched by a kernel instead of the copy engine, and a small result is written
    by the GEMM's own stores.  Same bits as the pageable path (which copies both ways), at sizes on both sides of the
    limits and from a pinned buffer at an odd offset (which falls back to the copy)."""
    import ctypes as C
    import torch
    rng = np.random.default_rng(m + k + n)
    a, bt = f16_normal(rng, (m, k)), f16_normal(rng, (n, k), 0.05)
    want = ctx.hgemm_nt(a, bt, m, n, k)                      # numpy arrays: pageable host memory
    assert_close_ref(want, oracle.hgemm_nt(a, bt), "pageable operands")
    dbt = ctx.upload(bt)
    pin = torch.empty(m * k + 8, dtype=torch.float16).pin_memory()
    out = torch.zeros((m, n), dtype=torch.float16).pin_memory()
    sz = C.c_size_t
    for off in (0, 4):                                      # 0: 16-byte aligned; 4 halves = 8 bytes off
        view = pin[off:off + m * k]
        view.copy_(torch.from_numpy(a.reshape(-1)))
        out.zero_()
        ctx._check(ctx.lib.md_hgemm_nt(ctx.h, C.c_void_p(view.data_ptr()), C.c_void_p(dbt.ptr),
                                       C.c_void_p(out.data_ptr()), sz(m), sz(n), sz(k)))
        np.testing.assert_array_equal(out.numpy(), want, err_msg=f"pinned operands, offset {off}")
