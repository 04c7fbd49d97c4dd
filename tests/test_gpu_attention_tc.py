"""GPU parity of the two multi-query attention kernels, each forced in turn: the tcgen05 kernel
(option attn_tc = 1) and the mma.sync kernel (attn_tc = 0), against the oracle's
multiMasklessSDPA / multiMaskedSDPA restatements (attention.zig:125-234, 416-541)."""
import numpy as np
import pytest

from conftest import assert_close_ref, f16_normal

pytestmark = pytest.mark.gpu


@pytest.fixture(params=[1, 0], ids=["tcgen05", "mma_sync"])
def forced(ctx, request):
    ctx.set_option("attn_tc", request.param)
    yield request.param
    ctx.set_option("attn_tc", -1)


@pytest.mark.parametrize("h,lq,lk,d", [(16, 729, 729, 72), (2, 5, 5, 72), (3, 37, 53, 72), (4, 170, 170, 64),
                                       (2, 128, 64, 64), (2, 129, 65, 64), (1, 1, 1, 64), (3, 257, 1000, 72),
                                       (1, 300, 2048, 64)])
def test_maskless(ctx, oracle, forced, h, lq, lk, d):
    rng = np.random.default_rng(lq * 7 + lk + d)
    q, k, v = f16_normal(rng, (h, lq, d)), f16_normal(rng, (h, lk, d)), f16_normal(rng, (h, lk, d))
    assert_close_ref(ctx.sdpa_maskless(q, k, v, h, lq, lk, d), oracle.sdpa_maskless(q, k, v), "maskless")


@pytest.mark.parametrize("pos,s", [(0, 1), (0, 7), (16, 37), (0, 761), (300, 70), (63, 130), (1000, 129)])
def test_causal_mask(ctx, oracle, forced, pos, s):
    m = ctx.create_attention_mask(pos, s)
    rng = np.random.default_rng(pos + s)
    h = 32 if s < 100 else 4
    q, k, v = f16_normal(rng, (h, s, 64)), f16_normal(rng, (h, pos + s, 64)), f16_normal(rng, (h, pos + s, 64))
    assert_close_ref(ctx.sdpa_masked(q, k, v, m, h, s, pos + s, 64), oracle.sdpa_masked(q, k, v, m), "masked")


def test_arbitrary_mask(ctx, oracle, forced):
    rng = np.random.default_rng(12)
    q, k, v = f16_normal(rng, (4, 150, 64)), f16_normal(rng, (4, 190, 64)), f16_normal(rng, (4, 190, 64))
    m = (rng.random((150, 190)) > 0.3).astype(np.uint8)
    m[:, 0] = 1  # every row keeps at least one key
    assert_close_ref(ctx.sdpa_masked(q, k, v, m, 4, 150, 190, 64), oracle.sdpa_masked(q, k, v, m), "random mask")


def test_large_scores_stay_finite(ctx, oracle, forced):
    """Scores far from zero: the running-max rescale must keep exp() in range in every tile."""
    rng = np.random.default_rng(5)
    q, k, v = f16_normal(rng, (2, 200, 64), 6.0), f16_normal(rng, (2, 300, 64), 6.0), f16_normal(rng, (2, 300, 64))
    got = ctx.sdpa_maskless(q, k, v, 2, 200, 300, 64)
    assert np.isfinite(got.astype(np.float32)).all()
    assert_close_ref(got, oracle.sdpa_maskless(q, k, v), "large scores")


def test_prefill_ignores_unwritten_cache_rows(ctx, oracle, forced):
    """Cache rows past pos + S hold NaN: no kernel may let them reach the output."""
    from test_gpu_attention import ref_attention_block
    rng = np.random.default_rng(21)
    S = 140
    kc_ref, vc_ref = np.zeros((32, 2048, 64), np.float16), np.zeros((32, 2048, 64), np.float16)
    poison = np.full((32, 2048, 64), np.nan, np.float16)
    kc, vc = ctx.upload(poison), ctx.upload(poison)
    qkv = f16_normal(rng, (S, 6144))
    ref = ref_attention_block(oracle, qkv, kc_ref, vc_ref, 0)
    out = ctx.alloc((S, 2048))
    ctx.sdpa_prefill_fused(ctx.upload(qkv), kc, vc, out, S, 32, 64, 2048, 0, 32)
    ctx.sync()
    got = out.numpy()
    assert np.isfinite(got.astype(np.float32)).all()
    assert_close_ref(got, ref, "prefill over a poisoned cache")


@pytest.mark.parametrize("crops", [1, 3, 13])
def test_vit_layout(ctx, oracle, forced, crops):
    """Heads interleaved inside the packed qkv rows (row stride 3456, head stride 72), one batch per crop."""
    rng = np.random.default_rng(crops + 40)
    T, H, d = 729, 16, 72
    qkv = f16_normal(rng, (crops * T, 3 * H * d))
    out = ctx.alloc((crops * T, H * d))
    ctx.sdpa_vit_fused(ctx.upload(qkv), out, crops, T, H, d)
    ctx.sync()
    got = out.numpy()
    for c in range(crops):
        blk = qkv[c * T:(c + 1) * T]
        q, k, v = [np.ascontiguousarray(blk[:, i * H * d:(i + 1) * H * d].reshape(T, H, d).transpose(1, 0, 2))
                   for i in range(3)]
        ref = np.ascontiguousarray(oracle.sdpa_maskless(q, k, v).transpose(1, 0, 2)).reshape(T, H * d)
        assert_close_ref(got[c * T:(c + 1) * T], ref, f"crop {c}")


_WALK: dict = {}


@pytest.mark.parametrize("per_sm", [0, 1, 2])
def test_ctas_that_walk_several_items_give_the_same_result(ctx, oracle, per_sm):
    """The tcgen05 kernel's grid is capped at attn_ctas_per_sm CTAs per SM; a CTA then walks several (query block,
    head, batch) items, carrying its rings, S / P buffers and wait parities from one item to the next.  13 crops are
    1248 items (4-9 per CTA); the causal case (320 items) has items of 2 to 20 key tiles in one CTA's walk.  per_sm = 0 gives
    every item its own CTA.  All three against the oracle, and bit-equal to one another."""
    ctx.set_option("attn_tc", 1)
    ctx.set_option("attn_ctas_per_sm", per_sm)
    try:
        rng = np.random.default_rng(77)
        crops, T, H, d = 13, 729, 16, 72
        qkv = f16_normal(rng, (crops * T, 3 * H * d))
        out = ctx.alloc((crops * T, H * d))
        ctx.sdpa_vit_fused(ctx.upload(qkv), out, crops, T, H, d)
        ctx.sync()
        got = out.numpy()
        for c in (0, 6, 12):
            blk = qkv[c * T:(c + 1) * T]
            q, k, v = [np.ascontiguousarray(blk[:, i * H * d:(i + 1) * H * d].reshape(T, H, d).transpose(1, 0, 2))
                       for i in range(3)]
            ref = np.ascontiguousarray(oracle.sdpa_maskless(q, k, v).transpose(1, 0, 2)).reshape(T, H * d)
            assert_close_ref(got[c * T:(c + 1) * T], ref, f"crop {c}")
        S = 1230
        qkv2 = f16_normal(rng, (S, 6144))
        kc, vc, o2 = ctx.alloc((32, 2048, 64)), ctx.alloc((32, 2048, 64)), ctx.alloc((S, 2048))
        ctx.sdpa_prefill_fused(ctx.upload(qkv2), kc, vc, o2, S, 32, 64, 2048, 0, 32)
        ctx.sync()
        got2 = o2.numpy()
    finally:
        ctx.set_option("attn_ctas_per_sm", 2)
        ctx.set_option("attn_tc", -1)
    _WALK[per_sm] = (got, got2)
    if per_sm == 0:   # the causal case against the oracle once; the other grids must equal this one bit for bit
        from test_gpu_attention import ref_attention_block
        kc_ref, vc_ref = np.zeros((32, 2048, 64), np.float16), np.zeros((32, 2048, 64), np.float16)
        assert_close_ref(got2, ref_attention_block(oracle, qkv2, kc_ref, vc_ref, 0), "causal prefill of 1230 rows")
    elif 0 in _WALK:
        np.testing.assert_array_equal(got, _WALK[0][0])
        np.testing.assert_array_equal(got2, _WALK[0][1])


def test_forced_tcgen05_rejects_other_head_dims(ctx, pkg):
    ctx.set_option("attn_tc", 1)
    try:
        z = np.zeros((2, 8, 48), np.float16)
        with pytest.raises(pkg.MdError):
            ctx.sdpa_maskless(z, z, z, 2, 8, 8, 48)
    finally:
        ctx.set_option("attn_tc", -1)
