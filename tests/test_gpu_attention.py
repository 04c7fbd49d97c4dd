"""GPU parity of the attention, rope and KV-cache entry points against the oracle."""
import numpy as np
import pytest

from conftest import assert_close_ref, f16_normal

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("h,lq,lk,d", [(16, 729, 729, 72), (2, 5, 5, 72), (3, 37, 53, 72), (4, 170, 170, 64),
                                       (2, 64, 64, 64), (2, 65, 63, 64), (1, 1, 9, 8), (2, 33, 40, 48)])
def test_sdpa_maskless(ctx, oracle, h, lq, lk, d):
    rng = np.random.default_rng(lq + d)
    q, k, v = f16_normal(rng, (h, lq, d)), f16_normal(rng, (h, lk, d)), f16_normal(rng, (h, lk, d))
    assert_close_ref(ctx.sdpa_maskless(q, k, v, h, lq, lk, d), oracle.sdpa_maskless(q, k, v), "maskless")


@pytest.mark.parametrize("pos,s", [(0, 1), (0, 7), (5, 1), (16, 37), (100, 3), (0, 761), (300, 70)])
def test_mask_and_masked_sdpa(ctx, oracle, pos, s):
    m = ctx.create_attention_mask(pos, s)
    np.testing.assert_array_equal(m.astype(bool), oracle.create_attention_mask(pos, s)[0])
    rng = np.random.default_rng(pos + s)
    h = 32 if s < 100 else 4
    q, k, v = f16_normal(rng, (h, s, 64)), f16_normal(rng, (h, pos + s, 64)), f16_normal(rng, (h, pos + s, 64))
    got = ctx.sdpa_masked(q, k, v, m, h, s, pos + s, 64)
    assert_close_ref(got, oracle.sdpa_masked(q, k, v, m), "masked")


def test_masked_sdpa_arbitrary_mask(ctx, oracle):
    rng = np.random.default_rng(11)
    q, k, v = f16_normal(rng, (4, 50, 64)), f16_normal(rng, (4, 90, 64)), f16_normal(rng, (4, 90, 64))
    m = (rng.random((50, 90)) > 0.3).astype(np.uint8)
    m[:, 0] = 1  # every row keeps at least one key
    assert_close_ref(ctx.sdpa_masked(q, k, v, m, 4, 50, 90, 64), oracle.sdpa_masked(q, k, v, m), "random mask")


@pytest.mark.parametrize("kv", [1, 2, 63, 127, 128, 129, 762, 961, 2048])
def test_sdpa_single(ctx, oracle, kv):
    rng = np.random.default_rng(kv)
    q, k, v = f16_normal(rng, (32, 1, 64)), f16_normal(rng, (32, kv, 64)), f16_normal(rng, (32, kv, 64))
    m = np.ones(kv, np.uint8)
    assert_close_ref(ctx.sdpa_single(q, k, v, m, kv), oracle.sdpa_single(q, k, v, m), f"single kv={kv}")
    if kv > 2:
        m[1::2] = 0
        assert_close_ref(ctx.sdpa_single(q, k, v, m, kv), oracle.sdpa_single(q, k, v, m), f"single masked kv={kv}")


def test_sdpa_single_too_long(ctx, pkg):
    z = np.zeros((32, 2049, 64), np.float16)
    with pytest.raises(pkg.MdError) as e:
        ctx.sdpa_single(np.zeros((32, 1, 64), np.float16), z, z, np.ones(2049, np.uint8), 2049)
    assert e.value.zig_error == "error.SequenceTooLong"


def test_rope(ctx, oracle, pkg):
    t = ctx.rope_table(32, 2048)
    np.testing.assert_allclose(t, oracle.rope_table(32, 2048), atol=3e-4)
    rng = np.random.default_rng(5)
    x = f16_normal(rng, (32, 9, 64))
    pos = np.arange(700, 709, dtype=np.uint64)
    tt = oracle.rope_table(32, 2048)
    got = ctx.rope_apply(x, tt, pos, 32, 9, 64, 16, 32)
    np.testing.assert_array_equal(got, oracle.rope_apply(x, tt, pos, 32))   # same table -> bit exact
    with pytest.raises(pkg.MdError) as e:
        ctx.rope_apply(x, tt, pos, 32, 9, 64, 16, 30)
    assert e.value.zig_error == "error.InvalidRotationDimension"


def test_kv_cache_roundtrip(ctx, oracle, pkg):
    rng = np.random.default_rng(2)
    kc, vc = ctx.alloc((32, 2048, 64)), ctx.alloc((32, 2048, 64))
    k1, v1 = f16_normal(rng, (32, 5, 64)), f16_normal(rng, (32, 5, 64))
    k2, v2 = f16_normal(rng, (32, 1, 64)), f16_normal(rng, (32, 1, 64))
    ctx.kv_update(kc, vc, k1, v1, 32, 2048, 64, 0, 5)
    ctx.kv_update(kc, vc, k2, v2, 32, 2048, 64, 5, 1)
    k, v = ctx.kv_active(kc, vc, 32, 2048, 64, 6)
    np.testing.assert_array_equal(k, np.concatenate([k1, k2], 1))
    np.testing.assert_array_equal(v, np.concatenate([v1, v2], 1))
    with pytest.raises(pkg.MdError) as e:
        ctx.kv_update(kc, vc, k1, v1, 32, 2048, 64, 2046, 5)
    assert e.value.zig_error == "error.SequenceTooLong"
    kc.free(), vc.free()


def ref_attention_block(oracle, qkv, kc, vc, pos):
    """The reference's sequence text_model.zig:198-294 on the oracle: split, transpose, rope,
    cache update, active cache, mask, SDPA, transpose back. qkv [S, 6144]; caches [32,2048,64]."""
    S = qkv.shape[0]
    q, k, v = [np.ascontiguousarray(qkv[:, i * 2048:(i + 1) * 2048].reshape(S, 32, 64).transpose(1, 0, 2))
               for i in range(3)]
    t = oracle.rope_table(32, 2048)
    ids = np.arange(pos, pos + S)
    qr, kr = oracle.rope_apply(q, t, ids, 32), oracle.rope_apply(k, t, ids, 32)
    n = oracle.kv_update(kc, vc, kr, v, pos)
    ka, va = oracle.kv_active(kc, vc, n)
    m = oracle.create_attention_mask(pos, S)
    o = oracle.sdpa_single(qr, ka, va, m) if S == 1 else oracle.sdpa_masked(qr, ka, va, m)
    return np.ascontiguousarray(o.transpose(1, 0, 2)).reshape(S, 2048)


@pytest.mark.parametrize("prefill", [1, 37, 130])
def test_fused_prefill_then_decode_matches_reference_sequence(ctx, oracle, prefill):
    rng = np.random.default_rng(prefill)
    kc_ref, vc_ref = np.zeros((32, 2048, 64), np.float16), np.zeros((32, 2048, 64), np.float16)
    kc, vc = ctx.upload(kc_ref), ctx.upload(vc_ref)
    qkv = f16_normal(rng, (prefill, 6144))
    ref = ref_attention_block(oracle, qkv, kc_ref, vc_ref, 0)
    out = ctx.alloc((prefill, 2048))
    ctx.sdpa_prefill_fused(ctx.upload(qkv), kc, vc, out, prefill, 32, 64, 2048, 0, 32)
    ctx.sync()
    assert_close_ref(out.numpy(), ref, "prefill fused")
    pos = prefill
    for step in range(4):
        row = f16_normal(rng, (1, 6144))
        ref = ref_attention_block(oracle, row, kc_ref, vc_ref, pos)
        o1 = ctx.alloc((1, 2048))
        ctx.sdpa_decode_fused(ctx.upload(row), kc, vc, o1, 32, 64, 2048, pos, 32)
        ctx.sync()
        assert_close_ref(o1.numpy(), ref, f"decode fused step {step}")
        pos += 1
    # the device cache now equals the reference's cache (K stored after rope, V raw)
    assert_close_ref(kc.numpy()[:, :pos], kc_ref[:, :pos], "key cache", rel=2e-3)
    np.testing.assert_array_equal(vc.numpy()[:, :pos], vc_ref[:, :pos])


def test_fused_chunked_prefill_with_offset(ctx, oracle):
    rng = np.random.default_rng(77)
    kc_ref, vc_ref = np.zeros((32, 2048, 64), np.float16), np.zeros((32, 2048, 64), np.float16)
    kc, vc = ctx.upload(kc_ref), ctx.upload(vc_ref)
    pos = 0
    for S in (70, 3, 200):
        qkv = f16_normal(rng, (S, 6144))
        ref = ref_attention_block(oracle, qkv, kc_ref, vc_ref, pos)
        out = ctx.alloc((S, 2048))
        ctx.sdpa_prefill_fused(ctx.upload(qkv), kc, vc, out, S, 32, 64, 2048, pos, 32)
        ctx.sync()
        assert_close_ref(out.numpy(), ref, f"prefill S={S} pos={pos}")
        pos += S


def test_fused_decode_at_long_context(ctx, oracle):
    rng = np.random.default_rng(9)
    pos = 2047
    kc_ref, vc_ref = f16_normal(rng, (32, 2048, 64)), f16_normal(rng, (32, 2048, 64))
    kc, vc = ctx.upload(kc_ref), ctx.upload(vc_ref)
    row = f16_normal(rng, (1, 6144))
    ref = ref_attention_block(oracle, row, kc_ref, vc_ref, pos)
    out = ctx.alloc((1, 2048))
    ctx.sdpa_decode_fused(ctx.upload(row), kc, vc, out, 32, 64, 2048, pos, 32)
    ctx.sync()
    assert_close_ref(out.numpy(), ref, "decode at 2047")


@pytest.mark.parametrize("pos", [0, 1, 127, 128, 129, 255, 256, 257, 383, 384, 385, 1000, 2047])
def test_fused_decode_with_one_cta_per_head_matches_reference(ctx, oracle, pos):
    """Option decode_loop = 1: one CTA per head walks all keys in turns of 128 (two turns in flight), no merge across
    CTAs.  Positions on both sides of every turn boundary, the empty cache and the last slot, against the oracle's
    rope + cache append + singleMaskedSDPA; the appended k / v rows must land in the cache as well."""
    rng = np.random.default_rng(1000 + pos)
    kc_ref, vc_ref = f16_normal(rng, (32, 2048, 64)), f16_normal(rng, (32, 2048, 64))
    kc_ref[:, pos:], vc_ref[:, pos:] = 0, 0
    kc, vc = ctx.upload(kc_ref), ctx.upload(vc_ref)
    row = f16_normal(rng, (1, 6144))
    ref = ref_attention_block(oracle, row, kc_ref, vc_ref, pos)
    out = ctx.alloc((1, 2048))
    ctx.set_option("decode_loop", 1)
    try:
        ctx.sdpa_decode_fused(ctx.upload(row), kc, vc, out, 32, 64, 2048, pos, 32)
        ctx.sync()
    finally:
        ctx.set_option("decode_loop", -1)
    assert_close_ref(out.numpy(), ref, f"one CTA per head at {pos}")
    assert_close_ref(kc.numpy()[:, pos], kc_ref[:, pos], "appended key", rel=2e-3)
    np.testing.assert_array_equal(vc.numpy()[:, pos], vc_ref[:, pos])


def test_fused_decode_rejects_full_cache(ctx, pkg):
    b = ctx.alloc((32, 2048, 64))
    with pytest.raises(pkg.MdError) as e:
        ctx.sdpa_decode_fused(b, b, b, b, 32, 64, 2048, 2048, 32)
    assert e.value.zig_error == "error.SequenceTooLong"


@pytest.mark.parametrize("crops", [1, 2, 5, 13])
def test_vit_fused_attention(ctx, oracle, crops):
    """qkv [crops*729, 3456] -> per-crop 729-token attention, output [crops*729, 1152]."""
    rng = np.random.default_rng(crops)
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
        assert_close_ref(got[c * T:(c + 1) * T], ref, f"vit crop {c}")
