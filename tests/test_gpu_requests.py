"""Independent requests end to end (the box-scale workload's unit of work): image -> vision encode -> prompt
embeddings around the image rows -> prefill -> greedy decode, several requests decoding together.  Checked against
the oracle's restatement of the same chain (moondream.zig:240-368 over vision_model.zig / text_model.zig) under
teacher forcing: the oracle generates, the GPU path is fed the oracle's tokens and must produce the same token at
every step whose top-2 logit gap in the oracle exceeds 0.05."""
import importlib

import numpy as np
import pytest

import __graft_entry__ as entry
from model_utils import text_weights, top2_gap, vision_weights

pytestmark = pytest.mark.gpu


def oracle_request(oracle, vw, tw, req, n_steps):
    """One request through the oracle: returns (first token, its gap, tokens [n_steps], gaps [n_steps])."""
    vis, txt = oracle.VisionModel(vw), oracle.TextModel(tw)
    feats = vis.encoder(oracle.preprocess_patchify(req.crops), joint_attention=False)
    image_rows = vis.projection(feats[0], feats[min(1, len(feats) - 1)])
    embeds = np.concatenate([txt.embed(req.ids[:1]), image_rows, txt.embed(req.ids[1:])])   # moondream.zig:286-303
    logits = txt.lm_head(txt.decoder(embeds))
    first, first_gap = oracle.argmax(logits), top2_gap(logits)
    toks, gaps, cur = [], [], first
    for _ in range(n_steps):
        logits = txt.lm_head(txt.decoder(txt.embed([cur])))
        cur = oracle.argmax(logits)
        toks.append(cur)
        gaps.append(top2_gap(logits))
    return first, first_gap, np.array(toks, np.uint32), np.array(gaps)


@pytest.mark.parametrize("max_streams,vision_capacity", [(3, 1), (8, 1), (8, 4)])
def test_requests_match_the_oracle_under_teacher_forcing(ctx, oracle, pkg, max_streams, vision_capacity):
    par = importlib.import_module(entry.PKG_NAME + ".parallel")
    models = importlib.import_module(entry.PKG_NAME + ".models")
    tw = text_weights(4031, n_layers=2, hidden=1024, vocab=4096)
    vw = vision_weights(3031, n_layers=2)
    # vision_capacity 4: the four images of the group go through the encoder in one pass (md_vision_encode_images)
    tm, vm = models.TextModel(ctx, tw), models.VisionModel(ctx, vw, max_crops=vision_capacity)
    rng = np.random.default_rng(31)
    n_req, n_steps = 4, 10
    requests = [par.Request(rng.integers(0, 256, (1, 378, 378, 3), dtype=np.uint8), rng.integers(0, 4096, 32))
                for _ in range(n_req)]
    ref = [oracle_request(oracle, vw, tw, r, n_steps) for r in requests]
    forced = {i: ref[i][2] for i in range(n_req)}
    served = par.serve_requests(ctx, vm, tm, requests, 1, 0, n_steps, max_streams=max_streams, forced=forced)
    tokens = par.gather_tokens(served, n_req)
    pinned_total = 0
    for i, (first, first_gap, toks, gaps) in enumerate(ref):
        got = tokens[i]
        assert got.shape == (1 + n_steps,)
        if first_gap > 0.05:
            assert got[0] == first, f"request {i}: first token"
        else:
            continue        # the prefill's token was a near tie: the forced continuation started from another token
        pinned = gaps > 0.05
        pinned_total += int(pinned.sum())
        np.testing.assert_array_equal(got[1:][pinned], toks[pinned], err_msg=f"request {i}")
    assert pinned_total >= n_steps     # the check is not vacuous
    tm.close(); vm.close()


def test_images_encoded_together_equal_images_encoded_alone(ctx, oracle, pkg):
    """md_vision_encode_images: n one-crop images in one pass against the oracle (features of an image paired with
    themselves, as the reference's two identical crops) and against one md_vision_encode per image."""
    models = importlib.import_module(entry.PKG_NAME + ".models")
    from conftest import assert_close_ref
    vw = vision_weights(3033, n_layers=2)
    vm = models.VisionModel(ctx, vw, max_crops=3)
    rng = np.random.default_rng(33)
    imgs = rng.integers(0, 256, (3, 378, 378, 3), dtype=np.uint8)
    ref = oracle.VisionModel(vw)
    feats = ref.encoder(oracle.preprocess_patchify(imgs), joint_attention=False)
    for _ in range(3):                  # the third pass replays the captured encode
        together = vm.encode_images(imgs)
    for i in range(3):
        assert_close_ref(together[i], ref.projection(feats[i], feats[i]), f"image {i} vs oracle")
        alone = vm.encode(imgs[i:i + 1])
        assert_close_ref(together[i], alone, f"image {i}: together vs alone", rel=2e-3)
    # a single-image encode after the batched one (another graph, the projection buffers keep their size)
    assert_close_ref(vm.encode(imgs[:1]), ref.projection(feats[0], feats[0]), "single encode afterwards")
    vm.close()


def test_requests_partition_is_the_same_work(ctx, pkg):
    """Serving a request list as rank r of `world` gives, put together, what one rank serving everything gives."""
    par = importlib.import_module(entry.PKG_NAME + ".parallel")
    models = importlib.import_module(entry.PKG_NAME + ".models")
    tw = text_weights(4032, n_layers=2, hidden=512, vocab=2048)
    vw = vision_weights(3032, n_layers=1)
    tm, vm = models.TextModel(ctx, tw), models.VisionModel(ctx, vw, max_crops=1)
    rng = np.random.default_rng(32)
    requests = [par.Request(rng.integers(0, 256, (1, 378, 378, 3), dtype=np.uint8), rng.integers(0, 2048, 32))
                for _ in range(5)]
    # groups of five and groups of two would take different decode attention kernels (another summation order); the
    # partition is what is under test, so both sides use the same one
    ctx.set_option("decode_loop", 0)
    try:
        alone = par.serve_requests(ctx, vm, tm, requests, 1, 0, 5, max_streams=8)
        merged = {}
        for r in range(3):
            merged.update(par.serve_requests(ctx, vm, tm, requests, 3, r, 5, max_streams=2))
    finally:
        ctx.set_option("decode_loop", -1)
    assert sorted(merged) == list(range(5))
    for i in range(5):
        np.testing.assert_array_equal(merged[i], alone[i])
    tm.close(); vm.close()


def test_comm_of_one_rank(ctx, pkg, oracle):
    """The communicator with a single rank needs no NCCL: symmetric allocation, barrier and both column-split forms
    degenerate to the plain GEMM."""
    import ctypes as C
    par = importlib.import_module(entry.PKG_NAME + ".parallel")
    h = C.c_void_p()
    ctx._check(ctx.lib.md_comm_init(ctx.h, C.c_char_p(bytes(128)), C.c_int(0), C.c_int(1), C.byref(h)))
    rng = np.random.default_rng(33)
    M, K, N = 200, 256, 512
    a = (rng.standard_normal((M, K))).astype(np.float16)
    b = (rng.standard_normal((N, K)) * 0.05).astype(np.float16)
    da, db = ctx.upload(a), ctx.upload(b)
    p = C.c_void_p()
    ctx._check(ctx.lib.md_comm_symm_alloc(h, C.c_size_t(M * N * 2), C.byref(p)))
    for fn, dst in ((ctx.lib.md_hgemm_colsplit_fused, p.value), (ctx.lib.md_hgemm_colsplit_allgather, ctx.alloc((M, N)).ptr)):
        ctx._check(fn(h, C.c_void_p(da.ptr), C.c_void_p(db.ptr), C.c_void_p(dst), C.c_size_t(M), C.c_size_t(N),
                      C.c_size_t(K), C.c_int(1)))
        ctx._check(ctx.lib.md_comm_barrier(h))
        out = np.empty((M, N), np.float16)
        ctx._check(ctx.lib.md_memcpy_d2h(ctx.h, C.c_void_p(out.ctypes.data), C.c_void_p(dst), C.c_size_t(out.nbytes)))
        from conftest import assert_close_ref
        assert_close_ref(out, oracle.hgemm_nt(a, b), "one-rank column split")
    st = ctx.lib.md_hgemm_colsplit_fused(h, C.c_void_p(da.ptr), C.c_void_p(db.ptr), C.c_void_p(da.ptr), C.c_size_t(M),
                                         C.c_size_t(N), C.c_size_t(K), C.c_int(1))
    assert st == 1      # MD_ERR_INVALID_ARG: C is not a buffer of this communicator
    ctx._check(ctx.lib.md_comm_symm_free(h, p))
    ctx._check(ctx.lib.md_comm_destroy(h))
