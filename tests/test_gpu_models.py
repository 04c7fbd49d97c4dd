"""GPU parity of the device-resident model runners against the oracle's restatement of
text_model.zig / vision_model.zig: hidden states and logits within 1e-2 * max|ref|, and identical
greedy tokens (teacher forcing) wherever the oracle's top-2 logit gap exceeds 0.05."""
import numpy as np
import pytest

import __graft_entry__ as entry
from conftest import assert_close_ref
from model_utils import text_weights, top2_gap, vision_weights

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def models_mod(pkg):
    import importlib
    return importlib.import_module(entry.PKG_NAME + ".models")


def run_text_parity(ctx, oracle, models_mod, w, prompt_rows, n_steps, seed):
    rng = np.random.default_rng(seed)
    ref = oracle.TextModel(w)
    gpu = models_mod.TextModel(ctx, w)
    req = gpu.request()
    ids = rng.integers(0, ref.vocab, prompt_rows)
    np.testing.assert_array_equal(gpu.text_encoder(ids), ref.embed(ids))
    embeds = ref.embed(ids)
    # prefill
    h_ref = ref.decoder(embeds)
    l_ref = ref.lm_head(h_ref)
    h_gpu, l_gpu, tok_gpu = gpu.forward(req, embeds)
    assert_close_ref(h_gpu, h_ref, "prefill hidden")
    assert_close_ref(l_gpu, l_ref, "prefill logits")
    tok_ref = oracle.argmax(l_ref)
    if top2_gap(l_ref) > 0.05:
        assert tok_gpu == tok_ref
    assert len(req) == prompt_rows
    # decode: the oracle generates; the GPU is fed the oracle's tokens (teacher forcing)
    ref_tokens, gaps, ref_logits = [], [], []
    cur = tok_ref
    for _ in range(n_steps):
        h = ref.decoder(ref.embed([cur]))
        l = ref.lm_head(h)
        cur = oracle.argmax(l)
        ref_tokens.append(cur); gaps.append(top2_gap(l)); ref_logits.append(l)
    toks, logits = gpu.generate(req, tok_ref, n_steps, forced=np.array(ref_tokens, np.uint32), want_logits=True)
    pinned = np.array(gaps) > 0.05
    assert pinned.sum() >= 1
    np.testing.assert_array_equal(toks[pinned], np.array(ref_tokens)[pinned])
    for i in (0, n_steps // 2, n_steps - 1):
        assert_close_ref(logits[i], ref_logits[i], f"decode logits step {i}")
    assert len(req) == prompt_rows + n_steps
    stats = {"pinned": int(pinned.sum()), "steps": n_steps, "match_all": int((toks == np.array(ref_tokens)).sum())}
    # free-running from the same state reproduces the teacher-forced tokens while they agree
    req.close(); gpu.close()
    return stats


def test_text_small_model(ctx, oracle, models_mod):
    w = text_weights(4001, n_layers=2, hidden=1024, vocab=4096)
    stats = run_text_parity(ctx, oracle, models_mod, w, prompt_rows=37, n_steps=12, seed=1)
    assert stats["match_all"] >= stats["pinned"]


def test_text_prefill_of_one_row_then_decode(ctx, oracle, models_mod):
    w = text_weights(4002, n_layers=2, hidden=512, vocab=2048)
    run_text_parity(ctx, oracle, models_mod, w, prompt_rows=1, n_steps=5, seed=2)


def test_text_free_running_generation_and_graph_reuse(ctx, oracle, models_mod):
    w = text_weights(4003, n_layers=2, hidden=512, vocab=2048)
    gpu = models_mod.TextModel(ctx, w)
    rng = np.random.default_rng(3)
    embeds = w["wte"][rng.integers(0, 2048, 20)]
    outs = []
    for _ in range(2):                      # second pass replays the graph captured by the first
        req = gpu.request() if not outs else req
        req.reset()
        _, _, tok = gpu.forward(req, embeds)
        outs.append(gpu.generate(req, tok, 16))
    np.testing.assert_array_equal(outs[0], outs[1])
    # teacher forcing with its own output changes nothing
    req.reset()
    _, _, tok = gpu.forward(req, embeds)
    np.testing.assert_array_equal(gpu.generate(req, tok, 16, forced=outs[0]), outs[0])
    req.close(); gpu.close()


def test_text_graphs_are_captured_again_when_the_context_moves_its_buffers(ctx, models_mod):
    """A request keeps the CUDA graphs of its decode step and its prefill.  They hold the addresses of the context's
    scratch buffer and rope table; another caller on the same context can make both move (here: a prefill attention
    over a longer cache, which needs a longer rope table and more scratch) and an option can change which kernels a
    step uses.  The runners must notice and capture again: same tokens before and after."""
    w = text_weights(4011, n_layers=2, hidden=512, vocab=2048)
    gpu = models_mod.TextModel(ctx, w)
    rng = np.random.default_rng(11)
    embeds = w["wte"][rng.integers(0, 2048, 24)]
    req = gpu.request()

    def run():
        req.reset()
        _, _, tok = gpu.forward(req, embeds)
        return tok, gpu.generate(req, tok, 12)

    first = [run() for _ in range(3)][-1]          # third pass replays both captured graphs
    # a foreign call on the same context: 4096-position cache -> the rope table is rebuilt, 9 MB of rotated q
    S, heads, d, max_seq = 2304, 32, 64, 4096
    qkv = ctx.upload((rng.standard_normal((S, 3 * heads * d)) * 0.5).astype(np.float16))
    kc, vc, out = ctx.alloc((heads, max_seq, d)), ctx.alloc((heads, max_seq, d)), ctx.alloc((S, heads * d))
    ctx.sdpa_prefill_fused(qkv, kc, vc, out, S, heads, d, max_seq, 0, 32)
    ctx.sync()
    for b in (qkv, kc, vc, out):
        b.free()
    again = run()
    assert again[0] == first[0]
    np.testing.assert_array_equal(again[1], first[1])
    # an option set after the capture takes effect on the next call (and gives the same tokens here)
    ctx.set_option("decode_fork", 0)
    try:
        n0 = ctx.launch_count()
        unforked = run()
        launched = ctx.launch_count() - n0
    finally:
        ctx.set_option("decode_fork", 1)
    assert launched > 0                                # the step was enqueued again, not replayed from the stale graph
    assert unforked[0] == first[0]
    assert (unforked[1] == first[1]).mean() >= 0.8     # other kernels, same rounding points
    req.close(); gpu.close()


def test_text_fused_decode_layer_matches_unfused_kernels(ctx, models_mod):
    """The 3-kernel decode layer (LayerNorm+qkv+fc1, attention, out-proj+fc2+residuals) against the same step
    run as separate LayerNorm / GEMV kernels: same rounding points, so logits agree to the parity bar."""
    w = text_weights(4006, n_layers=3, hidden=8192, vocab=4096)
    gpu = models_mod.TextModel(ctx, w)
    rng = np.random.default_rng(6)
    embeds = w["wte"][rng.integers(0, 4096, 70)]
    res = {}
    for fused in (1, 0):
        ctx.set_option("fused_decode", fused)
        try:
            req = gpu.request()
            _, _, tok = gpu.forward(req, embeds)
            forced = np.arange(1, 9, dtype=np.uint32) * 37 % 4096
            res[fused] = gpu.generate(req, tok, 8, forced=forced, want_logits=True)
            req.close()
        finally:
            ctx.set_option("fused_decode", 1)
    for i in range(8):
        assert_close_ref(res[1][1][i], res[0][1][i], f"fused vs unfused logits step {i}", rel=5e-3)
    gpu.close()


def test_text_forked_prefill_equals_the_sequential_prefill(ctx, models_mod):
    """Option prefill_fork (default on): fc1 -> fc2 as a second kernel chain beside qkv -> rope -> attention, joined
    in the out-projection's epilogue.  Same kernels on the same operands with the same roundings: hidden states and
    logits are bit-identical to the sequential form, for a fresh prompt and for a chunk appended at an offset."""
    w = text_weights(4009, n_layers=3, hidden=8192, vocab=4096)
    gpu = models_mod.TextModel(ctx, w)
    rng = np.random.default_rng(9)
    chunks = [w["wte"][rng.integers(0, 4096, n)] for n in (150, 37)]
    res = {}
    for fork in (1, 0):
        ctx.set_option("prefill_fork", fork)
        try:
            req = gpu.request()
            outs = []
            for c in chunks:
                h, lg, tok = gpu.forward(req, c, want_hidden=True, want_logits=True)
                outs.append((np.array(h), np.array(lg), int(tok)))
            res[fork] = outs
            req.close()
        finally:
            ctx.set_option("prefill_fork", 1)
    for (h1, l1, t1), (h0, l0, t0) in zip(res[1], res[0]):
        np.testing.assert_array_equal(h1, h0)
        np.testing.assert_array_equal(l1, l0)
        assert t1 == t0
    gpu.close()


def test_text_forked_decode_layer_matches_the_three_kernel_layer(ctx, models_mod):
    """Option decode_fork (default on): attention chain and MLP chain of a layer as concurrent kernel chains.
    Same rounding points as the three-kernel layer; single request and a batch."""
    w = text_weights(4008, n_layers=3, hidden=8192, vocab=4096)
    gpu = models_mod.TextModel(ctx, w)
    rng = np.random.default_rng(8)
    prompts = [w["wte"][rng.integers(0, 4096, n)] for n in (40, 3)]
    forced = np.arange(1, 9, dtype=np.uint32) * 43 % 4096
    res, batch_tokens = {}, {}
    for fork in (1, 0):
        ctx.set_option("decode_fork", fork)
        try:
            req = gpu.request()
            _, _, tok = gpu.forward(req, prompts[0])
            res[fork] = gpu.generate(req, tok, 8, forced=forced, want_logits=True)
            req.close()
            reqs = [gpu.request() for _ in prompts]
            firsts = [gpu.forward(r, pr)[2] for r, pr in zip(reqs, prompts)]
            batch_tokens[fork] = np.asarray(gpu.generate_batch(reqs, firsts, 6))
            for r in reqs:
                r.close()
        finally:
            ctx.set_option("decode_fork", 1)
    for i in range(8):
        assert_close_ref(res[1][1][i], res[0][1][i], f"forked vs three-kernel logits step {i}", rel=5e-3)
    assert (batch_tokens[1] == batch_tokens[0]).mean() >= 0.8  # random weights: near-ties may flip a token
    gpu.close()


@pytest.mark.parametrize("parts", [2, 4])
def test_text_split_mlp_decode_layer_matches_the_single_mlp_chain(ctx, oracle, models_mod, parts):
    """Option decode_mlp_split (default 2, single request): the MLP as 2 or 4 independent chains whose f32 partial sums
    of fc2 meet in the out-projection's epilogue (one rounding of the sum, then the bias, as the reference rounds
    fc2's output once).  Against the single MLP chain (logits within the parity bar) and against the oracle."""
    w = text_weights(4012, n_layers=3, hidden=8192, vocab=4096)
    gpu = models_mod.TextModel(ctx, w)
    ref = oracle.TextModel(w)
    rng = np.random.default_rng(12)
    ids = rng.integers(0, 4096, 33)
    forced = np.arange(1, 7, dtype=np.uint32) * 59 % 4096
    res = {}
    for split in (parts, 0):
        ctx.set_option("decode_mlp_split", split)
        try:
            req = gpu.request()
            _, _, tok = gpu.forward(req, ref.embed(ids))
            n0 = ctx.launch_count()
            res[split] = gpu.generate(req, 5, 6, forced=forced, want_logits=True)
            res[split] = res[split] + (ctx.launch_count() - n0,)
            req.close()
        finally:
            ctx.set_option("decode_mlp_split", 2)
    res[1] = res[parts]
    assert res[1][2] > res[0][2]          # more kernels per layer than the five of one MLP chain: the split form ran
    ref.decoder(ref.embed(ids))
    cur = 5
    for i in range(6):
        l_ref = ref.lm_head(ref.decoder(ref.embed([cur])))
        assert_close_ref(res[1][1][i], l_ref, f"split MLP vs oracle, step {i}")
        assert_close_ref(res[1][1][i], res[0][1][i], f"split MLP vs single chain, step {i}", rel=5e-3)
        cur = int(forced[i])
    gpu.close()


@pytest.mark.parametrize("cluster_merge", [1, 0], ids=["cluster_merge", "scratch_merge"])
def test_text_batched_decode_equals_single_requests(ctx, models_mod, cluster_merge):
    """One attention launch serves the whole batch (grid z = request), each request at its own position; both ways
    of merging the key splits (thread-block cluster, or global scratch + arrival counters) are exercised."""
    w = text_weights(4004, n_layers=2, hidden=512, vocab=2048)
    gpu = models_mod.TextModel(ctx, w)
    rng = np.random.default_rng(4)
    prompts = [w["wte"][rng.integers(0, 2048, n)] for n in (5, 130, 33)]
    singles, firsts = [], []
    for p in prompts:
        r = gpu.request()
        _, _, tok = gpu.forward(r, p)
        firsts.append(tok)
        singles.append(gpu.generate(r, tok, 10))
        r.close()
    reqs = [gpu.request() for _ in prompts]
    for r, p in zip(reqs, prompts):
        gpu.forward(r, p)
    ctx.set_option("decode_cluster", cluster_merge)
    try:
        batch = gpu.generate_batch(reqs, firsts, 10)
        r = gpu.request()  # and one single request under the same merge
        _, _, tok = gpu.forward(r, prompts[1])
        again = gpu.generate(r, tok, 10)
        r.close()
    finally:
        ctx.set_option("decode_cluster", -1)
    np.testing.assert_array_equal(batch, np.stack(singles))
    np.testing.assert_array_equal(again, singles[1])
    for r in reqs:
        r.close()
    gpu.close()


def test_text_batched_decode_with_one_cta_per_head_and_request_equals_single_requests(ctx, models_mod):
    """Option decode_loop: the attention of a batched step as one CTA per (head, request) walking all keys (no merge
    across CTAs).  Prompt lengths sit on both sides of the 128-key turn and of the two-turn unroll; 12 steps carry
    some requests across a boundary while decoding.  The single-request runs use the same kernel (same summation
    order), so the tokens must be equal; the kernel itself is checked against the oracle in test_gpu_attention.py."""
    w = text_weights(4024, n_layers=2, hidden=512, vocab=2048)
    gpu = models_mod.TextModel(ctx, w)
    rng = np.random.default_rng(24)
    prompts = [w["wte"][rng.integers(0, 2048, n)] for n in (1, 120, 128, 129, 250, 256, 257, 600)]
    ctx.set_option("decode_loop", 1)   # from one (head, request) pair on
    try:
        singles, firsts = [], []
        for p in prompts:
            r = gpu.request()
            _, _, tok = gpu.forward(r, p)
            firsts.append(tok)
            singles.append(gpu.generate(r, tok, 12))
            r.close()
        reqs = [gpu.request() for _ in prompts]
        for r, p in zip(reqs, prompts):
            gpu.forward(r, p)
        batch = gpu.generate_batch(reqs, firsts, 12)
    finally:
        ctx.set_option("decode_loop", -1)
    np.testing.assert_array_equal(batch, np.stack(singles))
    for r in reqs:
        r.close()
    gpu.close()


@pytest.mark.parametrize("split_ln", [0, 2])
def test_text_batched_decode_with_one_layernorm_kernel_equals_the_fused_kernels(ctx, models_mod, split_ln):
    """From decode_split_ln rows on the LayerNorm runs once as a kernel and plain GEMVs follow; below it every CTA of
    the fused kernels recomputes it.  Both forms must produce the tokens of the single-request runs."""
    w = text_weights(4014, n_layers=2, hidden=512, vocab=2048)
    gpu = models_mod.TextModel(ctx, w)
    rng = np.random.default_rng(14)
    prompts = [w["wte"][rng.integers(0, 2048, n)] for n in (3, 129, 40, 7, 64, 200, 1, 90)]
    singles, firsts = [], []
    for p in prompts:
        r = gpu.request()
        _, _, tok = gpu.forward(r, p)
        firsts.append(tok)
        singles.append(gpu.generate(r, tok, 8))
        r.close()
    reqs = [gpu.request() for _ in prompts]
    for r, p in zip(reqs, prompts):
        gpu.forward(r, p)
    ctx.set_option("decode_split_ln", split_ln)
    ctx.set_option("decode_loop", 0)   # the attention of the single-request runs (same summation order: same tokens)
    try:
        batch = gpu.generate_batch(reqs, firsts, 8)
    finally:
        ctx.set_option("decode_split_ln", 5)
        ctx.set_option("decode_loop", -1)
    np.testing.assert_array_equal(batch, np.stack(singles))
    for r in reqs:
        r.close()
    gpu.close()


def test_text_cache_overflow_is_an_error(ctx, pkg, models_mod):
    w = text_weights(4005, n_layers=1, hidden=256, vocab=512)
    gpu = models_mod.TextModel(ctx, w, max_seq=64)
    req = gpu.request()
    with pytest.raises(pkg.MdError) as e:
        gpu.forward(req, w["wte"][:65])
    assert e.value.zig_error == "error.SequenceTooLong"
    gpu.forward(req, w["wte"][:60])
    with pytest.raises(pkg.MdError):
        gpu.generate(req, 1, 5)
    req.close(); gpu.close()


def test_text_full_config4(ctx, oracle, models_mod):
    """benchmark config 4: 24 layers, prefill of 761 rows (729 image rows + 32 tokens), 200 greedy steps."""
    w = text_weights(4000)
    stats = run_text_parity(ctx, oracle, models_mod, w, prompt_rows=761, n_steps=200, seed=4)
    print("config 4 parity:", stats)
    assert stats["pinned"] >= 100


def run_vision(ctx, oracle, models_mod, w, crops, seed):
    rng = np.random.default_rng(seed)
    img = rng.integers(0, 256, (crops, 378, 378, 3), dtype=np.uint8)
    ref = oracle.VisionModel(w)
    patches = oracle.preprocess_patchify(img)
    f_ref = ref.encoder(patches, joint_attention=False)
    b = min(1, crops - 1)
    o_ref = ref.projection(f_ref[0], f_ref[b])
    gpu = models_mod.VisionModel(ctx, w, max_crops=crops)
    o_gpu, f_gpu = gpu.encode(img, want_features=True)
    assert_close_ref(f_gpu.reshape(f_ref.shape), f_ref, "vision features")
    assert_close_ref(o_gpu, o_ref, "projection output")
    gpu.close()
    return ref, img, o_gpu


def test_vision_small_two_identical_crops_match_the_reference_joint_attention(ctx, oracle, models_mod):
    """The reference feeds two identical crops and attends over both as one sequence
    (vision_model.zig:137-155,308-316); per-crop attention gives the same features."""
    w = vision_weights(3001, n_layers=2)
    rng = np.random.default_rng(7)
    one = rng.integers(0, 256, (1, 378, 378, 3), dtype=np.uint8)
    img = np.concatenate([one, one])
    ref = oracle.VisionModel(w)
    f_joint = ref.encoder(oracle.preprocess_patchify(img), joint_attention=True)
    gpu = models_mod.VisionModel(ctx, w, max_crops=2)
    o_gpu, f_gpu = gpu.encode(img, want_features=True)
    assert_close_ref(f_gpu.reshape(f_joint.shape), f_joint, "features vs joint attention")
    assert_close_ref(o_gpu, ref.projection(f_joint[0], f_joint[1]), "projection")
    gpu.close()


@pytest.mark.parametrize("crops", [1, 5, 13])
def test_vision_small_crops(ctx, oracle, models_mod, crops):
    run_vision(ctx, oracle, models_mod, vision_weights(3002, n_layers=2), crops, seed=crops)


@pytest.mark.parametrize("crops", [1, 5, 13])
def test_vision_full_config3(ctx, oracle, models_mod, crops):
    """benchmark config 3 at full depth (27 layers) for every crop count it names: 1, 5 and 13 crops per image
    (vision_model.zig:204-272 run per crop; features of every crop and the projection output checked)."""
    run_vision(ctx, oracle, models_mod, vision_weights(3000), crops, seed=10 + crops)
