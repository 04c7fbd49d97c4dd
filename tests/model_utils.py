"""Seeded random-init weights in the reference's layouts (weights.zig:439-478): text matrices
[out,in], vision / projection matrices [in,out]; weights and biases ~N(0,0.02), LayerNorm gamma 1,
beta 0, embeddings ~N(0,0.02)."""
import numpy as np


def _n(rng, shape, std=0.02):
    return (rng.standard_normal(shape, dtype=np.float32) * std).astype(np.float16)


def text_weights(seed, n_layers=24, dim=2048, hidden=8192, vocab=51200):
    rng = np.random.default_rng(seed)
    w = {k: [] for k in ("ln_w", "ln_b", "wqkv", "bqkv", "wout", "bout", "wfc1", "bfc1", "wfc2", "bfc2")}
    for _ in range(n_layers):
        w["ln_w"].append(np.ones(dim, np.float16)); w["ln_b"].append(np.zeros(dim, np.float16))
        w["wqkv"].append(_n(rng, (3 * dim, dim))); w["bqkv"].append(_n(rng, (3 * dim,)))
        w["wout"].append(_n(rng, (dim, dim))); w["bout"].append(_n(rng, (dim,)))
        w["wfc1"].append(_n(rng, (hidden, dim))); w["bfc1"].append(_n(rng, (hidden,)))
        w["wfc2"].append(_n(rng, (dim, hidden))); w["bfc2"].append(_n(rng, (dim,)))
    w["ln_out_w"], w["ln_out_b"] = np.ones(dim, np.float16), np.zeros(dim, np.float16)
    w["lm_w"], w["lm_b"] = _n(rng, (vocab, dim)), _n(rng, (vocab,))
    w["wte"] = _n(rng, (vocab, dim))
    return w


def vision_weights(seed, n_layers=27, dim=1152, hidden=4304, tokens=729, patch_dim=588, proj_hidden=8192,
                   proj_out=2048):
    rng = np.random.default_rng(seed)
    w = {k: [] for k in ("ln1_w", "ln1_b", "wqkv", "bqkv", "wout", "bout", "ln2_w", "ln2_b", "wfc1", "bfc1", "wfc2",
                         "bfc2")}
    for _ in range(n_layers):
        w["ln1_w"].append(np.ones(dim, np.float16)); w["ln1_b"].append(np.zeros(dim, np.float16))
        w["ln2_w"].append(np.ones(dim, np.float16)); w["ln2_b"].append(np.zeros(dim, np.float16))
        w["wqkv"].append(_n(rng, (dim, 3 * dim))); w["bqkv"].append(_n(rng, (3 * dim,)))
        w["wout"].append(_n(rng, (dim, dim))); w["bout"].append(_n(rng, (dim,)))
        w["wfc1"].append(_n(rng, (dim, hidden))); w["bfc1"].append(_n(rng, (hidden,)))
        w["wfc2"].append(_n(rng, (hidden, dim))); w["bfc2"].append(_n(rng, (dim,)))
    w["patch_w"], w["patch_b"] = _n(rng, (patch_dim, dim)), _n(rng, (dim,))
    w["pos_emb"] = _n(rng, (tokens, dim))
    w["norm_w"], w["norm_b"] = np.ones(dim, np.float16), np.zeros(dim, np.float16)
    w["proj_fc1_w"], w["proj_fc1_b"] = _n(rng, (2 * dim, proj_hidden)), _n(rng, (proj_hidden,))
    w["proj_fc2_w"], w["proj_fc2_b"] = _n(rng, (proj_hidden, proj_out)), _n(rng, (proj_out,))
    return w


def top2_gap(logits):
    l = np.asarray(logits, np.float32)
    part = np.partition(l, -2)
    return float(part[-1] - part[-2])
