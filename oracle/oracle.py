"""ctypes binding of the CPU oracle (test infrastructure, never the product path).

The oracle is the C++ restatement of the reference's CPU kernels in
``moondream_oracle.cpp``.  Only the tests, the smoke check and the CPU-baseline
leg of the benchmark may import this module.  All f16 arrays are numpy
``float16``; shapes follow the reference's tensors.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libmoondream_oracle.so")

ORC_OK = 0
ORC_ERR_INVALID_DIMENSION = -1
ORC_ERR_INCOMPATIBLE_SHAPES = -2
ORC_ERR_SEQUENCE_TOO_LONG = -3
ORC_ERR_INVALID_ROT_DIM = -4
ORC_ERR_INVALID_ARG = -5


class OracleError(RuntimeError):
    def __init__(self, code: int, what: str):
        super().__init__(f"{what}: oracle status {code}")
        self.code = code


def build(force: bool = False) -> str:
    """Compile the oracle with its Makefile if the shared object is missing or stale."""
    src = os.path.join(_HERE, "moondream_oracle.cpp")
    hdr = os.path.join(_HERE, "moondream_oracle.h")
    stale = (not os.path.exists(_LIB_PATH)) or any(
        os.path.getmtime(p) > os.path.getmtime(_LIB_PATH) for p in (src, hdr))
    if force or stale:
        subprocess.check_call(["make", "-C", _HERE, "-B", "libmoondream_oracle.so"],
                              stdout=subprocess.DEVNULL)
    return _LIB_PATH


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(_LIB_PATH)
        _lib.orc_set_threads.argtypes = [C.c_int]
        _lib.orc_get_threads.restype = C.c_int
    return _lib


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def _h(a) -> np.ndarray:
    a = np.ascontiguousarray(a)
    assert a.dtype == np.float16, a.dtype
    return a


def _check(rc: int, what: str):
    if rc != 0:
        raise OracleError(rc, what)


def set_threads(n: int) -> None:
    lib().orc_set_threads(int(n))


def get_threads() -> int:
    return int(lib().orc_get_threads())


_sz = C.c_size_t


def hgemm_nn(a, b):
    """hgemm.zig:362-426. a [M,K], b [K,N] -> [M,N]."""
    a, b = _h(a), _h(b)
    if a.ndim != 2 or b.ndim != 2:
        raise OracleError(ORC_ERR_INVALID_DIMENSION, "hgemm_nn")
    if b.shape[0] != a.shape[1]:
        raise OracleError(ORC_ERR_INCOMPATIBLE_SHAPES, "hgemm_nn")
    M, K = a.shape
    N = b.shape[1]
    c = np.empty((M, N), np.float16)
    _check(lib().orc_hgemm_nn(_p(a), _p(b), _p(c), _sz(M), _sz(N), _sz(K)), "hgemm_nn")
    return c


def hgemm_nt(a, b_t):
    """hgemm_trans.zig:400-488. a [M,K], b_t [N,K] -> [M,N]."""
    a, b_t = _h(a), _h(b_t)
    if a.ndim != 2 or b_t.ndim != 2:
        raise OracleError(ORC_ERR_INVALID_DIMENSION, "hgemm_nt")
    if b_t.shape[1] != a.shape[1]:
        raise OracleError(ORC_ERR_INCOMPATIBLE_SHAPES, "hgemm_nt")
    M, K = a.shape
    N = b_t.shape[0]
    c = np.empty((M, N), np.float16)
    _check(lib().orc_hgemm_nt(_p(a), _p(b_t), _p(c), _sz(M), _sz(N), _sz(K)), "hgemm_nt")
    return c


def naive_matmul_f16(a, b):
    """matmul_test.zig:83-106."""
    a, b = _h(a), _h(b)
    M, K = a.shape
    N = b.shape[1]
    c = np.empty((M, N), np.float16)
    _check(lib().orc_naive_matmul_f16(_p(a), _p(b), _p(c), _sz(M), _sz(N), _sz(K)), "naive")
    return c


def sgemm(a, b):
    a = np.ascontiguousarray(a, np.float32)
    b = np.ascontiguousarray(b, np.float32)
    M, K = a.shape
    N = b.shape[1]
    c = np.empty((M, N), np.float32)
    _check(lib().orc_sgemm(_p(a), _p(b), _p(c), _sz(M), _sz(N), _sz(K)), "sgemm")
    return c


def softmax_rows(x):
    x = np.array(x, np.float32, copy=True, order="C")
    rows = int(np.prod(x.shape[:-1]))
    _check(lib().orc_softmax_rows(_p(x), _sz(rows), _sz(x.shape[-1])), "softmax")
    return x


def sdpa_maskless(q, k, v):
    """attention.zig:125-234. q [h,Lq,d], k,v [h,Lk,d]."""
    q, k, v = _h(q), _h(k), _h(v)
    h, lq, d = q.shape
    lk = k.shape[1]
    out = np.empty_like(q)
    _check(lib().orc_sdpa_maskless(_p(q), _p(k), _p(v), _p(out), _sz(h), _sz(lq), _sz(lk), _sz(d)), "sdpa_maskless")
    return out


def create_attention_mask(pos: int, seq_len: int):
    """attention.zig:256-281 -> bool [1, seq_len, pos+seq_len]."""
    m = np.zeros((seq_len, pos + seq_len), np.uint8)
    _check(lib().orc_create_attention_mask(_p(m), _sz(pos), _sz(seq_len)), "mask")
    return m.astype(bool)[None]


def sdpa_masked(q, k, v, mask):
    """attention.zig:416-541."""
    q, k, v = _h(q), _h(k), _h(v)
    h, lq, d = q.shape
    lk = k.shape[1]
    m = np.ascontiguousarray(np.asarray(mask).reshape(lq, lk).astype(np.uint8))
    out = np.empty_like(q)
    _check(lib().orc_sdpa_masked(_p(q), _p(k), _p(v), _p(m), _p(out), _sz(h), _sz(lq), _sz(lk), _sz(d)),
           "sdpa_masked")
    return out


def sdpa_single(q, k, v, mask):
    """attention.zig:759-811. q [32,1,64], k,v [32,kv,64], mask [.., kv]."""
    q, k, v = _h(q), _h(k), _h(v)
    kv = k.shape[1]
    m = np.ascontiguousarray(np.asarray(mask).reshape(-1)[:kv].astype(np.uint8))
    out = np.empty((32, 1, 64), np.float16)
    _check(lib().orc_sdpa_single(_p(q), _p(k), _p(v), _p(m), _p(out), _sz(kv)), "sdpa_single")
    return out


def rope_table(dim: int, end: int, theta: float = 10000.0):
    """rope.zig:32-128 -> f32 [end, dim/2, 2]."""
    t = np.empty((end, dim // 2, 2), np.float32)
    _check(lib().orc_rope_table(_p(t), _sz(dim), _sz(end), C.c_float(theta)), "rope_table")
    return t


def rope_apply(x, freqs_cis, position_ids, rot_dim: int):
    """rope.zig:130-272. x [h,S,d]."""
    x = _h(x)
    if x.ndim != 3:
        raise OracleError(ORC_ERR_INVALID_DIMENSION, "rope_apply")
    h, s, d = x.shape
    f = np.ascontiguousarray(freqs_cis, np.float32)
    pos = np.ascontiguousarray(position_ids, np.uint64)
    out = np.empty_like(x)
    _check(lib().orc_rope_apply(_p(x), _p(out), _sz(h), _sz(s), _sz(d), _p(f), _sz(f.shape[-2]), _p(pos),
                                _sz(rot_dim)), "rope_apply")
    return out


EPS_F16 = np.float16(1e-5)


def layernorm(x, w, b, eps=EPS_F16):
    """ops.zig:1063-1419 over the last dim."""
    x, w, b = _h(x), _h(w), _h(b)
    cols = x.shape[-1]
    rows = x.size // cols
    y = np.empty_like(x)
    eps_bits = int(np.float16(eps).view(np.uint16))
    _check(lib().orc_layernorm(_p(x), _p(w), _p(b), _p(y), _sz(rows), _sz(cols), C.c_uint16(eps_bits)), "layernorm")
    return y


def gelu(x):
    """ops.zig:1635-1774 (returns a new array)."""
    y = np.array(_h(x), copy=True)
    _check(lib().orc_gelu(_p(y), _sz(y.size)), "gelu")
    return y


def bias_add(a, b):
    """ops.zig:1780-1953 (returns a new array)."""
    y = np.array(_h(a), copy=True)
    b = _h(b)
    cols = b.size
    _check(lib().orc_bias_add(_p(y), _p(b), _sz(y.size // cols), _sz(cols)), "bias_add")
    return y


def add(a, b):
    """ops.zig:312-323 (returns a new array)."""
    y = np.array(_h(a), copy=True)
    b = _h(b)
    _check(lib().orc_add(_p(y), _p(b), _sz(y.size)), "add")
    return y


def argmax(x) -> int:
    """sampling.zig:257-273."""
    x = _h(x).reshape(-1)
    idx = _sz(0)
    _check(lib().orc_argmax_f16(_p(x), _sz(x.size), C.byref(idx)), "argmax")
    return int(idx.value)


def kv_update(key_cache, value_cache, k_new, v_new, cur_len: int):
    """text_model.zig:476-515. caches [h,max_seq,d] modified in place."""
    h, max_seq, d = key_cache.shape
    k_new, v_new = _h(k_new), _h(v_new)
    s = k_new.shape[1]
    _check(lib().orc_kv_update(_p(key_cache), _p(value_cache), _p(k_new), _p(v_new), _sz(h), _sz(max_seq), _sz(d),
                               _sz(cur_len), _sz(s)), "kv_update")
    return cur_len + s


def kv_active(key_cache, value_cache, cur_len: int):
    """text_model.zig:436-474."""
    h, max_seq, d = key_cache.shape
    k = np.empty((h, cur_len, d), np.float16)
    v = np.empty((h, cur_len, d), np.float16)
    _check(lib().orc_kv_active(_p(key_cache), _p(value_cache), _p(k), _p(v), _sz(h), _sz(max_seq), _sz(d),
                               _sz(cur_len)), "kv_active")
    return k, v


def preprocess_patchify(img_u8, patch: int = 14):
    """vision_model.zig:137-183 + reshape_handler.zig. img uint8 [c,H,W,3] -> f16 [c,(H/p)(W/p),3pp]."""
    img = np.ascontiguousarray(img_u8, np.uint8)
    c, hh, ww, ch = img.shape
    assert ch == 3
    out = np.empty((c, (hh // patch) * (ww // patch), 3 * patch * patch), np.float16)
    _check(lib().orc_preprocess_patchify(_p(img), _p(out), _sz(c), _sz(hh), _sz(ww), _sz(patch)), "patchify")
    return out


# ---------------------------------------------------------------- models

def _ptr_array(arrs):
    return (C.c_void_p * len(arrs))(*[a.ctypes.data for a in arrs])


class _TextW(C.Structure):
    _fields_ = ([(n, C.c_size_t) for n in ("n_layers", "dim", "hidden", "n_heads", "head_dim", "vocab", "max_seq")] +
                [(n, C.c_void_p) for n in ("ln_w", "ln_b", "wqkv", "bqkv", "wout", "bout", "wfc1", "bfc1", "wfc2",
                                           "bfc2", "ln_out_w", "ln_out_b", "lm_w", "lm_b", "wte")])


class TextModel:
    """Host control flow of text_model.zig over a dict of numpy f16 weights.

    weights: per-layer lists ``ln_w ln_b wqkv bqkv wout bout wfc1 bfc1 wfc2 bfc2`` and
    ``ln_out_w ln_out_b lm_w lm_b wte``; matrices are [out,in]."""

    PER_LAYER = ("ln_w", "ln_b", "wqkv", "bqkv", "wout", "bout", "wfc1", "bfc1", "wfc2", "bfc2")

    def __init__(self, weights: dict, n_heads: int = 32, max_seq: int = 2048):
        self.w = weights
        L = len(weights["wqkv"])
        dim = weights["wqkv"][0].shape[1]
        self.n_layers, self.dim, self.n_heads, self.max_seq = L, dim, n_heads, max_seq
        self.head_dim = dim // n_heads
        self.vocab = weights["lm_w"].shape[0]
        self._keep = []
        s = _TextW()
        s.n_layers, s.dim, s.hidden = L, dim, weights["wfc1"][0].shape[0]
        s.n_heads, s.head_dim, s.vocab, s.max_seq = n_heads, self.head_dim, self.vocab, max_seq
        for name in self.PER_LAYER:
            arr = _ptr_array([_h(a) for a in weights[name]])
            self._keep.append(arr)
            setattr(s, name, C.cast(arr, C.c_void_p))
        for name in ("ln_out_w", "ln_out_b", "lm_w", "lm_b", "wte"):
            setattr(s, name, weights[name].ctypes.data)
        self.s = s
        self.reset()

    def reset(self):
        shape = (self.n_heads, self.max_seq, self.head_dim)
        self.key = [np.zeros(shape, np.float16) for _ in range(self.n_layers)]
        self.value = [np.zeros(shape, np.float16) for _ in range(self.n_layers)]
        self.cur_len = 0

    def embed(self, ids):
        return self.w["wte"][np.asarray(ids, np.int64)]

    def decoder(self, embeds):
        """text_model.zig:139-180; appends to the cache; returns hidden [S,dim]."""
        h = np.array(_h(embeds), copy=True)
        S = h.shape[0]
        kp, vp = _ptr_array(self.key), _ptr_array(self.value)
        _check(lib().orc_text_decoder(C.byref(self.s), _p(h), _sz(S), kp, vp, _sz(self.cur_len)), "text_decoder")
        self.cur_len += S
        return h

    def lm_head(self, hidden):
        hidden = _h(hidden)
        logits = np.empty((self.vocab,), np.float16)
        _check(lib().orc_lm_head(C.byref(self.s), _p(hidden), _sz(hidden.shape[0]), _p(logits)), "lm_head")
        return logits


class _VisW(C.Structure):
    _fields_ = ([(n, C.c_size_t) for n in ("n_layers", "dim", "n_heads", "head_dim", "hidden", "tokens", "patch_dim",
                                           "proj_hidden", "proj_out")] +
                [(n, C.c_void_p) for n in ("patch_w", "patch_b", "pos_emb", "ln1_w", "ln1_b", "wqkv", "bqkv", "wout",
                                           "bout", "ln2_w", "ln2_b", "wfc1", "bfc1", "wfc2", "bfc2", "norm_w",
                                           "norm_b", "proj_fc1_w", "proj_fc1_b", "proj_fc2_w", "proj_fc2_b")])


class VisionModel:
    """Host control flow of vision_model.zig; matrices are [in,out]."""

    PER_LAYER = ("ln1_w", "ln1_b", "wqkv", "bqkv", "wout", "bout", "ln2_w", "ln2_b", "wfc1", "bfc1", "wfc2", "bfc2")
    SINGLE = ("patch_w", "patch_b", "pos_emb", "norm_w", "norm_b", "proj_fc1_w", "proj_fc1_b", "proj_fc2_w",
              "proj_fc2_b")

    def __init__(self, weights: dict, n_heads: int = 16):
        self.w = weights
        s = _VisW()
        s.n_layers = len(weights["wqkv"])
        s.dim = weights["wqkv"][0].shape[0]
        s.n_heads, s.head_dim = n_heads, s.dim // n_heads
        s.hidden = weights["wfc1"][0].shape[1]
        s.tokens = weights["pos_emb"].shape[0]
        s.patch_dim = weights["patch_w"].shape[0]
        s.proj_hidden = weights["proj_fc1_w"].shape[1]
        s.proj_out = weights["proj_fc2_w"].shape[1]
        self._keep = []
        for name in self.PER_LAYER:
            arr = _ptr_array([_h(a) for a in weights[name]])
            self._keep.append(arr)
            setattr(s, name, C.cast(arr, C.c_void_p))
        for name in self.SINGLE:
            setattr(s, name, _h(weights[name]).ctypes.data)
        self.s = s

    def encoder(self, patches, joint_attention: bool = False):
        """vision_model.zig:204-272. patches [crops, tokens, patch_dim] -> [crops, tokens, dim]."""
        patches = _h(patches)
        crops = patches.shape[0]
        out = np.empty((crops, self.s.tokens, self.s.dim), np.float16)
        _check(lib().orc_vision_encoder(C.byref(self.s), _p(patches), _sz(crops), C.c_int(int(joint_attention)),
                                        _p(out)), "vision_encoder")
        return out

    def projection(self, feat_a, feat_b):
        feat_a, feat_b = _h(feat_a), _h(feat_b)
        out = np.empty((self.s.tokens, self.s.proj_out), np.float16)
        _check(lib().orc_vision_projection(C.byref(self.s), _p(feat_a), _p(feat_b), _p(out)), "projection")
        return out
