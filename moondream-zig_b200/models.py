"""ctypes binding of include/moondream_b200_model.h: the device-resident text decoder and
vision encoder built on the hot-path kernels.  Weights are numpy f16 arrays laid out as the
reference holds them (text matrices [out,in], vision matrices [in,out]); they are uploaded
once at construction."""
from __future__ import annotations

import ctypes as C

import numpy as np

_sz = C.c_size_t

TEXT_PER_LAYER = ("ln_w", "ln_b", "wqkv", "bqkv", "wout", "bout", "wfc1", "bfc1", "wfc2", "bfc2")
TEXT_SINGLE = ("ln_out_w", "ln_out_b", "lm_w", "lm_b", "wte")
VIS_PER_LAYER = ("ln1_w", "ln1_b", "wqkv", "bqkv", "wout", "bout", "ln2_w", "ln2_b", "wfc1", "bfc1", "wfc2", "bfc2")
VIS_SINGLE = ("norm_w", "norm_b", "proj_fc1_w", "proj_fc1_b", "proj_fc2_w", "proj_fc2_b")


class _TextW(C.Structure):
    _fields_ = ([(n, C.c_size_t) for n in ("n_layers", "dim", "hidden", "n_heads", "head_dim", "vocab", "max_seq",
                                           "rot_dim")] +
                [("rope_theta", C.c_float), ("eps_f16", C.c_uint16)] +
                [(n, C.c_void_p) for n in TEXT_PER_LAYER + TEXT_SINGLE])


class _VisW(C.Structure):
    _fields_ = ([(n, C.c_size_t) for n in ("n_layers", "dim", "n_heads", "head_dim", "hidden", "tokens", "patch", "img",
                                           "proj_hidden", "proj_out")] +
                [("eps_f16", C.c_uint16)] +
                [(n, C.c_void_p) for n in ("patch_w", "patch_b", "pos_emb") + VIS_PER_LAYER + VIS_SINGLE])


class _TorchBuf:
    """A CUDA torch tensor used in place of an uploaded weight (kept alive by this wrapper)."""

    def __init__(self, t):
        self.t, self.ptr, self.shape = t, t.data_ptr(), tuple(t.shape)


def _dev(ctx, a):
    """numpy f16 array -> uploaded DevBuf; CUDA torch tensor (f16, contiguous) -> used in place."""
    if hasattr(a, "data_ptr"):
        assert a.is_cuda and a.is_contiguous() and a.element_size() == 2
        return _TorchBuf(a)
    return ctx.upload(np.ascontiguousarray(a, np.float16))


def _f16_bits(v) -> int:
    return int(np.float16(v).view(np.uint16))


class TextRequest:
    """One KVCache (text_model.zig:349) plus the activation buffers of a step."""

    def __init__(self, model: "TextModel"):
        self.model = model
        h = C.c_void_p()
        model.ctx._check(model.lib.md_text_request_create(model.h, C.byref(h)))
        self.h = h

    def reset(self):
        self.model.ctx._check(self.model.lib.md_text_request_reset(self.h))

    def __len__(self):
        n = C.c_size_t()
        self.model.ctx._check(self.model.lib.md_text_request_len(self.h, C.byref(n)))
        return int(n.value)

    def close(self):
        if self.h:
            self.model.lib.md_text_request_destroy(self.h)
            self.h = None


class TextModel:
    def __init__(self, ctx, weights: dict, n_heads: int = 32, max_seq: int = 2048, rot_dim: int | None = None,
                 theta: float = 10000.0, eps=np.float16(1e-5)):
        self.ctx, self.lib = ctx, ctx.lib
        self.dev = {}
        s = _TextW()
        L = len(weights["wqkv"])
        dim = weights["wqkv"][0].shape[1]
        s.n_layers, s.dim, s.hidden = L, dim, weights["wfc1"][0].shape[0]
        s.n_heads, s.head_dim = n_heads, dim // n_heads
        s.vocab, s.max_seq = weights["lm_w"].shape[0], max_seq
        s.rot_dim = rot_dim if rot_dim is not None else (dim // n_heads) // 2
        s.rope_theta, s.eps_f16 = theta, _f16_bits(eps)
        self._keep = []
        for name in TEXT_PER_LAYER:
            bufs = [_dev(ctx, a) for a in weights[name]]
            self.dev[name] = bufs
            arr = (C.c_void_p * L)(*[b.ptr for b in bufs])
            self._keep.append(arr)
            setattr(s, name, C.cast(arr, C.c_void_p))
        for name in TEXT_SINGLE:
            b = _dev(ctx, weights[name])
            self.dev[name] = b
            setattr(s, name, b.ptr)
        self._create(s)

    def _create(self, s: _TextW):
        self.s = s
        self.dim, self.vocab, self.n_layers = int(s.dim), int(s.vocab), int(s.n_layers)
        h = C.c_void_p()
        self.ctx._check(self.lib.md_text_model_create(self.ctx.h, C.byref(s), C.byref(h)))
        self.h = h

    @classmethod
    def from_table(cls, ctx, table: _TextW, owner=None) -> "TextModel":
        """A model over weights that are already resident (e.g. a weight file's table); `owner` is kept alive."""
        self = cls.__new__(cls)
        self.ctx, self.lib, self.dev, self._keep = ctx, ctx.lib, {}, [owner]
        self._create(table)
        return self

    def request(self) -> TextRequest:
        return TextRequest(self)

    def text_encoder(self, ids, out_ptr: int | None = None):
        """text_model.zig:106-137.  With out_ptr (a device address) the rows are written there and nothing is returned."""
        ids = np.ascontiguousarray(ids, np.uint32)
        out = np.empty((ids.size, self.dim), np.float16) if out_ptr is None else None
        self.ctx._check(self.lib.md_text_encoder(self.h, C.c_void_p(ids.ctypes.data), _sz(ids.size),
                                                 C.c_void_p(out.ctypes.data if out_ptr is None else out_ptr)))
        return out

    def forward(self, req: TextRequest, embeds, want_hidden=True, want_logits=True, rows: int | None = None):
        """text_decoder + lm_head + argmax over S rows (text_model.zig:139-180,325-345).  embeds: a numpy array
        [S, dim], or a device address together with rows=S."""
        if isinstance(embeds, np.ndarray):
            embeds = np.ascontiguousarray(embeds, np.float16)
            S, src = embeds.shape[0], embeds.ctypes.data
        else:
            S, src = int(rows), int(embeds)
        hidden = np.empty((S, self.dim), np.float16) if want_hidden else None
        logits = np.empty((self.vocab,), np.float16) if want_logits else None
        tok = np.zeros(1, np.uint64)
        self.ctx._check(self.lib.md_text_forward(
            self.h, req.h, C.c_void_p(src), _sz(S),
            C.c_void_p(hidden.ctypes.data if want_hidden else 0), C.c_void_p(logits.ctypes.data if want_logits else 0),
            C.c_void_p(tok.ctypes.data)))
        return hidden, logits, int(tok[0])

    def generate(self, req: TextRequest, first: int, n_steps: int, forced=None, want_logits=False):
        """Greedy decode loop on the device (moondream.zig:323-368)."""
        toks = np.zeros(n_steps, np.uint32)
        f = np.ascontiguousarray(forced, np.uint32) if forced is not None else None
        logits = np.empty((n_steps, self.vocab), np.float16) if want_logits else None
        self.ctx._check(self.lib.md_text_generate(
            self.h, req.h, C.c_uint32(int(first)), _sz(n_steps), C.c_void_p(toks.ctypes.data),
            C.c_void_p(f.ctypes.data if f is not None else 0), C.c_void_p(logits.ctypes.data if want_logits else 0)))
        return (toks, logits) if want_logits else toks

    def generate_batch(self, reqs, first, n_steps: int, forced=None) -> np.ndarray:
        """Up to 8 requests advanced together; forced [batch, n_steps] = teacher forcing per request."""
        B = len(reqs)
        arr = (C.c_void_p * B)(*[r.h.value for r in reqs])
        f = np.ascontiguousarray(first, np.uint32)
        toks = np.zeros((B, n_steps), np.uint32)
        if forced is None:
            self.ctx._check(self.lib.md_text_generate_batch(self.h, arr, _sz(B), C.c_void_p(f.ctypes.data),
                                                            _sz(n_steps), C.c_void_p(toks.ctypes.data)))
        else:
            fo = np.ascontiguousarray(forced, np.uint32)
            assert fo.shape == (B, n_steps)
            self.ctx._check(self.lib.md_text_generate_batch_forced(self.h, arr, _sz(B), C.c_void_p(f.ctypes.data),
                                                                   _sz(n_steps), C.c_void_p(toks.ctypes.data),
                                                                   C.c_void_p(fo.ctypes.data)))
        return toks

    def close(self):
        if getattr(self, "h", None):
            self.lib.md_text_model_destroy(self.h)
            self.h = None


class VisionModel:
    def __init__(self, ctx, weights: dict, n_heads: int = 16, img: int = 378, patch: int = 14, max_crops: int = 2,
                 eps=np.float16(1e-5)):
        self.ctx, self.lib = ctx, ctx.lib
        self.dev = {}
        s = _VisW()
        L = len(weights["wqkv"])
        s.n_layers, s.dim = L, weights["wqkv"][0].shape[0]
        s.n_heads, s.head_dim = n_heads, s.dim // n_heads
        s.hidden = weights["wfc1"][0].shape[1]
        s.tokens, s.patch, s.img = weights["pos_emb"].shape[0], patch, img
        s.proj_hidden, s.proj_out = weights["proj_fc1_w"].shape[1], weights["proj_fc2_w"].shape[1]
        s.eps_f16 = _f16_bits(eps)
        self._keep = []
        for name in VIS_PER_LAYER:
            bufs = [_dev(ctx, a) for a in weights[name]]
            self.dev[name] = bufs
            arr = (C.c_void_p * L)(*[b.ptr for b in bufs])
            self._keep.append(arr)
            setattr(s, name, C.cast(arr, C.c_void_p))
        for name in ("patch_w", "patch_b", "pos_emb") + VIS_SINGLE:
            b = _dev(ctx, weights[name])
            self.dev[name] = b
            setattr(s, name, b.ptr)
        self._create(s, max_crops)

    def _create(self, s: _VisW, max_crops: int):
        self.s = s
        self.tokens, self.dim, self.proj_out, self.img = int(s.tokens), int(s.dim), int(s.proj_out), int(s.img)
        self.max_crops = int(max_crops)
        h = C.c_void_p()
        self.ctx._check(self.lib.md_vision_model_create(self.ctx.h, C.byref(s), _sz(max_crops), C.byref(h)))
        self.h = h

    @classmethod
    def from_table(cls, ctx, table: _VisW, max_crops: int = 2, owner=None) -> "VisionModel":
        self = cls.__new__(cls)
        self.ctx, self.lib, self.dev, self._keep = ctx, ctx.lib, {}, [owner]
        self._create(table, max_crops)
        return self

    def encode(self, crops_u8: np.ndarray, crop_a: int = 0, crop_b: int | None = None, want_features: bool = False,
               out_ptr: int | None = None):
        """vision_model.zig:160-202 without the file decode. crops uint8 [c, img, img, 3].  With out_ptr (a device
        address) the [tokens, proj_out] result stays on the device and nothing is returned."""
        crops_u8 = np.ascontiguousarray(crops_u8, np.uint8)
        c = crops_u8.shape[0]
        crop_b = min(1, c - 1) if crop_b is None else crop_b
        feats = np.empty((c * self.tokens, self.dim), np.float16) if want_features else None
        out = np.empty((self.tokens, self.proj_out), np.float16) if out_ptr is None else None
        self.ctx._check(self.lib.md_vision_encode(self.h, C.c_void_p(crops_u8.ctypes.data), _sz(c), _sz(crop_a),
                                                  _sz(crop_b), C.c_void_p(feats.ctypes.data if want_features else 0),
                                                  C.c_void_p(out.ctypes.data if out_ptr is None else out_ptr)))
        return (out, feats) if want_features else out

    def encode_images(self, images_u8: np.ndarray, out_ptrs=None):
        """n independent one-crop images in one pass (md_vision_encode_images).  images uint8 [n, img, img, 3].
        out_ptrs: n device addresses of [tokens, proj_out] buffers; without them a numpy array [n, tokens, proj_out]
        is returned."""
        images_u8 = np.ascontiguousarray(images_u8, np.uint8)
        n = images_u8.shape[0]
        out = None
        if out_ptrs is None:
            out = np.empty((n, self.tokens, self.proj_out), np.float16)
            out_ptrs = [out[i].ctypes.data for i in range(n)]
        arr = (C.c_void_p * n)(*[int(p) for p in out_ptrs])
        self.ctx._check(self.lib.md_vision_encode_images(self.h, C.c_void_p(images_u8.ctypes.data), _sz(n), arr))
        return out

    def close(self):
        if getattr(self, "h", None):
            self.lib.md_vision_model_destroy(self.h)
            self.h = None
