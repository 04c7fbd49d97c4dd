"""ctypes binding of libmoondream_b200 (the C ABI in include/moondream_b200.h).

Thin by design: every method forwards to one ``md_*`` entry point and raises
``MdError`` with the reference's error name when the status is not MD_OK.  There is
no CPU fallback: loading fails loudly if the CUDA library has not been built, and
``Context()`` fails if no sm_100a device is present.

Arguments may be numpy arrays (host, "drop-in" mode: the call stages them through
device memory and returns the result in a new numpy array) or ``DevBuf`` objects /
raw integer device pointers ("resident" mode).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libmoondream_b200.so")
HEADER_PATH = os.path.normpath(os.path.join(_HERE, "..", "include", "moondream_b200.h"))

MD_OK = 0
STATUS_NAMES = {
    0: "MD_OK", 1: "MD_ERR_INVALID_ARG", 2: "MD_ERR_INVALID_DIMENSION", 3: "MD_ERR_SHAPE",
    4: "MD_ERR_SEQUENCE_TOO_LONG", 5: "MD_ERR_INVALID_ROT_DIM", 6: "MD_ERR_UNSUPPORTED", 7: "MD_ERR_OOM",
    8: "MD_ERR_CUDA", 9: "MD_ERR_TIMEOUT", 10: "MD_ERR_NO_DEVICE", 11: "MD_ERR_IO", 12: "MD_ERR_FORMAT",
    13: "MD_ERR_NCCL",
}
# the Zig error each status maps back to in the shim
ZIG_ERRORS = {
    2: "error.InvalidTensorDimension", 3: "error.IncompatibleTensorShapes", 4: "error.SequenceTooLong",
    5: "error.InvalidRotationDimension", 7: "error.OutOfMemory",
}


class MdError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"{STATUS_NAMES.get(status, status)}: {message}")
        self.status = status
        self.zig_error = ZIG_ERRORS.get(status)
        if status in (11, 12) and ":" in message:  # the weight-file reader puts the Zig error name first
            self.zig_error = "error." + message.split(":", 1)[0]


def build(force: bool = False) -> str:
    """Compile the CUDA library in-tree (nvcc, sm_100a) if it is missing or stale."""
    csrc = os.path.join(_HERE, "csrc")
    srcs = [os.path.join(csrc, f) for f in os.listdir(csrc) if f.endswith((".cu", ".cuh"))] + [HEADER_PATH]
    inc = os.path.dirname(HEADER_PATH)
    srcs += [os.path.join(inc, f) for f in os.listdir(inc) if f.endswith(".h")]
    stale = (not os.path.exists(LIB_PATH)) or any(os.path.getmtime(s) > os.path.getmtime(LIB_PATH) for s in srcs)
    if force or stale:
        subprocess.check_call(["make", "-C", csrc, "-j8"] + (["-B"] if force else []), stdout=subprocess.DEVNULL)
    return LIB_PATH


_lib = None


def load() -> C.CDLL:
    """Load the shared library. Raises if it has not been built: there is no other path."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with __graft_entry__.build() or `make -C "
                f"{os.path.join(_HERE, 'csrc')}`; this package has no CPU fallback")
        _lib = C.CDLL(LIB_PATH)
        _lib.md_last_error.restype = C.c_char_p
        _lib.md_last_error.argtypes = [C.c_void_p]
    return _lib


class DevBuf:
    """A device allocation owned by a Context (freed with the context or by free())."""

    def __init__(self, ctx: "Context", ptr: int, nbytes: int, shape=None, dtype=np.float16):
        self.ctx, self.ptr, self.nbytes, self.shape, self.dtype = ctx, ptr, nbytes, shape, np.dtype(dtype)

    def numpy(self) -> np.ndarray:
        out = np.empty(self.shape if self.shape is not None else (self.nbytes // self.dtype.itemsize,), self.dtype)
        self.ctx._check(self.ctx.lib.md_memcpy_d2h(self.ctx.h, C.c_void_p(out.ctypes.data), C.c_void_p(self.ptr),
                                                   C.c_size_t(out.nbytes)))
        return out

    def view(self, offset_elems: int, shape, dtype=None) -> "DevBuf":
        dt = np.dtype(dtype or self.dtype)
        n = int(np.prod(shape)) * dt.itemsize
        return DevBuf(self.ctx, self.ptr + offset_elems * self.dtype.itemsize, n, tuple(shape), dt)

    def free(self):
        if self.ptr:
            self.ctx.lib.md_free(self.ctx.h, C.c_void_p(self.ptr))
            self.ptr = 0


def _sz(v):
    return C.c_size_t(int(v))


class Context:
    def __init__(self, device: int = 0):
        self.lib = load()
        h = C.c_void_p()
        st = self.lib.md_init(C.byref(h), C.c_int(device))
        if st != MD_OK:
            raise MdError(st, self.lib.md_last_error(None).decode())
        self.h = h
        self._owned = []

    # ---- plumbing
    def _check(self, st: int):
        if st != MD_OK:
            raise MdError(st, self.lib.md_last_error(self.h).decode())

    def close(self):
        if getattr(self, "h", None):
            for b in self._owned:
                b.free()
            self._owned = []
            self.lib.md_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def sync(self):
        self._check(self.lib.md_sync(self.h))

    def selftest_bounded_wait(self, limit_ms: int = 50):
        """Enqueue the kernel whose bounded wait runs out after limit_ms; the next sync raises MD_ERR_TIMEOUT."""
        self._check(self.lib.md_selftest_bounded_wait(self.h, C.c_uint(limit_ms)))

    def set_stream(self, cuda_stream: int | None):
        self._check(self.lib.md_set_stream(self.h, C.c_void_p(cuda_stream or 0)))

    def set_gemm_mode(self, mode: int):
        self._check(self.lib.md_set_gemm_mode(self.h, C.c_int(mode)))

    def set_option(self, key: str, value: int):
        self._check(self.lib.md_set_option(self.h, C.c_char_p(key.encode()), C.c_long(int(value))))

    def get_option(self, key: str) -> int:
        v = C.c_long()
        self._check(self.lib.md_get_option(self.h, C.c_char_p(key.encode()), C.byref(v)))
        return int(v.value)

    def graph_begin(self):
        self._check(self.lib.md_graph_begin(self.h))

    def graph_end(self):
        g = C.c_void_p()
        self._check(self.lib.md_graph_end(self.h, C.byref(g)))
        return g

    def graph_launch(self, g):
        self._check(self.lib.md_graph_launch(self.h, g))

    def graph_destroy(self, g):
        self._check(self.lib.md_graph_destroy(self.h, g))

    def launch_count(self) -> int:
        n = C.c_uint64()
        self._check(self.lib.md_launch_count(self.h, C.byref(n)))
        return int(n.value)

    def alloc(self, shape, dtype=np.float16) -> DevBuf:
        dt = np.dtype(dtype)
        n = int(np.prod(shape)) * dt.itemsize
        p = C.c_void_p()
        self._check(self.lib.md_alloc(self.h, _sz(n), C.byref(p)))
        b = DevBuf(self, p.value, n, tuple(np.atleast_1d(shape)), dt)
        self._owned.append(b)
        return b

    def upload(self, arr: np.ndarray) -> DevBuf:
        """Register a tensor once (weights): md_upload."""
        arr = np.ascontiguousarray(arr)
        p = C.c_void_p()
        self._check(self.lib.md_upload(self.h, C.c_void_p(arr.ctypes.data), _sz(arr.nbytes), C.byref(p)))
        b = DevBuf(self, p.value, arr.nbytes, arr.shape, arr.dtype)
        self._owned.append(b)
        return b

    @staticmethod
    def _ptr(x):
        if isinstance(x, DevBuf):
            return C.c_void_p(x.ptr)
        if isinstance(x, np.ndarray):
            assert x.flags["C_CONTIGUOUS"]
            return C.c_void_p(x.ctypes.data)
        if x is None:
            return C.c_void_p(0)
        return C.c_void_p(int(x))  # raw device pointer (e.g. torch tensor.data_ptr())

    def _out(self, like_device, shape, dtype=np.float16):
        """Output buffer: device when the inputs are device-resident, numpy otherwise."""
        if like_device:
            return self.alloc(shape, dtype)
        return np.empty(shape, dtype)

    @staticmethod
    def _on_device(*xs):
        return any(isinstance(x, (DevBuf, int)) for x in xs)

    # ---- matmul (hgemm.zig:362, hgemm_trans.zig:400)
    def hgemm_nn(self, a, b, M, N, K, out=None):
        out = out if out is not None else self._out(self._on_device(a, b), (M, N))
        self._check(self.lib.md_hgemm_nn(self.h, self._ptr(a), self._ptr(b), self._ptr(out), _sz(M), _sz(N), _sz(K)))
        return out

    def hgemm_nt(self, a, b_t, M, N, K, out=None):
        out = out if out is not None else self._out(self._on_device(a, b_t), (M, N))
        self._check(self.lib.md_hgemm_nt(self.h, self._ptr(a), self._ptr(b_t), self._ptr(out), _sz(M), _sz(N), _sz(K)))
        return out

    def hgemm_fused(self, a, b, out, M, N, K, b_layout, bias=None, gelu=False, residual=None):
        self._check(self.lib.md_hgemm_fused(self.h, self._ptr(a), self._ptr(b), self._ptr(out), _sz(M), _sz(N), _sz(K),
                                            C.c_int(b_layout), self._ptr(bias), C.c_int(int(gelu)),
                                            self._ptr(residual)))
        return out

    def check_matmul_shapes(self, a_shape, b_shape, b_transposed: bool):
        a = (C.c_size_t * len(a_shape))(*a_shape)
        b = (C.c_size_t * len(b_shape))(*b_shape)
        st = self.lib.md_check_matmul_shapes(a, _sz(len(a_shape)), b, _sz(len(b_shape)), C.c_int(int(b_transposed)))
        if st != MD_OK:
            raise MdError(st, f"matmul shapes {tuple(a_shape)} x {tuple(b_shape)}")

    # ---- attention (attention.zig:125, 256, 416, 759)
    def sdpa_maskless(self, q, k, v, n_heads, q_len, kv_len, d, out=None):
        out = out if out is not None else self._out(self._on_device(q, k, v), (n_heads, q_len, d))
        self._check(self.lib.md_sdpa_maskless(self.h, self._ptr(q), self._ptr(k), self._ptr(v), self._ptr(out),
                                              _sz(n_heads), _sz(q_len), _sz(kv_len), _sz(d)))
        return out

    def create_attention_mask(self, pos, seq_len, out=None):
        out = out if out is not None else np.empty((seq_len, pos + seq_len), np.uint8)
        self._check(self.lib.md_create_attention_mask(self.h, self._ptr(out), _sz(pos), _sz(seq_len)))
        return out

    def sdpa_masked(self, q, k, v, mask, n_heads, q_len, kv_len, d, out=None):
        out = out if out is not None else self._out(self._on_device(q, k, v), (n_heads, q_len, d))
        self._check(self.lib.md_sdpa_masked(self.h, self._ptr(q), self._ptr(k), self._ptr(v), self._ptr(mask),
                                            self._ptr(out), _sz(n_heads), _sz(q_len), _sz(kv_len), _sz(d)))
        return out

    def sdpa_single(self, q, k, v, mask, kv_len, out=None):
        out = out if out is not None else self._out(self._on_device(q, k, v), (32, 1, 64))
        self._check(self.lib.md_sdpa_single(self.h, self._ptr(q), self._ptr(k), self._ptr(v), self._ptr(mask),
                                            self._ptr(out), _sz(kv_len)))
        return out

    def sdpa_decode_fused(self, qkv_row, key_cache, value_cache, out, n_heads, d, max_seq, pos, rot_dim, theta=10000.0):
        self._check(self.lib.md_sdpa_decode_fused(self.h, self._ptr(qkv_row), self._ptr(key_cache),
                                                  self._ptr(value_cache), self._ptr(out), _sz(n_heads), _sz(d),
                                                  _sz(max_seq), _sz(pos), _sz(rot_dim), C.c_float(theta)))
        return out

    def sdpa_prefill_fused(self, qkv, key_cache, value_cache, out, S, n_heads, d, max_seq, pos, rot_dim,
                           theta=10000.0):
        self._check(self.lib.md_sdpa_prefill_fused(self.h, self._ptr(qkv), self._ptr(key_cache), self._ptr(value_cache),
                                                   self._ptr(out), _sz(S), _sz(n_heads), _sz(d), _sz(max_seq),
                                                   _sz(pos), _sz(rot_dim), C.c_float(theta)))
        return out

    def sdpa_vit_fused(self, qkv, out, crops, tokens, n_heads, d):
        self._check(self.lib.md_sdpa_vit_fused(self.h, self._ptr(qkv), self._ptr(out), _sz(crops), _sz(tokens),
                                               _sz(n_heads), _sz(d)))
        return out

    # ---- rope (rope.zig:32, 130)
    def rope_table(self, dim, end, theta=10000.0, out=None):
        out = out if out is not None else np.empty((end, dim // 2, 2), np.float32)
        self._check(self.lib.md_rope_table(self.h, self._ptr(out), _sz(dim), _sz(end), C.c_float(theta)))
        return out

    def rope_apply(self, x, freqs_cis, position_ids, n_heads, seq_len, d, freqs_half, rot_dim, out=None):
        out = out if out is not None else self._out(self._on_device(x), (n_heads, seq_len, d))
        self._check(self.lib.md_rope_apply(self.h, self._ptr(x), self._ptr(out), _sz(n_heads), _sz(seq_len), _sz(d),
                                           self._ptr(freqs_cis), _sz(freqs_half), self._ptr(position_ids),
                                           _sz(rot_dim)))
        return out

    # ---- KV cache (text_model.zig:436-515)
    def kv_update(self, key_cache, value_cache, k_new, v_new, n_heads, max_seq, d, cur_len, seq_len):
        self._check(self.lib.md_kv_update(self.h, self._ptr(key_cache), self._ptr(value_cache), self._ptr(k_new),
                                          self._ptr(v_new), _sz(n_heads), _sz(max_seq), _sz(d), _sz(cur_len),
                                          _sz(seq_len)))

    def kv_active(self, key_cache, value_cache, n_heads, max_seq, d, cur_len):
        k = np.empty((n_heads, cur_len, d), np.float16)
        v = np.empty((n_heads, cur_len, d), np.float16)
        self._check(self.lib.md_kv_active(self.h, self._ptr(key_cache), self._ptr(value_cache), self._ptr(k),
                                          self._ptr(v), _sz(n_heads), _sz(max_seq), _sz(d), _sz(cur_len)))
        return k, v

    # ---- glue (ops.zig)
    def layernorm(self, x, w, b, rows, cols, eps=np.float16(1e-5), out=None):
        out = out if out is not None else self._out(self._on_device(x), (rows, cols))
        bits = int(np.float16(eps).view(np.uint16))
        self._check(self.lib.md_layernorm(self.h, self._ptr(x), self._ptr(w), self._ptr(b), self._ptr(out), _sz(rows),
                                          _sz(cols), C.c_uint16(bits)))
        return out

    def gelu(self, x, n):
        self._check(self.lib.md_gelu(self.h, self._ptr(x), _sz(n)))
        return x

    def bias_add(self, a, b, rows, cols):
        self._check(self.lib.md_bias_add(self.h, self._ptr(a), self._ptr(b), _sz(rows), _sz(cols)))
        return a

    def add(self, a, b, n):
        self._check(self.lib.md_add(self.h, self._ptr(a), self._ptr(b), _sz(n)))
        return a

    def argmax(self, x, n) -> int:
        idx = np.zeros(1, np.uint64)
        self._check(self.lib.md_argmax(self.h, self._ptr(x), _sz(n), self._ptr(idx)))
        return int(idx[0])

    def preprocess_patchify(self, img, crops, height, width, patch=14, out_stride=None, out=None):
        pd = 3 * patch * patch
        out_stride = out_stride or pd
        shape = (crops * (height // patch) * (width // patch), out_stride)
        out = out if out is not None else self._out(self._on_device(img), shape)
        self._check(self.lib.md_preprocess_patchify(self.h, self._ptr(img), self._ptr(out), _sz(crops), _sz(height),
                                                    _sz(width), _sz(patch), _sz(out_stride)))
        return out
