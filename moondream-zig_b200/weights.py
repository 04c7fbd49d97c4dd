"""The moondream.bin weight file: ctypes binding of the md_weight_file_* reader
(include/moondream_b200_model.h; the format weights.zig:61-207 reads) and a writer producing the same
bytes as the reference's converter (weights.py:82-135: header, name, u64 dims, raw f16).

The writer takes the two weight dictionaries the model classes use (per-layer lists of [out,in] text
matrices and [in,out] vision matrices) and stacks the per-layer tensors on a leading axis, as
weights.py:137-154 does."""
from __future__ import annotations

import ctypes as C
import struct

import numpy as np

from . import MD_OK, MdError, load
from .models import TextModel, VisionModel, _TextW, _VisW

WEIGHTS_MAGIC = 0x4D4F4F4E  # "MOON" (weights.zig:10)
WEIGHTS_VERSION = 2         # weights.zig:11

_SIZES_TEXT = ("vocab", "dim", "hidden_dim", "n_layers", "n_heads", "head_dim", "seq_len")
_SIZES_VIS = ("img_channels", "img_dim", "patch_size", "num_patches", "vit_dim", "n_vit_layers", "n_vit_heads",
              "vit_head_dim", "hidden_features")


class ModelConfig(C.Structure):
    """md_model_config: config.zig:3-27."""
    _fields_ = ([(n, C.c_size_t) for n in _SIZES_TEXT] + [("rope_theta", C.c_float), ("partial_rotary_factor", C.c_float)] +
                [(n, C.c_size_t) for n in _SIZES_VIS])

    @classmethod
    def default(cls) -> "ModelConfig":
        cfg = cls()
        st = load().md_model_config_default(C.byref(cfg))
        if st != MD_OK:
            raise MdError(st, load().md_last_error(None).decode())
        return cfg

    @classmethod
    def scaled(cls, **sizes) -> "ModelConfig":
        """The default configuration with some sizes replaced (small files for tests)."""
        cfg = cls.default()
        for k, v in sizes.items():
            if k not in dict(cls._fields_):
                raise KeyError(k)
            setattr(cfg, k, v)
        return cfg


# file name -> (dictionary, key, stacked over layers); in the order weights.py:156-246 writes them
FILE_TENSORS = (
    ("word_token_embedding", "text", "wte", False),
    ("t_ln_w", "text", "ln_w", True), ("t_ln_b", "text", "ln_b", True),
    ("t_Wqkv_w", "text", "wqkv", True), ("t_Wqkv_b", "text", "bqkv", True),
    ("t_out_proj_w", "text", "wout", True), ("t_out_proj_bias", "text", "bout", True),
    ("t_fc1_w", "text", "wfc1", True), ("t_fc1_b", "text", "bfc1", True),
    ("t_fc2_w", "text", "wfc2", True), ("t_fc2_b", "text", "bfc2", True),
    ("t_linear_w", "text", "lm_w", False), ("t_linear_b", "text", "lm_b", False),
    ("t_ln_out_w", "text", "ln_out_w", False), ("t_ln_out_b", "text", "ln_out_b", False),
    ("v_patch_embedding_linear_w", "vision", "patch_w", False), ("v_patch_embedding_linear_b", "vision", "patch_b", False),
    ("v_pos_embedding", "vision", "pos_emb", False),
    ("v_Wqkv_w", "vision", "wqkv", True), ("v_Wqkv_b", "vision", "bqkv", True),
    ("v_out_proj_w", "vision", "wout", True), ("v_out_proj_b", "vision", "bout", True),
    ("v_fc1_w", "vision", "wfc1", True), ("v_fc1_b", "vision", "bfc1", True),
    ("v_fc2_w", "vision", "wfc2", True), ("v_fc2_b", "vision", "bfc2", True),
    ("v_norm1_w", "vision", "ln1_w", True), ("v_norm1_b", "vision", "ln1_b", True),
    ("v_norm2_w", "vision", "ln2_w", True), ("v_norm2_b", "vision", "ln2_b", True),
    ("v_norm_out_w", "vision", "norm_w", False), ("v_norm_out_b", "vision", "norm_b", False),
    ("v_proj_fc1_w", "vision", "proj_fc1_w", False), ("v_proj_fc1_b", "vision", "proj_fc1_b", False),
    ("v_proj_fc2_w", "vision", "proj_fc2_w", False), ("v_proj_fc2_b", "vision", "proj_fc2_b", False),
)


def write_tensor(f, name: str, array: np.ndarray) -> None:
    """One record (weights.py:82-135): u32 name length, u32 rank, u32 element count, name, u64 dims, f16 data."""
    a = np.ascontiguousarray(array)
    if a.dtype != np.float16:
        raise TypeError(f"{name}: expected float16, got {a.dtype}")
    raw = name.encode("utf-8")
    f.write(struct.pack("<III", len(raw), a.ndim, a.size & 0xFFFFFFFF))
    f.write(raw)
    f.write(struct.pack(f"<{a.ndim}Q", *a.shape))
    f.write(a.tobytes())


def write_weight_file(path: str, text: dict, vision: dict) -> None:
    """Write a moondream.bin from the two weight dictionaries."""
    src = {"text": text, "vision": vision}
    with open(path, "wb") as f:
        f.write(struct.pack("<II", WEIGHTS_MAGIC, WEIGHTS_VERSION))
        for name, which, key, stacked in FILE_TENSORS:
            a = np.stack(src[which][key]) if stacked else np.asarray(src[which][key])
            if name == "v_pos_embedding" and a.ndim == 2:
                a = a[None]  # the file holds [1, tokens, dim] (weights.zig:455)
            write_tensor(f, name, a)


class WeightFile:
    """An opened (parsed and validated) weight file; upload() makes it resident on a context's device."""

    def __init__(self, path: str, config: ModelConfig | None = None):
        self.lib = load()
        self.config = config if config is not None else ModelConfig.default()
        self.ctx = None
        h = C.c_void_p()
        st = self.lib.md_weight_file_open(C.c_char_p(path.encode()), C.byref(self.config), C.byref(h))
        if st != MD_OK:
            raise MdError(st, self.lib.md_last_error(None).decode())
        self.h = h

    def _check(self, st: int):
        if st != MD_OK:
            raise MdError(st, self.lib.md_last_error(self.ctx.h if self.ctx is not None else None).decode())

    def __len__(self) -> int:
        n = C.c_size_t()
        self._check(self.lib.md_weight_file_count(self.h, C.byref(n)))
        return int(n.value)

    def tensor(self, index: int):
        """(name, read-only f16 array over the mapped file) of record `index`."""
        name, rank, shape, data = C.c_char_p(), C.c_size_t(), (C.c_size_t * 4)(), C.c_void_p()
        self._check(self.lib.md_weight_file_tensor(self.h, C.c_size_t(index), C.byref(name), C.byref(rank), shape,
                                                   C.byref(data)))
        dims = tuple(int(shape[i]) for i in range(rank.value))
        n = int(np.prod(dims, dtype=np.int64)) if dims else 1
        if n == 0:
            return name.value.decode(), np.empty(dims, np.float16)
        buf = (C.c_uint16 * n).from_address(data.value)
        a = np.frombuffer(buf, np.float16).reshape(dims)
        a.flags.writeable = False
        return name.value.decode(), a

    def tensors(self) -> dict:
        return dict(self.tensor(i) for i in range(len(self)))

    def upload(self, ctx) -> "WeightFile":
        self._check(self.lib.md_weight_file_upload(self.h, ctx.h))
        self.ctx = ctx
        return self

    def text_model(self) -> TextModel:
        table = _TextW()
        self._check(self.lib.md_weight_file_text(self.h, C.byref(table)))
        return TextModel.from_table(self.ctx, table, owner=self)

    def vision_model(self, max_crops: int = 2) -> VisionModel:
        table = _VisW()
        self._check(self.lib.md_weight_file_vision(self.h, C.byref(table)))
        return VisionModel.from_table(self.ctx, table, max_crops, owner=self)

    def close(self):
        if getattr(self, "h", None):
            self.lib.md_weight_file_close(self.h)
            self.h = None
