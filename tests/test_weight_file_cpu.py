"""The moondream.bin reader (md_weight_file_open, host only) against files written by the package's writer:
record order, names, shapes and bytes, and every rejection weights.zig:61-207 makes, by its Zig error name."""
import importlib
import struct

import numpy as np
import pytest

import __graft_entry__ as entry
from model_utils import text_weights, vision_weights

SMALL = dict(vocab=96, dim=64, hidden_dim=128, n_layers=2, n_heads=2, head_dim=32, seq_len=64,
             img_dim=28, patch_size=14, num_patches=4, vit_dim=48, n_vit_layers=3, n_vit_heads=2, vit_head_dim=24,
             hidden_features=80)


@pytest.fixture(scope="module")
def wmod(pkg):
    return importlib.import_module(entry.PKG_NAME + ".weights")


def small_weights():
    tw = text_weights(3, n_layers=2, dim=64, hidden=128, vocab=96)
    # the projection input is vit_head_dim * n_heads(text) = 48 wide here (weights.zig:470)
    vw = vision_weights(4, n_layers=3, dim=48, hidden=80, tokens=4, patch_dim=588, proj_hidden=128, proj_out=64)
    vw["proj_fc1_w"] = vw["proj_fc1_w"][:48]
    return tw, vw


@pytest.fixture()
def small_file(wmod, tmp_path):
    tw, vw = small_weights()
    path = str(tmp_path / "moondream.bin")
    wmod.write_weight_file(path, tw, vw)
    return path, tw, vw, wmod.ModelConfig.scaled(**SMALL)


def test_default_config_is_the_reference_model(wmod):
    c = wmod.ModelConfig.default()
    assert (c.vocab, c.dim, c.hidden_dim, c.n_layers, c.n_heads, c.head_dim, c.seq_len) == (51200, 2048, 8192, 24, 32, 64,
                                                                                           2048)
    assert (c.img_channels, c.img_dim, c.patch_size, c.num_patches) == (3, 378, 14, 729)
    assert (c.vit_dim, c.n_vit_layers, c.n_vit_heads, c.vit_head_dim, c.hidden_features) == (1152, 27, 16, 72, 4304)
    assert c.rope_theta == 10000.0 and c.partial_rotary_factor == 0.5


def test_reader_returns_every_record_byte_for_byte(wmod, small_file):
    path, tw, vw, cfg = small_file
    wf = wmod.WeightFile(path, cfg)
    try:
        assert len(wf) == 36
        names = [wf.tensor(i)[0] for i in range(len(wf))]
        assert names == [t[0] for t in wmod.FILE_TENSORS]
        got = wf.tensors()
        src = {"text": tw, "vision": vw}
        for name, which, key, stacked in wmod.FILE_TENSORS:
            want = np.stack(src[which][key]) if stacked else np.asarray(src[which][key])
            if name == "v_pos_embedding":
                want = want[None]
            assert got[name].shape == want.shape, name
            assert np.array_equal(got[name].view(np.uint16), want.view(np.uint16)), name
    finally:
        wf.close()


def test_tables_need_a_resident_file(wmod, pkg, small_file):
    path, _, _, cfg = small_file
    wf = wmod.WeightFile(path, cfg)
    try:
        with pytest.raises(pkg.MdError) as e:
            wf.text_model()
        assert e.value.status == 1
    finally:
        wf.close()


def _expect(wmod, pkg, path, cfg, status, zig):
    with pytest.raises(pkg.MdError) as e:
        wmod.WeightFile(path, cfg)
    assert e.value.status == status, str(e.value)
    assert e.value.zig_error == "error." + zig, str(e.value)


def test_rejections_follow_the_reference(wmod, pkg, small_file, tmp_path):
    path, tw, vw, cfg = small_file
    raw = open(path, "rb").read()

    def variant(name, data):
        p = str(tmp_path / name)
        open(p, "wb").write(data)
        return p

    _expect(wmod, pkg, str(tmp_path / "absent.bin"), cfg, 11, "FileNotFound")
    _expect(wmod, pkg, variant("empty.bin", b""), cfg, 11, "InvalidRead")
    _expect(wmod, pkg, variant("magic.bin", struct.pack("<I", 0x4E4F4F4D) + raw[4:]), cfg, 12, "InvalidMagicNumber")
    _expect(wmod, pkg, variant("version.bin", raw[:4] + struct.pack("<I", 1) + raw[8:]), cfg, 12, "InvalidVersion")
    _expect(wmod, pkg, variant("short_version.bin", raw[:6]), cfg, 11, "InvalidRead")
    _expect(wmod, pkg, variant("tail.bin", raw + b"\0" * 5), cfg, 12, "InvalidHeader")
    _expect(wmod, pkg, variant("cut.bin", raw[:-2]), cfg, 11, "InvalidRead")
    _expect(wmod, pkg, variant("cut_name.bin", raw[:8 + 12 + 3]), cfg, 11, "InvalidRead")
    _expect(wmod, pkg, variant("cut_shape.bin", raw[:8 + 12 + 20 + 8]), cfg, 11, "InvalidRead")
    _expect(wmod, pkg, variant("name_len.bin", raw[:8] + struct.pack("<I", 257) + raw[12:]), cfg, 12, "InvalidNameLength")
    _expect(wmod, pkg, variant("rank.bin", raw[:12] + struct.pack("<I", 5) + raw[16:]), cfg, 12, "InvalidShapeLength")
    _expect(wmod, pkg, variant("unknown.bin", raw[:20] + b"W" + raw[21:]), cfg, 12, "UnknownTensorName")
    # a file of another configuration: the first tensor's shape already differs
    _expect(wmod, pkg, path, wmod.ModelConfig.default(), 12, "ShapeMismatch")
    # a transposed matrix is a shape mismatch, not a silent reinterpretation
    tw2 = dict(tw)
    tw2["wfc1"] = [np.ascontiguousarray(a.T) for a in tw["wfc1"]]
    p = str(tmp_path / "transposed.bin")
    wmod.write_weight_file(p, tw2, vw)
    _expect(wmod, pkg, p, cfg, 12, "ShapeMismatch")


def test_element_count_word_is_ignored_and_a_repeated_name_keeps_its_last_record(wmod, small_file, tmp_path):
    path, tw, vw, cfg = small_file
    raw = bytearray(open(path, "rb").read())
    raw[16:20] = struct.pack("<I", 7)  # third header word of the first record: written, never read (weights.zig:140-141)
    p = str(tmp_path / "again.bin")
    with open(p, "wb") as f:
        f.write(bytes(raw))
        wmod.write_tensor(f, "t_ln_out_b", np.full(64, 0.5, np.float16))
    wf = wmod.WeightFile(p, cfg)
    try:
        assert len(wf) == 37
        assert float(wf.tensors()["t_ln_out_b"][0]) == 0.5  # dict(): the later record wins, as in the C tables
    finally:
        wf.close()
