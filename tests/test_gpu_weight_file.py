"""A moondream.bin written by the package's writer, read by md_weight_file_open, made resident with
md_weight_file_upload and run through both models: outputs must equal, bit for bit, those of models built from
the same arrays uploaded one by one (the loader only moves bytes; weights.zig:61-207)."""
import importlib

import numpy as np
import pytest

import __graft_entry__ as entry
from conftest import f16_normal
from model_utils import text_weights, vision_weights

pytestmark = pytest.mark.gpu


def test_models_from_a_weight_file_equal_models_from_arrays(ctx, tmp_path):
    models = importlib.import_module(entry.PKG_NAME + ".models")
    wmod = importlib.import_module(entry.PKG_NAME + ".weights")
    tw = text_weights(5001, n_layers=2, hidden=1024, vocab=4096)
    vw = vision_weights(5002, n_layers=2, proj_hidden=1024)
    cfg = wmod.ModelConfig.scaled(n_layers=2, hidden_dim=1024, vocab=4096, n_vit_layers=2)
    path = str(tmp_path / "moondream.bin")
    wmod.write_weight_file(path, tw, vw)

    wf = wmod.WeightFile(path, cfg).upload(ctx)
    t_file, v_file = wf.text_model(), wf.vision_model(max_crops=2)
    t_arr, v_arr = models.TextModel(ctx, tw), models.VisionModel(ctx, vw, max_crops=2)
    try:
        rng = np.random.default_rng(9)
        embeds = f16_normal(rng, (70, 2048))
        outs = []
        for tm in (t_file, t_arr):
            req = tm.request()
            hidden, logits, tok = tm.forward(req, embeds)
            toks = tm.generate(req, tok, 6)
            outs.append((hidden, logits, tok, toks))
            req.close()
        assert np.array_equal(outs[0][0].view(np.uint16), outs[1][0].view(np.uint16))
        assert np.array_equal(outs[0][1].view(np.uint16), outs[1][1].view(np.uint16))
        assert outs[0][2] == outs[1][2] and np.array_equal(outs[0][3], outs[1][3])
        ids = np.array([0, 17, 4095], np.uint32)
        assert np.array_equal(t_file.text_encoder(ids).view(np.uint16), tw["wte"][ids].view(np.uint16))

        img = rng.integers(0, 256, (2, 378, 378, 3), dtype=np.uint8)
        o_file, f_file = v_file.encode(img, want_features=True)
        o_arr, f_arr = v_arr.encode(img, want_features=True)
        assert np.isfinite(o_file.astype(np.float32)).all()
        assert np.array_equal(f_file.view(np.uint16), f_arr.view(np.uint16))
        assert np.array_equal(o_file.view(np.uint16), o_arr.view(np.uint16))
    finally:
        for m in (t_file, v_file, t_arr, v_arr):
            m.close()
        wf.close()


def test_a_missing_tensor_is_reported_when_the_table_is_built(ctx, pkg, tmp_path):
    wmod = importlib.import_module(entry.PKG_NAME + ".weights")
    path = str(tmp_path / "partial.bin")
    import struct
    with open(path, "wb") as f:
        f.write(struct.pack("<II", wmod.WEIGHTS_MAGIC, wmod.WEIGHTS_VERSION))
        wmod.write_tensor(f, "t_ln_out_w", np.ones(2048, np.float16))
    wf = wmod.WeightFile(path).upload(ctx)
    try:
        with pytest.raises(pkg.MdError) as e:
            wf.text_model()
        assert e.value.status == 12 and e.value.zig_error == "error.MissingTensor"
    finally:
        wf.close()
