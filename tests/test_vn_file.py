"""The `.vn` container reader against files the reference's own writer produced (tests/golden/model_tiny_*.vn,
written by CometSparkNexLM.save_vn with safetensors and with its .npz fallback)."""

import os

import numpy as np
import pytest

from versenext_b200.vn_file import VNFileReader

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("name,fmt", [("model_tiny_st.vn", "safetensors"), ("model_tiny_npz.vn", "npz")])
def test_reader_returns_the_reference_state_dict(golden, name, fmt):
    g = golden("vn_reference.npz")
    want = {n[3:]: g[n] for n in g.files if n.startswith("sd.")}
    with VNFileReader(os.path.join(GOLDEN, name)) as r:
        meta = r.read_meta()
        assert meta["arch"] == "versenex" and r.vn_format_version in (1, 2) and r.weight_format == fmt
        assert meta["weight_count"] == len(want)
        cfg = r.read_config()
        assert cfg["vocab_size"] == 96 and cfg["dim"] == 32 and cfg["layer_pattern"] == ["mod", "trisparse"]
        got = r.read_weights()
        assert r.read_chat_template() is None and r.read_tokenizer() is None
    assert set(got) == set(want)
    for n, w in want.items():
        assert got[n].dtype == np.float32 and got[n].shape == w.shape
        np.testing.assert_array_equal(got[n], w, err_msg=n)


def test_reader_rejects_other_files(tmp_path):
    import zipfile
    p = tmp_path / "x.vn"
    with zipfile.ZipFile(p, "w") as z:
        z.writestr("config.yml", "{}")
    with pytest.raises(ValueError):
        VNFileReader(str(p)).read_meta()
    with zipfile.ZipFile(p, "w") as z:
        z.writestr("meta.json", '{"vn_format_version": 9}')
    with pytest.raises(ValueError):
        VNFileReader(str(p)).read_meta()
    with zipfile.ZipFile(p, "w") as z:
        z.writestr("meta.json", '{"vn_format_version": 2, "weight_format": "npz"}')
        z.writestr("config.yml", "{}")
    with pytest.raises(ValueError):
        VNFileReader(str(p)).read_weights()


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["model_tiny_st.vn", "model_tiny_npz.vn"])
def test_from_pretrained_matches_the_reference_forward(golden, name, tmp_path):
    import shutil
    import versenext_b200 as vn
    g = golden("vn_reference.npz")
    m = vn.VerseNexLM.from_pretrained(os.path.join(GOLDEN, name))
    got = np.asarray(m(g["tokens"]).data)
    assert float(np.max(np.abs(got - g["logits"])) / np.max(np.abs(g["logits"]))) < 1e-3
    # directory form: <dir>/model.vn
    shutil.copy(os.path.join(GOLDEN, name), tmp_path / "model.vn")
    m2 = vn.VerseNexLM.from_pretrained(str(tmp_path))
    np.testing.assert_array_equal(np.asarray(m2(g["tokens"]).data), got)
    (tmp_path / "empty").mkdir()
    with pytest.raises(FileNotFoundError):
        vn.VerseNexLM.from_pretrained(str(tmp_path / "empty"))
    with pytest.raises(ValueError):
        vn.VerseNexLM.from_pretrained(str(tmp_path / "model.pt"))
