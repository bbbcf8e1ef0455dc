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


def _delta_vn_case():
    from oracle import model as OM
    cfg = OM.Config(vocab_size=64, dim=32, n_layer=3, n_head=2, n_kv_head=1, layer_pattern=["trisparse", "vda", "dsa"],
                    window_size=8, num_global_tokens=3, use_alibi=False, use_rope=True, max_seq_len=64, init_std=0.2)
    return cfg, OM.init_state_dict(cfg, seed=302, gate_std=1.0)


def test_reader_on_a_file_with_delta_attention_layers(golden):
    """A model with vda / dsa layers written by the reference's writer: names of the modules' tensors, layer kinds in
    config.yml (the writer stores neither anchor_interval nor latent_dim: they come back as the defaults), and the
    oracle's forward on what was read."""
    from oracle import model as OM
    g = golden("vn_delta_reference.npz")
    cfg, sd = _delta_vn_case()
    with VNFileReader(os.path.join(GOLDEN, "model_tiny_delta.vn")) as r:
        r.read_meta()
        conf = r.read_config()
        got = r.read_weights()
    assert conf["layer_pattern"] == ["trisparse", "vda", "dsa"] and "anchor_interval" not in conf
    want = {n: w for n, w in sd.items() if not (n == "head.weight" and cfg.tie_weights)}
    assert set(got) - {"head.weight"} == set(want) - {"head.weight"}
    for n in ("blocks.1.attn.gmla.w_kv_down.weight", "blocks.1.attn.dsa.global_tokens.weight",
              "blocks.1.attn.kda.wk.weight", "blocks.1.attn.gate_logits", "blocks.2.attn.head_gate_logits"):
        np.testing.assert_array_equal(got[n], sd[n], err_msg=n)
    lg, _ = OM.forward(sd, cfg, g["tokens"])
    np.testing.assert_allclose(lg, g["logits"], rtol=2e-4, atol=2e-5)


@pytest.mark.gpu
def test_from_pretrained_with_delta_attention_layers(golden):
    import versenext_b200 as vn
    g = golden("vn_delta_reference.npz")
    m = vn.VerseNexLM.from_pretrained(os.path.join(GOLDEN, "model_tiny_delta.vn"))
    assert m.layer_pattern == ["trisparse", "vda", "dsa"] and m.anchor_interval == 128
    got = np.asarray(m(g["tokens"]).data)
    assert float(np.max(np.abs(got - g["logits"])) / np.max(np.abs(g["logits"]))) < 1e-3
