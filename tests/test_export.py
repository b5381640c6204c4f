"""Weight-directory exporter and loader round trip (no GPU): a randomly initialised HuggingFace GPT-2 of toy size is
written with webgpt_b200.export (the counterpart of other/conversion_scripts/convert_pretrained_pytorch.py), read
back through GPT's host-side loader in both on-disk conventions, and the CPU oracle run on the loaded tensors must
reproduce HuggingFace's own logits."""
import json
import os

import numpy as np
import pytest

from conftest import rel_err
from webgpt_b200 import GPT, export, synth


@pytest.fixture(scope="module")
def hf_model():
    torch = pytest.importorskip("torch")
    transformers = pytest.importorskip("transformers")
    torch.manual_seed(0)
    cfg = transformers.GPT2Config(n_layer=2, n_head=2, n_embd=32, n_positions=24, vocab_size=50,
                                  resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0)
    m = transformers.GPT2LMHeadModel(cfg).eval()
    with torch.no_grad():  # spread the values so LayerNorm scale/shift and biases matter
        for name, p in m.named_parameters():
            p.copy_(torch.randn_like(p) * (0.1 if p.dim() > 1 else 0.2) + (1.0 if "ln_" in name and name.endswith("weight") else 0.0))
    return m, cfg


def load_tensors(folder, **kw):
    g = GPT(folder, **kw)
    g.params = g.loadParameters(folder)   # host side only: no device is created
    names = synth.tensor_names(g.params)
    return g.params, [g._fetch(folder, n).reshape(synth.tensor_shape(g.params, n)) for n in names]


def test_state_dict_round_trip_both_layouts(hf_model, oracle, tmp_path):
    import torch
    m, cfg = hf_model
    ids = np.array([3, 14, 15, 9, 2, 6, 5, 35, 8, 9, 7, 49], np.uint32)
    with torch.no_grad():
        want = m(torch.tensor(ids.astype(np.int64))[None]).logits[0, -1].numpy()
    a = str(tmp_path / "in_out")
    written = export.export_model(m.state_dict(), cfg, a)
    assert not any(".attn.bias" in k or ".attn.masked_bias" in k or k == "lm_head.weight" for k in written)
    assert "transformer.h.1.attn.c_attn.bias" in written
    assert os.path.getsize(os.path.join(a, "transformer.h.0.attn.c_attn.weight_gpt.bin")) == 32 * 96 * 4
    params, tensors = load_tensors(a)
    assert params["n_ctx"] == 24 and params["weight_layout"] == "in_out"
    got = oracle.Model(params, tensors).run(ids)
    assert rel_err(got, want) < 2e-5
    # the nn.Linear convention: every block matrix stored [out, in]; the loader transposes it back
    b = str(tmp_path / "out_in")
    export.export_model(m.state_dict(), cfg, b, weight_layout="out_in")
    raw = np.fromfile(os.path.join(b, "transformer.h.1.mlp.c_fc.weight_gpt.bin"), "<f4").reshape(128, 32)
    assert np.array_equal(raw.T, m.state_dict()["transformer.h.1.mlp.c_fc.weight"].numpy())
    params_b, tensors_b = load_tensors(b)
    assert params_b["weight_layout"] == "out_in"
    for x, y in zip(tensors, tensors_b):
        assert np.array_equal(x, y)
    # a folder without the marker is taken as [in, out] unless the caller says otherwise
    with open(os.path.join(b, "params_gpt.json")) as f:
        cfg_json = json.load(f)
    del cfg_json["weight_layout"]
    cfg_json["block_size"] = cfg_json.pop("n_positions")   # nanoGPT's name, condensed/condensed.js:1726
    with open(os.path.join(b, "params_gpt.json"), "w") as f:
        json.dump(cfg_json, f)
    params_c, tensors_c = load_tensors(b, weight_layout="out_in")
    assert params_c["n_ctx"] == 24
    assert all(np.array_equal(x, y) for x, y in zip(tensors, tensors_c))


def test_bias_free_checkpoint_reads_zero_biases(hf_model, oracle, tmp_path):
    """bias: false in params_gpt.json (model.js:322) with the bias files absent, as nanoGPT writes them
    (condensed/condensed.js:1762-1782): every missing bias reads as zeros."""
    m, cfg = hf_model
    folder = str(tmp_path / "nobias")
    sd = {k: v for k, v in m.state_dict().items() if not k.endswith(".bias") or ".attn.bias" in k}
    export.export_model(sd, dict(cfg.to_dict(), bias=False), folder)
    assert not os.path.exists(os.path.join(folder, "transformer.h.0.ln_1.bias_gpt.bin"))
    params, tensors = load_tensors(folder)
    assert params["bias"] is False
    names = synth.tensor_names(params)
    for n, t in zip(names, tensors):
        if n.endswith(".bias"):
            assert not t.any(), n
    ids = np.array([1, 2, 3, 4], np.uint32)
    ref = oracle.Model(params, tensors).run(ids)
    assert np.isfinite(ref).all()
    # with the biases present but bias: true the same folder would fail to load a missing file
    with pytest.raises(FileNotFoundError):
        load_tensors(folder, params={**params, "bias": True})
