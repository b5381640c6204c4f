"""CPU checks of the C-ABI boundary: the library loads without a GPU, exports every declared symbol, and the
host-side mirror of the reference's helpers behaves like the reference's."""
import os
import re

import numpy as np
import pytest

from conftest import ROOT


def _declared():
    text = open(os.path.join(ROOT, "include", "webgpt_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(wgpt_[a-z0-9_]+)\s*\(", text)))


@pytest.fixture(scope="module")
def lib():
    from webgpt_b200 import build, _lib
    build.build()
    return _lib.load()


def test_exports_every_declared_symbol(lib):
    from webgpt_b200 import _lib
    names = _declared()
    assert len(names) >= 35
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/webgpt_b200.h but not exported"
    bound = set(_lib.SIGNATURES) | set(_lib._SPECIAL)
    assert bound == set(names), (bound ^ set(names))


def test_abi_version_and_no_gpu_is_loud(lib):
    import ctypes as C
    assert lib.wgpt_abi_version() == 1
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    h = C.c_void_p()
    rc = lib.wgpt_device_create(0, C.byref(h))
    assert rc < 0 and not h.value
    assert len(lib.wgpt_last_error()) > 0
    from webgpt_b200 import Device, WgptError
    with pytest.raises(WgptError):
        Device(0)


def test_null_handles_are_rejected(lib):
    assert lib.wgpt_device_synchronize(None) == -8
    assert lib.wgpt_model_finalize(None) == -8
    assert lib.wgpt_session_reset(None) == -8
    assert b"null" in lib.wgpt_last_error()


def test_product_never_touches_the_oracle():
    """The shipped package must not import, load or execute anything under oracle/."""
    pkg = os.path.join(ROOT, "webgpt_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                src = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in src.lower(), f"{f} mentions the oracle"


def test_host_helpers_match_reference_semantics():
    from webgpt_b200 import globals as G
    # selectTopK: stable descending sort -> lowest index first on ties (globals.js:66-74)
    r = G.selectTopK(np.array([0.5, 2.0, 2.0, -1.0], np.float32), 3)
    assert r["topKIndices"] == [1, 2, 0]
    assert G.selectTopK([1.0, 1.0, 1.0], 1)["topKIndices"] == [0]
    p = G.cpuSoftmax([1.0, 2.0, 3.0], 0.5)
    e = np.exp((np.array([1.0, 2.0, 3.0]) - 3.0) / 0.5)
    assert np.allclose(p, e / e.sum())
    assert G.sampleFromDistribution([0.2, 0.3, 0.5], rand=0.0) == 0
    assert G.sampleFromDistribution([0.2, 0.3, 0.5], rand=0.2) == 1
    assert G.sampleFromDistribution([0.2, 0.3, 0.5], rand=0.9999) == 2
    assert G.sampleFromDistribution([0.2, 0.3], rand=0.9) == 1  # falls through to the last index
    a = np.arange(6, dtype=np.float32)
    assert np.array_equal(G.transpose(a, 2, 3), np.array([0, 3, 1, 4, 2, 5], np.float32))
    with pytest.raises(ValueError):
        G.transpose(a, 2, 2)
    assert G.wgSize(65, 64) == 2


def test_load_parameters_checks():
    from webgpt_b200.model import GPT
    ok = GPT(None, params=dict(n_layer=1, n_head=2, n_embd=32, n_ctx=8, vocab_size=10)).loadParameters(None)
    assert ok["head_size"] == 16 and ok["hidden_size"] == 128 and ok["vocab_chunk_instances"] == 1
    assert ok["attention_scale"] == pytest.approx(0.25)
    for bad, msg in [(dict(n_embd=30), "divisible by 4"), (dict(n_head=3), "divisible by n_head"),
                     (dict(n_embd=24, n_head=4), "n_embd / n_head")]:
        p = dict(n_layer=1, n_head=2, n_embd=32, n_ctx=8, vocab_size=10)
        p.update(bad)
        with pytest.raises(ValueError, match=msg):
            GPT(None, params=p).loadParameters(None)


def test_weight_folder_round_trip(tmp_path):
    """The reference's on-disk format: raw little-endian f32 per tensor + params_gpt.json."""
    import json
    from webgpt_b200 import globals as G, synth
    from webgpt_b200.model import GPT
    params = synth.CONFIGS["tiny"]
    w = synth.make_weights(params, seed=8, ln_random=True)
    folder = str(tmp_path / "tiny_model")
    synth.write_weight_folder(folder, params, w)
    assert len(os.listdir(folder)) == 1 + 4 + 12 * params["n_layer"]
    for name in synth.tensor_names(params):
        back = G.fetchBin(os.path.join(folder, f"{name}_gpt.bin"))
        assert back.dtype == np.float32 and np.array_equal(back, w[name].ravel())
    loaded = GPT(folder).loadParameters(folder)
    assert {k: loaded[k] for k in params} == params
    # HF-style config without n_ctx
    p2 = dict(json.load(open(os.path.join(folder, "params_gpt.json"))))
    p2["n_positions"] = p2.pop("n_ctx")
    json.dump(p2, open(os.path.join(folder, "params_gpt.json"), "w"))
    assert GPT(folder).loadParameters(folder)["n_ctx"] == params["n_ctx"]
