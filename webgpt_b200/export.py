"""Weight-directory exporter: state dict -> the folder format GPT(folder) loads.

Mirrors other/conversion_scripts/convert_pretrained_pytorch.py:16-42 (one raw little-endian f32 file
"<state-dict key>_gpt.bin" per tensor, buffers and the tied head skipped, the model configuration written as
params_gpt.json), for any mapping of names to arrays: a torch state dict (tensors are converted with
.detach().cpu().numpy()) or a dict of numpy arrays. Two on-disk conventions exist in the reference:
  * "in_out": matmul weights as [in, out], what HuggingFace GPT-2 (Conv1D) stores and model.js reads
    (model.js:405-420, 456-468);
  * "out_in": matmul weights as [out, in], what nanoGPT's nn.Linear stores and condensed/condensed.js transposes
    at load (condensed/condensed.js:1765-1784), with block_size for the context length (:1726) and, for
    bias-free checkpoints, no bias files at all (:1762-1782, model.js:322).
The convention is recorded in params_gpt.json as "weight_layout" so that the loader does not have to guess.
"""
import json
import os

import numpy as np

IGNORED = (".attn.masked_bias", ".attn.bias", "lm_head.weight")  # convert_pretrained_pytorch.py:16
MATMUL_WEIGHTS = ("attn.c_attn.weight", "attn.c_proj.weight", "mlp.c_fc.weight", "mlp.c_proj.weight")


def _to_numpy(v):
    if hasattr(v, "detach"):
        v = v.detach().cpu().numpy()
    return np.ascontiguousarray(v, dtype="<f4")


def export_weights_to_files(state_dict, folder_name, transpose_matmul_weights=False):
    """convert_pretrained_pytorch.py:19-37. transpose_matmul_weights writes each 2-D matmul weight transposed (the
    commented-out branch of the script, :33-35), i.e. converts between the two conventions on the way out."""
    os.makedirs(folder_name, exist_ok=True)
    written = []
    for k, v in state_dict.items():
        if any(i in k for i in IGNORED):
            continue
        values = _to_numpy(v)
        if transpose_matmul_weights and any(k.endswith(w) for w in MATMUL_WEIGHTS):
            values = np.ascontiguousarray(values.T)
        values.tofile(os.path.join(folder_name, f"{k}_gpt.bin"))
        written.append(k)
    return written


def save_model_args_to_json(config, folder_name, weight_layout="in_out"):
    """convert_pretrained_pytorch.py:40-42: the whole configuration dictionary, plus the layout marker."""
    cfg = dict(config.to_dict() if hasattr(config, "to_dict") else config)
    cfg["weight_layout"] = weight_layout
    with open(os.path.join(folder_name, "params_gpt.json"), "w") as f:
        json.dump(cfg, f, indent=4, default=str)


def export_model(state_dict, config, folder_name, weight_layout="in_out", source_layout="in_out"):
    """Writes state_dict (whose matmul weights are in source_layout) as a folder in weight_layout."""
    assert weight_layout in ("in_out", "out_in") and source_layout in ("in_out", "out_in")
    written = export_weights_to_files(state_dict, folder_name, transpose_matmul_weights=weight_layout != source_layout)
    save_model_args_to_json(config, folder_name, weight_layout)
    return written
