"""Seeded synthetic weights and token ids with the shapes of the reference's models.

The reference ships its weights as Git-LFS blobs (weights/gpt2, weights/better_shakespeare;
model.js:270-454 loads them); the benchmark configurations ask for seeded N(0, 0.02) weights,
LayerNorm gamma = 1 / beta = 0, and uniform random token ids instead. Tensors come out in the
on-disk convention written by other/conversion_scripts/convert_pretrained_pytorch.py:31-37:
one f32 array per state-dict key, matmul weights as [in, out].
"""
import numpy as np

CONFIGS = {
    # nanoGPT shakespeare_char shape
    "char": dict(n_layer=6, n_head=6, n_embd=384, n_ctx=256, vocab_size=65),
    "gpt2": dict(n_layer=12, n_head=12, n_embd=768, n_ctx=1024, vocab_size=50257),
    "gpt2-xl": dict(n_layer=48, n_head=25, n_embd=1600, n_ctx=1024, vocab_size=50257),
    # small shapes for tests
    "tiny": dict(n_layer=2, n_head=2, n_embd=32, n_ctx=24, vocab_size=50),
    "small": dict(n_layer=3, n_head=4, n_embd=128, n_ctx=64, vocab_size=211),
}

LAYER_KEYS = [
    "ln_1.weight", "ln_1.bias", "attn.c_attn.weight", "attn.c_attn.bias", "attn.c_proj.weight", "attn.c_proj.bias",
    "ln_2.weight", "ln_2.bias", "mlp.c_fc.weight", "mlp.c_fc.bias", "mlp.c_proj.weight", "mlp.c_proj.bias",
]


def tensor_names(params):
    names = ["transformer.wte.weight", "transformer.wpe.weight", "transformer.ln_f.weight", "transformer.ln_f.bias"]
    for l in range(params["n_layer"]):
        names += [f"transformer.h.{l}.{k}" for k in LAYER_KEYS]
    return names


def tensor_shape(params, name):
    E, V, C = params["n_embd"], params["vocab_size"], params["n_ctx"]
    if name.endswith("wte.weight"):
        return (V, E)
    if name.endswith("wpe.weight"):
        return (C, E)
    if name.endswith("c_attn.weight"):
        return (E, 3 * E)
    if name.endswith("c_attn.bias"):
        return (3 * E,)
    if name.endswith("attn.c_proj.weight"):
        return (E, E)
    if name.endswith("c_fc.weight"):
        return (E, 4 * E)
    if name.endswith("c_fc.bias"):
        return (4 * E,)
    if name.endswith("mlp.c_proj.weight"):
        return (4 * E, E)
    return (E,)


def make_weights(params, seed=1234, std=0.02, ln_random=False):
    """Returns {name: f32 array}. Matrices, embeddings and biases ~ N(0, std); LayerNorm
    gamma = 1, beta = 0 unless ln_random (then gamma ~ 1 + N(0, 0.1), beta ~ N(0, 0.1), which
    exercises the scale/shift arithmetic in tests)."""
    out = {}
    for i, name in enumerate(tensor_names(params)):
        shape = tensor_shape(params, name)
        rng = np.random.default_rng([seed, i])
        is_ln = ".ln_" in name
        if is_ln and not ln_random:
            out[name] = np.ones(shape, np.float32) if name.endswith("weight") else np.zeros(shape, np.float32)
        elif is_ln:
            base = 1.0 if name.endswith("weight") else 0.0
            out[name] = (base + 0.1 * rng.standard_normal(shape, dtype=np.float32)).astype(np.float32)
        else:
            out[name] = (rng.standard_normal(shape, dtype=np.float32) * np.float32(std)).astype(np.float32)
    return out


def weight_list(params, weights):
    """Weights in tensor_names order (the order tensor_names gives)."""
    return [weights[n] for n in tensor_names(params)]


def make_tokens(vocab_size, n, seed=7, stream=0):
    rng = np.random.default_rng([seed, 1000 + stream])
    return rng.integers(0, vocab_size, size=n, dtype=np.uint32)


def make_int8_case(M, K, N, seed=11):
    """int8 weight-only GEMM inputs: q uniform in [-127,127] packed 4 per u32 little-endian along
    N (byte j of word w in row k = column 4w+j, other/int8-gemm.js:36-42), per-column scales
    ~ U(0.001, 0.02), activations ~ N(0,1)."""
    rng = np.random.default_rng([seed, M, K, N])
    q = rng.integers(-127, 128, size=(K, N), dtype=np.int8)
    packed = np.ascontiguousarray(q).view(np.uint32).reshape(K, N // 4).copy()
    scales = rng.uniform(0.001, 0.02, size=N).astype(np.float32)
    A = rng.standard_normal((M, K), dtype=np.float32)
    return A, q, packed, scales


def write_weight_folder(path, params, weights):
    """Writes a weight directory in the reference's on-disk format: params_gpt.json plus one raw little-endian
    f32 file "<state-dict key>_gpt.bin" per tensor (other/conversion_scripts/convert_pretrained_pytorch.py:19-42;
    read back by model.js:289-291, 341, 371, 379-383, 405-420)."""
    import json
    import os
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "params_gpt.json"), "w") as f:
        json.dump({k: params[k] for k in ("n_layer", "n_head", "n_embd", "n_ctx", "vocab_size")}, f, indent=4)
    for name in tensor_names(params):
        np.ascontiguousarray(weights[name], dtype="<f4").tofile(os.path.join(path, f"{name}_gpt.bin"))
