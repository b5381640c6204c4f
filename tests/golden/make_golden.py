"""Generates the committed golden vectors under tests/golden/.

Source of truth for gpt2_*.npz: HuggingFace transformers' GPT2LMHeadModel (CPU, f32) loaded with
the seeded synthetic weights of webgpt_b200.synth. The reference (0hq/WebGPT) implements the
same network on the same state-dict layout (other/conversion_scripts/convert_pretrained_pytorch.py
exports exactly this state dict; model.js:104-241 is its forward pass), and neither its
JavaScript nor its LFS-stored validation fixtures can be used in this environment, so an
independent implementation of the same mathematics pins the oracle instead.

attention_kat.npz restates the synthetic known-answer case of the reference's manual harness
(other/test.js:370-388): probabilities = head index + 1 under a causal mask, values = head
index + 1, whose expected output is (t + 1) * (h + 1)^2 for row t of head h.

Run from the repository root:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))

from webgpt_b200 import synth  # noqa: E402


def hf_model(params, weights):
    import torch
    from transformers import GPT2Config, GPT2LMHeadModel

    cfg = GPT2Config(vocab_size=params["vocab_size"], n_positions=params["n_ctx"], n_embd=params["n_embd"],
                     n_layer=params["n_layer"], n_head=params["n_head"], activation_function="gelu_new",
                     resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0, layer_norm_epsilon=1e-5)
    model = GPT2LMHeadModel(cfg).eval()
    sd = {k: torch.from_numpy(v.copy()) for k, v in weights.items()}
    sd["lm_head.weight"] = sd["transformer.wte.weight"]
    missing, unexpected = model.load_state_dict(sd, strict=False)
    assert not unexpected, unexpected
    assert all(".attn.bias" in m or ".attn.masked_bias" in m for m in missing), missing
    return model


def make_gpt2_case(name, cfg_name, n_prompt, n_new, seed, ln_random, std):
    import torch

    params = synth.CONFIGS[cfg_name]
    weights = synth.make_weights(params, seed=seed, std=std, ln_random=ln_random)
    prompt = synth.make_tokens(params["vocab_size"], n_prompt, seed=seed + 1)
    model = hf_model(params, weights)
    hist = [int(t) for t in prompt]
    step_logits = []
    with torch.no_grad():
        for _ in range(n_new):
            window = hist[-params["n_ctx"]:]
            out = model(torch.tensor([window], dtype=torch.long)).logits[0, -1].numpy().astype(np.float32)
            step_logits.append(out)
            hist.append(int(np.argmax(out)))
        full = model(torch.tensor([hist[:n_prompt]], dtype=torch.long), output_hidden_states=True)
    np.savez_compressed(
        os.path.join(HERE, name), config=cfg_name, seed=seed, ln_random=ln_random, std=std, prompt=prompt,
        history=np.array(hist, np.uint32), step_logits=np.stack(step_logits),
        prompt_last_hidden=full.hidden_states[-1][0].numpy().astype(np.float32),  # after ln_f
        prompt_emb=full.hidden_states[0][0].numpy().astype(np.float32))
    print(name, "history tail", hist[-5:])


def make_attention_kat():
    T, E, H = 15, 128, 4
    hs = E // H
    P = np.zeros((H * T, T), np.float32)
    for y in range(H * T):
        for x in range(T):
            P[y, x] = (y // T) + 1 if x <= y % T else 0
    V = np.zeros((T, E), np.float32)
    for x in range(E):
        V[:, x] = x // hs + 1
    expected = np.zeros((T, E), np.float32)
    for t in range(T):
        for c in range(E):
            h = c // hs
            expected[t, c] = (t + 1) * (h + 1) * (h + 1)
    np.savez_compressed(os.path.join(HERE, "attention_kat.npz"), P=P, V=V, expected=expected, H=H)


def make_sampling_kat():
    """Known answers of the sampling step (model.js:81-83) from the Python mirror of globals.js:47-74, which is
    written independently of the C oracle: rows of logits (distinct values, heavy ties with +0/-0, all equal),
    several top_k / temperature / uniform numbers each, the kept indices in order and the pick."""
    sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
    from webgpt_b200 import globals as G
    rng = np.random.default_rng(2024)
    V = 777
    rows = [
        (rng.standard_normal(V) * 4 - 30).astype(np.float32),
        (rng.standard_normal(V) * 4 + 10).astype(np.float32),
        np.round(rng.standard_normal(V) * 2).astype(np.float32),
        np.zeros(V, np.float32),
    ]
    rows[2][rows[2] == 0] *= rng.choice([-1.0, 1.0], size=int((rows[2] == 0).sum())).astype(np.float32)
    rows[3][1::2] = -0.0
    cases = []
    for ri, logits in enumerate(rows):
        for top_k in (1, 2, 3, 40, 100, 128):
            for temperature in (0.3, 1.0, 1.7):
                for u in (0.0, float(rng.random()), float(rng.random()), 0.9999999999):
                    sel = G.selectTopK(logits, top_k)
                    probs = G.cpuSoftmax(sel["topKProbs"], temperature)
                    pick = sel["topKIndices"][G.sampleFromDistribution(probs, u)]
                    cases.append((ri, top_k, temperature, u, pick))
    c = np.array(cases, np.float64)
    np.savez_compressed(os.path.join(HERE, "sampling_kat.npz"), logits=np.stack(rows), row=c[:, 0].astype(np.int32),
                        top_k=c[:, 1].astype(np.int32), temperature=c[:, 2], u=c[:, 3], pick=c[:, 4].astype(np.int32))


if __name__ == "__main__":
    make_attention_kat()
    make_sampling_kat()
    # std is larger than the benchmark's 0.02 so that greedy decoding does not collapse onto one token
    # window stays inside n_ctx
    make_gpt2_case("gpt2_tiny.npz", "tiny", n_prompt=5, n_new=8, seed=101, ln_random=True, std=0.2)
    # prompt 20 + 12 new tokens crosses n_ctx = 24: the window slides (model.js:69)
    make_gpt2_case("gpt2_tiny_slide.npz", "tiny", n_prompt=20, n_new=12, seed=202, ln_random=True, std=0.2)
    make_gpt2_case("gpt2_small.npz", "small", n_prompt=33, n_new=6, seed=303, ln_random=True, std=0.1)
