"""CPU tests of the oracle: golden vectors (independent HF implementation), the reference's
known-answer patterns, and numpy restatements of each kernel."""
import numpy as np
import pytest

from conftest import load_golden, rel_err
from webgpt_b200 import synth

TOL_LOGITS = 1e-3  # other/validation/validation.js:216; the target is far tighter
TIGHT = 2e-5


def _oracle_model(orc, g):
    params = synth.CONFIGS[str(g["config"])]
    w = synth.make_weights(params, seed=int(g["seed"]), std=float(g["std"]), ln_random=bool(g["ln_random"]))
    return params, orc.Model(params, synth.weight_list(params, w))


@pytest.mark.parametrize("name", ["gpt2_tiny.npz", "gpt2_tiny_slide.npz", "gpt2_small.npz"])
def test_generate_matches_golden(oracle, name):
    g = load_golden(name)
    params, m = _oracle_model(oracle, g)
    n_new = len(g["history"]) - len(g["prompt"])
    hist, trace = m.generate_greedy(g["prompt"], n_new, trace=True)
    assert np.array_equal(hist, g["history"])  # greedy ids identical (validation.js:301)
    for i in range(n_new):
        assert rel_err(trace[i], g["step_logits"][i]) < TIGHT


@pytest.mark.parametrize("name", ["gpt2_tiny.npz", "gpt2_small.npz"])
def test_taps_match_golden(oracle, name):
    g = load_golden(name)
    params, m = _oracle_model(oracle, g)
    _, taps = m.run(g["prompt"], taps=True)
    assert taps.shape[0] == 2 + 6 * params["n_layer"]
    assert np.max(np.abs(taps[0] - g["prompt_emb"])) < 1e-6
    assert np.max(np.abs(taps[-1] - g["prompt_last_hidden"])) < 1e-3  # validation.js tolerance
    assert rel_err(taps[-1], g["prompt_last_hidden"]) < TIGHT


def test_kv_cached_equals_recompute(oracle):
    g = load_golden("gpt2_small.npz")
    params, m = _oracle_model(oracle, g)
    ids = g["history"][:39]
    kv = m.kv_logits(ids)
    for t in (0, 1, 7, 38):
        assert rel_err(kv[t], m.run(ids[: t + 1])) < TIGHT
    new = m.kv_generate_greedy(g["prompt"], 6)
    assert np.array_equal(new, g["history"][len(g["prompt"]):])


def test_attention_values_known_answer(oracle):
    """other/test.js:370-388: head-indexed probabilities and values."""
    g = load_golden("attention_kat.npz")
    out = oracle.attn_values(g["P"], g["V"], int(g["H"]))
    assert np.array_equal(out, g["expected"])


def test_matmul_vs_numpy(oracle):
    rng = np.random.default_rng(0)
    for M, K, N in [(1, 8, 8), (3, 12, 16), (15, 128, 384), (33, 384, 128)]:
        A = rng.standard_normal((M, K), dtype=np.float32)
        B = rng.standard_normal((K, N), dtype=np.float32)
        b = rng.standard_normal(N, dtype=np.float32)
        ref = A.astype(np.float64) @ B.astype(np.float64) + b
        assert rel_err(oracle.matmul(A, B, b), ref) < 1e-5
        assert rel_err(oracle.matmul(A, B), ref - b) < 1e-5


def test_layernorm_softmax_gelu_vs_numpy(oracle):
    rng = np.random.default_rng(1)
    for M, N in [(1, 4), (3, 60), (15, 384), (2, 5000)]:
        x = (3 * rng.standard_normal((M, N))).astype(np.float32)
        gm = rng.standard_normal(N).astype(np.float32)
        bt = rng.standard_normal(N).astype(np.float32)
        x64 = x.astype(np.float64)
        mean = x64.mean(1, keepdims=True)
        sd = np.sqrt(x64.var(1, keepdims=True) + 1e-5)
        y, stats = oracle.layernorm(x, gm, bt, return_stats=True)
        assert np.max(np.abs(y - ((x64 - mean) / sd * gm + bt))) < 2e-5
        assert np.max(np.abs(stats[:, 0] - mean[:, 0])) < 1e-5 and np.max(np.abs(stats[:, 1] - sd[:, 0])) < 1e-5
        e = np.exp(x64 - x64.max(1, keepdims=True))
        assert np.max(np.abs(oracle.softmax(x) - e / e.sum(1, keepdims=True))) < 1e-6
        gl = 0.5 * x64 * (1 + np.tanh(0.7978845608 * (x64 + 0.044715 * x64 ** 3)))
        assert np.max(np.abs(oracle.gelu(x) - gl)) < 1e-5
    edge = np.array([[-11.0, -10.0, 10.0, 11.0, 0.0, -0.0, 50.0, -50.0]], np.float32)
    ge = oracle.gelu(edge)[0]
    assert ge[0] == 0.0 and ge[3] == 11.0 and ge[6] == 50.0 and ge[7] == 0.0  # clamps, instructions.js:724-727
    assert oracle.softmax(np.full((1, 7), -1e9, np.float32)).sum() == pytest.approx(1.0, abs=1e-6)


def test_attention_blocks_vs_numpy(oracle):
    rng = np.random.default_rng(2)
    T, E, H = 15, 128, 4  # T % 4 != 0: the reference's withCheck matmul variant
    hs = E // H
    x = rng.standard_normal((T, E), dtype=np.float32)
    W = [0.1 * rng.standard_normal((E, E), dtype=np.float32) for _ in range(4)]
    b = [0.1 * rng.standard_normal(E, dtype=np.float32) for _ in range(4)]
    scale = np.float32(1 / np.sqrt(hs))
    out = oracle.attention(x, H, scale, W[0], b[0], W[1], b[1], W[2], b[2], W[3], b[3])
    x64 = x.astype(np.float64)
    q, k, v = (x64 @ W[i] + b[i] for i in range(3))
    o = np.zeros((T, E))
    for h in range(H):
        sl = slice(h * hs, (h + 1) * hs)
        s = q[:, sl] @ k[:, sl].T * float(scale)
        s = np.where(np.tril(np.ones((T, T), bool)), s, -1e9)
        p = np.exp(s - s.max(1, keepdims=True))
        p /= p.sum(1, keepdims=True)
        o[:, sl] = p @ v[:, sl]
    assert rel_err(out, o @ W[3] + b[3]) < 1e-5
    # formatQ index arithmetic, instructions.js:1130-1135
    Q = np.arange(T * E, dtype=np.float32).reshape(T, E)
    Qf = oracle.format_q(Q, hs)
    assert np.array_equal(Qf.reshape(H, T, hs), Q.reshape(T, H, hs).transpose(1, 0, 2))
    S = oracle.attn_weights(Qf, Q, H, 1.0)
    assert np.all(S.reshape(H, T, T)[:, np.triu_indices(T, 1)[0], np.triu_indices(T, 1)[1]] == np.float32(-1e9))


def test_embed_deembed(oracle):
    rng = np.random.default_rng(3)
    V, E, T = 70, 16, 9
    wte = rng.standard_normal((V, E), dtype=np.float32)
    wpe = rng.standard_normal((T + 3, E), dtype=np.float32)
    idx = rng.integers(0, V, T).astype(np.uint32)
    assert np.array_equal(oracle.embed(idx, wte, wpe), wte[idx] + wpe[:T])
    x = rng.standard_normal(E, dtype=np.float32)
    assert rel_err(oracle.deembed(x, wte), wte.astype(np.float64) @ x) < 1e-5


def test_int8_pack_unpack_bit_exact(oracle):
    # exhaustive over one byte lane, in each of the four lanes (other/int8-gemm.js:126-131)
    for lane in range(4):
        words = (np.arange(256, dtype=np.uint32) << (8 * lane)).view(np.int32)
        got = oracle.int8_unpack(words).reshape(256, 4)
        assert np.array_equal(got[:, lane], np.arange(256, dtype=np.uint8).view(np.int8))
        assert np.all(np.delete(got, lane, axis=1) == 0)
    rng = np.random.default_rng(4)
    words = rng.integers(0, 2 ** 32, 4096, dtype=np.uint64).astype(np.uint32)
    assert np.array_equal(oracle.int8_unpack(words.view(np.int32)), words.view(np.int8))
    # quantise -> pack -> unpack round trip (other/int8-gemm.js:25-62); halves round toward +inf
    x = np.array([1.0, -1.0, 0.5, -0.5, 1.5, -1.5, 0.0, 0.25, 63.5, -63.5, 126.49, -126.51], np.float32)
    for absmax in (1.0, 127.0, 0.3):
        xs = x if absmax == 127.0 else (x / 127 * absmax).astype(np.float32)
        q = oracle.int8_unpack(oracle.int8_quantize(xs, absmax))
        want = [int(np.floor(float(v) / absmax * 127 + 0.5)) for v in xs]  # JS Math.round in f64
        assert list(q) == want
    q = oracle.int8_unpack(oracle.int8_quantize(x, 127.0))
    assert list(q[:6]) == [1, -1, 1, 0, 2, -1]  # exact halves go toward +infinity


def test_int8_matmul(oracle):
    for M, K, N in [(1, 64, 32), (3, 96, 64), (16, 128, 256)]:
        A, q, packed, scales = synth.make_int8_case(M, K, N)
        assert np.array_equal(oracle.int8_unpack(packed.view(np.int32).ravel()).reshape(K, N), q)
        ref = A.astype(np.float64) @ (q.astype(np.float64) * scales.astype(np.float64))
        out = oracle.int8_matmul(A, packed, scales, N)
        assert rel_err(out, ref) < 1e-5
        lit = oracle.int8_matmul(A, packed, scales, N, literal=True)
        assert rel_err(lit, ref) < 1e-5
        # the reference's own acceptance bound: |cpu - gpu| <= 0.1 per element (int8-gemm.js:321)
        assert np.max(np.abs(out - ref)) < 0.1


def test_model_rejects_bad_params(oracle):
    params = dict(synth.CONFIGS["tiny"], n_head=3)  # n_embd % n_head != 0, model.js:295
    with pytest.raises(ValueError):
        oracle.Model(params, [np.zeros(1, np.float32)] * (4 + 12 * params["n_layer"]))


def test_heatmap_known_values(oracle):
    """visuals.js:104-135 on hand-computed pixels."""
    v = np.array([0.0, 5.0, -5.0, 10.0, 15.0, -15.0, 17.0, -30.0, 1e9], np.float32)
    px = oracle.heatmap(v)
    assert px[0].tolist() == [0, 0, 0, 0]
    assert px[1].tolist() == [128, 0, 0, 0]      # 0.5 -> 127.5 -> rounds to 128
    assert px[2].tolist() == [0, 0, 128, 0]
    assert px[3].tolist() == [255, 0, 0, 0]      # exactly the threshold: no green yet
    assert px[4].tolist() == [255, 128, 0, 0]    # 1.5: green = 0.5
    assert px[5].tolist() == [0, 128, 255, 0]
    assert px[6].tolist() == [255, 179, 0, 0]    # green capped at 0.7 -> 178.5 -> 179
    assert px[7].tolist() == [0, 179, 255, 0]
    assert px[8].tolist() == [255, 179, 0, 0]


def _sample_cases():
    rng = np.random.default_rng(77)
    cases = []
    for V in (5, 257, 1000, 50257):
        cases.append(rng.standard_normal(V).astype(np.float32) * 4 - 30)           # distinct values
        cases.append(np.round(rng.standard_normal(V) * 2).astype(np.float32))      # many exact ties, +0 and -0
    z = np.zeros(64, np.float32)
    z[1::2] = -0.0
    cases.append(z)                                                                 # all equal under JS ordering
    return cases


def test_sample_topk_matches_host_mirror(oracle):
    """The C restatement of model.js:81-83 against the Python mirror of the same three helpers
    (globals.js:47-74), written independently: same kept indices in the same order, same pick."""
    from webgpt_b200 import globals as G
    rng = np.random.default_rng(5)
    for logits in _sample_cases():
        for top_k in (1, 2, 3, 40, 100):
            for temperature in (0.1, 0.7, 1.0, 2.0):
                for u in (0.0, float(rng.random()), float(rng.random()), 0.9999999999):
                    got, top = oracle.sample_topk(logits, top_k, temperature, u, return_top=True)
                    sel = G.selectTopK(logits, top_k)
                    assert [int(t) for t in top] == sel["topKIndices"]
                    probs = G.cpuSoftmax(sel["topKProbs"], temperature)
                    assert got == sel["topKIndices"][G.sampleFromDistribution(probs, u)]
    # top_k = 1 is the greedy pick
    x = _sample_cases()[1]
    assert oracle.sample_topk(x, 1, 1.0, 0.5) == int(oracle.lib().orc_argmax(oracle._f(x)[1], x.size))


def test_sampled_generation_kv_equals_recompute(oracle):
    params = synth.CONFIGS["tiny"]
    w = synth.make_weights(params, seed=3, std=0.15, ln_random=True)
    m = oracle.Model(params, synth.weight_list(params, w))
    prompt = synth.make_tokens(params["vocab_size"], 5, seed=1)
    n_new = params["n_ctx"] - 5
    u = np.random.default_rng(8).random(n_new)
    a = m.kv_generate_sample(prompt, n_new, 3, 0.8, u)
    b = m.generate_sample(prompt, n_new, 3, 0.8, u)
    assert np.array_equal(a, b[5:])
    assert len(set(int(t) for t in a)) > 1
    # top_k = 1 ignores the random numbers and equals the greedy loop
    assert np.array_equal(m.kv_generate_sample(prompt, n_new, 1, 0.8, u), m.kv_generate_greedy(prompt, n_new))


def test_sample_topk_golden(oracle):
    """The committed sampling known answers (tests/golden/sampling_kat.npz, made by make_golden.py from the Python
    mirror of globals.js:47-74) against the C restatement."""
    g = load_golden("sampling_kat.npz")
    for r, k, t, u, pick in zip(g["row"], g["top_k"], g["temperature"], g["u"], g["pick"]):
        assert oracle.sample_topk(g["logits"][r], int(k), float(t), float(u)) == int(pick)


def test_int8_quantize_matrix_matches_the_flat_quantiser(oracle):
    """The matrix form with one absmax for the matrix is the prototype's quantizeMatrix (other/int8-gemm.js:25-46)
    word for word; with per-column maxima each column equals the flat quantiser run on that column with its own
    absmax, and dequantised values stay within half a step of the weights."""
    rng = np.random.default_rng(3)
    K, N = 24, 16
    w = (rng.standard_normal((K, N)) * 0.05).astype(np.float32)
    w[:, 5] = 0.0                                  # a zero column
    w[3, 2] = np.float32(0.5) * np.abs(w[:, 2]).max() / np.float32(127)   # a rounding half
    packed, scale = oracle.int8_quantize_matrix(w, per_column=False)
    absmax = float(np.abs(w).max())
    assert np.array_equal(packed.reshape(-1), oracle.int8_quantize(w.reshape(-1), absmax))
    assert np.all(scale == np.float32(absmax / 127.0))
    packed, scale = oracle.int8_quantize_matrix(w, per_column=True)
    q = oracle.int8_unpack(packed.reshape(-1)).reshape(K, N)
    for n in range(N):
        a = float(np.abs(w[:, n]).max())
        if a == 0.0:
            assert not q[:, n].any() and scale[n] == 0.0
            continue
        col = np.repeat(w[:, n], 4)                # the flat quantiser packs 4 consecutive values
        ref = oracle.int8_unpack(oracle.int8_quantize(col, a))[::4]
        assert np.array_equal(q[:, n], ref)
        assert scale[n] == np.float32(a / 127.0)
    assert np.max(np.abs(q * scale[None, :] - w)) <= 0.5001 * scale.max()
