"""GPU parity of the model-level C ABI (GPT.run / GPT.generate) against golden vectors and the CPU oracle."""
import numpy as np
import pytest

from conftest import load_golden, rel_err
from webgpt_b200 import synth

pytestmark = pytest.mark.gpu

TOL_LOGITS = 1e-3   # required: max|d| / max|ref| per logits vector
TIGHT = 5e-5        # what the FP32 paths actually achieve


def make_gpt(params, weights, fused=True):
    from webgpt_b200 import GPT
    g = GPT(None, params=params, weights=weights, fused=fused)
    g.initialize()
    return g


def golden_model(name, fused=True):
    g = load_golden(name)
    params = synth.CONFIGS[str(g["config"])]
    w = synth.make_weights(params, seed=int(g["seed"]), std=float(g["std"]), ln_random=bool(g["ln_random"]))
    return g, params, w, make_gpt(params, w, fused)


@pytest.mark.parametrize("name", ["gpt2_tiny.npz", "gpt2_tiny_slide.npz", "gpt2_small.npz"])
@pytest.mark.parametrize("fused", [True, False])
def test_generate_matches_golden(name, fused):
    g, params, w, gpt = golden_model(name, fused)
    try:
        n_prompt = len(g["prompt"])
        n_new = len(g["history"]) - n_prompt
        got = list(gpt.generate(g["prompt"], n_new, 1))
        assert got == [int(t) for t in g["history"][n_prompt:]]  # identical greedy ids
        # teacher-forced logits at every step, window sliding as model.js:69
        for i in range(n_new):
            window = g["history"][: n_prompt + i][-params["n_ctx"]:]
            assert rel_err(gpt.run(window), g["step_logits"][i]) < TIGHT
    finally:
        gpt.destroy()


def test_kv_cached_steps_equal_recompute(oracle):
    g, params, w, gpt = golden_model("gpt2_small.npz")
    try:
        m = oracle.Model(params, synth.weight_list(params, w))
        ids = synth.make_tokens(params["vocab_size"], 40, seed=9)
        s = gpt.session()
        s.reset()
        first = s.forward(ids[:7])[0]      # prefill of 7
        assert rel_err(first, m.run(ids[:7])) < TIGHT
        for t in range(7, 40):             # then one token at a time through the cache
            lg = s.forward(ids[t:t + 1])[0]
            if t in (7, 8, 20, 39):
                assert rel_err(lg, m.run(ids[: t + 1])) < TIGHT
        assert s.length() == 40
        # chunked prefill (3 + 30 + 7) lands on the same logits as one pass
        s.reset()
        s.forward(ids[:3], want_logits=False)
        s.forward(ids[3:33], want_logits=False)
        assert rel_err(s.forward(ids[33:40])[0], m.run(ids)) < TIGHT
    finally:
        gpt.destroy()


def _walsh(n):
    h = np.array([[1]], np.int64)
    while h.shape[0] < n:
        h = np.block([[h, h], [h, -h]])
    return h


def kv_index_pattern():
    """A one-layer model whose arithmetic is exact in f32 whatever the summation order, built so that the residual
    stream after the block spells out which cache rows each head read.

    E = 128 in four blocks of 32, four heads of 32. Position t carries the balanced +-1 Walsh code c_t and token id
    the code d_id: x_t = 16 * [c_t, c_t, d_id, d_id]. Such a row has mean 0 and variance 256 exactly, and
    256 + 1e-5 rounds to 256 in f32, so ln_1 (gamma 1, beta 0) gives exactly x_t / 16, whether a kernel divides by
    the deviation or multiplies by its reciprocal. The query of head 0 is 64 * c_(t-1), of head 1 64 * c_(t//2), of
    head 2 64 * c_0, of head 3 64 * c_t; keys are c_j: the matching key scores 2048 / sqrt(32), every other visible
    key 0, and exp(-362) is exactly 0, so each head's softmax is exactly one-hot. Values are c_j (heads 0, 3) and
    d_id_j (heads 1, 2); the output projection is the identity; ln_2 has gamma = beta = 0 and the MLP weights are
    zero, so the block adds exactly the selected value rows: small integers everywhere, TF32-exact as well."""
    E, H, hs, n_ctx, V = 128, 4, 32, 32, 64
    params = dict(n_layer=1, n_head=H, n_embd=E, n_ctx=n_ctx, vocab_size=V)
    W = _walsh(32)[1:]                       # 31 balanced, mutually orthogonal rows
    c = lambda t: W[t % 31]
    d = lambda i: W[(7 * i + 3) % 31]
    z = np.zeros(32, np.int64)
    wte = np.stack([16 * np.concatenate([z, z, d(i), d(i)]) for i in range(V)])
    wpe = np.stack([16 * np.concatenate([c(t), c(t), z, z]) for t in range(n_ctx)])
    sel = [lambda t: max(t - 1, 0), lambda t: t // 2, lambda t: 0, lambda t: t]
    # M_f c_t = c_f(t): sum over t of outer(c_f(t), c_t) / 32; times 64 the entries are even integers
    def qmap(f):
        return sum(np.outer(c(f(t)), c(t)) for t in range(31)) * 2   # = 64 * M_f
    wq = np.zeros((E, E), np.int64)
    wk = np.zeros((E, E), np.int64)
    wv = np.zeros((E, E), np.int64)
    I = np.eye(32, dtype=np.int64)
    for hd in range(4):
        o = slice(32 * hd, 32 * hd + 32)
        wq[0:32, o] = qmap(sel[hd]).T      # q = h . Wq reads the position code of block 0
        wk[0:32, o] = I
        wv[(0 if hd in (0, 3) else 64):(32 if hd in (0, 3) else 96), o] = I
    w = synth.make_weights(params, seed=1, std=0.0)
    f32 = lambda a: np.ascontiguousarray(a, dtype=np.float32)
    w["transformer.wte.weight"] = f32(wte)
    w["transformer.wpe.weight"] = f32(wpe)
    w["transformer.h.0.attn.c_attn.weight"] = f32(np.concatenate([wq, wk, wv], axis=1))
    w["transformer.h.0.attn.c_proj.weight"] = f32(np.eye(E))
    w["transformer.h.0.ln_2.weight"] = np.zeros(E, np.float32)

    def expected(ids):
        x = np.stack([wte[i] + wpe[t] for t, i in enumerate(ids)])
        out = x.copy()
        for t in range(len(ids)):
            for hd in range(4):
                j = sel[hd](t)
                val = c(j) if hd in (0, 3) else d(int(ids[j]))
                out[t, 32 * hd:32 * hd + 32] += val
        return out.astype(np.float32)
    return params, w, expected


@pytest.mark.parametrize("precision", ["fp32", "tf32x3"])
def test_kv_slot_indexing_exact(precision):
    """KV slot indexing, bit for bit: with the exact index-encoding model above, the residual stream after the
    block must equal the integer prediction exactly for every row, however the 24 tokens were fed (24 x 1, 1 x 24,
    5 + 1 + 1 + 17, 23 + 1): row t of the cache depends on (token t, position t) only (positions 0..T-1 of
    instructions.js:812-819, the [T, E] K/V rows read by :1141-1214). The logits of the newest row must then be
    bit-identical across chunkings as well."""
    from webgpt_b200 import _lib
    params, w, expected = kv_index_pattern()
    gpt = make_gpt(params, w)
    try:
        gpt.device.set_precision(_lib.PRECISION_FP32 if precision == "fp32" else _lib.PRECISION_TF32X3)
        ids = synth.make_tokens(params["vocab_size"], 24, seed=3)
        want = expected(ids)
        s = gpt.session()
        logits = []
        for chunks in ([24], [1] * 24, [5, 1, 1, 17], [23, 1], [9, 15]):
            s.reset()
            pos = 0
            for c in chunks:
                lg = s.forward(ids[pos:pos + c])[0]
                tap = s.tap()
                assert tap.shape == (c, params["n_embd"])
                assert np.array_equal(tap, want[pos:pos + c]), (chunks, pos)
                pos += c
            logits.append(lg)
        for lg in logits[1:]:
            assert np.array_equal(lg, logits[0])
        # a reset forgets everything: token 0 alone reproduces row 0
        s.reset()
        s.forward(ids[:1])
        assert np.array_equal(s.tap(), want[:1])
    finally:
        gpt.destroy()


def test_batch_equals_singles(oracle):
    """n_seq independent sequences in one session give the same tokens as each sequence alone."""
    params = synth.CONFIGS["small"]
    w = synth.make_weights(params, seed=6, std=0.1, ln_random=True)
    gpt = make_gpt(params, w)
    try:
        m = oracle.Model(params, synth.weight_list(params, w))
        for n_seq in (3, 8, 12):
            prompts = np.stack([synth.make_tokens(params["vocab_size"], 9, seed=20, stream=i) for i in range(n_seq)])
            batch = gpt.session(n_seq).generate_greedy(prompts, 10)
            for i in (0, n_seq - 1):
                want = m.generate_greedy(prompts[i], 10)[9:]
                assert np.array_equal(batch[i], want)
    finally:
        gpt.destroy()


def test_char_config_greedy_vs_oracle(oracle):
    """The reference's CPU-runnable configuration (char-level GPT, prompt 32) at reduced length."""
    params = synth.CONFIGS["char"]
    w = synth.make_weights(params, seed=1234)
    gpt = make_gpt(params, w)
    try:
        m = oracle.Model(params, synth.weight_list(params, w))
        prompt = synth.make_tokens(params["vocab_size"], 32, seed=7)
        n_new = 24
        want, trace = m.generate_greedy(prompt, n_new, trace=True)
        got = gpt.session().generate_greedy(prompt, n_new)[0]
        # teacher-forced comparison: a near-tie may flip an id without being a kernel error
        hist = list(prompt)
        for i in range(n_new):
            lg = gpt.run(hist)
            assert rel_err(lg, trace[i]) < TIGHT
            hist.append(int(want[32 + i]))
        top2 = np.sort(trace, axis=1)[:, -2:]
        gap = (top2[:, 1] - top2[:, 0]) / np.abs(trace).max(axis=1)
        if gap.min() > 1e-4:
            assert np.array_equal(got, want[32:])
    finally:
        gpt.destroy()


def test_errors_are_reported_not_fatal():
    from webgpt_b200 import WgptError, _lib
    params = synth.CONFIGS["tiny"]
    w = synth.make_weights(params, seed=1)
    gpt = make_gpt(params, w)
    try:
        with pytest.raises(WgptError) as e:
            gpt.run(list(range(params["n_ctx"] + 1)))
        assert e.value.code == _lib.ERR_SHAPE
        with pytest.raises(WgptError, match="out of range"):
            gpt.run([1, 2, params["vocab_size"]])
        lg = gpt.run([1, 2, 3])  # the device is still usable afterwards
        assert np.isfinite(lg).all()
        with pytest.raises(WgptError) as e:
            _lib.call("wgpt_model_set_tensor", gpt.model_handle, b"transformer.wte.weight", lg.ctypes.data, 3)
        assert e.value.code == _lib.ERR_STATE
    finally:
        gpt.destroy()


def test_tap_is_pre_lnf_residual_stream(oracle):
    g, params, w, gpt = golden_model("gpt2_small.npz")
    try:
        m = oracle.Model(params, synth.weight_list(params, w))
        _, taps = m.run(g["prompt"], taps=True)
        gpt.run(g["prompt"])
        got = gpt.session().tap()
        assert got.shape == taps[-2].shape
        assert np.max(np.abs(got - taps[-2])) < 1e-3  # validation.js:216 bound on r2 of the last block
        assert rel_err(got, taps[-2]) < TIGHT
    finally:
        gpt.destroy()


def test_xl_shape_two_layers(oracle):
    """GPT-2 XL geometry (d=1600, 25 heads of 64, 4d=6400) cut to two layers and a small vocabulary: exercises
    K = 1600 / 6400 (not multiples of 128), the register-streaming GEMV where a block does not fit shared memory,
    and 25 heads, in prefill (tensor cores), single-token decode and a 3-sequence batch."""
    params = dict(n_layer=2, n_head=25, n_embd=1600, n_ctx=96, vocab_size=1000)
    w = synth.make_weights(params, seed=11, std=0.05, ln_random=True)
    gpt = make_gpt(params, w)
    try:
        m = oracle.Model(params, synth.weight_list(params, w))
        ids = synth.make_tokens(params["vocab_size"], 70, seed=12)
        assert rel_err(gpt.run(ids), m.run(ids)) < TIGHT
        s = gpt.session()
        s.reset()
        s.forward(ids[:66], want_logits=False)
        for t in range(66, 70):
            lg = s.forward(ids[t:t + 1])[0]
        assert rel_err(lg, m.run(ids)) < TIGHT
        prompts = np.stack([synth.make_tokens(params["vocab_size"], 5, seed=13, stream=i) for i in range(3)])
        got = gpt.session(3).generate_greedy(prompts, 6)
        for i in range(3):
            assert np.array_equal(got[i], m.generate_greedy(prompts[i], 6)[5:])
    finally:
        gpt.destroy()


def test_generate_longer_than_context_from_long_prompt(oracle):
    """Prompt longer than n_ctx: the first window is the newest n_ctx tokens and every step slides (model.js:69)."""
    params = synth.CONFIGS["tiny"]
    w = synth.make_weights(params, seed=21, std=0.2, ln_random=True)
    gpt = make_gpt(params, w)
    try:
        m = oracle.Model(params, synth.weight_list(params, w))
        prompt = synth.make_tokens(params["vocab_size"], params["n_ctx"] + 7, seed=22)
        want = m.generate_greedy(prompt, 5)[len(prompt):]
        got = gpt.session().generate_greedy(prompt, 5)[0]
        assert np.array_equal(got, want)
    finally:
        gpt.destroy()


def test_visuals_heatmap_matches_oracle(oracle, tmp_path):
    """Visuals.render: the tap of the last run coloured by the reference's fragment-shader arithmetic, bit-exact."""
    from webgpt_b200.visuals import Visuals
    g, params, w, gpt = golden_model("gpt2_small.npz")
    try:
        vis = Visuals(gpt)
        vis.init()
        gpt.run(g["prompt"])
        img = vis.render(ppm_path=str(tmp_path / "v.ppm"))
        m = oracle.Model(params, synth.weight_list(params, w))
        _, taps = m.run(g["prompt"], taps=True)
        T = len(g["prompt"])
        tap = gpt.session().tap()
        assert np.array_equal(img[:T], oracle.heatmap(tap))          # same bytes for the same floats
        assert np.mean(img[:T] != oracle.heatmap(taps[-2])) < 1e-3   # and for the oracle's own residual stream
        assert not img[T:].any()
        assert (tmp_path / "v.ppm").stat().st_size == len(b"P6\n128 64\n255\n") + 64 * 128 * 3
        # scaled inputs reach every branch of the colour map
        big = (np.random.default_rng(0).standard_normal((params["n_ctx"], params["n_embd"])) * 12).astype(np.float32)
        vis.embeddingsBuffer.write(big)
        assert np.array_equal(vis.render(), oracle.heatmap(big))
        vis.destroy()
    finally:
        gpt.destroy()


@pytest.mark.parametrize("fused", [True, False])
def test_load_from_weight_folder(tmp_path, fused):
    """GPT(folder) reads the reference's directory format and computes what GPT(weights=...) computes."""
    from webgpt_b200 import GPT
    params = synth.CONFIGS["tiny"]
    w = synth.make_weights(params, seed=8, std=0.2, ln_random=True)
    folder = str(tmp_path / "m")
    synth.write_weight_folder(folder, params, w)
    a = GPT(folder, fused=fused)
    a.initialize()
    b = make_gpt(params, w, fused)
    try:
        ids = synth.make_tokens(params["vocab_size"], 9, seed=2)
        assert np.array_equal(a.run(ids), b.run(ids))
    finally:
        a.destroy()
        b.destroy()


def test_load_linear_layout_and_bias_free_folder(tmp_path):
    """The second on-disk convention (nn.Linear [out, in] matrices and block_size, condensed/condensed.js:1726,
    1765-1784) and a bias-free checkpoint (bias files absent, model.js:322) load to the same logits as the same
    weights handed over in memory."""
    from webgpt_b200 import GPT, export
    params = synth.CONFIGS["tiny"]
    w = synth.make_weights(params, seed=8, std=0.2, ln_random=True)
    for k in w:
        if k.endswith(".bias"):
            w[k] = np.zeros_like(w[k])
    cfg = {"n_layer": 2, "n_head": 2, "n_embd": 32, "block_size": 24, "vocab_size": 50, "bias": False}
    sd = {k: v for k, v in w.items() if not k.endswith(".bias")}
    folder = str(tmp_path / "lin")
    export.export_model(sd, cfg, folder, weight_layout="out_in")
    a = GPT(folder)
    a.initialize()
    b = make_gpt(params, w)
    try:
        ids = synth.make_tokens(params["vocab_size"], 9, seed=2)
        assert np.array_equal(a.run(ids), b.run(ids))
        assert list(a.generate(ids, 5, 1)) == list(b.generate(ids, 5, 1))
    finally:
        a.destroy()
        b.destroy()


def test_sharded_generation_inside_the_library_equals_unsharded(oracle):
    """wgpt_generate_greedy_sharded: the sequences of one call split over several device handles, one host thread
    each, joined inside the library. With one GPU present the handles sit on the same GPU (two streams); with more,
    on different GPUs. The gathered ids must equal the unsharded ids and the oracle's."""
    import ctypes as C
    from webgpt_b200 import WgptError, _lib
    from webgpt_b200.sharding import MultiGPT
    params = synth.CONFIGS["small"]
    w = synth.make_weights(params, seed=6, std=0.1, ln_random=True)
    n_seq, n_prompt, n_new = 11, 9, 10
    prompts = np.stack([synth.make_tokens(params["vocab_size"], n_prompt, seed=20, stream=i) for i in range(n_seq)])
    n_dev = 1
    try:
        import torch
        n_dev = max(1, torch.cuda.device_count())
    except Exception:
        pass
    devices = [i % n_dev for i in range(max(2, min(n_dev, 4)))]
    multi = MultiGPT(params, w, devices)
    single = make_gpt(params, w)
    try:
        got = multi.generate_greedy(prompts, n_new)
        want = single.session(n_seq).generate_greedy(prompts, n_new)
        assert np.array_equal(got, want)
        m = oracle.Model(params, synth.weight_list(params, w))
        for i in (0, 5, n_seq - 1):
            assert np.array_equal(got[i], m.generate_greedy(prompts[i], n_new)[n_prompt:])
        # two sessions on one device handle are refused
        g = multi.gpts[0]
        from webgpt_b200.model import Session
        s1, s2 = Session(g, 1), Session(g, 1)
        arr = (C.c_void_p * 2)(s1.handle, s2.handle)
        out = np.empty((2, 2), np.uint32)
        with pytest.raises(WgptError) as e:
            _lib.call("wgpt_generate_greedy_sharded", arr, 2, prompts.ctypes.data, n_prompt, 2, out.ctypes.data)
        assert e.value.code == _lib.ERR_ARG
        s1.destroy()
        s2.destroy()
    finally:
        multi.destroy()
        single.destroy()


@pytest.mark.parametrize("precision,tol", [("tf32x3", 5e-5), ("tf32", 5e-3), ("fp32", 5e-5)])
def test_prefill_attention_head64_chunked(oracle, precision, tol):
    """Prefill attention for head size 64 (tensor-core kernel in the TF32 modes, CUDA-core kernel in FP32): windows of
    16..129 tokens appended to a cache that already holds earlier positions, with partial last tiles, against one
    oracle pass over the whole window (instructions.js:1101-1214: causal mask by absolute position)."""
    from webgpt_b200 import _lib
    params = dict(synth.CONFIGS["small"])
    params.update(n_embd=128, n_head=2, n_layer=2, n_ctx=256, vocab_size=96)
    w = synth.make_weights(params, seed=31, std=0.08, ln_random=True)
    m = oracle.Model(params, synth.weight_list(params, w))
    ids = synth.make_tokens(params["vocab_size"], 230, seed=9)
    ref = m.kv_logits(ids)  # ref[t] = logits after feeding ids[0..t]
    gpt = make_gpt(params, w)
    try:
        gpt.device.set_precision({"fp32": _lib.PRECISION_FP32, "tf32x3": _lib.PRECISION_TF32X3,
                                  "tf32": _lib.PRECISION_TF32}[precision])
        s = gpt.session()
        for chunks in ([230], [16, 129, 65, 20], [100, 1, 64, 17, 48], [3, 200, 27]):
            s.reset()
            pos = 0
            for c in chunks:
                lg = s.forward(ids[pos:pos + c])[0]
                pos += c
                assert rel_err(lg, ref[pos - 1]) < tol, (precision, chunks, pos)
    finally:
        gpt.destroy()
