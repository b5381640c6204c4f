"""GPU parity of on-device top-k sampling (model.js:81-83, globals.js:47-74) against the CPU oracle: the pick
is an index, so every comparison is exact."""
import numpy as np
import pytest

from webgpt_b200 import synth

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    from webgpt_b200 import Device
    d = Device(0)
    yield d
    d.destroy()


def device_picks(dev, rows, top_k, temperature, u):
    from webgpt_b200 import _lib
    rows = np.ascontiguousarray(rows, np.float32)
    n, V = rows.shape
    lg, ud, out = dev.tensor(rows), dev.tensor(np.ascontiguousarray(u, np.float64)), dev.buffer(n * 4)
    _lib.call("wgpt_sample_topk", dev.handle, lg.ptr, n, V, top_k, float(temperature), ud.ptr, out.ptr)
    got = out.read(np.uint32, n)
    for b in (lg, ud, out):
        b.destroy()
    return got


@pytest.mark.parametrize("V", [5, 130, 1000, 1024, 1025, 4097, 50257])
def test_sample_topk_rows(dev, oracle, V):
    rng = np.random.default_rng(V)
    n = 12
    distinct = (rng.standard_normal((n, V)) * 4 - 30).astype(np.float32)
    tied = np.round(rng.standard_normal((n, V)) * 2).astype(np.float32)   # few distinct values, +0 and -0 mixed
    tied[tied == 0] *= rng.choice([-1.0, 1.0], size=int((tied == 0).sum())).astype(np.float32)
    for rows in (distinct, tied):
        for top_k in sorted({1, 2, 3, min(40, V), min(100, V), min(128, V)}):
            for temperature in (0.3, 1.0, 1.7):
                u = rng.random(n)
                u[0], u[1] = 0.0, 0.9999999999
                got = device_picks(dev, rows, top_k, temperature, u)
                want = [oracle.sample_topk(rows[i], top_k, temperature, u[i]) for i in range(n)]
                assert [int(t) for t in got] == want, (V, top_k, temperature)


def test_sample_topk_all_equal_and_clustered(dev, oracle):
    """Worst cases of the candidate search: every logit equal (order is index order alone), and the largest values
    all falling into one thread's strided share of the row."""
    V = 50257
    flat = np.zeros((2, V), np.float32)
    flat[1, 1::2] = -0.0
    clustered = np.full((2, V), -50.0, np.float32)
    clustered[0, 7::1024] = np.linspace(5, 6, len(clustered[0, 7::1024]), dtype=np.float32)
    clustered[1, 1023::1024] = 3.0
    for rows in (flat, clustered):
        for top_k in (1, 49, 128):
            for u in ([0.0, 0.5], [0.97, 0.9999999]):
                got = device_picks(dev, rows, top_k, 1.0, np.array(u))
                want = [oracle.sample_topk(rows[i], top_k, 1.0, u[i]) for i in range(2)]
                assert [int(t) for t in got] == want


def test_sample_topk_rejects_bad_arguments(dev):
    from webgpt_b200 import WgptError, _lib
    a = dev.tensor(np.zeros(64, np.float32))
    u = dev.tensor(np.zeros(1, np.float64))
    for top_k, temperature, code in ((0, 1.0, _lib.ERR_SHAPE), (129, 1.0, _lib.ERR_SHAPE), (65, 1.0, _lib.ERR_SHAPE),
                                     (2, 0.0, _lib.ERR_ARG)):
        with pytest.raises(WgptError) as e:
            _lib.call("wgpt_sample_topk", dev.handle, a.ptr, 1, 64, top_k, temperature, u.ptr, a.ptr)
        assert e.value.code == code


def make_gpt(params, weights, fused=True):
    from webgpt_b200 import GPT
    g = GPT(None, params=params, weights=weights, fused=fused)
    g.initialize()
    return g


@pytest.mark.parametrize("config,n_prompt,n_new", [("tiny", 4, 10), ("small", 9, 40)])
@pytest.mark.parametrize("top_k,temperature", [(2, 1.0), (3, 0.8), (40, 1.3)])
def test_generate_sample_matches_oracle(oracle, config, n_prompt, n_new, top_k, temperature):
    params = synth.CONFIGS[config]
    w = synth.make_weights(params, seed=21, std=0.15, ln_random=True)
    m = oracle.Model(params, synth.weight_list(params, w))
    gpt = make_gpt(params, w)
    try:
        n_seq = 3
        prompts = np.stack([synth.make_tokens(params["vocab_size"], n_prompt, seed=40 + q) for q in range(n_seq)])
        u = np.random.default_rng(top_k).random((n_new, n_seq))
        got = gpt.session(n_seq).generate_sample(prompts, n_new, top_k, temperature, u)
        for q in range(n_seq):
            want = m.kv_generate_sample(prompts[q], n_new, top_k, temperature, u[:, q])
            assert np.array_equal(got[q], want), q
        assert len({int(t) for t in got.ravel()}) > 3  # the sampler does move between tokens
        # the same call again replays the captured decode step and must reproduce itself
        assert np.array_equal(gpt.session(n_seq).generate_sample(prompts, n_new, top_k, temperature, u), got)
        # top_k = 1 is the greedy pick whatever the random numbers
        one = gpt.session(n_seq).generate_sample(prompts, n_new, 1, temperature, u)
        assert np.array_equal(one, gpt.session(n_seq).generate_greedy(prompts, n_new))
    finally:
        gpt.destroy()


def test_generate_sample_sliding_window(oracle):
    """Past n_ctx the window slides and every step recomputes it (model.js:69); the step counter that indexes the
    random numbers keeps running through the switch."""
    params = synth.CONFIGS["tiny"]
    w = synth.make_weights(params, seed=22, std=0.15, ln_random=True)
    m = oracle.Model(params, synth.weight_list(params, w))
    gpt = make_gpt(params, w)
    try:
        prompt = synth.make_tokens(params["vocab_size"], 6, seed=2)
        n_new = params["n_ctx"] + 5
        u = np.random.default_rng(3).random(n_new)
        got = gpt.session().generate_sample(prompt, n_new, 3, 0.9, u)[0]
        assert np.array_equal(got, m.generate_sample(prompt, n_new, 3, 0.9, u)[6:])
    finally:
        gpt.destroy()


def test_gpt_generate_routes_agree(oracle):
    """GPT.generate(prompt, n, top_k, temperature) with the same random-number source: the fused route (picks on
    the device) and the pass-list route (logits read back, the three helpers on the host) yield the same ids."""
    params = synth.CONFIGS["small"]
    w = synth.make_weights(params, seed=23, std=0.15, ln_random=True)
    prompt = [int(t) for t in synth.make_tokens(params["vocab_size"], 7, seed=4)]
    outs = []
    for fused in (True, False):
        gpt = make_gpt(params, w, fused)
        try:
            rng = np.random.default_rng(11)
            outs.append(list(gpt.generate(prompt, 12, "3", "0.8", rand=lambda: float(rng.random()))))
        finally:
            gpt.destroy()
    assert outs[0] == outs[1]


def test_sample_topk_golden(dev):
    """Device picks against the committed known answers (made from the Python mirror of globals.js:47-74,
    independent of the C oracle)."""
    from conftest import load_golden
    g = load_golden("sampling_kat.npz")
    keys = sorted({(int(k), float(t)) for k, t in zip(g["top_k"], g["temperature"])})
    for k, t in keys:
        sel = [i for i in range(len(g["pick"])) if int(g["top_k"][i]) == k and float(g["temperature"][i]) == t]
        rows = g["logits"][g["row"][sel]]
        got = device_picks(dev, rows, k, t, g["u"][sel])
        assert [int(x) for x in got] == [int(x) for x in g["pick"][sel]], (k, t)
