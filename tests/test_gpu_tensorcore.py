"""GPU parity of the tcgen05 tensor-core GEMM (TF32 and 3xTF32) against the CPU oracle, through the C ABI."""
import numpy as np
import pytest

from conftest import rel_err
from webgpt_b200 import synth

pytestmark = pytest.mark.gpu

TOL_X3 = 5e-5    # 3 x TF32: the operands are exact to ~2^-21; what remains is the tensor core's own FP32
                 # accumulation, which truncates, so the error grows with K (measured 2.3e-5 at K = 3072)
TOL_TF32 = 3e-3  # single TF32 product


@pytest.fixture(scope="module")
def dev():
    from webgpt_b200 import Device
    d = Device(0)
    yield d
    d.destroy()


def run_nk(dev, A, Wt, b, mode):
    from webgpt_b200 import _lib
    M, K = A.shape
    N = Wt.shape[0]
    dev.set_precision(mode)
    a_d, w_d, b_d, o_d = dev.tensor(A), dev.tensor(Wt), dev.tensor(b), dev.buffer(M * N * 4)
    try:
        _lib.call("wgpt_matmul_nk", dev.handle, M, N, K, a_d.ptr, w_d.ptr, b_d.ptr, o_d.ptr)
        _lib.call("wgpt_device_check", dev.handle)
        return o_d.read(np.float32, M * N).reshape(M, N)
    finally:
        dev.set_precision(_lib.PRECISION_TF32X3)


@pytest.mark.parametrize("M,K,N", [(128, 32, 128), (128, 64, 128), (256, 768, 768), (100, 96, 200), (64, 768, 2304),
                                   (512, 3072, 768), (333, 1600, 136), (1024, 768, 3072)])
def test_gemm_tc_matches_oracle(dev, oracle, M, K, N):
    from webgpt_b200 import _lib
    rng = np.random.default_rng(M + K + N)
    A = rng.standard_normal((M, K), dtype=np.float32)
    Wt = (rng.standard_normal((N, K), dtype=np.float32) * 0.05).astype(np.float32)
    b = rng.standard_normal(N, dtype=np.float32)
    ref = oracle.matmul(A, np.ascontiguousarray(Wt.T), b)
    got3 = run_nk(dev, A, Wt, b, _lib.PRECISION_TF32X3)
    assert rel_err(got3, ref) < TOL_X3
    got1 = run_nk(dev, A, Wt, b, _lib.PRECISION_TF32)
    assert rel_err(got1, ref) < TOL_TF32
    got0 = run_nk(dev, A, Wt, b, _lib.PRECISION_FP32)
    assert rel_err(got0, ref) < 1e-5
    # deterministic
    assert np.array_equal(run_nk(dev, A, Wt, b, _lib.PRECISION_TF32X3), got3)


def test_gemm_tc_index_pattern(dev):
    """Small integers are exact in TF32: the product must be bit-exact, which pins tile, swizzle and row/column
    mapping (any misplaced element changes an integer)."""
    from webgpt_b200 import _lib
    M, K, N = 256, 96, 256
    A = ((np.arange(M)[:, None] * 7 + np.arange(K)[None, :] * 3) % 11 - 5).astype(np.float32)
    Wt = ((np.arange(N)[:, None] * 5 + np.arange(K)[None, :]) % 13 - 6).astype(np.float32)
    b = np.arange(N, dtype=np.float32)
    ref = A.astype(np.float64) @ Wt.astype(np.float64).T + b
    for mode in (_lib.PRECISION_TF32, _lib.PRECISION_TF32X3):
        assert np.array_equal(run_nk(dev, A, Wt, b, mode).astype(np.float64), ref)


@pytest.mark.parametrize("K,N", [(768, 2304), (3072, 768)])
def test_gemm_tc_full_size_properties(dev, K, N):
    """The batched configuration's prefill GEMMs at full size (M = 8192 rows), checked through properties that do
    not need a CPU product of the whole matrix: integer operands are exact (every tile, every k-block and the
    persistent tile loop contribute an integer that float64 reproduces on a row sample), additivity in A, a row
    sample of a random product against float64, and bit-identical repeats."""
    from webgpt_b200 import _lib
    M = 8192
    rng = np.random.default_rng(K)
    rows = rng.choice(M, 96, replace=False)
    Ai = rng.integers(-3, 4, (M, K)).astype(np.float32)
    Wi = rng.integers(-3, 4, (N, K)).astype(np.float32)
    zero = np.zeros(N, np.float32)
    for mode in (_lib.PRECISION_TF32, _lib.PRECISION_TF32X3):
        got = run_nk(dev, Ai, Wi, zero, mode)
        assert np.array_equal(got[rows].astype(np.float64), Ai[rows].astype(np.float64) @ Wi.astype(np.float64).T)
        assert got.sum(dtype=np.float64) == (Ai.sum(0, dtype=np.float64) @ Wi.astype(np.float64).T).sum()
    A1 = rng.standard_normal((M, K), dtype=np.float32)
    A2 = rng.standard_normal((M, K), dtype=np.float32)
    Wt = (rng.standard_normal((N, K), dtype=np.float32) * 0.05).astype(np.float32)
    b = rng.standard_normal(N, dtype=np.float32)
    y1 = run_nk(dev, A1, Wt, b, _lib.PRECISION_TF32X3)
    y2 = run_nk(dev, A2, Wt, zero, _lib.PRECISION_TF32X3)
    y12 = run_nk(dev, A1 + A2, Wt, b, _lib.PRECISION_TF32X3)
    assert rel_err(y12, y1.astype(np.float64) + y2) < TOL_X3
    ref = A1[rows].astype(np.float64) @ Wt.astype(np.float64).T + b
    assert rel_err(y1[rows], ref) < TOL_X3
    assert np.array_equal(run_nk(dev, A1, Wt, b, _lib.PRECISION_TF32X3), y1)


def test_model_in_tf32x3_matches_oracle(oracle):
    """Prefill and batched decode through the tensor cores: logits within 1e-3 (required) / 5e-5 (asserted)."""
    from webgpt_b200 import GPT, _lib
    params = synth.CONFIGS["small"]
    w = synth.make_weights(params, seed=6, std=0.1, ln_random=True)
    gpt = GPT(None, params=params, weights=w)
    gpt.initialize()
    try:
        gpt.device.set_precision(_lib.PRECISION_TF32X3)
        m = oracle.Model(params, synth.weight_list(params, w))
        ids = synth.make_tokens(params["vocab_size"], 50, seed=4)
        assert rel_err(gpt.run(ids), m.run(ids)) < 5e-5
        n_seq = 12
        prompts = np.stack([synth.make_tokens(params["vocab_size"], 9, seed=20, stream=i) for i in range(n_seq)])
        batch = gpt.session(n_seq).generate_greedy(prompts, 10)
        for i in (0, 5, n_seq - 1):
            assert np.array_equal(batch[i], m.generate_greedy(prompts[i], 10)[9:])
    finally:
        gpt.destroy()


def test_batched_decode_gpt2_width(oracle):
    """GPT-2 width (d = 768, 12 heads of 64) cut to two layers, 16 and 64 sequences decoded together: the layer
    products run split-K with exchanged operands, the attention adds the QKV slices itself, the residual products'
    second stage applies the next LayerNorm, and the de-embedding runs without split. Tokens must equal the
    oracle's for every checked sequence, logits within 5e-5."""
    from webgpt_b200 import GPT
    params = dict(n_layer=2, n_head=12, n_embd=768, n_ctx=48, vocab_size=1000)
    w = synth.make_weights(params, seed=31, std=0.05, ln_random=True)
    m = oracle.Model(params, synth.weight_list(params, w))
    gpt = GPT(None, params=params, weights=w)
    gpt.initialize()
    try:
        for n_seq in (16, 64):
            prompts = np.stack([synth.make_tokens(params["vocab_size"], 7, seed=50, stream=i) for i in range(n_seq)])
            batch = gpt.session(n_seq).generate_greedy(prompts, 12)
            for i in (0, n_seq // 2, n_seq - 1):
                assert np.array_equal(batch[i], m.kv_generate_greedy(prompts[i], 12)), (n_seq, i)
            # logits of one more decode step of every sequence against the oracle's recompute
            s = gpt.session(n_seq)
            s.reset()
            s.forward(prompts, want_logits=False)
            lg = s.forward(batch[:, :1])
            for i in (1, n_seq - 2):
                ref = m.run(np.concatenate([prompts[i], batch[i, :1]]))
                assert rel_err(lg[i], ref) < 5e-5
    finally:
        gpt.destroy()


def test_prefill_8192_rows_gpt2_width(oracle):
    """The batched configuration's prefill at full row count through the model path: 64 sequences x 128 tokens =
    8192 rows at GPT-2 width (one layer, small vocabulary), i.e. the persistent 128x128-tile products with the
    weights' low parts fetched by TMA. Logits of the last position of sampled sequences against the oracle."""
    from webgpt_b200 import GPT
    params = dict(n_layer=1, n_head=12, n_embd=768, n_ctx=136, vocab_size=512)
    w = synth.make_weights(params, seed=33, std=0.05, ln_random=True)
    m = oracle.Model(params, synth.weight_list(params, w))
    gpt = GPT(None, params=params, weights=w)
    gpt.initialize()
    try:
        n_seq, n_tok = 64, 128
        prompts = np.stack([synth.make_tokens(params["vocab_size"], n_tok, seed=60, stream=i) for i in range(n_seq)])
        s = gpt.session(n_seq)
        s.reset()
        lg = s.forward(prompts)
        for i in (0, 17, n_seq - 1):
            assert rel_err(lg[i], m.run(prompts[i])) < 5e-5, i
        s.reset()
        assert np.array_equal(s.forward(prompts), lg)  # bit-identical repeat
    finally:
        gpt.destroy()


def test_batched_decode_xl_width(oracle):
    """GPT-2 XL width (d = 1600, 25 heads of 64) cut to two layers, 16 sequences decoded together: 1600 and 4800
    are not multiples of the 128-wide feature tile, so the last tile of every split-K product is ragged and the
    q | k | v boundaries fall inside tiles."""
    from webgpt_b200 import GPT
    params = dict(n_layer=2, n_head=25, n_embd=1600, n_ctx=32, vocab_size=512)
    w = synth.make_weights(params, seed=35, std=0.04, ln_random=True)
    m = oracle.Model(params, synth.weight_list(params, w))
    gpt = GPT(None, params=params, weights=w)
    gpt.initialize()
    try:
        n_seq = 16
        prompts = np.stack([synth.make_tokens(params["vocab_size"], 6, seed=70, stream=i) for i in range(n_seq)])
        batch = gpt.session(n_seq).generate_greedy(prompts, 8)
        for i in (0, 7, n_seq - 1):
            assert np.array_equal(batch[i], m.kv_generate_greedy(prompts[i], 8)), i
        s = gpt.session(n_seq)
        s.reset()
        s.forward(prompts, want_logits=False)
        lg = s.forward(batch[:, :1])
        for i in (2, n_seq - 1):
            assert rel_err(lg[i], m.run(np.concatenate([prompts[i], batch[i, :1]]))) < 5e-5
    finally:
        gpt.destroy()


PAIR_SCRIPT = r"""
import numpy as np, sys
from webgpt_b200 import Device, _lib
dev = Device(0)
rng = np.random.default_rng(3)
worst = 0.0
for (M, K, N) in [(8192, 768, 2304), (1000, 100, 520), (4100, 64, 2312), (2048, 3072, 3072)]:
    A = rng.standard_normal((M, K), dtype=np.float32)
    Wt = (rng.standard_normal((N, K), dtype=np.float32) * 0.05).astype(np.float32)
    b = rng.standard_normal(N, dtype=np.float32)
    rows = rng.choice(M, 64, replace=False)
    ref = A[rows].astype(np.float64) @ Wt.astype(np.float64).T + b
    Ai = rng.integers(-3, 4, (M, K)).astype(np.float32)
    Wi = rng.integers(-3, 4, (N, K)).astype(np.float32)
    refi = Ai[rows].astype(np.float64) @ Wi.astype(np.float64).T
    for mode, tol in ((_lib.PRECISION_TF32X3, 5e-5), (_lib.PRECISION_TF32, 3e-3)):
        dev.set_precision(mode)
        outs = []
        for (a, w, bias) in ((A, Wt, b), (Ai, Wi, np.zeros(N, np.float32))):
            a_d, w_d, b_d, o_d = dev.tensor(a), dev.tensor(w), dev.tensor(bias), dev.buffer(M * N * 4)
            _lib.call("wgpt_matmul_nk", dev.handle, M, N, K, a_d.ptr, w_d.ptr, b_d.ptr, o_d.ptr)
            _lib.call("wgpt_device_check", dev.handle)
            outs.append(o_d.read(np.float32, M * N).reshape(M, N))
            for buf in (a_d, w_d, b_d, o_d): buf.destroy()
        err = float(np.max(np.abs(outs[0][rows] - ref)) / np.max(np.abs(ref)))
        assert err < tol, (M, K, N, mode, err)
        assert np.array_equal(outs[1][rows].astype(np.float64), refi), (M, K, N, mode)
        worst = max(worst, err)
print("PAIR_OK", worst)
"""


def test_pair_gemm_all_shapes():
    """The CTA-pair kernel (two SMs on one 256 x 256 tile) forced on for every product that fits it, TF32 and
    3xTF32, including ragged tiles: integer operands must come out exact, random ones within the mode's tolerance.
    The switch is read once per process, hence the child process."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, WGPT_PAIR_GEMM="2", PYTHONPATH=root)
    r = subprocess.run([sys.executable, "-c", PAIR_SCRIPT], env=env, cwd=root, capture_output=True, text=True,
                       timeout=300)
    assert r.returncode == 0 and "PAIR_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
