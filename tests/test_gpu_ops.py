"""GPU parity of each operator entry point of the C ABI against the CPU oracle (run with -m gpu)."""
import numpy as np
import pytest

from conftest import load_golden, rel_err

pytestmark = pytest.mark.gpu

TOL = 2e-5  # relative, FP32 paths (the reference's own bound is 1e-3 absolute, validation.js:216)
TOL_X3 = 5e-5  # products of 32 rows and more run on the tensor cores in 3xTF32 (see test_gpu_tensorcore.py)


@pytest.fixture(scope="module")
def dev():
    from webgpt_b200 import Device
    d = Device(0)
    yield d
    d.destroy()


@pytest.fixture(scope="module")
def ops(dev):
    from webgpt_b200 import globals as G
    G.initializeOperations(dev)
    yield G
    G.destroyOperations()


def run(inst):
    for p in inst["passes"]:
        assert p["flag"] == "compute"
        p["run"]()
    return inst["resultBuffer"]


@pytest.mark.parametrize("M,K,N", [(1, 8, 8), (1, 768, 2304), (3, 12, 16), (4, 384, 384), (8, 3072, 768),
                                   (15, 128, 384), (33, 384, 1536), (256, 768, 768), (1, 1600, 6400),
                                   (1024, 768, 2304), (100, 1600, 72)])
def test_matmul(dev, ops, oracle, M, K, N):
    rng = np.random.default_rng(M * 1000 + N)
    A = rng.standard_normal((M, K), dtype=np.float32)
    B = (rng.standard_normal((K, N), dtype=np.float32) * 0.05).astype(np.float32)
    b = rng.standard_normal(N, dtype=np.float32)
    out = run(ops.FastMatMulBlock.newInstance(M, N, K, dev.tensor(A), dev.tensor(B), dev.tensor(b)))
    got = out.read(np.float32, M * N).reshape(M, N)
    assert rel_err(got, oracle.matmul(A, B, b)) < (TOL if M < 32 else TOL_X3)
    # deterministic: the split-K sums are added in a fixed order
    out2 = run(ops.FastMatMulBlock.newInstance(M, N, K, dev.tensor(A), dev.tensor(B), dev.tensor(b)))
    assert np.array_equal(out2.read(np.float32, M * N).reshape(M, N), got)


def test_matmul_rejects_bad_shapes(dev, ops):
    from webgpt_b200 import WgptError, _lib
    with pytest.raises(ValueError, match="divisible by 16"):
        ops.FastMatMulBlock.newInstance(4, 12, 8, None, None, None)
    a = dev.tensor(np.zeros(64, np.float32))
    with pytest.raises(WgptError) as e:
        _lib.call("wgpt_matmul", dev.handle, 1, 12, 8, a.ptr, a.ptr, None, a.ptr)
    assert e.value.code == _lib.ERR_SHAPE and "divisible by 16" in e.value.message
    with pytest.raises(WgptError) as e:
        _lib.call("wgpt_matmul", dev.handle, 1, 8, 8, a.ptr + 4, a.ptr, None, a.ptr)
    assert e.value.code == _lib.ERR_ALIGN
    with pytest.raises(WgptError) as e:
        _lib.call("wgpt_gelu", dev.handle, 1, 6, a.ptr, a.ptr)
    assert "divisible by 4" in e.value.message


@pytest.mark.parametrize("M,N", [(1, 4), (3, 60), (15, 384), (1, 768), (2, 5000), (64, 1600)])
def test_elementwise_ops(dev, ops, oracle, M, N):
    rng = np.random.default_rng(M + N)
    x = (3 * rng.standard_normal((M, N))).astype(np.float32)
    y = rng.standard_normal((M, N), dtype=np.float32)
    g = rng.standard_normal(N, dtype=np.float32)
    b = rng.standard_normal(N, dtype=np.float32)
    xb, yb = dev.tensor(x), dev.tensor(y)
    got = run(ops.ResidualBlock.newInstance(M, N, xb, yb)).read(np.float32, M * N).reshape(M, N)
    assert np.array_equal(got, oracle.residual(x, y))  # one f32 add: bit exact
    got = run(ops.LayerNormBlock.newInstance(M, N, xb, dev.tensor(g), dev.tensor(b))).read(np.float32, M * N)
    assert np.max(np.abs(got.reshape(M, N) - oracle.layernorm(x, g, b))) < 2e-5
    got = run(ops.GeluBlock.newInstance(M, N, xb)).read(np.float32, M * N).reshape(M, N)
    assert np.max(np.abs(got - oracle.gelu(x))) < 2e-6
    got = run(ops.SoftmaxBlock.newInstance(M, N, xb)).read(np.float32, M * N).reshape(M, N)
    assert np.max(np.abs(got - oracle.softmax(x))) < 1e-6


def test_gelu_clamps_and_softmax_odd(dev, ops, oracle):
    edge = np.array([[-11.0, -10.0, 10.0, 11.0, 0.0, -0.0, 50.0, -50.0]], np.float32)
    got = run(ops.GeluBlock.newInstance(1, 8, dev.tensor(edge))).read(np.float32, 8)
    assert np.array_equal(got[[0, 3, 6, 7]], np.array([0.0, 11.0, 50.0, 0.0], np.float32))
    for cols in (1, 3, 15, 33, 257):
        x = np.random.default_rng(cols).standard_normal((5, cols)).astype(np.float32)
        got = run(ops.SoftmaxBlock.newInstance(5, cols, dev.tensor(x))).read(np.float32, 5 * cols).reshape(5, cols)
        assert np.max(np.abs(got - oracle.softmax(x))) < 1e-6


def test_embed_deembed(dev, ops, oracle):
    rng = np.random.default_rng(5)
    V, E, T = 211, 128, 33
    wte = rng.standard_normal((V, E), dtype=np.float32)
    wpe = rng.standard_normal((64, E), dtype=np.float32)
    idx = rng.integers(0, V, T).astype(np.uint32)
    wb, pb = dev.tensor(wte), dev.tensor(wpe)
    emb = run(ops.EmbedBlock.newInstance(idx, T, E, V, [wb], pb, ops.ResidualBlock))
    got = emb.read(np.float32, T * E).reshape(T, E)
    assert np.array_equal(got, oracle.embed(idx, wte, wpe))
    logits = run(ops.DeEmbedBlock.newInstance(E, V, V, T, V, emb, [wb])).read(np.float32, V)
    assert rel_err(logits, oracle.deembed(got[-1], wte)) < TOL
    from webgpt_b200 import WgptError
    bad = idx.copy()
    bad[3] = V
    with pytest.raises(WgptError, match="out of range"):
        run(ops.EmbedBlock.newInstance(bad, T, E, V, [wb], pb, ops.ResidualBlock))


@pytest.mark.parametrize("T,E,H", [(1, 32, 2), (3, 64, 4), (15, 128, 4), (33, 384, 6), (100, 768, 12), (40, 256, 2)])
def test_attention(dev, ops, oracle, T, E, H):
    rng = np.random.default_rng(T + E)
    hs = E // H
    x = rng.standard_normal((T, E), dtype=np.float32)
    W = [(rng.standard_normal((E, E), dtype=np.float32) / np.sqrt(E)).astype(np.float32) for _ in range(4)]
    b = [0.1 * rng.standard_normal(E, dtype=np.float32) for _ in range(4)]
    scale = 1 / np.sqrt(hs)
    t = dev.tensor
    inst = ops.AttentionBlock.newFusedInstance(T, E, scale, H, hs, t(x), t(W[0]), t(b[0]), t(W[1]), t(b[1]), t(W[2]),
                                               t(b[2]), t(W[3]), t(b[3]), ops.FastMatMulBlock, ops.SoftmaxBlock)
    got = run(inst).read(np.float32, T * E).reshape(T, E)
    ref = oracle.attention(x, H, np.float32(scale), W[0], b[0], W[1], b[1], W[2], b[2], W[3], b[3])
    assert rel_err(got, ref) < (TOL if T < 32 else TOL_X3)


def test_attention_known_answer(dev, ops):
    """The head-indexed pattern of other/test.js:370-388, pushed through the whole attention operator:
    identity-like projections make Q.K constant per head so the softmax is uniform over the visible keys, and
    V = head index + 1 must come back unchanged for every row."""
    T, E, H = 15, 128, 4
    hs = E // H
    g = load_golden("attention_kat.npz")
    x = g["V"]  # rows of (head index + 1)
    eye = np.eye(E, dtype=np.float32)
    z = np.zeros(E, np.float32)
    t = dev.tensor
    inst = ops.AttentionBlock.newFusedInstance(T, E, 1 / np.sqrt(hs), H, hs, t(x), t(eye), t(z), t(eye), t(z), t(eye),
                                               t(z), t(eye), t(z))
    got = run(inst).read(np.float32, T * E).reshape(T, E)
    assert np.max(np.abs(got - x)) < 1e-5


@pytest.mark.parametrize("M,K,N", [(1, 768, 3072), (1, 3072, 768), (16, 768, 3072), (16, 1600, 6400), (4, 64, 32),
                                   (3, 96, 64), (256, 768, 3072), (40, 128, 72)])
def test_int8_matmul(dev, oracle, M, K, N):
    from webgpt_b200 import _lib, synth
    A, q, packed, scales = synth.make_int8_case(M, K, N)
    out, a_d, b_d, s_d = dev.buffer(M * N * 4), dev.tensor(A), dev.tensor(packed), dev.tensor(scales)
    _lib.call("wgpt_int8_matmul", dev.handle, M, K, N, a_d.ptr, b_d.ptr, s_d.ptr, out.ptr)
    got = out.read(np.float32, M * N).reshape(M, N)
    assert rel_err(got, oracle.int8_matmul(A, packed, scales, N)) < TOL
    assert np.max(np.abs(got - oracle.int8_matmul(A, packed, scales, N, literal=True))) < 0.1  # int8-gemm.js:321


@pytest.mark.parametrize("K", [8, 64, 40])
def test_int8_unpack_bit_exact(dev, K):
    """One-hot activations and unit scales read the unpacked integers back out of the kernel exactly; every byte
    value appears in every lane."""
    from webgpt_b200 import _lib
    N = 1024
    vals = np.arange(K * N, dtype=np.int64)
    q = ((vals * 37 + vals // N) % 256).astype(np.uint8).view(np.int8).reshape(K, N)
    packed = np.ascontiguousarray(q).view(np.uint32).reshape(K, N // 4)
    for M in (1, K if K <= 16 else 16, K):
        A = np.eye(K, dtype=np.float32)[:M]
        out, a_d, b_d, s_d = dev.buffer(M * N * 4), dev.tensor(A), dev.tensor(packed), dev.tensor(np.ones(N, np.float32))
        _lib.call("wgpt_int8_matmul", dev.handle, M, K, N, a_d.ptr, b_d.ptr, s_d.ptr, out.ptr)
        got = out.read(np.float32, M * N).reshape(M, N)
        assert np.array_equal(got, q[:M].astype(np.float32))


@pytest.mark.parametrize("K", [16, 64, 48])
def test_int8_weight_handle_unpack_bit_exact(dev, K):
    """The re-laid-out copy of a weight handle (bytes [N, K]) holds exactly the prototype's codes: one-hot
    activations and unit scales read them back through the streaming kernel (1 to 4 rows), every byte value in every
    lane of the words."""
    import ctypes as C
    from webgpt_b200 import _lib
    N = 1024
    vals = np.arange(K * N, dtype=np.int64)
    q = ((vals * 37 + vals // N) % 256).astype(np.uint8).view(np.int8).reshape(K, N)
    packed = np.ascontiguousarray(q).view(np.uint32).reshape(K, N // 4)
    b_d, s_d = dev.tensor(packed), dev.tensor(np.ones(N, np.float32))
    h = C.c_void_p()
    _lib.call("wgpt_int8_weight_create", dev.handle, K, N, b_d.ptr, s_d.ptr, C.byref(h))
    for M, k0 in ((1, 0), (1, K - 1), (3, 5), (4, K - 4), (16, 0)):
        A = np.eye(K, dtype=np.float32)[k0:k0 + M]
        out, a_d = dev.buffer(M * N * 4), dev.tensor(A)
        _lib.call("wgpt_int8_matmul_w", dev.handle, M, h, a_d.ptr, out.ptr)
        assert np.array_equal(out.read(np.float32, M * N).reshape(M, N), q[k0:k0 + M].astype(np.float32))
    _lib.call("wgpt_int8_weight_destroy", h)


def test_pass_list_graph_replay(dev, ops, oracle):
    """A recorded pass list (wgpt_graph_*) replays to the same bits as eager execution, also after the inputs
    change in place (the recording holds addresses, not values)."""
    import ctypes as C
    from webgpt_b200 import _lib
    rng = np.random.default_rng(9)
    M, K, N = 4, 384, 768
    A = rng.standard_normal((M, K), dtype=np.float32)
    W = (rng.standard_normal((K, N), dtype=np.float32) * 0.05).astype(np.float32)
    b = rng.standard_normal(N, dtype=np.float32)
    a_d, w_d, b_d, y_d, z_d = dev.tensor(A), dev.tensor(W), dev.tensor(b), dev.buffer(M * N * 4), dev.buffer(M * N * 4)

    def passes():
        _lib.call("wgpt_matmul", dev.handle, M, N, K, a_d.ptr, w_d.ptr, b_d.ptr, y_d.ptr)
        _lib.call("wgpt_gelu", dev.handle, M, N, y_d.ptr, z_d.ptr)

    passes()
    eager = z_d.read(np.float32, M * N)
    _lib.call("wgpt_graph_begin", dev.handle)
    passes()
    g = C.c_void_p()
    _lib.call("wgpt_graph_end", dev.handle, C.byref(g))
    z_d.write(np.zeros(M * N, np.float32))
    _lib.call("wgpt_graph_launch", dev.handle, g)
    assert np.array_equal(z_d.read(np.float32, M * N), eager)
    A2 = (A * 0.5).astype(np.float32)
    a_d.write(A2)
    _lib.call("wgpt_graph_launch", dev.handle, g)
    ref = oracle.gelu(oracle.matmul(A2, W, b))
    assert rel_err(z_d.read(np.float32, M * N).reshape(M, N), ref) < TOL
    _lib.call("wgpt_graph_destroy", dev.handle, g)
    with pytest.raises(_lib.WgptError) as e:
        _lib.call("wgpt_graph_end", dev.handle, C.byref(g))
    assert e.value.code == _lib.ERR_STATE


def test_pass_list_records_embed_layernorm_matmul(oracle):
    """The reference's pass list starts with the embedding pass (model.js:118); recording embed -> layernorm ->
    matmul must succeed (the embed call only enqueues while recording) and replay to the eager result. Calls that
    would synchronise the stream are refused while recording."""
    import ctypes as C
    from webgpt_b200 import Device, WgptError, _lib
    dev = Device(0)
    try:
        rng = np.random.default_rng(10)
        T, E, V, N = 6, 64, 40, 128
        wte = rng.standard_normal((V, E), dtype=np.float32)
        wpe = rng.standard_normal((T, E), dtype=np.float32)
        g, b = rng.standard_normal(E, dtype=np.float32), rng.standard_normal(E, dtype=np.float32)
        W = (rng.standard_normal((E, N), dtype=np.float32) * 0.1).astype(np.float32)
        ids = rng.integers(0, V, size=T, dtype=np.uint32)
        t = dev.tensor
        ids_d, wte_d, wpe_d, g_d, b_d, w_d = t(ids), t(wte), t(wpe), t(g), t(b), t(W)
        x_d, h_d, y_d = dev.buffer(T * E * 4), dev.buffer(T * E * 4), dev.buffer(T * N * 4)

        def passes():
            _lib.call("wgpt_embed", dev.handle, ids_d.ptr, T, E, V, wte_d.ptr, wpe_d.ptr, x_d.ptr)
            _lib.call("wgpt_layernorm", dev.handle, T, E, x_d.ptr, g_d.ptr, b_d.ptr, h_d.ptr)
            _lib.call("wgpt_matmul", dev.handle, T, N, E, h_d.ptr, w_d.ptr, None, y_d.ptr)

        passes()
        eager = y_d.read(np.float32, T * N)
        ref = oracle.matmul(oracle.layernorm(oracle.embed(ids, wte, wpe), g, b), W)
        assert rel_err(eager.reshape(T, N), ref) < TOL
        _lib.call("wgpt_graph_begin", dev.handle)
        passes()
        for name, args in (("wgpt_device_synchronize", (dev.handle,)), ("wgpt_device_check", (dev.handle,)),
                           ("wgpt_buffer_read", (dev.handle, y_d.ptr, 0, eager.ctypes.data, 4)),
                           ("wgpt_buffer_write", (dev.handle, y_d.ptr, 0, eager.ctypes.data, 4))):
            with pytest.raises(WgptError) as e:
                _lib.call(name, *args)
            assert e.value.code == _lib.ERR_STATE
        graph = C.c_void_p()
        _lib.call("wgpt_graph_end", dev.handle, C.byref(graph))
        y_d.write(np.zeros(T * N, np.float32))
        _lib.call("wgpt_graph_launch", dev.handle, graph)
        _lib.call("wgpt_device_check", dev.handle)
        assert np.array_equal(y_d.read(np.float32, T * N), eager)
        _lib.call("wgpt_graph_destroy", dev.handle, graph)
    finally:
        dev.destroy()


def test_stale_pass_list_is_refused_after_workspace_growth():
    """A recorded pass list holds the address of the library's workspace (split-K partial sums). If a later call
    makes the workspace grow, the old block is freed; launching the old recording is refused with WGPT_ERR_STATE
    instead of touching freed memory (the stale recording never runs)."""
    import ctypes as C
    from webgpt_b200 import Device, WgptError, _lib
    dev = Device(0)
    try:
        rng = np.random.default_rng(11)
        A = rng.standard_normal((2, 256), dtype=np.float32)
        W = rng.standard_normal((256, 128), dtype=np.float32)
        a_d, w_d, y_d = dev.tensor(A), dev.tensor(W), dev.buffer(2 * 128 * 4)
        _lib.call("wgpt_matmul", dev.handle, 2, 128, 256, a_d.ptr, w_d.ptr, None, y_d.ptr)   # sizes the workspace
        _lib.call("wgpt_graph_begin", dev.handle)
        _lib.call("wgpt_matmul", dev.handle, 2, 128, 256, a_d.ptr, w_d.ptr, None, y_d.ptr)
        graph = C.c_void_p()
        _lib.call("wgpt_graph_end", dev.handle, C.byref(graph))
        _lib.call("wgpt_graph_launch", dev.handle, graph)                                    # fine: nothing moved
        big_a, big_w = dev.tensor(np.zeros((8, 4096), np.float32)), dev.tensor(np.zeros((4096, 4096), np.float32))
        big_y = dev.buffer(8 * 4096 * 4)
        _lib.call("wgpt_matmul", dev.handle, 8, 4096, 4096, big_a.ptr, big_w.ptr, None, big_y.ptr)  # workspace grows
        with pytest.raises(WgptError) as e:
            _lib.call("wgpt_graph_launch", dev.handle, graph)
        assert e.value.code == _lib.ERR_STATE and "recorded again" in e.value.message
        _lib.call("wgpt_graph_destroy", dev.handle, graph)
    finally:
        dev.destroy()


def test_matmul_long_shared_dimension_eight_rows(dev, ops, oracle):
    """8 rows with a shared dimension too long for one CTA's staging buffer: the K split grows until a slice fits."""
    rng = np.random.default_rng(12)
    M, K, N = 8, 16384, 256
    A = rng.standard_normal((M, K), dtype=np.float32)
    B = (rng.standard_normal((K, N), dtype=np.float32) * 0.02).astype(np.float32)
    out = run(ops.FastMatMulBlock.newInstance(M, N, K, dev.tensor(A), dev.tensor(B), dev.tensor(np.zeros(N, np.float32))))
    assert rel_err(out.read(np.float32, M * N).reshape(M, N), oracle.matmul(A, B)) < TOL


@pytest.mark.parametrize("per_column", [True, False])
@pytest.mark.parametrize("K,N", [(24, 16), (768, 3072), (1600, 6400), (100, 8)])
def test_int8_quantize_bit_exact(dev, oracle, K, N, per_column):
    """wgpt_int8_quantize against the oracle's quantiser: identical words and scales (JS double arithmetic,
    Math.round halves toward +infinity, & 0xff, 4 per word along N, other/int8-gemm.js:25-62), including a zero
    column and values that sit exactly on a rounding half; the result feeds wgpt_int8_matmul."""
    from webgpt_b200 import _lib
    rng = np.random.default_rng(K + N)
    w = (rng.standard_normal((K, N)) * 0.05).astype(np.float32)
    w[:, 3] = 0.0
    w[1, 2] = np.float32(2.5) * np.abs(w[:, 2]).max() / np.float32(127)
    w[2, 2] = -w[1, 2]
    ref_q, ref_s = oracle.int8_quantize_matrix(w, per_column=per_column)
    w_d, q_d, s_d = dev.tensor(w), dev.buffer(K * N), dev.buffer(N * 4)
    _lib.call("wgpt_int8_quantize", dev.handle, K, N, int(per_column), w_d.ptr, q_d.ptr, s_d.ptr)
    assert np.array_equal(q_d.read(np.int32, K * N // 4).reshape(K, N // 4), ref_q)
    assert np.array_equal(s_d.read(np.float32, N), ref_s)
    if N % 8 == 0 and K % 4 == 0:
        A = rng.standard_normal((2, K), dtype=np.float32)
        a_d, o_d = dev.tensor(A), dev.buffer(2 * N * 4)
        _lib.call("wgpt_int8_matmul", dev.handle, 2, K, N, a_d.ptr, q_d.ptr, s_d.ptr, o_d.ptr)
        got = o_d.read(np.float32, 2 * N).reshape(2, N)
        assert rel_err(got, oracle.int8_matmul(A, ref_q, ref_s, N)) < TOL
        assert np.max(np.abs(got - A @ w)) < 0.1     # the prototype's acceptance rule, other/int8-gemm.js:321


def test_bounded_wait_expiry_reports_timeout_and_device_survives(oracle):
    """A bounded device-side wait driven to its limit: the probe kernel's mbarrier is armed for more bytes than its
    first copy delivers, so the wait gives up after a handful of polls, the kernel flags the error word, drains
    with a second bounded wait and returns. wgpt_device_check then reports WGPT_ERR_TIMEOUT exactly once, and the
    same device computes a correct product afterwards."""
    import ctypes as C
    from webgpt_b200 import Device, WgptError, _lib
    dev = Device(0)
    try:
        first, drain = C.c_int32(-1), C.c_int32(-1)
        _lib.call("wgpt_device_probe_wait_expiry", dev.handle, 4, C.byref(first), C.byref(drain))
        assert first.value == 0      # the wait ran out
        assert drain.value == 1      # the drain wait completed: no copy was left in flight
        with pytest.raises(WgptError) as e:
            _lib.call("wgpt_device_check", dev.handle)
        assert e.value.code == _lib.ERR_TIMEOUT and "did not complete in time" in e.value.message
        _lib.call("wgpt_device_check", dev.handle)   # reported once, then clear
        rng = np.random.default_rng(13)
        A = rng.standard_normal((1, 768), dtype=np.float32)
        W = (rng.standard_normal((768, 768), dtype=np.float32) * 0.05).astype(np.float32)
        a_d, w_d, y_d = dev.tensor(A), dev.tensor(np.ascontiguousarray(W.T)), dev.buffer(768 * 4)
        _lib.call("wgpt_matmul_nk", dev.handle, 1, 768, 768, a_d.ptr, w_d.ptr, None, y_d.ptr)   # bulk-copy GEMV
        _lib.call("wgpt_device_check", dev.handle)
        assert rel_err(y_d.read(np.float32, 768).reshape(1, 768), oracle.matmul(A, W)) < TOL
    finally:
        dev.destroy()
