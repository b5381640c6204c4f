"""wgpt_matmul_static: the matmul entry point for callers that must not allocate on the device (servers that
own all of HBM through their own arena, latency-critical loops, hosts that forbid driver allocations while
serving). Its split-K scratch is a fixed array inside the library, shared by every call, so the checks here
are: same answer as wgpt_matmul, also on a second call that finds the first call's leftovers in the array,
a clear refusal beyond the array's size, and that free device memory does not move across a call (after one
warm-up call per GPU, which is when the CUDA runtime loads the library's device code). Collected last on
purpose."""
import numpy as np
import pytest

from conftest import rel_err

pytestmark = pytest.mark.gpu

TOL = 2e-5  # same relative bound as the other FP32 matmul tests


def test_static_scratch_matmul_matches_allocating_entry_point():
    from webgpt_b200 import Device, WgptError, _lib
    dev = Device(0)
    try:
        rng = np.random.default_rng(77)
        # two calls in a row with different shapes: the second one reuses an array full of the first one's sums
        for rows, K, N in [(8, 3072, 768), (1, 768, 2304), (3, 1600, 6400), (1, 768, 2304)]:
            A = rng.standard_normal((rows, K), dtype=np.float32)
            W = (rng.standard_normal((K, N), dtype=np.float32) * 0.05).astype(np.float32)
            b = rng.standard_normal(N, dtype=np.float32)
            a_d, w_d, b_d = dev.tensor(A), dev.tensor(W), dev.tensor(b)
            ref_d, got_d = dev.buffer(rows * N * 4), dev.buffer(rows * N * 4)
            _lib.call("wgpt_matmul", dev.handle, rows, N, K, a_d.ptr, w_d.ptr, b_d.ptr, ref_d.ptr)
            ref = ref_d.read(np.float32, rows * N)
            for _ in range(2):
                got_d.write(np.zeros(rows * N, np.float32))
                _lib.call("wgpt_matmul_static", dev.handle, rows, N, K, a_d.ptr, w_d.ptr, b_d.ptr, got_d.ptr)
                got = got_d.read(np.float32, rows * N)
                assert rel_err(got, ref) < TOL
            assert rel_err(got.reshape(rows, N), A.astype(np.float64) @ W.astype(np.float64) + b) < TOL
        # beyond the limits: more than 8 rows, or rows*cols larger than the built-in array
        with pytest.raises(WgptError) as e:
            _lib.call("wgpt_matmul_static", dev.handle, 9, N, K, a_d.ptr, w_d.ptr, b_d.ptr, got_d.ptr)
        assert e.value.code == _lib.ERR_SHAPE and "at most 8 rows" in e.value.message
        big_n = 2097152 + 8
        with pytest.raises(WgptError) as e:
            _lib.call("wgpt_matmul_static", dev.handle, 1, big_n, 4, a_d.ptr, w_d.ptr, None, got_d.ptr)
        assert e.value.code == _lib.ERR_SHAPE and "exceeds the built-in scratch" in e.value.message
    finally:
        dev.destroy()


def test_static_scratch_matmul_allocates_nothing():
    """After one warm-up call the driver's free-memory figure is the same before and after wgpt_matmul_static,
    on a shape whose split-K partial sums exceed the workspace a fresh device holds (none); the allocating entry
    point wgpt_matmul moves that figure on the same shape."""
    from webgpt_b200 import Device, _lib
    dev = Device(0)
    try:
        rng = np.random.default_rng(78)
        rows, K, N = 8, 4096, 4096   # split-K partials: a few MiB
        A = rng.standard_normal((rows, K), dtype=np.float32)
        W = (rng.standard_normal((K, N), dtype=np.float32) * 0.05).astype(np.float32)
        a_d, w_d = dev.tensor(A), dev.tensor(W)
        out_d = dev.buffer(rows * N * 4)
        _lib.call("wgpt_matmul_static", dev.handle, 1, 64, 64, a_d.ptr, w_d.ptr, None, out_d.ptr)  # warm-up
        dev.synchronize()
        free0, _ = dev.mem_info()
        for _ in range(3):
            _lib.call("wgpt_matmul_static", dev.handle, rows, N, K, a_d.ptr, w_d.ptr, None, out_d.ptr)
        dev.synchronize()
        free1, _ = dev.mem_info()
        assert free1 == free0
        got = out_d.read(np.float32, rows * N).reshape(rows, N)
        assert rel_err(got, A.astype(np.float64) @ W.astype(np.float64)) < TOL
        _lib.call("wgpt_matmul", dev.handle, rows, N, K, a_d.ptr, w_d.ptr, None, out_d.ptr)  # grows the workspace
        dev.synchronize()
        free2, _ = dev.mem_info()
        assert free2 < free1
    finally:
        dev.destroy()
