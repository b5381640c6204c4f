"""ctypes binding of the CPU oracle (liboracle.so built from oracle.c).

Test infrastructure only: imported by tests/, by the smoke check and by the CPU-baseline
leg of the benchmark. The product package never imports this module.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

f32p = C.POINTER(C.c_float)
u32p = C.POINTER(C.c_uint32)
i32p = C.POINTER(C.c_int32)


def build(force=False):
    so = os.path.join(_HERE, "liboracle.so")
    src = os.path.join(_HERE, "oracle.c")
    if force or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-s", "-B", "liboracle.so"], check=True, stdout=subprocess.DEVNULL,
                       stderr=subprocess.DEVNULL)
    return so


def usable_cores():
    """Cores this process may really use: the affinity mask, further limited by a cgroup CPU quota."""
    n = len(os.sched_getaffinity(0))
    try:
        quota, period = open("/sys/fs/cgroup/cpu.max").read().split()
        if quota != "max":
            n = min(n, max(1, int(float(quota) / float(period))))
    except Exception:
        pass
    return max(1, min(n, 64))


def lib():
    global _LIB
    if _LIB is None:
        # idle OpenMP workers must sleep, not spin: the team may be larger than the CPU share
        os.environ.setdefault("OMP_WAIT_POLICY", "passive")
        _LIB = C.CDLL(build())
        L = _LIB
        L.orc_set_threads(usable_cores())
        L.orc_gelu1.restype = C.c_float
        L.orc_gelu1.argtypes = [C.c_float]
        L.orc_model_create.restype = C.c_void_p
        L.orc_model_create.argtypes = [C.c_int] * 5 + [C.POINTER(f32p)]
        L.orc_model_destroy.argtypes = [C.c_void_p]
        L.orc_model_num_taps.argtypes = [C.c_void_p]
        L.orc_model_run.argtypes = [C.c_void_p, u32p, C.c_int, f32p, f32p]
        L.orc_generate_greedy.argtypes = [C.c_void_p, u32p, C.c_int, C.c_int, u32p, f32p]
        L.orc_argmax.restype = C.c_uint32
        L.orc_argmax.argtypes = [f32p, C.c_int]
        L.orc_kv_create.restype = C.c_void_p
        L.orc_kv_create.argtypes = [C.c_void_p]
        L.orc_kv_destroy.argtypes = [C.c_void_p]
        L.orc_kv_reset.argtypes = [C.c_void_p]
        L.orc_kv_step.argtypes = [C.c_void_p, C.c_uint32, f32p]
        L.orc_kv_generate_greedy.argtypes = [C.c_void_p, u32p, C.c_int, C.c_int, u32p]
        f64p = C.POINTER(C.c_double)
        L.orc_sample_topk.restype = C.c_uint32
        L.orc_sample_topk.argtypes = [f32p, C.c_int, C.c_int, C.c_double, C.c_double, u32p]
        L.orc_kv_generate_sample.argtypes = [C.c_void_p, u32p, C.c_int, C.c_int, C.c_int, C.c_double, f64p, u32p]
        L.orc_generate_sample.argtypes = [C.c_void_p, u32p, C.c_int, C.c_int, C.c_int, C.c_double, f64p, u32p]
        L.orc_int8_quantize.argtypes = [f32p, C.c_size_t, C.c_double, i32p]
        L.orc_int8_unpack.argtypes = [i32p, C.c_size_t, C.POINTER(C.c_int8)]
        L.orc_int8_quantize_matrix.argtypes = [f32p, C.c_int, C.c_int, C.c_int, i32p, f32p]
    return _LIB


def _f(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a, a.ctypes.data_as(f32p)


def _u(a):
    a = np.ascontiguousarray(a, dtype=np.uint32)
    return a, a.ctypes.data_as(u32p)


def matmul(A, B, bias=None):
    A, pa = _f(A)
    B, pb = _f(B)
    M, K = A.shape
    N = B.shape[1]
    out = np.empty((M, N), np.float32)
    pbias = None
    if bias is not None:
        bias, pbias = _f(bias)
    lib().orc_matmul(pa, pb, pbias, out.ctypes.data_as(f32p), M, K, N)
    return out


def residual(a, b):
    a, pa = _f(a)
    b, pb = _f(b)
    out = np.empty_like(a)
    lib().orc_residual(pa, pb, out.ctypes.data_as(f32p), a.shape[0], a.shape[1])
    return out


def layernorm(x, gamma, beta, return_stats=False):
    x, px = _f(x)
    gamma, pg = _f(gamma)
    beta, pb = _f(beta)
    out = np.empty_like(x)
    stats = np.empty((x.shape[0], 2), np.float32)
    lib().orc_layernorm(px, pg, pb, out.ctypes.data_as(f32p), stats.ctypes.data_as(f32p), x.shape[0], x.shape[1])
    return (out, stats) if return_stats else out


def softmax(x):
    x, px = _f(x)
    out = np.empty_like(x)
    lib().orc_softmax(px, out.ctypes.data_as(f32p), x.shape[0], x.shape[1])
    return out


def gelu(x):
    x, px = _f(x)
    out = np.empty_like(x)
    x2 = x.reshape(-1, x.shape[-1])
    lib().orc_gelu(px, out.ctypes.data_as(f32p), x2.shape[0], x2.shape[1])
    return out


def embed(idx, wte, wpe):
    idx, pi = _u(idx)
    wte, pw = _f(wte)
    wpe, pp = _f(wpe)
    E = wte.shape[1]
    out = np.empty((len(idx), E), np.float32)
    lib().orc_embed(pi, len(idx), E, pw, pp, out.ctypes.data_as(f32p))
    return out


def deembed(x_last, wte):
    x_last, px = _f(x_last)
    wte, pw = _f(wte)
    V, E = wte.shape
    out = np.empty(V, np.float32)
    lib().orc_deembed(px, E, V, pw, out.ctypes.data_as(f32p))
    return out


def format_q(Q, hs):
    Q, pq = _f(Q)
    T, E = Q.shape
    out = np.empty((E // hs * T, hs), np.float32)
    lib().orc_format_q(pq, out.ctypes.data_as(f32p), T, E, hs)
    return out


def attn_weights(Qf, Kmat, H, scale):
    Qf, pq = _f(Qf)
    Kmat, pk = _f(Kmat)
    T, E = Kmat.shape
    out = np.empty((H * T, T), np.float32)
    lib().orc_attn_weights(pq, pk, out.ctypes.data_as(f32p), T, E, H, C.c_float(scale))
    return out


def attn_values(P, V, H):
    P, pp = _f(P)
    V, pv = _f(V)
    T, E = V.shape
    out = np.empty((T, E), np.float32)
    lib().orc_attn_values(pp, pv, out.ctypes.data_as(f32p), T, E, H)
    return out


def attention(x, H, scale, wq, bq, wk, bk, wv, bv, wo, bo):
    arrs = [_f(a) for a in (x, wq, bq, wk, bk, wv, bv, wo, bo)]
    T, E = arrs[0][0].shape
    out = np.empty((T, E), np.float32)
    p = [a[1] for a in arrs]
    lib().orc_attention(p[0], T, E, H, C.c_float(scale), *p[1:], out.ctypes.data_as(f32p))
    return out


def int8_quantize(x, absmax):
    x, px = _f(x)
    out = np.empty(x.size // 4, np.int32)
    lib().orc_int8_quantize(px, x.size, float(absmax), out.ctypes.data_as(i32p))
    return out


def int8_quantize_matrix(w, per_column=True):
    """Returns (packed [K, N/4] int32, scale [N] f32) for a row-major [K, N] matrix."""
    w, pw = _f(w)
    K, N = w.shape
    packed = np.empty((K, N // 4), np.int32)
    scale = np.empty(N, np.float32)
    lib().orc_int8_quantize_matrix(pw, K, N, int(per_column), packed.ctypes.data_as(i32p), scale.ctypes.data_as(f32p))
    return packed, scale


def int8_unpack(packed):
    packed = np.ascontiguousarray(packed, dtype=np.int32)
    out = np.empty(packed.size * 4, np.int8)
    lib().orc_int8_unpack(packed.ctypes.data_as(i32p), packed.size, out.ctypes.data_as(C.POINTER(C.c_int8)))
    return out


def int8_matmul(A, Bq, scale, N, literal=False):
    A, pa = _f(A)
    Bq = np.ascontiguousarray(Bq, dtype=np.int32)
    scale, ps = _f(scale)
    M, K = A.shape
    out = np.empty((M, N), np.float32)
    lib().orc_int8_matmul(pa, Bq.ctypes.data_as(i32p), ps, out.ctypes.data_as(f32p), M, K, N, int(literal))
    return out


def sample_topk(logits, top_k, temperature, u, return_top=False):
    """model.js:81-83 with the random number supplied: returns the sampled vocabulary index."""
    logits, pl = _f(logits)
    k = min(int(top_k), logits.size)
    top = np.empty(k, np.uint32)
    idx = lib().orc_sample_topk(pl, logits.size, int(top_k), float(temperature), float(u), top.ctypes.data_as(u32p))
    return (int(idx), top) if return_top else int(idx)


def heatmap(buf):
    buf, pb = _f(buf)
    out = np.empty(buf.shape + (4,), np.uint8)
    lib().orc_heatmap.argtypes = [f32p, C.c_size_t, C.POINTER(C.c_uint8)]
    lib().orc_heatmap(pb, buf.size, out.ctypes.data_as(C.POINTER(C.c_uint8)))
    return out


TENSORS_PER_LAYER = 12


class Model:
    """orc_model over a weight list in the on-disk order (see oracle.c)."""

    def __init__(self, params, tensors):
        self.params = dict(params)
        self._keep = [np.ascontiguousarray(t, dtype=np.float32) for t in tensors]
        n = 4 + TENSORS_PER_LAYER * params["n_layer"]
        assert len(self._keep) == n, (len(self._keep), n)
        arr = (f32p * n)(*[t.ctypes.data_as(f32p) for t in self._keep])
        self._h = lib().orc_model_create(params["n_layer"], params["n_head"], params["n_embd"], params["n_ctx"],
                                         params["vocab_size"], arr)
        if not self._h:
            raise ValueError("orc_model_create rejected the parameters")

    def __del__(self):
        if getattr(self, "_h", None):
            lib().orc_model_destroy(self._h)
            self._h = None

    def run(self, idx, taps=False):
        idx, pi = _u(idx)
        V, E = self.params["vocab_size"], self.params["n_embd"]
        logits = np.empty(V, np.float32)
        tp = None
        tbuf = None
        if taps:
            tbuf = np.empty((lib().orc_model_num_taps(self._h), len(idx), E), np.float32)
            tp = tbuf.ctypes.data_as(f32p)
        rc = lib().orc_model_run(self._h, pi, len(idx), logits.ctypes.data_as(f32p), tp)
        if rc:
            raise ValueError(f"orc_model_run failed: {rc}")
        return (logits, tbuf) if taps else logits

    def generate_greedy(self, prompt, n_new, trace=False):
        prompt, pp = _u(prompt)
        hist = np.empty(len(prompt) + n_new, np.uint32)
        tr = np.empty((n_new, self.params["vocab_size"]), np.float32) if trace else None
        rc = lib().orc_generate_greedy(self._h, pp, len(prompt), n_new, hist.ctypes.data_as(u32p),
                                       tr.ctypes.data_as(f32p) if trace else None)
        if rc:
            raise ValueError(f"orc_generate_greedy failed: {rc}")
        return (hist, tr) if trace else hist

    def kv_generate_greedy(self, prompt, n_new):
        prompt, pp = _u(prompt)
        kv = lib().orc_kv_create(self._h)
        out = np.empty(n_new, np.uint32)
        rc = lib().orc_kv_generate_greedy(kv, pp, len(prompt), n_new, out.ctypes.data_as(u32p))
        lib().orc_kv_destroy(kv)
        if rc:
            raise ValueError(f"orc_kv_generate_greedy failed: {rc}")
        return out

    def kv_generate_sample(self, prompt, n_new, top_k, temperature, uniforms):
        """Top-k sampling through the KV cache; uniforms holds one number in [0,1) per new token."""
        prompt, pp = _u(prompt)
        u = np.ascontiguousarray(uniforms, dtype=np.float64)
        assert len(u) >= n_new
        kv = lib().orc_kv_create(self._h)
        out = np.empty(n_new, np.uint32)
        rc = lib().orc_kv_generate_sample(kv, pp, len(prompt), n_new, top_k, float(temperature),
                                          u.ctypes.data_as(C.POINTER(C.c_double)), out.ctypes.data_as(u32p))
        lib().orc_kv_destroy(kv)
        if rc:
            raise ValueError(f"orc_kv_generate_sample failed: {rc}")
        return out

    def generate_sample(self, prompt, n_new, top_k, temperature, uniforms):
        """Top-k sampling by full-window recompute (the reference's loop); returns prompt + new ids."""
        prompt, pp = _u(prompt)
        u = np.ascontiguousarray(uniforms, dtype=np.float64)
        assert len(u) >= n_new
        hist = np.empty(len(prompt) + n_new, np.uint32)
        rc = lib().orc_generate_sample(self._h, pp, len(prompt), n_new, top_k, float(temperature),
                                       u.ctypes.data_as(C.POINTER(C.c_double)), hist.ctypes.data_as(u32p))
        if rc:
            raise ValueError(f"orc_generate_sample failed: {rc}")
        return hist

    def kv_logits(self, ids):
        """Feeds ids one by one through the KV cache; returns the logits after each."""
        kv = lib().orc_kv_create(self._h)
        V = self.params["vocab_size"]
        out = np.empty((len(ids), V), np.float32)
        for i, t in enumerate(ids):
            rc = lib().orc_kv_step(kv, int(t), out[i].ctypes.data_as(f32p))
            assert rc == 0
        lib().orc_kv_destroy(kv)
        return out


def num_threads():
    return lib().orc_num_threads()
