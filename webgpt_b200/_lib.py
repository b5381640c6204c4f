"""ctypes binding of libwebgpt_b200.so — the only route from Python to the kernels.

There is no fallback: if the shared library is missing or no B200 is present, loading or the first device
call raises.
"""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libwebgpt_b200.so")

OK = 0
ERR_SHAPE, ERR_ALIGN, ERR_OOM, ERR_CUDA, ERR_TIMEOUT, ERR_STATE, ERR_UNSUPPORTED, ERR_ARG = -1, -2, -3, -4, -5, -6, -7, -8
PRECISION_FP32, PRECISION_TF32X3, PRECISION_TF32 = 0, 1, 2

MAX_TOP_K = 128  # WGPT_MAX_TOP_K
_ERR_NAMES = {ERR_SHAPE: "WGPT_ERR_SHAPE", ERR_ALIGN: "WGPT_ERR_ALIGN", ERR_OOM: "WGPT_ERR_OOM",
              ERR_CUDA: "WGPT_ERR_CUDA", ERR_TIMEOUT: "WGPT_ERR_TIMEOUT", ERR_STATE: "WGPT_ERR_STATE",
              ERR_UNSUPPORTED: "WGPT_ERR_UNSUPPORTED", ERR_ARG: "WGPT_ERR_ARG"}


class WgptError(RuntimeError):
    """Raised for any non-zero status; mirrors the reference's `throw new Error(message)`."""

    def __init__(self, code, message):
        super().__init__(f"{_ERR_NAMES.get(code, code)}: {message}")
        self.code = code
        self.message = message


class Params(C.Structure):
    _fields_ = [(k, C.c_int32) for k in ("n_layer", "n_head", "n_embd", "n_ctx", "vocab_size", "bias")]


vp, vpp = C.c_void_p, C.POINTER(C.c_void_p)
i32, u64, f32 = C.c_int32, C.c_uint64, C.c_float

# name -> argument types; every function returns int32 status unless listed in _SPECIAL
SIGNATURES = {
    "wgpt_device_create": [i32, vpp],
    "wgpt_device_destroy": [vp],
    "wgpt_device_synchronize": [vp],
    "wgpt_device_set_precision": [vp, i32],
    "wgpt_device_launch_count": [vp, C.POINTER(u64)],
    "wgpt_device_mem_info": [vp, C.POINTER(u64), C.POINTER(u64)],
    "wgpt_buffer_create": [vp, u64, vpp],
    "wgpt_buffer_destroy": [vp, vp],
    "wgpt_buffer_write": [vp, vp, u64, vp, u64],
    "wgpt_buffer_read": [vp, vp, u64, vp, u64],
    "wgpt_buffer_copy": [vp, vp, u64, vp, u64, u64],
    "wgpt_host_alloc": [u64, vpp],
    "wgpt_host_free": [vp],
    "wgpt_event_create": [vp, vpp],
    "wgpt_event_record": [vp, vp],
    "wgpt_event_elapsed_ms": [vp, vp, vp, C.POINTER(f32)],
    "wgpt_event_destroy": [vp, vp],
    "wgpt_graph_begin": [vp],
    "wgpt_graph_end": [vp, vpp],
    "wgpt_graph_launch": [vp, vp],
    "wgpt_graph_destroy": [vp, vp],
    "wgpt_matmul": [vp, i32, i32, i32, vp, vp, vp, vp],
    "wgpt_matmul_nk": [vp, i32, i32, i32, vp, vp, vp, vp],
    "wgpt_device_check": [vp],
    "wgpt_device_probe_wait_expiry": [vp, C.c_uint32, C.POINTER(i32), C.POINTER(i32)],
    "wgpt_matmul_static": [vp, i32, i32, i32, vp, vp, vp, vp],
    "wgpt_residual": [vp, i32, i32, vp, vp, vp],
    "wgpt_layernorm": [vp, i32, i32, vp, vp, vp, vp],
    "wgpt_softmax": [vp, i32, i32, vp, vp],
    "wgpt_gelu": [vp, i32, i32, vp, vp],
    "wgpt_embed": [vp, vp, i32, i32, i32, vp, vp, vp],
    "wgpt_deembed": [vp, i32, i32, i32, vp, vp, vp],
    "wgpt_attention": [vp, i32, i32, f32, i32, i32] + [vp] * 10,
    "wgpt_int8_matmul": [vp, i32, i32, i32, vp, vp, vp, vp],
    "wgpt_int8_quantize": [vp, i32, i32, i32, vp, vp, vp],
    "wgpt_int8_weight_create": [vp, i32, i32, vp, vp, vpp],
    "wgpt_int8_weight_destroy": [vp],
    "wgpt_int8_matmul_w": [vp, i32, vp, vp, vp],
    "wgpt_model_create": [vp, C.POINTER(Params), vpp],
    "wgpt_model_set_tensor": [vp, C.c_char_p, vp, u64],
    "wgpt_model_finalize": [vp],
    "wgpt_model_destroy": [vp],
    "wgpt_session_create": [vp, i32, vpp],
    "wgpt_session_destroy": [vp],
    "wgpt_session_reset": [vp],
    "wgpt_session_length": [vp, C.POINTER(i32)],
    "wgpt_session_forward": [vp, vp, i32, vp],
    "wgpt_model_run": [vp, vp, i32, vp],
    "wgpt_generate_greedy": [vp, vp, i32, i32, vp],
    "wgpt_generate_greedy_sharded": [vpp, i32, vp, i32, i32, vp],
    "wgpt_session_set_prompts": [vp, vp, i32],
    "wgpt_session_generate": [vp, i32],
    "wgpt_session_get_new_ids": [vp, i32, vp],
    "wgpt_generate_sample": [vp, vp, i32, i32, i32, C.c_double, vp, vp],
    "wgpt_session_generate_sample": [vp, i32, i32, C.c_double, vp],
    "wgpt_sample_topk": [vp, vp, i32, i32, i32, C.c_double, vp, vp],
    "wgpt_visuals_render": [vp, vp, i32, i32, vp],
    "wgpt_session_tap": [vp, vp, u64, C.POINTER(u64)],
}
_SPECIAL = {"wgpt_abi_version": (i32, []), "wgpt_last_error": (C.c_char_p, [])}

_lib = None


def load():
    """Loads the shared library (no device call is made)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: run `python -m webgpt_b200.build` (needs nvcc)")
        lib = C.CDLL(LIB_PATH)
        for name, args in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = i32
            fn.argtypes = args
        for name, (res, args) in _SPECIAL.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def check(rc):
    if rc != OK:
        raise WgptError(rc, load().wgpt_last_error().decode("utf-8", "replace"))


def call(name, *args):
    check(getattr(load(), name)(*args))
