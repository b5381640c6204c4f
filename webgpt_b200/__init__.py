"""webgpt_b200: the GPT-2 forward hot path of 0hq/WebGPT on B200 (sm_100a) behind a C ABI.

`GPT` mirrors the reference's model.js class, `globals`/`instructions` mirror its operator singletons and
instruction classes; all compute happens in libwebgpt_b200.so (CUDA). Importing the package does not touch
the GPU; creating a Device does, and raises if the library or a B200 is missing.
"""
from . import synth  # noqa: F401
from ._lib import WgptError  # noqa: F401

__all__ = ["synth", "WgptError", "GPT", "Device"]


def __getattr__(name):
    if name == "GPT":
        from .model import GPT
        return GPT
    if name == "Device":
        from .device import Device
        return Device
    raise AttributeError(name)
