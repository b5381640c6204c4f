"""Device and buffer objects over the C ABI (the counterpart of GPUDevice / GPUBuffer in the reference)."""
import ctypes as C

import numpy as np

from . import _lib


class Buffer:
    """A device allocation. `ptr` is the device address handed to the C ABI."""

    def __init__(self, device, nbytes, dims=None):
        self.device = device
        self.nbytes = int(nbytes)
        self.dims = tuple(dims) if dims is not None else None
        p = C.c_void_p()
        _lib.call("wgpt_buffer_create", device.handle, self.nbytes, C.byref(p))
        self.ptr = p.value
        self.destroyed = False

    def write(self, array, offset=0):
        a = np.ascontiguousarray(array)
        if offset + a.nbytes > self.nbytes:
            raise ValueError("write exceeds the buffer")
        _lib.call("wgpt_buffer_write", self.device.handle, self.ptr, offset, a.ctypes.data, a.nbytes)
        return self

    def read(self, dtype=np.float32, count=None, offset=0):
        n = (self.nbytes - offset) // np.dtype(dtype).itemsize if count is None else count
        out = np.empty(n, dtype)
        _lib.call("wgpt_buffer_read", self.device.handle, self.ptr, offset, out.ctypes.data, out.nbytes)
        return out

    def destroy(self):
        if not self.destroyed:
            self.destroyed = True
            _lib.call("wgpt_buffer_destroy", self.device.handle, self.ptr)

    def __del__(self):
        try:
            if not self.destroyed and self.device.handle:
                self.destroy()
        except Exception:
            pass


class Device:
    """One B200 and its stream (model.js:27-28 requestAdapter/requestDevice)."""

    def __init__(self, ordinal=0):
        self.handle = None
        h = C.c_void_p()
        _lib.call("wgpt_device_create", ordinal, C.byref(h))
        self.handle = h
        self.ordinal = ordinal

    def buffer(self, nbytes, dims=None):
        return Buffer(self, nbytes, dims)

    def tensor(self, array):
        a = np.ascontiguousarray(array)
        return Buffer(self, a.nbytes, a.shape).write(a)

    def synchronize(self):
        _lib.call("wgpt_device_synchronize", self.handle)

    def copy(self, src, src_offset, dst, dst_offset, size):
        _lib.call("wgpt_buffer_copy", self.handle, src.ptr, src_offset, dst.ptr, dst_offset, size)

    def set_precision(self, mode):
        _lib.call("wgpt_device_set_precision", self.handle, mode)

    def launch_count(self):
        n = C.c_uint64()
        _lib.call("wgpt_device_launch_count", self.handle, C.byref(n))
        return n.value

    def mem_info(self):
        """(free, total) device memory in bytes as the driver reports them."""
        f, t = C.c_uint64(), C.c_uint64()
        _lib.call("wgpt_device_mem_info", self.handle, C.byref(f), C.byref(t))
        return f.value, t.value

    def event(self):
        e = C.c_void_p()
        _lib.call("wgpt_event_create", self.handle, C.byref(e))
        return e

    def record(self, event):
        _lib.call("wgpt_event_record", self.handle, event)

    def elapsed_ms(self, start, stop):
        ms = C.c_float()
        _lib.call("wgpt_event_elapsed_ms", self.handle, start, stop, C.byref(ms))
        return ms.value

    def destroy(self):
        if self.handle:
            h, self.handle = self.handle, None
            _lib.call("wgpt_device_destroy", h)
