"""class Visuals with the surface of the reference's visuals.js, headless.

The reference draws the residual stream of the last forward pass (the model's externalBuffer tap,
model.js:211-222) onto a canvas with a fragment shader (visuals.js:81-137). There is no canvas or swap chain
here: render() runs the same per-pixel arithmetic as a CUDA kernel into a device buffer and returns the image
as an [n_ctx, n_embd, 4] uint8 array (RGBA), optionally also writing it as a binary PPM file.
"""
import numpy as np

from . import _lib


class Visuals:
    def __init__(self, model):
        self.model = model
        self.device = model.device
        self.params = model.params
        self.initialized = False

    def init(self):
        """visuals.js:11-19: allocate the embeddings buffer and hook it up as the model's externalBuffer."""
        n = self.params["n_ctx"] * self.params["n_embd"]
        self.embeddingsBuffer = self.device.buffer(n * 4, [self.params["n_ctx"], self.params["n_embd"]])
        self.embeddingsBuffer.write(np.zeros(n, np.float32))
        self.imageBuffer = self.device.buffer(n * 4)
        self.updateModelBuffer()
        self.initialized = True

    def updateModelBuffer(self):
        """visuals.js:48-50."""
        self.model.externalBuffer = self.embeddingsBuffer

    def render(self, ppm_path=None):
        """visuals.js:213-236. Rows beyond the last window's length keep what an earlier, longer window left
        there, as the reference's buffer does."""
        p = self.params
        _lib.call("wgpt_visuals_render", self.device.handle, self.embeddingsBuffer.ptr, p["n_ctx"], p["n_embd"],
                  self.imageBuffer.ptr)
        img = self.imageBuffer.read(np.uint8).reshape(p["n_ctx"], p["n_embd"], 4)
        if ppm_path:
            with open(ppm_path, "wb") as f:
                f.write(b"P6\n%d %d\n255\n" % (p["n_embd"], p["n_ctx"]))
                f.write(np.ascontiguousarray(img[:, :, :3]).tobytes())
        return img

    def destroy(self):
        """visuals.js:238-242."""
        self.model.externalBuffer = None
        self.embeddingsBuffer.destroy()
        self.imageBuffer.destroy()
        self.initialized = False
