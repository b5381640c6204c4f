"""Operator ("instruction") classes with the surface of the reference's instructions.js.

Each class keeps the reference's name, its `newInstance(...)` argument order and its return shape
`{"resultBuffer", "passes"}`; a pass is either `{"flag": "compute", "run": callable}` (one call into the C
ABI that enqueues the kernels) or `{"flag": "copy", src, srcOffset, dst, dstOffset, size}`, executed in order
by GPT.run the way model.js:245-257 replays its pass list. Result buffers are cached by shape and recycled
between runs like Block.initResultBuffer / clearBufferCache (instructions.js:57-65,123-130).
Shape violations raise with the reference's messages (they come back from the C ABI as WGPT_ERR_SHAPE).
"""
from . import _lib


class Block:
    """instructions.js:7-139 (bind-group and pipeline plumbing has no counterpart: kernels are precompiled)."""

    def __init__(self):
        self.name = ""
        self.device = None

    def initialize(self, device):
        self.device = device
        self.boundBufferCache = {}
        self.unboundBufferCache = {}

    def bufferSize(self, dimA, dimB=1):
        return int(dimA) * int(dimB) * 4

    def initResultBuffer(self, dims):
        key = "result_" + ",".join(str(d) for d in dims)
        pool = self.unboundBufferCache.get(key)
        if pool:
            buf = pool.pop()
            if not pool:
                del self.unboundBufferCache[key]
            self.boundBufferCache.setdefault(key, []).append(buf)
            return buf
        return self.initBuffer(["storage", "copy_from"], dims, key)

    def initBuffer(self, ops, dims, key=""):
        d = list(dims) + [1, 1]
        buf = self.device.buffer(self.bufferSize(d[0], d[1]) * (d[2] if len(dims) > 2 else 1), dims)
        self.boundBufferCache.setdefault(key, []).append(buf)
        return buf

    def clearBufferCache(self):
        for pool in self.unboundBufferCache.values():
            for b in pool:
                b.destroy()
        self.unboundBufferCache = self.boundBufferCache
        self.boundBufferCache = {}

    def destroyBuffers(self):
        for cache in (self.unboundBufferCache, self.boundBufferCache):
            for pool in cache.values():
                for b in pool:
                    b.destroy()
        self.unboundBufferCache = {}
        self.boundBufferCache = {}

    def destroy(self):
        self.destroyBuffers()

    def _compute(self, fn, *args):
        """A compute pass. Buffer arguments are held by the pass (as a bind group holds its buffers in the
        reference) and resolved to device addresses when the pass runs."""
        dev = self.device

        def run():
            _lib.call(fn, dev.handle, *[a.ptr if hasattr(a, "ptr") else a for a in args])

        return {"flag": "compute", "run": run, "buffers": [a for a in args if hasattr(a, "ptr")]}


class FastMatMulBlockClass(Block):
    def __init__(self):
        super().__init__()
        self.name = "fastMatMul"

    def newInstance(self, rows, cols, shared, inputBuffer, weightsBuffer, biasBuffer):
        """instructions.js:157-177. weightsBuffer is [shared, cols]."""
        if cols % 8 != 0:
            raise ValueError("Cols must be divisible by 16.")
        resultBuffer = self.initResultBuffer([rows, cols])
        bias = biasBuffer
        return {"resultBuffer": resultBuffer,
                "passes": [self._compute("wgpt_matmul", rows, cols, shared, inputBuffer, weightsBuffer, bias,
                                         resultBuffer)]}


class ResidualBlockClass(Block):
    def __init__(self):
        super().__init__()
        self.name = "residual"

    def newInstance(self, rows, cols, outputBuf, residualBuf):
        """instructions.js:336-356."""
        if cols % 4 != 0:
            raise ValueError("Cols must be divisible by 4.")
        resultBuffer = self.initResultBuffer([rows, cols])
        return {"resultBuffer": resultBuffer,
                "passes": [self._compute("wgpt_residual", rows, cols, outputBuf, residualBuf, resultBuffer)]}


class LayerNormBlockClass(Block):
    def __init__(self):
        super().__init__()
        self.name = "layerNorm"

    def newInstance(self, rows, cols, inputBuffer, gammaBuffer, betaBuffer):
        """instructions.js:409-448 (statistics and normalisation are one kernel here)."""
        if cols % 4 != 0:
            raise ValueError("Cols must be divisible by 4.")
        resultBuffer = self.initResultBuffer([rows, cols])
        return {"resultBuffer": resultBuffer,
                "passes": [self._compute("wgpt_layernorm", rows, cols, inputBuffer, gammaBuffer, betaBuffer,
                                         resultBuffer)]}


class SoftmaxBlockClass(Block):
    def __init__(self):
        super().__init__()
        self.name = "softmax"

    def newInstance(self, rows, cols, inputBuffer, transpose=False):
        """instructions.js:567-588. The transposed store (:594) is never used by the model and is not offered."""
        if transpose:
            raise NotImplementedError("transposed softmax output is not used by the model path")
        resultBuffer = self.initResultBuffer([rows, cols])
        return {"resultBuffer": resultBuffer,
                "passes": [self._compute("wgpt_softmax", rows, cols, inputBuffer, resultBuffer)]}


class GeluBlockClass(Block):
    def __init__(self):
        super().__init__()
        self.name = "gelu"

    def newInstance(self, rows, cols, inputBuf):
        """instructions.js:683-703."""
        if cols % 4 != 0:
            raise ValueError("Cols must be divisible by 4.")
        resultBuffer = self.initResultBuffer([rows, cols])
        return {"resultBuffer": resultBuffer,
                "passes": [self._compute("wgpt_gelu", rows, cols, inputBuf, resultBuffer)]}


class EmbedBlockClass(Block):
    def __init__(self):
        super().__init__()
        self.name = "embed"

    def newInstance(self, idx, seq_length, n_embd, vocab_chunk_size, embdBuffers, posEmbdBuffer, ResidualBlock):
        """instructions.js:790-827. idx is a host sequence of token ids; the reference issues one buffer copy per
        token, here the ids are uploaded and gathered by one kernel. embdBuffers is the list of wte chunks; this
        build always loads a single chunk (no 128 MiB binding limit), so vocab_chunk_size == vocab size."""
        import numpy as np

        if len(embdBuffers) != 1:
            raise ValueError("embeddings are loaded as one chunk")
        ids = self.initBuffer(["storage", "copy_to"], [seq_length], f"ids_{seq_length}")
        ids.write(np.asarray(idx, dtype=np.uint32)[:seq_length])
        resultBuffer = self.initResultBuffer([seq_length, n_embd])
        return {"resultBuffer": resultBuffer,
                "passes": [self._compute("wgpt_embed", ids, seq_length, n_embd, vocab_chunk_size,
                                         embdBuffers[0], posEmbdBuffer, resultBuffer)]}


class DeEmbedBlockClass(Block):
    def __init__(self):
        super().__init__()
        self.name = "deembed"

    def newInstance(self, n_embd, vocab_size, padded_vocab_size, seq_length, vocab_chunk_size, embedBuffer,
                    deEmbeddingsBuffers):
        """instructions.js:844-888. deEmbeddingsBuffers is the single untransposed wte table."""
        if len(deEmbeddingsBuffers) != 1:
            raise ValueError("embeddings are loaded as one chunk")
        resultBuffer = self.initBuffer(["map_read", "copy_to"], [vocab_size], f"logits_{vocab_size}")
        return {"resultBuffer": resultBuffer,
                "passes": [self._compute("wgpt_deembed", n_embd, vocab_size, seq_length, embedBuffer,
                                         deEmbeddingsBuffers[0], resultBuffer)]}


class AttentionBlockClass(Block):
    def __init__(self):
        super().__init__()
        self.name = "attention"

    def newFusedInstance(self, seq_length, n_embd, attentionDotProductScale, n_head, head_size, inputBuffer,
                         qWeightsBuffer, qBiasBuffer, kWeightsBuffer, kBiasBuffer, vWeightsBuffer, vBiasBuffer,
                         linearWeightsBuffer, linearBiasBuffer, FastMatMulBlock=None, SoftmaxBlock=None):
        """instructions.js:985-1099: the eight passes of the reference collapse into one enqueue."""
        resultBuffer = self.initResultBuffer([seq_length, n_embd])
        return {"resultBuffer": resultBuffer,
                "passes": [self._compute("wgpt_attention", seq_length, n_embd, float(attentionDotProductScale), n_head,
                                         head_size, inputBuffer, qWeightsBuffer, qBiasBuffer,
                                         kWeightsBuffer, kBiasBuffer, vWeightsBuffer, vBiasBuffer,
                                         linearWeightsBuffer, linearBiasBuffer, resultBuffer)]}
