"""Operator singletons and host helpers with the surface of the reference's globals.js."""
import math
import random

import numpy as np

from .instructions import (AttentionBlockClass, DeEmbedBlockClass, EmbedBlockClass, FastMatMulBlockClass,
                           GeluBlockClass, LayerNormBlockClass, ResidualBlockClass, SoftmaxBlockClass)

# globals.js:1-8
FastMatMulBlock = FastMatMulBlockClass()
AttentionBlock = AttentionBlockClass()
ResidualBlock = ResidualBlockClass()
EmbedBlock = EmbedBlockClass()
DeEmbedBlock = DeEmbedBlockClass()
GeluBlock = GeluBlockClass()
LayerNormBlock = LayerNormBlockClass()
SoftmaxBlock = SoftmaxBlockClass()

# globals.js:11
operations = [FastMatMulBlock, AttentionBlock, ResidualBlock, EmbedBlock, DeEmbedBlock, GeluBlock, LayerNormBlock,
              SoftmaxBlock]


def initializeOperations(device):  # globals.js:13
    for op in operations:
        op.initialize(device)


def destroyOperationBuffers():  # globals.js:17
    for op in operations:
        op.destroyBuffers()


def clearOperationCache():  # globals.js:21
    for op in operations:
        op.clearBufferCache()


def destroyOperations():  # globals.js:25
    for op in operations:
        op.destroy()


def fetchBin(path):
    """globals.js:39-43 with a file path in place of a URL: raw little-endian f32."""
    return np.fromfile(path, dtype="<f4")


def wgSize(dim, size):  # globals.js:45
    return math.ceil(dim / size)


def sampleFromDistribution(probs, rand=None):
    """globals.js:47-57. `rand` replaces Math.random() for reproducible tests."""
    r = random.random() if rand is None else rand
    c = 0.0
    for i, p in enumerate(probs):
        c += p
        if r < c:
            return i
    return len(probs) - 1


def cpuSoftmax(logits, temperature=1.0):
    """globals.js:59-64 (f64 arithmetic like JS numbers)."""
    logits = [float(v) for v in logits]
    m = max(logits)
    e = [math.exp((v - m) / temperature) for v in logits]
    s = sum(e)
    return [v / s for v in e]


def selectTopK(probs, top_k):
    """globals.js:66-74: stable descending sort, so equal values keep index order."""
    probs = np.asarray(probs)
    order = np.argsort(-probs.astype(np.float64), kind="stable")
    idx = [int(i) for i in order[:top_k]]
    return {"topKIndices": idx, "topKProbs": [float(probs[i]) for i in idx]}


def zeros(dim):  # globals.js:78
    return np.zeros(dim, np.float32)


def transpose(array, input_rows, input_cols):
    """globals.js:80-94."""
    a = np.asarray(array, np.float32)
    if a.size != input_rows * input_cols:
        raise ValueError("Transpose dims failed")
    return np.ascontiguousarray(a.reshape(input_rows, input_cols).T).ravel()


def formatAsMatrix(floatArray, dimA, dimB):  # globals.js:103
    return [np.asarray(floatArray)[i * dimB:(i + 1) * dimB] for i in range(dimA)]
