"""class GPT with the surface of the reference's model.js, driving the B200 kernels through the C ABI.

Two execution routes share one weight source:
  * the fused route (default): weights live in a `wgpt_model`, `run` is one `wgpt_model_run` call and
    `generate` is one `wgpt_generate_greedy` (top_k = 1) or `wgpt_generate_sample` call with the KV cache and
    the pick on the device;
  * the pass-list route (`fused=False`): `run` builds the reference's pass list from the instruction classes
    (model.js:114-241) and replays it (model.js:245-257), one C-ABI call per operator.
Token ids go in and come out as integers; the reference's tokenizers (tokenizer.js) are host-side string code
outside this package, so `prompt` may be a list of ids, or a string when a tokenizer object with
encode/decode is supplied.
"""
import ctypes as C
import json
import math
import os
import random
import time

import numpy as np

from . import _lib, globals as G, synth
from .device import Device


class Session:
    """KV cache + activations of n_seq equal-length sequences (wgpt_session)."""

    def __init__(self, gpt, n_seq=1):
        self.gpt = gpt
        self.n_seq = n_seq
        h = C.c_void_p()
        _lib.call("wgpt_session_create", gpt.model_handle, n_seq, C.byref(h))
        self.handle = h

    def reset(self):
        _lib.call("wgpt_session_reset", self.handle)

    def length(self):
        n = C.c_int32()
        _lib.call("wgpt_session_length", self.handle, C.byref(n))
        return n.value

    def forward(self, ids, want_logits=True):
        ids = np.ascontiguousarray(ids, dtype=np.uint32).reshape(self.n_seq, -1)
        V = self.gpt.params["vocab_size"]
        logits = np.empty((self.n_seq, V), np.float32) if want_logits else None
        _lib.call("wgpt_session_forward", self.handle, ids.ctypes.data, ids.shape[1],
                  logits.ctypes.data if want_logits else None)
        return logits

    def generate_greedy(self, prompts, n_new):
        prompts = np.ascontiguousarray(prompts, dtype=np.uint32).reshape(self.n_seq, -1)
        out = np.empty((self.n_seq, n_new), np.uint32)
        _lib.call("wgpt_generate_greedy", self.handle, prompts.ctypes.data, prompts.shape[1], n_new, out.ctypes.data)
        return out

    def generate_sample(self, prompts, n_new, top_k, temperature, uniforms):
        """Top-k sampling on the device (model.js:81-83); uniforms is [n_new, n_seq] numbers in [0,1)."""
        prompts = np.ascontiguousarray(prompts, dtype=np.uint32).reshape(self.n_seq, -1)
        u = np.ascontiguousarray(uniforms, dtype=np.float64).reshape(n_new, self.n_seq)
        out = np.empty((self.n_seq, n_new), np.uint32)
        _lib.call("wgpt_generate_sample", self.handle, prompts.ctypes.data, prompts.shape[1], n_new, int(top_k),
                  float(temperature), u.ctypes.data, out.ctypes.data)
        return out

    def tap(self):
        rows_max = self.n_seq * self.gpt.params["n_ctx"]
        E = self.gpt.params["n_embd"]
        buf = self.gpt.device.buffer(rows_max * E * 4)
        n = C.c_uint64()
        _lib.call("wgpt_session_tap", self.handle, buf.ptr, rows_max * E, C.byref(n))
        out = buf.read(np.float32, n.value).reshape(-1, E)
        buf.destroy()
        return out

    def destroy(self):
        if self.handle:
            h, self.handle = self.handle, None
            _lib.call("wgpt_session_destroy", h)


class GPT:
    def __init__(self, folder, type="bpe", *, weights=None, params=None, fused=True, device_ordinal=0,
                 tokenizer=None, weight_layout=None):
        """model.js:2-21. `folder` is a weight directory in the reference's format; alternatively pass
        `params` + `weights` (a dict of state-dict-keyed arrays, e.g. from synth.make_weights)."""
        self.folder = folder
        self.tokenizerType = type
        self.initialized = False
        self.device = None
        self.model = None
        self.tokenizer = tokenizer
        self.params = dict(params) if params else None
        self.minBufferOffset = 1
        self.defaultPrompt = None
        self.defaultTopK = None
        self.defaultTemperature = None
        self.defaultTokens = None
        self.externalBuffer = None
        self.unloadDeletionStack = []
        self._weights = weights
        self._weight_layout = weight_layout  # None: what params_gpt.json says ("in_out" when it says nothing)
        self._fused = fused
        self._ordinal = device_ordinal
        self.model_handle = None
        self._session = None
        self.averageKernelTime = None

    # ------------------------------------------------------------------ lifecycle
    def initialize(self):
        """model.js:23-51."""
        if self.initialized:
            print("Model already initialized")
            return
        self.device = Device(self._ordinal)  # raises when no B200 / no library: there is no other path
        G.initializeOperations(self.device)
        self.model, self.params = self.loadModel(self.folder)
        if self.tokenizerType == "bpe":
            self.defaultTopK, self.defaultTemperature, self.defaultTokens = 3, 1, 30
        else:
            self.defaultTopK, self.defaultTemperature, self.defaultTokens = 2, 1, 80
        self.initialized = True

    def destroy(self):
        if self._session:
            self._session.destroy()
            self._session = None
        self.unloadBuffers()
        G.destroyOperations()
        if self.model_handle:
            _lib.call("wgpt_model_destroy", self.model_handle)
            self.model_handle = None
        if self.device:
            self.device.destroy()
            self.device = None
        self.initialized = False

    # ------------------------------------------------------------------ generation
    def generate(self, prompt, max_new_tokens, top_k, temperature=1.0, rand=None):
        """model.js:53-102: yields one token per step (a decoded string with a tokenizer, else the id)."""
        if not self.initialized:
            print("Model not loaded yet")
            return
        history = list(self.tokenizer.encode(prompt)) if self.tokenizer and isinstance(prompt, str) else [int(t) for t in prompt]
        dec = (lambda t: self.tokenizer.decode([t])) if self.tokenizer else (lambda t: t)
        if self._fused and top_k == 1:
            # Greedy: one call; KV cache, arg-max and window handling are inside the library.
            t0 = time.perf_counter()
            new = self.session().generate_greedy(np.array(history, np.uint32), max_new_tokens)[0]
            self.averageKernelTime = (time.perf_counter() - t0) * 1e3 / max_new_tokens
            for t in new:
                yield dec(int(t))
            return
        top_k, temperature = int(top_k), float(temperature)  # the page passes both as strings (index.html:89-91)
        if self._fused and top_k <= _lib.MAX_TOP_K:
            # Sampled: also one call. The random numbers are drawn here, one per token in order as
            # sampleFromDistribution would draw them (globals.js:48), and the picks happen on the device.
            u = np.array([(rand() if rand else random.random()) for _ in range(max_new_tokens)], np.float64)
            t0 = time.perf_counter()
            new = self.session().generate_sample(np.array(history, np.uint32), max_new_tokens, top_k, temperature, u)[0]
            self.averageKernelTime = (time.perf_counter() - t0) * 1e3 / max_new_tokens
            for t in new:
                yield dec(int(t))
            return
        warmupRuns, totalTime = 3, 0.0
        n_ctx = self.params["n_ctx"]
        for i in range(max_new_tokens):
            idx_cond = history[-n_ctx:]
            t0 = time.perf_counter()
            logits = self.run(idx_cond)
            lapsed = (time.perf_counter() - t0) * 1e3
            if i >= warmupRuns:
                totalTime += lapsed
            top = G.selectTopK(logits, top_k)
            probs = G.cpuSoftmax(top["topKProbs"], temperature)
            idx_next = top["topKIndices"][G.sampleFromDistribution(probs, rand() if rand else None)]
            history.append(idx_next)
            yield dec(idx_next)
        if max_new_tokens > warmupRuns:
            self.averageKernelTime = totalTime / (max_new_tokens - warmupRuns)

    def session(self, n_seq=1):
        if self._session is None or self._session.n_seq != n_seq:
            if self._session:
                self._session.destroy()
            self._session = Session(self, n_seq)
        return self._session

    def run(self, idx):
        """model.js:104-268: logits (vocab_size floats) of the last position of the window idx."""
        idx = [int(t) for t in idx]
        if self._fused:
            ids = np.array(idx, np.uint32)
            logits = np.empty(self.params["vocab_size"], np.float32)
            s = self.session()
            _lib.call("wgpt_model_run", s.handle, ids.ctypes.data, len(idx), logits.ctypes.data)
            if self.externalBuffer is not None:
                n = C.c_uint64()
                _lib.call("wgpt_session_tap", s.handle, self.externalBuffer.ptr, self.externalBuffer.nbytes // 4,
                          C.byref(n))
            return logits
        return self._run_passes(idx)

    def _run_passes(self, idx):
        m, p = self.model, self.params
        seq_length = len(idx)
        n_embd, n_head, head_size, hidden = p["n_embd"], p["n_head"], p["head_size"], p["hidden_size"]
        self.computePasses = []

        def push(inst):
            self.computePasses.extend(inst["passes"])
            return inst["resultBuffer"]

        intermediate = push(G.EmbedBlock.newInstance(idx, seq_length, n_embd, p["vocab_chunk_size"],
                                                     m["embeddingsBuffers"], m["posEmbdBuffer"], G.ResidualBlock))
        residual = intermediate
        for b in m["layer_buffers"]:
            intermediate = push(G.LayerNormBlock.newInstance(seq_length, n_embd, intermediate,
                                                             b["normAttentionGammaBuffer"], b["normAttentionBetaBuffer"]))
            intermediate = push(G.AttentionBlock.newFusedInstance(
                seq_length, n_embd, p["attention_scale"], n_head, head_size, intermediate,
                b["qkvWeightArray"][0], b["qkvBiasArray"][0], b["qkvWeightArray"][1], b["qkvBiasArray"][1],
                b["qkvWeightArray"][2], b["qkvBiasArray"][2], b["linearWeightsBuffer"], b["linearBiasBuffer"],
                G.FastMatMulBlock, G.SoftmaxBlock))
            intermediate = residual = push(G.ResidualBlock.newInstance(seq_length, n_embd, intermediate, residual))
            intermediate = push(G.LayerNormBlock.newInstance(seq_length, n_embd, intermediate,
                                                             b["normLinearGammaBuffer"], b["normLinearBetaBuffer"]))
            intermediate = push(G.FastMatMulBlock.newInstance(seq_length, hidden, n_embd, intermediate,
                                                              b["firstLayerWeightsBuffer"], b["firstLayerBiasBuffer"]))
            intermediate = push(G.GeluBlock.newInstance(seq_length, hidden, intermediate))
            intermediate = push(G.FastMatMulBlock.newInstance(seq_length, n_embd, hidden, intermediate,
                                                              b["secondLayerWeightsBuffer"], b["secondLayerBiasBuffer"]))
            intermediate = residual = push(G.ResidualBlock.newInstance(seq_length, n_embd, intermediate, residual))
        if self.externalBuffer is not None:  # model.js:211-222
            self.computePasses.append({"flag": "copy", "src": intermediate, "srcOffset": 0, "dst": self.externalBuffer,
                                       "dstOffset": 0, "size": self.bufferSize(seq_length, n_embd)})
        intermediate = push(G.LayerNormBlock.newInstance(seq_length, n_embd, intermediate, m["normGammaBuffer"],
                                                         m["normBetaBuffer"]))
        result = push(G.DeEmbedBlock.newInstance(n_embd, p["vocab_size"],
                                                 p["vocab_chunk_size"] * p["vocab_chunk_instances"], seq_length,
                                                 p["vocab_chunk_size"], intermediate, m["deEmbeddingsBuffers"]))
        for ps in self.computePasses:  # model.js:245-257
            if ps["flag"] == "compute":
                ps["run"]()
            elif ps["flag"] == "copy":
                self.device.copy(ps["src"], ps["srcOffset"], ps["dst"], ps["dstOffset"], ps["size"])
        out = result.read(np.float32, p["vocab_size"])  # model.js:261-263
        G.clearOperationCache()
        return out

    # ------------------------------------------------------------------ loading
    def _fetch(self, folder, key):
        """One tensor in the [in, out] convention of model.js, flattened. Folders in nanoGPT's nn.Linear [out, in]
        convention (condensed/condensed.js:1765-1784) are transposed here, as that loader does; bias-free
        checkpoints have no bias files and read as zeros (condensed/condensed.js:1762-1782, model.js:322)."""
        if self._weights is not None:
            return np.ascontiguousarray(self._weights[key], dtype=np.float32).ravel()
        path = os.path.join(folder, f"{key}_gpt.bin")
        shape = synth.tensor_shape(self.params, key)
        if key.endswith(".bias") and not self.params.get("bias", True) and not os.path.exists(path):
            return np.zeros(shape, np.float32).ravel()
        data = G.fetchBin(path)
        if self.params.get("weight_layout", "in_out") == "out_in" and len(shape) == 2 and ".h." in key:
            data = np.ascontiguousarray(data.reshape(shape[1], shape[0]).T).ravel()
        return data

    def loadModel(self, folder):
        """model.js:270-287."""
        if self.initialized:
            print("Model already loaded")
            return
        weightsFolder = os.path.join("weights", folder) if (folder and not os.path.isdir(folder)) else folder
        params = self.loadParameters(weightsFolder)
        self.params = params
        output = {}
        if self._fused:
            P = _lib.Params(params["n_layer"], params["n_head"], params["n_embd"], params["n_ctx"],
                            params["vocab_size"], 1 if params["bias"] else 0)
            h = C.c_void_p()
            _lib.call("wgpt_model_create", self.device.handle, C.byref(P), C.byref(h))
            self.model_handle = h
            for name in synth.tensor_names(params):
                data = self._fetch(weightsFolder, name)
                _lib.call("wgpt_model_set_tensor", h, name.encode(), data.ctypes.data, data.size)
            _lib.call("wgpt_model_finalize", h)
            return output, params
        output.update(self.loadEmbeddings(params, weightsFolder))
        output.update(self.loadPositionalEmbeddings(params, weightsFolder))
        output["layer_buffers"] = self.loadLayers(params, weightsFolder)
        output.update(self.loadFinalLayerNorm(params, weightsFolder))
        return output, params

    def loadParameters(self, weightsFolder):
        """model.js:289-337. CUDA has no storage-binding limit, so the vocabulary is always one chunk."""
        if self.params is not None:
            params = dict(self.params)
        else:
            with open(os.path.join(weightsFolder, "params_gpt.json")) as f:
                params = json.load(f)
            # the exporters write the HF config (n_positions beside or instead of n_ctx) or nanoGPT's model args
            # (block_size, as condensed/condensed.js:1726 reads it)
            if "n_ctx" not in params:
                params["n_ctx"] = params.get("n_positions", params.get("block_size"))
            if self._weight_layout is not None:
                params["weight_layout"] = self._weight_layout
            if params.get("weight_layout", "in_out") not in ("in_out", "out_in"):
                raise ValueError("Model load failed: weight_layout must be 'in_out' or 'out_in'.")
        if params["n_embd"] % 4 != 0:
            raise ValueError("Model load failed: n_embd must be divisible by 4.")
        if params["n_embd"] % params["n_head"] != 0:
            raise ValueError("Model load failed: n_embd must be divisible by n_head.")
        if (params["n_embd"] // params["n_head"]) % 4 != 0:
            raise ValueError("Model load failed: n_embd / n_head must be divisible by 4.")
        params["vocab_chunk_size"] = params["vocab_size"]
        params["vocab_chunk_instances"] = 1
        params["head_size"] = params["n_embd"] // params["n_head"]
        params["hidden_size"] = params["n_embd"] * 4
        params["attention_scale"] = 1 / math.sqrt(params["n_embd"] / params["n_head"])
        params["bias"] = True if params.get("bias") is None else params["bias"]
        return params

    def loadEmbeddings(self, params, weightsFolder):
        """model.js:339-367. One untransposed table serves both the gather and the de-embedding."""
        wte = self._fetch(weightsFolder, "transformer.wte.weight")
        buf = self.initTensor(wte, [params["vocab_size"], params["n_embd"]], ["copy_from", "storage"])
        return {"embeddingsBuffers": [buf], "deEmbeddingsBuffers": [buf]}

    def loadPositionalEmbeddings(self, params, weightsFolder):
        """model.js:369-375."""
        wpe = self._fetch(weightsFolder, "transformer.wpe.weight")
        return {"posEmbdBuffer": self.initTensor(wpe, [params["n_ctx"], params["n_embd"]], ["copy_from"])}

    def loadFinalLayerNorm(self, params, weightsFolder):
        """model.js:377-389."""
        E = params["n_embd"]
        return {"normGammaBuffer": self.fetchAndInitTensor(weightsFolder, "transformer.ln_f.weight", [E], ["storage"]),
                "normBetaBuffer": self.fetchAndInitTensor(weightsFolder, "transformer.ln_f.bias", [E], ["storage"])}

    def loadLayers(self, params, weightsFolder):
        """model.js:391-401."""
        return [self.loadLayer(params, weightsFolder, i) for i in range(params["n_layer"])]

    def loadLayer(self, params, weightsFolder, layerIndex):
        """model.js:403-454."""
        E, F = params["n_embd"], params["hidden_size"]
        pre = f"transformer.h.{layerIndex}."
        f = lambda k, dims: self.fetchAndInitTensor(weightsFolder, pre + k, dims, ["storage"])  # noqa: E731
        return {
            "normAttentionGammaBuffer": f("ln_1.weight", [E]),
            "normAttentionBetaBuffer": f("ln_1.bias", [E]),
            "qkvWeightArray": self.fetchAndSplitQKVWeightTensors(weightsFolder, pre + "attn.c_attn.weight", [E, 3 * E], ["storage"]),
            "qkvBiasArray": self.fetchAndSplitQKVBiasTensors(weightsFolder, pre + "attn.c_attn.bias", [E], ["storage"]),
            "linearWeightsBuffer": f("attn.c_proj.weight", [E, E]),
            "linearBiasBuffer": f("attn.c_proj.bias", [E]),
            "normLinearGammaBuffer": f("ln_2.weight", [E]),
            "normLinearBetaBuffer": f("ln_2.bias", [E]),
            "firstLayerWeightsBuffer": f("mlp.c_fc.weight", [E, F]),
            "firstLayerBiasBuffer": f("mlp.c_fc.bias", [F]),
            "secondLayerWeightsBuffer": f("mlp.c_proj.weight", [F, E]),
            "secondLayerBiasBuffer": f("mlp.c_proj.bias", [E]),
        }

    def fetchAndSplitQKVWeightTensors(self, weightsFolder, key, dims, ops):
        """model.js:456-468: [E,3E] -> three [E,E] matrices (columns Q | K | V)."""
        E = dims[0]
        data = self._fetch(weightsFolder, key).reshape(E, 3 * E)
        return [self.initTensor(np.ascontiguousarray(data[:, i * E:(i + 1) * E]), [E, E], ops) for i in range(3)]

    def fetchAndSplitQKVBiasTensors(self, weightsFolder, key, dims, ops):
        """model.js:470-482."""
        E = dims[0]
        data = self._fetch(weightsFolder, key)
        return [self.initTensor(data[i * E:(i + 1) * E], [E], ops) for i in range(3)]

    def fetchAndInitTensor(self, weightsFolder, key, dims, ops):
        """model.js:484-488."""
        return self.initTensor(self._fetch(weightsFolder, key), dims, ops)

    def initTensor(self, data, dims, ops):
        """model.js:490-500."""
        d = list(dims) + [1, 1]
        buf = self.device.buffer(self.bufferSize(d[0], d[1], d[2]), dims)
        buf.write(np.ascontiguousarray(data, dtype=np.float32))
        self.unloadDeletionStack.append(buf)
        return buf

    def unloadBuffers(self):
        """model.js:502-505."""
        for b in self.unloadDeletionStack:
            b.destroy()
        self.unloadDeletionStack = []

    def bufferSize(self, dimX, dimY=1, dimZ=1):
        """model.js:507-512."""
        return int(math.ceil(dimX * dimY * dimZ * 4 / self.minBufferOffset) * self.minBufferOffset)
