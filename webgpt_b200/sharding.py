"""Sequence sharding across GPUs: the only way this path scales out.

Independent sequences (each with its own ids, KV cache and logits; GPT.run has no cross-sequence state,
model.js:104-268) are split into contiguous blocks, one block per rank; weights are replicated; no collective
touches the data path. torch.distributed is used only to line ranks up (barrier), to take the maximum of the
per-rank device times, and to bring the generated ids back to rank 0.
"""
import numpy as np


def shard_range(n_seq, world, rank):
    """Contiguous block of sequence indices owned by `rank`: sizes differ by at most one, earlier ranks get the
    larger blocks. Returns (start, stop)."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    base, extra = divmod(n_seq, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def max_over_ranks(value, dist=None):
    """Largest `value` over all ranks (the job is as slow as its slowest GPU)."""
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return float(value)
    import torch
    dev = "cuda" if dist.get_backend() == "nccl" else "cpu"
    t = torch.tensor([float(value)], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def gather_ids(local_ids, n_seq, dist=None):
    """Rank 0 receives the [n_seq, n_new] ids of all sequences in order; other ranks receive None.
    local_ids is this rank's [stop - start, n_new] block."""
    local_ids = np.ascontiguousarray(local_ids, dtype=np.uint32)
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return local_ids
    world, rank = dist.get_world_size(), dist.get_rank()
    blocks = [None] * world if rank == 0 else None
    dist.gather_object(local_ids, blocks, dst=0)
    if rank != 0:
        return None
    out = np.concatenate([b.reshape(-1, local_ids.shape[1]) for b in blocks], axis=0)
    assert out.shape[0] == n_seq
    return out


def generate_sharded(generate_block, prompts, n_new, dist=None):
    """Runs generate_block(prompts_block, n_new) -> ids on this rank's block of `prompts` ([n_seq, n_prompt]) and
    gathers the result on rank 0."""
    prompts = np.asarray(prompts)
    world = dist.get_world_size() if dist is not None and dist.is_initialized() else 1
    rank = dist.get_rank() if world > 1 else 0
    a, b = shard_range(prompts.shape[0], world, rank)
    local = generate_block(prompts[a:b], n_new) if b > a else np.empty((0, n_new), np.uint32)
    return gather_ids(local, prompts.shape[0], dist if world > 1 else None)


class MultiGPT:
    """The same model on several GPUs of one process (weights replicated), for generating many independent
    sequences with one call: sequences are split into contiguous blocks (shard_range), one block per device, and
    wgpt_generate_greedy_sharded runs one host thread per device inside the library."""

    def __init__(self, params, weights, devices):
        from .model import GPT
        self.gpts = [GPT(None, params=params, weights=weights, device_ordinal=d) for d in devices]
        for g in self.gpts:
            g.initialize()
        self.params = self.gpts[0].params

    def generate_greedy(self, prompts, n_new):
        import ctypes as C
        from . import _lib
        prompts = np.ascontiguousarray(prompts, dtype=np.uint32)
        n_seq, n_prompt = prompts.shape
        world = len(self.gpts)
        sessions = []
        for r, g in enumerate(self.gpts):
            a, b = shard_range(n_seq, world, r)
            if b > a:
                sessions.append(g.session(b - a))
        arr = (C.c_void_p * len(sessions))(*[s.handle for s in sessions])
        out = np.empty((n_seq, n_new), np.uint32)
        _lib.call("wgpt_generate_greedy_sharded", arr, len(sessions), prompts.ctypes.data, n_prompt, n_new,
                  out.ctypes.data)
        return out

    def destroy(self):
        for g in self.gpts:
            g.destroy()
        self.gpts = []
