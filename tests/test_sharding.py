"""Host logic of the multi-GPU path on CPU: two gloo ranks each generate their block of sequences (with the CPU
oracle standing in for the device) and rank 0 must end up with exactly the unsharded result."""
import os
import sys

import numpy as np
import pytest

from conftest import ROOT
from webgpt_b200 import sharding, synth


def test_shard_range_partitions_exactly():
    for n in (0, 1, 7, 64, 65):
        for world in (1, 2, 3, 8):
            spans = [sharding.shard_range(n, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        sharding.shard_range(4, 2, 2)


def _worker(rank, world, port, out_path):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    from oracle import oracle as orc
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    params = synth.CONFIGS["tiny"]
    w = synth.make_weights(params, seed=3, std=0.2, ln_random=True)
    m = orc.Model(params, synth.weight_list(params, w))
    prompts = np.stack([synth.make_tokens(params["vocab_size"], 6, seed=5, stream=i) for i in range(5)])

    def block(p, n_new):
        return np.stack([m.generate_greedy(row, n_new)[len(row):] for row in p])

    ids = sharding.generate_sharded(block, prompts, 4, dist)
    slow = sharding.max_over_ranks(1.0 + rank, dist)
    assert slow == float(world)
    if rank == 0:
        np.save(out_path, ids)
    else:
        assert ids is None
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_sharded_generation_equals_unsharded(tmp_path, oracle):
    import torch.multiprocessing as mp
    out = str(tmp_path / "ids.npy")
    port = 29500 + os.getpid() % 1000
    mp.spawn(_worker, args=(2, port, out), nprocs=2, join=True)
    got = np.load(out)
    params = synth.CONFIGS["tiny"]
    w = synth.make_weights(params, seed=3, std=0.2, ln_random=True)
    m = oracle.Model(params, synth.weight_list(params, w))
    prompts = np.stack([synth.make_tokens(params["vocab_size"], 6, seed=5, stream=i) for i in range(5)])
    want = np.stack([m.generate_greedy(row, 4)[6:] for row in prompts])
    assert np.array_equal(got, want)
    # single-process path: same function, no process group
    assert np.array_equal(sharding.generate_sharded(lambda p, n: want[: len(p)], prompts, 4), want)
