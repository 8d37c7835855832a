"""The multi-GPU host logic on CPU: two gloo ranks shard a ragged request set, run a stand-in
forward pass, gather the logits, and rank 0 must hold exactly what a single rank computes."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
N_CLASSES = 16


def fake_forward(batch):
    """Deterministic per-request logits that depend on every token and on nothing else."""
    out = np.zeros((len(batch), N_CLASSES), np.float32)
    for i, ids in enumerate(batch):
        a = np.asarray(ids, np.int64)
        for c in range(N_CLASSES):
            out[i, c] = np.float32(((a * (c + 3) + 7 * np.arange(a.size)) % 1013).sum() % 997) / np.float32(100.0)
    return out


def make_requests():
    rng = np.random.default_rng(5)
    lengths = np.exp(rng.uniform(np.log(8), np.log(700), 23)).astype(int)
    return [rng.integers(0, 1000, n).tolist() for n in lengths]


def worker(rank, world, port, result_path):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch.distributed as dist
    from system1_omni_b200 import dispatch
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        out = dispatch.run_sharded(make_requests(), fake_forward, N_CLASSES, rank, world, dist=dist, b=1e-3)
        if rank == 0:
            np.save(result_path, out)
        else:
            assert out is None
    finally:
        dist.destroy_process_group()


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_two_ranks_equal_one_rank(tmp_path):
    import torch.multiprocessing as mp
    from system1_omni_b200 import dispatch
    requests = make_requests()
    single = dispatch.run_sharded(requests, fake_forward, N_CLASSES, 0, 1)
    assert np.array_equal(single, fake_forward(requests))
    path = str(tmp_path / "rank0.npy")
    mp.spawn(worker, args=(2, free_port(), path), nprocs=2, join=True)
    assert np.array_equal(np.load(path), single)


def test_shards_are_balanced_and_complete():
    from system1_omni_b200 import dispatch
    rng = np.random.default_rng(0)
    lengths = np.exp(rng.uniform(np.log(512), np.log(16384), 64)).astype(np.int32)     # the 27B config's request set
    for world in (2, 4, 8):
        where = dispatch.shard(lengths, world, a=1.0, b=2e-5)
        cost = lengths + 2e-5 * lengths.astype(np.float64) ** 2
        loads = np.array([cost[where == r].sum() for r in range(world)])
        assert loads.max() / loads.mean() < 1.15
        assert np.bincount(where, minlength=world).sum() == 64
    # packs respect the reference's limits and keep order
    groups = dispatch.packs([4000, 100, 50, 5000] + [10] * 40)
    assert [list(g) for g in groups][:3] == [[0], [1, 2], [3]]
    assert all(len(g) <= 16 for g in groups)
