"""The multi-GPU host logic on CPU: two gloo ranks shard a ragged request set, run a stand-in
forward pass, gather the logits, and rank 0 must hold exactly what a single rank computes."""
import ctypes as C
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
        import torch

        def gather(block):
            mine = torch.from_numpy(block)
            every = [torch.zeros_like(mine) for _ in range(world)]
            dist.all_gather(every, mine)
            return [t.numpy() for t in every]

        out = dispatch.run_sharded(make_requests(), fake_forward, N_CLASSES, rank, world, gather=gather, b=1e-3)
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
    from system1_omni_b200 import model as M
    rng = np.random.default_rng(0)
    lengths = np.exp(rng.uniform(np.log(512), np.log(16384), 64)).astype(np.int32)     # the 27B config's request set
    for world in (1, 2, 4, 8):
        cost = lengths + 2e-5 * lengths.astype(np.float64) ** 2
        seen = []
        for rank in range(world):
            where, mine, packs = dispatch.layout(lengths, world, rank, a=1.0, b=2e-5)
            assert np.array_equal(where, M.assign_requests(lengths, world, 1.0, 2e-5))
            assert sorted(mine.tolist()) == np.flatnonzero(where == rank).tolist()
            # run order: by length, so that short prompts share packs
            assert np.all(np.diff(lengths[mine]) >= 0)
            # packs cover the rank's requests in order and respect the reference's limits
            assert [j for g in packs for j in g] == list(range(len(mine)))
            for g in packs:
                assert len(g) <= 16 and (len(g) == 1 or lengths[mine[list(g)]].sum() <= 4096)
            seen += mine.tolist()
        assert sorted(seen) == list(range(64))
        loads = np.array([cost[where == r].sum() for r in range(world)])
        assert loads.max() / loads.mean() < 1.15
    # the pack limits themselves, order kept (batching.rs:9-25)
    groups = M.ranges([4000, 100, 50, 5000] + [10] * 40)
    assert [list(g) for g in groups][:3] == [[0], [1, 2], [3]]
    assert all(len(g) <= 16 for g in groups)


def test_unequal_speeds_shift_load_to_the_faster_ranks():
    """Requests go where they finish earliest: finish times (load / speed) come out balanced, equal
    speeds reproduce the unweighted assignment, and invalid speeds are refused."""
    from system1_omni_b200 import dispatch
    from system1_omni_b200 import lib as L
    rng = np.random.default_rng(3)
    lengths = np.exp(rng.uniform(np.log(512), np.log(16384), 64)).astype(np.int32)
    cost = lengths + 2e-5 * lengths.astype(np.float64) ** 2
    world = 8
    plain = dispatch.layout(lengths, world, 0, a=1.0, b=2e-5)[0]
    assert np.array_equal(plain, dispatch.layout(lengths, world, 0, a=1.0, b=2e-5, speed=np.ones(world))[0])
    speed = np.array([0.95, 1.0, 1.05, 1.0, 1.0, 1.02, 0.97, 1.0])
    where = dispatch.layout(lengths, world, 0, a=1.0, b=2e-5, speed=speed)[0]
    for rank in range(1, world):        # every rank derives the same assignment
        assert np.array_equal(where, dispatch.layout(lengths, world, rank, a=1.0, b=2e-5, speed=speed)[0])
    finish = np.array([cost[where == r].sum() for r in range(world)]) / speed
    unweighted = np.array([cost[plain == r].sum() for r in range(world)]) / speed
    assert finish.max() / finish.mean() < 1.02
    assert finish.max() < unweighted.max()
    load = np.array([cost[where == r].sum() for r in range(world)])
    assert load[2] > load[0]            # the fastest rank carries more than the slowest
    bad = np.array([1.0, 0.0] + [1.0] * 6)
    out = np.zeros(64, np.int32)
    rc = L.load().s1_assign_requests_weighted(lengths.ctypes.data_as(C.c_void_p), 64, world, 1.0, 2e-5,
                                              bad.ctypes.data_as(C.c_void_p), out.ctypes.data_as(C.c_void_p))
    assert rc == 3000
