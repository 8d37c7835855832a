"""The dispatcher of include/s1_dispatch.h on GPUs: one rank against the public forward call, the
queue-only entry point under many outstanding passes, a device-side wait that runs out surfacing
as a host error, and - where the box has two GPUs - two NCCL ranks against one."""
import ctypes as C
import os
import subprocess
import sys

import numpy as np
import pytest

from helpers import random_weights, tiny_config

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
N_CLASSES = 5


def make_requests(cfg, n=11, seed=3):
    rng = np.random.default_rng(seed)
    lengths = np.exp(rng.uniform(np.log(5), np.log(900), n)).astype(np.int32)
    lengths[2] = 4100                      # longer than a pack's token limit: runs alone
    return lengths, [rng.integers(0, cfg.vocab, int(t)).astype(np.int32) for t in lengths]


@pytest.fixture(scope="module")
def setup(cs1):
    from system1_omni_b200 import lib as L
    from system1_omni_b200 import model as M
    L.set_device(0)
    cfg = tiny_config()
    model = M.Model(cfg, device=0)
    model.set_tensors(random_weights(cfg, seed=4))
    yield cfg, model
    model.close()


def test_one_rank_equals_the_public_call(setup):
    from system1_omni_b200 import dispatch as D
    from system1_omni_b200 import model as M
    cfg, model = setup
    lengths, prompts = make_requests(cfg)
    head = np.random.default_rng(1).normal(0, 1, (N_CLASSES, cfg.hidden)).astype(np.float32)
    bias = np.linspace(-1, 1, N_CLASSES).astype(np.float32)
    d = D.Dispatcher(0, 1, 0)
    try:
        d.plan(model, lengths, N_CLASSES)
        assert sorted(d.local.tolist()) == list(range(len(prompts)))
        d.stage(np.concatenate(prompts))
        for resident in (False, True, False):
            if resident:
                d.upload()
            d.enqueue(resident)
            assert d.pack_ms().shape == (d.n_packs,)
            got, _ = d.collect(head, bias)
            # the same packs through the public call
            _, mine, packs = D.layout(lengths, 1, 0)
            for group in packs:
                reqs = [int(mine[j]) for j in group]
                last = model.forward_batch([prompts[i] for i in reqs])
                for row, i in zip(last, reqs):
                    want = M.head_logits(head, row, bias)
                    assert np.array_equal(want.view(np.uint32), got[i].view(np.uint32)), (resident, i)
    finally:
        d.close()


def make_candidates(cfg, seed=12):
    """A 128-token prefix and nine candidates of 3..70 tokens (the shape of the multi-candidate request)."""
    rng = np.random.default_rng(seed)
    prefix = rng.integers(0, cfg.vocab, 128).astype(np.int32)
    return prefix, [rng.integers(0, cfg.vocab, int(t)).astype(np.int32) for t in rng.integers(3, 71, 9)]


def test_candidates_on_one_rank_equal_the_one_shot_prompts(setup):
    """s1_dispatch_candidates with one rank: every candidate's logits equal, bit for bit, those of
    the whole prompt (prefix + candidate) run in one piece - whole-tile GEMMs make a row's bits
    independent of what it is packed with and of where the prefix came from."""
    from system1_omni_b200 import dispatch as D
    from system1_omni_b200 import model as M
    cfg, model = setup
    prefix_ids, cands = make_candidates(cfg)
    head = np.random.default_rng(2).normal(0, 1, (N_CLASSES, cfg.hidden)).astype(np.float32)
    bias = np.linspace(1, -1, N_CLASSES).astype(np.float32)
    d = D.Dispatcher(0, 1, 0)
    prefix = model.capture_prefix(prefix_ids.tolist())
    try:
        got, rank_of = d.candidates(model, prefix, cands, head, bias)
        assert np.all(rank_of == 0)
        for i, c in enumerate(cands):
            last = model.forward_batch([np.concatenate([prefix_ids, c])])[0]
            assert np.array_equal(M.head_logits(head, last, bias).view(np.uint32), got[i].view(np.uint32)), i
    finally:
        prefix.close()
        d.close()


def test_many_queued_passes_keep_their_own_offsets(setup):
    """More passes than the executor's ring of pinned offset slots, alternating between two length
    vectors, queued without a wait in between: every pass must gather its own last rows."""
    from system1_omni_b200 import lib as L
    cfg, model = setup
    lib = L.load()
    rng = np.random.default_rng(8)
    vectors = [np.array([40, 7, 90], np.int32), np.array([64, 73], np.int32)]
    ids = [rng.integers(0, cfg.vocab, int(v.sum())).astype(np.int32) for v in vectors]
    want = [model.forward_batch(np.split(i, np.cumsum(v)[:-1])) for i, v in zip(ids, vectors)]
    passes = 40
    rows = L.DeviceBuffer(passes * 3 * cfg.hidden * 2)
    pinned = []
    for k in range(passes):
        v, i = vectors[k % 2], ids[k % 2]
        p = C.c_void_p()
        L.check(lib.s1_host_alloc(C.byref(p), i.nbytes), "pinned")
        np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_int32)), shape=(i.size,))[:] = i
        pinned.append(p)
        L.check(lib.s1_model_forward_queue(model.handle, p, v.ctypes.data_as(C.c_void_p), v.size,
                                           rows.at(k * 3 * cfg.hidden * 2)), "forward_queue")
    out = np.zeros((passes, 3, cfg.hidden), np.uint16)
    L.check(lib.s1_model_read_rows(model.handle, out.ctypes.data_as(C.c_void_p), rows.at(), out.nbytes), "read rows")
    for p in pinned:
        lib.s1_host_free(p)
    import oracle as O
    for k in range(passes):
        n = vectors[k % 2].size
        assert np.array_equal(O.bf16_to_f32(out[k, :n]), want[k % 2]), k


def test_a_wait_that_runs_out_becomes_a_host_error(setup):
    """A bounded device-side wait that gives up must not pass silently: the kernel records a code
    and returns, the next call that reads results back returns CS1_ERR_DEVICE_CHECK, the words
    are cleared, and the context keeps working. The wait here is on a barrier nothing completes,
    with a limit of 200 microseconds; no fault, no trap."""
    from system1_omni_b200 import lib as L
    cfg, model = setup
    lib = L.load()
    prompt = [list(range(1, 50))]
    before = model.forward_batch(prompt)
    assert L.device_status() == (0, 0, 0)
    L.check(lib.s1_selftest_wait_runs_out(200, model.stream), "self-test")
    with pytest.raises(L.CudaError) as err:
        model.forward_batch(prompt)
    assert err.value.code == 2001
    assert L.device_status() == (0, 0, 0)              # cleared by the call that reported it
    assert np.array_equal(model.forward_batch(prompt), before)
    # the status entry point itself reports and clears
    L.check(lib.s1_selftest_wait_runs_out(200, model.stream), "self-test")
    assert L.device_status() == (99, 0, 0)
    assert L.device_status() == (0, 0, 0)
    # and a plain GEMM after it is as before
    assert np.array_equal(model.forward_batch(prompt), before)


RANK_SCRIPT = r"""
import os, sys
import numpy as np
sys.path.insert(0, {root!r}); sys.path.insert(0, os.path.join({root!r}, "tests"))
from helpers import random_weights, tiny_config
from test_dispatch_gpu import make_candidates, make_requests, N_CLASSES
from system1_omni_b200 import dispatch as D, lib as L, model as M
rank, world = int(sys.argv[1]), int(sys.argv[2])
L.load(); L.set_device(rank)
cfg = tiny_config()
model = M.Model(cfg, device=rank)
model.set_tensors(random_weights(cfg, seed=4))
lengths, prompts = make_requests(cfg)
head = np.random.default_rng(1).normal(0, 1, (N_CLASSES, cfg.hidden)).astype(np.float32)
d = D.Dispatcher(rank, world, rank, rendezvous=sys.argv[3])
d.plan(model, lengths, N_CLASSES)
d.stage(np.concatenate(prompts))
for _ in range(3):
    out, us = d.run(head)
assert d.max_over_ranks(rank) == world - 1
assert np.array_equal(d.allgather([rank, 2.5]), [[r, 2.5] for r in range(world)])
# the multi-candidate request: every rank captures the prefix, the candidates are shared out
prefix_ids, cands = make_candidates(cfg)
prefix = model.capture_prefix(prefix_ids.tolist())
d.set_speed([1.0, 1.6][:world] if world == 2 else None)      # unequal on purpose: the faster rank takes more
scores, where = d.candidates(model, prefix, cands, head)
d.barrier()
if rank == 0:
    np.save(sys.argv[4], out)
    np.save(sys.argv[4] + ".cand.npy", scores)
    np.save(sys.argv[4] + ".where.npy", where)
prefix.close(); d.close(); model.close()
"""


def test_two_ranks_equal_one_rank(setup, tmp_path):
    """Two processes, one GPU each, NCCL gather: rank 0 holds bit for bit what one rank computes
    when it runs the same packs (a prompt's bits depend on its pack, not on its GPU)."""
    from system1_omni_b200 import dispatch as D
    from system1_omni_b200 import lib as L
    from system1_omni_b200 import model as M
    if L.device_count() < 2:
        pytest.skip("needs two GPUs")
    cfg, model = setup
    lengths, prompts = make_requests(cfg)
    head = np.random.default_rng(1).normal(0, 1, (N_CLASSES, cfg.hidden)).astype(np.float32)
    script = tmp_path / "rank.py"
    script.write_text(RANK_SCRIPT.format(root=ROOT))
    rv, result = str(tmp_path / "nccl.id"), str(tmp_path / "rank0.npy")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    procs = [subprocess.Popen([sys.executable, str(script), str(r), "2", rv, result], env=env) for r in range(2)]
    for p in procs:
        assert p.wait(timeout=600) == 0
    got = np.load(result)
    for rank in range(2):
        _, mine, packs = D.layout(lengths, 2, rank)
        for group in packs:
            reqs = [int(mine[j]) for j in group]
            last = model.forward_batch([prompts[i] for i in reqs])
            for row, i in zip(last, reqs):
                assert np.array_equal(M.head_logits(head, row).view(np.uint32), got[i].view(np.uint32)), i
    # the multi-candidate request: both ranks took part (the faster one more), and every candidate's
    # logits equal those of its whole prompt run on one GPU
    scores, where = np.load(result + ".cand.npy"), np.load(result + ".where.npy")
    prefix_ids, cands = make_candidates(cfg)
    assert set(where.tolist()) == {0, 1}
    tokens = np.array([len(c) for c in cands])
    assert tokens[where == 1].sum() > tokens[where == 0].sum()
    for i, c in enumerate(cands):
        last = model.forward_batch([np.concatenate([prefix_ids, c])])[0]
        assert np.array_equal(M.head_logits(head, last).view(np.uint32), scores[i].view(np.uint32)), i
