"""Request sharding across the GPUs of one box: replicated weights, whole requests per rank,
one small gather of decision logits. The reference serves from a single device
(src/models/qwen3_5/native/src/model.rs:625 pins device 0), so this layer has no counterpart
there; per-request results must equal single-GPU execution, which the tests check.

`Dispatcher` mirrors the C ABI of include/s1_dispatch.h (one process per GPU, NCCL bound by
the library itself at run time; no torch). `layout` is the plan alone, on the host.
`run_sharded` drives the same plan with a caller-supplied forward and gather, which is how the
multi-rank logic is covered on CPU (gloo ranks, a stand-in forward).
"""
import ctypes as C
import importlib.util
import os

import numpy as np

from . import lib as L
from . import model as M


def layout(lengths, world, rank, a=1.0, b=4e-6, speed=None):
    """(rank_of [n], this rank's request indices in run order, packs as ranges over that order).
    speed: relative speed of every rank's GPU (None = equal)."""
    lengths = np.ascontiguousarray(lengths, dtype=np.int32)
    sp = None if speed is None else np.ascontiguousarray(speed, dtype=np.float64)
    if sp is not None and sp.size != world:
        raise ValueError("one speed per rank")
    n = lengths.size
    rank_of = np.zeros(max(n, 1), np.int32)
    local = np.zeros(max(n, 1), np.int32)
    starts = np.zeros(max(n, 1), np.int32)
    n_local = C.c_int(0)
    packs = L.load().s1_dispatch_layout_weighted(lengths.ctypes.data_as(C.c_void_p), n, world, a, b,
                                                 None if sp is None else sp.ctypes.data_as(C.c_void_p), rank,
                                                 rank_of.ctypes.data_as(C.c_void_p), local.ctypes.data_as(C.c_void_p),
                                                 C.byref(n_local), starts.ctypes.data_as(C.c_void_p))
    if packs < 0:
        raise L.CudaError(-packs, "dispatch layout")
    edges = [int(x) for x in starts[:packs]] + [n_local.value]
    return rank_of[:n].copy(), local[:n_local.value].copy(), [range(edges[i], edges[i + 1]) for i in range(packs)]


def nccl_library():
    """Path of the libnccl.so.2 that ships with the Python environment, or None (loader default)."""
    spec = importlib.util.find_spec("nvidia")
    for root in (spec.submodule_search_locations if spec else []):
        path = os.path.join(root, "nccl", "lib", "libnccl.so.2")
        if os.path.exists(path):
            return path
    return None


def rendezvous_path():
    """A file name all ranks of one launch agree on and no other launch uses: the launcher's
    process id (the ranks are its children) and the master port."""
    key = f"{os.environ.get('MASTER_PORT', '0')}_{os.getppid()}_{os.environ.get('TORCHELASTIC_RUN_ID', 'none')}"
    root = "/dev/shm" if os.path.isdir("/dev/shm") else "/tmp"
    return os.path.join(root, f"s1_dispatch_{key}.id")


class Dispatcher:
    """One rank of the dispatcher of include/s1_dispatch.h."""

    def __init__(self, rank=0, world=1, device=0, rendezvous=None, nccl=None):
        self.rank, self.world = rank, world
        self.handle = C.c_void_p()
        rv = (rendezvous or rendezvous_path()).encode() if world > 1 else None
        lib_path = nccl if nccl is not None else nccl_library()
        L.check(L.load().s1_dispatch_create(rank, world, device, rv, lib_path.encode() if lib_path else None,
                                            C.byref(self.handle)), "dispatch create")
        self.n = self.n_classes = 0

    def close(self):
        if getattr(self, "handle", None) and self.handle.value:
            L.load().s1_dispatch_destroy(self.handle)
            self.handle = C.c_void_p()

    def set_cost(self, a, b):
        L.check(L.load().s1_dispatch_set_cost(self.handle, float(a), float(b)), "dispatch cost")

    def set_speed(self, speed):
        """Relative speed of every rank's GPU (None = equal); used by the next plan."""
        if speed is None:
            L.check(L.load().s1_dispatch_set_speed(self.handle, None, self.world), "dispatch speed")
            return
        sp = np.ascontiguousarray(speed, dtype=np.float64)
        L.check(L.load().s1_dispatch_set_speed(self.handle, sp.ctypes.data_as(C.c_void_p), sp.size), "dispatch speed")

    def plan(self, model, lengths, n_classes):
        lengths = np.ascontiguousarray(lengths, dtype=np.int32)
        L.check(L.load().s1_dispatch_plan(self.handle, model.handle, lengths.ctypes.data_as(C.c_void_p), lengths.size,
                                          n_classes), "dispatch plan")
        self.n, self.n_classes = int(lengths.size), int(n_classes)
        n_local, tokens, packs = C.c_int(), C.c_longlong(), C.c_int()
        rank_of = np.zeros(self.n, np.int32)
        L.check(L.load().s1_dispatch_info(self.handle, C.byref(n_local), C.byref(tokens), C.byref(packs),
                                          rank_of.ctypes.data_as(C.c_void_p)), "dispatch info")
        local = np.zeros(max(n_local.value, 1), np.int32)
        starts = np.zeros(max(packs.value, 1), np.int32)
        L.check(L.load().s1_dispatch_local(self.handle, local.ctypes.data_as(C.c_void_p),
                                           starts.ctypes.data_as(C.c_void_p)), "dispatch local")
        self.rank_of, self.local = rank_of, local[:n_local.value].copy()
        self.pack_start = starts[:packs.value].copy()
        self.local_tokens, self.n_packs = int(tokens.value), int(packs.value)
        return self

    def stage(self, ids_all):
        ids_all = np.ascontiguousarray(ids_all, dtype=np.int32)
        L.check(L.load().s1_dispatch_stage(self.handle, ids_all.ctypes.data_as(C.c_void_p)), "dispatch stage")

    def upload(self):
        L.check(L.load().s1_dispatch_upload(self.handle), "dispatch upload")

    def enqueue(self, resident=False):
        L.check(L.load().s1_dispatch_enqueue(self.handle, int(resident)), "dispatch enqueue")

    def pack_ms(self):
        out = np.zeros(max(self.n_packs, 1), np.float32)
        L.check(L.load().s1_dispatch_pack_ms(self.handle, out.ctypes.data_as(C.c_void_p)), "dispatch pack ms")
        return out[:self.n_packs]

    def collect(self, head, bias=None):
        """Rank 0: (float32 [n, n_classes] in request order, gather microseconds); others (None, us)."""
        head = np.ascontiguousarray(head, dtype=np.float32)
        b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
        out = np.zeros((self.n, self.n_classes), np.float32) if self.rank == 0 else None
        us = C.c_double(0)
        L.check(L.load().s1_dispatch_collect(self.handle, head.ctypes.data_as(C.c_void_p),
                                             None if b is None else b.ctypes.data_as(C.c_void_p),
                                             None if out is None else out.ctypes.data_as(C.c_void_p), C.byref(us)),
                "dispatch collect")
        return out, us.value

    def run(self, head, bias=None):
        """One end-to-end step from staged ids: queue every pack, read back, head, gather."""
        self.enqueue(False)
        return self.collect(head, bias)

    def candidates(self, model, prefix, candidates, head, bias=None):
        """One multi-candidate request: `candidates` (lists of token ids, the same on every rank)
        continue `prefix` (captured on this rank's model) on the ranks they are assigned to.
        Rank 0: (float32 [n, n_classes] in candidate order, rank_of [n]); others (None, rank_of)."""
        head = np.ascontiguousarray(head, dtype=np.float32)
        b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
        lengths = np.array([len(c) for c in candidates], np.int32)
        ids = np.ascontiguousarray(np.concatenate([np.asarray(c, np.int32) for c in candidates]), dtype=np.int32)
        out = np.zeros((len(candidates), head.shape[0]), np.float32) if self.rank == 0 else None
        rank_of = np.zeros(len(candidates), np.int32)
        L.check(L.load().s1_dispatch_candidates(self.handle, model.handle, prefix.handle, ids.ctypes.data_as(C.c_void_p),
                                                lengths.ctypes.data_as(C.c_void_p), len(candidates),
                                                head.ctypes.data_as(C.c_void_p),
                                                None if b is None else b.ctypes.data_as(C.c_void_p), head.shape[0],
                                                None if out is None else out.ctypes.data_as(C.c_void_p),
                                                rank_of.ctypes.data_as(C.c_void_p)), "dispatch candidates")
        return out, rank_of

    def barrier(self):
        L.check(L.load().s1_dispatch_barrier(self.handle), "dispatch barrier")

    def max_over_ranks(self, x):
        v = np.array([float(x)], np.float64)
        L.check(L.load().s1_dispatch_allreduce_max(self.handle, v.ctypes.data_as(C.c_void_p), 1), "dispatch max")
        return float(v[0])

    def allgather(self, values):
        v = np.ascontiguousarray(values, dtype=np.float64).ravel()
        out = np.zeros((self.world, v.size), np.float64)
        L.check(L.load().s1_dispatch_allgather(self.handle, v.ctypes.data_as(C.c_void_p), v.size,
                                               out.ctypes.data_as(C.c_void_p)), "dispatch allgather")
        return out


def run_sharded(requests, forward, n_classes, rank, world, gather=None, a=1.0, b=4e-6, speed=None):
    """The dispatcher's plan with a caller-supplied forward and gather.

    forward(list_of_requests) -> float32 [n, n_classes] logits of one pack on this rank.
    gather(block: float32 [most * n_classes]) -> list of every rank's block (an all-gather).
    Every rank calls this with the same `requests`; rank 0 gets float32 [len(requests), n_classes]
    in request order, other ranks get None. With world == 1 no communication happens.
    """
    lengths = np.array([len(r) for r in requests], np.int32)
    rank_of, mine, packs = layout(lengths, world, rank, a, b, speed)
    local = np.zeros((len(mine), n_classes), np.float32)
    for group in packs:
        idx = list(group)
        local[idx] = forward([requests[mine[j]] for j in idx])
    if world == 1:
        out = np.zeros((len(requests), n_classes), np.float32)
        out[mine] = local
        return out
    most = int(np.bincount(rank_of, minlength=world).max())
    block = np.zeros(most * n_classes, np.float32)
    block[: local.size] = local.ravel()
    gathered = gather(block)
    if rank != 0:
        return None
    out = np.zeros((len(requests), n_classes), np.float32)
    for r in range(world):
        theirs = layout(lengths, world, r, a, b, speed)[1]
        out[theirs] = np.asarray(gathered[r], np.float32).reshape(most, n_classes)[: len(theirs)]
    return out
