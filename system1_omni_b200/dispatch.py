"""Request sharding across the GPUs of one box: replicated weights, whole requests per rank,
one small gather of decision logits. The reference serves from a single device
(src/models/qwen3_5/native/src/model.rs:625 pins device 0), so this layer has no counterpart
there; per-request results must equal single-GPU execution, which the tests check.

One process per GPU. `torch.distributed` is used for the gather only (backend nccl on GPUs,
gloo in the CPU tests); the forward pass itself never communicates.
"""
import numpy as np

from . import model as M


def shard(lengths, world, a=1.0, b=0.0):
    """rank_of[i] for every request: longest processing time first on cost a*T + b*T^2."""
    return M.assign_requests(lengths, world, a, b)


def packs(lengths):
    """Order-preserving groups of at most 16 prompts / 4096 tokens (the reference's pack limits)."""
    return M.ranges(lengths)


def run_sharded(requests, forward, n_classes, rank, world, dist=None, device=None, a=1.0, b=0.0):
    """Run `requests` (lists of token ids) across `world` ranks.

    forward(list_of_requests) -> float32 [n, n_classes] logits on this rank's GPU/host.
    Every rank calls this with the same `requests`; rank 0 gets float32 [len(requests), n_classes]
    in request order, other ranks get None. With world == 1 no communication happens.
    """
    lengths = np.array([len(r) for r in requests], np.int32)
    rank_of = shard(lengths, world, a, b)
    mine = [i for i in range(len(requests)) if rank_of[i] == rank]
    local = np.zeros((len(mine), n_classes), np.float32)
    my_lengths = [len(requests[i]) for i in mine]
    for group in packs(my_lengths):
        idx = list(group)
        local[idx] = forward([requests[mine[j]] for j in idx])
    if world == 1:
        return local
    import torch
    # a fixed-size block per rank: [count, logits...] padded to the largest share
    most = int(np.bincount(rank_of, minlength=world).max())
    block = torch.zeros(most * n_classes, dtype=torch.float32)
    block[: local.size] = torch.from_numpy(local.ravel())
    if device is not None:
        block = block.to(device)
    gathered = [torch.zeros_like(block) for _ in range(world)]
    dist.all_gather(gathered, block)
    if rank != 0:
        return None
    out = np.zeros((len(requests), n_classes), np.float32)
    for r in range(world):
        theirs = [i for i in range(len(requests)) if rank_of[i] == r]
        rows = gathered[r].cpu().numpy().reshape(most, n_classes)[: len(theirs)]
        out[theirs] = rows
    return out
