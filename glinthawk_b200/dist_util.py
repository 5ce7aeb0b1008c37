"""Multi-process helpers: one process per GPU, contexts sharded by request, no collective on the attention path.

``torch.distributed`` is used for exactly two things: a barrier around timed regions and the maximum over ranks
of a device-measured duration.  Everything here also runs on CPU ranks (gloo), which is how it is tested.
"""
from __future__ import annotations

import os

import numpy as np
import torch
import torch.distributed as dist

from .workload import Workload, assign_contexts


def rank_world() -> tuple[int, int, int]:
    return (int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")),
            int(os.environ.get("LOCAL_RANK", "0")))


def max_over_ranks(value: float, device: torch.device | str = "cpu") -> float:
    """The slowest rank decides: every multi-GPU duration is reported as the maximum over ranks."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(value)
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sum_over_ranks(value: float, device: torch.device | str = "cpu") -> float:
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(value)
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


def weak_scaling_lengths(wl: Workload, seed: int, rank: int, headroom: int, batch: int | None = None) -> np.ndarray:
    """Weak scaling: every rank serves its own contexts, and the per-GPU work is exactly the same on every rank —
    the same multiset of cached lengths (so that the maximum over ranks measures the machine, not the luck of
    the draw), in a rank-specific order; the cached values themselves differ by rank (seeded by the caller)."""
    lens = wl.lengths(seed, headroom)[: batch or wl.batch]
    return np.random.default_rng(seed + 7919 * (rank + 1)).permutation(lens) if rank > 0 else lens


def strong_scaling_lengths(wl: Workload, seed: int, rank: int, world: int, headroom: int) -> tuple[np.ndarray, np.ndarray]:
    """One fixed set of requests divided among the ranks: returns (global indices, lengths) of this rank's share.
    Every rank computes the same assignment from the same seed, so no communication is needed."""
    lens = wl.lengths(seed, headroom)
    mine = assign_contexts(lens, world)[rank]
    return mine, lens[mine]


def strong_share_on_local_contexts(lens_global, lens_local, share_of: int, n_shares: int) -> np.ndarray:
    """A rank that already holds its own copy of the request set in another order (weak_scaling_lengths gives every
    rank the same multiset of lengths, permuted) picks, among its local contexts, the ones that stand for share
    `share_of` of the fixed request set divided `n_shares` ways: the k-th shortest local context stands for the k-th
    shortest request.  Returns sorted local indices; their lengths are exactly the share's lengths."""
    lens_global, lens_local = np.asarray(lens_global), np.asarray(lens_local)
    mine = assign_contexts(lens_global, n_shares)[share_of]
    order_global = np.argsort(lens_global, kind="stable")
    order_local = np.argsort(lens_local, kind="stable")
    place = np.empty(len(lens_global), dtype=np.int64)
    place[order_global] = np.arange(len(lens_global))
    return np.sort(order_local[place[mine]])
