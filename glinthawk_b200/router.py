"""Request -> GPU assignment on the GPUs of one box (include/glinthawk_router.h): which rank's slot pool holds a
prompt's KV.  The reference's counterpart is the tier router's bookkeeping (src/compute/routerman.hh:295-331,
src/compute/common.hh:44-104).  Host-only."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from ._lib import lib
from .stage import GlinthawkAttnError

POSITION, BALANCED = _lib.GH_ROUTE_POSITION, _lib.GH_ROUTE_BALANCED


def _p(a: np.ndarray | None) -> C.c_void_p:
    return C.c_void_p(0 if a is None else a.ctypes.data)


class ContextRouter:
    """``n_ranks`` GPUs, each serving ``per_rank_batch`` prompts of a full batch out of ``slots_per_rank`` slots."""

    def __init__(self, n_ranks: int, per_rank_batch: int, slots_per_rank: int, policy: int = POSITION):
        self._h = None
        h = C.c_void_p()
        rc = lib.gh_router_create(C.byref(h), n_ranks, per_rank_batch, slots_per_rank, policy)
        if rc != _lib.GH_OK:
            raise GlinthawkAttnError(rc, "gh_router_create")
        self._h, self.n_ranks, self.per_rank_batch = h, n_ranks, per_rank_batch

    def close(self) -> None:
        if self._h:
            lib.gh_router_destroy(self._h)
            self._h = None

    def __del__(self):
        self.close()

    @staticmethod
    def _ck(rc: int, what: str) -> None:
        if rc != _lib.GH_OK:
            raise GlinthawkAttnError(rc, what)

    def is_context_available(self) -> bool:
        """ParentTierRouter::is_context_available: room for one more full batch on every rank."""
        return lib.gh_router_is_context_available(self._h) == 1

    def assign_ranks(self, prompt_ids, expected_tokens=None) -> np.ndarray:
        """ParentTierRouter::assign_ranks for one batch; prompts that already have a rank keep it."""
        ids = np.ascontiguousarray(prompt_ids, dtype=np.uint64)
        tok = None if expected_tokens is None else np.ascontiguousarray(expected_tokens, dtype=np.uint32)
        assert tok is None or tok.shape == ids.shape
        ranks = np.zeros(len(ids), dtype=np.uint32)
        self._ck(lib.gh_router_assign_ranks(self._h, len(ids), _p(ids), _p(tok), _p(ranks)), "gh_router_assign_ranks")
        return ranks

    def lookup(self, prompt_id: int) -> int:
        rank = C.c_uint32(0)
        self._ck(lib.gh_router_lookup(self._h, prompt_id, C.byref(rank)), "gh_router_lookup")
        return rank.value

    def note_tokens(self, prompt_ids, cached_tokens) -> None:
        ids = np.ascontiguousarray(prompt_ids, dtype=np.uint64)
        tok = np.ascontiguousarray(cached_tokens, dtype=np.uint32)
        assert tok.shape == ids.shape
        self._ck(lib.gh_router_note_tokens(self._h, len(ids), _p(ids), _p(tok)), "gh_router_note_tokens")

    def release(self, prompt_ids) -> None:
        ids = np.ascontiguousarray(prompt_ids, dtype=np.uint64)
        self._ck(lib.gh_router_release(self._h, len(ids), _p(ids)), "gh_router_release")

    def loads(self) -> tuple[np.ndarray, np.ndarray]:
        """(free slots, cached tokens) per rank."""
        free, tok = np.zeros(self.n_ranks, dtype=np.uint32), np.zeros(self.n_ranks, dtype=np.uint64)
        self._ck(lib.gh_router_loads(self._h, _p(free), _p(tok)), "gh_router_loads")
        return free, tok

    def cut(self, ranks) -> tuple[np.ndarray, np.ndarray]:
        """A batch cut into per-rank shards: (batch indices grouped by rank, prompts per rank)."""
        ranks = np.ascontiguousarray(ranks, dtype=np.uint32)
        order, counts = np.zeros(len(ranks), dtype=np.uint32), np.zeros(self.n_ranks, dtype=np.uint32)
        self._ck(lib.gh_router_cut(self.n_ranks, len(ranks), _p(ranks), _p(order), _p(counts)), "gh_router_cut")
        return order, counts
