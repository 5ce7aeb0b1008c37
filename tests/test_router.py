"""Request -> GPU router (include/glinthawk_router.h) against the reference's bookkeeping rules
(src/compute/routerman.hh:295-331, src/compute/common.hh:44-104).  Host-only."""
import threading

import numpy as np
import pytest

from glinthawk_b200 import _lib
from glinthawk_b200.router import BALANCED, POSITION, ContextRouter
from glinthawk_b200.stage import GlinthawkAttnError
from glinthawk_b200.workload import WORKLOADS, assign_contexts


def test_position_policy_is_the_references_slicing():
    """SliceConcurrency::tier_rank for one tier of n nodes with equal attention concurrency: batch index i belongs to
    node i / concurrency, and the cutting plan is that many prompts per node."""
    r = ContextRouter(8, 32, 64)
    ids = np.arange(1000, 1256)
    ranks = r.assign_ranks(ids)
    assert (ranks == np.arange(256) // 32).all()
    order, counts = r.cut(ranks)
    assert (counts == 32).all() and (order == np.arange(256)).all()
    free, _ = r.loads()
    assert (free == 32).all()


def test_context_availability_follows_the_free_slots():
    """ParentTierRouter::is_context_available: true while every node has at least its share of a batch free."""
    r = ContextRouter(4, 8, 20)
    assert r.is_context_available()
    r.assign_ranks(np.arange(32))
    assert r.is_context_available()  # 12 free each, 8 needed
    r.assign_ranks(np.arange(32, 64))
    assert not r.is_context_available()  # 4 free each
    # a short batch may still go in as long as its ranks have room ...
    ranks = r.assign_ranks(np.arange(64, 68))
    assert (ranks == 0).all()
    # ... and a full one is refused without touching anything
    before = r.loads()[0].copy()
    with pytest.raises(GlinthawkAttnError) as e:
        r.assign_ranks(np.arange(100, 132))
    assert e.value.status == _lib.GH_ERR_NO_SLOT
    assert (r.loads()[0] == before).all()
    with pytest.raises(GlinthawkAttnError) as e:
        r.lookup(100)
    assert e.value.status == _lib.GH_ERR_NOT_FOUND
    # finished prompts make room again (the reference never releases)
    r.release(np.arange(32))
    assert r.is_context_available()
    assert (r.assign_ranks(np.arange(100, 132)) == np.arange(32) // 8).all()


def test_a_prompt_keeps_its_rank():
    """assign_ranks only touches prompts that are not routed yet (routerman.hh:316-328): a prompt that comes back at
    another batch position stays where its KV is, and takes no second slot."""
    r = ContextRouter(4, 4, 16, BALANCED)
    first = r.assign_ranks(np.arange(16), np.full(16, 100))
    free0 = r.loads()[0].copy()
    perm = np.random.default_rng(0).permutation(16)
    again = r.assign_ranks(np.arange(16)[perm], np.full(16, 999))
    assert (again == first[perm]).all()
    assert (r.loads()[0] == free0).all()
    assert all(r.lookup(i) == first[i] for i in range(16))
    # a batch that mixes old and new prompts: the new ones fill what is left of each rank's slice
    r.release([0, 5])
    mixed = r.assign_ranks([1, 2, 3, 4, 100, 6, 7, 8, 9, 10, 11, 12, 13, 14, 15, 101], np.full(16, 100))
    _, counts = r.cut(mixed)
    assert (counts == 4).all()
    assert {int(mixed[4]), int(mixed[15])} == {int(first[0]), int(first[5])}


def test_balanced_policy_evens_out_cached_tokens():
    """Contexts of the headline workload's length distribution on 8 ranks: equal prompt counts per rank, and a
    largest token load close to the mean (the position policy is off by what the draw happens to give)."""
    lens = WORKLOADS["llama2_70b_gqa"].lengths(20240)
    ids = np.arange(256)
    bal, pos = ContextRouter(8, 32, 64, BALANCED), ContextRouter(8, 32, 64, POSITION)
    rb, rp = bal.assign_ranks(ids, lens), pos.assign_ranks(ids, lens)
    assert (np.bincount(rb, minlength=8) == 32).all() and (np.bincount(rp, minlength=8) == 32).all()
    tb, tp = bal.loads()[1].astype(np.int64), pos.loads()[1].astype(np.int64)
    assert tb.sum() == tp.sum() == int(lens.sum())
    assert tb.max() <= 1.02 * tb.mean()
    assert tb.max() <= tp.max()
    # next to the unconstrained longest-first placement of a fixed set (no equal-count rule): within a few percent
    lpt = max(int(lens[idx].sum()) for idx in assign_contexts(lens, 8))
    assert tb.max() <= 1.03 * lpt
    # the loads follow the prompts as they grow and leave
    bal.note_tokens(ids, lens + 10)
    assert bal.loads()[1].sum() == int(lens.sum()) + 2560
    bal.release(ids[rb == 3])
    assert bal.loads()[1][3] == 0 and bal.loads()[0][3] == 64


def test_new_prompts_go_where_the_load_is_lowest():
    r = ContextRouter(2, 2, 8, BALANCED)
    assert list(r.assign_ranks([1, 2, 3, 4], [4000, 10, 10, 10])) == [0, 1, 1, 0]
    r.note_tokens([2, 3], [3000, 3000])  # rank 1 now holds 6000 tokens against 4010
    # the lighter rank takes new prompts until its slice of the batch is full, the rest go elsewhere
    assert list(r.assign_ranks([5, 6, 7], [500, 400, 300])) == [0, 0, 1]
    assert list(r.loads()[1]) == [4910, 6300]


def test_two_routers_fed_the_same_calls_agree():
    """No communication between the ranks of a box: every process replays the same calls."""
    rng = np.random.default_rng(5)
    a, b = ContextRouter(8, 16, 40, BALANCED), ContextRouter(8, 16, 40, BALANCED)
    live: list[int] = []
    nxt = 0
    for _ in range(30):
        n_new = int(rng.integers(1, 64))
        ids = np.arange(nxt, nxt + n_new)
        lens = rng.integers(16, 4096, n_new)
        try:
            ra = a.assign_ranks(ids, lens)
        except GlinthawkAttnError:
            with pytest.raises(GlinthawkAttnError):
                b.assign_ranks(ids, lens)
        else:
            assert (ra == b.assign_ranks(ids, lens)).all()
            live += list(ids)
            nxt += n_new
        gone = [live.pop(int(rng.integers(len(live)))) for _ in range(min(len(live), int(rng.integers(0, 40))))]
        a.release(gone)
        b.release(gone)
        assert all((x == y).all() for x, y in zip(a.loads(), b.loads()))
    free, tokens = a.loads()
    assert int((40 - free).sum()) == len(live)


def test_bad_calls_are_refused_and_change_nothing():
    with pytest.raises(GlinthawkAttnError):
        ContextRouter(0, 4, 4)
    with pytest.raises(GlinthawkAttnError):
        ContextRouter(4, 0, 4)
    with pytest.raises(GlinthawkAttnError):
        ContextRouter(4, 4, 4, policy=7)
    r = ContextRouter(2, 2, 4)
    for bad in ([1, 1], [1, 2, 3, 4, 5]):  # the same prompt twice; more than a full batch
        with pytest.raises(GlinthawkAttnError) as e:
            r.assign_ranks(bad)
        assert e.value.status == _lib.GH_ERR_INVALID
    assert (r.loads()[0] == 4).all()
    r.assign_ranks([1, 2])
    for bad in ([1, 9], [1, 1]):
        with pytest.raises(GlinthawkAttnError) as e:
            r.release(bad)
        assert e.value.status == _lib.GH_ERR_NOT_FOUND
    with pytest.raises(GlinthawkAttnError):
        r.note_tokens([9], [5])
    assert list(r.loads()[0]) == [2, 4]
    with pytest.raises(GlinthawkAttnError):
        r.cut([0, 2])


def test_threads_share_one_router():
    """One mutex, like the reference's ctx_mutex_: admission on one thread, releases on another."""
    r = ContextRouter(4, 8, 4096)
    errors: list[Exception] = []

    def admit(base):
        try:
            for k in range(100):
                r.assign_ranks(np.arange(base + 32 * k, base + 32 * k + 32))
        except Exception as e:  # pragma: no cover
            errors.append(e)

    ts = [threading.Thread(target=admit, args=(b,)) for b in (0, 10_000, 20_000, 30_000)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    assert not errors
    assert (r.loads()[0] == 4096 - 3200).all()
    r.release(np.concatenate([np.arange(b, b + 3200) for b in (0, 10_000, 20_000, 30_000)]))
    assert (r.loads()[0] == 4096).all()
