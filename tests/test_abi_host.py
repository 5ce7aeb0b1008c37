"""CPU-only checks of the drop-in boundary: the shared library loads without a GPU, exports every symbol the
public header declares, reports errors as status codes, and its host-side planner behaves."""
import ctypes as C

import numpy as np
import pytest
import torch

from glinthawk_b200 import _lib
from glinthawk_b200.shapes import SHAPES
from glinthawk_b200.stage import GlinthawkAttnError, plan_batch, plan_projection


def test_library_exports_every_declared_symbol():
    names = _lib.declared_symbols()
    assert len(names) >= 27
    for n in names:
        assert hasattr(_lib.lib, n), f"{n} is declared in include/glinthawk_attn.h but not exported"
    assert set(names) == set(_lib._PROTOS), "binding table and header disagree"


def test_status_strings():
    assert _lib.lib.gh_status_string(0) == b"ok"
    assert b"slot" in _lib.lib.gh_status_string(_lib.GH_ERR_NO_SLOT)


def test_create_rejects_bad_config():
    h = C.c_void_p(0)
    cfg = _lib.Config(C.sizeof(_lib.Config), 6, 4, 48, 256, 1, _lib.GH_F32, 4, 4, 0, 0, 0, 0, 0, 0)  # 6 % 4 != 0
    assert _lib.lib.gh_attn_create(C.byref(cfg), C.byref(h)) == _lib.GH_ERR_INVALID
    cfg = _lib.Config(C.sizeof(_lib.Config) - 4, 6, 6, 48, 256, 1, _lib.GH_F32, 4, 4, 0, 0, 0, 0, 0, 0)
    assert _lib.lib.gh_attn_create(C.byref(cfg), C.byref(h)) == _lib.GH_ERR_INVALID
    cfg = _lib.Config(C.sizeof(_lib.Config), 6, 6, 48, 256, 1, _lib.GH_F32, 4096, 4, 0, 0, 0, 0, 0, 0)  # batch > 1024
    assert _lib.lib.gh_attn_create(C.byref(cfg), C.byref(h)) == _lib.GH_ERR_INVALID


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the behaviour on a machine without a GPU")
def test_create_without_gpu_fails_loudly():
    """No CPU fallback: without a device the stage cannot be created."""
    h = C.c_void_p(0)
    cfg = _lib.Config(C.sizeof(_lib.Config), 6, 6, 48, 256, 1, _lib.GH_F32, 4, 4, 0, 0, 0, 0, 0, 0)
    assert _lib.lib.gh_attn_create(C.byref(cfg), C.byref(h)) == _lib.GH_ERR_CUDA
    assert not h.value


def test_null_handle_is_an_error_not_a_crash():
    assert _lib.lib.gh_attn_destroy(None) == _lib.GH_ERR_INVALID
    assert _lib.lib.gh_attn_last_error(None) == b"null handle"
    s = C.c_int32(0)
    assert _lib.lib.gh_slot_acquire(None, 1, C.byref(s)) == _lib.GH_ERR_INVALID


def _check_plan(pos, items, chunk, tile):
    pos = np.asarray(pos, dtype=np.int64)
    covered = {i: [] for i in range(len(pos))}
    for ctx, b, e, split in items:
        assert 0 <= b < e
        assert b % tile == 0, "split boundaries must sit on tile multiples"
        covered[ctx].append((b, e, split))
    for i, p in enumerate(pos):
        if p == 0xFFFFFFFF:
            assert covered[i] == []
            continue
        segs = sorted(covered[i])
        assert segs[0][0] == 0 and segs[-1][1] == p + 1
        for (b0, e0, s0), (b1, e1, s1) in zip(segs, segs[1:]):
            assert e0 == b1 and s1 == s0 + 1
        assert all(e - b <= chunk for b, e, _ in segs)
    lens = [e - b for _, b, e, _ in items]
    assert lens == sorted(lens, reverse=True), "items must be ordered longest first"


def test_plan_covers_every_token_exactly_once():
    rng = np.random.default_rng(0)
    pos = rng.integers(0, 4096, size=256).astype(np.uint32)
    for fixed in (0, 64, 320, 1024):
        items, chunk = plan_batch(pos, blocks_per_item=8, fixed_chunk=fixed)
        _check_plan(pos, items, chunk, 64)
        assert chunk % 64 == 0


def test_plan_edge_cases():
    items, chunk = plan_batch([0], blocks_per_item=8)
    assert items.tolist() == [[0, 0, 1, 0]]
    items, chunk = plan_batch([0xFFFFFFFF, 5, 0xFFFFFFFF], blocks_per_item=1)
    assert items.tolist() == [[1, 0, 6, 0]]
    items, chunk = plan_batch([0xFFFFFFFF] * 4, blocks_per_item=1)
    assert len(items) == 0
    # a fixed split length is honoured (rounded to the tile) and splits are balanced
    items, chunk = plan_batch([1000], blocks_per_item=8, fixed_chunk=300)
    assert chunk == 320
    _check_plan([1000], items, chunk, 64)
    assert len(items) == 4
    # a tiny item buffer forces longer splits instead of failing
    pos = np.full(8, 4095, dtype=np.uint32)
    items, chunk = plan_batch(pos, blocks_per_item=8, fixed_chunk=64, max_items=16)
    assert len(items) <= 16
    _check_plan(pos, items, chunk, 64)
    # more active contexts than items: refused
    with pytest.raises(Exception):
        plan_batch(np.zeros(32, dtype=np.uint32), blocks_per_item=1, max_items=16)


def test_plan_cuts_contexts_only_when_it_pays():
    # plenty of contexts for every block slot: cutting would only add per-item overhead
    pos = np.random.default_rng(1).integers(15, 4096, size=256).astype(np.uint32)
    items, chunk = plan_batch(pos, blocks_per_item=8)
    assert len(items) == 256 and chunk >= pos.max() + 1
    _check_plan(pos, items, chunk, 64)
    # one long context alone on the GPU: cut down to the minimum split length
    items, chunk = plan_batch([4095], blocks_per_item=8)
    assert chunk == 256 and len(items) == 16
    # a few long contexts among short ones: the long ones are cut, the plan stays valid
    pos = np.array([4095, 4000, 100, 50, 20, 3000], dtype=np.uint32)
    items, chunk = plan_batch(pos, blocks_per_item=8)
    assert 256 <= chunk < 4096
    _check_plan(pos, items, chunk, 64)


@pytest.mark.parametrize("shape_name", ["mini_mha", "mini_g4", "mini_g16", "l7b_4k", "l70b_4k", "l3_8b_8k", "l3_405b"])
@pytest.mark.parametrize("sm_count", [148, 132, 1, 7])
def test_projection_work_is_dealt_completely_and_evenly(shape_name, sm_count):
    """The fused projection deals (feature tile, k-block) units to the CTAs as contiguous runs.  Every unit must be
    covered exactly once, the runs must differ by at most one unit's worth, and the piece numbering the finishing
    kernel relies on (piece index within its tile, pieces per tile, bounded by max_segs) must be consistent."""
    sh = SHAPES[shape_name]
    plan, pieces = plan_projection(sh, sm_count=sm_count, max_pieces=1 << 16)
    n_tiles, kb = plan["n_tiles"], plan["kblocks"]
    assert n_tiles == (sh.dim + 2 * sh.kv_dim) // 128 and kb == sh.dim // 64
    assert plan["ctas"] <= sm_count
    covered = np.zeros((n_tiles, kb), dtype=np.int32)
    per_cta = np.zeros(plan["ctas"], dtype=np.int64)
    seen = {}
    for cta, tile, k0, k1, seg, nsegs in pieces:
        assert 0 <= k0 < k1 <= kb and 0 <= seg < nsegs <= plan["max_segs"]
        covered[tile, k0:k1] += 1
        per_cta[cta] += k1 - k0
        seen.setdefault(tile, []).append((k0, k1, seg, nsegs))
    assert (covered == 1).all(), "every (tile, k-block) unit exactly once"
    assert per_cta.max() == plan["units_per_cta"] and per_cta.sum() == n_tiles * kb
    assert (per_cta[:-1] == plan["units_per_cta"]).all(), "only the last CTA may run short"
    for tile, segs in seen.items():
        segs.sort()
        assert [s[2] for s in segs] == list(range(len(segs))), "pieces are numbered in k order"
        assert all(s[3] == len(segs) for s in segs), "every piece knows how many pieces its tile has"
    # the order inside a CTA is the order of the units
    for cta in range(plan["ctas"]):
        mine = pieces[pieces[:, 0] == cta]
        start = mine[:, 1] * kb + mine[:, 2]
        assert (np.diff(start) > 0).all()


def test_projection_plan_refuses_shapes_the_kernel_does_not_take():
    with pytest.raises(GlinthawkAttnError) as e:
        plan_projection(SHAPES["tiny15m"])
    assert e.value.status == _lib.GH_ERR_UNSUPPORTED

