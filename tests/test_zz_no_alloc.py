"""gh_decode_noalloc — the decode entry point for callers that cannot allocate device memory.

Some users of this library run where cudaMalloc is not an option: a worker that handed all of its GPU memory to
weights and context slots at start-up (and treats a failed allocation as fatal), or a serving loop that must not
take the device-wide synchronisation an allocation implies.  For them the library carries its split-K scratch as
a fixed array inside its own image.  This file checks that entry point, through the C ABI, against the regular
fused entry point (gh_op_attention_fused) on the same inputs and against the CPU oracle's layer-step on them —
twice in a row with different batches, because the second call finds the array as the first one left it.  It is
named so that pytest collects it last.
"""
import numpy as np
import pytest
import torch

from glinthawk_b200 import _lib
from glinthawk_b200.stage import GlinthawkAttnError, decode_noalloc
from tests import cases, gpu_util

pytestmark = pytest.mark.gpu


def _both_ways(oracle, shape_name, dtype, pos, seed, inactive=()):
    case = cases.make_case("noalloc", shape_name, dtype, pos, seed, inactive=inactive)
    # The oracle's layer-step appends and rotates first; the attention part of it is what the entry point computes,
    # so the device gets the caches with the oracle's appended rows in place and the oracle's rotated q.
    oracle_step = oracle.layer_step(case)
    host_caches = []
    for c, p, row in zip(case.cache, case.pos, oracle_step.rows):
        c = c.copy()
        if row is not None:
            c[int(p)] = row
        host_caches.append(c)
    caches = [gpu_util.to_dev(c, dtype) for c in host_caches]  # ordinary device buffers: nothing from a slot pool
    bases = [c.data_ptr() if a else 0 for c, a in zip(caches, case.active)]
    q = gpu_util.to_dev(oracle_step.q, dtype)

    stage = gpu_util.make_stage(case)  # the existing entry point needs a handle; the new one does not
    want = torch.zeros_like(q)
    stage.attention_fused(q, bases, want, case.B, case.pos)
    torch.cuda.synchronize()
    stage.close()

    got = torch.zeros_like(q)
    decode_noalloc(case.shape, gpu_util.TORCH_DT[dtype], bases, case.pos, q, got)
    torch.cuda.synchronize()
    return case, got, want, cases.as_f32(oracle_step.xb, dtype)


@pytest.mark.parametrize("shape_name,dtype", [("mini_g8", cases.F16), ("tiny15m", cases.F32), ("mini_g4", cases.BF16)])
def test_noalloc_matches_existing_entry_point_twice_in_a_row(oracle, shape_name, dtype):
    S = cases.SHAPES[shape_name].seq_len
    # first call: long contexts, so several are cut into work items and leave partial records and counters behind
    first = [S - 1, S - 2, 300 % S, 0, S // 2]
    # second call: a different batch size and different lengths on top of the stale scratch
    second = [5, S - 1, 64, 63, 129 % S, S - 3, 1]
    for pos, seed, inactive in ((first, 1, ()), (second, 2, (2,))):
        case, got, want, oracle_xb = _both_ways(oracle, shape_name, dtype, pos, seed, inactive)
        tol = cases.TOL_XB[dtype]
        for i in range(case.B):
            if case.active[i]:
                np.testing.assert_allclose(got[i].float().cpu().numpy(), want[i].float().cpu().numpy(), rtol=0,
                                           atol=tol, err_msg=f"context {i} against gh_op_attention_fused")
                np.testing.assert_allclose(got[i].float().cpu().numpy(), oracle_xb[i], rtol=0,
                                           atol=tol, err_msg=f"context {i} against the oracle")
            else:
                assert torch.count_nonzero(got[i]) == 0  # inactive prompts are skipped


def test_noalloc_refuses_sizes_beyond_its_limits():
    sh = cases.SHAPES["mini_g8"]
    q = torch.zeros((65, sh.dim), dtype=torch.float16, device="cuda")
    with pytest.raises(GlinthawkAttnError) as e:
        decode_noalloc(sh, torch.float16, [q.data_ptr()] * 65, [0] * 65, q, q.clone())
    assert e.value.status == _lib.GH_ERR_INVALID and "GH_NOALLOC_MAX_BATCH" in str(e.value)
    big = cases.SHAPES["l3_405b"]  # 128 heads x 128 = 16384 query elements
    with pytest.raises(GlinthawkAttnError) as e:
        decode_noalloc(big, torch.float16, [q.data_ptr()], [0], q, q.clone())
    assert "GH_NOALLOC_MAX_Q_ELEMS" in str(e.value)
