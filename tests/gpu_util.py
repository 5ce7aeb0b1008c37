"""Runs a seeded parity case on the GPU through the C ABI (test helper)."""
from __future__ import annotations

import numpy as np
import torch

from glinthawk_b200.stage import AttentionStage
from tests import cases

TORCH_DT = {cases.F16: torch.float16, cases.F32: torch.float32, cases.BF16: torch.bfloat16}


def to_dev(a: np.ndarray, dtype: int) -> torch.Tensor:
    if dtype == cases.BF16:
        return torch.from_numpy(a.view(np.int16)).cuda().view(torch.bfloat16)
    return torch.from_numpy(a).cuda()


def to_host(t: torch.Tensor, dtype: int) -> np.ndarray:
    if dtype == cases.BF16:
        return t.view(torch.int16).cpu().numpy().view(np.uint16)
    return t.cpu().numpy()


def make_stage(case: cases.Case, *, layers: int = 2, paged: bool = False, force_generic: bool = False,
               decode_chunk: int = 0, max_contexts: int | None = None) -> AttentionStage:
    st = AttentionStage(case.shape, TORCH_DT[case.dtype], n_layers_hosted=layers, max_batch=max(case.B, 1),
                        max_contexts=max_contexts or case.B, paged=paged, force_generic=force_generic,
                        decode_chunk=decode_chunk)
    st.set_rope_tables(to_dev(case.fcr, case.dtype), to_dev(case.fci, case.dtype))
    return st


def load_case(st: AttentionStage, case: cases.Case, layer: int, first_id: int = 1) -> np.ndarray:
    """Binds one slot per context (ids first_id..), uploads the pre-filled cache, returns the slots
    (-1 for inactive prompts)."""
    ids = np.array([first_id + i if a else 0 for i, a in enumerate(case.active)], dtype=np.uint32)
    slots = st.get_contexts(ids)
    assert slots is not None
    for i in range(case.B):
        if not case.active[i]:
            assert slots[i] == -1
            continue
        p = int(case.pos[i])
        st.prepare(int(slots[i]), layer, p, False)
        if p > 0:
            st.layer_view(int(slots[i]), layer, p).copy_(to_dev(case.cache[i][:p], case.dtype))
    return slots


def run_step(st: AttentionStage, case: cases.Case, slots, layer: int, *, fused_call: bool = True) -> cases.StepResult:
    q = to_dev(case.q, case.dtype)
    kv = to_dev(case.kv_new, case.dtype)
    xb = torch.zeros_like(q)
    st.batch_begin(slots, case.pos)
    if fused_call:
        st.step(layer, q, kv, xb)
    else:
        st.append(layer, q, kv)
        st.decode(layer, q, xb)
    torch.cuda.synchronize()
    rows = []
    for i in range(case.B):
        if not case.active[i]:
            rows.append(None)
            continue
        p = int(case.pos[i])
        rows.append(to_host(st.layer_view(int(slots[i]), layer, p + 1)[p], case.dtype))
    assert st.stats().device_error == 0
    return cases.StepResult(rows, to_host(q, case.dtype), to_host(xb, case.dtype))


def assert_step_close(res: cases.StepResult, want: cases.StepResult, case: cases.Case, *, xb_atol=None) -> None:
    kvd = case.shape.kv_dim
    atol = cases.TOL_XB[case.dtype] if xb_atol is None else xb_atol
    for i in range(case.B):
        if not case.active[i]:
            continue
        got_row, want_row = np.asarray(res.rows[i]), np.asarray(want.rows[i])
        assert np.array_equal(got_row[kvd:].view(np.uint8), want_row[kvd:].view(np.uint8)), "V must be bit-exact"
        np.testing.assert_allclose(cases.as_f32(got_row[:kvd], case.dtype), cases.as_f32(want_row[:kvd], case.dtype),
                                   rtol=cases.TOL_K_REL, atol=1e-3, err_msg=f"rotated K, context {i}")
        np.testing.assert_allclose(cases.as_f32(res.q[i], case.dtype), cases.as_f32(want.q[i], case.dtype),
                                   rtol=cases.TOL_K_REL, atol=1e-3, err_msg=f"rotated q, context {i}")
        np.testing.assert_allclose(cases.as_f32(res.xb[i], case.dtype), cases.as_f32(want.xb[i], case.dtype), rtol=0,
                                   atol=atol, err_msg=f"attention output, context {i}")
