"""Runs a seeded parity case on the GPU through the C ABI (test helper)."""
from __future__ import annotations

import numpy as np
import torch

from glinthawk_b200._lib import GH_ERR_CAPACITY  # noqa: F401  (re-exported for the tests)
from glinthawk_b200.stage import AttentionStage, GlinthawkAttnError  # noqa: F401
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


def _ordered(x: np.ndarray, dtype: int) -> np.ndarray:
    """Storage bit patterns as integers whose difference counts representable values between two numbers."""
    if dtype == cases.F32:
        b = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.int64)
        mag, sign = b & 0x7FFFFFFF, b >> 31
    else:
        b = np.ascontiguousarray(x).view(np.uint16).astype(np.int64)
        mag, sign = b & 0x7FFF, b >> 15
    return np.where(sign == 1, -mag, mag)


def assert_rotation_close(got, want, unrotated, dtype: int, what: str) -> None:
    """The rotation is computed in fp32 and rounded once to the storage type, on the device as in the reference
    (src/arch/amd64/llama2/ops.hh:150-162), so a rotated value may differ from the reference's by at most one unit
    in the last place of the STORAGE type (both sides round the same fp32 value, or two that straddle a rounding
    boundary).  The one thing that can move the fp32 value itself is the order of its three roundings (a compiler
    may fuse x0*c - x1*s into one multiply-add): that is worth 2^-22 of the larger operand of the pair, which only
    shows where the two products nearly cancel."""
    got, want = np.asarray(got), np.asarray(want)
    ulps = np.abs(_ordered(got, dtype) - _ordered(want, dtype))
    x = np.abs(cases.as_f32(np.asarray(unrotated), dtype)).reshape(-1, 2)
    slack = np.repeat(x.max(axis=1), 2).reshape(got.shape) * np.float32(2.0 ** -22)
    diff = np.abs(cases.as_f32(got, dtype).astype(np.float64) - cases.as_f32(want, dtype).astype(np.float64))
    bad = (ulps > 1) & (diff > slack)
    assert not bad.any(), (f"{what}: {int(bad.sum())} of {bad.size} values differ by more than one unit in the last "
                           f"place (worst {int(ulps[bad].max())} ulps, |diff| {diff[bad].max():.3g})")


def assert_step_close(res: cases.StepResult, want: cases.StepResult, case: cases.Case, *, xb_atol=None) -> None:
    kvd = case.shape.kv_dim
    atol = cases.TOL_XB[case.dtype] if xb_atol is None else xb_atol
    for i in range(case.B):
        if not case.active[i]:
            continue
        got_row, want_row = np.asarray(res.rows[i]), np.asarray(want.rows[i])
        assert np.array_equal(got_row[kvd:].view(np.uint8), want_row[kvd:].view(np.uint8)), "V must be bit-exact"
        assert_rotation_close(got_row[:kvd], want_row[:kvd], case.kv_new[i][:kvd], case.dtype, f"rotated K, context {i}")
        assert_rotation_close(res.q[i], want.q[i], case.q[i], case.dtype, f"rotated q, context {i}")
        np.testing.assert_allclose(cases.as_f32(res.xb[i], case.dtype), cases.as_f32(want.xb[i], case.dtype), rtol=0,
                                   atol=atol, err_msg=f"attention output, context {i}")


def _exact_causal_attention(sh, dtype, pos0, q_rot, cache):
    """Softmax attention in float64 over the given rotated queries [B][T][dim] and cache rows, every token seeing the
    keys up to its own position."""
    B, T = q_rot.shape[:2]
    out = np.zeros(q_rot.shape, dtype=np.float64)
    group, hs = sh.n_heads // sh.n_kv_heads, sh.head_size
    for i, p in enumerate(pos0):
        rows = cases.as_f32(cache[i][:p + T], dtype).astype(np.float64)
        k = rows[:, :sh.kv_dim].reshape(-1, sh.n_kv_heads, hs)
        v = rows[:, sh.kv_dim:].reshape(-1, sh.n_kv_heads, hs)
        qi = cases.as_f32(q_rot[i], dtype).astype(np.float64).reshape(T, sh.n_heads, hs)
        visible = np.arange(p + T)[None, :] <= (p + np.arange(T))[:, None]
        for h in range(sh.n_heads):
            s = qi[:, h] @ k[:, h // group].T / np.sqrt(hs)
            s = np.where(visible, s, -np.inf)
            w = np.exp(s - s.max(axis=1, keepdims=True))
            out[i, :, h * hs:(h + 1) * hs] = (w / w.sum(axis=1, keepdims=True)) @ v[:, h // group]
    return out


def check_prefill(oracle, shape_name, dtype, pos0, chunk_lens, k_ramp=0.0, seed=321, exact_attention=False):
    """Feeds `chunk_lens` consecutive prompt chunks to contexts whose slots already hold `pos0[i]` tokens, and
    compares everything the calls leave behind with token-by-token reference layer-steps on a growing cache.
    `k_ramp` > 0 scales the new K rows by (1 + k_ramp * position): the scores then grow along the keys by far more
    than the kernel lets a row's running maximum lag, so the accumulator is rescaled again and again.
    `exact_attention` replaces the reference's attention output by the exact softmax over the reference's own
    rotated queries and cache rows (the appended rows and q are still held to the reference's)."""
    sh = cases.SHAPES[shape_name]
    T = int(sum(chunk_lens))
    rng = np.random.default_rng(seed)
    B = len(pos0)
    base = cases.make_case("pf", shape_name, dtype, [p + T - 1 for p in pos0], seed=9)
    q = cases.store(rng.standard_normal((B, T, sh.dim), dtype=np.float32), dtype)
    kv32 = rng.standard_normal((B, T, 2 * sh.kv_dim), dtype=np.float32)
    if k_ramp:
        for i, p in enumerate(pos0):
            kv32[i, :, :sh.kv_dim] *= (1.0 + k_ramp * (p + np.arange(T, dtype=np.float32)))[:, None]
    kv = cases.store(kv32, dtype)

    # oracle: token by token
    cache = [c.copy() for c in base.cache]
    want_xb = np.zeros_like(q)
    want_q = np.zeros_like(q)
    for t in range(T):
        step = cases.Case("pf", sh, dtype, np.array([p + t for p in pos0], dtype=np.uint32), base.active,
                          [c[: p + t + 1] for c, p in zip(cache, pos0)], np.ascontiguousarray(q[:, t]),
                          np.ascontiguousarray(kv[:, t]), base.fcr, base.fci)
        res = oracle.layer_step(step)
        for i, p in enumerate(pos0):
            cache[i][p + t] = res.rows[i]
        want_xb[:, t], want_q[:, t] = res.xb, res.q

    want_xb = cases.as_f32(want_xb, dtype)
    if exact_attention:
        want_xb = _exact_causal_attention(sh, dtype, pos0, want_q, cache)

    st = make_stage(base, layers=2, paged=True)
    slots = st.get_contexts(np.arange(1, B + 1, dtype=np.uint32))
    for i, p in enumerate(pos0):
        st.prepare(int(slots[i]), 1, max(p, 1) - 1, False)
        if p > 0:
            st.layer_view(int(slots[i]), 1, p).copy_(to_dev(base.cache[i][:p], dtype))
    got_xb, got_q = np.zeros_like(q), np.zeros_like(q)
    t0 = 0
    for n in chunk_lens:
        q_d = to_dev(np.ascontiguousarray(q[:, t0:t0 + n]), dtype)
        kv_d = to_dev(np.ascontiguousarray(kv[:, t0:t0 + n]), dtype)
        xb_d = torch.zeros_like(q_d)
        st.prefill_chunk(1, slots, [p + t0 for p in pos0], n, q_d, kv_d, xb_d)
        torch.cuda.synchronize()
        got_xb[:, t0:t0 + n], got_q[:, t0:t0 + n] = to_host(xb_d, dtype), to_host(q_d, dtype)
        t0 += n
    assert st.stats().device_error == 0
    tol = cases.TOL_XB[dtype]
    np.testing.assert_allclose(cases.as_f32(got_xb, dtype), want_xb, rtol=0, atol=tol)
    assert_rotation_close(got_q, want_q, q, dtype, "rotated q of the chunk")
    for i, p in enumerate(pos0):
        got = to_host(st.layer_view(int(slots[i]), 1, p + T), dtype)
        kvd = sh.kv_dim
        assert np.array_equal(got[p:, kvd:].view(np.uint8), cache[i][p:p + T, kvd:].view(np.uint8)), "V rows bit-exact"
        assert_rotation_close(got[p:, :kvd], cache[i][p:p + T, :kvd], kv[i][:, :kvd], dtype, f"rotated K rows, context {i}")
    kernel = st.stats().last_kernel
    st.close()
    return kernel


# One rounding of a sum of magnitude ~1 to the storage type may flip in the last place (the GPU adds the products in
# another order than the reference's serial loop): 2^-10 relative for fp16, 2^-7 for bf16; the rotation then mixes
# two such values.
PROJ_RTOL = {cases.F16: 1e-3, cases.BF16: 8e-3}
PROJ_ATOL = {cases.F16: 4e-3, cases.BF16: 3e-2}


def run_project(case: cases.ProjCase, inactive=()):
    """project_append on fresh slots; returns q_out, the appended rows (None where inactive) and the stage."""
    sh, B, dt = case.shape, case.B, case.dtype
    tdt = TORCH_DT[dt]
    st = AttentionStage(sh, tdt, n_layers_hosted=2, max_batch=B, max_contexts=B, paged=True)
    st.set_rope_tables(to_dev(case.fcr, dt), to_dev(case.fci, dt))
    slots = st.get_contexts(np.arange(1, B + 1, dtype=np.uint32)).astype(np.int32)
    slots[list(inactive)] = -1
    pos = case.pos.copy()
    pos[list(inactive)] = 0xFFFFFFFF  # an inactive prompt's position is nobody's business: it must never be used
    st.batch_begin(slots, pos)
    q_out = torch.full((B, sh.dim), float("nan"), device="cuda", dtype=tdt)
    st.project_append(1, to_dev(case.x, dt), to_dev(case.rms_w, dt), to_dev(case.wq, dt),
                      to_dev(case.wkv, dt), q_out)
    torch.cuda.synchronize()
    assert st.stats().device_error == 0
    rows = []
    for i in range(B):
        if slots[i] < 0:
            rows.append(None)
            continue
        p = int(case.pos[i])
        rows.append(to_host(st.layer_view(int(slots[i]), 1, p + 1), dt)[p])
    return to_host(q_out, dt), rows, st, slots


def check_project(case, want, q_out, rows):
    dt = case.dtype
    for i, row in enumerate(rows):
        if row is not None:  # (the q of an inactive prompt is unspecified, as its xb is in the reference)
            np.testing.assert_allclose(cases.as_f32(q_out[i], dt), cases.as_f32(want.q_rot[i], dt), rtol=PROJ_RTOL[dt],
                                       atol=PROJ_ATOL[dt], err_msg=f"q of prompt {i}")
            np.testing.assert_allclose(cases.as_f32(row, dt), cases.as_f32(want.rows[i], dt), rtol=PROJ_RTOL[dt], atol=PROJ_ATOL[dt],
                                       err_msg=f"slot row of prompt {i}")
