"""The CPU restatement (oracle/attn_oracle.c) against fixtures produced by the reference's own amd64 code, and —
where a prebuilt reference library is present — against that code run live."""
import zlib
from pathlib import Path

import numpy as np
import pytest

from tests import cases

GOLDEN = Path(__file__).resolve().parent / "golden"


def _crc(case):
    crc = 0
    for a in [*case.cache, case.q, case.kv_new, case.fcr, case.fci, case.pos]:
        crc = zlib.crc32(np.ascontiguousarray(a).tobytes(), crc)
    return crc


def _f32(a, dtype):
    return cases.as_f32(np.asarray(a), dtype)


# fp32: the reference is built with -ffast-math (vectorised expf, reassociated sums), the restatement is not.
# fp16: every intermediate is rounded to fp16 in both, so at most a last-place flip survives.
ORACLE_VS_REF_ABS = {cases.F32: 2e-6, cases.F16: 1e-3}


def check_against(res, gold_rows, gold_q, gold_xb, case, atol):
    for i in range(case.B):
        if not case.active[i]:
            continue
        kvd = case.shape.kv_dim
        # V is a raw copy everywhere: bit-exact
        assert np.array_equal(res.rows[i][kvd:].view(np.uint8), np.asarray(gold_rows[i][kvd:]).view(np.uint8))
        np.testing.assert_allclose(_f32(res.rows[i][:kvd], case.dtype), _f32(gold_rows[i][:kvd], case.dtype),
                                   rtol=cases.TOL_K_REL, atol=1e-3)
        np.testing.assert_allclose(_f32(res.q[i], case.dtype), _f32(gold_q[i], case.dtype), rtol=cases.TOL_K_REL,
                                   atol=1e-3)
        np.testing.assert_allclose(_f32(res.xb[i], case.dtype), _f32(gold_xb[i], case.dtype), rtol=0, atol=atol)


@pytest.mark.parametrize("spec", cases.GOLDEN_SPECS, ids=lambda s: s["name"])
def test_oracle_matches_reference_fixture(oracle, spec):
    case = cases.golden_case(spec)
    gold = np.load(GOLDEN / f"{case.name}.npz")
    assert int(gold["input_crc"]) == _crc(case), "seeded inputs drifted: regenerate tests/golden"
    res = oracle.layer_step(case)
    check_against(res, gold["rows"], gold["q"], gold["xb"], case, ORACLE_VS_REF_ABS[case.dtype])


@pytest.mark.parametrize("spec", cases.GOLDEN_SPECS[:10], ids=lambda s: s["name"])
def test_fixture_reproduced_by_reference_library(reference, spec):
    """Where the reference library travels with the repository, it must reproduce its own fixtures."""
    case = cases.golden_case(spec)
    gold = np.load(GOLDEN / f"{case.name}.npz")
    res = reference.layer_step(case)
    check_against(res, gold["rows"], gold["q"], gold["xb"], case, ORACLE_VS_REF_ABS[case.dtype])


@pytest.mark.parametrize("dtype", [cases.F32, cases.F16])
def test_oracle_per_op_against_reference(oracle, reference, dtype):
    """Score matrix after softmax (the only place `att` is observable) agrees op by op."""
    case = cases.make_case("per_op", "mini_g4", dtype, [0, 17, 200], seed=7)
    a = oracle.layer_step(case, keep_att=True)
    b = reference.layer_step(case, keep_att=True)
    for i, p in enumerate(case.pos):
        np.testing.assert_allclose(a.att[i, :, : p + 1].astype(np.float32), b.att[i, :, : p + 1].astype(np.float32),
                                   rtol=0, atol=2e-6 if dtype == cases.F32 else 1e-3)
        sums = a.att[i, :, : p + 1].astype(np.float32).sum(axis=1)
        np.testing.assert_allclose(sums, 1.0, atol=5e-3 if dtype == cases.F16 else 1e-5)


def test_oracle_bf16_roundtrip_and_step(oracle):
    x = np.random.default_rng(0).standard_normal(4096).astype(np.float32)
    b = cases.to_bf16_bits(x)
    assert np.abs(cases.from_bf16_bits(b) - x).max() <= np.abs(x).max() * 2.0 ** -8
    # a bf16 layer-step stays close to the fp32 step on the same bf16-rounded inputs
    c32 = cases.make_case("bf", "mini_g4", cases.F32, [40, 300], seed=11, round_inputs_to=cases.BF16)
    c16 = cases.make_case("bf", "mini_g4", cases.BF16, [40, 300], seed=11)
    r32, r16 = oracle.layer_step(c32), oracle.layer_step(c16)
    np.testing.assert_allclose(cases.from_bf16_bits(r16.xb), r32.xb, rtol=0, atol=cases.TOL_XB[cases.BF16])


def test_oracle_convert_and_copy(oracle):
    import ctypes as C
    x = np.random.default_rng(1).standard_normal(1000).astype(np.float32)
    h = np.zeros(1000, np.float16)
    oracle.op("convert_and_copy", cases.F16, C.c_void_p(h.ctypes.data), cases.F32, C.c_void_p(x.ctypes.data),
              C.c_uint64(1000))
    assert np.array_equal(h, x.astype(np.float16))
    back = np.zeros(1000, np.float32)
    oracle.op("convert_and_copy", cases.F32, C.c_void_p(back.ctypes.data), cases.F16, C.c_void_p(h.ctypes.data),
              C.c_uint64(1000))
    assert np.array_equal(back, h.astype(np.float32))


# ---- the stage's producer: rmsnorm + q / kv projections (+ rotation and append) -------------------------------

# fp32: sums of `dim` products, reassociated by -ffast-math in the reference build.  fp16: one rounding of a sum of
# magnitude ~1, so a last-place flip (2^-10 relative) is the most that survives.
PROJ_ABS = {cases.F32: 2e-5, cases.F16: 4e-3}


def _proj_crc(case):
    crc = 0
    for a in [case.x, case.rms_w, case.wq, case.wkv, case.fcr, case.fci, case.pos]:
        crc = zlib.crc32(np.ascontiguousarray(a).tobytes(), crc)
    return crc


def check_proj(res, gold, case):
    atol = PROJ_ABS[case.dtype]
    for name in ("xb", "q", "kv", "q_rot", "rows"):
        np.testing.assert_allclose(_f32(getattr(res, name), case.dtype), _f32(gold[name], case.dtype), rtol=cases.TOL_K_REL,
                                   atol=atol, err_msg=name)


@pytest.mark.parametrize("spec", cases.GOLDEN_PROJ_SPECS, ids=lambda s: s["name"])
def test_oracle_producer_matches_reference_fixture(oracle, spec):
    case = cases.golden_proj_case(spec)
    gold = np.load(GOLDEN / f"{case.name}.npz")
    assert int(gold["input_crc"]) == _proj_crc(case), "seeded inputs drifted: regenerate tests/golden"
    check_proj(oracle.pre_attention(case), gold, case)


@pytest.mark.parametrize("spec", cases.GOLDEN_PROJ_SPECS, ids=lambda s: s["name"])
def test_producer_fixture_reproduced_by_reference_library(oracle, reference, spec):
    case = cases.golden_proj_case(spec)
    gold = np.load(GOLDEN / f"{case.name}.npz")
    check_proj(reference.pre_attention(case, oracle), gold, case)

