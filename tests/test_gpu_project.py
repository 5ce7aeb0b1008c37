"""The stage's producer fused to the append (gh_attn_project_append) against the CPU restatement of the reference's
rmsnorm, matmul, copy_kv_cache and apply_rope, on a GPU."""
import numpy as np
import pytest
import torch

from glinthawk_b200 import _lib
from glinthawk_b200.shapes import SHAPES
from glinthawk_b200.stage import AttentionStage, GlinthawkAttnError
from tests import cases, gpu_util

pytestmark = pytest.mark.gpu

_run, _check = gpu_util.run_project, gpu_util.check_project


@pytest.mark.parametrize("shape_name,dtype,n", [("mini_mha", cases.F16, 5), ("mini_g4", cases.F16, 7), ("mini_g4", cases.BF16, 33),
                                                ("mini_g8", cases.F16, 16), ("mini_g16", cases.BF16, 3)])
def test_projection_rope_and_append_match_the_reference_operations(oracle, shape_name, dtype, n):
    sh = SHAPES[shape_name]
    pos = np.random.default_rng(n).integers(0, sh.seq_len, n)
    pos[0], pos[-1] = 0, sh.seq_len - 1
    case = cases.make_proj_case("proj", shape_name, dtype, pos, seed=40 + n)
    want = oracle.pre_attention(case)
    q_out, rows, st, _ = _run(case)
    _check(case, want, q_out, rows)
    st.close()


def test_projection_fixture_from_the_reference(oracle):
    """The same call against the committed outputs of the reference's own rmsnorm and matmul."""
    from pathlib import Path
    for spec in cases.GOLDEN_PROJ_SPECS[:2]:
        case = cases.golden_proj_case(spec)
        gold = np.load(Path(__file__).resolve().parent / "golden" / f"{case.name}.npz")
        q_out, rows, st, _ = _run(case)
        np.testing.assert_allclose(cases.as_f32(q_out, case.dtype), cases.as_f32(gold["q_rot"], case.dtype),
                                   rtol=gpu_util.PROJ_RTOL[case.dtype], atol=gpu_util.PROJ_ATOL[case.dtype])
        np.testing.assert_allclose(cases.as_f32(np.stack(rows), case.dtype), cases.as_f32(gold["rows"], case.dtype),
                                   rtol=gpu_util.PROJ_RTOL[case.dtype], atol=gpu_util.PROJ_ATOL[case.dtype])
        st.close()


def test_inactive_prompts_get_no_row_and_large_batches_go_in_slices(oracle):
    """300 prompts (two slices of the tensor-core tile's 256 columns), every seventh inactive: their slots stay
    untouched, everybody else's row and q match."""
    sh = SHAPES["mini_g4"]
    n = 300
    pos = np.random.default_rng(3).integers(0, sh.seq_len, n)
    case = cases.make_proj_case("proj300", "mini_g4", cases.F16, pos, seed=77)
    want = oracle.pre_attention(case)
    inactive = list(range(3, n, 7))
    q_out, rows, st, slots = _run(case, inactive=inactive)
    _check(case, want, q_out, rows)
    assert all(rows[i] is None for i in inactive)
    st.close()


@pytest.mark.parametrize("shape_name,dtype", [("l70b_4k", cases.F16), ("l3_8b_8k", cases.BF16), ("l3_405b", cases.F16)])
def test_full_size_weights_cut_across_all_sms(oracle, shape_name, dtype):
    """The real matrices (Llama2-70B: 8192 x 8192 and 2048 x 8192, 80 tiles of 128 k-blocks; Llama3-8B; Llama3-405B:
    16384 x 16384, 144 tiles of 256 k-blocks) dealt to one CTA per SM, so most tiles are finished from several CTAs'
    partial sums."""
    sh = SHAPES[shape_name]
    pos = np.array([0, 1, 100, 1000, sh.seq_len - 1, 17, 33, sh.seq_len // 2], dtype=np.uint32)
    case = cases.make_proj_case("projfull", shape_name, dtype, pos, seed=5)
    want = oracle.pre_attention(case)
    q_out, rows, st, _ = _run(case)
    _check(case, want, q_out, rows)
    # the same call again gives the same bits: the pieces are added in a fixed order
    q2, rows2, st2, _ = _run(case)
    assert np.array_equal(q_out.view(np.uint16), q2.view(np.uint16))
    assert all(np.array_equal(a.view(np.uint16), b.view(np.uint16)) for a, b in zip(rows, rows2))
    st.close()
    st2.close()


def test_projection_then_decode_equals_the_reference_layer_step(oracle):
    """project_append followed by decode against: reference projections, then the reference's layer-step on a cache
    that already holds a prefix."""
    shape_name, dt = "mini_g4", cases.F16
    sh = SHAPES[shape_name]
    pos = [0, 9, 64, 200, 511]
    base = cases.make_case("pd", shape_name, dt, pos, seed=12)
    proj = cases.make_proj_case("pd", shape_name, dt, pos, seed=13)
    pre = oracle.pre_attention(proj)
    step = cases.Case("pd", sh, dt, base.pos, base.active, base.cache, pre.q, pre.kv, base.fcr, base.fci)
    want = oracle.layer_step(step)

    st = gpu_util.make_stage(step, layers=2, paged=True)
    slots = gpu_util.load_case(st, step, layer=1)
    st.batch_begin(slots, step.pos)
    q_out = torch.zeros((len(pos), sh.dim), device="cuda", dtype=torch.float16)
    xb = torch.zeros_like(q_out)
    st.project_append(1, gpu_util.to_dev(proj.x, dt), gpu_util.to_dev(proj.rms_w, dt), gpu_util.to_dev(proj.wq, dt),
                      gpu_util.to_dev(proj.wkv, dt), q_out)
    st.decode(1, q_out, xb)
    torch.cuda.synchronize()
    assert st.stats().device_error == 0
    np.testing.assert_allclose(gpu_util.to_host(xb, dt).astype(np.float32), want.xb.astype(np.float32), rtol=0,
                               atol=cases.TOL_XB[dt])
    st.close()


def test_the_operation_level_entry_point_takes_the_reference_arguments(oracle):
    """gh_op_project_append: destination rows as device pointers (what copy_kv_cache and apply_rope receive), a null
    pointer for an inactive prompt, the RoPE tables as arguments."""
    case = cases.make_proj_case("projop", "mini_g8", cases.F16, [0, 3, 77, 511, 200], seed=91)
    want = oracle.pre_attention(case)
    sh, B, dt = case.shape, case.B, case.dtype
    st = AttentionStage(sh, torch.float16, n_layers_hosted=1, max_batch=B, max_contexts=B)
    rows_d = torch.full((B, 2 * sh.kv_dim), float("nan"), device="cuda", dtype=torch.float16)
    ptrs = [rows_d[i].data_ptr() for i in range(B)]
    ptrs[2] = 0  # inactive
    pos = case.pos.copy()
    pos[2] = 0xFFFFFFFF  # ... and its position is a value that must never index the tables
    q_out = torch.zeros((B, sh.dim), device="cuda", dtype=torch.float16)
    st.pre_attention_rope_append(B, gpu_util.to_dev(case.x, dt), gpu_util.to_dev(case.rms_w, dt), gpu_util.to_dev(case.wq, dt),
                                 gpu_util.to_dev(case.wkv, dt), q_out, pos, gpu_util.to_dev(case.fcr, dt),
                                 gpu_util.to_dev(case.fci, dt), ptrs)
    torch.cuda.synchronize()
    assert st.stats().device_error == 0
    got = gpu_util.to_host(rows_d, dt)
    assert np.isnan(got[2].astype(np.float32)).all(), "the inactive prompt's row is not touched"
    _check(case, want, gpu_util.to_host(q_out, dt), [got[i] if i != 2 else None for i in range(B)])
    st.close()


def test_unsupported_shapes_are_refused():
    sh = SHAPES["tiny15m"]  # fp32, dim 288
    st = AttentionStage(sh, torch.float32, n_layers_hosted=1, max_batch=2, max_contexts=2)
    cos = torch.ones(sh.seq_len, sh.head_size // 2, device="cuda")
    st.set_rope_tables(cos, torch.zeros_like(cos))
    s = st.get_context(1)
    st.batch_begin([s], [0])
    x = torch.zeros(1, sh.dim, device="cuda")
    w = torch.zeros(sh.dim, sh.dim, device="cuda")
    with pytest.raises(GlinthawkAttnError) as e:
        st.project_append(0, x, x[0], w, torch.zeros(2 * sh.kv_dim, sh.dim, device="cuda"), torch.zeros_like(x))
    assert e.value.status == _lib.GH_ERR_UNSUPPORTED
    st.close()
