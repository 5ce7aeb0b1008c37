"""Llama2::forward_attention on the reference's wire format: a serialized BatchedInferenceState goes in, the same
bytes come back with the attention output over the queries buffer and the next stage advanced
(src/models/common/state.hh:17-50, 561-594; src/models/llama2/model.hh:611-725).  The byte layout used here is the
one oracle/model_harness.cc asserts, at compile time, against the reference's own structs."""
import numpy as np
import pytest
import torch

from glinthawk_b200 import _lib
from glinthawk_b200.stage import AttentionStage, GlinthawkAttnError
from tests import cases, gpu_util

pytestmark = pytest.mark.gpu

METADATA = np.dtype([("id", "<u8"), ("batch_size", "<u4"), ("dtype", "u1"), ("route_id", "<u4"), ("model_id", "<u4"),
                     ("next_layer", "<u4"), ("next_stage", "u1"), ("next_tier", "i1"), ("next_rank", "u1"),
                     ("has_activations", "u1"), ("has_queries", "u1"), ("has_kvs", "u1"), ("is_sharded", "u1")])
PROMPT = np.dtype([("active", "u1"), ("prompt_id", "u1", (32,)), ("context_id", "<u4"), ("token", "<u4"),
                   ("token_pos", "<u4"), ("temperature", "u1"), ("prompt_length", "<u4"),
                   ("max_completion_length", "<u4"), ("finished", "u1"), ("kv_tier", "i1"), ("kv_rank", "u1")])
ATTENTION, POST_ATTENTION = 1, 2


def serialize(case: cases.Case, wire_dtype: int, next_layer: int, with_activations: bool, context_ids) -> np.ndarray:
    assert METADATA.itemsize == 32 and PROMPT.itemsize == 57
    md = np.zeros(1, dtype=METADATA)
    md["id"], md["batch_size"], md["dtype"] = 0x1122334455667788, case.B, wire_dtype
    md["route_id"], md["model_id"], md["next_layer"], md["next_stage"] = 7, 9, next_layer, ATTENTION
    md["has_activations"], md["has_queries"], md["has_kvs"] = int(with_activations), 1, 1
    pr = np.zeros(case.B, dtype=PROMPT)
    pr["active"] = case.active
    pr["prompt_id"] = np.arange(32 * case.B, dtype=np.uint8).reshape(case.B, 32)
    pr["context_id"], pr["token_pos"], pr["token"] = context_ids, case.pos, 31337
    npdt = cases.NP_DTYPE[wire_dtype]
    parts = [md.tobytes(), pr.tobytes()]
    if with_activations:
        parts.append(np.full((case.B, case.shape.dim), 0.5, dtype=npdt).tobytes())
    parts += [cases.as_f32(case.q, case.dtype).astype(npdt).tobytes(), cases.as_f32(case.kv_new, case.dtype).astype(npdt).tobytes()]
    return np.frombuffer(b"".join(parts), dtype=np.uint8).copy()


@pytest.mark.parametrize("wire_dtype,with_activations", [(cases.F16, False), (cases.F32, True)])
def test_serialized_state_through_the_attention_stage(oracle, wire_dtype, with_activations):
    case = cases.make_case("wire", "mini_g8", cases.F16, [0, 64, 333, 129, 511], seed=61, inactive=[3])
    want = oracle.layer_step(case)
    st = AttentionStage(case.shape, torch.float16, n_layers_hosted=2, max_batch=8, max_contexts=8, paged=True)
    st.set_rope_tables(gpu_util.to_dev(case.fcr, case.dtype), gpu_util.to_dev(case.fci, case.dtype))
    ids = np.array([500, 501, 502, 503, 504], dtype=np.uint32)
    first_layer = 10  # hosted layers 0, 1 stand for model layers 10, 11
    # the contexts exist already (bound by earlier states) and hold the cached rows of model layer 11
    slots = st.get_contexts(np.where(case.active, ids, 0).astype(np.uint32))
    for i in range(case.B):
        p = int(case.pos[i])
        if case.active[i] and p > 0:
            st.prepare(int(slots[i]), 1, p)
            st.layer_view(int(slots[i]), 1, p).copy_(gpu_util.to_dev(case.cache[i][:p], case.dtype))
    state = serialize(case, wire_dtype, first_layer + 1, with_activations, ids)
    before = state.copy()
    st.forward_attention_state(state, first_layer_hosted=first_layer)

    md = state[:32].view(METADATA)[0]
    assert md["next_stage"] == POST_ATTENTION and md["id"] == 0x1122334455667788 and md["has_kvs"] == 1
    npdt, sz = cases.NP_DTYPE[wire_dtype], np.dtype(cases.NP_DTYPE[wire_dtype]).itemsize
    off_q = 32 + 57 * case.B + (case.B * case.shape.dim * sz if with_activations else 0)
    off_kv = off_q + case.B * case.shape.dim * sz
    changed = np.flatnonzero(state != before)
    assert set(changed[changed < off_q].tolist()) <= {25} and changed.max() < off_kv, \
        "only next_stage (byte 25) and the queries buffer may change"
    xb = state[off_q:off_kv].view(npdt).reshape(case.B, case.shape.dim).astype(np.float32)
    for i in range(case.B):
        if case.active[i]:
            np.testing.assert_allclose(xb[i], cases.as_f32(want.xb[i], case.dtype), rtol=0, atol=cases.TOL_XB[case.dtype])
            p = int(case.pos[i])
            row = gpu_util.to_host(st.layer_view(int(st.lookup(int(ids[i]))), 1, p + 1)[p], case.dtype)
            assert np.array_equal(row[case.shape.kv_dim:], want.rows[i][case.shape.kv_dim:]), "V row bit-exact"
            gpu_util.assert_rotation_close(row[:case.shape.kv_dim], want.rows[i][:case.shape.kv_dim],
                                           case.kv_new[i][:case.shape.kv_dim], case.dtype, f"K row {i}")
    assert st.lookup(int(ids[3])) is None, "an inactive prompt binds no slot"

    # a state whose next stage is not attention, a layer that is not hosted, a truncated state: refused
    not_attention, wrong_layer, truncated = before.copy(), before.copy(), before[:-16].copy()
    not_attention[25] = POST_ATTENTION
    wrong_layer[21:25].view("<u4")[0] = 99
    for bad, status in ((not_attention, _lib.GH_ERR_STATE), (wrong_layer, _lib.GH_ERR_INVALID), (truncated, _lib.GH_ERR_INVALID)):
        with pytest.raises(GlinthawkAttnError) as e:
            st.forward_attention_state(bad, first_layer_hosted=first_layer)
        assert e.value.status == status
    st.close()


def test_a_prompt_at_position_zero_of_the_first_hosted_layer_starts_its_slot_afresh(oracle):
    """model.hh:617-621: prepare( layer, pos, pos == 0 && layer is the first served ) drops what the slot held."""
    case = cases.make_case("wire0", "l70b_4k", cases.F16, [0, 0], seed=62)  # 4 KiB rows: 3000 of them span six pages
    want = oracle.layer_step(case)
    st = AttentionStage(case.shape, torch.float16, n_layers_hosted=2, max_batch=2, max_contexts=2, paged=True)
    st.set_rope_tables(gpu_util.to_dev(case.fcr, case.dtype), gpu_util.to_dev(case.fci, case.dtype))
    slots = st.get_contexts(np.array([1, 2], dtype=np.uint32))
    for s in slots:  # a previous prompt's rows
        st.prepare(int(s), 0, 3000)
        st.prepare(int(s), 1, 3000)
    mapped_before = st.stats().bytes_mapped
    state = serialize(case, cases.F16, 0, False, np.array([1, 2], dtype=np.uint32))
    st.forward_attention_state(state)
    assert st.stats().bytes_mapped < mapped_before, "the old rows' pages went back to the pool"
    off_q = 32 + 57 * 2
    xb = state[off_q:off_q + 2 * case.shape.dim * 2].view(np.float16).reshape(2, -1).astype(np.float32)
    np.testing.assert_allclose(xb, cases.as_f32(want.xb, case.dtype), rtol=0, atol=cases.TOL_XB[case.dtype])
    st.close()
