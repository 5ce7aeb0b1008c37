"""Slot pool, context views, paging and the error conventions of the boundary, on a GPU."""
import numpy as np
import pytest
import torch

from glinthawk_b200 import _lib
from glinthawk_b200.shapes import SHAPES
from glinthawk_b200.stage import AttentionStage, GlinthawkAttnError

pytestmark = pytest.mark.gpu


def test_context_manager_semantics():
    st = AttentionStage(SHAPES["tiny15m"], torch.float32, n_layers_hosted=2, max_batch=8, max_contexts=3)
    a, b = st.get_context(11), st.get_context(22)
    assert a != b and st.get_context(11) == a and st.lookup(22) == b and st.lookup(99) is None
    assert st.get_context(0) == -1  # NULL_CONTEXT -> the empty context
    # all-or-nothing for a batch: two new ids, one slot left -> nothing is bound
    assert st.get_contexts([11, 33, 44]) is None
    assert st.stats().slots_free == 1 and st.lookup(33) is None
    slots = st.get_contexts([11, 0, 33])
    assert slots.tolist() == [a, -1, st.lookup(33)]
    with pytest.raises(GlinthawkAttnError) as e:
        st.get_context(55)
    assert e.value.status == _lib.GH_ERR_NO_SLOT
    assert st.release_context(22) and not st.release_context(22)
    assert st.get_context(55) == b  # the freed slot is reused
    st.close()


def test_context_views_follow_the_reference_layout():
    sh = SHAPES["mini_g4"]
    st = AttentionStage(sh, torch.float16, n_layers_hosted=3, max_batch=4, max_contexts=2)
    s0, s1 = st.get_context(1), st.get_context(2)
    row = 2 * sh.kv_dim * 2
    assert st.slot_bytes() == 3 * sh.seq_len * row
    base = st.layer_ptr(s0, 0)
    assert st.layer_ptr(s0, 2) - base == 2 * sh.seq_len * row      # layers packed consecutively
    assert st.token_ptr(s0, 1, 7) - st.layer_ptr(s0, 1) == 7 * row  # token t at + t * 2 * kv_dim elements
    assert st.layer_ptr(s1, 0) - base >= st.slot_bytes()
    assert st.layer_ptr(-1, 0) == 0 and st.token_ptr(-1, 0, 3) == 0  # empty context -> null views
    with pytest.raises(GlinthawkAttnError):
        st.layer_ptr(s0, 3)
    with pytest.raises(GlinthawkAttnError) as e:
        st.token_ptr(s0, 0, sh.seq_len)
    assert e.value.status == _lib.GH_ERR_CAPACITY
    st.close()


def test_paged_slots_map_on_demand_and_release():
    sh = SHAPES["l70b_4k"]  # row 4 KiB -> 512 tokens per 2 MiB page, 16 MiB per layer
    st = AttentionStage(sh, torch.float16, n_layers_hosted=2, max_batch=4, max_contexts=4, paged=True)
    s = st.get_context(7)
    assert st.stats().bytes_mapped == 0 and st.stats().bytes_reserved >= 4 * st.slot_bytes()
    st.prepare(s, 0, 0)
    one = st.stats().bytes_mapped
    assert one == 2 << 20
    st.prepare(s, 0, 100)
    assert st.stats().bytes_mapped == one  # same page
    st.prepare(s, 1, 511)
    assert st.stats().bytes_mapped == 2 * one
    st.prepare(s, 1, 512)  # the 513th token of layer 1 starts a new page
    assert st.stats().bytes_mapped == 3 * one
    v = st.layer_view(s, 1, 1024)
    v.fill_(1.0)
    torch.cuda.synchronize()
    assert float(v.float().sum()) == 1024 * 2 * sh.kv_dim
    st.prepare(s, 0, 0, can_release=True)  # a new prompt starts in this slot
    assert st.stats().bytes_mapped == one
    st.release_context(7)
    assert st.stats().bytes_mapped == 0
    # a slot whose pages went back to the pool can be bound and filled again
    s2 = st.get_context(8)
    st.prepare(s2, 1, 2000)
    st.layer_view(s2, 1, 2001).fill_(2.0)
    torch.cuda.synchronize()
    assert st.stats().bytes_mapped == 4 * one
    st.close()


def test_paged_budget_is_an_error_status():
    sh = SHAPES["l70b_4k"]
    st = AttentionStage(sh, torch.float16, n_layers_hosted=2, max_batch=4, max_contexts=4, paged=True,
                        page_budget=2 << 20)
    s = st.get_context(1)
    st.prepare(s, 0, 10)
    with pytest.raises(GlinthawkAttnError) as e:
        st.prepare(s, 1, 10)
    assert e.value.status == _lib.GH_ERR_OOM
    st.close()


def test_error_conventions():
    sh = SHAPES["tiny15m"]
    st = AttentionStage(sh, torch.float32, n_layers_hosted=1, max_batch=2, max_contexts=2)
    q = torch.zeros(2, sh.dim, device="cuda")
    kv = torch.zeros(2, 2 * sh.kv_dim, device="cuda")
    with pytest.raises(GlinthawkAttnError) as e:
        st.decode(0, q, q.clone())
    assert e.value.status == _lib.GH_ERR_STATE  # no batch yet
    s = st.get_context(1)
    with pytest.raises(GlinthawkAttnError) as e:
        st.batch_begin([s], [sh.seq_len])
    assert e.value.status == _lib.GH_ERR_CAPACITY
    with pytest.raises(GlinthawkAttnError) as e:
        st.batch_begin([5], [0])
    assert e.value.status == _lib.GH_ERR_INVALID
    with pytest.raises(GlinthawkAttnError):
        st.batch_begin([s, s, s], [0, 0, 0])  # larger than max_batch
    st.batch_begin([s, -1], [0, 0])
    with pytest.raises(GlinthawkAttnError) as e:
        st.append(0, q, kv)
    assert e.value.status == _lib.GH_ERR_STATE  # RoPE tables not set
    with pytest.raises(GlinthawkAttnError):
        st.decode(1, q, q.clone())  # layer not hosted
    # the handle stays usable after every error
    cos = torch.ones(sh.seq_len, sh.head_size // 2, device="cuda")
    st.set_rope_tables(cos, torch.zeros_like(cos))
    st.append(0, q, kv)
    torch.cuda.synchronize()
    assert st.stats().device_error == 0 and st.stats().kernel_launches >= 1
    st.close()


def test_misaligned_device_buffers_are_refused_before_any_launch():
    """The kernels move q, K/V rows and outputs in 16-byte pieces.  A pointer that is not 16-byte aligned comes back
    as GH_ERR_INVALID with nothing launched, and the handle keeps working."""
    sh = SHAPES["mini_g4"]
    st = AttentionStage(sh, torch.float16, n_layers_hosted=1, max_batch=2, max_contexts=2)
    cos = torch.ones(sh.seq_len, sh.head_size // 2, device="cuda", dtype=torch.float16)
    st.set_rope_tables(cos, torch.zeros_like(cos))
    s = st.get_context(1)
    st.batch_begin([s, -1], [0, 0])
    big = torch.zeros(2 * sh.dim + 8, device="cuda", dtype=torch.float16)
    q_odd = big[4:4 + 2 * sh.dim].view(2, sh.dim)  # 8 bytes off
    q = torch.zeros(2, sh.dim, device="cuda", dtype=torch.float16)
    kv = torch.zeros(2, 2 * sh.kv_dim, device="cuda", dtype=torch.float16)
    launches = st.stats().kernel_launches
    for call in (lambda: st.append(0, q_odd, kv), lambda: st.decode(0, q_odd, q.clone()), lambda: st.decode(0, q, q_odd),
                 lambda: st.step(0, q_odd, kv, q.clone()),
                 lambda: st.prefill_chunk(0, [s], [0], 2, q_odd.view(1, 2, sh.dim), kv.view(1, 2, -1), q.clone().view(1, 2, -1))):
        with pytest.raises(GlinthawkAttnError) as e:
            call()
        assert e.value.status == _lib.GH_ERR_INVALID and "aligned" in str(e.value)
    assert st.stats().kernel_launches == launches
    st.step(0, q, kv, q.clone())
    torch.cuda.synchronize()
    assert st.stats().device_error == 0 and st.stats().kernel_launches > launches
    st.close()


def test_a_batch_of_inactive_prompts_only_is_a_no_op():
    """The reference's batches keep their size when prompts finish: a batch can consist of empty contexts only
    (src/compute/contextman.hh:128-171).  Every entry point then succeeds and writes nothing."""
    sh = SHAPES["mini_g4"]
    st = AttentionStage(sh, torch.float16, n_layers_hosted=1, max_batch=3, max_contexts=3, paged=True)
    cos = torch.ones(sh.seq_len, sh.head_size // 2, device="cuda", dtype=torch.float16)
    st.set_rope_tables(cos, torch.zeros_like(cos))
    st.batch_begin([-1, -1, -1], [0, 5, 9])
    q = torch.ones(3, sh.dim, device="cuda", dtype=torch.float16)
    kv = torch.ones(3, 2 * sh.kv_dim, device="cuda", dtype=torch.float16)
    xb = torch.full_like(q, 3.0)
    st.step(0, q, kv, xb)
    st.prefill_chunk(0, [-1, -1], [0, 0], 4, torch.ones(2, 4, sh.dim, device="cuda", dtype=torch.float16),
                     torch.ones(2, 4, 2 * sh.kv_dim, device="cuda", dtype=torch.float16),
                     torch.full((2, 4, sh.dim), 3.0, device="cuda", dtype=torch.float16))
    x = torch.ones(3, sh.dim, device="cuda", dtype=torch.float16)
    w = torch.zeros(sh.dim, sh.dim, device="cuda", dtype=torch.float16)
    st.project_append(0, x, x[0].contiguous(), w, torch.zeros(2 * sh.kv_dim, sh.dim, device="cuda", dtype=torch.float16),
                      torch.empty_like(q))
    torch.cuda.synchronize()
    stats = st.stats()
    assert stats.device_error == 0 and stats.bytes_mapped == 0, "no page was mapped for anybody"
    assert (xb == 3.0).all() and (q == 1.0).all()
    st.close()


def test_fill_normal_statistics():
    sh = SHAPES["tiny15m"]
    st = AttentionStage(sh, torch.float32, n_layers_hosted=1, max_batch=1, max_contexts=1)
    x = torch.empty(1 << 20, device="cuda")
    st.fill_normal(x, x.numel(), torch.float32, seed=3)
    y = torch.empty(1 << 20, device="cuda", dtype=torch.float16)
    st.fill_normal(y, y.numel(), torch.float16, seed=3)
    torch.cuda.synchronize()
    assert abs(float(x.mean())) < 5e-3 and abs(float(x.std()) - 1.0) < 5e-3
    assert torch.equal(x.half(), y)  # same counter stream in every dtype
    z = torch.empty(1 << 19, device="cuda")
    st.fill_normal(z, z.numel(), torch.float32, seed=3, offset=1 << 19)
    torch.cuda.synchronize()
    assert torch.equal(z, x[1 << 19:])
    st.close()


def test_create_that_cannot_fit_reports_out_of_memory_and_leaks_nothing():
    """Static slots for 4096 Llama2-70B contexts would need 5 TB: creation fails with a status (the reference aborts
    the process, src/arch/cuda/llama2/ops.cuh:113-115), and what had been allocated before the failure is released."""
    free0, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        with pytest.raises(GlinthawkAttnError) as e:
            AttentionStage(SHAPES["l70b_4k"], torch.float16, n_layers_hosted=80, max_batch=8, max_contexts=4096)
        assert e.value.status == _lib.GH_ERR_OOM
    free1, _ = torch.cuda.mem_get_info()
    assert free0 - free1 < (64 << 20)
    # the same shape with paged slots only reserves address space
    st = AttentionStage(SHAPES["l70b_4k"], torch.float16, n_layers_hosted=80, max_batch=8, max_contexts=512, paged=True)
    assert st.stats().bytes_mapped == 0 and st.stats().bytes_reserved >= 512 * st.slot_bytes()
    st.close()
