"""The CUDA path against the CPU oracle at the benchmark configurations' real batch sizes.

The golden fixtures hold two to six contexts per shape; here one layer-step runs with the whole batch of each
configuration (256 lognormal contexts of Llama2-70B, 64 of Llama2-7B, 128 of Llama2-13B over two consecutive steps,
every fourth of the 448 Llama3-8B decode contexts, and 512-token prompt chunks that end at the last row of an
8192-token slot).  The cached rows are generated on the device and downloaded for the oracle, so that set-up takes
seconds instead of minutes.
"""
import threading

import numpy as np
import pytest
import torch

from glinthawk_b200.rope import rope_tables
from glinthawk_b200.stage import AttentionStage
from glinthawk_b200.workload import WORKLOADS
from tests import cases, gpu_util

pytestmark = pytest.mark.gpu


def device_case(workload: str, pos, seed: int, *, layers: int = 1, layer: int = 0):
    """A stage whose slots hold pos[i] device-generated rows each, and the same case for the oracle."""
    wl = WORKLOADS[workload]
    sh = wl.shape
    dtype = {"f16": cases.F16, "bf16": cases.BF16, "f32": cases.F32}[wl.dtype]
    tdt = gpu_util.TORCH_DT[dtype]
    pos = np.asarray(pos, dtype=np.uint32)
    B = len(pos)
    st = AttentionStage(sh, tdt, n_layers_hosted=layers, max_batch=B, max_contexts=B, paged=True)
    cos, sin = rope_tables(sh.head_size, sh.seq_len, sh.rope_theta)
    fcr, fci = cases.store(cos, dtype), cases.store(sin, dtype)
    st.set_rope_tables(gpu_util.to_dev(fcr, dtype), gpu_util.to_dev(fci, dtype))
    slots = st.get_contexts(np.arange(1, B + 1, dtype=np.uint32))
    row = 2 * sh.kv_dim
    cache = []
    for i in range(B):
        p = int(pos[i])
        st.prepare(int(slots[i]), layer, p)
        if p > 0:
            st.fill_normal(st.layer_ptr(int(slots[i]), layer), p * row, tdt, seed, offset=i * sh.seq_len * row)
    torch.cuda.synchronize()
    for i in range(B):
        p = int(pos[i])
        c = np.zeros((p + 1, row), dtype=np.uint16 if dtype == cases.BF16 else cases.NP_DTYPE[dtype])
        if p > 0:
            c[:p] = gpu_util.to_host(st.layer_view(int(slots[i]), layer, p), dtype)
        cache.append(c)
    rng = np.random.default_rng(seed)
    q = cases.store(rng.standard_normal((B, sh.dim), dtype=np.float32), dtype)
    kv_new = cases.store(rng.standard_normal((B, row), dtype=np.float32), dtype)
    case = cases.Case(workload, sh, dtype, pos, np.ones(B, dtype=bool), cache, q, kv_new, fcr, fci, seed)
    return st, slots, case


def test_llama2_70b_all_256_contexts(oracle):
    wl = WORKLOADS["llama2_70b_gqa"]
    pos = wl.lengths(20240, headroom=1).astype(np.uint32)
    pos[0], pos[1], pos[2] = 16, 4095, 0  # the shortest length of the distribution, the slot's last row, an empty slot
    st, slots, case = device_case("llama2_70b_gqa", pos, seed=5)
    want = oracle.layer_step(case)
    got = gpu_util.run_step(st, case, slots, layer=0)
    gpu_util.assert_step_close(got, want, case)
    assert st.stats().last_kernel == 1
    st.close()


def test_llama2_7b_all_64_contexts(oracle):
    pos = np.random.default_rng(3).integers(128, 4096, size=64).astype(np.uint32)
    pos[5] = 4095
    st, slots, case = device_case("llama2_7b_layer", pos, seed=6)
    want = oracle.layer_step(case)
    got = gpu_util.run_step(st, case, slots, layer=0)
    gpu_util.assert_step_close(got, want, case)
    st.close()


def test_llama2_13b_128_contexts_two_consecutive_steps(oracle):
    pos = np.random.default_rng(4).integers(512, 4095, size=128).astype(np.uint32)
    st, slots, case = device_case("llama2_13b", pos, seed=7)
    rng = np.random.default_rng(70)
    for step in range(2):
        want = oracle.layer_step(case)
        got = gpu_util.run_step(st, case, slots, layer=0)
        gpu_util.assert_step_close(got, want, case)
        if step == 0:  # the next token: the caches now hold the oracle's appended rows, the slots the device's
            grown = []
            for c, p, r in zip(case.cache, case.pos, want.rows):
                c = np.concatenate([c, np.zeros((1, c.shape[1]), c.dtype)])
                c[int(p)] = r
                grown.append(c)
            for i in range(case.B):
                st.prepare(int(slots[i]), 0, int(case.pos[i]) + 1)
            case = cases.Case(case.name, case.shape, case.dtype, case.pos + 1, case.active, grown,
                              cases.store(rng.standard_normal(case.q.shape, dtype=np.float32), case.dtype),
                              cases.store(rng.standard_normal(case.kv_new.shape, dtype=np.float32), case.dtype),
                              case.fcr, case.fci)
    st.close()


def test_llama3_8b_bf16_every_fourth_decode_context(oracle):
    wl = WORKLOADS["llama3_8b_decode"]
    pos = wl.lengths(20240, headroom=1)[::4].astype(np.uint32)
    pos[0] = 8191
    st, slots, case = device_case("llama3_8b_decode", pos, seed=8)
    want = oracle.layer_step(case)
    got = gpu_util.run_step(st, case, slots, layer=0)
    gpu_util.assert_step_close(got, want, case)
    st.close()


def test_llama3_8b_prompt_chunks_up_to_the_last_row_of_the_slot(oracle):
    """512-token chunks into a fresh slot, behind 3584 cached tokens, and ending exactly at row 8191."""
    kernel = gpu_util.check_prefill(oracle, "l3_8b_8k", cases.BF16, pos0=[0, 3584, 7680], chunk_lens=[512])
    assert kernel == 2


def test_current_batch_survives_many_other_uploads(oracle):
    """A batch description must stay intact however many prompt chunks and pointer-array operations are issued
    between gh_attn_batch_begin and a later layer's step: each of those uploads a description of its own."""
    case = cases.make_case("ring", "mini_g4", cases.F16, [40, 300, 7, 129, 511, 64], seed=77)
    want = oracle.layer_step(case)
    st = AttentionStage(case.shape, torch.float16, n_layers_hosted=3, max_batch=8, max_contexts=12, paged=True)
    st.set_rope_tables(gpu_util.to_dev(case.fcr, case.dtype), gpu_util.to_dev(case.fci, case.dtype))
    slots = gpu_util.load_case(st, case, layer=2)
    q = gpu_util.to_dev(case.q, case.dtype)
    kv = gpu_util.to_dev(case.kv_new, case.dtype)
    xb = torch.zeros_like(q)
    st.batch_begin(slots, case.pos)

    # 24 prompt-chunk calls (two uploads each) into other slots, and 24 pointer-array operations
    sh = case.shape
    other = st.get_contexts(np.arange(100, 104, dtype=np.uint32))
    pf_q = torch.randn((4, 16, sh.dim), device="cuda").half()
    pf_kv = torch.randn((4, 16, 2 * sh.kv_dim), device="cuda").half()
    pf_xb = torch.zeros_like(pf_q)
    for n in range(24):
        st.prefill_chunk(0, other, [16 * n] * 4, 16, pf_q, pf_kv, pf_xb)
    for s in other:
        st.prepare(int(s), 1, 0)
    rows = [st.token_ptr(int(s), 1, 0) for s in other]
    for n in range(24):
        st.copy_kv_cache(rows, pf_kv[:, 0].contiguous(), 4)

    st.step(2, q, kv, xb)
    torch.cuda.synchronize()
    assert st.stats().device_error == 0
    got_rows = [gpu_util.to_host(st.layer_view(int(s), 2, int(p) + 1)[int(p)], case.dtype) for s, p in zip(slots, case.pos)]
    got = cases.StepResult(got_rows, gpu_util.to_host(q, case.dtype), gpu_util.to_host(xb, case.dtype))
    gpu_util.assert_step_close(got, want, case)
    st.close()


def test_slot_map_from_a_second_thread_while_steps_run(oracle):
    """The reference looks contexts up on a bookkeeping thread while the execution thread runs the model
    (src/compute/kernel.hh:139-170, under the mutex of src/compute/contextman.hh:82-184).  Here one thread binds and
    looks up ids while the main thread runs layer-steps; the steps' results and the map both stay right."""
    case = cases.make_case("mt", "mini_g8", cases.F16, [100, 511, 3, 64], seed=88)
    want = oracle.layer_step(case)
    st = AttentionStage(case.shape, torch.float16, n_layers_hosted=2, max_batch=4, max_contexts=260, paged=True)
    st.set_rope_tables(gpu_util.to_dev(case.fcr, case.dtype), gpu_util.to_dev(case.fci, case.dtype))
    slots = gpu_util.load_case(st, case, layer=0)
    stop, seen, errors = threading.Event(), {}, []

    def bookkeeping():
        try:
            n = 0
            while not stop.is_set():
                cid = 1000 + (n % 256)
                slot = st.get_context(cid)
                if seen.setdefault(cid, slot) != slot or st.lookup(cid) != slot:
                    errors.append(f"context {cid} moved")
                for i, s in enumerate(slots):
                    if st.lookup(1 + i) != int(s):
                        errors.append(f"context {1 + i} lost its slot")
                n += 1
        except Exception as e:  # noqa: BLE001
            errors.append(repr(e))

    t = threading.Thread(target=bookkeeping)
    t.start()
    try:
        for _ in range(50):
            for i in range(case.B):  # the step overwrites row pos: start every pass from the same slot contents
                p = int(case.pos[i])
                st.layer_view(int(slots[i]), 0, p + 1)[p].zero_()
            got = gpu_util.run_step(st, case, slots, layer=0)
            gpu_util.assert_step_close(got, want, case)
    finally:
        stop.set()
        t.join()
    assert not errors, errors[:3]
    assert len(set(seen.values())) == len(seen) and not set(seen.values()) & {int(s) for s in slots}
    st.close()


def test_timed_out_wait_is_reported_and_can_be_cleared():
    """The error word is sticky on the device; the host refuses work once it has seen it and goes on after
    gh_attn_clear_device_error.  The word is set here by hand (nothing on the GPU is made to hang)."""
    from glinthawk_b200 import _lib
    case = cases.make_case("flag", "mini_g8", cases.F16, [10, 70], seed=5)
    st = gpu_util.make_stage(case)
    slots = gpu_util.load_case(st, case, layer=0)
    assert st.stats().device_error == 0
    assert _lib.lib.gh_attn_inject_device_error(st._h, 2) == 0
    with pytest.raises(gpu_util.GlinthawkAttnError) as e:
        st.synchronize()
    assert e.value.status == _lib.GH_ERR_CUDA
    q = gpu_util.to_dev(case.q, case.dtype)
    with pytest.raises(gpu_util.GlinthawkAttnError):
        st.batch_begin(slots, case.pos)
        st.step(0, q, gpu_util.to_dev(case.kv_new, case.dtype), torch.zeros_like(q))
    st.clear_device_error()
    assert st.stats().device_error == 0
    got = gpu_util.run_step(st, case, slots, layer=0)
    assert np.isfinite(cases.as_f32(got.xb, case.dtype)).all()
    st.close()


@pytest.mark.parametrize("paged", [False, True])
def test_reference_operations_on_own_slots_share_one_description(oracle, paged):
    """The adapter's sequence for a layer — copy_kv_cache + apply_rope (as one call or as two) and the fused attention
    call, with host arrays of row pointers — over three layers and two steps.  The pointers name the stage's own
    slots, so the calls run on the kernels of the fused path; the description is planned once per step."""
    pos = [40, 300, 7, 129, 510, 64]
    case = cases.make_case("ops_own", "mini_g8", cases.F16, pos, seed=91, inactive=[2])
    st = gpu_util.make_stage(case, layers=3, paged=paged)
    slots = None
    for layer in range(3):
        slots = gpu_util.load_case(st, case, layer) if slots is None else slots
        for i in range(case.B):
            if case.active[i]:
                st.prepare(int(slots[i]), layer, int(case.pos[i]) + 1)
                if layer and case.pos[i]:
                    st.layer_view(int(slots[i]), layer, int(case.pos[i])).copy_(
                        gpu_util.to_dev(case.cache[i][: int(case.pos[i])], case.dtype))
    fcr, fci = gpu_util.to_dev(case.fcr, case.dtype), gpu_util.to_dev(case.fci, case.dtype)
    cur, rng = case, np.random.default_rng(5)
    for step in range(2):
        want = oracle.layer_step(cur)
        plans_before = None
        for layer in range(3):
            rows = [st.token_ptr(int(s), layer, int(p)) if s >= 0 else 0 for s, p in zip(slots, cur.pos)]
            bases = [st.layer_ptr(int(s), layer) if s >= 0 else 0 for s in slots]
            q = gpu_util.to_dev(cur.q, cur.dtype)
            kv = gpu_util.to_dev(cur.kv_new, cur.dtype)
            xb = torch.zeros_like(q)
            if layer == 1:  # the two operations on their own
                st.copy_kv_cache(rows, kv, cur.B)
                st.apply_rope(cur.B, cur.pos, fcr, fci, q, rows)
            else:
                st.copy_kv_cache_apply_rope(cur.B, cur.pos, fcr, fci, q, rows, kv)
            st.attention_fused(q, bases, xb, cur.B, cur.pos)
            torch.cuda.synchronize()
            stats = st.stats()
            assert stats.device_error == 0 and stats.last_kernel == 1
            got_rows = [gpu_util.to_host(st.layer_view(int(s), layer, int(p) + 1)[int(p)], cur.dtype) if s >= 0 else None
                        for s, p in zip(slots, cur.pos)]
            got = cases.StepResult(got_rows, gpu_util.to_host(q, cur.dtype), gpu_util.to_host(xb, cur.dtype))
            gpu_util.assert_step_close(got, want, cur)
            assert torch.count_nonzero(xb[2]) == 0, "inactive prompt untouched"
            if plans_before is None:
                plans_before = stats.batch_plans
            assert stats.batch_plans == plans_before, "later layers of a step reuse the first layer's description"
        grown = [np.concatenate([c[: int(p)], (r if r is not None else c[int(p)])[None, :], np.zeros((1, c.shape[1]), c.dtype)])
                 for c, p, r in zip(cur.cache, cur.pos, want.rows)]
        cur = cases.Case(cur.name, cur.shape, cur.dtype, cur.pos + 1, cur.active, grown,
                         rng.standard_normal(cur.q.shape).astype(cur.q.dtype),
                         rng.standard_normal(cur.kv_new.shape).astype(cur.kv_new.dtype), cur.fcr, cur.fci)
    st.close()


def test_consecutive_calls_execute_in_order_although_launches_overlap():
    """Every kernel of the path is launched as a programmatic dependent of the one before it, so that its blocks are
    placed while the last blocks of the previous kernel still run.  Calls must still execute strictly one after the
    other: here layer 1 takes layer 0's OUTPUT buffer as its q (rotated in place by layer 1's append) and writes its
    own output over layer 0's q, on the full 256-context batch; the result must be what the same calls give with the
    device drained between them."""
    wl = WORKLOADS["llama2_70b_gqa"]
    sh = wl.shape
    lens = wl.lengths(20240, headroom=4).astype(np.uint32)
    B = len(lens)

    def run(drain: bool):
        st = AttentionStage(sh, torch.float16, n_layers_hosted=2, max_batch=B, max_contexts=B, paged=True)
        cos, sin = rope_tables(sh.head_size, sh.seq_len, sh.rope_theta)
        st.set_rope_tables(torch.from_numpy(cos).cuda().half(), torch.from_numpy(sin).cuda().half())
        slots = st.get_contexts(np.arange(1, B + 1, dtype=np.uint32))
        row = 2 * sh.kv_dim
        for i in range(B):
            for l in range(2):
                st.prepare(int(slots[i]), l, int(lens[i]))
                st.fill_normal(st.layer_ptr(int(slots[i]), l), int(lens[i]) * row, torch.float16, 3,
                               offset=(2 * i + l) * sh.seq_len * row)
        a = torch.empty((B, sh.dim), dtype=torch.float16, device="cuda")
        b = torch.zeros_like(a)
        kv = torch.empty((B, row), dtype=torch.float16, device="cuda")
        st.fill_normal(a, a.numel(), torch.float16, 4)
        st.fill_normal(kv, kv.numel(), torch.float16, 5)
        torch.cuda.synchronize()
        st.batch_begin(slots, lens)
        st.step(0, a, kv, b)      # q = a, output -> b
        if drain:
            torch.cuda.synchronize()
        st.step(1, b, kv, a)      # q = layer 0's output, output -> over layer 0's q
        torch.cuda.synchronize()
        assert st.stats().device_error == 0
        out = (a.clone(), b.clone())
        st.close()
        return out

    a0, b0 = run(drain=True)
    a1, b1 = run(drain=False)
    assert torch.equal(a0, a1) and torch.equal(b0, b1)
    assert torch.isfinite(a0.float()).all() and float(a0.float().abs().max()) > 0


def test_copy_and_rope_in_one_call_on_foreign_rows(oracle):
    """gh_op_copy_kv_cache_apply_rope with token rows that are NOT in the stage's slots (plain device buffers): the
    pointer array travels to the device with the call, the result is that of the two operations."""
    case = cases.make_case("foreign_rows", "mini_g4", cases.BF16, [3, 200, 77, 510], seed=12, inactive=[1])
    want = oracle.layer_step(case)
    st = gpu_util.make_stage(case)
    rows_d = torch.full((case.B, 2 * case.shape.kv_dim), float("nan"), device="cuda", dtype=torch.bfloat16)
    ptrs = [rows_d[i].data_ptr() if case.active[i] else 0 for i in range(case.B)]
    q = gpu_util.to_dev(case.q, case.dtype)
    q_before = q.clone()
    st.copy_kv_cache_apply_rope(case.B, case.pos, gpu_util.to_dev(case.fcr, case.dtype), gpu_util.to_dev(case.fci, case.dtype),
                                q, ptrs, gpu_util.to_dev(case.kv_new, case.dtype))
    torch.cuda.synchronize()
    got_rows, got_q = gpu_util.to_host(rows_d, case.dtype), gpu_util.to_host(q, case.dtype)
    kvd = case.shape.kv_dim
    for i in range(case.B):
        if not case.active[i]:
            assert torch.isnan(rows_d[i].float()).all() and torch.equal(q[i], q_before[i]), "inactive prompt untouched"
            continue
        assert np.array_equal(got_rows[i][kvd:], want.rows[i][kvd:]), "V bit-exact"
        gpu_util.assert_rotation_close(got_rows[i][:kvd], want.rows[i][:kvd], case.kv_new[i][:kvd], case.dtype, f"K {i}")
        gpu_util.assert_rotation_close(got_q[i], want.q[i], case.q[i], case.dtype, f"q {i}")
    st.close()


def test_the_appended_row_is_attended_although_old_rows_are_fetched_ahead_of_the_append(oracle):
    """The decode kernel's producers start fetching a context's old rows while the append in front of the kernel has
    not run yet (it waits for the previous layer's launch to complete); the tile that holds the new row must come
    after it.  Three layers are issued back to back, without draining the device, on contexts whose positions sit
    on and around the 32-token tile boundaries, next to long contexts that keep the previous layer's launch busy.
    Every new K row is a multiple of its group's (identical) query heads, so nearly all of a head's weight lies on the
    new row: an output computed from a tile that was fetched before the append wrote it would be nowhere near."""
    wl = WORKLOADS["llama2_70b_gqa"]
    sh = wl.shape
    dtype, tdt = cases.F16, torch.float16
    rng = np.random.default_rng(31)
    pos = np.array([0, 1, 30, 31, 32, 33, 63, 64, 65, 95, 96, 127, 128, 129, 1023, 1024]
                   + list(rng.integers(2500, 4090, size=12)), dtype=np.uint32)
    B, L, row = len(pos), 3, 2 * sh.kv_dim
    group, hs = sh.n_heads // sh.n_kv_heads, sh.head_size
    st = AttentionStage(sh, tdt, n_layers_hosted=L, max_batch=B, max_contexts=B, paged=True)
    cos, sin = rope_tables(sh.head_size, sh.seq_len, sh.rope_theta)
    fcr, fci = cases.store(cos, dtype), cases.store(sin, dtype)
    st.set_rope_tables(gpu_util.to_dev(fcr, dtype), gpu_util.to_dev(fci, dtype))
    slots = st.get_contexts(np.arange(1, B + 1, dtype=np.uint32))
    layer_cases, dev = [], []
    for l in range(L):
        cache = []
        for i in range(B):
            p = int(pos[i])
            st.prepare(int(slots[i]), l, p)
            if p > 0:
                st.fill_normal(st.layer_ptr(int(slots[i]), l), p * row, tdt, 50 + l, offset=i * sh.seq_len * row)
        torch.cuda.synchronize()
        for i in range(B):
            p = int(pos[i])
            c = np.zeros((p + 1, row), dtype=cases.NP_DTYPE[dtype])
            if p > 0:
                c[:p] = gpu_util.to_host(st.layer_view(int(slots[i]), l, p), dtype)
            cache.append(c)
        u = rng.standard_normal((B, sh.n_kv_heads, 1, hs), dtype=np.float32)
        q = cases.store(np.broadcast_to(u, (B, sh.n_kv_heads, group, hs)).reshape(B, sh.dim), dtype)
        kv_new = np.concatenate([3.0 * u.reshape(B, sh.kv_dim), rng.standard_normal((B, sh.kv_dim), dtype=np.float32)], axis=1)
        kv_new = cases.store(kv_new, dtype)
        layer_cases.append(cases.Case(f"early{l}", sh, dtype, pos, np.ones(B, dtype=bool), cache, q, kv_new, fcr, fci, 31))
        dev.append((gpu_util.to_dev(q, dtype), gpu_util.to_dev(kv_new, dtype), torch.zeros((B, sh.dim), dtype=tdt, device="cuda")))
    torch.cuda.synchronize()
    st.batch_begin(slots, pos)
    for l in range(L):
        st.step(l, *dev[l])
    torch.cuda.synchronize()
    assert st.stats().device_error == 0
    for l in range(L):
        want = oracle.layer_step(layer_cases[l])
        rows = [gpu_util.to_host(st.layer_view(int(slots[i]), l, int(pos[i]) + 1)[int(pos[i])], dtype) for i in range(B)]
        got = cases.StepResult(rows, gpu_util.to_host(dev[l][0], dtype), gpu_util.to_host(dev[l][2], dtype))
        gpu_util.assert_step_close(got, want, layer_cases[l])
        # the construction holds: every head's output is its group's new V row to within rounding
        v_new = cases.as_f32(layer_cases[l].kv_new[:, sh.kv_dim:], dtype).reshape(B, sh.n_kv_heads, 1, hs)
        xb = cases.as_f32(got.xb, dtype).reshape(B, sh.n_kv_heads, group, hs)
        assert np.abs(xb - v_new).max() < 2e-2
    st.close()
