"""Parity of the CUDA path, called through the C ABI, with the CPU oracle and with the fixtures produced by
the reference's own amd64 backend.  Tolerances are the contract's: V bit-exact, rotated K/q within 1e-3
relative, attention output within 2e-2 absolute (fp16/bf16) or 1e-4 (fp32)."""
from pathlib import Path

import numpy as np
import pytest
import torch

from tests import cases, gpu_util

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"


@pytest.mark.parametrize("spec", cases.GOLDEN_SPECS, ids=lambda s: s["name"])
def test_fused_step_matches_reference_fixture(spec):
    case = cases.golden_case(spec)
    gold = np.load(GOLDEN / f"{case.name}.npz")
    want = cases.StepResult([r for r in gold["rows"]], gold["q"], gold["xb"])
    st = gpu_util.make_stage(case)
    slots = gpu_util.load_case(st, case, layer=1)
    res = gpu_util.run_step(st, case, slots, layer=1)
    gpu_util.assert_step_close(res, want, case)
    st.close()


@pytest.mark.parametrize("spec", cases.GOLDEN_SPECS[:10], ids=lambda s: s["name"])
@pytest.mark.parametrize("variant", ["generic", "paged", "chunk64", "two_calls"])
def test_fused_step_variants_match_oracle(oracle, spec, variant):
    """The same cases through the CUDA-core kernel, paged slots, the smallest split length (every context cut
    into 64-token items, so the partial-record merge runs everywhere), and append/decode as two calls."""
    case = cases.golden_case(spec)
    want = oracle.layer_step(case)
    st = gpu_util.make_stage(case, force_generic=variant == "generic", paged=variant == "paged",
                             decode_chunk=64 if variant == "chunk64" else 0)
    slots = gpu_util.load_case(st, case, layer=0)
    res = gpu_util.run_step(st, case, slots, layer=0, fused_call=variant != "two_calls")
    gpu_util.assert_step_close(res, want, case)
    st.close()


@pytest.mark.parametrize("dtype", [cases.F16, cases.BF16, cases.F32])
@pytest.mark.parametrize("shape_name", ["mini_mha", "mini_g4", "mini_g8", "mini_g16", "tiny15m"])
def test_fused_step_all_dtypes(oracle, shape_name, dtype):
    S = cases.SHAPES[shape_name].seq_len
    pos = [0, 1, 63, 64, 65, 127, 128, S // 2, S - 1]
    case = cases.make_case("dt", shape_name, dtype, pos, seed=1000 + dtype)
    want = oracle.layer_step(case)
    st = gpu_util.make_stage(case, decode_chunk=128)
    slots = gpu_util.load_case(st, case, layer=1)
    res = gpu_util.run_step(st, case, slots, layer=1)
    gpu_util.assert_step_close(res, want, case)
    st.close()


def test_consecutive_decode_steps_grow_the_cache(oracle):
    """Several layer-steps in a row on two layers: each step sees the rows the previous ones appended."""
    case = cases.make_case("multi", "mini_g8", cases.F16, [10, 62, 300], seed=5)
    st = gpu_util.make_stage(case, layers=2, paged=True)
    slots = {l: None for l in (0, 1)}
    slots = gpu_util.load_case(st, case, layer=0)
    for i in range(case.B):  # same pre-filled rows in layer 1
        p = int(case.pos[i])
        st.prepare(int(slots[i]), 1, p, False)
        st.layer_view(int(slots[i]), 1, p).copy_(gpu_util.to_dev(case.cache[i][:p], case.dtype))
    cur = case
    rng = np.random.default_rng(99)
    for step in range(4):
        want = oracle.layer_step(cur)
        for layer in (0, 1):
            res = gpu_util.run_step(st, cur, slots, layer)
            gpu_util.assert_step_close(res, want, cur)
        # next token: the cache now holds the appended rows
        new_cache = [np.concatenate([c[: int(p)], r[None, :], np.zeros((1, c.shape[1]), c.dtype)])
                     for c, p, r in zip(cur.cache, cur.pos, want.rows)]
        cur = cases.Case(cur.name, cur.shape, cur.dtype, cur.pos + 1, cur.active, new_cache,
                         rng.standard_normal(cur.q.shape).astype(cur.q.dtype),
                         rng.standard_normal(cur.kv_new.shape).astype(cur.kv_new.dtype), cur.fcr, cur.fci)
    st.close()


@pytest.mark.parametrize("dtype", [cases.F16, cases.F32, cases.BF16])
def test_reference_operations_one_by_one(oracle, dtype):
    """copy_kv_cache, apply_rope, attention_0_gemm, attention_softmax, attention_2_gemm with the reference's
    argument lists, each checked on its own output (including the score matrix `att`)."""
    case = cases.make_case("ops", "mini_g4", dtype, [0, 17, 200, 90], seed=21, inactive=[3])
    sh = case.shape
    want = oracle.layer_step(case, keep_att=True)
    st = gpu_util.make_stage(case)
    slots = gpu_util.load_case(st, case, layer=1)
    layer_ptrs = [st.layer_ptr(int(s), 1) if s >= 0 else 0 for s in slots]
    token_ptrs = [st.token_ptr(int(s), 1, int(p)) if s >= 0 else 0 for s, p in zip(slots, case.pos)]
    q = gpu_util.to_dev(case.q, dtype)
    kv = gpu_util.to_dev(case.kv_new, dtype)
    att = torch.zeros((case.B, sh.n_heads, sh.seq_len), dtype=q.dtype, device="cuda")
    xb = torch.zeros_like(q)

    st.copy_kv_cache(token_ptrs, kv, case.B)
    torch.cuda.synchronize()
    for i in range(case.B):
        if case.active[i]:
            row = gpu_util.to_host(st.layer_view(int(slots[i]), 1, int(case.pos[i]) + 1)[int(case.pos[i])], dtype)
            assert np.array_equal(row.view(np.uint8), case.kv_new[i].view(np.uint8)), "raw copy before RoPE"

    st.apply_rope(case.B, case.pos, gpu_util.to_dev(case.fcr, dtype), gpu_util.to_dev(case.fci, dtype), q, token_ptrs)
    st.attention_0_gemm(q, layer_ptrs, att, case.B, case.pos)
    st.attention_softmax(att, case.pos, None, case.B)
    st.attention_2_gemm(att, layer_ptrs, xb, case.B, case.pos)
    torch.cuda.synchronize()

    rows = [gpu_util.to_host(st.layer_view(int(s), 1, int(p) + 1)[int(p)], dtype) if s >= 0 else None
            for s, p in zip(slots, case.pos)]
    res = cases.StepResult(rows, gpu_util.to_host(q, dtype), gpu_util.to_host(xb, dtype))
    # unfused ops round where the reference rounds: much tighter than the contract
    gpu_util.assert_step_close(res, want, case, xb_atol={cases.F32: 2e-6, cases.F16: 2e-3, cases.BF16: 1.6e-2}[dtype])
    att_h = gpu_util.to_host(att, dtype)
    for i, p in enumerate(case.pos):
        if case.active[i]:
            np.testing.assert_allclose(cases.as_f32(att_h[i, :, : p + 1], dtype),
                                       cases.as_f32(want.att[i, :, : p + 1], dtype), rtol=0,
                                       atol={cases.F32: 1e-6, cases.F16: 1e-3, cases.BF16: 8e-3}[dtype])

    # the fused stand-in for the three attention calls gives the same xb from the same arguments
    xb2 = torch.zeros_like(q)
    st.attention_fused(q, layer_ptrs, xb2, case.B, case.pos)
    torch.cuda.synchronize()
    for i in range(case.B):
        if case.active[i]:
            np.testing.assert_allclose(cases.as_f32(gpu_util.to_host(xb2, dtype)[i], dtype),
                                       cases.as_f32(want.xb[i], dtype), rtol=0, atol=cases.TOL_XB[dtype])
    # inactive prompts are skipped: their xb row is untouched
    assert torch.count_nonzero(xb[3]) == 0 and torch.count_nonzero(xb2[3]) == 0
    st.close()


def test_attention_fused_on_foreign_memory(oracle):
    """Layer contexts that do not live in the stage's own arena (plain cudaMalloc'd buffers) still work."""
    case = cases.make_case("foreign", "mini_g8", cases.F16, [70, 400], seed=31)
    want = oracle.layer_step(case)
    st = gpu_util.make_stage(case)
    bufs = []
    for i in range(case.B):
        c = case.cache[i].copy()
        c[int(case.pos[i])] = want.rows[i]
        bufs.append(gpu_util.to_dev(c, case.dtype))
    q = gpu_util.to_dev(want.q, case.dtype)
    xb = torch.zeros_like(q)
    st.attention_fused(q, [b.data_ptr() for b in bufs], xb, case.B, case.pos)
    torch.cuda.synchronize()
    assert st.stats().last_kernel == 0
    np.testing.assert_allclose(xb.float().cpu().numpy(), want.xb.astype(np.float32), rtol=0, atol=cases.TOL_XB[cases.F16])
    st.close()


@pytest.mark.parametrize("io_dtype", [cases.F16, cases.F32])
def test_forward_attention_with_host_buffers(oracle, io_dtype):
    """The piped-mode entry point: q and the new [K,V] rows arrive in host memory, possibly in another dtype
    (the reference mixes fp16 pre/post-attention with fp32 attention), and xb goes back to the host."""
    case = cases.make_case("host", "mini_g8", cases.F16, [5, 64, 333], seed=41)
    want = oracle.layer_step(case)
    st = gpu_util.make_stage(case)
    slots = gpu_util.load_case(st, case, layer=0)
    npdt = cases.NP_DTYPE[io_dtype]
    q_h = torch.from_numpy(case.q.astype(npdt)).pin_memory()
    kv_h = torch.from_numpy(case.kv_new.astype(npdt)).pin_memory()
    xb_h = torch.zeros_like(q_h).pin_memory()
    st.batch_begin(slots, case.pos)
    st.forward_attention_host(0, io_dtype, q_h, kv_h, xb_h)
    torch.cuda.synchronize()
    np.testing.assert_allclose(xb_h.numpy().astype(np.float32), want.xb.astype(np.float32), rtol=0,
                               atol=cases.TOL_XB[cases.F16])
    st.close()


def test_convert_and_copy():
    case = cases.make_case("cc", "tiny15m", cases.F32, [3], seed=1)
    st = gpu_util.make_stage(case)
    x = np.random.default_rng(3).standard_normal(5000).astype(np.float32)
    d16 = torch.zeros(5000, dtype=torch.float16, device="cuda")
    st.convert_and_copy(d16, torch.float16, x, torch.float32, 5000, 0)  # host fp32 -> device fp16
    assert np.array_equal(d16.cpu().numpy(), x.astype(np.float16))
    back = np.zeros(5000, dtype=np.float32)
    st.convert_and_copy(back, torch.float32, d16, torch.float16, 5000, 1)  # device fp16 -> host fp32
    assert np.array_equal(back, x.astype(np.float16).astype(np.float32))
    same = np.zeros(5000, dtype=np.float16)
    st.convert_and_copy(same, torch.float16, d16, torch.float16, 5000, 1)
    assert np.array_equal(same, x.astype(np.float16))
    with pytest.raises(Exception):
        st.convert_and_copy(same, torch.float16, same, torch.float16, 10, 3)  # host-to-host is rejected
    st.close()


def test_layers_in_flight_on_several_streams(oracle):
    """One batch, four layers, each layer's host-buffer call on its own stream (what an end-to-end driver does to
    overlap copies with kernels).  Every context is cut into 64-token items, so every launch uses split partial
    records and arrival counters; launches in flight together must not share them."""
    pos = [130, 511, 64, 300, 1, 447]
    layer_cases = [cases.make_case(f"l{l}", "mini_g8", cases.F16, pos, seed=500 + l) for l in range(4)]
    wants = [oracle.layer_step(c) for c in layer_cases]
    st = gpu_util.make_stage(layer_cases[0], layers=4, decode_chunk=64, paged=True)
    slots = gpu_util.load_case(st, layer_cases[0], layer=0)
    for l in range(1, 4):
        for i, p in enumerate(pos):
            st.prepare(int(slots[i]), l, p, False)
            if p > 0:
                st.layer_view(int(slots[i]), l, p).copy_(gpu_util.to_dev(layer_cases[l].cache[i][:p], cases.F16))
    torch.cuda.synchronize()
    q_h = [torch.from_numpy(c.q).pin_memory() for c in layer_cases]
    kv_h = [torch.from_numpy(c.kv_new).pin_memory() for c in layer_cases]
    xb_h = [torch.zeros_like(q).pin_memory() for q in q_h]
    streams = [torch.cuda.Stream() for _ in range(3)]
    main = torch.cuda.current_stream()
    for rep in range(3):  # repeat so that scratch sets and staging buffers are reused across streams
        st.batch_begin(slots, pos, stream=main)
        ready = torch.cuda.Event()
        ready.record(main)
        for s in streams:
            s.wait_event(ready)
        for l in range(4):
            st.forward_attention_host(l, cases.F16, q_h[l], kv_h[l], xb_h[l], stream=streams[(l + rep) % 3])
        torch.cuda.synchronize()
        for l in range(4):
            np.testing.assert_allclose(xb_h[l].numpy().astype(np.float32), wants[l].xb.astype(np.float32), rtol=0,
                                       atol=cases.TOL_XB[cases.F16], err_msg=f"layer {l}, repetition {rep}")
    assert st.stats().device_error == 0
    st.close()


@pytest.mark.parametrize("shape_name,dtype", [("mini_g4", cases.BF16), ("mini_g8", cases.F16), ("tiny15m", cases.F32),
                                              ("mini_mha", cases.F16), ("mini_g16", cases.F16), ("mini_g4", cases.F16)])
def test_prefill_chunk_equals_token_by_token_reference_steps(oracle, shape_name, dtype):
    """A multi-token prompt chunk in one call.  The reference has no such operation — it feeds prompts one token
    per forward pass — so the oracle is n_tokens consecutive reference layer-steps on a growing cache.  Fresh slot,
    short prefix, longer prefix; 37 tokens leave the last query block ragged."""
    gpu_util.check_prefill(oracle, shape_name, dtype, pos0=[0, 5, 100], chunk_lens=[37])


@pytest.mark.parametrize("dtype", [cases.F16, cases.BF16])
def test_prefill_in_several_chunks_continues_where_the_last_one_ended(oracle, dtype):
    """A prompt fed as three chunks of different sizes: the later chunks attend to rows the earlier calls wrote."""
    kernel = gpu_util.check_prefill(oracle, "mini_g4", dtype, pos0=[0, 17], chunk_lens=[64, 40, 9])
    assert kernel == 2, "head size 128 in a 16-bit type runs the tcgen05 kernel"


@pytest.mark.parametrize("shape_name,dtype", [("mini_g4", cases.BF16), ("mini_g8", cases.F16)])
def test_prefill_with_scores_that_keep_growing_along_the_keys(oracle, shape_name, dtype):
    """The tcgen05 kernel lets a row's running maximum lag behind by up to 2^8 and rescales its accumulator only
    then.  Keys that grow with their position push every row's maximum up by much more than that from tile to
    tile, over several tiles of 64 keys, with and without a cached prefix.

    The yardstick for the attention output here is the exact softmax: the reference stores its scores in the 16-bit
    type between its three operations (src/arch/amd64/llama2/ops.hh:170-298), and at scores of this size that rounding
    alone moves the reference's own output by up to 0.5."""
    gpu_util.check_prefill(oracle, shape_name, dtype, pos0=[0, 150], chunk_lens=[200], k_ramp=0.125, seed=5, exact_attention=True)


def test_prefill_skips_inactive_contexts_and_refuses_chunks_past_the_slot(oracle):
    """Slot -1 = inactive prompt: nothing of it is appended or written, the others are unaffected.  A chunk that would
    run past the slot capacity is refused before anything is launched."""
    shape_name, dtype, T = "mini_g4", cases.F16, 40
    sh = cases.SHAPES[shape_name]
    pos0 = [0, 30, 11]
    base = cases.make_case("pfi", shape_name, dtype, [p + T - 1 for p in pos0], seed=21)
    rng = np.random.default_rng(8)
    q = cases.store(rng.standard_normal((3, T, sh.dim), dtype=np.float32), dtype)
    kv = cases.store(rng.standard_normal((3, T, 2 * sh.kv_dim), dtype=np.float32), dtype)
    st = gpu_util.make_stage(base, layers=1, paged=True)
    slots = st.get_contexts(np.arange(1, 4, dtype=np.uint32)).astype(np.int32)
    for i, p in enumerate(pos0):
        st.prepare(int(slots[i]), 0, max(p, 1) - 1, False)
        if p > 0:
            st.layer_view(int(slots[i]), 0, p).copy_(gpu_util.to_dev(base.cache[i][:p], dtype))
    q_d, kv_d = gpu_util.to_dev(q, dtype), gpu_util.to_dev(kv, dtype)
    xb_all, xb_two = torch.zeros_like(q_d), torch.full_like(q_d, 7.0)
    st.prefill_chunk(0, slots, pos0, T, q_d.clone(), kv_d, xb_all)      # everybody
    with_middle = gpu_util.to_host(xb_all, dtype)
    mapped = st.stats().bytes_mapped
    for i, p in enumerate(pos0):  # start again from the same prefixes
        st.layer_view(int(slots[i]), 0, p + T)[p:].zero_()
    masked = slots.copy()
    masked[1] = -1
    q_in = q_d.clone()
    st.prefill_chunk(0, masked, pos0, T, q_in, kv_d, xb_two)            # the middle one inactive
    torch.cuda.synchronize()
    got = gpu_util.to_host(xb_two, dtype)
    assert np.array_equal(got[0], with_middle[0]) and np.array_equal(got[2], with_middle[2])
    assert (got[1].astype(np.float32) == 7.0).all(), "xb of the inactive prompt is not written"
    assert torch.equal(q_in[1], q_d[1]), "q of the inactive prompt is not rotated"
    assert not st.layer_view(int(slots[1]), 0, pos0[1] + T)[pos0[1]:].any(), "nothing is appended for it"
    assert st.stats().bytes_mapped == mapped
    launches = st.stats().kernel_launches
    with pytest.raises(gpu_util.GlinthawkAttnError) as e:
        st.prefill_chunk(0, slots, [0, sh.seq_len - T + 1, 0], T, q_d, kv_d, xb_all)
    assert e.value.status == gpu_util.GH_ERR_CAPACITY and st.stats().kernel_launches == launches
    assert st.stats().device_error == 0
    st.close()


@pytest.mark.parametrize("force_generic", [False, True])
def test_garbage_beyond_the_current_position_is_never_read_into_the_result(oracle, force_generic):
    """A slot keeps whatever its previous owner left behind the current position (the reference never clears
    contexts either).  NaNs and infinities planted in every row after `pos` must not reach the output, although
    the tensor-core kernel fetches whole 32-token tiles that include those rows."""
    pos = [0, 5, 30, 31, 32, 33, 63, 64, 100, 254]
    case = cases.make_case("nan", "mini_g8", cases.F16, pos, seed=71)
    want = oracle.layer_step(case)
    st = gpu_util.make_stage(case, force_generic=force_generic)
    slots = gpu_util.load_case(st, case, layer=0)
    for i, p in enumerate(pos):
        tail = st.layer_view(int(slots[i]), 0, case.shape.seq_len)[p + 1:]
        tail[0::3] = float("nan")
        tail[1::3] = float("inf")
        tail[2::3] = -float("inf")
    res = gpu_util.run_step(st, case, slots, layer=0)
    assert np.isfinite(cases.as_f32(res.xb, cases.F16)).all()
    gpu_util.assert_step_close(res, want, case)
    st.close()


def test_largest_batch_and_all_inactive_batch(oracle):
    """MAX_BATCH_SIZE (1024, src/models/llama2/base.hh:26) contexts in one call, a third of them inactive; then a
    batch with no active prompt at all, which must leave every buffer untouched."""
    rng = np.random.default_rng(8)
    B = 1024
    pos = rng.integers(0, 48, size=B)
    pos[:4] = [0, 47, 31, 32]
    inactive = list(range(2, B, 3))
    case = cases.make_case("big", "mini_g4", cases.F16, pos, seed=72, inactive=inactive)
    want = oracle.layer_step(case)
    st = gpu_util.make_stage(case, layers=1)
    slots = gpu_util.load_case(st, case, layer=0)
    res = gpu_util.run_step(st, case, slots, layer=0)
    gpu_util.assert_step_close(res, want, case)
    q = gpu_util.to_dev(case.q, cases.F16)
    xb = torch.full_like(q, 3.0)
    q0 = q.clone()
    none = np.full(B, -1, dtype=np.int32)
    st.batch_begin(none, case.pos)
    st.step(0, q, gpu_util.to_dev(case.kv_new, cases.F16), xb)
    torch.cuda.synchronize()
    assert torch.equal(q, q0) and bool((xb == 3.0).all())
    st.close()


def test_slot_reuse_after_release_starts_clean(oracle):
    """A released slot is handed to the next context (contextman.hh:193-195 recycles contexts the same way); the new
    context's results depend only on what it appended itself."""
    first = cases.make_case("a", "mini_g8", cases.F16, [400], seed=81)
    second = cases.make_case("b", "mini_g8", cases.F16, [37], seed=82)
    for paged in (False, True):
        st = gpu_util.make_stage(first, paged=paged, max_contexts=1)
        slots = gpu_util.load_case(st, first, layer=0, first_id=10)
        gpu_util.run_step(st, first, slots, layer=0)
        assert st.release_context(10)
        slots2 = gpu_util.load_case(st, second, layer=0, first_id=11)
        assert slots2[0] == slots[0]
        res = gpu_util.run_step(st, second, slots2, layer=0)
        gpu_util.assert_step_close(res, oracle.layer_step(second), second)
        st.close()
