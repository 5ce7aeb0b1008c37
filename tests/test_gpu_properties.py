"""Size-independent properties at the benchmark configurations' full sizes (where the CPU oracle would take minutes):
constant-V reproduction, uniform attention, split invariance, agreement of the two decode kernels, batch-order
invariance, and the append round trip.  Inputs are generated on the device."""
import numpy as np
import pytest
import torch

from glinthawk_b200.rope import rope_tables
from glinthawk_b200.shapes import SHAPES
from glinthawk_b200.stage import AttentionStage
from glinthawk_b200.workload import WORKLOADS

pytestmark = pytest.mark.gpu
TDT = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}


def build(workload: str, *, batch=None, layers=1, seed=7, headroom=4, **kw):
    wl = WORKLOADS[workload]
    sh, tdt = wl.shape, TDT[wl.dtype]
    B = batch or wl.batch
    lens = wl.lengths(seed, headroom)[:B]
    st = AttentionStage(sh, tdt, n_layers_hosted=layers, max_batch=B, max_contexts=B, paged=True, **kw)
    cos, sin = rope_tables(sh.head_size, sh.seq_len, sh.rope_theta)
    st.set_rope_tables(torch.from_numpy(cos).cuda().to(tdt), torch.from_numpy(sin).cuda().to(tdt))
    slots = st.get_contexts(np.arange(1, B + 1, dtype=np.uint32))
    row = 2 * sh.kv_dim
    for i in range(B):
        for l in range(layers):
            st.prepare(int(slots[i]), l, int(lens[i]) + headroom - 1)
            st.fill_normal(st.layer_ptr(int(slots[i]), l), int(lens[i]) * row, tdt, seed,
                           offset=(i * layers + l) * sh.seq_len * row)
    q = torch.empty((B, sh.dim), dtype=tdt, device="cuda")
    kv = torch.empty((B, row), dtype=tdt, device="cuda")
    st.fill_normal(q, q.numel(), tdt, seed + 1)
    st.fill_normal(kv, kv.numel(), tdt, seed + 2)
    torch.cuda.synchronize()
    return wl, st, slots, lens, q, kv


def decode_only(st, slots, pos, q, layer=0):
    xb = torch.zeros_like(q)
    st.batch_begin(slots, pos)
    st.decode(layer, q, xb)
    torch.cuda.synchronize()
    assert st.stats().device_error == 0
    return xb


@pytest.mark.parametrize("workload", ["llama2_7b_layer", "llama2_70b_gqa", "llama3_8b_decode"])
def test_append_round_trip_and_softmax_weights_sum_to_one(workload):
    wl, st, slots, lens, q, kv = build(workload, batch=64)
    sh = wl.shape
    pos = lens.astype(np.uint32)  # the token being appended
    q0 = q.clone()
    xb = torch.zeros_like(q)
    st.batch_begin(slots, pos)
    st.step(0, q, kv, xb)
    torch.cuda.synchronize()
    kvd = sh.kv_dim
    for i in range(0, len(slots), 7):
        row = st.layer_view(int(slots[i]), 0, int(pos[i]) + 1)[int(pos[i])]
        assert torch.equal(row[kvd:], kv[i, kvd:]), "V row must be a bit-exact copy"
        # a rotation preserves the norm of every (even, odd) pair
        k_in = kv[i, :kvd].float().view(-1, 2)
        k_out = row[:kvd].float().view(-1, 2)
        torch.testing.assert_close(k_out.norm(dim=1), k_in.norm(dim=1), rtol=4e-3 if wl.dtype == "f16" else 2e-2,
                                   atol=4e-3 if wl.dtype == "f16" else 2e-2)
        torch.testing.assert_close(q[i].float().view(-1, 2).norm(dim=1), q0[i].float().view(-1, 2).norm(dim=1),
                                   rtol=4e-3 if wl.dtype == "f16" else 2e-2, atol=4e-3 if wl.dtype == "f16" else 2e-2)
    # position 0 rotates by angle 0: appending at pos 0 leaves K and q unchanged
    fresh = st.get_contexts  # noqa: F841  (slots are all taken; reuse slot 0 from scratch)
    st.prepare(int(slots[0]), 0, 0, can_release=True)
    q1 = q0[:1].clone()
    st.batch_begin(slots[:1], np.zeros(1, dtype=np.uint32))
    st.append(0, q1, kv[:1])
    torch.cuda.synchronize()
    assert torch.equal(q1, q0[:1]) and torch.equal(st.layer_view(int(slots[0]), 0, 1)[0], kv[0])

    # constant V along the token axis: the output equals that constant whatever the scores are
    wl, st2, slots2, lens2, q2, _ = build(workload, batch=64, seed=11)
    const = torch.linspace(-2, 2, sh.kv_dim, device="cuda").to(q2.dtype)
    for i in range(len(slots2)):
        st2.layer_view(int(slots2[i]), 0, int(lens2[i]))[:, kvd:] = const
    xb2 = decode_only(st2, slots2, (lens2 - 1).astype(np.uint32), q2)
    want = const.view(sh.n_kv_heads, 1, sh.head_size).expand(-1, sh.gqa_size, -1).reshape(-1).float()
    tol = 4e-3 if wl.dtype == "f16" else 3e-2
    assert float((xb2.float() - want).abs().max()) <= tol
    st.close()
    st2.close()


@pytest.mark.parametrize("workload", ["llama2_7b_layer", "llama2_70b_gqa", "llama3_8b_decode"])
def test_uniform_attention_is_the_mean_of_v(workload):
    wl, st, slots, lens, q, _ = build(workload, batch=32)
    sh = wl.shape
    q.zero_()  # all scores equal -> uniform weights
    pos = (lens - 1).astype(np.uint32)
    xb = decode_only(st, slots, pos, q)
    for i in range(0, len(slots), 5):
        v = st.layer_view(int(slots[i]), 0, int(lens[i]))[:, sh.kv_dim:].float().mean(dim=0)
        want = v.view(sh.n_kv_heads, 1, sh.head_size).expand(-1, sh.gqa_size, -1).reshape(-1)
        torch.testing.assert_close(xb[i].float(), want, rtol=0, atol=2e-3 if wl.dtype == "f16" else 1e-2)
    st.close()


@pytest.mark.parametrize("workload", ["llama2_7b_layer", "llama2_70b_gqa", "llama3_8b_decode"])
def test_split_invariance_and_kernel_agreement(workload):
    """Cutting contexts into 64-token or 512-token items, or using the CUDA-core kernel, changes only rounding."""
    results = {}
    for name, kw in (("auto", {}), ("chunk64", dict(decode_chunk=64)), ("chunk512", dict(decode_chunk=512)),
                     ("generic", dict(force_generic=True))):
        wl, st, slots, lens, q, _ = build(workload, batch=48, **kw)
        results[name] = decode_only(st, slots, (lens - 1).astype(np.uint32), q).float()
        if name != "generic":
            assert st.stats().last_kernel == 1
        st.close()
    tol = 2e-3 if WORKLOADS[workload].dtype == "f16" else 1.5e-2
    for name in ("chunk64", "chunk512", "generic"):
        assert float((results[name] - results["auto"]).abs().max()) <= tol, name


def test_batch_order_does_not_matter():
    wl, st, slots, lens, q, _ = build("llama2_70b_gqa", batch=96)
    pos = (lens - 1).astype(np.uint32)
    xb = decode_only(st, slots, pos, q)
    perm = np.random.default_rng(0).permutation(len(slots))
    xb_p = decode_only(st, slots[perm], pos[perm], q[torch.from_numpy(perm).cuda()].contiguous())
    assert torch.equal(xb_p, xb[torch.from_numpy(perm).cuda()]), "a context's result must not depend on its neighbours"
    # inactive prompts interleaved: the others are unaffected, their own rows untouched
    s2 = slots.copy()
    s2[::3] = -1
    xb_i = torch.full_like(q, 7.0)
    st.batch_begin(s2, pos)
    st.decode(0, q, xb_i)
    torch.cuda.synchronize()
    keep = torch.from_numpy(s2 >= 0).cuda()
    # (with a third of the batch gone the planner may cut long contexts that it left whole before: same values up to
    # the rounding of a different summation order, not the same bits)
    assert float((xb_i[keep].float() - xb[keep].float()).abs().max()) <= 2e-3 and bool((xb_i[~keep] == 7.0).all())
    st.close()


def test_full_llama2_70b_batch_many_steps_stay_finite_and_consistent():
    """256 contexts, 2 layers, 6 consecutive decode steps on paged slots: positions advance, pages are mapped as
    contexts grow, results stay finite and the two layers (filled identically) agree bit for bit."""
    wl = WORKLOADS["llama2_70b_gqa"]
    sh, tdt = wl.shape, torch.float16
    B, steps = 256, 6
    lens = wl.lengths(3, steps + 1)
    lens[:8] = [15, 16, 63, 64, 511, 512, 1023, 4096 - steps - 1]  # page and tile edges
    st = AttentionStage(sh, tdt, n_layers_hosted=2, max_batch=B, max_contexts=B, paged=True)
    cos, sin = rope_tables(sh.head_size, sh.seq_len, sh.rope_theta)
    st.set_rope_tables(torch.from_numpy(cos).cuda().half(), torch.from_numpy(sin).cuda().half())
    slots = st.get_contexts(np.arange(1, B + 1, dtype=np.uint32))
    row = 2 * sh.kv_dim
    for i in range(B):
        for l in range(2):
            st.prepare(int(slots[i]), l, int(lens[i]) - 1)  # only what is cached; growth maps more on demand
            st.fill_normal(st.layer_ptr(int(slots[i]), l), int(lens[i]) * row, tdt, 5, offset=i * sh.seq_len * row)
    mapped0 = st.stats().bytes_mapped
    pos = lens.astype(np.uint32)
    for step in range(steps):
        q = torch.empty((B, sh.dim), dtype=tdt, device="cuda")
        kv = torch.empty((B, row), dtype=tdt, device="cuda")
        st.fill_normal(q, q.numel(), tdt, 100 + step)
        st.fill_normal(kv, kv.numel(), tdt, 200 + step)
        outs = []
        st.batch_begin(slots, pos)
        for l in range(2):
            ql, xb = q.clone(), torch.zeros_like(q)
            st.step(l, ql, kv, xb)
            outs.append(xb)
        torch.cuda.synchronize()
        assert bool(torch.isfinite(outs[0]).all()) and torch.equal(outs[0], outs[1])
        assert float(outs[0].float().abs().max()) < 8.0
        pos += 1
    assert st.stats().bytes_mapped > mapped0 and st.stats().device_error == 0
    st.close()


def test_pipelined_layer_steps_give_the_same_bits_as_strict_ones():
    """pipeline_steps = 1 lets the append launch of the next layer-step begin while the decode launch before it is
    still running.  With separate q / kv / xb buffers per layer (what the option demands) every layer's output and
    every appended row must be bit-identical to the strictly ordered run, over several steps of 8 layers at the
    benchmark's batch."""
    outs = []
    for pipelined in (False, True):
        wl, st, slots, lens, q, kv = build("llama2_70b_gqa", batch=256, layers=8, headroom=8, pipeline_steps=pipelined)
        sh = wl.shape
        tdt = q.dtype
        qs = torch.empty((8, *q.shape), dtype=tdt, device="cuda")
        kvs = torch.empty((8, *kv.shape), dtype=tdt, device="cuda")
        st.fill_normal(qs, qs.numel(), tdt, 31)
        st.fill_normal(kvs, kvs.numel(), tdt, 32)
        xbs = torch.zeros_like(qs)
        pos = lens.astype(np.uint32).copy()
        for _ in range(3):
            st.batch_begin(slots, pos)
            for l in range(8):
                st.step(l, qs[l], kvs[l], xbs[l])
            pos += 1
        torch.cuda.synchronize()
        assert st.stats().device_error == 0
        rows = torch.stack([st.layer_view(int(slots[i]), 7, int(pos[i]))[-3:].clone() for i in range(0, 256, 17)])
        outs.append((xbs.clone(), qs.clone(), rows))
        st.close()
    for a, b in zip(*outs):
        assert torch.equal(a, b)

