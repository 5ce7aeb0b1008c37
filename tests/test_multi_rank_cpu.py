"""The N > 1 path on CPU ranks (gloo, world size 2): request sharding and the rank reductions bench.py relies on."""
import os
import socket

import numpy as np
import torch.distributed as dist
import torch.multiprocessing as mp

from glinthawk_b200 import dist_util
from glinthawk_b200.stage import plan_batch
from glinthawk_b200.workload import WORKLOADS, algorithmic_bytes, assign_contexts


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        wl = WORKLOADS["llama2_70b_gqa"]
        assert dist_util.rank_world() == (rank, world, rank)
        # weak scaling: every rank has its own 256 contexts
        weak = dist_util.weak_scaling_lengths(wl, 20240, rank, headroom=16)
        # strong scaling: one request set, divided without communication
        idx, lens = dist_util.strong_scaling_lengths(wl, 20240, rank, world, headroom=16)
        items, chunk = plan_batch(lens.astype(np.uint32), blocks_per_item=wl.shape.n_kv_heads)
        covered = sum(int(e - b) for _, b, e, _ in items)
        total_tokens = dist_util.sum_over_ranks(float((lens + 1).sum()))
        total_ctx = dist_util.sum_over_ranks(float(len(idx)))
        slowest = dist_util.max_over_ranks(10.0 + rank)  # the slowest rank decides the reported time
        dist.barrier()
        out.put((rank, weak[:4].tolist(), idx.tolist(), int((lens + 1).sum()), covered, total_tokens, total_ctx, slowest))
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_shard_requests_without_overlap():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, out)) for r in range(world)]
    for p in procs:
        p.start()
    results = sorted(out.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    wl = WORKLOADS["llama2_70b_gqa"]
    lens = wl.lengths(20240, 16)
    (r0, weak0, idx0, tok0, cov0, total_tokens, total_ctx, slowest), (r1, weak1, idx1, tok1, cov1, *_rest) = results
    assert weak0 != weak1, "weak scaling: every rank has its own contexts (same lengths, different order)"
    assert sorted(idx0 + idx1) == list(range(wl.batch)) and not set(idx0) & set(idx1)
    assert tok0 == cov0 and tok1 == cov1, "every cached token is covered by exactly one work item"
    assert total_tokens == float((lens + 1).sum()) and total_ctx == wl.batch
    assert abs(tok0 - tok1) <= lens.max() + 1, "token load is balanced to within one context"
    assert slowest == 11.0


def test_assign_contexts_balances_tokens_not_counts():
    rng = np.random.default_rng(5)
    lens = np.clip(np.rint(np.exp(rng.normal(np.log(1024), 0.8, 256))), 16, 4096).astype(np.int64)
    for n in (1, 2, 4, 8):
        parts = assign_contexts(lens, n)
        assert sorted(np.concatenate(parts).tolist()) == list(range(256))
        loads = [int((lens[p] + 1).sum()) for p in parts]
        assert max(loads) - min(loads) <= lens.max() + 1
    # degenerate: more ranks than contexts leaves some ranks empty but loses nothing
    parts = assign_contexts([5, 9], 4)
    assert sorted(np.concatenate(parts).tolist()) == [0, 1] and sum(len(p) == 0 for p in parts) == 2


def test_algorithmic_bytes_formula():
    sh = WORKLOADS["llama2_70b_gqa"].shape
    b = algorithmic_bytes([1, 100], sh, 2)
    row = 2 * 1024 * 2
    assert b["kv_read"] == 101 * row and b["appended"] == 2 * row
    assert b["decode_kernel"] == 101 * row + 2 * 2 * 8192 * 2


def _handoff_worker(rank: int, world: int, port: int, out):
    import torch

    from glinthawk_b200.handoff import AttentionLink, StageShapes, run_attention_rank, run_dense_rank

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        shapes = StageShapes(batch=6, dim=64, row_elems=32, dtype=torch.float32, device="cpu")
        link = AttentionLink(peer=1 - rank, shapes=shapes)
        n_layers = 5
        if rank == 0:  # dense stages: produce q / kv, consume xb
            got = {}
            gen = torch.Generator().manual_seed(3)
            inputs = [(torch.randn(6, 64, generator=gen), torch.randn(6, 32, generator=gen)) for _ in range(n_layers)]
            run_dense_rank(link, n_layers, lambda l: inputs[l], lambda l, xb: got.__setitem__(l, xb.clone()))
            ok = all(torch.allclose(got[l], inputs[l][0] * 2 + inputs[l][1].sum(dim=1, keepdim=True) + l)
                     for l in range(n_layers))
            out.put(("dense", ok))
        else:  # attention rank: a stand-in for the attention step with a checkable result
            run_attention_rank(link, n_layers, lambda l, q, kv: q * 2 + kv.sum(dim=1, keepdim=True) + l)
            out.put(("attention", True))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def _layer_link_worker(rank: int, world: int, port: int, out):
    import torch

    from glinthawk_b200.handoff import LayerLink, attention_side_step, dense_side_step

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        link = LayerLink(1 - rank, dist.new_group([0, 1]), dist.new_group([0, 1]))
        n_layers, B = 7, 5
        gen = torch.Generator().manual_seed(11)
        q_src, kv_src = torch.randn(n_layers, B, 64, generator=gen), torch.randn(n_layers, B, 32, generator=gen)
        for step in range(2):
            if rank == 0:
                xb_rx = torch.zeros(n_layers, B, 64)
                dense_side_step(link, n_layers, q_src + step, kv_src, xb_rx)
                want = (q_src + step) * 2 + kv_src.sum(dim=2, keepdim=True) + torch.arange(n_layers).view(-1, 1, 1)
                out.put(("dense", step, bool(torch.allclose(xb_rx, want))))
            else:
                q, kv, xb = torch.zeros(n_layers, B, 64), torch.zeros(n_layers, B, 32), torch.zeros(n_layers, B, 64)

                def step_layer(l):
                    xb[l] = q[l] * 2 + kv[l].sum(dim=1, keepdim=True) + l

                attention_side_step(link, n_layers, q, kv, xb, step_layer)
                out.put(("attention", step, True))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_layer_by_layer_handoff_with_one_group_per_direction():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = [ctx.Process(target=_layer_link_worker, args=(r, world, port, out)) for r in range(world)]
    for p in procs:
        p.start()
    results = [out.get(timeout=120) for _ in range(4)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(ok for _, _, ok in results) and {(s, st) for s, st, _ in results} == {
        ("dense", 0), ("dense", 1), ("attention", 0), ("attention", 1)}


def test_stage_handoff_protocol_between_two_ranks():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = [ctx.Process(target=_handoff_worker, args=(r, world, port, out)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict(out.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert results == {"dense": True, "attention": True}


def test_reference_arm_under_torchrun_prints_one_line_from_rank_zero(tmp_path):
    """`bench.py --impl reference` launched the way the multi-GPU runs launch it: rank 0 times the reference's CPU
    code and prints the JSON line, the other rank leaves with status 0 and prints nothing.  (No GPU involved.)"""
    import json
    import subprocess
    import sys
    from pathlib import Path

    import pytest

    from tests import cases
    if cases.Reference.try_load() is None:
        pytest.skip("the reference library is not built here")
    root = Path(__file__).resolve().parents[1]
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), str(root / "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1",
           "--warmup", "1", "--layers", "1", "--cpu-contexts", "2"]
    res = subprocess.run(cmd, cwd=tmp_path, capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [ln for ln in res.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1, res.stdout
    out = json.loads(lines[0])
    assert out["impl"] == "reference" and out["n_gpus"] == 2 and out["value"] > 0
    assert out["cpu_baseline"]["kind"] in ("reference", "port") and out["e2e"]["h2d_bytes_per_step"] == 0



def test_strong_share_is_found_among_a_rank_s_own_permuted_contexts():
    wl = WORKLOADS["llama2_70b_gqa"]
    lens = wl.lengths(20240, 40)
    for world in (2, 4, 8):
        covered = []
        for rank in range(world):
            local = dist_util.weak_scaling_lengths(wl, 20240, rank, 40)
            sel = dist_util.strong_share_on_local_contexts(lens, local, rank, world)
            want = np.sort(lens[assign_contexts(lens, world)[rank]])
            assert np.array_equal(np.sort(local[sel]), want) and len(set(sel.tolist())) == len(sel)
            covered.append(want)
        assert np.array_equal(np.sort(np.concatenate(covered)), np.sort(lens)), "the shares make up the whole request set"
        loads = [int((c + 1).sum()) for c in covered]
        assert max(loads) - min(loads) <= lens.max() + 1


def _router_worker(rank: int, world: int, port: int, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from glinthawk_b200.router import BALANCED, ContextRouter
        wl = WORKLOADS["llama2_70b_gqa"]
        lens = wl.lengths(20240, 16)
        router = ContextRouter(world, wl.batch // world, wl.batch, BALANCED)  # every rank replays the same calls
        ranks = router.assign_ranks(np.arange(wl.batch), lens)
        mine = np.flatnonzero(ranks == rank)
        # a second batch: a quarter of the prompts have finished, new ones take their place
        gone = np.arange(0, wl.batch, 4)
        router.release(gone)
        ranks2 = router.assign_ranks(np.concatenate([np.setdiff1d(np.arange(wl.batch), gone), 1000 + gone]),
                                     np.concatenate([np.delete(lens, gone), lens[gone]]))
        tokens_mine = float(router.loads()[1][rank])
        total = dist_util.sum_over_ranks(tokens_mine)
        worst = dist_util.max_over_ranks(tokens_mine)
        dist.barrier()
        out.put((rank, mine.tolist(), ranks2.tolist(), total, worst))
    finally:
        dist.destroy_process_group()


def test_two_ranks_route_the_same_requests_without_talking():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = [ctx.Process(target=_router_worker, args=(r, world, port, out)) for r in range(world)]
    for p in procs:
        p.start()
    results = sorted(out.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    wl = WORKLOADS["llama2_70b_gqa"]
    lens = wl.lengths(20240, 16)
    (_, mine0, again0, total, worst), (_, mine1, again1, *_rest) = results
    assert sorted(mine0 + mine1) == list(range(wl.batch)) and len(mine0) == len(mine1) == wl.batch // 2
    assert again0 == again1, "both processes hold the same table after the same calls"
    assert total == float(lens.sum()) and worst <= 1.02 * total / world
