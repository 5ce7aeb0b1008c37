"""Hand-off of stage activations between ranks over NCCL point-to-point (NVLink inside one box).

In the reference an attention-only node receives, per layer, the batch's query rows and new K/V rows from the node
that ran the dense pre-attention stage, and returns the attention output to the node that runs the post-attention
stage; the tensors travel as a serialized ``BatchedInferenceState`` over TCP, through host memory on both sides
(src/worker/worker.hh:728-757, src/models/common/state.hh:561-594, src/models/llama2/model.hh:632-722).  Here the
same three tensors move device to device with ``torch.distributed`` P2P operations; the attention path itself still
has no collective.  The classes work on any backend, so the protocol is tested with gloo on CPU ranks.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass
class StageShapes:
    batch: int
    dim: int        # n_heads * head_size: width of q and of the attention output
    row_elems: int  # 2 * kv_dim: width of a new [K,V] row
    dtype: torch.dtype
    device: torch.device | str


class AttentionLink:
    """One end of the link between a dense-stage rank and the attention rank that owns the contexts' KV."""

    def __init__(self, peer: int, shapes: StageShapes):
        self.peer, self.s = peer, shapes

    def _buf(self, width: int) -> torch.Tensor:
        return torch.empty((self.s.batch, width), dtype=self.s.dtype, device=self.s.device)

    # dense-stage side ------------------------------------------------------------------------------
    def send_inputs(self, q: torch.Tensor, kv_new: torch.Tensor) -> list:
        ops = [dist.P2POp(dist.isend, q, self.peer), dist.P2POp(dist.isend, kv_new, self.peer)]
        return dist.batch_isend_irecv(ops)

    def recv_output(self, xb: torch.Tensor | None = None):
        xb = self._buf(self.s.dim) if xb is None else xb
        return xb, dist.batch_isend_irecv([dist.P2POp(dist.irecv, xb, self.peer)])

    # attention side ----------------------------------------------------------------------------------
    def recv_inputs(self, q: torch.Tensor | None = None, kv_new: torch.Tensor | None = None):
        q = self._buf(self.s.dim) if q is None else q
        kv_new = self._buf(self.s.row_elems) if kv_new is None else kv_new
        ops = [dist.P2POp(dist.irecv, q, self.peer), dist.P2POp(dist.irecv, kv_new, self.peer)]
        return q, kv_new, dist.batch_isend_irecv(ops)

    def send_output(self, xb: torch.Tensor) -> list:
        return dist.batch_isend_irecv([dist.P2POp(dist.isend, xb, self.peer)])


def wait_all(reqs) -> None:
    for r in reqs:
        r.wait()


def run_attention_rank(link: AttentionLink, n_layers: int, step_fn) -> None:
    """Attention side of one decode step.  Both ranks walk through the same sequence of transfer groups — group g
    carries layer g's inputs one way and layer g-1's output the other way — because NCCL matches point-to-point
    operations between two ranks strictly in the order they were issued."""
    xb = None
    q = kv = None
    for g in range(n_layers + 1):
        ops, nq, nkv = [], None, None
        if g < n_layers:
            nq, nkv = link._buf(link.s.dim), link._buf(link.s.row_elems)
            ops += [dist.P2POp(dist.irecv, nq, link.peer), dist.P2POp(dist.irecv, nkv, link.peer)]
        if g >= 1:
            xb = step_fn(g - 1, q, kv)  # enqueued on the current stream; the send below is ordered after it
            ops.append(dist.P2POp(dist.isend, xb, link.peer))
        wait_all(dist.batch_isend_irecv(ops))
        q, kv = nq, nkv


def run_dense_rank(link: AttentionLink, n_layers: int, make_inputs, consume_output) -> None:
    """Dense-stage side: ``make_inputs(layer) -> (q, kv_new)``, ``consume_output(layer, xb)``; mirrors
    run_attention_rank group by group."""
    for g in range(n_layers + 1):
        ops, xb, keep = [], None, None
        if g < n_layers:
            keep = make_inputs(g)
            ops += [dist.P2POp(dist.isend, keep[0], link.peer), dist.P2POp(dist.isend, keep[1], link.peer)]
        if g >= 1:
            xb = link._buf(link.s.dim)
            ops.append(dist.P2POp(dist.irecv, xb, link.peer))
        wait_all(dist.batch_isend_irecv(ops))
        if g >= 1:
            consume_output(g - 1, xb)


def main() -> None:
    """Two ranks, one GPU each (launch with torch.distributed.run): rank 0 plays the dense stages, rank 1 owns the
    contexts and runs the attention stage; q / new K,V rows / xb cross NVLink once per layer.  Prints one JSON line
    with the step time, and checks the returned xb against the attention rank's own copy."""
    import argparse
    import json
    import os

    import numpy as np

    from .rope import rope_tables
    from .stage import AttentionStage
    from .workload import WORKLOADS

    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="llama2_70b_gqa")
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--steps", type=int, default=5)
    args = ap.parse_args()

    rank, local = int(os.environ["RANK"]), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    from datetime import timedelta

    dist.init_process_group("nccl", device_id=dev, timeout=timedelta(seconds=60))  # fail fast, never hang
    wl = WORKLOADS[args.workload]
    sh = wl.shape
    tdt = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}[wl.dtype]
    B, L = wl.batch, args.layers
    shapes = StageShapes(B, sh.dim, 2 * sh.kv_dim, tdt, dev)
    link = AttentionLink(1 - rank, shapes)
    gen = torch.Generator(device=dev).manual_seed(1234)
    q_all = torch.randn((L, B, sh.dim), device=dev, generator=gen).to(tdt)
    kv_all = torch.randn((L, B, 2 * sh.kv_dim), device=dev, generator=gen).to(tdt)  # same seed on both ranks
    times = []
    if rank == 1:
        lens = wl.lengths(7, args.steps + 2)
        stage = AttentionStage(sh, tdt, n_layers_hosted=L, max_batch=B, max_contexts=B, paged=True, device=local)
        cos, sin = rope_tables(sh.head_size, sh.seq_len, sh.rope_theta)
        stage.set_rope_tables(torch.from_numpy(cos).to(dev).to(tdt), torch.from_numpy(sin).to(dev).to(tdt))
        slots = stage.get_contexts(np.arange(1, B + 1, dtype=np.uint32))
        for i in range(B):
            for l in range(L):
                stage.prepare(int(slots[i]), l, int(lens[i]) + args.steps)
                stage.fill_normal(stage.layer_ptr(int(slots[i]), l), int(lens[i]) * 2 * sh.kv_dim, tdt, 5,
                                  offset=(i * L + l) * sh.seq_len * 2 * sh.kv_dim)
        pos = lens.astype(np.uint32)
        outs = {}

        def step_fn(layer, q, kv):
            xb = torch.empty_like(q)
            stage.step(layer, q, kv, xb)
            outs[layer] = xb
            return xb

    for step in range(args.steps):
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        if rank == 1:
            stage.batch_begin(slots, pos)
            run_attention_rank(link, L, step_fn)
            pos += 1
        else:
            got = {}
            run_dense_rank(link, L, lambda l: (q_all[l].clone(), kv_all[l]), lambda l, xb: got.__setitem__(l, xb))
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    # verification: the attention rank sends its last step's outputs once more through a plain collective
    check = torch.zeros((L, B, sh.dim), dtype=tdt, device=dev)
    if rank == 1:
        check = torch.stack([outs[l] for l in range(L)])
    dist.broadcast(check, src=1)
    if rank == 0:
        same = all(torch.equal(got[l], check[l]) for l in range(L))
        per_layer = (B * sh.dim * 2 + B * 2 * sh.kv_dim) * q_all.element_size()
        print(json.dumps({"mode": "stage hand-off over NCCL P2P", "workload": wl.name, "layers": L, "contexts": B,
                          "ms_per_step": min(times), "ms_per_layer": min(times) / L, "handoff_bytes_per_layer": per_layer,
                          "outputs_identical": bool(same)}))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
