"""Hand-off of stage activations between ranks over NCCL point-to-point (NVLink inside one box).

In the reference an attention-only node receives, per layer, the batch's query rows and new K/V rows from the node
that ran the dense pre-attention stage, and returns the attention output to the node that runs the post-attention
stage; the tensors travel as a serialized ``BatchedInferenceState`` over TCP, through host memory on both sides
(src/worker/worker.hh:728-757, src/models/common/state.hh:561-594, src/models/llama2/model.hh:632-722).  Here the
same three tensors move device to device with ``torch.distributed`` P2P operations; the attention path itself still
has no collective.  What the attention side runs on the tensors once they are on its GPU is ``gh_attn_step``, the
device-buffer form of ``Llama2::forward_attention``.  The classes work on any backend, so the protocol is tested with
gloo on CPU ranks; ``bench.py`` times it on pairs of GPUs.
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


@dataclass
class LayerLink:
    """A pair's two directions as process groups of their own (each gets its own NCCL communicator and stream):
    `inputs` carries q and the new K/V rows to the attention side, `outputs` carries xb back.  Traffic of one direction
    never queues behind traffic of the other, so the inputs of later layers arrive while earlier layers compute."""
    peer: int
    inputs: object
    outputs: object


def attention_side_step(link: LayerLink, n_layers: int, q_all, kv_all, xb_all, step_layer, ahead: int = 8) -> None:
    """Attention side of one decode step over all layers.  The receives of q / K,V rows run `ahead` layers in front of
    the compute, in layer order (the order the dense side sends them in); layer l's kernels are enqueued once its
    inputs are in (`step_layer(l)` reads q_all[l], kv_all[l] and writes xb_all[l] on the current stream), and
    xb_all[l] goes back while layer l+1 computes.  On NCCL a wait only orders streams; the host runs ahead, and it
    posts only a few receives before the first layer's kernels so that the GPU does not sit idle behind it."""
    def post(l):
        return dist.batch_isend_irecv([dist.P2POp(dist.irecv, q_all[l], link.peer, group=link.inputs),
                                       dist.P2POp(dist.irecv, kv_all[l], link.peer, group=link.inputs)])

    recvs = {l: post(l) for l in range(min(ahead, n_layers))}
    sends = []
    for l in range(n_layers):
        wait_all(recvs.pop(l))
        step_layer(l)
        sends.append(dist.batch_isend_irecv([dist.P2POp(dist.isend, xb_all[l], link.peer, group=link.outputs)]))
        if l + ahead < n_layers:
            recvs[l + ahead] = post(l + ahead)
    for s_ in sends:
        wait_all(s_)


def dense_side_step(link: LayerLink, n_layers: int, q_all, kv_all, xb_rx) -> None:
    """Dense-stage side, mirroring attention_side_step: every layer's inputs go out in layer order, every layer's xb
    is received into xb_rx[l] in layer order."""
    works = []
    for l in range(n_layers):
        works.append(dist.batch_isend_irecv([dist.P2POp(dist.isend, q_all[l], link.peer, group=link.inputs),
                                             dist.P2POp(dist.isend, kv_all[l], link.peer, group=link.inputs)]))
        works.append(dist.batch_isend_irecv([dist.P2POp(dist.irecv, xb_rx[l], link.peer, group=link.outputs)]))
    for w in works:
        wait_all(w)


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
