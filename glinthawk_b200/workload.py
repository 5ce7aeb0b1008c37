"""Synthetic workloads for the benchmark and the full-size tests, and request-to-GPU assignment.

The reference drives its end-to-end runs with prompt/response lengths sampled from a ShareGPT dump
(py/process_sharegpt.py:48-88); that data is not available here, so seeded length distributions with the sizes
of the benchmark configurations stand in for it.  Contexts are assigned to GPUs whole (a context's KV lives on
exactly one device), as the reference's tier router does (src/compute/routerman.hh:311-331); here the
assignment balances the number of cached tokens, not the number of contexts.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from .shapes import SHAPES, AttnShape


@dataclass(frozen=True)
class Workload:
    name: str
    shape: AttnShape
    dtype: str          # "f16" | "bf16" | "f32"
    n_layers: int       # attention layers a token passes through in one step
    batch: int          # contexts decoding one token each
    length_dist: str    # how the cached lengths are drawn
    description: str
    prefill_contexts: int = 0   # additional contexts that append a prompt chunk into a fresh slot every step
    prefill_tokens: int = 0     # tokens per prompt chunk
    prefill_pos0: int = 0       # tokens those slots already hold when the chunk arrives (0 = fresh slots)

    def lengths(self, seed: int, headroom: int = 0) -> np.ndarray:
        """Cached tokens per context before the first step; every context keeps `headroom` free positions."""
        rng = np.random.default_rng(seed)
        S = self.shape.seq_len
        if self.length_dist == "lognormal_1024_0.8":
            x = np.exp(rng.normal(np.log(1024.0), 0.8, size=self.batch))
            lens = np.clip(np.rint(x), 16, S)
        elif self.length_dist.startswith("uniform_"):
            lo, hi = (int(v) for v in self.length_dist.split("_")[1:])
            lens = rng.integers(lo, hi + 1, size=self.batch)
        else:
            raise ValueError(self.length_dist)
        return np.minimum(lens, S - headroom).astype(np.int64)


WORKLOADS = {w.name: w for w in [
    Workload("llama2_70b_gqa", SHAPES["l70b_4k"], "f16", 80, 256, "lognormal_1024_0.8",
             "Llama2-70B GQA attention stage, 80 layers, fp16, 64 q / 8 kv heads, head 128, slots of 4096, "
             "256 contexts, lengths lognormal(median 1024, sigma 0.8) clipped to 16..4096"),
    Workload("llama2_70b_long", SHAPES["l70b_4k"], "f16", 4, 256, "uniform_2048_4095",
             "Llama2-70B GQA attention stage, 4 layers, fp16, 256 contexts, lengths uniform 2048..4096 (the same kernel "
             "without the short contexts of the lognormal mix)"),
    Workload("llama2_7b_layer", SHAPES["l7b_4k"], "f16", 1, 64, "uniform_128_4095",
             "Llama2-7B attention layer, fp16, 32 heads (MHA), head 128, 64 contexts, lengths uniform 128..4096"),
    Workload("llama2_13b", SHAPES["l13b_4k"], "f16", 40, 128, "uniform_512_4095",
             "Llama2-13B attention stage, 40 layers, fp16, 40 heads (MHA), 128 contexts, lengths uniform 512..4096"),
    Workload("llama3_8b_decode", SHAPES["l3_8b_8k"], "bf16", 1, 448, "uniform_256_8191",
             "Llama3-8B GQA decode part, one layer, bf16, 32 q / 8 kv heads, 448 contexts, lengths uniform 256..8192"),
    Workload("llama3_8b_mixed", SHAPES["l3_8b_8k"], "bf16", 1, 448, "uniform_256_8191",
             "Llama3-8B GQA mixed prefill + decode, one layer, bf16, 32 q / 8 kv heads, head 128, slots of 8192: "
             "448 contexts decode one token each (lengths uniform 256..8192), 64 contexts append a 512-token prompt "
             "chunk into fresh slots", prefill_contexts=64, prefill_tokens=512),
    Workload("llama3_8b_late_chunk", SHAPES["l3_8b_8k"], "bf16", 1, 64, "uniform_256_8191",
             "Llama3-8B GQA, one layer, bf16: 32 contexts append the last 512-token chunk of a 4096-token prompt "
             "(3584 tokens already cached) next to 64 contexts decoding one token each (lengths uniform 256..8192)",
             prefill_contexts=32, prefill_tokens=512, prefill_pos0=3584),
]}


def assign_contexts(lengths, n_ranks: int) -> list[np.ndarray]:
    """Whole contexts to ranks, longest first onto the least-loaded rank (ties: lowest rank).  Returns, per rank,
    the sorted indices of its contexts.  Deterministic, so every rank computes the same assignment."""
    lengths = np.asarray(lengths, dtype=np.int64)
    order = np.argsort(-lengths, kind="stable")
    load = np.zeros(n_ranks, dtype=np.int64)
    count = np.zeros(n_ranks, dtype=np.int64)
    owner = np.empty(len(lengths), dtype=np.int64)
    for i in order:
        r = int(np.lexsort((np.arange(n_ranks), count, load))[0])
        owner[i] = r
        load[r] += lengths[i] + 1
        count[r] += 1
    return [np.flatnonzero(owner == r) for r in range(n_ranks)]


def algorithmic_bytes(lengths_after_append, shape: AttnShape, elem: int) -> dict:
    """Bytes one layer-step must move, per kernel: K and V of every attended token read once (the query heads
    of a group share them), the appended row read and written, q read and xb written."""
    n = np.asarray(lengths_after_append, dtype=np.int64)
    row = 2 * shape.kv_dim * elem
    B = len(n)
    qx = B * shape.dim * elem
    return {
        "kv_read": int(n.sum()) * row,
        "appended": B * row,
        "decode_kernel": int(n.sum()) * row + 2 * qx,
        "append_kernel": 2 * B * row + 2 * qx + B * shape.head_size * elem,
    }
