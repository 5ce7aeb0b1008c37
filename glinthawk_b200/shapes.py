"""Model shapes of the attention stage.

The reference fixes shapes at compile time as ``ModelConfig`` structs (src/models/llama2/variants.hh:37-186);
here they are run-time values.  Names match the shape table compiled into the reference harness used by the
parity tests, so that the same name selects the same shape on both sides.
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class AttnShape:
    name: str
    dim: int
    n_heads: int
    n_kv_heads: int
    seq_len: int
    n_layers: int
    rope_theta: float = 10000.0

    @property
    def head_size(self) -> int:
        return self.dim // self.n_heads

    @property
    def gqa_size(self) -> int:
        return self.n_heads // self.n_kv_heads

    @property
    def kv_dim(self) -> int:
        return self.dim // self.gqa_size

    def row_bytes(self, elem: int) -> int:
        return 2 * self.kv_dim * elem


SHAPES = {s.name: s for s in [
    AttnShape("tiny15m", 288, 6, 6, 256, 6),              # stories15M shape
    AttnShape("s110m", 768, 12, 12, 1024, 12),            # Stories_110M, variants.hh:173-186
    AttnShape("l7b_4k", 4096, 32, 32, 4096, 32),          # Llama2_7B_Chat shape (variants.hh:158-171), 4K slots
    AttnShape("l13b_4k", 5120, 40, 40, 4096, 40),         # Llama2_13B_Chat shape (variants.hh:143-156), 4K slots
    AttnShape("l70b_4k", 8192, 64, 8, 4096, 80),          # Llama2_70B_Chat_4K, variants.hh:113-116
    AttnShape("l3_8b_8k", 4096, 32, 8, 8192, 32, 500000.0),  # Llama3_8B shape (variants.hh:83-96), 8K slots
    AttnShape("l3_405b", 16384, 128, 8, 2048, 126, 500000.0),  # Llama3_405B, variants.hh:53-66
    AttnShape("mini_mha", 512, 4, 4, 512, 2),
    AttnShape("mini_g4", 1024, 8, 2, 512, 2),
    AttnShape("mini_g8", 2048, 16, 2, 512, 2),
    AttnShape("mini_g16", 4096, 32, 2, 512, 2),
]}
