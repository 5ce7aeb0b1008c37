"""RoPE tables as the reference's converters write them into the base weights.

``tools/bin2glint.py:19-25`` (Llama 2, theta 1e4) and ``tools/llama3/llamasplit2glint.py:47-58,121-123`` (Llama 3,
theta 5e5): ``freq_k = 1 / theta**(2k / head_size)`` in fp32, ``angle[t][k] = t * freq_k`` in fp32, cos and sin in
fp32, then stored in the model dtype (``base.hh:110-112``: ``freq_cis_real`` / ``freq_cis_imag`` of
``seq_len * head_size / 2`` elements each).
"""
from __future__ import annotations

import numpy as np


def rope_tables(head_size: int, seq_len: int, theta: float = 10000.0) -> tuple[np.ndarray, np.ndarray]:
    """fp32 cos and sin tables of shape [seq_len, head_size // 2]; cast to the model dtype to store them."""
    k2 = np.arange(0, head_size, 2, dtype=np.float32)[: head_size // 2]
    freqs = (np.float32(1.0) / np.power(np.float32(theta), k2 / np.float32(head_size))).astype(np.float32)
    t = np.arange(seq_len, dtype=np.float32)
    ang = np.outer(t, freqs).astype(np.float32)
    return np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)
