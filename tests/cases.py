"""Seeded parity cases and thin wrappers around the two CPU checkers (test infrastructure).

* ``Oracle``    — the plain-C restatement in ``oracle/attn_oracle.c``.
* ``Reference`` — the reference project's own amd64 operations, prebuilt into ``oracle/_ref`` from the reference
  tree (present only where it was built or carried along).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field

import numpy as np

from glinthawk_b200.rope import rope_tables
from glinthawk_b200.shapes import SHAPES, AttnShape
from oracle import build as oracle_build

F16, F32, BF16 = 0, 1, 2
NP_DTYPE = {F16: np.float16, F32: np.float32}

# Tolerances of the parity contract.
TOL_XB = {F16: 2e-2, BF16: 2e-2, F32: 1e-4}  # absolute, attention output
TOL_K_REL = 1e-3                             # relative, rotated K (and q); V is bit-exact


def to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """fp32 -> bf16 bit patterns (uint16), round to nearest even."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = u + 0x7FFF + ((u >> 16) & 1)
    return (u >> 16).astype(np.uint16)


def from_bf16_bits(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << 16).view(np.float32)


def store(x: np.ndarray, dtype: int) -> np.ndarray:
    """fp32 values -> array in the storage representation (bf16 as uint16 bit patterns)."""
    return to_bf16_bits(x) if dtype == BF16 else x.astype(NP_DTYPE[dtype])


def as_f32(x: np.ndarray, dtype: int) -> np.ndarray:
    return from_bf16_bits(x) if dtype == BF16 else x.astype(np.float32)


@dataclass
class Case:
    name: str
    shape: AttnShape
    dtype: int
    pos: np.ndarray                      # uint32 [B]
    active: np.ndarray                   # bool [B]
    cache: list[np.ndarray]              # per context [(pos+1), 2*kv_dim] storage dtype (row pos is overwritten)
    q: np.ndarray                        # [B, dim]
    kv_new: np.ndarray                   # [B, 2*kv_dim]
    fcr: np.ndarray                      # [S, hs/2]
    fci: np.ndarray
    seed: int = 0
    extra: dict = field(default_factory=dict)

    @property
    def B(self) -> int:
        return len(self.pos)


def make_case(name: str, shape_name: str, dtype: int, pos, seed: int, *, q_scale: float = 1.0,
              inactive=(), round_inputs_to: int | None = None) -> Case:
    """N(0,1) cache, q, k, v from ``default_rng(seed)``; RoPE tables by the converter formula, stored in dtype.

    ``round_inputs_to=BF16`` with ``dtype=F32`` gives fp32 arrays whose values are exactly bf16-representable:
    the inputs the reference's fp32 operations are run on to check a bf16 device path."""
    sh = SHAPES[shape_name]
    rng = np.random.default_rng(seed)
    pos = np.asarray(pos, dtype=np.uint32)
    B = len(pos)

    def gen(*shape):
        x = rng.standard_normal(shape, dtype=np.float32)
        if round_inputs_to == BF16:
            x = from_bf16_bits(to_bf16_bits(x))
        return store(x, dtype)

    cache = [gen(int(p) + 1, 2 * sh.kv_dim) for p in pos]
    q = store(as_f32(gen(B, sh.dim), dtype) * np.float32(q_scale), dtype)
    kv_new = gen(B, 2 * sh.kv_dim)
    cos, sin = rope_tables(sh.head_size, sh.seq_len, sh.rope_theta)
    if round_inputs_to == BF16:
        cos, sin = from_bf16_bits(to_bf16_bits(cos)), from_bf16_bits(to_bf16_bits(sin))
    active = np.ones(B, dtype=bool)
    active[list(inactive)] = False
    return Case(name, sh, dtype, pos, active, cache, q, kv_new, store(cos, dtype), store(sin, dtype), seed)


@dataclass
class StepResult:
    rows: list[np.ndarray]   # the appended [K|V] row of every context after RoPE (None for inactive)
    q: np.ndarray            # q after in-place rotation
    xb: np.ndarray           # attention output [B, dim]
    att: np.ndarray | None = None


def _vp(a):
    return C.c_void_p(a.ctypes.data) if a is not None else C.c_void_p(0)


@dataclass
class ProjCase:
    """Inputs of the stage's producer (src/models/llama2/model.hh:326-343): the residual stream, the rmsnorm weight
    and the two projection matrices, plus the batch's token positions for the rotation and the append."""
    name: str
    shape: AttnShape
    dtype: int
    pos: np.ndarray       # uint32 [B]
    x: np.ndarray         # [B, dim]
    rms_w: np.ndarray     # [dim]
    wq: np.ndarray        # [dim, dim]          (row r = output feature r)
    wkv: np.ndarray       # [2*kv_dim, dim]
    fcr: np.ndarray
    fci: np.ndarray

    @property
    def B(self) -> int:
        return len(self.pos)


def make_proj_case(name: str, shape_name: str, dtype: int, pos, seed: int) -> ProjCase:
    """x ~ N(0,1), rmsnorm weights around 1, projection weights ~ N(0, 1/dim) so that q, k, v come out ~ N(0,1)."""
    sh = SHAPES[shape_name]
    rng = np.random.default_rng(seed)
    pos = np.asarray(pos, dtype=np.uint32)
    B = len(pos)
    x = store(rng.standard_normal((B, sh.dim), dtype=np.float32), dtype)
    rms_w = store(1.0 + 0.1 * rng.standard_normal(sh.dim, dtype=np.float32), dtype)
    scale = np.float32(1.0 / np.sqrt(sh.dim))
    wq = store(rng.standard_normal((sh.dim, sh.dim), dtype=np.float32) * scale, dtype)
    wkv = store(rng.standard_normal((2 * sh.kv_dim, sh.dim), dtype=np.float32) * scale, dtype)
    cos, sin = rope_tables(sh.head_size, sh.seq_len, sh.rope_theta)
    return ProjCase(name, sh, dtype, pos, x, rms_w, wq, wkv, store(cos, dtype), store(sin, dtype))


@dataclass
class ProjResult:
    xb: np.ndarray           # rmsnorm output [B, dim]
    q: np.ndarray            # projected q [B, dim], before rotation
    kv: np.ndarray           # projected [K|V] rows [B, 2*kv_dim], before rotation
    q_rot: np.ndarray        # q after apply_rope
    rows: np.ndarray         # the rows as copy_kv_cache + apply_rope leave them in the slots [B, 2*kv_dim]


class Oracle:
    def __init__(self):
        self.lib = oracle_build.load_oracle()

    def layer_step(self, case: Case, keep_att: bool = False) -> StepResult:
        sh, B = case.shape, case.B
        cache = [c.copy() for c in case.cache]
        q, xb = case.q.copy(), np.zeros_like(case.q)
        att = np.zeros((B, sh.n_heads, sh.seq_len), dtype=case.q.dtype)
        bases = (C.c_void_p * B)(*[c.ctypes.data if a else 0 for c, a in zip(cache, case.active)])
        rc = self.lib.gho_layer_step(case.dtype, C.c_uint64(B), _vp(case.pos), bases, _vp(case.fcr), _vp(case.fci),
                                     _vp(q), _vp(case.kv_new), _vp(att), _vp(xb), C.c_uint64(sh.n_kv_heads),
                                     C.c_uint64(sh.gqa_size), C.c_uint64(sh.head_size), C.c_uint64(sh.seq_len))
        assert rc == 0
        rows = [c[int(p)].copy() if a else None for c, p, a in zip(cache, case.pos, case.active)]
        return StepResult(rows, q, xb, att if keep_att else None)

    def timed_layer_step(self, case: Case):
        """As Reference.timed_layer_step, for the C restatement."""
        sh, B = case.shape, case.B
        cache = [c.copy() for c in case.cache]
        q, xb = case.q.copy(), np.zeros_like(case.q)
        att = np.zeros((B, sh.n_heads, sh.seq_len), dtype=case.q.dtype)
        bases = (C.c_void_p * B)(*[c.ctypes.data if a else 0 for c, a in zip(cache, case.active)])
        args = (case.dtype, C.c_uint64(B), _vp(case.pos), bases, _vp(case.fcr), _vp(case.fci), _vp(q), _vp(case.kv_new),
                _vp(att), _vp(xb), C.c_uint64(sh.n_kv_heads), C.c_uint64(sh.gqa_size), C.c_uint64(sh.head_size),
                C.c_uint64(sh.seq_len))
        keep = (cache, q, xb, att, case)

        def run():
            assert self.lib.gho_layer_step(*args) == 0
            return keep is not None

        return run

    def _rotate_and_append(self, case: "ProjCase", q: np.ndarray, kv: np.ndarray):
        """copy_kv_cache + apply_rope on one-row slots: what the reference does with the projections next
        (src/models/llama2/model.hh:345-360)."""
        sh, B = case.shape, case.B
        rows = np.zeros_like(kv)
        q_rot = q.copy()
        ptrs = (C.c_void_p * B)(*[rows[i].ctypes.data for i in range(B)])
        assert self.lib.gho_copy_kv_cache(case.dtype, ptrs, _vp(kv), C.c_uint64(B), C.c_uint64(sh.kv_dim)) == 0
        assert self.lib.gho_apply_rope(case.dtype, C.c_uint64(B), _vp(case.pos), _vp(case.fcr), _vp(case.fci), _vp(q_rot),
                                       ptrs, C.c_uint64(sh.n_kv_heads), C.c_uint64(sh.gqa_size),
                                       C.c_uint64(sh.head_size)) == 0
        return q_rot, rows

    def pre_attention(self, case: "ProjCase") -> "ProjResult":
        sh, B = case.shape, case.B
        xb, q = np.zeros_like(case.x), np.zeros_like(case.x)
        kv = np.zeros((B, 2 * sh.kv_dim), dtype=case.x.dtype)
        rc = self.lib.gho_pre_attention(case.dtype, C.c_uint64(B), _vp(case.x), _vp(case.rms_w), _vp(case.wq), _vp(case.wkv),
                                        _vp(xb), _vp(q), _vp(kv), C.c_uint64(sh.dim), C.c_uint64(sh.kv_dim))
        assert rc == 0
        q_rot, rows = self._rotate_and_append(case, q, kv)
        return ProjResult(xb, q, kv, q_rot, rows)

    def op(self, name: str, *args):
        fn = getattr(self.lib, "gho_" + name)
        rc = fn(*args)
        assert rc == 0, f"oracle {name} -> {rc}"


class Reference:
    """ctypes view of ``oracle/_ref/libghref_*.so`` (see ``oracle/ref_harness.cc``)."""

    def __init__(self, lib, flavour: str = ""):
        self.lib = lib
        self.flavour = flavour  # which build of the reference this is: native, v4 (AVX-512) or v3 (AVX2)
        lib.ghref_shape_name.restype = C.c_char_p
        self.names = [lib.ghref_shape_name(i).decode() for i in range(lib.ghref_shape_count())]

    @classmethod
    def try_load(cls, flavour: str | None = None):
        lib = oracle_build.load_ref(flavour)
        return cls(lib, flavour or oracle_build.ref_flavour() or "") if lib is not None else None

    def threads(self) -> int:
        return self.lib.ghref_threads()

    def timed_layer_step(self, case: Case):
        """A closure that runs the reference's five operations on the case and nothing else: buffers are set up here,
        outside whatever the caller times.  Every call appends the same rows again and rotates q once more."""
        assert case.dtype in (F16, F32), "the reference's amd64 backend has no bf16"
        sh, B = case.shape, case.B
        idx = self.names.index(sh.name)
        cache = [c.copy() for c in case.cache]
        q, xb = case.q.copy(), np.zeros_like(case.q)
        att = np.zeros((B, sh.n_heads, sh.seq_len), dtype=case.q.dtype)
        bases = (C.c_void_p * B)(*[c.ctypes.data if a else 0 for c, a in zip(cache, case.active)])
        args = (idx, case.dtype, C.c_uint64(B), _vp(case.pos), bases, _vp(case.fcr), _vp(case.fci), _vp(q),
                _vp(case.kv_new), _vp(att), _vp(xb))
        keep = (cache, q, xb, att, case)  # noqa: F841  (the closure keeps the buffers alive)

        def run():
            assert self.lib.ghref_layer_step(*args) == 0
            return keep is not None

        return run

    def layer_step(self, case: Case, keep_att: bool = False) -> StepResult:
        assert case.dtype in (F16, F32), "the reference's amd64 backend has no bf16"
        sh, B = case.shape, case.B
        idx = self.names.index(sh.name)
        cache = [c.copy() for c in case.cache]
        q, xb = case.q.copy(), np.zeros_like(case.q)
        att = np.zeros((B, sh.n_heads, sh.seq_len), dtype=case.q.dtype)
        bases = (C.c_void_p * B)(*[c.ctypes.data if a else 0 for c, a in zip(cache, case.active)])
        rc = self.lib.ghref_layer_step(idx, case.dtype, C.c_uint64(B), _vp(case.pos), bases, _vp(case.fcr),
                                       _vp(case.fci), _vp(q), _vp(case.kv_new), _vp(att), _vp(xb))
        assert rc == 0
        rows = [c[int(p)].copy() if a else None for c, p, a in zip(cache, case.pos, case.active)]
        return StepResult(rows, q, xb, att if keep_att else None)


    def pre_attention(self, case: "ProjCase", oracle: "Oracle") -> "ProjResult":
        """The reference's own rmsnorm and matmul; rotation and append as in layer_step (through the oracle's
        restatement of the two operations, which the layer-step fixtures pin)."""
        assert case.dtype in (F16, F32), "the reference's amd64 backend has no bf16"
        sh, B = case.shape, case.B
        idx = self.names.index(sh.name)
        xb, q = np.zeros_like(case.x), np.zeros_like(case.x)
        kv = np.zeros((B, 2 * sh.kv_dim), dtype=case.x.dtype)
        rc = self.lib.ghref_pre_attention(idx, case.dtype, C.c_uint64(B), _vp(case.x), _vp(case.rms_w), _vp(case.wq),
                                          _vp(case.wkv), _vp(xb), _vp(q), _vp(kv))
        assert rc == 0
        q_rot, rows = oracle._rotate_and_append(case, q, kv)
        return ProjResult(xb, q, kv, q_rot, rows)


# The producer's golden cases: one per storage type the reference has, small matrices.
GOLDEN_PROJ_SPECS = [
    dict(name="proj_mini_mha_f16", shape_name="mini_mha", dtype=F16, pos=[0, 5, 64, 300, 511], seed=201),
    dict(name="proj_mini_g4_f16", shape_name="mini_g4", dtype=F16, pos=[1, 2, 3, 100, 101, 102, 400], seed=202),
    dict(name="proj_tiny15m_f32", shape_name="tiny15m", dtype=F32, pos=[0, 17, 255], seed=203),
]


def golden_proj_case(spec: dict) -> ProjCase:
    return make_proj_case(spec["name"], spec["shape_name"], spec["dtype"], spec["pos"], spec["seed"])


# The golden cases: small enough for the checkers to finish in well under a second each, covering every head
# size / group size / dtype the kernels dispatch on, the edges of the 64-token tile, position 0, the last
# position of a slot, an inactive prompt, and a large-magnitude query that moves the running maximum.
GOLDEN_SPECS = [
    dict(name="tiny15m_f32", shape_name="tiny15m", dtype=F32, pos=[0, 7, 31, 255], seed=101),
    dict(name="tiny15m_f16", shape_name="tiny15m", dtype=F16, pos=[3, 64, 100, 200], seed=102),
    dict(name="s110m_f16", shape_name="s110m", dtype=F16, pos=[0, 63, 1023], seed=103),
    dict(name="mini_mha_f16", shape_name="mini_mha", dtype=F16, pos=[0, 1, 63, 64, 65, 511], seed=104),
    dict(name="mini_g4_f16", shape_name="mini_g4", dtype=F16, pos=[5, 127, 128, 300, 511], seed=105),
    dict(name="mini_g8_f16", shape_name="mini_g8", dtype=F16, pos=[0, 62, 191, 192, 511], seed=106),
    dict(name="mini_g8_f32", shape_name="mini_g8", dtype=F32, pos=[9, 64, 257], seed=107),
    dict(name="mini_g16_f16", shape_name="mini_g16", dtype=F16, pos=[15, 255, 256, 400], seed=108),
    dict(name="mini_g8_f16_inactive", shape_name="mini_g8", dtype=F16, pos=[33, 0, 130, 77], seed=109, inactive=[1, 3]),
    dict(name="mini_g8_f16_bigq", shape_name="mini_g8", dtype=F16, pos=[100, 511], seed=110, q_scale=6.0),
    dict(name="l70b_4k_f16", shape_name="l70b_4k", dtype=F16, pos=[15, 1023, 2500, 4095], seed=111),
    dict(name="l7b_4k_f16", shape_name="l7b_4k", dtype=F16, pos=[127, 3000], seed=112),
    dict(name="l13b_4k_f16", shape_name="l13b_4k", dtype=F16, pos=[511, 2047], seed=113),
    dict(name="l3_8b_8k_f32_bf16in", shape_name="l3_8b_8k", dtype=F32, pos=[300, 8191], seed=114, round_inputs_to=BF16),
    dict(name="l3_405b_f16", shape_name="l3_405b", dtype=F16, pos=[40, 2047], seed=115),
]


def golden_case(spec: dict) -> Case:
    return make_case(**spec)
