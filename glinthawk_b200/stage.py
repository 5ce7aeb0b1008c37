"""Host-side wrapper of the attention stage for Python callers (tests, benchmark).

Method names, argument order and argument meaning follow the reference's ``LlamaOperations``
(src/arch/cuda/llama2/ops.cuh:26-77), its context views (src/models/llama2/context.hh:61-190) and
``PreallocatingContextManager`` (src/compute/contextman.hh:57-87); every method is one call into the C ABI of
``include/glinthawk_attn.h``.  torch is used only to own device memory and streams.
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from . import _lib
from ._lib import lib
from .shapes import AttnShape

_TORCH_DTYPE = {_lib.GH_F16: torch.float16, _lib.GH_F32: torch.float32, _lib.GH_BF16: torch.bfloat16}
_CODE = {v: k for k, v in _TORCH_DTYPE.items()}
_ELEM = {_lib.GH_F16: 2, _lib.GH_F32: 4, _lib.GH_BF16: 2}
_TYPESTR = {_lib.GH_F16: "<f2", _lib.GH_F32: "<f4", _lib.GH_BF16: "<i2"}


class GlinthawkAttnError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"[{status}: {lib.gh_status_string(status).decode()}] {message}")
        self.status = status


class _DevView:
    """Exposes raw device memory through the CUDA array interface so torch can wrap it without copying."""

    def __init__(self, ptr: int, shape: tuple[int, ...], typestr: str):
        self.__cuda_array_interface__ = {"shape": shape, "typestr": typestr, "data": (ptr, False), "version": 2}


def dtype_code(dtype) -> int:
    return dtype if isinstance(dtype, int) else _CODE[dtype]


def _ptr(t) -> C.c_void_p:
    if t is None:
        return C.c_void_p(0)
    if isinstance(t, torch.Tensor):
        assert t.is_contiguous()
        return C.c_void_p(t.data_ptr())
    if isinstance(t, np.ndarray):
        assert t.flags.c_contiguous
        return C.c_void_p(t.ctypes.data)
    return C.c_void_p(int(t))


def _stream(stream) -> C.c_void_p:
    if stream is None:
        return C.c_void_p(torch.cuda.current_stream().cuda_stream)
    return C.c_void_p(stream.cuda_stream if hasattr(stream, "cuda_stream") else int(stream))


class AttentionStage:
    """One attention-stage instance on one GPU: slot pool + operations."""

    def __init__(self, shape: AttnShape, dtype, *, n_layers_hosted: int | None = None, max_batch: int = 64,
                 max_contexts: int = 64, paged: bool = False, device: int = 0, decode_chunk: int = 0,
                 page_budget: int = 0, force_generic: bool = False, seq_len: int | None = None,
                 pipeline_steps: bool = False):
        self.shape = shape
        self.dtype_code = dtype_code(dtype)
        self.torch_dtype = _TORCH_DTYPE[self.dtype_code]
        self.elem = _ELEM[self.dtype_code]
        self.device = device
        self.seq_len = seq_len or shape.seq_len
        self.n_layers = n_layers_hosted or shape.n_layers
        cfg = _lib.Config(C.sizeof(_lib.Config), shape.n_heads, shape.n_kv_heads, shape.head_size, self.seq_len,
                          self.n_layers, self.dtype_code, max_batch, max_contexts,
                          _lib.GH_BACKING_PAGED if paged else _lib.GH_BACKING_STATIC, device, decode_chunk,
                          page_budget, 1 if force_generic else 0, 1 if pipeline_steps else 0)
        self._h = C.c_void_p(0)
        rc = lib.gh_attn_create(C.byref(cfg), C.byref(self._h))
        if rc != _lib.GH_OK:
            self._h = C.c_void_p(0)
            raise GlinthawkAttnError(rc, "gh_attn_create failed (a CUDA device is required; there is no CPU path)")
        self.row_elems = 2 * shape.kv_dim
        self._rope = None

    # -- plumbing -------------------------------------------------------------------------------------
    def _ck(self, rc: int) -> None:
        if rc != _lib.GH_OK:
            raise GlinthawkAttnError(rc, lib.gh_attn_last_error(self._h).decode())

    def close(self) -> None:
        if self._h:
            lib.gh_attn_destroy(self._h)
            self._h = C.c_void_p(0)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def stats(self) -> _lib.Stats:
        s = _lib.Stats()
        self._ck(lib.gh_attn_get_stats(self._h, C.byref(s)))
        return s

    def synchronize(self, stream=None) -> None:
        """Waits for `stream`; raises when a kernel of this stage has reported a timed-out wait."""
        self._ck(lib.gh_attn_synchronize(self._h, _stream(stream)))

    def clear_device_error(self) -> None:
        self._ck(lib.gh_attn_clear_device_error(self._h))

    def set_rope_tables(self, freq_cis_real: torch.Tensor, freq_cis_imag: torch.Tensor) -> None:
        assert freq_cis_real.dtype == self.torch_dtype and freq_cis_imag.dtype == self.torch_dtype
        self._rope = (freq_cis_real.contiguous(), freq_cis_imag.contiguous())  # keep them alive
        self._ck(lib.gh_attn_set_rope_tables(self._h, _ptr(self._rope[0]), _ptr(self._rope[1])))

    # -- PreallocatingContextManager ------------------------------------------------------------------
    def get_context(self, context_id: int) -> int:
        slot = C.c_int32(-1)
        self._ck(lib.gh_slot_acquire(self._h, context_id, C.byref(slot)))
        return slot.value

    def get_contexts(self, context_ids) -> np.ndarray | None:
        """All-or-nothing, like the reference: None when the pool cannot serve the whole batch."""
        ids = np.ascontiguousarray(context_ids, dtype=np.uint32)
        slots = np.empty(len(ids), dtype=np.int32)
        rc = lib.gh_slots_acquire_batch(self._h, len(ids), _ptr(ids), _ptr(slots))
        if rc == _lib.GH_ERR_NO_SLOT:
            return None
        self._ck(rc)
        return slots

    def lookup(self, context_id: int) -> int | None:
        slot = C.c_int32(-1)
        rc = lib.gh_slot_lookup(self._h, context_id, C.byref(slot))
        return slot.value if rc == _lib.GH_OK else None

    def release_context(self, context_id: int) -> bool:
        rc = lib.gh_slot_release(self._h, context_id)
        if rc == _lib.GH_ERR_NOT_FOUND:
            return False
        self._ck(rc)
        return True

    # -- Context / LayerContext / TokenContext ---------------------------------------------------------
    def prepare(self, slot: int, layer: int, pos: int, can_release: bool = False) -> None:
        self._ck(lib.gh_slot_prepare(self._h, slot, layer, pos, int(can_release)))

    def layer_ptr(self, slot: int, layer: int) -> int:
        p = C.c_void_p(0)
        self._ck(lib.gh_slot_layer_ptr(self._h, slot, layer, C.byref(p)))
        return p.value or 0

    def token_ptr(self, slot: int, layer: int, token: int) -> int:
        p = C.c_void_p(0)
        self._ck(lib.gh_slot_token_ptr(self._h, slot, layer, token, C.byref(p)))
        return p.value or 0

    def slot_bytes(self) -> int:
        return lib.gh_slot_bytes(self._h)

    def layer_view(self, slot: int, layer: int, n_tokens: int) -> torch.Tensor:
        """torch view [n_tokens, 2 * kv_dim] of a slot's rows (the rows must be prepared)."""
        ptr = self.layer_ptr(slot, layer)
        v = torch.as_tensor(_DevView(ptr, (n_tokens, self.row_elems), _TYPESTR[self.dtype_code]),
                            device=f"cuda:{self.device}")
        return v.view(torch.bfloat16) if self.dtype_code == _lib.GH_BF16 else v

    # -- fused hot path -----------------------------------------------------------------------------------
    def batch_begin(self, slots, pos, stream=None) -> None:
        slots = np.ascontiguousarray(slots, dtype=np.int32)
        pos = np.ascontiguousarray(pos, dtype=np.uint32)
        assert len(slots) == len(pos)
        self._ck(lib.gh_attn_batch_begin(self._h, len(slots), _ptr(slots), _ptr(pos), _stream(stream)))

    def append(self, layer: int, q_inout: torch.Tensor, kv_new: torch.Tensor, stream=None) -> None:
        self._ck(lib.gh_attn_append(self._h, layer, _ptr(q_inout), _ptr(kv_new), _stream(stream)))

    def decode(self, layer: int, q: torch.Tensor, xb: torch.Tensor, stream=None) -> None:
        self._ck(lib.gh_attn_decode(self._h, layer, _ptr(q), _ptr(xb), _stream(stream)))

    def step(self, layer: int, q_inout: torch.Tensor, kv_new: torch.Tensor, xb: torch.Tensor, stream=None) -> None:
        self._ck(lib.gh_attn_step(self._h, layer, _ptr(q_inout), _ptr(kv_new), _ptr(xb), _stream(stream)))

    def prefill_chunk(self, layer: int, slots, pos0, n_tokens: int, q_inout, kv_new, xb, stream=None) -> None:
        """n_tokens prompt tokens per context in one call; equals n_tokens consecutive step() calls."""
        slots = np.ascontiguousarray(slots, dtype=np.int32)
        pos0 = np.ascontiguousarray(pos0, dtype=np.uint32)
        self._ck(lib.gh_attn_prefill_chunk(self._h, layer, len(slots), _ptr(slots), _ptr(pos0), n_tokens,
                                           _ptr(q_inout), _ptr(kv_new), _ptr(xb), _stream(stream)))

    def project_append(self, layer: int, x, rms_weight, wq, wkv, q_out, stream=None) -> None:
        """rmsnorm + q / kv projections + RoPE + K/V append for the current batch (the reference's pre_attention_ops
        followed by copy_kv_cache and apply_rope); q_out receives the rotated queries."""
        self._ck(lib.gh_attn_project_append(self._h, layer, _ptr(x), _ptr(rms_weight), _ptr(wq), _ptr(wkv), _ptr(q_out),
                                            _stream(stream)))

    def forward_attention_host(self, layer: int, io_dtype, q_host, kv_host, xb_host, stream=None) -> None:
        self._ck(lib.gh_attn_forward_attention_host(self._h, layer, dtype_code(io_dtype), _ptr(q_host), _ptr(kv_host),
                                                    _ptr(xb_host), _stream(stream)))

    def forward_attention_state(self, state: np.ndarray, first_layer_hosted: int = 0, stream=None) -> None:
        """Llama2::forward_attention on a serialized BatchedInferenceState (a writable uint8 array), in place."""
        assert state.dtype == np.uint8 and state.flags.c_contiguous and state.flags.writeable
        self._ck(lib.gh_attn_forward_attention_state(self._h, first_layer_hosted, _ptr(state), state.nbytes, _stream(stream)))

    # -- the reference's operations, argument for argument -------------------------------------------
    @staticmethod
    def _ptr_array(ptrs) -> np.ndarray:
        return np.ascontiguousarray([int(p or 0) for p in ptrs], dtype=np.uint64)

    def copy_kv_cache(self, token_contexts, state_kv: torch.Tensor, batch_size: int, stream=None) -> None:
        rows = self._ptr_array(token_contexts)
        self._ck(lib.gh_op_copy_kv_cache(self._h, _ptr(rows), _ptr(state_kv), batch_size, _stream(stream)))

    def apply_rope(self, batch_size: int, token_positions, freq_cis_real, freq_cis_imag, state_q, token_contexts,
                   stream=None) -> None:
        rows = self._ptr_array(token_contexts)
        pos = np.ascontiguousarray(token_positions, dtype=np.uint32)
        self._ck(lib.gh_op_apply_rope(self._h, batch_size, _ptr(pos), _ptr(freq_cis_real), _ptr(freq_cis_imag),
                                      _ptr(state_q), _ptr(rows), _stream(stream)))

    def copy_kv_cache_apply_rope(self, batch_size: int, token_positions, freq_cis_real, freq_cis_imag, state_q,
                                 token_contexts, state_kv, stream=None) -> None:
        """copy_kv_cache then apply_rope on the same rows, as one launch."""
        rows = self._ptr_array(token_contexts)
        pos = np.ascontiguousarray(token_positions, dtype=np.uint32)
        self._ck(lib.gh_op_copy_kv_cache_apply_rope(self._h, batch_size, _ptr(pos), _ptr(freq_cis_real), _ptr(freq_cis_imag),
                                                    _ptr(state_q), _ptr(rows), _ptr(state_kv), _stream(stream)))

    def pre_attention_rope_append(self, batch_size: int, x, rms_att_weight, wq, wkv, state_q, token_positions,
                                  freq_cis_real, freq_cis_imag, token_contexts, stream=None) -> None:
        """pre_attention_ops (with the cache update) + apply_rope of the reference in one call, on tcgen05."""
        rows = self._ptr_array(token_contexts)
        pos = np.ascontiguousarray(token_positions, dtype=np.uint32)
        self._ck(lib.gh_op_project_append(self._h, batch_size, _ptr(x), _ptr(rms_att_weight), _ptr(wq), _ptr(wkv),
                                          _ptr(state_q), _ptr(pos), _ptr(freq_cis_real), _ptr(freq_cis_imag), _ptr(rows),
                                          _stream(stream)))

    def attention_0_gemm(self, query, layer_contexts, att, batch_size: int, token_positions, stream=None) -> None:
        bases = self._ptr_array(layer_contexts)
        pos = np.ascontiguousarray(token_positions, dtype=np.uint32)
        self._ck(lib.gh_op_attention_0_gemm(self._h, _ptr(query), _ptr(bases), _ptr(att), batch_size, _ptr(pos),
                                            _stream(stream)))

    def attention_softmax(self, att, token_positions, temp_buffer, batch_size: int, stream=None) -> None:
        pos = np.ascontiguousarray(token_positions, dtype=np.uint32)
        self._ck(lib.gh_op_attention_softmax(self._h, _ptr(att), _ptr(pos), _ptr(temp_buffer), batch_size,
                                             _stream(stream)))

    def attention_2_gemm(self, att, layer_contexts, xb, batch_size: int, token_positions, stream=None) -> None:
        bases = self._ptr_array(layer_contexts)
        pos = np.ascontiguousarray(token_positions, dtype=np.uint32)
        self._ck(lib.gh_op_attention_2_gemm(self._h, _ptr(att), _ptr(bases), _ptr(xb), batch_size, _ptr(pos),
                                            _stream(stream)))

    def attention_fused(self, query, layer_contexts, xb, batch_size: int, token_positions, stream=None) -> None:
        bases = self._ptr_array(layer_contexts)
        pos = np.ascontiguousarray(token_positions, dtype=np.uint32)
        self._ck(lib.gh_op_attention_fused(self._h, _ptr(query), _ptr(bases), _ptr(xb), batch_size, _ptr(pos),
                                           _stream(stream)))

    def convert_and_copy(self, dst, dst_dtype, src, src_dtype, size: int, copy_type: int) -> None:
        self._ck(lib.gh_op_convert_and_copy(self._h, _ptr(dst), dtype_code(dst_dtype), _ptr(src),
                                            dtype_code(src_dtype), size, copy_type))

    # -- helpers ---------------------------------------------------------------------------------------
    def fill_normal(self, dst, n: int, dtype, seed: int, offset: int = 0, stream=None) -> None:
        self._ck(lib.gh_fill_normal(self._h, _ptr(dst), n, dtype_code(dtype), seed, offset, _stream(stream)))


def plan_batch(pos, *, blocks_per_item: int, sm_count: int = 148, tile: int = 64, fixed_chunk: int = 0,
               max_items: int = 4096):
    """Host-only view of the split plan (no device needed): returns (items[n,4], chunk)."""
    pos = np.ascontiguousarray(pos, dtype=np.uint32)
    items = np.zeros((max_items, 4), dtype=np.int32)
    n, chunk = C.c_uint32(0), C.c_uint32(0)
    rc = lib.gh_plan_batch(blocks_per_item, sm_count, tile, fixed_chunk, max_items, len(pos), _ptr(pos), _ptr(items),
                           C.byref(n), C.byref(chunk))
    if rc != _lib.GH_OK:
        raise GlinthawkAttnError(rc, "gh_plan_batch")
    return items[: n.value].copy(), chunk.value


def plan_projection(shape: AttnShape, *, sm_count: int = 148, max_pieces: int = 8192):
    """Host-only view of how the fused projection deals (feature tile, k-block) units to the SMs: returns
    (plan dict, pieces[n, 6] = {cta, tile, k0, k1, piece index, pieces of the tile})."""
    plan = np.zeros(5, dtype=np.uint32)
    pieces = np.zeros((max_pieces, 6), dtype=np.int32)
    n = C.c_uint32(0)
    rc = lib.gh_plan_projection(shape.n_heads, shape.head_size, shape.kv_dim, sm_count, _ptr(plan), _ptr(pieces),
                                max_pieces, C.byref(n))
    if rc != _lib.GH_OK:
        raise GlinthawkAttnError(rc, "gh_plan_projection")
    keys = ("ctas", "units_per_cta", "max_segs", "n_tiles", "kblocks")
    return dict(zip(keys, (int(v) for v in plan))), pieces[: n.value].copy()


def decode_noalloc(shape: AttnShape, dtype, layer_contexts, token_positions, query, xb, stream=None) -> None:
    """``gh_decode_noalloc``: fused decode attention for callers that must not allocate device memory (a worker
    whose GPU memory is fully handed out at start-up, a loop that cannot take cudaMalloc's device-wide
    synchronisation).  Needs no stage; scratch is a fixed array inside the library.  Raises with the library's
    message when a size limit is exceeded."""
    bases = np.ascontiguousarray([int(p or 0) for p in layer_contexts], dtype=np.uint64)
    pos = np.ascontiguousarray(token_positions, dtype=np.uint32)
    sh = _lib.NoallocShape(C.sizeof(_lib.NoallocShape), shape.n_heads, shape.n_kv_heads, shape.head_size,
                           dtype_code(dtype))
    rc = lib.gh_decode_noalloc(C.byref(sh), len(pos), _ptr(bases), _ptr(pos), _ptr(query), _ptr(xb), _stream(stream))
    if rc != _lib.GH_OK:
        raise GlinthawkAttnError(rc, lib.gh_decode_noalloc_error().decode())
