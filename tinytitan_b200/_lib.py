"""ctypes binding of libtinytitan_cuda.so (the C ABI declared in include/tinytitan_cuda.h).

The library is the product; this module only loads it. There is no fallback: when the shared
object is missing the import fails with an instruction to build it.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# TINYTITAN_CUDA_LIB selects another build of the same library (e.g. one compiled with experiment flags)
LIB_PATH = os.environ.get("TINYTITAN_CUDA_LIB") or os.path.join(_HERE, "libtinytitan_cuda.so")

TT_OK, TT_ERR_INVALID_ARG, TT_ERR_UNSUPPORTED_SHAPE, TT_ERR_OOM, TT_ERR_CUDA, TT_ERR_TIMEOUT, TT_ERR_BUSY = range(7)
TT_F16, TT_BF16 = 0, 1
TT_GDN_A_LOG_PREEXP, TT_GDN_V_TILED, TT_GDN_GATES_F32 = 1, 2, 4


class TinyTitanError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"[{status}] {message}")
        self.status = status


class InvalidArgument(TinyTitanError, ValueError):
    """The reference's precondition failures."""


class UnsupportedShape(TinyTitanError, NotImplementedError):
    pass


class ContextOptions(C.Structure):
    _fields_ = [("workspace_bytes", C.c_size_t), ("max_sessions", C.c_uint32), ("reserved", C.c_uint32)]


class KVFormat(C.Structure):
    _fields_ = [("bits", C.c_uint32), ("stride_bytes", C.c_uint32), ("value_bytes", C.c_uint32),
                ("group_size", C.c_uint32)]


class AttnSession(C.Structure):
    _fields_ = [("q", C.c_void_p), ("out", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p),
                ("seq_len", C.c_uint32), ("q_rows", C.c_uint32), ("kv_start", C.c_uint32),
                ("reserved", C.c_uint32)]


class AttnBatchParams(C.Structure):
    _fields_ = [("head_dim", C.c_uint32), ("n_q_heads", C.c_uint32), ("n_kv_heads", C.c_uint32),
                ("kv_token_stride_elements", C.c_uint32), ("q_row_stride_elements", C.c_uint32),
                ("out_row_stride_elements", C.c_uint32), ("scale", C.c_float), ("io_dtype", C.c_uint32)]


class SplitGeometry(C.Structure):
    _fields_ = [("effective_length", C.c_uint32), ("num_chunks", C.c_uint32), ("chunk_length", C.c_uint32),
                ("partial_threadgroups", C.c_uint32), ("use_swa_grouped_partial", C.c_uint32)]


class PrefillParams(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in (
        "start_position", "query_count", "head_dim", "n_q_heads", "n_kv_heads", "kv_valid_count",
        "sliding_window", "kv_token_stride_elements", "q_token_stride_elements",
        "o_token_stride_elements")] + [("scale", C.c_float)] + [(n, C.c_uint32) for n in (
            "kv_bits", "kv_token_stride_bytes", "kv_value_bytes", "kv_group_size")]


class GdnShape(C.Structure):
    _fields_ = [("n_k_heads", C.c_uint32), ("n_v_heads", C.c_uint32), ("key_dim", C.c_uint32),
                ("value_dim", C.c_uint32), ("flags", C.c_uint32), ("readout_scale", C.c_float)]


class GdnPreSession(C.Structure):
    _fields_ = [("tail", C.c_void_p), ("qkv", C.c_void_p), ("conv_out", C.c_void_p)]


class GdnSession(C.Structure):
    _fields_ = [("conv_out", C.c_void_p), ("a", C.c_void_p), ("b", C.c_void_p), ("state", C.c_void_p),
                ("y", C.c_void_p), ("checkpoint_state", C.c_void_p)]


ALLOC_FN = C.CFUNCTYPE(C.c_void_p, C.c_void_p, C.c_size_t)
RELEASE_FN = C.CFUNCTYPE(None, C.c_void_p, C.c_void_p)
COPY_FN = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t)
ZERO_FN = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_void_p, C.c_size_t)


class Allocator(C.Structure):
    _fields_ = [("user", C.c_void_p), ("alloc", ALLOC_FN), ("release", RELEASE_FN), ("copy", COPY_FN),
                ("zero", ZERO_FN), ("download", COPY_FN), ("upload", COPY_FN)]


class Arch(C.Structure):
    _fields_ = [("n_layers", C.c_uint32), ("layer_kind", C.POINTER(C.c_uint8))] + [(n, C.c_uint32) for n in (
        "n_kv_heads", "head_dim", "n_full_kv_heads", "full_head_dim", "sliding_window", "gdn_k_heads",
        "gdn_v_heads", "gdn_key_dim", "gdn_value_dim", "gdn_conv_kernel")]


class KVViewC(C.Structure):
    _fields_ = [("buffer", C.c_void_p), ("offset", C.c_size_t), ("stride", C.c_uint32),
                ("valid_token_count", C.c_uint32), ("precision_bits", C.c_uint32), ("value_bytes", C.c_uint32),
                ("group_size", C.c_uint32), ("ring_capacity", C.c_uint32)]


# name -> (restype, argtypes); every symbol include/tinytitan_cuda.h declares.
_u32, _vp, _f32p = C.c_uint32, C.c_void_p, C.POINTER(C.c_float)
class AttnExchange(C.Structure):
    _fields_ = [("peer_buffers", C.POINTER(C.c_void_p)), ("rank", C.c_uint32), ("world", C.c_uint32),
                ("epoch", C.c_uint32), ("reserved", C.c_uint32), ("out", C.c_void_p)]


SIGNATURES = {
    "tt_context_create": (_vp, [C.c_int, C.POINTER(ContextOptions), C.POINTER(C.c_int)]),
    "tt_context_destroy": (None, [_vp]),
    "tt_last_error_string": (C.c_char_p, [_vp]),
    "tt_status_string": (C.c_char_p, [C.c_int]),
    "tt_ctx_poll_status": (C.c_int, [_vp, _vp, C.POINTER(_u32)]),
    "tt_stream_synchronize": (C.c_int, [_vp, _vp]),
    "tt_ctx_launch_count": (C.c_uint64, [_vp]),
    "tt_ctx_profile_enable": (C.c_int, [_vp, C.c_int]),
    "tt_ctx_profile_collect": (C.c_int, [_vp, _f32p, _u32, C.POINTER(_u32)]),
    "tt_attn_decode": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32, _u32, C.c_float,
                                 C.POINTER(KVFormat), _vp, _u32]),
    "tt_attn_decode_window": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32, C.c_float,
                                        C.POINTER(KVFormat), _vp]),
    "tt_attn_decode_batched": (C.c_int, [_vp, _vp, C.POINTER(AttnSession), _u32, C.POINTER(AttnBatchParams)]),
    "tt_attn_decode_partial": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32, _u32, C.c_float, _u32,
                                         _u32, _vp, _vp, _vp]),
    "tt_attn_combine": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _u32, _u32, _u32, _vp, _u32]),
    "tt_attn_exchange_bytes": (C.c_size_t, [_u32, _u32, _u32]),
    "tt_peer_buffer_create": (C.c_int, [_vp, C.c_size_t, C.POINTER(_vp), C.c_char_p]),
    "tt_peer_buffer_open": (C.c_int, [_vp, C.c_char_p, C.POINTER(_vp)]),
    "tt_peer_buffer_close": (C.c_int, [_vp, _vp]),
    "tt_peer_buffer_destroy": (C.c_int, [_vp, _vp]),
    "tt_attn_exchange_combine": (C.c_int, [_vp, _vp, _vp, _vp, _vp, C.POINTER(_vp), _u32, _u32, _u32, _u32, _u32, _vp,
                                           _u32]),
    "tt_attn_decode_exchange": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32, _u32, C.c_float, _u32, _u32,
                                          C.POINTER(AttnExchange)]),
    "tt_attn_decode_noalloc": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32, _u32, C.c_float]),
    "tt_attn_prefill_causal_selected": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _vp, C.POINTER(PrefillParams), _u32, _u32, _vp, _u32,
                                                  _vp, _u32, _vp, _vp]),
    "tt_qsa_pool_blocks": (C.c_int, [_vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32, _u32, _vp, C.c_float, C.c_float]),
    "tt_qsa_query_norm_rope": (C.c_int, [_vp, _vp, _vp, _u32, _u32, _u32, _u32, _vp, C.c_float, C.c_float]),
    "tt_qsa_block_scores": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32, _u32]),
    "tt_qsa_select_keys": (C.c_int, [_vp, _vp, _vp, _u32, _u32, _u32, _u32, _u32, _vp, _u32, _vp, _u32, _vp]),
    "tt_kv_window_create": (_vp, [_u32, _u32, _u32, _u32, _u32, C.POINTER(Allocator), C.POINTER(C.c_int)]),
    "tt_kv_window_destroy": (None, [_vp]),
    "tt_kv_window_bytes": (C.c_size_t, [_vp]),
    "tt_kv_window_host_arena_bytes": (C.c_size_t, [_vp]),
    "tt_kv_window_tokens": (_u32, [_vp]),
    "tt_kv_window_prefill_chunk_tokens": (_u32, [_vp, _u32, _u32]),
    "tt_kv_window_base": (C.c_int, [_vp, _u32, _u32, C.POINTER(_vp), C.POINTER(_vp)]),
    "tt_kv_window_write_slot": (C.c_int, [_vp, _u32, _u32, _u32, C.POINTER(_vp), C.POINTER(_vp)]),
    "tt_kv_window_row_of": (C.c_int, [_vp, _u32, _u32, _u32, C.POINTER(C.c_int64)]),
    "tt_kv_window_prepare_decode": (C.c_int, [_vp, _u32, _u32, _u32, _vp, _u32, _vp, _vp]),
    "tt_kv_window_begin_prefill": (C.c_int, [_vp, _u32, _u32, _u32, _u32, C.POINTER(_vp), C.POINTER(_vp)]),
    "tt_kv_window_prepare_prefill": (C.c_int, [_vp, _u32, _u32, _u32, _u32, _vp, _u32, _vp, _vp, _vp, _vp, _u32]),
    "tt_kv_window_commit": (C.c_int, [_vp, _u32, _u32, _u32]),
    "tt_kv_window_reset_slot": (C.c_int, [_vp, _u32]),
    "tt_kv_window_host_row": (C.c_int, [_vp, _u32, _u32, _u32, C.c_int, _vp]),
    "tt_kv_window_counters": (None, [_vp, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]),
    "tt_gdn_decode_pre": (C.c_int, [_vp, _vp, C.POINTER(GdnPreSession), _u32, _vp, _u32, _u32, _u32, _u32]),
    "tt_gdn_prefill_pre": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32, _u32, C.c_int]),
    "tt_ctx_set_exchange_poll_limit": (C.c_int, [_vp, _u32]),
    "tt_attn_decode_noalloc_status": (C.c_int, [_vp, C.POINTER(_u32)]),
    "tt_attn_reference_split_geometry": (None, [_u32, _u32, _u32, _u32, C.c_int, C.POINTER(SplitGeometry)]),
    "tt_attn_plan_splits": (C.c_int, [C.POINTER(_u32), C.POINTER(_u32), _u32, _u32, _u32, _u32, _u32, C.c_size_t,
                                      C.POINTER(_u32), C.POINTER(_u32)]),
    "tt_attn_plan_verify_splits": (C.c_int, [C.POINTER(_u32), C.POINTER(_u32), _u32, _u32, _u32, _u32, _u32, C.c_size_t,
                                             C.POINTER(_u32), C.POINTER(_u32), C.POINTER(_u32)]),
    "tt_attn_pre": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32, C.c_float, C.c_float,
                              _u32, _u32, _u32]),
    "tt_attn_gate_mul": (C.c_int, [_vp, _vp, _vp, _vp, _u32]),
    "tt_kv_quantize_affine": (C.c_int, [_vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32, _u32, _u32, _u32]),
    "tt_attn_prefill_causal": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _vp, C.POINTER(PrefillParams), _u32, _u32]),
    "tt_attn_prefill_path": (C.c_int, [_vp, _vp, _vp, _vp, C.POINTER(PrefillParams), _u32]),
    "tt_gdn_step": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, C.POINTER(GdnShape), _u32, _u32, _vp]),
    "tt_gdn_step_batched": (C.c_int, [_vp, _vp, C.POINTER(GdnSession), _u32, _vp, _vp, C.POINTER(GdnShape), _u32,
                                      _u32]),
    "tt_gdn_scan_chunked": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, C.POINTER(GdnShape), _u32, _u32,
                                      _u32]),
    "tt_gdn_conv_mix": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _vp, _u32, _u32, _u32, C.c_int]),
    "tt_gdn_conv_tail_update": (C.c_int, [_vp, _vp, _vp, _vp, _u32, _u32, _u32]),
    "tt_gdn_conv_tail_checkpoint": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _u32, _u32]),
    "tt_gdn_qk_norm": (C.c_int, [_vp, _vp, _vp, _u32, _u32, _u32, _u32]),
    "tt_gdn_gated_norm": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _vp, _u32, _u32, _u32, C.c_int]),
    "tt_kv_row_layout": (None, [_u32, _u32, C.POINTER(_u32), C.POINTER(_u32)]),
    "tt_kv_cache_create": (_vp, [C.POINTER(Arch), _u32, _u32, _u32, C.c_int, _u32, C.POINTER(Allocator),
                                 C.POINTER(C.c_int)]),
    "tt_kv_cache_destroy": (None, [_vp]),
    "tt_kv_cache_reserve": (C.c_int, [_vp, _u32, _u32]),
    "tt_kv_cache_k_slot": (C.c_int, [_vp, _u32, _u32, _u32, C.POINTER(_vp)]),
    "tt_kv_cache_v_slot": (C.c_int, [_vp, _u32, _u32, _u32, C.POINTER(_vp)]),
    "tt_kv_cache_key_view": (C.c_int, [_vp, _u32, _u32, _u32, C.POINTER(KVViewC)]),
    "tt_kv_cache_value_view": (C.c_int, [_vp, _u32, _u32, _u32, C.POINTER(KVViewC)]),
    "tt_kv_cache_advance": (C.c_int, [_vp, _u32, _u32]),
    "tt_kv_cache_rewind": (C.c_int, [_vp, _u32, _u32]),
    "tt_kv_cache_reset": (C.c_int, [_vp]),
    "tt_kv_cache_reset_slot": (C.c_int, [_vp, _u32]),
    "tt_kv_cache_position": (_u32, [_vp, _u32]),
    "tt_kv_cache_capacity": (_u32, [_vp, _u32]),
    "tt_kv_cache_stride": (_u32, [_vp, _u32]),
    "tt_kv_cache_layer_kind": (_u32, [_vp, _u32]),
    "tt_kv_cache_buffer_length": (C.c_size_t, [_vp, _u32]),
    "tt_kv_cache_worst_case_bytes": (C.c_size_t, [C.POINTER(Arch), _u32, _u32, _u32]),
    "tt_kv_cache_snapshot_bytes": (C.c_size_t, [_vp, _u32]),
    "tt_kv_cache_snapshot_export": (C.c_int, [_vp, _vp, C.c_size_t, C.POINTER(C.c_size_t)]),
    "tt_kv_cache_snapshot_restore": (C.c_int, [_vp, _u32, _vp, C.c_size_t]),
    "tt_gdn_state_snapshot_bytes": (C.c_size_t, [_vp]),
    "tt_gdn_state_snapshot_export": (C.c_int, [_vp, _vp, C.c_size_t, C.POINTER(C.c_size_t)]),
    "tt_gdn_state_snapshot_restore": (C.c_int, [_vp, _vp, C.c_size_t]),
    "tt_gdn_state_create": (_vp, [C.POINTER(Arch), _u32, C.c_int, C.POINTER(Allocator), C.POINTER(C.c_int)]),
    "tt_gdn_state_destroy": (None, [_vp]),
    "tt_gdn_state_state_slot": (C.c_int, [_vp, _u32, _u32, C.POINTER(_vp)]),
    "tt_gdn_state_conv_tail_slot": (C.c_int, [_vp, _u32, _u32, C.POINTER(_vp)]),
    "tt_gdn_state_speculative_state_slot": (C.c_int, [_vp, _u32, _u32, C.POINTER(_vp)]),
    "tt_gdn_state_reset": (C.c_int, [_vp]),
    "tt_gdn_state_reset_slot": (C.c_int, [_vp, _u32]),
    "tt_gdn_state_speculative_restore": (C.c_int, [_vp, _vp]),
    "tt_gdn_state_bind_stream": (C.c_int, [_vp, _vp]),
    "tt_kv_cache_bind_stream": (C.c_int, [_vp, _vp]),
    "tt_kv_cache_write_rows": (C.c_int, [_vp, _vp, _u32, _vp, _vp, _u32, _vp, _vp, _u32]),
    "tt_gdn_state_bytes_per_layer": (C.c_size_t, [_vp]),
    "tt_gdn_state_conv_tail_bytes_per_layer": (C.c_size_t, [_vp]),
    "tt_gdn_state_is_linear": (C.c_int, [_vp, _u32]),
    "tt_gdn_state_worst_case_bytes": (C.c_size_t, [C.POINTER(Arch), _u32]),
}

_lib = None


def lib():
    """The loaded library. Raises when it has not been built (no fallback exists)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `make -C tinytitan_b200/csrc` "
                "(or __graft_entry__.build()); this package has no CPU or PyTorch fallback")
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(status: int, ctx=None) -> None:
    if status == TT_OK:
        return
    message = lib().tt_last_error_string(ctx).decode() if ctx else ""
    if not message:
        message = lib().tt_status_string(status).decode()
    if status == TT_ERR_INVALID_ARG:
        raise InvalidArgument(status, message)
    if status == TT_ERR_UNSUPPORTED_SHAPE:
        raise UnsupportedShape(status, message)
    raise TinyTitanError(status, message)
