"""Host-side mirror of the reference's attention operator classes over the C ABI.

The classes keep the names, argument meaning and error behaviour of the Swift operators they
stand in for, so call sites and tests read like the reference's:

  Attention         sources/TinyTitan/Kernels/Attention/Attention.swift:270-470
  PrefillAttention  sources/TinyTitan/Kernels/Attention/PrefillAttention.swift:5-55, :165-258
  GDN               sources/TinyTitan/Kernels/GDN/GDN.swift:318-396

A "buffer" is a torch CUDA tensor or an integer device address; `*_offset` arguments are byte
offsets as in the reference. `command_buffer` is the CUDA stream handle (default: torch's
current stream); every encode* call enqueues and returns.
"""
from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass
from typing import Optional, Sequence

from . import _lib as L


def _addr(buf, offset: int = 0) -> int:
    if buf is None:
        return 0
    base = buf.data_ptr() if hasattr(buf, "data_ptr") else int(buf)
    return base + int(offset)


def _stream(command_buffer) -> int:
    if command_buffer is not None:
        return int(getattr(command_buffer, "cuda_stream", command_buffer))
    import torch
    return int(torch.cuda.current_stream().cuda_stream)


def _dtype_of(buf, default=L.TT_F16) -> int:
    dt = getattr(buf, "dtype", None)
    if dt is None:
        return default
    import torch
    if dt == torch.bfloat16:
        return L.TT_BF16
    return L.TT_F16


class Context:
    """One per device and per runner: device scratch allocated once, not re-entrant."""

    def __init__(self, device: int = 0, workspace_bytes: int = 0, max_sessions: int = 0):
        err = C.c_int(0)
        opts = L.ContextOptions(workspace_bytes, max_sessions, 0)
        self.handle = L.lib().tt_context_create(device, C.byref(opts), C.byref(err))
        if not self.handle:
            L.check(err.value or L.TT_ERR_CUDA)
            raise L.TinyTitanError(L.TT_ERR_CUDA, "tt_context_create failed")
        self.device = device

    def close(self):
        if getattr(self, "handle", None):
            L.lib().tt_context_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def check(self, status: int):
        L.check(status, self.handle)

    def poll_status(self, command_buffer=None) -> int:
        flags = C.c_uint32(0)
        self.check(L.lib().tt_ctx_poll_status(self.handle, _stream(command_buffer), C.byref(flags)))
        return flags.value

    def synchronize(self, command_buffer=None):
        self.check(L.lib().tt_stream_synchronize(self.handle, _stream(command_buffer)))

    PROFILE_DECODE_PARTIAL = 1
    PROFILE_GDN_STEP = 2
    PROFILE_EXCHANGE = 4

    def profile_enable(self, enabled=True):
        """`enabled`: False/0 off, True/1 the split-KV pass-1 kernel, or a mask of PROFILE_*."""
        self.check(L.lib().tt_ctx_profile_enable(self.handle, int(enabled)))

    def profile_collect(self):
        """Durations (ms), in launch order, of the profiled launches recorded since the last collect."""
        buf = (C.c_float * 256)()
        n = C.c_uint32(0)
        self.check(L.lib().tt_ctx_profile_collect(self.handle, buf, 256, C.byref(n)))
        return [buf[i] for i in range(n.value)]

    def set_exchange_poll_limit(self, polls: int):
        """Polls (~0.25 us each) the exchange kernels wait for peers before giving up; 0 = default."""
        self.check(L.lib().tt_ctx_set_exchange_poll_limit(self.handle, polls))

    @property
    def launch_count(self) -> int:
        return int(L.lib().tt_ctx_launch_count(self.handle))


@dataclass
class KVFormat:
    bits: int = 16
    stride: int = 0
    value_bytes: int = 0
    group_size: int = 64


@dataclass
class AttentionSplitGeometry:
    effective_length: int
    num_chunks: int
    chunk_length: int
    partial_threadgroups: int
    use_swa_grouped_partial: bool


@dataclass
class DecodeSession:
    """One row group of a batched / few-token decode step (tt_attn_session)."""
    q: object
    out: object
    k: object
    v: object
    seq_len: int
    q_rows: int = 1
    kv_start: int = 0
    q_offset: int = 0
    out_offset: int = 0
    k_offset: int = 0
    v_offset: int = 0


class Attention:
    max_q_heads = 96
    max_head_dim = 512

    def __init__(self, context: Context):
        self.context = context

    @staticmethod
    def default_scale(head_dim: int) -> float:
        return 1.0 / math.sqrt(head_dim)

    @staticmethod
    def split_geometry(num_q_heads: int, num_kv_heads: int, seq_len: int, kv_start: int,
                       prefer_gqa_swa: bool) -> AttentionSplitGeometry:
        g = L.SplitGeometry()
        L.lib().tt_attn_reference_split_geometry(num_q_heads, num_kv_heads, seq_len, kv_start,
                                                 int(prefer_gqa_swa), C.byref(g))
        return AttentionSplitGeometry(g.effective_length, g.num_chunks, g.chunk_length,
                                      g.partial_threadgroups, bool(g.use_swa_grouped_partial))

    def _encode(self, command_buffer, q, q_offset, k, k_offset, v, v_offset, out, out_offset, head_dim,
                num_q_heads, num_kv_heads, seq_len, kv_start, scale, kv_format, keep_mask, ring_capacity):
        if num_kv_heads <= 0 or num_q_heads % num_kv_heads != 0:
            raise L.InvalidArgument(L.TT_ERR_INVALID_ARG, "numQHeads must be a multiple of numKVHeads for GQA")
        if head_dim > self.max_head_dim:
            raise L.InvalidArgument(L.TT_ERR_INVALID_ARG, "head_dim must be <= 512")
        fmt = None
        if kv_format is not None:
            fmt = L.KVFormat(kv_format.bits, kv_format.stride, kv_format.value_bytes, kv_format.group_size)
        sc = self.default_scale(head_dim) if scale is None else scale
        self.context.check(L.lib().tt_attn_decode(
            self.context.handle, _stream(command_buffer), _addr(q, q_offset), _addr(k, k_offset),
            _addr(v, v_offset), _addr(out, out_offset), head_dim, num_q_heads, num_kv_heads, seq_len, kv_start,
            sc, C.byref(fmt) if fmt is not None else None, _addr(keep_mask), ring_capacity))

    def encode_full(self, q, k, v, out, head_dim, num_q_heads, num_kv_heads, seq_len, scale=None,
                    kv_format: Optional[KVFormat] = None, keep_mask=None, command_buffer=None, q_offset=0,
                    k_offset=0, v_offset=0, out_offset=0):
        """Attention.encodeFull (Attention.swift:270-307)."""
        if seq_len <= 0:
            raise L.InvalidArgument(L.TT_ERR_INVALID_ARG, "full attention requires at least one KV position")
        self._encode(command_buffer, q, q_offset, k, k_offset, v, v_offset, out, out_offset, head_dim, num_q_heads,
                     num_kv_heads, seq_len, 0, scale, kv_format, keep_mask, 0)

    def encode_window(self, q, k, v, out, head_dim, num_q_heads, num_kv_heads, sel_rows, sel_count, scale=None,
                      kv_format: Optional[KVFormat] = None, command_buffer=None):
        """encodeFull(windowSelection:): attention over sel_count keys, key s at row sel_rows[s]."""
        fmt = None
        if kv_format is not None:
            fmt = L.KVFormat(kv_format.bits, kv_format.stride, kv_format.value_bytes, kv_format.group_size)
        self.context.check(L.lib().tt_attn_decode_window(
            self.context.handle, _stream(command_buffer), _addr(q), _addr(k), _addr(v), _addr(out), head_dim,
            num_q_heads, num_kv_heads, sel_count, self.default_scale(head_dim) if scale is None else scale,
            C.byref(fmt) if fmt is not None else None, _addr(sel_rows)))

    def encode_swa(self, q, k, v, out, head_dim, num_q_heads, num_kv_heads, seq_len, window, scale=None,
                   ring_capacity=0, kv_format: Optional[KVFormat] = None, command_buffer=None, q_offset=0,
                   k_offset=0, v_offset=0, out_offset=0):
        """Attention.encodeSWA (Attention.swift:233-266): keys [max(0, seqLen-window), seqLen)."""
        kv_start = seq_len - window if seq_len > window else 0
        self._encode(command_buffer, q, q_offset, k, k_offset, v, v_offset, out, out_offset, head_dim, num_q_heads,
                     num_kv_heads, seq_len, kv_start, scale, kv_format, None, ring_capacity)

    def encode_batched(self, sessions: Sequence[DecodeSession], head_dim, num_q_heads, num_kv_heads,
                       kv_token_stride_elements=None, q_row_stride_elements=None, out_row_stride_elements=None,
                       scale=None, io_dtype=None, command_buffer=None):
        """All rows of a batched decode / verify step in one launch pair (tt_attn_decode_batched)."""
        n = len(sessions)
        arr = (L.AttnSession * max(n, 1))()
        for i, s in enumerate(sessions):
            arr[i] = L.AttnSession(_addr(s.q, s.q_offset), _addr(s.out, s.out_offset), _addr(s.k, s.k_offset),
                                   _addr(s.v, s.v_offset), s.seq_len, s.q_rows, s.kv_start, 0)
        tight_q = num_q_heads * head_dim
        p = L.AttnBatchParams(head_dim, num_q_heads, num_kv_heads,
                              kv_token_stride_elements or num_kv_heads * head_dim,
                              q_row_stride_elements or tight_q, out_row_stride_elements or tight_q,
                              self.default_scale(head_dim) if scale is None else scale,
                              io_dtype if io_dtype is not None else (_dtype_of(sessions[0].q) if n else L.TT_F16))
        self.context.check(L.lib().tt_attn_decode_batched(self.context.handle, _stream(command_buffer), arr, n,
                                                          C.byref(p)))

    def prepare_batch(self, sessions: Sequence[DecodeSession], head_dim, num_q_heads, num_kv_heads,
                      kv_token_stride_elements=None, q_row_stride_elements=None, out_row_stride_elements=None,
                      scale=None, io_dtype=None):
        """The argument block of encode_batched built once, for a step that is replayed with the
        same buffers (the reference re-encodes the same bindings every token as well)."""
        n = len(sessions)
        arr = (L.AttnSession * max(n, 1))()
        for i, s in enumerate(sessions):
            arr[i] = L.AttnSession(_addr(s.q, s.q_offset), _addr(s.out, s.out_offset), _addr(s.k, s.k_offset),
                                   _addr(s.v, s.v_offset), s.seq_len, s.q_rows, s.kv_start, 0)
        tight_q = num_q_heads * head_dim
        p = L.AttnBatchParams(head_dim, num_q_heads, num_kv_heads,
                              kv_token_stride_elements or num_kv_heads * head_dim,
                              q_row_stride_elements or tight_q, out_row_stride_elements or tight_q,
                              self.default_scale(head_dim) if scale is None else scale,
                              io_dtype if io_dtype is not None else (_dtype_of(sessions[0].q) if n else L.TT_F16))
        return (arr, n, p)

    def encode_prepared(self, batch, command_buffer=None):
        arr, n, p = batch
        self.context.check(L.lib().tt_attn_decode_batched(self.context.handle, _stream(command_buffer), arr, n,
                                                          C.byref(p)))

    def encode_pre(self, q_packed, q_out, gate_out, k_rows, q_norm_weight, k_norm_weight, head_dim, num_q_heads,
                   num_kv_heads, rotary_dim, theta, eps, position, rows=1, k_row_stride_elements=None,
                   command_buffer=None):
        """Split [query; gate], per-head q/k RMS norm, NeoX partial RoPE (encodeGatedFullPostProjection)."""
        self.context.check(L.lib().tt_attn_pre(
            self.context.handle, _stream(command_buffer), _addr(q_packed), _addr(q_out), _addr(gate_out), _addr(k_rows),
            _addr(q_norm_weight), _addr(k_norm_weight), head_dim, num_q_heads, num_kv_heads, rotary_dim, theta, eps,
            position, rows, k_row_stride_elements or num_kv_heads * head_dim))

    def encode_gate_mul(self, out, gate, count, command_buffer=None):
        """out *= sigmoid(gate): the full-attention output gate."""
        self.context.check(L.lib().tt_attn_gate_mul(self.context.handle, _stream(command_buffer), _addr(out),
                                                    _addr(gate), count))

    def encode_partial(self, q, k, v, head_dim, num_q_heads, num_kv_heads, seq_len, kv_start, m_out, d_out, o_out,
                       scale=None, kv_token_stride_elements=0, io_dtype=None, command_buffer=None):
        """Pass 1 alone: one unnormalised (m, d, o) triple per q head for this device's keys."""
        self.context.check(L.lib().tt_attn_decode_partial(
            self.context.handle, _stream(command_buffer), _addr(q), _addr(k), _addr(v), head_dim, num_q_heads,
            num_kv_heads, seq_len, kv_start, self.default_scale(head_dim) if scale is None else scale,
            kv_token_stride_elements, io_dtype if io_dtype is not None else _dtype_of(q), _addr(m_out), _addr(d_out),
            _addr(o_out)))

    def encode_combine(self, m, d, o, n_parts, num_q_heads, head_dim, out, io_dtype=None, command_buffer=None):
        """Pass 2 alone: log-sum-exp merge of n_parts triples."""
        self.context.check(L.lib().tt_attn_combine(
            self.context.handle, _stream(command_buffer), _addr(m), _addr(d), _addr(o), n_parts, num_q_heads,
            head_dim, _addr(out), io_dtype if io_dtype is not None else _dtype_of(out)))

    def encode_exchange_combine(self, m, d, o, exchange, num_q_heads, head_dim, out, io_dtype=None, command_buffer=None):
        """Cross-GPU merge in one kernel: this rank's triple goes to every rank's exchange buffer over
        peer memory, the kernel waits (bounded) for the others' and merges. `exchange` is a PeerExchange."""
        self.context.check(L.lib().tt_attn_exchange_combine(
            self.context.handle, _stream(command_buffer), _addr(m), _addr(d), _addr(o), exchange.pointer_array,
            exchange.rank, exchange.world, num_q_heads, head_dim, exchange.next_epoch(), _addr(out),
            io_dtype if io_dtype is not None else _dtype_of(out)))


    def encode_decode_exchange(self, q, k, v, head_dim, num_q_heads, num_kv_heads, seq_len, kv_start, exchange, out,
                               scale=None, kv_token_stride_elements=0, io_dtype=None, command_buffer=None):
        """One step of a session split over GPUs in two launches: pass 1 over this GPU's rows, then the
        local merge fused with the peer exchange and the cross-GPU merge."""
        x = L.AttnExchange(exchange.pointer_array, exchange.rank, exchange.world, exchange.next_epoch(), 0, _addr(out))
        self.context.check(L.lib().tt_attn_decode_exchange(
            self.context.handle, _stream(command_buffer), _addr(q), _addr(k), _addr(v), head_dim, num_q_heads,
            num_kv_heads, seq_len, kv_start, scale if scale is not None else head_dim ** -0.5,
            kv_token_stride_elements, io_dtype if io_dtype is not None else _dtype_of(q), C.byref(x)))


class PeerExchange:
    """One exchange buffer per rank, mapped into every rank of the group (one process per GPU, one node).

    `gather_handles(handle_bytes) -> list of every rank's handle bytes` is the host channel; with
    torch.distributed it is an all_gather_object."""

    def __init__(self, context: Context, rank: int, world: int, num_q_heads: int, head_dim: int, gather_handles):
        self.context, self.rank, self.world = context, rank, world
        self.bytes = L.lib().tt_attn_exchange_bytes(world, num_q_heads, head_dim)
        mine = C.c_void_p()
        handle = C.create_string_buffer(64)
        context.check(L.lib().tt_peer_buffer_create(context.handle, self.bytes, C.byref(mine), handle))
        self.local = mine.value
        handles = gather_handles(handle.raw)
        self.opened = []
        ptrs = []
        for r in range(world):
            if r == rank:
                ptrs.append(self.local)
                continue
            p = C.c_void_p()
            context.check(L.lib().tt_peer_buffer_open(context.handle, handles[r], C.byref(p)))
            self.opened.append(p.value)
            ptrs.append(p.value)
        self.pointer_array = (C.c_void_p * world)(*ptrs)
        self.epoch = 0

    def next_epoch(self) -> int:
        self.epoch += 1
        return self.epoch

    def close(self):
        """Unmap the peers' buffers and free this rank's (every rank must have stopped using them)."""
        for p in self.opened:
            L.lib().tt_peer_buffer_close(self.context.handle, p)
        self.opened = []
        if self.local:
            L.lib().tt_peer_buffer_destroy(self.context.handle, self.local)
            self.local = None


def quantize_kv_rows(context: Context, source, destination, element_count: int, bits: int, tokens: int,
                     source_stride_elements=None, destination_stride_bytes=None, values_bytes=None, group_size=64,
                     command_buffer=None, source_offset=0, destination_offset=0):
    """kv_cache_quantize_affine: fp16 rows -> the cache's packed row format (codes, scales, biases)."""
    packed = (element_count * bits + 7) // 8
    vb = values_bytes if values_bytes is not None else (packed + 1) & ~1
    groups = (element_count + group_size - 1) // group_size
    context.check(L.lib().tt_kv_quantize_affine(
        context.handle, _stream(command_buffer), _addr(source, source_offset), _addr(destination, destination_offset),
        source_stride_elements or element_count, destination_stride_bytes or vb + groups * 4, vb, element_count, bits,
        group_size, tokens))


@dataclass
class PrefillAttentionParams:
    """PrefillAttentionParams (PrefillAttention.swift:5-55), same fields and defaults."""
    start_position: int
    query_count: int
    head_dim: int
    num_q_heads: int
    num_kv_heads: int
    kv_valid_count: int
    sliding_window: int
    kv_token_stride_elements: int
    q_token_stride_elements: int
    o_token_stride_elements: int
    scale: float
    kv_bits: int = 16
    kv_token_stride_bytes: int = 0
    kv_value_bytes: int = 0
    kv_group_size: int = 64

    def to_c(self) -> "L.PrefillParams":
        return L.PrefillParams(self.start_position, self.query_count, self.head_dim, self.num_q_heads,
                               self.num_kv_heads, self.kv_valid_count, self.sliding_window,
                               self.kv_token_stride_elements, self.q_token_stride_elements,
                               self.o_token_stride_elements, self.scale, self.kv_bits,
                               self.kv_token_stride_bytes, self.kv_value_bytes, self.kv_group_size)


class PrefillAttention:
    def __init__(self, context: Context):
        self.context = context

    def encode_causal(self, q, k, v, out, params: PrefillAttentionParams, kv_ring_capacity=0, io_dtype=None,
                      command_buffer=None, q_offset=0, k_offset=0, v_offset=0, out_offset=0, keep_mask=None,
                      keep_stride=0, keep_indices=None, keep_index_stride=0, keep_counts=None, keep_rows=None):
        """PrefillAttention.encodeCausal (PrefillAttention.swift:165-258); the keep* arguments are its
        per-query key selection (mask, compact index list with counts, window rows)."""
        cp = params.to_c()
        if keep_mask is not None or keep_indices is not None or keep_counts is not None or keep_rows is not None:
            self.context.check(L.lib().tt_attn_prefill_causal_selected(
                self.context.handle, _stream(command_buffer), _addr(q, q_offset), _addr(k, k_offset),
                _addr(v, v_offset), _addr(out, out_offset), C.byref(cp), kv_ring_capacity,
                io_dtype if io_dtype is not None else _dtype_of(q), _addr(keep_mask) or None, keep_stride,
                _addr(keep_indices) or None, keep_index_stride, _addr(keep_counts) or None, _addr(keep_rows) or None))
            return
        self.context.check(L.lib().tt_attn_prefill_causal(
            self.context.handle, _stream(command_buffer), _addr(q, q_offset), _addr(k, k_offset),
            _addr(v, v_offset), _addr(out, out_offset), C.byref(cp), kv_ring_capacity,
            io_dtype if io_dtype is not None else _dtype_of(q)))

    @staticmethod
    def selected_path(q, k, v, out, params: PrefillAttentionParams, kv_ring_capacity=0, q_offset=0, k_offset=0,
                      v_offset=0, out_offset=0) -> str:
        cp = params.to_c()
        path = L.lib().tt_attn_prefill_path(_addr(q, q_offset), _addr(k, k_offset), _addr(v, v_offset),
                                            _addr(out, out_offset), C.byref(cp), kv_ring_capacity)
        return "tcgen05" if path == 1 else "generic"


@dataclass(frozen=True)
class SparseIndexerConfig:
    """SparseIndexerConfig of the reference's ArchConfig (ModelTypes.swift:129-133)."""
    num_heads: int = 4
    head_dim: int = 128
    budget: int = 2048
    compress_ratio: int = 4


class QSAIndexer:
    """Device side of QSAIndexer (sources/TinyTitan/Kernels/Attention/QSAIndexer.swift): pooled-key cache
    maintenance, block scores and the key selection. The caller owns the buffers (raw keys, pooled
    blocks, scores, selection), like the Swift class; projections are the caller's GEMVs."""

    def __init__(self, context: Context, config: SparseIndexerConfig, rope_theta: float = 1e7, eps: float = 1e-6,
                 budget: Optional[int] = None):
        self.context, self.config = context, config
        self.heads, self.head_dim, self.compress_ratio = config.num_heads, config.head_dim, config.compress_ratio
        self.budget = config.budget if budget is None else budget
        self.rope_theta, self.eps = rope_theta, eps

    @property
    def selection_width(self) -> int:
        """Cells a query keeps: the budget plus the tail block's extra members."""
        return self.budget + self.compress_ratio - 1

    def encode_pool(self, raw_keys, pooled, first_block, block_count, visible_keys, key_norm_weight=None,
                    command_buffer=None):
        """encodePoolPrefill / the repool of encodeAppendKey: pool + norm + rotation of a block range."""
        self.context.check(L.lib().tt_qsa_pool_blocks(
            self.context.handle, _stream(command_buffer), _addr(raw_keys), _addr(pooled), self.head_dim, first_block,
            block_count, self.compress_ratio, visible_keys, _addr(key_norm_weight) or None, self.eps, self.rope_theta))

    def encode_pool_prefill(self, raw_keys, pooled, start_position, tokens, key_norm_weight, command_buffer=None):
        first = start_position // self.compress_ratio
        last = (start_position + tokens - 1) // self.compress_ratio
        self.encode_pool(raw_keys, pooled, first, last - first + 1, start_position + tokens, key_norm_weight, command_buffer)

    def encode_append_key(self, raw_keys, pooled, position, key_norm_weight, command_buffer=None):
        """Repool the block token `position` joined (its raw key is already in the cache)."""
        self.encode_pool(raw_keys, pooled, position // self.compress_ratio, 1, position + 1, key_norm_weight, command_buffer)

    def encode_query(self, query, rows, position, query_norm_weight, command_buffer=None):
        self.context.check(L.lib().tt_qsa_query_norm_rope(
            self.context.handle, _stream(command_buffer), _addr(query), self.head_dim, self.heads, rows, position,
            _addr(query_norm_weight), self.eps, self.rope_theta))

    def encode_scores(self, query, pooled, scores, blocks, rows=1, score_stride=None, command_buffer=None):
        """encodeScores (rows = 1) / encodeScoresPrefill after the query's norm and rotation."""
        self.context.check(L.lib().tt_qsa_block_scores(
            self.context.handle, _stream(command_buffer), _addr(query), _addr(pooled), _addr(scores), self.head_dim,
            self.heads, blocks, rows, score_stride or blocks))

    def encode_select_keys(self, scores, score_stride, start_position, rows, keep=None, keep_stride=0, indices=None,
                           index_stride=0, counts=None, command_buffer=None):
        """encodeSelectKeys / selectKeysCompact (rows = 1) and selectKeysPrefill, mask and compact list at once."""
        self.context.check(L.lib().tt_qsa_select_keys(
            self.context.handle, _stream(command_buffer), _addr(scores), score_stride, start_position, rows,
            self.compress_ratio, self.selection_width, _addr(keep) or None, keep_stride, _addr(indices) or None,
            index_stride, _addr(counts) or None))


@dataclass(frozen=True)
class LinearAttentionConfig:
    """LinearAttentionConfig (sources/TinyTitanCore/Format/ModelTypes+Configs.swift:147-188)."""
    num_k_heads: int
    num_v_heads: int
    key_head_dim: int
    value_head_dim: int
    conv_kernel_size: int = 4

    @property
    def qkv_dim(self) -> int:
        return 2 * self.num_k_heads * self.key_head_dim + self.num_v_heads * self.value_head_dim

    @property
    def value_dim(self) -> int:
        return self.num_v_heads * self.value_head_dim


@dataclass
class GDNSession:
    conv_out: object
    a_proj: object
    b_proj: object
    state: object
    y: object
    checkpoint_state: object = None
    conv_out_offset: int = 0
    a_proj_offset: int = 0
    b_proj_offset: int = 0
    state_offset: int = 0
    y_offset: int = 0
    checkpoint_state_offset: int = 0


class GDN:
    def __init__(self, context: Context, config: LinearAttentionConfig, a_log_preexp=False, v_tiled=False,
                 readout_scale=1.0, gates_f32=False):
        self.context = context
        self.config = config
        flags = (L.TT_GDN_A_LOG_PREEXP if a_log_preexp else 0) | (L.TT_GDN_V_TILED if v_tiled else 0) | \
                (L.TT_GDN_GATES_F32 if gates_f32 else 0)
        self.shape = L.GdnShape(config.num_k_heads, config.num_v_heads, config.key_head_dim,
                                config.value_head_dim, flags, readout_scale)

    # ---- the elementwise kernels around the delta rule (GDN.swift:185-313, :399-427) ----
    def encode_conv_decode(self, tail, qkv, conv_weight, out, command_buffer=None, tail_offset=0, qkv_offset=0,
                           conv_weight_offset=0, out_offset=0):
        """GDN.encodeConvDecode: conv + SiLU of one row, the tail shifted in place."""
        self.context.check(L.lib().tt_gdn_conv_mix(
            self.context.handle, _stream(command_buffer), _addr(tail, tail_offset), _addr(qkv, qkv_offset),
            _addr(conv_weight, conv_weight_offset), _addr(out, out_offset), self.config.qkv_dim,
            self.config.conv_kernel_size, 1, 1))

    def encode_decode_prologue(self, sessions, conv_weight, command_buffer=None):
        """encodeConvDecode + encodeQKNorm for a batch of sessions in one launch; `sessions` is a sequence of
        (tail, qkv, conv_out) buffers (tensors or device addresses)."""
        n = len(sessions)
        arr = (L.GdnPreSession * max(n, 1))()
        for i, (tail, qkv, conv_out) in enumerate(sessions):
            arr[i] = L.GdnPreSession(_addr(tail), _addr(qkv), _addr(conv_out))
        self.context.check(L.lib().tt_gdn_decode_pre(
            self.context.handle, _stream(command_buffer), arr, n, _addr(conv_weight), self.config.num_k_heads,
            self.config.key_head_dim, self.config.qkv_dim, self.config.conv_kernel_size))

    def encode_prefill_prologue(self, tail, qkv_rows, conv_weight, conv_out, rows, checkpoint_tail=None, update_tail=True,
                                command_buffer=None):
        """encodeConvPrefill + encodeConvTailCheckpoint + encodeConvTailUpdate + encodeQKNorm over a chunk of rows in
        one launch (bit-identical to the four separate calls)."""
        self.context.check(L.lib().tt_gdn_prefill_pre(
            self.context.handle, _stream(command_buffer), _addr(tail), _addr(qkv_rows), _addr(conv_weight),
            _addr(conv_out), _addr(checkpoint_tail) if checkpoint_tail is not None else None, self.config.num_k_heads,
            self.config.key_head_dim, self.config.qkv_dim, self.config.conv_kernel_size, rows, int(update_tail)))

    def encode_conv_prefill(self, tail, qkv_rows, conv_weight, out, rows, command_buffer=None, tail_offset=0,
                            qkv_rows_offset=0, conv_weight_offset=0, out_offset=0):
        """GDN.encodeConvPrefill: conv over [tail | chunk rows]; the tail is read-only here."""
        self.context.check(L.lib().tt_gdn_conv_mix(
            self.context.handle, _stream(command_buffer), _addr(tail, tail_offset), _addr(qkv_rows, qkv_rows_offset),
            _addr(conv_weight, conv_weight_offset), _addr(out, out_offset), self.config.qkv_dim,
            self.config.conv_kernel_size, rows, 0))

    def encode_conv_tail_update(self, tail, qkv_rows, rows, command_buffer=None, tail_offset=0, qkv_rows_offset=0):
        """GDN.encodeConvTailUpdate: tail := last (kernel-1) raw rows of [tail | chunk]."""
        self.context.check(L.lib().tt_gdn_conv_tail_update(
            self.context.handle, _stream(command_buffer), _addr(tail, tail_offset), _addr(qkv_rows, qkv_rows_offset),
            self.config.qkv_dim, self.config.conv_kernel_size, rows))

    def encode_conv_tail_checkpoint(self, tail, qkv, checkpoint, command_buffer=None, tail_offset=0, qkv_offset=0,
                                    checkpoint_offset=0):
        """GDN.encodeConvTailCheckpoint: the tail as it stands after row 0 alone."""
        self.context.check(L.lib().tt_gdn_conv_tail_checkpoint(
            self.context.handle, _stream(command_buffer), _addr(tail, tail_offset), _addr(qkv, qkv_offset),
            _addr(checkpoint, checkpoint_offset), self.config.qkv_dim, self.config.conv_kernel_size))

    def encode_qk_norm(self, conv_out, rows=1, row_stride=None, command_buffer=None, conv_out_offset=0):
        """GDN.encodeQKNorm: per-head RMS norm of the q and k slices, delta-rule scales folded in."""
        self.context.check(L.lib().tt_gdn_qk_norm(
            self.context.handle, _stream(command_buffer), _addr(conv_out, conv_out_offset), self.config.num_k_heads,
            self.config.key_head_dim, row_stride or self.config.qkv_dim, rows))

    def encode_gated_norm(self, y, z, norm_weight, out, rows=1, sigmoid_gate=False, command_buffer=None, y_offset=0,
                          z_offset=0, norm_weight_offset=0, out_offset=0):
        """GDN.encodeGatedNorm: rmsnorm(y) * weight * silu(z) (or sigmoid(z)) per value head."""
        self.context.check(L.lib().tt_gdn_gated_norm(
            self.context.handle, _stream(command_buffer), _addr(y, y_offset), _addr(z, z_offset),
            _addr(norm_weight, norm_weight_offset), _addr(out, out_offset), self.config.num_v_heads,
            self.config.value_head_dim, rows, int(sigmoid_gate)))

    def encode_delta_step_decode(self, conv_out, a_proj, b_proj, a_log, dt_bias, state, y, command_buffer=None,
                                 conv_out_offset=0, a_proj_offset=0, b_proj_offset=0, a_log_offset=0,
                                 dt_bias_offset=0, state_offset=0, y_offset=0):
        """GDN.encodeDeltaStepDecode (GDN.swift:318-347)."""
        self.encode_delta_step_prefill(conv_out, a_proj, b_proj, a_log, dt_bias, state, y, rows=1,
                                       command_buffer=command_buffer, conv_out_offset=conv_out_offset,
                                       a_proj_offset=a_proj_offset, b_proj_offset=b_proj_offset,
                                       a_log_offset=a_log_offset, dt_bias_offset=dt_bias_offset,
                                       state_offset=state_offset, y_offset=y_offset)

    def encode_delta_step_prefill(self, conv_out, a_proj, b_proj, a_log, dt_bias, state, y, rows,
                                  checkpoint_state=None, row_stride=None, command_buffer=None, conv_out_offset=0,
                                  a_proj_offset=0, b_proj_offset=0, a_log_offset=0, dt_bias_offset=0,
                                  state_offset=0, checkpoint_state_offset=0, y_offset=0):
        """GDN.encodeDeltaStepPrefill (GDN.swift:351-396): rows applied in order, exact arithmetic."""
        self.context.check(L.lib().tt_gdn_step(
            self.context.handle, _stream(command_buffer), _addr(conv_out, conv_out_offset),
            _addr(a_proj, a_proj_offset), _addr(b_proj, b_proj_offset), _addr(a_log, a_log_offset),
            _addr(dt_bias, dt_bias_offset), _addr(state, state_offset), _addr(y, y_offset), C.byref(self.shape),
            rows, row_stride or self.config.qkv_dim,
            _addr(checkpoint_state, checkpoint_state_offset) if checkpoint_state is not None else None))

    def encode_delta_step_batched(self, sessions: Sequence[GDNSession], a_log, dt_bias, rows=1, row_stride=None,
                                  command_buffer=None):
        n = len(sessions)
        arr = (L.GdnSession * max(n, 1))()
        for i, s in enumerate(sessions):
            arr[i] = L.GdnSession(_addr(s.conv_out, s.conv_out_offset), _addr(s.a_proj, s.a_proj_offset),
                                  _addr(s.b_proj, s.b_proj_offset), _addr(s.state, s.state_offset),
                                  _addr(s.y, s.y_offset),
                                  _addr(s.checkpoint_state, s.checkpoint_state_offset)
                                  if s.checkpoint_state is not None else None)
        self.context.check(L.lib().tt_gdn_step_batched(
            self.context.handle, _stream(command_buffer), arr, n, _addr(a_log), _addr(dt_bias),
            C.byref(self.shape), rows, row_stride or self.config.qkv_dim))

    def prepare_batch(self, sessions: Sequence[GDNSession]):
        n = len(sessions)
        arr = (L.GdnSession * max(n, 1))()
        for i, s in enumerate(sessions):
            arr[i] = L.GdnSession(_addr(s.conv_out, s.conv_out_offset), _addr(s.a_proj, s.a_proj_offset),
                                  _addr(s.b_proj, s.b_proj_offset), _addr(s.state, s.state_offset),
                                  _addr(s.y, s.y_offset),
                                  _addr(s.checkpoint_state, s.checkpoint_state_offset)
                                  if s.checkpoint_state is not None else None)
        return (arr, n)

    def encode_prepared(self, batch, a_log, dt_bias, rows=1, row_stride=None, command_buffer=None):
        arr, n = batch
        self.context.check(L.lib().tt_gdn_step_batched(
            self.context.handle, _stream(command_buffer), arr, n, _addr(a_log), _addr(dt_bias),
            C.byref(self.shape), rows, row_stride or self.config.qkv_dim))

    def encode_delta_scan_chunked(self, conv_out, a_proj, b_proj, a_log, dt_bias, state, y, rows, chunk=64,
                                  row_stride=None, command_buffer=None, state_offset=0):
        """Chunk-parallel form of encode_delta_step_prefill (tt_gdn_scan_chunked)."""
        self.context.check(L.lib().tt_gdn_scan_chunked(
            self.context.handle, _stream(command_buffer), _addr(conv_out), _addr(a_proj), _addr(b_proj),
            _addr(a_log), _addr(dt_bias), _addr(state, state_offset), _addr(y), C.byref(self.shape), rows,
            row_stride or self.config.qkv_dim, chunk))
