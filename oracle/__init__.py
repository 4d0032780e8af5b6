"""CPU oracle for the attention + Gated-DeltaNet path (TEST INFRASTRUCTURE ONLY).

ctypes/numpy front end of ``oracle/tt_oracle.c`` (own restatement) and, when
it has been built, of ``oracle/_ref/libtinytitan_ref.so`` (the reference's two
delta-rule C kernels compiled unmodified from their sources). Only the test
suite, the smoke check and the bench's CPU-baseline leg may import this
package; the product library never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_f32p = C.POINTER(C.c_float)
_u8p = C.POINTER(C.c_uint8)


def build(quiet: bool = True) -> None:
    """Compile liboracle.so (and _ref when the reference tree is present)."""
    subprocess.run(["make", "-C", _HERE], check=True,
                   stdout=subprocess.DEVNULL if quiet else None)


def _load(path: str):
    return C.CDLL(path) if os.path.exists(path) else None


_lib = None
_ref = None


def lib():
    global _lib
    if _lib is None:
        so = os.path.join(_HERE, "liboracle.so")
        if not os.path.exists(so):
            build()
        _lib = C.CDLL(so)
        _lib.tt_oracle_max_threads.restype = C.c_int
        _lib.tt_oracle_delta_rule_chunk.restype = C.c_int
        _lib.tt_oracle_gdn_scan_heads.restype = C.c_int
        _lib.tt_oracle_cpu_engine_attention_batch.restype = C.c_int
        _lib.tt_oracle_cpu_engine_attention_head.restype = C.c_int
    return _lib


def ref():
    """The compiled reference kernels, or None when oracle/_ref was not built."""
    global _ref
    if _ref is None:
        _ref = _load(os.path.join(_HERE, "_ref", "libtinytitan_ref.so"))
        if _ref is not None:
            _ref.tinytitan_delta_rule_chunk.restype = C.c_int
    return _ref


def max_threads() -> int:
    return int(lib().tt_oracle_max_threads())


def _f(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _p(a: np.ndarray):
    return a.ctypes.data_as(_f32p)


# --------------------------------------------------------------------------
# attention
# --------------------------------------------------------------------------
def attn_decode(q, k, v, n_kv_heads: int, scale: float, window: int = -1) -> np.ndarray:
    """q [Hq,hd], k/v [S,Hkv,hd] -> [Hq,hd] (materialised-softmax reference)."""
    q, k, v = _f(q), _f(k), _f(v)
    hq, hd = q.shape
    s = k.shape[0]
    out = np.empty((hq, hd), np.float32)
    lib().tt_oracle_attn_decode(_p(q), _p(k), _p(v), hd, hq, n_kv_heads, s, window,
                                C.c_float(scale), _p(out))
    return out


def attn_decode_split(q, k, v, n_kv_heads: int, scale: float, seq_len: int, kv_start: int = 0,
                      keep=None, ring_capacity: int = 0, n_chunks: int = 16,
                      kv_stride: int | None = None) -> np.ndarray:
    """Split-KV partial + combine form; k/v are [rows, kv_stride] fp32."""
    q = _f(q)
    hq, hd = q.shape
    k = _f(k).reshape(k.shape[0], -1)
    v = _f(v).reshape(v.shape[0], -1)
    stride = kv_stride or k.shape[1]
    out = np.empty((hq, hd), np.float32)
    kp = None
    if keep is not None:
        keep = np.ascontiguousarray(keep, dtype=np.uint8)
        kp = keep.ctypes.data_as(_u8p)
    lib().tt_oracle_attn_decode_split(_p(q), _p(k), _p(v), hd, hq, n_kv_heads, C.c_size_t(stride),
                                      seq_len, kv_start, C.c_float(scale), kp, ring_capacity,
                                      n_chunks, _p(out))
    return out


def attn_partial(q_row, k, v, n_kv_heads: int, kv_head: int, p_start: int, p_end: int,
                 scale: float, keep=None, ring_capacity: int = 0):
    q_row = _f(q_row)
    hd = q_row.shape[0]
    k = _f(k).reshape(k.shape[0], -1)
    v = _f(v).reshape(v.shape[0], -1)
    m = C.c_float()
    d = C.c_float()
    o = np.empty(hd, np.float32)
    kp = None
    if keep is not None:
        keep = np.ascontiguousarray(keep, dtype=np.uint8)
        kp = keep.ctypes.data_as(_u8p)
    lib().tt_oracle_attn_partial(_p(q_row), _p(k), _p(v), hd, n_kv_heads, kv_head,
                                 C.c_size_t(k.shape[1]), p_start, p_end, C.c_float(scale), kp,
                                 ring_capacity, C.byref(m), C.byref(d), _p(o))
    return m.value, d.value, o


def attn_combine(m, d, o) -> np.ndarray:
    m, d, o = _f(m), _f(d), _f(o)
    n, hd = o.shape
    out = np.empty(hd, np.float32)
    lib().tt_oracle_attn_combine(_p(m), _p(d), _p(o), n, hd, _p(out))
    return out


def attn_prefill(q, k, v, q_stride: int, kv_stride: int, head_dim: int, q_heads: int,
                 kv_heads: int, start: int, chunk: int, kv_valid: int, window: int,
                 scale: float, threads: int = 0) -> np.ndarray:
    """Strided causal prefill reference; q/k/v are flat fp32 buffers; out [T,Hq,hd]."""
    q, k, v = _f(q).ravel(), _f(k).ravel(), _f(v).ravel()
    out = np.empty((chunk, q_heads, head_dim), np.float32)
    lib().tt_oracle_attn_prefill(_p(q), _p(k), _p(v), C.c_size_t(q_stride), C.c_size_t(kv_stride),
                                 head_dim, q_heads, kv_heads, start, chunk, kv_valid, window,
                                 C.c_float(scale), threads or max_threads(), _p(out))
    return out


def cpu_engine_attention(query, keys, values, kv_heads: int, scale: float, threads: int = 1):
    """The reference CPU engine's decode attention: query [H,dim], keys/values [S,Hkv*dim]."""
    query, keys, values = _f(query), _f(keys), _f(values)
    heads, dim = query.shape
    cached = keys.shape[0]
    out = np.empty((heads, dim), np.float32)
    lib().tt_oracle_cpu_engine_attention(_p(query), _p(keys), _p(values), heads, kv_heads, dim,
                                         cached, C.c_float(scale), threads, _p(out))
    return out


def cpu_engine_attention_sessions(query, keys, values, cached, row_base, kv_heads: int,
                                  scale: float, threads: int):
    """query [N,H,dim]; keys/values one shared fp32 store [rows, Hkv*dim]."""
    query, keys, values = _f(query), _f(keys), _f(values)
    n, heads, dim = query.shape
    cached = np.ascontiguousarray(cached, dtype=np.int32)
    row_base = np.ascontiguousarray(row_base, dtype=np.int64)
    out = np.empty((n, heads, dim), np.float32)
    lib().tt_oracle_cpu_engine_attention_sessions(
        _p(query), _p(keys), _p(values), cached.ctypes.data_as(C.POINTER(C.c_int)),
        row_base.ctypes.data_as(C.POINTER(C.c_longlong)), n, heads, kv_heads, dim,
        C.c_float(scale), threads, _p(out))
    return out


def cpu_engine_attention_batch(query, keys, values, kv_heads: int, base_position: int,
                               scale: float, threads: int = 0):
    """Batched prefill attention of the CPU engine. query [T,H,dim]; keys/values [P,Hkv*dim]."""
    query, keys, values = _f(query), _f(keys), _f(values)
    t, heads, dim = query.shape
    positions = keys.shape[0]
    out = np.empty((t, heads, dim), np.float32)
    rc = lib().tt_oracle_cpu_engine_attention_batch(
        _p(query), t, heads, dim, _p(keys), _p(values), positions, kv_heads, base_position,
        C.c_float(scale), threads or max_threads(), _p(out))
    if rc:
        raise RuntimeError(f"attention mask limit past the cache (rc={rc})")
    return out


# --------------------------------------------------------------------------
# gated delta rule
# --------------------------------------------------------------------------
def _delta_rule_call(fn, query, key, value, a, b, decay_log, decay_bias, key_heads, inverse, state):
    query, key, value = _f(query).ravel(), _f(key).ravel(), _f(value)
    heads, dv = value.shape
    dk = key.size // key_heads
    a, b, decay_log, decay_bias = _f(a), _f(b), _f(decay_log), _f(decay_bias)
    state = np.array(state, dtype=np.float32, copy=True).reshape(heads, dv, dk)
    readout = np.empty((heads, dv), np.float32)
    fn(_p(query), _p(key), _p(value), _p(a), _p(b), _p(decay_log), _p(decay_bias),
       C.c_size_t(heads), C.c_size_t(key_heads), C.c_size_t(dk), C.c_size_t(dv),
       C.c_float(inverse), _p(state), _p(readout))
    return readout, state


def delta_rule(query, key, value, a, b, decay_log, decay_bias, key_heads, inverse, state):
    """Own restatement of the CPU one-token rule. Returns (readout [H,dv], new state)."""
    return _delta_rule_call(lib().tt_oracle_delta_rule, query, key, value, a, b, decay_log,
                            decay_bias, key_heads, inverse, state)


def ref_delta_rule(query, key, value, a, b, decay_log, decay_bias, key_heads, inverse, state):
    """The compiled reference kernel tinytitan_delta_rule."""
    return _delta_rule_call(ref().tinytitan_delta_rule, query, key, value, a, b, decay_log,
                            decay_bias, key_heads, inverse, state)


def _chunk_call(fn, queries, keys, values, alphas, betas, state):
    queries, keys, values = _f(queries), _f(keys), _f(values)
    alphas, betas = _f(alphas), _f(betas)
    t, dk = keys.shape
    dv = values.shape[1]
    state = np.array(state, dtype=np.float32, copy=True).reshape(dv, dk)
    ro = np.empty((t, dv), np.float32)
    rc = fn(_p(queries), C.c_size_t(dk), _p(keys), C.c_size_t(dk), _p(values), C.c_size_t(dv),
            _p(alphas), C.c_size_t(1), _p(betas), C.c_size_t(1), C.c_size_t(t), C.c_size_t(dk),
            C.c_size_t(dv), _p(state), _p(ro), C.c_size_t(dv))
    if rc:
        raise MemoryError("chunk kernel scratch allocation failed")
    return ro, state


def delta_rule_chunk(queries, keys, values, alphas, betas, state):
    """Own restatement of the chunked rule, one head. Returns (readouts [T,dv], state)."""
    return _chunk_call(lib().tt_oracle_delta_rule_chunk, queries, keys, values, alphas, betas, state)


def ref_delta_rule_chunk(queries, keys, values, alphas, betas, state):
    return _chunk_call(ref().tinytitan_delta_rule_chunk, queries, keys, values, alphas, betas, state)


def gdn_step_rows(conv_out, a, b, a_log, dt_bias, hk, hv, dk, dv, state, a_preexp=False,
                  v_tiled=False, readout_scale=1.0, want_checkpoint=False):
    """GPU-kernel form of the rule over rows sequentially (all-fp32 arithmetic).

    conv_out [rows, C] with C >= 2*hk*dk + hv*dv; a/b [rows, hv]. Returns
    (y [rows, hv*dv], state', checkpoint or None)."""
    conv_out = _f(conv_out)
    rows, stride = conv_out.shape
    a, b, a_log, dt_bias = _f(a).reshape(rows, hv), _f(b).reshape(rows, hv), _f(a_log), _f(dt_bias)
    state = np.array(state, dtype=np.float32, copy=True).reshape(hv, dv, dk)
    ck = np.empty_like(state) if want_checkpoint else None
    y = np.empty((rows, hv * dv), np.float32)
    lib().tt_oracle_gdn_step_rows(_p(conv_out), C.c_size_t(stride), _p(a), _p(b), _p(a_log),
                                  _p(dt_bias), hk, hv, dk, dv, rows, int(a_preexp), int(v_tiled),
                                  C.c_float(readout_scale), _p(state),
                                  _p(ck) if ck is not None else None, _p(y))
    return y, state, ck


def gdn_scan_heads(q, k, v, alpha, beta, hk, hv, dk, dv, chunk, state, threads=0, use_ref=False):
    """Chunked scan over all heads. q/k [T,hk*dk], v [T,hv*dv], alpha/beta [T,hv]."""
    q, k, v, alpha, beta = _f(q), _f(k), _f(v), _f(alpha), _f(beta)
    t = q.shape[0]
    state = np.array(state, dtype=np.float32, copy=True).reshape(hv, dv, dk)
    y = np.empty((t, hv * dv), np.float32)
    fn = None
    if use_ref:
        fn = C.cast(ref().tinytitan_delta_rule_chunk, C.c_void_p)
    rc = lib().tt_oracle_gdn_scan_heads(fn, _p(q), _p(k), _p(v), _p(alpha), _p(beta), t, hk, hv,
                                        dk, dv, chunk, threads or max_threads(), _p(state), _p(y))
    if rc:
        raise MemoryError("chunk kernel scratch allocation failed")
    return y, state


def delta_rule_sessions(query, key, value, a, b, decay_log, decay_bias, key_heads, inverse, state,
                        threads=0, use_ref=False):
    """One-token CPU rule over N sessions. query/key [N,Hk*dk], value [N,H,dv], a/b [N,H]."""
    query, key, value, a, b = _f(query), _f(key), _f(value), _f(a), _f(b)
    decay_log, decay_bias = _f(decay_log), _f(decay_bias)
    n, heads, dv = value.shape
    dk = key.shape[1] // key_heads
    state = np.array(state, dtype=np.float32, copy=True).reshape(n, heads, dv, dk)
    ro = np.empty((n, heads, dv), np.float32)
    fn = None
    if use_ref:
        fn = C.cast(ref().tinytitan_delta_rule_range, C.c_void_p)
    lib().tt_oracle_delta_rule_sessions(fn, _p(query), _p(key), _p(value), _p(a), _p(b),
                                        _p(decay_log), _p(decay_bias), n, heads, key_heads, dk, dv,
                                        C.c_float(inverse), threads or max_threads(), _p(state),
                                        _p(ro))
    return ro, state


# --------------------------------------------------------------------------
# the whole Gated-DeltaNet chain of one layer, token by token (numpy, fp32 with the GPU path's
# fp16 rounding points). Follows sources/TinyTitanValidation/Support/Reference/GDN/
# GDNReference.swift:45-123: conv + SiLU (rounded to fp16, :55-64), tail shift (:65-66), q/k RMS
# norm with folded scales 1/Dk and 1/sqrt(Dk) (rounded, :68-81), delta rule (y rounded, :84-107),
# gated output norm rmsnorm(y) * w * silu(z) (:109-121).
# --------------------------------------------------------------------------
class GDNChainReference:
    def __init__(self, hk, hv, dk, dv, taps, conv_w, a_log, dt_bias, norm_w, fp16_points=True):
        """fp16_points=False keeps every intermediate in fp32 (the all-fp32 model the reference's
        numpy implementation tools/qwen35_reference.py:231-290 computes)."""
        self.hk, self.hv, self.dk, self.dv, self.taps = hk, hv, dk, dv, taps
        if not fp16_points:
            self._h = lambda x: np.asarray(x, np.float32)
        self.c = 2 * hk * dk + hv * dv
        self.conv_w = _f(conv_w).reshape(self.c, taps)
        self.a_log, self.dt_bias, self.norm_w = _f(a_log), _f(dt_bias), _f(norm_w)
        self.tail = np.zeros((taps - 1, self.c), np.float32)
        self.state = np.zeros((hv, dv, dk), np.float32)

    @staticmethod
    def _h(x):
        return np.asarray(x, np.float32).astype(np.float16).astype(np.float32)

    def conv(self, qkv_raw):
        x = _f(qkv_raw)
        acc = x * self.conv_w[:, self.taps - 1]
        for j in range(self.taps - 1):
            acc = acc + self.tail[j] * self.conv_w[:, j]
        acc = acc.astype(np.float32)
        out = self._h(acc / (1 + np.exp(-acc)))
        self.tail = np.concatenate([self.tail[1:], self._h(x)[None]], 0)
        return out

    def qk_norm(self, conv):
        n = conv.copy()
        for hi in range(2 * self.hk):
            is_q = hi < self.hk
            head = hi if is_q else hi - self.hk
            base = (0 if is_q else self.hk * self.dk) + head * self.dk
            sl = conv[base:base + self.dk]
            inv = np.float32(1) / np.sqrt(np.float32((sl * sl).sum(dtype=np.float32) / self.dk + 1e-6))
            scale = np.float32(1 / self.dk) if is_q else np.float32(1 / np.sqrt(self.dk))
            n[base:base + self.dk] = self._h(sl * inv * scale)
        return n

    def gated_norm(self, y, z, sigmoid_gate=False):
        y, z = _f(y).reshape(self.hv, self.dv), _f(z).reshape(self.hv, self.dv)
        inv = 1 / np.sqrt((y * y).sum(-1, keepdims=True, dtype=np.float32) / self.dv + 1e-6)
        gate = 1 / (1 + np.exp(-z)) if sigmoid_gate else z / (1 + np.exp(-z))
        return (y * inv * self.norm_w[None] * gate).astype(np.float32).reshape(-1)

    def step(self, qkv_raw, a, b, z):
        normed = self.qk_norm(self.conv(qkv_raw))
        y, self.state, _ = gdn_step_rows(normed[None], _f(a)[None], _f(b)[None], self.a_log, self.dt_bias,
                                         self.hk, self.hv, self.dk, self.dv, self.state)
        y = self._h(y[0])
        return self.gated_norm(y, z), y, normed


# --------------------------------------------------------------------------
# the elementwise step either side of decode attention (numpy, fp32 with the GPU path's fp16
# rounding points). Follows Primitives/rmsnorm.metal:101-128 (per-head RMS norm, bf16 weight, fp16
# store), Primitives/rope.metal:32-49, :80-108 (NeoX rotation of the first `rotary` elements, fp16
# store) and Primitives/utility.metal:142-160 (out * sigmoid(gate)); the call order is
# RealForwardRunner+DecodeFullAttention.swift:123-185.
# --------------------------------------------------------------------------
def _half(x):
    return np.asarray(x, np.float32).astype(np.float16).astype(np.float32)


def attn_norm_rope(x, weight, eps: float, rotary: int, theta: float, position: int, fp16_points: bool = True):
    """One head: RMS norm with `weight`, then NeoX rotation of x[:rotary] at `position`."""
    h = _half if fp16_points else (lambda a: np.asarray(a, np.float32))
    x = np.asarray(x, np.float32)
    inv = np.float32(1) / np.sqrt(np.float32((x * x).sum(dtype=np.float32) / x.size + eps))
    y = h(x * inv * np.asarray(weight, np.float32))
    half = rotary // 2
    pair = np.arange(half, dtype=np.float32)
    angle = np.float32(position) * np.power(np.float32(theta), -(2 * pair) / np.float32(rotary)).astype(np.float32)
    c, s = np.cos(angle).astype(np.float32), np.sin(angle).astype(np.float32)
    out = y.copy()
    out[:half] = h(y[:half] * c - y[half:rotary] * s)
    out[half:rotary] = h(y[:half] * s + y[half:rotary] * c)
    return out


def attn_gate_mul(out, gate, fp16_points: bool = True):
    """Sigmoid output gate: out * 1/(1+exp(-gate))."""
    h = _half if fp16_points else (lambda a: np.asarray(a, np.float32))
    out, gate = np.asarray(out, np.float32), np.asarray(gate, np.float32)
    return h(out / (np.float32(1) + np.exp(-gate)))


# --------------------------------------------------------------------------
# affine KV quantisation (numpy). Follows
# sources/TinyTitanCore/Metal/Quant/kv_cache_quantize.metal:4-72 (bias = group min, scale =
# (max-min)/levels in fp32, code = round-half-away(clamp((x-bias)/scale)), fp16 scale/bias stored
# after the packed codes) and the loader attn_load_kv (attention.metal:89-117).
# --------------------------------------------------------------------------
def kv_quantize_rows(rows, bits: int, group_size: int = 64):
    """rows fp32 [tokens, elements] (fp16-representable). Returns (packed uint8 rows, dequantised fp32)."""
    x = _f(rows)
    tokens, n = x.shape
    groups = (n + group_size - 1) // group_size
    packed_bytes = (n * bits + 7) // 8
    value_bytes = (packed_bytes + 1) & ~1
    stride = value_bytes + groups * 4
    levels = np.float32(15 if bits == 4 else 255)
    out = np.zeros((tokens, stride), np.uint8)
    deq = np.zeros_like(x)
    for g in range(groups):
        sl = x[:, g * group_size:(g + 1) * group_size]
        mn, mx = sl.min(1, keepdims=True), sl.max(1, keepdims=True)
        scale = np.where(mx > mn, (mx - mn) / levels, np.float32(0)).astype(np.float32)
        safe = np.where(scale > 0, scale, np.float32(1))
        q = np.where(scale > 0, np.floor(np.clip((sl - mn) / safe, 0, levels).astype(np.float32) + np.float32(0.5)), 0)
        q = q.astype(np.uint8)
        s16, b16 = scale.astype(np.float16), mn.astype(np.float16)
        out[:, value_bytes + 2 * g:value_bytes + 2 * g + 2] = s16.view(np.uint8).reshape(tokens, 2)
        out[:, value_bytes + 2 * (groups + g):value_bytes + 2 * (groups + g) + 2] = b16.view(np.uint8).reshape(tokens, 2)
        deq[:, g * group_size:(g + 1) * group_size] = q.astype(np.float32) * s16.astype(np.float32) + b16.astype(np.float32)
        cols = np.arange(g * group_size, min(n, (g + 1) * group_size))
        if bits == 8:
            out[:, cols] = q
        else:
            lo, hi = q[:, 0::2], q[:, 1::2]
            byte = lo.copy()
            byte[:, :hi.shape[1]] |= (hi << 4)
            out[:, cols[0] // 2:cols[0] // 2 + byte.shape[1]] = byte
    return out, deq, stride, value_bytes


# --------------------------------------------------------------------------
# Qwen Sparse Attention's block indexer (numpy). Follows
# sources/TinyTitanCore/Metal/Attention/qsa.metal:14-126 (pool: mean of the raw members present,
# stored fp16; scores: sum over heads of max(0, q.pooled)), the norm and rotation the host encodes
# after pooling (QSAIndexer.swift:196-238: rmsnorm_bf16w_perhead then rope_neox_subdim_strided with
# rotary = head_dim at position block * ratio) and the selection rule of
# QSAIndexer+Scratch.swift:211-251 (selectKeys) / QSAIndexer.swift:391-498 (selectKeysPrefill).
# --------------------------------------------------------------------------
def qsa_pool_blocks(raw, ratio: int, n_kv: int, first_block: int, block_count: int, weight=None,
                    eps: float = 1e-6, theta: float = 1e7):
    """raw fp32 [cells, D] (fp16-representable). Returns {block: pooled row} for the blocks that exist."""
    raw = _f(raw)
    out = {}
    for block in range(first_block, first_block + block_count):
        first = block * ratio
        if first >= n_kv:
            continue
        count = min(ratio, n_kv - first)
        acc = np.zeros(raw.shape[1], np.float32)
        for m in range(count):
            acc = acc + raw[first + m]
        row = _half(acc / np.float32(count))
        if weight is not None:
            row = attn_norm_rope(row, weight, eps, raw.shape[1], theta, block * ratio)
        out[block] = row
    return out


def qsa_block_scores(query, pooled):
    """query [T, H, D], pooled [B, D] -> scores [T, B] = sum_h max(0, q[t,h] . pooled[b])."""
    q, p = _f(query), _f(pooled)
    dots = np.einsum("thd,bd->thb", q.astype(np.float64), p.astype(np.float64))
    return np.maximum(dots, 0.0).sum(axis=1).astype(np.float32)


def qsa_select_keys(scores, visible: int, ratio: int, width: int):
    """One query's selection. Returns (keep uint8 [visible], ascending kept indices capped at `width`)."""
    keep = np.zeros(visible, np.uint8)
    if visible <= width:
        keep[:] = 1
        return keep, np.arange(visible, dtype=np.uint32)
    complete = (visible // ratio) * ratio
    keep[complete:] = 1                                   # the query's own ragged tail
    remaining = width - (visible - complete)
    if remaining > 0:
        blocks = complete // ratio
        s = np.asarray(scores, np.float32)[:blocks] + np.float32(0)   # -0.0 ties +0.0
        ranked = sorted(range(blocks), key=lambda b: (-float(s[b]), b))
        for block in ranked:
            if remaining <= 0:
                break
            take = min(ratio, remaining)
            keep[block * ratio:block * ratio + take] = 1
            remaining -= take
    return keep, np.nonzero(keep)[0].astype(np.uint32)[:width]


def attn_prefill_selected(q, k, v, head_dim, q_heads, kv_heads, start, kv_valid, window, scale, keys_of_row,
                          rows_of_row=None):
    """Causal prefill where query row t attends only the logical keys keys_of_row[t] that fall in its
    visible range; rows_of_row[t][i] (optional) is the cache row holding keys_of_row[t][i]
    (attention_prefill_causal_qsa_tiled, prefill.metal:914-1054). q [T, Hq*hd], k/v [rows, Hkv*hd]."""
    q, k, v = _f(q), _f(k), _f(v)
    t_count = q.shape[0]
    out = np.zeros((t_count, q_heads, head_dim), np.float32)
    for t in range(t_count):
        abs_q = start + t
        first = abs_q + 1 - window if (window != 0 and abs_q + 1 > window) else 0
        last = min(kv_valid, abs_q + 1)
        keys = np.asarray(keys_of_row[t], np.int64)
        phys = keys if rows_of_row is None else np.asarray(rows_of_row[t], np.int64)
        ok = (keys >= first) & (keys < last)
        if not ok.any():
            continue
        kk = k[phys[ok]].reshape(-1, kv_heads, head_dim)
        vv = v[phys[ok]].reshape(-1, kv_heads, head_dim)
        out[t] = attn_decode(q[t].reshape(q_heads, head_dim), kk, vv, kv_heads, scale)
    return out
