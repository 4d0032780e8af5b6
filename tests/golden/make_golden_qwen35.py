#!/usr/bin/env python3
"""Generates tests/golden/qwen35_*.npz by RUNNING the reference's own numpy model.

`tools/qwen35_reference.py` of the reference tree holds `Reference.attention` (q/gate split,
per-head RMS norm, partial NeoX RoPE, GQA softmax against the growing KV list, sigmoid output
gate; `:292-322`, RoPE `:213-229`) and `Reference.gdn` (causal conv + SiLU, L2 norm, gated delta
rule, gated RMS norm; `:231-290`). Both read weights only through `self.w.get(name)`. This script
imports that file unmodified, builds a `Reference` without its checkpoint loader and hands it a
weight table of seeded synthetic tensors whose projections are 0/1 selection matrices, so that
the layer input `x` IS `[query;gate | k | v]` (or `[qkv | z | a | b]`) and the layer output is the
gated attention / gated-norm row itself. Everything between those two points is the reference's
code, executed here.

    python tests/golden/make_golden_qwen35.py --ref /path/to/TinyTitan
    (or TINYTITAN_REF=/path/to/TinyTitan)

Only the reference's OUTPUTS are stored; the tests regenerate the inputs from the same seeds with
the `*_inputs` functions below.

  qwen35_attention.npz  per case: out [T, H*hd] (gated attention rows), keys [T, Hkv, hd] (the
                        normed + rotated K rows the reference appended to its cache)
  qwen35_gdn.npz        out [T, Hv*dv], state checksums + a few state rows, the conv tail
"""
from __future__ import annotations

import argparse
import importlib.util
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))

EPS = 1e-6
ROPE_THETA = 10_000_000.0
ROTARY = 64

# name -> (q heads, kv heads, head_dim, rows already in the cache, positions decoded)
ATTENTION_CASES = {
    "h8_kv2_d256_from0": (8, 2, 256, 0, 64),          # Qwen3.5-2B geometry, from an empty cache
    "h16_kv2_d256_from1000": (16, 2, 256, 1000, 64),  # Qwen3.6-35B-A3B geometry, 1000 cached rows
}
GDN_CASE = dict(hk=16, hv=32, dk=128, dv=128, conv_k=4, tokens=12)


def _f16(x):
    return np.asarray(x, np.float32).astype(np.float16).astype(np.float32)


def _bf16(x):
    """Round to nearest-even bf16, returned widened to fp32."""
    u = np.asarray(x, np.float32).view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) >> 16 << 16
    return u.astype(np.uint32).view(np.float32)


def attention_inputs(name: str) -> dict:
    """Seeded inputs of one attention case; every value is exactly representable in the dtype the
    GPU path stores it in (fp16 activations and cache rows, bf16 norm weights)."""
    hq, hkv, hd, cached, steps = ATTENTION_CASES[name]
    r = np.random.default_rng([0x51A5, hq, hkv, hd, cached])
    return dict(
        hq=hq, hkv=hkv, hd=hd, cached=cached, steps=steps,
        packed=_f16(r.normal(size=(steps, hq, 2 * hd))),      # per head [query ; gate], as q_proj emits it
        k=_f16(r.normal(size=(steps, hkv, hd))),              # k_proj rows (before norm and RoPE)
        v=_f16(r.normal(size=(steps, hkv, hd))),
        q_norm=_bf16(r.uniform(0.5, 1.5, size=hd)), k_norm=_bf16(r.uniform(0.5, 1.5, size=hd)),
        cache_k=_f16(r.normal(size=(cached, hkv, hd))),       # rows already in the cache (stored as they are)
        cache_v=_f16(r.normal(size=(cached, hkv, hd))),
    )


def gdn_inputs() -> dict:
    c = dict(GDN_CASE)
    hk, hv, dk, dv, taps, t = c["hk"], c["hv"], c["dk"], c["dv"], c["conv_k"], c["tokens"]
    conv_dim = 2 * hk * dk + hv * dv
    r = np.random.default_rng([0x6D17, hk, hv, dk])
    c.update(
        qkv=_f16(r.normal(size=(t, conv_dim))), z=_f16(r.normal(size=(t, hv * dv))),
        a=_f16(r.normal(size=(t, hv))), b=_f16(r.normal(size=(t, hv))),
        conv_w=_bf16(r.uniform(-0.4, 0.4, size=(conv_dim, taps))),
        a_log=_bf16(r.uniform(-1.0, 1.5, size=hv)), dt_bias=_bf16(r.uniform(-0.5, 0.5, size=hv)),
        norm_w=_bf16(r.uniform(0.5, 1.5, size=dv)),
    )
    return c


class _Table:
    """Stands in for the reference's `Weights`: `.get(name)` by suffix."""

    def __init__(self, entries: dict):
        self.entries = entries

    def get(self, name: str):
        for suffix, value in self.entries.items():
            if name.endswith(suffix):
                return value
        raise KeyError(name)


def _select(rows: int, cols: int, first_col: int):
    """0/1 matrix that copies x[first_col : first_col + rows]; sparse, so the product is exact."""
    from scipy.sparse import csr_matrix
    idx = np.arange(rows)
    return csr_matrix((np.ones(rows, np.float32), (idx, first_col + idx)), shape=(rows, cols))


def load_reference_module(ref_root: str):
    path = os.path.join(ref_root, "tools", "qwen35_reference.py")
    spec = importlib.util.spec_from_file_location("qwen35_reference", path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules["qwen35_reference"] = mod
    spec.loader.exec_module(mod)
    return mod


def _bare_reference(mod, **fields):
    ref = object.__new__(mod.Reference)      # skip __init__: it opens a checkpoint directory
    ref.eps, ref.rope_theta, ref.rotary = EPS, ROPE_THETA, ROTARY
    for key, value in fields.items():
        setattr(ref, key, value)
    ref.reset()
    return ref


def run_attention(mod, name: str) -> dict:
    c = attention_inputs(name)
    hq, hkv, hd = c["hq"], c["hkv"], c["hd"]
    nq, nkv = hq * 2 * hd, hkv * hd
    hidden = nq + 2 * nkv
    ref = _bare_reference(mod, heads=hq, kv_heads=hkv, head_dim=hd, w=_Table({
        "q_proj.weight": _select(nq, hidden, 0), "k_proj.weight": _select(nkv, hidden, nq),
        "v_proj.weight": _select(nkv, hidden, nq + nkv), "o_proj.weight": _select(hq * hd, hq * hd, 0),
        "q_norm.weight": c["q_norm"], "k_norm.weight": c["k_norm"]}))
    if c["cached"]:
        ref.kv[0] = (c["cache_k"].copy(), c["cache_v"].copy())
    ref.position = c["cached"]
    out = np.empty((c["steps"], hq * hd), np.float32)
    for t in range(c["steps"]):
        x = np.concatenate([c["packed"][t].ravel(), c["k"][t].ravel(), c["v"][t].ravel()]).astype(np.float32)
        out[t] = ref.attention(0, x)
        ref.position += 1
    keys = np.asarray(ref.kv[0][0][c["cached"]:], np.float32)
    return {f"{name}.out": out, f"{name}.keys": keys}


def run_gdn(mod) -> dict:
    c = gdn_inputs()
    hk, hv, dk, dv, taps = c["hk"], c["hv"], c["dk"], c["dv"], c["conv_k"]
    conv_dim, zdim = 2 * hk * dk + hv * dv, hv * dv
    hidden = conv_dim + zdim + 2 * hv
    ref = _bare_reference(mod, hk=hk, hv=hv, dk=dk, dv=dv, conv_k=taps, w=_Table({
        "in_proj_qkv.weight": _select(conv_dim, hidden, 0), "in_proj_z.weight": _select(zdim, hidden, conv_dim),
        "in_proj_a.weight": _select(hv, hidden, conv_dim + zdim), "in_proj_b.weight": _select(hv, hidden, conv_dim + zdim + hv),
        "conv1d.weight": c["conv_w"].reshape(conv_dim, 1, taps), "A_log": c["a_log"], "dt_bias": c["dt_bias"],
        "norm.weight": c["norm_w"], "out_proj.weight": _select(zdim, zdim, 0)}))
    out = np.empty((c["tokens"], zdim), np.float32)
    for t in range(c["tokens"]):
        x = np.concatenate([c["qkv"][t], c["z"][t], c["a"][t], c["b"][t]]).astype(np.float32)
        out[t] = ref.gdn(0, x)
    state = np.asarray(ref.gdn_state[0], np.float64)
    return {"out": out, "state_sum": np.array([state.sum(), np.abs(state).sum()]),
            "state_rows": np.asarray(ref.gdn_state[0][::8, ::32, :], np.float32),     # heads 0,8,16,24; rows 0,32,64,96
            "tail": np.asarray(ref.gdn_conv[0], np.float32)}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("TINYTITAN_REF"),
                    help="root of the TinyTitan source tree (or set TINYTITAN_REF)")
    args = ap.parse_args()
    if not args.ref:
        ap.error("pass --ref or set TINYTITAN_REF")
    mod = load_reference_module(args.ref)
    out = {}
    for name in ATTENTION_CASES:
        out.update(run_attention(mod, name))
    np.savez_compressed(os.path.join(HERE, "qwen35_attention.npz"), **out)
    np.savez_compressed(os.path.join(HERE, "qwen35_gdn.npz"), **run_gdn(mod))
    print("wrote qwen35_attention.npz, qwen35_gdn.npz")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
