#!/usr/bin/env python3
"""Benchmark of the attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl tinytitan|reference]

Workload (config.workload "C2"): Qwen3.6-35B-A3B-shaped batched decode. Every rank owns 32
independent sessions with context lengths drawn uniformly from [1024, 32768] (fixed seed):
one full-attention SDPA decode step (16 q heads, 2 KV heads, head_dim 256, fp16 KV cache in
the reference's slot layout) and one Gated-DeltaNet decode step (16 k heads, 32 v heads,
d 128, fp32 state) per session per step. Ranks share nothing (weak scaling, no collective).

  value   tokens/s with every input already resident in HBM, CUDA-event timed, max over ranks
  e2e     the same step driven from pinned HOST buffers through the C-ABI operators: the
          step's inputs (q rows, the new K/V row of every session, the GDN conv/a/b rows)
          are copied host->device, the outputs (attention rows, GDN y) device->host, inside
          the timed region. The KV cache and the GDN state are the managers' persistent device
          state (as in the reference), not per-step inputs.
  roofline   the split-KV pass-1 kernel against the measured HBM copy bandwidth
  cpu_baseline / --impl reference   the reference's CPU path on the host cores (bounded sample)

Timing: the `--steps`-long loop is one batch (barrier + synchronize on both sides, CUDA events, max
over ranks); batches are repeated until at least half a second has been timed, `ms_per_step` is the
MEDIAN batch divided by the steps, the spread of the batches is reported next to it, and the clocks
are sampled while the batches run.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np

HQ, HKV, HD = 16, 2, 256
GK, GV, GD = 16, 32, 128
N_SESSIONS = 32
SCALE = 0.0625
METRIC = "decode_attention_tok_per_s"
UNIT = "tok/s"


def session_lengths(rank: int):
    """The same drawn lengths on every rank: per-GPU work is fixed as N grows (weak scaling)."""
    rng = np.random.default_rng(20261125)
    return [int(x) for x in rng.integers(1024, 32769, size=32)][:N_SESSIONS]


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def config_dict(world, lens):
    """The workload description both arms print (same string for the GPU and the CPU arm)."""
    alg = algorithmic_bytes(lens)
    return {"workload": "C2: Qwen3.6-35B-A3B-shaped batched decode, 32 sessions per GPU, S~U[1024,32768] "
                        "(seeded), SDPA 16/2/256 fp16 KV + GDN step 16/32/128 fp32 state, one layer of each per step",
            "sessions_per_gpu": len(lens), "sum_context": sum(lens),
            "l2": "inputs larger than L2: %.2f GB of KV + 0.13 GB of GDN state streamed per step" % (alg / 1e9),
            "parallelism": f"sessions x{world} (no collective)"}


def algorithmic_bytes(lens):
    """Decode SDPA bytes per step: K and V rows once per KV head, plus q and out rows."""
    return sum(lens) * HKV * HD * 2 * 2 + len(lens) * HQ * HD * 2 * 2


# ------------------------------------------------------------------------------------------
# CPU arm: the reference's CPU path for the same step on the host cores (bounded sample).
# Attention: the C restatement of CPUQwen35.attention (oracle port; the Swift original cannot
# be built here). GDN: the reference's own tinytitan_delta_rule compiled from its sources
# (oracle/_ref) when present, else the port.
# ------------------------------------------------------------------------------------------
CPU_SAMPLE_SESSIONS = 8


def cpu_step_setup(lens, threads=None):
    import oracle
    rng = np.random.default_rng(7)
    sample = lens[:CPU_SAMPLE_SESSIONS]
    bases = np.concatenate([[0], np.cumsum(sample)[:-1]]).astype(np.int64)
    total = int(sum(sample))
    keys = rng.standard_normal((total, HKV * HD), dtype=np.float32)
    values = rng.standard_normal((total, HKV * HD), dtype=np.float32)
    query = rng.standard_normal((len(sample), HQ, HD), dtype=np.float32)
    n = len(sample)
    unit = lambda x: x / np.sqrt((x * x).sum(-1, keepdims=True) + 1e-6)
    gq = unit(rng.standard_normal((n, GK, GD), dtype=np.float32)).reshape(n, -1)
    gk = unit(rng.standard_normal((n, GK, GD), dtype=np.float32)).reshape(n, -1)
    gv = rng.standard_normal((n, GV, GD), dtype=np.float32)
    ga = rng.standard_normal((n, GV), dtype=np.float32)
    gb = rng.standard_normal((n, GV), dtype=np.float32)
    state = (0.02 * rng.standard_normal((n, GV, GD, GD), dtype=np.float32))
    zeros = np.zeros(GV, np.float32)
    use_ref = oracle.ref() is not None
    threads = threads or oracle.max_threads()

    def step():
        oracle.cpu_engine_attention_sessions(query, keys, values, sample, bases, HKV, SCALE, threads)
        oracle.delta_rule_sessions(gq, gk, gv, ga, gb, zeros, zeros, GK, 1.0 / np.sqrt(GD), state,
                                   threads=threads, use_ref=use_ref)

    desc = (f"first {n} of the 32 sessions (sum S = {total} keys): decode attention = C port of "
            f"CPUQwen35.attention over (session, head) pairs + GDN step = "
            f"{'reference tinytitan_delta_rule_range (oracle/_ref)' if use_ref else 'C port of tinytitan_delta_rule'}"
            f", {threads} host threads")
    return step, n, threads, desc, ("reference+port" if use_ref else "port")


def time_cpu(lens, steps, warmup, threads=None):
    step, n, threads, desc, kind = cpu_step_setup(lens, threads)
    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    # attention is the C port of the Swift engine (the Swift original cannot be built here), so the arm is a
    # "port" even when the GDN half runs the reference's own compiled kernel
    return {"value": n / dt, "unit": UNIT, "cores": threads, "kind": "port", "sample": desc, "ms_per_step": dt * 1e3,
            "gdn_kernel": kind}


def cpu_side_baselines():
    """The reference's CPU path for the other kernels, on bounded samples (reported only)."""
    import oracle
    out = {}
    threads = oracle.max_threads()
    rng = np.random.default_rng(11)
    # prefill attention: CPUQwen35 attentionHead (gather + scores GEMM + masked softmax + PV GEMM) for all 16
    # heads over a 1024-token prompt; the GEMM is a plain loop (the reference calls Accelerate's cblas_sgemm)
    t = 1024
    q = rng.standard_normal((t, HQ, HD), dtype=np.float32)
    k = rng.standard_normal((t, HKV * HD), dtype=np.float32); v = rng.standard_normal((t, HKV * HD), dtype=np.float32)
    t0 = time.perf_counter()
    oracle.cpu_engine_attention_batch(q, k, v, HKV, 0, SCALE, threads=threads)
    dt = time.perf_counter() - t0
    flops = 4.0 * HQ * HD * (t * (t + 1) / 2)
    out["prefill_attention"] = {"TFLOPs_causal": flops / dt / 1e12, "seconds": dt, "cores": threads, "kind": "port",
                                "sample": f"{t}-token prompt, 16/2/256, all heads over {threads} threads, loop GEMM"}
    # GDN prefill scan: the reference's tinytitan_delta_rule_chunk at its default chunk 8 and at 64
    t = 512
    unit = lambda x: x / np.sqrt((x * x).sum(-1, keepdims=True) + 1e-6)
    gq = unit(rng.standard_normal((t, GK, GD), dtype=np.float32)).reshape(t, -1)
    gk = unit(rng.standard_normal((t, GK, GD), dtype=np.float32)).reshape(t, -1)
    gv = rng.standard_normal((t, GV * GD), dtype=np.float32)
    al = rng.uniform(0.5, 1.0, size=(t, GV)).astype(np.float32); be = rng.uniform(0.1, 0.9, size=(t, GV)).astype(np.float32)
    st = (0.02 * rng.standard_normal((GV, GD, GD))).astype(np.float32)
    use_ref = oracle.ref() is not None
    for chunk in (8, 64):
        t0 = time.perf_counter()
        oracle.gdn_scan_heads(gq, gk, gv, al, be, GK, GV, GD, GD, chunk, st, threads=threads, use_ref=use_ref)
        dt = time.perf_counter() - t0
        out[f"gdn_scan_chunk{chunk}"] = {"tokens_per_s": t / dt, "seconds": dt, "cores": threads,
                                         "kind": "reference" if use_ref else "port",
                                         "sample": f"{t} tokens, 16/32 heads d128, tinytitan_delta_rule_chunk, heads over threads"}
    return out


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    lens = session_lengths(0)
    # a CPU step of the 8-session sample is ~60 ms on 16 cores: K steps and W warm-ups as asked
    steps, warmup = max(1, args.steps), max(0, args.warmup)
    res = time_cpu(lens, steps, warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": res["value"], "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": res["ms_per_step"], "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": config_dict(args.gpus, lens),
        "cpu_baseline": {"value": res["value"], "unit": UNIT, "cores": res["cores"], "kind": "port",
                         "sample": res["sample"]},
        "e2e": {"value": res["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))
    return 0


# ------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------
class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 100 ms while the timed batches run."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index, self.proc = gpu_index, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.gpu_index)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, smax, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); smax = float(f[2])
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": smax, "reasons": sorted(reasons),
                "samples": len(sm)}


def device_view(ptr, n, dtype):
    import torch
    typestr = {torch.float32: "<f4", torch.float16: "<f2"}[dtype]

    class Raw:
        __cuda_array_interface__ = {"shape": (n,), "typestr": typestr, "data": (ptr, False), "version": 2}
    return torch.as_tensor(Raw(), device="cuda")


class Workload:
    """Config-2 state on one GPU: a KV cache and a GDN state in the reference's slot layouts,
    the step's device-side inputs/outputs, and the prepared operator calls."""

    def __init__(self, rank: int, device: int):
        import torch
        import tinytitan_b200 as tt
        self.tt, self.torch = tt, torch
        self.lens = session_lengths(rank)
        self.ctx = tt.Context(device)
        arch = tt.ArchConfig([tt.FULL, tt.LINEAR], HKV, HD, HKV, HD, 0, tt.LinearAttentionConfig(GK, GV, GD, GD, 4))
        self.kv = tt.KVCacheManager(arch, max_context=32768, slots=N_SESSIONS)
        self.kv.reserve(32768)
        self.gdn_state = tt.GDNStateManager(arch, slots=N_SESSIONS)
        gen = torch.Generator(device="cuda"); gen.manual_seed(1234 + rank)
        cap, stride = self.kv.capacity(0), self.kv.stride(0)
        self.cap, self.row_elems = cap, stride // 2
        kview, vview = self.kv.key_view(0, 0, 0), self.kv.value_view(0, 0, 0)
        self.k_all = device_view(kview.buffer, N_SESSIONS * cap * self.row_elems, torch.float16).view(N_SESSIONS * cap, self.row_elems)
        self.v_all = device_view(vview.buffer, N_SESSIONS * cap * self.row_elems, torch.float16).view(N_SESSIONS * cap, self.row_elems)
        for s, n in enumerate(self.lens):   # N(0,1) rows, only the live ones
            self.k_all[s * cap:s * cap + n].normal_(generator=gen)
            self.v_all[s * cap:s * cap + n].normal_(generator=gen)
            self.kv.advance(s, n)
        n_state = GV * GD * GD
        self.state_all = device_view(self.gdn_state.state_slot(1, 0), N_SESSIONS * n_state, torch.float32)
        self.state_all.normal_(0.0, 0.02, generator=gen)
        la = arch.linear_attention
        # The step's inputs live in ONE device buffer and its outputs in another, so the end-to-end
        # step moves them with a single host->device and a single device->host copy.
        n_q, n_conv, n_g, n_kv = N_SESSIONS * HQ * HD, N_SESSIONS * la.qkv_dim, N_SESSIONS * GV, 2 * N_SESSIONS * self.row_elems
        self.d_in = torch.empty(n_q + n_conv + 2 * n_g + n_kv, device="cuda", dtype=torch.float16)
        o = 0
        def take(n, shape):
            nonlocal o
            v = self.d_in[o:o + n].view(*shape); o += n
            return v
        self.q = take(n_q, (N_SESSIONS, HQ * HD))
        self.d_newkv = take(n_kv, (2, N_SESSIONS, self.row_elems))
        self.conv = take(n_conv, (N_SESSIONS, la.qkv_dim))
        self.a = take(n_g, (N_SESSIONS, GV))
        self.b = take(n_g, (N_SESSIONS, GV))
        self.d_out = torch.empty(N_SESSIONS * (HQ * HD + GV * GD), device="cuda", dtype=torch.float16)
        self.out = self.d_out[:N_SESSIONS * HQ * HD].view(N_SESSIONS, HQ * HD)
        self.y = self.d_out[N_SESSIONS * HQ * HD:].view(N_SESSIONS, GV * GD)
        self.q.copy_(torch.randn(N_SESSIONS, HQ * HD, device="cuda", generator=gen).half())
        qk = torch.randn(N_SESSIONS, 2 * GK, GD, device="cuda", generator=gen)
        qk = qk / qk.norm(dim=-1, keepdim=True)
        qk[:, :GK] *= GD ** -0.5
        vv = torch.randn(N_SESSIONS, GV * GD, device="cuda", generator=gen)
        self.conv.copy_(torch.cat([qk.reshape(N_SESSIONS, -1), vv], dim=1).half())
        # g = sigmoid(n) and beta = sigmoid(n') through the raw parameters: A_log = 0, dt_bias = 0, a = -n
        self.a.copy_((-torch.randn(N_SESSIONS, GV, device="cuda", generator=gen)).half())
        self.b.copy_(torch.randn(N_SESSIONS, GV, device="cuda", generator=gen).half())
        self.a_log = torch.zeros(GV, device="cuda", dtype=torch.bfloat16)
        self.dt_bias = torch.zeros(GV, device="cuda", dtype=torch.bfloat16)
        self.attn = tt.Attention(self.ctx)
        self.gdn = tt.GDN(self.ctx, la)
        esz = 2
        sessions = [tt.DecodeSession(self.q, self.out, kview.buffer, vview.buffer, n, 1, 0,
                                     q_offset=s * HQ * HD * esz, out_offset=s * HQ * HD * esz,
                                     k_offset=s * cap * stride, v_offset=s * cap * stride)
                    for s, n in enumerate(self.lens)]
        self.attn_batch = self.attn.prepare_batch(sessions, HD, HQ, HKV, scale=SCALE, io_dtype=tt.TT_F16)
        gs = [tt.GDNSession(self.conv, self.a, self.b, self.gdn_state.state_slot(1, s), self.y,
                            conv_out_offset=s * la.qkv_dim * esz, a_proj_offset=s * GV * esz,
                            b_proj_offset=s * GV * esz, y_offset=s * GV * GD * esz) for s in range(N_SESSIONS)]
        self.gdn_batch = self.gdn.prepare_batch(gs)
        # where each session's newest token goes: (slot, position S_i - 1), written by tt_kv_cache_write_rows
        self.new_slots = np.arange(N_SESSIONS, dtype=np.uint32)
        self.new_positions = np.array([n - 1 for n in self.lens], np.uint32)
        # pinned host side of the end-to-end step
        self.d_newkv.copy_(torch.randn(2, N_SESSIONS, self.row_elems, device="cuda", generator=gen).half())
        self.h_in = torch.empty(self.d_in.shape, dtype=torch.float16).pin_memory().copy_(self.d_in.cpu())
        self.h_out = torch.empty(self.d_out.shape, dtype=torch.float16).pin_memory()
        self.h2d = self.h_in.numel() * 2
        self.d2h = self.h_out.numel() * 2
        torch.cuda.synchronize()

    def step(self):
        self.attn.encode_prepared(self.attn_batch)
        self.gdn.encode_prepared(self.gdn_batch, self.a_log, self.dt_bias)

    def step_e2e(self):
        """One step driven from pinned host buffers: every byte of the step's inputs crosses host->device and
        every byte of its outputs device->host inside the step. One stream: sending the GDN layer's inputs and
        the attention rows over a second stream while the other layer computes measured the same 0.23 ms (the
        two copies are ~25 us of the step and the event hops cost what the overlap saves)."""
        t = self.torch
        self.d_in.copy_(self.h_in, non_blocking=True)                # q, new K/V rows, conv/a/b rows: one copy
        # the projections' write into kSlot / vSlot of every session: one launch of the library's own
        self.kv.write_rows(0, self.new_slots, self.new_positions, self.d_newkv[0], self.d_newkv[1], self.row_elems * 2)
        self.step()
        self.h_out.copy_(self.d_out, non_blocking=True)              # attention rows and GDN y: one copy
        t.cuda.current_stream().synchronize()   # the caller reads the step's result


def timed_loop(torch, dist, world, fn, steps):
    """One batch: barrier + synchronize on both sides, CUDA events on the launching stream, max over ranks."""
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    start.record()
    for _ in range(steps):
        fn()
    end.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    ms = torch.tensor([start.elapsed_time(end)], device="cuda")
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return float(ms.item())


def timed_batches(torch, dist, world, fn, steps, min_seconds=0.5, max_batches=400):
    """`steps`-long batches repeated until `min_seconds` have been timed (at least 3 batches). Returns the
    per-batch milliseconds; the count is fixed from the first batch so that every rank runs the same number."""
    first = timed_loop(torch, dist, world, fn, steps)
    n = int(min(max_batches, max(3, -(-min_seconds * 1e3 // max(first, 1e-3)))))
    return [first] + [timed_loop(torch, dist, world, fn, steps) for _ in range(n - 1)]


class _Skip(Exception):
    """Raised inside a side measurement that was not asked for."""


def aux_measurements(w, pk, only=None, c5_sessions=64):
    """Other kernels of the path on their own configurations (rank 0, outside the timed region).
    `only`: run just the named case (a smaller, profiler-sized run); `c5_sessions`: sessions of config 5."""
    torch, tt = w.torch, w.tt
    aux = {}

    def want(name):
        if only is not None and name != only:
            raise _Skip()

    def ev_time(fn, reps, warm=3):
        for _ in range(warm):
            fn()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize(); s.record()
        for _ in range(reps):
            fn()
        e.record(); torch.cuda.synchronize()
        return s.elapsed_time(e) / reps

    # GDN decode step alone (128 MiB of state read + written per step)
    def kernel_ms(fn, reps):
        """Mean device time of the GDN step kernel alone (event pairs the library records per launch)."""
        w.ctx.profile_enable(w.ctx.PROFILE_GDN_STEP)
        for _ in range(reps):
            fn()
        t = w.ctx.profile_collect()
        w.ctx.profile_enable(False)
        return sum(t) / max(1, len(t))

    if only in (None, "gdn_step_c2"):
        ms = ev_time(lambda: w.gdn.encode_prepared(w.gdn_batch, w.a_log, w.dt_bias), 50)
        kms = kernel_ms(lambda: w.gdn.encode_prepared(w.gdn_batch, w.a_log, w.dt_bias), 50)
        gdn_bytes = N_SESSIONS * GV * GD * GD * 4 * 2 + N_SESSIONS * (2 * GK * GD + GV * GD) * 2 + N_SESSIONS * GV * GD * 2
        aux["gdn_step_c2"] = {"ms": ms, "kernel_ms": kms, "GBps": gdn_bytes / kms / 1e6,
                              "frac_hbm": gdn_bytes / kms / 1e6 / pk["hbm_gbs"],
                              "note": "GBps and frac_hbm from kernel_ms (per-launch events); ms is one Python call per step; "
                                      "launched back to back, so about half of the 134 MB state is still in L2 -- "
                                      "the cold-L2 figure is gdn_step_in_step in the main line"}
    # config 3: causal prefill, 8192 tokens, 16/2/256, bf16, tcgen05 kernel
    try:
        want("prefill_c3")
        T = 8192
        g = torch.Generator(device="cuda"); g.manual_seed(3)
        q = torch.randn(T, HQ * HD, device="cuda", generator=g).bfloat16()
        k = torch.randn(T, HKV * HD, device="cuda", generator=g).bfloat16()
        v = torch.randn(T, HKV * HD, device="cuda", generator=g).bfloat16()
        o = torch.empty_like(q)
        p = tt.PrefillAttentionParams(0, T, HD, HQ, HKV, T, 0, HKV * HD, HQ * HD, HQ * HD, SCALE)
        pa = tt.PrefillAttention(w.ctx)
        ms = ev_time(lambda: pa.encode_causal(q, k, v, o, p), 10)
        flops = 4.0 * HQ * HD * (T * (T + 1) / 2)
        aux["prefill_c3_bf16"] = {"ms": ms, "TFLOPs": flops / ms / 1e9, "frac_tensor": flops / ms / 1e9 / pk["bf16_tflops"],
                                  "path": tt.PrefillAttention.selected_path(q, k, v, o, p)}
        del q, k, v, o
    except _Skip:
        pass
    except Exception as exc:  # reported, never hidden
        aux["prefill_c3_bf16"] = {"error": str(exc)}
    # config 3: GDN prefill over 8192 tokens, 16/32 heads, d 128: chunk-parallel scan vs the exact sequential kernel
    try:
        want("gdn_scan_c3")
        T = 8192
        g = torch.Generator(device="cuda"); g.manual_seed(5)
        cfg = tt.LinearAttentionConfig(GK, GV, GD, GD)
        qk = torch.randn(T, 2 * GK, GD, device="cuda", generator=g)
        qk = qk / qk.norm(dim=-1, keepdim=True); qk[:, :GK] *= GD ** -0.5
        conv = torch.cat([qk.reshape(T, -1), torch.randn(T, GV * GD, device="cuda", generator=g)], 1).half().contiguous()
        a = (-torch.randn(T, GV, device="cuda", generator=g)).half(); b = torch.randn(T, GV, device="cuda", generator=g).half()
        st = 0.02 * torch.randn(GV, GD, GD, device="cuda", generator=g)
        y = torch.empty(T, GV * GD, device="cuda", dtype=torch.float16)
        gdn = tt.GDN(w.ctx, cfg)
        ms_scan = ev_time(lambda: gdn.encode_delta_scan_chunked(conv, a, b, w.a_log, w.dt_bias, st, y, T), 5, warm=2)
        ms_seq = ev_time(lambda: gdn.encode_delta_step_prefill(conv, a, b, w.a_log, w.dt_bias, st, y, T), 3, warm=1)
        scan_bytes = T * (2 * GK * GD + GV * GD) * 2 + T * GV * GD * 2 + 2 * GV * GD * GD * 4 + T * GV * 4
        scan_flops = (T / 64) * GV * 9.44e6
        aux["gdn_scan_c3"] = {"ms": ms_scan, "GBps_algorithmic": scan_bytes / ms_scan / 1e6,
                              "frac_hbm": scan_bytes / ms_scan / 1e6 / pk["hbm_gbs"], "TFLOPs": scan_flops / ms_scan / 1e9,
                              "sequential_kernel_ms": ms_seq, "tokens_per_s": T / ms_scan * 1e3}
        del conv, y
    except _Skip:
        pass
    except Exception as exc:
        aux["gdn_scan_c3"] = {"error": str(exc)}
    # config 4 on one GPU: one session, S = 262144, 16/2/256 (the per-GPU share at N GPUs is S/N of this)
    try:
        want("decode_c4")
        s4 = 262144
        g = torch.Generator(device="cuda"); g.manual_seed(6)
        k4 = torch.randn(s4, HKV * HD, device="cuda", generator=g).half()
        v4 = torch.randn(s4, HKV * HD, device="cuda", generator=g).half()
        q4 = torch.randn(HQ, HD, device="cuda", generator=g).half(); o4 = torch.empty_like(q4)
        ms = ev_time(lambda: w.attn.encode_full(q4, k4, v4, o4, HD, HQ, HKV, s4, scale=SCALE), 30)
        w.ctx.profile_enable(w.ctx.PROFILE_DECODE_PARTIAL)
        for _ in range(30):
            w.attn.encode_full(q4, k4, v4, o4, HD, HQ, HKV, s4, scale=SCALE)
        t = w.ctx.profile_collect()
        w.ctx.profile_enable(False)
        kms = sum(t) / max(1, len(t))
        b4 = s4 * HKV * HD * 2 * 2 + HQ * HD * 2 * 2
        aux["decode_c4_1gpu"] = {"ms": ms, "pass1_kernel_ms": kms, "GBps": b4 / ms / 1e6,
                                 "frac_hbm": b4 / ms / 1e6 / pk["hbm_gbs"], "pass1_frac_hbm": b4 / kms / 1e6 / pk["hbm_gbs"]}
        del k4, v4
    except _Skip:
        pass
    except Exception as exc:
        aux["decode_c4_1gpu"] = {"error": str(exc)}
    # config 5: 64 sessions x 4 draft rows, S = 16384 (+3), 32/2/256; GDN 4-row step with 64 value heads. Once with
    # all 64 sessions on this GPU and once with 8 (the share of one GPU when the batch is sharded over 8).
    def verify_case(n5, suffix):
        w5, s5, hq5 = 4, 16384 + 3, 32
        batch, keep = make_decode_batch(torch, tt, w.attn, [s5] * n5, hq5, w5, 8)
        ms = ev_time(lambda: w.attn.encode_prepared(batch), 10)
        w.ctx.profile_enable(w.ctx.PROFILE_DECODE_PARTIAL)
        for _ in range(10):
            w.attn.encode_prepared(batch)
        t = w.ctx.profile_collect()
        w.ctx.profile_enable(False)
        kms = sum(t) / max(1, len(t))
        b5 = n5 * s5 * HKV * HD * 2 * 2 + 2 * n5 * w5 * hq5 * HD * 2
        # host cost of one call: the split planner simulates the dispatch when the batch's tile counts change
        # (a fresh context = a cold plan) and reuses the plan otherwise
        cold_ctx = tt.Context(w.ctx.device)
        cold_attn = tt.Attention(cold_ctx)
        torch.cuda.synchronize()
        t0 = time.perf_counter(); cold_attn.encode_prepared(batch); cold_us = (time.perf_counter() - t0) * 1e6
        t0 = time.perf_counter(); cold_attn.encode_prepared(batch); warm_us = (time.perf_counter() - t0) * 1e6
        torch.cuda.synchronize()
        cold_ctx.close()
        aux["verify_c5" + suffix] = {"sessions": n5, "ms": ms, "pass1_kernel_ms": kms, "GBps": b5 / ms / 1e6,
                                     "frac_hbm": b5 / ms / 1e6 / pk["hbm_gbs"], "pass1_frac_hbm": b5 / kms / 1e6 / pk["hbm_gbs"],
                                     "tok_per_s": n5 * w5 / ms * 1e3, "host_us_first_call_cold_plan": cold_us,
                                     "host_us_next_call_cached_plan": warm_us,
                                     "note": "ms = whole call (pass 1 + merge; tables travel in the kernel parameters up to 16 sessions, else one upload), one Python call per step"}
        del batch, keep
        gdn5, gb, z5, keep2, cfg5 = make_gdn_batch(torch, tt, w.ctx, n5, 64, w5, 9)
        ms = ev_time(lambda: gdn5.encode_prepared(gb, z5, z5, rows=w5), 10)
        kms = kernel_ms(lambda: gdn5.encode_prepared(gb, z5, z5, rows=w5), 10)
        bg = n5 * 64 * GD * GD * 4 * 2 + n5 * w5 * (cfg5.qkv_dim + 64 * GD) * 2
        aux["gdn_verify_c5" + suffix] = {"sessions": n5, "ms": ms, "kernel_ms": kms, "GBps": bg / kms / 1e6,
                                         "frac_hbm": bg / kms / 1e6 / pk["hbm_gbs"]}

    try:
        want("verify_c5")
        if only is None:
            verify_case(64, "_1gpu")
            verify_case(8, "_8sessions_share_of_one_gpu")
        else:
            verify_case(c5_sessions, "_1gpu")
    except _Skip:
        pass
    except Exception as exc:
        aux["verify_c5_1gpu_error"] = str(exc)
    # config 1: one session, S = 4096, 8/2/256; 32 distinct caches are rotated so HBM is really read
    try:
        want("decode_c1")
        s1, hq1 = 4096, 8
        g = torch.Generator(device="cuda"); g.manual_seed(4)
        ks = torch.randn(32, s1, HKV * HD, device="cuda", generator=g).half()
        vs = torch.randn(32, s1, HKV * HD, device="cuda", generator=g).half()
        q1 = torch.randn(hq1, HD, device="cuda", generator=g).half(); o1 = torch.empty_like(q1)
        state = {"i": 0}

        def one():
            i = state["i"] = (state["i"] + 1) % 32
            w.attn.encode_full(q1, ks[i], vs[i], o1, HD, hq1, HKV, s1, scale=SCALE)
        ms = ev_time(one, 64)
        b1 = s1 * HKV * HD * 2 * 2 + hq1 * HD * 2 * 2
        aux["decode_c1"] = {"ms": ms, "GBps": b1 / ms / 1e6, "frac_hbm": b1 / ms / 1e6 / pk["hbm_gbs"],
                            "note": "32 rotating caches (268 MB) so the 8 MiB working set does not sit in L2; "
                                    "one Python call per step, so this includes ~10 us of host overhead"}
        # the same 32 calls replayed from one CUDA graph: device-side time per call without the host
        try:
            graph = torch.cuda.CUDAGraph()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for _ in range(32):
                    one()
                torch.cuda.synchronize()
                with torch.cuda.graph(graph, stream=side):
                    for _ in range(32):
                        one()
            torch.cuda.synchronize()
            msg = ev_time(graph.replay, 20) / 32
            aux["decode_c1"]["graph_ms"] = msg
            aux["decode_c1"]["graph_GBps"] = b1 / msg / 1e6
            aux["decode_c1"]["graph_frac_hbm"] = b1 / msg / 1e6 / pk["hbm_gbs"]
        except Exception as exc:
            aux["decode_c1"]["graph_error"] = str(exc)
    except _Skip:
        pass
    except Exception as exc:
        aux["decode_c1"] = {"error": str(exc)}
    return aux


def split_kv_c4(w, torch, dist, rank, world, pk):
    """Config 4 on `world` GPUs: one session of 262,144 keys (16/2/256 fp16) whose KV rows are split
    along the sequence; one decode step = pass 1 on the local rows + the cross-GPU merge, once with
    an NCCL all-gather followed by the merge kernel and once with exchange and merge fused in one
    kernel over peer memory. Device time per step, max over ranks."""
    from tinytitan_b200 import sharding
    s4 = 262144
    lo, hi = sharding.kv_split_ranges(s4, world)[rank]
    g = torch.Generator(device="cuda"); g.manual_seed(600 + rank)
    k = torch.randn(hi - lo, HKV * HD, device="cuda", generator=g).half()
    v = torch.randn(hi - lo, HKV * HD, device="cuda", generator=g).half()
    g.manual_seed(6)
    q = torch.randn(HQ, HD, device="cuda", generator=g).half()
    out_a, out_b = torch.empty_like(q), torch.empty_like(q)
    plain = sharding.LongContextDecode(w.attn, HD, HQ, HKV, SCALE)
    fused = sharding.LongContextDecode(w.attn, HD, HQ, HKV, SCALE, fused=True)

    def timed(fn, reps=100):
        for _ in range(5):
            fn()
        dist.barrier(); torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record(); torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / reps], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    ms_nccl = timed(lambda: plain.step(q, k, v, hi - lo, out_a))
    ms_fused = timed(lambda: fused.step(q, k, v, hi - lo, out_b))
    # Where the fused step's time goes: every rank's own kernel durations (event pairs the library records
    # around pass 1 and around the merge + exchange kernel, whose duration INCLUDES its wait for the slowest
    # peer) next to the wall figure above. wall - (pass 1 + exchange) on the fastest rank is launch gaps and
    # host time; exchange(max over ranks) - exchange(min over ranks) is the skew the flag wait absorbs.
    w.ctx.profile_enable(w.ctx.PROFILE_DECODE_PARTIAL | w.ctx.PROFILE_EXCHANGE)
    dist.barrier(); torch.cuda.synchronize()
    for _ in range(100):
        fused.step(q, k, v, hi - lo, out_b)
    torch.cuda.synchronize()
    rec = w.ctx.profile_collect()
    w.ctx.profile_enable(False)
    mine = torch.tensor([statistics.mean(rec[0::2]) if rec else 0.0, statistics.mean(rec[1::2]) if rec else 0.0], device="cuda")
    allr = [torch.zeros_like(mine) for _ in range(world)]
    dist.all_gather(allr, mine)
    p1 = [float(t[0]) for t in allr]; ex = [float(t[1]) for t in allr]
    agree = float((out_a.float() - out_b.float()).abs().max().item())
    status = w.ctx.poll_status()
    fused.close()
    bytes_total = s4 * HKV * HD * 2 * 2 + HQ * HD * 2 * 2
    return {"S": s4, "keys_per_gpu": hi - lo, "ms_nccl_allgather": ms_nccl, "ms_fused_exchange": ms_fused,
            "GBps_aggregate_fused": bytes_total / ms_fused / 1e6,
            "frac_hbm_aggregate_fused": bytes_total / ms_fused / 1e6 / (pk["hbm_gbs"] * world),
            "fused_kernels_ms": {"pass1_min": min(p1), "pass1_max": max(p1), "merge_exchange_min": min(ex),
                                 "merge_exchange_max": max(ex),
                                 "launch_and_host_ms": ms_fused - (min(p1) + min(ex)),
                                 "skew_absorbed_by_the_flag_wait_ms": max(ex) - min(ex)},
            "max_abs_diff_between_paths": agree, "device_status": status,
            "note": "one Python call per step on every rank; device time, max over ranks"}


def make_decode_batch(torch, tt, attn, lens, hq, q_rows, seed):
    """A batched decode call over freshly drawn sessions of the given lengths (one KV store, slot layout)."""
    g = torch.Generator(device="cuda"); g.manual_seed(seed)
    n = len(lens)
    cap = max(lens) + 8
    k = torch.randn(n * cap, HKV * HD, device="cuda", generator=g).half()
    v = torch.randn(n * cap, HKV * HD, device="cuda", generator=g).half()
    q = torch.randn(n, q_rows, hq * HD, device="cuda", generator=g).half()
    o = torch.empty_like(q)
    row = HKV * HD * 2
    ses = [tt.DecodeSession(q, o, k, v, lens[i], q_rows, 0, q_offset=i * q_rows * hq * HD * 2, out_offset=i * q_rows * hq * HD * 2,
                            k_offset=i * cap * row, v_offset=i * cap * row) for i in range(n)]
    batch = attn.prepare_batch(ses, HD, hq, HKV, scale=SCALE, io_dtype=tt.TT_F16)
    return batch, (k, v, q, o)


def make_gdn_batch(torch, tt, ctx, n, hv, rows, seed):
    g = torch.Generator(device="cuda"); g.manual_seed(seed)
    cfg = tt.LinearAttentionConfig(GK, hv, GD, GD)
    st = 0.02 * torch.randn(n, hv * GD * GD, device="cuda", generator=g)
    qk = torch.randn(n * rows, 2 * GK, GD, device="cuda", generator=g)
    qk = qk / qk.norm(dim=-1, keepdim=True); qk[:, :GK] *= GD ** -0.5
    conv = torch.cat([qk.reshape(n * rows, -1), torch.randn(n * rows, hv * GD, device="cuda", generator=g)], 1).half().contiguous()
    a = (-torch.randn(n * rows, hv, device="cuda", generator=g)).half(); b = torch.randn(n * rows, hv, device="cuda", generator=g).half()
    y = torch.empty(n * rows, hv * GD, device="cuda", dtype=torch.float16)
    z = torch.zeros(hv, device="cuda", dtype=torch.bfloat16)
    gdn = tt.GDN(ctx, cfg)
    gs = [tt.GDNSession(conv[i * rows:(i + 1) * rows], a[i * rows:(i + 1) * rows], b[i * rows:(i + 1) * rows], st[i],
                        y[i * rows:(i + 1) * rows]) for i in range(n)]
    return gdn, gdn.prepare_batch(gs), z, (st, conv, a, b, y), cfg


def sharded_configs(w, torch, dist, rank, world, pk):
    """Configs 2 and 5 as stated: a FIXED batch (32 drawn sessions; 64 verify sessions of 4 draft rows at
    context 16384) split over the `world` GPUs with no collective. The whole batch is first timed on rank 0
    alone, then every rank runs its shard; value = sessions of the whole batch / max-over-ranks step time,
    efficiency = t(1 GPU) / (world * t(world GPUs))."""
    from tinytitan_b200 import sharding
    tt = w.tt
    out = {}

    def device_ms(fn, reps, everyone=True):
        for _ in range(3):
            fn()
        if everyone:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record(); torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / reps], device="cuda")
        if everyone:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def one_config(name, lens, hq, q_rows, hv, reps):
        # whole batch on rank 0 alone
        t1 = torch.zeros(1, device="cuda")
        if rank == 0:
            batch, keep = make_decode_batch(torch, tt, w.attn, lens, hq, q_rows, 900)
            gdn, gb, z, keep2, _ = make_gdn_batch(torch, tt, w.ctx, len(lens), hv, q_rows, 901)
            t1[0] = device_ms(lambda: (w.attn.encode_prepared(batch), gdn.encode_prepared(gb, z, z, rows=q_rows)), reps, everyone=False)
            del batch, keep, gb, keep2
            torch.cuda.empty_cache()
        dist.broadcast(t1, 0)
        shard = sharding.shard_sessions(lens, world, "greedy")[rank]
        mine = [lens[i] for i in shard]
        batch, keep = make_decode_batch(torch, tt, w.attn, mine, hq, q_rows, 910 + rank)
        gdn, gb, z, keep2, cfg = make_gdn_batch(torch, tt, w.ctx, len(mine), hv, q_rows, 920 + rank)
        tn = device_ms(lambda: (w.attn.encode_prepared(batch), gdn.encode_prepared(gb, z, z, rows=q_rows)), reps)
        my_bytes = sum(mine) * HKV * HD * 2 * 2 + 2 * len(mine) * q_rows * hq * HD * 2 + \
            len(mine) * hv * GD * GD * 4 * 2 + len(mine) * q_rows * (cfg.qkv_dim + hv * GD) * 2
        b = torch.tensor([float(my_bytes)], device="cuda")
        dist.all_reduce(b, op=dist.ReduceOp.MAX)
        assert w.ctx.poll_status() == 0
        out[name] = {"sessions_total": len(lens), "sessions_per_gpu": len(mine), "rows_per_session": q_rows,
                     "ms_step_1gpu_whole_batch": float(t1.item()), "ms_step": tn,
                     "tok_per_s": len(lens) * q_rows / tn * 1e3,
                     "speedup_over_1gpu": float(t1.item()) / tn, "efficiency": float(t1.item()) / tn / world,
                     "frac_hbm_per_gpu_heaviest_shard": float(b.item()) / tn / 1e6 / pk["hbm_gbs"],
                     "note": "attention + GDN step of the shard per step, device time, max over ranks; greedy byte balancing"}
        del batch, keep, gb, keep2

    one_config("c2_strong", session_lengths(0) if N_SESSIONS == 32 else session_lengths(0), HQ, 1, GV, 200)
    one_config("c5_sharded", [16384 + 3] * 64, 32, 4, 64, 50)
    return out


# ncu (dram__bytes_read.sum + dram__bytes_write.sum) of attn_decode_partial_kernel per algorithmic
# byte, from an 8-session capture of this workload (221.9 MB of DRAM traffic for 216.9 MB of
# algorithmic bytes). Traffic grows in proportion to the keys processed, so a full launch is this
# ratio times its algorithmic bytes.
TRAFFIC_PER_ALGORITHMIC_BYTE = 1.023


def run_gpu_arm(args):
    import torch
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    pk = peaks()
    w = Workload(rank, local_rank)
    if args.case is not None:
        # one side measurement alone (a small, profiler-sized run); not a benchmark line
        if rank == 0:
            print(json.dumps({"case": args.case, "sessions": args.sessions, "c5_sessions": args.c5_sessions,
                              "aux": aux_measurements(w, pk, only=args.case, c5_sessions=args.c5_sessions)}))
        return 0
    sampler = ClockSampler(local_rank)

    for _ in range(max(3, args.warmup)):
        w.step()
    torch.cuda.synchronize()
    sampler.start()
    launches0 = w.ctx.launch_count
    batch_ms = timed_batches(torch, dist, world, w.step, args.steps, args.min_seconds)
    launches = (w.ctx.launch_count - launches0) // len(batch_ms)       # per batch of `steps` steps
    # per-launch device time of the dominant kernels (the library's own event pairs), one more batch
    w.ctx.profile_enable(w.ctx.PROFILE_DECODE_PARTIAL | w.ctx.PROFILE_GDN_STEP)
    timed_loop(torch, dist, world, w.step, min(args.steps, 128))
    both_ms = w.ctx.profile_collect()
    w.ctx.profile_enable(False)
    # a step launches the decode pass 1 and then the GDN step: the record alternates
    partial_ms, gdn_ms = both_ms[0::2], both_ms[1::2]
    assert w.ctx.poll_status() == 0, "device status word is not clean"

    for _ in range(3):
        w.step_e2e()
    e2e_steps = args.steps
    e2e_ms = timed_batches(torch, dist, world, w.step_e2e, e2e_steps, args.min_seconds)
    clocks = sampler.stop()
    clocks["note"] = "sampled every 100 ms over the timed batches of the device-resident and the end-to-end step"

    c4 = strong = None
    if world > 1 and not args.no_aux:
        try:
            c4 = split_kv_c4(w, torch, dist, rank, world, pk)
        except Exception as exc:   # the same code runs on every rank, so a failure is common to all
            c4 = {"error": str(exc)}
        try:
            strong = sharded_configs(w, torch, dist, rank, world, pk)
        except Exception as exc:
            strong = {"error": str(exc)}

    ms_total = statistics.median(batch_ms)
    ms_e2e = statistics.median(e2e_ms)
    ms_per_step = ms_total / args.steps
    value = world * N_SESSIONS / (ms_per_step * 1e-3)
    e2e_value = world * N_SESSIONS / (ms_e2e / e2e_steps * 1e-3)
    if rank == 0:
        alg = algorithmic_bytes(w.lens)
        kernel_ms = statistics.mean(partial_ms) if partial_ms else None
        achieved = alg / kernel_ms / 1e6 if kernel_ms else None
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "timing": {"batches": len(batch_ms), "steps_per_batch": args.steps, "statistic": "median batch",
                       "ms_per_step_min": min(batch_ms) / args.steps, "ms_per_step_max": max(batch_ms) / args.steps,
                       "timed_seconds": sum(batch_ms) / 1e3},
            "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": config_dict(world, w.lens),
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": w.h2d, "d2h_bytes_per_step": w.d2h,
                    "steps": e2e_steps, "ms_per_step": ms_e2e / e2e_steps, "batches": len(e2e_ms),
                    "ms_per_step_min": min(e2e_ms) / e2e_steps, "ms_per_step_max": max(e2e_ms) / e2e_steps},
            "gpu_launches": int(launches),
            "clocks": clocks,
            "roofline": {"bound": "hbm", "kernel": "attn_decode_partial_kernel<256,1,2,half>", "achieved": achieved,
                         "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": (achieved / pk["hbm_gbs"]) if achieved else None,
                         "peak_source": pk["source"], "algorithmic_bytes_per_launch": alg, "kernel_ms": kernel_ms,
                         "launches_timed": len(partial_ms),
                         "traffic": (TRAFFIC_PER_ALGORITHMIC_BYTE * alg) if TRAFFIC_PER_ALGORITHMIC_BYTE else None},
            "hbm_GBps_step": (alg + N_SESSIONS * GV * GD * GD * 8) / ms_per_step / 1e6,
            "gdn_step_in_step": ({"kernel_ms": statistics.mean(gdn_ms),
                                  "frac_hbm": N_SESSIONS * GV * GD * GD * 8 / statistics.mean(gdn_ms) / 1e6 / pk["hbm_gbs"],
                                  "note": "the GDN step kernel between two decode passes (cold L2), state bytes only"}
                                 if gdn_ms else None),
        }
        if world == 1 and not args.no_aux:
            line["aux"] = aux_measurements(w, pk)
            cpu = time_cpu(w.lens, 3, 1)
            line["cpu_baseline"] = {k: cpu[k] for k in ("value", "unit", "cores", "kind", "sample")}
            # the reference runs decode attention on ONE thread (CPUQwen35.swift:313-348): the same sample, one thread
            one = time_cpu(w.lens, 2, 1, threads=1)
            line["cpu_baseline"]["single_thread"] = {"value": one["value"], "unit": UNIT, "cores": 1, "ms_per_step": one["ms_per_step"]}
            line["aux"]["cpu"] = cpu_side_baselines()
        else:
            line["cpu_baseline"] = None
            if c4 is not None:
                line["aux"] = {"decode_c4_split_kv": c4}
                if isinstance(strong, dict):
                    line["aux"].update(strong)
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="tinytitan", choices=["tinytitan", "reference"])
    ap.add_argument("--no-aux", action="store_true", help="skip the side measurements and the CPU baseline")
    ap.add_argument("--sessions", type=int, default=32,
                    help="sessions per GPU (32 is the benchmark; a smaller count is for profiler captures only)")
    ap.add_argument("--case", default=None,
                    choices=["gdn_step_c2", "prefill_c3", "gdn_scan_c3", "decode_c4", "verify_c5", "decode_c1"],
                    help="run one side measurement alone and exit (for profiler captures)")
    ap.add_argument("--c5-sessions", type=int, default=64, help="sessions of the config-5 side measurement")
    ap.add_argument("--min-seconds", type=float, default=0.5,
                    help="batches of --steps steps are repeated until this much time has been measured (0: three batches; "
                         "for profiler captures)")
    args = ap.parse_args()
    global N_SESSIONS
    N_SESSIONS = args.sessions
    if args.impl == "reference":
        return run_reference_arm(args)
    return run_gpu_arm(args)


if __name__ == "__main__":
    raise SystemExit(main())
