"""Helpers shared by the GPU parity tests."""
import numpy as np
import torch

import tinytitan_b200 as tt

TOL = 2e-3  # max abs error vs the fp32 oracle on fp16 I/O (the bar the north star states)

_ctx = None


def context() -> tt.Context:
    global _ctx
    if _ctx is None:
        _ctx = tt.Context(0)
    return _ctx


def dev(a, dtype=torch.float16):
    return torch.as_tensor(np.ascontiguousarray(a)).to(device="cuda", dtype=dtype).contiguous()


def host(t):
    return t.detach().float().cpu().numpy()


def rounded(a, dtype=torch.float16):
    """fp32 numpy copy of `a` after rounding to the storage dtype (what the kernels read)."""
    return torch.as_tensor(np.ascontiguousarray(a), dtype=torch.float32).to(dtype).float().numpy()


def bf16_tol(ref):
    """Tolerance for bf16 outputs: the fp16 bar plus one bf16 rounding step of the value."""
    return TOL + np.abs(ref) * 2.0 ** -8


class _RawDevice:
    def __init__(self, ptr, n, typestr):
        self.__cuda_array_interface__ = {"shape": (n,), "typestr": typestr, "data": (ptr, False), "version": 2}


def device_view(ptr: int, n: int, dtype=torch.float32):
    """A torch tensor over `n` elements of raw device memory owned by one of the managers."""
    typestr = {torch.float32: "<f4", torch.float16: "<f2", torch.uint8: "|u1"}[dtype]
    return torch.as_tensor(_RawDevice(ptr, n, typestr), device="cuda")
