"""Tensor-level wrappers over the C ABI (include/bitmtp_b200.h).

Each function validates metadata, allocates the outputs as torch tensors on the
inputs' device and enqueues one native call on torch's current stream.  None
of them computes anything in PyTorch.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch

from . import native
from .native import check


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream(device) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _require_cuda(*tensors: torch.Tensor) -> None:
    dev = tensors[0].device
    for t in tensors:
        if not t.is_cuda or not t.is_contiguous():
            raise RuntimeError("bitmtp_b200 operators take contiguous CUDA tensors")
        if t.device != dev:
            raise RuntimeError("bitmtp_b200 operators need all tensors on one CUDA device")


def t2_gemv(a_int8: torch.Tensor, b_packed: torch.Tensor, s: torch.Tensor, ws: torch.Tensor, *,
            out_kind: int = native.OUT_BF16, path: int = native.PATH_AUTO,
            want_groups: bool = False, pdl: bool = False, out: Optional[torch.Tensor] = None,
            ldc: Optional[int] = None):
    """C = ((A x ternary(B)) scaled per 128-group by ws) / s.

    a_int8 [W, K] int8, b_packed [N, K/4] int8/uint8, s [W] or [W,1] fp32,
    ws [N, K/128] bf16.  Returns C ([W, N] bf16 or fp32 per `out_kind`), or
    (C, G) with G int32 [W, N, K/128] when `want_groups`.
    """
    _require_cuda(a_int8, b_packed, s, ws)
    W, K = a_int8.shape
    N = b_packed.shape[0]
    if b_packed.shape[1] * 4 != K or tuple(ws.shape) != (N, K // 128):
        raise RuntimeError("t2_gemv: packed weight / scale shape mismatch")
    if a_int8.dtype != torch.int8 or ws.dtype != torch.bfloat16 or s.dtype != torch.float32:
        raise RuntimeError("t2_gemv: invalid activation, scale or multiplier dtype")
    if s.numel() != W:
        raise RuntimeError("t2_gemv: one activation multiplier per row is required")
    dt = torch.bfloat16 if out_kind == native.OUT_BF16 else torch.float32
    if out is None:
        out = torch.empty((W, N), dtype=dt, device=a_int8.device)
        ldc = N
    elif ldc is None:
        ldc = out.stride(0)
    G = torch.empty((W, N, K // 128), dtype=torch.int32, device=a_int8.device) if want_groups else None
    rc = native.lib().bm_t2_gemv(_ptr(a_int8), _ptr(b_packed), _ptr(out), _ptr(s), _ptr(ws),
                                 W, N, K, ldc, out_kind, path, _ptr(G), int(pdl),
                                 _stream(a_int8.device))
    check(rc, f"bm_t2_gemv(W={W}, N={N}, K={K})")
    return (out, G) if want_groups else out


def gemv_bytes(W: int, N: int, K: int, out_kind: int = native.OUT_BF16) -> int:
    return int(native.lib().bm_t2_gemv_bytes(W, N, K, out_kind))
