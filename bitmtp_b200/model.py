"""Packed T2-g128 inference model on the B200 kernels.

Host-side mirror of `bonsai_sft.gpu.model` of the reference for the packed
ternary decode path: same operator names (`t2g128_int8xint2_linear`,
`packed_int8_linear`, `T2LinearKernel`), same module tree and state-dict keys,
same forward entry points (`forward_sdlm_decode_graph_kernel`,
`forward_sdlm_prefill`, `prepare_merged_weights`, `prepare_t2_lm_head`).  Every
tensor expression of the reference's forward is one call into
libbitmtp_b200.so; PyTorch only owns the memory and the stream.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch
from torch import nn

from . import native, ops
from .contracts import require_kernel_shape, require_native_shape

SDLMLayerCache = Tuple[torch.Tensor, torch.Tensor]

_t2_lib = None


def load_t2_kernel() -> None:
    """Load libbitmtp_b200.so (the reference loads libbonsai_t2.so here:
    src/bonsai_sft/gpu/model.py:206-219).  Raises if the library is not built."""
    global _t2_lib
    _t2_lib = native.lib()


def _validate_packed_inputs(a, b, s, ws, *, kind: str = "t2g128", bits: int = 2,
                            activation_dtype=torch.int8, validate_registry: bool = False):
    """Metadata checks ahead of the native call, in the reference's order and with its
    messages (src/bonsai_sft/gpu/model.py:96-115).  They run before the library is
    loaded, so a bad call fails without touching CUDA."""
    if a.dim() not in (2, 3) or b.dim() != 2:
        raise ValueError(f"{kind}: expected rank-2/3 activation and rank-2 weight")
    m = a.numel() // a.shape[-1] if a.shape[-1] else 0
    n, k = b.shape[0], b.shape[1] * (8 // bits)
    if validate_registry:
        require_kernel_shape(kind, m, n, k)
    else:
        require_native_shape(m, n, k)
    if a.shape[-1] != k:
        raise RuntimeError(f"{kind}: activation width mismatch: {a.shape[-1]} != {k}")
    if tuple(ws.shape) != (n, k // 128):
        raise RuntimeError(f"{kind}: invalid weight scale shape {tuple(ws.shape)}")
    if a.dtype != activation_dtype or b.dtype != torch.int8 or ws.dtype != torch.bfloat16:
        raise RuntimeError(f"{kind}: invalid activation, packed-weight, or scale dtype")
    if s.dtype != torch.float32 or s.shape[-1:] != (1,) or s.numel() != m:
        raise RuntimeError(f"{kind}: activation scales must be float32 with one value per row")
    tensors = (a, b, s, ws)
    if not all(t.is_cuda and t.is_contiguous() for t in tensors):
        raise RuntimeError(f"{kind}: inputs and scales must be contiguous CUDA tensors")
    if not all(t.device == a.device for t in tensors):
        raise RuntimeError(f"{kind}: inputs and scales must share one CUDA device")
    return m, n, k


def t2g128_int8xint2_linear(a_int8: torch.Tensor, b_packed: torch.Tensor, s: torch.Tensor,
                            ws: torch.Tensor, *, validate_registry: bool = False) -> torch.Tensor:
    """W2A8 linear on natural-order packed weights; returns bf16 `[..., N]`.

    Same call as the reference wrapper (src/bonsai_sft/gpu/model.py:222-256):
    a_int8 `[M, K]` or `[B, S, K]` int8, b_packed `[N, K/4]` int8, s `[..., 1]`
    fp32 (127/absmax, the output is divided by it), ws `[N, K/128]` bf16.  It goes
    through the library's drop-in symbol of the same name.  `validate_registry`
    restricts (M, N, K) to the reference's registered triples.
    """
    m, n, k = _validate_packed_inputs(a_int8, b_packed, s, ws, validate_registry=validate_registry)
    if _t2_lib is None:
        load_t2_kernel()
    out_shape = (*a_int8.shape[:-1], n)
    out = torch.empty(out_shape, dtype=torch.bfloat16, device=a_int8.device)
    stream = torch.cuda.current_stream(a_int8.device)
    _t2_lib.t2g128_int8xint2_linear(
        ctypes.c_void_p(a_int8.data_ptr()), ctypes.c_void_p(b_packed.data_ptr()),
        ctypes.c_void_p(out.data_ptr()), ctypes.c_void_p(s.data_ptr()),
        ctypes.c_void_p(ws.data_ptr()), m, n, k, ctypes.c_void_p(stream.cuda_stream))
    return out


def packed_int8_linear(a_int8, b_packed, s, ws, *, validate_registry: bool = False):
    """Dispatch by packed width (src/bonsai_sft/gpu/model.py:259-268).  Only the
    ternary layout (K/4 bytes per row) exists in this build."""
    K = a_int8.shape[-1]
    if b_packed.shape[-1] * 4 == K:
        return t2g128_int8xint2_linear(a_int8, b_packed, s, ws, validate_registry=validate_registry)
    raise ValueError(f"unknown packed weight layout A.K={K}, B.shape={tuple(b_packed.shape)}")
