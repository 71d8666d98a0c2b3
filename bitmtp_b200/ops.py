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


def t2_gemv_prepared(a_prep: torch.Tensor, a_sums: torch.Tensor, b_packed: torch.Tensor,
                     s: torch.Tensor, ws: torch.Tensor, *, out: torch.Tensor, ldc: Optional[int] = None,
                     out_kind: int = native.OUT_BF16, pdl: bool = False) -> torch.Tensor:
    """The GEMV on GEMV-ready activations (q_prep / asum of a quantising operator)."""
    W, K = a_prep.shape
    N = b_packed.shape[0]
    rc = native.lib().bm_t2_gemv_prepared(_ptr(a_prep), _ptr(a_sums), _ptr(b_packed), _ptr(out), _ptr(s),
                                          _ptr(ws), W, N, K, ldc if ldc is not None else out.stride(0),
                                          out_kind, int(pdl), _stream(a_prep.device))
    check(rc, f"bm_t2_gemv_prepared(W={W}, N={N}, K={K})")
    return out


def gemv_bytes(W: int, N: int, K: int, out_kind: int = native.OUT_BF16) -> int:
    return int(native.lib().bm_t2_gemv_bytes(W, N, K, out_kind))


# --------------------------------------------------------------------------- fused operators
def quant_rows(x: torch.Tensor, *, pdl: bool = False, prepared: bool = False):
    """bf16 [M, K] -> (int8 [M, K], fp32 [M, 1]); with `prepared`, the GEMV-ready form
    (q_prep int8 [M, K], asum int32 [M, K/128], s fp32 [M, 1]) instead."""
    _require_cuda(x)
    M, K = x.shape
    s = torch.empty((M, 1), dtype=torch.float32, device=x.device)
    q = qp = asum = None
    if prepared:
        qp = torch.empty((M, K), dtype=torch.int8, device=x.device)
        asum = torch.empty((M, K // 128), dtype=torch.int32, device=x.device)
    else:
        q = torch.empty((M, K), dtype=torch.int8, device=x.device)
    check(native.lib().bm_quant_rows(_ptr(x), M, K, _ptr(q), _ptr(qp), _ptr(asum), _ptr(s), int(pdl),
                                     _stream(x.device)), "bm_quant_rows")
    return (qp, asum, s) if prepared else (q, s)


def rmsnorm_fused(x: torch.Tensor, w: torch.Tensor, eps: float, *, M: Optional[int] = None,
                  gather: Optional[torch.Tensor] = None, res: Optional[torch.Tensor] = None,
                  row0: int = 0, want_h: bool = False, want_q: bool = True, want_n: bool = False,
                  want_prep: bool = False, pdl: bool = False, out=None):
    """(gather | residual add) + RMSNorm + (quantise | store).  Returns a dict with the
    requested outputs among h (bf16), q (int8), qp + asum (GEMV-ready int8 + int32 group
    sums), s (fp32 [M,1]), n (bf16).  Buffers passed in `out` are used as they are."""
    dim = x.shape[-1]
    if M is None:
        M = gather.shape[0] if gather is not None else x.shape[0] - row0
    dev = x.device
    out = dict(out) if out else {}
    if want_h and "h" not in out:
        out["h"] = torch.empty((M, dim), dtype=torch.bfloat16, device=dev)
    if want_prep and "qp" not in out:
        out["qp"] = torch.empty((M, dim), dtype=torch.int8, device=dev)
        out["asum"] = torch.empty((M, dim // 128), dtype=torch.int32, device=dev)
    if want_q and "q" not in out and "qp" not in out:
        out["q"] = torch.empty((M, dim), dtype=torch.int8, device=dev)
    if ("q" in out or "qp" in out) and "s" not in out:
        out["s"] = torch.empty((M, 1), dtype=torch.float32, device=dev)
    if want_n and "n" not in out:
        out["n"] = torch.empty((M, dim), dtype=torch.bfloat16, device=dev)
    rc = native.lib().bm_rmsnorm_fused(_ptr(x), _ptr(gather), int(x.shape[0]) if gather is not None else 0, _ptr(res), _ptr(w), float(eps), M, dim,
                                       row0, _ptr(out.get("h")), _ptr(out.get("q")), _ptr(out.get("qp")),
                                       _ptr(out.get("asum")), _ptr(out.get("s")), _ptr(out.get("n")),
                                       int(pdl), _stream(dev))
    check(rc, f"bm_rmsnorm_fused(M={M}, dim={dim})")
    return out


def silu_mul_quant(gu: torch.Tensor, *, want_inner: bool = False, pdl: bool = False, out=None,
                   prep=None):
    """gate|up bf16 [M, 2F] -> INT8 codes of silu(gate)*up + multiplier.  `out` = (q, s)
    buffers (natural order), `prep` = (qp, asum) buffers (GEMV-ready); either or both."""
    _require_cuda(gu)
    M, F2 = gu.shape
    F = F2 // 2
    q = s = None
    if out is not None:
        q, s = out
    elif prep is None:
        q = torch.empty((M, F), dtype=torch.int8, device=gu.device)
    if s is None:
        s = torch.empty((M, 1), dtype=torch.float32, device=gu.device)
    qp, asum = prep if prep is not None else (None, None)
    inner = torch.empty((M, F), dtype=torch.bfloat16, device=gu.device) if want_inner else None
    check(native.lib().bm_silu_mul_quant(_ptr(gu), M, F, _ptr(q), _ptr(qp), _ptr(asum), _ptr(s),
                                         _ptr(inner), int(pdl), _stream(gu.device)), "bm_silu_mul_quant")
    return (q, s, inner) if want_inner else (q, s)


def qknorm_rope_kvappend(xqkv, q_w, k_w, eps, cos_t, sin_t, positions, H, Hkv, k_layer, v_layer,
                         sigma, *, pdl: bool = False, q_out=None):
    """k_layer / v_layer: bf16 [Hkv, kv_rows, 128] views of one layer of the shared buffer."""
    M = xqkv.shape[0]
    kv_rows = k_layer.shape[-2]
    if q_out is None:
        q_out = torch.empty((M, H, 128), dtype=torch.bfloat16, device=xqkv.device)
    rc = native.lib().bm_qknorm_rope_kvappend(
        _ptr(xqkv), _ptr(q_w), _ptr(k_w), float(eps), _ptr(cos_t), _ptr(sin_t), _ptr(positions),
        M, H, Hkv, _ptr(k_layer), _ptr(v_layer), kv_rows, sigma, _ptr(q_out), int(pdl),
        _stream(xqkv.device))
    check(rc, "bm_qknorm_rope_kvappend")
    return q_out


def new_step_state(device) -> torch.Tensor:
    return torch.zeros(4, dtype=torch.int32, device=device)


def set_step_state(state: torch.Tensor, cache_len: int, n_pend: int, role: int, P: int) -> None:
    check(native.lib().bm_set_step_state(_ptr(state), int(cache_len), int(n_pend), int(role), int(P),
                                         _stream(state.device)), "bm_set_step_state")


def kv_copy_rows(kv: torch.Tensor, kv_rows: int, src_row: int, dst_row: int, n: int) -> None:
    """kv: contiguous bf16 buffer whose trailing dims are [kv_rows, 128]."""
    planes = kv.numel() // (kv_rows * 128)
    check(native.lib().bm_kv_copy_rows(_ptr(kv), planes, kv_rows, int(src_row), int(dst_row), int(n),
                                       _stream(kv.device)), "bm_kv_copy_rows")


def attention_scratch(M: int, H: int, sigma: int, device) -> torch.Tensor:
    n = int(native.lib().bm_verify_attention_scratch_bytes(M, H, sigma))
    return torch.zeros((n + 15) // 16 * 16, dtype=torch.uint8, device=device)


def verify_attention(q, k_layer, v_layer, sigma, state, scratch, *, pdl: bool = False, out=None,
                     prep=None):
    """Returns (att bf16 [M, H*128], q int8 [M, H*128] or None, s fp32 [M, 1]).  `prep` =
    (qp, asum) buffers additionally (or, with out[1] None, instead) receive the GEMV-ready
    codes."""
    M, H, _ = q.shape
    Hkv, kv_rows = k_layer.shape[-3], k_layer.shape[-2]
    dev = q.device
    if out is None:
        out = (torch.empty((M, H * 128), dtype=torch.bfloat16, device=dev),
               torch.empty((M, H * 128), dtype=torch.int8, device=dev),
               torch.empty((M, 1), dtype=torch.float32, device=dev))
    qp, asum = prep if prep is not None else (None, None)
    rc = native.lib().bm_verify_attention(_ptr(q), _ptr(k_layer), _ptr(v_layer), M, H, Hkv, kv_rows,
                                          sigma, _ptr(state), _ptr(scratch), _ptr(out[0]),
                                          _ptr(out[1]), _ptr(qp), _ptr(asum), _ptr(out[2]), int(pdl),
                                          _stream(dev))
    check(rc, "bm_verify_attention")
    return out


def logit_scratch(device) -> torch.Tensor:
    """Zeroed scratch for the many-CTA logit reductions (bm_logit_scratch_bytes); one per stream of calls."""
    return torch.zeros(int(native.lib().bm_logit_scratch_bytes()), dtype=torch.uint8, device=device)


def argmax_rows(logits: torch.Tensor, *, out=None, scratch: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Row argmax, lowest index on ties.  With `scratch` (logit_scratch) each row is spread over 16-128 CTAs."""
    rows, vocab = logits.shape
    idx = out if out is not None else torch.empty(rows, dtype=torch.int64, device=logits.device)
    if scratch is not None and rows <= 32:
        check(native.lib().bm_argmax_rows_split(_ptr(logits), rows, vocab, logits.stride(0), _ptr(idx), None,
                                                _ptr(scratch), _stream(logits.device)), "bm_argmax_rows_split")
        return idx
    check(native.lib().bm_argmax_rows(_ptr(logits), rows, vocab, logits.stride(0), _ptr(idx), None,
                                      _stream(logits.device)), "bm_argmax_rows")
    return idx


def draft_chain(logits: torch.Tensor, tau: float, *, bufs=None, scratch: Optional[torch.Tensor] = None):
    """Returns (idx int64 [D], iter_accept int32 [1] (device), conf fp32 [D]).  With `scratch`
    (logit_scratch) a row is reduced by many CTAs: one launch with a 16-CTA cluster per row, or, where the
    device cannot hold the clusters, the argmax and the confidence launch on 16-128 CTAs per row."""
    D, vocab = logits.shape
    dev = logits.device
    if bufs is None:
        bufs = (torch.empty(D, dtype=torch.int64, device=dev), torch.empty(D, device=dev),
                torch.empty(D, device=dev), torch.empty(1, dtype=torch.int32, device=dev))
    idx, mx, conf, n = bufs
    if scratch is not None and D <= 32:
        check(native.lib().bm_draft_chain_split(_ptr(logits), D, vocab, logits.stride(0), float(tau), _ptr(idx),
                                                _ptr(mx), _ptr(conf), _ptr(n), _ptr(scratch), _stream(dev)),
              "bm_draft_chain_split")
        return idx, n, conf
    check(native.lib().bm_draft_chain(_ptr(logits), D, vocab, logits.stride(0), float(tau), _ptr(idx),
                                      _ptr(mx), _ptr(conf), _ptr(n), _stream(dev)), "bm_draft_chain")
    return idx, n, conf


def pack_t2_g128(w: torch.Tensor, *, want_frozen: bool = False):
    """Freeze + pack bf16 weights [N, K] on the device: (packed int8 [N, K/4], scale bf16 [N, K/128]) and, with
    `want_frozen`, the bf16 weights on the ternary grid.  Same bytes as the converter's CPU packer."""
    _require_cuda(w)
    if w.dtype != torch.bfloat16 or w.dim() != 2 or w.shape[1] % 128:
        raise RuntimeError("pack_t2_g128 takes a bf16 [N, K] tensor with K a multiple of 128")
    N, K = w.shape
    packed = torch.empty((N, K // 4), dtype=torch.int8, device=w.device)
    scale = torch.empty((N, K // 128), dtype=torch.bfloat16, device=w.device)
    frozen = torch.empty_like(w) if want_frozen else None
    check(native.lib().bm_pack_t2_g128(_ptr(w), N, K, _ptr(packed), _ptr(scale), _ptr(frozen), _stream(w.device)),
          f"bm_pack_t2_g128(N={N}, K={K})")
    return (packed, scale, frozen) if want_frozen else (packed, scale)


def t2_gemm_wide(a_prep: torch.Tensor, a_sums: torch.Tensor, b_packed: torch.Tensor, s: torch.Tensor, ws: torch.Tensor,
                 *, out: torch.Tensor, pdl: bool = False) -> torch.Tensor:
    """The packed product for many rows (a prompt): out bf16 [T, N], each row what t2_gemv_prepared gives it."""
    T, K = a_prep.shape
    N = b_packed.shape[0]
    rc = native.lib().bm_t2_gemm_wide(_ptr(a_prep), _ptr(a_sums), _ptr(b_packed), _ptr(out), _ptr(s), _ptr(ws), T, N, K,
                                      out.stride(0), int(pdl), _stream(a_prep.device))
    check(rc, f"bm_t2_gemm_wide(T={T}, N={N}, K={K})")
    return out


def prompt_attention_scratch(T: int, hist0: int, slab_rows: int, H: int, Hkv: int, device) -> torch.Tensor:
    n = int(native.lib().bm_prompt_attention_scratch_bytes(T, hist0, slab_rows, H, Hkv))
    if n < 0:
        raise RuntimeError(f"prompt attention does not take T={T}, hist0={hist0}, slab_rows={slab_rows}")
    return torch.zeros((n + 15) // 16 * 16, dtype=torch.uint8, device=device)


def prompt_attention(q: torch.Tensor, k_layer, v_layer, hist0: int, slab_rows: int, scratch: torch.Tensor, *,
                     att: torch.Tensor, amax: torch.Tensor, pdl: bool = False) -> None:
    """Causal attention of T prompt rows whose K / V rows already sit at [hist0, hist0 + T) of the layer's
    planes; q bf16 [T, H, 128] rotated queries.  att bf16 [T, H*128], amax uint32 [T] (zero on entry)."""
    T, H, _ = q.shape
    Hkv, kv_rows = k_layer.shape[-3], k_layer.shape[-2]
    rc = native.lib().bm_prompt_attention(_ptr(q), _ptr(k_layer), _ptr(v_layer), T, int(hist0), int(slab_rows), H, Hkv,
                                          kv_rows, _ptr(scratch), _ptr(att), _ptr(amax), int(pdl), _stream(q.device))
    check(rc, f"bm_prompt_attention(T={T}, hist0={hist0})")


def dense_head(h: torch.Tensor, w: torch.Tensor, *, out: torch.Tensor, w_scale: Optional[torch.Tensor] = None,
               h_scale_out: Optional[torch.Tensor] = None, pdl: bool = False) -> torch.Tensor:
    """Dense draft head: bf16 rows h [R, K] against the bf16 table w [N, K], or against its e4m3 copy
    (w.dtype float8_e4m3fn, `w_scale` the per-tensor fp32 scale).  `out` fp32 [R, >= N] receives the
    bf16-rounded logits."""
    R, K = h.shape
    N = w.shape[0]
    fp8 = w.dtype == torch.float8_e4m3fn
    if not fp8 and w.dtype != torch.bfloat16:
        raise RuntimeError("dense_head: the table must be bf16 or float8_e4m3fn")
    if fp8 and (w_scale is None or w_scale.dtype != torch.float32):
        raise RuntimeError("dense_head: an e4m3 table needs its fp32 per-tensor scale")
    rc = native.lib().bm_dense_head(_ptr(h), _ptr(w), int(fp8), _ptr(w_scale), R, N, K, _ptr(out), out.stride(0),
                                    _ptr(h_scale_out), int(pdl), _stream(h.device))
    check(rc, f"bm_dense_head(R={R}, N={N}, K={K}, fp8={fp8})")
    return out


def verify_accept(draft: torch.Tensor, verify: torch.Tensor, D: int, *, out=None) -> torch.Tensor:
    n = out if out is not None else torch.empty(1, dtype=torch.int32, device=draft.device)
    check(native.lib().bm_verify_accept(_ptr(draft), _ptr(verify), D, _ptr(n), _stream(draft.device)),
          "bm_verify_accept")
    return n


# --------------------------------------------------------------------------- fused SwiGLU
def gate_up_silu(a_prep: torch.Tensor, a_sums: torch.Tensor, w_gu: torch.Tensor, s: torch.Tensor,
                 w_gu_scale: torch.Tensor, *, inner: torch.Tensor, amax: torch.Tensor, pdl: bool = False) -> None:
    """inner[W, F] = bf16(silu(g) * u) straight from the merged gate|up GEMV; amax[W] (uint32 bits, zero
    on entry) collects the row absmax."""
    W, K = a_prep.shape
    F = w_gu.shape[0] // 2
    rc = native.lib().bm_t2_gemv_gate_up_silu(_ptr(a_prep), _ptr(a_sums), _ptr(w_gu), _ptr(w_gu_scale), _ptr(s), W, F,
                                              K, _ptr(inner), _ptr(amax), int(pdl), _stream(a_prep.device))
    check(rc, f"bm_t2_gemv_gate_up_silu(W={W}, F={F}, K={K})")


def quant_rows_amax(x: torch.Tensor, amax: torch.Tensor, *, prep: Tuple[torch.Tensor, torch.Tensor], s: torch.Tensor,
                    amax_zero: Optional[torch.Tensor] = None, q: Optional[torch.Tensor] = None,
                    pdl: bool = False) -> None:
    """INT8 codes of bf16 rows whose absmax bits are in `amax`; clears `amax_zero` for the next producer."""
    M, K = x.shape
    rc = native.lib().bm_quant_rows_amax(_ptr(x), _ptr(amax), _ptr(amax_zero), M, K, _ptr(q), _ptr(prep[0]),
                                         _ptr(prep[1]), _ptr(s), int(pdl), _stream(x.device))
    check(rc, f"bm_quant_rows_amax(M={M}, K={K})")


def rope_verify_attention(xqkv, q_w, k_w, eps, cos_t, sin_t, positions, H, Hkv, k_layer, v_layer, sigma, state,
                          scratch, *, out, prep=None, pdl=False):
    """qknorm_rope_kvappend + verify_attention with the first folded into the attention's chunk kernel.
    `out` = (att or None, q or None, s), `prep` = (qp, asum)."""
    M = xqkv.shape[0]
    kv_rows = k_layer.shape[-2]
    qp, asum = prep if prep is not None else (None, None)
    rc = native.lib().bm_rope_verify_attention(
        _ptr(xqkv), _ptr(q_w), _ptr(k_w), float(eps), _ptr(cos_t), _ptr(sin_t), _ptr(positions), _ptr(k_layer),
        _ptr(v_layer), M, H, Hkv, kv_rows, sigma, _ptr(state), _ptr(scratch), _ptr(out[0]), _ptr(out[1]), _ptr(qp),
        _ptr(asum), _ptr(out[2]), int(pdl), _stream(xqkv.device))
    check(rc, "bm_rope_verify_attention")


def rope_verify_attention_rows(xqkv, q_w, k_w, eps, cos_t, sin_t, positions, H, Hkv, k_layer, v_layer, sigma, state,
                               scratch, *, att, amax, pdl=False):
    """rope_verify_attention without the quantisation: bf16 rows into `att`, row absmax bits into `amax`
    (uint32 [M], zero on entry); follow with quant_rows_amax(att, amax, ...)."""
    M = xqkv.shape[0]
    kv_rows = k_layer.shape[-2]
    rc = native.lib().bm_rope_verify_attention_rows(
        _ptr(xqkv), _ptr(q_w), _ptr(k_w), float(eps), _ptr(cos_t), _ptr(sin_t), _ptr(positions), _ptr(k_layer),
        _ptr(v_layer), M, H, Hkv, kv_rows, sigma, _ptr(state), _ptr(scratch), _ptr(att), _ptr(amax), int(pdl),
        _stream(xqkv.device))
    check(rc, "bm_rope_verify_attention_rows")


def zero_words(t: torch.Tensor) -> None:
    """Stream-ordered clear of a 32-bit tensor (no torch in-place op: workspaces may be inference tensors)."""
    check(native.lib().bm_zero_words(_ptr(t), t.numel(), _stream(t.device)), "bm_zero_words")


def stage_replay_inputs(kind: int, src_a: torch.Tensor, src_b: Optional[torch.Tensor], n_pend: int, cache_len: int,
                        M: int, D: int, mask_id: int, role: int, P: int, tok: torch.Tensor, pos: torch.Tensor,
                        state: torch.Tensor) -> None:
    """Tokens, positions and the step record of one replay in one launch (bm_stage_replay_inputs)."""
    rc = native.lib().bm_stage_replay_inputs(int(kind), _ptr(src_a), _ptr(src_b), int(n_pend), int(cache_len), int(M),
                                             int(D), int(mask_id), int(role), int(P), _ptr(tok), _ptr(pos), _ptr(state),
                                             _stream(tok.device))
    check(rc, "bm_stage_replay_inputs")


def commit_stage_draft(src: torch.Tensor, n_commit: int, verified: bool, gen_dst: torch.Tensor, pending: torch.Tensor,
                       *, stage=None) -> None:
    """Committed ids -> output buffer and pending rows, and (with `stage` = (cache_len, M, D, mask_id, role, P,
    tok, pos, state)) the next draft replay's inputs, in one launch (bm_commit_stage_draft)."""
    if stage is None:
        rc = native.lib().bm_commit_stage_draft(_ptr(src), int(n_commit), int(verified), _ptr(gen_dst), _ptr(pending),
                                                0, 0, 1, 0, 0, 0, 1, None, None, None, _stream(src.device))
    else:
        cache_len, M, D, mask_id, role, P, tok, pos, state = stage
        rc = native.lib().bm_commit_stage_draft(_ptr(src), int(n_commit), int(verified), _ptr(gen_dst), _ptr(pending),
                                                1, int(cache_len), int(M), int(D), int(mask_id), int(role), int(P),
                                                _ptr(tok), _ptr(pos), _ptr(state), _stream(src.device))
    check(rc, "bm_commit_stage_draft")


def gemv_row_fused(src_mode: int, x: torch.Tensor, w: torch.Tensor, ws: torch.Tensor, *, out: torch.Tensor,
                   gather: Optional[torch.Tensor] = None, res: Optional[torch.Tensor] = None,
                   norm_w: Optional[torch.Tensor] = None, eps: float = 0.0, h_out: Optional[torch.Tensor] = None,
                   amax_in: Optional[torch.Tensor] = None, amax_zero: Optional[torch.Tensor] = None, silu: bool = False,
                   amax_out: Optional[torch.Tensor] = None, out_kind: int = native.OUT_BF16, pdl: bool = False) -> None:
    """Width-1 GEMV that quantises its own bf16 input row (bm_t2_gemv_row_fused): src_mode 1 = row with known
    absmax, 2 = (gather | add) + RMSNorm; `silu`: merged gate|up weights with the SiLU epilogue."""
    K = w.shape[1] * 4
    N = w.shape[0] // 2 if silu else w.shape[0]
    rc = native.lib().bm_t2_gemv_row_fused(
        int(src_mode), _ptr(x), _ptr(gather), int(x.shape[0]) if gather is not None else 0, _ptr(res), _ptr(norm_w), float(eps), _ptr(h_out), _ptr(amax_in),
        _ptr(amax_zero), _ptr(w), _ptr(ws), N, K, _ptr(out), out.shape[-1], int(out_kind), int(silu), _ptr(amax_out),
        int(pdl), _stream(x.device))
    check(rc, f"bm_t2_gemv_row_fused(mode={src_mode}, N={N}, K={K})")
