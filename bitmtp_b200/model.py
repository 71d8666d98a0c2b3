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
import math
import os
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


# ===========================================================================
# Modules (same tree and state-dict keys as the reference, model.py:274-304, 607-656,
# 689-760, 1015-1076, 1143-1166)
# ===========================================================================
@dataclass
class ModelArgs:
    """Bonsai-1.7B (Qwen3) defaults, same fields as the reference (model.py:689-713)."""
    dim: int = 2048
    n_layers: int = 28
    n_heads: int = 16
    n_kv_heads: int = 8
    head_dim: int = 128
    ffn_dim: int = 6144
    vocab_size: int = 151669
    norm_eps: float = 1.0e-6
    rope_theta: float = 1.0e6
    rope_original_max: int = 8192
    rope_factor: float = 4.0
    rope_mscale: float = 1.0
    rope_mscale_all_dim: float = 0.0
    rope_beta_fast: float = 32.0
    rope_beta_slow: float = 1.0
    tie_word_embeddings: bool = True
    use_kernel: bool = True
    kernel_kind: str = "t2g128"
    block_size: int = 8
    causal_attn: bool = True
    mask_token_id: int = 151654


class RMSNorm(nn.Module):
    """RMSNorm weight holder; `forward` runs the native kernel (bf16 rows in, bf16 rows out)."""

    def __init__(self, hidden_size: int, eps: float = 1e-6):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden_size), requires_grad=False)
        self.eps = eps

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        out = ops.rmsnorm_fused(x2, self.weight.data, self.eps, want_q=False, want_n=True)
        return out["n"].reshape(x.shape)

    def forward_and_quant(self, x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        out = ops.rmsnorm_fused(x.contiguous(), self.weight.data, self.eps)
        return out["q"], out["s"]


class T2LinearKernel(nn.Module):
    """Q2_0_g128 W2A8 linear: `weight` int8 [out, in/4] (four natural-order ternary codes
    per byte, 1/2/3 = -1/0/+1), `weight_scale` bf16 [out, in/128] (model.py:607-630)."""

    MAX_ROWS = 16

    def __init__(self, in_features: int, out_features: int, bias: bool = False):
        super().__init__()
        assert bias is False
        assert in_features % 128 == 0
        self.in_features = in_features
        self.out_features = out_features
        self.weight = nn.Parameter(torch.zeros(out_features, in_features // 4, dtype=torch.int8),
                                   requires_grad=False)
        self.register_buffer("weight_scale",
                             torch.zeros(out_features, in_features // 128, dtype=torch.bfloat16),
                             persistent=True)

    def quant_input(self, x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """Per-token absmax INT8 quantisation (model.py:632-636)."""
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        q, s = ops.quant_rows(x2)
        return q.reshape(x.shape), s.reshape(*x.shape[:-1], 1)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """Any number of rows: the native kernel takes up to 32 at a time, so long inputs
        (prefill) go through it in slabs.  The reference falls back to a dense bf16 GEMM
        on unpacked weights for unregistered widths (model.py:650-656); the integer path
        gives the same quantised product without the bf16 roundings and without the dense
        copy of the weights."""
        x2 = x.reshape(-1, self.in_features).contiguous()
        q, s = ops.quant_rows(x2)
        out = torch.empty((x2.shape[0], self.out_features), dtype=torch.bfloat16, device=x.device)
        for r0 in range(0, x2.shape[0], self.MAX_ROWS):
            r1 = min(r0 + self.MAX_ROWS, x2.shape[0])
            ops.t2_gemv(q[r0:r1], self.weight.data, s[r0:r1], self.weight_scale, out=out[r0:r1],
                        ldc=self.out_features)
        return out.reshape(*x.shape[:-1], self.out_features)


def _yarn_inv_freq(head_dim: int, base: float, factor: float, original_max: int,
                   beta_fast: float = 32.0, beta_slow: float = 1.0) -> torch.Tensor:
    """YaRN inverse frequencies, computed on the CPU in the reference's operation order
    (model.py:342-368) so that the bf16 tables are the same bits everywhere."""
    dim = head_dim
    pos_freqs = base ** (torch.arange(0, dim, 2).float() / dim)
    extrap = 1.0 / pos_freqs
    interp = 1.0 / (factor * pos_freqs)

    def correction(num_rotations: float) -> float:
        return (dim * math.log(original_max / (num_rotations * 2 * math.pi))) / (2 * math.log(base))

    low = max(math.floor(correction(beta_fast)), 0)
    high = min(math.ceil(correction(beta_slow)), dim - 1)
    if low == high:
        high += 0.001
    ramp = torch.clamp((torch.arange(dim // 2, dtype=torch.float32) - low) / (high - low), 0.0, 1.0)
    keep = 1.0 - ramp
    return interp * (1.0 - keep) + extrap * keep


def _yarn_attention_factor(scale: float, mscale: float = 1.0, mscale_all_dim: float = 0.0) -> float:
    """cos/sin post-scaling (model.py:371-379)."""
    if scale <= 1.0:
        return 1.0

    def g(s, m):
        return 0.1 * m * math.log(s) + 1.0
    if mscale and mscale_all_dim:
        return g(scale, mscale) / g(scale, mscale_all_dim)
    return g(scale, mscale)


class Attention(nn.Module):
    def __init__(self, args: ModelArgs):
        super().__init__()
        self.args = args
        self.head_dim = args.head_dim
        self.n_local_heads = args.n_heads
        self.n_local_kv_heads = args.n_kv_heads
        self.heads_per_group = args.n_heads // args.n_kv_heads
        self.q_dim = args.n_heads * args.head_dim
        self.k_dim = args.n_kv_heads * args.head_dim
        self.v_dim = self.k_dim
        self.q_proj = T2LinearKernel(args.dim, self.q_dim)
        self.k_proj = T2LinearKernel(args.dim, self.k_dim)
        self.v_proj = T2LinearKernel(args.dim, self.v_dim)
        self.o_proj = T2LinearKernel(self.q_dim, args.dim)
        self.q_norm = RMSNorm(self.head_dim, eps=args.norm_eps)
        self.k_norm = RMSNorm(self.head_dim, eps=args.norm_eps)
        self.register_buffer("inv_freq", _yarn_inv_freq(
            self.head_dim, args.rope_theta, args.rope_factor, args.rope_original_max,
            args.rope_beta_fast, args.rope_beta_slow), persistent=False)
        self.rope_mscale = _yarn_attention_factor(args.rope_factor, args.rope_mscale,
                                                  args.rope_mscale_all_dim)

    def prepare_merged_weights(self, max_positions: int = 256, tables=None) -> None:
        """Concatenate q|k|v rows and scales; build the bf16 RoPE tables (model.py:931-956).
        The tables are computed on the CPU and copied over, and shared between layers."""
        dev = self.q_proj.weight.device
        self.wqkv_weight = torch.cat([self.q_proj.weight.data, self.k_proj.weight.data,
                                      self.v_proj.weight.data], dim=0).contiguous()
        self.wqkv_scale = torch.cat([self.q_proj.weight_scale.data, self.k_proj.weight_scale.data,
                                     self.v_proj.weight_scale.data], dim=0).contiguous()
        self._qkv_split = [self.q_dim, self.k_dim, self.v_dim]
        if tables is None:
            tables = rope_tables(self.inv_freq.detach().float().cpu(), self.rope_mscale, max_positions)
            tables = (tables[0].to(dev), tables[1].to(dev))
        self.rope_cos, self.rope_sin = tables
        self._attn_scale = 1.0 / math.sqrt(self.head_dim)


def rope_tables(inv_freq_cpu: torch.Tensor, mscale: float, max_positions: int):
    """bf16 cos/sin tables [max_positions, head_dim] (model.py:950-955), on the CPU.  The
    inverse frequencies are rounded to bf16 first: the reference casts the whole module,
    this buffer included, to bf16 when it builds the model (generate.py:50)."""
    inv_freq_cpu = inv_freq_cpu.to(torch.bfloat16).float()
    pos = torch.arange(max_positions, dtype=torch.float32)
    freqs = torch.outer(pos, inv_freq_cpu)
    emb = torch.cat((freqs, freqs), dim=-1)
    return (emb.cos() * mscale).to(torch.bfloat16), (emb.sin() * mscale).to(torch.bfloat16)


class FeedForward(nn.Module):
    def __init__(self, args: ModelArgs):
        super().__init__()
        self.gate_proj = T2LinearKernel(args.dim, args.ffn_dim)
        self.up_proj = T2LinearKernel(args.dim, args.ffn_dim)
        self.down_proj = T2LinearKernel(args.ffn_dim, args.dim)

    def prepare_merged_weights(self) -> None:
        """gate|up by output row (model.py:1042-1051)."""
        self.w_gu = torch.cat([self.gate_proj.weight.data, self.up_proj.weight.data], dim=0).contiguous()
        self.w_gu_scale = torch.cat([self.gate_proj.weight_scale.data,
                                     self.up_proj.weight_scale.data], dim=0).contiguous()
        self._gu_split = [self.gate_proj.out_features, self.up_proj.out_features]


class TransformerBlock(nn.Module):
    def __init__(self, args: ModelArgs):
        super().__init__()
        self.attention = Attention(args)
        self.feed_forward = FeedForward(args)
        self.input_layernorm = RMSNorm(args.dim, eps=args.norm_eps)
        self.post_attention_layernorm = RMSNorm(args.dim, eps=args.norm_eps)


# ===========================================================================
# Transformer: the captured forward
# ===========================================================================
class StepWorkspace:
    """Every intermediate of one replay width M, allocated once.  A captured graph bakes
    these addresses in; graphs of the same width share one workspace because replays on
    a stream never overlap."""

    def __init__(self, args: ModelArgs, M: int, n_pad: int, device):
        bf, i8, f32 = torch.bfloat16, torch.int8, torch.float32
        q_dim = args.n_heads * args.head_dim
        qkv = q_dim + 2 * args.n_kv_heads * args.head_dim

        def buf(shape, dtype):
            return torch.empty(shape, dtype=dtype, device=device)

        self.M = M
        self.h = buf((M, args.dim), bf)
        self.q = buf((M, args.dim), i8)
        self.s = buf((M, 1), f32)
        self.xqkv = buf((M, qkv), bf)
        self.qrot = buf((M, args.n_heads, args.head_dim), bf)
        self.att = buf((M, q_dim), bf)
        self.att_q = buf((M, q_dim), i8)
        self.att_s = buf((M, 1), f32)
        self.attn_out = buf((M, args.dim), bf)
        self.gu = buf((M, 2 * args.ffn_dim), bf)
        self.iq = buf((M, args.ffn_dim), i8)
        self.is_ = buf((M, 1), f32)
        self.ffn_out = buf((M, args.dim), bf)
        self.hq = buf((M, args.dim), i8)
        self.hs = buf((M, 1), f32)
        self.hn = buf((M, args.dim), bf)            # normed logit rows of the dense draft heads
        # per-128-group sums that travel with the GEMV-ready codes in q / att_q / iq / hq
        i32 = torch.int32
        self.q_sum = buf((M, args.dim // 128), i32)
        self.att_sum = buf((M, q_dim // 128), i32)
        self.i_sum = buf((M, args.ffn_dim // 128), i32)
        self.h_sum = buf((M, args.dim // 128), i32)
        self.inner = buf((M, args.ffn_dim), bf)
        self.inner_amax = torch.zeros((2, M), dtype=i32, device=device)   # row absmax bits, two slots used in turn
        self.att_amax = torch.zeros((2, M), dtype=i32, device=device)
        self.h2 = buf((M, args.dim), bf)            # second residual buffer of the width-1 fused path
        self.n_pad = n_pad


class Transformer(nn.Module):
    def __init__(self, args: ModelArgs):
        super().__init__()
        self.args = args
        self.embed_tokens = nn.Embedding(args.vocab_size, args.dim)
        self.layers = nn.ModuleList([TransformerBlock(args) for _ in range(args.n_layers)])
        self.norm = RMSNorm(args.dim, eps=args.norm_eps)
        if not args.tie_word_embeddings:
            raise NotImplementedError("only tied-embedding T2 checkpoints are in scope")
        self._lm_head_weight_ref = None
        self._lm_head_t2_w = None
        # prompt waves of a shape seen before are replayed as CUDA graphs (BM_PROMPT_GRAPHS=0: always eager)
        self.use_prompt_graphs = os.environ.get("BM_PROMPT_GRAPHS", "1") != "0"
        self._workspaces = {}
        # Programmatic dependent launch between the kernels of a replay: every kernel lets its
        # successor start early (GEMVs then request their weight tiles while the predecessor
        # is still running) and waits for its predecessor before touching activations.
        self.use_pdl = os.environ.get("BM_PDL", "1") != "0"
        # SiLU(gate) * up inside the gate|up GEMV + a flat quantisation kernel instead of GEMV + one SiLU
        # CTA per row (BM_FUSED_FFN=0 restores the latter)
        self.fused_ffn = os.environ.get("BM_FUSED_FFN", "1") != "0"
        # q/k norm + RoPE + KV append folded into the attention kernel (BM_FUSED_ROPE=0: own launch)
        self.fused_rope = os.environ.get("BM_FUSED_ROPE", "1") != "0"
        # width-1 replays: RMSNorm / quantisation inside the consuming GEMV, 6 launches per layer instead
        # of 10 (BM_FUSED_AR=0: the general sequence)
        self.fused_ar = os.environ.get("BM_FUSED_AR", "1") != "0"

    def tie_weights(self) -> None:
        # plain attribute, not a registered parameter: the state dict keeps the reference's keys
        object.__setattr__(self, "_lm_head_weight_ref", self.embed_tokens.weight)

    def _lm_head_weight(self) -> torch.Tensor:
        w = self._lm_head_weight_ref
        return self.embed_tokens.weight if w is None else w

    @torch.no_grad()
    def prepare_t2_lm_head(self) -> None:
        """Pack the tied head on its exact Q2_0_g128 grid (model.py:1223-1243).  The
        reference pads to its one registered head size (151936 rows); here the row count is
        padded to a multiple of 32, which is that same number for the real vocabularies."""
        if self._lm_head_t2_w is not None:
            return
        from .synthetic import pack_t2_g128
        W = self._lm_head_weight().data.to(torch.bfloat16)
        vocab, dim = W.shape
        n_pad = (vocab + 31) // 32 * 32
        dev = W.device
        # packed in slabs on the CPU: the converter's packer is CPU code and the dense
        # fp32 view of the whole table would not be worth its 1.2 GB on the device
        Wc = W.cpu()
        packed = torch.zeros(n_pad, dim // 4, dtype=torch.int8)
        scale = torch.zeros(n_pad, dim // 128, dtype=torch.bfloat16)
        for r0 in range(0, vocab, 16384):
            r1 = min(r0 + 16384, vocab)
            p, s = pack_t2_g128(Wc[r0:r1].contiguous())
            packed[r0:r1], scale[r0:r1] = p, s
        # pad rows keep code bytes 0 and scale 0: their logits are 0 * anything = 0 and are
        # sliced off before any argmax
        self._lm_head_t2_w = packed.to(dev)
        self._lm_head_t2_scale = scale.to(dev)
        self._lm_head_t2_vocab = vocab
        self._lm_head_n_pad = n_pad

    @torch.no_grad()
    def prepare_fp8_lm_head(self) -> None:
        """Per-tensor e4m3 copy of the tied head for the `draft_fp8` role (model.py:1169-1194): rows padded
        to a multiple of 16, w_scale = bf16(amax|W| / 448) kept as an fp32 device scalar, table =
        (W / w_scale) cast to e4m3.  A one-time conversion at load; the per-step work is bm_dense_head."""
        if getattr(self, "_lm_head_fp8_w", None) is not None:
            return
        fp8_max = torch.finfo(torch.float8_e4m3fn).max
        W = self._lm_head_weight().data
        vocab, dim = W.shape
        vocab_pad = (vocab + 15) // 16 * 16
        Wp = W
        if vocab_pad != vocab:
            Wp = torch.zeros(vocab_pad, dim, dtype=W.dtype, device=W.device)
            Wp[:vocab].copy_(W)
        w_scale = (Wp.abs().amax() / fp8_max).clamp_min(1e-12).to(torch.float32)
        out = torch.empty(vocab_pad, dim, dtype=torch.float8_e4m3fn, device=W.device)
        for r0 in range(0, vocab_pad, 16384):          # in slabs: no second full-size temporary
            out[r0:r0 + 16384] = (Wp[r0:r0 + 16384] / w_scale).to(torch.float8_e4m3fn)
        self._lm_head_fp8_w = out
        self._lm_head_w_scale = w_scale.reshape(1).contiguous()
        self._lm_head_fp8_max = fp8_max
        self._lm_head_vocab = vocab

    @torch.no_grad()
    def prepare_bf16_lm_head(self) -> None:
        """Table of the `draft_bf16` role (model.py:1276-1282): the tied bf16 embedding itself; a zero-padded
        copy only when the vocabulary is not a multiple of 16 rows."""
        if getattr(self, "_lm_head_bf16_w", None) is not None:
            return
        W = self._lm_head_weight().data
        vocab, dim = W.shape
        if vocab % 16 == 0 and W.is_contiguous():
            self._lm_head_bf16_w = W
        else:
            Wp = torch.zeros((vocab + 15) // 16 * 16, dim, dtype=W.dtype, device=W.device)
            Wp[:vocab].copy_(W)
            self._lm_head_bf16_w = Wp
        self._lm_head_vocab = vocab

    def prepare_merged_weights(self, max_positions: int = 256) -> None:
        """model.py:1444-1447; the RoPE tables are built once and shared by all layers."""
        dev = self.embed_tokens.weight.device
        a0 = self.layers[0].attention
        cos, sin = rope_tables(a0.inv_freq.detach().float().cpu(), a0.rope_mscale, max_positions)
        tables = (cos.to(dev), sin.to(dev))
        for layer in self.layers:
            layer.attention.prepare_merged_weights(max_positions, tables=tables)
            layer.feed_forward.prepare_merged_weights()
        self.max_positions = max_positions

    def _ar_fused_supported(self, M: int) -> bool:
        a = self.args
        return (self.fused_ar and M == 1 and a.dim == 2048 and a.n_heads % 4 == 0 and a.head_dim == 128
                and (a.n_heads * a.head_dim) % 256 == 0 and a.ffn_dim % 256 == 0)

    def _layers_ar_fused(self, W, token_values, positions, kv_full, kv_rows, sigma, attn_mask, attn_scratch,
                         pdl, attn_pdl) -> None:
        """Width-1 layer stack in six launches per layer: each projection quantises (and, for qkv and
        gate|up, normalises) its own input row.  The residual stream alternates between W.h2 and W.h and
        ends in W.h, where the final norm expects it."""
        a = self.args
        eps = a.norm_eps
        ops.zero_words(W.inner_amax[0])
        ops.zero_words(W.att_amax[0])
        for i, layer in enumerate(self.layers):
            at, ff = layer.attention, layer.feed_forward
            k_l, v_l = kv_full[i]
            if i == 0:
                ops.gemv_row_fused(2, self.embed_tokens.weight.data, at.wqkv_weight, at.wqkv_scale, out=W.xqkv,
                                   gather=token_values, norm_w=layer.input_layernorm.weight.data, eps=eps,
                                   h_out=W.h2, pdl=pdl)
            else:
                ops.gemv_row_fused(2, W.ffn_out, at.wqkv_weight, at.wqkv_scale, out=W.xqkv, res=W.h,
                                   norm_w=layer.input_layernorm.weight.data, eps=eps, h_out=W.h2, pdl=pdl)
            ops.rope_verify_attention_rows(W.xqkv, at.q_norm.weight.data, at.k_norm.weight.data, eps, at.rope_cos,
                                           at.rope_sin, positions, a.n_heads, a.n_kv_heads,
                                           _LayerView(k_l, kv_rows), _LayerView(v_l, kv_rows), sigma, attn_mask,
                                           attn_scratch, att=W.att, amax=W.att_amax[i & 1], pdl=attn_pdl)
            ops.gemv_row_fused(1, W.att, at.o_proj.weight.data, at.o_proj.weight_scale, out=W.attn_out,
                               amax_in=W.att_amax[i & 1], amax_zero=W.att_amax[(i + 1) & 1], pdl=pdl)
            ops.gemv_row_fused(2, W.h2, ff.w_gu, ff.w_gu_scale, out=W.inner, res=W.attn_out,
                               norm_w=layer.post_attention_layernorm.weight.data, eps=eps, h_out=W.h, silu=True,
                               amax_out=W.inner_amax[i & 1], pdl=pdl)
            ops.gemv_row_fused(1, W.inner, ff.down_proj.weight.data, ff.down_proj.weight_scale, out=W.ffn_out,
                               amax_in=W.inner_amax[i & 1], amax_zero=W.inner_amax[(i + 1) & 1], pdl=pdl)

    def _layers_by_operator(self, W, token_values, positions, kv_full, kv_rows, sigma, attn_mask, attn_scratch,
                            pdl, attn_pdl) -> None:
        """The layer stack as ten launches per layer (every geometry, every width)."""
        a = self.args
        M = W.M
        eps = a.norm_eps
        L0 = self.layers[0]
        # INT8 activations go from their producer to the next GEMV in GEMV-ready order
        # (16-runs transposed 4x4, plus per-group sums), so no GEMV CTA permutes or sums them.
        qsink = {"h": W.h, "qp": W.q, "asum": W.q_sum, "s": W.s}
        fused_ffn = self.fused_ffn and M <= 16 and a.ffn_dim % 16 == 0 and a.dim % 256 == 0
        if fused_ffn:
            ops.zero_words(W.inner_amax[0])           # slot of layer 0; every layer clears the next one's
        if self.fused_rope:
            ops.zero_words(W.att_amax[0])
        ops.rmsnorm_fused(self.embed_tokens.weight.data, L0.input_layernorm.weight.data, eps, M=M,
                          gather=token_values, pdl=pdl, out=qsink)
        for i, layer in enumerate(self.layers):
            at, ff = layer.attention, layer.feed_forward
            if i > 0:
                ops.rmsnorm_fused(W.ffn_out, layer.input_layernorm.weight.data, eps, M=M, res=W.h,
                                  pdl=pdl, out=qsink)
            ops.t2_gemv_prepared(W.q, W.q_sum, at.wqkv_weight, W.s, at.wqkv_scale, out=W.xqkv,
                                 ldc=W.xqkv.shape[1], pdl=pdl)
            k_l, v_l = kv_full[i]
            if self.fused_rope:
                # one attention launch (q/k norm, RoPE and KV append folded in; the last CTA of a query group
                # merges the split-KV partials and gathers the row absmax by atomic max), then the INT8 codes
                # from the flat quantisation kernel
                ops.rope_verify_attention_rows(W.xqkv, at.q_norm.weight.data, at.k_norm.weight.data, eps,
                                               at.rope_cos, at.rope_sin, positions, a.n_heads, a.n_kv_heads,
                                               _LayerView(k_l, kv_rows), _LayerView(v_l, kv_rows), sigma, attn_mask,
                                               attn_scratch, att=W.att, amax=W.att_amax[i & 1], pdl=attn_pdl)
                ops.quant_rows_amax(W.att, W.att_amax[i & 1], prep=(W.att_q, W.att_sum), s=W.att_s,
                                    amax_zero=W.att_amax[(i + 1) & 1], pdl=pdl)
            else:
                ops.qknorm_rope_kvappend(W.xqkv, at.q_norm.weight.data, at.k_norm.weight.data, eps,
                                         at.rope_cos, at.rope_sin, positions, a.n_heads, a.n_kv_heads,
                                         _LayerView(k_l, kv_rows), _LayerView(v_l, kv_rows), sigma,
                                         pdl=pdl, q_out=W.qrot)
                ops.verify_attention(W.qrot, _LayerView(k_l, kv_rows), _LayerView(v_l, kv_rows), sigma,
                                     attn_mask, attn_scratch, pdl=attn_pdl, out=(None, None, W.att_s),
                                     prep=(W.att_q, W.att_sum))
            ops.t2_gemv_prepared(W.att_q, W.att_sum, at.o_proj.weight.data, W.att_s,
                                 at.o_proj.weight_scale, out=W.attn_out, ldc=a.dim, pdl=pdl)
            ops.rmsnorm_fused(W.h, layer.post_attention_layernorm.weight.data, eps, M=M,
                              res=W.attn_out, pdl=pdl, out=qsink)
            if fused_ffn:
                # SiLU(gate) * up in the GEMV epilogue (the row absmax gathered by atomic max), then
                # the INT8 codes from a flat grid: the work of the one-CTA-per-row SiLU kernel spread
                # over all SMs
                ops.gate_up_silu(W.q, W.q_sum, ff.w_gu, W.s, ff.w_gu_scale, inner=W.inner,
                                 amax=W.inner_amax[i & 1], pdl=pdl)
                ops.quant_rows_amax(W.inner, W.inner_amax[i & 1], prep=(W.iq, W.i_sum), s=W.is_,
                                    amax_zero=W.inner_amax[(i + 1) & 1], pdl=pdl)
            else:
                ops.t2_gemv_prepared(W.q, W.q_sum, ff.w_gu, W.s, ff.w_gu_scale, out=W.gu,
                                     ldc=W.gu.shape[1], pdl=pdl)
                ops.silu_mul_quant(W.gu, pdl=pdl, out=(None, W.is_), prep=(W.iq, W.i_sum))
            ops.t2_gemv_prepared(W.iq, W.i_sum, ff.down_proj.weight.data, W.is_,
                                 ff.down_proj.weight_scale, out=W.ffn_out, ldc=a.dim, pdl=pdl)

    def workspace(self, M: int) -> StepWorkspace:
        ws = self._workspaces.get(M)
        if ws is None:
            self.prepare_t2_lm_head()
            ws = StepWorkspace(self.args, M, self._lm_head_n_pad, self.embed_tokens.weight.device)
            self._workspaces[M] = ws
        return ws

    @torch.no_grad()
    def forward_sdlm_decode_graph_kernel(
        self,
        token_values: torch.Tensor,      # int64 [M]
        positions: torch.Tensor,         # int64 [M]
        kv_full: List[SDLMLayerCache],   # per layer (k, v) views [1, n_kv, sigma+M, head_dim]
        block_size: int,                 # M (replay width)
        attn_mask: torch.Tensor,         # int32 [4] step state (see below)
        logits_start: int = 0,
        logits_end: int = -1,
        lm_head_precision: str = "t2",
        *,
        attn_scratch: Optional[torch.Tensor] = None,
        logits_buf: Optional[torch.Tensor] = None,
        stable_state: bool = False,
    ) -> torch.Tensor:
        """The replay body (reference: model.py:1363-1404, 1119-1137, 958-1009, 1053-1064).

        Same arguments as the reference with one change of meaning: `attn_mask` is not an
        additive [1,1,M,sigma+M] tensor but the 16-byte device record
        {cache_len, n_pend, role, P} written by `ops.set_step_state`; the attention kernel
        derives the same visibility from it.  K and V rows of this replay are written in
        place at rows [sigma, sigma+M) of every layer's views.  Returns fp32 logits
        [logits_end - logits_start, vocab] holding bf16-rounded values, as the reference's
        `.float()` of a bf16 head output does.

        `stable_state`: the caller guarantees that `attn_mask` and the history rows were
        written by launches that finished before this forward's first launch (a captured
        replay); the attention then reads them without waiting for the preceding kernel.
        """
        if lm_head_precision not in ("t2", "fp8", "bf16_raw"):
            raise RuntimeError(f"unsupported lm_head precision: {lm_head_precision!r}")
        a = self.args
        M = int(block_size)
        if logits_end == -1:
            logits_end = M
        rows = logits_end - logits_start
        W = self.workspace(M)
        pdl = self.use_pdl
        attn_pdl = (native.PDL_OVERLAP | native.PDL_STABLE_STATE) if (pdl and stable_state) else int(pdl)
        k0 = kv_full[0][0]
        kv_rows = k0.stride(-3) // a.head_dim
        sigma = k0.shape[-2] - M
        dev = token_values.device
        if attn_scratch is None:
            attn_scratch = ops.attention_scratch(M, a.n_heads, sigma, dev)
        if logits_buf is None:
            logits_buf = torch.empty((rows, W.n_pad), dtype=torch.float32, device=dev)
        eps = a.norm_eps
        if self._ar_fused_supported(M) and token_values.is_contiguous() and positions.is_contiguous():
            self._layers_ar_fused(W, token_values, positions, kv_full, kv_rows, sigma, attn_mask, attn_scratch,
                                  pdl, attn_pdl)
        else:
            self._layers_by_operator(W, token_values, positions, kv_full, kv_rows, sigma, attn_mask, attn_scratch,
                                     pdl, attn_pdl)
        if rows == 0:
            # layers only: the caller takes the logit rows it wants with head_from_workspace
            return logits_buf[:, : self._lm_head_t2_vocab]
        return self.head_from_workspace(M, logits_start, rows, logits_buf, lm_head_precision)

    def head_from_workspace(self, M: int, row0: int, rows: int, logits_buf: torch.Tensor,
                            precision: str = "t2") -> torch.Tensor:
        """Final norm and head over rows [row0, row0 + rows) of the width-M workspace as the layer loop
        left it: h + ffn_out, RMSNorm, then by `precision` (reference: model.py:1402-1404, 1245-1296)
          t2        INT8 quantisation + the packed T2 head
          fp8       the e4m3 copy of the tied table with per-tensor scales (prepare_fp8_lm_head)
          bf16_raw  the bf16 tied table itself
        Returns fp32 logits [rows, vocab]."""
        W = self.workspace(M)
        pdl = self.use_pdl
        if precision in ("fp8", "bf16_raw"):
            ops.rmsnorm_fused(W.h, self.norm.weight.data, self.args.norm_eps, M=rows, res=W.ffn_out, row0=row0,
                              pdl=pdl, want_q=False, out={"n": W.hn})
            if precision == "fp8":
                self.prepare_fp8_lm_head()
                ops.dense_head(W.hn[:rows], self._lm_head_fp8_w, out=logits_buf, w_scale=self._lm_head_w_scale, pdl=pdl)
            else:
                self.prepare_bf16_lm_head()
                ops.dense_head(W.hn[:rows], self._lm_head_bf16_w, out=logits_buf, pdl=pdl)
            return logits_buf[:, : self._lm_head_vocab]
        ops.rmsnorm_fused(W.h, self.norm.weight.data, self.args.norm_eps, M=rows, res=W.ffn_out, row0=row0,
                          pdl=pdl, out={"qp": W.hq, "asum": W.h_sum, "s": W.hs})
        ops.t2_gemv_prepared(W.hq[:rows], W.h_sum[:rows], self._lm_head_t2_w, W.hs[:rows],
                             self._lm_head_t2_scale, out_kind=native.OUT_F32_OF_BF16, out=logits_buf,
                             ldc=W.n_pad, pdl=pdl)
        return logits_buf[:, : self._lm_head_t2_vocab]

    def wide_prefill_supported(self) -> bool:
        """The many-row prompt path needs every projection's row count to be a multiple of 128 and the
        flat quantisation's K % 256 == 0; every released geometry and the test geometries have both."""
        a = self.args
        q_dim, kv_dim = a.n_heads * a.head_dim, a.n_kv_heads * a.head_dim
        return (all(n % 128 == 0 for n in (q_dim + 2 * kv_dim, a.dim, 2 * a.ffn_dim)) and q_dim % 256 == 0
                and a.dim % 256 == 0 and a.ffn_dim % 128 == 0 and os.environ.get("BM_WIDE_PREFILL", "1") != "0")

    @torch.no_grad()
    def prefill_rows_wide(self, token_values: torch.Tensor, positions: torch.Tensor, kv_planes: List[SDLMLayerCache],
                          kv_rows: int, hist0: int, ws: "PromptWorkspace", scratch: torch.Tensor) -> None:
        """One wave of the prompt forward on the many-row kernels: T = len(token_values) rows at positions
        hist0 .. hist0 + T - 1, whose K / V rows are written in place at rows [hist0, hist0 + T) of every
        layer's planes (`kv_planes[i]` = (k, v) [1, n_kv, kv_rows, hd]); rows [0, hist0) are history.
        Same arithmetic, row for row, as the slab-by-slab prefill (forward_sdlm_prefill), so K / V rows and
        the residual stream equal it bit for bit: every projection is bm_t2_gemm_wide (tensor cores, each
        weight byte read once per 32 rows), the attention one launch over AR-causal slabs of PREFILL_CHUNK
        rows.  Leaves the residual stream in ws.h / ws.ffn_out (reference: model.py:1306-1340)."""
        a = self.args
        T = int(token_values.shape[0])
        eps, pdl = a.norm_eps, self.use_pdl
        pos = positions
        L0 = self.layers[0]
        h, q, q_sum, s = ws.h[:T], ws.q[:T], ws.q_sum[:T], ws.s[:T]
        qsink = {"h": h, "qp": q, "asum": q_sum, "s": s}
        ops.zero_words(ws.att_amax[0])
        ops.rmsnorm_fused(self.embed_tokens.weight.data, L0.input_layernorm.weight.data, eps, M=T,
                          gather=token_values, pdl=pdl, out=qsink)
        for i, layer in enumerate(self.layers):
            at, ff = layer.attention, layer.feed_forward
            if i > 0:
                ops.rmsnorm_fused(ws.ffn_out[:T], layer.input_layernorm.weight.data, eps, M=T, res=h, pdl=pdl, out=qsink)
            ops.t2_gemm_wide(q, q_sum, at.wqkv_weight, s, at.wqkv_scale, out=ws.xqkv[:T], pdl=pdl)
            k_l, v_l = kv_planes[i]
            kl, vl = _LayerView(k_l, kv_rows), _LayerView(v_l, kv_rows)
            ops.qknorm_rope_kvappend(ws.xqkv[:T], at.q_norm.weight.data, at.k_norm.weight.data, eps, at.rope_cos,
                                     at.rope_sin, pos, a.n_heads, a.n_kv_heads, kl, vl, hist0, pdl=pdl, q_out=ws.qrot[:T])
            ops.prompt_attention(ws.qrot[:T], kl, vl, hist0, PREFILL_CHUNK, scratch, att=ws.att[:T],
                                 amax=ws.att_amax[i & 1][:T], pdl=pdl)
            ops.quant_rows_amax(ws.att[:T], ws.att_amax[i & 1][:T], prep=(ws.att_q[:T], ws.att_sum[:T]), s=ws.att_s[:T],
                                amax_zero=ws.att_amax[(i + 1) & 1][:T], pdl=pdl)
            ops.t2_gemm_wide(ws.att_q[:T], ws.att_sum[:T], at.o_proj.weight.data, ws.att_s[:T], at.o_proj.weight_scale,
                             out=ws.attn_out[:T], pdl=pdl)
            ops.rmsnorm_fused(h, layer.post_attention_layernorm.weight.data, eps, M=T, res=ws.attn_out[:T], pdl=pdl,
                              out=qsink)
            ops.t2_gemm_wide(q, q_sum, ff.w_gu, s, ff.w_gu_scale, out=ws.gu[:T], pdl=pdl)
            ops.silu_mul_quant(ws.gu[:T], pdl=pdl, out=(None, ws.is_[:T]), prep=(ws.iq[:T], ws.i_sum[:T]))
            ops.t2_gemm_wide(ws.iq[:T], ws.i_sum[:T], ff.down_proj.weight.data, ws.is_[:T], ff.down_proj.weight_scale,
                             out=ws.ffn_out[:T], pdl=pdl)

    @torch.no_grad()
    def prefill_wide(self, token_values: torch.Tensor, kv_planes: List[SDLMLayerCache], kv_rows: int,
                     logits_buf: Optional[torch.Tensor] = None) -> torch.Tensor:
        """The whole prompt through prefill_rows_wide in waves of PREFILL_WAVE rows, then the packed head on
        the last row (the only logit row a decode loop uses).  Returns fp32 logits [1, vocab]."""
        seq = int(token_values.shape[0])
        dev = token_values.device
        a = self.args
        self.prepare_t2_lm_head()
        wave = min(PREFILL_WAVE, (seq + PREFILL_CHUNK - 1) // PREFILL_CHUNK * PREFILL_CHUNK)
        ws = getattr(self, "_prompt_ws", None)
        if ws is None or ws.T < wave:
            ws = self._prompt_ws = PromptWorkspace(a, max(wave, PREFILL_WAVE if seq > PREFILL_WAVE else wave), dev)
        ids = token_values.to(torch.int64).contiguous()
        n = 0
        cache = self.__dict__.setdefault("_prompt_waves", {})
        for c0 in range(0, seq, wave):
            n = min(wave, seq - c0)
            # Per (rows, first position, KV buffer): the attention scratch, the position ids and, from the
            # second prompt of that shape on, a CUDA graph of the wave (about 280 launches whose host cost
            # would otherwise exceed their device time).  The graph reads its ids from ws.tokens.
            key = (n, c0, kv_planes[0][0].data_ptr(), kv_rows)
            rec = cache.get(key)
            if rec is None:
                if len(cache) > 32:
                    cache.clear()
                rec = cache[key] = {"scratch": ops.prompt_attention_scratch(n, c0, PREFILL_CHUNK, a.n_heads,
                                                                            a.n_kv_heads, dev),
                                    "pos": torch.arange(c0, c0 + n, device=dev, dtype=torch.int64), "uses": 0,
                                    "graph": None}
            rec["uses"] += 1
            ws.tokens[:n].copy_(ids[c0:c0 + n])
            if rec["graph"] is None and rec["uses"] >= 2 and self.use_prompt_graphs \
                    and not torch.cuda.is_current_stream_capturing():
                torch.cuda.synchronize(dev)
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    self.prefill_rows_wide(ws.tokens[:n], rec["pos"], kv_planes, kv_rows, c0, ws, rec["scratch"])
                rec["graph"] = g
            if rec["graph"] is not None:
                rec["graph"].replay()
            else:
                self.prefill_rows_wide(ws.tokens[:n], rec["pos"], kv_planes, kv_rows, c0, ws, rec["scratch"])
        if logits_buf is None:
            logits_buf = torch.empty((1, self._lm_head_n_pad), dtype=torch.float32, device=dev)
        # final norm + packed head on the last row of the last wave
        W1 = self.workspace(1)
        ops.rmsnorm_fused(ws.h, self.norm.weight.data, a.norm_eps, M=1, res=ws.ffn_out, row0=n - 1, pdl=self.use_pdl,
                          out={"qp": W1.hq, "asum": W1.h_sum, "s": W1.hs})
        ops.t2_gemv_prepared(W1.hq[:1], W1.h_sum[:1], self._lm_head_t2_w, W1.hs[:1], self._lm_head_t2_scale,
                             out_kind=native.OUT_F32_OF_BF16, out=logits_buf, ldc=self._lm_head_n_pad, pdl=self.use_pdl)
        return logits_buf[:, : self._lm_head_t2_vocab]

    @torch.no_grad()
    def forward_sdlm_prefill(self, token_values: torch.Tensor, cache: List[SDLMLayerCache],
                             positions: Optional[torch.Tensor] = None, block_size: int = 1,
                             fast: bool = False, causal_attn: bool = True) -> torch.Tensor:
        """Variable-length causal prompt forward (reference: model.py:1306-1340).

        Runs the packed integer path in AR-causal slabs of PREFILL_CHUNK rows: each slab
        writes its K/V rows in place (sigma == cache_len == slab start) and attends to the
        rows before it.  The reference unpacks every layer to dense bf16 and calls cuBLAS on
        fake-quantised activations, the same quantised product with bf16 roundings between
        the steps.  `cache[i]` is replaced by (k, v) views [1, n_kv, seq, head_dim]; returns
        fp32 logits [seq, vocab]."""
        if block_size > 1:
            raise NotImplementedError("block-diffusion prefill masks are outside the decode path")
        a = self.args
        seq = int(token_values.shape[0])
        dev = token_values.device
        if positions is None:
            positions = torch.arange(seq, device=dev, dtype=torch.int64)
        positions = positions.to(torch.int64).contiguous()
        kv = torch.zeros(2, a.n_layers, 1, a.n_kv_heads, seq + PREFILL_CHUNK, a.head_dim,
                         dtype=torch.bfloat16, device=dev)
        state = ops.new_step_state(dev)
        scratch = ops.attention_scratch(PREFILL_CHUNK, a.n_heads, seq, dev)
        self.prepare_t2_lm_head()
        logits = torch.empty((seq, self._lm_head_n_pad), dtype=torch.float32, device=dev)
        for c0 in range(0, seq, PREFILL_CHUNK):
            n = min(PREFILL_CHUNK, seq - c0)
            ops.set_step_state(state, c0, 0, native.ROLE_AR, n - a.block_size)
            kv_full = [(kv[0, i][:, :, : c0 + n, :], kv[1, i][:, :, : c0 + n, :])
                       for i in range(a.n_layers)]
            self.forward_sdlm_decode_graph_kernel(
                token_values[c0:c0 + n].contiguous(), positions[c0:c0 + n].contiguous(), kv_full, n,
                state, 0, n, "t2", attn_scratch=scratch, logits_buf=logits[c0:c0 + n])
        for i in range(a.n_layers):
            cache[i] = (kv[0, i][:, :, :seq, :], kv[1, i][:, :, :seq, :])
        return logits[:, : self._lm_head_t2_vocab]


PREFILL_CHUNK = 16
PREFILL_WAVE = 256          # prompt rows one pass of the many-row path takes


class PromptWorkspace:
    """Intermediates of one wave of the many-row prompt path (Transformer.prefill_rows_wide)."""

    def __init__(self, args: ModelArgs, T: int, device):
        bf, i8, f32, i32 = torch.bfloat16, torch.int8, torch.float32, torch.int32
        q_dim = args.n_heads * args.head_dim
        qkv = q_dim + 2 * args.n_kv_heads * args.head_dim

        def buf(shape, dtype):
            return torch.empty(shape, dtype=dtype, device=device)

        self.T = T
        self.h = buf((T, args.dim), bf)
        self.q, self.q_sum, self.s = buf((T, args.dim), i8), buf((T, args.dim // 128), i32), buf((T, 1), f32)
        self.xqkv = buf((T, qkv), bf)
        self.qrot = buf((T, args.n_heads, args.head_dim), bf)
        self.att = buf((T, q_dim), bf)
        self.att_amax = torch.zeros((2, T), dtype=i32, device=device)
        self.att_q, self.att_sum, self.att_s = buf((T, q_dim), i8), buf((T, q_dim // 128), i32), buf((T, 1), f32)
        self.attn_out = buf((T, args.dim), bf)
        self.gu = buf((T, 2 * args.ffn_dim), bf)
        self.iq, self.i_sum, self.is_ = buf((T, args.ffn_dim), i8), buf((T, args.ffn_dim // 128), i32), buf((T, 1), f32)
        self.ffn_out = buf((T, args.dim), bf)
        self.tokens = torch.zeros(T, dtype=torch.int64, device=device)


class _LayerView:
    """Adapter handing ops the base pointer of a [1, n_kv, rows, hd] view together with the
    row count of the buffer it was sliced from."""

    def __init__(self, view: torch.Tensor, kv_rows: int):
        self._v = view
        self.shape = (view.shape[-3], kv_rows, view.shape[-1])

    def data_ptr(self):
        return self._v.data_ptr()


def make_sdlm_cache(args: ModelArgs, device, dtype: torch.dtype = torch.bfloat16) -> List[SDLMLayerCache]:
    """Empty (length-0) per-layer cache list for the prefill path (model.py:1453-1469)."""
    return [(torch.zeros(1, args.n_kv_heads, 0, args.head_dim, dtype=dtype, device=device),
             torch.zeros(1, args.n_kv_heads, 0, args.head_dim, dtype=dtype, device=device))
            for _ in range(args.n_layers)]
