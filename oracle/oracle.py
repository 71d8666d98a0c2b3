"""Python face of the CPU oracle.  TEST INFRASTRUCTURE ONLY.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs import
this module; the package under bitmtp_b200/ never does.

Arrays are numpy; bf16 tensors travel as uint16 bit patterns.  The arithmetic
lives in oracle/bm_oracle.c (see its header for the reference lines each
function restates); `gemv_numpy` is an independent numpy twin of the GEMV used
to check the C code against itself, and `OracleModel.forward` strings the
operators together in the order of the reference's captured forward
(src/bonsai_sft/gpu/model.py:1363-1404, 1119-1137, 958-1009, 1053-1064).
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, List, Optional, Tuple

import numpy as np

from .build import build_oracle

ROLE_DRAFT, ROLE_VERIFY, ROLE_AR = 0, 1, 2
ROLE_IDS = {"draft": ROLE_DRAFT, "draft_fp8": ROLE_DRAFT, "draft_bf16": ROLE_DRAFT,
            "verify": ROLE_VERIFY, "ar": ROLE_AR}

_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        so = build_oracle()
        L = ctypes.CDLL(so)
        vp, ci, cf = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
        L.bmo_num_threads.restype = ci
        L.bmo_set_num_threads.argtypes = [ci]
        L.bmo_t2_gemv.argtypes = [vp, vp, vp, vp, ci, ci, ci, vp, vp, vp]
        L.bmo_quant_rows.argtypes = [vp, ci, ci, vp, vp]
        L.bmo_rmsnorm.argtypes = [vp, vp, cf, ci, ci, vp]
        L.bmo_rmsnorm_quant.argtypes = [vp, vp, cf, ci, ci, vp, vp]
        L.bmo_add_rmsnorm_quant.argtypes = [vp, vp, vp, cf, ci, ci, vp, vp, vp]
        L.bmo_add_bf16.argtypes = [vp, vp, ctypes.c_size_t, vp]
        L.bmo_silu_mul_quant.argtypes = [vp, ci, ci, vp, vp, vp]
        L.bmo_qknorm_rope_kvappend.argtypes = [vp, vp, vp, cf, vp, vp, vp, ci, ci, ci, vp, vp,
                                               ci, ci, vp]
        L.bmo_attention.argtypes = [vp, vp, vp, ci, ci, ci, ci, ci, ci, ci, ci, ci, vp]
        L.bmo_visible.argtypes = [ci] * 7
        L.bmo_visible.restype = ci
        L.bmo_argmax_rows.argtypes = [vp, ci, ci, vp]
        L.bmo_draft_chain.argtypes = [vp, ci, ci, cf, vp, vp]
        L.bmo_draft_chain.restype = ci
        L.bmo_verify_accept.argtypes = [vp, vp, ci]
        L.bmo_verify_accept.restype = ci
        L.bmo_embed.argtypes = [vp, vp, ci, ci, vp]
        L.bmo_expf.argtypes = [cf]
        L.bmo_expf.restype = cf
        L.bmo_logf.argtypes = [cf]
        L.bmo_logf.restype = cf
        L.bmo_f32_to_bf16.argtypes = [cf]
        L.bmo_f32_to_bf16.restype = ctypes.c_uint16
        _lib = L
    return _lib


def _p(a: Optional[np.ndarray]):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"], "oracle arrays must be contiguous"
    return a.ctypes.data_as(ctypes.c_void_p)


# --------------------------------------------------------------------------- bf16 helpers
def f32_to_bf16(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even fp32 -> bf16 bit patterns (uint16)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    return r.astype(np.uint16)


def bf16_to_f32(h: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(h, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def torch_to_u16(t) -> np.ndarray:
    """torch.bfloat16 tensor (CPU) -> uint16 numpy view of its bits."""
    import torch
    assert t.dtype == torch.bfloat16
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def u16_to_torch(a: np.ndarray):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).view(torch.bfloat16)


# --------------------------------------------------------------------------- packing
def pack_t2(codes: np.ndarray) -> np.ndarray:
    """Ternary values in {-1,0,1}, shape [N, K] -> packed uint8 [N, K/4].

    Element j of a row occupies bits 2*(j%4) of byte j/4 and is stored as
    value+2 (src/bonsai_sft/gpu/convert_bonsai_mtp_to_gpu.py:127-144).
    """
    c = (codes.astype(np.int16) + 2).astype(np.uint8).reshape(codes.shape[0], -1, 4)
    return (c[..., 0] | (c[..., 1] << 2) | (c[..., 2] << 4) | (c[..., 3] << 6)).astype(np.uint8)


def unpack_t2(packed: np.ndarray) -> np.ndarray:
    """Packed uint8 [N, K/4] -> ternary int8 [N, K] (code - 2)."""
    p = packed.astype(np.uint8)
    out = np.empty((p.shape[0], p.shape[1], 4), dtype=np.int8)
    for i in range(4):
        out[..., i] = ((p >> (2 * i)) & 3).astype(np.int8) - 2
    return out.reshape(p.shape[0], -1)


# --------------------------------------------------------------------------- operators
def t2_gemv(A: np.ndarray, B: np.ndarray, ws: np.ndarray, s: np.ndarray,
            want_groups: bool = False):
    """Returns (out_f32 [W,N], out_bf16 uint16 [W,N], G int32 [W,N,K/128] or None)."""
    W, K = A.shape
    N = B.shape[0]
    assert B.shape[1] * 4 == K and ws.shape == (N, K // 128)
    A = np.ascontiguousarray(A, dtype=np.int8)
    B = np.ascontiguousarray(B).view(np.uint8)
    ws = np.ascontiguousarray(ws, dtype=np.uint16)
    s = np.ascontiguousarray(s, dtype=np.float32).reshape(-1)
    o32 = np.empty((W, N), dtype=np.float32)
    o16 = np.empty((W, N), dtype=np.uint16)
    G = np.empty((W, N, K // 128), dtype=np.int32) if want_groups else None
    lib().bmo_t2_gemv(_p(A), _p(B), _p(ws), _p(s), W, N, K, _p(o32), _p(o16), _p(G))
    return o32, o16, G


def gemv_numpy(A: np.ndarray, B: np.ndarray, ws: np.ndarray, s: np.ndarray):
    """Independent numpy twin of bmo_t2_gemv: same group sums, same fp32 order."""
    W, K = A.shape
    N = B.shape[0]
    ng = K // 128
    t = unpack_t2(B.view(np.uint8)).astype(np.int32).reshape(N, ng, 128)
    a = A.astype(np.int32).reshape(W, ng, 128)
    G = np.einsum("wgk,ngk->wng", a, t).astype(np.int32)
    sc = bf16_to_f32(ws)                                   # [N, ng]
    slot = np.zeros((W, N, 16), dtype=np.float32)
    for g in range(ng):
        prod = G[:, :, g].astype(np.float64) * sc[None, :, g].astype(np.float64)
        # fma(G, sc, slot): the product of a <2^24 integer and a bf16 is exact in
        # fp64, and so is adding an fp32 to it, so one rounding to fp32 is an fma.
        slot[:, :, g % 16] = (prod + slot[:, :, g % 16].astype(np.float64)).astype(np.float32)
    step = 1
    while step < 16:
        for i in range(0, 16, 2 * step):
            slot[:, :, i] = slot[:, :, i] + slot[:, :, i + step]
        step *= 2
    inv = (np.float32(1.0) / s.reshape(W, 1).astype(np.float32)).astype(np.float32)
    y = (slot[:, :, 0] * inv).astype(np.float32)
    return y, f32_to_bf16(y), G


def quant_rows(x_u16: np.ndarray):
    M, K = x_u16.shape
    q = np.empty((M, K), dtype=np.int8)
    s = np.empty((M,), dtype=np.float32)
    lib().bmo_quant_rows(_p(np.ascontiguousarray(x_u16)), M, K, _p(q), _p(s))
    return q, s


def rmsnorm(x_u16, w_u16, eps: float):
    M, dim = x_u16.shape
    out = np.empty((M, dim), dtype=np.uint16)
    lib().bmo_rmsnorm(_p(np.ascontiguousarray(x_u16)), _p(w_u16), eps, M, dim, _p(out))
    return out


def rmsnorm_quant(x_u16, w_u16, eps: float):
    M, dim = x_u16.shape
    q = np.empty((M, dim), dtype=np.int8)
    s = np.empty((M,), dtype=np.float32)
    lib().bmo_rmsnorm_quant(_p(np.ascontiguousarray(x_u16)), _p(w_u16), eps, M, dim, _p(q), _p(s))
    return q, s


def add_rmsnorm_quant(x_u16, res_u16, w_u16, eps: float):
    M, dim = x_u16.shape
    h = np.empty((M, dim), dtype=np.uint16)
    q = np.empty((M, dim), dtype=np.int8)
    s = np.empty((M,), dtype=np.float32)
    lib().bmo_add_rmsnorm_quant(_p(np.ascontiguousarray(x_u16)), _p(np.ascontiguousarray(res_u16)),
                                _p(w_u16), eps, M, dim, _p(h), _p(q), _p(s))
    return h, q, s


def add_bf16(x_u16, res_u16):
    out = np.empty_like(x_u16)
    lib().bmo_add_bf16(_p(np.ascontiguousarray(x_u16)), _p(np.ascontiguousarray(res_u16)),
                       x_u16.size, _p(out))
    return out


def silu_mul_quant(gu_u16, want_inner: bool = False):
    M, F2 = gu_u16.shape
    F = F2 // 2
    q = np.empty((M, F), dtype=np.int8)
    s = np.empty((M,), dtype=np.float32)
    inner = np.empty((M, F), dtype=np.uint16) if want_inner else None
    lib().bmo_silu_mul_quant(_p(np.ascontiguousarray(gu_u16)), M, F, _p(q), _p(s), _p(inner))
    return (q, s, inner) if want_inner else (q, s)


def qknorm_rope_kvappend(xqkv, q_w, k_w, eps, cos_t, sin_t, positions, H, Hkv,
                         k_layer, v_layer, sigma):
    """k_layer / v_layer: uint16 [Hkv, kv_rows, 128], written in place at rows [sigma, sigma+M)."""
    M = xqkv.shape[0]
    kv_rows = k_layer.shape[1]
    assert k_layer.flags["C_CONTIGUOUS"] and v_layer.flags["C_CONTIGUOUS"]
    q_out = np.empty((M, H, 128), dtype=np.uint16)
    pos = np.ascontiguousarray(positions, dtype=np.int64)
    lib().bmo_qknorm_rope_kvappend(_p(np.ascontiguousarray(xqkv)), _p(q_w), _p(k_w), eps,
                                   _p(cos_t), _p(sin_t), _p(pos), M, H, Hkv,
                                   _p(k_layer), _p(v_layer), kv_rows, sigma, _p(q_out))
    return q_out


def attention(q, k_layer, v_layer, sigma, cache_len, n_pend, P, role):
    M, H, _ = q.shape
    Hkv, kv_rows, _ = k_layer.shape
    out = np.empty((M, H * 128), dtype=np.uint16)
    lib().bmo_attention(_p(np.ascontiguousarray(q)), _p(k_layer), _p(v_layer), M, H, Hkv, kv_rows,
                        sigma, cache_len, n_pend, P, role, _p(out))
    return out


def visible(role, r, c, sigma, cache_len, n_pend, P) -> bool:
    return bool(lib().bmo_visible(role, r, c, sigma, cache_len, n_pend, P))


def mask_matrix(role: int, M: int, sigma: int, cache_len: int, n_pend: int, P: int) -> np.ndarray:
    """Boolean [M, sigma+M] visibility matrix of one replay."""
    out = np.zeros((M, sigma + M), dtype=bool)
    for r in range(M):
        for c in range(sigma + M):
            out[r, c] = visible(role, r, c, sigma, cache_len, n_pend, P)
    return out


def argmax_rows(logits: np.ndarray) -> np.ndarray:
    rows, vocab = logits.shape
    idx = np.empty((rows,), dtype=np.int64)
    lib().bmo_argmax_rows(_p(np.ascontiguousarray(logits, dtype=np.float32)), rows, vocab, _p(idx))
    return idx


def draft_chain(logits: np.ndarray, tau: float):
    D, vocab = logits.shape
    idx = np.empty((D,), dtype=np.int64)
    conf = np.empty((D,), dtype=np.float32)
    n = lib().bmo_draft_chain(_p(np.ascontiguousarray(logits, dtype=np.float32)), D, vocab,
                              tau, _p(idx), _p(conf))
    return idx, int(n), conf


def verify_accept(draft: np.ndarray, verify: np.ndarray, D: int) -> int:
    d = np.ascontiguousarray(draft, dtype=np.int64)
    v = np.ascontiguousarray(verify, dtype=np.int64)
    return int(lib().bmo_verify_accept(_p(d), _p(v), D))


# --------------------------------------------------------------------------- whole forward
class OracleModel:
    """Weights of one packed checkpoint as numpy arrays + the captured forward.

    `state` is the dict `model_state_t2g128.pt` holds (torch tensors) and
    `cfg` the dict of `bonsai_gpu_config.json`.  Weight merging (q|k|v and
    gate|up by output row) and the T2 packing of the tied head follow
    src/bonsai_sft/gpu/model.py:931-956, 1042-1051, 1223-1243.
    """

    def __init__(self, cfg: dict, state: dict, max_positions: int, head=None):
        """`head`: optional (packed codes int8/uint8 [vocab, dim/4], scales bf16 [vocab, dim/128]) of the
        tied head when the caller already holds it on the T2 grid (vocab a multiple of 8); otherwise the
        embedding is packed here."""
        import torch
        self.cfg = dict(cfg)
        self.dim, self.L = cfg["dim"], cfg["n_layers"]
        self.H, self.Hkv, self.hd = cfg["n_heads"], cfg["n_kv_heads"], cfg["head_dim"]
        assert self.hd == 128
        self.F, self.vocab, self.eps = cfg["ffn_dim"], cfg["vocab_size"], float(cfg["norm_eps"])
        self.D = cfg["block_size"]

        def u16(k):
            return torch_to_u16(state[k].to(torch.bfloat16))

        def u8(k):
            return np.ascontiguousarray(state[k].cpu().numpy().view(np.uint8))

        self.embed = u16("embed_tokens.weight")
        self.norm = u16("norm.weight")
        self.layers: List[Dict[str, np.ndarray]] = []
        for i in range(self.L):
            a, f = f"layers.{i}.attention.", f"layers.{i}.feed_forward."
            self.layers.append(dict(
                in_ln=u16(f"layers.{i}.input_layernorm.weight"),
                post_ln=u16(f"layers.{i}.post_attention_layernorm.weight"),
                wqkv=np.concatenate([u8(a + "q_proj.weight"), u8(a + "k_proj.weight"),
                                     u8(a + "v_proj.weight")], 0),
                wqkv_s=np.concatenate([u16(a + "q_proj.weight_scale"), u16(a + "k_proj.weight_scale"),
                                       u16(a + "v_proj.weight_scale")], 0),
                wo=u8(a + "o_proj.weight"), wo_s=u16(a + "o_proj.weight_scale"),
                q_norm=u16(a + "q_norm.weight"), k_norm=u16(a + "k_norm.weight"),
                wgu=np.concatenate([u8(f + "gate_proj.weight"), u8(f + "up_proj.weight")], 0),
                wgu_s=np.concatenate([u16(f + "gate_proj.weight_scale"),
                                      u16(f + "up_proj.weight_scale")], 0),
                wdown=u8(f + "down_proj.weight"), wdown_s=u16(f + "down_proj.weight_scale"),
            ))
        if head is not None and head[0].shape[0] % 8 == 0:
            self.head_w = np.ascontiguousarray(head[0].cpu().numpy().view(np.uint8))
            self.head_s = torch_to_u16(head[1].to(torch.bfloat16))
        else:
            self.head_w, self.head_s = self._pack_head(state["embed_tokens.weight"])
        self.cos, self.sin = rope_tables(cfg, max_positions)

    @staticmethod
    def _pack_head(embed):
        """Tied head on its T2 grid, padded to a multiple of 8 rows (model.py:1223-1243)."""
        import torch
        W = embed.detach().cpu().to(torch.bfloat16)
        vocab, dim = W.shape
        npad = (vocab + 7) // 8 * 8
        Wp = torch.zeros(npad, dim, dtype=torch.bfloat16)
        Wp[:vocab].copy_(W)
        groups = Wp.float().view(npad, dim // 128, 128)
        scale = groups.abs().amax(dim=-1).to(torch.bfloat16)
        denom = scale.float().unsqueeze(-1).clamp_min(1e-30)
        q = torch.round(groups / denom).clamp(-1, 1).to(torch.int8).view(npad, dim)
        return pack_t2(q.numpy()), torch_to_u16(scale)

    def new_kv(self, sigma: int, m_max: int) -> np.ndarray:
        """uint16 [2, L, 1, Hkv, sigma+m_max, 128], zero-filled (fast_runtime.py:130-138)."""
        return np.zeros((2, self.L, 1, self.Hkv, sigma + m_max, 128), dtype=np.uint16)

    def forward(self, tokens, positions, kv: np.ndarray, sigma: int, role: int, cache_len: int,
                n_pend: int, logits_start: int = 0, logits_end: int = -1) -> np.ndarray:
        """One captured forward of width M=len(tokens).  Returns logits fp32
        [logits_end-logits_start, vocab]: the bf16-rounded head output widened to fp32
        (model.py:1403)."""
        L = lib()
        M = len(tokens)
        P = M - self.D
        if logits_end == -1:
            logits_end = M
        tokens = np.ascontiguousarray(tokens, dtype=np.int64)
        h = np.empty((M, self.dim), dtype=np.uint16)
        L.bmo_embed(_p(self.embed), _p(tokens), M, self.dim, _p(h))
        q, s = rmsnorm_quant(h, self.layers[0]["in_ln"], self.eps)
        ffn_out = None
        for i, ly in enumerate(self.layers):
            if i > 0:
                h, q, s = add_rmsnorm_quant(ffn_out, h, ly["in_ln"], self.eps)
            _, xqkv, _ = t2_gemv(q, ly["wqkv"], ly["wqkv_s"], s)
            k_layer, v_layer = kv[0, i, 0], kv[1, i, 0]
            xq = qknorm_rope_kvappend(xqkv, ly["q_norm"], ly["k_norm"], self.eps, self.cos,
                                      self.sin, positions, self.H, self.Hkv, k_layer, v_layer, sigma)
            att = attention(xq, k_layer, v_layer, sigma, cache_len, n_pend, P, role)
            oq, os_ = quant_rows(att)
            _, attn_out, _ = t2_gemv(oq, ly["wo"], ly["wo_s"], os_)
            h, fq, fs = add_rmsnorm_quant(h, attn_out, ly["post_ln"], self.eps)
            _, gu, _ = t2_gemv(fq, ly["wgu"], ly["wgu_s"], fs)
            iq, is_ = silu_mul_quant(gu)
            _, ffn_out, _ = t2_gemv(iq, ly["wdown"], ly["wdown_s"], is_)
        h = add_bf16(h, ffn_out)
        hn = rmsnorm(np.ascontiguousarray(h[logits_start:logits_end]), self.norm, self.eps)
        hq, hs = quant_rows(hn)
        _, lg16, _ = t2_gemv(hq, self.head_w, self.head_s, hs)
        return bf16_to_f32(lg16[:, : self.vocab])


def rope_tables(cfg: dict, max_positions: int) -> Tuple[np.ndarray, np.ndarray]:
    """bf16 cos/sin tables [max_positions, 128] with YaRN scaling
    (src/bonsai_sft/gpu/model.py:342-379, 950-955).  Computed with torch CPU
    ops in the reference's own order; both the oracle and the GPU runtime
    consume the resulting table, so its transcendental functions never enter a
    parity comparison."""
    import math
    import torch
    dim = cfg["head_dim"]
    base, factor = float(cfg["rope_theta"]), float(cfg["rope_factor"])
    original_max = cfg["rope_original_max"]
    beta_fast, beta_slow = 32.0, 1.0
    pos_freqs = base ** (torch.arange(0, dim, 2).float() / dim)
    inv_extrap = 1.0 / pos_freqs
    inv_interp = 1.0 / (factor * pos_freqs)

    def corr(num_rot):
        return (dim * math.log(original_max / (num_rot * 2 * math.pi))) / (2 * math.log(base))

    low = max(math.floor(corr(beta_fast)), 0)
    high = min(math.ceil(corr(beta_slow)), dim - 1)
    if low == high:
        high += 0.001
    ramp = torch.clamp((torch.arange(dim // 2, dtype=torch.float32) - low) / (high - low), 0.0, 1.0)
    extrap_factor = 1.0 - ramp
    inv_freq = inv_interp * (1.0 - extrap_factor) + inv_extrap * extrap_factor
    # build_model casts the whole module, buffers included, to bf16
    # (src/bonsai_sft/gpu/generate.py:50), so the tables are built from bf16-rounded
    # inverse frequencies
    inv_freq = inv_freq.to(torch.bfloat16).float()
    mscale = 1.0 if factor <= 1.0 else 0.1 * 1.0 * math.log(factor) + 1.0
    pos = torch.arange(max_positions, dtype=torch.float32)
    freqs = torch.outer(pos, inv_freq.float())
    emb = torch.cat((freqs, freqs), dim=-1)
    cos = (emb.cos() * mscale).to(torch.bfloat16)
    sin = (emb.sin() * mscale).to(torch.bfloat16)
    return torch_to_u16(cos), torch_to_u16(sin)
