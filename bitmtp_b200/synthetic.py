"""Seeded synthetic weights, activations and checkpoints.

Stand-ins for the real Bonsai checkpoints and prompts (not available offline):
ternary codes i.i.d. uniform over {-1,0,+1}, one bf16 scale per 128 K-elements
drawn U[0.01,0.05], bf16 N(0,1) activations.  Everything is generated with a
CPU torch.Generator, so the CPU oracle and the GPU path see identical bytes.
"""
from __future__ import annotations

import json
import os
from typing import Dict, Tuple

import torch

GROUP = 128


def pack_t2_g128(w_frozen: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """bf16 weights on the {-s,0,+s} grid -> (int8 [N,K/4] codes, bf16 [N,K/128] scales).

    Same layout as the reference converter (element j of a row in bits 2*(j%4)
    of byte j/4, stored as value+2; scale = per-group absmax):
    src/bonsai_sft/gpu/convert_bonsai_mtp_to_gpu.py:127-144.
    """
    assert w_frozen.dtype == torch.bfloat16
    n, k = w_frozen.shape
    assert k % GROUP == 0
    wg = w_frozen.float().view(n, k // GROUP, GROUP)
    scale = wg.abs().amax(dim=-1).to(torch.bfloat16)
    q = torch.round(wg / scale.float().unsqueeze(-1).clamp_min(1e-30)).clamp(-1, 1)
    code = (q.to(torch.int16).view(n, k // 4, 4) + 2).to(torch.uint8)
    packed = code[..., 0] | (code[..., 1] << 2) | (code[..., 2] << 4) | (code[..., 3] << 6)
    return packed.view(torch.int8).contiguous(), scale.contiguous()


def ternary_weight(n: int, k: int, gen: torch.Generator):
    """Returns (packed int8 [n,k/4], scale bf16 [n,k/128], dense bf16 [n,k])."""
    q = torch.randint(-1, 2, (n, k), generator=gen, dtype=torch.int8)
    sc = (torch.rand(n, k // GROUP, generator=gen) * 0.04 + 0.01).to(torch.bfloat16)
    w = (q.float().view(n, k // GROUP, GROUP) * sc.float().unsqueeze(-1)).view(n, k).to(torch.bfloat16)
    packed, scale = pack_t2_g128(w)
    return packed, scale, w


def gemv_case(w: int, n: int, k: int, seed: int = 0) -> Dict[str, torch.Tensor]:
    """One GEMV problem: packed weights + INT8-quantised N(0,1) activations (CPU tensors)."""
    gen = torch.Generator().manual_seed(seed)
    packed, scale, _ = ternary_weight(n, k, gen)
    x = torch.randn(w, k, generator=gen).to(torch.bfloat16)
    xf = x.float()
    s = 127.0 / xf.abs().amax(dim=-1, keepdim=True).clamp_min(1e-5)
    a = (xf * s).round().clamp(-128, 127).to(torch.int8)
    return {"A": a, "B": packed, "ws": scale, "s": s.reshape(-1).contiguous(), "x": x}


BONSAI_1P7B = dict(dim=2048, n_layers=28, n_heads=16, n_kv_heads=8, head_dim=128, ffn_dim=6144,
                   vocab_size=151936)
BONSAI_4B = dict(dim=2560, n_layers=36, n_heads=32, n_kv_heads=8, head_dim=128, ffn_dim=9728,
                 vocab_size=151936)
TINY = dict(dim=256, n_layers=2, n_heads=2, n_kv_heads=1, head_dim=128, ffn_dim=512,
            vocab_size=1000)


def make_config(geometry: Dict[str, int], block_size: int = 8) -> Dict:
    """`bonsai_gpu_config.json` content (convert_bonsai_mtp_to_gpu.py:257-275)."""
    cfg = dict(geometry)
    cfg.update(norm_eps=1e-6, rope_theta=1.0e6, rope_original_max=8192, rope_factor=4.0,
               tie_word_embeddings=True, block_size=block_size, causal_attn=True,
               mask_token_id=min(151654, geometry["vocab_size"] - 1), kernel_kind="t2g128",
               quantize_embedding=True)
    return cfg


def make_state(cfg: Dict, seed: int = 0) -> Dict[str, torch.Tensor]:
    """Random-init packed state dict with the key names of `model_state_t2g128.pt`
    (convert_bonsai_mtp_to_gpu.py:37-66, 221-242).  Norm weights are 1; the
    embedding is bf16 on the ternary grid so that re-packing it as the tied
    head is lossless."""
    gen = torch.Generator().manual_seed(seed)
    dim, ffn = cfg["dim"], cfg["ffn_dim"]
    qd, kd = cfg["n_heads"] * cfg["head_dim"], cfg["n_kv_heads"] * cfg["head_dim"]
    sd: Dict[str, torch.Tensor] = {}
    _, _, emb = ternary_weight(cfg["vocab_size"], dim, gen)
    sd["embed_tokens.weight"] = emb
    sd["norm.weight"] = torch.ones(dim, dtype=torch.bfloat16)
    for i in range(cfg["n_layers"]):
        p = f"layers.{i}."
        sd[p + "input_layernorm.weight"] = torch.ones(dim, dtype=torch.bfloat16)
        sd[p + "post_attention_layernorm.weight"] = torch.ones(dim, dtype=torch.bfloat16)
        sd[p + "attention.q_norm.weight"] = torch.ones(cfg["head_dim"], dtype=torch.bfloat16)
        sd[p + "attention.k_norm.weight"] = torch.ones(cfg["head_dim"], dtype=torch.bfloat16)
        for name, (n, k) in (("attention.q_proj", (qd, dim)), ("attention.k_proj", (kd, dim)),
                             ("attention.v_proj", (kd, dim)), ("attention.o_proj", (dim, qd)),
                             ("feed_forward.gate_proj", (ffn, dim)),
                             ("feed_forward.up_proj", (ffn, dim)),
                             ("feed_forward.down_proj", (dim, ffn))):
            packed, scale, _ = ternary_weight(n, k, gen)
            sd[p + name + ".weight"] = packed
            sd[p + name + ".weight_scale"] = scale
    return sd


def write_checkpoint(out_dir: str, cfg: Dict, seed: int = 0) -> str:
    """Write `bonsai_gpu_config.json` + `model_state_t2g128.pt` in the reference's layout."""
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "bonsai_gpu_config.json"), "w") as f:
        json.dump(cfg, f, indent=2)
    torch.save(make_state(cfg, seed), os.path.join(out_dir, "model_state_t2g128.pt"))
    return out_dir


class AcceptancePolicy:
    """How many draft tokens a benchmark or test run accepts per step, in place of the measured
    confidence chain / prefix match (random-init weights accept almost nothing by themselves).

    kind  "free"         keep the measured counts
          "forced"       the whole block: chain length D, verifier accepts D
          "categorical"  a seeded draw a in 1..D per step with p(k) proportional to r**k
                         (r = 0.9082925: mean 4.0 at D = 8); the chain length becomes a, and
                         a verifier replay in the same step accepts a - 1 (+ its own token =
                         a committed).  A verifier replay with no chain before it (the
                         speculative policy) draws its own a.
    The draws come from a splitmix64 stream, so every host reproduces them from the seed."""

    R = 0.9082925

    def __init__(self, kind: str, D: int, seed: int = 0):
        if kind not in ("free", "forced", "categorical"):
            raise ValueError(f"unknown acceptance policy {kind!r}")
        self.kind, self.D = kind, int(D)
        self._state = (int(seed) * 0x9E3779B97F4A7C15 + 0x1234567) & 0xFFFFFFFFFFFFFFFF
        self._a = None
        w = [self.R ** k for k in range(1, self.D + 1)]
        tot = sum(w)
        self.p = [x / tot for x in w]
        self.draws: list = []

    def _uniform(self) -> float:
        self._state = (self._state + 0x9E3779B97F4A7C15) & 0xFFFFFFFFFFFFFFFF
        z = self._state
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & 0xFFFFFFFFFFFFFFFF
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & 0xFFFFFFFFFFFFFFFF
        z ^= z >> 31
        return (z >> 11) / float(1 << 53)

    def _draw(self) -> int:
        u, acc = self._uniform(), 0.0
        a = self.D
        for k, pk in enumerate(self.p, start=1):
            acc += pk
            if u < acc:
                a = k
                break
        self.draws.append(a)
        return a

    def chain_count(self):
        """Replacement for the confidence-chain length of this step, or None to keep it."""
        if self.kind == "free":
            return None
        if self.kind == "forced":
            return self.D
        self._a = self._draw()
        return self._a

    def accept_count(self):
        """Replacement for the verifier's accepted-prefix length, or None to keep it."""
        if self.kind == "free":
            return None
        if self.kind == "forced":
            return self.D
        a = self._a if self._a is not None else self._draw()
        self._a = None
        return a - 1


def acceptance_hooks(FG, policy: "AcceptancePolicy"):
    """Replacements for the decode loops' confidence-chain and prefix-accept reductions
    (`FG._fused_draft_chain`, `FG._fused_verify_accept`; FG = bitmtp_b200.fast_generate) that apply
    an AcceptancePolicy.  The kernels still run.  A replaced chain length is handed to the loop as a
    host value, so the loop still reads only the ids from the device (one copy) and no extra kernel
    runs inside a timed region; a replaced accepted-prefix length is written over the kernel's count
    in place, so that it stays part of the record the loop reads in one copy."""
    chain, accept = FG._fused_draft_chain, FG._fused_verify_accept

    def hooked_chain(logits, threshold, out=None):
        idx, n = chain(logits, threshold, out)
        a = policy.chain_count()
        return idx, (n if a is None else torch.tensor([a], dtype=torch.int64))

    def hooked_accept(draft, verify, Dd, out=None):
        n = accept(draft, verify, Dd, out)
        a = policy.accept_count()
        return n if a is None else n.fill_(a)

    return hooked_chain, hooked_accept


def random_prompt(length: int, vocab: int, seed: int = 0) -> torch.Tensor:
    gen = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (1, length), generator=gen, dtype=torch.int64)


def device_ternary(n: int, k: int, gen: torch.Generator, device):
    """Random packed ternary weight generated on `device`: (packed int8 [n,k/4], scale bf16
    [n,k/128]).  Codes are uniform over {1,2,3} (= -1,0,+1), scales U[0.01,0.05].  Used by
    the benchmarks, where only the distribution matters; parity tests use the CPU-seeded
    generators above."""
    codes = torch.randint(1, 4, (n, k // 4, 4), generator=gen, device=device, dtype=torch.uint8)
    packed = codes[..., 0] | (codes[..., 1] << 2) | (codes[..., 2] << 4) | (codes[..., 3] << 6)
    scale = (torch.rand(n, k // GROUP, generator=gen, device=device) * 0.04 + 0.01).to(torch.bfloat16)
    return packed.view(torch.int8).contiguous(), scale.contiguous()


def device_state(cfg: Dict, device, seed: int = 0) -> Dict[str, torch.Tensor]:
    """Random-init packed state dict built directly on `device` (seconds instead of a
    minute for the 1.7B geometry).  Also returns the packed tied head under the private
    keys `_head.weight` / `_head.weight_scale`, so that the loader need not re-pack the
    embedding on the CPU."""
    gen = torch.Generator(device=device).manual_seed(seed)
    dim, ffn = cfg["dim"], cfg["ffn_dim"]
    qd, kd = cfg["n_heads"] * cfg["head_dim"], cfg["n_kv_heads"] * cfg["head_dim"]
    sd: Dict[str, torch.Tensor] = {}
    vocab = cfg["vocab_size"]
    hp, hs = device_ternary(vocab, dim, gen, device)
    emb = torch.empty(vocab, dim, dtype=torch.bfloat16, device=device)
    for r0 in range(0, vocab, 16384):
        r1 = min(r0 + 16384, vocab)
        p = hp[r0:r1].view(torch.uint8)
        q = torch.stack([(p >> (2 * i)) & 3 for i in range(4)], dim=-1).to(torch.int8) - 2
        w = q.view(r1 - r0, dim // GROUP, GROUP).float() * hs[r0:r1].float().unsqueeze(-1)
        emb[r0:r1] = w.view(r1 - r0, dim).to(torch.bfloat16)
    sd["embed_tokens.weight"] = emb
    sd["_head.weight"], sd["_head.weight_scale"] = hp, hs
    one = lambda n: torch.ones(n, dtype=torch.bfloat16, device=device)
    sd["norm.weight"] = one(dim)
    for i in range(cfg["n_layers"]):
        p = f"layers.{i}."
        sd[p + "input_layernorm.weight"] = one(dim)
        sd[p + "post_attention_layernorm.weight"] = one(dim)
        sd[p + "attention.q_norm.weight"] = one(cfg["head_dim"])
        sd[p + "attention.k_norm.weight"] = one(cfg["head_dim"])
        for name, (n, k) in (("attention.q_proj", (qd, dim)), ("attention.k_proj", (kd, dim)),
                             ("attention.v_proj", (kd, dim)), ("attention.o_proj", (dim, qd)),
                             ("feed_forward.gate_proj", (ffn, dim)),
                             ("feed_forward.up_proj", (ffn, dim)),
                             ("feed_forward.down_proj", (dim, ffn))):
            sd[p + name + ".weight"], sd[p + name + ".weight_scale"] = device_ternary(n, k, gen, device)
    return sd
