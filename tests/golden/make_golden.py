#!/usr/bin/env python
"""Generate the golden fixtures of tests/golden/ from the reference's own Python code.

Run where the reference project is checked out (its root is the directory that holds `src/bonsai_sft`):

    python tests/golden/make_golden.py --ref REFERENCE_ROOT [--only ops,masks,kats,forward,streams]

(`--ref` defaults to the environment variable BITMTP_REFERENCE.)

The script imports `bonsai_sft.gpu` from the reference under its eager profile
(`orin-d8`, so every `compile_helper` is the identity and the tensor expressions
run as written, on CPU), feeds it seeded inputs and records inputs + outputs as
small .npz / .json files.  The fixtures travel with the repository; the reference
does not.  tests/test_oracle_golden.py checks the CPU oracle against them, and
the GPU tests check the CUDA path against the oracle.

What each file pins:
  ops.npz      quant_input, _fused_norm_quant, _fused_add_norm_quant, RMSNorm.forward,
               silu*up + quant, _fused_qkv_qknorm_rope_kv_write, the explicit attention
               path, the rope tables, _pack_t2_g128 / _unpack_to_bf16 and integer group
               sums + fp64 scaled outputs of a GEMV computed from the unpacked weights
  masks.npz    every draft / verify / ar mask GraphAtlas builds for the D=8 and D=4
               width sets
  kats.json    accept-prefix, confidence-chain and width-selector known answers
  forward.npz  logits of the reference's captured forward on a tiny model (native
               GEMV replaced by the integer restatement, everything else unmodified)
  streams.json token streams of the reference's own decode loops driven over the
               CPU oracle forward (forced acceptance and free-running)
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)


def load_reference(ref_root: str):
    sys.path.insert(0, os.path.join(ref_root, "src"))
    from bonsai_sft.gpu.runtime_config import select_runtime_profile
    select_runtime_profile("orin-d8")
    from bonsai_sft.gpu import model as RM, fast_runtime as RR, fast_generate as RG, contracts as RC
    from bonsai_sft.gpu import convert_bonsai_mtp_to_gpu as RCV
    return types.SimpleNamespace(model=RM, runtime=RR, generate=RG, contracts=RC, convert=RCV)


def u16(t: torch.Tensor) -> np.ndarray:
    return t.detach().contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def bf16_randn(gen, *shape, scale=1.0):
    return (torch.randn(*shape, generator=gen) * scale).to(torch.bfloat16)


# ----------------------------------------------------------------------------- ops
def make_ops(ref, out_path):
    from bitmtp_b200 import synthetic
    RM = ref.model
    gen = torch.Generator().manual_seed(1234)
    rec = {}

    # --- packing + GEMV group sums, config 0 of the baseline (K=2048, N=6144, W=1, seed 0)
    for tag, (W, N, K, seed) in {"cfg0": (1, 6144, 2048, 0), "w9": (9, 256, 2560, 5)}.items():
        case = synthetic.gemv_case(W, N, K, seed=seed)
        g2 = torch.Generator().manual_seed(seed)
        q = torch.randint(-1, 2, (N, K), generator=g2, dtype=torch.int8)
        sc = (torch.rand(N, K // 128, generator=g2) * 0.04 + 0.01).to(torch.bfloat16)
        w = (q.float().view(N, K // 128, 128) * sc.float().unsqueeze(-1)).view(N, K).to(torch.bfloat16)
        packed, scale = ref.convert._pack_t2_g128(w)
        assert torch.equal(packed, case["B"]) and torch.equal(scale, case["ws"]), "packer mismatch"
        lin = RM.T2LinearKernel(K, N)
        lin.weight.data.copy_(packed)
        lin.weight_scale.copy_(scale)
        wb = lin._unpack_to_bf16()
        assert torch.equal(wb, w)
        xq, s = lin.quant_input(case["x"])
        assert torch.equal(xq, case["A"]) and torch.equal(s.reshape(-1), case["s"])
        rows = torch.randperm(N, generator=gen)[:48].sort().values
        codes = torch.round(wb[rows].float().view(48, K // 128, 128)
                            / scale[rows].float().unsqueeze(-1)).to(torch.int64)
        G = torch.einsum("wgk,ngk->wng", xq.to(torch.int64).view(W, K // 128, 128), codes)
        y64 = (G.double() * scale[rows].double().unsqueeze(0)).sum(-1) / s.double().reshape(W, 1)
        rec[f"gemv_{tag}_shape"] = np.array([W, N, K, seed])
        rec[f"gemv_{tag}_rows"] = rows.numpy()
        rec[f"gemv_{tag}_G"] = G.numpy().astype(np.int32)
        rec[f"gemv_{tag}_y64"] = y64.numpy()
        rec[f"gemv_{tag}_sha_packed"] = np.frombuffer(sha(packed.numpy()).encode(), dtype=np.uint8)
        rec[f"gemv_{tag}_sha_scale"] = np.frombuffer(sha(u16(scale)).encode(), dtype=np.uint8)
        # the reference's own CPU-capable arithmetic for the same product (bf16 fallback)
        fb = torch.nn.functional.linear(RM.Q1Linear.act_quant(case["x"]), wb[rows])
        rec[f"gemv_{tag}_fallback_bf16"] = u16(fb)

    # --- activation quantisation
    x = bf16_randn(gen, 5, 2048, scale=3.0)
    x[3].zero_()
    lin = RM.T2LinearKernel(2048, 128)
    q, s = lin.quant_input(x)
    rec.update(quant_x=u16(x), quant_q=q.numpy(), quant_s=s.numpy().reshape(-1))

    # --- fused norm helpers
    for dim in (2048, 2560):
        x = bf16_randn(gen, 4, dim, scale=2.0)
        res = bf16_randn(gen, 4, dim, scale=0.7)
        w = (1.0 + 0.1 * torch.randn(dim, generator=gen)).to(torch.bfloat16)
        q, s = RM._fused_norm_quant(x, w, 1e-6)
        h2, q2, s2 = RM._fused_add_norm_quant(x, res, w, 1e-6)
        norm = RM.RMSNorm(dim, eps=1e-6).to(torch.bfloat16)
        norm.weight.data.copy_(w)
        n = norm(x)
        rec.update({f"norm{dim}_x": u16(x), f"norm{dim}_res": u16(res), f"norm{dim}_w": u16(w),
                    f"norm{dim}_q": q.numpy(), f"norm{dim}_s": s.numpy().reshape(-1),
                    f"norm{dim}_h2": u16(h2), f"norm{dim}_q2": q2.numpy(),
                    f"norm{dim}_s2": s2.numpy().reshape(-1), f"norm{dim}_n": u16(n)})

    # --- SiLU * up + quant
    F = 768
    gu = bf16_randn(gen, 3, 2 * F, scale=3.0)
    g, u = gu.split([F, F], dim=-1)
    inner = torch.nn.functional.silu(g) * u
    q, s = lin.quant_input(inner)
    rec.update(silu_gu=u16(gu), silu_inner=u16(inner), silu_q=q.numpy(), silu_s=s.numpy().reshape(-1))

    # --- q/k norm + rope + kv write, tables from Attention.prepare_merged_weights
    args = RM.ModelArgs(dim=256, n_layers=1, n_heads=4, n_kv_heads=2, head_dim=128, ffn_dim=512,
                        vocab_size=512, use_kernel=True, kernel_kind="t2g128")
    att = RM.Attention(args).to(torch.bfloat16)
    att.prepare_merged_weights(max_positions=700)
    att.q_norm.weight.data.copy_((1.0 + 0.1 * torch.randn(128, generator=gen)).to(torch.bfloat16))
    att.k_norm.weight.data.copy_((1.0 + 0.1 * torch.randn(128, generator=gen)).to(torch.bfloat16))
    M, sigma = 5, 24
    xqkv = bf16_randn(gen, M, (4 + 2 * 2) * 128, scale=2.0)
    pos = torch.tensor([0, 3, 77, 600, 699], dtype=torch.int64)
    kfull = torch.zeros(1, 2, sigma + M, 128, dtype=torch.bfloat16)
    vfull = torch.zeros(1, 2, sigma + M, 128, dtype=torch.bfloat16)
    xq = RM._fused_qkv_qknorm_rope_kv_write(
        xqkv, att.q_norm.weight, att.k_norm.weight, att.q_norm.eps, att.rope_cos, att.rope_sin, pos,
        kfull, vfull, att.q_dim, att.k_dim, 4, 2, 128, sigma)
    rec.update(rope_xqkv=u16(xqkv), rope_qw=u16(att.q_norm.weight.data), rope_kw=u16(att.k_norm.weight.data),
               rope_pos=pos.numpy(), rope_cos=u16(att.rope_cos), rope_sin=u16(att.rope_sin),
               rope_q=u16(xq[0].permute(1, 0, 2).contiguous()), rope_k=u16(kfull[0]), rope_v=u16(vfull[0]),
               rope_sigma=np.array([sigma]))

    # --- attention, explicit path of Attention.forward_sdlm_graph_kernel (model.py:996-1003)
    H, Hkv, sigma, M, D = 4, 2, 96, 9, 8
    cases = []
    for ci, (role, cache_len, n_pend, Mw) in enumerate([("verify", 70, 0, 9), ("draft", 41, 1, 9),
                                                         ("draft", 64, 4, 12), ("ar", 33, 0, 1)]):
        q = bf16_randn(gen, 1, H, Mw, 128, scale=1.5)
        k = bf16_randn(gen, 1, Hkv, sigma + Mw, 128, scale=1.5)
        v = bf16_randn(gen, 1, Hkv, sigma + Mw, 128)
        mask = reference_mask(ref, role, Mw, sigma, cache_len, n_pend, D)
        hpg = H // Hkv
        k_exp = k.unsqueeze(2).expand(-1, -1, hpg, -1, -1).reshape(1, H, sigma + Mw, 128)
        v_exp = v.unsqueeze(2).expand(-1, -1, hpg, -1, -1).reshape(1, H, sigma + Mw, 128)
        attn = torch.matmul(q, k_exp.transpose(2, 3)) * (1.0 / np.sqrt(128)) + mask
        attn = torch.nn.functional.softmax(attn, dim=-1, dtype=torch.float32).to(q.dtype)
        out = torch.matmul(attn, v_exp).squeeze(0).permute(1, 0, 2).contiguous().view(Mw, H * 128)
        # fp32 evaluation of the same softmax, for a tighter bound than the bf16 path gives
        a32 = torch.matmul(q.float(), k_exp.float().transpose(2, 3)) * (1.0 / np.sqrt(128)) + mask.float()
        o32 = torch.matmul(torch.softmax(a32, -1), v_exp.float()).squeeze(0).permute(1, 0, 2).reshape(Mw, H * 128)
        rec.update({f"attn{ci}_q": u16(q[0].permute(1, 0, 2).contiguous()), f"attn{ci}_k": u16(k[0]),
                    f"attn{ci}_v": u16(v[0]), f"attn{ci}_out": u16(out), f"attn{ci}_out32": o32.numpy(),
                    f"attn{ci}_meta": np.array([oracle_role(role), Mw, sigma, cache_len, n_pend, D, H, Hkv])})
        cases.append(ci)
    rec["attn_cases"] = np.array(cases)
    np.savez_compressed(out_path, **rec)
    print("wrote", out_path, os.path.getsize(out_path) >> 10, "KiB")


def oracle_role(role: str) -> int:
    return {"draft": 0, "verify": 1, "ar": 2}[role]


# ----------------------------------------------------------------------------- masks
def reference_atlas(ref, D: int, sigma: int, m_set, roles=("draft", "verify", "ar")):
    """A GraphAtlas object without captured graphs: enough state for the reference's own
    mask builders (the construction its CPU tests use, tests/test_bonsai_cpu.py:13-42)."""
    GA = ref.runtime.GraphAtlas
    atlas = GA.__new__(GA)
    atlas.device = torch.device("cpu")
    atlas.dtype = torch.bfloat16
    atlas.D = D
    atlas.segment_ladder = (sigma,)
    atlas.m_set = tuple(sorted(m_set))
    atlas.M_max = max(m_set)
    atlas.roles = tuple(roles)
    atlas.graphs = {}
    for M in atlas.m_set:
        if M == 1:
            atlas.graphs[(1, sigma, "ar")] = None
        else:
            for role in roles:
                if role != "ar":
                    atlas.graphs[(M, sigma, role)] = None
    atlas._build_mask_templates()
    atlas._build_verify_templates()
    return atlas


def reference_mask(ref, role: str, M: int, sigma: int, cache_len: int, n_pend: int, D: int):
    m_set = {M, D + 1, 1} | ({D} if M >= D else set())
    atlas = reference_atlas(ref, D, sigma, m_set)
    graph = types.SimpleNamespace(role=role, M=M, sigma=sigma, P=M - D,
                                  attn_mask=torch.full((1, 1, M, sigma + M), float("-inf"),
                                                       dtype=torch.bfloat16))
    if role == "ar" and (M, sigma) not in atlas.verify_templates:
        tmpl = torch.full((1, 1, M, sigma + M), float("-inf"), dtype=torch.bfloat16)
        for r in range(M):
            tmpl[:, :, r, sigma:sigma + r + 1] = 0.0
        atlas.verify_templates[(M, sigma)] = tmpl
    atlas.prepare_step(graph, cache_len, n_pend)
    return graph.attn_mask


def make_masks(ref, out_path):
    rec, index = {}, []
    sigma = 24
    for D, m_set in ((8, (1, 8, 9, 10, 12, 16, 17)), (4, (1, 4, 5, 6, 7, 8, 9))):
        atlas = reference_atlas(ref, D, sigma, m_set)
        for M in m_set:
            for role in (("ar",) if M == 1 else ("draft", "verify")):
                P = M - D
                pend_range = range(0, max(P, 0) + 2) if role == "draft" else (0,)
                for n_pend in pend_range:
                    for cache_len in (1, 2, 7, sigma):
                        if role == "draft" and M < D:
                            continue
                        graph = types.SimpleNamespace(
                            role=role, M=M, sigma=sigma, P=P,
                            attn_mask=torch.zeros(1, 1, M, sigma + M, dtype=torch.bfloat16))
                        atlas.prepare_step(graph, cache_len, n_pend)
                        vis = (graph.attn_mask[0, 0] == 0).numpy()
                        assert np.isneginf(graph.attn_mask[0, 0].float().numpy()[~vis]).all()
                        key = f"m_{len(index)}"
                        rec[key] = np.packbits(vis, axis=None)
                        index.append([oracle_role(role), D, M, sigma, cache_len, n_pend])
    rec["index"] = np.array(index, dtype=np.int32)
    np.savez_compressed(out_path, **rec)
    print("wrote", out_path, len(index), "masks", os.path.getsize(out_path) >> 10, "KiB")


# ----------------------------------------------------------------------------- known answers
def make_kats(ref, out_path):
    RG = ref.generate
    kats = {}
    # prefix acceptance (tests/test_bonsai_strict_verifier.py:18-36)
    verify = torch.arange(9)
    acc = []
    for prefix in range(9):
        draft = torch.arange(8)
        if prefix < 8:
            draft[prefix] = 99
        acc.append({"draft": draft.tolist(), "verify": verify.tolist(), "D": 8,
                    "accept": int(RG._fused_verify_accept(draft, verify, 8).item())})
    tied = torch.tensor([[3.0, 3.0], [0.0, 0.0], [2.0, 2.0]]).argmax(-1)
    for d in ([1, 0], [0, 1], [0, 0]):
        acc.append({"draft": d, "verify": tied.tolist(), "D": 2,
                    "accept": int(RG._fused_verify_accept(torch.tensor(d), tied, 2).item())})
    kats["verify_accept"] = acc
    # confidence chain (tests/test_orin_runtime.py:152-154) plus seeded random blocks
    chains = []
    logits = torch.tensor([[0., 0.], [20., 0.], [0., 0.], [20., 0.]])
    tok, n = RG._fused_draft_chain(logits, .9)
    chains.append({"logits": logits.tolist(), "tau": .9, "tokens": tok.tolist(), "length": int(n.item())})
    gen = torch.Generator().manual_seed(77)
    for i in range(6):
        lg = (torch.randn(8, 64, generator=gen) * 2).to(torch.bfloat16).float()
        for r in range(8):
            if (i + r) % 3:
                lg[r, (7 * r + i) % 64] = 12.0
        tok, n = RG._fused_draft_chain(lg, .9)
        chains.append({"logits": lg.tolist(), "tau": .9, "tokens": tok.tolist(), "length": int(n.item())})
    kats["draft_chain"] = chains
    # width selector (tests/test_generation_artifact_preflight.py:118-126)
    sel = {}
    for D, m_set in ((8, (1, 8, 9, 10, 12, 16, 17)), (4, (1, 4, 5, 6, 7, 8, 9))):
        atlas = types.SimpleNamespace(D=D, m_set=m_set)
        sel[str(D)] = {"m_set": list(m_set),
                       "widths": [RG._select_M_for_pending(atlas, n) for n in range(1, D + 2)]}
    kats["select_M"] = sel
    # registry
    RC = ref.contracts
    kats["registry"] = {"Q1_M": sorted(RC.Q1_M), "BONSAI_17B_NK": sorted(map(list, RC.BONSAI_17B_NK)),
                        "T2_4B_M": sorted(RC.T2_4B_M), "T2_4B_NK": sorted(map(list, RC.T2_4B_NK))}
    with open(out_path, "w") as f:
        json.dump(kats, f)
    print("wrote", out_path)


# ----------------------------------------------------------------------------- whole forward
def oracle_gemv_as_torch(O):
    """Drop-in for the reference's native call: the integer restatement, bf16 out."""
    def fn(a_int8, b_packed, s, ws):
        K = a_int8.shape[-1]
        a2 = a_int8.reshape(-1, K).numpy()
        _, y16, _ = O.t2_gemv(a2, b_packed.numpy().view(np.uint8), u16(ws), s.reshape(-1).numpy())
        return O.u16_to_torch(y16).reshape(*a_int8.shape[:-1], b_packed.shape[0])
    return fn


def build_reference_model(ref, O, cfg, state, max_positions):
    RM = ref.model
    RM.packed_int8_linear = oracle_gemv_as_torch(O)
    RM.t2g128_int8xint2_linear = RM.packed_int8_linear
    args = RM.ModelArgs(dim=cfg["dim"], n_layers=cfg["n_layers"], n_heads=cfg["n_heads"],
                        n_kv_heads=cfg["n_kv_heads"], head_dim=cfg["head_dim"], ffn_dim=cfg["ffn_dim"],
                        vocab_size=cfg["vocab_size"], norm_eps=cfg["norm_eps"],
                        rope_theta=cfg["rope_theta"], rope_original_max=cfg["rope_original_max"],
                        rope_factor=cfg["rope_factor"], tie_word_embeddings=True, use_kernel=True,
                        kernel_kind="t2g128", block_size=cfg["block_size"], causal_attn=True,
                        mask_token_id=cfg["mask_token_id"])
    m = RM.Transformer(args).to(torch.bfloat16)
    missing, unexpected = m.load_state_dict(state, strict=False)
    assert not unexpected and all("lm_head" in k for k in missing), (missing, unexpected)
    m.tie_weights()
    m._force_a8_lm_head = True
    m.eval()
    m.prepare_merged_weights(max_positions=max_positions)
    return m


def make_forward(ref, out_path):
    """Reference captured forward (model.py:1363-1404) on a tiny model vs nothing: records its
    logits; the oracle test compares OracleModel.forward with them."""
    from oracle import oracle as O
    from bitmtp_b200 import synthetic
    cfg = synthetic.make_config(synthetic.TINY, block_size=8)
    state = synthetic.make_state(cfg, seed=3)
    sigma, m_max = 64, 17
    m = build_reference_model(ref, O, cfg, state, sigma + m_max)
    # the reference pads the packed head to 151936 rows; shrink that for a 1000-word vocabulary
    head_w, head_s = O.OracleModel._pack_head(state["embed_tokens.weight"])
    m._lm_head_t2_w = torch.from_numpy(head_w.view(np.int8))
    m._lm_head_t2_scale = O.u16_to_torch(head_s)
    m._lm_head_t2_vocab = cfg["vocab_size"]
    rec = {"cfg": np.frombuffer(json.dumps(cfg).encode(), dtype=np.uint8), "seed": np.array([3]),
           "sigma": np.array([sigma]), "m_max": np.array([m_max])}
    gen = torch.Generator().manual_seed(11)
    L, Hkv = cfg["n_layers"], cfg["n_kv_heads"]
    cases = [("ar", 1, 20, 0), ("verify", 9, 30, 0), ("draft", 9, 30, 1), ("draft", 12, 25, 3),
             ("draft", 16, 40, 8)]
    for ci, (role, M, cache_len, n_pend) in enumerate(cases):
        D = cfg["block_size"]
        kv = (torch.randn(2, L, 1, Hkv, sigma + m_max, 128, generator=gen) * 0.5).to(torch.bfloat16)
        kv0 = kv.clone()
        tokens = torch.randint(0, cfg["vocab_size"], (M,), generator=gen)
        positions = torch.arange(cache_len, cache_len + M)
        mask = reference_mask(ref, role, M, sigma, cache_len, n_pend, D)
        kv_full = [(kv[0, i][:, :, :sigma + M, :], kv[1, i][:, :, :sigma + M, :]) for i in range(L)]
        if role == "draft":
            ls, le = M - D, M
        elif role == "verify":
            ls, le = 0, min(D + 1, M)
        else:
            ls, le = 0, M
        logits = m.forward_sdlm_decode_graph_kernel(tokens, positions, kv_full, M, mask, ls, le, "t2")
        rec.update({f"c{ci}_meta": np.array([oracle_role(role), M, cache_len, n_pend, ls, le]),
                    f"c{ci}_tokens": tokens.numpy(), f"c{ci}_positions": positions.numpy(),
                    f"c{ci}_kv_in": u16(kv0), f"c{ci}_logits": logits.numpy(),
                    f"c{ci}_kv_out_sha": np.frombuffer(sha(u16(kv)).encode(), dtype=np.uint8),
                    f"c{ci}_kv_rows": u16(kv[:, :, 0, :, sigma:sigma + M, :])})
    rec["n_cases"] = np.array([len(cases)])
    np.savez_compressed(out_path, **rec)
    print("wrote", out_path, os.path.getsize(out_path) >> 10, "KiB")


# ----------------------------------------------------------------------------- token streams
PREFILL_CHUNK = 16


class OracleBackedModel:
    """What the reference's decode loops need from a `Transformer`: `.args` and a prefill.

    The prefill runs the packed integer path in AR-causal chunks of PREFILL_CHUNK rows
    (rows are written in place, sigma == cache_len == chunk start), which is also what the
    B200 runtime does; the reference's own prefill multiplies fake-quantised bf16
    activations with unpacked bf16 weights in cuBLAS, i.e. the same quantised product with
    bf16 roundings in between."""

    def __init__(self, om, args):
        self.om, self.args = om, args

    def forward_sdlm_prefill(self, token_values, cache, positions=None, block_size=1, fast=False,
                             causal_attn=True):
        om = self.om
        seq = int(token_values.shape[0])
        kv = om.new_kv(seq, PREFILL_CHUNK)
        logits = np.empty((seq, om.vocab), dtype=np.float32)
        toks = token_values.numpy()
        for c0 in range(0, seq, PREFILL_CHUNK):
            n = min(PREFILL_CHUNK, seq - c0)
            logits[c0:c0 + n] = om.forward(toks[c0:c0 + n], np.arange(c0, c0 + n), kv, sigma=c0, role=2,
                                           cache_len=c0, n_pend=0)
        from oracle import oracle as O
        for i in range(om.L):
            cache[i] = (O.u16_to_torch(kv[0, i, :, :, :seq, :].copy()),
                        O.u16_to_torch(kv[1, i, :, :, :seq, :].copy()))
        return torch.from_numpy(logits)


    def forward_sdlm_decode(self, token_values, positions, cache, block_size, cache_len=None, causal_attn=True):
        """The eager block decode the reference's confidence loop opens with (fast_generate.py:322-351): the D rows
        [anchor, MASK ...] over the prompt's K/V with the key just before the block hidden
        (model.py:462-505) - a draft-role forward with nothing pending, by the oracle."""
        from oracle import oracle as O
        om = self.om
        D = int(token_values.shape[0])
        past = int(cache[0][0].shape[2]) if cache_len is None else int(cache_len)
        kv = om.new_kv(past, D)
        for i in range(om.L):
            kv[0, i, 0, :, :past, :] = O.torch_to_u16(cache[i][0][0, :, :past, :])
            kv[1, i, 0, :, :past, :] = O.torch_to_u16(cache[i][1][0, :, :past, :])
        lg = om.forward(token_values.numpy(), positions.numpy(), kv, sigma=past, role=0, cache_len=past, n_pend=0,
                        logits_start=0, logits_end=D)
        return torch.from_numpy(lg), None, None


def make_cpu_atlas(ref, om, args, segment_ladder, m_set, roles, check_masks=True):
    """A GraphAtlas whose graphs replay the CPU oracle forward; everything else (mask
    templates, prepare_step, commit_kv, migrate_segment, select_segment) is the reference's
    own code running on CPU tensors."""
    from oracle import oracle as O
    GA = ref.runtime.GraphAtlas
    atlas = GA.__new__(GA)
    atlas.model, atlas.args = None, args
    atlas.device, atlas.dtype = torch.device("cpu"), torch.bfloat16
    atlas.segment_ladder = tuple(sorted(set(segment_ladder)))
    atlas.m_set = tuple(sorted(set(m_set)))
    atlas.roles = tuple(roles)
    atlas.D, atlas.M_max = args.block_size, max(m_set)
    atlas.vocab_size, atlas.n_layers = args.vocab_size, args.n_layers
    atlas.n_kv, atlas.head_dim = args.n_kv_heads, args.head_dim
    atlas._allocate_shared_kv()
    atlas._allocate_input_bufs()
    atlas.graphs = {}
    D = atlas.D
    for sigma in atlas.segment_ladder:
        kv_np = atlas.kv_buffers[sigma].view(torch.int16).numpy().view(np.uint16)
        for M in atlas.m_set:
            for role in (("ar",) if M == 1 else tuple(r for r in roles if r != "ar")):
                if M == 1 and "ar" not in roles:
                    continue
                P = M - D
                ls, le = {"ar": (0, M), "draft": (P, M), "verify": (0, min(D + 1, M))}[role]
                g = types.SimpleNamespace(
                    tokens_buf=atlas.tokens_m[M], positions_buf=atlas.positions_m[M],
                    attn_mask=torch.full((1, 1, M, sigma + M), float("-inf"), dtype=torch.bfloat16),
                    logits_out=torch.zeros(le - ls, args.vocab_size), M=M, sigma=sigma, role=role, P=P,
                    logits_start=ls, logits_end=le, lm_head_precision="t2", state=None)

                def replay(g=g, kv_np=kv_np):
                    cache_len, n_pend = g.state
                    rid = oracle_role(g.role)
                    if check_masks:
                        want = (g.attn_mask[0, 0] == 0).numpy()
                        got = O.mask_matrix(rid, g.M, g.sigma, cache_len, n_pend, g.P)
                        assert np.array_equal(want, got), (g.role, g.M, cache_len, n_pend)
                    lg = om.forward(g.tokens_buf.numpy(), g.positions_buf.numpy(), kv_np, g.sigma, rid,
                                    cache_len, n_pend, g.logits_start, g.logits_end)
                    g.logits_out.copy_(torch.from_numpy(lg))

                g.cuda_graph = types.SimpleNamespace(replay=replay)
                atlas.graphs[(M, sigma, role)] = g
    atlas._build_mask_templates()
    atlas._build_verify_templates()
    real_prepare = GA.prepare_step

    def prepare_step(graph, cache_len, n_pend, causal_attn=True):
        real_prepare(atlas, graph, cache_len, n_pend, causal_attn)
        graph.state = (int(cache_len), int(n_pend))

    atlas.prepare_step = prepare_step
    return atlas


def run_reference_loop(ref, O, cfg, state, mode, prompt, new_tokens, accept_kind, ladder, m_set, accept_seed=0,
                       eos_ids=(), exact_m1_verify=False):
    RG = ref.generate
    om = O.OracleModel(cfg, state, max_positions=max(ladder) + max(m_set))
    args = ref.model.ModelArgs(dim=cfg["dim"], n_layers=cfg["n_layers"], n_heads=cfg["n_heads"],
                               n_kv_heads=cfg["n_kv_heads"], head_dim=cfg["head_dim"],
                               ffn_dim=cfg["ffn_dim"], vocab_size=cfg["vocab_size"],
                               block_size=cfg["block_size"], mask_token_id=cfg["mask_token_id"],
                               use_kernel=True, kernel_kind="t2g128")
    model = OracleBackedModel(om, args)
    roles = ("ar",) if mode == "ar" else ("ar", "draft", "verify")
    atlas = make_cpu_atlas(ref, om, args, ladder, m_set, roles)
    D = cfg["block_size"]
    torch.cuda.synchronize = lambda *a, **k: None
    torch.cuda.empty_cache = lambda *a, **k: None
    orig_chain, orig_accept, orig_conf = RG._fused_draft_chain, RG._fused_verify_accept, RG._confidence_accept
    from bitmtp_b200 import synthetic
    policy = synthetic.AcceptancePolicy(accept_kind, D, seed=accept_seed)

    def conf_accept(logits, threshold, eos_ids, Dd):
        # _confidence_accept (fast_generate.py:354-386) with the oracle's confidences and, where the plan says
        # so, the policy's chain length; no end-of-sequence id is special for random-init weights
        idx, n, _ = O.draft_chain(logits.numpy(), float(threshold))
        a = policy.chain_count()
        n = n if a is None else a
        toks, hit = [], False
        for t in idx[:n]:                      # truncate at the first end-of-sequence id, which is not emitted
            if int(t) in eos_ids:
                hit = True
                break
            toks.append(int(t))
        return toks, len(toks), hit

    def chain(logits, threshold):
        idx, n, _ = O.draft_chain(logits.numpy(), float(threshold))
        a = policy.chain_count()
        return torch.from_numpy(idx), torch.tensor(n if a is None else a)

    def accept(draft_tokens, verify_tokens, Dd):
        a = policy.accept_count()
        return orig_accept(draft_tokens, verify_tokens, Dd) if a is None else torch.tensor(a)

    RG._fused_draft_chain, RG._fused_verify_accept, RG._confidence_accept = chain, accept, conf_accept
    try:
        fn = {"ar": RG.fast_ar_generate, "spec": RG.fast_speculative_generate,
              "hybrid": RG.fast_hybrid_generate, "conf": RG.fast_confidence_generate}[mode]
        kw = dict(exact_m1_verify=True) if exact_m1_verify else {}
        out, stats = fn(model, atlas, prompt, max_gen_len=new_tokens, eos_ids=frozenset(eos_ids), **kw)
    finally:
        RG._fused_draft_chain, RG._fused_verify_accept, RG._confidence_accept = orig_chain, orig_accept, orig_conf
    keep = {k: v for k, v in stats.items() if not k.endswith("_time") and k != "ttft"}
    return out.tolist(), keep


def make_streams(ref, out_path, full=False):
    from oracle import oracle as O
    from bitmtp_b200 import synthetic
    O.lib()
    records = []
    geoms = {"tiny": synthetic.TINY,
             "tiny_g4": dict(synthetic.TINY, n_heads=4, n_kv_heads=1, dim=512, ffn_dim=768)}
    # acceptance: "free" = measured, "forced" = whole block, "categorical" = seeded draw per step
    # (synthetic.AcceptancePolicy, seed = prompt length)
    plans = [("tiny", 8, "ar", "free", 24, 20), ("tiny", 8, "spec", "free", 40, 48),
             ("tiny", 8, "hybrid", "free", 40, 48), ("tiny", 8, "hybrid", "forced", 40, 64),
             ("tiny", 8, "spec", "forced", 33, 40), ("tiny_g4", 8, "hybrid", "forced", 50, 40),
             ("tiny_g4", 8, "hybrid", "free", 50, 40), ("tiny", 4, "hybrid", "forced", 21, 30),
             ("tiny", 4, "spec", "free", 21, 30), ("tiny", 8, "hybrid", "categorical", 37, 96),
             ("tiny_g4", 8, "spec", "categorical", 29, 60), ("tiny", 4, "hybrid", "categorical", 19, 40),
             # the confidence policy: its first block is the reference's eager block decode
             ("tiny", 8, "conf", "free", 24, 40), ("tiny", 8, "conf", "forced", 33, 48),
             ("tiny_g4", 8, "conf", "categorical", 29, 60), ("tiny", 4, "conf", "categorical", 19, 40)]
    for (gname, D, mode, accept_kind, plen, ntok) in plans:
        cfg = synthetic.make_config(geoms[gname], block_size=D)
        state = synthetic.make_state(cfg, seed=7)
        prompt = synthetic.random_prompt(plen, cfg["vocab_size"], seed=plen)
        m_set = (1, 8, 9, 10, 12, 16, 17) if D == 8 else (1, 4, 5, 6, 7, 8, 9)
        toks, stats = run_reference_loop(ref, O, cfg, state, mode, prompt, ntok, accept_kind, (64, 256), m_set,
                                         accept_seed=plen)
        records.append(dict(geometry=gname, cfg=cfg, state_seed=7, prompt_seed=plen, prompt_len=plen,
                            new_tokens=ntok, mode=mode, forced=accept_kind == "forced", accept=accept_kind,
                            accept_seed=plen, ladder=[64, 256], m_set=list(m_set), tokens=toks, stats=stats))
        print(gname, D, mode, accept_kind, len(toks), "tokens", "iters", stats.get("n_iters"),
              "verify paths", stats.get("n_verify_path"))
    # End-of-sequence handling: the same loops with one id of their own stream declared end-of-sequence (the
    # id nearest to 60 % of the stream that has not occurred before it), so that the policies stop inside a block.
    for (gname, D, mode, accept_kind, plen, ntok) in [("tiny", 8, "ar", "free", 24, 20), ("tiny", 8, "spec", "forced", 33, 40),
                                                      ("tiny_g4", 8, "spec", "categorical", 29, 60),
                                                      ("tiny", 8, "hybrid", "categorical", 37, 96),
                                                      ("tiny", 8, "hybrid", "forced", 40, 64),
                                                      ("tiny_g4", 8, "conf", "categorical", 29, 60),
                                                      ("tiny", 8, "conf", "forced", 33, 48)]:
        base = next(r for r in records if (r["geometry"], r["cfg"]["block_size"], r["mode"], r["accept"], r["prompt_len"])
                    == (gname, D, mode, accept_kind, plen) and not r.get("eos_ids"))
        toks = base["tokens"]
        firsts = [i for i in range(2, len(toks)) if toks[i] not in toks[:i]]
        k = min(firsts, key=lambda i: abs(i - 0.6 * len(toks))) if firsts else 0     # a one-id stream: its first output
        eos = [toks[k]]
        cfg = base["cfg"]
        state = synthetic.make_state(cfg, seed=7)
        prompt = synthetic.random_prompt(plen, cfg["vocab_size"], seed=plen)
        got, stats = run_reference_loop(ref, O, cfg, state, mode, prompt, ntok, accept_kind, (64, 256), base["m_set"],
                                        accept_seed=plen, eos_ids=eos)
        assert got == toks[:len(got)] and len(got) < len(toks), (mode, len(got), len(toks))
        records.append(dict(base, tokens=got, stats=stats, eos_ids=eos))
        print(gname, D, mode, accept_kind, "eos", eos, "at", k, "->", len(got), "tokens")
    # The width-1 verifier (`exact_m1_verify=True`): every draft token is checked by AR replays instead of one
    # width-(D+1) replay; the accepted length is then measured, not drawn.
    for (gname, D, mode, accept_kind, plen, ntok) in [("tiny_g4", 8, "spec", "categorical", 29, 40),
                                                      ("tiny", 8, "hybrid", "categorical", 37, 64),
                                                      ("tiny", 4, "hybrid", "categorical", 19, 40)]:
        cfg = synthetic.make_config(geoms[gname], block_size=D)
        state = synthetic.make_state(cfg, seed=7)
        prompt = synthetic.random_prompt(plen, cfg["vocab_size"], seed=plen)
        m_set = (1, 8, 9, 10, 12, 16, 17) if D == 8 else (1, 4, 5, 6, 7, 8, 9)
        toks, stats = run_reference_loop(ref, O, cfg, state, mode, prompt, ntok, accept_kind, (64, 256), m_set,
                                         accept_seed=plen, exact_m1_verify=True)
        records.append(dict(geometry=gname, cfg=cfg, state_seed=7, prompt_seed=plen, prompt_len=plen,
                            new_tokens=ntok, mode=mode, forced=False, accept=accept_kind, accept_seed=plen,
                            ladder=[64, 256], m_set=list(m_set), tokens=toks, stats=stats, exact_m1_verify=True))
        print(gname, D, mode, accept_kind, "exact-m1", len(toks), "tokens", "verify paths", stats.get("n_verify_path"),
              "accepted", stats.get("accepted_drafts"))
    with open(out_path, "w") as f:
        json.dump(records, f)
    print("wrote", out_path)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("BITMTP_REFERENCE"), required="BITMTP_REFERENCE" not in os.environ,
                    help="root of the reference checkout")
    ap.add_argument("--only", default="ops,masks,kats,forward,streams")
    a = ap.parse_args()
    ref = load_reference(a.ref)
    todo = set(a.only.split(","))
    with torch.no_grad():
        if "ops" in todo:
            make_ops(ref, os.path.join(HERE, "ops.npz"))
        if "masks" in todo:
            make_masks(ref, os.path.join(HERE, "masks.npz"))
        if "kats" in todo:
            make_kats(ref, os.path.join(HERE, "kats.json"))
        if "forward" in todo:
            make_forward(ref, os.path.join(HERE, "forward.npz"))
        if "streams" in todo:
            make_streams(ref, os.path.join(HERE, "streams.json"))


if __name__ == "__main__":
    main()
