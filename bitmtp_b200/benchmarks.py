"""Decode workloads behind bench.py: the Bonsai-architecture hybrid MTP decode on synthetic
weights (GPU arm) and its bounded CPU counterpart on the oracle (reference arm).

Definitions follow the reference's benchmark adapter: decode speed = timed decode tokens /
decode seconds, the first token and the prefill excluded
(benchmarks/bonsai_adapter.py:55-58, src/bonsai_sft/gpu/fast_generate.py:1147-1172).
"""
from __future__ import annotations

import json
import os
import time

import torch

GEOMETRIES = {"1p7b": "BONSAI_1P7B", "4b": "BONSAI_4B", "tiny": "TINY"}
D8_WIDTHS = (1, 8, 9, 10, 12, 16, 17)


def _forced_hooks(FG, D):
    chain, accept = FG._fused_draft_chain, FG._fused_verify_accept

    def forced_chain(logits, threshold):
        idx, n = chain(logits, threshold)
        return idx, torch.full_like(n, D)

    def forced_accept(draft, verify, Dd):
        return torch.full_like(accept(draft, verify, Dd), Dd)

    return forced_chain, forced_accept


def build_decode(model_name: str, device, prompt_len: int, new_tokens: int, seed: int = 0):
    """(model, atlas, cfg) for a synthetic checkpoint of the named geometry."""
    from . import generate, synthetic
    from .fast_runtime import GraphAtlas
    geometry = getattr(synthetic, GEOMETRIES[model_name])
    cfg = synthetic.make_config(geometry, block_size=8)
    sd = synthetic.device_state(cfg, device, seed=seed)
    head_w, head_s = sd.pop("_head.weight"), sd.pop("_head.weight_scale")
    model = generate.model_from_state(generate.args_from_config(cfg), sd, device)
    n_pad = (cfg["vocab_size"] + 31) // 32 * 32
    if n_pad != cfg["vocab_size"]:
        model.prepare_t2_lm_head()
    else:
        model._lm_head_t2_w, model._lm_head_t2_scale = head_w, head_s
        model._lm_head_t2_vocab, model._lm_head_n_pad = cfg["vocab_size"], n_pad
    need = prompt_len + new_tokens + max(D8_WIDTHS)
    ladder = tuple(s for s in (256, 1024, 4096) if s >= need)[:1] or (4096,)
    model.prepare_merged_weights(max_positions=ladder[0] + max(D8_WIDTHS))
    atlas = GraphAtlas(model, model.args, device, segment_ladder=ladder, m_set=D8_WIDTHS,
                       roles=("ar", "draft", "verify"), capture_verbose=False)
    return model, atlas, cfg
