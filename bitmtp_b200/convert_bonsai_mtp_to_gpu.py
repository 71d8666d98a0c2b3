"""Hugging Face Bonsai (Qwen3) safetensors -> packed T2-g128 GPU checkpoint.

Writes the same directory the reference's converter writes
(src/bonsai_sft/gpu/convert_bonsai_mtp_to_gpu.py:150-278), so that either runtime loads it:

    bonsai_gpu_config.json   dim, n_layers, n_heads, n_kv_heads, head_dim, ffn_dim, vocab_size,
                             norm_eps, rope_theta, rope_original_max, rope_factor,
                             tie_word_embeddings, block_size, causal_attn, mask_token_id,
                             kernel_kind="t2g128", quantize_embedding
    model_state_t2g128.pt    torch.save(dict): embed_tokens.weight bf16 [vocab, dim] on the
                             ternary grid; norm weights bf16; for each of the seven projections
                             per layer `.weight` int8 [out, in/4] (four natural-order codes per
                             byte, value+2) and `.weight_scale` bf16 [out, in/128]
    model_state_fp16.pt      optional: the same tensors unpacked (frozen bf16 grid)

Same command line:
    python -m bitmtp_b200.convert_bonsai_mtp_to_gpu --src HF_DIR --out OUT_DIR [--no-kernel] [--no-fp16]
With the defaults this is offline CPU code and touches no CUDA.  Two additions of this build:
    --device cuda:0   freeze and pack each tensor with the device kernel (bm_pack_t2_g128); same bytes
    --safetensors     also write model_state_t2g128.safetensors (same tensors, same names), which
                      `generate.build_model` memory-maps straight to the device when it is present
"""
from __future__ import annotations

import argparse
import json
import os
from typing import Dict

import torch

from .checkpoint_validation import validate_hf_checkpoint, validate_sdlm_config
from .contracts import validate_public_model_scope
from .synthetic import GROUP, pack_t2_g128

# HF name fragment -> GPU name fragment (convert_bonsai_mtp_to_gpu.py:37-66)
_RENAMES = (("model.embed_tokens.", "embed_tokens."), ("model.norm.", "norm."),
            ("model.layers.", "layers."), (".self_attn.", ".attention."), (".mlp.", ".feed_forward."))
_PROJECTIONS = ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj")
_EMBED = "embed_tokens.weight"


def hf_to_gpu_key(name: str) -> str:
    for old, new in _RENAMES:
        name = name.replace(old, new, 1)
    return name


def is_ternary_tensor(gpu_key: str) -> bool:
    return gpu_key == _EMBED or any(gpu_key.endswith(f".{p}.weight") for p in _PROJECTIONS)


@torch.no_grad()
def freeze_ternary_g128(w: torch.Tensor) -> torch.Tensor:
    """Latent weights -> the {-s, 0, +s} grid with s the absmax of each 128-group, the
    deterministic rounding the QAT forward applies (src/bonsai_sft/ternary_modules.py:22-34,
    86-93).  Computed in fp32, returned in the input dtype."""
    n, k = w.shape
    g = w.float().view(n, k // GROUP, GROUP)
    s = g.abs().amax(dim=-1, keepdim=True).clamp_min(1e-8)
    return (torch.round(g / s).clamp_(-1, 1) * s).view(n, k).to(w.dtype)


def gpu_config(hf: dict) -> dict:
    """bonsai_gpu_config.json from the HF config (convert_bonsai_mtp_to_gpu.py:257-275)."""
    rope = hf["rope_scaling"]
    return {
        "dim": hf["hidden_size"], "n_layers": hf["num_hidden_layers"],
        "n_heads": hf["num_attention_heads"], "n_kv_heads": hf["num_key_value_heads"],
        "head_dim": hf["head_dim"], "ffn_dim": hf["intermediate_size"],
        "vocab_size": hf["vocab_size"], "norm_eps": hf["rms_norm_eps"],
        "rope_theta": hf["rope_theta"],
        "rope_original_max": rope["original_max_position_embeddings"], "rope_factor": rope["factor"],
        "tie_word_embeddings": bool(hf["tie_word_embeddings"]),
        "block_size": int(hf.get("block_size", 8)), "causal_attn": bool(hf.get("causal_attn", True)),
        "mask_token_id": int(hf.get("text_mask_token_id", 151654)),
        "kernel_kind": "t2g128", "quantize_embedding": True,
    }


@torch.no_grad()
def freeze_and_pack(t: torch.Tensor, device: str = "cpu"):
    """(frozen bf16 [N, K], packed int8 [N, K/4], scale bf16 [N, K/128]) of one bf16 weight, all on the CPU.
    `device` "cpu" runs the torch expressions above; a CUDA device runs the packing kernel instead
    (identical bytes; tests/test_pack_gpu.py compares the two)."""
    if torch.device(device).type == "cpu":
        frozen = freeze_ternary_g128(t)
        return (frozen,) + tuple(pack_t2_g128(frozen))
    from . import ops
    packed, scale, frozen = ops.pack_t2_g128(t.to(device).contiguous(), want_frozen=True)
    return frozen.cpu(), packed.cpu(), scale.cpu()


@torch.no_grad()
def convert(src_ckpt_dir: str, out_dir: str, pack_kernel: bool = True, pack_fp16: bool = True,
            quant: str = "ternary", quantize_embedding: bool = True, *, device: str = "cpu",
            safetensors_copy: bool = False) -> None:
    """Freeze the HF weights on the ternary g128 grid and write the packed checkpoint.
    The source is checked first (checkpoint_validation.py); nothing is written unless every tensor
    converted; an existing output is never touched."""
    if quant != "ternary":
        raise ValueError("quant must be 'ternary' (this build converts T2-g128 checkpoints only)")
    if os.path.lexists(out_dir):
        raise ValueError("conversion output already exists; use a new output directory")
    if not pack_kernel and not pack_fp16:
        raise ValueError("at least one output format must be enabled")
    if not quantize_embedding:
        raise ValueError("ternary requires quantized embedding/head; --keep-embedding-fp is Q1-only")
    from safetensors import safe_open
    # source config, shard containers and every core tensor's key / shape / dtype, before anything is written
    hf, shards = validate_hf_checkpoint(src_ckpt_dir)
    validate_sdlm_config(src_ckpt_dir, hf)
    cfg = gpu_config(hf)
    packed: Dict[str, torch.Tensor] = {}
    dense: Dict[str, torch.Tensor] = {}
    for shard in shards:
        with safe_open(os.path.join(src_ckpt_dir, shard), framework="pt", device="cpu") as f:
            for name in f.keys():
                if name.startswith("lm_head.") and cfg["tie_word_embeddings"]:
                    continue                              # tied to the embedding at load
                key = hf_to_gpu_key(name)
                t = f.get_tensor(name).to(torch.bfloat16)
                if not is_ternary_tensor(key) or t.dim() != 2 or t.shape[1] % GROUP != 0:
                    packed[key] = dense[key] = t          # norms stay bf16
                    continue
                frozen, codes, scale = freeze_and_pack(t, device)
                dense[key] = frozen
                if key == _EMBED:
                    packed[key] = frozen                  # gathered, not multiplied: stays bf16
                else:
                    packed[key], packed[key.replace(".weight", ".weight_scale")] = codes, scale
    expect = 2 + cfg["n_layers"] * (4 + 2 * len(_PROJECTIONS))
    if len(packed) != expect:
        raise ValueError(f"checkpoint has {len(packed)} converted tensors, expected {expect}")
    os.makedirs(out_dir, exist_ok=False)
    if pack_fp16:
        torch.save(dense, os.path.join(out_dir, "model_state_fp16.pt"))
    if pack_kernel:
        torch.save(packed, os.path.join(out_dir, "model_state_t2g128.pt"))
        if safetensors_copy:
            from safetensors.torch import save_file
            save_file({k: v.contiguous() for k, v in packed.items()},
                      os.path.join(out_dir, "model_state_t2g128.safetensors"))
    with open(os.path.join(out_dir, "bonsai_gpu_config.json"), "w") as f:
        json.dump(cfg, f, indent=2)
    print(f"[convert] wrote {out_dir}: {len(packed)} tensors, kernel_kind=t2g128")


def make_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(description="Convert public Bonsai T2 checkpoints: 1.7B D4/D8 or 4B D8.")
    ap.add_argument("--src", required=True, help="HF safetensors directory of SFT or MTP checkpoint")
    ap.add_argument("--out", required=True, help="output directory")
    ap.add_argument("--no-kernel", action="store_true", help="skip the packed T2 dump")
    ap.add_argument("--no-fp16", action="store_true", help="skip the frozen bf16 dump")
    ap.add_argument("--quant", choices=("ternary",), default="ternary")
    ap.add_argument("--keep-embedding-fp", action="store_true",
                    help="legacy compatibility flag; rejected by the T2-only release")
    ap.add_argument("--device", default="cpu", help="cpu (default), or a CUDA device to pack with the device kernel")
    ap.add_argument("--safetensors", action="store_true",
                    help="also write model_state_t2g128.safetensors for memory-mapped loading")
    return ap


def main(argv=None):
    ap = make_parser()
    args = ap.parse_args(argv)
    try:
        with open(os.path.join(args.src, "config.json")) as f:
            validate_public_model_scope(json.load(f), hf=True, quant=args.quant,
                                        quantize_embedding=not args.keep_embedding_fp)
    except (OSError, ValueError, TypeError) as error:
        ap.error(str(error))
    convert(args.src, args.out, pack_kernel=not args.no_kernel, pack_fp16=not args.no_fp16,
            quant=args.quant, quantize_embedding=not args.keep_embedding_fp, device=args.device,
            safetensors_copy=args.safetensors)


if __name__ == "__main__":
    main()
