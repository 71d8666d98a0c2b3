"""Model loading for the packed T2-g128 runtime.

Mirror of the loader half of `bonsai_sft.gpu.generate`
(src/bonsai_sft/gpu/generate.py:30-68): `load_args_from_ckpt` and `build_model` read
`bonsai_gpu_config.json` + `model_state_t2g128.pt` in the reference's layout.  The
reference file also holds uncaptured eager decoders; the captured runtime
(`fast_runtime`, `fast_generate`) is the path this build provides.
"""
from __future__ import annotations

import json
import os

import torch

from .model import ModelArgs, Transformer

_BONSAI_EOS_IDS = frozenset([151643, 151645])  # <|endoftext|>, <|im_end|>


def args_from_config(cfg: dict, use_kernel: bool = True) -> ModelArgs:
    return ModelArgs(
        dim=cfg["dim"], n_layers=cfg["n_layers"], n_heads=cfg["n_heads"],
        n_kv_heads=cfg["n_kv_heads"], head_dim=cfg["head_dim"], ffn_dim=cfg["ffn_dim"],
        vocab_size=cfg["vocab_size"], norm_eps=cfg["norm_eps"], rope_theta=cfg["rope_theta"],
        rope_original_max=cfg["rope_original_max"], rope_factor=cfg["rope_factor"],
        tie_word_embeddings=cfg["tie_word_embeddings"], block_size=cfg["block_size"],
        causal_attn=cfg["causal_attn"], mask_token_id=cfg["mask_token_id"],
        use_kernel=use_kernel, kernel_kind=cfg.get("kernel_kind", "q1"))


def load_args_from_ckpt(ckpt_dir: str, use_kernel: bool) -> ModelArgs:
    with open(os.path.join(ckpt_dir, "bonsai_gpu_config.json"), "r") as f:
        return args_from_config(json.load(f), use_kernel)


def model_from_state(args: ModelArgs, state: dict, device) -> Transformer:
    """Instantiate on `device` and load a packed state dict (tensors may live anywhere)."""
    if args.kernel_kind != "t2g128" or not args.use_kernel:
        raise RuntimeError("bitmtp_b200 serves packed T2-g128 checkpoints through its kernels only "
                           f"(kernel_kind={args.kernel_kind!r}, use_kernel={args.use_kernel})")
    with torch.device("meta"):
        m = Transformer(args)
    m = m.to_empty(device=device)
    for mod in m.modules():                       # non-persistent buffers are not in the state dict
        if hasattr(mod, "inv_freq"):
            from .model import _yarn_inv_freq
            mod.inv_freq = _yarn_inv_freq(args.head_dim, args.rope_theta, args.rope_factor,
                                          args.rope_original_max, args.rope_beta_fast,
                                          args.rope_beta_slow).to(device)
    # floating-point parameters are bf16, packed codes stay int8
    for p in m.parameters():
        if p.is_floating_point():
            p.data = p.data.to(torch.bfloat16)
    missing, unexpected = m.load_state_dict(state, strict=False)
    real_missing = [k for k in missing if "lm_head" not in k]
    if real_missing:
        raise RuntimeError(f"Missing weights: {real_missing[:5]}")
    if unexpected:
        raise RuntimeError(f"Unexpected weights: {unexpected[:5]}")
    m.tie_weights()
    m._force_a8_lm_head = True
    m.eval()
    return m


def build_model(ckpt_dir: str, use_kernel: bool, device) -> Transformer:
    """generate.py:48-68: read the config, build the module tree in bf16, load
    `model_state_t2g128.pt`, tie the head to the embedding.  When the converter also wrote
    `model_state_t2g128.safetensors`, that file is memory-mapped and each tensor copied straight to
    the device, with no unpickling and no host copy of the whole state."""
    args = load_args_from_ckpt(ckpt_dir, use_kernel=use_kernel)
    return model_from_state(args, load_packed_state(ckpt_dir, device), device)


def load_packed_state(ckpt_dir: str, device) -> dict:
    st = os.path.join(ckpt_dir, "model_state_t2g128.safetensors")
    if os.path.isfile(st):
        from safetensors.torch import load_file
        return load_file(st, device=str(device))
    return torch.load(os.path.join(ckpt_dir, "model_state_t2g128.pt"), map_location=device)
