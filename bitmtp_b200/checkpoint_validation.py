"""Read-only checks of a Hugging Face Bonsai (Qwen3) checkpoint before the converter writes anything.

Same acceptance rules and error texts as the reference's preflight
(src/bonsai_sft/gpu/checkpoint_validation.py:17-126) and its MTP metadata check
(src/bonsai_sft/export_ternary.py:32-54): the config fields the GPU model needs, every core tensor of
every layer present exactly once across the safetensors shards, with the expected shape and a
floating-point dtype.  Only metadata is read (safetensors headers); tensor values are not inspected.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Tuple

GROUP = 128
_FLOAT_DTYPES = ("F16", "BF16", "F32", "F64")

# (config key, must be an integer)
_POSITIVE_FIELDS = (("hidden_size", True), ("num_hidden_layers", True), ("num_attention_heads", True),
                    ("num_key_value_heads", True), ("head_dim", True), ("intermediate_size", True),
                    ("vocab_size", True), ("rms_norm_eps", False), ("rope_theta", False))


def _require_positive(value, name: str, integer: bool) -> None:
    ok = type(value) is int if integer else type(value) in (int, float)
    if not ok or not math.isfinite(value) or value <= 0:
        kind = "integer" if integer else "number"
        raise ValueError(f"config.json: {name} must be a positive {kind}")


def expected_tensor_shapes(config: dict) -> Dict[str, Tuple[int, ...]]:
    """HF tensor name -> shape for everything the GPU model consumes.  Projections are sized from the
    query / key-value widths (heads x head_dim), which differ from the hidden size on the 4B model."""
    dim, vocab, hd = config["hidden_size"], config["vocab_size"], config["head_dim"]
    q_dim, kv_dim = config["num_attention_heads"] * hd, config["num_key_value_heads"] * hd
    ffn = config["intermediate_size"]
    per_layer = {
        "input_layernorm": (dim,), "post_attention_layernorm": (dim,),
        "self_attn.q_norm": (hd,), "self_attn.k_norm": (hd,),
        "self_attn.q_proj": (q_dim, dim), "self_attn.k_proj": (kv_dim, dim), "self_attn.v_proj": (kv_dim, dim),
        "self_attn.o_proj": (dim, q_dim),
        "mlp.gate_proj": (ffn, dim), "mlp.up_proj": (ffn, dim), "mlp.down_proj": (dim, ffn),
    }
    shapes: Dict[str, Tuple[int, ...]] = {"model.embed_tokens.weight": (vocab, dim), "model.norm.weight": (dim,)}
    if not config["tie_word_embeddings"]:
        shapes["lm_head.weight"] = (vocab, dim)
    for layer in range(config["num_hidden_layers"]):
        for name, shape in per_layer.items():
            shapes[f"model.layers.{layer}.{name}.weight"] = shape
    return shapes


def validate_hf_config(config) -> None:
    if not isinstance(config, dict):
        raise ValueError("config.json must contain a JSON object")
    for key, integer in _POSITIVE_FIELDS:
        _require_positive(config.get(key), key, integer)
    if type(config.get("tie_word_embeddings")) is not bool:
        raise ValueError("config.json: tie_word_embeddings must be an explicit boolean")
    rope = config.get("rope_scaling")
    if not isinstance(rope, dict):
        raise ValueError("config.json: Bonsai rope_scaling metadata is required")
    _require_positive(rope.get("original_max_position_embeddings"),
                      "rope_scaling.original_max_position_embeddings", True)
    _require_positive(rope.get("factor"), "rope_scaling.factor", False)
    if config["num_attention_heads"] % config["num_key_value_heads"]:
        raise ValueError("config.json: attention heads must be divisible by key/value heads")
    if config["head_dim"] % 2:
        raise ValueError("config.json: head_dim must be even for rotary embedding")
    widths = (("hidden_size", config["hidden_size"]), ("intermediate_size", config["intermediate_size"]),
              ("query projection width", config["num_attention_heads"] * config["head_dim"]))
    for name, width in widths:
        if width % GROUP:
            raise ValueError(f"config.json: {name} must be divisible by group size {GROUP}")
    _require_positive(config.get("block_size", 8), "block_size", True)
    if type(config.get("causal_attn", True)) is not bool:
        raise ValueError("config.json: causal_attn must be a boolean")
    mask = config.get("text_mask_token_id", 151654)
    if type(mask) is not int or not 0 <= mask < config["vocab_size"]:
        raise ValueError("config.json: text_mask_token_id must index the checkpoint vocabulary")


def validate_hf_checkpoint(src_ckpt_dir: str) -> Tuple[dict, List[str]]:
    """(config, shard file names) of a complete HF checkpoint; ValueError otherwise.  Creates nothing."""
    from safetensors import safe_open
    config_path = os.path.join(src_ckpt_dir, "config.json")
    if not os.path.isfile(config_path):
        raise ValueError(f"missing HF config.json: {config_path}")
    try:
        with open(config_path, encoding="utf-8") as f:
            config = json.load(f)
    except (OSError, ValueError) as error:
        raise ValueError(f"cannot read valid HF config.json: {config_path}") from error
    validate_hf_config(config)

    shards = sorted(n for n in os.listdir(src_ckpt_dir)
                    if n.endswith(".safetensors") and os.path.isfile(os.path.join(src_ckpt_dir, n)))
    if not shards:
        raise ValueError("No HF safetensors weight shards found. A config/card or .bin-only checkpoint is not "
                         "sufficient; export the complete HF model with save_pretrained(..., "
                         "safe_serialization=True) before conversion.")
    required = expected_tensor_shapes(config)
    accepted = dict(required)
    if config["tie_word_embeddings"]:
        accepted["lm_head.weight"] = (config["vocab_size"], config["hidden_size"])     # present in some exports, ignored
    seen = set()
    for shard in shards:
        try:
            with safe_open(os.path.join(src_ckpt_dir, shard), framework="pt", device="cpu") as reader:
                names = list(reader.keys())
                if not names:
                    raise ValueError(f"empty safetensors shard: {shard}")
                for name in names:
                    if name in seen:
                        raise ValueError(f"duplicate tensor key across shards: {name}")
                    if name not in accepted:
                        raise ValueError(f"unsupported tensor key for Bonsai GPU conversion: {name}")
                    view = reader.get_slice(name)
                    shape = tuple(view.get_shape())
                    if shape != accepted[name]:
                        raise ValueError(f"tensor shape mismatch for {name}: {shape} != {accepted[name]}")
                    if view.get_dtype() not in _FLOAT_DTYPES:
                        raise ValueError(f"{name} must contain floating-point HF weights, not packed/integer weights")
                    seen.add(name)
        except Exception as error:
            raise ValueError(f"invalid HF safetensors shard {shard}: {error}") from error
    missing = sorted(set(required) - seen)
    if missing:
        raise ValueError(f"incomplete HF checkpoint: missing {len(missing)} core tensors: {missing[:5]}")
    return config, shards


def validate_sdlm_config(ckpt_dir: str, config: dict):
    """`sdlm_config.json`, when the checkpoint carries one, must agree with config.json on the MTP fields."""
    path = os.path.join(ckpt_dir, "sdlm_config.json")
    if not os.path.isfile(path):
        return None
    with open(path, encoding="utf-8") as f:
        saved = json.load(f)
    if not isinstance(saved, dict):
        raise ValueError("sdlm_config.json must contain a JSON object")
    for key, kind in (("block_size", int), ("causal_attn", bool), ("text_mask_token_id", int)):
        value = saved.get(key)
        if type(value) is not kind:
            raise ValueError(f"sdlm_config.json: invalid or missing {key}")
        other = config.get(key)
        if type(other) is not kind or other != value:
            raise ValueError(f"sdlm_config.json conflicts with config.json: {key}")
    if saved["block_size"] <= 0:
        raise ValueError("sdlm_config.json: block_size must be positive")
    if not 0 <= saved["text_mask_token_id"] < config["vocab_size"]:
        raise ValueError("sdlm_config.json: text_mask_token_id is outside the vocabulary")
    return saved
