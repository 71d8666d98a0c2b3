"""Single-prompt CUDA-graph generation on the B200 kernels; not a quality or speed benchmark.

Same command line as the reference's `python -m bonsai_sft.gpu.run_generation`
(src/bonsai_sft/gpu/run_generation.py:21-52): checkpoint and tokenizer directories, block
size, mode, prompt, and the threshold / chain / margin / precision options.  `--check-only`
validates options and local artifacts without importing torch or touching CUDA.
"""
from __future__ import annotations

import argparse
import json
import math
from pathlib import Path

from .contracts import (require_native_shape, validate_public_device_scope,
                        validate_public_model_scope, validate_verification_options)
from .runtime_config import (RUNTIME_PROFILES, is_orin_profile, select_runtime_profile,
                             validate_profile_device, validate_profile_model,
                             validate_profile_options)

WIDTHS = {4: (1, 4, 5, 6, 7, 8, 9), 8: (1, 8, 9, 10, 12, 16, 17)}
DRAFT_ROLE = {"native": "draft", "fp8": "draft_fp8", "bf16": "draft_bf16"}


def make_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(description=__doc__)
    p.add_argument("--ckpt", type=Path, required=True, help="Converted GPU checkpoint directory.")
    p.add_argument("--hf-ckpt", "--hf_ckpt", dest="hf_ckpt", type=Path, required=True,
                   help="Local Hugging Face tokenizer directory for the same checkpoint.")
    p.add_argument("--block-size", type=int, choices=(4, 8), required=True,
                   help="Must match bonsai_gpu_config.json; not a checkpoint override.")
    p.add_argument("--mode", choices=("ar", "conf", "spec", "hybrid"), required=True)
    p.add_argument("--runtime-profile", choices=RUNTIME_PROFILES, default="b200",
                   help="Kept for command-line compatibility; every profile runs the same kernels.")
    src = p.add_mutually_exclusive_group(required=True)
    src.add_argument("--prompt", help="Raw prompt text, unless --chat is supplied.")
    src.add_argument("--prompt-file", type=Path, help="Read a UTF-8 prompt from a local file.")
    p.add_argument("--chat", action="store_true", help="Apply the checkpoint chat template, thinking disabled.")
    p.add_argument("--max-new-tokens", type=int, default=128)
    p.add_argument("--max-context", type=int, default=4096,
                   help="One captured KV segment; must fit prompt + output + maximum graph width.")
    p.add_argument("--threshold", type=float, default=0.9)
    p.add_argument("--min-chain", type=int, default=None,
                   help="Hybrid gate: default 6 for D8, 3 for D4.")
    p.add_argument("--margin", type=float, default=0.0,
                   help="Compatibility argument; only 0 is accepted by strict verification.")
    p.add_argument("--exact-m1-verify", action="store_true",
                   help="Use the same width-1 graph as AR; requires margin 0.")
    p.add_argument("--draft-precision", choices=("native", "fp8", "bf16"), default="native",
                   help="Head of the draft role: native packed T2, or the dense tied table as e4m3 / bf16.")
    p.add_argument("--verify-precision", choices=("native",), default="native")
    p.add_argument("--device", default="cuda:0")
    p.add_argument("--no-flex-attention", action="store_true",
                   help="Accepted and ignored: attention is always the native kernel.")
    p.add_argument("--check-only", action="store_true",
                   help="Validate options and local artifacts only; never initialize CUDA or generate.")
    return p


def validate_options(args):
    """Option combinations, in the reference's order (run_generation.py:55-81).
    Returns (widths, roles, min_chain)."""
    validate_verification_options(args.margin, args.exact_m1_verify)
    validate_profile_options(args)
    if not math.isfinite(args.threshold) or not 0 <= args.threshold <= 1:
        raise ValueError("threshold must be finite and between 0 and 1")
    if args.max_new_tokens < 1 or args.max_context < 1:
        raise ValueError("max-new-tokens and max-context must be positive")
    default_chain = 3 if (is_orin_profile(args.runtime_profile) or args.block_size == 4) else 6
    min_chain = default_chain if args.min_chain is None else args.min_chain
    if not 1 <= min_chain <= args.block_size + 1:
        raise ValueError("min-chain must be in [1, block-size + 1]")
    if args.min_chain is not None and args.mode != "hybrid":
        raise ValueError("min-chain is only used by hybrid mode")
    verifying = args.mode in ("spec", "hybrid")
    if not verifying and (args.exact_m1_verify or args.margin != 0 or args.verify_precision != "native"):
        raise ValueError("verification options are only used by spec/hybrid modes")
    if args.mode == "ar" and args.draft_precision != "native":
        raise ValueError("AR does not use a draft projection")
    if args.verify_precision != "native":
        raise ValueError("strict verification requires the native verifier projection")
    widths = (1,) if args.mode == "ar" else WIDTHS[args.block_size]
    roles = ["ar"]
    if args.mode != "ar":
        roles.append(DRAFT_ROLE[args.draft_precision])
    if verifying:
        roles.append("verify")
    return widths, tuple(roles), min_chain


def validate_artifacts(args, widths) -> dict:
    """Local files and kernel shapes (run_generation.py:84-123).  Reads JSON only."""
    config_path = args.ckpt / "bonsai_gpu_config.json"
    if not config_path.is_file():
        raise ValueError(f"missing GPU checkpoint configuration: {config_path}")
    config = json.loads(config_path.read_text())
    validate_public_model_scope(config)
    validate_profile_model(args.runtime_profile, config)
    if config.get("block_size") != args.block_size:
        raise ValueError("block-size does not match the converted checkpoint configuration")
    kind = config.get("kernel_kind", "q1")
    if kind != "t2g128":
        raise ValueError(f"unsupported kernel_kind: {kind!r} (this build serves t2g128 checkpoints)")
    state = args.ckpt / "model_state_t2g128.pt"
    if not state.is_file() and not (args.ckpt / "model_state_t2g128.safetensors").is_file():
        raise ValueError(f"missing packed checkpoint: {state}")
    tok = args.hf_ckpt
    if not (tok / "tokenizer_config.json").is_file():
        raise ValueError(f"missing tokenizer_config.json in {tok}")
    if not ((tok / "tokenizer.json").is_file()
            or all((tok / f).is_file() for f in ("vocab.json", "merges.txt"))):
        raise ValueError(f"need tokenizer.json or both vocab.json and merges.txt in {tok}")
    if args.prompt_file is not None and not args.prompt_file.is_file():
        raise ValueError(f"missing prompt file: {args.prompt_file}")
    dim = config["dim"]
    qw = config["n_heads"] * config["head_dim"]
    kvw = config["n_kv_heads"] * config["head_dim"]
    shapes = ((qw + 2 * kvw, dim), (dim, qw), (2 * config["ffn_dim"], dim), (dim, config["ffn_dim"]),
              ((config["vocab_size"] + 31) // 32 * 32, dim))
    for m in widths:
        for n, k in shapes:
            require_native_shape(m, n, k)
    from .native import SO_PATH                       # path constant only; nothing is loaded
    if not Path(SO_PATH).is_file():
        raise ValueError(f"missing native library: {SO_PATH}; build it with `python -m bitmtp_b200.native`")
    return config


def main(argv=None):
    parser = make_parser()
    args = parser.parse_args(argv)
    try:
        widths, roles, min_chain = validate_options(args)
        config = validate_artifacts(args, widths)
    except (ValueError, RuntimeError, KeyError) as error:
        parser.error(str(error))
    if args.check_only:
        print(json.dumps({"status": "local_artifacts_and_options_checked", "gpu_executed": False,
                          "runtime_profile": args.runtime_profile, "mode": args.mode,
                          "kernel_kind": config.get("kernel_kind"), "widths": widths, "roles": roles,
                          "margin": args.margin,
                          "min_chain": min_chain if args.mode == "hybrid" else None}, indent=2))
        return

    select_runtime_profile(args.runtime_profile)
    import torch
    from transformers import AutoTokenizer
    from .fast_generate import (fast_ar_generate, fast_confidence_generate, fast_hybrid_generate,
                                fast_speculative_generate)
    from .fast_runtime import GraphAtlas
    from .generate import build_model

    if not torch.cuda.is_available():
        parser.error("CUDA is required for generation; --check-only performs artifact checks without CUDA")
    device = torch.device(args.device)
    if device.type != "cuda":
        parser.error("device must be a CUDA device")
    torch.cuda.set_device(device)
    capability = torch.cuda.get_device_capability(device)
    try:
        validate_public_device_scope(config, capability)
        validate_profile_device(args.runtime_profile, capability)
    except ValueError as error:
        parser.error(str(error))
    tokenizer = AutoTokenizer.from_pretrained(str(args.hf_ckpt), local_files_only=True,
                                              trust_remote_code=False)
    prompt = args.prompt_file.read_text() if args.prompt_file else args.prompt
    if args.chat:
        prompt = tokenizer.apply_chat_template([{"role": "user", "content": prompt}], tokenize=False,
                                               add_generation_prompt=True, enable_thinking=False)
    input_ids = tokenizer(prompt, return_tensors="pt").input_ids
    if input_ids.shape[1] == 0:
        parser.error("prompt must tokenize to at least one token")
    if input_ids.shape[1] + args.max_new_tokens + max(widths) > args.max_context:
        parser.error("max-context is too small for prompt + output + maximum graph width")
    model = build_model(str(args.ckpt), use_kernel=True, device=device)
    model.prepare_merged_weights(max_positions=args.max_context + max(widths))
    atlas = GraphAtlas(model, model.args, device, segment_ladder=(args.max_context,), m_set=widths,
                       roles=roles)
    draft = dict(use_fp8_draft=args.draft_precision == "fp8", use_bf16_draft=args.draft_precision == "bf16")
    verify = dict(exact_m1_verify=args.exact_m1_verify, rabv_margin=args.margin)
    ids = input_ids.to(device)
    n = args.max_new_tokens
    if args.mode == "ar":
        output, stats = fast_ar_generate(model, atlas, ids, max_gen_len=n)
    elif args.mode == "conf":
        output, stats = fast_confidence_generate(model, atlas, ids, threshold=args.threshold,
                                                 max_gen_len=n, **draft)
    elif args.mode == "spec":
        output, stats = fast_speculative_generate(model, atlas, ids, max_gen_len=n, **draft, **verify)
    else:
        output, stats = fast_hybrid_generate(model, atlas, ids, threshold=args.threshold,
                                             hybrid_m=min_chain, max_gen_len=n, **draft, **verify)
    print(json.dumps({"mode": args.mode, "block_size": args.block_size, "margin": args.margin,
                      "runtime_profile": args.runtime_profile, "threshold": args.threshold,
                      "min_chain": min_chain if args.mode == "hybrid" else None, "roles": roles,
                      "exact_m1_verify": args.exact_m1_verify,
                      "text": tokenizer.decode(output.tolist(), skip_special_tokens=True),
                      "token_ids": output.tolist(), "generation_stats": stats,
                      "note": "Single-prompt generation only; not a quality or speed benchmark."},
                     ensure_ascii=False, indent=2))


if __name__ == "__main__":
    main()
