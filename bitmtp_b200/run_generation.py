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


def _default_min_chain(args) -> int:
    """3 where a block has four draft positions (D4, and the reference's Orin profiles), otherwise 6."""
    return 3 if (args.block_size == 4 or is_orin_profile(args.runtime_profile)) else 6


def _roles_for(mode: str, draft_precision: str):
    """Graph roles a mode replays: AR always (first token, exact-M1 verify), a draft role for every MTP mode,
    the verifier for the two modes that check drafts."""
    roles = ("ar",)
    if mode != "ar":
        roles += (DRAFT_ROLE[draft_precision],)
    if mode in ("spec", "hybrid"):
        roles += ("verify",)
    return roles


def validate_options(args):
    """Option combinations, judged in the reference's order and with its messages
    (run_generation.py:55-81).  Returns (widths, roles, min_chain)."""
    validate_verification_options(args.margin, args.exact_m1_verify)
    validate_profile_options(args)
    mode, verifying = args.mode, args.mode in ("spec", "hybrid")
    min_chain = _default_min_chain(args) if args.min_chain is None else args.min_chain
    verify_options_set = args.exact_m1_verify or args.margin != 0 or args.verify_precision != "native"
    # (condition that must hold, message when it does not), first failure wins
    rules = (
        (math.isfinite(args.threshold) and 0 <= args.threshold <= 1, "threshold must be finite and between 0 and 1"),
        (args.max_new_tokens >= 1 and args.max_context >= 1, "max-new-tokens and max-context must be positive"),
        (1 <= min_chain <= args.block_size + 1, "min-chain must be in [1, block-size + 1]"),
        (args.min_chain is None or mode == "hybrid", "min-chain is only used by hybrid mode"),
        (verifying or not verify_options_set, "verification options are only used by spec/hybrid modes"),
        (mode != "ar" or args.draft_precision == "native", "AR does not use a draft projection"),
        (args.verify_precision == "native", "strict verification requires the native verifier projection"),
    )
    for holds, message in rules:
        if not holds:
            raise ValueError(message)
    widths = (1,) if mode == "ar" else WIDTHS[args.block_size]
    return widths, _roles_for(mode, args.draft_precision), min_chain


def _layer_shapes(config: dict):
    """(N, K) of the merged projections of a layer and of the padded packed head."""
    dim, hd = config["dim"], config["head_dim"]
    q_dim, kv_dim = config["n_heads"] * hd, config["n_kv_heads"] * hd
    head_rows = (config["vocab_size"] + 31) // 32 * 32
    return ((q_dim + 2 * kv_dim, dim), (dim, q_dim), (2 * config["ffn_dim"], dim), (dim, config["ffn_dim"]),
            (head_rows, dim))


def _require_file(path: Path, what: str) -> None:
    if not path.is_file():
        raise ValueError(f"missing {what}: {path}")


def validate_artifacts(args, widths) -> dict:
    """Local files and kernel shapes (run_generation.py:84-123).  Reads JSON only; neither torch nor the native
    library is touched."""
    _require_file(args.ckpt / "bonsai_gpu_config.json", "GPU checkpoint configuration")
    config = json.loads((args.ckpt / "bonsai_gpu_config.json").read_text())
    validate_public_model_scope(config)
    validate_profile_model(args.runtime_profile, config)
    if config.get("block_size") != args.block_size:
        raise ValueError("block-size does not match the converted checkpoint configuration")
    kind = config.get("kernel_kind", "q1")
    if kind != "t2g128":
        raise ValueError(f"unsupported kernel_kind: {kind!r} (this build serves t2g128 checkpoints)")
    if not any((args.ckpt / name).is_file() for name in ("model_state_t2g128.pt", "model_state_t2g128.safetensors")):
        raise ValueError(f"missing packed checkpoint: {args.ckpt / 'model_state_t2g128.pt'}")
    tok = args.hf_ckpt
    if not (tok / "tokenizer_config.json").is_file():
        raise ValueError(f"missing tokenizer_config.json in {tok}")
    bpe_pair = all((tok / name).is_file() for name in ("vocab.json", "merges.txt"))
    if not ((tok / "tokenizer.json").is_file() or bpe_pair):
        raise ValueError(f"need tokenizer.json or both vocab.json and merges.txt in {tok}")
    if args.prompt_file is not None:
        _require_file(args.prompt_file, "prompt file")
    for n, k in _layer_shapes(config):
        for m in widths:
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
