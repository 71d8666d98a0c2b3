"""The reference's own GPU decode loops, timed.  BASELINE MEASUREMENT ONLY.

Runs the UNMODIFIED reference runtime (`bonsai_sft.gpu` as installed under baseline/_ref by
oracle/build.py: its model, its GraphAtlas, its fast_ar_generate / fast_hybrid_generate, its CUDA
kernel built into oracle/_ref) on the synthetic random-init checkpoint the benchmark uses, and
prints one JSON line with its decode tokens/s (reference definition: timed decode tokens / decode
seconds, src/bonsai_sft/gpu/fast_generate.py:1147-1172).  None of this repository's kernels or
runtime modules is loaded here; `bitmtp_b200.synthetic` (pure torch) only supplies the weights.

    python oracle/reference_decode.py --model 1p7b --prompt-len 256 --new-tokens 512
                                      [--profile standard|eager] [--no-flex]

--profile standard  the reference's default: fused helpers through torch.compile, FlexAttention
--profile eager     its `orin-d8` profile (same tensor expressions, not compiled) with the explicit
                    matmul/softmax attention; used when the compiled profile cannot run on the box
Forced acceptance: the confidence-chain length is replaced by D (every block is committed whole),
as on this repository's side of the benchmark.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
REF_SITE = os.path.join(ROOT, "baseline", "_ref")


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="1p7b", choices=["1p7b", "4b"])
    ap.add_argument("--prompt-len", type=int, default=256)
    ap.add_argument("--new-tokens", type=int, default=512)
    ap.add_argument("--profile", default="standard", choices=["standard", "eager"])
    ap.add_argument("--no-flex", action="store_true")
    ap.add_argument("--reps", type=int, default=2)
    args = ap.parse_args()
    if not os.path.isdir(os.path.join(REF_SITE, "bonsai_sft")):
        print(json.dumps({"unavailable": "baseline/_ref holds no copy of the reference's Python package"}))
        return 0
    sys.path.insert(0, REF_SITE)
    sys.path.insert(1, ROOT)
    import torch
    if not torch.cuda.is_available():
        print(json.dumps({"unavailable": "no CUDA device"}))
        return 0
    from bonsai_sft.gpu.runtime_config import select_runtime_profile
    select_runtime_profile("standard" if args.profile == "standard" else "orin-d8")
    from bonsai_sft.gpu import fast_generate as RG, fast_runtime as RF, model as RM
    from bitmtp_b200 import synthetic

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    geometry = synthetic.BONSAI_1P7B if args.model == "1p7b" else synthetic.BONSAI_4B
    cfg = synthetic.make_config(geometry, block_size=8)
    D = cfg["block_size"]
    margs = RM.ModelArgs(dim=cfg["dim"], n_layers=cfg["n_layers"], n_heads=cfg["n_heads"],
                         n_kv_heads=cfg["n_kv_heads"], head_dim=cfg["head_dim"], ffn_dim=cfg["ffn_dim"],
                         vocab_size=cfg["vocab_size"], norm_eps=cfg["norm_eps"], rope_theta=cfg["rope_theta"],
                         rope_original_max=cfg["rope_original_max"], rope_factor=cfg["rope_factor"],
                         tie_word_embeddings=True, block_size=D, causal_attn=True,
                         mask_token_id=cfg["mask_token_id"], use_kernel=True, kernel_kind="t2g128")
    t_build = time.time()
    model = RM.Transformer(margs).to(device=dev, dtype=torch.bfloat16)
    sd = synthetic.device_state(cfg, dev, seed=0)
    sd = {k: v for k, v in sd.items() if not k.startswith("_head")}
    missing, unexpected = model.load_state_dict(sd, strict=False)
    if [k for k in missing if "lm_head" not in k] or unexpected:
        print(json.dumps({"unavailable": f"state dict mismatch: missing {missing[:3]} unexpected {unexpected[:3]}"}))
        return 0
    del sd
    model.tie_weights()
    model._force_a8_lm_head = True
    model.eval()
    need = args.prompt_len + args.new_tokens + 17
    sigma = next((s for s in (256, 1024, 4096) if s >= need), 4096)
    widths = (1, 9, 16)      # AR; first draft after the prompt and the verifier; steady-state draft with 8 pending rows
    model.prepare_merged_weights(max_positions=sigma + max(widths))
    flex = (args.profile == "standard") and not args.no_flex
    atlas = RF.GraphAtlas(model, margs, dev, segment_ladder=(sigma,), m_set=widths, roles=("ar", "draft", "verify"),
                          capture_verbose=False, use_flex_attention=flex)
    torch.cuda.synchronize()
    build_s = time.time() - t_build
    prompt = synthetic.random_prompt(args.prompt_len, cfg["vocab_size"], seed=100).to(dev)

    def timed(fn, **kw):
        best = None
        for i in range(1 + args.reps):
            out, st = fn(model, atlas, prompt, max_gen_len=args.new_tokens, eos_ids=(), **kw)
            if i and (best is None or st["decode_time"] < best["decode_time"]):
                best = st
        return {"tok_s": round(best["timed_decode_tokens"] / best["decode_time"], 1),
                "decode_ms": round(best["decode_time"] * 1e3, 1), "prefill_ms": round(best["prefill_time"] * 1e3, 1),
                "tokens": int(best["decode_tokens"]), "iters": int(best["n_iters"])}

    res = {"impl": "reference runtime on this GPU", "profile": args.profile, "flex_attention": bool(atlas.use_flex_attention),
           "model": args.model, "prompt_len": args.prompt_len, "new_tokens": args.new_tokens, "segment": sigma,
           "build_and_capture_s": round(build_s, 1), "torch": torch.__version__}
    res["ar"] = timed(RG.fast_ar_generate)
    orig_chain, orig_accept = RG._fused_draft_chain, RG._fused_verify_accept

    def forced_chain(logits, threshold):
        idx, _ = orig_chain(logits, threshold)            # the reductions still run
        return idx, torch.full((), D, dtype=torch.int64, device=logits.device)

    def forced_accept(draft_tokens, verify_tokens, Dd):
        orig_accept(draft_tokens, verify_tokens, Dd)
        return torch.full((), Dd, dtype=torch.int64, device=draft_tokens.device)

    RG._fused_draft_chain, RG._fused_verify_accept = forced_chain, forced_accept
    try:
        res["hybrid_forced"] = timed(RG.fast_hybrid_generate)
    finally:
        RG._fused_draft_chain, RG._fused_verify_accept = orig_chain, orig_accept
    print(json.dumps(res), flush=True)
    return 0


if __name__ == "__main__":
    try:
        sys.exit(main())
    except Exception as e:                      # one JSON line in every case: the caller parses stdout
        import traceback
        traceback.print_exc()
        print(json.dumps({"unavailable": f"{type(e).__name__}: {e}"[:400]}), flush=True)
        sys.exit(0)
