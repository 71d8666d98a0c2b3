"""The reference's OWN evaluation adapter (benchmarks/bonsai_adapter.py), unchanged, over this package's decode
loops: its per-request accounting (`BonsaiMTPWrap._call`: token partition, drafted / accepted / bonus / path
invariants per policy, request receipts) and its aggregate (`get_stats`) are run for all four policies of its
D8 and D4 recipes, with the generate callables built exactly as its `init()` builds them (same functions, same
keyword arguments) but on a CPU atlas over the oracle forward, since `init()` itself needs a GPU, lm-eval and the
released tokenizer.  Where no checkout of the reference is at hand (BITMTP_REFERENCE, or a `reference` directory
beside this repository) the module is skipped.  Nothing of the reference is copied.
"""
import importlib
import os
import sys

import pytest
import torch

from bitmtp_b200 import fast_generate as FG, generate, synthetic
from oracle import oracle as O
from tests.cpu_atlas import CpuAtlas, OracleModel, patched_host_ops

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.environ.get("BITMTP_REFERENCE", os.path.join(os.path.dirname(ROOT), "reference"))

pytestmark = pytest.mark.skipif(not os.path.isfile(os.path.join(REF, "benchmarks", "bonsai_adapter.py")),
                                reason="no checkout of the reference at hand")


@pytest.fixture(scope="module")
def adapter():
    """The reference's `benchmarks` package, imported from where it lies."""
    saved_path = list(sys.path)
    saved_mods = {k: v for k, v in sys.modules.items() if k == "benchmarks" or k.startswith("benchmarks.")}
    for k in saved_mods:
        del sys.modules[k]
    sys.path.insert(0, REF)
    try:
        yield importlib.import_module("benchmarks.bonsai_adapter"), importlib.import_module("benchmarks.profiles")
    finally:
        sys.path[:] = saved_path
        for k in [k for k in sys.modules if k == "benchmarks" or k.startswith("benchmarks.")]:
            del sys.modules[k]
        sys.modules.update(saved_mods)


def _callable_like_init(wrap, model, atlas):
    """The generate callable of BonsaiMTPWrap.init() for wrap.mode (benchmarks/bonsai_adapter.py:161-182): the same
    functions with the same keyword arguments, resolved in this package."""
    eos = ()                                    # random-init weights: no end-of-sequence id is special
    if wrap.mode == "ar":
        return lambda ids, max_t: FG.fast_ar_generate(model, atlas, ids, max_gen_len=max_t, eos_ids=eos)
    if wrap.mode == "confidence":
        return lambda ids, max_t: FG.fast_confidence_generate(
            model, atlas, ids, threshold=wrap.threshold, max_gen_len=max_t, eos_ids=eos,
            use_fp8_draft=wrap.use_fp8_draft, use_bf16_draft=wrap.use_bf16_draft)
    if wrap.mode == "speculative":
        return lambda ids, max_t: FG.fast_speculative_generate(
            model, atlas, ids, max_gen_len=max_t, eos_ids=eos, use_fp8_draft=wrap.use_fp8_draft,
            use_bf16_draft=wrap.use_bf16_draft, rabv_margin=0.0)
    return lambda ids, max_t: FG.fast_hybrid_generate(
        model, atlas, ids, threshold=wrap.threshold, hybrid_m=wrap.min_chain, max_gen_len=max_t, eos_ids=eos,
        use_fp8_draft=wrap.use_fp8_draft, use_bf16_draft=wrap.use_bf16_draft, rabv_margin=0.0)


@pytest.mark.parametrize("recipe,accept", [
    ("bonsai_1p7b_h20_d8_ar", "free"), ("bonsai_1p7b_h20_d8_confidence", "free"),
    ("bonsai_1p7b_h20_d8_speculative", "free"), ("bonsai_1p7b_h20_d8_hybrid", "free"),
    ("bonsai_1p7b_h20_d8_hybrid", "forced"), ("bonsai_1p7b_h20_d4_hybrid", "free"),
    ("bonsai_1p7b_h20_d4_speculative", "forced"), ("bonsai_1p7b_rtx3090_d4_hybrid", "free")])
def test_adapter_accounting_over_this_runtime(adapter, recipe, accept):
    mod, profiles = adapter
    profile = dict(profiles.PROFILES[recipe])
    if profile["mode"] in ("confidence", "hybrid"):
        profile["draft_projection"] = "native"          # the CPU atlas has the packed head only (both are in the recipe's set)
        if profile["device_profile"] == "rtx3090":
            profile["draft_projection"] = "bf16_raw"    # its only admitted value; the role name is all the loops read of it
    wrap = mod.BonsaiMTPWrap(0, profile, checkpoint="unused", tokenizer_path="unused")
    D = wrap.block_size
    cfg = synthetic.make_config(synthetic.TINY, block_size=D)
    state = synthetic.make_state(cfg, seed=5)
    m_set = wrap.replay_widths                          # the recipe's width schedule, as its init() passes it
    ladder = (64, 256)
    om = O.OracleModel(cfg, state, max_positions=max(ladder) + max(m_set))
    args = generate.args_from_config(cfg)
    draft = "draft_bf16" if wrap.use_bf16_draft else "draft_fp8" if wrap.use_fp8_draft else "draft"
    roles = ("ar",) if wrap.mode == "ar" else (draft, "ar") if wrap.mode == "confidence" else (draft, "verify", "ar")
    atlas = CpuAtlas(om, args, ladder, m_set, roles)
    wrap.device = torch.device("cpu")
    wrap._fn = _callable_like_init(wrap, OracleModel(om, args), atlas)
    policy = synthetic.AcceptancePolicy(accept, D, seed=3)
    lengths = (7, 19, 33)
    with patched_host_ops(D, policy):
        outs = [wrap._call(synthetic.random_prompt(n, cfg["vocab_size"], seed=n)[0].tolist(), max_gen=24)
                for n in lengths]
    assert all(0 < len(o) <= 24 for o in outs)
    st = wrap.get_stats()
    assert st["sequence_record_count"] == len(lengths)
    assert st["decode_speed"] > 0 and st["total_speed"] > 0
    if wrap.mode == "ar":
        assert st["draft_iters"] == 0
    else:
        assert st["drafted_tokens"] == D * st["draft_iters"] > 0
        assert st["accepted_drafts"] + st["verifier_bonus_tokens"] == sum(len(o) for o in outs) - (
            0 if wrap.mode == "confidence" else len(outs))
    assert len(wrap._request_receipts) == len(lengths)


@pytest.mark.parametrize("recipe,geometry,D", [("bonsai_1p7b_h20_d8_hybrid", "BONSAI_1P7B", 8),
                                               ("bonsai_1p7b_h20_d4_hybrid", "BONSAI_1P7B", 4),
                                               ("bonsai_4b_h20_d8_hybrid", "BONSAI_4B", 8),
                                               ("bonsai_1p7b_h20_sft_ar", "BONSAI_1P7B", 8)])
def test_adapter_accepts_this_packages_model_arguments(adapter, recipe, geometry, D):
    """`validate_bonsai_config(profile, vars(m.args))`, the check the adapter's init() runs on the loaded model
    (benchmarks/bonsai_adapter.py:121-122): every field it reads exists in this package's ModelArgs with the type
    it insists on, for the released geometries (vocabulary 151669)."""
    _, profiles = adapter
    cfg = synthetic.make_config(dict(getattr(synthetic, geometry), vocab_size=151669), block_size=D)
    profiles.validate_bonsai_config(profiles.PROFILES[recipe], vars(generate.args_from_config(cfg)))
    wrong = dict(vars(generate.args_from_config(cfg)), kernel_kind="q1")
    with pytest.raises(ValueError):
        profiles.validate_bonsai_config(profiles.PROFILES[recipe], wrong)
