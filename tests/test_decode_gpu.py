"""End-to-end GPU parity: the captured forward against the CPU oracle forward (logits and
appended KV rows, bit for bit) and the decode loops over real CUDA graphs against the token
streams recorded from the reference's loops."""
import json
import os

import numpy as np
import pytest
import torch

from bitmtp_b200 import fast_generate as FG, generate, native, ops, synthetic
from bitmtp_b200.synthetic import acceptance_hooks
from bitmtp_b200.fast_runtime import GraphAtlas
from bitmtp_b200.model import make_sdlm_cache

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "streams.json")
RECORDS = json.load(open(GOLDEN))
_MODELS = {}


def _model(cfg, seed, max_positions):
    key = (json.dumps(cfg, sort_keys=True), seed, max_positions)
    if key not in _MODELS:
        state = synthetic.make_state(cfg, seed=seed)
        m = generate.model_from_state(generate.args_from_config(cfg), state, DEV)
        m.prepare_merged_weights(max_positions=max_positions)
        _MODELS[key] = (m, state)
    return _MODELS[key]


FORWARD_CASES = [("ar", 1, 20, 0), ("ar", 16, 0, 0), ("ar", 7, 48, 0), ("verify", 9, 30, 0),
                 ("draft", 9, 30, 1), ("draft", 12, 25, 3), ("draft", 16, 40, 8), ("draft", 17, 33, 9),
                 ("draft", 10, 64, 1)]


@pytest.mark.parametrize("geom", ["tiny", "g4"])
@pytest.mark.parametrize("role,M,cache_len,n_pend", FORWARD_CASES)
def test_forward_matches_oracle(oracle, geom, role, M, cache_len, n_pend):
    geometry = synthetic.TINY if geom == "tiny" else dict(synthetic.TINY, n_heads=4, n_kv_heads=1,
                                                          dim=512, ffn_dim=768)
    cfg = synthetic.make_config(geometry, block_size=8)
    sigma, m_max = 64, 17
    model, state = _model(cfg, 3, sigma + m_max)
    om = oracle.OracleModel(cfg, state, max_positions=sigma + m_max)
    D, L, Hkv = 8, cfg["n_layers"], cfg["n_kv_heads"]
    gen = torch.Generator().manual_seed(M * 100 + cache_len)
    kv = (torch.randn(2, L, 1, Hkv, sigma + m_max, 128, generator=gen) * 0.5).to(torch.bfloat16)
    tokens = torch.randint(0, cfg["vocab_size"], (M,), generator=gen)
    positions = torch.arange(max(cache_len - 1, 0), max(cache_len - 1, 0) + M)
    rid = oracle.ROLE_IDS[role]
    ls, le = {"ar": (0, M), "verify": (0, min(D + 1, M)), "draft": (M - D, M)}[role]
    kv_np = oracle.torch_to_u16(kv).copy()
    want = om.forward(tokens.numpy(), positions.numpy(), kv_np, sigma, rid, cache_len, n_pend, ls, le)

    kvd = kv.to(DEV)
    state_t = ops.new_step_state(DEV)
    ops.set_step_state(state_t, cache_len, min(n_pend, max(M - D, 0)), rid, M - D)
    kv_full = [(kvd[0, i][:, :, : sigma + M, :], kvd[1, i][:, :, : sigma + M, :]) for i in range(L)]
    logits = model.forward_sdlm_decode_graph_kernel(tokens.to(DEV), positions.to(DEV), kv_full, M,
                                                    state_t, ls, le, "t2")
    torch.cuda.synchronize()
    assert native.lib().bm_device_error() == 0
    assert np.array_equal(logits.cpu().numpy().view(np.uint32), want.view(np.uint32)), "logits differ"
    assert np.array_equal(oracle.torch_to_u16(kvd.cpu()), kv_np), "KV buffer differs"


@pytest.mark.parametrize("rec", RECORDS, ids=lambda r: f"{r['geometry']}-D{r['cfg']['block_size']}-{r['mode']}-"
                                                         f"{r['accept']}" + ("-eos" if r.get("eos_ids") else "") +
                                                         ("-m1verify" if r.get("exact_m1_verify") else ""))
def test_token_streams_match_reference_loops(rec, monkeypatch):
    if rec.get("exact_m1_verify"):
        pytest.skip("the width-1 verifier streams are pinned on the CPU atlas (test_host_loops_cpu.py); not yet run on a GPU")
    cfg = rec["cfg"]
    model, _ = _model(cfg, rec["state_seed"], max(rec["ladder"]) + max(rec["m_set"]))
    roles = ("ar",) if rec["mode"] == "ar" else ("ar", "draft", "verify")
    atlas = GraphAtlas(model, model.args, torch.device(DEV), segment_ladder=tuple(rec["ladder"]),
                       m_set=tuple(rec["m_set"]), roles=roles, capture_verbose=False)
    if rec["accept"] != "free":
        policy = synthetic.AcceptancePolicy(rec["accept"], cfg["block_size"], seed=rec["accept_seed"])
        fc, fa = acceptance_hooks(FG, policy)
        monkeypatch.setattr(FG, "_fused_draft_chain", fc)
        monkeypatch.setattr(FG, "_fused_verify_accept", fa)
    prompt = synthetic.random_prompt(rec["prompt_len"], cfg["vocab_size"], seed=rec["prompt_seed"])
    fn = {"ar": FG.fast_ar_generate, "spec": FG.fast_speculative_generate,
          "hybrid": FG.fast_hybrid_generate, "conf": FG.fast_confidence_generate}[rec["mode"]]
    extra = dict(exact_m1_verify=True) if rec.get("exact_m1_verify") else {}
    out, stats = fn(model, atlas, prompt, max_gen_len=rec["new_tokens"], eos_ids=frozenset(rec.get("eos_ids", ())), **extra)
    assert native.lib().bm_device_error() == 0
    assert out.cpu().tolist() == rec["tokens"]
    for key, want in rec["stats"].items():
        assert stats[key] == pytest.approx(want), key
    # graphs of one segment share one KV buffer (the observable the reference's adapter checks)
    sig = atlas.segment_ladder[0]
    ptrs = {g.kv_full[0][0].data_ptr() for (M, s, r), g in atlas.graphs.items() if s == sig}
    assert ptrs == {atlas.kv_buffers[sig].data_ptr()}


@pytest.mark.parametrize("cache_len", [0, 37, 200])
def test_width1_fused_layers_equal_operator_path(cache_len):
    """The six-launch width-1 layer (RMSNorm / quantisation inside the consuming GEMV) against the general
    launch sequence on the 1.7B layer geometry: logits, residual stream and KV rows bit for bit."""
    geometry = dict(synthetic.BONSAI_1P7B, n_layers=3, vocab_size=4096)
    cfg = synthetic.make_config(geometry, block_size=8)
    sigma, m_max = 256, 17
    model, _ = _model(cfg, 5, sigma + m_max)
    assert model._ar_fused_supported(1)
    L, Hkv, M = cfg["n_layers"], cfg["n_kv_heads"], 1
    gen = torch.Generator().manual_seed(cache_len + 1)
    kv = (torch.randn(2, L, 1, Hkv, sigma + m_max, 128, generator=gen) * 0.5).to(torch.bfloat16)
    tokens = torch.randint(0, cfg["vocab_size"], (M,), generator=gen).to(DEV)
    positions = torch.arange(cache_len, cache_len + M).to(DEV)
    state_t = ops.new_step_state(DEV)
    ops.set_step_state(state_t, cache_len, 0, native.ROLE_AR, M - 8)
    outs = {}
    for fused in (False, True):
        kvd = kv.to(DEV)
        kv_full = [(kvd[0, i][:, :, : sigma + M, :], kvd[1, i][:, :, : sigma + M, :]) for i in range(L)]
        model.fused_ar = fused
        try:
            for rep in range(2):
                logits = model.forward_sdlm_decode_graph_kernel(tokens, positions, kv_full, M, state_t, 0, M, "t2")
        finally:
            model.fused_ar = True
        torch.cuda.synchronize()
        assert native.lib().bm_device_error() == 0
        outs[fused] = (logits.clone(), kvd.clone(), model.workspace(M).h.clone())
    assert torch.equal(outs[True][0].view(torch.int32), outs[False][0].view(torch.int32)), "logits differ"
    assert torch.equal(outs[True][1].view(torch.int16), outs[False][1].view(torch.int16)), "KV rows differ"
    assert torch.equal(outs[True][2].view(torch.int16), outs[False][2].view(torch.int16)), "residual stream differs"


def test_confidence_stream_with_categorical_acceptance_equals_cpu_loop(oracle):
    """Confidence-only decode with a seeded accepted length per step walks the draft widths
    9, 10, 12 and 16 (n_pend = 1..8).  The captured graphs must produce the token stream the same
    loop produces over the CPU oracle forward, with the same draws."""
    from tests.cpu_atlas import CpuAtlas, OracleModel, patched_host_ops
    cfg = synthetic.make_config(synthetic.TINY, block_size=8)
    ladder, m_set, roles = (256,), (1, 8, 9, 10, 12, 16, 17), ("ar", "draft", "verify")
    model, state = _model(cfg, 7, max(ladder) + max(m_set))
    prompt = synthetic.random_prompt(31, cfg["vocab_size"], seed=31)
    new_tokens = 120

    om = oracle.OracleModel(cfg, state, max_positions=max(ladder) + max(m_set))
    cpu_atlas = CpuAtlas(om, model.args, ladder, m_set, roles)
    policy = synthetic.AcceptancePolicy("categorical", 8, seed=5)
    with patched_host_ops(8, policy):
        want, want_stats = FG.fast_confidence_generate(OracleModel(om, model.args), cpu_atlas, prompt,
                                                       max_gen_len=new_tokens, eos_ids=())
    widths = {M for (_, M, _, _, _) in cpu_atlas.log}
    assert {9, 10, 12, 16} <= widths, widths

    atlas = GraphAtlas(model, model.args, torch.device(DEV), segment_ladder=ladder, m_set=m_set, roles=roles,
                       capture_verbose=False)
    policy = synthetic.AcceptancePolicy("categorical", 8, seed=5)
    saved = FG._fused_draft_chain, FG._fused_verify_accept
    FG._fused_draft_chain, FG._fused_verify_accept = acceptance_hooks(FG, policy)
    try:
        got, stats = FG.fast_confidence_generate(model, atlas, prompt, max_gen_len=new_tokens, eos_ids=())
    finally:
        FG._fused_draft_chain, FG._fused_verify_accept = saved
    assert native.lib().bm_device_error() == 0
    assert got.cpu().tolist() == want.tolist()
    for key in ("n_iters", "draft_iters", "accepted_drafts", "n_conf_path", "n_verify_path", "decode_tokens"):
        assert stats[key] == want_stats[key], key


@pytest.mark.parametrize("geometry,seq", [("tiny", 37), ("tiny", 16), ("tiny", 5), ("layers3", 70), ("layers3", 300),
                                          ("cut4b", 200), ("tiny", 129)])
def test_atlas_prefill_equals_operator_prefill(geometry, seq, monkeypatch):
    """GraphAtlas.prefill against Transformer.forward_sdlm_prefill (the slab-by-slab prompt forward,
    every operator launched from the host, rows written in place): the prompt's K/V rows in every layer
    and the last row's logits, bit for bit.  Prompts longer than a slab go through the many-row kernels
    (bm_t2_gemm_wide, bm_prompt_attention; 300 rows = two waves), shorter ones through the captured slab
    graph; with BM_WIDE_PREFILL=0 every length goes through the slab graphs."""
    geo = {"tiny": synthetic.TINY, "layers3": dict(synthetic.BONSAI_1P7B, n_layers=3, vocab_size=4096),
           "cut4b": dict(synthetic.BONSAI_4B, n_layers=2, vocab_size=4096)}[geometry]
    if geometry == "tiny" and seq == 129:
        monkeypatch.setenv("BM_WIDE_PREFILL", "0")
    cfg = synthetic.make_config(geo, block_size=8)
    sigma, m_set = 128 if seq <= 128 else 512, (1, 9, 16)
    model, _ = _model(cfg, 5, sigma + max(m_set))
    atlas = GraphAtlas(model, model.args, torch.device(DEV), segment_ladder=(sigma,), m_set=m_set,
                       roles=("ar", "draft", "verify"), capture_verbose=False)
    assert sigma in atlas.prefill_graphs and atlas.prefill_graphs[sigma].n_kernels > 0
    prompt = synthetic.random_prompt(seq, cfg["vocab_size"], seed=seq)[0].to(DEV)

    cache = make_sdlm_cache(model.args, device=torch.device(DEV))
    want_logits = model.forward_sdlm_prefill(token_values=prompt, cache=cache)[-1:].clone()
    # three times: the first call launches every kernel from the host, the second captures the wave into a
    # CUDA graph and replays it, the third replays
    for call in range(3):
        atlas.kv_buffers[sigma].zero_()
        got_logits = atlas.prefill(prompt, sigma)
        torch.cuda.synchronize()
        assert native.lib().bm_device_error() == 0
        assert torch.equal(got_logits.view(torch.int32), want_logits.view(torch.int32)), f"last-row logits differ (call {call})"
        shared = atlas.kv_buffers[sigma]
        for i, (ck, cv) in enumerate(cache):
            assert torch.equal(shared[0, i, 0, :, :seq, :].view(torch.int16), ck[0].view(torch.int16)), f"K layer {i}"
            assert torch.equal(shared[1, i, 0, :, :seq, :].view(torch.int16), cv[0].view(torch.int16)), f"V layer {i}"
            assert not shared[:, i, 0, :, seq:sigma, :].any(), "rows past the prompt were written"
