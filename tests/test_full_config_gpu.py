"""Parity at the benchmark's own sizes.

1. The full decode configuration the headline number is quoted on: Bonsai-1.7B architecture (28 layers,
   hidden 2048, 16 query / 8 KV heads, MLP 6144, vocabulary 151936), seeded 256-token prompt, 512 new
   tokens, block size 8, forced full-block acceptance, one 1024-row segment, hybrid and speculative
   policies.  The captured CUDA graphs must produce, token for token
   and statistic for statistic, what the same decode loop produces over the CPU oracle forward.
2. The 4B layer geometry (hidden 2560, 32 query / 8 KV heads, MLP 9728, 4096-row segment) cut to two
   layers: the captured forward against the oracle forward, logits and every K/V row bit for bit, for
   every role and every width a block-size-8 decode replays, including a history that fills the whole
   segment; and one hybrid stream with the seeded categorical acceptance of mean 4.

Synthetic seeded weights and prompts stand in for the real checkpoints and prompts.
"""
import numpy as np
import pytest
import torch

from bitmtp_b200 import fast_generate as FG, generate, native, ops, synthetic
from bitmtp_b200.fast_runtime import GraphAtlas
from bitmtp_b200.synthetic import acceptance_hooks

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
WIDTHS = (1, 8, 9, 10, 12, 16, 17)
ROLES = ("ar", "draft", "verify")


def _build(cfg, seed, max_positions, oracle):
    """The same random-init checkpoint as a GPU model and as an oracle model."""
    sd = synthetic.device_state(cfg, DEV, seed=seed)
    head = (sd.pop("_head.weight"), sd.pop("_head.weight_scale"))
    cpu_state = {k: v.cpu() for k, v in sd.items()}
    model = generate.model_from_state(generate.args_from_config(cfg), sd, DEV)
    if cfg["vocab_size"] % 32 == 0:
        model._lm_head_t2_w, model._lm_head_t2_scale = head
        model._lm_head_t2_vocab = model._lm_head_n_pad = cfg["vocab_size"]
    model.prepare_merged_weights(max_positions=max_positions)
    om = oracle.OracleModel(cfg, cpu_state, max_positions=max_positions, head=(head[0].cpu(), head[1].cpu()))
    return model, om


@pytest.fixture(scope="module")
def full_1p7b(oracle):
    cfg = synthetic.make_config(synthetic.BONSAI_1P7B, block_size=8)
    model, om = _build(cfg, 0, 1024 + 17, oracle)
    atlas = GraphAtlas(model, model.args, torch.device(DEV), segment_ladder=(1024,), m_set=WIDTHS, roles=ROLES,
                       capture_verbose=False)
    yield cfg, model, om, atlas
    del atlas, model
    torch.cuda.empty_cache()


@pytest.mark.parametrize("mode", ["hybrid", "spec"])
def test_full_1p7b_forced_stream_equals_oracle_loop(full_1p7b, oracle, mode):
    from tests.cpu_atlas import CpuAtlas, OracleModel, patched_host_ops
    cfg, model, om, atlas = full_1p7b
    D, prompt_len, new_tokens = 8, 256, 512
    prompt = synthetic.random_prompt(prompt_len, cfg["vocab_size"], seed=100)
    fn = {"hybrid": FG.fast_hybrid_generate, "spec": FG.fast_speculative_generate}[mode]

    cpu_atlas = CpuAtlas(om, model.args, (1024,), WIDTHS, ROLES)
    with patched_host_ops(D, synthetic.AcceptancePolicy("forced", D)):
        want, want_stats = fn(OracleModel(om, model.args), cpu_atlas, prompt, max_gen_len=new_tokens, eos_ids=())

    saved = FG._fused_draft_chain, FG._fused_verify_accept
    FG._fused_draft_chain, FG._fused_verify_accept = acceptance_hooks(FG, synthetic.AcceptancePolicy("forced", D))
    try:
        got, stats = fn(model, atlas, prompt, max_gen_len=new_tokens, eos_ids=())
    finally:
        FG._fused_draft_chain, FG._fused_verify_accept = saved
    assert native.lib().bm_device_error() == 0
    got, want = got.cpu().tolist(), want.tolist()
    assert len(want) == new_tokens
    first_diff = next((i for i, (a, b) in enumerate(zip(got, want)) if a != b), None)
    assert got == want, f"streams part at token {first_diff}"
    for key in ("n_iters", "draft_iters", "drafted_tokens", "accepted_drafts", "verifier_bonus_tokens",
                "n_conf_path", "n_verify_path", "decode_tokens", "timed_decode_tokens", "committed_tokens"):
        assert stats[key] == want_stats[key], key
    replayed = {(role, M) for (role, M, _, _, _) in cpu_atlas.log}
    assert replayed == ({("draft", 9), ("draft", 16)} if mode == "hybrid" else {("draft", 9), ("verify", 9)})


GEOM_4B_CUT = dict(synthetic.BONSAI_4B, n_layers=2, vocab_size=8192)
CASES_4B = [("ar", 1, 700, 0), ("verify", 9, 1500, 0), ("draft", 9, 33, 1), ("draft", 10, 2049, 2),
            ("draft", 12, 600, 4), ("draft", 16, 3000, 8), ("draft", 17, 95, 9), ("draft", 16, 4096, 8),
            ("ar", 16, 0, 0)]


@pytest.fixture(scope="module")
def cut_4b(oracle):
    cfg = synthetic.make_config(GEOM_4B_CUT, block_size=8)
    model, om = _build(cfg, 11, 4096 + 17, oracle)
    yield cfg, model, om
    del model
    torch.cuda.empty_cache()


@pytest.mark.parametrize("role,M,cache_len,n_pend", CASES_4B)
def test_4b_geometry_forward_matches_oracle(cut_4b, oracle, role, M, cache_len, n_pend):
    cfg, model, om = cut_4b
    sigma, m_max, D, L, Hkv = 4096, 17, 8, cfg["n_layers"], cfg["n_kv_heads"]
    gen = torch.Generator().manual_seed(M * 1000 + cache_len)
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
    logits = model.forward_sdlm_decode_graph_kernel(tokens.to(DEV), positions.to(DEV), kv_full, M, state_t, ls, le, "t2")
    torch.cuda.synchronize()
    assert native.lib().bm_device_error() == 0
    assert np.array_equal(logits.cpu().numpy().view(np.uint32), want.view(np.uint32)), "logits differ"
    assert np.array_equal(oracle.torch_to_u16(kvd.cpu()), kv_np), "KV buffer differs"


def test_4b_geometry_hybrid_stream_with_categorical_acceptance(cut_4b, oracle):
    from tests.cpu_atlas import CpuAtlas, OracleModel, patched_host_ops
    cfg, model, om = cut_4b
    D, ladder = 8, (4096,)
    prompt = synthetic.random_prompt(70, cfg["vocab_size"], seed=5)
    new_tokens = 160
    cpu_atlas = CpuAtlas(om, model.args, ladder, WIDTHS, ROLES)
    with patched_host_ops(D, synthetic.AcceptancePolicy("categorical", D, seed=2)):
        want, want_stats = FG.fast_hybrid_generate(OracleModel(om, model.args), cpu_atlas, prompt,
                                                   max_gen_len=new_tokens, eos_ids=())
    assert {("draft", 9), ("draft", 16), ("verify", 9)} <= {(r, M) for (r, M, _, _, _) in cpu_atlas.log}
    atlas = GraphAtlas(model, model.args, torch.device(DEV), segment_ladder=ladder, m_set=WIDTHS, roles=ROLES,
                       capture_verbose=False)
    saved = FG._fused_draft_chain, FG._fused_verify_accept
    FG._fused_draft_chain, FG._fused_verify_accept = acceptance_hooks(
        FG, synthetic.AcceptancePolicy("categorical", D, seed=2))
    try:
        got, stats = FG.fast_hybrid_generate(model, atlas, prompt, max_gen_len=new_tokens, eos_ids=())
    finally:
        FG._fused_draft_chain, FG._fused_verify_accept = saved
    assert native.lib().bm_device_error() == 0
    assert got.cpu().tolist() == want.tolist()
    for key in ("n_iters", "draft_iters", "accepted_drafts", "verifier_bonus_tokens", "n_conf_path",
                "n_verify_path", "decode_tokens"):
        assert stats[key] == want_stats[key], key
