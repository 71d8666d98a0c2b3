"""The dense draft heads (`draft_fp8`, `draft_bf16` roles): bm_dense_head against an fp32 PyTorch
evaluation of the SAME quantised operands, and the roles through the atlas and the decode loops.

The reference computes these two heads with cuBLASLt (torch._scaled_mm, F.linear), whose fp32
summation order is not reproducible on a CPU either, so parity here is a stated tolerance, not
bit-equality: every logit within one bf16 step of the fp32 result (2^-7 relative to the row's
scale covers a value that rounds across a bf16 boundary), the per-tensor activation scale exactly,
and the greedy token equal wherever the top-2 gap of the fp32 result exceeds that tolerance."""
import pytest
import torch

from bitmtp_b200 import fast_generate as FG, generate, native, ops, synthetic
from bitmtp_b200.fast_runtime import GraphAtlas

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
FP8_MAX = 448.0


def _table(n, k, seed):
    gen = torch.Generator().manual_seed(seed)
    _, _, w = synthetic.ternary_weight(n, k, gen)            # bf16 on the ternary grid, like the tied embedding
    h = (torch.randn(24, k, generator=gen) * 1.7).to(torch.bfloat16)
    return w.to(DEV), h.to(DEV)


def _check(got, ref32, rows):
    ref = ref32.to(torch.bfloat16).float()
    scale = ref32.abs().amax(dim=1, keepdim=True)
    tol = scale * 2.0 ** -7
    assert torch.all((got - ref).abs() <= tol), float(((got - ref).abs() / scale).max())
    top2 = ref32.topk(2, dim=1).values
    clear = (top2[:, 0] - top2[:, 1]) > 2 * tol[:, 0]
    assert torch.equal(got.argmax(1)[clear], ref32.argmax(1)[clear])
    assert int(clear.sum()) >= rows // 2


@pytest.mark.parametrize("R", [1, 8, 9, 17])
@pytest.mark.parametrize("N,K", [(4096, 2048), (5008, 2560), (151936, 2048)])
def test_bf16_head_against_fp32_matmul(R, N, K):
    if N > 100000 and R not in (8, 17):
        pytest.skip("the full-size table is checked at the two widths a draft replay uses")
    w, h = _table(N, K, seed=N + R)
    h = h[:R].contiguous()
    out = torch.zeros(R, N + 32, dtype=torch.float32, device=DEV)
    ops.dense_head(h, w, out=out)
    torch.cuda.synchronize()
    ref32 = h.float() @ w.float().T
    _check(out[:, :N], ref32, R)
    assert float(out[:, N:].abs().sum()) == 0.0                      # columns past N are not touched
    assert native.lib().bm_device_error() == 0


@pytest.mark.parametrize("R", [1, 8, 9, 17])
@pytest.mark.parametrize("N,K", [(4096, 2048), (5008, 2560), (151936, 2048)])
def test_fp8_head_against_fp32_matmul_of_the_same_e4m3_operands(R, N, K):
    if N > 100000 and R not in (8, 17):
        pytest.skip("the full-size table is checked at the two widths a draft replay uses")
    w, h = _table(N, K, seed=N + 3 * R)
    h = h[:R].contiguous()
    # the reference's expressions (model.py:1185-1187, 1267-1269), evaluated with torch on the device
    w_scale = (w.abs().amax() / FP8_MAX).clamp_min(1e-12).to(torch.float32)
    w8 = (w / w_scale).to(torch.float8_e4m3fn)
    h_scale = (h.abs().amax() / FP8_MAX).clamp_min(1e-12).to(torch.float32)
    h8 = (h / h_scale).to(torch.float8_e4m3fn)
    out = torch.zeros(R, N, dtype=torch.float32, device=DEV)
    got_scale = torch.zeros(1, dtype=torch.float32, device=DEV)
    ops.dense_head(h, w8, out=out, w_scale=w_scale.reshape(1).contiguous(), h_scale_out=got_scale)
    torch.cuda.synchronize()
    assert float(got_scale) == float(h_scale), "per-tensor activation scale"
    ref32 = (h8.float() @ w8.float().T) * (h_scale * w_scale)
    _check(out, ref32, R)
    assert native.lib().bm_device_error() == 0


@pytest.mark.parametrize("role,kw", [("draft_fp8", {"use_fp8_draft": True}), ("draft_bf16", {"use_bf16_draft": True})])
def test_dense_draft_roles_through_the_atlas_and_the_loops(role, kw):
    """The roles capture, report their head precision, share the segment's KV buffer with the other
    graphs, and a hybrid generation with forced acceptance runs on them; the draft logits of a replay
    equal the head applied to the replay's own normed rows."""
    cfg = synthetic.make_config(dict(synthetic.TINY, vocab_size=1008), block_size=8)
    state = synthetic.make_state(cfg, seed=7)
    model = generate.model_from_state(generate.args_from_config(cfg), state, DEV)
    model.prepare_merged_weights(max_positions=256 + 17)
    atlas = GraphAtlas(model, model.args, torch.device(DEV), segment_ladder=(256,), m_set=(1, 8, 9, 10, 12, 16, 17),
                       roles=("ar", role, "verify"), capture_verbose=False)
    want_precision = {"draft_fp8": "fp8", "draft_bf16": "bf16_raw"}[role]
    assert atlas.graphs[(16, 256, role)].lm_head_precision == want_precision
    assert atlas.graphs[(9, 256, "verify")].lm_head_precision == "t2"
    assert {g.kv_full[0][0].data_ptr() for g in atlas.graphs.values()} == {atlas.kv_buffers[256].data_ptr()}
    prompt = synthetic.random_prompt(30, cfg["vocab_size"], seed=3)
    saved = FG._fused_draft_chain, FG._fused_verify_accept
    FG._fused_draft_chain, FG._fused_verify_accept = synthetic.acceptance_hooks(FG, synthetic.AcceptancePolicy("forced", 8))
    try:
        out, stats = FG.fast_hybrid_generate(model, atlas, prompt, max_gen_len=64, eos_ids=(), **kw)
    finally:
        FG._fused_draft_chain, FG._fused_verify_accept = saved
    assert out.numel() == 64 and stats["n_verify_path"] == 0 and stats["n_conf_path"] >= 8
    assert native.lib().bm_device_error() == 0
    # the last draft replay: logits of rows P..M against the head on the workspace's normed rows
    g = atlas.graphs[(16, 256, role)]
    hn = model.workspace(16).hn[:8].float()
    W = model.embed_tokens.weight.data
    if role == "draft_bf16":
        ref32 = hn @ W.float().T
    else:
        w8 = model._lm_head_fp8_w[: cfg["vocab_size"]].float()
        h_scale = (hn.abs().amax() / FP8_MAX).to(torch.bfloat16).float().clamp_min(1e-12)
        h8 = (model.workspace(16).hn[:8] / h_scale).to(torch.float8_e4m3fn).float()
        ref32 = (h8 @ w8.T) * (h_scale * model._lm_head_w_scale)
    _check(g.logits_out[:, : cfg["vocab_size"]], ref32, 8)


def test_cli_accepts_the_dense_draft_precisions():
    from bitmtp_b200 import run_generation as RG
    for prec, role in (("fp8", "draft_fp8"), ("bf16", "draft_bf16")):
        args = RG.make_parser().parse_args(["--ckpt", "x", "--hf-ckpt", "y", "--block-size", "8", "--mode", "hybrid",
                                            "--prompt", "hi", "--draft-precision", prec])
        widths, roles, _ = RG.validate_options(args)
        assert role in roles and "verify" in roles


@pytest.mark.parametrize("mode,draft", [("ar", None), ("confidence", "draft"), ("hybrid", "draft_fp8"),
                                        ("speculative", "draft_bf16")])
def test_atlas_passes_the_checks_of_the_reference_evaluation_adapter(mode, draft):
    """What the reference's lm-eval / EvalPlus adapter asserts right after it builds its atlas
    (benchmarks/bonsai_adapter.py:118-157), with its constructor arguments and its role ordering: ladder, width
    schedule and role tuple come back unchanged, every captured graph reports the head precision of its role, and
    every graph's per-layer K / V views start at the segment's shared buffer."""
    cfg = synthetic.make_config(dict(synthetic.TINY, vocab_size=1008), block_size=8)
    state = synthetic.make_state(cfg, seed=11)
    model = generate.model_from_state(generate.args_from_config(cfg), state, DEV)
    model.prepare_merged_weights(max_positions=512 + 17)
    ladder, widths = (128, 512), ((1,) if mode == "ar" else (1, 8, 9, 10, 12, 16, 17))
    roles = ("ar",) if mode == "ar" else ((draft, "ar") if mode == "confidence" else (draft, "verify", "ar"))
    atlas = GraphAtlas(model, model.args, torch.device(DEV), dtype=torch.bfloat16, segment_ladder=ladder, m_set=widths,
                       roles=roles, capture_verbose=False)
    assert atlas.segment_ladder == ladder and atlas.m_set == widths and tuple(atlas.roles) == tuple(roles)
    expected = {"ar": "t2", "verify": "t2", "draft": "t2", "draft_fp8": "fp8", "draft_bf16": "bf16_raw"}
    assert atlas.graphs, "no graph captured"
    for (width, sigma, role), graph in atlas.graphs.items():
        assert role in expected and graph.lm_head_precision == expected[role]
        shared = atlas.kv_buffers[sigma]
        for layer, (key_view, value_view) in enumerate(graph.kv_full):
            assert key_view.data_ptr() == shared[0, layer].data_ptr()
            assert value_view.data_ptr() == shared[1, layer].data_ptr()
    assert native.lib().bm_device_error() == 0
