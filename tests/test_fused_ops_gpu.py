"""GPU parity of the fused operators and the block-verify attention against the CPU
oracle, through the C ABI.  Everything here is compared bit for bit: INT8 codes,
fp32 multipliers, bf16 rows."""
import numpy as np
import pytest
import torch

from bitmtp_b200 import native, ops, synthetic

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _bf16(gen, *shape, scale=1.0):
    return (torch.randn(*shape, generator=gen) * scale).to(torch.bfloat16)


def _u16(O, t):
    return O.torch_to_u16(t.cpu())


@pytest.mark.parametrize("M,K", [(1, 2048), (9, 6144), (16, 9728), (17, 256), (3, 2560), (5, 64)])
def test_quant_rows(oracle, M, K):
    gen = torch.Generator().manual_seed(M * 7 + K)
    x = _bf16(gen, M, K, scale=3.0)
    x[0, 0] = 0.0
    if M > 2:
        x[2].zero_()                                  # all-zero row: the 1e-5 clamp
    q, s = ops.quant_rows(x.to(DEV))
    qo, so = oracle.quant_rows(_u16(oracle, x))
    assert np.array_equal(q.cpu().numpy(), qo)
    assert np.array_equal(s.cpu().numpy().reshape(-1).view(np.uint32), so.view(np.uint32))


@pytest.mark.parametrize("M,dim", [(1, 2048), (16, 2048), (9, 2560), (17, 256), (4, 4096)])
def test_rmsnorm_variants(oracle, M, dim):
    gen = torch.Generator().manual_seed(M + dim)
    x, res = _bf16(gen, M, dim, scale=2.0), _bf16(gen, M, dim, scale=0.5)
    w = (1.0 + 0.1 * torch.randn(dim, generator=gen)).to(torch.bfloat16)
    eps = 1e-6
    xd, rd, wd = x.to(DEV), res.to(DEV), w.to(DEV)
    xu, ru, wu = _u16(oracle, x), _u16(oracle, res), _u16(oracle, w)
    # norm + quant
    o = ops.rmsnorm_fused(xd, wd, eps)
    qo, so = oracle.rmsnorm_quant(xu, wu, eps)
    assert np.array_equal(o["q"].cpu().numpy(), qo)
    assert np.array_equal(o["s"].cpu().numpy().reshape(-1).view(np.uint32), so.view(np.uint32))
    # add + norm + quant, returning h
    o = ops.rmsnorm_fused(xd, wd, eps, res=rd, want_h=True)
    ho, qo, so = oracle.add_rmsnorm_quant(xu, ru, wu, eps)
    assert np.array_equal(_u16(oracle, o["h"]), ho)
    assert np.array_equal(o["q"].cpu().numpy(), qo)
    assert np.array_equal(o["s"].cpu().numpy().reshape(-1).view(np.uint32), so.view(np.uint32))
    # plain norm with bf16 output, on a row window
    row0 = 1 if M > 2 else 0
    o = ops.rmsnorm_fused(xd, wd, eps, row0=row0, M=M - row0, want_q=False, want_n=True)
    no = oracle.rmsnorm(np.ascontiguousarray(xu[row0:]), wu, eps)
    assert np.array_equal(_u16(oracle, o["n"]), no)


def test_embedding_gather_norm(oracle):
    gen = torch.Generator().manual_seed(5)
    table = _bf16(gen, 1000, 2048, scale=0.03)
    w = torch.ones(2048, dtype=torch.bfloat16)
    tok = torch.tensor([5, 999, 0, 17, 5], dtype=torch.int64)
    o = ops.rmsnorm_fused(table.to(DEV), w.to(DEV), 1e-6, gather=tok.to(DEV), want_h=True)
    rows = np.ascontiguousarray(_u16(oracle, table)[tok.numpy()])
    qo, so = oracle.rmsnorm_quant(rows, _u16(oracle, w), 1e-6)
    assert np.array_equal(_u16(oracle, o["h"]), rows)
    assert np.array_equal(o["q"].cpu().numpy(), qo)
    assert np.array_equal(o["s"].cpu().numpy().reshape(-1).view(np.uint32), so.view(np.uint32))


@pytest.mark.parametrize("M,F", [(1, 6144), (16, 6144), (9, 9728), (3, 512)])
def test_silu_mul_quant(oracle, M, F):
    gen = torch.Generator().manual_seed(M + F)
    gu = _bf16(gen, M, 2 * F, scale=4.0)
    gu[0, :4] = torch.tensor([-100.0, 100.0, 0.0, -20.0], dtype=torch.bfloat16)
    q, s, inner = ops.silu_mul_quant(gu.to(DEV), want_inner=True)
    qo, so, io = oracle.silu_mul_quant(_u16(oracle, gu), want_inner=True)
    assert np.array_equal(_u16(oracle, inner), io)
    assert np.array_equal(q.cpu().numpy(), qo)
    assert np.array_equal(s.cpu().numpy().reshape(-1).view(np.uint32), so.view(np.uint32))


def _rope_tables(oracle, max_pos):
    from bitmtp_b200 import synthetic
    cfg = synthetic.make_config(synthetic.TINY)
    return oracle.rope_tables(cfg, max_pos)


@pytest.mark.parametrize("M,H,Hkv", [(1, 16, 8), (16, 16, 8), (9, 32, 8), (17, 2, 1)])
def test_qknorm_rope_kvappend(oracle, M, H, Hkv):
    gen = torch.Generator().manual_seed(M + H)
    sigma, kv_rows = 40, 40 + 17
    xqkv = _bf16(gen, M, (H + 2 * Hkv) * 128, scale=2.0)
    qw = (1.0 + 0.1 * torch.randn(128, generator=gen)).to(torch.bfloat16)
    kw = (1.0 + 0.1 * torch.randn(128, generator=gen)).to(torch.bfloat16)
    cos, sin = _rope_tables(oracle, 600)
    pos = torch.randint(0, 600, (M,), generator=gen, dtype=torch.int64)
    k0 = _bf16(gen, Hkv, kv_rows, 128)
    v0 = _bf16(gen, Hkv, kv_rows, 128)
    ku, vu = _u16(oracle, k0).copy(), _u16(oracle, v0).copy()
    qo = oracle.qknorm_rope_kvappend(_u16(oracle, xqkv), _u16(oracle, qw), _u16(oracle, kw), 1e-6,
                                     cos, sin, pos.numpy(), H, Hkv, ku, vu, sigma)
    kd, vd = k0.to(DEV), v0.to(DEV)
    q = ops.qknorm_rope_kvappend(xqkv.to(DEV), qw.to(DEV), kw.to(DEV), 1e-6,
                                 oracle.u16_to_torch(cos).to(DEV), oracle.u16_to_torch(sin).to(DEV),
                                 pos.to(DEV), H, Hkv, kd, vd, sigma)
    assert np.array_equal(_u16(oracle, q), qo)
    assert np.array_equal(_u16(oracle, kd), ku)
    assert np.array_equal(_u16(oracle, vd), vu)


ATTN_CASES = [
    # (M, H, Hkv, sigma, cache_len, n_pend, D, role)
    (1, 16, 8, 256, 77, 0, 8, "ar"),
    (1, 2, 1, 64, 0, 0, 8, "ar"),
    (9, 16, 8, 256, 100, 1, 8, "draft"),
    (10, 16, 8, 256, 129, 2, 8, "draft"),
    (12, 16, 8, 256, 33, 3, 8, "draft"),
    (16, 16, 8, 1024, 700, 8, 8, "draft"),
    (16, 32, 8, 256, 64, 5, 8, "draft"),
    (8, 2, 1, 64, 31, 0, 8, "draft"),
    (9, 16, 8, 256, 100, 0, 8, "verify"),
    (9, 32, 8, 1024, 513, 0, 8, "verify"),
    (5, 2, 1, 64, 20, 1, 4, "draft"),
    (16, 16, 8, 256, 0, 0, 8, "ar"),
    (17, 16, 8, 256, 40, 9, 8, "draft"),
    (16, 16, 8, 4096, 2500, 8, 8, "draft"),    # long segment: the three-CTAs-per-SM build of the chunk kernel
    (9, 32, 8, 4096, 3000, 0, 8, "verify"),
    (16, 16, 8, 256, 256, 8, 8, "draft"),      # the history fills the whole segment (cache_len == sigma)
    (9, 16, 8, 64, 64, 0, 8, "verify"),
    # grids that are resident at once run as thread-block clusters (merge through distributed shared memory)
    (1, 16, 8, 1024, 1000, 0, 8, "ar"),        # nine CTAs per cluster, all with rows
    (1, 32, 8, 1024, 513, 0, 8, "ar"),
    (8, 16, 8, 1024, 700, 0, 8, "draft"),      # 288 CTAs in 32 clusters, three of nine CTAs without rows
    (4, 16, 8, 1920, 1901, 0, 4, "draft"),     # the largest cluster (16)
    (4, 16, 8, 1920, 0, 0, 4, "ar"),           # only the CTA of the replay's own rows works
]


@pytest.mark.parametrize("M,H,Hkv,sigma,cache_len,n_pend,D,role", ATTN_CASES)
def test_verify_attention(oracle, M, H, Hkv, sigma, cache_len, n_pend, D, role):
    gen = torch.Generator().manual_seed(M * 31 + cache_len)
    kv_rows = sigma + 17
    q = _bf16(gen, M, H, 128, scale=1.5)
    k = _bf16(gen, Hkv, kv_rows, 128, scale=1.5)
    v = _bf16(gen, Hkv, kv_rows, 128)
    rid = oracle.ROLE_IDS[role]
    P = M - D
    att_o = oracle.attention(_u16(oracle, q), _u16(oracle, k), _u16(oracle, v), sigma, cache_len,
                             n_pend, P, rid)
    qo, so = oracle.quant_rows(att_o)
    state = ops.new_step_state(DEV)
    ops.set_step_state(state, cache_len, n_pend, rid, P)
    scratch = ops.attention_scratch(M, H, sigma, DEV)
    for rep in range(2):                               # second call: scratch counters were left zero
        att, qq, s = ops.verify_attention(q.to(DEV), k.to(DEV), v.to(DEV), sigma, state, scratch)
        torch.cuda.synchronize()
        assert np.array_equal(_u16(oracle, att), att_o), f"attention rows differ (call {rep})"
        assert np.array_equal(qq.cpu().numpy(), qo)
        assert np.array_equal(s.cpu().numpy().reshape(-1).view(np.uint32), so.view(np.uint32))
    assert int(scratch[:256].sum().item()) == 0


def test_attention_clamps_a_record_beyond_the_segment(oracle):
    """A step record that claims more history than the segment holds (a stale record, a wrong segment
    passed through the C ABI) must not index past the scratch or the K/V planes: the kernels clamp the
    length to sigma, so the call equals the one with cache_len == sigma."""
    M, H, Hkv, sigma, D = 9, 16, 8, 64, 8
    gen = torch.Generator().manual_seed(5)
    q = _bf16(gen, M, H, 128, scale=1.5).to(DEV)
    k = _bf16(gen, Hkv, sigma + 17, 128, scale=1.5).to(DEV)
    v = _bf16(gen, Hkv, sigma + 17, 128).to(DEV)
    scratch = ops.attention_scratch(M, H, sigma, DEV)
    outs = []
    for claimed in (sigma, sigma + 1000):
        state = ops.new_step_state(DEV)
        ops.set_step_state(state, claimed, 1, native.ROLE_DRAFT, M - D)
        att, qq, s = ops.verify_attention(q, k, v, sigma, state, scratch)
        torch.cuda.synchronize()
        outs.append((att.clone(), qq.clone(), s.clone()))
    assert native.lib().bm_device_error() == 0
    for a, b in zip(outs[0], outs[1]):
        assert torch.equal(a.view(torch.uint8), b.view(torch.uint8))


def test_argmax_of_nan_rows_stays_inside_the_row(oracle):
    """A row of NaNs (a corrupt scale upstream) must still give an index inside the row: the id stays on
    the device and feeds the next replay's embedding gather.  NaN counts as the maximum and the lowest
    index wins, as torch.argmax does; the gather itself clamps ids it is given."""
    vocab = 5000
    lg = torch.randn(4, vocab)
    lg[0] = float("nan")
    lg[1, 1234] = float("nan")
    lg[1, 4000] = float("nan")
    lg[2] = float("-inf")
    want = torch.argmax(lg, dim=-1)
    assert want.tolist()[:3] == [0, 1234, 0]
    assert np.array_equal(oracle.argmax_rows(lg.numpy()), want.numpy())
    d = lg.to(DEV)
    assert torch.equal(ops.argmax_rows(d).cpu(), want)
    assert torch.equal(ops.argmax_rows(d, scratch=ops.logit_scratch(DEV)).cpu(), want)
    # out-of-table ids are clamped by the gathering RMSNorm
    table = _bf16(torch.Generator().manual_seed(1), 10, 256).to(DEV)
    w = torch.ones(256, dtype=torch.bfloat16, device=DEV)
    ids = torch.tensor([2 ** 31 - 1, -5, 3], dtype=torch.int64, device=DEV)
    got = ops.rmsnorm_fused(table, w, 1e-6, gather=ids, want_q=False, want_h=True)["h"]
    assert torch.equal(got.view(torch.int16), table[[9, 0, 3]].view(torch.int16))


def test_kv_copy_rows():
    gen = torch.Generator().manual_seed(3)
    kv = _bf16(gen, 2, 3, 1, 2, 50, 128).to(DEV)
    ref = kv.clone()
    ops.kv_copy_rows(kv, 50, 40, 7, 5)
    ref[..., 7:12, :] = ref[..., 40:45, :]
    assert torch.equal(kv, ref)


def test_logit_reductions(oracle):
    gen = torch.Generator().manual_seed(9)
    D, vocab = 8, 151936
    logits = (torch.randn(D, vocab, generator=gen) * 3).to(torch.bfloat16).float()
    logits[1, 777] = 60.0
    logits[2, 5] = 60.0
    logits[3, 100] = logits[3].max()
    logits[3, 90000] = logits[3].max()                 # tie: the lower index wins
    lg = logits.to(DEV)
    idx = ops.argmax_rows(lg)
    assert np.array_equal(idx.cpu().numpy(), oracle.argmax_rows(logits.numpy()))
    for tau in (0.9, 0.5):
        i2, n, conf = ops.draft_chain(lg, tau)
        io, no, co = oracle.draft_chain(logits.numpy(), tau)
        assert np.array_equal(i2.cpu().numpy(), io)
        assert int(n.item()) == no
        assert np.array_equal(conf.cpu().numpy().view(np.uint32), co.view(np.uint32))
    a = torch.tensor([1, 2, 3, 4, 5, 6, 7, 8], dtype=torch.int64)
    b = torch.tensor([1, 2, 3, 9, 5, 6, 7, 8, 0], dtype=torch.int64)
    assert int(ops.verify_accept(a.to(DEV), b.to(DEV), 8).item()) == oracle.verify_accept(a.numpy(), b.numpy(), 8) == 3


def _permute16(q_nat: np.ndarray) -> np.ndarray:
    """Natural-order codes -> GEMV-ready order: every run of 16 transposed 4x4."""
    M, K = q_nat.shape
    return q_nat.reshape(M, K // 16, 4, 4).transpose(0, 1, 3, 2).reshape(M, K).copy()


@pytest.mark.parametrize("M,K", [(1, 2048), (16, 6144), (9, 2560), (5, 256)])
def test_prepared_outputs_and_prepared_gemv(oracle, M, K):
    """q_prep is the 4x4 transpose of q per 16-run, asum the per-group code sums, and the
    GEMV on them equals the GEMV on natural-order codes bit for bit."""
    from bitmtp_b200 import synthetic
    gen = torch.Generator().manual_seed(M + K)
    x = _bf16(gen, M, K, scale=2.0)
    q, s = ops.quant_rows(x.to(DEV))
    qp, asum, s2 = ops.quant_rows(x.to(DEV), prepared=True)
    qn = q.cpu().numpy()
    assert np.array_equal(qp.cpu().numpy(), _permute16(qn))
    assert np.array_equal(asum.cpu().numpy(), qn.astype(np.int32).reshape(M, K // 128, 128).sum(-1))
    assert torch.equal(s, s2)
    N = 512
    packed, scale, _ = synthetic.ternary_weight(N, K, gen)
    Bd, wsd = packed.to(DEV), scale.to(DEV)
    want = ops.t2_gemv(q, Bd, s, wsd, out_kind=native.OUT_F32)
    got = torch.empty_like(want)
    ops.t2_gemv_prepared(qp, asum, Bd, s, wsd, out=got, out_kind=native.OUT_F32)
    assert torch.equal(got, want)
    y32, _, _ = oracle.t2_gemv(qn, packed.numpy().view(np.uint8), oracle.torch_to_u16(scale),
                               s.cpu().numpy().reshape(-1))
    assert np.array_equal(got.cpu().numpy().view(np.uint32), y32.view(np.uint32))


def test_prepared_from_norm_silu_attention(oracle):
    gen = torch.Generator().manual_seed(77)
    # rmsnorm
    x = _bf16(gen, 9, 2048, scale=2.0)
    w = (1.0 + 0.1 * torch.randn(2048, generator=gen)).to(torch.bfloat16)
    a = ops.rmsnorm_fused(x.to(DEV), w.to(DEV), 1e-6)
    b = ops.rmsnorm_fused(x.to(DEV), w.to(DEV), 1e-6, want_q=False, want_prep=True)
    qn = a["q"].cpu().numpy()
    assert np.array_equal(b["qp"].cpu().numpy(), _permute16(qn))
    assert np.array_equal(b["asum"].cpu().numpy(), qn.astype(np.int32).reshape(9, 16, 128).sum(-1))
    # silu
    gu = _bf16(gen, 5, 2 * 6144, scale=3.0).to(DEV)
    q, s = ops.silu_mul_quant(gu)
    qp = torch.empty_like(q)
    asum = torch.empty(5, 48, dtype=torch.int32, device=DEV)
    s2 = torch.empty_like(s)
    ops.silu_mul_quant(gu, out=(None, s2), prep=(qp, asum))
    qn = q.cpu().numpy()
    assert np.array_equal(qp.cpu().numpy(), _permute16(qn)) and torch.equal(s, s2)
    assert np.array_equal(asum.cpu().numpy(), qn.astype(np.int32).reshape(5, 48, 128).sum(-1))
    # attention
    M, H, Hkv, sigma = 9, 16, 8, 256
    qv = _bf16(gen, M, H, 128).to(DEV)
    k = _bf16(gen, Hkv, sigma + 17, 128).to(DEV)
    v = _bf16(gen, Hkv, sigma + 17, 128).to(DEV)
    st = ops.new_step_state(DEV)
    ops.set_step_state(st, 100, 1, 0, 1)
    scr = ops.attention_scratch(M, H, sigma, DEV)
    att, qq, ss = ops.verify_attention(qv, k, v, sigma, st, scr)
    qp = torch.empty_like(qq)
    asum = torch.empty(M, H, dtype=torch.int32, device=DEV)
    out2 = (torch.empty_like(att), None, torch.empty_like(ss))
    ops.verify_attention(qv, k, v, sigma, st, scr, out=out2, prep=(qp, asum))
    qn = qq.cpu().numpy()
    assert torch.equal(out2[0], att) and torch.equal(out2[2], ss)
    assert np.array_equal(qp.cpu().numpy(), _permute16(qn))
    assert np.array_equal(asum.cpu().numpy(), qn.astype(np.int32).reshape(M, H, 128).sum(-1))


@pytest.mark.parametrize("M,F,K", [(1, 6144, 2048), (9, 6144, 2048), (16, 6144, 2048), (8, 9728, 2560), (16, 768, 512),
                                   (5, 512, 256)])
def test_gate_up_silu_gemv_and_amax_quant(M, F, K):
    """SiLU(gate)*up in the GEMV epilogue + quantisation with the gathered absmax against the unfused
    chain GEMV -> bm_silu_mul_quant (each checked against the oracle elsewhere): inner rows, absmax,
    codes, GEMV-ready codes, group sums and multipliers bit for bit; two calls on reused buffers."""
    from bitmtp_b200 import synthetic
    case = synthetic.gemv_case(M, 2 * F, K, seed=M + F)
    A, B, ws, s = (case[k].to(DEV) for k in ("A", "B", "ws", "s"))
    prep = A.view(M, -1, 4, 4).transpose(2, 3).contiguous().view(M, -1)
    asum = A.view(M, -1, 128).to(torch.int32).sum(-1).to(torch.int32).contiguous()
    gu = torch.empty(M, 2 * F, dtype=torch.bfloat16, device=DEV)
    ops.t2_gemv_prepared(prep, asum, B, s, ws, out=gu)
    ref_qp = torch.empty(M, F, dtype=torch.int8, device=DEV)
    ref_sum = torch.empty(M, F // 128, dtype=torch.int32, device=DEV)
    ref_q = torch.empty(M, F, dtype=torch.int8, device=DEV)
    ref_s = torch.empty(M, 1, dtype=torch.float32, device=DEV)
    _, _, ref_inner = ops.silu_mul_quant(gu, want_inner=True, out=(ref_q, ref_s), prep=(ref_qp, ref_sum))

    amax = torch.zeros(2, M, dtype=torch.int32, device=DEV)
    inner = torch.empty(M, F, dtype=torch.bfloat16, device=DEV)
    q = torch.empty(M, F, dtype=torch.int8, device=DEV)
    qp = torch.empty(M, F, dtype=torch.int8, device=DEV)
    isum = torch.empty(M, F // 128, dtype=torch.int32, device=DEV)
    s_out = torch.empty(M, 1, dtype=torch.float32, device=DEV)
    for rep in range(2):
        slot, nxt = rep & 1, (rep + 1) & 1
        ops.gate_up_silu(prep, asum, B, s, ws, inner=inner, amax=amax[slot])
        ops.quant_rows_amax(inner, amax[slot], prep=(qp, isum), s=s_out, amax_zero=amax[nxt], q=q)
        torch.cuda.synchronize()
        assert int(amax[nxt].abs().sum()) == 0, "the other slot was not cleared"
        assert torch.equal(inner.view(torch.int16), ref_inner.view(torch.int16)), f"inner rows differ (call {rep})"
        assert torch.equal(amax[slot].view(torch.float32), ref_inner.float().abs().amax(dim=1)), "absmax differs"
        assert torch.equal(q, ref_q) and torch.equal(qp, ref_qp), "codes differ"
        assert torch.equal(isum, ref_sum), "group sums differ"
        assert torch.equal(s_out.view(torch.int32), ref_s.view(torch.int32)), "multipliers differ"
    assert native.lib().bm_device_error() == 0


@pytest.mark.parametrize("M,H,Hkv,sigma,cache_len,n_pend,D,role", ATTN_CASES)
def test_rope_folded_into_attention(oracle, M, H, Hkv, sigma, cache_len, n_pend, D, role):
    """bm_rope_verify_attention (q/k norm + RoPE + KV append inside the chunk kernel) against the two
    separate calls: attention rows, codes, multipliers and the KV planes bit for bit."""
    gen = torch.Generator().manual_seed(M * 17 + cache_len + H)
    kv_rows = sigma + 17
    xqkv = _bf16(gen, M, (H + 2 * Hkv) * 128, scale=2.0).to(DEV)
    qw = (1.0 + 0.1 * torch.randn(128, generator=gen)).to(torch.bfloat16).to(DEV)
    kw = (1.0 + 0.1 * torch.randn(128, generator=gen)).to(torch.bfloat16).to(DEV)
    cos, sin = _rope_tables(oracle, sigma + 40)
    cos, sin = oracle.u16_to_torch(cos).to(DEV), oracle.u16_to_torch(sin).to(DEV)
    pos = (torch.arange(M) + max(cache_len - 1, 0)).to(torch.int64).to(DEV)
    k0 = _bf16(gen, Hkv, kv_rows, 128, scale=1.5)
    v0 = _bf16(gen, Hkv, kv_rows, 128)
    rid = oracle.ROLE_IDS[role]
    state = ops.new_step_state(DEV)
    ops.set_step_state(state, cache_len, n_pend, rid, M - D)
    scratch = ops.attention_scratch(M, H, sigma, DEV)

    ka, va = k0.to(DEV), v0.to(DEV)
    q = ops.qknorm_rope_kvappend(xqkv, qw, kw, 1e-6, cos, sin, pos, H, Hkv, ka, va, sigma)
    att_a, q_a, s_a = ops.verify_attention(q, ka, va, sigma, state, scratch)

    kb, vb = k0.to(DEV), v0.to(DEV)
    att_b = torch.empty_like(att_a)
    q_b = torch.empty_like(q_a)
    s_b = torch.empty_like(s_a)
    for rep in range(2):
        ops.rope_verify_attention(xqkv, qw, kw, 1e-6, cos, sin, pos, H, Hkv, kb, vb, sigma, state, scratch,
                                  out=(att_b, q_b, s_b))
        torch.cuda.synchronize()
        assert torch.equal(att_a.view(torch.int16), att_b.view(torch.int16)), f"attention rows differ (call {rep})"
        assert torch.equal(q_a, q_b) and torch.equal(s_a.view(torch.int32), s_b.view(torch.int32))
        assert torch.equal(ka.view(torch.int16), kb.view(torch.int16)), "K planes differ"
        assert torch.equal(va.view(torch.int16), vb.view(torch.int16)), "V planes differ"
    if H % 4 == 0:
        # rows-only variant (merge spread over head groups) + quantisation with the gathered absmax
        kc, vc = k0.to(DEV), v0.to(DEV)
        amax = torch.zeros(2, M, dtype=torch.int32, device=DEV)
        att_c = torch.zeros_like(att_a)
        q_c, s_c = torch.empty_like(q_a), torch.empty_like(s_a)
        qp_c = torch.empty_like(q_a)
        sum_c = torch.empty(M, H, dtype=torch.int32, device=DEV)
        for rep in range(2):
            slot = rep & 1
            ops.rope_verify_attention_rows(xqkv, qw, kw, 1e-6, cos, sin, pos, H, Hkv, kc, vc, sigma, state, scratch,
                                           att=att_c, amax=amax[slot])
            ops.quant_rows_amax(att_c, amax[slot], prep=(qp_c, sum_c), s=s_c, amax_zero=amax[1 - slot], q=q_c)
            torch.cuda.synchronize()
            assert torch.equal(att_a.view(torch.int16), att_c.view(torch.int16)), f"rows differ (split merge, call {rep})"
            assert torch.equal(q_a, q_c) and torch.equal(s_a.view(torch.int32), s_c.view(torch.int32))
            assert torch.equal(ka.view(torch.int16), kc.view(torch.int16)) and torch.equal(va.view(torch.int16), vc.view(torch.int16))
    assert native.lib().bm_device_error() == 0


@pytest.mark.parametrize("M,D,n_pend,cache_len", [(9, 8, 1, 40), (10, 8, 2, 7), (12, 8, 3, 100), (16, 8, 8, 300),
                                                  (17, 8, 9, 12), (16, 8, 5, 1), (5, 4, 1, 9), (9, 4, 5, 64)])
def test_stage_replay_inputs_matches_the_tensor_fills(M, D, n_pend, cache_len):
    """bm_stage_replay_inputs against the per-step tensor fills of the decode loops (draft, verify, AR)."""
    MASK = 151654
    P = M - D
    gen = torch.Generator().manual_seed(M * 31 + n_pend)
    pending = torch.randint(0, 150000, (18,), generator=gen, dtype=torch.int64).to(DEV)
    draft = torch.randint(0, 150000, (D,), generator=gen, dtype=torch.int64).to(DEV)
    ar = torch.arange(32, dtype=torch.int64, device=DEV)
    # draft
    tok = torch.full((M,), -7, dtype=torch.int64, device=DEV)
    pos = torch.full((M,), -7, dtype=torch.int64, device=DEV)
    tok[:n_pend] = pending[:n_pend]
    if n_pend < P:
        tok[n_pend:P] = 0
        pos[n_pend:P] = 0
    tok[P:P + 1] = pending[n_pend - 1:n_pend]
    if P + 1 < M:
        tok[P + 1:] = MASK
    pos[:n_pend] = ar[:n_pend] + cache_len
    pos[P:P + D] = ar[:D] + (cache_len + n_pend - 1)
    tok2, pos2 = torch.full_like(tok, -1), torch.full_like(pos, -1)
    st = ops.new_step_state(DEV)
    ops.stage_replay_inputs(0, pending, None, n_pend, cache_len, M, D, MASK, native.ROLE_DRAFT, P, tok2, pos2, st)
    assert torch.equal(tok, tok2) and torch.equal(pos, pos2)
    assert st.cpu().tolist() == [cache_len, max(0, min(n_pend, max(P, 0))), native.ROLE_DRAFT, P]
    # verify (width D + 1)
    tokv = torch.cat([pending[n_pend - 1:n_pend], draft])
    posv = ar[:D + 1] + (cache_len - 1)
    tok3, pos3 = torch.empty_like(tokv), torch.empty_like(posv)
    ops.stage_replay_inputs(1, pending, draft, n_pend, cache_len, D + 1, D, 0, native.ROLE_VERIFY, 1, tok3, pos3, st)
    assert torch.equal(tokv, tok3) and torch.equal(posv, pos3)
    assert st.cpu().tolist() == [cache_len, 0, native.ROLE_VERIFY, 1]
    # AR
    tok4, pos4 = torch.empty(1, dtype=torch.int64, device=DEV), torch.empty(1, dtype=torch.int64, device=DEV)
    ops.stage_replay_inputs(2, draft[2:3], None, 0, cache_len, 1, 0, 0, native.ROLE_AR, 1 - D, tok4, pos4, st)
    assert int(tok4) == int(draft[2]) and int(pos4) == cache_len
    assert st.cpu().tolist() == [cache_len, 0, native.ROLE_AR, 1 - D]
    # prompt slab (width M, n_pend real rows taken from an offset of the prompt)
    tok5, pos5 = torch.full((M,), -1, dtype=torch.int64, device=DEV), torch.full((M,), -1, dtype=torch.int64, device=DEV)
    ops.stage_replay_inputs(3, pending[1:], None, n_pend, cache_len, M, D, 0, native.ROLE_AR, P, tok5, pos5, st)
    assert tok5.tolist() == pending[1:1 + n_pend].tolist() + [0] * (M - n_pend)
    assert pos5.tolist() == [cache_len + i for i in range(n_pend)] + [0] * (M - n_pend)
    assert st.cpu().tolist() == [cache_len, 0, native.ROLE_AR, P]


ROW_FUSED = [(1, 2048, 2048, False), (1, 2048, 6144, False), (1, 2560, 9728, False), (1, 1024, 2560, False),
             (2, 4096, 2048, False), (2, 2048, 2048, False), (2, 6144, 2048, True), (2, 512, 2048, True)]


@pytest.mark.parametrize("src_mode,N,K,silu", ROW_FUSED)
def test_width1_row_fused_register_kernel_equals_staged_kernel(src_mode, N, K, silu):
    """bm_t2_gemv_row_fused picks the register-only kernel for layers of a few MB; BM_PDL_STAGED keeps it
    on the shared-memory-staged kernel.  Outputs, the stored residual row, the absmax words and the
    cleared word must be identical."""
    gen = torch.Generator().manual_seed(N + K + src_mode)
    rows = 2 * N if silu else N
    w, ws, _ = synthetic.ternary_weight(rows, K, gen)
    w, ws = w.to(DEV), ws.to(DEV)
    x = (torch.randn(1, K, generator=gen) * 1.3).to(torch.bfloat16).to(DEV)
    res = torch.randn(1, K, generator=gen).to(torch.bfloat16).to(DEV)
    norm_w = (1.0 + 0.1 * torch.randn(K, generator=gen)).to(torch.bfloat16).to(DEV)
    amax_in = x.float().abs().max().reshape(1).view(torch.int32).to(DEV)

    def run(pdl):
        out = torch.zeros(1, N, dtype=torch.bfloat16, device=DEV)
        h_out = torch.zeros(1, K, dtype=torch.bfloat16, device=DEV)
        amax_zero = torch.full((1,), 77, dtype=torch.int32, device=DEV)
        amax_out = torch.zeros(1, dtype=torch.int32, device=DEV)
        kw = dict(out=out, silu=silu, amax_out=amax_out if silu else None, pdl=pdl)
        if src_mode == 1:
            ops.gemv_row_fused(1, x, w, ws, amax_in=amax_in, amax_zero=amax_zero, **kw)
        else:
            ops.gemv_row_fused(2, x, w, ws, res=res, norm_w=norm_w, eps=1e-6, h_out=h_out, **kw)
        torch.cuda.synchronize()
        return out, h_out, amax_zero, amax_out

    a, b = run(0), run(native.PDL_STAGED)
    assert native.lib().bm_device_error() == 0
    for name, u, v in zip(("output", "residual row", "cleared word", "absmax word"), a, b):
        assert torch.equal(u.view(torch.int16) if u.dtype == torch.bfloat16 else u,
                           v.view(torch.int16) if v.dtype == torch.bfloat16 else v), name
    assert float(a[0].float().abs().sum()) > 0


@pytest.mark.parametrize("rows,vocab,ld", [(8, 151936, 151936), (9, 151669, 151936), (1, 1000, 1000), (17, 4099, 4100),
                                           (32, 300, 333)])
def test_split_logit_reductions_equal_the_single_cta_kernels(rows, vocab, ld):
    """bm_argmax_rows_split / bm_draft_chain_split (many CTAs per row: last-arriver combine, or one cluster per row) against
    bm_argmax_rows / bm_draft_chain: indices, confidences (bit for bit) and chain lengths, with ties in
    the rows, ragged vocabulary sizes and unaligned leading dimensions; three calls in a row on one scratch
    show that the ticket counters are left clean."""
    gen = torch.Generator().manual_seed(rows * 7 + vocab)
    base = torch.randn(rows, ld, generator=gen) * 3.0
    base[:, vocab:] = 1e9                                     # padding columns must never win
    if vocab > 600:
        base[0, 17] = base[0, 512] = base[0].max() + 1.0        # a tie across two ranges: lowest index wins
    lg = base.to(DEV)[:, :vocab]
    scratch = ops.logit_scratch(DEV)
    want_idx = ops.argmax_rows(lg)
    for _ in range(3):
        got_idx = ops.argmax_rows(lg, scratch=scratch)
        assert torch.equal(got_idx, want_idx)
    if vocab > 600:
        assert int(want_idx[0]) == 17
    for tau in (0.0, 1e-6, 0.5):
        idx0, n0, conf0 = ops.draft_chain(lg, tau)
        for _ in range(2):
            idx1, n1, conf1 = ops.draft_chain(lg, tau, scratch=scratch)
            assert torch.equal(idx1, idx0)
            assert torch.equal(conf1.view(torch.int32), conf0.view(torch.int32))
            assert int(n1) == int(n0)
    torch.cuda.synchronize()
    assert native.lib().bm_device_error() == 0
    assert int(scratch[: 4 * 65].view(torch.int32).abs().sum()) == 0


@pytest.mark.parametrize("M,D,n_commit,verified,cache_len", [(16, 8, 8, False, 300), (9, 8, 5, True, 41), (12, 8, 3, False, 7),
                                                              (9, 8, 1, False, 64), (5, 4, 1, True, 20), (17, 8, 9, False, 100)])
def test_commit_and_stage_draft_in_one_launch(M, D, n_commit, verified, cache_len):
    """bm_commit_stage_draft against the copies of a step's commit followed by bm_stage_replay_inputs kind 0."""
    MASK, P = 151654, M - D
    gen = torch.Generator().manual_seed(M * 13 + n_commit)
    src = torch.randint(0, 150000, (17,), generator=gen, dtype=torch.int64).to(DEV)
    n_pend = 1 if verified else n_commit
    # the plain sequence
    gen_a = torch.full((40,), -1, dtype=torch.int64, device=DEV)
    pend_a = torch.full((18,), -2, dtype=torch.int64, device=DEV)
    gen_a[5:5 + n_commit] = src[:n_commit]
    if verified:
        pend_a[0:1] = src[n_commit - 1:n_commit]
    else:
        pend_a[:n_commit] = src[:n_commit]
    tok_a, pos_a = torch.full((M,), -1, dtype=torch.int64, device=DEV), torch.full((M,), -1, dtype=torch.int64, device=DEV)
    st_a = ops.new_step_state(DEV)
    ops.stage_replay_inputs(0, pend_a, None, n_pend, cache_len, M, D, MASK, native.ROLE_DRAFT, P, tok_a, pos_a, st_a)
    # one launch
    gen_b = torch.full((40,), -1, dtype=torch.int64, device=DEV)
    pend_b = torch.full((18,), -2, dtype=torch.int64, device=DEV)
    tok_b, pos_b = torch.full((M,), -1, dtype=torch.int64, device=DEV), torch.full((M,), -1, dtype=torch.int64, device=DEV)
    st_b = ops.new_step_state(DEV)
    ops.commit_stage_draft(src, n_commit, verified, gen_b[5:], pend_b,
                           stage=(cache_len, M, D, MASK, native.ROLE_DRAFT, P, tok_b, pos_b, st_b))
    for name, a, b in (("output ids", gen_a, gen_b), ("pending ids", pend_a, pend_b), ("tokens", tok_a, tok_b),
                       ("positions", pos_a, pos_b), ("step record", st_a, st_b)):
        assert torch.equal(a, b), name
    # commit only
    gen_c = torch.full((40,), -1, dtype=torch.int64, device=DEV)
    pend_c = torch.full((18,), -2, dtype=torch.int64, device=DEV)
    ops.commit_stage_draft(src, n_commit, verified, gen_c[5:], pend_c)
    assert torch.equal(gen_c, gen_a) and torch.equal(pend_c, pend_a)
