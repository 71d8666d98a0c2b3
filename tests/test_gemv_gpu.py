"""GPU parity of the T2-g128 GEMV against the CPU oracle, through the C ABI.

Bar: int32 group sums bit-exact; fp32 outputs bit-exact against the oracle's
fixed summation order (which implies the 1e-3 relative bound the spec asks
for, checked separately against an fp64 evaluation); bf16 outputs bit-exact.
"""
import numpy as np
import pytest
import torch

from bitmtp_b200 import native, ops, synthetic

pytestmark = pytest.mark.gpu

REL_TOL = 1e-3   # max |y - y64| / max |y64| demanded of the scaled fp32 output


def _run(case, path, out_kind, want_groups=True):
    dev = torch.device("cuda:0")
    A, B, ws, s = (case[k].to(dev) for k in ("A", "B", "ws", "s"))
    out = ops.t2_gemv(A, B, s, ws, out_kind=out_kind, path=path, want_groups=want_groups)
    torch.cuda.synchronize()
    assert native.lib().bm_device_error() == 0
    return out


def _oracle(O, case):
    return O.t2_gemv(case["A"].numpy(), case["B"].numpy().view(np.uint8),
                     O.torch_to_u16(case["ws"]), case["s"].numpy(), want_groups=True)


def _check(O, case, path):
    y32, y16, G = _oracle(O, case)
    out, Gd = _run(case, path, native.OUT_F32)
    assert np.array_equal(Gd.cpu().numpy(), G), "int32 group sums differ"
    got = out.cpu().numpy()
    assert np.array_equal(got.view(np.uint32), y32.view(np.uint32)), "fp32 output not bit-exact"
    # fp64 evaluation of the same sums: the spec's 1e-3 bound
    sc = O.bf16_to_f32(O.torch_to_u16(case["ws"])).astype(np.float64)
    y64 = (G.astype(np.float64) * sc[None]).sum(-1) / case["s"].numpy().astype(np.float64)[:, None]
    assert np.abs(got - y64).max() / np.abs(y64).max() <= REL_TOL
    outb = _run(case, path, native.OUT_BF16, want_groups=False)
    assert np.array_equal(O.torch_to_u16(outb.cpu()), y16), "bf16 output not bit-exact"


SMALL = [(1, 8, 128), (2, 16, 256), (3, 24, 128), (4, 64, 384), (5, 40, 2048), (8, 72, 2560),
         (9, 64, 2048), (16, 128, 4096), (17, 32, 256), (12, 200, 1024), (10, 8, 6144)]


@pytest.mark.parametrize("W,N,K", SMALL)
@pytest.mark.parametrize("path", [native.PATH_DP4A, native.PATH_MMA])
def test_small_shapes_both_consumers(oracle, W, N, K, path):
    case = synthetic.gemv_case(W, N, K, seed=W * 1000 + N + K)
    if path == native.PATH_MMA and K % 256 != 0:
        # the MMA consumer needs an even number of groups; the ABI says so with EINVAL
        dev = torch.device("cuda:0")
        A, B, ws, s = (case[k].to(dev) for k in ("A", "B", "ws", "s"))
        with pytest.raises(native.NativeError):
            ops.t2_gemv(A, B, s, ws, path=path)
        return
    _check(oracle, case, path)


LAYER_NK = [(2048, 2048), (1024, 2048), (4096, 2048), (6144, 2048), (2048, 6144), (12288, 2048),
            (6144, 2560), (2560, 4096), (19456, 2560), (2560, 9728)]


@pytest.mark.parametrize("N,K", LAYER_NK)
@pytest.mark.parametrize("W", [1, 2, 4, 8, 9, 16])
def test_layer_shapes_auto_path(oracle, N, K, W):
    _check(oracle, synthetic.gemv_case(W, N, K, seed=0), native.PATH_AUTO)


def test_config0_reference_case(oracle):
    """K=2048, N=6144, W=1, seed 0: the single-GEMV configuration of the baseline."""
    case = synthetic.gemv_case(1, 6144, 2048, seed=0)
    for path in (native.PATH_DP4A, native.PATH_MMA):
        _check(oracle, case, path)


@pytest.mark.parametrize("N,K,W", [(12288, 2048, 16), (12288, 2048, 3), (151936, 2048, 16),
                                   (28672, 8192, 16), (19456, 2560, 9), (2560, 9728, 16)])
def test_large_tiles_without_group_output(oracle, N, K, W):
    """The production instantiations (16- and 32-row tiles) are only reached when no group
    sums are requested; check their scaled outputs bit for bit."""
    case = synthetic.gemv_case(W, N, K, seed=21)
    y32, y16, _ = oracle.t2_gemv(case["A"].numpy(), case["B"].numpy().view(np.uint8),
                                 oracle.torch_to_u16(case["ws"]), case["s"].numpy())
    dev = torch.device("cuda:0")
    A, B, ws, s = (case[k].to(dev) for k in ("A", "B", "ws", "s"))
    out = ops.t2_gemv(A, B, s, ws, out_kind=native.OUT_F32)
    assert np.array_equal(out.cpu().numpy().view(np.uint32), y32.view(np.uint32))
    outb = ops.t2_gemv(A, B, s, ws)
    assert np.array_equal(oracle.torch_to_u16(outb.cpu()), y16)
    assert native.lib().bm_device_error() == 0


@pytest.mark.parametrize("W", [1, 10, 12, 17])
def test_head_shape(oracle, W):
    _check(oracle, synthetic.gemv_case(W, 151936, 2048, seed=3), native.PATH_AUTO)


@pytest.mark.parametrize("W", [1, 8])
def test_wide_stress_shape(oracle, W):
    _check(oracle, synthetic.gemv_case(W, 28672, 8192, seed=4), native.PATH_AUTO)


def test_row_independent_of_width():
    """A token's output row is bit-identical at every width and on both consumers."""
    dev = torch.device("cuda:0")
    case = synthetic.gemv_case(17, 4096, 2048, seed=7)
    A, B, ws, s = (case[k].to(dev) for k in ("A", "B", "ws", "s"))
    full = ops.t2_gemv(A, B, s, ws, out_kind=native.OUT_F32, path=native.PATH_MMA)
    for W in (1, 2, 4, 9, 16):
        for path in (native.PATH_DP4A, native.PATH_MMA):
            part = ops.t2_gemv(A[:W].contiguous(), B, s[:W].contiguous(), ws,
                               out_kind=native.OUT_F32, path=path)
            assert torch.equal(part, full[:W])


def test_legacy_symbol_and_logit_kind(oracle):
    """The reference's own C symbol (bf16 out) and the fp32-of-bf16 logit store."""
    import ctypes
    dev = torch.device("cuda:0")
    case = synthetic.gemv_case(9, 4096, 2048, seed=11)
    A, B, ws, s = (case[k].to(dev) for k in ("A", "B", "ws", "s"))
    out = torch.empty(9, 4096, dtype=torch.bfloat16, device=dev)
    native.lib().t2g128_int8xint2_linear(A.data_ptr(), B.data_ptr(), out.data_ptr(), s.data_ptr(),
                                         ws.data_ptr(), 9, 4096, 2048,
                                         ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    _, y16, _ = _oracle(oracle, case)
    assert np.array_equal(oracle.torch_to_u16(out.cpu()), y16)
    lg = ops.t2_gemv(A, B, s, ws, out_kind=native.OUT_F32_OF_BF16)
    assert np.array_equal(lg.cpu().numpy(), oracle.bf16_to_f32(y16))


def test_rejects_bad_shapes():
    dev = torch.device("cuda:0")
    case = synthetic.gemv_case(1, 16, 128, seed=1)
    A, B, ws, s = (case[k].to(dev) for k in ("A", "B", "ws", "s"))
    L = native.lib()
    st = torch.cuda.current_stream().cuda_stream
    out = torch.empty(1, 16, dtype=torch.bfloat16, device=dev)
    args = lambda W, N, K: (A.data_ptr(), B.data_ptr(), out.data_ptr(), s.data_ptr(), ws.data_ptr(),
                            W, N, K, N, 0, 0, None, 0, st)
    assert L.bm_t2_gemv(*args(1, 12, 128)) == native.BM_EINVAL     # N not a multiple of 8
    assert L.bm_t2_gemv(*args(1, 16, 192)) == native.BM_EINVAL     # K not a multiple of 128
    assert L.bm_t2_gemv(*args(0, 16, 128)) == native.BM_EINVAL
    assert L.bm_t2_gemv(*args(33, 16, 128)) == native.BM_EINVAL


def test_linearity_property_full_size():
    """Size-independent property at the head size: G(a1 + a2) = G(a1) + G(a2) exactly,
    checked through fp32 outputs with unit scales-free comparison of group sums."""
    dev = torch.device("cuda:0")
    case = synthetic.gemv_case(2, 151936, 2048, seed=5)
    B, ws = case["B"].to(dev), case["ws"].to(dev)
    a1 = torch.randint(-60, 61, (1, 2048), dtype=torch.int8, device=dev)
    a2 = torch.randint(-60, 61, (1, 2048), dtype=torch.int8, device=dev)
    one = torch.ones(1, device=dev)
    _, g1 = ops.t2_gemv(a1, B, one, ws, want_groups=True)
    _, g2 = ops.t2_gemv(a2, B, one, ws, want_groups=True)
    _, g12 = ops.t2_gemv((a1 + a2).contiguous(), B, one, ws, want_groups=True)
    assert torch.equal(g12, g1 + g2)


ROWWARP = [(1, 16, 512), (2, 64, 512), (3, 48, 1024), (8, 2048, 2048), (5, 2048, 6144), (4, 6144, 2560),
           (8, 2560, 9728), (7, 12288, 2048), (1, 151936, 2048), (8, 28672, 8192), (6, 4096, 4096),
           # shards of the 8192 -> 28672 layer split over 2, 4 and 8 GPUs: two and four warps share a 16-row block
           (1, 14336, 8192), (8, 7168, 8192), (1, 3584, 8192), (8, 3584, 8192)]


@pytest.mark.parametrize("W,N,K", ROWWARP)
def test_row_per_warp_consumer(oracle, W, N, K):
    """The W <= 8 streaming kernel (a warp per 16-row block, tiled TMA panels), forced at
    every size: group sums, fp32 and bf16 outputs bit for bit."""
    _check(oracle, synthetic.gemv_case(W, N, K, seed=W * 77 + N + K), native.PATH_ROWWARP)


DIRECT = [(1, 8, 128), (2, 16, 384), (3, 24, 2048), (4, 64, 2560), (1, 1024, 2048), (1, 2048, 2048),
          (2, 4096, 2048), (4, 6144, 2048), (1, 2048, 6144), (3, 2560, 9728), (1, 12288, 2048), (4, 2048, 10240),
          (1, 6144, 2560), (2, 104, 8192)]


@pytest.mark.parametrize("W,N,K", DIRECT)
def test_direct_consumer(oracle, W, N, K):
    """The W <= 4 kernel that works from registers (a warp per row, one memory round trip), forced at
    every size incl. a single CTA, ragged last CTAs and K that is not a multiple of 2048: group sums,
    fp32 and bf16 outputs bit for bit."""
    _check(oracle, synthetic.gemv_case(W, N, K, seed=W * 131 + N + K), native.PATH_DIRECT)


@pytest.mark.parametrize("W,N,K", [(1, 2048, 2048), (4, 1024, 2560), (2, 2048, 6144)])
def test_direct_consumer_on_prepared_activations(oracle, W, N, K):
    """GEMV-ready activations (4x4-transposed 16-runs + group sums) through the automatic choice,
    which is the direct kernel at these sizes."""
    dev = torch.device("cuda:0")
    case = synthetic.gemv_case(W, N, K, seed=W + N + K)
    y32, _, _ = oracle.t2_gemv(case["A"].numpy(), case["B"].numpy().view(np.uint8),
                               oracle.torch_to_u16(case["ws"]), case["s"].numpy())
    A = case["A"].to(dev)
    prep = A.view(W, -1, 4, 4).transpose(2, 3).contiguous().view(W, -1)
    asum = A.view(W, -1, 128).to(torch.int32).sum(-1).to(torch.int32).contiguous()
    out = torch.empty(W, N, dtype=torch.float32, device=dev)
    ops.t2_gemv_prepared(prep, asum, case["B"].to(dev), case["s"].to(dev), case["ws"].to(dev), out=out,
                         out_kind=native.OUT_F32)
    torch.cuda.synchronize()
    assert native.lib().bm_device_error() == 0
    assert np.array_equal(out.cpu().numpy().view(np.uint32), y32.view(np.uint32))


def test_direct_rejects_what_it_cannot_serve():
    dev = torch.device("cuda:0")
    for (W, N, K) in [(5, 64, 512), (1, 64, 12288)]:
        case = synthetic.gemv_case(W, N, K, seed=1)
        A, B, ws, s = (case[k].to(dev) for k in ("A", "B", "ws", "s"))
        with pytest.raises(native.NativeError):
            ops.t2_gemv(A, B, s, ws, path=native.PATH_DIRECT)


def test_row_per_warp_rejects_what_it_cannot_serve():
    dev = torch.device("cuda:0")
    for (W, N, K) in [(9, 64, 512), (2, 24, 512), (2, 64, 256)]:
        case = synthetic.gemv_case(W, N, K, seed=1)
        A, B, ws, s = (case[k].to(dev) for k in ("A", "B", "ws", "s"))
        with pytest.raises(native.NativeError):
            ops.t2_gemv(A, B, s, ws, path=native.PATH_ROWWARP)


def test_prepared_activations_on_the_head_shape(oracle):
    """GEMV-ready activations through the automatic choice, which is the row-per-warp kernel
    for the 151936-row head at W <= 8 and the cooperative tiles at W = 16."""
    dev = torch.device("cuda:0")
    for W in (1, 8, 16):
        case = synthetic.gemv_case(W, 151936, 2048, seed=50 + W)
        y32, _, _ = oracle.t2_gemv(case["A"].numpy(), case["B"].numpy().view(np.uint8),
                                   oracle.torch_to_u16(case["ws"]), case["s"].numpy())
        A = case["A"].to(dev)
        # GEMV-ready form of the same codes: 4x4 byte transpose per 16-run + group sums
        prep = A.view(W, -1, 4, 4).transpose(2, 3).contiguous().view(W, -1)
        asum = A.view(W, -1, 128).to(torch.int32).sum(-1).to(torch.int32).contiguous()
        out = torch.empty(W, 151936, dtype=torch.float32, device=dev)
        ops.t2_gemv_prepared(prep, asum, case["B"].to(dev), case["s"].to(dev), case["ws"].to(dev), out=out,
                             out_kind=native.OUT_F32)
        assert np.array_equal(out.cpu().numpy().view(np.uint32), y32.view(np.uint32))
    assert native.lib().bm_device_error() == 0


def test_launch_counter_counts_this_librarys_launches():
    """bm_launch_count: +1 per GEMV call, +2 for the many-CTA confidence chain (argmax + confidence)."""
    dev = torch.device("cuda:0")
    lib = native.lib()
    case = synthetic.gemv_case(1, 64, 256, seed=3)
    A, B, ws, s = (case[k].to(dev) for k in ("A", "B", "ws", "s"))
    before = lib.bm_launch_count()
    ops.t2_gemv(A, B, s, ws)
    assert lib.bm_launch_count() - before == 1
    logits = torch.randn(8, 1000, device=dev)
    scratch = ops.logit_scratch(dev)
    before = lib.bm_launch_count()
    ops.draft_chain(logits, 0.5, scratch=scratch)
    assert lib.bm_launch_count() - before in (1, 2)       # one cluster launch, or argmax + confidence where clusters do not fit
    torch.cuda.synchronize()


@pytest.mark.parametrize("T", [1, 31, 32, 33, 100, 256])
@pytest.mark.parametrize("N,K", [(128, 256), (256, 512), (4096, 2048), (2048, 6144), (6144, 2560), (2560, 9728),
                                 (2048, 4096)])
def test_many_row_product_equals_the_gemv_row_for_row(T, N, K):
    """bm_t2_gemm_wide against the decode GEMV on the same GEMV-ready rows, 16 rows at a time: every bf16
    output bit for bit.  The GEMV itself is compared with the oracle above, so this pins the prompt GEMM to the
    oracle at every prompt length incl. ragged last tiles, K with 2 to 76 groups (slots with zero, one and
    several groups) and the 4B shapes."""
    if N * K > 2048 * 6144 and T not in (33, 256):
        pytest.skip("large shapes at two prompt lengths")
    dev = torch.device("cuda:0")
    gen = torch.Generator(device=dev).manual_seed(N + K + T)
    B, ws = synthetic.device_ternary(N, K, gen, dev)
    x = (torch.randn(T, K, device=dev, generator=gen) * 1.3).to(torch.bfloat16)
    qp, asum, s = ops.quant_rows(x, prepared=True)
    want = torch.empty(T, N, dtype=torch.bfloat16, device=dev)
    for r0 in range(0, T, 16):
        r1 = min(T, r0 + 16)
        ops.t2_gemv_prepared(qp[r0:r1], asum[r0:r1], B, s[r0:r1], ws, out=want[r0:r1])
    got = torch.full((T + 1, N + 128), 7.0, dtype=torch.bfloat16, device=dev)           # guard row and columns
    ops.t2_gemm_wide(qp, asum, B, s, ws, out=got[:T, :N])
    torch.cuda.synchronize()
    assert native.lib().bm_device_error() == 0
    assert torch.equal(got[:T, :N].view(torch.int16), want.view(torch.int16))
    assert bool((got[T] == 7.0).all()) and bool((got[:, N:] == 7.0).all()), "wrote outside the output"
