"""This library's GEMV against the reference's own CUDA kernel on the same device buffers.

The reference kernel (src/bonsai_sft/gpu/t2g128_kernels/t2g128_kernels.cu) is compiled from its
source by oracle/build.py into oracle/_ref/libbonsai_t2.so; the tests are skipped where that file
has not been built.  Both kernels round their fp32 result to bf16.  They differ in the fp32 order
(the reference multiplies 16-element partial dot products by the group scale in each of 8 lanes and
sums across lanes; this library scales exact int32 group sums) and in the final step (fast-math
division against a multiplication by 1/s), so a result that lies next to a bf16 rounding boundary
may land one bf16 step apart.  Tolerance: every element within one bf16 step (2^-7 relative) or
1e-5 of the row maximum; at least 99 % of the elements identical."""
import ctypes

import pytest
import torch

from bitmtp_b200 import model as BM, native, ops, synthetic
from oracle.build import reference_kernel_path

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

CASES = [(1, 1024, 2048), (8, 1024, 2048), (1, 2048, 2048), (9, 2048, 2048), (1, 4096, 2048), (16, 4096, 2048),
         (1, 6144, 2048), (4, 6144, 2048), (17, 6144, 2048), (1, 12288, 2048), (12, 12288, 2048),
         (1, 2048, 6144), (10, 2048, 6144), (16, 2048, 6144), (1, 151936, 2048), (8, 151936, 2048),
         (1, 6144, 2560), (16, 19456, 2560), (9, 2560, 4096), (1, 2560, 9728), (16, 2560, 9728)]


@pytest.fixture(scope="module")
def ref_lib():
    path = reference_kernel_path()
    if not path:
        pytest.skip("oracle/_ref/libbonsai_t2.so has not been built (python -m oracle.build with BITMTP_REFERENCE set)")
    lib = ctypes.CDLL(path)
    vp = ctypes.c_void_p
    lib.t2g128_int8xint2_linear.argtypes = [vp, vp, vp, vp, vp, ctypes.c_int, ctypes.c_int, ctypes.c_int, vp]
    lib.t2g128_int8xint2_linear.restype = None
    return lib


@pytest.mark.parametrize("W,N,K", CASES, ids=lambda v: str(v))
def test_gemv_agrees_with_reference_cuda_kernel(ref_lib, W, N, K):
    case = synthetic.gemv_case(W, N, K, seed=W + N % 97)
    A, B, ws, s = (case[k].to(DEV) for k in ("A", "B", "ws", "s"))
    ref = torch.full((W, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    ref_lib.t2g128_int8xint2_linear(A.data_ptr(), B.data_ptr(), ref.data_ptr(), s.data_ptr(), ws.data_ptr(), W, N, K,
                                    torch.cuda.current_stream().cuda_stream)
    ours = ops.t2_gemv(A, B, s, ws, out_kind=native.OUT_BF16)
    # the drop-in symbol of the same name, through the reference-facing wrapper
    shim = BM.t2g128_int8xint2_linear(A, B, s.view(W, 1), ws)
    torch.cuda.synchronize()
    assert native.lib().bm_device_error() == 0
    assert not torch.isnan(ref.float()).any(), "the reference kernel left outputs unwritten"
    assert torch.equal(ours.view(torch.int16), shim.view(torch.int16))
    r, o = ref.float(), ours.float()
    tol = torch.maximum(r.abs() * 2.0 ** -7, r.abs().amax(dim=1, keepdim=True) * 1e-5)
    bad = (o - r).abs() > tol
    assert not bad.any(), f"{int(bad.sum())} elements beyond one bf16 step, worst {float(((o - r).abs() / r.abs().clamp_min(1e-20)).max())}"
    same = (ours.view(torch.int16) == ref.view(torch.int16)).float().mean().item()
    assert same >= 0.99, f"only {same:.4f} of the elements are bit-identical"
