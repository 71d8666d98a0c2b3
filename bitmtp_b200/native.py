"""Loader and build recipe for libbitmtp_b200.so (the hand-written sm_100a kernels).

The library is built in-tree (`python -m bitmtp_b200.native` or
`__graft_entry__.build()`) and loaded with ctypes, as the reference loads
`libbonsai_t2.so` (src/bonsai_sft/gpu/model.py:206-219).  There is no CPU or
PyTorch fallback: if the library is missing, or a call returns a non-zero
status, the caller gets an exception.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
SO_PATH = os.path.join(HERE, "libbitmtp_b200.so")
SOURCES = ["bm_lib.cu"]
HEADERS = ["bm_math.h", "bm_common.cuh", "t2_gemv.cuh", "fused_ops.cuh", "verify_attn.cuh", "t2_gemv_rowwarp.cuh",
           "t2_gemv_direct.cuh", "dense_head.cuh", "t2_gemm_wide.cuh"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    # No implicit multiply-add fusion and no fast-math: the kernels share
    # bm_math.h with the CPU oracle and must round exactly as it does.
    "-fmad=false", "-Xcompiler", "-fPIC", "-shared",
]

BM_OK = 0
BM_EINVAL = 22
BM_ETOOBIG = 27
BM_ECAPTURE = 16
STATIC_ATTN_SCRATCH_BYTES = 8 << 20     # BM_STATIC_ATTN_SCRATCH_BYTES of the header
OUT_BF16, OUT_F32, OUT_F32_OF_BF16 = 0, 1, 2
PATH_AUTO, PATH_DP4A, PATH_MMA, PATH_ROWWARP, PATH_DIRECT = 0, 1, 2, 3, 4
ROLE_DRAFT, ROLE_VERIFY, ROLE_AR = 0, 1, 2
PDL_OVERLAP, PDL_STABLE_STATE, PDL_STAGED = 1, 2, 4

_lib = None


def _stale() -> bool:
    if not os.path.exists(SO_PATH):
        return True
    t = os.path.getmtime(SO_PATH)
    deps = [os.path.join(CSRC, f) for f in SOURCES + HEADERS]
    deps.append(os.path.join(HERE, "..", "include", "bitmtp_b200.h"))
    return any(os.path.exists(p) and os.path.getmtime(p) > t for p in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile the CUDA library for sm_100a if sources are newer than the .so."""
    if not force and not _stale():
        return SO_PATH
    nvcc = os.environ.get("NVCC", "nvcc")
    cmd = [nvcc] + NVCC_FLAGS + [os.path.join(CSRC, s) for s in SOURCES] + ["-o", SO_PATH + ".tmp"]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
        print(" ".join(cmd), file=sys.stderr)
    subprocess.run(cmd, check=True)
    os.replace(SO_PATH + ".tmp", SO_PATH)
    return SO_PATH


class NativeError(RuntimeError):
    pass


def lib() -> ctypes.CDLL:
    """The loaded library.  Raises if it has not been built: there is no fallback."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(SO_PATH):
        raise NativeError(
            f"{SO_PATH} is missing: build it with `python -m bitmtp_b200.native` "
            "(nvcc, sm_100a). bitmtp_b200 has no CPU or PyTorch fallback.")
    L = ctypes.CDLL(SO_PATH)
    vp, ci = ctypes.c_void_p, ctypes.c_int
    L.bm_version.restype = ctypes.c_char_p
    L.bm_sm_count.restype = ci
    L.bm_device_error.restype = ci
    L.bm_launch_count.restype = ctypes.c_ulonglong
    L.bm_t2_gemv.argtypes = [vp, vp, vp, vp, vp, ci, ci, ci, ci, ci, ci, vp, ci, vp]
    L.bm_t2_gemv.restype = ci
    L.bm_t2_gemv_bytes.argtypes = [ci, ci, ci, ci]
    L.bm_t2_gemv_bytes.restype = ctypes.c_int64
    L.t2g128_int8xint2_linear.argtypes = [vp, vp, vp, vp, vp, ci, ci, ci, vp]
    L.t2g128_int8xint2_linear.restype = None
    _declare_optional(L)
    _lib = L
    return L


def _declare_optional(L) -> None:
    """Prototypes of the fused operators, the attention and the logit reductions."""
    vp, ci, cf = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    protos = {
        "bm_quant_rows": [vp, ci, ci, vp, vp, vp, vp, ci, vp],
        "bm_rmsnorm_fused": [vp, vp, ci, vp, vp, cf, ci, ci, ci, vp, vp, vp, vp, vp, vp, ci, vp],
        "bm_silu_mul_quant": [vp, ci, ci, vp, vp, vp, vp, vp, ci, vp],
        "bm_qknorm_rope_kvappend": [vp, vp, vp, cf, vp, vp, vp, ci, ci, ci, vp, vp, ci, ci, vp, ci, vp],
        "bm_set_step_state": [vp, ci, ci, ci, ci, vp],
        "bm_kv_copy_rows": [vp, ci, ci, ci, ci, ci, vp],
        "bm_verify_attention_scratch_bytes": [ci, ci, ci],
        "bm_verify_attention": [vp, vp, vp, ci, ci, ci, ci, ci, vp, vp, vp, vp, vp, vp, vp, ci, vp],
        "bm_verify_attention_static": [vp, vp, vp, ci, ci, ci, ci, ci, vp, vp, vp, vp, vp, vp, ci, vp],
        "bm_zero_words": [vp, ci, vp],
        "bm_t2_gemv_row_fused": [ci, vp, vp, ci, vp, vp, cf, vp, vp, vp, vp, vp, ci, ci, vp, ci, ci, ci, vp, ci, vp],
        "bm_stage_replay_inputs": [ci, vp, vp, ci, ci, ci, ci, ctypes.c_longlong, ci, ci, vp, vp, vp, vp],
        "bm_rope_verify_attention_rows": [vp, vp, vp, cf, vp, vp, vp, vp, vp, ci, ci, ci, ci, ci, vp, vp, vp, vp, ci, vp],
        "bm_rope_verify_attention": [vp, vp, vp, cf, vp, vp, vp, vp, vp, ci, ci, ci, ci, ci, vp, vp, vp, vp, vp, vp, vp,
                                     ci, vp],
        "bm_t2_gemv_gate_up_silu": [vp, vp, vp, vp, vp, ci, ci, ci, vp, vp, ci, vp],
        "bm_quant_rows_amax": [vp, vp, vp, ci, ci, vp, vp, vp, vp, ci, vp],
        "bm_t2_gemv_nsplit": [vp, vp, vp, vp, ci, ci, ci, ci, ci, ci, ci, ctypes.POINTER(vp), ctypes.POINTER(vp),
                              ctypes.POINTER(vp), vp, ci, ci, vp],
        "bm_t2_gemv_prepared": [vp, vp, vp, vp, vp, vp, ci, ci, ci, ci, ci, ci, vp],
        "bm_dense_head": [vp, vp, ci, vp, ci, ci, ci, vp, ci, vp, ci, vp],
        "bm_t2_gemm_wide": [vp, vp, vp, vp, vp, vp, ci, ci, ci, ci, ci, vp],
        "bm_pack_t2_g128": [vp, ci, ci, vp, vp, vp, vp],
        "bm_prompt_attention_scratch_bytes": [ci, ci, ci, ci, ci],
        "bm_prompt_attention": [vp, vp, vp, ci, ci, ci, ci, ci, ci, vp, vp, vp, ci, vp],
        "bm_argmax_rows": [vp, ci, ci, ci, vp, vp, vp],
        "bm_draft_chain": [vp, ci, ci, ci, cf, vp, vp, vp, vp, vp],
        "bm_verify_accept": [vp, vp, ci, vp, vp],
        "bm_argmax_rows_split": [vp, ci, ci, ci, vp, vp, vp, vp],
        "bm_draft_chain_split": [vp, ci, ci, ci, cf, vp, vp, vp, vp, vp, vp],
        "bm_logit_scratch_bytes": [],
        "bm_commit_stage_draft": [vp, ci, ci, vp, vp, ci, ci, ci, ci, ctypes.c_longlong, ci, ci, vp, vp, vp, vp],
    }
    for name, args in protos.items():
        fn = getattr(L, name)
        fn.argtypes = args
        fn.restype = ctypes.c_int64 if name.endswith("_bytes") else ci


def check(status: int, what: str) -> None:
    if status != BM_OK:
        detail = "invalid shape or alignment" if status == BM_EINVAL else f"status {status}"
        if status >= 1000:
            detail = f"CUDA error {status - 1000}"
        raise NativeError(f"{what} failed: {detail}")


def exported_symbols():
    """Names declared in include/bitmtp_b200.h (parsed from the header text)."""
    import re
    hdr = os.path.join(HERE, "..", "include", "bitmtp_b200.h")
    text = open(hdr).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = re.findall(r"\b(bm_[a-z0-9_]+|t2g128_int8xint2_linear)\s*\(", text)
    return sorted(set(names))


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
