"""Build recipe for the CPU oracle (test infrastructure, never imported by the package).

`python -m oracle.build` compiles oracle/bm_oracle.c into oracle/libbm_oracle.so.
The flags matter for parity:
  -ffp-contract=off   gcc must not fuse a*b+c on its own; every fused
                      multiply-add in the oracle is an explicit fmaf()
  -march=x86-64-v3    fmaf() becomes one vfmadd instruction (hardware FMA is
                      exact by definition, so the result does not depend on it,
                      only the speed does) and the int8 dot products vectorise
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "bm_oracle.c")
OUT = os.path.join(HERE, "libbm_oracle.so")
HDR = os.path.join(HERE, "..", "bitmtp_b200", "csrc", "bm_math.h")


def _stale() -> bool:
    if not os.path.exists(OUT):
        return True
    t = os.path.getmtime(OUT)
    return any(os.path.getmtime(p) > t for p in (SRC, HDR, __file__))


def build_oracle(force: bool = False, verbose: bool = False) -> str:
    """Compile the oracle if its sources are newer than the library; return the .so path."""
    if not force and not _stale():
        return OUT
    # The system gcc ships libgomp; a $CC wrapper may not, so it is not consulted.
    cc = "/usr/bin/gcc" if os.path.exists("/usr/bin/gcc") else "gcc"
    cmd = [
        cc, "-O3", "-std=gnu11", "-fopenmp", "-fPIC", "-shared",
        "-ffp-contract=off", "-fno-fast-math", "-march=x86-64-v3", "-fvisibility=hidden",
        "-Wall", "-Wno-unknown-pragmas", SRC, "-o", OUT + ".tmp", "-lm",
    ]
    if verbose:
        print(" ".join(cmd), file=sys.stderr)
    subprocess.run(cmd, check=True)
    os.replace(OUT + ".tmp", OUT)
    return OUT


# ----------------------------------------------------------------------------- the reference's own kernel
REF_DIR = os.path.join(HERE, "_ref")
REF_OUT = os.path.join(REF_DIR, "libbonsai_t2.so")
REF_SRC_REL = os.path.join("src", "bonsai_sft", "gpu", "t2g128_kernels", "t2g128_kernels.cu")


def build_reference_kernel(reference_root: str, force: bool = False, verbose: bool = False) -> str:
    """Compile the reference's CUDA GEMV (one source file, read where it lies in the reference
    checkout, never copied) into oracle/_ref/libbonsai_t2.so with the flags of its own
    compile.sh (-O3 -std=c++17 --use_fast_math -Xcompiler -fPIC -shared), targeting sm_100a,
    which that script does not list.  The GPU tests compare this library's GEMV outputs with it
    and the benchmark's reference arm times it; nothing else loads it.  Returns the path, or ""
    when the reference checkout or nvcc is absent (the prebuilt file, if any, stays in use)."""
    src = os.path.join(reference_root, REF_SRC_REL)
    nvcc = "/usr/local/cuda/bin/nvcc" if os.path.exists("/usr/local/cuda/bin/nvcc") else "nvcc"
    if not os.path.exists(src):
        return REF_OUT if os.path.exists(REF_OUT) else ""
    if not force and os.path.exists(REF_OUT) and os.path.getmtime(REF_OUT) >= os.path.getmtime(src):
        return REF_OUT
    os.makedirs(REF_DIR, exist_ok=True)
    cmd = [nvcc, "-O3", "-std=c++17", "--use_fast_math", "-Xcompiler", "-fPIC", "-shared",
           "-gencode", "arch=compute_100a,code=sm_100a", src, "-o", REF_OUT + ".tmp"]
    if verbose:
        print(" ".join(cmd), file=sys.stderr)
    subprocess.run(cmd, check=True)
    os.replace(REF_OUT + ".tmp", REF_OUT)
    return REF_OUT


REF_SITE = os.path.join(HERE, "..", "baseline", "_ref")


def install_reference_python(reference_root: str, force: bool = False) -> str:
    """Install the reference's Python package, unmodified, into the git-ignored baseline/_ref with pip
    (offline, no dependency resolution: its pins name older torch / transformers than this image has)
    and place the reference kernel built above where its ctypes loader looks for it
    (src/bonsai_sft/gpu/model.py:206-219).  Only the benchmark's reference arm imports from there
    (oracle/reference_decode.py, bench.py's reference_cpu_linear_path).  The source tree is read-only,
    so pip builds from a temporary copy.  Returns the site directory, or "" when nothing was installed."""
    import shutil
    import tempfile
    site = os.path.abspath(REF_SITE)
    pkg = os.path.join(site, "bonsai_sft")
    if not os.path.isdir(os.path.join(reference_root, "src", "bonsai_sft")):
        return site if os.path.isdir(pkg) else ""
    if force or not os.path.isdir(pkg):
        tmp = tempfile.mkdtemp(prefix="bitmtp_ref_")
        try:
            src = os.path.join(tmp, "reference")
            shutil.copytree(reference_root, src, symlinks=True)
            os.makedirs(site, exist_ok=True)
            subprocess.run([sys.executable, "-m", "pip", "install", "--quiet", "--no-index", "--no-build-isolation",
                            "--no-deps", "--upgrade", "--find-links", "/opt/wheelhouse", "--target", site, src],
                           check=True)
        finally:
            shutil.rmtree(tmp, ignore_errors=True)
    if os.path.exists(REF_OUT) and os.path.isdir(pkg):
        dst = os.path.join(pkg, "gpu", "t2g128_kernels", "libbonsai_t2.so")
        if not os.path.exists(dst) or os.path.getmtime(dst) < os.path.getmtime(REF_OUT):
            shutil.copyfile(REF_OUT, dst)
    return site if os.path.isdir(pkg) else ""


def reference_kernel_path() -> str:
    """Path of the built reference kernel library, "" if it has not been built."""
    return REF_OUT if os.path.exists(REF_OUT) else ""


if __name__ == "__main__":
    print(build_oracle(force="--force" in sys.argv, verbose=True))
    root = os.environ.get("BITMTP_REFERENCE", "")
    if root:
        print(build_reference_kernel(root, force="--force" in sys.argv, verbose=True) or "reference checkout not found")
        print(install_reference_python(root, force="--force" in sys.argv) or "reference package not installed")
