"""bitmtp_b200: B200 (sm_100a) implementation of BitMTP's packed T2-g128 decode path.

Module names mirror `bonsai_sft.gpu` of the reference so that its users find the
same entry points: `model` (packed linear operators and the captured forward),
`fast_runtime` (GraphAtlas), `fast_generate` (decode policies), `generate`
(build_model), `contracts`, `runtime_config`, `run_generation` and
`convert_bonsai_mtp_to_gpu` (CLIs).  Compute goes through `native` (ctypes over
libbitmtp_b200.so); nothing here falls back to PyTorch arithmetic.
"""
__version__ = "0.1.0"
