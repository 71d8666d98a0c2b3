"""bm_verify_attention_static: the attention entry point that allocates nothing.

Called through the C ABI with caller-owned inputs and outputs; its results must equal those
of bm_verify_attention (caller scratch) bit for bit, on two calls in a row that share the
library's built-in scratch array.  The file name sorts last so that the test also runs after
every other GPU test has used the device."""
import numpy as np
import pytest
import torch

from bitmtp_b200 import native, ops

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _bf16(gen, *shape, scale=1.0):
    return (torch.randn(*shape, generator=gen) * scale).to(torch.bfloat16)


def _p(t):
    return None if t is None else t.data_ptr()


def _case(seed, M, H, Hkv, sigma, cache_len, n_pend, role, D=8):
    gen = torch.Generator().manual_seed(seed)
    kv_rows = sigma + 17
    q = _bf16(gen, M, H, 128, scale=1.5).to(DEV)
    k = _bf16(gen, Hkv, kv_rows, 128, scale=1.5).to(DEV)
    v = _bf16(gen, Hkv, kv_rows, 128).to(DEV)
    state = ops.new_step_state(DEV)
    ops.set_step_state(state, cache_len, n_pend, role, M - D)
    return q, k, v, state, kv_rows


def _outputs(M, H):
    return (torch.zeros((M, H * 128), dtype=torch.bfloat16, device=DEV),
            torch.zeros((M, H * 128), dtype=torch.int8, device=DEV),
            torch.zeros((M, H * 128), dtype=torch.int8, device=DEV),
            torch.zeros((M, H * 128 // 128), dtype=torch.int32, device=DEV),
            torch.zeros((M, 1), dtype=torch.float32, device=DEV))


def _run_static(q, k, v, state, kv_rows, M, H, Hkv, sigma, outs):
    att, qq, qp, asum, s = outs
    stream = torch.cuda.current_stream().cuda_stream
    return native.lib().bm_verify_attention_static(
        _p(q), _p(k), _p(v), M, H, Hkv, kv_rows, sigma, _p(state), _p(att), _p(qq), _p(qp), _p(asum),
        _p(s), 0, stream)


def test_static_scratch_attention_matches_caller_scratch_twice():
    lib = native.lib()
    shapes = [(16, 16, 8, 1024, 700, 8, native.ROLE_DRAFT), (9, 16, 8, 256, 100, 0, native.ROLE_VERIFY)]
    for call, (M, H, Hkv, sigma, cache_len, n_pend, role) in enumerate(shapes):
        q, k, v, state, kv_rows = _case(100 + call, M, H, Hkv, sigma, cache_len, n_pend, role)
        want = _outputs(M, H)
        scratch = ops.attention_scratch(M, H, sigma, DEV)
        stream = torch.cuda.current_stream().cuda_stream
        rc = lib.bm_verify_attention(_p(q), _p(k), _p(v), M, H, Hkv, kv_rows, sigma, _p(state),
                                     _p(scratch), *[_p(t) for t in want], 0, stream)
        assert rc == 0
        got = _outputs(M, H)
        assert _run_static(q, k, v, state, kv_rows, M, H, Hkv, sigma, got) == 0
        torch.cuda.synchronize()
        for name, a, b in zip(("att", "codes", "prepared codes", "group sums", "multipliers"), got, want):
            assert torch.equal(a.view(torch.uint8), b.view(torch.uint8)), f"{name} differ on call {call}"
        assert float(want[0].float().abs().sum()) > 0.0
    assert lib.bm_device_error() == 0


def test_static_scratch_back_to_back_overlapped_calls():
    """Two calls on one stream with programmatic overlap and no synchronisation in between: the second
    call's CTAs may start while the first call's last CTAs still merge out of the shared array.  Every
    write to the array comes after the kernel's wait for its predecessor, so both results must still
    equal the caller-scratch results."""
    lib = native.lib()
    pdl = native.PDL_OVERLAP | native.PDL_STABLE_STATE
    shapes = [(16, 16, 8, 1024, 700, 8, native.ROLE_DRAFT), (9, 32, 8, 256, 100, 0, native.ROLE_VERIFY)]
    cases, wants, gots = [], [], []
    for call, (M, H, Hkv, sigma, cache_len, n_pend, role) in enumerate(shapes):
        q, k, v, state, kv_rows = _case(200 + call, M, H, Hkv, sigma, cache_len, n_pend, role)
        want = _outputs(M, H)
        scratch = ops.attention_scratch(M, H, sigma, DEV)
        stream = torch.cuda.current_stream().cuda_stream
        assert lib.bm_verify_attention(_p(q), _p(k), _p(v), M, H, Hkv, kv_rows, sigma, _p(state), _p(scratch),
                                       *[_p(t) for t in want], 0, stream) == 0
        cases.append((q, k, v, state, kv_rows, M, H, Hkv, sigma))
        wants.append(want)
        gots.append(_outputs(M, H))
    torch.cuda.synchronize()
    stream = torch.cuda.current_stream().cuda_stream
    for (q, k, v, state, kv_rows, M, H, Hkv, sigma), got in zip(cases, gots):
        att, qq, qp, asum, s = got
        assert lib.bm_verify_attention_static(_p(q), _p(k), _p(v), M, H, Hkv, kv_rows, sigma, _p(state), _p(att),
                                              _p(qq), _p(qp), _p(asum), _p(s), pdl, stream) == 0
    torch.cuda.synchronize()
    for call, (got, want) in enumerate(zip(gots, wants)):
        for name, a, b in zip(("att", "codes", "prepared codes", "group sums", "multipliers"), got, want):
            assert torch.equal(a.view(torch.uint8), b.view(torch.uint8)), f"{name} differ on call {call}"
    assert lib.bm_device_error() == 0


def test_static_scratch_attention_rejects_oversize():
    lib = native.lib()
    # the limit, from host-only arithmetic: 16 rows x 16 heads fit up to sigma = 7808
    assert lib.bm_verify_attention_scratch_bytes(16, 16, 7808) <= native.STATIC_ATTN_SCRATCH_BYTES
    assert lib.bm_verify_attention_scratch_bytes(16, 16, 7809) > native.STATIC_ATTN_SCRATCH_BYTES
    M, H, Hkv, sigma = 32, 32, 8, 4096
    assert lib.bm_verify_attention_scratch_bytes(M, H, sigma) > native.STATIC_ATTN_SCRATCH_BYTES
    q, k, v, state, kv_rows = _case(7, M, H, Hkv, 64, 10, 0, native.ROLE_DRAFT, D=24)
    outs = _outputs(M, H)
    # the size check comes before anything is launched, so the small buffers are never read
    rc = _run_static(q, k, v, state, sigma + 17, M, H, Hkv, sigma, outs)
    assert rc == native.BM_ETOOBIG
    q16, k16, v16, state16, _ = _case(8, 16, 16, 8, 64, 10, 0, native.ROLE_DRAFT)
    outs16 = _outputs(16, 16)
    assert _run_static(q16, k16, v16, state16, 7809 + 17, 16, 16, 8, 7809, outs16) == native.BM_ETOOBIG
    torch.cuda.synchronize()
    assert float(outs[0].float().abs().sum()) == 0.0 and float(outs16[0].float().abs().sum()) == 0.0
