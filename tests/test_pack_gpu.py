"""Device freeze + pack (bm_pack_t2_g128) against the converter's CPU expressions: same packed bytes, same
bf16 scales, same frozen grid, on latent weights, on weights that are already on the grid, and on the
degenerate groups (all zero, one outlier, exact half-way ratios).  Then a whole checkpoint converted with
`--device cuda:0` against the CPU conversion of the same source."""
import pytest
import torch

from bitmtp_b200 import convert_bonsai_mtp_to_gpu as CV, native, ops
from bitmtp_b200.synthetic import pack_t2_g128

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _cpu(w):
    frozen = CV.freeze_ternary_g128(w)
    return (frozen,) + tuple(pack_t2_g128(frozen))


def _same(w):
    frozen, codes, scale = _cpu(w)
    g_codes, g_scale, g_frozen = ops.pack_t2_g128(w.to(DEV), want_frozen=True)
    torch.cuda.synchronize()
    assert torch.equal(g_codes.cpu(), codes)
    assert torch.equal(g_scale.cpu().view(torch.int16), scale.view(torch.int16))
    assert torch.equal(g_frozen.cpu().view(torch.int16), frozen.view(torch.int16))
    two = ops.pack_t2_g128(w.to(DEV))
    assert len(two) == 2 and torch.equal(two[0].cpu(), codes)
    assert native.lib().bm_device_error() == 0


@pytest.mark.parametrize("N,K", [(1, 128), (7, 384), (2048, 2048), (6144, 2048), (2048, 6144), (5008, 2560)])
def test_latent_weights(N, K):
    gen = torch.Generator().manual_seed(N * 31 + K)
    _same((torch.randn(N, K, generator=gen) * 0.02).to(torch.bfloat16))


def test_frozen_weights_are_a_fixed_point():
    gen = torch.Generator().manual_seed(5)
    w = (torch.randn(512, 1024, generator=gen) * 0.05).to(torch.bfloat16)
    frozen = CV.freeze_ternary_g128(w)
    _same(frozen)
    codes, scale, again = ops.pack_t2_g128(frozen.to(DEV), want_frozen=True)
    assert torch.equal(again.cpu().view(torch.int16), frozen.view(torch.int16))


def test_degenerate_groups():
    gen = torch.Generator().manual_seed(9)
    w = (torch.randn(64, 512, generator=gen) * 0.3).to(torch.bfloat16)
    w[0] = 0                                         # all-zero groups: scale 0, every code 2
    w[1, :128] = 0
    w[1, 5] = 3.0                                    # one outlier, everything else rounds to zero
    w[2, :128] = 0.5
    w[2, 0] = 1.0                                    # ratios of exactly one half: round half to even -> 0
    w[3, :128] = -1.5
    w[3, 7] = 1.0                                    # the absmax element is negative
    w[4, 128:256] = 1e-30                            # below the 1e-8 floor of the freeze scale
    w[5, :128] = float(torch.finfo(torch.bfloat16).max)
    _same(w)
    codes, scale, _ = ops.pack_t2_g128(w.to(DEV), want_frozen=True)
    assert int(codes[0].view(torch.uint8).min()) == 0xAA == int(codes[0].view(torch.uint8).max())
    assert float(scale[0].abs().max()) == 0.0


def test_rejects_what_the_packer_cannot_take():
    w = torch.zeros(4, 128, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(RuntimeError):
        ops.pack_t2_g128(w.float())
    with pytest.raises(RuntimeError):
        ops.pack_t2_g128(torch.zeros(4, 192, dtype=torch.bfloat16, device=DEV))
    with pytest.raises(RuntimeError):
        ops.pack_t2_g128(torch.zeros(4, 128, dtype=torch.bfloat16))


def test_whole_checkpoint_converted_on_the_device(tmp_path):
    from .test_boundary_cpu import tiny_hf_checkpoint
    src = tiny_hf_checkpoint(tmp_path)
    CV.convert(str(src), str(tmp_path / "cpu"))
    CV.convert(str(src), str(tmp_path / "gpu"), device=DEV, safetensors_copy=True)
    for name in ("model_state_t2g128.pt", "model_state_fp16.pt"):
        a, b = torch.load(tmp_path / "cpu" / name), torch.load(tmp_path / "gpu" / name)
        assert sorted(a) == sorted(b)
        for k in a:
            assert a[k].dtype == b[k].dtype and torch.equal(a[k], b[k]), (name, k)
    from bitmtp_b200 import generate
    st = generate.load_packed_state(str(tmp_path / "gpu"), DEV)
    ref = torch.load(tmp_path / "cpu" / "model_state_t2g128.pt")
    assert all(st[k].is_cuda and torch.equal(st[k].cpu(), ref[k]) for k in ref)
