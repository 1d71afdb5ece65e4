"""CPU checks of the oracle's two block-scaled formats (MXFP8, NVFP4), which the reference has no code for ("parity
unpinned"): the rounding tables and the properties the formats guarantee, so that the GPU parity tests compare against
a restatement that is at least self-consistent."""
import torch

from oracle import moe_oracle as orc


def test_e2m1_rounds_to_nearest_even_and_saturates():
    v = torch.tensor([0.0, 0.24, 0.25, 0.26, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 5.01, 6.0, 100.0, -0.26, -0.0, -100.0])
    want = [0, 0, 0, 1, 2, 2, 4, 4, 6, 6, 7, 7, 7, 9, 8, 15]
    assert orc.e2m1_codes(v).tolist() == want


def test_nvfp4_every_representable_value_survives():
    # x = code value * scale * g is reproduced exactly when the block's largest value is 6 * scale * g
    g = torch.tensor([0.125])
    vals = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0, 6.0])
    for scale in (0.015625, 1.0, 448.0):
        x = (vals * scale * g).reshape(1, 16)
        q, s = orc.quant_nvfp4(x, g)
        assert s.view(torch.float8_e4m3fn).float().item() == scale
        assert torch.equal(orc.dequant_nvfp4(q, s, g), x)


def test_nvfp4_quantiser_is_idempotent_and_bounded():
    gen = torch.Generator().manual_seed(0)
    x = torch.randn(64, 256, generator=gen) * 3.0
    g = orc.nvfp4_global_scale(x)
    q, s = orc.quant_nvfp4(x, g)
    dq = orc.dequant_nvfp4(q, s, g)
    q2, s2 = orc.quant_nvfp4(dq, g)
    assert torch.equal(orc.dequant_nvfp4(q2, s2, g), dq)
    # the error of a value is at most half the widest e2m1 step (2 = 6 - 4) of its block's scale, plus the part of
    # the block's amax that the e4m3 rounding of the scale cuts off (1/16 relative)
    step = (s.view(torch.float8_e4m3fn).float() * g).repeat_interleave(16, dim=-1)
    amax = x.reshape(64, 16, 16).abs().amax(dim=-1).repeat_interleave(16, dim=-1)
    assert bool(((dq - x).abs() <= step * 1.0 + amax / 16 + 1e-6).all())
    assert orc.cosine(dq, x) > 0.99


def test_nvfp4_zero_block_and_packing_order():
    x = torch.zeros(1, 32)
    x[0, 16] = 1.0       # element 0 of the second block -> low nibble of byte 8
    x[0, 17] = -3.0      # element 1 -> high nibble of byte 8
    g = torch.tensor([3.0 / 6.0 / 2.0])   # block scale byte = e4m3(2.0)
    q, s = orc.quant_nvfp4(x, g)
    assert s[0, 0].item() == 0 and torch.count_nonzero(q[0, :8]) == 0
    assert s.view(torch.float8_e4m3fn).float()[0, 1].item() == 2.0
    # 1.0 / (2 * 0.25) = 2.0 -> code 4; -3.0 / 0.5 = -6 -> code 15
    assert q[0, 8].item() == (4 | (15 << 4))


def test_mx_scale_is_the_smallest_power_of_two_that_fits():
    gen = torch.Generator().manual_seed(1)
    x = torch.randn(16, 128, generator=gen) * torch.logspace(-3, 3, 16).view(16, 1)
    q, s = orc.quant_mx(x)
    scale = torch.pow(2.0, s.float() - 127.0)
    amax = x.reshape(16, 4, 32).abs().amax(dim=-1)
    assert bool((amax / scale <= 448.0).all()) and bool((amax / (scale / 2) > 448.0).all())
    assert orc.cosine(orc.dequant_mx(q, s), x) > 0.999
