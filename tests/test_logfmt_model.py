"""The PyTorch model of the 10-bit logarithmic row format (CPU): range, zeros, error bound."""
import torch

from nixl_b200.ops.logfmt import logfmt10_codes, logfmt10_roundtrip, logfmt10_row_bytes


def test_codes_fit_nine_bits_and_zero_is_exact():
    torch.manual_seed(1)
    x = torch.randn(16, 1024).bfloat16()
    x[0, :128] = 0
    x[1, 7] = 0
    codes, neg, pmin, per_step = logfmt10_codes(x)
    assert codes.min().item() == 0 and codes.max().item() == 511
    assert torch.all(codes[0, :128] == 0) and codes[1, 7].item() == 0
    assert torch.equal(neg, x < 0)
    y = logfmt10_roundtrip(x)
    assert torch.all(y[0, :128] == 0) and y[1, 7].item() == 0
    assert pmin.shape == (16, 8) and per_step.shape == (16, 8)


def test_a_group_within_four_octaves_is_coded_exactly():
    torch.manual_seed(3)
    x = ((torch.rand(8, 512) * 0.9 + 0.1) * torch.where(torch.rand(8, 512) < 0.5, -1.0, 1.0)).bfloat16()  # |x| in [0.1, 1): < 4 octaves
    x[:, ::17] = 0
    assert torch.equal(logfmt10_roundtrip(x), x.float())


def test_relative_error_stays_within_half_a_step():
    torch.manual_seed(2)
    x = (torch.randn(32, 2048) * torch.logspace(-3, 3, 32).unsqueeze(1)).bfloat16()
    _, _, _, per_step = logfmt10_codes(x)
    y = logfmt10_roundtrip(x)
    xf = x.float()
    rel = (y - xf).abs() / xf.abs().clamp(min=1e-30)
    # Half a step of `per_step` patterns plus half a pattern for the decoder's rounding to a
    # whole pattern; one pattern is at most 2^-7 of the value.
    bound = ((per_step + 1) * 0.5 * 2.0 ** -7).repeat_interleave(128, dim=-1)
    live = xf != 0
    assert torch.all(rel[live] <= bound[live] * 1.01 + 1e-6)
    assert ((y - xf).norm() / xf.norm()).item() < 6e-3


def test_extremes_of_a_group_are_kept_and_a_wide_range_is_clipped_from_below():
    x = torch.zeros(1, 128)
    x[0, 0], x[0, 1], x[0, 2] = 3.0, -0.01, 2.0 ** -40   # the last lies more than 32 octaves below the largest
    y = logfmt10_roundtrip(x)
    assert y[0, 0].item() == 3.0
    assert abs(y[0, 1].item() + 0.01) / 0.01 < 0.04
    assert 0 < y[0, 2].item() <= 3.0 * 2.0 ** -32 * 1.001
    single = torch.full((1, 128), -0.75)
    assert torch.equal(logfmt10_roundtrip(single), single)
    big = torch.full((1, 128), float("inf"))
    assert torch.isfinite(logfmt10_roundtrip(big)).all()


def test_row_bytes():
    assert logfmt10_row_bytes(7168) == 7168 * 10 // 8 + 56 * 8 == 9408
    assert logfmt10_row_bytes(7168) / (7168 * 2) < 0.66
