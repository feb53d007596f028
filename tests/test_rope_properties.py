"""What the llama3 frequency scaling must do, stated as properties rather than as its formula, and checked on
both statements of the formula (the part's table and the plain implementation's): short wavelengths are kept,
long ones are divided by the factor, the band between is a blend that joins both ends without a jump and
never leaves the range between them.  Parameter sets: the tiny configurations and the Llama 3.1 8B / 3.2 3B
values (the reference has no such scaling to compare with: kvcore/model/layer/rotary_embedding.py:62-69 is
the plain table only)."""
from __future__ import annotations

import math

import pytest
import torch

import plain_llama
from kvcore_b200.parts.rope import rope_inverse_frequencies

CASES = {
    "tiny B": dict(head_dim=32, theta=500000.0, factor=8.0, low=1.0, high=4.0, original=64),
    "tiny D": dict(head_dim=128, theta=500000.0, factor=8.0, low=1.0, high=4.0, original=128),
    "8B": dict(head_dim=128, theta=500000.0, factor=8.0, low=1.0, high=4.0, original=8192),
    "3B": dict(head_dim=128, theta=500000.0, factor=32.0, low=1.0, high=4.0, original=8192),
    "odd": dict(head_dim=96, theta=10000.0, factor=3.0, low=2.0, high=5.0, original=1000),
}


def tables(case):
    """(plain table, the part's table, unscaled table), all float64."""
    config = dict(hidden_size=case["head_dim"], num_attention_heads=1, head_dim=case["head_dim"], rope_theta=case["theta"],
                  rope_scaling=dict(rope_type="llama3", factor=case["factor"], low_freq_factor=case["low"],
                                    high_freq_factor=case["high"], original_max_position_embeddings=case["original"]))
    plain = plain_llama.rope_inv_freq(config).to(torch.float64)
    part = rope_inverse_frequencies(case["head_dim"], case["theta"], "llama3", case["factor"], case["low"], case["high"],
                                    case["original"]).to(torch.float64)
    base = torch.tensor([case["theta"] ** (-(2.0 * j) / case["head_dim"]) for j in range(case["head_dim"] // 2)],
                        dtype=torch.float64)
    return plain, part, base


@pytest.mark.parametrize("name", sorted(CASES))
def test_llama3_scaling_keeps_divides_and_blends(name):
    case = CASES[name]
    plain, part, base = tables(case)
    torch.testing.assert_close(part, plain, rtol=2e-7, atol=0.0)          # the part keeps its table in 32-bit
    wavelen = 2.0 * math.pi / base
    short, long_ = case["original"] / case["high"], case["original"] / case["low"]
    for table in (plain, part):
        ratio = table / base
        kept, divided = wavelen < short, wavelen > long_
        band = ~(kept | divided)
        assert kept.any() and divided.any(), "the case should reach both ends"
        torch.testing.assert_close(ratio[kept], torch.ones_like(ratio[kept]), rtol=2e-7, atol=0.0)
        torch.testing.assert_close(ratio[divided], torch.full_like(ratio[divided], 1.0 / case["factor"]), rtol=2e-7, atol=0.0)
        # inside the band: between the two ends, and falling as the wavelength grows
        assert bool(((ratio[band] <= 1.0 + 1e-6) & (ratio[band] >= 1.0 / case["factor"] - 1e-6)).all())
        order = torch.argsort(wavelen)
        along = ratio[order]
        assert bool((along[1:] <= along[:-1] + 1e-6).all()), "the scaling must not grow with the wavelength"
        # the frequencies themselves still fall from one component to the next
        assert bool((table[1:] < table[:-1]).all())


def test_the_blend_joins_both_ends():
    """At a wavelength just inside either edge of the band the blend equals the value outside it (no jump):
    probed with a table whose base is chosen so that components land next to the edges."""
    original, factor, low, high, dim = 8192.0, 8.0, 1.0, 4.0, 64
    for edge, want in ((original / high, 1.0), (original / low, 1.0 / factor)):
        for nudge in (1.0 - 1e-9, 1.0 + 1e-9):
            # theta such that component j = 1 has exactly the wavelength edge * nudge: f = theta^(-2/dim)
            f = 2.0 * math.pi / (edge * nudge)
            theta = f ** (-dim / 2.0)
            config = dict(hidden_size=dim, num_attention_heads=1, head_dim=dim, rope_theta=theta,
                          rope_scaling=dict(rope_type="llama3", factor=factor, low_freq_factor=low, high_freq_factor=high,
                                            original_max_position_embeddings=int(original)))
            plain = float(plain_llama.rope_inv_freq(config)[1]) / f
            part = float(rope_inverse_frequencies(dim, theta, "llama3", factor, low, high, int(original)).to(torch.float64)[1]) / f
            assert abs(plain - want) < 1e-6 and abs(part - want) < 1e-6, (edge, nudge, plain, part)


def test_linear_scaling_divides_everything_and_default_changes_nothing():
    base = rope_inverse_frequencies(64, 10000.0).to(torch.float64)
    linear = rope_inverse_frequencies(64, 10000.0, "linear", 4.0).to(torch.float64)
    torch.testing.assert_close(linear * 4.0, base, rtol=2e-7, atol=0.0)
    config = dict(hidden_size=64, num_attention_heads=1, head_dim=64, rope_theta=10000.0)
    torch.testing.assert_close(plain_llama.rope_inv_freq(config).to(torch.float64), base, rtol=2e-7, atol=0.0)
