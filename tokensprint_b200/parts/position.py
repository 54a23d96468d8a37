"""Rotary position encoding (rotate-half pairing) as a part of its own."""

from __future__ import annotations

from typing import Optional

import torch

from tokensprint_b200 import ops
from tokensprint_b200.parts.base import BuildContext, PositionEncoding, StepContext, register_part


def rope_inverse_frequencies(dim: int, theta: float) -> torch.Tensor:
    """inv_freq[j] = 1 / theta^(2j/dim), j = 0..dim/2-1, float32 on the host.

    The reference's formula and dtype (engine/nn/rope.py:28-29).
    """
    idx = torch.arange(0, dim, step=2, dtype=torch.float32)
    return 1.0 / (theta ** (idx / dim))


def rope_inverse_frequencies_exact(dim: int, theta: float) -> torch.Tensor:
    """theta^(-2j/dim), j = 0..dim/2-1, worked out in float64 and rounded once to float32."""
    idx = torch.arange(0, dim, step=2, dtype=torch.float64)
    return torch.pow(torch.tensor(float(theta), dtype=torch.float64), -idx / dim).to(torch.float32)


@register_part("position_encoding", "rotary")
class RotaryEncoding(PositionEncoding):
    """x'[j] = x[j] cos - x[j+r/2] sin, x'[j+r/2] = x[j+r/2] cos + x[j] sin over the first
    `dim` (= r) entries of each head, angle = position * inv_freq[j] in float32
    (engine/nn/rope.py:105-123, engine/kernels/triton/rope.py:22-65).  The rotation
    itself runs inside the fused q/k kernel; this part owns the frequencies.

    `pairing` "half" (the default) is the above; "neighbours" turns entry 2i with entry 2i+1 by
    the same angles (mixers whose kernels take a pairing ask for it through `pairing`; the fused
    q/k kernels of the attention mixer know the half pairing only, so `rotary_inv_freq()` answers
    None for the other and that mixer falls back to `apply`, which this part does not offer).
    `exact_frequencies`: the inverse frequencies are worked out in float64 before they are rounded."""

    graph_safe = True

    def __init__(self, ctx: BuildContext, *, dim: int, theta: float, pairing: str = "half", exact_frequencies: bool = False) -> None:
        if dim % 2:
            raise ValueError(f"rotary width must be even, got {dim}")
        if pairing not in ops.ROTARY_PAIRINGS:
            raise ValueError(f"rotary pairing must be one of {sorted(ops.ROTARY_PAIRINGS)}, got {pairing!r}")
        self.dim, self.theta, self.pairing = int(dim), float(theta), pairing
        make = rope_inverse_frequencies_exact if exact_frequencies else rope_inverse_frequencies
        self.inv_freq = make(self.dim, self.theta).to(ctx.device)

    def rotary_inv_freq(self) -> Optional[torch.Tensor]:
        return self.inv_freq if self.pairing == "half" else None

    def frequencies(self) -> torch.Tensor:
        """[dim/2] float32 inverse frequencies, whatever the pairing (for kernels that take one)."""
        return self.inv_freq

    def rotary_cos_sin(self, step: StepContext) -> Optional[torch.Tensor]:
        """The table of the step, made by the first layer that asks and used by all layers with the
        same width and base (angles, cosines and sines in float32, as in the rotating kernels)."""
        key = ("rotary_cos_sin", self.dim, self.theta)
        table = step.shared.get(key)
        if table is None:
            table = step.shared[key] = ops.rope_cos_sin(step.positions, self.inv_freq, step.num_tokens)
        return table
