"""SiluAndMul on the F3 kernel (reference: layers/activation.py:6-13), and the dense feed-forward with a clamped
gated unit that several of the listed-layer decoders share."""
import torch
from torch import nn

from .. import ops
from .linear import MergedColumnParallelLinear, RowParallelLinear


class SiluAndMul(nn.Module):

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.silu_and_mul(x)


class ClampedGatedFeedForward(nn.Module):
    """W_down(g sigmoid(alpha g) (u + 1)), g = min(W_gate h, limit), u = clamp(W_up h, -limit, limit)."""

    def __init__(self, width: int, ff: int, limit: float, alpha: float = 1.702):
        super().__init__()
        self.limit, self.alpha = float(limit), float(alpha)
        self.gate_up_proj = MergedColumnParallelLinear(width, [ff, ff])
        self.down_proj = RowParallelLinear(ff, width)

    def forward(self, h):
        return self.down_proj(ops.glu_clamped(self.gate_up_proj(h), self.alpha, self.limit))
