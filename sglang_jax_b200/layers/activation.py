"""Gated activations."""
from torch import nn

from .. import ops
from ..ops import reference


class SiluAndMul(nn.Module):
    def forward(self, x):
        return ops.silu_and_mul(x)


class GeluAndMul(nn.Module):
    def __init__(self, approximate="tanh"):
        super().__init__()
        self.approximate = approximate

    def forward(self, x):
        return reference.gelu_and_mul(x, self.approximate)
