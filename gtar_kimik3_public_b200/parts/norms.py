"""The norms that read the residual stream, each fused with the add of a pending branch output into it: RMSNorm,
``weight * (x * rsqrt(mean(x^2) + eps))`` in 32-bit (src/layers/rmsnorm.py:11-16), and layer norm with a weight and no
bias."""

from __future__ import annotations

import torch

from ..ops import functional as F
from .base import Norm, TensorSpec, register_part


class RMSNorm(Norm):
    graph_safe = True

    def __init__(self, size: int, eps: float, weight_offset: float = 0.0, weight_name: str = "weight"):
        """``weight_offset``: the file stores the weight minus this number (1.0 for a weight kept around zero); the
        sum is formed once at load, in 32-bit, and the kernels multiply by it as by any weight.  ``weight_name``: the
        tensor's name relative to the part ("" where the part's prefix is the whole name)."""
        self.size = int(size)
        self.eps = float(eps)
        self.weight_offset = float(weight_offset)
        self.weight_name = weight_name
        self.weight: torch.Tensor | None = None

    def tensor_specs(self):
        init = (0.0, 0.1) if self.weight_offset else None
        return {self.weight_name: TensorSpec((self.size,), "vector", init=init)}

    def load(self, tensors):
        weight = tensors[self.weight_name]
        if self.weight_offset:
            weight = weight.float() + self.weight_offset
        self.weight = weight.contiguous()

    def weight_bytes(self):
        return self.weight.numel() * self.weight.element_size()

    def decode_record(self):
        return {"kind": "rmsnorm", "size": self.size, "eps": self.eps, "weight": self.weight}

    def forward(self, h, delta, out_dtype, rows=None):
        return F.add_rmsnorm(h, delta, self.weight, self.eps, out_dtype, rows)


register_part("norm", "rmsnorm", RMSNorm)


class LayerNorm(Norm):
    """Layer norm with a weight and no bias, ``(x - mean) / sqrt(mean((x - mean)^2) + eps) * weight`` in 32-bit, fused with
    the add of a pending branch output into the stream; ``delta_scale`` multiplies that branch as it is added (a model
    that scales every branch by one constant gives it to all its norms)."""

    graph_safe = True

    def __init__(self, size: int, eps: float, weight_name: str = "weight", delta_scale: float = 1.0):
        self.size, self.eps, self.weight_name, self.delta_scale = int(size), float(eps), weight_name, float(delta_scale)
        self.weight: torch.Tensor | None = None

    def tensor_specs(self):
        return {self.weight_name: TensorSpec((self.size,), "vector")}

    def load(self, tensors):
        self.weight = tensors[self.weight_name].float().contiguous()

    def weight_bytes(self):
        return self.weight.numel() * self.weight.element_size()

    def forward(self, h, delta, out_dtype, rows=None):
        return F.add_layernorm(h, delta, self.weight, self.eps, out_dtype, rows, self.delta_scale)

    def forward_conv_single(self, h, delta, conv_weight, state, ctx, update_state: bool):
        """The norm and the short convolution over time behind it as one kernel, in steps of one token a sequence."""
        return F.add_layernorm_conv_single(h, delta, self.weight, self.eps, conv_weight, state, ctx.tok_pos, ctx.tok_seq, ctx.slots,
                                           ctx.dtype, self.delta_scale, update_state)


register_part("norm", "layernorm", LayerNorm)
