"""SwiGLU feed-forward: ``down(silu(gate(x)) * up(x))`` (src/layers/swiglu.py:9-14), with the gate
and up projections as one packed matrix product whose rows alternate gate, up, gate, up, ... so
that the activation can be applied where the product is written (each output channel's two
numbers sit side by side in the accumulator)."""

from __future__ import annotations

import torch

from ..ops import functional as F
from ..ops.linear import linear, linear_normed, linear_on_stream_ok, linear_residual
from .base import FeedForward, StepContext, TensorSpec, register_part


class SwiGLUFeedForward(FeedForward):
    graph_safe = True

    def __init__(self, hidden_size: int, intermediate_size: int):
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.w_gate_up = self.w_down = None

    def tensor_specs(self):
        h, i = self.hidden_size, self.intermediate_size
        return {
            "gate_proj.weight": TensorSpec((i, h)),
            "up_proj.weight": TensorSpec((i, h)),
            "down_proj.weight": TensorSpec((h, i)),
        }

    def load(self, tensors):
        gate, up = tensors["gate_proj.weight"], tensors["up_proj.weight"]
        if gate.dtype != up.dtype:
            gate, up = gate.float(), up.float()
        self.w_gate_up = torch.stack([gate, up], dim=1).reshape(2 * gate.shape[0], gate.shape[1]).contiguous()
        self.w_down = tensors["down_proj.weight"].contiguous()

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_gate_up, self.w_down))

    def decode_record(self):
        if self.w_gate_up.dtype != torch.bfloat16 or self.w_down.dtype != torch.bfloat16:
            return None
        return {"kind": "swiglu", "hidden": self.hidden_size, "inter": self.intermediate_size, "w_gu": self.w_gate_up,
                "w_down": self.w_down}

    def forward(self, x, ctx: StepContext) -> torch.Tensor:
        return linear(linear(x, self.w_gate_up, swiglu=True), self.w_down)

    def on_stream_ok(self, h: torch.Tensor, norm_weight, ctx: StepContext) -> bool:
        return ctx.dtype == torch.bfloat16 and linear_on_stream_ok(h, norm_weight, self.w_gate_up, self.w_down)

    def forward_on_stream(self, h: torch.Tensor, norm_weight: torch.Tensor, norm_eps: float, ctx: StepContext) -> None:
        """``h += down(silu(gate(y)) * up(y))`` with ``y = rmsnorm(h)`` formed inside the gate|up product and the add
        in the down product's output stage."""
        linear_residual(linear_normed(h, norm_weight, norm_eps, self.w_gate_up, swiglu=True), self.w_down, h)


register_part("feed_forward", "swiglu", SwiGLUFeedForward)


class GeluFeedForward(FeedForward):
    """``down(gelu(up(x)))`` with the tanh form of GELU, ``0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))``; no gate,
    no biases.  Tensor names are given by the builder (defaults ``up.weight`` / ``down.weight``)."""

    graph_safe = True

    def __init__(self, hidden_size: int, intermediate_size: int, up_name: str = "up.weight", down_name: str = "down.weight"):
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.up_name, self.down_name = up_name, down_name
        self.w_up = self.w_down = None

    def tensor_specs(self):
        h, i = self.hidden_size, self.intermediate_size
        return {self.up_name: TensorSpec((i, h)), self.down_name: TensorSpec((h, i))}

    def load(self, tensors):
        self.w_up = tensors[self.up_name].contiguous()
        self.w_down = tensors[self.down_name].contiguous()

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_up, self.w_down))

    def forward(self, x, ctx: StepContext) -> torch.Tensor:
        return linear(linear(x, self.w_up, gelu=True), self.w_down)


register_part("feed_forward", "gelu", GeluFeedForward)


class ReluSquaredFeedForward(FeedForward):
    """``down(relu(up(x))^2)``: no gate, no biases.  The activation is the output stage of the few-token product and a
    kernel of its own behind the many-token product."""

    graph_safe = True

    def __init__(self, hidden_size: int, intermediate_size: int, up_name: str = "up.weight", down_name: str = "down.weight"):
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.up_name, self.down_name = up_name, down_name
        self.w_up = self.w_down = None

    def tensor_specs(self):
        h, i = self.hidden_size, self.intermediate_size
        return {self.up_name: TensorSpec((i, h)), self.down_name: TensorSpec((h, i))}

    def load(self, tensors):
        self.w_up = tensors[self.up_name].contiguous()
        self.w_down = tensors[self.down_name].contiguous()

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_up, self.w_down))

    def forward(self, x, ctx: StepContext) -> torch.Tensor:
        return linear(linear(x, self.w_up, relu_squared=True), self.w_down)


register_part("feed_forward", "relu_squared", ReluSquaredFeedForward)


class XieluFeedForward(FeedForward):
    """``down(act(up(x)))`` with an activation that is quadratic above zero and exponential below, joined smoothly at
    zero, shaped by two stored numbers ``p`` and ``q`` (tensor ``act`` ``[2]``):

        z > 0:   softplus(p) z^2 + z / 2          z <= 0:   (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2

    No gate, no biases.  The two constants are formed once at load, in 32-bit; the activation is the output stage of the
    few-token product (applied to its 32-bit sums) and a kernel of its own behind the many-token product."""

    graph_safe = True

    def __init__(self, hidden_size: int, intermediate_size: int, up_name: str = "up", down_name: str = "down", act_name: str = "act"):
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.up_name, self.down_name, self.act_name = up_name, down_name, act_name
        self.w_up = self.w_down = None
        self.up_const = self.down_const = 0.0

    def tensor_specs(self):
        h, i = self.hidden_size, self.intermediate_size
        return {self.up_name: TensorSpec((i, h)), self.down_name: TensorSpec((h, i)),
                self.act_name: TensorSpec((2,), "vector", init=(0.5, 0.4))}

    def load(self, tensors):
        self.w_up = tensors[self.up_name].contiguous()
        self.w_down = tensors[self.down_name].contiguous()
        p, q = torch.nn.functional.softplus(tensors[self.act_name].float()).tolist()
        self.up_const, self.down_const = p, 0.5 + q

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_up, self.w_down))

    def forward(self, x, ctx: StepContext) -> torch.Tensor:
        return linear(linear(x, self.w_up, xielu=(self.up_const, self.down_const)), self.w_down)


register_part("feed_forward", "xielu", XieluFeedForward)
