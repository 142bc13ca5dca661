"""A feed-forward of many small gated experts, of which every token uses a few.

Expert ``e``: ``W_down[e] (silu(W_gate[e] x) * (W_up[e] x))``, no biases.  Router: ``z = W_r x`` in 32-bit, scores
``s = sigmoid(z)``; the choice goes by ``s + correction`` (a stored vector), the weights by ``s`` alone.  The experts form
``n_groups`` equal groups of neighbours; a group's score is the sum of its two largest choice scores, and only experts of
the best ``keep_groups`` groups can be chosen (the others count as minus infinity).  The ``top`` largest choice scores are
chosen; a chosen expert's output is weighted by ``s * route_scale`` (not renormalised) and the weighted outputs are added.

Tensors: ``e<i>.gate``, ``e<i>.up`` ``[ff, hidden]``, ``e<i>.down`` ``[hidden, ff]``, ``router`` ``[experts, hidden]``,
``correction`` ``[experts]``; stacked at load into ``[E, 2, ff, hidden]`` and ``[E, hidden, ff]``.

With ``logit_weights`` the router is plainer: scores are the logits plus a stored bias, ``s = z + b`` (the bias tensor's
name is the builder's, ``bias_name``), the ``top`` largest are chosen, and the chosen experts' weights are the softmax
over the chosen scores alone (times ``route_scale``).

The result is 32-bit (it goes into the residual stream); ``forward_added`` folds another branch's output into the
same sum, for blocks whose branches read one norm.
"""

from __future__ import annotations

import torch

from ..ops import functional as F
from ..ops.linear import grouped_product_ok, linear_grouped
from .base import FeedForward, StepContext, TensorSpec, register_part


class RoutedExperts(FeedForward):
    graph_safe = True

    def __init__(self, hidden_size: int, expert_size: int, n_experts: int, top: int, route_scale: float = 1.0,
                 n_groups: int = 1, keep_groups: int = 1, logit_weights: bool = False, bias_name: str = "correction"):
        self.hidden_size, self.ff, self.n_experts, self.top = int(hidden_size), int(expert_size), int(n_experts), int(top)
        self.route_scale, self.n_groups, self.keep = float(route_scale), int(n_groups), int(keep_groups)
        if self.n_experts % self.n_groups or not 1 <= self.keep <= self.n_groups:
            raise ValueError(f"{self.n_experts} experts do not form {self.n_groups} equal groups of which {self.keep} are kept")
        if not 1 <= self.top <= self.keep * (self.n_experts // self.n_groups):
            raise ValueError(f"{self.top} experts cannot be chosen from {self.keep} groups of {self.n_experts // self.n_groups}")
        self.logit_weights, self.bias_name = bool(logit_weights), bias_name
        self.w_gate_up = self.w_down = self.w_router = self.correction = None
        # from this many (token, expert) pairs on, a bfloat16 step sorts its pairs by expert and runs each expert's rows
        # through one tensor-core product; below, every pair streams its expert's weights by itself
        self.grouped_from_pairs = 256

    def tensor_specs(self):
        W, ff = self.hidden_size, self.ff
        specs = {}
        for e in range(self.n_experts):
            specs[f"e{e}.gate"] = TensorSpec((ff, W))
            specs[f"e{e}.up"] = TensorSpec((ff, W))
            specs[f"e{e}.down"] = TensorSpec((W, ff))
        specs["router"] = TensorSpec((self.n_experts, W), init=(0.0, 0.5))
        specs[self.bias_name] = TensorSpec((self.n_experts,), "vector", init=(0.0, 0.3))
        return specs

    def load(self, tensors):
        E = self.n_experts
        mats = [tensors[f"e{e}.{part}"] for e in range(E) for part in ("gate", "up", "down")]
        kind = torch.float32 if any(m.dtype == torch.float32 for m in mats) else mats[0].dtype
        self.w_gate_up = torch.stack([torch.stack([tensors[f"e{e}.gate"].to(kind), tensors[f"e{e}.up"].to(kind)]) for e in range(E)]).contiguous()
        self.w_down = torch.stack([tensors[f"e{e}.down"].to(kind) for e in range(E)]).contiguous()
        self.w_router = tensors["router"].float().contiguous()
        self.correction = tensors[self.bias_name].float().contiguous()

    def weight_bytes(self):
        """What a single token reads: its ``top`` experts and the router."""
        per_expert = (self.w_gate_up[0].numel() + self.w_down[0].numel()) * self.w_down.element_size()
        return self.top * per_expert + self.w_router.numel() * 4

    def route(self, x: torch.Tensor):
        return F.route_groups(x, self.w_router, self.correction, self.top, self.n_groups, self.keep, self.route_scale,
                              logits=self.logit_weights)

    def forward_added(self, x: torch.Tensor, ctx: StepContext, add: torch.Tensor | None) -> torch.Tensor:
        """``add + experts(x)`` as one 32-bit sum (``add``: another branch's output for the same tokens, or None)."""
        ids, weights = self.route(x)
        if x.shape[0] * self.top >= self.grouped_from_pairs and self.ff % 8 == 0 and grouped_product_ok(x, self.w_down):
            # many tokens: the pairs in the order of their experts, each expert's rows through one product
            ends, place_of, pair_at = F.experts_sort(ids, self.n_experts)
            rows = F.gather_rows(x, pair_at, self.top)
            act = F.swiglu(linear_grouped(rows, self.w_gate_up.view(self.n_experts, 2 * self.ff, self.hidden_size), ends))
            return F.experts_combine(linear_grouped(act, self.w_down, ends), place_of, weights, add)
        return F.experts_pairwise(x, self.w_gate_up, self.w_down, ids, weights, add)

    def forward(self, x, ctx: StepContext) -> torch.Tensor:
        return self.forward_added(x, ctx, None)


register_part("feed_forward", "routed_experts", RoutedExperts)
