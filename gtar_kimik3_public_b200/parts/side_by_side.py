"""Two mixers side by side: both read the same input, and the result is ``left_scale * left(x) + right_scale * right(x)``
(the sum formed in 32-bit).  The two keep what they need between steps independently: the pair's cache request is the
list of both mixers' requests, the left one's first.  Their tensors sit under the prefixes ``left.`` and ``right.``."""

from __future__ import annotations

from ..ops import functional as F
from .base import Mixer, StepContext, register_part


def _as_list(request) -> list:
    if request is None:
        return []
    return list(request) if isinstance(request, (list, tuple)) else [request]


class SideBySide(Mixer):
    def __init__(self, left: Mixer, right: Mixer, left_scale: float = 1.0, right_scale: float = 1.0,
                 names: dict[str, str] | None = None):
        self.left, self.right, self.left_scale, self.right_scale = left, right, float(left_scale), float(right_scale)
        self.names = {"left": "left.", "right": "right.", **(names or {})}

    @property
    def graph_safe(self) -> bool:
        return self.left.graph_safe and self.right.graph_safe

    def children(self):
        return [(self.names["left"], self.left), (self.names["right"], self.right)]

    def tensor_specs(self):
        return {prefix + name: spec for prefix, part in self.children() for name, spec in part.tensor_specs().items()}

    def load(self, tensors):
        for prefix, part in self.children():
            part.load({name: tensors[prefix + name] for name in part.tensor_specs() if prefix + name in tensors})

    def weight_bytes(self):
        return self.left.weight_bytes() + self.right.weight_bytes()

    def cache_request(self):
        return _as_list(self.left.cache_request()) + _as_list(self.right.cache_request())

    @staticmethod
    def _views(request, views: list):
        """The storage of one of the two, in the form its own request has: one view, None, or a tuple."""
        if request is None:
            return None
        if isinstance(request, (list, tuple)):
            return tuple(views.pop(0) for _ in request)
        return views.pop(0)

    def forward(self, x, ctx: StepContext, cache):
        views = list(cache) if isinstance(cache, (list, tuple)) else ([] if cache is None else [cache])
        left = self.left.forward(x, ctx, self._views(self.left.cache_request(), views))
        right = self.right.forward(x, ctx, self._views(self.right.cache_request(), views))
        return F.scaled_sum(left, self.left_scale, right, self.right_scale)


register_part("mixer", "side_by_side", SideBySide)
