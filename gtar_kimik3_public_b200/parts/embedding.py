"""Token embedding (``h0 = E[ids]``, src/models/transformer.py:55,61) and the output head
(``logits = z @ W.T``, tied to the embedding table or its own; transformer.py:75-77,101)."""

from __future__ import annotations

import torch

from ..ops import functional as F
from ..ops.linear import linear
from .base import Part, TensorSpec


class TokenEmbedding(Part):
    graph_safe = True

    def __init__(self, vocab_size: int, hidden_size: int, weight_name: str = "weight", scale: float = 1.0):
        """``scale`` multiplies every row as it enters the 32-bit stream (1.0: the table's rows as they are)."""
        self.vocab_size, self.hidden_size = int(vocab_size), int(hidden_size)
        self.weight_name, self.scale = weight_name, float(scale)
        self.weight: torch.Tensor | None = None

    def tensor_specs(self):
        return {self.weight_name: TensorSpec((self.vocab_size, self.hidden_size))}

    def load(self, tensors):
        self.weight = tensors[self.weight_name].contiguous()

    def forward(self, ids: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        return F.embed_rows(self.weight, ids, out, self.scale)


class OutputHead(Part):
    graph_safe = True

    """Logits in float32.  ``tied_to`` names an embedding whose table is used instead of an own matrix.  ``softcap``:
    the logits become ``softcap * tanh(logits / softcap)`` (None: they stay as they are).  ``scale``: a constant on
    the logits (applied to the 32-bit products, before a cap)."""

    def __init__(self, hidden_size: int, vocab_size: int, tied_to: TokenEmbedding | None = None, weight_name: str = "weight",
                 softcap: float | None = None, scale: float = 1.0):
        self.hidden_size, self.vocab_size, self.tied_to = int(hidden_size), int(vocab_size), tied_to
        self.weight_name, self.softcap, self.scale = weight_name, (None if softcap is None else float(softcap)), float(scale)
        self._weight: torch.Tensor | None = None

    def tensor_specs(self):
        # A tied model's file may still carry the head (the reference's state dict does): it is
        # accepted and not read.
        return {self.weight_name: TensorSpec((self.vocab_size, self.hidden_size), optional=self.tied_to is not None)}

    def load(self, tensors):
        if self.tied_to is None:
            self._weight = tensors[self.weight_name].contiguous()

    @property
    def weight(self) -> torch.Tensor:
        return self.tied_to.weight if self.tied_to is not None else self._weight

    def weight_bytes(self):
        return self.weight.numel() * self.weight.element_size()

    def forward(self, z: torch.Tensor) -> torch.Tensor:
        logits = linear(z, self.weight, torch.float32)
        if self.scale != 1.0:
            logits = F.scale_(logits, self.scale)
        return F.softcap_(logits, self.softcap) if self.softcap is not None else logits
