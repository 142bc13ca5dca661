"""The Zasorax decoder put together from parts.

Token embedding times a constant; per layer an ``OutNormBlock`` (the sublayers read the stream itself; an RMS norm with a
weight on each sublayer's RESULT before it is added) around one of two mixers and a feed-forward (dense with the xIELU
activation, routed experts, or none); the model's last norm; an output head of its own.  The mixers, by the layer's
``type``, are both the scored attention of this library under different rules:

* ``attention``: norms over the whole query row and the whole key row, no rotation, a number per head on the products, a
  learned term by distance from a table with logarithmically widening rows, keys of the token's own chunk only, a learned
  sink per head in the softmax; with ``kv_from`` the layer reads the pages of an earlier layer of the same sizes;
* ``attention_2``: causal, q and k rotated (part of each head) and then brought to unit root mean square, values turned by
  their own position and read-outs turned back by the reader's, one added to the softmax's denominator, a sigmoid gate
  per head.

Each layer's sizes come from its own entry of the config, so layers may differ in everything and come in any order.
Tensor names: ``embed``, ``l<i>.norm1``, ``l<i>.mix.*``, ``l<i>.norm2``, ``l<i>.mlp.*``, ``final.norm``, ``head``.
"""

from __future__ import annotations

import math

from ..config.zasorax import DEFAULT_BIAS_ROWS, ZasoraxConfig
from ..parts.base import build_part
from ..parts.embedding import OutputHead, TokenEmbedding
from .model import ModelPlan, RunEntry


def build_zasorax_plan(config: ZasoraxConfig) -> ModelPlan:
    width, eps = config.width, config.eps
    positions: dict = {}

    def rotation(dims: int, base: float):
        """One table per distinct rotation (layers with the same constants read the same tables)."""
        key = (int(dims), float(base))
        if key not in positions:
            positions[key] = build_part("position", "rope", dim=key[0], base=key[1], precise=True)
        return positions[key]

    def norm(name: str):
        return build_part("norm", "rmsnorm", size=width, eps=eps, weight_name=name)

    # pages are kept as far back as the furthest look of the layer that owns them and of every layer that reads them
    readers: dict[int, list[dict]] = {}
    for i, spec in enumerate(config.layers):
        owner = spec["mixer"].get("kv_from")
        readers.setdefault(i if owner is None else owner, []).append(spec["mixer"])

    layers, run_list = [], []
    for i, spec in enumerate(config.layers):
        m = spec["mixer"]
        source = m.get("kv_from")
        common = dict(hidden_size=width, n_q_heads=m["heads"], n_kv_heads=m["kv_heads"], key_dim=m["dim"], value_dim=m["vdim"],
                      scale=m["scale"], norm_eps=eps, own_kv=source is None)
        if spec["type"] == "attention":
            # what the random-weights mode writes (half the rows must lie below bias_max); a model file's tensor has the last word
            rows = m.get("bias_rows") or max(2, min(DEFAULT_BIAS_ROWS, 2 * (math.ceil(m["bias_max"]) - 1)))
            chunks = [(r.get("mask") or {}).get("size") for r in readers[i if source is None else source]]
            span = None if None in chunks else max(chunks)  # a reader without chunks needs every page kept
            mixer = build_part("mixer", "scored_attention", wide_norm=True, temperature=True, distance_table=(rows, m["bias_max"]),
                               chunk=(m.get("mask") or {}).get("size"), sink="learned", cache_span=span, **common)
        else:
            rot = m["rot"]
            mixer = build_part("mixer", "scored_attention", position=rotation(rot["dims"], rot["base"]), unit_qk=True, sink="zero",
                               value_position=rotation(m["vdim"], rot["base"]), head_gate=True, **common)
        mlp = spec.get("mlp")
        ffn = None
        if mlp is not None and mlp["kind"] == "dense":
            ffn = build_part("feed_forward", "xielu", hidden_size=width, intermediate_size=mlp["ff"])
        elif mlp is not None:
            r = mlp["router"]
            ffn = build_part("feed_forward", "routed_experts", hidden_size=width, expert_size=mlp["expert"]["ff"], n_experts=r["experts"],
                             top=r["top"], logit_weights=True, bias_name="router.b")
        layers.append(build_part("block", "out_norm", norm_1=norm("norm1"), mixer=mixer, norm_2=norm("norm2") if ffn is not None else None,
                                 feed_forward=ffn, first=i == 0))
        run_list.append(RunEntry(i, cache_of=source))
    return ModelPlan(
        embedding=TokenEmbedding(config.vocab, width, weight_name="embed", scale=config.embedding_scale),
        layers=layers,
        final_norm=norm("norm"),
        head=OutputHead(width, config.vocab, weight_name="head"),
        run_list=run_list,
        positions=list(positions.values()),
        embedding_prefix="",
        layer_prefix="l{}.",
        final_norm_prefix="final.",
        head_prefix="",
    )
