"""The Rezulorn decoder put together from parts.

Token embedding; per layer a ``ConvPreNormBlock`` (layer norms with a weight and no bias, a short causal convolution
in front of each sublayer, every branch times one constant) around one of three mixers and a feed-forward with the
square of relu (or none); the model's last layer norm; an output head of its own whose logits are scaled by a constant.
The mixers, by the layer's ``type``:

* ``lightning``: linear attention with a fixed decay per head, SiLU on q, k and v, one RMS norm with a weight over all
  heads' read-outs, a sigmoid gate;
* ``attention``: softmax attention without rotation, a logarithmic distance term taken off the scores, a sliding window
  that keeps the first tokens;
* ``parallel``: two mixers side by side on the same input, their results summed with two constants: causal attention
  with rotated, unit-length q and k whose weights are sigmoids of the scores plus a number per head (left), and linear
  attention with rotated q and k, k times ``dim ** -0.5``, every head's read-out divided by its root mean square, a SiLU
  gate (right).

Each layer's sizes come from its own entry of the config, so layers may differ in everything and come in any order.
Tensor names: ``embed``, ``l<i>.norm1``, ``l<i>.canon1``, ``l<i>.mix.*``, ``l<i>.norm2``, ``l<i>.canon2``, ``l<i>.mlp.*``,
``final.norm``, ``head``.
"""

from __future__ import annotations

from ..config.rezulorn import RezulornConfig
from ..parts.base import build_part
from ..parts.embedding import OutputHead, TokenEmbedding
from .model import ModelPlan, RunEntry


def build_rezulorn_plan(config: RezulornConfig) -> ModelPlan:
    width, eps, mult = config.width, config.eps, config.residual_mult
    positions: dict = {}

    def rotation(rot: dict | None):
        """One table per distinct rotation (layers with the same constants read the same tables)."""
        if not rot:
            return None
        divisor = float((rot.get("scaling") or {}).get("factor", 1.0))
        key = (int(rot["dims"]), float(rot["base"]), divisor)
        if key not in positions:
            positions[key] = build_part("position", "rope", dim=key[0], base=key[1], precise=True, divisor=divisor)
        return positions[key]

    def norm(name: str):
        return build_part("norm", "layernorm", size=width, eps=eps, weight_name=name, delta_scale=mult)

    def softmax_kind(m: dict, **rules):
        mask = m.get("mask") or {}
        return build_part("mixer", "scored_attention", hidden_size=width, n_q_heads=m["heads"], n_kv_heads=m["kv_heads"],
                          key_dim=m["dim"], value_dim=m["vdim"], scale=m["scale"], norm_eps=eps, position=rotation(m.get("rot")),
                          window=mask.get("size"), keep_first=mask.get("keep_first") or 0, **rules)

    def decay_kind(m: dict, **rules):
        return build_part("mixer", "decay_linear_attention", hidden_size=width, n_heads=m["heads"], key_dim=m["dim"],
                          value_dim=m["vdim"], decay=m["decay"], norm_eps=eps, position=rotation(m.get("rot")), **rules)

    layers = []
    for spec in config.layers:
        m = spec["mixer"]
        if spec["type"] == "lightning":
            mixer = decay_kind(m, activation="silu", read_norm="all", gate="sigmoid")
        elif spec["type"] == "attention":
            mixer = softmax_kind(m, distance_bias=True, weights="softmax")
        else:
            left = softmax_kind(m["left"], unit_qk=True, weights="sigmoid", head_bias=True)
            right = decay_kind(m["right"], k_scale=float(m["right"]["dim"]) ** -0.5, read_norm="head", gate="silu")
            mixer = build_part("mixer", "side_by_side", left=left, right=right, left_scale=m.get("left_scale", 1.0),
                               right_scale=m.get("right_scale", 1.0))
        mlp = spec.get("mlp")
        ffn = None
        if mlp is not None:
            ffn = build_part("feed_forward", "relu_squared", hidden_size=width, intermediate_size=mlp["ff"], up_name="up",
                             down_name="down")
        layers.append(build_part("block", "pre_norm_conv", width=width, norm_1=norm("norm1"), mixer=mixer,
                                 norm_2=norm("norm2") if ffn is not None else None, feed_forward=ffn, conv_taps=config.taps))
    return ModelPlan(
        embedding=TokenEmbedding(config.vocab, width, weight_name="embed"),
        layers=layers,
        final_norm=norm("norm"),
        head=OutputHead(width, config.vocab, weight_name="head", scale=config.logit_scale),
        run_list=[RunEntry(i) for i in range(len(layers))],
        positions=list(positions.values()),
        embedding_prefix="",
        layer_prefix="l{}.",
        final_norm_prefix="final.",
        head_prefix="",
    )
