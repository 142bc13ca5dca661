"""Pre-norm residual block: ``h += mixer(norm_in(h)); h += ffn(norm_post(h))``
(src/models/transformer.py:47-48).  The adds are fused into the norm that follows them: the
block hands its last branch output on as ``pending`` instead of adding it itself.  Beside it: the block with
convolutions over time in front of its sublayers, the block whose branches share one norm, the block that norms
every branch on both sides, and the block that norms every branch on its way OUT only."""

from __future__ import annotations

import torch

from ..ops import functional as F
from .base import Block, FeedForward, Mixer, Norm, StepContext, register_part


class PreNormBlock(Block):
    def __init__(self, input_norm: Norm, mixer: Mixer, post_norm: Norm, feed_forward: FeedForward,
                 names: dict[str, str] | None = None):
        self.input_norm, self.mixer, self.post_norm, self.feed_forward = input_norm, mixer, post_norm, feed_forward
        # tensor-name prefixes of the four parts inside the layer
        self.names = names or {
            "input_norm": "input_layernorm.",
            "mixer": "self_attn.",
            "post_norm": "post_attention_layernorm.",
            "feed_forward": "mlp.",
        }

    def children(self):
        return [(self.names[k], getattr(self, k)) for k in ("input_norm", "mixer", "post_norm", "feed_forward")]

    def tensor_specs(self):
        return {prefix + name: spec for prefix, part in self.children() for name, spec in part.tensor_specs().items()}

    def load(self, tensors):
        for prefix, part in self.children():
            part.load({name[len(prefix):]: t for name, t in tensors.items() if name.startswith(prefix)})

    def weight_bytes(self):
        return sum(part.weight_bytes() for _, part in self.children())

    def decode_record(self) -> dict | None:
        """What the persistent decode kernel needs of this layer (weights, constants, sizes), or None when one of
        the four parts is not of the kind that kernel computes; each part answers for itself."""
        pieces = {}
        for key, part in (("in", self.input_norm), ("mixer", self.mixer), ("post", self.post_norm), ("ffn", self.feed_forward)):
            describe = getattr(part, "decode_record", None)
            piece = describe() if describe is not None else None
            if piece is None:
                return None
            pieces[key] = piece
        norm_in, norm_post, mixer, ffn = pieces["in"], pieces["post"], pieces["mixer"], pieces["ffn"]
        if mixer.get("kind") != "gqa" or ffn.get("kind") != "swiglu" or norm_in.get("kind") != "rmsnorm" or norm_post.get("kind") != "rmsnorm":
            return None
        if not (norm_in["size"] == norm_post["size"] == mixer["hidden"] == ffn["hidden"]):
            return None
        if norm_in["weight"].dtype != norm_post["weight"].dtype:
            return None
        return {**mixer, "inter": ffn["inter"], "w_gu": ffn["w_gu"], "w_down": ffn["w_down"], "norm_in": norm_in["weight"],
                "norm_post": norm_post["weight"], "eps_in": norm_in["eps"], "eps_post": norm_post["eps"],
                "norm_dtype": norm_in["weight"].dtype}

    @staticmethod
    def _plain_rmsnorm(norm):
        """(weight, eps) of a norm that is nothing but an RMSNorm with a weight, else None."""
        describe = getattr(norm, "decode_record", None)
        record = describe() if describe is not None else None
        return (record["weight"], record["eps"]) if record and record.get("kind") == "rmsnorm" else None

    def forward(self, h, pending, ctx: StepContext, cache):
        # Few-token steps: a branch may work on the stream itself (``forward_on_stream``: its norm inside its first
        # product, its add inside its last), which saves the two norm kernels of the layer.  A part that offers no such
        # method, a norm of another kind or sizes the kernels do not take leave the branch as it is below.
        if pending is None and ctx.n_tokens <= 16:
            norm = self._plain_rmsnorm(self.input_norm)
            ok = getattr(self.mixer, "on_stream_ok", None)
            if norm is not None and ok is not None and ok(h, norm[0], ctx, cache):
                self.mixer.forward_on_stream(h, norm[0], norm[1], ctx, cache)
                norm = self._plain_rmsnorm(self.post_norm)
                ok = getattr(self.feed_forward, "on_stream_ok", None)
                if norm is not None and ok is not None and ok(h, norm[0], ctx):
                    self.feed_forward.forward_on_stream(h, norm[0], norm[1], ctx)
                    return h, None
                x = self.post_norm.forward(h, None, ctx.dtype)
                return h, self.feed_forward.forward(x, ctx)
        x = self.input_norm.forward(h, pending, ctx.dtype)
        branch = self.mixer.forward(x, ctx, cache)
        x = self.post_norm.forward(h, branch, ctx.dtype)
        return h, self.feed_forward.forward(x, ctx)


register_part("block", "pre_norm", PreNormBlock)


class ConvPreNormBlock(Block):
    """Pre-norm residual block whose sublayers read their input through a short causal convolution over time:

        a = norm_1(x);  a += conv_1(a);  x += m * mixer(a)
        b = norm_2(x);  b += conv_2(b);  x += m * feed_forward(b)            (left out for a layer without feed-forward)

    ``conv``: ``taps`` taps per channel, no bias, zeros before the sequence's start; tap ``j`` multiplies the input
    ``taps - 1 - j`` positions back.  The last ``taps - 1`` inputs of each convolution are part of a sequence's state, beside
    what the mixer keeps.  The constant ``m`` on the branches belongs to the norms, which add a pending branch into the
    stream (``delta_scale``): the norm after a branch, the next layer's first norm or the model's last.  The norms'
    results feed the convolutions in 32-bit; the convolutions hand on the run's type.
    """

    def __init__(self, width: int, norm_1: Norm, mixer: Mixer, norm_2: Norm | None, feed_forward: FeedForward | None,
                 conv_taps: int = 0, names: dict[str, str] | None = None):
        if (feed_forward is None) != (norm_2 is None):
            raise ValueError("a feed-forward comes with the norm before it, or not at all")
        self.width, self.conv_taps = int(width), int(conv_taps)
        self.norm_1, self.mixer, self.norm_2, self.feed_forward = norm_1, mixer, norm_2, feed_forward
        self.names = {"mixer": "mix.", "feed_forward": "mlp.", "conv_1": "canon1", "conv_2": "canon2", **(names or {})}
        self.conv_1 = self.conv_2 = None

    def children(self):
        parts = [("", self.norm_1), (self.names["mixer"], self.mixer)]
        if self.feed_forward is not None:
            parts += [("", self.norm_2), (self.names["feed_forward"], self.feed_forward)]
        return parts

    def _own_specs(self):
        from .base import TensorSpec

        if not self.conv_taps:
            return {}
        keys = ["conv_1"] + (["conv_2"] if self.feed_forward is not None else [])
        return {self.names[k]: TensorSpec((self.width, self.conv_taps), "matrix", init=(0.0, 0.3)) for k in keys}

    def tensor_specs(self):
        specs = {prefix + name: spec for prefix, part in self.children() for name, spec in part.tensor_specs().items()}
        specs.update(self._own_specs())
        return specs

    def load(self, tensors):
        for prefix, part in self.children():
            part.load({name: tensors[prefix + name] for name in part.tensor_specs() if prefix + name in tensors})
        if self.conv_taps:
            # [taps, width]: the kernels read tap by tap
            self.conv_1 = tensors[self.names["conv_1"]].float().t().contiguous()
            if self.feed_forward is not None:
                self.conv_2 = tensors[self.names["conv_2"]].float().t().contiguous()

    def weight_bytes(self):
        own = sum(t.numel() * t.element_size() for t in (self.conv_1, self.conv_2) if t is not None)
        return own + sum(part.weight_bytes() for _, part in self.children())

    def n_conv_states(self) -> int:
        if self.conv_taps <= 1:
            return 0
        return 2 if self.feed_forward is not None else 1

    def cache_request(self):
        request = self.mixer.cache_request()
        n_own = self.n_conv_states()
        if not n_own:
            return request
        from .base import StateRequest

        own = [StateRequest((self.conv_taps - 1, self.width), torch.float32)] * n_own
        if request is None:
            return own
        return [*request, *own] if isinstance(request, (list, tuple)) else [request, *own]

    def _normed_through_conv(self, norm, h, pending, weight, state, ctx: StepContext):
        """``norm(h + pending)`` through the convolution; one kernel where every sequence brings one token and the norm has
        that form, else the norm's kernel and the convolution's."""
        if ctx.all_single and hasattr(norm, "forward_conv_single") and F.add_layernorm_conv_single_fits(h.shape[1], weight.shape[0]):
            keep = state is not None and not ctx.extras.get("cache_read_only", False)
            return norm.forward_conv_single(h, pending, weight, state, ctx, keep)
        return self._through_conv(norm.forward(h, pending, torch.float32), weight, state, ctx)

    def _through_conv(self, a, weight, state, ctx: StepContext):
        keep = state is not None and not ctx.extras.get("cache_read_only", False)
        # one token a sequence: the convolution's kernel moves the states on itself
        g = F.causal_conv(a, weight, state, ctx.tok_pos, ctx.tok_seq, ctx.cu_q, ctx.slots, ctx.dtype,
                          update_single_token_state=keep and ctx.all_single)
        if keep and not ctx.all_single:
            F.conv_state(a, state, ctx.cu_q, ctx.slots, ctx.n_seqs)
        return g

    def forward(self, h, pending, ctx: StepContext, cache):
        states = [None, None]
        n_own = self.n_conv_states()
        if n_own:
            mixer_request = self.mixer.cache_request()
            *views, = cache
            states[:n_own] = views[len(views) - n_own:]
            views = views[:len(views) - n_own]
            cache = tuple(views) if isinstance(mixer_request, (list, tuple)) else (views[0] if views else None)
        if self.conv_taps:
            a = self._normed_through_conv(self.norm_1, h, pending, self.conv_1, states[0], ctx)
        else:
            a = self.norm_1.forward(h, pending, ctx.dtype)
        branch = self.mixer.forward(a, ctx, cache)
        if self.feed_forward is None:
            return h, branch
        if self.conv_taps:
            b = self._normed_through_conv(self.norm_2, h, branch, self.conv_2, states[1], ctx)
        else:
            b = self.norm_2.forward(h, branch, ctx.dtype)
        return h, self.feed_forward.forward(b, ctx)


register_part("block", "pre_norm_conv", ConvPreNormBlock)


class ParallelBlock(Block):
    """A layer whose two branches read ONE norm: ``n = norm(x); x += mixer(n) + feed_forward(n)`` (the feed-forward may be
    absent).  The sum of the two branches is formed in 32-bit and handed on as ``pending``, so that the add into the
    stream happens inside the next norm."""

    def __init__(self, norm: Norm, mixer: Mixer, feed_forward: FeedForward | None, names: dict[str, str] | None = None):
        self.norm, self.mixer, self.feed_forward = norm, mixer, feed_forward
        self.names = {"norm": "", "mixer": "mix.", "feed_forward": "mlp.", **(names or {})}

    def children(self):
        parts = [(self.names["norm"], self.norm), (self.names["mixer"], self.mixer)]
        if self.feed_forward is not None:
            parts.append((self.names["feed_forward"], self.feed_forward))
        return parts

    def tensor_specs(self):
        return {prefix + name: spec for prefix, part in self.children() for name, spec in part.tensor_specs().items()}

    def load(self, tensors):
        for prefix, part in self.children():
            part.load({name: tensors[prefix + name] for name in part.tensor_specs() if prefix + name in tensors})

    def weight_bytes(self):
        return sum(part.weight_bytes() for _, part in self.children())

    def forward(self, h, pending, ctx: StepContext, cache):
        x = self.norm.forward(h, pending, ctx.dtype)
        branch = self.mixer.forward(x, ctx, cache)
        if self.feed_forward is None:
            return h, branch
        added = getattr(self.feed_forward, "forward_added", None)
        if added is not None:
            return h, added(x, ctx, branch)
        return h, branch.float() + self.feed_forward.forward(x, ctx).float()


register_part("block", "parallel", ParallelBlock)


class SandwichBlock(Block):
    """A layer that norms every branch before AND after it, scales it per channel, passes the mixer's input
    through a short causal convolution over time, and mixes the results of all earlier layers into what it hands on:

        a = norm_in(x);  a += conv(a)                      (conv: ``taps`` taps per channel, zeros before the start)
        x += scale_1 * norm_out_1(mixer(a))
        x += scale_2 * norm_out_2(feed_forward(norm_mid(x)))          (left out for a layer without feed-forward)
        X_(i+1) = x;   handed on: sum_{j <= i+1} mix[j] * X_j         (X_0 the embedding output, i this layer's place)

    The last ``taps - 1`` inputs of the convolution are part of a sequence's state.  Every sum into the stream, the
    norm of the branch before it, the depth mix and the norm that reads the result are one kernel (``branch_merge``);
    the norm at the head of the NEXT layer is formed there too when the next layer is of this kind (``next_block``).
    The step keeps the streams ``X_j`` (``ctx.extras["kept_streams"]``, made by the model).
    """

    def __init__(self, width: int, place: int, norm_in: Norm, mixer: Mixer, norm_out_1: Norm, norm_mid: Norm | None,
                 feed_forward: FeedForward | None, norm_out_2: Norm | None, conv_taps: int = 0,
                 names: dict[str, str] | None = None):
        self.width, self.place, self.conv_taps = int(width), int(place), int(conv_taps)
        self.norm_in, self.mixer, self.norm_out_1 = norm_in, mixer, norm_out_1
        self.norm_mid, self.feed_forward, self.norm_out_2 = norm_mid, feed_forward, norm_out_2
        if (feed_forward is None) != (norm_mid is None) or (feed_forward is None) != (norm_out_2 is None):
            raise ValueError("a feed-forward comes with the norms before and after it, or not at all")
        self.names = {"mixer": "mix.", "feed_forward": "mlp.", "scale_1": "ls1", "scale_2": "ls2", "conv": "canon1",
                      "mix": "dwa", **(names or {})}
        self.next_block: SandwichBlock | None = None
        self.scale_1 = self.scale_2 = self.conv = self.mix = None

    def children(self):
        parts = [("", self.norm_in), (self.names["mixer"], self.mixer), ("", self.norm_out_1)]
        if self.feed_forward is not None:
            parts += [("", self.norm_mid), (self.names["feed_forward"], self.feed_forward), ("", self.norm_out_2)]
        return parts

    def _own_specs(self):
        from .base import TensorSpec

        specs = {self.names["scale_1"]: TensorSpec((self.width,), "vector", init=(1.0, 0.2)),
                 self.names["mix"]: TensorSpec((self.place + 2,), "vector", init=(0.4, 0.3))}
        if self.feed_forward is not None:
            specs[self.names["scale_2"]] = TensorSpec((self.width,), "vector", init=(1.0, 0.2))
        if self.conv_taps:
            specs[self.names["conv"]] = TensorSpec((self.width, self.conv_taps), "matrix", init=(0.0, 0.3))
        return specs

    def tensor_specs(self):
        specs = {prefix + name: spec for prefix, part in self.children() for name, spec in part.tensor_specs().items()}
        specs.update(self._own_specs())
        return specs

    def load(self, tensors):
        for prefix, part in self.children():
            part.load({name: tensors[prefix + name] for name in part.tensor_specs() if prefix + name in tensors})
        for _, part in self.children():
            if isinstance(part, Norm) and getattr(part, "weight", None) is not None:
                part.weight = part.weight.float().contiguous()  # the merging kernel multiplies by 32-bit weights
        n = self.names
        self.scale_1 = tensors[n["scale_1"]].float().contiguous()
        self.mix = tensors[n["mix"]].float().contiguous()
        if self.feed_forward is not None:
            self.scale_2 = tensors[n["scale_2"]].float().contiguous()
        if self.conv_taps:
            self.conv = tensors[n["conv"]].float().t().contiguous()  # [taps, width]: the kernels read tap by tap

    def weight_bytes(self):
        own = sum(t.numel() * t.element_size() for t in (self.scale_1, self.scale_2, self.conv, self.mix) if t is not None)
        return own + sum(part.weight_bytes() for _, part in self.children())

    def cache_request(self):
        request = self.mixer.cache_request()
        if self.conv_taps <= 1:
            return request
        from .base import StateRequest

        own = StateRequest((self.conv_taps - 1, self.width), torch.float32)
        if request is None:
            return [own]
        return [*request, own] if isinstance(request, (list, tuple)) else [request, own]

    def input_dtype(self, ctx: StepContext) -> torch.dtype:
        """What the norm at the head of the layer is wanted in: 32-bit where the convolution reads it."""
        return torch.float32 if self.conv_taps else ctx.dtype

    def forward(self, h, pending, ctx: StepContext, cache):
        if pending is not None:
            raise ValueError("a layer of this kind takes its stream whole: the layer before must not leave a branch unadded")
        kept = ctx.extras.get("kept_streams")
        if kept is None or kept.shape[0] < self.place + 2:
            raise ValueError("the model's plan must keep the streams of a step for layers that mix earlier results")
        state = None
        if self.conv_taps > 1:
            *views, state = cache
            cache = views[0] if len(views) == 1 else (tuple(views) if views else None)
        a = ctx.extras.pop("normed_input", None)
        if a is None:
            a = self.norm_in.forward(h, None, self.input_dtype(ctx))
        if self.conv_taps:
            keep = state is not None and not ctx.extras.get("cache_read_only", False)
            # one token a sequence: the convolution's kernel moves the states on itself
            g = F.causal_conv(a, self.conv, state, ctx.tok_pos, ctx.tok_seq, ctx.cu_q, ctx.slots, ctx.dtype,
                              update_single_token_state=keep and ctx.all_single)
            if keep and not ctx.all_single:
                F.conv_state(a, state, ctx.cu_q, ctx.slots, ctx.n_seqs)
        else:
            g = a
        y = self.mixer.forward(g, ctx, cache)
        # the embedding output is one of the kept streams: the first layer's sums go to a stream of their own
        stream = torch.empty_like(h) if h.data_ptr() == kept.data_ptr() else h
        follower = self.next_block
        if self.feed_forward is None:
            return self._close(h, y, self.norm_out_1, self.scale_1, kept, follower, ctx, stream), None
        _, z = F.branch_merge(h, y, self.norm_out_1.weight, self.norm_out_1.eps, self.scale_1,
                              next_weight=self.norm_mid.weight, next_eps=self.norm_mid.eps, next_dtype=ctx.dtype, x_out=stream)
        y = self.feed_forward.forward(z, ctx)
        return self._close(stream, y, self.norm_out_2, self.scale_2, kept, follower, ctx, stream), None

    def _close(self, x, y, norm, scale, kept, follower, ctx, stream):
        """The layer's last sum: the result is kept, the depth mix goes on, and the next layer's head norm is formed."""
        next_weight = next_eps = None
        next_dtype = torch.float32
        if follower is not None:
            next_weight, next_eps, next_dtype = follower.norm_in.weight, follower.norm_in.eps, follower.input_dtype(ctx)
        _, z = F.branch_merge(x, y, norm.weight, norm.eps, scale, kept=kept, n_kept=self.place + 1, mix=self.mix,
                              next_weight=next_weight, next_eps=next_eps or 0.0, next_dtype=next_dtype, x_out=stream)
        if z is not None:
            ctx.extras["normed_input"] = z
        return stream


register_part("block", "sandwich", SandwichBlock)


class OutNormBlock(Block):
    """A layer whose sublayers read the stream itself and whose results are normed before they are added:

        x += norm_1(mixer(x));   x += norm_2(feed_forward(x))            (the second left out for a layer without feed-forward)

    The stream is 32-bit; what a sublayer multiplies is the stream in the run's type.  The norm of a branch, its add into
    the stream and the copy that the next sublayer reads are one kernel; the copy for the next LAYER travels in the
    step's extras, so only the model's first layer forms one by itself."""

    def __init__(self, norm_1: Norm, mixer: Mixer, norm_2: Norm | None, feed_forward: FeedForward | None,
                 names: dict[str, str] | None = None, first: bool = False):
        """``first``: the model's first layer, which nothing hands a copy of the stream."""
        if (feed_forward is None) != (norm_2 is None):
            raise ValueError("a feed-forward comes with the norm behind it, or not at all")
        self.norm_1, self.mixer, self.norm_2, self.feed_forward = norm_1, mixer, norm_2, feed_forward
        self.first = bool(first)
        self.names = {"mixer": "mix.", "feed_forward": "mlp.", **(names or {})}

    def children(self):
        parts = [("", self.norm_1), (self.names["mixer"], self.mixer)]
        if self.feed_forward is not None:
            parts += [("", self.norm_2), (self.names["feed_forward"], self.feed_forward)]
        return parts

    def tensor_specs(self):
        return {prefix + name: spec for prefix, part in self.children() for name, spec in part.tensor_specs().items()}

    def load(self, tensors):
        for prefix, part in self.children():
            part.load({name: tensors[prefix + name] for name in part.tensor_specs() if prefix + name in tensors})
        for norm in (self.norm_1, self.norm_2):
            if norm is not None:
                norm.weight = norm.weight.float().contiguous()  # the merging kernel multiplies by 32-bit weights

    def weight_bytes(self):
        return sum(part.weight_bytes() for _, part in self.children())

    def forward(self, h, pending, ctx: StepContext, cache):
        if pending is not None:
            raise ValueError("a layer of this kind takes its stream whole: the layer before must not leave a branch unadded")
        x = ctx.extras.pop("stream_copy", None)
        if x is None or self.first:
            x = F.stream_cast(h, ctx.dtype)
        copy = None if ctx.dtype == torch.float32 else ctx.dtype  # a 32-bit run reads the stream itself
        branch = self.mixer.forward(x, ctx, cache)
        _, x = F.branch_merge(h, branch, self.norm_1.weight, self.norm_1.eps, copy_dtype=copy)
        if self.feed_forward is not None:
            branch = self.feed_forward.forward(h if x is None else x, ctx)
            _, x = F.branch_merge(h, branch, self.norm_2.weight, self.norm_2.eps, copy_dtype=copy)
        if x is not None:
            ctx.extras["stream_copy"] = x
        return h, None


register_part("block", "out_norm", OutNormBlock)
