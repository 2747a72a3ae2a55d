"""A layer put together from its parts, and the arrangements that wire them."""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from ..config.specs import BlockSpec
from ..weights.loader import ParamSpec
from .context import StageContext
from .registry import lookup, register_arrangement


class StreamConnection:
    """One sublayer's connection to the S residual streams of a model that keeps several: `inp` [S] weighs the
    streams into the sublayer's input, and after the sublayer x_t <- sum_s mix[s, t] x_s + out[t] * y for all t
    at once (`mix` is indexed [from, to])."""

    def __init__(self, streams: int):
        self.streams = streams
        self.inp = self.out = self.mix = None

    def parameters(self) -> Dict[str, ParamSpec]:
        S = self.streams
        lone = S == 1          # one stream may come without connection tensors: it is then the plain residual stream
        return {"in": ParamSpec((S,), role="scale", init=("one_plus_normal", 0.1), optional=lone),
                "out": ParamSpec((S,), role="scale", init=("one_plus_normal", 0.1), optional=lone),
                "mix": ParamSpec((S, S), role="scale", init=("normal", 0.5), optional=lone)}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        # an absent tensor stays None, which the streams' kernel reads as ones (in, out) or the identity (mix)
        self.inp, self.out, self.mix = (tensors[k].contiguous() if k in tensors else None for k in ("in", "out", "mix"))


class PendingUpdate:
    """A sublayer's output that has not joined the streams yet, with the coefficients it joins them by: the
    kernel that norms the next sublayer's input applies it on the way."""

    def __init__(self, y, connection: StreamConnection):
        self.y, self.connection = y, connection


def _stream_y(y):
    from ..csrc import ops
    return ops.as_tensor(y) if isinstance(y, ops.PartialSum) and y.rounds_to is not None else y


def streams_norm(streams: torch.Tensor, pending: Optional[PendingUpdate], inp: Optional[torch.Tensor], norm,
                 out_dtype: torch.dtype, rows: Optional[torch.Tensor] = None, fan: bool = False) -> torch.Tensor:
    """Apply the pending update (if any), then `norm` of sum_t inp[t] x_t (inp None: the sum of the streams, what
    a model's final norm reads) for all rows or for `rows`.  `fan`: the streams are still one (the embedding, in
    streams[0]) and are written out to their places on the way."""
    from ..csrc import ops
    c = pending.connection if pending is not None else None
    return ops.stream_norm(streams, _stream_y(pending.y) if pending is not None else None,
                           c.mix if c is not None else None, c.out if c is not None else None, inp, norm.weight,
                           norm.eps, getattr(norm, "center", False), out_dtype, rows=rows, fan=fan)


class InputConvolution:
    """What a sublayer reads instead of the stream x itself: u_t = x_t + sum_j w[:, j] * x_(t - taps + 1 + j), a causal
    convolution over time on each channel (`w` [hidden, taps], the last tap on the token itself, zeros before the
    sequence's start), in 32-bit, stored in the compute dtype.  The last taps - 1 rows of x are kept per request."""

    def __init__(self, hidden_size: int, taps: int):
        if taps < 1:
            raise ValueError("an input convolution needs at least one tap")
        self.hidden, self.taps = hidden_size, taps
        self.weight: Optional[torch.Tensor] = None

    def parameters(self) -> Dict[str, ParamSpec]:
        return {"": ParamSpec((self.hidden, self.taps), role="scale", init=("normal", 0.2))}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors[""].contiguous()

    def forward(self, x: torch.Tensor, kept: Optional[torch.Tensor], batch, out_dtype: torch.dtype) -> torch.Tensor:
        from ..csrc import ops
        return ops.short_conv(x, self.weight, kept, batch, out_dtype)


class Block:
    """Holds one layer's mixer, feed-forward and norms, each chosen by the layer's spec."""

    STATE_NAME = "block"          # the name of the state a layer's arrangement keeps per request, beside its mixer's

    def __init__(self, spec: BlockSpec, hidden_size: int, compute_dtype: torch.dtype, device):
        self.spec = spec
        self.dtype = compute_dtype
        self.mixer_norm = lookup("norm", spec.mixer_norm.kind)(spec.mixer_norm, hidden_size)
        self.feed_forward_norm = lookup("norm", spec.feed_forward_norm.kind)(spec.feed_forward_norm, hidden_size)
        self.mixer = lookup("mixer", spec.mixer.kind)(spec.mixer, hidden_size, compute_dtype, device)
        # a layer may be its mixer only: then it has no feed-forward and no norm for one
        self.feed_forward = None
        if spec.feed_forward is not None:
            self.feed_forward = lookup("feed_forward", spec.feed_forward.kind)(
                spec.feed_forward, hidden_size, compute_dtype, device)
        else:
            self.feed_forward_norm = None
        # norms on the sublayers' outputs, for arrangements that have them beside the ones in front
        self.mixer_post_norm = self.feed_forward_post_norm = None
        if getattr(spec, "mixer_post_norm", None) is not None:
            self.mixer_post_norm = lookup("norm", spec.mixer_post_norm.kind)(spec.mixer_post_norm, hidden_size)
        if getattr(spec, "feed_forward_post_norm", None) is not None and spec.feed_forward is not None:
            self.feed_forward_post_norm = lookup("norm", spec.feed_forward_post_norm.kind)(spec.feed_forward_post_norm, hidden_size)
        self.arrangement = lookup("arrangement", spec.arrangement)
        # a model with several residual streams: one connection per sublayer
        self.connections = None
        if spec.connections is not None:
            n = spec.connections[0]
            self.connections = (StreamConnection(n), StreamConnection(n) if self.feed_forward is not None else None)
        # a causal convolution over time in front of each sublayer
        self.input_convs = None
        taps = getattr(spec, "input_conv", None)
        if taps is not None:
            self.input_convs = (InputConvolution(hidden_size, taps),
                                InputConvolution(hidden_size, taps) if self.feed_forward is not None else None)
        self.residual_scale = float(getattr(spec, "residual_scale", 1.0))
        self.hidden = hidden_size

    def state_need(self):
        """What the layer keeps per request beside its mixer's cache: the last taps - 1 rows of the stream in front of
        each sublayer that reads it through a convolution, [sublayers, taps - 1, hidden] float32 (ring rows by
        position); None without a convolution or with a single tap."""
        from ..cache import StateNeed
        if self.input_convs is None or self.input_convs[0].taps < 2:
            return None
        subs = 2 if self.feed_forward is not None else 1
        return StateNeed((subs, self.input_convs[0].taps - 1, self.hidden), "float32", name=self.STATE_NAME)

    def _children(self):
        s = self.spec
        out = [(s.mixer_norm_name, self.mixer_norm), (s.mixer.weight_prefix, self.mixer)]
        if self.feed_forward is not None:
            out += [(s.feed_forward_norm_name, self.feed_forward_norm), (s.feed_forward.weight_prefix, self.feed_forward)]
        if self.mixer_post_norm is not None:
            out.append((s.mixer_post_norm_name, self.mixer_post_norm))
        if self.feed_forward_post_norm is not None:
            out.append((s.feed_forward_post_norm_name, self.feed_forward_post_norm))
        if self.connections is not None:
            out += [(name, c) for name, c in zip(s.connections[1:], self.connections) if c is not None]
        if self.input_convs is not None:
            out += [(name, c) for name, c in zip(s.input_conv_names, self.input_convs) if c is not None]
        return out

    def parts(self):
        """The parts that may offer a prelude, a graph variant or weights to count."""
        return [p for p in (self.mixer, self.feed_forward) if p is not None]

    def parameters(self) -> Dict[str, ParamSpec]:
        out = {}
        for prefix, part in self._children():
            for name, p in part.parameters().items():
                out[f"{prefix}.{name}" if name else prefix] = p      # '' : the tensor is named like the part
        return out

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        for prefix, part in self._children():
            mine = {n[len(prefix) + 1:]: t for n, t in tensors.items() if n.startswith(prefix + ".")}
            if prefix in tensors and "" in part.parameters():
                mine[""] = tensors[prefix]
            part.load({n: t for n, t in mine.items() if n in part.parameters()})

    def forward(self, h: torch.Tensor, delta: Optional[torch.Tensor], ctx: StageContext
                ) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        return self.arrangement(self, h, delta, ctx)


@register_arrangement("pre_norm")
def pre_norm(block: Block, h: torch.Tensor, delta: Optional[torch.Tensor], ctx: StageContext):
    """h += mixer(norm1(h)); h += ffn(norm2(h))  (src/model/qwen3.cpp:948-968).

    `h` is the float32 residual stream; `delta` is the previous layer's feed-forward output
    that has not been added yet (None if nothing is pending).  Each add is fused into the norm
    that follows it, so the layer returns its own feed-forward output as the next pending delta,
    unless the part added it to `h` itself (in the epilogue of its last product).
    """
    from ..csrc import ops
    if not getattr(block.mixer_norm, "accepts_partials", False):
        delta = ops.as_tensor(delta)
    x = block.mixer_norm.forward(h, block.dtype, delta=delta, write_sum=delta is not None)
    ctx.partials_ok = getattr(block.feed_forward_norm, "accepts_partials", False)
    ctx.residual = h                                            # a part may add its result here itself and return None
    a = block.mixer.forward(x, ctx)
    if block.feed_forward is None:                              # a layer that is its mixer only: its output is what is pending
        return h, a
    y = block.feed_forward_norm.forward(h, block.dtype, delta=a, write_sum=a is not None)
    extra = {}
    if getattr(block.feed_forward, "supports_partials", False):
        extra["partials_ok"] = True                             # the next norm (or `pre_norm` above) adds the splits
    if getattr(block.feed_forward, "supports_residual", False):
        extra["residual"] = h
    f = block.feed_forward.forward(y, **extra)
    return h, f


@register_arrangement("branch_norm")
def branch_norm(block: Block, h: torch.Tensor, delta: Optional[torch.Tensor], ctx: StageContext):
    """h += norm1(mixer(h)); h += norm2(ffn(h)): the norms sit on the sublayers' outputs and the
    sublayers read the stream itself.

    `h` is the float32 residual stream and is complete on entry and on return (nothing is pending, so
    `delta` passes through as None).  A sublayer's products want their input in the compute dtype: the
    kernel that adds a normed output to the stream also writes the new stream in that dtype, and hands
    it to the next sublayer, across layers too, through `batch.tables["stream_copy"]` (a pair of the
    stream it is a copy of and the copy); the first layer of a model finds there what the embedding
    kernel wrote.  In the float32 mode the stream is its own copy.
    """
    from ..csrc import ops
    if delta is not None:
        ops.residual_add(h, ops.as_tensor(delta))
    tables = ctx.batch.tables
    narrow = None if block.dtype == torch.float32 else block.dtype
    held = tables.pop("stream_copy", None)
    if narrow is None:
        x = h
    elif held is not None and held[0] is h:
        x = held[1]
    else:
        x = h.to(narrow)
    ctx.partials_ok = True                                      # the norm kernel adds a product's k-splits as it reads
    ctx.residual = None                                         # the norm stands between the product and the stream
    a = block.mixer.forward(x, ctx)
    x = block.mixer_norm.add_normed(h, a, narrow)
    if block.feed_forward is not None:
        extra = {"partials_ok": True} if getattr(block.feed_forward, "supports_partials", False) else {}
        f = block.feed_forward.forward(x if narrow is not None else h, **extra)
        x = block.feed_forward_norm.add_normed(h, f, narrow)
    if narrow is not None:
        tables["stream_copy"] = (h, x)
    return h, None


@register_arrangement("sandwich_norm")
def sandwich_norm(block: Block, h: torch.Tensor, delta, ctx: StageContext):
    """h += norm1b(mixer(norm1(h))); h += norm2b(ffn(norm2(h))): a norm in front of every sublayer and one on its
    output.  `h` is the float32 residual stream; a sublayer's output does not join it when the sublayer returns: it
    travels on (across layers too) as a `PendingNormed` with the norm of its way, and the kernel that makes the next
    sublayer's normed input adds it as it reads.  The norms must take a `PendingNormed` as their `delta`."""
    from .norms import PendingNormed
    x = block.mixer_norm.forward(h, block.dtype, delta=delta, write_sum=delta is not None)
    ctx.partials_ok = True                                      # the norm kernel adds a product's k-splits as it reads
    ctx.residual = None                                         # a norm stands between the product and the stream
    pending = PendingNormed(block.mixer.forward(x, ctx), block.mixer_post_norm)
    if block.feed_forward is not None:
        x = block.feed_forward_norm.forward(h, block.dtype, delta=pending, write_sum=True)
        extra = {"partials_ok": True} if getattr(block.feed_forward, "supports_partials", False) else {}
        pending = PendingNormed(block.feed_forward.forward(x, **extra), block.feed_forward_post_norm)
    return h, pending


@register_arrangement("post_norm")
def post_norm(block: Block, h: torch.Tensor, delta: Optional[torch.Tensor], ctx: StageContext):
    """h <- norm1(a * h + mixer(u(h))); h <- norm2(a * h + ffn(u(h))) with a = the layer's `residual_scale`: the norm
    follows the sum and the sublayers read the stream itself, through the layer's input convolution if it has one
    (u = h + conv(h), else u = h).  `h` is the float32 residual stream, complete on entry and on return.  The kernel
    of the norm also keeps the rows the convolution will want in the request's next step."""
    from ..csrc import ops
    if delta is not None:
        ops.residual_add(h, ops.as_tensor(delta))
    b, kept = ctx.batch, ctx.block_state

    def read(sub: int):
        if block.input_convs is not None:
            return block.input_convs[sub].forward(h, kept[:, sub] if kept is not None else None, b, block.dtype)
        return h if block.dtype == torch.float32 else h.to(block.dtype)

    ctx.partials_ok = True                                      # the norm kernel adds a product's k-splits as it reads
    ctx.residual = None                                         # the norm stands between the product and the stream
    a = block.mixer.forward(read(0), ctx)
    ops.scaled_add_norm(h, a, block.mixer_norm.weight, block.residual_scale, block.mixer_norm.eps,
                        kept[:, 0] if kept is not None else None, b)
    if block.feed_forward is not None:
        extra = {"partials_ok": True} if getattr(block.feed_forward, "supports_partials", False) else {}
        f = block.feed_forward.forward(read(1), **extra)
        ops.scaled_add_norm(h, f, block.feed_forward_norm.weight, block.residual_scale, block.feed_forward_norm.eps,
                            kept[:, 1] if kept is not None else None, b)
    return h, None


@register_arrangement("hyper_pre_norm")
def hyper_pre_norm(block: Block, h: torch.Tensor, delta, ctx: StageContext):
    """The pre-norm layer over S residual streams (`h`: float32 [S, T, hidden]).  For each sublayer with its
    `StreamConnection` c: u = sum_s c.inp[s] x_s; y = sublayer(norm(u)); x_t <- sum_s c.mix[s, t] x_s + c.out[t] y.
    The update is not applied when the sublayer returns: it travels on as a `PendingUpdate` (across layers too)
    and the kernel that makes the next sublayer's normed input applies it as it reads the streams."""
    c1, c2 = block.connections
    # nothing pending: the model's first layer, whose streams are still the embedding in h[0]
    x = streams_norm(h, delta, c1.inp, block.mixer_norm, block.dtype, fan=delta is None)
    ctx.partials_ok = True                                      # the streams' kernel adds a product's k-splits as it reads
    ctx.residual = None
    pending = PendingUpdate(block.mixer.forward(x, ctx), c1)
    if block.feed_forward is not None:
        x = streams_norm(h, pending, c2.inp, block.feed_forward_norm, block.dtype)
        extra = {"partials_ok": True} if getattr(block.feed_forward, "supports_partials", False) else {}
        pending = PendingUpdate(block.feed_forward.forward(x, **extra), c2)
    return h, pending
