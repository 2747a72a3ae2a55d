"""Typed descriptions of the parts a model is assembled from.

A model is data: a list of distinct layers (`BlockSpec`), each naming its
mixer, feed-forward, norms and position encoding with every size and constant
as a field, and an `order` list saying which layer runs when.  Nothing here
knows about a particular architecture; an architecture's config class turns its
own config.json keys into a `ModelPlan` (see `config/qwen3.py`).

The reference hard-wires one arrangement (src/model/qwen3.cpp:841-1059) and one
set of sizes for all layers (src/model/qwen3.cpp:1067-1071); here the same
arrangement is one value of `BlockSpec.arrangement`.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple


@dataclass(frozen=True)
class NormSpec:
    """A normalisation over the last dimension.  kind 'rmsnorm': x*rsqrt(mean(x^2)+eps)*w.
    `weight_name` is the local name of its weight tensor ('' when the tensor is named like the norm
    itself, e.g. 'l0.norm1' instead of 'l0.norm1.weight')."""
    kind: str
    eps: float
    weight_name: str = "weight"
    # kind 'layernorm': (x - mean) * rsqrt(mean((x - mean)^2) + eps) * w, a weight and no bias.
    # kind 'tanh': tanh(alpha * x) * w + b elementwise, no mean and no variance; tensors '<weight>', 'alpha' [], 'b'.


@dataclass(frozen=True)
class PositionSpec:
    """How a mixer encodes token positions.

    kind 'rope': half-split rotation of pairs (i, i+rotary_dim/2) by the angle
    position * theta**(-2i/rotary_dim).  kind 'none': no encoding.  kind 'sinusoid_added' (a model's
    `embedding_position`, not a mixer's): the vector with entry 2i = sin(p * theta**(-2i/width)) and
    entry 2i+1 = cos of the same angle is added to the token's embedding.
    kind 'rope_pairs': the rotation of NEIGHBOURING pairs (2i, 2i+1) of the first rotary_dim entries by the angle
    position * f_i, f_i = theta**(-2i/rotary_dim); `params` scaling = (factor, original, fast, slow) stretches the
    frequencies: with pair(t) = rotary_dim * ln(original / (2 pi t)) / (2 ln theta), lo = max(floor(pair(fast)), 0),
    hi = min(ceil(pair(slow)), rotary_dim - 1) and ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), the frequency
    is f_i / factor * ramp_i + f_i * (1 - ramp_i); `params` magnitude multiplies cos and sin.
    `params` carries what other kinds need.
    """
    kind: str
    theta: float = 10000.0
    rotary_dim: int = 0
    params: Tuple[Tuple[str, Any], ...] = ()


@dataclass(frozen=True)
class MixerSpec:
    """The token-mixing part of a layer.

    kind 'attention': grouped-query causal attention over the paged cache.
    `window` = None attends to every earlier key; an integer w attends to the
    last w keys (the query's own included).  `has_kv` = False makes a mixer that
    projects only queries and reads the keys and values another stage wrote (the
    stage that runs it must then name that stage in `cache_from`).  `params`
    carries what other kinds of mixer need.

    kind 'gated_attention': the same attention with more of it configurable: values of their own width
    (`value_dim`), biases on the q/k/v projections (`bias`), the q/k norm per head or over a token's whole
    projection (`qk_norm_scope` 'head' | 'projection'), a query temperature (`query_temperature` = (coef,
    every): q *= 1 + coef * ln(floor((p+1)/every) + 1)), an output gate on the concatenated heads
    (`output_gate` 'sigmoid': times sigmoid(W_g x)).
    kind 'gla': gated linear attention, a recurrent state [head_dim, value_dim] per head with a decay per
    key channel; `params`: tau (alpha = sigmoid(z)^(1/tau)), rank (of the low-rank decay projection; None:
    taken from the stored tensor).
    kind 'parallel': the mixers in `branches` side by side on the same input, their results added with
    the weights `branch_scales`.
    `output_gate_scope` 'channel': one gate value per output channel (W_g is [heads * value_dim, hidden]);
    'head': one per head (W_g is [heads, hidden]).  `distance_bias` = (rows, far): a learned table
    [rows, heads] is added to the scaled scores, its row chosen by the distance n = i - j between query and
    key: n itself below rows/2, then logarithmic steps that reach the last row at n = far.
    kind 'retention': linear attention with one fixed decay per head (`params`: decay, a tuple of one number
    per head; eps of the per-head output norm), a rotation on q and k (`position`), keys scaled by
    head_dim^-1/2, a weightless per-head RMS norm of the output and a silu gate.
    kind 'mlstm': a matrix memory with exponential input and forget gates, a normaliser vector and a
    running maximum per head (`params`: gate_cap, eps).
    `tensor_names` renames a mixer's tensors: pairs (the mixer's own name for a tensor, its name in the
    model's files, without the mixer's prefix).
    `head_temperature`: a learned number per query head (tensor 'temp' [heads]) multiplies the scaled score.
    `log_distance_bias`: r1[h] * ln(1 + r2[h] * (i - j)) is taken off the score of query i and key j, with two
    learned numbers per query head (tensors 'r1', 'r2' [heads]); unlike `distance_bias` it has no farthest row.
    kind 'latent_attention': softmax attention whose keys and values are made from a cached latent: queries
    through a normed low-rank latent (`params`: q_rank), per token one normed latent of `params` kv_rank entries
    and one rotated key part of `params` rot_dim entries shared by all heads go to the pages; per head the
    unrotated key (`head_dim` entries) and the value (`value_dim`) are linear maps of the latent; `position`
    rotates the rot_dim part of queries and keys; `window`, `scale`, `output_gate` as for attention; `params`
    eps (of the two latent norms), keep_window (the pages keep so many positions: the widest window among the
    stages that read them; None: all).  With `has_kv` False the mixer has no latent projection of its own and
    reads the pages of the stage named by `cache_from`.
    """
    kind: str
    num_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0
    qk_norm: Optional[NormSpec] = None
    position: PositionSpec = PositionSpec(kind="none")
    window: Optional[int] = None
    scale: Optional[float] = None          # None = 1/sqrt(head_dim)
    has_kv: bool = True
    weight_prefix: str = "self_attn"
    params: Tuple[Tuple[str, Any], ...] = ()
    value_dim: Optional[int] = None        # None = head_dim
    bias: bool = False
    qk_norm_scope: str = "head"
    query_temperature: Optional[Tuple[float, int]] = None
    output_gate: Optional[str] = None
    branches: Tuple["MixerSpec", ...] = ()
    branch_scales: Tuple[float, ...] = ()
    tensor_names: Tuple[Tuple[str, str], ...] = ()
    output_gate_scope: str = "channel"
    distance_bias: Optional[Tuple[int, float]] = None
    head_temperature: bool = False
    log_distance_bias: bool = False
    keep_first: int = 0                    # with a window: the sequence's first so many keys stay visible to every later query
    softmax_sink: Optional[float] = None   # a score whose exponential joins the softmax's denominator and carries no value


@dataclass(frozen=True)
class FeedForwardSpec:
    """The per-token part of a layer.  kind 'swiglu': down(act(gate(x)) * up(x)) with act = silu, or what
    `params` activation names ('silu', 'gelu_tanh': 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))).
    kind 'moe': routed experts; `intermediate_size` is one expert's, `params`: experts, top, groups
    (count, keep) or None, route_scale, limit (the experts' clamp), expert_prefix (expert e's tensors are
    '<expert_prefix><e>.gate' and so on).
    `tensor_names`: pairs (the part's own name for a tensor, its name in the model's files)."""
    kind: str
    intermediate_size: int = 0
    weight_prefix: str = "mlp"
    params: Tuple[Tuple[str, Any], ...] = ()
    tensor_names: Tuple[Tuple[str, str], ...] = ()


@dataclass(frozen=True)
class BlockSpec:
    """One layer: which parts it has and how they are wired.

    arrangement 'pre_norm': h += mixer(norm1(h)); h += ffn(norm2(h)).
    arrangement 'branch_norm': h += norm1(mixer(h)); h += norm2(ffn(h)): the norms sit on the sublayers'
    outputs, and the sublayers read the stream itself.
    arrangement 'hyper_pre_norm': the pre-norm layer over `streams` copies of the residual stream (see
    `connections`).
    arrangement 'post_norm': h <- norm1(residual_scale * h + mixer(u(h))); h <- norm2(residual_scale * h + ffn(u(h))):
    the norm comes after the sum and the sublayers read the stream itself, or, with `input_conv` = taps, the stream
    plus its causal convolution over time, channel by channel: u_t = h_t + sum_j w[:, j] * h_(t - taps + 1 + j) with
    zeros before the sequence's start (tensors `input_conv_names`, one [hidden, taps] per sublayer; the last taps - 1
    rows of h are kept per request, layer and sublayer).
    arrangement 'sandwich_norm': h += norm1b(mixer(norm1(h))); h += norm2b(ffn(norm2(h))): a norm in front of each
    sublayer and one on its output (`mixer_post_norm`, `feed_forward_post_norm`, named `mixer_post_norm_name` and
    `feed_forward_post_norm_name`).
    `feed_forward` None: a layer that is its mixer only.
    `connections` = (streams, name of the mixer's connection tensors, name of the feed-forward's): each
    sublayer has tensors `<name>.in` [streams], `<name>.out` [streams], `<name>.mix` [streams, streams]; its
    input is sum_s in[s] x_s and afterwards x_t <- sum_s mix[s, t] x_s + out[t] * y for all t at once.
    """
    arrangement: str
    mixer: MixerSpec
    feed_forward: Optional[FeedForwardSpec]
    mixer_norm: NormSpec
    feed_forward_norm: NormSpec
    weight_prefix: str = ""
    mixer_norm_name: str = "input_layernorm"
    feed_forward_norm_name: str = "post_attention_layernorm"
    connections: Optional[Tuple[int, str, str]] = None
    residual_scale: float = 1.0
    input_conv: Optional[int] = None
    input_conv_names: Tuple[str, str] = ("conv1", "conv2")
    mixer_post_norm: Optional[NormSpec] = None
    feed_forward_post_norm: Optional[NormSpec] = None
    mixer_post_norm_name: str = "post_mixer_layernorm"
    feed_forward_post_norm_name: str = "post_feed_forward_layernorm"


@dataclass(frozen=True)
class StageSpec:
    """One entry of the run order: which layer runs, and whose cache it uses.

    A layer named by two stages shares its weights between them, but each stage
    has a cache (or state) of its own, unless `cache_from` names an EARLIER stage
    (by its index in the order) whose cache this stage reads without writing.
    """
    block: int
    cache_from: Optional[int] = None


@dataclass(frozen=True)
class ModelPlan:
    """Everything needed to build a model: sizes, layers, their order, names."""
    hidden_size: int
    vocab_size: int
    blocks: Tuple[BlockSpec, ...]
    order: Tuple[StageSpec, ...]            # the layers in the order they run; may repeat
    final_norm: NormSpec
    tie_word_embeddings: bool
    max_position: int
    embedding_name: str = "model.embed_tokens.weight"
    final_norm_name: str = "model.norm.weight"
    output_name: str = "lm_head.weight"
    embedding_position: Optional[PositionSpec] = None     # an encoding added to the embeddings themselves
    embedding_scale: float = 1.0                          # the token's row is multiplied by this (in 32-bit)
    streams: int = 0                                      # > 0: the layers keep so many copies of the residual stream
                                                          # (equal at the start, summed before the final norm)

    def validate(self) -> None:
        if self.hidden_size <= 0 or self.vocab_size <= 0:
            raise ValueError("hidden_size and vocab_size must be positive")
        if not self.blocks:
            raise ValueError("a model needs at least one layer")
        if not self.order:
            raise ValueError("the run order is empty")
        for s, st in enumerate(self.order):
            if not 0 <= st.block < len(self.blocks):
                raise ValueError(f"stage {s} names layer {st.block}, but there are {len(self.blocks)} layers")
            mixer = self.blocks[st.block].mixer
            conn = self.blocks[st.block].connections
            if (conn[0] if conn else 0) != self.streams:
                raise ValueError(f"stage {s}: the layer's connections do not fit the model's {self.streams} streams")
            if st.cache_from is not None:
                if not 0 <= st.cache_from < s:
                    raise ValueError(f"stage {s}: cache_from={st.cache_from} is not an earlier stage")
                if self.order[st.cache_from].cache_from is not None:
                    raise ValueError(f"stage {s}: cache_from={st.cache_from} itself borrows a cache")
            elif not mixer.has_kv:
                raise ValueError(f"stage {s}: its mixer writes no keys and values, so cache_from must be set")
