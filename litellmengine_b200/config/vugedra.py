"""Typed configuration of the Vugedra design, read from its config.json.

The file names the design with `"architecture": "Vugedra"` and gives `vocab`, `width`, `norm.eps` and a list
`layers`.  A layer entry has `type` ('attention', 'gla' or 'latent_attention'), the sizes and constants of its mixer
under `mixer`, its feed-forward under `mlp` ({"kind": "dense", "ff": n}, {"kind": "moe", ...}, or null for a layer
without one), and optionally `weights_of: j`: the layer then has no tensors of its own and runs layer j's, with a
cache or a recurrent state of its own.  Tensors of layer i start with `l<i>.`; linear weights are [out, in].

What the design fixes, and therefore lives here and in the parts rather than in the file:
  * the norm computes no mean and no variance: tanh(alpha x) * w + b with one learned alpha ('<norm>.alpha') and a
    bias ('<norm>.b') beside the weight; a layer has one in front of each sublayer and one on its output,
    x += norm1b(mixer(norm1(x))), x += norm2b(ff(norm2(x))); the model's last norm is of the same kind;
  * 'attention' = grouped-query softmax attention with biased q/k/v, an RMS norm over a token's WHOLE q and k
    projections, a rotation of neighbouring pairs over the first `rot.dims` entries of a head with stretched
    frequencies (`rot.scaling`), a sliding window (`mask.size`) that keeps the sequence's first `mask.keep_first`
    keys, one more term exp(0) in the softmax's denominator, a sigmoid output gate per head;
  * 'gla' = gated linear attention: a decay per key channel alpha = sigmoid(z)^(1/tau) from a low-rank projection
    whose rank is the stored tensors' inner size, a per-head RMS norm of the output with one weight shared by the
    heads, a silu output gate;
  * 'latent_attention' = queries through a normed latent of `q_rank`; per token a normed latent of `kv_rank` and one
    rotated key part of `rot_dim` shared by all heads are cached; per head the unrotated key and the value are maps
    of the latent; the same rotation of neighbouring pairs on the rot_dim part; causal; a sigmoid gate per head;
  * the dense feed-forward is down(silu(gate x) * (up x)); the routed one scores its router outputs by softmax,
    chooses `top` of them by score + a stored correction, weighs them by their scores over the chosen ones' sum;
    the last `router.identity` outputs are no experts (the token's own input comes back); a shared expert
    (`mlp.shared`) runs for every token;
  * the output head is a tensor of its own.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .registry import ConfigError, register_architecture
from .specs import BlockSpec, FeedForwardSpec, MixerSpec, ModelPlan, NormSpec, PositionSpec, StageSpec
from .tobovik import _FF_NAMES, _freeze, _gla_spec, _need, _thaw

MAX_POSITION = 1 << 20        # nothing of the design is tabulated by absolute position
SINK_SCORE = 0.0              # the score of the term that joins the attention softmax's denominator without a value
YARN_MAGNITUDE = 0.1          # cos and sin are multiplied by YARN_MAGNITUDE * ln(factor) + 1

_ATTN_NAMES = (("q", "q"), ("k", "k"), ("v", "v"), ("g", "g"), ("o", "o"), ("q_bias", "q.b"), ("k_bias", "k.b"),
               ("v_bias", "v.b"), ("q_norm", "q.norm"), ("k_norm", "k.norm"))
_LATENT_NAMES = (("dq", "dq"), ("dq_norm", "dq.norm"), ("uq", "uq"), ("dkv", "dkv"), ("dkv_norm", "dkv.norm"),
                 ("uk", "uk"), ("uv", "uv"), ("g", "g"), ("o", "o"))


def _rotation(rot: Optional[Dict[str, Any]], where: str, limit: int) -> PositionSpec:
    """`rot` = {base, dims, scaling: {factor, original, fast, slow}} (scaling may be absent) as a position spec of
    kind 'rope_pairs'; no `rot`: no rotation."""
    if rot is None:
        return PositionSpec(kind="none")
    base, dims = _need(rot, "base", float, where), _need(rot, "dims", int, where)
    if dims % 2 or dims > limit or not base > 1.0:
        raise ConfigError(f"config field {where}dims must be even and at most {limit}, {where}base above 1")
    params = ()
    sc = rot.get("scaling")
    if sc is not None:
        w = where + "scaling."
        factor, original = _need(sc, "factor", float, w), _need(sc, "original", float, w)
        fast, slow = _need(sc, "fast", float, w), _need(sc, "slow", float, w)
        if not (factor > 0 and original > 0 and fast > 0 and slow > 0):
            raise ConfigError(f"config field {where}scaling: factor, original, fast and slow must be positive")
        params = (("scaling", (factor, original, fast, slow)), ("magnitude", YARN_MAGNITUDE * math.log(factor) + 1.0))
    return PositionSpec(kind="rope_pairs", theta=base, rotary_dim=dims, params=params)


def _attention_spec(m: Dict[str, Any], where: str, eps: float) -> MixerSpec:
    heads, kv = _need(m, "heads", int, where), _need(m, "kv_heads", int, where)
    if heads % kv:
        raise ConfigError(f"config field {where}heads must be a multiple of {where}kv_heads")
    dim = _need(m, "dim", int, where)
    window, keep = None, 0
    if m.get("mask") is not None:
        window = _need(m["mask"], "size", int, where + "mask.")
        k = m["mask"].get("keep_first", 0)
        if isinstance(k, bool) or not isinstance(k, int) or k < 0:
            raise ConfigError(f"config field {where}mask.keep_first must be a non-negative integer")
        keep = k
    return MixerSpec(kind="gated_attention", num_heads=heads, num_kv_heads=kv, head_dim=dim,
                     value_dim=_need(m, "vdim", int, where), qk_norm=NormSpec("rmsnorm", eps), qk_norm_scope="projection",
                     position=_rotation(m.get("rot"), where + "rot.", dim), window=window, keep_first=keep,
                     softmax_sink=SINK_SCORE, scale=_need(m, "scale", float, where), bias=True, output_gate="sigmoid",
                     output_gate_scope="head", weight_prefix="mix", tensor_names=_ATTN_NAMES)


def _latent_spec(m: Dict[str, Any], where: str, eps: float) -> MixerSpec:
    rot_dim = _need(m, "rot_dim", int, where)
    window = None if m.get("mask") is None else _need(m["mask"], "size", int, where + "mask.")
    return MixerSpec(kind="latent_attention", num_heads=_need(m, "heads", int, where), num_kv_heads=1,
                     head_dim=_need(m, "dim", int, where), value_dim=_need(m, "vdim", int, where),
                     position=_rotation(m.get("rot"), where + "rot.", rot_dim), window=window,
                     scale=_need(m, "scale", float, where), output_gate="sigmoid", output_gate_scope="head",
                     weight_prefix="mix", tensor_names=_LATENT_NAMES,
                     params=(("q_rank", _need(m, "q_rank", int, where)), ("kv_rank", _need(m, "kv_rank", int, where)),
                             ("rot_dim", rot_dim), ("eps", eps), ("keep_window", window)))


def _feed_forward_spec(mlp: Dict[str, Any], where: str) -> FeedForwardSpec:
    kind = _need(mlp, "kind", str, where)
    if kind == "dense":
        return FeedForwardSpec(kind="swiglu", intermediate_size=_need(mlp, "ff", int, where), weight_prefix="mlp",
                               tensor_names=_FF_NAMES)
    if kind != "moe":
        raise ConfigError(f"{where}kind={kind!r} is not a feed-forward of this design ('dense', 'moe')")
    router = mlp.get("router")
    experts, top = _need(router, "experts", int, where + "router."), _need(router, "top", int, where + "router.")
    identity = router.get("identity", 0)
    if isinstance(identity, bool) or not isinstance(identity, int) or identity < 0:
        raise ConfigError(f"config field {where}router.identity must be a non-negative integer")
    if top > experts + identity:
        raise ConfigError(f"config field {where}router.top exceeds the router's outputs")
    shared = None if mlp.get("shared") is None else _need(mlp["shared"], "ff", int, where + "shared.")
    return FeedForwardSpec(kind="moe", intermediate_size=_need(mlp.get("expert"), "ff", int, where + "expert."),
                           weight_prefix="mlp",
                           params=(("experts", experts), ("top", top), ("groups", None), ("route_scale", 1.0),
                                   ("score", "softmax"), ("correction", True), ("identity", identity),
                                   ("activation", "silu"), ("shared", shared), ("expert_prefix", "e")))


@register_architecture("Vugedra")
@dataclass(frozen=True)
class VugedraConfig:
    vocab: int
    width: int
    eps: float
    layers: Tuple[Any, ...]           # the file's layer entries, kept as read (nested tuples of pairs)

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "VugedraConfig":
        vocab, width = _need(d, "vocab", int, ""), _need(d, "width", int, "")
        eps = _need(d.get("norm"), "eps", float, "norm.")
        if not eps > 0:
            raise ConfigError("config field norm.eps must be positive")
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("Missing required config field: layers")
        cfg = cls(vocab=vocab, width=width, eps=eps, layers=tuple(_freeze(x) for x in layers))
        cfg.plan()                    # every other check is the plan's
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.eps}, "layers": [_thaw(x) for x in self.layers]}

    # what the engine's entry points ask of any configuration
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def torch_dtype(self) -> str:
        return "bfloat16"

    def owner_of(self, i: int) -> int:
        """The layer whose tensors layer i runs (itself, unless it says `weights_of`)."""
        layers = [_thaw(x) for x in self.layers]
        seen = set()
        while layers[i].get("weights_of") is not None:
            if i in seen:
                raise ConfigError(f"layers[{i}].weights_of runs in a circle")
            seen.add(i)
            j = layers[i]["weights_of"]
            if isinstance(j, bool) or not isinstance(j, int) or not 0 <= j < len(layers):
                raise ConfigError(f"layers[{i}].weights_of must name a layer, got {j!r}")
            i = j
        return i

    def plan(self) -> ModelPlan:
        norm = NormSpec(kind="tanh", eps=self.eps, weight_name="")
        layers = [_thaw(x) for x in self.layers]
        owners = [self.owner_of(i) for i in range(len(layers))]
        block_of, blocks = {}, []
        for i in sorted(set(owners)):
            e, where = layers[i], f"layers[{i}]."
            kind, m = _need(e, "type", str, where), e.get("mixer")
            if not isinstance(m, dict):
                raise ConfigError(f"Missing required config field: {where}mixer")
            if kind == "attention":
                mixer = _attention_spec(m, where + "mixer.", self.eps)
            elif kind == "gla":
                mixer = _gla_spec(m, where + "mixer.", "mix", self.eps)
            elif kind == "latent_attention":
                mixer = _latent_spec(m, where + "mixer.", self.eps)
            else:
                raise ConfigError(f"{where}type={kind!r} is not a mixer of this design "
                                  "('attention', 'gla', 'latent_attention')")
            ffn = None if e.get("mlp") is None else _feed_forward_spec(e["mlp"], where + "mlp.")
            block_of[i] = len(blocks)
            blocks.append(BlockSpec(arrangement="sandwich_norm", mixer=mixer, feed_forward=ffn, mixer_norm=norm,
                                    feed_forward_norm=norm, weight_prefix=f"l{i}", mixer_norm_name="norm1",
                                    feed_forward_norm_name="norm2", mixer_post_norm=norm, feed_forward_post_norm=norm,
                                    mixer_post_norm_name="norm1b", feed_forward_post_norm_name="norm2b"))
        # a layer that says `weights_of` runs its owner's mixer, feed-forward and norms: the owner's entry counts
        plan = ModelPlan(
            hidden_size=self.width, vocab_size=self.vocab, blocks=tuple(blocks),
            order=tuple(StageSpec(block=block_of[j]) for j in owners), final_norm=norm,
            tie_word_embeddings=False, max_position=MAX_POSITION, embedding_name="embed",
            final_norm_name="final.norm", output_name="head")
        plan.validate()
        return plan
