"""Typed configuration of the Komazen design, read from its config.json.

The file names the design with `"architecture": "Komazen"` and gives `vocab`, `width`, `norm.eps`,
`embedding.scale`, `postln_alpha`, `canon.taps` and a list `layers`.  A layer entry has `type` ('attention' or
'latent_attention'), the sizes and constants of its mixer under `mixer`, and its feed-forward under `mlp`
({"kind": "dense", "ff": n}, or null for a layer without one).  Tensors of layer i start with `l<i>.`; linear
weights are [out, in].

What the design fixes, and therefore lives here and in the parts rather than in the file:
  * the token's embedding row is multiplied by `embedding.scale`; there is no position vector;
  * the norm comes AFTER the sum: x <- norm1(alpha x + mixer(u)), x <- norm2(alpha x + ff(u)) with RMS norms
    (plain weight, eps inside the root) and alpha = `postln_alpha`;
  * what a sublayer reads is u = x + conv(x), a causal convolution over time on each channel with `canon.taps`
    taps (tensors `canon1`, `canon2` [width, taps], the last tap on the token itself, zeros before the
    sequence's start); the last taps - 1 rows of x are part of a request's state, per layer and sublayer;
  * 'attention' = grouped-query softmax attention over all earlier keys, no rotation: q and k RMS-normed per
    head with one weight [dim] for all heads, score = q.k * scale * temp[h] - r1[h] ln(1 + r2[h] (i - j));
  * 'latent_attention' = queries through a normed latent of `q_rank`; per token a normed latent of `kv_rank`
    and one rotated key part of `rot_dim` shared by all heads are cached; per head the unrotated key and the
    value are maps of the latent; a half-split rotation (`rot.base`, `rot.dims`) on the rot_dim part of q and
    k; a sliding window of `mask.size` keys; a sigmoid output gate per channel; with `kv_from`: j the layer has
    no latent projection and reads what layer j cached;
  * the feed-forward is down(gelu_tanh(gate u) * (up u));
  * a final RMS norm precedes the output head, which is a tensor of its own.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

from .registry import ConfigError, register_architecture
from .specs import BlockSpec, FeedForwardSpec, MixerSpec, ModelPlan, NormSpec, PositionSpec, StageSpec
from .tobovik import _freeze, _need, _thaw

MAX_POSITION = 1 << 20        # nothing of the design is tabulated by absolute position

_ATTN_NAMES = (("q", "q"), ("k", "k"), ("v", "v"), ("o", "o"), ("q_norm", "q.norm"), ("k_norm", "k.norm"),
               ("temp", "temp"), ("r1", "r1"), ("r2", "r2"))
_LATENT_NAMES = (("dq", "dq"), ("dq_norm", "dq.norm"), ("uq", "uq"), ("dkv", "dkv"), ("dkv_norm", "dkv.norm"),
                 ("uk", "uk"), ("uv", "uv"), ("g", "g"), ("o", "o"))


def _attention_spec(m: Dict[str, Any], where: str, eps: float) -> MixerSpec:
    heads, kv = _need(m, "heads", int, where), _need(m, "kv_heads", int, where)
    if heads % kv:
        raise ConfigError(f"config field {where}heads must be a multiple of {where}kv_heads")
    return MixerSpec(kind="gated_attention", num_heads=heads, num_kv_heads=kv, head_dim=_need(m, "dim", int, where),
                     value_dim=_need(m, "vdim", int, where), position=PositionSpec(kind="none"), window=None,
                     scale=_need(m, "scale", float, where), qk_norm=NormSpec(kind="rmsnorm", eps=eps),
                     qk_norm_scope="head", head_temperature=True, log_distance_bias=True, weight_prefix="mix",
                     tensor_names=_ATTN_NAMES)


def _window(m: Dict[str, Any], where: str) -> Optional[int]:
    return None if m.get("mask") is None else _need(m["mask"], "size", int, where + "mask.")


def _rotation(m: Dict[str, Any], where: str) -> Tuple[float, int]:
    rot_dim = _need(m, "rot_dim", int, where)
    rot = m.get("rot")
    base, dims = _need(rot, "base", float, where + "rot."), _need(rot, "dims", int, where + "rot.")
    if dims % 2 or dims > rot_dim or not base > 0:
        raise ConfigError(f"config field {where}rot: dims must be even and at most {where}rot_dim, base positive")
    return base, dims


def _latent_spec(m: Dict[str, Any], where: str, eps: float, keep_window: Optional[int]) -> MixerSpec:
    base, dims = _rotation(m, where)
    return MixerSpec(kind="latent_attention", num_heads=_need(m, "heads", int, where), num_kv_heads=1,
                     head_dim=_need(m, "dim", int, where), value_dim=_need(m, "vdim", int, where),
                     position=PositionSpec(kind="rope", theta=base, rotary_dim=dims), window=_window(m, where),
                     scale=_need(m, "scale", float, where), has_kv=m.get("kv_from") is None, output_gate="sigmoid",
                     weight_prefix="mix", tensor_names=_LATENT_NAMES,
                     params=(("q_rank", _need(m, "q_rank", int, where)), ("kv_rank", _need(m, "kv_rank", int, where)),
                             ("rot_dim", _need(m, "rot_dim", int, where)), ("eps", eps), ("keep_window", keep_window)))


@register_architecture("Komazen")
@dataclass(frozen=True)
class KomazenConfig:
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    alpha: float                      # the stream's weight in the sum that each norm follows
    taps: int                         # of the causal convolution in front of every sublayer
    layers: Tuple[Any, ...]           # the file's layer entries, kept as read (nested tuples of pairs)

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "KomazenConfig":
        vocab, width = _need(d, "vocab", int, ""), _need(d, "width", int, "")
        eps = _need(d.get("norm"), "eps", float, "norm.")
        if not eps > 0:
            raise ConfigError("config field norm.eps must be positive")
        scale = 1.0 if d.get("embedding") is None else _need(d["embedding"], "scale", float, "embedding.")
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("Missing required config field: layers")
        cfg = cls(vocab=vocab, width=width, eps=eps, embedding_scale=scale, alpha=_need(d, "postln_alpha", float, ""),
                  taps=_need(d.get("canon"), "taps", int, "canon."), layers=tuple(_freeze(x) for x in layers))
        cfg.plan()                    # every other check is the plan's
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
                "embedding": {"scale": self.embedding_scale}, "postln_alpha": self.alpha, "canon": {"taps": self.taps},
                "layers": [_thaw(x) for x in self.layers]}

    # what the engine's entry points ask of any configuration
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def torch_dtype(self) -> str:
        return "bfloat16"

    def _sources(self, entries: List[dict]) -> Dict[int, int]:
        """layer -> the layer whose cached latent it reads, checked."""
        out = {}
        for i, e in enumerate(entries):
            m = e.get("mixer") if isinstance(e.get("mixer"), dict) else {}
            j = m.get("kv_from")
            if e.get("type") != "latent_attention" or j is None:
                continue
            where = f"layers[{i}].mixer."
            if isinstance(j, bool) or not isinstance(j, int) or not 0 <= j < i:
                raise ConfigError(f"config field {where}kv_from must name an earlier layer")
            o = entries[j].get("mixer") if isinstance(entries[j].get("mixer"), dict) else {}
            if entries[j].get("type") != "latent_attention" or o.get("kv_from") is not None:
                raise ConfigError(f"config field {where}kv_from: layer {j} keeps no latent of its own")
            if any(m.get(k) != o.get(k) for k in ("kv_rank", "rot_dim", "rot")):
                raise ConfigError(f"config field {where}kv_from: kv_rank, rot_dim and rot must equal layer {j}'s")
            out[i] = j
        return out

    def plan(self) -> ModelPlan:
        norm = NormSpec(kind="rmsnorm", eps=self.eps, weight_name="")
        entries = [_thaw(x) for x in self.layers]
        sources = self._sources(entries)
        blocks = []
        for i, e in enumerate(entries):
            where = f"layers[{i}]."
            kind, m = _need(e, "type", str, where), e.get("mixer")
            if not isinstance(m, dict):
                raise ConfigError(f"Missing required config field: {where}mixer")
            if kind == "attention":
                mixer = _attention_spec(m, where + "mixer.", self.eps)
            elif kind == "latent_attention":
                # the pages keep what the widest window among their readers still sees
                windows = [_window(entries[k]["mixer"], f"layers[{k}].mixer.") for k in [i] + [a for a, b in sources.items() if b == i]]
                keep = None if any(w is None for w in windows) else max(windows)
                mixer = _latent_spec(m, where + "mixer.", self.eps, keep)
            else:
                raise ConfigError(f"{where}type={kind!r} is not a mixer of this design ('attention', 'latent_attention')")
            ffn = None
            if e.get("mlp") is not None:
                mlp = e["mlp"]
                if _need(mlp, "kind", str, where + "mlp.") != "dense":
                    raise ConfigError(f"{where}mlp.kind={mlp['kind']!r} is not built (only 'dense')")
                ffn = FeedForwardSpec(kind="swiglu", intermediate_size=_need(mlp, "ff", int, where + "mlp."),
                                      weight_prefix="mlp", params=(("activation", "gelu_tanh"),),
                                      tensor_names=(("gate", "gate"), ("up", "up"), ("down", "down")))
            blocks.append(BlockSpec(arrangement="post_norm", mixer=mixer, feed_forward=ffn, mixer_norm=norm,
                                    feed_forward_norm=norm, weight_prefix=f"l{i}", mixer_norm_name="norm1",
                                    feed_forward_norm_name="norm2", residual_scale=self.alpha, input_conv=self.taps,
                                    input_conv_names=("canon1", "canon2")))
        plan = ModelPlan(
            hidden_size=self.width, vocab_size=self.vocab, blocks=tuple(blocks),
            order=tuple(StageSpec(block=i, cache_from=sources.get(i)) for i in range(len(blocks))), final_norm=norm,
            tie_word_embeddings=False, max_position=MAX_POSITION, embedding_name="embed",
            final_norm_name="final.norm", output_name="head", embedding_scale=self.embedding_scale)
        plan.validate()
        return plan
