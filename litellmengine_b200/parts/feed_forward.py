"""Feed-forward parts."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..config.specs import FeedForwardSpec
from ..csrc import ops
from ..weights.loader import ParamSpec
from .registry import register_feed_forward


@register_feed_forward("swiglu")
class SwiGLU:
    """down(act(gate(x)) * up(x)), no biases, act = silu (src/model/qwen3.cpp:143-152,
    src/ops/silu_and_mul.cu:44-46) or what the spec's `params` name as `activation` ('gelu_tanh').  Gate and up are
    one fused product [g | u]."""

    graph_safe = True          # forward only launches kernels on the current stream
    any_division_safe = True   # and nothing in it is shaped by the number of entries of the step

    def __init__(self, spec: FeedForwardSpec, hidden_size: int, compute_dtype: torch.dtype, device):
        if spec.intermediate_size <= 0:
            raise ValueError("intermediate_size must be positive")
        self.hidden, self.inter, self.dtype = hidden_size, spec.intermediate_size, compute_dtype
        names = dict(getattr(spec, "tensor_names", ()))
        self._gate, self._up, self._down = (names.get("gate", "gate_proj.weight"), names.get("up", "up_proj.weight"),
                                            names.get("down", "down_proj.weight"))
        self.activation = dict(getattr(spec, "params", ())).get("activation", "silu")
        if self.activation not in ops.ACTIVATIONS:
            raise ValueError(f"activation {self.activation!r}: one of {sorted(ops.ACTIVATIONS)}")
        self.w_gate_up: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None

    def parameters(self) -> Dict[str, ParamSpec]:
        return {self._gate: ParamSpec((self.inter, self.hidden)),
                self._up: ParamSpec((self.inter, self.hidden)),
                self._down: ParamSpec((self.hidden, self.inter))}

    def load(self, t: Dict[str, torch.Tensor]) -> None:
        g, u = t[self._gate], t[self._up]
        dt = torch.float32 if torch.float32 in (g.dtype, u.dtype) else g.dtype
        self.w_gate_up = torch.cat([g.to(dt), u.to(dt)], dim=0).contiguous()
        self.w_down = t[self._down].contiguous()
        ops.prepare_streaming(self.w_gate_up)       # a tiled copy for decode steps (bfloat16 on a GPU only)
        ops.prepare_streaming(self.w_down)

    supports_partials = True   # forward(x, partials_ok=True) may return an ops.PartialSum
    supports_residual = True   # forward(x, residual=h) may add its result to h itself and return None

    def forward(self, x: torch.Tensor, partials_ok: bool = False, residual: Optional[torch.Tensor] = None):
        act = ops.linear_silu_mul(x, self.w_gate_up, self.dtype, self.activation)
        if residual is not None and ops.linear_into(act, self.w_down, residual):
            return None                                                               # joined the residual in the product
        return ops.linear(act, self.w_down, out_dtype=torch.float32, partials_ok=partials_ok)


@register_feed_forward("moe")
class RoutedExperts:
    """A mixture of experts.  Router: scores s = sigmoid(W_r x) in 32-bit; experts form groups of neighbours, a
    group's score is the sum of its two largest scores, and the `top` largest scores among the experts of the
    `keep` best groups are chosen; their weights are s / (sum of the chosen s + 1e-20) * route_scale.  Expert:
    down(g * sigmoid(1.702 g) * (u + 1)) with g = min(gate x, limit), u = clamp(up x, -limit, limit), no biases.
    The result is the weighted sum of the chosen experts' outputs.

    The experts' [gate; up] matrices are stacked into one and their down matrices stand side by side along the
    input axis.  Three ways to run, chosen by the step's size; all give the same sums up to rounding.
    Prompt portions in bfloat16: the (token, choice) pairs are sorted by expert and each expert's rows go through
    its own matrices in the library's grouped matrix product (exactly the chosen experts' flops).  Steps whose
    pairs are fewer than the experts (decode steps of a model with many experts): two kernels that read only the
    chosen experts' matrices.  Otherwise (decode steps that touch most experts anyway; the 32-bit mode): one
    product gives every expert's gate and up values, the activation kernel multiplies each expert's activations
    by the token's weight for it (zero for experts that were not chosen) and ONE down product adds the chosen
    experts' outputs up.

    Options of the spec's `params`: `score` 'sigmoid' (above) or 'softmax' (over all router outputs); `correction`:
    a stored vector (tensor 'correction') is added to the scores for the CHOICE only, the weights are made of the
    scores themselves; `identity` = n: the router has n more outputs than experts, and a token that picks one of
    them gets its own input back times the weight; `activation` 'silu': an expert is down(silu(gate x) * (up x))
    without clamps; `shared` = ff: one more gated feed-forward of that size (tensors 'shared.gate', 'shared.up',
    'shared.down', the routed experts' activation) runs for every token and is added."""

    graph_safe = True
    any_division_safe = True
    supports_partials = True
    ACT_ALPHA = 1.702
    SORTED_FROM = 32           # steps of more tokens than the weight-streaming product takes sort their tokens by expert

    def __init__(self, spec: FeedForwardSpec, hidden_size: int, compute_dtype: torch.dtype, device):
        p = dict(spec.params)
        self.hidden, self.ff, self.dtype = hidden_size, spec.intermediate_size, compute_dtype
        self.E, self.top = int(p["experts"]), int(p["top"])
        self.groups = tuple(p["groups"]) if p.get("groups") else None
        self.route_scale = float(p.get("route_scale", 1.0))
        # the experts' activation as (clamp, slope inside the sigmoid, what is added to the up value)
        self.activation = p.get("activation", "clamped_swish")
        if self.activation == "clamped_swish":
            self.limit, self.act_alpha, self.act_shift = float(p["limit"]), self.ACT_ALPHA, 1.0
        elif self.activation == "silu":
            self.limit, self.act_alpha, self.act_shift = float("inf"), 1.0, 0.0
        else:
            raise ValueError(f"activation {self.activation!r}: 'clamped_swish' or 'silu'")
        self.score = p.get("score", "sigmoid")
        self.identity = int(p.get("identity", 0) or 0)
        self.has_correction = bool(p.get("correction", False))
        self.correction = None
        self.shared = None
        if p.get("shared"):
            self.shared = SwiGLU(FeedForwardSpec(kind="swiglu", intermediate_size=int(p["shared"]),
                                                 params=(("activation", "silu"),),
                                                 tensor_names=(("gate", "gate"), ("up", "up"), ("down", "down"))),
                                 hidden_size, compute_dtype, device)
        self.prefix = p.get("expert_prefix", "e")
        if self.ff <= 0 or self.E <= 0 or self.identity < 0 or not 0 < self.top <= self.E + self.identity:
            raise ValueError("routed experts need a positive size, experts and 0 < top <= the router's outputs")
        if self.score not in ("sigmoid", "softmax"):
            raise ValueError(f"score {self.score!r}: 'sigmoid' or 'softmax'")
        if self.groups is not None and self.identity:
            raise ValueError("expert groups and router outputs without an expert exclude one another")
        if self.groups is not None:
            count, keep = self.groups
            if self.E % count or not 0 < keep <= count or keep * (self.E // count) < self.top:
                raise ValueError("the expert groups do not fit the experts that are chosen")
        self.w_router = self.w_gate_up = self.w_down = None

    def parameters(self) -> Dict[str, ParamSpec]:
        out = {"router": ParamSpec((self.E + self.identity, self.hidden), role="scale", init=("normal", 0.5))}
        if self.has_correction:
            out["correction"] = ParamSpec((self.E + self.identity,), role="scale", init=("normal", 0.05))
        if self.shared is not None:
            out.update({f"shared.{n}": ps for n, ps in self.shared.parameters().items()})
        for e in range(self.E):
            out[f"{self.prefix}{e}.gate"] = ParamSpec((self.ff, self.hidden))
            out[f"{self.prefix}{e}.up"] = ParamSpec((self.ff, self.hidden))
            out[f"{self.prefix}{e}.down"] = ParamSpec((self.hidden, self.ff))
        return out

    def load(self, t: Dict[str, torch.Tensor]) -> None:
        self.w_router = t["router"].float().contiguous()
        if self.has_correction:
            self.correction = t["correction"].float().contiguous()
        if self.shared is not None:
            self.shared.load({n: t[f"shared.{n}"] for n in self.shared.parameters()})
        rows = [t[f"{self.prefix}{e}.{k}"] for e in range(self.E) for k in ("gate", "up")]
        downs = [t[f"{self.prefix}{e}.down"] for e in range(self.E)]
        dt = torch.float32 if any(x.dtype == torch.float32 for x in rows + downs) else rows[0].dtype
        self.w_gate_up = torch.cat([x.to(dt) for x in rows], dim=0).contiguous()          # [E * 2 * ff, hidden]
        self.w_down = torch.cat([x.to(dt) for x in downs], dim=1).contiguous()             # [hidden, E * ff]
        ops.prepare_streaming(self.w_gate_up)
        ops.prepare_streaming(self.w_down)

    def _route(self, x: torch.Tensor, lists: bool):
        """(dense weights or None, ids, weights, the tokens' share of their own input or None)."""
        got = ops.moe_route(x, self.w_router, self.top, self.groups, self.route_scale, lists=lists, score=self.score,
                            correction=self.correction, identity=self.identity)
        if lists:
            return got if self.identity else got + (None,)
        return (got[0], None, None, got[1]) if self.identity else (got, None, None, None)

    def forward(self, x: torch.Tensor, partials_ok: bool = False):
        T = x.shape[0]
        act = (self.limit, self.act_alpha)
        plain = self.identity == 0 and self.shared is None        # nothing joins the experts' sum
        if (T * self.top < self.E and x.dtype == self.w_gate_up.dtype == self.w_down.dtype and self.hidden <= 12288
                and self.top * self.ff <= 12288):
            _, ids, weights, own = self._route(x, True)
            out = ops.moe_sparse(x, self.w_gate_up, self.w_down, ids, weights, self.ff, *act, shift=self.act_shift)
        elif (T > self.SORTED_FROM and x.dtype == torch.bfloat16 and self.w_gate_up.dtype == self.w_down.dtype == torch.bfloat16
                and self.hidden % 8 == 0 and self.ff % 8 == 0 and self.E <= 4096 and ops.grouped_product_available()):
            _, ids, weights, own = self._route(x, True)
            out = ops.moe_sorted(x, self.w_gate_up, self.w_down, ids, weights, self.E, self.ff, *act, shift=self.act_shift)
        else:
            dense, _, _, own = self._route(x, False)
            gate_up = ops.linear(x, self.w_gate_up, out_dtype=torch.float32, partials_ok=True)
            a = ops.moe_act(gate_up, dense, self.E, self.ff, *act, self.dtype, shift=self.act_shift)
            out = ops.linear(a, self.w_down, out_dtype=torch.float32, partials_ok=partials_ok and plain)
        if plain:
            return out
        # the token's own input times what it gave to outputs without an expert, and the shared expert, join in 32-bit
        shared = self.shared.forward(x, partials_ok=True) if self.shared is not None else None
        if isinstance(shared, ops.PartialSum) and shared.rounds_to is not None:
            shared = ops.as_tensor(shared)
        return ops.moe_finish(ops.as_tensor(out), x, own, shared)
