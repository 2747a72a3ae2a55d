"""Latent attention: softmax attention whose keys and values are linear maps of a small cached latent."""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from ..cache import PagedNeed
from ..config.specs import MixerSpec
from ..csrc import ops
from ..weights.loader import ParamSpec
from .context import StageContext
from .registry import lookup, register_mixer


@register_mixer("latent_attention")
class LatentAttentionMixer:
    """H heads; per head D unrotated and P rotated query/key entries and V value entries; latents of Q (queries) and
    R (keys and values) entries.  For a token with layer input x:

        cq = rmsnorm(W_dq x) * w_dq             q[h] = W_uq[h] cq = [qn[h] (D) | qr[h] (P)],  qr rotated by position
        [d | kr] = W_dkv x                      c = rmsnorm(d) * w_dkv (R),  kr (P) rotated by position, shared by all heads
        key[h] = [W_uk[h] c | kr]               value[h] = W_uv[h] c
        score(i, j) = (qn_i[h] . W_uk[h] c_j + qr_i[h] . kr_j) * scale        over the keys of the window, softmax
        out = W_o (concat_h(sum_j p_j value_j[h]) * sigmoid(W_g x))      (the gate one value per channel, or per head)

    Only the row [c | kr] (R + P entries, ONE "kv head") goes to the pages.  The per-head maps are folded into the
    query and the output, q_abs[h] = W_uk[h]^T qn[h] and sum_j p_j value_j[h] = W_uv[h] sum_j p_j c_j, so attention
    runs straight over the cached rows with key width R + P and the values the first R entries of the same rows:
    nothing per head is ever materialised per key, in prompts or in decoding.  A mixer whose spec says `has_kv`
    False has no W_dkv and reads the rows another stage cached (the stage's `cache_from`), with maps, queries,
    window and everything else of its own.

    One product yields [dq | dkv | g] per token in float32; `latent_prepare` norms both latents, rotates kr and
    writes the page row; W_uq; `latent_q_split` rotates qr and lays qn out head-major; a batched product with
    W_uk^T fills q_abs; attention (bfloat16: the tensor-core kernel in which all heads of a token share each staged
    tile of rows; float32: the general kernel); a batched product with W_uv^T; the gate; W_o."""

    graph_safe = True           # kernels and library products on the current stream only
    any_division_safe = True    # nothing is shaped by the number of entries

    _DEFAULT_NAMES = {"dq": "q_down.weight", "dq_norm": "q_down_norm.weight", "uq": "q_up.weight",
                      "dkv": "kv_down.weight", "dkv_norm": "kv_down_norm.weight", "uk": "k_up.weight",
                      "uv": "v_up.weight", "g": "g_proj.weight", "o": "o_proj.weight"}

    def __init__(self, spec: MixerSpec, hidden_size: int, compute_dtype: torch.dtype, device):
        p = dict(spec.params)
        self.H, self.D, self.V = spec.num_heads, spec.head_dim, spec.value_dim or spec.head_dim
        self.Q, self.R, self.P = int(p["q_rank"]), int(p["kv_rank"]), int(p.get("rot_dim", 0))
        if min(self.H, self.D, self.V, self.Q, self.R) <= 0 or self.P < 0:
            raise ValueError("latent attention needs positive heads, widths and ranks")
        if self.R > 512 or self.R + self.P > 1024:
            raise ValueError("latent attention: the attention kernel takes latents up to 512 and rows up to 1024 entries")
        if spec.output_gate not in (None, "sigmoid"):
            raise ValueError(f"output_gate {spec.output_gate!r}: 'sigmoid' or None")
        if spec.window is not None and spec.window <= 0:
            raise ValueError("an attention window must be positive")
        self.eps = float(p.get("eps", 1e-6))
        self.keep_window = p.get("keep_window", spec.window)
        self.spec, self.hidden, self.dtype, self.device = spec, hidden_size, compute_dtype, torch.device(device)
        self.scale = spec.scale if spec.scale is not None else 1.0 / math.sqrt(float(self.D + self.P))
        self.names = dict(self._DEFAULT_NAMES, **dict(spec.tensor_names))
        self.rot_dims, self.inv_freq, self.rot_pairs, self.rot_mag = 0, None, False, 1.0
        if spec.position.kind == "rope" and self.P:
            pos = lookup("position", "rope")(spec.position, self.P, device)       # the rotation's frequencies, float32
            self.rot_dims, self.inv_freq = pos.rotary_dim, pos.inv_freq
        elif spec.position.kind == "rope_pairs" and self.P:                       # neighbouring pairs, stretched frequencies
            self.inv_freq, self.rot_dims, self.rot_mag, self.rot_pairs = lookup("position", "rope_pairs")(
                spec.position, self.P, device).kernel_args()
        elif spec.position.kind != "none":
            raise ValueError("latent attention rotates by 'rope', by 'rope_pairs' or not at all")
        if spec.output_gate_scope not in ("channel", "head"):
            raise ValueError(f"output_gate_scope {spec.output_gate_scope!r}: 'channel' or 'head'")
        self.gate_per_head = bool(spec.output_gate) and spec.output_gate_scope == "head"
        self.dq_off = 0
        self.dkv_off = self.Q
        self.g_off = self.Q + (self.R + self.P if spec.has_kv else 0)
        self.gate_width = 0 if not spec.output_gate else (self.H if self.gate_per_head else self.H * self.V)
        # bfloat16 on the tensor-core kernel over the cached rows; float32 (and other latent sizes) on the general kernel
        self.tensor_core = (compute_dtype == torch.bfloat16 and self.device.type == "cuda"
                            and ops.latent_attention_supported(self.R, self.P))
        self.w_in = self.w_uq = self.w_uk_t = self.w_uv_t = self.w_o = None
        self.wq_norm = self.wkv_norm = None

    def parameters(self) -> Dict[str, ParamSpec]:
        n, s = self.names, self.spec
        p = {n["dq"]: ParamSpec((self.Q, self.hidden)),
             n["dq_norm"]: ParamSpec((self.Q,), role="scale", init=("one_plus_normal", 0.01)),
             n["uq"]: ParamSpec((self.H * (self.D + self.P), self.Q)),
             n["uk"]: ParamSpec((self.H * self.D, self.R)), n["uv"]: ParamSpec((self.H * self.V, self.R)),
             n["o"]: ParamSpec((self.hidden, self.H * self.V))}
        if s.has_kv:
            p[n["dkv"]] = ParamSpec((self.R + self.P, self.hidden))
            p[n["dkv_norm"]] = ParamSpec((self.R,), role="scale", init=("one_plus_normal", 0.01))
        if s.output_gate:
            p[n["g"]] = ParamSpec((self.gate_width, self.hidden))
        return p

    def load(self, t: Dict[str, torch.Tensor]) -> None:
        n, s = self.names, self.spec
        rows = [t[n["dq"]]] + ([t[n["dkv"]]] if s.has_kv else []) + ([t[n["g"]]] if s.output_gate else [])
        dt = torch.float32 if any(x.dtype == torch.float32 for x in rows) else rows[0].dtype
        self.w_in = torch.cat([x.to(dt) for x in rows], dim=0).contiguous()
        self.w_uq, self.w_o = t[n["uq"]].contiguous(), t[n["o"]].contiguous()
        # per head: [D, R] (q_abs = qn W_uk) and [R, V] (value = latent sum times W_uv^T), the batched products' right sides
        self.w_uk_t = t[n["uk"]].view(self.H, self.D, self.R).contiguous()
        self.w_uv_t = t[n["uv"]].view(self.H, self.V, self.R).transpose(1, 2).contiguous()
        self.wq_norm = t[n["dq_norm"]].float().contiguous()
        if s.has_kv:
            self.wkv_norm = t[n["dkv_norm"]].float().contiguous()
        for w in (self.w_in, self.w_uq, self.w_o):
            ops.prepare_streaming(w)

    def cache_need(self):
        if not self.spec.has_kv:
            return None
        return PagedNeed(1, self.R + self.P, self.keep_window, 0)       # keys only: the values are part of the key rows

    def forward(self, x: torch.Tensor, ctx: StageContext):
        b, s = ctx.batch, self.spec
        if s.has_kv != ctx.writes_cache:
            raise RuntimeError("a latent attention mixer keeps its own latent, or reads another stage's, as its spec says")
        H, D, P, R, V, T = self.H, self.D, self.P, self.R, self.V, x.shape[0]
        proj = ops.as_tensor(ops.linear(x, self.w_in, out_dtype=torch.float32))
        cq = ops.latent_prepare(proj, self.dq_off, self.dkv_off, self.Q, R, P, self.rot_dims, self.wq_norm, self.wkv_norm,
                                self.eps, self.inv_freq, ctx.cache_keys if s.has_kv else None, b, ctx.block_table,
                                ctx.page_size, ctx.status, self.dtype, rot_pairs=self.rot_pairs, rot_mag=self.rot_mag)
        q = ops.as_tensor(ops.linear(cq, self.w_uq, out_dtype=torch.float32))
        qn, packed = ops.latent_q_split(q, b.positions, self.inv_freq, H, D, P, R, self.rot_dims, self.dtype,
                                        rot_pairs=self.rot_pairs, rot_mag=self.rot_mag)
        # q_abs[h] = qn[h] W_uk[h], written into the first R columns of head h of the packed query
        torch.bmm(qn, self.w_uk_t if self.w_uk_t.dtype == qn.dtype else self.w_uk_t.to(qn.dtype),
                  out=packed.view(T, H, R + P)[:, :, :R].permute(1, 0, 2))
        lat = torch.empty((T, H * R), dtype=self.dtype, device=x.device)
        if self.tensor_core:
            ops.latent_attention(packed, ctx.cache_keys, b.positions, b.token_entry, b.entry_slot, ctx.block_table, H, R, P,
                                 ctx.page_size, s.window, self.scale, ctx.status, lat)
        else:
            ops.paged_attention_generic_kv(packed, ctx.cache_keys, None, b.positions, b.token_entry, b.entry_slot,
                                           ctx.block_table, H, 1, R + P, R, ctx.page_size, s.window, self.scale, ctx.status,
                                           lat, values_in_keys=True)
        heads = torch.empty((T, H * V), dtype=self.dtype, device=x.device)
        torch.bmm(lat.view(T, H, R).permute(1, 0, 2), self.w_uv_t if self.w_uv_t.dtype == lat.dtype else self.w_uv_t.to(lat.dtype),
                  out=heads.view(T, H, V).permute(1, 0, 2))
        if s.output_gate:
            ops.gate_mul(heads, proj, self.g_off, heads, 0, s.output_gate, per_head=V if self.gate_per_head else 0)
        return ops.linear(heads, self.w_o, out_dtype=torch.float32, partials_ok=getattr(ctx, "partials_ok", False))
