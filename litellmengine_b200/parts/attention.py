"""The attention mixer: grouped-query causal attention over the paged cache."""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, Optional

import numpy as np
import torch

from ..cache import PagedNeed
from ..config.specs import MixerSpec
from ..csrc import ops
from ..weights.loader import ParamSpec
from .context import StageContext, StepPrelude
from .registry import lookup, register_mixer


class AttentionWork(StepPrelude):
    """How the attention kernels cut a step: rows of entries that bring one token go to the
    split-key decode kernel, longer portions are cut into tiles of `ops.PREFILL_TILE_ROWS` query
    rows (entry, first row inside it) for the tensor-core prompt kernel, longest walk first.
    Both lists are padded with -1 up to what a step of as many tokens could need at most, so that
    a launch over the whole padded list does the same work (a kernel's block that meets -1 returns
    at once): that is how a captured graph of a step of T tokens serves every later step of T
    tokens, however they are divided among requests."""
    name = "attention_work"

    @dataclass
    class Views:
        decode_rows: torch.Tensor        # int32 [num_decode] rows of entries that bring a single token
        prefill_tiles: torch.Tensor      # int32 [num_prefill_tiles, 2]
        num_decode: int
        num_prefill_tiles: int
        padded_rows: torch.Tensor        # the same lists over their padding: [rows_cap], [tiles_cap, 2]
        padded_tiles: torch.Tensor

    def sections(self, max_tokens: int, max_entries: int):
        self.max_entries = max_entries
        return {"decode_rows": max_tokens,
                "prefill_tiles": 2 * (max_tokens // ops.PREFILL_TILE_ROWS + max_entries + 1)}

    def caps(self, num_tokens: int):
        """The most rows and tiles a step of `num_tokens` tokens can have."""
        return (min(num_tokens, self.max_entries),
                num_tokens // ops.PREFILL_TILE_ROWS + min(num_tokens // 2, self.max_entries) + 1)

    def fill(self, facts, out):
        R = ops.PREFILL_TILE_ROWS
        single = facts.q_len == 1
        n_dec = int(single.sum())
        rows_cap, tiles_cap = self.caps(facts.num_tokens)
        tiles_cap = min(tiles_cap, len(out["prefill_tiles"]) // 2)
        out["decode_rows"][:n_dec] = facts.q_start[single]
        out["decode_rows"][n_dec:rows_cap] = -1
        n_tiles = 0
        if n_dec < len(facts.q_len):
            tiles = [(i, q0) for i in np.nonzero(~single)[0] for q0 in range(0, int(facts.q_len[i]), R)]
            # longest first: a tile late in a long prompt walks the most keys, so it should start early
            tiles.sort(key=lambda t: -(int(facts.past[t[0]]) + t[1]))
            n_tiles = len(tiles)
            out["prefill_tiles"][:2 * n_tiles] = np.asarray(tiles, dtype=np.int64).reshape(-1)
        out["prefill_tiles"][2 * n_tiles:2 * tiles_cap] = -1
        return n_dec, n_tiles, rows_cap, tiles_cap

    def views(self, dev, filled):
        n_dec, n_tiles, rows_cap, tiles_cap = filled
        return AttentionWork.Views(dev["decode_rows"][:n_dec], dev["prefill_tiles"][:2 * n_tiles].view(n_tiles, 2),
                                   n_dec, n_tiles, dev["decode_rows"][:rows_cap],
                                   dev["prefill_tiles"][:2 * tiles_cap].view(tiles_cap, 2))


@register_mixer("attention")
class AttentionMixer:
    """q/k/v projections without bias fused into one product, per-head RMSNorm of q and k,
    rotation, cache write, attention over the pages, output projection
    (src/model/qwen3.cpp:357-449,464-481,550-567).  kv head of query head h is h // (heads /
    kv_heads); scores are scaled by 1/sqrt(head_dim) unless the spec gives a scale
    (src/ops/attention.cu:204-207)."""

    graph_safe = True          # forward only launches kernels on the current stream
    any_division_safe = True   # and nothing in it is shaped by the number of entries of the step

    def __init__(self, spec: MixerSpec, hidden_size: int, compute_dtype: torch.dtype, device):
        if spec.num_heads <= 0 or spec.num_kv_heads <= 0 or spec.num_heads % spec.num_kv_heads:
            raise ValueError("attention heads must be a positive multiple of kv heads")
        if spec.head_dim <= 0 or spec.head_dim % 16 or spec.head_dim > 256:
            raise ValueError(f"head_dim {spec.head_dim}: the attention kernels take multiples of 16 up to 256")
        if spec.window is not None and spec.window <= 0:
            raise ValueError("an attention window must be positive")
        self.spec = spec
        self.hidden = hidden_size
        self.nq, self.nkv, self.d = spec.num_heads, spec.num_kv_heads, spec.head_dim
        self.scale = spec.scale if spec.scale is not None else 1.0 / math.sqrt(float(self.d))
        self.dtype = compute_dtype
        self.device = torch.device(device)
        self.position = lookup("position", spec.position.kind)(spec.position, self.d, device)
        self.q_norm = self.k_norm = None
        if spec.qk_norm is not None:
            cls = lookup("norm", spec.qk_norm.kind)
            self.q_norm = cls(spec.qk_norm, self.d)
            self.k_norm = cls(spec.qk_norm, self.d) if spec.has_kv else None
        self.w_qkv: Optional[torch.Tensor] = None
        self.w_o: Optional[torch.Tensor] = None

    def parameters(self) -> Dict[str, ParamSpec]:
        p = {"q_proj.weight": ParamSpec((self.nq * self.d, self.hidden)),
             "o_proj.weight": ParamSpec((self.hidden, self.nq * self.d))}
        if self.spec.has_kv:
            p["k_proj.weight"] = ParamSpec((self.nkv * self.d, self.hidden))
            p["v_proj.weight"] = ParamSpec((self.nkv * self.d, self.hidden))
        if self.q_norm is not None:
            p["q_norm.weight"] = self.q_norm.parameters()["weight"]
        if self.k_norm is not None:
            p["k_norm.weight"] = self.k_norm.parameters()["weight"]
        return p

    def load(self, t: Dict[str, torch.Tensor]) -> None:
        parts = [t["q_proj.weight"]]
        if self.spec.has_kv:
            parts += [t["k_proj.weight"], t["v_proj.weight"]]
        # Row concatenation, so one product yields [q | k | v] per token.  A float32 member
        # keeps the fused matrix in float32.
        dt = torch.float32 if any(x.dtype == torch.float32 for x in parts) else parts[0].dtype
        self.w_qkv = torch.cat([x.to(dt) for x in parts], dim=0).contiguous()
        self.w_o = t["o_proj.weight"].contiguous()
        ops.prepare_streaming(self.w_qkv)           # a tiled copy for decode steps (bfloat16 on a GPU only)
        ops.prepare_streaming(self.w_o)
        if self.q_norm is not None:
            self.q_norm.load({"weight": t["q_norm.weight"]})
        if self.k_norm is not None:
            self.k_norm.load({"weight": t["k_norm.weight"]})

    def cache_need(self):
        if not self.spec.has_kv:
            return None
        return PagedNeed(self.nkv, self.d, self.spec.window)

    def step_prelude(self):
        return AttentionWork()

    @property
    def graph_variant_group(self):
        return ("attention", self.nkv)

    def graph_variant(self, batch, padded: bool) -> int:
        """The decode kernel's key splits: the one launch choice here that depends on lengths."""
        work = batch.preludes.get(AttentionWork.name)
        if work is None:
            return 0
        n_dec = work.padded_rows.shape[0] if padded else work.num_decode
        return decode_key_splits(self.device, n_dec, self.nkv, batch.max_kv_len) if n_dec else 0

    def forward(self, x: torch.Tensor, ctx: StageContext) -> torch.Tensor:
        b = ctx.batch
        qkv = ops.linear(x, self.w_qkv, out_dtype=torch.float32, partials_ok=True)   # normalised, rotated in 32-bit
        has_kv = self.spec.has_kv and ctx.writes_cache
        if self.spec.has_kv and not ctx.writes_cache:
            raise RuntimeError("a mixer with its own keys and values was given a borrowed cache")
        eps = self.spec.qk_norm.eps if self.spec.qk_norm is not None else 0.0
        qw = self.q_norm.weight if self.q_norm is not None else None
        kw = self.k_norm.weight if self.k_norm is not None else None
        cache, table = (ctx.cache, ctx.block_table) if has_kv else (None, None)
        if hasattr(self.position, "rotation"):
            # a rotation (or nothing): norms, rotation and cache write in one kernel
            rot = self.position.rotation(b)
            q = ops.qk_norm_rope_kv_write(
                qkv, cache, b.positions, b.token_entry, b.entry_slot, table, qw, kw, eps,
                rot.inv_freq if rot is not None else None, rot.rotary_dim if rot is not None else 0,
                self.nq, self.nkv, self.d, ctx.page_size, has_kv, ctx.status, q_dtype=self.dtype,
                angles=rot.angles if rot is not None else None)
        else:
            # an encoding of the part's own: norms, then the part, then the cache write
            q32, k32 = ops.qk_head_norm(qkv, qw, kw, eps, self.nq, self.nkv, self.d, has_kv)
            T = q32.shape[0]
            q32, k32 = self.position.apply(q32.view(T, self.nq, self.d),
                                           k32.view(T, self.nkv, self.d) if k32 is not None else None, b)
            q = ops.qk_store(q32.reshape(T, self.nq * self.d).contiguous(),
                             k32.reshape(T, self.nkv * self.d).contiguous() if k32 is not None else None, qkv, cache,
                             b.positions, b.token_entry, b.entry_slot, table, self.nq, self.nkv, self.d,
                             ctx.page_size, has_kv, ctx.status, self.dtype)
        a = attention_over_pages(q, ctx, self.nq, self.nkv, self.d, self.spec.window, self.scale)
        # joins the float32 residual; may stay a sum of k-splits if the layer's norm adds them itself
        residual = getattr(ctx, "residual", None)
        if residual is not None and ops.linear_into(a, self.w_o, residual):
            return None                                           # added to the residual in the product's epilogue
        return ops.linear(a, self.w_o, out_dtype=torch.float32, partials_ok=getattr(ctx, "partials_ok", False))


class BranchMixer:
    """What a mixer offers so that it can stand alone or beside others under `ParallelMixer`: after
    `load`, `w_in` [in_width, hidden] (every projection of the layer input it wants, as one matrix) and
    `w_o` [hidden, out_width]; `mix` reads its columns of a float32 projection and writes its columns of
    the layer's output buffer, which `w_o` then maps to the hidden size.  Standing alone that is three
    steps; a parent that runs several branches fuses their `w_in` into one product and their `w_o`
    into another and calls `mix` of each on its own column ranges."""

    in_width = 0
    out_width = 0
    w_in: Optional[torch.Tensor] = None
    w_o: Optional[torch.Tensor] = None

    def mix(self, proj: torch.Tensor, col0: int, ctx: StageContext, out: torch.Tensor, out_col0: int,
            out_scale: float) -> None:
        raise NotImplementedError

    def forward(self, x: torch.Tensor, ctx: StageContext):
        proj = ops.linear(x, self.w_in, out_dtype=torch.float32)
        out = torch.empty((x.shape[0], self.out_width), dtype=self.dtype, device=x.device)
        self.mix(proj, 0, ctx, out, 0, 1.0)
        return ops.linear(out, self.w_o, out_dtype=torch.float32, partials_ok=getattr(ctx, "partials_ok", False))

    def fused_by_parent(self) -> None:
        """A parent holds the fused matrices now; the branch keeps no copies."""
        self.w_in = self.w_o = None


@register_mixer("gated_attention")
class GatedAttentionMixer(BranchMixer):
    """Grouped-query causal softmax attention over the paged cache with the options of `MixerSpec`:
    values of their own width, biased q/k/v projections, a q/k norm per head or over the token's whole
    projection, a query temperature q *= 1 + coef * ln(floor((p + 1) / every) + 1), and an output gate
    sigmoid(W_g x) on the concatenated heads before the output projection.  No rotation: a model that
    uses this mixer encodes positions elsewhere.  One product yields [q | k | v | g] per token in
    float32; one kernel adds the biases, normalises, applies the temperature and writes keys and values
    to their pages; the attention kernel applies the gate as it stores.  The gate may be one value per head
    (`output_gate_scope` 'head').  `distance_bias` = (rows, far) adds a learned bias table[bucket(i - j), head]
    to the scaled score of query i and key j (see `distance_bucket`); the mixer expands the stored table
    [rows, heads] into one row per distance once, when it is loaded.  `head_temperature`: a learned number per query
    head multiplies the scaled score; `log_distance_bias`: r1[h] * ln(1 + r2[h] * (i - j)) is taken off it (two learned
    numbers per query head, evaluated inside the attention kernel: no table, no farthest distance)."""

    graph_safe = True
    any_division_safe = True

    _DEFAULT_NAMES = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "g": "g_proj.weight",
                      "o": "o_proj.weight", "q_bias": "q_proj.bias", "k_bias": "k_proj.bias", "v_bias": "v_proj.bias",
                      "q_norm": "q_norm.weight", "k_norm": "k_norm.weight", "rel": "distance_bias",
                      "temp": "head_temperature", "r1": "log_bias.r1", "r2": "log_bias.r2"}

    def __init__(self, spec: MixerSpec, hidden_size: int, compute_dtype: torch.dtype, device):
        if spec.num_heads <= 0 or spec.num_kv_heads <= 0 or spec.num_heads % spec.num_kv_heads:
            raise ValueError("attention heads must be a positive multiple of kv heads")
        self.dv = spec.value_dim or spec.head_dim
        if not 0 < spec.head_dim <= 256 or not 0 < self.dv <= 256:
            raise ValueError("key and value widths must be between 1 and 256")
        if spec.position.kind not in ("none", "rope_pairs"):
            raise ValueError("the gated attention mixer rotates neighbouring pairs ('rope_pairs') or not at all")
        if spec.qk_norm_scope not in ("head", "projection"):
            raise ValueError(f"qk_norm_scope {spec.qk_norm_scope!r}: 'head' or 'projection'")
        if spec.output_gate not in (None, "sigmoid"):
            raise ValueError(f"output_gate {spec.output_gate!r}: 'sigmoid' or None")
        if not spec.has_kv:
            raise ValueError("the gated attention mixer keeps its own keys and values")
        if spec.output_gate_scope not in ("channel", "head"):
            raise ValueError(f"output_gate_scope {spec.output_gate_scope!r}: 'channel' or 'head'")
        if spec.window is not None and spec.window <= 0:
            raise ValueError("an attention window must be positive")
        self.spec, self.hidden, self.dtype, self.device = spec, hidden_size, compute_dtype, torch.device(device)
        self.nq, self.nkv, self.d = spec.num_heads, spec.num_kv_heads, spec.head_dim
        self.scale = spec.scale if spec.scale is not None else 1.0 / math.sqrt(float(self.d))
        self.names = dict(self._DEFAULT_NAMES, **dict(spec.tensor_names))
        # a rotation after the norm, inside the kernel that prepares q, k and v
        self.rotation = None
        if spec.position.kind != "none":
            self.rotation = lookup("position", spec.position.kind)(spec.position, self.d, device).kernel_args()
        self.keep_first = int(getattr(spec, "keep_first", 0)) if spec.window is not None else 0
        self.sink = getattr(spec, "softmax_sink", None)
        if self.keep_first < 0:
            raise ValueError("keep_first must not be negative")
        self.q_off, self.k_off = 0, self.nq * self.d
        self.v_off = self.k_off + self.nkv * self.d
        self.g_off = self.v_off + self.nkv * self.dv
        self.gate_per_head = spec.output_gate is not None and spec.output_gate_scope == "head"
        self.gate_width = 0 if not spec.output_gate else (self.nq if self.gate_per_head else self.nq * self.dv)
        self.in_width = self.g_off + self.gate_width
        self.out_width = self.nq * self.dv
        self.biases = None
        self.q_norm_w = self.k_norm_w = None
        self.dist_table = None                  # float32 [distances, heads], made from the stored table when loaded
        if spec.distance_bias is not None:
            rows, far = spec.distance_bias
            if rows != -1 and not far > rows // 2 >= 1:
                raise ValueError("distance_bias: the farthest distance must exceed half the number of rows")
        # the tuned bfloat16 kernels read keys and values of one width from one tensor, add no bias to the
        # scores and leave the gate to a kernel that takes one value per channel
        self.head_temp = self.log_r1 = self.log_r2 = None     # float32 [heads] each, when the spec asks for them
        # the scores or the key walk carry more than the tuned kernels know
        scored = spec.head_temperature or spec.log_distance_bias
        walked = self.keep_first > 0 or self.sink is not None          # kept first keys, a sink: the general kernel
        self._tuned = (compute_dtype == torch.bfloat16 and self.dv == self.d and self.device.type == "cuda"
                       and spec.distance_bias is None and not self.gate_per_head and not scored and not walked
                       and ops.fast_attention_supported(self.d, self.nq // self.nkv))
        # with a bias by distance or a gate per head: prompt portions still take a tensor-core kernel (the
        # mma.sync one, which adds the bias to its scores and gates as it stores), single tokens the general one
        if scored and spec.distance_bias is not None:
            raise ValueError("a distance table and a logarithmic distance bias or head temperature exclude one another")
        self._tuned_prompt = (not self._tuned and compute_dtype == torch.bfloat16 and self.dv == self.d
                              and self.device.type == "cuda" and (self.gate_per_head or not spec.output_gate)
                              and ops.prefill_attention_supported(self.d))
        self._tuned_decode = self._tuned_prompt and ops.fast_attention_supported(self.d, self.nq // self.nkv)
        self.dist_table_t = None
        self.analytic = False                   # dist_table_t holds (temperature, r1, r2) per head instead of a table

    def parameters(self) -> Dict[str, ParamSpec]:
        n, s = self.names, self.spec
        p = {n["q"]: ParamSpec((self.nq * self.d, self.hidden)), n["k"]: ParamSpec((self.nkv * self.d, self.hidden)),
             n["v"]: ParamSpec((self.nkv * self.dv, self.hidden)), n["o"]: ParamSpec((self.hidden, self.nq * self.dv))}
        if s.output_gate:
            p[n["g"]] = ParamSpec((self.gate_width, self.hidden))
        if s.distance_bias is not None:
            p[n["rel"]] = ParamSpec((s.distance_bias[0], self.nq), role="scale", init=("normal", 0.5))
        if s.head_temperature:
            p[n["temp"]] = ParamSpec((self.nq,), role="scale", init=("one_plus_normal", 0.2))
        if s.log_distance_bias:
            p[n["r1"]] = ParamSpec((self.nq,), role="scale", init=("one_plus_normal", 0.15))
            p[n["r2"]] = ParamSpec((self.nq,), role="scale", init=("one_plus_normal", 0.15))     # stays positive
        if s.bias:
            for key, size in (("q_bias", self.nq * self.d), ("k_bias", self.nkv * self.d), ("v_bias", self.nkv * self.dv)):
                p[n[key]] = ParamSpec((size,), role="scale", init=("normal", 0.02))
        if s.qk_norm is not None:
            whole = s.qk_norm_scope == "projection"
            p[n["q_norm"]] = ParamSpec((self.nq * self.d if whole else self.d,), role="scale", init=("one_plus_normal", 0.01))
            p[n["k_norm"]] = ParamSpec((self.nkv * self.d if whole else self.d,), role="scale", init=("one_plus_normal", 0.01))
        return p

    def load(self, t: Dict[str, torch.Tensor]) -> None:
        n, s = self.names, self.spec
        rows = [t[n["q"]], t[n["k"]], t[n["v"]]] + ([t[n["g"]]] if s.output_gate else [])
        dt = torch.float32 if any(x.dtype == torch.float32 for x in rows) else rows[0].dtype
        self.w_in = torch.cat([x.to(dt) for x in rows], dim=0).contiguous()
        self.w_o = t[n["o"]].contiguous()
        if s.bias:
            self.biases = tuple(t[n[k]].contiguous() for k in ("q_bias", "k_bias", "v_bias"))
        if s.qk_norm is not None:
            self.q_norm_w, self.k_norm_w = t[n["q_norm"]].contiguous(), t[n["k_norm"]].contiguous()
        if s.head_temperature:
            self.head_temp = t[n["temp"]].float().contiguous()
        if s.log_distance_bias:
            self.log_r1, self.log_r2 = t[n["r1"]].float().contiguous(), t[n["r2"]].float().contiguous()
        if s.head_temperature or s.log_distance_bias:
            # for the tensor-core kernels: (temperature, r1, r2) per head; they evaluate the bias themselves
            one = torch.ones(self.nq, dtype=torch.float32, device=self.w_in.device)
            self.dist_table_t = torch.stack([self.head_temp if self.head_temp is not None else one,
                                             self.log_r1 if self.log_r1 is not None else one * 0,
                                             self.log_r2 if self.log_r2 is not None else one * 0], dim=1).contiguous()
            self.analytic = True
        if s.distance_bias is not None:
            rel = t[n["rel"]].float()
            rows, far = rel.shape[0], float(s.distance_bias[1])
            if not far > rows // 2 >= 1:
                raise ValueError("distance_bias: the farthest distance must exceed half the number of rows")
            # from distance ceil(far) on the row no longer changes; a window never asks beyond its size
            count = int(math.ceil(far)) + 1
            if s.window is not None:
                count = min(count, s.window)
            index = torch.tensor([distance_bucket(d, rows, far) for d in range(count)], dtype=torch.long, device=rel.device)
            self.dist_table = rel[index].contiguous()
            # for the tensor-core kernel: a row per head, in the exp2 domain
            self.dist_table_t = (self.dist_table.t() * math.log2(math.e)).contiguous()
        ops.prepare_streaming(self.w_in)
        ops.prepare_streaming(self.w_o)

    def cache_need(self):
        return PagedNeed(self.nkv, self.d, self.spec.window, None if self.dv == self.d else self.dv, self.keep_first)

    def step_prelude(self):
        return AttentionWork() if self._tuned or self._tuned_prompt else None

    @property
    def graph_variant_group(self):
        return ("attention", self.nkv) if self._tuned else ("gated_attention", self.nkv, self.spec.window)

    def _decode_reach(self, batch) -> int:
        """The most keys a single token of this step walks: the longest cached length, or the window."""
        return min(batch.max_kv_len, self.spec.window) if self.spec.window else batch.max_kv_len

    def graph_variant(self, batch, padded: bool) -> int:
        if self._tuned:
            return AttentionMixer.graph_variant(self, batch, padded)
        if not self._tuned_decode:
            return 0
        work = batch.preludes.get(AttentionWork.name)       # the decode kernel's key splits, as the step will choose them
        n_dec = 0 if work is None else (work.padded_rows.shape[0] if padded else work.num_decode)
        n_tiles = 0 if work is None else (work.padded_tiles.shape[0] if padded else work.num_prefill_tiles)
        return decode_key_splits(self.device, n_dec, self.nkv, self._decode_reach(batch)) if n_dec and not n_tiles else 0

    def mix(self, proj, col0, ctx, out, out_col0, out_scale):
        b, s = ctx.batch, self.spec
        if not ctx.writes_cache:
            raise RuntimeError("a mixer with its own keys and values was given a borrowed cache")
        q = ops.attention_prepare(
            proj, col0 + self.q_off, col0 + self.k_off, col0 + self.v_off, self.biases, self.q_norm_w, self.k_norm_w,
            s.qk_norm_scope if s.qk_norm is not None else None, s.qk_norm.eps if s.qk_norm is not None else 0.0,
            s.query_temperature, ctx.cache_keys, ctx.cache_values, b.positions, b.token_entry, b.entry_slot,
            ctx.block_table, self.nq, self.nkv, self.d, self.dv, ctx.page_size, ctx.status, self.dtype,
            rotation=self.rotation)
        if self._tuned and ctx.cache is not None and b.preludes.get(AttentionWork.name) is not None:
            a = attention_over_pages(q, ctx, self.nq, self.nkv, self.d, s.window, self.scale)
            ops.gate_mul(a, proj, col0 + self.g_off, out, out_col0, s.output_gate, out_scale)
            return
        work = b.preludes.get(AttentionWork.name) if self._tuned_prompt and ctx.cache is not None else None
        padded = getattr(b, "any_division", False)
        if work is not None:
            # prompt portions on the tensor cores (bias added to the scores, gate and scale as the kernel stores);
            # single tokens in the split-key decode kernel where it takes the group (bias likewise, the gate in a
            # small kernel after it), else in the general kernel by the list of their rows
            n_tiles = work.padded_tiles.shape[0] if padded else work.num_prefill_tiles
            n_dec = work.padded_rows.shape[0] if padded else work.num_decode
            gate = proj if s.output_gate else None
            if (n_tiles and self.analytic and gate is None and out_col0 == 0 and out_scale == 1.0 and out.is_contiguous()
                    and out.shape[1] == self.nq * self.d
                    and ops.prefill_tcgen05_biased_supported(self.d, ctx.page_size, self.nq // self.nkv)):
                # temperature and logarithmic bias in the softmax warps of the tcgen05 kernel (two heads of a group a CTA)
                ops.paged_attention_prefill_tcgen05_biased(
                    q, out, ctx.cache, work.padded_tiles if padded else work.prefill_tiles, n_tiles, b.entry_slot,
                    b.entry_q_start, b.entry_q_len, b.entry_kv_len, ctx.block_table, self.nq, self.nkv, self.d,
                    ctx.page_size, s.window, self.scale, ctx.status, self.dist_table_t)
            elif n_tiles:
                ops.paged_attention_prefill_biased(
                    q, out, out_col0, ctx.cache, work.padded_tiles if padded else work.prefill_tiles, n_tiles, b.entry_slot,
                    b.entry_q_start, b.entry_q_len, b.entry_kv_len, ctx.block_table, self.nq, self.nkv, self.d, ctx.page_size,
                    s.window, self.scale, ctx.status, dist_bias_t=self.dist_table_t, head_gate=gate,
                    gate_off=col0 + self.g_off, out_scale=out_scale, analytic_bias=self.analytic,
                    keep_first=self.keep_first, sink=self.sink)
            if not n_dec:
                return
            rows = work.padded_rows if padded else (None if n_dec == b.num_tokens else work.decode_rows)
            if self._tuned_decode and not n_tiles:
                # without a gate, a scale or a column offset the kernel writes where the output product reads
                direct = (gate is None and out_col0 == 0 and out_scale == 1.0 and out.is_contiguous()
                          and tuple(out.shape) == tuple(q.shape))
                a = out if direct else torch.empty_like(q)
                splits = decode_key_splits(q.device, n_dec, self.nkv, self._decode_reach(b))
                ops.paged_attention_decode(q, a, ctx.cache, rows, n_dec, b.positions, b.token_entry, b.entry_slot,
                                           ctx.block_table, self.nq, self.nkv, self.d, ctx.page_size, s.window, self.scale, splits,
                                           ctx.status, dist_bias_t=self.dist_table_t, analytic_bias=self.analytic,
                                           keep_first=self.keep_first, sink=self.sink)
                if not direct:
                    ops.gate_mul(a, gate, col0 + self.g_off, out, out_col0, s.output_gate, out_scale,
                                 per_head=self.dv if self.gate_per_head else 0)
                return
        else:
            rows = None
        ops.paged_attention_generic_kv(
            q, ctx.cache_keys, ctx.cache_values, b.positions, b.token_entry, b.entry_slot, ctx.block_table, self.nq,
            self.nkv, self.d, self.dv, ctx.page_size, s.window, self.scale, ctx.status, out, out_col0,
            gate=proj if s.output_gate else None, gate_off=col0 + self.g_off, out_scale=out_scale,
            dist_bias=self.dist_table, gate_per_head=self.gate_per_head, rows=rows, head_scale=self.head_temp,
            log_bias=(self.log_r1, self.log_r2) if self.log_r1 is not None else None, keep_first=self.keep_first,
            sink=self.sink)


def distance_bucket(n: int, rows: int, far: float) -> int:
    """Row of a distance-bias table for the distance n >= 0 between a query and a key: the first rows // 2
    distances have a row each; farther ones share rows in logarithmic steps, and from `far` on it is the last."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


_slots = {}


def _cta_slots(device) -> int:
    n = _slots.get(device)
    if n is None:
        n = _slots[device] = 2 * torch.cuda.get_device_properties(device).multi_processor_count
    return n


# Key splits of the decode kernel by the longest cached length, in steps: a captured graph holds its
# number of splits, so steps whose lengths give the same number share a graph.
_SPLIT_STEPS = (1, 2, 3, 4, 6, 8, 12, 16, 24, 32, 48, 64)


def decode_key_splits(device, n_dec: int, nkv: int, max_kv_len: int) -> int:
    """Two rules, measured.  (1) A split costs its launch and its share of the merge, a key costs its
    bytes: for a few rows the best number grows as the square root of the length (one row: 8, 12,
    16, 24 splits at 1,024, 2,304, 4,096, 16,384 keys), at least 64 keys a split.  (2) The grid runs in
    waves of two CTAs per SM: below that ceiling take the fewest splits that fill at least 0.85 of the
    waves they start, else the fullest (at 4,096 keys 20 rows: 5 splits, 40 rows: 4, 48 rows: 2,
    where one split took a quarter longer; 8, 16, 32, 64 rows stay at 4, 2, 1, 1; at 384 keys 48 rows
    stay at one split: 1.71 ms a step on the 0.6B shape against 1.79 with two)."""
    by_length = max(1, min(math.ceil(math.sqrt(max_kv_len / 16.0)), -(-max_kv_len // 64)))
    most = max(s for s in _SPLIT_STEPS if s <= by_length)
    if n_dec * nkv > _cta_slots(device):             # more CTAs than slots already: a split only evens out the waves,
        most = max(1, min(most, max_kv_len // 512))  # which pays for its merge kernel from about 512 keys a split
    key = (device, n_dec * nkv, most)
    got = _split_choice.get(key)
    if got is None:
        slots, ctas = _cta_slots(device), max(1, n_dec * nkv)
        fill = lambda s: ctas * s / (-(-ctas * s // slots) * slots)
        enough = [s for s in range(1, most + 1) if fill(s) >= 0.85]
        got = _split_choice[key] = enough[0] if enough else max(range(1, most + 1), key=lambda s: (fill(s), -s))
    return got


_split_choice: Dict[tuple, int] = {}


def attention_over_pages(q: torch.Tensor, ctx: StageContext, nq: int, nkv: int, d: int,
                         window: Optional[int], scale: float) -> torch.Tensor:
    """Pick the attention kernels for this batch.  Every choice reads the same pages and gives
    the same result up to rounding.  bfloat16 with a head size and group the tuned kernels
    take: single tokens go to the split-key decode kernel, longer portions to the tensor-core
    prefill kernel (a mixed batch launches both, each over its own rows).  Everything else,
    float32 included, goes through the generic kernel."""
    b = ctx.batch
    cache = ctx.cache
    work = b.preludes.get(AttentionWork.name)
    if (work is not None and q.dtype == torch.bfloat16 and cache.dtype == torch.bfloat16
            and ops.fast_attention_supported(d, nq // nkv)):
        out = torch.empty_like(q)
        # A step that is being captured as a graph of "any step of this many tokens" launches both
        # kernels over the padded lists; otherwise over what this step has.
        padded = getattr(b, "any_division", False)
        n_dec = work.padded_rows.shape[0] if padded else work.num_decode
        n_tiles = work.padded_tiles.shape[0] if padded else work.num_prefill_tiles
        if n_dec:
            splits = decode_key_splits(q.device, n_dec, nkv, b.max_kv_len)
            rows = work.padded_rows if padded else (None if n_dec == b.num_tokens else work.decode_rows)
            ops.paged_attention_decode(q, out, cache, rows, n_dec, b.positions, b.token_entry, b.entry_slot,
                                       ctx.block_table, nq, nkv, d, ctx.page_size, window, scale, splits, ctx.status)
        if n_tiles:
            kernel = (ops.paged_attention_prefill_tcgen05
                      if ops.prefill_tcgen05_supported(d, ctx.page_size)
                      else ops.paged_attention_prefill)       # tcgen05/TMEM/TMA where it applies, mma.sync otherwise
            kernel(q, out, cache, work.padded_tiles if padded else work.prefill_tiles, n_tiles, b.entry_slot,
                   b.entry_q_start, b.entry_q_len, b.entry_kv_len, ctx.block_table, nq, nkv, d, ctx.page_size, window,
                   scale, ctx.status)
        return out
    return ops.paged_attention_generic(q, cache, b.positions, b.token_entry, b.entry_slot,
                                       ctx.block_table, nq, nkv, d, ctx.page_size, window, scale, ctx.status)
