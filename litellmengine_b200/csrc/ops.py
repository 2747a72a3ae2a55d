"""Python faces of the CUDA kernels: argument checks, then one ctypes call per launch.

Every function takes CUDA tensors, launches on torch's current stream, allocates only its
result (or writes into `out`), and raises if the kernel refuses the sizes.  There is no CPU
or library fallback here: a tensor that is not on a CUDA device is an error, and a missing
compiler or library surfaces as `BuildError`.
"""
from __future__ import annotations

import ctypes
import os
import weakref
from ctypes import c_float, c_int, c_int32, c_longlong, c_uint32, c_uint64, c_void_p
from typing import Dict, Optional

import torch

from . import build

_libs: Dict[str, ctypes.CDLL] = {}

_REFUSALS = {
    -1: "a size this kernel does not take",
    -2: "a dtype combination this kernel is not built for",
    -3: "a pointer or stride that is not 16-byte aligned",
}


class KernelError(RuntimeError):
    pass


def lib(family: str) -> ctypes.CDLL:
    l = _libs.get(family)
    if l is None:
        l = ctypes.CDLL(build.ensure_built(family))
        _libs[family] = l
    return l


def loaded_libraries():
    return {k: v._name for k, v in _libs.items()}


def _fn(family: str, name: str, argtypes, restype=c_int):
    f = getattr(lib(family), name)
    if f.argtypes is None:
        f.argtypes = argtypes
        f.restype = restype
    return f


class PartialSum:
    """A product left as its k-splits: float32 [splits, rows, cols] whose sum over the first axis
    is the result.  The engine's norm and q/k kernels add the splits while they read, which
    saves a kernel per product in decode steps; `as_tensor` adds them for anyone else."""

    def __init__(self, parts: torch.Tensor, rounds_to: Optional[torch.dtype] = None):
        self.parts = parts
        self.rounds_to = rounds_to      # the product's own dtype when it is not float32: the sum is rounded to it

    @property
    def shape(self):
        return self.parts.shape[1:]

    @property
    def dtype(self):
        return self.parts.dtype


def as_tensor(x):
    if not isinstance(x, PartialSum):
        return x
    total = x.parts.sum(dim=0)
    return total.to(x.rounds_to) if x.rounds_to is not None else total


launch_count = 0          # launches of the engine's own kernels since import (library products are not counted)


def _check(code: int, what: str) -> None:
    global launch_count
    if code == 0:
        launch_count += 1
        return
    if code < 0:
        raise KernelError(f"{what}: refused, {_REFUSALS.get(code, f'code {code}')}")
    raise KernelError(f"{what}: CUDA error {code} at launch")


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return 0
    if t.dtype == torch.bfloat16:
        return 1
    raise KernelError(f"dtype {t.dtype} is not float32 or bfloat16")


def _dev(*tensors) -> None:
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise KernelError("tensor is not on a CUDA device; the engine has no CPU path")
        if not t.is_contiguous():
            raise KernelError("tensor is not contiguous")


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


_bound_stream: Optional[int] = None


def _stream() -> int:
    return _bound_stream if _bound_stream is not None else torch.cuda.current_stream().cuda_stream


class bound_stream:
    """Inside this scope every launch goes to the stream that was current at its entry, looked up
    once (asking for the current stream costs as much as three launches).  For code that does not
    switch streams while it runs: a model's forward pass."""

    def __enter__(self):
        global _bound_stream
        self._prev = _bound_stream
        _bound_stream = torch.cuda.current_stream().cuda_stream
        return self

    def __exit__(self, *exc):
        global _bound_stream
        _bound_stream = self._prev
        return False


def _i32(t: Optional[torch.Tensor], what: str) -> None:
    if t is not None and t.dtype != torch.int32:
        raise KernelError(f"{what} must be int32, got {t.dtype}")


# ------------------------------------------------------------------------------------------
def embedding(ids: torch.Tensor, table: torch.Tensor, status: torch.Tensor,
              out: Optional[torch.Tensor] = None, feedback: Optional[torch.Tensor] = None,
              scale: float = 1.0) -> torch.Tensor:
    """float32 [T, H] = table[ids] * scale; an id -1-j takes its token from feedback[j] (int32, on the device)."""
    _dev(ids, table, status, out, feedback)
    _i32(ids, "ids")
    if feedback is not None:
        _i32(feedback, "feedback")
    T, (V, H) = ids.numel(), table.shape
    if out is None:
        out = torch.empty((T, H), dtype=torch.float32, device=table.device)
    f = _fn("embedding", "llm_embedding_gather",
            [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_float, c_void_p])
    _check(f(_ptr(ids), _ptr(table), _dt(table), _ptr(out), T, H, V, _ptr(status), _ptr(feedback),
             feedback.numel() if feedback is not None else 0, float(scale), _stream()), "embedding")
    return out


def embedding_sinusoid(ids: torch.Tensor, table: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor,
                       status: torch.Tensor, feedback: Optional[torch.Tensor] = None,
                       copy_dtype: Optional[torch.dtype] = None):
    """float32 [T, H] = table[ids] + the sinusoidal vector of each token's position (entry 2i: sin(p * f_i),
    entry 2i+1: cos(p * f_i), f = `inv_freq`, float64 [ceil(H/2)]).  With `copy_dtype` the same rows come back a
    second time in that dtype.  Returns (stream, copy or None)."""
    _dev(ids, table, positions, inv_freq, status, feedback)
    _i32(ids, "ids")
    _i32(positions, "positions")
    T, (V, H) = ids.numel(), table.shape
    if inv_freq.dtype != torch.float64 or inv_freq.numel() != (H + 1) // 2:
        raise KernelError("inv_freq must be float64 [ceil(hidden/2)]")
    out = torch.empty((T, H), dtype=torch.float32, device=table.device)
    copy = torch.empty((T, H), dtype=copy_dtype, device=table.device) if copy_dtype is not None else None
    f = _fn("embedding", "llm_embedding_sinusoid",
            [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int,
             c_void_p, c_void_p, c_void_p])
    _check(f(_ptr(ids), _ptr(table), _dt(table), _ptr(out), _ptr(copy), _dt(copy) if copy is not None else 0, T, H, V,
             _ptr(status), _ptr(feedback), feedback.numel() if feedback is not None else 0, _ptr(positions),
             _ptr(inv_freq), _stream()), "embedding_sinusoid")
    return out, copy


def scatter_int32(dst: torch.Tensor, index: torch.Tensor, value: torch.Tensor, count: torch.Tensor,
                  max_count: int, status: torch.Tensor) -> None:
    """dst.flat[index[i]] = value[i] for i < count[0] (count is a device scalar; None: for i < max_count)."""
    _dev(dst, index, value, count, status)
    for t, n in ((dst, "dst"), (index, "index"), (value, "value"), (count, "count")):
        _i32(t, n)
    f = _fn("embedding", "llm_scatter_int32",
            [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p])
    _check(f(_ptr(dst), dst.numel(), _ptr(index), _ptr(value), _ptr(count), max_count, _ptr(status), _stream()),
           "scatter_int32")


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out_dtype: torch.dtype,
            delta: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None,
            write_sum: bool = False, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out = rmsnorm(x (+ delta)) * weight over the last dim; with `write_sum`, x += delta in place.
    `rows` (int32) selects which rows are normalised (out has len(rows) rows)."""
    parts, part_stride = 1, 0
    if isinstance(delta, PartialSum):
        parts, part_stride = delta.parts.shape[0], delta.parts.stride(0)
        delta = delta.parts[0]
    _dev(x, weight, delta, rows, out)
    _i32(rows, "rows")
    H = x.shape[-1]
    if weight.dtype != torch.float32 or weight.numel() != H:
        raise KernelError("norm weight must be float32 of the row length")
    if delta is not None and delta.shape != x.shape:
        raise KernelError("delta must have x's shape")
    n = rows.numel() if rows is not None else x.numel() // H
    if out is None:
        out = torch.empty((n, H), dtype=out_dtype, device=x.device)
    f = _fn("norm", "llm_rmsnorm",
            [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_float,
             c_int, c_int, c_longlong, c_void_p])
    _check(f(_ptr(x), _dt(x), _ptr(delta), _dt(delta) if delta is not None else 0, _ptr(weight), _ptr(out),
             _dt(out), _ptr(rows), n, H, float(eps), 1 if write_sum else 0, parts, part_stride, _stream()), "rmsnorm")
    return out


def rmsnorm_add(h: torch.Tensor, y: torch.Tensor, weight: torch.Tensor, eps: float,
                copy_dtype: Optional[torch.dtype] = None) -> Optional[torch.Tensor]:
    """h (float32, in place) += rmsnorm(y) * weight, row by row: a norm on a sublayer's output joined with
    the residual add.  With `copy_dtype`, returns the new h in that dtype (what the next sublayer reads).
    y may be a `PartialSum`: the kernel adds the k-splits as it reads."""
    parts, part_stride = 1, 0
    if isinstance(y, PartialSum):
        parts, part_stride = y.parts.shape[0], y.parts.stride(0)
        y = y.parts[0]
    _dev(h, weight)
    if not y.is_cuda or y.dim() != 2 or y.stride(1) != 1:
        raise KernelError("y must be a CUDA matrix with unit stride along its rows")
    T, H = h.shape
    if h.dtype != torch.float32 or tuple(y.shape) != (T, H) or weight.dtype != torch.float32 or weight.numel() != H:
        raise KernelError("rmsnorm_add wants a float32 stream, a y of its shape and a float32 weight of the row length")
    copy = torch.empty((T, H), dtype=copy_dtype, device=h.device) if copy_dtype is not None else None
    f = _fn("norm", "llm_rmsnorm_add",
            [c_void_p, c_void_p, c_int, c_longlong, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_int, c_longlong,
             c_void_p])
    _check(f(_ptr(h), _ptr(y), _dt(y), y.stride(0), _ptr(weight), _ptr(copy), _dt(copy) if copy is not None else 0,
             T, H, float(eps), parts, part_stride, _stream()), "rmsnorm_add")
    return copy


def tanh_norm(h: torch.Tensor, y, post, pre, out_dtype: Optional[torch.dtype] = None,
              rows: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """The elementwise norm n(v) = tanh(alpha v) * w + b around a residual add, in 32-bit: v = h + post(y) (written back
    into the float32 stream h unless `rows` picks rows), returned as pre(v) in `out_dtype`.  `post` and `pre` are
    (alpha float32 [1], w float32 [H], b float32 [H]) or None: without `post`, y joins as it is; without `pre`, nothing
    is returned.  y: None, a matrix [T, H] (float32 or bfloat16), or a `PartialSum` whose k-splits are added as they
    are read."""
    parts, part_stride = 1, 0
    if isinstance(y, PartialSum):
        parts, part_stride = y.parts.shape[0], y.parts.stride(0)
        y = y.parts[0]
    _dev(h, rows)
    _i32(rows, "rows")
    if h.dtype != torch.float32 or h.dim() != 2 or not h.is_contiguous():
        raise KernelError("tanh_norm wants a contiguous float32 stream [T, H]")
    T, H = h.shape
    if y is not None and (not y.is_cuda or tuple(y.shape) != (T, H) or y.stride(1) != 1):
        raise KernelError("y must be a CUDA matrix of the stream's shape with unit stride along its rows")
    for norm in (post, pre):
        if norm is not None:
            a, w, b = norm
            _dev(a, w, b)
            if any(t.dtype != torch.float32 for t in (a, w, b)) or a.numel() != 1 or w.numel() != H or b.numel() != H:
                raise KernelError("a tanh norm is (alpha [1], weight [H], bias [H]) in float32")
    n = rows.numel() if rows is not None else T
    out = torch.empty((n, H), dtype=out_dtype, device=h.device) if pre is not None else None
    pa, pw, pb = post if post is not None else (None, None, None)
    na, nw, nb = pre if pre is not None else (None, None, None)
    f = _fn("tanh_norm", "llm_tanh_norm",
            [c_void_p, c_void_p, c_int, c_longlong, c_int, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
             c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p])
    _check(f(_ptr(h), _ptr(y), _dt(y) if y is not None else 0, y.stride(0) if y is not None else 0, parts, part_stride,
             _ptr(pa), _ptr(pw), _ptr(pb), _ptr(na), _ptr(nw), _ptr(nb), _ptr(out), _dt(out) if out is not None else 0,
             _ptr(rows), n, H, _stream()), "tanh_norm")
    return out


ACTIVATIONS = {"silu": 0, "gelu_tanh": 1}


def silu_and_mul(gate_up, out: Optional[torch.Tensor] = None, activation: str = "silu") -> torch.Tensor:
    """[T, 2I] -> [T, I]: act(first half) * second half, act = silu or the tanh form of gelu.  A `PartialSum` is
    added up on the way."""
    act = ACTIVATIONS[activation]
    if isinstance(gate_up, PartialSum):
        parts = gate_up.parts
        _dev(parts, out)
        S, T, two_i = parts.shape
        if out is None:
            out = torch.empty((T, two_i // 2), dtype=gate_up.rounds_to or torch.float32, device=parts.device)
        f = _fn("activation", "llm_silu_and_mul_parts", [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
        _check(f(_ptr(parts), S, _ptr(out), _dt(out), T, two_i // 2, act, _stream()), "silu_and_mul")
        return out
    _dev(gate_up, out)
    T, two_i = gate_up.shape
    inter = two_i // 2
    if out is None:
        out = torch.empty((T, inter), dtype=gate_up.dtype, device=gate_up.device)
    f = _fn("activation", "llm_silu_and_mul", [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(gate_up), _ptr(out), _dt(gate_up), T, inter, act, _stream()), "silu_and_mul")
    return out


def residual_add(h: torch.Tensor, delta: torch.Tensor) -> torch.Tensor:
    """h (float32) += delta, in place."""
    delta = as_tensor(delta)
    _dev(h, delta)
    if h.dtype != torch.float32 or h.shape != delta.shape:
        raise KernelError("residual_add wants a float32 residual and a delta of its shape")
    f = _fn("activation", "llm_residual_add", [c_void_p, c_void_p, c_int, c_longlong, c_void_p])
    _check(f(_ptr(h), _ptr(delta), _dt(delta), h.numel(), _stream()), "residual_add")
    return h


def qk_norm_rope_kv_write(qkv: torch.Tensor, cache: Optional[torch.Tensor], positions, token_entry, entry_slot,
                          block_table: Optional[torch.Tensor], q_norm_w, k_norm_w, eps: float, inv_freq,
                          rotary_dim: int, nq: int, nkv: int, d: int, page_size: int, has_kv: bool,
                          status: torch.Tensor, q_out: Optional[torch.Tensor] = None,
                          q_dtype: Optional[torch.dtype] = None, angles: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Normalise and rotate q and k, write k and v into the cache pages, return q [T, nq*d]
    in `q_dtype` (default: qkv's).
    cache: [num_pages, 2, nkv, page_size, d] of one stage (None with has_kv False).
    angles: the step's table from `rope_angles`, which saves every layer the sines and cosines."""
    parts, part_stride = 1, 0
    if isinstance(qkv, PartialSum):
        parts, part_stride = qkv.parts.shape[0], qkv.parts.stride(0)
        qkv = qkv.parts[0]
    _dev(qkv, cache, positions, token_entry, entry_slot, block_table, q_norm_w, k_norm_w, inv_freq, status, q_out)
    for t, n in ((positions, "positions"), (token_entry, "token_entry"), (entry_slot, "entry_slot"),
                 (block_table, "block_table")):
        _i32(t, n)
    T = qkv.shape[0]
    heads_total = nq + (2 * nkv if has_kv else 0)
    if qkv.shape[1] != heads_total * d:
        raise KernelError(f"qkv row is {qkv.shape[1]}, expected {heads_total * d}")
    if has_kv:
        if cache is None or block_table is None or tuple(cache.shape[1:]) != (2, nkv, page_size, d):
            raise KernelError("cache must be [pages, 2, kv_heads, page_size, head_dim]")
    for w in (q_norm_w, k_norm_w):
        if w is not None and (w.dtype != torch.float32 or w.numel() != d):
            raise KernelError("q/k norm weight must be float32 [head_dim]")
    if inv_freq is not None and (inv_freq.dtype != torch.float32 or inv_freq.numel() * 2 != rotary_dim):
        raise KernelError("inv_freq must be float32 [rotary_dim/2]")
    if angles is not None and (inv_freq is None or angles.dtype != torch.float32 or not angles.is_contiguous()
                               or tuple(angles.shape) != (T, inv_freq.numel(), 2)):
        raise KernelError("angles must be float32 [T, rotary_dim/2, 2] from rope_angles")
    if q_out is None:
        q_out = torch.empty((T, nq * d), dtype=q_dtype or qkv.dtype, device=qkv.device)
    f = _fn("rope_cache", "llm_qk_norm_rope_kv_write",
            [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
             c_void_p, c_void_p, c_float, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
             c_void_p, c_int, c_longlong, c_void_p, c_void_p])
    _check(f(_ptr(qkv), _dt(qkv), _ptr(q_out), _dt(q_out), _ptr(cache),
             _dt(cache) if cache is not None else _dt(q_out),
             _ptr(positions), _ptr(token_entry), _ptr(entry_slot), _ptr(block_table),
             block_table.shape[1] if block_table is not None else 0, _ptr(q_norm_w), _ptr(k_norm_w), float(eps),
             _ptr(inv_freq), rotary_dim if inv_freq is not None else 0, T, nq, nkv, d, page_size,
             1 if has_kv else 0, cache.shape[0] if cache is not None else 0, _ptr(status), parts, part_stride,
             _ptr(angles), _stream()),
           "qk_norm_rope_kv_write")
    return q_out


def qk_head_norm(qkv, q_norm_w, k_norm_w, eps: float, nq: int, nkv: int, d: int, has_kv: bool):
    """The first half of `qk_norm_rope_kv_write` alone: the per-head norms of q and k (a null weight:
    no norm), nothing rotated, nothing written to the cache.  Returns float32 q [T, nq*d] and k
    [T, nkv*d] (None without keys), for a position part that encodes them itself."""
    parts, part_stride = 1, 0
    if isinstance(qkv, PartialSum):
        parts, part_stride = qkv.parts.shape[0], qkv.parts.stride(0)
        qkv = qkv.parts[0]
    _dev(qkv, q_norm_w, k_norm_w)
    T = qkv.shape[0]
    if qkv.shape[1] != (nq + (2 * nkv if has_kv else 0)) * d:
        raise KernelError(f"qkv row is {qkv.shape[1]}, expected {(nq + (2 * nkv if has_kv else 0)) * d}")
    for w in (q_norm_w, k_norm_w):
        if w is not None and (w.dtype != torch.float32 or w.numel() != d):
            raise KernelError("q/k norm weight must be float32 [head_dim]")
    q = torch.empty((T, nq * d), dtype=torch.float32, device=qkv.device)
    k = torch.empty((T, nkv * d), dtype=torch.float32, device=qkv.device) if has_kv else None
    f = _fn("rope_cache", "llm_qk_head_norm",
            [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_int, c_int, c_int, c_int, c_int, c_int,
             c_longlong, c_void_p])
    _check(f(_ptr(qkv), _dt(qkv), _ptr(q), _ptr(k), _ptr(q_norm_w), _ptr(k_norm_w), float(eps), T, nq, nkv, d,
             1 if has_kv else 0, parts, part_stride, _stream()), "qk_head_norm")
    return q, k


def qk_store(q: torch.Tensor, k: Optional[torch.Tensor], qkv, cache: Optional[torch.Tensor], positions, token_entry,
             entry_slot, block_table: Optional[torch.Tensor], nq: int, nkv: int, d: int, page_size: int, has_kv: bool,
             status: torch.Tensor, q_dtype: torch.dtype) -> torch.Tensor:
    """The second half: q (float32, encoded by the position part) rounded to `q_dtype`; k (float32,
    encoded) and the v columns of `qkv` written into the pages of `cache`."""
    parts, part_stride = 1, 0
    if isinstance(qkv, PartialSum):
        parts, part_stride = qkv.parts.shape[0], qkv.parts.stride(0)
        qkv = qkv.parts[0]
    _dev(q, k, qkv, cache, positions, token_entry, entry_slot, block_table, status)
    T = qkv.shape[0]
    if q.dtype != torch.float32 or tuple(q.shape) != (T, nq * d) or (has_kv and (
            k is None or k.dtype != torch.float32 or tuple(k.shape) != (T, nkv * d))):
        raise KernelError("q and k must be float32 [T, heads * head_dim]")
    if has_kv and (cache is None or block_table is None or tuple(cache.shape[1:]) != (2, nkv, page_size, d)):
        raise KernelError("cache must be [pages, 2, kv_heads, page_size, head_dim]")
    q_out = torch.empty((T, nq * d), dtype=q_dtype, device=q.device)
    f = _fn("rope_cache", "llm_qk_store",
            [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
             c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_longlong, c_void_p])
    _check(f(_ptr(q), _ptr(k), _ptr(qkv), _dt(qkv), _ptr(q_out), _dt(q_out), _ptr(cache),
             _dt(cache) if cache is not None else _dt(q_out), _ptr(positions), _ptr(token_entry), _ptr(entry_slot),
             _ptr(block_table), block_table.shape[1] if block_table is not None else 0, T, nq, nkv, d, page_size,
             1 if has_kv else 0, cache.shape[0] if cache is not None else 0, _ptr(status), parts, part_stride,
             _stream()), "qk_store")
    return q_out


ROPE_TABLE_MIN_TOKENS = 64     # steps of fewer tokens compute their angles inside the kernel, before it waits


def rope_angles(positions: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """(sin, cos) of float32(position) * inv_freq for every token of a step: float32 [T, rotary_dim/2, 2],
    computed once for all layers (a prompt portion's rotation kernel is bound by its instructions, and
    most of them are these)."""
    _dev(positions, inv_freq)
    _i32(positions, "positions")
    T, half = positions.numel(), inv_freq.numel()
    out = torch.empty((T, half, 2), dtype=torch.float32, device=positions.device)
    f = _fn("rope_cache", "llm_rope_angles", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p])
    _check(f(_ptr(positions), _ptr(inv_freq), _ptr(out), T, half, _stream()), "rope_angles")
    return out


def paged_attention_generic(q: torch.Tensor, cache: torch.Tensor, positions, token_entry, entry_slot,
                            block_table: torch.Tensor, nq: int, nkv: int, d: int, page_size: int,
                            window: Optional[int], scale: float, status: torch.Tensor,
                            out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal attention of every token in q [T, nq*d] over its request's pages."""
    _dev(q, cache, positions, token_entry, entry_slot, block_table, status, out)
    for t, n in ((positions, "positions"), (token_entry, "token_entry"), (entry_slot, "entry_slot"),
                 (block_table, "block_table")):
        _i32(t, n)
    T = q.shape[0]
    if q.shape[1] != nq * d or tuple(cache.shape[1:]) != (2, nkv, page_size, d):
        raise KernelError("q must be [T, heads*head_dim] and cache [pages, 2, kv_heads, page_size, head_dim]")
    if out is None:
        out = torch.empty_like(q)
    f = _fn("attention_generic", "llm_paged_attention_generic",
            [c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
             c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p])
    _check(f(_ptr(q), _ptr(out), _dt(q), _ptr(cache), _dt(cache), _ptr(positions), _ptr(token_entry),
             _ptr(entry_slot), _ptr(block_table), block_table.shape[1], T, nq, nkv, d, page_size,
             int(window) if window else 0, float(scale), cache.shape[0], _ptr(status), _stream()),
           "paged_attention_generic")
    return out


NORM_SCOPES = {None: 0, "none": 0, "head": 1, "projection": 2}


def attention_prepare(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, biases, q_norm_w, k_norm_w,
                      norm_scope, eps: float, temperature, keys: Optional[torch.Tensor],
                      values: Optional[torch.Tensor], positions, token_entry, entry_slot,
                      block_table: Optional[torch.Tensor], nq: int, nkv: int, dk: int, dv: int, page_size: int,
                      status: torch.Tensor, q_dtype: torch.dtype, rotation=None) -> torch.Tensor:
    """From a float32 projection [T, n] whose columns hold q (from q_off), k (from k_off) and v (from v_off):
    add the biases (`biases` = (bq, bk, bv), any of them None), normalise q and k in 32-bit (`norm_scope`
    'head': each head by itself with a weight [dk]; 'projection': all heads of a token together with a
    weight over the whole projection; None), multiply q by the query temperature 1 + coef * ln(floor((p + 1)
    / every) + 1) (`temperature` = (coef, every) or None), return q [T, nq*dk] in `q_dtype` and write k and
    v into the token's place in `keys` [pages, nkv, page, dk] and `values` [pages, nkv, page, dv] (views
    with any page stride).  keys None: a mixer that writes no keys and values.  `rotation` = (freq, dims, mag,
    pairs): after the norm the first `dims` entries of every q and k head turn by position * freq[i] (float32
    [dims / 2]), pairs of neighbours (2i, 2i + 1) if `pairs` else (i, i + dims / 2), sine and cosine times `mag`."""
    if proj.dtype != torch.float32 or proj.dim() != 2 or proj.stride(1) != 1 or not proj.is_cuda:
        raise KernelError("proj must be a float32 CUDA matrix with unit stride along its rows")
    bq, bk, bv = biases if biases is not None else (None, None, None)
    _dev(bq, bk, bv, q_norm_w, k_norm_w, positions, token_entry, entry_slot, block_table, status)
    T, n = proj.shape
    if max(q_off + nq * dk, (k_off + nkv * dk) if keys is not None else 0, (v_off + nkv * dv) if keys is not None else 0) > n:
        raise KernelError("the projection is narrower than its q, k and v pieces")
    scope = NORM_SCOPES[norm_scope]
    for w, size in ((q_norm_w, nq * dk if scope == 2 else dk), (k_norm_w, nkv * dk if scope == 2 else dk)):
        if w is not None and (w.dtype != torch.float32 or w.numel() != size):
            raise KernelError(f"a q/k norm weight must be float32 [{size}]")
    for b, size in ((bq, nq * dk), (bk, nkv * dk), (bv, nkv * dv)):
        if b is not None and (b.dtype != torch.float32 or b.numel() != size):
            raise KernelError(f"a projection bias must be float32 [{size}]")
    kps = vps = pages = 0
    if keys is not None:
        for c, w in ((keys, dk), (values, dv)):
            if (c is None or not c.is_cuda or c.dim() != 4 or tuple(c.shape[1:]) != (nkv, page_size, w)
                    or c[0].stride() != (page_size * w, w, 1)):
                raise KernelError("keys / values must be [pages, kv_heads, page_size, width] with dense pages")
        if keys.dtype != values.dtype or block_table is None:
            raise KernelError("keys and values must share a dtype and come with a block table")
        kps, vps, pages = keys.stride(0), values.stride(0), keys.shape[0]
    coef, every = (float(temperature[0]), int(temperature[1])) if temperature is not None else (0.0, 0)
    freq, rot_dims, rot_mag, rot_pairs = rotation if rotation is not None else (None, 0, 1.0, False)
    if freq is not None and (not freq.is_cuda or freq.dtype != torch.float32 or freq.numel() != rot_dims // 2):
        raise KernelError("the rotation's frequencies must be float32 [dims / 2] on the device")
    q = torch.empty((T, nq * dk), dtype=q_dtype, device=proj.device)
    f = _fn("attention_prepare", "llm_attention_prepare",
            [c_void_p, c_longlong, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_float,
             c_float, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_longlong, c_longlong, c_void_p, c_void_p,
             c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_float,
             c_int, c_void_p])
    _check(f(_ptr(proj), proj.stride(0), q_off, k_off, v_off, _ptr(bq), _ptr(bk), _ptr(bv), _ptr(q_norm_w),
             _ptr(k_norm_w), scope, float(eps), coef, every, _ptr(q), _dt(q), _ptr(keys), _ptr(values),
             _dt(keys) if keys is not None else 0, kps, vps, _ptr(positions), _ptr(token_entry), _ptr(entry_slot),
             _ptr(block_table), block_table.shape[1] if block_table is not None else 0, T, nq, nkv, dk, dv, page_size,
             pages, _ptr(status), _ptr(freq), int(rot_dims), float(rot_mag), 1 if rot_pairs else 0, _stream()),
           "attention_prepare")
    return q


def gate_mul(a: torch.Tensor, gate: Optional[torch.Tensor], gate_off: int, out: torch.Tensor, out_off: int,
             kind: Optional[str], scale: float = 1.0, per_head: int = 0) -> None:
    """out[:, out_off : out_off + w] = a * gate_fn(gate[:, gate_off : gate_off + w]) * scale for a contiguous
    a [T, w]; gate is float32; `kind` 'sigmoid', 'silu' or None (no gate: scale and place only).  `per_head` > 0:
    one gate value per head of that many channels (gate[:, gate_off + channel // per_head])."""
    _dev(a)
    T, w = a.shape
    if kind is None:
        gate = None
    if (gate is not None and (gate.dtype != torch.float32 or gate.stride(1) != 1)) or out.stride(1) != 1 or out.dtype != a.dtype:
        raise KernelError("gate must be float32, out of a's dtype, both with unit stride along rows")
    f = _fn("attention_prepare", "llm_gate_mul",
            [c_void_p, c_int, c_void_p, c_longlong, c_int, c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_float, c_int,
             c_void_p])
    _check(f(_ptr(a), _dt(a), _ptr(gate), gate.stride(0) if gate is not None else 0, gate_off, _ptr(out), out.stride(0),
             out_off, T, w, {None: 0, "sigmoid": 1, "silu": 2}[kind], float(scale), int(per_head), _stream()), "gate_mul")


def paged_attention_generic_kv(q: torch.Tensor, keys: torch.Tensor, values: torch.Tensor, positions, token_entry,
                               entry_slot, block_table: torch.Tensor, nq: int, nkv: int, dk: int, dv: int,
                               page_size: int, window: Optional[int], scale: float, status: torch.Tensor,
                               out: torch.Tensor, out_off: int = 0, gate: Optional[torch.Tensor] = None,
                               gate_off: int = 0, out_scale: float = 1.0, dist_bias: Optional[torch.Tensor] = None,
                               gate_per_head: bool = False, rows: Optional[torch.Tensor] = None,
                               head_scale: Optional[torch.Tensor] = None, log_bias=None,
                               values_in_keys: bool = False, keep_first: int = 0,
                               sink: Optional[float] = None) -> torch.Tensor:
    """Causal attention of every token in q [T, nq*dk] over its request's pages of `keys` [pages, nkv, page,
    dk] and `values` [pages, nkv, page, dv] (views with any page stride), written into columns out_off ..
    out_off + nq*dv of `out`, times sigmoid(gate[:, gate_off + ...]) (float32, optional; one value per output
    channel, or per head with `gate_per_head`) and `out_scale`.  `dist_bias` (float32 [len, nq]): row min(i - j,
    len - 1) is added to the scaled scores of query i and key j.  `rows` (int32): only these tokens are worked on
    (-1 entries are padding).  `head_scale` (float32 [nq]) multiplies each head's scaled scores; `log_bias` = (r1, r2),
    float32 [nq] each, takes r1[h] * ln(1 + r2[h] * (i - j)) off them.  `values_in_keys`: `values` is None and the
    values are the first dv entries of the key rows.  `keep_first`: with a window, the sequence's first so many keys
    stay visible to every later query.  `sink`: a score whose exponential joins the softmax's denominator without a
    value (None: ordinary softmax)."""
    r1, r2 = log_bias if log_bias is not None else (None, None)
    _dev(q, positions, token_entry, entry_slot, block_table, status, dist_bias, rows, head_scale, r1, r2)
    _i32(rows, "rows")
    for v in (head_scale, r1, r2):
        if v is not None and (v.dtype != torch.float32 or v.numel() != nq):
            raise KernelError("head_scale and the log bias's numbers must be float32 [heads]")
    value_row = 0
    if values_in_keys:
        if values is not None or dv > dk:
            raise KernelError("values_in_keys: no values tensor, and dv at most dk")
        values, value_row = keys, dk
    if dist_bias is not None and (dist_bias.dtype != torch.float32 or dist_bias.dim() != 2 or dist_bias.shape[1] != nq):
        raise KernelError("dist_bias must be float32 [distances, heads]")
    T = q.shape[0]
    for c, w in ((keys, dk), (values, dk if values_in_keys else dv)):
        if (not c.is_cuda or c.dim() != 4 or tuple(c.shape[1:]) != (nkv, page_size, w)
                or c[0].stride() != (page_size * w, w, 1)):
            raise KernelError("keys / values must be [pages, kv_heads, page_size, width] with dense pages")
    if q.shape[1] != nq * dk or out.dtype != q.dtype or out.stride(1) != 1 or out.shape[0] != T:
        raise KernelError("q must be [T, heads*dk] and out a matrix of q's dtype with T rows")
    if gate is not None and (gate.dtype != torch.float32 or gate.stride(1) != 1):
        raise KernelError("gate must be float32 with unit stride along rows")
    f = _fn("attention_generic", "llm_paged_attention_generic_kv",
            [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_longlong, c_longlong, c_void_p, c_void_p, c_void_p,
             c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_longlong,
             c_int, c_float, c_longlong, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
             c_longlong, c_int, c_int, c_float, c_void_p])
    _check(f(_ptr(q), _ptr(out), _dt(q), _ptr(keys), _ptr(values), _dt(keys), keys.stride(0), values.stride(0),
             _ptr(positions), _ptr(token_entry), _ptr(entry_slot), _ptr(block_table), block_table.shape[1],
             rows.numel() if rows is not None else T, nq, nkv,
             dk, dv, page_size, int(window) if window else 0, float(scale), keys.shape[0], _ptr(gate),
             gate.stride(0) if gate is not None else 0, gate_off, float(out_scale), out.stride(0), out_off,
             _ptr(status), _ptr(dist_bias), dist_bias.shape[0] if dist_bias is not None else 0,
             1 if gate_per_head else 0, _ptr(rows), _ptr(head_scale), _ptr(r1), _ptr(r2), value_row,
             int(keep_first) if window else 0, 0 if sink is None else 1, float(sink or 0.0), _stream()),
           "paged_attention_generic_kv")
    return out


# ---- a short convolution in front of a sublayer, the norm after the sum ------------------------------
def short_conv(x: torch.Tensor, w: torch.Tensor, kept: Optional[torch.Tensor], batch, out_dtype: torch.dtype) -> torch.Tensor:
    """u[t] = x[t] + sum_j w[:, j] * x_(t - taps + 1 + j) along each request's tokens, channel by channel, in 32-bit,
    stored in `out_dtype`.  x: the float32 stream [T, W]; w: float32 [W, taps]; `kept`: float32 [slots, taps - 1, W]
    (a view with any slot stride), the rows of the last taps - 1 positions of each request at ring row position mod
    (taps - 1), read for tokens whose predecessors are not in this step; rows before a sequence's start are zero.
    `batch` gives positions, token_entry, entry_slot, entry_q_start."""
    _dev(x, w, batch.positions, batch.token_entry, batch.entry_slot, batch.entry_q_start)
    T, W = x.shape
    if x.dtype != torch.float32 or w.dtype != torch.float32 or w.dim() != 2 or w.shape[0] != W:
        raise KernelError("short_conv wants a float32 stream [T, W] and float32 taps [W, taps]")
    taps = w.shape[1]
    if taps > 1 and (kept is None or kept.dtype != torch.float32 or tuple(kept.shape[1:]) != (taps - 1, W)
                     or kept[0].stride() != (W, 1)):
        raise KernelError("kept rows must be float32 [slots, taps - 1, W] with dense slots")
    out = torch.empty((T, W), dtype=out_dtype, device=x.device)
    f = _fn("conv_norm", "llm_short_conv",
            [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
             c_int, c_void_p])
    _check(f(_ptr(x), _ptr(w), _ptr(out), _dt(out), _ptr(kept) if taps > 1 else None, kept.stride(0) if taps > 1 else 0,
             _ptr(batch.positions), _ptr(batch.token_entry), _ptr(batch.entry_slot), _ptr(batch.entry_q_start), T, W, taps,
             _stream()), "short_conv")
    return out


def scaled_add_norm(x: torch.Tensor, y, weight: torch.Tensor, alpha: float, eps: float, kept: Optional[torch.Tensor],
                    batch) -> torch.Tensor:
    """x (float32 [T, W], in place) <- rmsnorm(alpha * x + y) * weight, row by row in 32-bit: the norm that follows
    the sum.  y may be a `PartialSum`.  `kept` (float32 [slots, R, W], any slot stride): the OLD row of each token
    among the last R of its portion is stored at ring row position mod R of its request (what the convolution in
    front of the sublayer reads in the request's next step)."""
    parts, part_stride = 1, 0
    if isinstance(y, PartialSum):
        if y.rounds_to is not None:
            y = as_tensor(y)
        else:
            parts, part_stride = y.parts.shape[0], y.parts.stride(0)
            y = y.parts[0]
    _dev(x, weight)
    T, W = x.shape
    if not y.is_cuda or y.dim() != 2 or y.stride(1) != 1 or tuple(y.shape) != (T, W):
        raise KernelError("y must be a CUDA matrix of x's shape with unit stride along its rows")
    if x.dtype != torch.float32 or weight.dtype != torch.float32 or weight.numel() != W:
        raise KernelError("scaled_add_norm wants a float32 stream and a float32 weight of the row length")
    R = 0
    if kept is not None:
        R = kept.shape[1]
        if kept.dtype != torch.float32 or kept.dim() != 3 or kept.shape[2] != W or (R and kept[0].stride() != (W, 1)):
            raise KernelError("kept rows must be float32 [slots, R, W] with dense slots")
    f = _fn("conv_norm", "llm_scaled_add_norm",
            [c_void_p, c_void_p, c_int, c_longlong, c_int, c_longlong, c_void_p, c_float, c_float, c_void_p, c_longlong, c_int,
             c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p])
    _check(f(_ptr(x), _ptr(y), _dt(y), y.stride(0), parts, part_stride, _ptr(weight), float(alpha), float(eps),
             _ptr(kept) if R else None, kept.stride(0) if R else 0, R, _ptr(batch.positions), _ptr(batch.token_entry),
             _ptr(batch.entry_slot), _ptr(batch.entry_q_start), _ptr(batch.entry_q_len), T, W, _stream()), "scaled_add_norm")
    return x


# ---- latent attention ---------------------------------------------------------------------------
def latent_prepare(proj: torch.Tensor, dq_off: int, dkv_off: int, Q: int, R: int, P: int, dims: int, wq: torch.Tensor,
                   wkv: Optional[torch.Tensor], eps: float, inv_freq: Optional[torch.Tensor], keys: Optional[torch.Tensor],
                   batch, block_table: Optional[torch.Tensor], page_size: int, status: torch.Tensor,
                   q_dtype: torch.dtype, rot_pairs: bool = False, rot_mag: float = 1.0) -> torch.Tensor:
    """From the float32 projection [T, n] with the query latent in columns dq_off .. + Q and (if `keys`) the key/value
    latent and the shared key part in columns dkv_off .. + R + P: returns rmsnorm(query latent) * wq as [T, Q] in
    `q_dtype` and writes [rmsnorm(latent) * wkv | rotated key part] into the token's row of `keys` [pages, 1, page, R +
    P].  The rotation turns the first `dims` entries of the key part (half-split pairs, or with `rot_pairs` neighbours
    2i and 2i + 1) by position * inv_freq, sine and cosine times `rot_mag`."""
    if proj.dtype != torch.float32 or proj.dim() != 2 or proj.stride(1) != 1 or not proj.is_cuda:
        raise KernelError("proj must be a float32 CUDA matrix with unit stride along its rows")
    _dev(wq, wkv, inv_freq, batch.positions, batch.token_entry, batch.entry_slot, block_table, status)
    T, n = proj.shape
    if dq_off + Q > n or (keys is not None and dkv_off + R + P > n):
        raise KernelError("the projection is narrower than its pieces")
    if wq.dtype != torch.float32 or wq.numel() != Q or (wkv is not None and (wkv.dtype != torch.float32 or wkv.numel() != R)):
        raise KernelError("the latent norms' weights must be float32 of the latents' sizes")
    if inv_freq is not None and (inv_freq.dtype != torch.float32 or inv_freq.numel() < dims // 2):
        raise KernelError("inv_freq must be float32 [dims / 2]")
    kps = pages = 0
    if keys is not None:
        if (not keys.is_cuda or keys.dim() != 4 or tuple(keys.shape[1:]) != (1, page_size, R + P)
                or keys[0].stride() != (page_size * (R + P), R + P, 1) or block_table is None):
            raise KernelError("keys must be [pages, 1, page_size, R + P] with dense pages, and come with a block table")
        kps, pages = keys.stride(0), keys.shape[0]
    cq = torch.empty((T, Q), dtype=q_dtype, device=proj.device)
    f = _fn("latent_attention", "llm_latent_prepare",
            [c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_float, c_void_p, c_void_p,
             c_int, c_void_p, c_int, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p,
             c_int, c_float, c_void_p])
    _check(f(_ptr(proj), proj.stride(0), dq_off, dkv_off, Q, R, P, dims, _ptr(wq), _ptr(wkv), float(eps), _ptr(inv_freq),
             _ptr(cq), _dt(cq), _ptr(keys), _dt(keys) if keys is not None else 0, kps, _ptr(batch.positions),
             _ptr(batch.token_entry), _ptr(batch.entry_slot), _ptr(block_table),
             block_table.shape[1] if block_table is not None else 0, T, page_size, pages, _ptr(status),
             1 if rot_pairs else 0, float(rot_mag), _stream()),
           "latent_prepare")
    return cq


def latent_q_split(q: torch.Tensor, positions: torch.Tensor, inv_freq: Optional[torch.Tensor], H: int, D: int, P: int,
                   R: int, dims: int, dtype: torch.dtype, rot_pairs: bool = False, rot_mag: float = 1.0):
    """q: float32 [T, H * (D + P)], per head [D unrotated | P to rotate].  Returns (qn [H, T, D] in `dtype`, the
    unrotated parts head-major; packed [T, H * (R + P)] in `dtype` whose columns R .. R + P of every head hold the
    rotated parts and whose first R columns per head are left for the caller to fill)."""
    _dev(q, positions, inv_freq)
    T = q.shape[0]
    if q.dtype != torch.float32 or q.shape[1] != H * (D + P):
        raise KernelError("q must be float32 [T, heads * (D + P)]")
    qn = torch.empty((H, T, D), dtype=dtype, device=q.device)
    packed = torch.empty((T, H * (R + P)), dtype=dtype, device=q.device)
    f = _fn("latent_attention", "llm_latent_q_split",
            [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
             c_void_p])
    _check(f(_ptr(q), _ptr(qn), _ptr(packed), _dt(qn), _ptr(positions), _ptr(inv_freq), T, H, D, P, R, dims,
             1 if rot_pairs else 0, float(rot_mag), _stream()),
           "latent_q_split")
    return qn, packed


def latent_attention_supported(R: int, P: int) -> bool:
    """Whether the tensor-core kernel over cached latent rows takes a latent of R and a rotated part of P entries."""
    return bool(_fn("latent_attention", "llm_latent_attention_supported", [c_int, c_int])(R, P))


def latent_attention(q: torch.Tensor, rows_cache: torch.Tensor, positions, token_entry, entry_slot,
                     block_table: torch.Tensor, H: int, R: int, P: int, page_size: int, window: Optional[int], scale: float,
                     status: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """Causal softmax attention of the packed queries q (bfloat16 [T, H * (R + P)]) over each token's pages of
    `rows_cache` (bfloat16 [pages, 1, page, R + P]): the scores run over all R + P entries of a row, the values are
    its first R entries.  `window`: a token sees itself and the window - 1 rows before it (None: all).  Writes the
    weighted latent sums into `out` (bfloat16 [T, H * R])."""
    _dev(q, rows_cache, positions, token_entry, entry_slot, block_table, status, out)
    T, DK = q.shape[0], R + P
    if q.dtype != torch.bfloat16 or rows_cache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("latent_attention runs in bfloat16")
    if q.dim() != 2 or q.shape[1] != H * DK or not q.is_contiguous() or tuple(out.shape) != (T, H * R) or not out.is_contiguous():
        raise KernelError("q must be a dense [T, heads * (R + P)] and out a dense [T, heads * R]")
    if (rows_cache.dim() != 4 or tuple(rows_cache.shape[1:]) != (1, page_size, DK)
            or rows_cache[0].stride() != (page_size * DK, DK, 1)):
        raise KernelError("rows_cache must be [pages, 1, page_size, R + P] with dense pages")
    splits = _fn("latent_attention", "llm_latent_attention_splits", [c_int, c_int, c_int, c_int, c_int])(
        T, H, int(window or 0), block_table.shape[1], page_size)
    part_acc = part_ml = None
    if splits > 1:          # few tokens: a token's rows are dealt to several CTAs, whose sums a second kernel merges
        part_acc = torch.empty((T, splits, H, R), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((T, splits, H, 2), dtype=torch.float32, device=q.device)
    f = _fn("latent_attention", "llm_latent_attention",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
             c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p])
    _check(f(_ptr(q), _ptr(out), _ptr(part_acc), _ptr(part_ml), splits, _ptr(rows_cache), rows_cache.stride(0), _ptr(positions),
             _ptr(token_entry), _ptr(entry_slot), _ptr(block_table), block_table.shape[1], T, H, R, P, page_size,
             int(window or 0), float(scale), rows_cache.shape[0], _ptr(status), _stream()), "latent_attention")
    return out


# ---- gated linear attention ------------------------------------------------------------------
GLA_FULL, GLA_LOCAL, GLA_OUT = 0, 1, 2


def gla_supported(d: int, v: int) -> bool:
    return bool(_fn("linear_attention", "llm_gla_supported", [c_int, c_int])(d, v))


def gla_decay(proj: torch.Tensor, a_off: int, rank: int, w2t: torch.Tensor, b2: Optional[torch.Tensor],
              tau: float) -> torch.Tensor:
    """The decays alpha = sigmoid(proj[:, a_off : a_off + rank] @ w2t + b2) ^ (1 / tau) as float32 [T, channels]
    (computed as exp(ln(sigmoid(z)) / tau), which neither side of z overflows); `w2t` is the projection's
    second half transposed, float32 [rank, channels]."""
    _dev(w2t, b2)
    if proj.dtype != torch.float32 or proj.stride(1) != 1 or w2t.dtype != torch.float32 or w2t.shape[0] != rank:
        raise KernelError("gla_decay wants a float32 projection and a float32 w2t [rank, channels]")
    T, C = proj.shape[0], w2t.shape[1]
    la = torch.empty((T, C), dtype=torch.float32, device=proj.device)
    f = _fn("linear_attention", "llm_gla_decay",
            [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_float, c_void_p, c_int, c_int, c_void_p])
    _check(f(_ptr(proj), proj.stride(0), a_off, rank, _ptr(w2t), _ptr(b2), float(tau), _ptr(la), T, C, _stream()),
           "gla_decay")
    return la


def gla_scan(proj: torch.Tensor, offs, alpha: torch.Tensor, norm_w: torch.Tensor, eps: float, q_scale: float,
             out_scale: float, out: torch.Tensor, out_off: int, state: torch.Tensor, entry_slot, entry_q_start,
             entry_q_len, items: Optional[torch.Tensor], num_items: int, mode: int,
             scratch_s: Optional[torch.Tensor], scratch_a: Optional[torch.Tensor], H: int, D: int, V: int) -> None:
    """The recurrence S <- diag(alpha) S + k v^T, o = S^T q over the tokens of each work item, per head, with
    the per-head RMS norm of o (weight `norm_w` [V]), the silu output gate and `out_scale` applied before
    the store into columns out_off .. out_off + H*V of `out`.  `offs` = (q, k, v, g) column offsets in the
    float32 projection; `alpha` float32 [T, H*D] from `gla_decay`; `state` float32 [slots, H, D, V]; see
    csrc/linear_attention.cu for the modes."""
    la = alpha
    _dev(la, norm_w, state, entry_slot, entry_q_start, entry_q_len, items, scratch_s, scratch_a)
    if (proj.dtype != torch.float32 or proj.stride(1) != 1 or la.dtype != torch.float32 or state.dtype != torch.float32
            or tuple(state.shape[1:]) != (H, D, V) or norm_w.dtype != torch.float32 or norm_w.numel() != V
            or out.stride(1) != 1):
        raise KernelError("gla_scan: float32 projection, decays and state [slots, H, D, V]; norm weight [V]")
    q_off, k_off, v_off, g_off = offs
    f = _fn("linear_attention", "llm_gla_scan",
            [c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_float, c_float, c_float, c_void_p,
             c_int, c_longlong, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p,
             c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(proj), proj.stride(0), q_off, k_off, v_off, g_off, _ptr(la), _ptr(norm_w), float(eps),
             float(q_scale), float(out_scale), _ptr(out), _dt(out), out.stride(0), out_off, _ptr(state),
             _ptr(entry_slot), _ptr(entry_q_start), _ptr(entry_q_len), _ptr(items), num_items, mode,
             _ptr(scratch_s), _ptr(scratch_a), H, D, V, _stream()), "gla_scan")


def gla_step(proj: torch.Tensor, offs, alpha: torch.Tensor, norm_w: torch.Tensor, eps: float, q_scale: float,
             out_scale: float, out: torch.Tensor, out_off: int, state: torch.Tensor, entry_slot, entry_q_start,
             num_entries: int, H: int, D: int, V: int, decay=None) -> None:
    """`gla_scan` for a step whose entries all bring one token: the state is streamed through once instead
    of being held, which is what a decode step wants (same arguments, same result up to summation order).
    With `alpha` None the kernel makes the decays itself from `decay` = (a_off, rank, w2t, b2, tau), the
    arguments of `gla_decay`: one launch fewer."""
    la = alpha
    a_off, rank, w2t, b2, tau = decay if decay is not None else (0, 0, None, None, 1.0)
    if la is None and w2t is None:
        raise KernelError("gla_step wants the decays or what they are made from")
    _dev(la, norm_w, state, entry_slot, entry_q_start, w2t, b2)
    if (proj.dtype != torch.float32 or proj.stride(1) != 1 or (la is not None and la.dtype != torch.float32) or state.dtype != torch.float32
            or tuple(state.shape[1:]) != (H, D, V) or norm_w.dtype != torch.float32 or norm_w.numel() != V
            or out.stride(1) != 1):
        raise KernelError("gla_step: float32 projection, decays and state [slots, H, D, V]; norm weight [V]")
    q_off, k_off, v_off, g_off = offs
    f = _fn("linear_attention", "llm_gla_step",
            [c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_float, c_float, c_float, c_void_p,
             c_int, c_longlong, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
             c_void_p, c_float, c_void_p])
    _check(f(_ptr(proj), proj.stride(0), q_off, k_off, v_off, g_off, _ptr(la), _ptr(norm_w), float(eps),
             float(q_scale), float(out_scale), _ptr(out), _dt(out), out.stride(0), out_off, _ptr(state),
             _ptr(entry_slot), _ptr(entry_q_start), num_entries, H, D, V, a_off, rank, _ptr(w2t), _ptr(b2), float(tau),
             _stream()), "gla_step")


def gla_chain(state: torch.Tensor, scratch_s: torch.Tensor, scratch_a: torch.Tensor, chains: torch.Tensor,
              num_chains: int, entry_slot, H: int, D: int, V: int) -> None:
    """Per (chain, head): walk the chain's chunks in order, leaving in scratch_s[c] the state that enters
    chunk c and in the request's slot the state after the last one."""
    _dev(state, scratch_s, scratch_a, chains, entry_slot)
    f = _fn("linear_attention", "llm_gla_chain",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(state), _ptr(scratch_s), _ptr(scratch_a), _ptr(chains), num_chains, _ptr(entry_slot), H, D, V,
             _stream()), "gla_chain")


# ---- recurrences with a decay per (token, head) or per head (retention, matrix memories) -------------
def rotate_qk(proj: torch.Tensor, q_off: int, k_off: int, heads_q: int, heads_k: int, D: int, dims: int,
              inv_freq: torch.Tensor, positions: torch.Tensor) -> None:
    """In place on the float32 projection: pairs (i, i + dims/2) of every head of q (from column q_off) and of k
    (from k_off) turn by the angle float(position) * inv_freq[i]."""
    _dev(inv_freq, positions)
    _i32(positions, "positions")
    if (proj.dtype != torch.float32 or proj.stride(1) != 1 or inv_freq.dtype != torch.float32
            or inv_freq.numel() * 2 != dims):
        raise KernelError("rotate_qk wants a float32 projection and inv_freq float32 [dims/2]")
    f = _fn("linear_attention", "llm_rotate_qk",
            [c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p])
    _check(f(_ptr(proj), proj.stride(0), q_off, k_off, heads_q, heads_k, D, dims, _ptr(inv_freq), _ptr(positions),
             proj.shape[0], _stream()), "rotate_qk")


def recur_gates(proj: torch.Tensor, i_off: int, f_off: int, i_bias: torch.Tensor, f_bias: torch.Tensor, cap: float,
                state: torch.Tensor, m_off: int, head_stride: int, entry_slot, entry_q_start, entry_q_len,
                num_entries: int, H: int) -> torch.Tensor:
    """The gates of a matrix memory over the tokens of each entry, in order: float32 [3, T, H] = (keep, put,
    floor) per (token, head), see csrc/linear_attention.cu; the running maximum in `state` moves on."""
    _dev(i_bias, f_bias, state, entry_slot, entry_q_start, entry_q_len)
    if proj.dtype != torch.float32 or proj.stride(1) != 1 or state.dtype != torch.float32:
        raise KernelError("recur_gates wants a float32 projection and state")
    T = proj.shape[0]
    gates = torch.empty((3, T, H), dtype=torch.float32, device=proj.device)
    f = _fn("linear_attention", "llm_recur_gates",
            [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_float, c_void_p, c_longlong, c_void_p, c_longlong,
             c_longlong, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p])
    _check(f(_ptr(proj), proj.stride(0), i_off, f_off, _ptr(i_bias), _ptr(f_bias), float(cap), _ptr(gates), T,
             _ptr(state), m_off, head_stride, state.stride(0), _ptr(entry_slot), _ptr(entry_q_start),
             _ptr(entry_q_len), num_entries, H, _stream()), "recur_gates")
    return gates


GATE_KINDS = {None: 0, "sigmoid": 1, "silu": 2}


def recur_scan(proj: torch.Tensor, offs, alpha: torch.Tensor, a_tok: int, a_head: int,
               kscale: Optional[torch.Tensor], nfloor: Optional[torch.Tensor], norm_w: Optional[torch.Tensor],
               norm_stride: int, gate: Optional[str], eps: float, q_scale: float, out_scale: float, out: torch.Tensor,
               out_off: int, state: torch.Tensor, head_stride: int, entry_slot, entry_q_start, entry_q_len,
               items: Optional[torch.Tensor], num_items: int, mode: int, scratch_s: Optional[torch.Tensor],
               scratch_a: Optional[torch.Tensor], H: int, D: int, V: int) -> None:
    """`gla_scan` for recurrences whose decay is one number per (token, head): alpha[token * a_tok + head * a_head]
    (a_tok 0: a constant per head).  `kscale` [T, H]: the input scale e; `nfloor` [T, H]: the state keeps a
    normaliser n beside S and o is divided by max(|n . q|, floor) + 1e-6.  `norm_w` None: a weightless output
    norm; else its index is head * norm_stride + channel.  `state` [slots, ...] holds per head S [D, V], then
    n [D], then what else the mixer keeps, `head_stride` floats a head."""
    _dev(alpha, kscale, nfloor, norm_w, state, entry_slot, entry_q_start, entry_q_len, items, scratch_s, scratch_a)
    if proj.dtype != torch.float32 or proj.stride(1) != 1 or alpha.dtype != torch.float32 or state.dtype != torch.float32 \
            or out.stride(1) != 1:
        raise KernelError("recur_scan: float32 projection, decays and state")
    q_off, k_off, v_off, g_off = offs
    f = _fn("linear_attention", "llm_recur_scan",
            [c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_float, c_float, c_float, c_void_p,
             c_int, c_longlong, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p,
             c_void_p, c_int, c_int, c_int, c_int, c_longlong, c_longlong, c_void_p, c_void_p, c_int, c_int, c_longlong,
             c_longlong, c_void_p])
    _check(f(_ptr(proj), proj.stride(0), q_off, k_off, v_off, g_off, _ptr(alpha), _ptr(norm_w), float(eps),
             float(q_scale), float(out_scale), _ptr(out), _dt(out), out.stride(0), out_off, _ptr(state),
             _ptr(entry_slot), _ptr(entry_q_start), _ptr(entry_q_len), _ptr(items), num_items, mode,
             _ptr(scratch_s), _ptr(scratch_a), H, D, V, 1, a_tok, a_head, _ptr(kscale), _ptr(nfloor), norm_stride,
             GATE_KINDS[gate], head_stride, state.stride(0), _stream()), "recur_scan")


def recur_step(proj: torch.Tensor, offs, alpha: Optional[torch.Tensor], a_strides, norm_w: Optional[torch.Tensor],
               norm_stride: int, gate: Optional[str], eps: float, q_scale: float, out_scale: float, out: torch.Tensor,
               out_off: int, state: torch.Tensor, head_stride: int, entry_slot, entry_q_start, num_entries: int,
               H: int, D: int, V: int, rotation=None, gates=None) -> None:
    """`recur_scan` for a step whose entries all bring one token.  `alpha` with `a_strides` = (token, head,
    channel) strides: the decays as they are.  `rotation` = (inv_freq, dims, positions): q and k are rotated
    inside the kernel.  `gates` = (i_off, f_off, i_bias, f_bias, cap): a matrix memory's gates are made inside
    the kernel (alpha None), the state keeps a normaliser and the running maximum after it."""
    inv_freq, dims, positions = rotation if rotation is not None else (None, 0, None)
    i_off, f_off, i_bias, f_bias, cap = gates if gates is not None else (0, 0, None, None, 0.0)
    if alpha is None and gates is None:
        raise KernelError("recur_step wants the decays or what they are made from")
    _dev(alpha, norm_w, state, entry_slot, entry_q_start, inv_freq, positions, i_bias, f_bias)
    if proj.dtype != torch.float32 or proj.stride(1) != 1 or state.dtype != torch.float32 or out.stride(1) != 1:
        raise KernelError("recur_step: float32 projection and state")
    a_tok, a_head, a_chan = a_strides if alpha is not None else (0, 0, 0)
    q_off, k_off, v_off, g_off = offs
    f = _fn("linear_attention", "llm_recur_step",
            [c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_float, c_float, c_float, c_void_p,
             c_int, c_longlong, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
             c_void_p, c_float, c_longlong, c_longlong, c_longlong, c_int, c_int, c_longlong, c_longlong, c_void_p,
             c_int, c_void_p, c_float, c_int, c_int, c_void_p, c_void_p, c_void_p])
    _check(f(_ptr(proj), proj.stride(0), q_off, k_off, v_off, g_off, _ptr(alpha), _ptr(norm_w), float(eps),
             float(q_scale), float(out_scale), _ptr(out), _dt(out), out.stride(0), out_off, _ptr(state),
             _ptr(entry_slot), _ptr(entry_q_start), num_entries, H, D, V, 0, 0, None, None, 1.0, a_tok, a_head, a_chan,
             norm_stride, GATE_KINDS[gate], head_stride, state.stride(0), _ptr(inv_freq), dims, _ptr(positions),
             float(cap), i_off, f_off, _ptr(i_bias), _ptr(f_bias), _stream()), "recur_step")


def recur_chain(state: torch.Tensor, head_stride: int, scratch_s: torch.Tensor, scratch_a: torch.Tensor,
                chains: torch.Tensor, num_chains: int, entry_slot, H: int, D: int, V: int, normaliser: bool) -> None:
    """`gla_chain` over states that may keep a normaliser n [D] after S [D, V]."""
    _dev(state, scratch_s, scratch_a, chains, entry_slot)
    f = _fn("linear_attention", "llm_recur_chain",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_longlong, c_longlong,
             c_void_p])
    _check(f(_ptr(state), _ptr(scratch_s), _ptr(scratch_a), _ptr(chains), num_chains, _ptr(entry_slot), H, D, V,
             1 if normaliser else 0, head_stride, state.stride(0), _stream()), "recur_chain")


# ---- several residual streams ----------------------------------------------------------------------------
def stream_norm(streams: torch.Tensor, y, mix: Optional[torch.Tensor], outw: Optional[torch.Tensor],
                inw: Optional[torch.Tensor], weight: Optional[torch.Tensor], eps: float, center: bool,
                out_dtype: Optional[torch.dtype], rows: Optional[torch.Tensor] = None,
                write_back: bool = True, fan: bool = False) -> Optional[torch.Tensor]:
    """streams: float32 [S, T, H] (or [T, H]: one stream).  With y (a sublayer's output that has not been added
    yet, possibly an `ops.PartialSum`): x_t <- sum_s mix[s, t] x_s + outw[t] * y for all t (mix None: the identity,
    outw None: ones), written back unless `rows` is given.  Then, with `weight`: the norm (`center`: layer norm,
    else RMS norm) of u = sum_t inw[t] x_t (inw None: the plain sum) times `weight`, returned in `out_dtype` for
    all rows or for `rows`.  `fan`: only streams[0] holds data yet (a model's embedding); every stream is read from
    there and written to its own place."""
    parts, part_stride = 1, 0
    if isinstance(y, PartialSum):
        parts, part_stride = y.parts.shape[0], y.parts.stride(0)
        y = y.parts[0]
    if fan and (y is not None or rows is not None):
        raise KernelError("stream_norm: the first fan-out takes no pending update and no row selection")
    _dev(streams, y, mix, outw, inw, weight, rows)
    _i32(rows, "rows")
    if streams.dtype != torch.float32:
        raise KernelError("the residual streams are float32")
    S = streams.shape[0] if streams.dim() == 3 else 1
    T, H = streams.shape[-2], streams.shape[-1]
    for t, n in ((mix, S * S), (outw, S), (inw, S), (weight, H)):
        if t is not None and (t.dtype != torch.float32 or t.numel() != n):
            raise KernelError("stream_norm: a coefficient tensor of the wrong size or type")
    if y is not None and tuple(y.shape) != (T, H):
        raise KernelError("y must have a stream's shape")
    n = rows.numel() if rows is not None else T
    out = torch.empty((n, H), dtype=out_dtype, device=streams.device) if weight is not None else None
    f = _fn("streams", "llm_stream_norm",
            [c_void_p, c_longlong, c_longlong, c_int, c_void_p, c_int, c_int, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p,
             c_float, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(streams), T * H, 0 if fan else T * H, S, _ptr(y), _dt(y) if y is not None else 0, parts, part_stride, _ptr(mix), _ptr(outw),
             _ptr(inw), _ptr(weight), float(eps), 1 if center else 0, _ptr(out), _dt(out) if out is not None else 0,
             _ptr(rows), n, H, 1 if (write_back and rows is None and (y is not None or fan)) else 0, _stream()), "stream_norm")
    return out


# ---- routed experts ----------------------------------------------------------------------------------------
def moe_route(x: torch.Tensor, w_router: torch.Tensor, top: int, groups, route_scale: float, lists: bool = False,
              score: str = "sigmoid", correction: Optional[torch.Tensor] = None, identity: int = 0):
    """Per token of x [T, W]: scores of `w_router` (float32 [E, W]; `score` 'sigmoid', or 'softmax' over all E), the
    `top` best among the experts of the best groups (`groups` = (count, keep) or None), weights normalised and
    scaled.  `correction` (float32 [E]) is added to the scores for the choice only.  The last `identity` router
    outputs are no experts: a token that picks one gets its own input back times the weight.  Returns the dense
    float32 weights [T, E - identity] (zero where not chosen) and, with `lists`, ids int32 [T, top] (-1 for an
    identity pick) and weights float32 [T, top]; with `identity`, also the float32 [T] share of a token's own input."""
    _dev(x, w_router, correction)
    T, W = x.shape
    E = w_router.shape[0]
    if w_router.dtype != torch.float32 or w_router.shape[1] != W:
        raise KernelError("the router's matrix must be float32 [experts, hidden]")
    if correction is not None and (correction.dtype != torch.float32 or correction.numel() != E):
        raise KernelError("the router's correction must be float32 [router outputs]")
    if score not in ("sigmoid", "softmax") or not 0 <= identity < E:
        raise KernelError("score 'sigmoid' or 'softmax'; identity outputs fewer than the router's")
    dense = torch.empty((T, E - identity), dtype=torch.float32, device=x.device)
    idw = torch.empty((T,), dtype=torch.float32, device=x.device) if identity else None
    ids = torch.empty((T, top), dtype=torch.int32, device=x.device) if lists else None
    wts = torch.empty((T, top), dtype=torch.float32, device=x.device) if lists else None
    count, keep = groups if groups is not None else (0, 0)
    f = _fn("moe", "llm_moe_route",
            [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
             c_int, c_void_p, c_int, c_void_p, c_void_p])
    _check(f(_ptr(x), _dt(x), _ptr(w_router), _ptr(dense), _ptr(ids), _ptr(wts), T, W, E, top, count, keep,
             float(route_scale), 1 if score == "softmax" else 0, _ptr(correction), identity, _ptr(idw), _stream()), "moe_route")
    out = (dense, ids, wts) if lists else dense
    if identity:
        return (out + (idw,)) if lists else (out, idw)
    return out


def moe_finish(out: torch.Tensor, x: Optional[torch.Tensor], idw: Optional[torch.Tensor], shared=None) -> torch.Tensor:
    """out (float32 [T, W], in place) += idw[t] * x[t] + shared[t]: a token's share of its own input (`idw` float32 [T]
    with x [T, W], or None) and the output of an expert that every token runs (float32 [T, W], a `PartialSum` or None)."""
    parts, part_stride = 1, 0
    if isinstance(shared, PartialSum):
        parts, part_stride = shared.parts.shape[0], shared.parts.stride(0)
        shared = shared.parts[0]
    _dev(out, x, idw, shared)
    T, W = out.shape
    if out.dtype != torch.float32 or not out.is_contiguous():
        raise KernelError("moe_finish wants a contiguous float32 sum")
    if idw is not None and (x is None or tuple(x.shape) != (T, W) or not x.is_contiguous() or idw.dtype != torch.float32 or idw.numel() != T):
        raise KernelError("moe_finish: x [T, W] and float32 weights [T]")
    if shared is not None and (shared.dtype != torch.float32 or tuple(shared.shape) != (T, W) or not shared.is_contiguous()):
        raise KernelError("moe_finish: the shared expert's output must be float32 [T, W]")
    f = _fn("moe", "llm_moe_finish", [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_longlong, c_int, c_int, c_void_p])
    _check(f(_ptr(out), _ptr(x) if idw is not None else None, _dt(x) if idw is not None else 0, _ptr(idw), _ptr(shared), parts,
             part_stride, T, W, _stream()), "moe_finish")
    return out


def moe_act(gate_up, dense: torch.Tensor, E: int, ff: int, limit: float, alpha: float,
            out_dtype: torch.dtype, shift: float = 1.0) -> torch.Tensor:
    """act [T, E*ff] = dense[t, e] * g * sigmoid(alpha g) * (u + shift), g = min(gate, limit), u = clamp(up, +-limit),
    from the float32 product [T, E*2*ff] (per expert: ff gate columns, then ff up columns; may be a `PartialSum`)."""
    parts, part_stride = 1, 0
    if isinstance(gate_up, PartialSum):
        parts, part_stride = gate_up.parts.shape[0], gate_up.parts.stride(0)
        gate_up = gate_up.parts[0]
    _dev(gate_up, dense)
    T = gate_up.shape[0]
    if gate_up.dtype != torch.float32 or gate_up.shape[1] != 2 * E * ff or tuple(dense.shape) != (T, E):
        raise KernelError("moe_act wants the float32 product [T, experts * 2 * ff] and the weights [T, experts]")
    act = torch.empty((T, E * ff), dtype=out_dtype, device=gate_up.device)
    f = _fn("moe", "llm_moe_act",
            [c_void_p, c_int, c_longlong, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_float, c_float, c_void_p])
    _check(f(_ptr(gate_up), parts, part_stride, _ptr(dense), _ptr(act), _dt(act), T, E, ff, float(limit), float(alpha),
             float(shift), _stream()), "moe_act")
    return act


def moe_sparse(x: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor,
               ff: int, limit: float, alpha: float, shift: float = 1.0) -> torch.Tensor:
    """The routed feed-forward for steps of few tokens: only the chosen experts' matrices are read.  x [T, W] and
    the matrices in one dtype (bfloat16 or float32); `ids`, `weights` [T, top] from `moe_route`.  Returns the
    float32 sum [T, W] of the chosen experts' weighted outputs."""
    _dev(x, w_gate_up, w_down, ids, weights)
    _i32(ids, "ids")
    T, W = x.shape
    top = ids.shape[1]
    E = w_gate_up.shape[0] // (2 * ff)
    if (w_gate_up.shape != (E * 2 * ff, W) or w_down.shape != (W, E * ff) or w_gate_up.dtype != x.dtype
            or w_down.dtype != x.dtype or weights.dtype != torch.float32):
        raise KernelError("moe_sparse: x, [E*2*ff, W] and [W, E*ff] in one dtype, float32 weights [T, top]")
    act = torch.empty((T * top, ff), dtype=x.dtype, device=x.device)
    out = torch.empty((T, W), dtype=torch.float32, device=x.device)
    f = _fn("moe", "llm_moe_sparse",
            [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
             c_int, c_float, c_float, c_float, c_void_p])
    code = f(_ptr(x), _dt(x), _ptr(w_gate_up), _ptr(w_down), _dt(w_down), _ptr(ids), _ptr(weights), _ptr(act), _ptr(out),
             T, W, ff, E, top, float(limit), float(alpha), float(shift), _stream())
    _check(code, "moe_sparse")
    global launch_count
    launch_count += 1                      # two kernels in one call
    return out


def grouped_product_available() -> bool:
    """Whether the tensor library offers a grouped matrix product with row offsets on the device."""
    return hasattr(torch, "_grouped_mm")


def moe_sorted(x: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor,
               E: int, ff: int, limit: float, alpha: float, shift: float = 1.0) -> torch.Tensor:
    """The routed feed-forward for prompt portions: the (token, choice) pairs are sorted by expert (the engine's
    kernels), each expert's rows go through ITS matrices in the library's grouped matrix product (bfloat16 in,
    bfloat16 out, 32-bit accumulation; the row offsets stay on the device), the activation takes each row's
    routing weight, and a token's rows are added in 32-bit.  Returns float32 [T, W]."""
    _dev(x, w_gate_up, w_down, ids, weights)
    T, W = x.shape
    top = ids.shape[1]
    pairs = T * top
    dev = x.device
    offs = torch.empty(E, dtype=torch.int32, device=dev)
    pos = torch.empty(pairs, dtype=torch.int32, device=dev)
    row_pair = torch.zeros(pairs, dtype=torch.int32, device=dev)      # rows no pair takes (a pick without an expert) read token 0
    _check(_fn("moe", "llm_moe_sort", [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p])(
        _ptr(ids), pairs, E, _ptr(offs), _ptr(pos), _ptr(row_pair), _stream()), "moe_sort")
    rows_fn = _fn("moe", "llm_moe_rows",
                  [c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_float, c_float, c_void_p])
    xs = torch.empty((pairs, W), dtype=x.dtype, device=dev)
    _check(rows_fn(0, _ptr(x), _dt(x), _ptr(row_pair), None, _ptr(xs), pairs, W, top, 0.0, 0.0, 0.0, _stream()), "moe_gather")
    gu = torch._grouped_mm(xs, w_gate_up.view(E, 2 * ff, W).transpose(1, 2), offs=offs)
    act = torch.empty((pairs, ff), dtype=x.dtype, device=dev)
    _check(rows_fn(1, _ptr(gu), _dt(gu), _ptr(row_pair), _ptr(weights), _ptr(act), pairs, ff, top, float(limit), float(alpha),
                   float(shift), _stream()), "moe_act_pairs")
    y = torch._grouped_mm(act, w_down.view(W, E, ff).permute(1, 2, 0), offs=offs)
    out = torch.empty((T, W), dtype=torch.float32, device=dev)
    _check(rows_fn(2, _ptr(y), _dt(y), _ptr(pos), None, _ptr(out), T, W, top, 0.0, 0.0, 0.0, _stream()), "moe_combine")
    return out


def fast_attention_supported(d: int, group: int) -> bool:
    """Whether the tuned bfloat16 kernels (tensor-core prefill, split-key decode) take this shape."""
    if d % 64 != 0:          # they are written for head sizes 64 and 128: do not compile them just to hear "no"
        return False
    a = _fn("attention_decode", "llm_paged_decode_supported", [c_int, c_int])
    b = _fn("attention_prefill", "llm_paged_prefill_supported", [c_int])
    return bool(a(d, group)) and bool(b(d))


PREFILL_TILE_ROWS = 128
_scratch: Dict[str, torch.Tensor] = {}
_scratch_retired = []          # outgrown buffers stay alive: a captured graph may still point at them


def decode_scratch(device, floats: int) -> Optional[torch.Tensor]:
    """The float32 scratch the split-key decode kernel merges through; grown on demand, never
    freed (launches on one stream are ordered, so one buffer per device serves them all)."""
    if floats <= 0:
        return None
    key = str(device)
    t = _scratch.get(key)
    if t is None or t.numel() < floats:
        if t is not None:
            _scratch_retired.append(t)
        t = torch.empty(max(2 * floats, 1 << 22), dtype=torch.float32, device=device)
        _scratch[key] = t
    return t


def paged_attention_decode(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, rows: Optional[torch.Tensor],
                           n_rows: int, positions, token_entry, entry_slot, block_table: torch.Tensor, nq: int,
                           nkv: int, d: int, page_size: int, window: Optional[int], scale: float, num_splits: int,
                           status: torch.Tensor, dist_bias_t: Optional[torch.Tensor] = None,
                           analytic_bias: bool = False, keep_first: int = 0, sink: Optional[float] = None) -> torch.Tensor:
    """Attention for single decoded tokens (rows of q named by `rows`, or rows 0..n_rows-1), written
    into the same rows of `out`.  bfloat16 only.  `dist_bias_t` float32 [nq, distances]: a bias by distance TIMES
    log2(e); row min(p - j, distances - 1) of a head joins the scaled score of the query at p and key j.
    `keep_first`: with a window, the sequence's first so many keys stay visible (one more split walks them, beside
    the `num_splits` of the window).  `sink`: a score whose exponential joins the softmax's denominator without a value."""
    keep_first = int(keep_first) if window else 0
    if keep_first:
        num_splits += 1
    _dev(q, out, cache, rows, positions, token_entry, entry_slot, block_table, status, dist_bias_t)
    if dist_bias_t is not None and (dist_bias_t.dtype != torch.float32 or dist_bias_t.dim() != 2 or dist_bias_t.shape[0] != nq):
        raise KernelError("dist_bias_t must be float32 [heads, distances]")
    dist_len = 0 if dist_bias_t is None else (-1 if analytic_bias else dist_bias_t.shape[1])
    if analytic_bias and (dist_bias_t is None or dist_bias_t.shape[1] != 3):
        raise KernelError("an analytic bias comes as float32 [heads, 3]: temperature, r1, r2")
    if q.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("the decode attention kernel is bfloat16 only")
    if q.shape[1] != nq * d or tuple(cache.shape[1:]) != (2, nkv, page_size, d):
        raise KernelError("q must be [T, heads*head_dim] and cache [pages, 2, kv_heads, page_size, head_dim]")
    need = _fn("attention_decode", "llm_paged_decode_scratch_floats", [c_int, c_int, c_int, c_int],
               restype=c_longlong)(n_rows, nq, d, num_splits)
    scratch = decode_scratch(q.device, int(need))
    f = _fn("attention_decode", "llm_paged_attention_decode_ex",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
             c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float,
             c_void_p])
    _check(f(_ptr(q), _ptr(out), _ptr(cache), _ptr(rows), n_rows, _ptr(positions), _ptr(token_entry),
             _ptr(entry_slot), _ptr(block_table), block_table.shape[1], nq, nkv, d, page_size,
             int(window) if window else 0, float(scale), cache.shape[0], num_splits, _ptr(scratch), _ptr(status),
             _ptr(dist_bias_t), dist_len, keep_first, 0 if sink is None else 1, float(sink or 0.0), _stream()),
           "paged_attention_decode")
    if num_splits > 1:
        global launch_count
        launch_count += 1                         # the merge kernel
    return out


def paged_attention_prefill(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, tiles: torch.Tensor,
                            n_tiles: int, entry_slot, entry_q_start, entry_q_len, entry_kv_len,
                            block_table: torch.Tensor, nq: int, nkv: int, d: int, page_size: int,
                            window: Optional[int], scale: float, status: torch.Tensor) -> torch.Tensor:
    """Attention for prompt portions: `tiles` int32 [n_tiles, 2] = (entry, first row of a
    PREFILL_TILE_ROWS-row tile inside the entry).  bfloat16 only."""
    _dev(q, out, cache, tiles, entry_slot, entry_q_start, entry_q_len, entry_kv_len, block_table, status)
    if q.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("the prefill attention kernel is bfloat16 only")
    if q.shape[1] != nq * d or tuple(cache.shape[1:]) != (2, nkv, page_size, d):
        raise KernelError("q must be [T, heads*head_dim] and cache [pages, 2, kv_heads, page_size, head_dim]")
    f = _fn("attention_prefill", "llm_paged_attention_prefill",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
             c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p])
    _check(f(_ptr(q), _ptr(out), _ptr(cache), _ptr(tiles), n_tiles, _ptr(entry_slot), _ptr(entry_q_start),
             _ptr(entry_q_len), _ptr(entry_kv_len), _ptr(block_table), block_table.shape[1], nq, nkv, d,
             page_size, int(window) if window else 0, float(scale), cache.shape[0], _ptr(status), _stream()),
           "paged_attention_prefill")
    return out


def prefill_attention_supported(d: int) -> bool:
    """Whether the tensor-core kernel for prompt portions (`paged_attention_prefill*`) takes this head size."""
    if d % 64 != 0:
        return False
    return bool(_fn("attention_prefill", "llm_paged_prefill_supported", [c_int])(d))


def paged_attention_prefill_biased(q: torch.Tensor, out: torch.Tensor, out_off: int, cache: torch.Tensor, tiles: torch.Tensor,
                                   n_tiles: int, entry_slot, entry_q_start, entry_q_len, entry_kv_len,
                                   block_table: torch.Tensor, nq: int, nkv: int, d: int, page_size: int,
                                   window: Optional[int], scale: float, status: torch.Tensor,
                                   dist_bias_t: Optional[torch.Tensor] = None, head_gate: Optional[torch.Tensor] = None,
                                   gate_off: int = 0, out_scale: float = 1.0, analytic_bias: bool = False,
                                   keep_first: int = 0, sink: Optional[float] = None) -> torch.Tensor:
    """`keep_first`: with a window, the sequence's first so many keys stay visible to every later query.  `sink`: a score
    whose exponential joins the softmax's denominator without a value.  `analytic_bias`: `dist_bias_t` is float32 [nq, 3], per head a temperature on the scaled score and the numbers
    r1, r2 of the bias r1 * ln(1 + r2 * (i - j)) that is taken off it (evaluated in the kernel; no table).
    `paged_attention_prefill` with what other attention layers add: `dist_bias_t` float32 [nq, distances], a bias by
    distance TIMES log2(e) (row min(i - j, distances - 1) of the head joins the scaled score); `head_gate` float32
    [T, ...] with one value per (token, head) from column gate_off, whose sigmoid multiplies the head's output;
    `out_scale`; the result goes to columns out_off .. out_off + nq*d of `out` (bfloat16, any row stride)."""
    _dev(q, cache, tiles, entry_slot, entry_q_start, entry_q_len, entry_kv_len, block_table, status, dist_bias_t)
    if q.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or out.stride(1) != 1:
        raise KernelError("the prefill attention kernel is bfloat16 only")
    if q.shape[1] != nq * d or tuple(cache.shape[1:]) != (2, nkv, page_size, d):
        raise KernelError("q must be [T, heads*head_dim] and cache [pages, 2, kv_heads, page_size, head_dim]")
    if dist_bias_t is not None and (dist_bias_t.dtype != torch.float32 or dist_bias_t.dim() != 2 or dist_bias_t.shape[0] != nq):
        raise KernelError("dist_bias_t must be float32 [heads, distances]")
    dist_len = 0 if dist_bias_t is None else (-1 if analytic_bias else dist_bias_t.shape[1])
    if analytic_bias and (dist_bias_t is None or dist_bias_t.shape[1] != 3):
        raise KernelError("an analytic bias comes as float32 [heads, 3]: temperature, r1, r2")
    if head_gate is not None and (head_gate.dtype != torch.float32 or head_gate.stride(1) != 1):
        raise KernelError("head_gate must be float32 with unit stride along rows")
    f = _fn("attention_prefill", "llm_paged_attention_prefill_ex",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
             c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p, c_int, c_void_p, c_longlong, c_int,
             c_float, c_longlong, c_int, c_int, c_int, c_float, c_void_p])
    _check(f(_ptr(q), _ptr(out), _ptr(cache), _ptr(tiles), n_tiles, _ptr(entry_slot), _ptr(entry_q_start),
             _ptr(entry_q_len), _ptr(entry_kv_len), _ptr(block_table), block_table.shape[1], nq, nkv, d,
             page_size, int(window) if window else 0, float(scale), cache.shape[0], _ptr(status), _ptr(dist_bias_t),
             dist_len, _ptr(head_gate),
             head_gate.stride(0) if head_gate is not None else 0, gate_off, float(out_scale), out.stride(0), out_off,
             int(keep_first) if window else 0, 0 if sink is None else 1, float(sink or 0.0),
             _stream()), "paged_attention_prefill_biased")
    return out


def prefill_tcgen05_supported(d: int, page_size: int) -> bool:
    f = _fn("attention_prefill_tcgen05", "llm_paged_prefill_tcgen05_supported", [c_int, c_int])
    return bool(f(d, page_size))


def paged_attention_prefill_tcgen05(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, tiles: torch.Tensor,
                                    n_tiles: int, entry_slot, entry_q_start, entry_q_len, entry_kv_len,
                                    block_table: torch.Tensor, nq: int, nkv: int, d: int, page_size: int,
                                    window: Optional[int], scale: float, status: torch.Tensor) -> torch.Tensor:
    """The prompt-portion attention on tcgen05/TMEM with TMA loads (head size 128, pages of 8..64);
    same arguments as `paged_attention_prefill`."""
    _dev(q, out, cache, tiles, entry_slot, entry_q_start, entry_q_len, entry_kv_len, block_table, status)
    if q.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("the tcgen05 prefill attention kernel is bfloat16 only")
    if q.shape[1] != nq * d or tuple(cache.shape[1:]) != (2, nkv, page_size, d):
        raise KernelError("q must be [T, heads*head_dim] and cache [pages, 2, kv_heads, page_size, head_dim]")
    f = _fn("attention_prefill_tcgen05", "llm_paged_attention_prefill_tcgen05",
            [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
             c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p])
    _check(f(_ptr(q), _ptr(out), _ptr(cache), q.shape[0], _ptr(tiles), n_tiles, _ptr(entry_slot), _ptr(entry_q_start),
             _ptr(entry_q_len), _ptr(entry_kv_len), _ptr(block_table), block_table.shape[1], nq, nkv, d, page_size,
             int(window) if window else 0, float(scale), cache.shape[0], _ptr(status), _stream()),
           "paged_attention_prefill_tcgen05")
    return out


def prefill_tcgen05_biased_supported(d: int, page_size: int, group: int) -> bool:
    f = _fn("attention_prefill_tcgen05", "llm_paged_prefill_tcgen05_biased_supported", [c_int, c_int, c_int])
    return bool(f(d, page_size, group))


def paged_attention_prefill_tcgen05_biased(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, tiles: torch.Tensor,
                                           n_tiles: int, entry_slot, entry_q_start, entry_q_len, entry_kv_len,
                                           block_table: torch.Tensor, nq: int, nkv: int, d: int, page_size: int,
                                           window: Optional[int], scale: float, status: torch.Tensor,
                                           head_bias: torch.Tensor) -> torch.Tensor:
    """`paged_attention_prefill_tcgen05` for scores with a temperature per head and a logarithmic distance bias:
    `head_bias` float32 [nq, 3] = (t, r1, r2) per query head, weight of key j for the query at i =
    exp(q.k * scale * t - r1 * ln(1 + r2 * (i - j))).  Even groups of query heads per kv head only; `out` is
    bfloat16 [T, nq*d], contiguous."""
    _dev(q, out, cache, tiles, entry_slot, entry_q_start, entry_q_len, entry_kv_len, block_table, status, head_bias)
    if q.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("the tcgen05 prefill attention kernel is bfloat16 only")
    if q.shape[1] != nq * d or tuple(cache.shape[1:]) != (2, nkv, page_size, d) or not out.is_contiguous() \
            or tuple(out.shape) != tuple(q.shape):
        raise KernelError("q and out must be [T, heads*head_dim] and cache [pages, 2, kv_heads, page_size, head_dim]")
    if head_bias.dtype != torch.float32 or tuple(head_bias.shape) != (nq, 3) or not head_bias.is_contiguous():
        raise KernelError("head_bias must be float32 [heads, 3]: temperature, r1, r2")
    f = _fn("attention_prefill_tcgen05", "llm_paged_attention_prefill_tcgen05_biased",
            [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
             c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p, c_void_p])
    _check(f(_ptr(q), _ptr(out), _ptr(cache), q.shape[0], _ptr(tiles), n_tiles, _ptr(entry_slot), _ptr(entry_q_start),
             _ptr(entry_q_len), _ptr(entry_kv_len), _ptr(block_table), block_table.shape[1], nq, nkv, d, page_size,
             int(window) if window else 0, float(scale), cache.shape[0], _ptr(status), _ptr(head_bias), _stream()),
           "paged_attention_prefill_tcgen05_biased")
    return out


def argmax_rows(logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _dev(logits, out)
    if logits.dtype != torch.float32 or logits.dim() != 2:
        raise KernelError("logits must be float32 [rows, vocab]")
    R, V = logits.shape
    if out is None:
        out = torch.empty((R,), dtype=torch.int32, device=logits.device)
    scratch = decode_scratch(logits.device, R * 64 * 2)
    f = _fn("sampling", "llm_argmax_rows", [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p])
    _check(f(_ptr(logits), R, V, _ptr(out), _ptr(scratch), _stream()), "argmax_rows")
    return out


def sample_rows(logits: torch.Tensor, row_slot: torch.Tensor, sampler_state: torch.Tensor,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token per row by the row's slot state {seed_lo, seed_hi, counter, temperature bits};
    temperature <= 0 takes the argmax.  Advances the counters of sampled rows."""
    _dev(logits, row_slot, sampler_state, out)
    _i32(row_slot, "row_slot")
    _i32(sampler_state, "sampler_state")
    if logits.dtype != torch.float32 or logits.dim() != 2:
        raise KernelError("logits must be float32 [rows, vocab]")
    if sampler_state.dim() != 2 or sampler_state.shape[1] != 4:
        raise KernelError("sampler_state must be int32 [slots, 4]")
    R, V = logits.shape
    if out is None:
        out = torch.empty((R,), dtype=torch.int32, device=logits.device)
    f = _fn("sampling", "llm_sample_rows", [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p])
    _check(f(_ptr(logits), R, V, _ptr(row_slot), _ptr(sampler_state), _ptr(out), _stream()), "sample_rows")
    return out


def sampler_uniform(seed: int, counter: int) -> float:
    """The u in [0,1) that the sampling kernel draws for (seed, counter); runs on the host."""
    f = _fn("sampling", "llm_sampler_uniform", [c_uint64, c_uint32], restype=c_float)
    return float(f(seed & 0xFFFFFFFFFFFFFFFF, counter & 0xFFFFFFFF))


# ------------------------------------------------------------------------------------------
_skinny_scratch: Dict[str, torch.Tensor] = {}


def skinny_scratch(device, floats: int) -> Optional[torch.Tensor]:
    """Scratch for the streaming product's k-splits; grown on demand, never freed."""
    if floats <= 0:
        return None
    key = str(device)
    t = _skinny_scratch.get(key)
    if t is None or t.numel() < floats:
        if t is not None:
            _scratch_retired.append(t)
        t = torch.empty(max(2 * floats, 1 << 22), dtype=torch.float32, device=device)
        _skinny_scratch[key] = t
    return t


SKINNY_MAX_ROWS = 16     # rows up to which `linear` takes the engine's own streaming kernel
SKINNY_SMALL_MAX_ROWS = 32    # and for small (latency-bound) products, see `skinny_small`
_skinny_small: Dict[tuple, bool] = {}


def skinny_small(n: int, k: int) -> bool:
    """Whether an [n, k] product has fewer items than would give every CTA slot of the streaming kernel
    four: then latency bounds it, not bytes, and the kernel takes it up to 32 rows."""
    got = _skinny_small.get((n, k))
    if got is None:
        got = _skinny_small[(n, k)] = bool(_fn("gemm_skinny", "llm_linear_skinny_small", [c_int, c_int])(n, k))
    return got



# ---- weights stored tile by tile for the streaming product ----------------------------------
# The streaming product reads the plain [N, K] weights box by box through the copy engine, or, 2.5 %
# (batch 8) to 4.5 % (batch 1) faster per decode step, a second copy of them stored in its
# shared-memory order.  That copy doubles the weights' memory, so it is made only for models whose
# weights are a small share of the device: `begin_model` decides once per model.
_TILED_POLICY = os.environ.get("LLM_TILED", "auto")   # on | auto | off
_TILED_SHARE = 0.125                                   # auto: models whose matrices take up to this share of the device's memory
_tiled: Dict[int, torch.Tensor] = {}                   # weight.data_ptr() -> its tiled copy
_tiled_allowed = _TILED_POLICY != "off"          # until a model says otherwise (`begin_model`)
TILE_ROWS, TILE_K = 64, 256


def begin_model(matrix_bytes: int, device) -> bool:
    """Called before a model's weights are loaded with the bytes of its bfloat16 matrices: decides
    whether `prepare_streaming` makes tiled copies for them (all of them or none).  `LLM_TILED=on` /
    `off` overrides the rule."""
    global _tiled_allowed
    device = torch.device(device)
    if _TILED_POLICY == "off" or device.type != "cuda":
        _tiled_allowed = False
    elif _TILED_POLICY == "on":
        _tiled_allowed = True
    else:
        _, total = torch.cuda.mem_get_info(device)
        _tiled_allowed = matrix_bytes <= _TILED_SHARE * total
    return _tiled_allowed


def tile_weight(weight: torch.Tensor) -> torch.Tensor:
    """bfloat16 [N, K] -> the same values as [N/64 tiles, K/256 steps] blocks of 32 KB, each four
    sub-tiles of [64 rows][64 k-values] with 128-byte rows whose 16-byte chunks are XOR-swizzled by
    the row (chunk c of row r at position c ^ (r % 8)), zero-padded at the edges.  A stage of the
    streaming product is one block for up to 8 tokens and half a block for 9 to 16; a K-major tcgen05 operand of 128 rows x 64
    k-values is two sub-tiles."""
    N, K = weight.shape
    tn, nk = -(-N // TILE_ROWS), -(-K // TILE_K)
    padded = torch.zeros((tn * TILE_ROWS, nk * TILE_K), dtype=weight.dtype, device=weight.device)
    padded[:N, :K] = weight
    v = padded.view(tn, TILE_ROWS, nk, TILE_K // 64, 8, 8)               # [tile, row, step, sub, chunk, 8 values]
    r = torch.arange(TILE_ROWS, device=weight.device)[:, None]
    p = torch.arange(8, device=weight.device)[None, :]
    src = p ^ (r & 7)                                                     # the chunk that lands at position p of row r
    idx = src[None, :, None, None, :, None].expand(tn, TILE_ROWS, nk, TILE_K // 64, 8, 8)
    return torch.gather(v, 4, idx).permute(0, 2, 3, 1, 4, 5).contiguous().view(tn, nk, TILE_ROWS * TILE_K)


def prepare_streaming(weight: Optional[torch.Tensor]) -> None:
    """Keep a tiled copy of a bfloat16 weight for decode steps of up to 16 tokens, if `begin_model`
    allowed copies for the model being loaded.  The copy lives as long as the weight."""
    if (weight is None or not _tiled_allowed or not weight.is_cuda or weight.dtype != torch.bfloat16
            or weight.dim() != 2 or weight.shape[1] % 8 != 0):
        return
    key = weight.data_ptr()
    if key in _tiled:
        return
    _tiled[key] = tile_weight(weight)
    weakref.finalize(weight, _tiled.pop, key, None)


_tiled_generation = 0


def release_streaming() -> int:
    """Drop every tiled copy (the weights themselves stay; products fetch them box by box from their
    plain layout from then on).  Returns how many copies went.  Captured CUDA graphs that read the copies must
    not be replayed afterwards: `streaming_generation` changes, and the runner drops its graphs."""
    global _tiled_generation
    n = len(_tiled)
    if n:
        torch.cuda.synchronize()                 # nothing in flight still reads them
        _tiled.clear()
        _tiled_generation += 1
    return n


def streaming_generation() -> int:
    """Counts the times the tiled copies were dropped."""
    return _tiled_generation


def linear_skinny(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype,
                  out: Optional[torch.Tensor] = None, partials_ok: bool = False):
    """x [M <= 32, K] @ weight[N, K]^T with the engine's own weight-streaming kernel (bfloat16
    operands, float32 accumulation, float32 or bfloat16 result).  With `partials_ok` a product
    that is cut into k-splits comes back as a `PartialSum` instead of being added up."""
    _dev(x, weight, out)
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16:
        raise KernelError("the skinny product takes bfloat16 operands")
    M, K = x.shape
    N = weight.shape[0]
    if weight.shape[1] != K:
        raise KernelError("x and weight disagree on K")
    global launch_count
    tiled = _tiled.get(weight.data_ptr())
    g = _fn("gemm_skinny", "llm_linear_skinny_tiled" if tiled is not None else "llm_linear_skinny_boxes",
            [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_void_p, c_void_p])
    st, wp = stream_status(x.device), _ptr(tiled if tiled is not None else weight)
    f = lambda xp, _w, yp, dt, sp, sn, m, n, k, keep, stream: g(xp, wp, yp, dt, sp, sn, m, n, k, keep, _ptr(st), stream)
    splits = _fn("gemm_skinny", "llm_linear_skinny_splits", [c_int, c_int, c_int])(M, N, K)
    if partials_ok and splits > 1 and out is None:
        parts = torch.empty((splits, M, N), dtype=torch.float32, device=x.device)
        _check(f(_ptr(x), _ptr(weight), None, 0, _ptr(parts), parts.numel(), M, N, K, 1, _stream()), "linear_skinny")
        return PartialSum(parts, None if out_dtype == torch.float32 else out_dtype)
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
    scratch = skinny_scratch(x.device, splits * M * N if splits > 1 else 0)
    _check(f(_ptr(x), _ptr(weight), _ptr(out), _dt(out), _ptr(scratch), scratch.numel() if scratch is not None else 0,
             M, N, K, 0, _stream()), "linear_skinny")
    launch_count += 1 if splits > 1 else 0        # the kernel that adds the k-splits
    return out


_stream_status: Dict[str, torch.Tensor] = {}


def stream_status(device) -> torch.Tensor:
    """The status word of the engine's matrix products (code 8: a bounded wait of the weight-streaming
    product ran out; 9: of the paired product)."""
    key = str(device)
    t = _stream_status.get(key)
    if t is None:
        t = _stream_status[key] = torch.zeros(2, dtype=torch.int32, device=device)
    return t


def linear_pair(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype,
                out: Optional[torch.Tensor] = None, accumulate: bool = False) -> torch.Tensor:
    """x [T, K] @ weight[N, K]^T for prompt portions with the engine's own tcgen05 kernel, in which
    two CTAs of a cluster share a tile of 256 tokens x 256 features (bfloat16 operands, float32
    accumulation in tensor memory, float32 or bfloat16 result).  With `accumulate` the product is
    added to the float32 `out` in place."""
    if accumulate and (out is None or out.dtype != torch.float32):
        raise KernelError("accumulating wants a float32 out")
    _dev(x, weight, out)
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16:
        raise KernelError("the paired product takes bfloat16 operands")
    T, K = x.shape
    N = weight.shape[0]
    if weight.shape[1] != K:
        raise KernelError("x and weight disagree on K")
    if out is None:
        out = torch.empty((T, N), dtype=out_dtype, device=x.device)
    if out.shape != (T, N) or not out.is_contiguous():
        raise KernelError("out must be a contiguous [T, N]")
    f = _fn("gemm_pair_tcgen05", "llm_linear_pair",
            [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(f(_ptr(x), _ptr(weight), _ptr(out), _dt(out), 1 if accumulate else 0, T, N, K, _ptr(stream_status(x.device)),
             _stream()), "linear_pair")
    return out


def linear_pair_silu_mul(x: torch.Tensor, w_gate_up: torch.Tensor, out: Optional[torch.Tensor] = None,
                         activation: str = "silu") -> torch.Tensor:
    """act(x @ gate^T) * (x @ up^T), act = silu or the tanh form of gelu, for w_gate_up = [gate; up] of 2 I rows, as bfloat16 [T, I]: the
    paired tcgen05 product with the activation in its epilogue (gate and up are rounded to bfloat16
    before the activation, as the separate kernel would read them)."""
    _dev(x, w_gate_up, out)
    if x.dtype != torch.bfloat16 or w_gate_up.dtype != torch.bfloat16:
        raise KernelError("the paired product takes bfloat16 operands")
    T, K = x.shape
    if w_gate_up.shape[1] != K or w_gate_up.shape[0] % 2 != 0:
        raise KernelError("x and the gate/up weight disagree")
    inter = w_gate_up.shape[0] // 2
    if out is None:
        out = torch.empty((T, inter), dtype=torch.bfloat16, device=x.device)
    f = _fn("gemm_pair_tcgen05", "llm_linear_pair_silu_mul", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p,
                                                              c_void_p])
    _check(f(_ptr(x), _ptr(w_gate_up), _ptr(out), T, inter, K, ACTIVATIONS[activation], _ptr(stream_status(x.device)), _stream()),
           "linear_pair_silu_mul")
    return out


_PAIR_POLICY = os.environ.get("LLM_PAIR", "auto")       # auto | all | off: which prompt-portion products take the paired kernel
PAIR_MIN_ROWS = 129                                      # fewer rows leave the second CTA of a pair idle
# Thousandths of the clusters' time that a product's tiles must fill for the paired kernel to be taken
# under `auto`; None: only under `all`.  With the activation in its epilogue it saves a kernel and wins
# from 0.85 on (prefill of the Qwen3-8B shape, 2,048 / 4,096 / 8,192 tokens: 26.9 / 56.2 / 123.9 ms
# against 27.9 / 58.8 / 124.1 with the library product and the activation kernel).  Alone it is level with
# the library kernel by kernel, but a prefill is power-bound and the clocks settle lower with it: taking
# the other products too gave 57.6 and 127.1 ms at 4,096 and 8,192 tokens, and adding into the residual
# 28.9 ms at 2,048.
_PAIR_NEEDS = {"plain": None, "silu": 850, "into": None}


def _pair_takes(x: torch.Tensor, weight: torch.Tensor, n: int, kind: str) -> bool:
    """Whether the paired tcgen05 product is the faster way for these operands: bfloat16 on the GPU,
    enough rows, and tiles that keep the clusters busy."""
    if (_PAIR_POLICY == "off" or not x.is_cuda or x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16
            or x.shape[0] < PAIR_MIN_ROWS or not x.is_contiguous() or not weight.is_contiguous()):
        return False
    eff = _fn("gemm_pair_tcgen05", "llm_linear_pair_efficiency", [c_int, c_int, c_int, c_int])(
        x.shape[0], n, x.shape[1], 1 if kind == "silu" else 0)
    if eff <= 0:
        return False
    need = _PAIR_NEEDS[kind]
    return _PAIR_POLICY == "all" or (need is not None and eff >= need)


def linear_into(x: torch.Tensor, weight: torch.Tensor, residual: torch.Tensor) -> bool:
    """residual (float32 [T, N]) += x @ weight^T in the product's epilogue, if the paired kernel takes
    these operands; False, and nothing done, if not."""
    if (residual.dtype != torch.float32 or not residual.is_contiguous() or residual.shape != (x.shape[0], weight.shape[0])
            or not _pair_takes(x, weight, weight.shape[0], "into")):
        return False
    linear_pair(x, weight, torch.float32, out=residual, accumulate=True)
    return True


def linear_silu_mul(x: torch.Tensor, w_gate_up: torch.Tensor, out_dtype: torch.dtype, activation: str = "silu"):
    """act(x @ gate^T) * (x @ up^T) for w_gate_up = [gate; up]: one kernel where the paired product
    takes it, else the product (which may stay a sum of k-splits) followed by the activation kernel."""
    if out_dtype == torch.bfloat16 and _pair_takes(x, w_gate_up, w_gate_up.shape[0] // 2, "silu"):
        return linear_pair_silu_mul(x, w_gate_up, activation=activation)
    return silu_and_mul(linear(x, w_gate_up, out_dtype=out_dtype, partials_ok=True), activation=activation)


def linear(x: torch.Tensor, weight: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
           partials_ok: bool = False):
    """x [T, K] @ weight[N, K]^T.  Up to 16 bfloat16 rows (decode steps; up to 32 for the small products
    of small models) go through the engine's
    own weight-streaming kernel: alone it is level with the library for N = 4096..24576 and
    faster for K = 12288 (32 us against 36) and N = 151936 (203 against 218), and in a step it
    starts fetching weights while the kernel before it drains (a whole decode step of the
    Qwen3-8B shape at batch 8: 4.35 ms against 4.77 with the library products).  Everything else
    goes through the library matrix product (under `LLM_PAIR=all`, prompt portions take the paired tcgen05
    product `linear_pair`; by default only the gate/up product does, through `linear_silu_mul`) (the reference uses cuBLAS for all its products,
    src/layers/linear.cu:169-215).  bfloat16 operands accumulate in float32; a float32 weight
    keeps its product in true float32 (no TF32), whatever x is."""
    _dev(x, weight)
    rows = x.shape[0]
    if (x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.shape[1] % 8 == 0 and weight.data_ptr() % 16 == 0
            and rows >= 1 and (rows <= SKINNY_MAX_ROWS
                               or (rows <= SKINNY_SMALL_MAX_ROWS and skinny_small(weight.shape[0], weight.shape[1])))):
        return linear_skinny(x, weight, out_dtype or x.dtype, partials_ok=partials_ok)
    if x.shape[0] >= PAIR_MIN_ROWS and (out_dtype or x.dtype) in (torch.float32, torch.bfloat16) and _pair_takes(
            x, weight, weight.shape[0], "plain"):
        return linear_pair(x, weight, out_dtype or x.dtype)
    if weight.dtype == torch.float32:
        y = torch.mm(x if x.dtype == torch.float32 else x.float(), weight.t())
        want = out_dtype or x.dtype
        return y if want == torch.float32 else y.to(want)
    if x.dtype != weight.dtype:
        x = x.to(weight.dtype)
    if out_dtype is not None and out_dtype != x.dtype:
        return torch.mm(x, weight.t(), out_dtype=out_dtype)
    return torch.mm(x, weight.t())


def configure_library_products() -> None:
    """No reduced-precision modes in the library products: float32 stays IEEE float32 and
    bfloat16 products reduce in float32."""
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
    try:
        torch.set_float32_matmul_precision("highest")
    except Exception:
        pass
