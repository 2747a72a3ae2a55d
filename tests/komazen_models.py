"""Small Komazen configurations for the tests, and random weights for them.

The configurations differ from one another in every size and option: widths that are no powers of two, one to
four convolution taps (one tap keeps no rows between steps), stream weights above and below one, grouped and
ungrouped query heads, key and value widths that differ and that agree, latent ranks that differ from the head
sizes, a rotation over the whole rotated part and over a part of it, windows shorter than a page and over
several, a latent layer without a window, layers that read an earlier layer's cached latent with a wider and
with a narrower window than its owner's, a single head, a layer without a feed-forward.  Weights are drawn so
that activations are of order one and a lost key, a lost row of the convolution or a wrong constant moves the
logits by far more than rounding.  This file does not import the engine.
"""
from __future__ import annotations

from typing import Dict

import numpy as np
import torch


def _attn(heads, kv, dim, vdim, scale):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}


def _latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, window, base, dims=None, kv_from=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale,
         "rot": {"base": base, "dims": rot_dim if dims is None else dims}}
    if window:
        m["mask"] = {"size": window}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _layer(kind, mixer, ff):
    return {"type": kind, "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def _config(vocab, width, eps, scale, alpha, taps, layers):
    return {"architecture": "Komazen", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": scale},
            "postln_alpha": alpha, "canon": {"taps": taps}, "layers": layers}


# A: three taps, a window shorter than a page, a reader whose window is wider than its owner's, a layer without feed-forward
KOMA_A = _config(101, 40, 1e-5, 3.5, 1.7, 3, [
    _layer("attention", _attn(4, 2, 16, 24, 0.3), 56),
    _layer("latent_attention", _latent(3, 8, 4, 16, 20, 12, 0.35, 9, 500.0), 48),
    _layer("attention", _attn(2, 1, 8, 8, 0.5), None),
    _layer("latent_attention", _latent(2, 16, 4, 8, 24, 12, 0.25, 21, 500.0, kv_from=1), 40),
])
KOMA_A_PAGE = 16

# B: one tap (nothing kept between steps), ungrouped heads, a partial rotation, a latent layer without a window, page of 4
KOMA_B = _config(131, 48, 3e-6, 1.0, 0.6, 1, [
    _layer("latent_attention", _latent(4, 12, 8, 20, 16, 24, 0.2, 0, 1.0e4, dims=4), 64),
    _layer("attention", _attn(3, 3, 32, 32, 0.2), 72),
    _layer("latent_attention", _latent(1, 24, 8, 12, 40, 24, 0.3, 7, 1.0e4, dims=4, kv_from=0), None),
])
KOMA_B_PAGE = 4

# C: four taps, head size 64, a window over several pages, longer sequences, a reader with a narrower window
KOMA_C = _config(211, 64, 1e-5, 8.0, 3.0, 4, [
    _layer("latent_attention", _latent(4, 32, 16, 48, 48, 40, 0.15, 130, 20000.0), 96),
    _layer("attention", _attn(4, 2, 64, 64, 0.125), 96),
    _layer("latent_attention", _latent(2, 64, 16, 32, 32, 40, 0.1, 33, 20000.0, kv_from=0), 96),
])
KOMA_C_PAGE = 16

# D: two taps, odd sizes throughout, a single attention head, key width above value width
KOMA_D = _config(89, 36, 1e-6, 0.5, 1.0, 2, [
    _layer("attention", _attn(1, 1, 20, 12, 0.4), 30),
    _layer("latent_attention", _latent(5, 6, 2, 10, 14, 6, 0.5, 5, 50.0), 22),
    _layer("attention", _attn(6, 3, 4, 12, 1.0), 26),
])
KOMA_D_PAGE = 8

# E: latent ranks of 64 and 128, which the bfloat16 run takes on the tensor-core kernel over the cached rows: more heads
# than half a block of heads, a reader of other head sizes, a window that ends in the middle of a tile of rows
KOMA_E = _config(97, 72, 1e-5, 2.0, 1.5, 3, [
    _layer("latent_attention", _latent(18, 8, 32, 12, 36, 64, 0.2, 50, 3000.0), 80),
    _layer("attention", _attn(3, 1, 16, 24, 0.25), 64),
    _layer("latent_attention", _latent(5, 24, 32, 16, 28, 64, 0.15, 77, 3000.0, kv_from=0), 80),
    _layer("latent_attention", _latent(2, 16, 16, 40, 24, 128, 0.2, 0, 700.0), None),
])
KOMA_E_PAGE = 32

# F: attention heads of 128, which the bfloat16 run takes on the tensor cores: two query heads a key head (prompt portions
# on the kernel with accumulators in tensor memory) and one (the mma.sync kernel); a latent of 256
KOMA_F = _config(113, 64, 1e-5, 4.0, 2.0, 3, [
    _layer("attention", _attn(4, 2, 128, 128, 0.09), 96),
    _layer("latent_attention", _latent(4, 16, 32, 24, 40, 256, 0.2, 140, 5000.0), 80),
    _layer("attention", _attn(2, 2, 128, 128, 0.08), None),
])
KOMA_F_PAGE = 16


def tensor_shapes(cfg: dict) -> Dict[str, tuple]:
    """Names and shapes of a model's tensors, written out from the design's naming rules."""
    W, taps = cfg["width"], cfg["canon"]["taps"]
    out = {"embed": (cfg["vocab"], W), "final.norm": (W,), "head": (cfg["vocab"], W)}
    for i, e in enumerate(cfg["layers"]):
        p, m = f"l{i}.mix", e["mixer"]
        out[f"l{i}.norm1"] = (W,)
        out[f"l{i}.canon1"] = (W, taps)
        if e["type"] == "attention":
            H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            out.update({f"{p}.q": (H * D, W), f"{p}.k": (G * D, W), f"{p}.v": (G * V, W), f"{p}.o": (W, H * V),
                        f"{p}.q.norm": (D,), f"{p}.k.norm": (D,), f"{p}.temp": (H,), f"{p}.r1": (H,), f"{p}.r2": (H,)})
        else:
            H, D, P, V, Q, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["q_rank"], m["kv_rank"]
            out.update({f"{p}.dq": (Q, W), f"{p}.dq.norm": (Q,), f"{p}.uq": (H * (D + P), Q), f"{p}.uk": (H * D, R),
                        f"{p}.uv": (H * V, R), f"{p}.g": (H * V, W), f"{p}.o": (W, H * V)})
            if m.get("kv_from") is None:
                out.update({f"{p}.dkv": (R + P, W), f"{p}.dkv.norm": (R,)})
        if e.get("mlp"):
            ff = e["mlp"]["ff"]
            out.update({f"l{i}.norm2": (W,), f"l{i}.canon2": (W, taps), f"l{i}.mlp.gate": (ff, W), f"l{i}.mlp.up": (ff, W),
                        f"l{i}.mlp.down": (W, ff)})
    return out


def random_weights(cfg: dict, seed: int, sharp: float = 2.5) -> Dict[str, torch.Tensor]:
    """float32 tensors whose values are exactly representable in bfloat16 (so a bfloat16 run and a float32 run hold
    the same model).  Matrices N(0, 1/fan_in); what makes queries (`q`, `uq`) times `sharp` so that softmax is
    peaked and single keys matter; the taps N(0, 0.4); the temperatures 1 + N(0, 0.3); the distance bias's two
    numbers uniform in [0.2, 1.5] (positive, so that the logarithm's argument stays above one); norm weights
    1 + N(0, 0.1)."""
    rng = np.random.RandomState(seed)
    w = {}
    for name, shape in tensor_shapes(cfg).items():
        if ".canon" in name:
            t = rng.normal(0.0, 0.4, shape)
        elif name.endswith(".r1") or name.endswith(".r2"):
            t = rng.uniform(0.2, 1.5, shape)
        elif name.endswith(".temp"):
            t = 1.0 + rng.normal(0.0, 0.3, shape)
        elif len(shape) == 1:
            t = 1.0 + rng.normal(0.0, 0.1, shape)
        elif name == "embed":
            t = rng.normal(0.0, 1.0, shape)
        else:
            t = rng.normal(0.0, shape[1] ** -0.5, shape)
            if name.endswith(".mix.q") or name.endswith(".mix.uq"):
                t = t * sharp
        w[name] = torch.from_numpy(np.asarray(t, dtype=np.float32)).to(torch.bfloat16).to(torch.float32)
    return w


def random_tokens(cfg: dict, n: int, seed: int) -> list:
    return np.random.RandomState(seed).randint(0, cfg["vocab"], size=n).tolist()
