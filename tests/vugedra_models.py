"""Small Vugedra configurations for the tests, and random weights for them.

The configurations differ from one another in every size and option: widths that are no multiples of four or
eight, grouped, ungrouped and single heads, key and value widths that differ and that agree, rotations over a part
of a head and over all of it, with and without stretched frequencies, windows shorter than a page and over several,
kept first keys fewer than a page, more than a page and more than the window, an attention layer without a mask and
without a rotation, latents of sizes that the tensor-core kernel takes and that it does not, routers with one, two
and all outputs chosen, with none, one and several outputs that are no experts, with and without a shared expert
whose size differs from the experts', dense feed-forwards, layers without one, layers that run an earlier and a
LATER layer's tensors.  Weights are drawn so that activations are of order one and a lost key, a lost state or a
wrong constant moves the logits by far more than rounding.  This file does not import the engine.
"""
from __future__ import annotations

from typing import Dict

import numpy as np
import torch


def _rot(base, dims, scaling=None):
    r = {"base": base, "dims": dims}
    if scaling:
        r["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return r


def _attn(heads, kv, dim, vdim, scale, window=None, keep=None, rot=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if window:
        m["mask"] = {"size": window}
        if keep is not None:
            m["mask"]["keep_first"] = keep
    if rot:
        m["rot"] = rot
    return m


def _gla(heads, dim, vdim, tau):
    return {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}


def _latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, rot):
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
            "scale": scale, "rot": rot}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(experts, top, ff, identity=None, shared=None):
    router = {"experts": experts, "top": top}
    if identity is not None:
        router["identity"] = identity
    m = {"kind": "moe", "expert": {"ff": ff}, "router": router}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def _layer(kind, mixer, mlp, weights_of=None):
    e = {"type": kind, "mixer": mixer, "mlp": mlp}
    if weights_of is not None:
        e["weights_of"] = weights_of
    return e


def _config(vocab, width, eps, layers):
    return {"architecture": "Vugedra", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}


# A: a window shorter than a page with three kept keys, a partial rotation with stretched frequencies, one output of the
# router that is no expert, a shared expert wider than the experts, a layer that runs an earlier layer's tensors
_A0 = _attn(4, 2, 16, 24, 0.3, window=9, keep=3, rot=_rot(500.0, 8, (4.0, 16, 4.0, 0.5)))
VUG_A = _config(101, 40, 1e-5, [
    _layer("attention", _A0, _dense(56)),
    _layer("gla", _gla(3, 8, 12, 4.0), _moe(5, 2, 16, identity=1, shared=24)),
    _layer("latent_attention", _latent(3, 8, 4, 16, 20, 12, 0.35, _rot(300.0, 4, (2.0, 8, 2.0, 0.25))), _moe(4, 1, 24)),
    _layer("attention", _A0, _dense(56), weights_of=0),
    _layer("gla", _gla(2, 16, 8, 1.0), None),
])
VUG_A_PAGE = 16

# B: pages of 4, ungrouped heads, a rotation over the whole head without stretching, a window without kept keys, an
# attention layer with no mask and no rotation at all, top = every output of the router, a width that is no multiple of 4
VUG_B = _config(131, 30, 3e-6, [
    _layer("latent_attention", _latent(4, 12, 8, 20, 16, 24, 0.2, _rot(1.0e4, 8)), _moe(3, 5, 20, identity=2)),
    _layer("attention", _attn(3, 3, 8, 8, 0.4, window=5, rot=_rot(50.0, 8)), _dense(44)),
    _layer("attention", _attn(2, 1, 12, 6, 0.3), None),
    _layer("gla", _gla(5, 4, 6, 16.0), _moe(6, 3, 12, shared=10)),
])
VUG_B_PAGE = 4

# C: longer sequences: a window over several pages with more kept keys than a page holds, head size 64, a latent of 64
# with a rotated part of 16 (the tensor-core kernel over cached rows in the 16-bit mode), a layer that runs a LATER one's tensors
_C_MOE = _moe(6, 3, 32, identity=3, shared=32)
VUG_C = _config(211, 64, 1e-5, [
    _layer("gla", _gla(2, 32, 64, 8.0), _C_MOE, weights_of=3),
    _layer("attention", _attn(4, 2, 64, 64, 0.125, window=130, keep=20, rot=_rot(2.0e4, 32, (8.0, 64, 16.0, 1.0))), _dense(96)),
    _layer("latent_attention", _latent(4, 32, 16, 48, 48, 64, 0.15, _rot(2.0e4, 16, (2.0, 128, 8.0, 1.0))), _moe(8, 2, 32, identity=2)),
    _layer("gla", _gla(2, 32, 64, 8.0), _C_MOE),
])
VUG_C_PAGE = 16

# D: odd sizes throughout, a single attention head, more kept keys than the window is wide, key width above value width,
# a window of one key, a router without outputs that are no experts and without a shared expert
VUG_D = _config(89, 36, 1e-6, [
    _layer("attention", _attn(1, 1, 20, 12, 0.4, window=3, keep=7, rot=_rot(100.0, 6, (3.0, 10, 2.0, 0.5))), _moe(7, 2, 10)),
    _layer("latent_attention", _latent(5, 6, 2, 10, 14, 6, 0.5, _rot(50.0, 2)), _dense(22)),
    _layer("attention", _attn(6, 3, 4, 12, 1.0, window=1, keep=1, rot=_rot(10.0, 4)), _dense(26)),
    _layer("gla", _gla(1, 24, 20, 2.0), _dense(30)),
])
VUG_D_PAGE = 8

# E: attention heads of 128 in groups of two and of one, a window that ends in the middle of a page, kept keys; a latent
# of 128 with a rotated part of 32 and more heads than sixteen
VUG_E = _config(113, 64, 1e-5, [
    _layer("attention", _attn(4, 2, 128, 128, 0.09, window=140, keep=6, rot=_rot(1.0e4, 64, (2.0, 64, 32.0, 1.0))), _moe(4, 2, 40, identity=1, shared=48)),
    _layer("latent_attention", _latent(18, 8, 32, 12, 36, 128, 0.2, _rot(3000.0, 32, (4.0, 32, 8.0, 1.0))), _dense(80)),
    _layer("attention", _attn(2, 2, 128, 128, 0.08, window=33, keep=0, rot=_rot(1.0e4, 128)), None),
    _layer("gla", _gla(2, 64, 32, 16.0), _dense(72)),
])
VUG_E_PAGE = 16


def owner(cfg: dict, i: int) -> int:
    while cfg["layers"][i].get("weights_of") is not None:
        i = cfg["layers"][i]["weights_of"]
    return i


GLA_RANK = 5          # of the low-rank decay projection; only the tensors know it


def _norm_shapes(name, W):
    return {name: (W,), name + ".alpha": (), name + ".b": (W,)}


def tensor_shapes(cfg: dict) -> Dict[str, tuple]:
    """Names and shapes of a model's tensors, written out from the design's naming rules."""
    W = cfg["width"]
    out = {"embed": (cfg["vocab"], W), "head": (cfg["vocab"], W)}
    out.update(_norm_shapes("final.norm", W))
    for i, e in enumerate(cfg["layers"]):
        if e.get("weights_of") is not None:
            continue
        p, m = f"l{i}.mix", e["mixer"]
        out.update(_norm_shapes(f"l{i}.norm1", W))
        out.update(_norm_shapes(f"l{i}.norm1b", W))
        if e["type"] == "attention":
            H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            out.update({f"{p}.q": (H * D, W), f"{p}.k": (G * D, W), f"{p}.v": (G * V, W), f"{p}.o": (W, H * V),
                        f"{p}.q.b": (H * D,), f"{p}.k.b": (G * D,), f"{p}.v.b": (G * V,), f"{p}.q.norm": (H * D,),
                        f"{p}.k.norm": (G * D,), f"{p}.g": (H, W)})
        elif e["type"] == "gla":
            H, D, V = m["heads"], m["dim"], m["vdim"]
            out.update({f"{p}.q": (H * D, W), f"{p}.k": (H * D, W), f"{p}.v": (H * V, W), f"{p}.g": (H * V, W),
                        f"{p}.o": (W, H * V), f"{p}.norm": (V,), f"{p}.a1": (GLA_RANK, W), f"{p}.a2": (H * D, GLA_RANK),
                        f"{p}.a2.b": (H * D,)})
        else:
            H, D, P, V, Q, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["q_rank"], m["kv_rank"]
            out.update({f"{p}.dq": (Q, W), f"{p}.dq.norm": (Q,), f"{p}.uq": (H * (D + P), Q), f"{p}.dkv": (R + P, W),
                        f"{p}.dkv.norm": (R,), f"{p}.uk": (H * D, R), f"{p}.uv": (H * V, R), f"{p}.g": (H, W),
                        f"{p}.o": (W, H * V)})
        mlp = e.get("mlp")
        if not mlp:
            continue
        out.update(_norm_shapes(f"l{i}.norm2", W))
        out.update(_norm_shapes(f"l{i}.norm2b", W))
        f = f"l{i}.mlp"
        if mlp["kind"] == "dense":
            out.update({f"{f}.gate": (mlp["ff"], W), f"{f}.up": (mlp["ff"], W), f"{f}.down": (W, mlp["ff"])})
            continue
        E, I, ff = mlp["router"]["experts"], mlp["router"].get("identity", 0), mlp["expert"]["ff"]
        out.update({f"{f}.router": (E + I, W), f"{f}.correction": (E + I,)})
        for x in range(E):
            out.update({f"{f}.e{x}.gate": (ff, W), f"{f}.e{x}.up": (ff, W), f"{f}.e{x}.down": (W, ff)})
        if mlp.get("shared"):
            s = mlp["shared"]["ff"]
            out.update({f"{f}.shared.gate": (s, W), f"{f}.shared.up": (s, W), f"{f}.shared.down": (W, s)})
    return out


def random_weights(cfg: dict, seed: int, sharp: float = 2.5) -> Dict[str, torch.Tensor]:
    """float32 tensors whose values are exactly representable in bfloat16 (so a 16-bit run and a 32-bit run hold the
    same model).  Matrices N(0, 1/fan_in); what makes queries times `sharp` so that softmax is peaked and single keys
    matter; routers times 3 and corrections N(0, 0.15), so that the correction changes choices and few calls are
    close; the decay's bias N(0, 2), so that channels forget at very different rates; the norms' alphas in
    [0.5, 1.5], their biases N(0, 0.1), vectors that multiply 1 + N(0, 0.1)."""
    rng = np.random.RandomState(seed)
    w = {}
    for name, shape in tensor_shapes(cfg).items():
        if name.endswith(".alpha"):
            t = rng.uniform(0.5, 1.5, shape)
        elif name.endswith(".a2.b"):
            t = rng.normal(0.0, 2.0, shape)
        elif name.endswith(".correction"):
            t = rng.normal(0.0, 0.15, shape)
        elif name.endswith(".b"):
            t = rng.normal(0.0, 0.1, shape)
        elif len(shape) == 1:
            t = 1.0 + rng.normal(0.0, 0.1, shape)
        elif name == "embed":
            t = rng.normal(0.0, 1.0, shape)
        else:
            t = rng.normal(0.0, shape[1] ** -0.5, shape)
            if name.endswith(".mix.q") or name.endswith(".mix.uq"):
                t = t * sharp
            if name.endswith(".router"):
                t = t * 3.0
            if name.endswith(".a2"):
                t = t * 2.0
        w[name] = torch.from_numpy(np.asarray(t, dtype=np.float32)).to(torch.bfloat16).to(torch.float32)
    return w


def random_tokens(cfg: dict, n: int, seed: int) -> list:
    return np.random.RandomState(seed).randint(0, cfg["vocab"], size=n).tolist()
