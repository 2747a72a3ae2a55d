"""A plain, slow restatement of the Komazen design: whole sequences, no cache, no state carried
between calls, one function per mechanism.  It shares no code with the engine; the tests compare
the engine with it.

Notation.  x [T, W] is the residual stream, u a sublayer's input (the stream plus its causal
convolution), p the position of a token in its sequence (from 0), `w` a dict of tensors by name,
`pre` a name prefix, `m` a mixer's entry of the configuration.  `act` rounds activations the way a
run mode would (identity for the 32-bit mode); what the design keeps in 32-bit stays unrounded.
Everything runs in float64 unless `act` rounds it.
"""
import math

import torch

F64 = torch.float64


def identity(x):
    return x


def bf16_round(x):
    """What a 16-bit run mode does to an activation between two kernels."""
    return x.to(torch.bfloat16).to(x.dtype)


def bf16_round_jittered(seed):
    """The same rounding after a relative nudge of up to half a unit in the last place: another
    implementation's rounding of the same exact value."""
    g = torch.Generator().manual_seed(seed)

    def act(x):
        nudge = (torch.rand(x.shape, generator=g, dtype=torch.float64) - 0.5) * 2.0 ** -8
        return (x * (1.0 + nudge.to(x.dtype))).to(torch.bfloat16).to(x.dtype)
    return act


def rms_unit(x, eps):
    return x * torch.rsqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)


def rms_norm(x, weight, eps):
    return rms_unit(x, eps) * weight


def embed(ids, w, scale):
    return w["embed"][torch.as_tensor(ids, dtype=torch.long)].to(F64) * scale


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def input_convolution(x, taps_w):
    """u_t = x_t + sum_j taps_w[:, j] * x_(t - taps + 1 + j), rows before the sequence's start are zero.
    taps_w is [W, taps]; the last tap weighs the token itself."""
    T, taps = x.shape[0], taps_w.shape[1]
    u = x.clone()
    for j in range(taps):
        back = taps - 1 - j
        if back < T:
            u[back:] += taps_w[:, j] * x[:T - back]
    return u


def rotate_half(t, positions, dims, base):
    """t [T, heads, n]: entry i of the first `dims` pairs with entry i + dims/2; the pair (a, b) at position
    p becomes (a cos - b sin, b cos + a sin) of the angle p * base^(-2i/dims).  The rest passes."""
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F64)
    ang = torch.as_tensor(positions, dtype=F64)[:, None] * f[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = t[..., :half], t[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, t[..., dims:]], dim=-1)


def softmax_core(scores, v, visible):
    """scores [H, T, S], visible [T, S] bool, v [H, S, V]: ordinary softmax over the visible keys."""
    scores = scores.masked_fill(~visible[None], float("-inf"))
    return torch.softmax(scores, dim=-1) @ v


def biased_attention_core(q, k, v, scale, temp, r1, r2, first_position=0):
    """q [T, H, D], k [S, G, D], v [S, G, V]; the query rows sit at positions first_position.. of the S keys.
    score(i, j) = q_i.k_j * scale * temp[h] - r1[h] * ln(1 + r2[h] * (i - j)); causal."""
    T, H, _ = q.shape
    S, G, _ = k.shape
    rep = H // G
    kk, vv = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
    i = torch.arange(first_position, first_position + T)[:, None]
    j = torch.arange(S)[None, :]
    dist = (i - j).clamp(min=0).to(F64)
    s = torch.einsum("thd,shd->hts", q, kk) * scale * temp[:, None, None]
    s = s - r1[:, None, None] * torch.log1p(r2[:, None, None] * dist[None])
    return softmax_core(s, vv.permute(1, 0, 2), j <= i).permute(1, 0, 2)          # [T, H, V]


def biased_attention(u, w, pre, m, eps, act=identity):
    """The 'attention' mixer on its input u [T, W] (already convolved)."""
    T = u.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    x = act(u)
    q = (x @ w[pre + "q"].T).view(T, H, D)
    k = (x @ w[pre + "k"].T).view(T, G, D)
    v = (x @ w[pre + "v"].T).view(T, G, V)
    q = act(rms_norm(q, w[pre + "q.norm"], eps))
    k = act(rms_norm(k, w[pre + "k.norm"], eps))
    o = biased_attention_core(q, k, act(v), m["scale"], w[pre + "temp"], w[pre + "r1"], w[pre + "r2"])
    return act(o.reshape(T, H * V)) @ w[pre + "o"].T


def latent_kv(u, w, pre, m, eps, act=identity):
    """What a latent attention layer caches per token: the normed latent c [T, kv_rank] and the rotated
    key part shared by all heads [T, rot_dim]."""
    T = u.shape[0]
    R, rot = m["kv_rank"], m["rot_dim"]
    d = act(u) @ w[pre + "dkv"].T
    c = rms_norm(d[:, :R], w[pre + "dkv.norm"], eps)
    kr = rotate_half(d[:, None, R:], range(T), m["rot"]["dims"], m["rot"]["base"])[:, 0]
    return act(c), act(kr)


def latent_attention(u, w, pre, m, eps, act=identity, shared=None):
    """The 'latent_attention' mixer on its input u.  `shared` = (c, rotated key part) of the layer whose
    cache this layer reads instead of making its own."""
    T = u.shape[0]
    H, D, rot, V, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    x = act(u)
    cq = act(rms_norm(x @ w[pre + "dq"].T, w[pre + "dq.norm"], eps))
    q = (cq @ w[pre + "uq"].T).view(T, H, D + rot)
    qn, qr = q[..., :D], rotate_half(q[..., D:], range(T), m["rot"]["dims"], m["rot"]["base"])
    c, kr = shared if shared is not None else latent_kv(u, w, pre, m, eps, act)
    kn = (c @ w[pre + "uk"].T).view(T, H, D)
    v = (c @ w[pre + "uv"].T).view(T, H, V)
    s = (torch.einsum("thd,shd->hts", act(qn), act(kn)) + torch.einsum("thd,sd->hts", act(qr), kr)) * m["scale"]
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    visible = j <= i
    if m.get("mask") is not None:
        visible = visible & (i - j < m["mask"]["size"])
    o = softmax_core(s, act(v).permute(1, 0, 2), visible).permute(1, 0, 2).reshape(T, H * V)
    gate = torch.sigmoid(x @ w[pre + "g"].T)
    return act(o * gate) @ w[pre + "o"].T


def dense_ff(u, w, pre, act=identity):
    x = act(u)
    return act(gelu_tanh(x @ w[pre + "gate"].T) * (x @ w[pre + "up"].T)) @ w[pre + "down"].T


def forward(cfg, w, ids, act=identity, layers_out=None):
    """Logits [T, vocab] of one whole sequence.  `w`: float64 tensors by name.  layers_out: a list that
    receives the stream after every layer."""
    eps, alpha = cfg["norm"]["eps"], cfg["postln_alpha"]
    x = embed(ids, w, cfg["embedding"]["scale"])
    kept = {}
    for i, layer in enumerate(cfg["layers"]):
        pre, m = f"l{i}.", layer["mixer"]
        u = input_convolution(x, w[pre + "canon1"])
        if layer["type"] == "attention":
            y = biased_attention(u, w, pre + "mix.", m, eps, act)
        elif layer["type"] == "latent_attention":
            src = m.get("kv_from")
            if src is None:
                kept[i] = latent_kv(u, w, pre + "mix.", m, eps, act)
            y = latent_attention(u, w, pre + "mix.", m, eps, act, shared=kept[i if src is None else src])
        else:
            raise ValueError(layer["type"])
        x = rms_norm(alpha * x + y, w[pre + "norm1"], eps)
        if layer.get("mlp") is not None:
            y = dense_ff(input_convolution(x, w[pre + "canon2"]), w, pre + "mlp.", act)
            x = rms_norm(alpha * x + y, w[pre + "norm2"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return rms_norm(x, w["final.norm"], eps) @ w["head"].T
