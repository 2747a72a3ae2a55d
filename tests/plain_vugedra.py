"""A plain, slow restatement of the Vugedra design: whole sequences, no cache, no state carried
between calls, one function per mechanism.  It shares no code with the engine; the tests compare
the engine with it.

Notation.  x [T, W] is the residual stream, u a sublayer's (normed) input, p the position of a token
in its sequence (from 0), `w` a dict of tensors by name, `pre` a name prefix, `m` a mixer's entry of
the configuration.  `act` rounds activations the way a run mode would (identity for the 32-bit mode);
what the design keeps in 32-bit stays unrounded.  Everything runs in float64 unless `act` rounds it.
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


def embed(ids, w):
    return w["embed"][torch.as_tensor(ids, dtype=torch.long)].to(F64)


def tanh_norm(x, w, name):
    """The design's norm: no mean, no variance.  tanh(alpha x) * weight + bias, alpha one number."""
    return torch.tanh(w[name + ".alpha"].to(F64) * x) * w[name].to(F64) + w[name + ".b"].to(F64)


def silu(z):
    return z * torch.sigmoid(z)


def rotation_table(positions, rot):
    """cos and sin [T, dims/2] of the angles p * f_i, f_i = base^(-2i/dims), with the frequencies stretched
    by `scaling` where it is given: pairs whose wavelength is long against the original context are slowed
    by `factor`, short ones are kept, a linear ramp over the pair index between the two; cos and sin are
    then both multiplied by 0.1 ln(factor) + 1."""
    dims, base = int(rot["dims"]), float(rot["base"])
    half = dims // 2
    f = [base ** (-2.0 * i / dims) for i in range(half)]
    mag = 1.0
    sc = rot.get("scaling")
    if sc:
        factor, orig = float(sc["factor"]), float(sc["original"])

        def pair_of(turns):
            return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
        lo = max(math.floor(pair_of(float(sc["fast"]))), 0)
        hi = min(math.ceil(pair_of(float(sc["slow"]))), dims - 1)
        for i in range(half):
            ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
            f[i] = f[i] / factor * ramp + f[i] * (1.0 - ramp)
        mag = 0.1 * math.log(factor) + 1.0
    ang = torch.as_tensor(positions, dtype=F64)[:, None] * torch.tensor(f, dtype=F64)[None, :]
    return torch.cos(ang) * mag, torch.sin(ang) * mag


def rotate_pairs(t, positions, rot):
    """t [T, heads, n]: of the first rot.dims entries, entry 2i pairs with entry 2i + 1; the pair (a, b)
    becomes (a cos - b sin, b cos + a sin).  The rest passes."""
    if not rot:
        return t
    dims = int(rot["dims"])
    c, s = rotation_table(positions, rot)
    c, s = c[:, None, :], s[:, None, :]
    a, b = t[..., 0:dims:2], t[..., 1:dims:2]
    out = t.clone()
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def visible_keys(T, mask):
    """[T, T] bool: query i sees key j if j <= i and (i - j < size or j < keep_first); without a mask every j <= i."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    vis = j <= i
    if mask:
        vis = vis & ((i - j < int(mask["size"])) | (j < int(mask.get("keep_first", 0))))
    return vis


def softmax_core(scores, v, visible, sink):
    """scores [H, T, S], visible [T, S] bool, v [H, S, V].  sink: one more term exp(0) in the denominator
    that carries no value."""
    scores = scores.masked_fill(~visible[None], float("-inf"))
    if not sink:
        return torch.softmax(scores, dim=-1) @ v
    top = torch.clamp(scores.max(dim=-1, keepdim=True).values, min=0.0)
    e = torch.exp(scores - top)
    return (e / (e.sum(dim=-1, keepdim=True) + torch.exp(-top))) @ v


def attention(u, w, pre, m, eps, act=identity):
    T = u.shape[0]
    H, G, D, V = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    g = lambda n: w[pre + n].to(F64)
    q = u @ g("q").T + g("q.b")
    k = u @ g("k").T + g("k.b")
    v = u @ g("v").T + g("v.b")
    q = rms_unit(q, eps) * g("q.norm")          # over the whole projection, before the heads are split
    k = rms_unit(k, eps) * g("k.norm")
    pos = list(range(T))
    q = act(rotate_pairs(q.view(T, H, D), pos, m.get("rot")))
    k = act(rotate_pairs(k.view(T, G, D), pos, m.get("rot")))
    v = act(v.view(T, G, V))
    rep = H // G
    kh = k.permute(1, 0, 2).repeat_interleave(rep, dim=0)
    vh = v.permute(1, 0, 2).repeat_interleave(rep, dim=0)
    scores = (q.permute(1, 0, 2) @ kh.transpose(1, 2)) * float(m["scale"])
    o = softmax_core(scores, vh, visible_keys(T, m.get("mask")), sink=True)      # [H, T, V]
    gate = torch.sigmoid(u @ g("g").T)                                          # [T, H]
    o = o.permute(1, 0, 2) * gate[:, :, None]
    return act(o.reshape(T, H * V)) @ g("o").T


def decay_log(u, w, pre, tau):
    """ln alpha [T, heads*dim] with alpha = sigmoid(z)^(1/tau), z = W_a2 (W_a1 u) + b."""
    z = (u @ w[pre + "a1"].to(F64).T) @ w[pre + "a2"].to(F64).T + w[pre + "a2.b"].to(F64)
    return torch.nn.functional.logsigmoid(z) / tau


def gla(u, w, pre, m, eps, act=identity, state=None):
    """S_t = diag(alpha_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t per head, token by token."""
    T = u.shape[0]
    H, D, V = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    g = lambda n: w[pre + n].to(F64)
    q = (u @ g("q").T).view(T, H, D) * D ** -0.5
    k = (u @ g("k").T).view(T, H, D)
    v = (u @ g("v").T).view(T, H, V)
    a = torch.exp(decay_log(u, w, pre, float(m["tau"]))).view(T, H, D)
    S = torch.zeros(H, D, V, dtype=F64) if state is None else state
    o = torch.zeros(T, H, V, dtype=F64)
    for t in range(T):
        S = a[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = rms_unit(o, eps) * g("norm")
    o = o.reshape(T, H * V) * silu(u @ g("g").T)
    return act(o) @ g("o").T, S


def latent_attention(u, w, pre, m, eps, act=identity):
    T = u.shape[0]
    H, D, R, V, C = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    g = lambda n: w[pre + n].to(F64)
    cq = act(rms_unit(u @ g("dq").T, eps) * g("dq.norm"))
    q = (cq @ g("uq").T).view(T, H, D + R)
    down = u @ g("dkv").T
    c = act(rms_unit(down[:, :C], eps) * g("dkv.norm"))
    pos = list(range(T))
    kr = act(rotate_pairs(down[:, None, C:], pos, m.get("rot")))                # [T, 1, R], shared by the heads
    qr = rotate_pairs(q[..., D:], pos, m.get("rot"))
    kn = (c @ g("uk").T).view(T, H, D)
    vv = (c @ g("uv").T).view(T, H, V)
    qh = act(torch.cat([q[..., :D], qr], dim=-1)).permute(1, 0, 2)
    kh = torch.cat([kn, kr.expand(T, H, R)], dim=-1).permute(1, 0, 2)
    scores = (qh @ kh.transpose(1, 2)) * float(m["scale"])
    o = softmax_core(scores, vv.permute(1, 0, 2), visible_keys(T, m.get("mask")), sink=False)
    gate = torch.sigmoid(u @ g("g").T)
    o = o.permute(1, 0, 2) * gate[:, :, None]
    return act(o.reshape(T, H * V)) @ g("o").T


def gated_ff(u, w, pre, act=identity):
    g = lambda n: w[pre + n].to(F64)
    return act(silu(u @ g("gate").T) * (u @ g("up").T)) @ g("down").T


def route(u, w, pre, router):
    """Per token the chosen experts and their weights: softmax over all router outputs; the choice is by
    score + correction, the weights are the chosen scores themselves divided by their sum."""
    z = u @ w[pre + "router"].to(F64).T
    s = torch.softmax(z, dim=-1)
    pick = torch.topk(s + w[pre + "correction"].to(F64), int(router["top"]), dim=-1).indices
    chosen = torch.gather(s, 1, pick)
    return pick, chosen / (chosen.sum(dim=-1, keepdim=True) + 1e-20)


def routed_ff(u, w, pre, mlp, act=identity, route_input=None):
    """Experts 0 .. experts-1 are feed-forwards; the `identity` router outputs after them return the token's
    input itself.  A shared expert, where the entry has one, runs for every token."""
    router = mlp["router"]
    E = int(router["experts"])
    pick, weight = route(u if route_input is None else route_input, w, pre, router)
    out = torch.zeros(u.shape[0], w[pre + "router"].shape[1], dtype=F64)
    for t in range(u.shape[0]):
        for e, a in zip(pick[t].tolist(), weight[t].tolist()):
            y = gated_ff(u[t:t + 1], w, f"{pre}e{e}.", act)[0] if e < E else u[t]
            out[t] += a * y
    if mlp.get("shared") is not None:
        out = out + gated_ff(u, w, pre + "shared.", act)
    return out


def owner(layers, i):
    while layers[i].get("weights_of") is not None:
        i = layers[i]["weights_of"]
    return i


def forward(cfg, w, ids, act=identity, collect=None):
    """Logits [T, vocab] of one whole sequence.  `collect`, a list, receives the stream after every layer."""
    eps = float(cfg["norm"]["eps"])
    x = embed(ids, w)
    layers = cfg["layers"]
    for i in range(len(layers)):
        j = owner(layers, i)
        e, pre = layers[j], f"l{j}."
        u = act(tanh_norm(x, w, pre + "norm1"))
        kind = e["type"]
        if kind == "attention":
            y = attention(u, w, pre + "mix.", e["mixer"], eps, act)
        elif kind == "gla":
            y, _ = gla(u, w, pre + "mix.", e["mixer"], eps, act)
        elif kind == "latent_attention":
            y = latent_attention(u, w, pre + "mix.", e["mixer"], eps, act)
        else:
            raise ValueError(kind)
        x = x + tanh_norm(y, w, pre + "norm1b")
        if e.get("mlp") is not None:
            u = act(tanh_norm(x, w, pre + "norm2"))
            if e["mlp"]["kind"] == "dense":
                y = gated_ff(u, w, pre + "mlp.", act)
            else:
                y = routed_ff(u, w, pre + "mlp.", e["mlp"], act)
            x = x + tanh_norm(y, w, pre + "norm2b")
        if collect is not None:
            collect.append(x.clone())
    return act(tanh_norm(x, w, "final.norm")) @ w["head"].to(F64).T
