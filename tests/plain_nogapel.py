"""A plain, slow Nogapel: one function per mechanism, float64 on the CPU, whole sequences, nothing shared with
the library.  `weights` is {tensor name: torch tensor}; `cfg` the config.json dictionary.

Notation: T tokens, W model width; a linear map is y = x @ M.T for a stored M [out, in].
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms_norm(x, weight, eps):
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def relu_squared(z):
    return torch.clamp(z, min=0.0) ** 2


def frequencies(rot):
    """f_i = base^(-2i/dims), i < dims/2; with `scaling` the long wavelengths are slowed down by `factor`, the
    short ones kept, and those between blended linearly in original/wavelength."""
    dims = rot["dims"]
    out = []
    sc = rot.get("scaling")
    for i in range(dims // 2):
        f = float(rot["base"]) ** (-2.0 * i / dims)
        if sc:
            wavelength = 2.0 * math.pi / f
            if wavelength < sc["original"] / sc["high"]:
                pass
            elif wavelength > sc["original"] / sc["low"]:
                f = f / sc["factor"]
            else:
                s = (sc["original"] / wavelength - sc["low"]) / (sc["high"] - sc["low"])
                f = (1.0 - s) * f / sc["factor"] + s * f
        out.append(f)
    return torch.tensor(out, dtype=F64)


def rotate_interleaved(x, positions, rot):
    """x [T, heads, D]: elements (2i, 2i + 1), i < dims/2, of every head turn by position * f_i; the rest pass."""
    dims = rot["dims"]
    a = positions.to(F64)[:, None] * frequencies(rot)[None, :]          # [T, dims/2]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def short_conv(u, w):
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros before the start."""
    T, C = u.shape
    taps = w.shape[1]
    y = torch.zeros(T, C, dtype=F64)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                y[t] += w[:, j] * u[s]
    return y


def masked_softmax_attention(q, k, v, scale, window, sink):
    """q [T, H, D], k [T, G, D], v [T, G, Dv] -> [T, H, Dv].  Query i sees key j when 0 <= i - j (< window, if one
    is given).  `sink` [H] or None: exp(sink[h]) joins the denominator, with no key and no value."""
    T, H, _ = q.shape
    G = k.shape[1]
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if window is not None:
        ok = ok & (i - j < window)
    out = torch.zeros(T, H, v.shape[2], dtype=F64)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        s = s.masked_fill(~ok, float("-inf"))
        if sink is None:
            p = torch.softmax(s, dim=-1)
        else:
            m = torch.maximum(s.max(dim=-1, keepdim=True).values, sink[h])
            e = torch.exp(s - m)
            p = e / (e.sum(-1, keepdim=True) + torch.exp(sink[h] - m))
        out[:, h] = p @ v[:, g]
    return out


def attention_mixer(h, w, p, m, eps, positions, v_first):
    """`p` the tensor-name prefix ('l0.mix.'), `m` the mixer's config.  `v_first`: None in the first layer with
    v_mix (and in layers without it), else that layer's values [T, G, Dv].  Returns (output [T, W], values)."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q, k, v = h @ w[p + "q"].T, h @ w[p + "k"].T, h @ w[p + "v"].T
    if m.get("conv"):
        q, k, v = short_conv(q, w[p + "q.conv"]), short_conv(k, w[p + "k.conv"]), short_conv(v, w[p + "v.conv"])
    q, k, v = q.view(T, H, D), k.view(T, G, D), v.view(T, G, Dv)
    q, k = rms_norm(q, w[p + "q.norm"], eps), rms_norm(k, w[p + "k.norm"], eps)
    if m.get("rot"):
        q, k = rotate_interleaved(q, positions, m["rot"]), rotate_interleaved(k, positions, m["rot"])
    if v_first is not None:
        lam = w[p + "vmix"]
        v = (1.0 - lam) * v + lam * v_first
    window = m["mask"]["size"] if m.get("mask") else None
    o = masked_softmax_attention(q, k, v, m["scale"], window, None)
    return o.reshape(T, H * Dv) @ w[p + "o"].T, v


def latent_attention_mixer(h, w, p, m, eps, positions):
    T = h.shape[0]
    H, D, R, Dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    cq = rms_norm(h @ w[p + "dq"].T, w[p + "dq.norm"], eps)
    q = (cq @ w[p + "uq"].T).view(T, H, D + R)
    dkv = h @ w[p + "dkv"].T
    c = rms_norm(dkv[:, :rank], w[p + "dkv.norm"], eps)
    rot = {"base": m["rot"]["base"], "dims": R, "scaling": m["rot"].get("scaling")}
    k_rot = rotate_interleaved(dkv[:, rank:].view(T, 1, R), positions, rot)
    q_rot = rotate_interleaved(q[..., D:], positions, rot)
    k_plain = (c @ w[p + "uk"].T).view(T, H, D)
    v = (c @ w[p + "uv"].T).view(T, H, Dv)
    qq = torch.cat([q[..., :D], q_rot], dim=-1)
    kk = torch.cat([k_plain, k_rot.expand(T, H, R)], dim=-1)
    o = masked_softmax_attention(qq, kk, v, m["scale"], None, w[p + "sink"])
    return o.reshape(T, H * Dv) @ w[p + "o"].T


def dense_feed_forward(h, w, p):
    return relu_squared(h @ w[p + "up"].T) @ w[p + "down"].T


def token_side_input(x, tokens, w, p, layer, dim, eps):
    """x <- x + rmsnorm(proj(gelu(gate x) * e)) * norm, e = the layer's slice of the side table's row."""
    e = w["side.embed"][tokens][:, layer * dim:(layer + 1) * dim]
    y = (gelu_tanh(x @ w[p + "gate"].T) * e) @ w[p + "proj"].T
    return x + rms_norm(y, w[p + "norm"], eps)


def forward(cfg, weights, tokens, capture=None):
    """Logits [T, vocab] of one sequence from its first token on; `capture` (a list) receives the residual after
    every layer."""
    w = {k: v.to(F64) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    positions = torch.arange(tokens.numel())
    x = rms_norm(w["embed"][tokens], w["embed.norm"], eps)
    side = cfg.get("token_side")
    v_first = None
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = rms_norm(x, w[p + "norm1"], eps)
        m = L["mixer"]
        if L["type"] == "attention":
            mixes = bool(m.get("v_mix"))
            y, v = attention_mixer(h, w, p + "mix.", m, eps, positions, v_first if mixes else None)
            if mixes and v_first is None:
                v_first = v
        elif L["type"] == "latent_attention":
            y = latent_attention_mixer(h, w, p + "mix.", m, eps, positions)
        else:
            raise ValueError(L["type"])
        if L.get("mlp"):
            y = y + dense_feed_forward(h, w, p + "mlp.")
        x = x + y
        if side:
            x = token_side_input(x, tokens, w, p + "side.", i, side["dim"], eps)
        if capture is not None:
            capture.append(x.clone())
    return rms_norm(x, w["final.norm"], eps) @ w["head"].T
