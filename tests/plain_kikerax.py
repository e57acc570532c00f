"""A plain, slow implementation of the Kikerax decoder: float64, whole sequences, one function per mechanism.

It shares nothing with the library: it takes the dictionary that config.json holds and a dictionary of tensors by
name, and runs one sequence from its first token.  Notation: x the residual [T, W], h a sublayer's input, p positions.

    layer        x <- x + rmsnorm(mixer(x)) w1;  x <- x + rmsnorm(ff(x)) w2        (the sublayers read x itself)
    attention    two softmax maps per head over the same values, combined with one number lambda per layer
    parallel     a * softmax attention whose values are its un-normed keys  +  b * a gated linear recurrent unit
    ff           W_down gelu(W_up h), or routed experts chosen from the best groups plus a shared expert
    head         softcap(E rmsnorm(x) w)
"""
from __future__ import annotations

import math

import torch

F = torch.float64


def rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.log1p(torch.exp(-z.abs())) + torch.clamp(z, min=0.0)


def lin(W, name, x, bias=False):
    y = x @ W[name].to(F).T
    if bias:
        y = y + W[name + ".b"].to(F)
    return y


# ---- positions ---------------------------------------------------------------------------------------------------
def rotary_frequencies(rot):
    """(frequencies [dims / 2], amplitude of the sines and cosines) of a `rot` object, with its scaling rule."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if not sc:
        return torch.tensor(f, dtype=F), 1.0
    factor, original = float(sc["factor"]), float(sc["original"])

    def turn_dim(turns):           # the (real-valued) pair index whose wave makes `turns` turns over `original` positions
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(turn_dim(float(sc["fast"]))), 0)
    hi = min(math.ceil(turn_dim(float(sc["slow"]))), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / factor * ramp + fi * (1.0 - ramp))
    return torch.tensor(out, dtype=F), 0.1 * math.log(factor) + 1.0


def rotate(x, pos, rot):
    """x [T, n, dim]: the first rot.dims elements of every vector turn in pairs (2i, 2i + 1) by pos * f_i."""
    if not rot:
        return x
    f, amp = rotary_frequencies(rot)
    dims = int(rot["dims"])
    ang = pos.to(F)[:, None] * f[None, :]                       # [T, dims / 2]
    c, s = (torch.cos(ang) * amp)[:, None, :], (torch.sin(ang) * amp)[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


# ---- attention ---------------------------------------------------------------------------------------------------
def visible(T, mask):
    """[T, T] booleans: query i sees key j."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if mask:
        ok = ok & ((i // int(mask["size"])) == (j // int(mask["size"])))
    return ok


def softmax_attention(q, k, v, scale, ok, softcap=None):
    """q [T, H, d], k [T, G, d], v [T, G, dv] -> [T, H, dv]; query head h reads key/value head h // (H / G)."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=F)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        if softcap:
            s = softcap * torch.tanh(s / softcap)
        s = s.masked_fill(~ok, float("-inf"))
        out[:, h] = torch.softmax(s, dim=-1) @ v[:, g]
    return out


def differential_attention(h, W, pre, m, eps):
    T = h.shape[0]
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    pos = torch.arange(T)
    q = lin(W, pre + "q", h, True).view(T, H, 2, d)
    k = lin(W, pre + "k", h, True).view(T, G, 2, d)
    v = lin(W, pre + "v", h, True).view(T, G, dv)
    q = rms(q, eps) * W[pre + "q.norm"].to(F)
    k = rms(k, eps) * W[pre + "k.norm"].to(F)
    q = rotate(q.reshape(T, 2 * H, d), pos, m.get("rot")).view(T, H, 2, d)
    k = rotate(k.reshape(T, 2 * G, d), pos, m.get("rot")).view(T, G, 2, d)
    ok = visible(T, m.get("mask"))
    a1 = softmax_attention(q[:, :, 0], k[:, :, 0], v, float(m["scale"]), ok)
    a2 = softmax_attention(q[:, :, 1], k[:, :, 1], v, float(m["scale"]), ok)
    diff = float(m["diff"])
    lam = (math.exp(float((W[pre + "lq1"].to(F) * W[pre + "lk1"].to(F)).sum()))
           - math.exp(float((W[pre + "lq2"].to(F) * W[pre + "lk2"].to(F)).sum())) + diff)
    o = rms(a1 - lam * a2, eps) * (1.0 - diff)
    o = o * torch.sigmoid(lin(W, pre + "g", h))[:, :, None]
    return lin(W, pre + "o", o.reshape(T, H * dv), True)


def query_temperature(T, qt):
    p = torch.arange(T, dtype=F)
    return 1.0 + float(qt["coef"]) * torch.log(torch.floor((p + 1.0) / float(qt["every"])) + 1.0)


def keyed_value_attention(h, W, pre, m, eps):
    """Softmax attention whose values are the keys as projected (before their norm); no rotation."""
    T = h.shape[0]
    H, G, d = int(m["heads"]), int(m["kv_heads"]), int(m["dim"])
    q = lin(W, pre + "q", h).view(T, H, d)
    k = lin(W, pre + "k", h).view(T, G, d)
    v = k
    q = rms(q, eps) * W[pre + "q.norm"].to(F)
    k = rms(k, eps) * W[pre + "k.norm"].to(F)
    if m.get("q_temp"):
        q = q * query_temperature(T, m["q_temp"])[:, None, None]
    o = softmax_attention(q, k, v, float(m["scale"]), visible(T, None), m.get("softcap"))
    o = o * torch.sigmoid(lin(W, pre + "g", h))[:, :, None]
    return lin(W, pre + "o", o.reshape(T, H * d))


# ---- the gated linear recurrent unit ------------------------------------------------------------------------------
def causal_conv(x, w, b):
    """x [T, C], w [C, taps] (last column: the current token), b [C]; zeros before the first token."""
    T, C = x.shape
    taps = w.shape[1]
    pad = torch.cat([torch.zeros(taps - 1, C, dtype=F), x])
    out = b.to(F).expand(T, C).clone()
    for j in range(taps):
        out = out + pad[j:j + T] * w[:, j].to(F)
    return out


def recurrent_block(h, W, pre, m):
    T = h.shape[0]
    width, blocks = int(m["width"]), int(m["blocks"])
    n = width // blocks
    y = gelu_tanh(lin(W, pre + "y", h, True))
    u = causal_conv(lin(W, pre + "x", h, True), W[pre + "conv"], W[pre + "conv.b"])
    ub = u.view(T, blocks, n)
    r = torch.sigmoid(torch.einsum("bon,tbn->tbo", W[pre + "ra"].to(F), ub) + W[pre + "ra.b"].to(F)).reshape(T, width)
    i = torch.sigmoid(torch.einsum("bon,tbn->tbo", W[pre + "ri"].to(F), ub) + W[pre + "ri.b"].to(F)).reshape(T, width)
    log_a = -8.0 * r * softplus(W[pre + "lam"].to(F))
    a = torch.exp(log_a)
    S = torch.zeros(width, dtype=F)
    out = torch.zeros(T, width, dtype=F)
    for t in range(T):
        S = a[t] * S + torch.sqrt(1.0 - a[t] * a[t]) * i[t] * u[t]
        out[t] = S
    return lin(W, pre + "o", out * y)


def parallel_mixer(h, W, pre, m, eps):
    left = keyed_value_attention(h, W, pre + "left.", m["left"], eps)
    right = recurrent_block(h, W, pre + "right.", m["right"])
    return float(m["left_scale"]) * left + float(m["right_scale"]) * right


# ---- feed-forward ------------------------------------------------------------------------------------------------
def dense_ff(h, W, pre):
    return lin(W, pre + "down", gelu_tanh(lin(W, pre + "up", h)))


def gated_expert(h, W, pre):
    return lin(W, pre + "down", silu(lin(W, pre + "gate", h)) * lin(W, pre + "up", h))


def router_choice(z, correction, r):
    """z [E] router logits -> (chosen experts, their weights)."""
    E, top = int(r["experts"]), int(r["top"])
    s = torch.sigmoid(z)
    c = s + correction
    groups = r.get("groups")
    if groups:
        n, keep = int(groups["count"]), int(groups["keep"])
        per = E // n
        gs = torch.stack([torch.topk(c[g * per:(g + 1) * per], min(2, per)).values.sum() for g in range(n)])
        kept = set(torch.topk(gs, keep).indices.tolist())
        c = torch.stack([c[e] if e // per in kept else torch.tensor(float("-inf"), dtype=F) for e in range(E)])
    idx = torch.topk(c, top).indices
    w = s[idx]
    return idx, w / (w.sum() + 1e-20) * float(r.get("scale", 1.0))


def routed_ff(h, W, pre, mlp, forced=None, own=None):
    """`forced` ([T, top] expert numbers): these experts are used instead of the router's own choice, with the weights
    their scores give; `own` (a list) receives the router's own choices either way."""
    T = h.shape[0]
    r = mlp["router"]
    z = lin(W, pre + "router", h)
    corr = W[pre + "correction"].to(F) if pre + "correction" in W else torch.zeros(int(r["experts"]), dtype=F)
    out = torch.zeros(T, h.shape[1], dtype=F)
    for t in range(T):
        idx, w = router_choice(z[t], corr, r)
        if own is not None:
            own.append(sorted(idx.tolist()))
        if forced is not None:
            idx = torch.as_tensor(forced[t], dtype=torch.long)
            w = torch.sigmoid(z[t])[idx]
            w = w / (w.sum() + 1e-20) * float(r.get("scale", 1.0))
        for e, we in zip(idx.tolist(), w):
            out[t] += we * gated_expert(h[t:t + 1], W, f"{pre}e{e}.")[0]
    if mlp.get("shared"):
        out = out + gated_expert(h, W, pre + "shared.")
    return out


# ---- the model ---------------------------------------------------------------------------------------------------
def forward(cfg, W, tokens, layers_out=None, forced=None, own_choices=None):
    """Logits [T, vocab] of one sequence from its first token; `layers_out` (a list) receives x after every layer.
    `forced` {layer: [T, top]} replaces the routers' choices in those layers, `own_choices` (a dictionary) receives
    every routed layer's own choices."""
    eps = float(cfg["norm"]["eps"])
    x = W["embed"].to(F)[torch.as_tensor(tokens, dtype=torch.long)]
    for i, L in enumerate(cfg["layers"]):
        pre = f"l{i}."
        if L["type"] == "attention":
            y = differential_attention(x, W, pre + "mix.", L["mixer"], eps)
        elif L["type"] == "parallel":
            y = parallel_mixer(x, W, pre + "mix.", L["mixer"], eps)
        else:
            raise ValueError(L["type"])
        x = x + rms(y, eps) * W[pre + "norm1"].to(F)
        mlp = L.get("mlp")
        if mlp:
            if mlp["kind"] == "dense":
                y = dense_ff(x, W, pre + "mlp.")
            else:
                own = None if own_choices is None else own_choices.setdefault(i, [])
                y = routed_ff(x, W, pre + "mlp.", mlp, None if forced is None else forced.get(i), own)
            x = x + rms(y, eps) * W[pre + "norm2"].to(F)
        if layers_out is not None:
            layers_out.append(x.clone())
    logits = (rms(x, eps) * W["final.norm"].to(F)) @ W["embed"].to(F).T
    cap = cfg.get("logit_softcap")
    if cap:
        logits = float(cap) * torch.tanh(logits / float(cap))
    return logits
