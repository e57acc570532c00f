"""Small Nogapel configurations and weights for the tests.

The weights are drawn here, not by the library's random mode, with spreads chosen so that faults show: attention scores
a few units wide (a single key can carry a row), convolution taps of both signs, norm weights away from one, mixing
weights away from zero and one, sinks that take a real share of a row, side vectors that move the residual.
"""
from __future__ import annotations

import json
import os
import tempfile

import torch


def attention(heads, kv_heads, dim, vdim, window=None, conv=None, v_mix=None, rot_dims=None, base=10000.0,
              scaling=None, scale=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
         "scale": (3.0 / dim ** 0.5) if scale is None else scale}
    if window is not None:
        m["mask"] = {"size": window}
    if conv is not None:
        m["conv"] = conv
    if v_mix is not None:
        m["v_mix"] = v_mix
    if rot_dims is not None:
        m["rot"] = {"base": base, "dims": rot_dims}
        if scaling is not None:
            m["rot"]["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return m


def latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, base=10000.0, scaling=None, scale=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
         "scale": (3.0 / (dim + rot_dim) ** 0.5) if scale is None else scale, "rot": {"base": base, "dims": rot_dim}}
    if scaling is not None:
        m["rot"]["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return m


def layer(mixer, ff):
    kind = "latent_attention" if "kv_rank" in mixer else "attention"
    return {"type": kind, "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def model(layers, width, vocab, side=None, eps=1e-5):
    cfg = {"architecture": "Nogapel", "layers": layers, "norm": {"eps": eps}, "vocab": vocab, "width": width}
    if side is not None:
        cfg["token_side"] = {"dim": side}
    return cfg


# A: sizes that are no multiples of 8 (the float32-pipe products in both precisions); the latent layer first, so that
# the first layer with value mixing is not layer 0; grouped keys, values of another size than keys, a rotation of part
# of the head with frequency scaling whose three branches all occur, short windows, two to five taps, a layer without
# a feed-forward, one attention layer outside the value mixing.
MIXED_A = model([
    layer(latent(3, 12, 6, 10, 14, 18, base=300.0, scaling=(4.0, 1.0, 4.0, 64)), 44),
    layer(attention(4, 2, 12, 10, window=11, conv=3, v_mix=True, rot_dims=8, base=200.0, scaling=(8.0, 1.0, 4.0, 64)), 50),
    layer(attention(6, 3, 10, 6, window=30, conv=2, rot_dims=10), None),
    layer(attention(2, 2, 20, 10, window=7, conv=5, v_mix=True, rot_dims=20, base=5000.0), 28),
    layer(latent(2, 20, 10, 14, 9, 26), 36),
    layer(attention(4, 2, 6, 10, window=64, conv=4, v_mix=True), 20),
], width=52, vocab=97, side=6)

# B: multiples of 8 and 16, so that the bfloat16 path runs the tensor-core products; a latent row of 128 and of 64
# elements (both tensor-core attention kernels), attention heads whose keys and values have one size 64, a window
# that ends inside a page and one that spans pages; other eps.
MIXED_B = model([
    layer(attention(4, 1, 64, 64, window=37, conv=3, v_mix=True, rot_dims=64, base=2.5e5, scaling=(4.0, 1.0, 8.0, 256)), 192),
    layer(latent(4, 48, 16, 40, 64, 112), 128),
    layer(latent(8, 16, 16, 32, 32, 48, base=500.0), 64),
    layer(attention(2, 1, 64, 64, window=100, conv=2, v_mix=True, rot_dims=32), 256),
], width=128, vocab=384, side=16, eps=1e-6)

# C: what the other two make equal or absent: no side vectors, a window of one, no rotation, one tap, eight taps, no
# convolution, one head, more key/value heads than one with value mixing, a layer that sees everything, a latent whose
# rotated part is larger than its plain part, a key size of four.
MIXED_C = model([
    layer(attention(2, 2, 4, 8, window=1, conv=1, v_mix=True), 40),
    layer(attention(1, 1, 40, 40, conv=8, rot_dims=40, base=50.0, scaling=(0.5, 2.0, 3.0, 16)), None),
    layer(latent(1, 4, 12, 8, 5, 7), 24),
    layer(attention(4, 2, 8, 8, window=3, v_mix=True, rot_dims=2), 16),
], width=40, vocab=64)


def draw_config(seed: int) -> dict:
    """A configuration whose every size, option and constant is drawn from the seed."""
    import random
    rng = random.Random(seed)
    n_layers = rng.randint(1, 5)
    G, Dv = rng.choice([1, 2, 3]), rng.choice([8, 24, 64, 128])          # shared by the layers that mix values
    layers = []
    for _ in range(n_layers):
        if rng.random() < 0.45:
            rd = rng.choice([2, 8, 16, 32, 64])
            rank = rng.choice([8, 24, 32, 64, 96, 192])
            sc = rng.choice([None, None, (rng.choice([2.0, 8.0]), 1.0, rng.choice([2.0, 4.0]), rng.choice([16, 256]))])
            m = latent(rng.choice([1, 2, 5, 8]), rng.choice([4, 16, 32, 64]), rd, rng.choice([8, 20, 64]),
                       rng.choice([8, 24, 64]), rank, base=rng.choice([100.0, 1e4, 5e5]), scaling=sc)
        else:
            mixes = rng.random() < 0.6
            g = G if mixes else rng.choice([1, 2, 4])
            D = rng.choice([8, 16, 20, 32, 64, 128])
            dv = Dv if mixes else rng.choice([D, D, 8, 24])
            sc = rng.choice([None, None, (rng.choice([2.0, 8.0]), 1.0, rng.choice([2.0, 4.0]), rng.choice([16, 256]))])
            rot = rng.choice([None, D, max(2, D // 4 * 2)])
            m = attention(g * rng.choice([1, 2, 4]), g, D, dv, window=rng.choice([None, 1, 7, 30, 64, 100]),
                          conv=rng.choice([None, 1, 2, 4, 8]), v_mix=mixes if rng.random() < 0.8 or mixes else None,
                          rot_dims=rot, base=rng.choice([100.0, 1e4, 1e6]), scaling=sc if rot else None)
        layers.append(layer(m, rng.choice([None, 24, 64, 256])))
    return model(layers, width=rng.choice([24, 40, 64, 128, 264]), vocab=rng.choice([50, 131, 449]),
                 side=rng.choice([None, 1, 4, 16, 40]), eps=rng.choice([1e-5, 1e-6]))


def draw_weights(cfg: dict, seed: int) -> dict:
    """{name: bfloat16 tensor} for a configuration."""
    g = torch.Generator().manual_seed(seed)
    W = {}

    def rn(shape, std, mean=0.0):
        if isinstance(shape, int):
            shape = (shape,)
        return (torch.randn(*shape, generator=g) * std + mean).to(torch.bfloat16)

    width, vocab, n = cfg["width"], cfg["vocab"], len(cfg["layers"])
    W["embed"] = rn((vocab, width), 1.0)
    W["embed.norm"] = rn(width, 0.2, 1.0)
    W["head"] = rn((vocab, width), 2.0 * width ** -0.5)
    W["final.norm"] = rn(width, 0.15, 1.0)
    side = (cfg.get("token_side") or {}).get("dim")
    if side:
        W["side.embed"] = rn((vocab, n * side), 1.0)
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        W[p + "norm1"] = rn(width, 0.15, 1.0)
        q = p + "mix."
        if L["type"] == "attention":
            H, D = m["heads"], m["dim"]
            G, Dv = m.get("kv_heads", H), m.get("vdim", D)
            W[q + "q"] = rn((H * D, width), width ** -0.5)
            W[q + "k"] = rn((G * D, width), width ** -0.5)
            W[q + "v"] = rn((G * Dv, width), width ** -0.5)
            W[q + "q.norm"], W[q + "k.norm"] = rn(D, 0.3, 1.0), rn(D, 0.3, 1.0)
            if m.get("conv"):
                for name, rows in (("q", H * D), ("k", G * D), ("v", G * Dv)):
                    W[q + name + ".conv"] = rn((rows, m["conv"]), 0.5, 0.3)
            if m.get("v_mix"):
                W[q + "vmix"] = torch.tensor(0.15 + 0.7 * torch.rand((), generator=g).item()).to(torch.bfloat16)
            W[q + "o"] = rn((width, H * Dv), (H * Dv) ** -0.5)
        else:
            H, D, R, Dv, qr, kr = (m[k] for k in ("heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank"))
            W[q + "dq"] = rn((qr, width), width ** -0.5)
            W[q + "dq.norm"] = rn(qr, 0.3, 1.0)
            W[q + "uq"] = rn((H * (D + R), qr), qr ** -0.5)
            W[q + "dkv"] = rn((kr + R, width), width ** -0.5)
            W[q + "dkv.norm"] = rn(kr, 0.3, 1.0)
            W[q + "uk"] = rn((H * D, kr), kr ** -0.5)
            W[q + "uv"] = rn((H * Dv, kr), kr ** -0.5)
            W[q + "sink"] = rn(H, 1.5, 1.0)
            W[q + "o"] = rn((width, H * Dv), (H * Dv) ** -0.5)
        if L.get("mlp"):
            ff = L["mlp"]["ff"]
            W[p + "mlp.up"] = rn((ff, width), 1.5 * width ** -0.5)
            W[p + "mlp.down"] = rn((width, ff), ff ** -0.5)
        if side:
            W[p + "side.gate"] = rn((side, width), 1.5 * width ** -0.5)
            W[p + "side.proj"] = rn((width, side), side ** -0.5)
            W[p + "side.norm"] = rn(width, 0.3, 0.8)
    return W


def write_model(cfg: dict, W: dict, root=None) -> str:
    from cpi_b200.weights.safetensors_io import write_safetensors
    d = tempfile.mkdtemp(prefix="nogapel_tiny_", dir=root)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(d, "model.safetensors"), {k: v.contiguous() for k, v in W.items()})
    return d


def tokens(n: int, vocab: int, seed: int) -> list:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()
