"""Small Kikerax configurations and weights for the tests.

The weights are drawn here, not by the library's random mode, with spreads chosen so that faults show: attention scores
a few units wide (a single key can carry a row), norm weights away from one, biases that matter, lambdas away from
zero, gates on both sides of a half, decays spread between fast and slow, router rows that separate the experts and
corrections of both signs that change the choice.
"""
from __future__ import annotations

import json
import os
import tempfile

import torch


def differential(heads, kv_heads, dim, vdim, diff=0.4, chunk=None, rot_dims=None, base=10000.0, scaling=None, scale=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "diff": diff,
         "scale": (3.0 / dim ** 0.5) if scale is None else scale}
    if chunk is not None:
        m["mask"] = {"size": chunk}
    if rot_dims is not None:
        m["rot"] = {"base": base, "dims": rot_dims}
        if scaling is not None:
            m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return m


def pair(heads, kv_heads, dim, width, blocks, conv, softcap=None, q_temp=None, scales=(0.7, 1.2), scale=None):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": (3.0 / dim ** 0.5) if scale is None else scale}
    if softcap is not None:
        left["softcap"] = softcap
    if q_temp is not None:
        left["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    return {"left": left, "right": {"width": width, "blocks": blocks, "conv": conv},
            "left_scale": scales[0], "right_scale": scales[1]}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, groups=None, shared=None, scale=1.5):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "scale": scale}}
    if groups is not None:
        m["router"]["groups"] = {"count": groups[0], "keep": groups[1]}
    if shared is not None:
        m["shared"] = {"ff": shared}
    return m


def layer(mixer, mlp):
    return {"type": "parallel" if "left" in mixer else "attention", "mixer": mixer, "mlp": mlp}


def model(layers, width, vocab, eps=1e-5, logit_softcap=None):
    cfg = {"architecture": "Kikerax", "layers": layers, "norm": {"eps": eps}, "vocab": vocab, "width": width}
    if logit_softcap is not None:
        cfg["logit_softcap"] = logit_softcap
    return cfg


# A: sizes that are no multiples of 8 (the float32-pipe products in both precisions); the pair first; grouped keys with
# three query heads per key head, values larger and smaller than keys, a rotation of part of a head under the scaled
# frequency rule (kept, stretched and blended pairs all occur), short chunks that end inside a page, a temperature that
# changes every three positions, a tight soft cap, three blocks, groups of experts of which two are kept, a layer
# without a feed-forward.
MIXED_A = model([
    layer(pair(4, 1, 12, 36, 3, 3, softcap=4.0, q_temp=(0.5, 3), scales=(0.6, 1.3)), moe(6, 2, 20, groups=(3, 2), shared=28)),
    layer(differential(6, 2, 10, 14, diff=0.35, chunk=11, rot_dims=6, base=300.0, scaling=(4.0, 64, 8.0, 1.0)), dense(44)),
    layer(pair(2, 2, 20, 30, 5, 2, softcap=9.0, scales=(1.1, 0.5)), None),
    layer(differential(2, 1, 12, 6, diff=0.6, chunk=30, rot_dims=12, base=50.0, scaling=(8.0, 32, 4.0, 0.5)), moe(4, 1, 36, shared=12, scale=0.8)),
], width=52, vocab=97, logit_softcap=6.0)

# B: multiples of 8 and 16, so that the bfloat16 path runs the tensor-core products and, where keys and values have one
# size of 64 and nothing acts on a score, the tensor-core attention kernels: both maps of a layer with a chunk that
# spans pages, and a pair's left side without a soft cap; sixteen experts in four groups; other eps.
MIXED_B = model([
    layer(differential(4, 2, 64, 64, diff=0.5, chunk=100, rot_dims=32, base=2.5e5, scaling=(2.0, 128, 16.0, 2.0)), dense(256)),
    layer(pair(4, 2, 64, 256, 2, 4, q_temp=(0.3, 16), scales=(0.8, 0.9)), moe(16, 4, 64, groups=(4, 2), shared=96, scale=2.5)),
    layer(differential(2, 2, 32, 64, diff=0.3, chunk=37, rot_dims=8), moe(8, 3, 32, groups=(2, 1))),
    layer(pair(8, 2, 16, 128, 8, 3, softcap=20.0, q_temp=(0.2, 40)), dense(192)),
], width=128, vocab=384, eps=1e-6, logit_softcap=12.0)

# C: what the other two make different or present: as many key heads as query heads, one head, one block, one tap, one
# expert a token, no groups, no shared expert, no soft cap, no temperature, no chunks, no rotation, a rotation of the
# whole head without scaling, a chunk of one position, scales of one, no cap on the logits, a layer without a
# feed-forward.
MIXED_C = model([
    layer(differential(1, 1, 8, 8, diff=0.2), dense(24)),
    layer(pair(1, 1, 8, 16, 1, 1, scales=(1.0, 1.0)), moe(3, 1, 16)),
    layer(differential(2, 2, 4, 20, diff=0.7, chunk=1, rot_dims=4, base=20.0), None),
    layer(differential(3, 3, 16, 16, diff=0.5, chunk=5, rot_dims=2), moe(5, 5, 8, shared=8)),
    layer(pair(3, 3, 4, 24, 2, 8), dense(40)),
], width=40, vocab=64)


def draw_config(seed: int) -> dict:
    """A configuration whose every size, option and constant is drawn from the seed."""
    import random
    rng = random.Random(seed)
    layers = []
    for _ in range(rng.randint(1, 5)):
        G = rng.choice([1, 2, 3])
        if rng.random() < 0.5:
            D = rng.choice([4, 8, 16, 32, 64, 128])
            rot = rng.choice([None, D, max(2, D // 4 * 2)])
            sc = rng.choice([None, (rng.choice([2.0, 8.0]), rng.choice([16, 256]), rng.choice([8.0, 32.0]), rng.choice([0.5, 1.0]))])
            m = differential(G * rng.choice([1, 2, 4]), G, D, rng.choice([D, D, 8, 24, 2 * D]), diff=rng.choice([0.2, 0.5, 0.8]),
                             chunk=rng.choice([None, 1, 7, 30, 64, 100]), rot_dims=rot, base=rng.choice([100.0, 1e4, 1e6]),
                             scaling=sc if rot else None)
        else:
            blocks = rng.choice([1, 2, 4, 6])
            m = pair(G * rng.choice([1, 2, 4]), G, rng.choice([4, 8, 20, 64, 128]), blocks * rng.choice([4, 8, 16, 40]),
                     blocks, rng.choice([1, 2, 4, 7]), softcap=rng.choice([None, 5.0, 30.0]),
                     q_temp=rng.choice([None, (0.4, 2), (0.1, 64)]), scales=(rng.choice([0.5, 1.0]), rng.choice([0.9, 1.4])))
        kind = rng.random()
        if kind < 0.2:
            mlp = None
        elif kind < 0.55:
            mlp = dense(rng.choice([24, 64, 256]))
        else:
            groups = rng.choice([None, (1, 1), (2, 1), (2, 2), (4, 2)])
            per = rng.choice([1, 2, 4])
            E = (groups[0] if groups else rng.choice([1, 3])) * per
            room = (groups[1] if groups else 1) * per if groups else E
            mlp = moe(E, rng.randint(1, room), rng.choice([8, 32, 64]), groups=groups, shared=rng.choice([None, 16, 48]),
                      scale=rng.choice([1.0, 2.5]))
        layers.append(layer(m, mlp))
    return model(layers, width=rng.choice([24, 40, 64, 128, 264]), vocab=rng.choice([50, 131, 449]),
                 eps=rng.choice([1e-5, 1e-6]), logit_softcap=rng.choice([None, 8.0, 30.0]))


def draw_weights(cfg: dict, seed: int) -> dict:
    """{name: bfloat16 tensor} for a configuration."""
    g = torch.Generator().manual_seed(seed)
    W = {}

    def rn(shape, std, mean=0.0):
        if isinstance(shape, int):
            shape = (shape,)
        return (torch.randn(*shape, generator=g) * std + mean).to(torch.bfloat16)

    width, vocab = cfg["width"], cfg["vocab"]
    W["embed"] = rn((vocab, width), 1.0)
    W["final.norm"] = rn(width, 0.15, 1.0)
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        W[p + "norm1"] = rn(width, 0.15, 0.7)
        q = p + "mix."
        if L["type"] == "attention":
            H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            W[q + "q"], W[q + "q.b"] = rn((2 * H * D, width), width ** -0.5), rn(2 * H * D, 0.3)
            W[q + "k"], W[q + "k.b"] = rn((2 * G * D, width), width ** -0.5), rn(2 * G * D, 0.3)
            W[q + "v"], W[q + "v.b"] = rn((G * Dv, width), width ** -0.5), rn(G * Dv, 0.3)
            W[q + "q.norm"], W[q + "k.norm"] = rn(D, 0.3, 1.0), rn(D, 0.3, 1.0)
            for n in ("lq1", "lk1", "lq2", "lk2"):
                W[q + n] = rn(D, 0.6 * D ** -0.5)
            W[q + "g"] = rn((H, width), 1.5 * width ** -0.5)
            W[q + "o"], W[q + "o.b"] = rn((width, H * Dv), (H * Dv) ** -0.5), rn(width, 0.3)
        else:
            l, r = m["left"], m["right"]
            H, G, D = l["heads"], l["kv_heads"], l["dim"]
            a = q + "left."
            W[a + "q"], W[a + "k"] = rn((H * D, width), width ** -0.5), rn((G * D, width), width ** -0.5)
            W[a + "q.norm"], W[a + "k.norm"] = rn(D, 0.3, 1.0), rn(D, 0.3, 1.0)
            W[a + "g"] = rn((H, width), 1.5 * width ** -0.5)
            W[a + "o"] = rn((width, H * D), (H * D) ** -0.5)
            b, C, B = q + "right.", r["width"], r["blocks"]
            n = C // B
            W[b + "y"], W[b + "y.b"] = rn((C, width), width ** -0.5), rn(C, 0.3)
            W[b + "x"], W[b + "x.b"] = rn((C, width), width ** -0.5), rn(C, 0.3)
            W[b + "conv"], W[b + "conv.b"] = rn((C, r["conv"]), 0.5, 0.3), rn(C, 0.2)
            W[b + "ra"], W[b + "ra.b"] = rn((B, n, n), 1.5 * n ** -0.5), rn((B, n), 0.5)
            W[b + "ri"], W[b + "ri.b"] = rn((B, n, n), 1.5 * n ** -0.5), rn((B, n), 0.5)
            W[b + "lam"] = rn(C, 1.5, -2.0)               # softplus of these: decays from a token to hundreds
            W[b + "o"] = rn((width, C), C ** -0.5)
        mlp = L.get("mlp")
        if mlp:
            W[p + "norm2"] = rn(width, 0.15, 0.7)
            f = p + "mlp."
            if mlp["kind"] == "dense":
                W[f + "up"], W[f + "down"] = rn((mlp["ff"], width), 1.5 * width ** -0.5), rn((width, mlp["ff"]), mlp["ff"] ** -0.5)
            else:
                E, ff = mlp["router"]["experts"], mlp["expert"]["ff"]
                W[f + "router"] = rn((E, width), 3.0 * width ** -0.5)
                W[f + "correction"] = rn(E, 0.3)
                names = [f"e{e}." for e in range(E)] + (["shared."] if mlp.get("shared") else [])
                for nm in names:
                    n_ff = mlp["shared"]["ff"] if nm == "shared." else ff
                    W[f + nm + "gate"] = rn((n_ff, width), 1.5 * width ** -0.5)
                    W[f + nm + "up"] = rn((n_ff, width), 1.5 * width ** -0.5)
                    W[f + nm + "down"] = rn((width, n_ff), n_ff ** -0.5)
    return W


def write_model(cfg: dict, W: dict, root=None) -> str:
    from cpi_b200.weights.safetensors_io import write_safetensors
    d = tempfile.mkdtemp(prefix="kikerax_tiny_", dir=root)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(d, "model.safetensors"), {k: v.contiguous() for k, v in W.items()})
    return d


def tokens(n: int, vocab: int, seed: int) -> list:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()
