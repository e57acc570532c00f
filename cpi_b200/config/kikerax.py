"""Typed configuration of the Kikerax decoder, read from config.json keys.

A Kikerax layer adds to the residual the RMS norm of its mixer's output and then the RMS norm of its feed-forward's
output; both sublayers read the residual itself.  The mixer is differential attention (two softmax maps per head over
the same values, biases, a shared per-head norm weight, a rotation of part of each head with the YaRN frequency rule,
a chunked mask, a gate per head), or a pair side by side: softmax attention whose values are its projected keys
(query temperature, soft-capped scores, a gate per head) and a recurrent block around a real-gated linear recurrent
unit.  The feed-forward is dense (gelu) or routed experts chosen from the best groups, with a shared expert.  Every
size and every constant that can differ between models is a key of config.json:

    architecture  "Kikerax"          vocab, width          norm {eps}          logit_softcap | absent
    layers        [{type: "attention" | "parallel", mixer {...}, mlp {...} | null}, ...]

attention:  heads, kv_heads, dim, vdim, scale, diff, mask {size} | absent,
            rot {base, dims, scaling {factor, original, fast, slow} | absent} | absent
parallel:   left {heads, kv_heads, dim, vdim (= dim), scale, softcap | absent, q_temp {coef, every} | absent},
            right {width, blocks, conv}, left_scale, right_scale
mlp:        {kind: "dense", ff}  |  {kind: "moe", expert {ff}, router {experts, top, scale | absent,
            groups {count, keep} | absent}, shared {ff} | absent}
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from .common import ConfigError
from .veredra import _need, _pos_int

MIXER_TYPES = ("attention", "parallel")


@dataclass(frozen=True)
class KikeraxLayer:
    type: str
    mixer: dict                    # the validated keys of the mixer, defaults filled in
    mlp: Optional[dict]            # the validated keys of the feed-forward, None: the layer has none


@dataclass(frozen=True)
class KikeraxConfig:
    architecture: str
    vocab: int
    width: int
    layers: tuple
    eps: float
    logit_softcap: Optional[float]
    initializer_range: float

    @staticmethod
    def from_json_dict(raw: dict) -> "KikeraxConfig":
        vocab, width = _pos_int(raw, "vocab", "the model"), _pos_int(raw, "width", "the model")
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, L in enumerate(layers_raw):
            where = f"layers[{i}]"
            if not isinstance(L, dict) or L.get("type") not in MIXER_TYPES:
                raise ConfigError(f"config.json: {where}.type must be one of {', '.join(MIXER_TYPES)}")
            m = L.get("mixer")
            if not isinstance(m, dict):
                raise ConfigError(f"config.json: {where}.mixer must be an object with the mixer's sizes")
            mixer = _differential(m, where + ".mixer") if L["type"] == "attention" else _parallel(m, where + ".mixer")
            layers.append(KikeraxLayer(L["type"], mixer, _mlp(L.get("mlp"), where + ".mlp")))
        norm = raw.get("norm")
        if not isinstance(norm, dict):
            raise ConfigError("config.json: 'norm' must be an object with 'eps'")
        cap = raw.get("logit_softcap")
        if cap is not None and not float(_need(raw, "logit_softcap", "the model")) > 0:
            raise ConfigError("config.json: logit_softcap must be positive")
        return KikeraxConfig(
            architecture=str(raw.get("architecture") or (raw.get("architectures") or ["Kikerax"])[0]),
            vocab=vocab, width=width, layers=tuple(layers), eps=float(_need(norm, "eps", "norm")),
            logit_softcap=None if cap is None else float(cap),
            initializer_range=float(raw.get("initializer_range", 0.02)))


def _heads(m: dict, where: str) -> dict:
    out = {"heads": _pos_int(m, "heads", where)}
    out["kv_heads"] = _pos_int(m, "kv_heads", where, default=out["heads"])
    if out["heads"] % out["kv_heads"]:
        raise ConfigError(f"config.json: {where}: {out['heads']} heads over {out['kv_heads']} kv_heads")
    out["dim"] = _pos_int(m, "dim", where)
    out["vdim"] = _pos_int(m, "vdim", where, default=out["dim"])
    out["scale"] = float(_need(m, "scale", where))
    return out


def _rot(m: dict, where: str, limit: int) -> Optional[dict]:
    r = m.get("rot")
    if not r:
        return None
    if not isinstance(r, dict):
        raise ConfigError(f"config.json: {where}.rot must be an object")
    dims = _pos_int(r, "dims", where + ".rot")
    if dims % 2 or dims > limit:
        raise ConfigError(f"config.json: {where}.rot.dims = {dims} must be even and at most {limit}")
    out = {"base": float(_need(r, "base", where + ".rot")), "dims": dims, "scaling": None}
    if not out["base"] > 1:
        raise ConfigError(f"config.json: {where}.rot.base must be larger than 1")
    sc = r.get("scaling")
    if sc:
        w = where + ".rot.scaling"
        out["scaling"] = {k: float(_need(sc, k, w)) for k in ("factor", "original", "fast", "slow")}
        if any(not v > 0 for v in out["scaling"].values()):
            raise ConfigError(f"config.json: {w}: factor, original, fast and slow must be positive")
    return out


def _differential(m: dict, where: str) -> dict:
    out = _heads(m, where)
    out["diff"] = float(_need(m, "diff", where))
    out["rot"] = _rot(m, where, out["dim"])
    out["mask"] = None
    if m.get("mask"):
        out["mask"] = {"size": _pos_int(m["mask"], "size", where + ".mask")}
    return out


def _parallel(m: dict, where: str) -> dict:
    l, r = m.get("left"), m.get("right")
    if not isinstance(l, dict) or not isinstance(r, dict):
        raise ConfigError(f"config.json: {where} needs the objects 'left' and 'right'")
    left = _heads(l, where + ".left")
    if left["vdim"] != left["dim"]:
        raise ConfigError(f"config.json: {where}.left: the values are the keys, so vdim = {left['vdim']} must equal "
                          f"dim = {left['dim']}")
    cap = l.get("softcap")
    left["softcap"] = None if cap is None else float(_need(l, "softcap", where + ".left"))
    if left["softcap"] is not None and not left["softcap"] > 0:
        raise ConfigError(f"config.json: {where}.left.softcap must be positive")
    left["q_temp"] = None
    if l.get("q_temp"):
        qt = l["q_temp"]
        left["q_temp"] = {"coef": float(_need(qt, "coef", where + ".left.q_temp")),
                          "every": float(_need(qt, "every", where + ".left.q_temp"))}
        if not left["q_temp"]["every"] > 0:
            raise ConfigError(f"config.json: {where}.left.q_temp.every must be positive")
    right = {"width": _pos_int(r, "width", where + ".right"), "blocks": _pos_int(r, "blocks", where + ".right", default=1),
             "conv": _pos_int(r, "conv", where + ".right", default=1)}
    if right["width"] % right["blocks"]:
        raise ConfigError(f"config.json: {where}.right: {right['width']} channels in {right['blocks']} blocks")
    return {"left": left, "right": right,
            "left_scale": float(m["left_scale"]) if m.get("left_scale") is not None else 1.0,
            "right_scale": float(m["right_scale"]) if m.get("right_scale") is not None else 1.0}


def _mlp(m, where: str) -> Optional[dict]:
    if m is None:
        return None
    if not isinstance(m, dict) or m.get("kind") not in ("dense", "moe"):
        raise ConfigError(f"config.json: {where}.kind must be 'dense' or 'moe' (or mlp null)")
    if m["kind"] == "dense":
        return {"kind": "dense", "ff": _pos_int(m, "ff", where)}
    e, r = m.get("expert"), m.get("router")
    if not isinstance(e, dict) or not isinstance(r, dict):
        raise ConfigError(f"config.json: {where} needs the objects 'expert' and 'router'")
    out = {"kind": "moe", "ff": _pos_int(e, "ff", where + ".expert"),
           "experts": _pos_int(r, "experts", where + ".router"), "top": _pos_int(r, "top", where + ".router"),
           "scale": float(r["scale"]) if r.get("scale") is not None else 1.0, "groups": 1, "keep": 1,
           "shared_ff": None}
    g = r.get("groups")
    if g:
        out["groups"] = _pos_int(g, "count", where + ".router.groups")
        out["keep"] = _pos_int(g, "keep", where + ".router.groups", default=out["groups"])
    if out["experts"] % out["groups"] or out["keep"] > out["groups"]:
        raise ConfigError(f"config.json: {where}.router: {out['experts']} experts in {out['groups']} groups of which "
                          f"{out['keep']} are kept")
    if out["top"] > out["keep"] * (out["experts"] // out["groups"]):
        raise ConfigError(f"config.json: {where}.router.top = {out['top']} exceeds the experts of the kept groups")
    if m.get("shared"):
        out["shared_ff"] = _pos_int(m["shared"], "ff", where + ".shared")
    return out
