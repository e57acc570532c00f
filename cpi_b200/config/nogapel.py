"""Typed configuration of the Nogapel decoder, read from config.json keys.

A Nogapel layer norms the residual once and feeds that to a mixer and a feed-forward side by side; both outputs are
added to the residual.  The mixer is softmax attention with a sliding window (q, k and v pass a short per-channel
convolution over time; q and k heads a weighted RMS norm and a rotation of their first elements; values may be mixed
with those of the first such layer), or attention over a cached latent (queries through a low rank, one normed latent
and one rotated key part per position, a learned sink in the softmax).  After the two sublayers every layer may take
a small vector looked up by token id, gated by a projection of the residual.  Every size and every constant that can
differ between models is a key of config.json:

    architecture  "Nogapel"          vocab, width          norm {eps}          token_side {dim} | absent
    layers        [{type: "attention" | "latent_attention", mixer {...}, mlp {kind: "dense", ff} | null}, ...]

attention:         heads, kv_heads, dim, vdim, scale, conv (taps) | absent, v_mix (bool) | absent,
                   rot {base, dims, scaling {factor, low, high, original} | absent} | absent, mask {size} | absent
latent_attention:  heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, rot {base, dims (= rot_dim), scaling | absent}
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from .common import ConfigError
from .veredra import _need, _pos_int

MIXER_TYPES = ("attention", "latent_attention")


@dataclass(frozen=True)
class NogapelLayer:
    type: str
    mixer: dict                    # the validated keys of the mixer, defaults filled in
    ff: Optional[int]              # hidden size of the dense feed-forward, None: the layer has none


@dataclass(frozen=True)
class NogapelConfig:
    architecture: str
    vocab: int
    width: int
    layers: tuple
    eps: float
    side_dim: Optional[int]        # elements of the per-layer token vector, None: the model has none
    initializer_range: float

    @staticmethod
    def from_json_dict(raw: dict) -> "NogapelConfig":
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
            mixer = _attention(m, where + ".mixer") if L["type"] == "attention" else _latent(m, where + ".mixer")
            layers.append(NogapelLayer(L["type"], mixer, _mlp(L.get("mlp"), where + ".mlp")))
        mixing = [L.mixer for L in layers if L.type == "attention" and L.mixer["v_mix"]]
        for m in mixing[1:]:
            if (m["kv_heads"], m["vdim"]) != (mixing[0]["kv_heads"], mixing[0]["vdim"]):
                raise ConfigError("config.json: layers with v_mix share the first such layer's values, so their "
                                  "kv_heads and vdim must be equal")
        norm = raw.get("norm")
        if not isinstance(norm, dict):
            raise ConfigError("config.json: 'norm' must be an object with 'eps'")
        side = raw.get("token_side")
        if side is not None and not isinstance(side, dict):
            raise ConfigError("config.json: 'token_side' must be an object with 'dim'")
        return NogapelConfig(
            architecture=str(raw.get("architecture") or (raw.get("architectures") or ["Nogapel"])[0]),
            vocab=vocab, width=width, layers=tuple(layers), eps=float(_need(norm, "eps", "norm")),
            side_dim=None if not side else _pos_int(side, "dim", "token_side"),
            initializer_range=float(raw.get("initializer_range", 0.02)))


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
    sc = r.get("scaling")
    if sc:
        w = where + ".rot.scaling"
        out["scaling"] = {k: float(_need(sc, k, w)) for k in ("factor", "low", "high", "original")}
        if not out["scaling"]["factor"] > 0 or out["scaling"]["high"] == out["scaling"]["low"]:
            raise ConfigError(f"config.json: {w} needs a positive factor and low != high")
    return out


def _attention(m: dict, where: str) -> dict:
    out = {"heads": _pos_int(m, "heads", where)}
    out["kv_heads"] = _pos_int(m, "kv_heads", where, default=out["heads"])
    if out["heads"] % out["kv_heads"]:
        raise ConfigError(f"config.json: {where}: {out['heads']} heads over {out['kv_heads']} kv_heads")
    out["dim"] = _pos_int(m, "dim", where)
    out["vdim"] = _pos_int(m, "vdim", where, default=out["dim"])
    out["scale"] = float(_need(m, "scale", where))
    out["conv"] = None if m.get("conv") is None else _pos_int(m, "conv", where)
    out["v_mix"] = bool(m.get("v_mix", False))
    out["rot"] = _rot(m, where, out["dim"])
    out["mask"] = None
    if m.get("mask"):
        out["mask"] = {"size": _pos_int(m["mask"], "size", where + ".mask")}
    return out


def _latent(m: dict, where: str) -> dict:
    out = {k: _pos_int(m, k, where) for k in ("heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank")}
    out["scale"] = float(_need(m, "scale", where))
    if out["rot_dim"] % 2:
        raise ConfigError(f"config.json: {where}.rot_dim = {out['rot_dim']} must be even")
    out["rot"] = _rot(m, where, out["rot_dim"])
    if out["rot"] is not None and out["rot"]["dims"] != out["rot_dim"]:
        raise ConfigError(f"config.json: {where}.rot.dims = {out['rot']['dims']} must equal rot_dim = {out['rot_dim']}")
    return out


def _mlp(m, where: str) -> Optional[int]:
    if m is None:
        return None
    if not isinstance(m, dict) or m.get("kind") != "dense":
        raise ConfigError(f"config.json: {where}.kind must be 'dense' (or mlp null)")
    return _pos_int(m, "ff", where)
