"""Kikerax configuration and spec on the CPU: keys, defaults, errors that name the key, the tensor list, the plain
implementation's own consistency."""
from __future__ import annotations

import copy

import pytest
import torch

import kikerax_tiny as V
import plain_kikerax as P
from cpi_b200.config.common import ConfigError
from cpi_b200.config.kikerax import KikeraxConfig
from cpi_b200.config.registry import architecture_of
from cpi_b200.engine.model import tensor_requirements


@pytest.mark.parametrize("cfg", [V.MIXED_A, V.MIXED_B, V.MIXED_C] + [V.draw_config(s) for s in range(1, 13)])
def test_the_tensor_list_is_the_drawn_weights(cfg):
    arch = architecture_of(cfg)
    assert arch.name == "Kikerax"
    spec = arch.build_spec(arch.parse_config(cfg))
    spec.validate()
    need = {r.name: tuple(r.shape) for r in tensor_requirements(spec)}
    have = {k: tuple(v.shape) for k, v in V.draw_weights(cfg, 1).items()}
    assert need == have


def test_defaults_and_parts():
    cfg = KikeraxConfig.from_json_dict(V.MIXED_C)
    spec = architecture_of(V.MIXED_C).build_spec(cfg)
    assert cfg.logit_softcap is None and "logit_softcap" not in spec.head.params
    assert [l.block.kind for l in spec.layers] == ["post_norm"] * 5
    assert [l.mixer.kind for l in spec.layers] == ["attention", "parallel", "attention", "attention", "parallel"]
    first = spec.layers[0].mixer
    assert first["window"]["kind"] == "full" and first["position"].kind == "none" and first["differential"] == {"lambda_init": 0.2}
    left = spec.layers[1].mixer["branches"][0]["mixer"]
    assert left["value_source"] == "keys" and left["score_softcap"] is None and left["query_temperature"] is None
    assert spec.layers[1].mixer["combine"] == {"kind": "weighted_sum", "scales": [1.0, 1.0]}
    moe = spec.layers[1].feed_forward
    assert moe["router_rule"]["groups"] == 1 and moe["router_rule"]["keep"] == 1 and moe["shared"] is None
    assert spec.layers[2].feed_forward is None and spec.layers[2].feed_forward_norm is None
    a = architecture_of(V.MIXED_A).build_spec(KikeraxConfig.from_json_dict(V.MIXED_A))
    rope = a.layers[1].mixer["position"]
    assert rope["pairing"] == "interleaved" and rope["rotary_dims"] == 6 and rope["scaling"]["rope_type"] == "yarn"
    assert a.layers[1].mixer["window"] == {"kind": "chunk", "size": 11} and a.head["logit_softcap"] == 6.0
    assert a.layers[0].mixer["branches"][0]["mixer"]["query_temperature"] == {"floor_scale": 3.0, "attn_scale": 0.5}


@pytest.mark.parametrize("change,word", [
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["layers"][0].update(type="other"), "type"),
    (lambda c: c["layers"][1]["mixer"].pop("diff"), "diff"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=4), "kv_heads"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7), "dims"),
    (lambda c: c["layers"][1]["mixer"]["rot"]["scaling"].pop("fast"), "fast"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(vdim=10), "vdim"),
    (lambda c: c["layers"][0]["mixer"]["right"].update(blocks=5), "blocks"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(softcap=-1.0), "softcap"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=5), "top"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=4), "groups"),
    (lambda c: c["layers"][1]["mlp"].update(kind="sparse"), "kind"),
    (lambda c: c.update(logit_softcap=0.0), "logit_softcap"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_errors_name_the_key(change, word):
    cfg = copy.deepcopy(V.MIXED_A)
    change(cfg)
    with pytest.raises(ConfigError) as e:
        KikeraxConfig.from_json_dict(cfg)
    assert word in str(e.value)


def test_plain_implementation_is_causal_and_its_state_is_the_prefix():
    """The plain functions know no cache: a prefix's logits do not depend on what follows, and the recurrent block over
    a prefix is the block over the whole sequence cut off."""
    cfg = V.MIXED_A
    W = V.draw_weights(cfg, 3)
    toks = V.tokens(40, cfg["vocab"], 1)
    whole = P.forward(cfg, W, toks)
    assert (P.forward(cfg, W, toks[:23]) - whole[:23]).abs().max() < 1e-9
    z = torch.tensor([0.3, -1.0, 2.0, 0.1, 0.0, 1.0], dtype=torch.float64)
    corr = torch.tensor([0.0, 3.0, -3.0, 0.0, 0.0, 0.0], dtype=torch.float64)
    idx, w = P.router_choice(z, corr, {"experts": 6, "top": 2, "scale": 2.0, "groups": {"count": 3, "keep": 1}})
    assert sorted(idx.tolist()) == [0, 1] and abs(float(w.sum()) - 2.0) < 1e-9        # the correction picks, the score weighs
    s = torch.sigmoid(z)
    assert abs(float(w[idx.tolist().index(1)]) - 2.0 * float(s[1] / (s[0] + s[1]))) < 1e-9
