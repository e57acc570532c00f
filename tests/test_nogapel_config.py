"""Nogapel without a GPU: config.json parsing, the spec that is built from it, the tensor list, the cache groups of
its two mixers, and the frequency rule."""
from __future__ import annotations

import copy

import pytest
import torch

import nogapel_tiny as V
import plain_nogapel as P
from cpi_b200.config.common import ConfigError
from cpi_b200.config.nogapel import NogapelConfig
from cpi_b200.config.registry import architecture_of
from cpi_b200.engine.model import tensor_requirements
from cpi_b200.models.nogapel import build_spec


def test_the_family_is_registered_and_parses_every_key():
    assert architecture_of(V.MIXED_A).name == "Nogapel"
    cfg = NogapelConfig.from_json_dict(V.MIXED_A)
    assert (cfg.vocab, cfg.width, cfg.eps, cfg.side_dim, len(cfg.layers)) == (97, 52, 1e-5, 6, 6)
    l0, l1, l2 = cfg.layers[:3]
    assert l0.type == "latent_attention" and l0.ff == 44
    assert {k: l0.mixer[k] for k in ("heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank")} == {
        "heads": 3, "dim": 12, "rot_dim": 6, "vdim": 10, "q_rank": 14, "kv_rank": 18}
    assert l0.mixer["rot"] == {"base": 300.0, "dims": 6, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64.0}}
    assert l1.type == "attention" and l1.mixer["mask"] == {"size": 11} and l1.mixer["conv"] == 3 and l1.mixer["v_mix"]
    assert l2.ff is None and not l2.mixer["v_mix"] and l2.mixer["rot"]["scaling"] is None
    c = NogapelConfig.from_json_dict(V.MIXED_C)
    assert c.side_dim is None and c.layers[1].mixer["mask"] is None and c.layers[3].mixer["conv"] is None
    assert c.layers[0].mixer["rot"] is None


@pytest.mark.parametrize("change,word", [
    (lambda c: c["layers"][0].update(type="mamba"), "type"),
    (lambda c: c["layers"][0].pop("mixer"), "mixer"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=14), "dims"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=5), "dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=4), "rot_dim"),
    (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][1]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][3]["mixer"].update(vdim=12), "v_mix"),
    (lambda c: c["layers"][1]["mlp"].update(kind="moe"), "kind"),
    (lambda c: c["layers"][1]["mixer"]["rot"]["scaling"].pop("low"), "low"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c.pop("vocab"), "vocab"),
    (lambda c: c.update(layers=[]), "layers"),
])
def test_bad_configurations_are_refused_by_name(change, word):
    c = copy.deepcopy(V.MIXED_A)
    change(c)
    with pytest.raises(ConfigError) as e:
        NogapelConfig.from_json_dict(c)
    assert word in str(e.value)


def test_the_spec_names_parts_and_the_first_mixing_layer():
    spec = build_spec(NogapelConfig.from_json_dict(V.MIXED_A))
    spec.validate()
    assert [(e.layer, e.before, e.after) for e in spec.run_order] == [(i, None, f"side{i}") for i in range(6)]
    assert all(L.block.kind == "parallel_residual" and L.feed_forward_norm is None for L in spec.layers)
    kinds = [L.mixer.kind for L in spec.layers]
    assert kinds == ["latent_attention", "attention", "attention", "attention", "latent_attention", "attention"]
    roles = [None if L.mixer.kind != "attention" or L.mixer["value_mix"] is None else L.mixer["value_mix"]["role"]
             for L in spec.layers]
    assert roles == [None, "first", None, "later", None, "later"]
    a = spec.layers[1].mixer
    assert a["window"] == {"kind": "sliding", "size": 11} and a["conv"] == 3 and a["qk_norm_weight"] == "shared"
    assert a["position"]["pairing"] == "interleaved" and a["position"]["rotary_dims"] == 8
    assert a["position"]["scaling"]["rope_type"] == "llama3"
    assert spec.layers[2].feed_forward is None and spec.layers[0].feed_forward.kind == "dense_mlp"
    assert spec.layers[0].feed_forward["activation"] == "relu_squared"
    j = dict(spec.junctions)
    assert j["side3"].kind == "token_gated_input" and j["side3"]["offset"] == 18 and j["side3"]["table_width"] == 36
    assert spec.embedding["norm"].kind == "rmsnorm"
    c = build_spec(NogapelConfig.from_json_dict(V.MIXED_C))
    assert c.junctions == () and all(e.after is None for e in c.run_order)
    assert c.layers[1].mixer["window"]["kind"] == "full" and c.layers[0].mixer["position"].kind == "none"


@pytest.mark.parametrize("cfg", [V.MIXED_A, V.MIXED_B, V.MIXED_C] + [V.draw_config(s) for s in range(1, 9)])
def test_tensor_list_is_the_folder_s(cfg):
    W = V.draw_weights(cfg, 1)
    spec = build_spec(NogapelConfig.from_json_dict(cfg))
    reqs = {r.name: tuple(r.shape) for r in tensor_requirements(spec)}
    assert reqs == {n: tuple(t.shape) for n, t in W.items()}


def test_cache_groups_a_latent_stream_and_windowed_keys_and_values():
    from cpi_b200.engine.model import DecoderModel
    spec = build_spec(NogapelConfig.from_json_dict(V.MIXED_A))
    reqs, states = DecoderModel(spec, torch.float32, "cpu").cache_requirements()
    lat, att = reqs[0], reqs[1]
    assert lat.window_kind == "full" and lat.streams == (("latent", 1, 24),)
    assert att.window_kind == "sliding" and att.window_size == 11 and dict((s[0], s[1:]) for s in att.streams) == {
        "k": (2, 12), "v": (2, 10)}
    assert [s.name for s in states[1]] == ["conv"] and tuple(states[1][0].shape) == (2, 4 * 12 + 2 * 12 + 2 * 10)
    assert states.get(0, []) == []


def test_plain_pieces_agree_with_each_other():
    """The plain implementation's own pieces: a window as large as the sequence is no window; a sink of minus
    infinity is no sink; one tap with weight one is the identity."""
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(9, 2, 6, generator=g, dtype=torch.float64) for _ in range(3))
    a = P.masked_softmax_attention(q, k, v, 0.5, None, None)
    assert torch.allclose(a, P.masked_softmax_attention(q, k, v, 0.5, 9, None))
    assert torch.allclose(a, P.masked_softmax_attention(q, k, v, 0.5, None, torch.full((2,), -1e30, dtype=torch.float64)))
    assert not torch.allclose(a, P.masked_softmax_attention(q, k, v, 0.5, 8, None))
    u = torch.randn(5, 3, generator=g, dtype=torch.float64)
    assert torch.equal(P.short_conv(u, torch.ones(3, 1, dtype=torch.float64)), u)
    w = torch.zeros(3, 2, dtype=torch.float64)
    w[:, 0] = 1.0
    assert torch.equal(P.short_conv(u, w)[1:], u[:-1]) and P.short_conv(u, w)[0].abs().max() == 0
