"""Kikerax as a `ModelSpec`: every layer is a `post_norm` block (the norms act on the sublayers' outputs, the sublayers
read the residual itself).  The mixer is `attention` with two score maps (`differential`), biases, a shared per-head
norm weight, an interleaved partial rotation under the yarn rule, a chunk window and an output gate; or `parallel` with
constant weights over an `attention` branch whose values are its projected keys (query temperature, soft-capped
scores, output gate) and an `rglru` branch.  The feed-forward is `dense_mlp` with gelu or `moe_swiglu` with the
grouped sigmoid choice and a shared expert.  The head is the embedding table, its logits soft-capped.

Tensor names: `embed`, `final.norm`; layer i under `l<i>.`: `norm1`, `norm2`,
`mix.{q,k,v,o}` with `.b` each, `mix.{q.norm,k.norm,lq1,lk1,lq2,lk2,g}`, or
`mix.left.{q,k,q.norm,k.norm,g,o}` and `mix.right.{y,y.b,x,x.b,conv,conv.b,ra,ra.b,ri,ri.b,lam,o}`;
`mlp.{up,down}` or `mlp.{router,correction,e<n>.{gate,up,down},shared.{gate,up,down}}`.
"""
from __future__ import annotations

from ..config.kikerax import KikeraxConfig
from ..config.registry import Architecture, register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, RunEntry


def _position(rot, head_dim) -> PartSpec:
    if rot is None:
        return PartSpec("none", {})
    sc = rot["scaling"]
    scaling = None if sc is None else {
        "rope_type": "yarn", "factor": sc["factor"], "original_max_position_embeddings": sc["original"],
        "beta_fast": sc["fast"], "beta_slow": sc["slow"]}
    return PartSpec("rope", {"head_dim": head_dim, "theta": rot["base"], "pairing": "interleaved",
                             "rotary_dims": rot["dims"], "scaling": scaling, "frequency_math": "float64"})


def _attention(cfg: KikeraxConfig, m: dict, names: str, **more) -> dict:
    return {"hidden_size": cfg.width, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
            "value_dim": m["vdim"], "softmax_scale": m["scale"], "qk_norm": True, "qk_norm_scope": "head",
            "qk_norm_order": "before_rope", "qk_norm_weight": "shared", "qk_norm_eps": cfg.eps, "output_gate": True,
            "tensor_names": {"q": names + "q", "k": names + "k", "v": names + "v", "o": names + "o",
                             "q_bias": names + "q.b", "k_bias": names + "k.b", "v_bias": names + "v.b",
                             "o_bias": names + "o.b", "q_norm": names + "q.norm", "k_norm": names + "k.norm",
                             "g": names + "g", "lq1": names + "lq1", "lk1": names + "lk1", "lq2": names + "lq2",
                             "lk2": names + "lk2"}, **more}


def _mixer_spec(cfg: KikeraxConfig, layer) -> PartSpec:
    m = layer.mixer
    if layer.type == "attention":
        window = {"kind": "full", "size": 0} if m["mask"] is None else {"kind": "chunk", "size": m["mask"]["size"]}
        return PartSpec("attention", _attention(
            cfg, m, "mix.", position=_position(m["rot"], m["dim"]), window=window, bias=True, output_bias=True,
            differential={"lambda_init": m["diff"]}, query_temperature=None))
    l, r = m["left"], m["right"]
    qt = l["q_temp"]
    left = PartSpec("attention", _attention(
        cfg, l, "mix.left.", position=PartSpec("none", {}), window={"kind": "full", "size": 0}, value_source="keys",
        score_softcap=l["softcap"],
        query_temperature=None if qt is None else {"floor_scale": qt["every"], "attn_scale": qt["coef"]}))
    n = "mix.right."
    right = PartSpec("rglru", {
        "hidden_size": cfg.width, "width": r["width"], "blocks": r["blocks"], "conv": r["conv"], "decay_scale": 8.0,
        "tensor_names": {"y": n + "y", "y_bias": n + "y.b", "x": n + "x", "x_bias": n + "x.b", "conv": n + "conv",
                         "conv_bias": n + "conv.b", "ra": n + "ra", "ra_bias": n + "ra.b", "ri": n + "ri",
                         "ri_bias": n + "ri.b", "lam": n + "lam", "o": n + "o"}})
    return PartSpec("parallel", {
        "hidden_size": cfg.width, "branches": [{"name": "left", "mixer": left}, {"name": "right", "mixer": right}],
        "combine": {"kind": "weighted_sum", "scales": [m["left_scale"], m["right_scale"]]}})


def _ff_spec(cfg: KikeraxConfig, mlp) -> PartSpec:
    W = cfg.width
    if mlp["kind"] == "dense":
        return PartSpec("dense_mlp", {"hidden_size": W, "intermediate_size": mlp["ff"], "activation": "gelu_tanh",
                                      "tensor_names": {"up": "mlp.up", "down": "mlp.down"}})
    shared = None
    if mlp["shared_ff"] is not None:
        shared = {"intermediate_size": mlp["shared_ff"],
                  "tensor_names": {"gate": "mlp.shared.gate", "up": "mlp.shared.up", "down": "mlp.shared.down"}}
    return PartSpec("moe_swiglu", {
        "hidden_size": W, "num_experts": mlp["experts"], "top_k": mlp["top"], "expert_size": mlp["ff"],
        "router_gate": "sigmoid_normed", "router_name": "mlp.router",
        "router_rule": {"choice_bias": "mlp.correction", "groups": mlp["groups"], "keep": mlp["keep"],
                        "scale": mlp["scale"]},
        "expert_layout": "per_expert",
        "expert_names": {"gate": "mlp.e{e}.gate", "up": "mlp.e{e}.up", "down": "mlp.e{e}.down"}, "shared": shared})


def build_spec(cfg: KikeraxConfig) -> ModelSpec:
    W = cfg.width
    norm = {"size": W, "eps": cfg.eps}
    layers = []
    for i, L in enumerate(cfg.layers):
        has_ff = L.mlp is not None
        layers.append(LayerSpec(
            prefix=f"l{i}.", block=PartSpec("post_norm", {}), mixer=_mixer_spec(cfg, L),
            feed_forward=_ff_spec(cfg, L.mlp) if has_ff else None,
            mixer_norm=PartSpec("rmsnorm", {**norm, "weight": "norm1"}),
            feed_forward_norm=PartSpec("rmsnorm", {**norm, "weight": "norm2"}) if has_ff else None))
    head = {"weight": "embed", "vocab_size": cfg.vocab, "hidden_size": W}
    if cfg.logit_softcap is not None:
        head["logit_softcap"] = cfg.logit_softcap
    return ModelSpec(
        architecture=cfg.architecture, hidden_size=W, vocab_size=cfg.vocab,
        embedding=PartSpec("token_embedding", {"weight": "embed", "vocab_size": cfg.vocab, "hidden_size": W}),
        layers=tuple(layers), run_order=tuple(RunEntry(i) for i in range(len(layers))),
        final_norm=PartSpec("rmsnorm", {**norm, "weight": "final.norm"}),
        head=PartSpec("linear_head", head), initializer_range=cfg.initializer_range)


register_architecture(Architecture("Kikerax", KikeraxConfig.from_json_dict, build_spec))
