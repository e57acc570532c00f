"""Nogapel as a `ModelSpec`: every layer norms the residual once and runs a mixer and a dense feed-forward (relu
squared, no gate) side by side on that (block `parallel_residual`); the mixer is sliding-window attention whose q, k
and v pass a short convolution over time (mixer `attention` with `conv`, a shared per-head norm weight, interleaved
rotation with the llama3 frequency rule, and values mixed with those of the first such layer), or attention over a
cached latent with a sink (mixer `latent_attention`); after the sublayers a layer takes its slice of a per-token side
vector through a gate (junction `token_gated_input`, named by the run entry's `after`); the embedding output is normed.

Tensor names: `embed`, `embed.norm`, `side.embed`, `final.norm`, `head`; layer i under `l<i>.`: `norm1`,
`mix.{q,k,v,o,q.norm,k.norm,q.conv,k.conv,v.conv,vmix}` or `mix.{dq,dq.norm,uq,dkv,dkv.norm,uk,uv,sink,o}`,
`mlp.{up,down}`, `side.{gate,proj,norm}`.
"""
from __future__ import annotations

from ..config.nogapel import NogapelConfig
from ..config.registry import Architecture, register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, RunEntry


def _position(rot, head_dim) -> PartSpec:
    if rot is None:
        return PartSpec("none", {})
    sc = rot["scaling"]
    scaling = None if sc is None else {
        "rope_type": "llama3", "factor": sc["factor"], "low_freq_factor": sc["low"], "high_freq_factor": sc["high"],
        "original_max_position_embeddings": sc["original"]}
    return PartSpec("rope", {"head_dim": head_dim, "theta": rot["base"], "pairing": "interleaved",
                             "rotary_dims": rot["dims"], "scaling": scaling, "frequency_math": "float64"})


def _mixer_spec(cfg: NogapelConfig, layer, first_mixing: bool) -> PartSpec:
    m, W = layer.mixer, cfg.width
    if layer.type == "attention":
        window = {"kind": "full", "size": 0} if m["mask"] is None else {"kind": "sliding", "size": m["mask"]["size"]}
        return PartSpec("attention", {
            "hidden_size": W, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
            "value_dim": m["vdim"], "softmax_scale": m["scale"], "position": _position(m["rot"], m["dim"]),
            "qk_norm": True, "qk_norm_scope": "head", "qk_norm_order": "before_rope", "qk_norm_weight": "shared",
            "qk_norm_eps": cfg.eps, "window": window, "query_temperature": None, "conv": m["conv"],
            "value_mix": None if not m["v_mix"] else {"role": "first" if first_mixing else "later", "channel": "v_first"},
            "tensor_names": {"q": "mix.q", "k": "mix.k", "v": "mix.v", "o": "mix.o", "q_norm": "mix.q.norm",
                             "k_norm": "mix.k.norm", "q_conv": "mix.q.conv", "k_conv": "mix.k.conv",
                             "v_conv": "mix.v.conv", "v_mix": "mix.vmix"}})
    return PartSpec("latent_attention", {
        "hidden_size": W, "heads": m["heads"], "head_dim": m["dim"], "rot_dim": m["rot_dim"], "value_dim": m["vdim"],
        "q_rank": m["q_rank"], "kv_rank": m["kv_rank"], "softmax_scale": m["scale"], "norm_eps": cfg.eps,
        "position": _position(m["rot"], m["rot_dim"]), "sink": True,
        "tensor_names": {"dq": "mix.dq", "dq_norm": "mix.dq.norm", "uq": "mix.uq", "dkv": "mix.dkv",
                         "dkv_norm": "mix.dkv.norm", "uk": "mix.uk", "uv": "mix.uv", "o": "mix.o", "sink": "mix.sink"}})


def build_spec(cfg: NogapelConfig) -> ModelSpec:
    W, n = cfg.width, len(cfg.layers)
    norm = {"size": W, "eps": cfg.eps}
    layers, junctions, order = [], [], []
    seen_mixing = False
    for i, L in enumerate(cfg.layers):
        mixing = L.type == "attention" and L.mixer["v_mix"]
        layers.append(LayerSpec(
            prefix=f"l{i}.", block=PartSpec("parallel_residual", {}),
            mixer=_mixer_spec(cfg, L, mixing and not seen_mixing),
            feed_forward=None if L.ff is None else PartSpec("dense_mlp", {
                "hidden_size": W, "intermediate_size": L.ff, "activation": "relu_squared",
                "tensor_names": {"up": "mlp.up", "down": "mlp.down"}}),
            mixer_norm=PartSpec("rmsnorm", {**norm, "weight": "norm1"}),
            feed_forward_norm=None))
        seen_mixing = seen_mixing or mixing
        after = None
        if cfg.side_dim is not None:
            after = f"side{i}"
            junctions.append((after, PartSpec("token_gated_input", {
                "hidden_size": W, "vocab_size": cfg.vocab, "dim": cfg.side_dim, "table": "side.embed",
                "table_width": n * cfg.side_dim, "offset": i * cfg.side_dim, "gate": f"l{i}.side.gate",
                "proj": f"l{i}.side.proj", "norm": f"l{i}.side.norm", "eps": cfg.eps})))
        order.append(RunEntry(i, after=after))
    return ModelSpec(
        architecture=cfg.architecture, hidden_size=W, vocab_size=cfg.vocab,
        embedding=PartSpec("token_embedding", {"weight": "embed", "vocab_size": cfg.vocab, "hidden_size": W,
                                               "norm": PartSpec("rmsnorm", {**norm, "weight": "embed.norm"})}),
        layers=tuple(layers), run_order=tuple(order),
        final_norm=PartSpec("rmsnorm", {**norm, "weight": "final.norm"}),
        head=PartSpec("linear_head", {"weight": "head", "vocab_size": cfg.vocab, "hidden_size": W}),
        initializer_range=cfg.initializer_range, junctions=tuple(junctions),
        # a mixing weight that a folder stores for an attention layer without value mixing is not read
        ignored_tensor_prefixes=tuple(f"l{i}.mix.vmix" for i, L in enumerate(cfg.layers)
                                      if L.type == "attention" and not L.mixer["v_mix"]))


register_architecture(Architecture("Nogapel", NogapelConfig.from_json_dict, build_spec))
