"""Attention mixer: grouped-query attention over the paged cache, with a window and a position part.

Reference forward of one token (src/engine/llama4_cpu_engine.cpp:304-325): q, k, v projections
without bias, per-head weightless RMS norm of q and k, RoPE, cache write, causal softmax attention
with scale 1/sqrt(D), output projection added to the residual.  This part generalises it by
parameters: any head counts and head size, the position part (rotary or none), the norm on or off and
before or after the rotation, a window (all keys, the query's chunk, or the last n keys), and an
optional temperature on the query; and by batch: any mix of sequences and positions in one call.

params: hidden_size, num_heads, num_kv_heads, head_dim, softmax_scale, position (PartSpec), qk_norm,
qk_norm_eps, qk_norm_order ("before_rope" | "after_rope"), window {"kind", "size"},
query_temperature (None or {"floor_scale", "attn_scale"}).
Tensors under the prefix: self_attn.{q,k,v,o}_proj.weight  ([out, in]).

Further parameters, all off by default: value_dim (values of another size than keys), bias (q, k and v
projections have one), qk_norm_scope "projection" (one RMS norm over all heads of q, one over all of k, with
weights, before the rotation; "head" is the weightless per-head norm above), sink (a learned number per head whose
exponential joins the softmax denominator without a key or a value), a position part that rotates only the first
elements of a head, and tensor_names {"q", "k", "v", "o", "q_bias", "k_bias", "v_bias", "q_norm", "k_norm", "sink"}.
A mixer that uses one of them prepares q, k and v with the general kernel (`qkv_prepare`), from float32 projection
rows, so that a row is rounded once, after its norm and rotation.  There the weightless per-head norm comes after
the rotation (qk_norm_order "after_rope").  A sliding window may carry `keep_first`: the sequence's first positions
stay visible to every later query, at their own positions.

Also served by the general preparation: `conv` (taps: q, k and v each pass a causal convolution over time per channel,
directly after the projection, tensors "q_conv" / "k_conv" / "v_conv" [channels, taps]; the last taps - 1 projected
rows of a sequence are per-slot state), `qk_norm_weight` "shared" (the per-head norm comes before the rotation and
carries a weight [head_dim] that all heads share, tensors "q_norm" / "k_norm"), a rotation of interleaved pairs, and
`value_mix` {"role": "first" | "later", "channel": name} (tensor "v_mix", one number m): the layer with role "first"
leaves its values of the step's tokens in a buffer named by the channel, a "later" layer caches and attends to
(1 - m) v + m v_first of the same token.

Further, also through the general preparation: `value_source` "keys" (there is no value projection: the cached values
are the keys as projected, before their norm; keys and values then have one size); `score_softcap` c (a scaled score s
becomes c tanh(s / c)); the query temperature together with the per-head norm before the rotation; `output_gate`
(tensor "g" [heads, hidden]: head n's output is multiplied by sigmoid(g_n . h), h being the mixer's input);
`output_bias` (tensor "o_bias"); and `differential` {"lambda_init": c}: q and k hold two score maps per head (stored
head by head as [map 1, map 2]; the rows are reordered map by map at load), each map is a softmax attention of its own
over the same values, the second map's keys live in a cache stream "k2", and with one number per layer
lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + c (tensors "lq1", "lk1", "lq2", "lk2" [head_dim]) a head's output is
rmsnorm(a1 - lambda a2) (1 - c), the norm over the head's values without a weight (`qk_norm_eps`).  A rotation whose
encoding carries an amplitude multiplies its sines and cosines by it.

`attend(...)` below is the choice of the attention kernel for prepared queries and a paged cache; other mixers that
end in softmax attention over pages (`latent_attention`) call it too.
"""
from __future__ import annotations

import math

import torch

from ..cache.manager import KVRequirement, StateRequirement
from ..csrc import lib as K
from ..phases import phase
from ..weights.store import TensorReq
from .base import Mixer, RotaryEncoding, ScoreBias, build_part, register_mixer
from .linear import MODE_ADD, MODE_STORE, project


# set to False to run every attention through the general kernel (tests compare the two families)
use_tensor_core_kernels = True


@register_mixer("attention")
class AttentionMixer(Mixer):
    graph_safe = True
    def __init__(self, spec, prefix="", workspace=None, owns_cache=True):
        super().__init__(spec, prefix)
        p = spec.params
        self.has_kv = bool(owns_cache)      # False: every run entry of this layer reads another's cache
        self.hidden = int(p["hidden_size"])
        self.nh, self.nkv, self.d = int(p["num_heads"]), int(p["num_kv_heads"]), int(p["head_dim"])
        if self.nh % self.nkv:
            raise ValueError(f"attention: {self.nh} heads cannot be grouped over {self.nkv} key/value heads")
        self.dv = int(p.get("value_dim") or self.d)
        self.bias = bool(p.get("bias", False))
        self.norm_scope = p.get("qk_norm_scope", "head")
        if self.norm_scope not in ("head", "projection"):
            raise ValueError(f"attention: unknown qk_norm_scope '{self.norm_scope}'")
        self.has_sink = bool(p.get("sink", False))
        rot = p["position"].get("rotary_dims") if p["position"].kind == "rope" else None
        self.rot_dims = self.d if rot is None else int(rot)
        self.taps = None if p.get("conv") is None else int(p["conv"])
        if self.taps is not None and not 1 <= self.taps <= 8:
            raise ValueError(f"attention: a convolution of {self.taps} taps (supported: 1 to 8)")
        self.norm_weight_shared = p.get("qk_norm_weight") == "shared"
        if p.get("qk_norm_weight") not in (None, "shared"):
            raise ValueError(f"attention: unknown qk_norm_weight '{p.get('qk_norm_weight')}'")
        vm = p.get("value_mix")
        if vm is not None and vm.get("role") not in ("first", "later"):
            raise ValueError("attention: value_mix.role must be 'first' or 'later'")
        self.value_mix = None if vm is None else (vm["role"], str(vm.get("channel", "v_first")))
        self.values_from_keys = p.get("value_source", "projection") == "keys"
        if p.get("value_source", "projection") not in ("projection", "keys"):
            raise ValueError(f"attention: unknown value_source '{p.get('value_source')}'")
        if self.values_from_keys and self.dv != self.d:
            raise ValueError(f"attention: values that are the keys have the keys' size, not {self.dv} beside {self.d}")
        self.softcap = float(p.get("score_softcap") or 0.0)
        self.has_gate, self.has_o_bias = bool(p.get("output_gate", False)), bool(p.get("output_bias", False))
        df = p.get("differential")
        self.diff = None if df is None else float(df["lambda_init"])
        self.maps = 1 if self.diff is None else 2
        self.lam = 0.0
        extended = self.values_from_keys or self.has_gate or self.diff is not None
        if self.diff is not None and (self.values_from_keys or vm is not None or p.get("sink") or p.get("conv") is not None):
            raise ValueError("attention: two score maps do not combine with values from keys, value mixing, a sink or a convolution")
        self.general = (extended or self.bias or self.dv != self.d or self.rot_dims != self.d or self.d % 16 != 0
                        or (bool(p.get("qk_norm", False)) and self.norm_scope == "projection")
                        or self.taps is not None or self.norm_weight_shared or self.value_mix is not None)
        limit = K.GENERAL_ATTENTION_MAX_DIM if self.general else 256
        if not 1 <= self.d <= limit or not 1 <= self.dv <= limit or (not self.general and self.d < 16):
            raise ValueError(f"attention: head sizes {self.d} / {self.dv} are not supported (up to {limit})")
        self.scale = float(p["softmax_scale"])
        self.position = build_part("position", p["position"])
        self.qk_norm = bool(p.get("qk_norm", False))
        self.qk_norm_eps = float(p.get("qk_norm_eps", 0.0))
        self.norm_before_rope = p.get("qk_norm_order", "after_rope") == "before_rope"
        w = p.get("window") or {"kind": "full", "size": 0}
        if w["kind"] not in K.WINDOW_KINDS:
            raise ValueError(f"attention: unknown window kind '{w['kind']}'")
        self.window_kind, self.window_size = w["kind"], int(w.get("size", 0))
        t = p.get("query_temperature")
        self.temperature = None if t is None else (float(t["floor_scale"]), float(t["attn_scale"]))
        self.ws = workspace
        self.w_qkv = self.w_o = None
        self.rotary = self.score_bias = None
        self.b_qkv = self.w_qnorm = self.w_knorm = self.sink = self.w_conv = self.w_vmix = self.b_o = None
        self.keep_first = int(w.get("keep_first") or 0) if self.window_kind == "sliding" else 0
        if self.keep_first < 0:
            raise ValueError(f"attention: keep_first must not be negative, not {self.keep_first}")
        head_norm = self.qk_norm and self.norm_scope == "head"
        if self.norm_weight_shared and not (head_norm and self.norm_before_rope):
            raise ValueError("attention: a per-head norm weight shared by the heads belongs to the per-head norm "
                             "before the rotation (qk_norm, qk_norm_scope 'head', qk_norm_order 'before_rope')")
        if self.value_mix is not None and not self.has_kv:
            raise ValueError("attention: value mixing needs a layer that writes its own cache")
        if self.general and ((head_norm and self.norm_before_rope and not self.norm_weight_shared)
                             or (self.qk_norm and not head_norm and not self.norm_before_rope)):
            raise ValueError("attention: biases, a norm over the whole projection, a partial rotation or values of "
                             "another size do not combine with a weightless per-head norm before the rotation or a "
                             "whole-projection norm after it")
        a = "self_attn."
        self.tn = {"q": a + "q_proj.weight", "k": a + "k_proj.weight", "v": a + "v_proj.weight",
                   "o": a + "o_proj.weight", "q_bias": a + "q_proj.bias", "k_bias": a + "k_proj.bias",
                   "v_bias": a + "v_proj.bias", "q_norm": a + "q_norm.weight", "k_norm": a + "k_norm.weight",
                   "sink": a + "sinks", "q_conv": a + "q_conv.weight", "k_conv": a + "k_conv.weight",
                   "v_conv": a + "v_conv.weight", "v_mix": a + "v_mix", "g": a + "g_proj.weight",
                   "o_bias": a + "o_proj.bias", "lq1": a + "lambda_q1", "lk1": a + "lambda_k1", "lq2": a + "lambda_q2",
                   "lk2": a + "lambda_k2"}
        self.tn.update(p.get("tensor_names") or {})
        self.tn = {k: self.prefix + v for k, v in self.tn.items()}

    # ---- weights ---------------------------------------------------------------------------------
    def _names(self):
        return self.tn["q"], self.tn["k"], self.tn["v"], self.tn["o"]

    def requirements(self):
        q, k, v, o = self._names()
        M = self.maps
        reqs = [TensorReq(q, (M * self.nh * self.d, self.hidden)), TensorReq(o, (self.hidden, self.nh * self.dv))]
        if self.has_kv:
            reqs.append(TensorReq(k, (M * self.nkv * self.d, self.hidden)))
            if not self.values_from_keys:
                reqs.append(TensorReq(v, (self.nkv * self.dv, self.hidden)))
        if self.bias:
            reqs.append(TensorReq(self.tn["q_bias"], (M * self.nh * self.d,)))
            if self.has_kv:
                reqs.append(TensorReq(self.tn["k_bias"], (M * self.nkv * self.d,)))
                if not self.values_from_keys:
                    reqs.append(TensorReq(self.tn["v_bias"], (self.nkv * self.dv,)))
        if self.has_gate:
            reqs.append(TensorReq(self.tn["g"], (self.nh, self.hidden)))
        if self.has_o_bias:
            reqs.append(TensorReq(self.tn["o_bias"], (self.hidden,)))
        if self.diff is not None:
            reqs += [TensorReq(self.tn[n], (self.d,)) for n in ("lq1", "lk1", "lq2", "lk2")]
        if self.qk_norm and self.norm_scope == "projection":
            reqs.append(TensorReq(self.tn["q_norm"], (self.nh * self.d,), init="ones+normal"))
            if self.has_kv:
                reqs.append(TensorReq(self.tn["k_norm"], (self.nkv * self.d,), init="ones+normal"))
        if self.norm_weight_shared:
            reqs.append(TensorReq(self.tn["q_norm"], (self.d,), init="ones+normal"))
            if self.has_kv:
                reqs.append(TensorReq(self.tn["k_norm"], (self.d,), init="ones+normal"))
        if self.taps is not None:
            reqs.append(TensorReq(self.tn["q_conv"], (self.nh * self.d, self.taps), init="const:0.3+normal"))
            if self.has_kv:
                reqs += [TensorReq(self.tn["k_conv"], (self.nkv * self.d, self.taps), init="const:0.3+normal"),
                         TensorReq(self.tn["v_conv"], (self.nkv * self.dv, self.taps), init="const:0.3+normal")]
        if self.value_mix is not None:       # the first layer's number is stored too, and unused
            reqs.append(TensorReq(self.tn["v_mix"], (), init="const:0.5"))
        if self.has_sink:
            reqs.append(TensorReq(self.tn["sink"], (self.nh,)))
        return reqs

    def load(self, source, device):
        q, k, v, o = self._names()

        def by_map(t, heads):
            # rows stored head by head as [map 1, map 2] -> all heads' first maps, then all second maps
            if self.maps == 1:
                return t
            return t.reshape(heads, self.maps, self.d, *t.shape[1:]).transpose(0, 1).reshape(t.shape)

        parts = [by_map(source.get(q, device), self.nh)]
        if self.has_kv:
            parts.append(by_map(source.get(k, device), self.nkv))
            if not self.values_from_keys:
                parts.append(source.get(v, device))
        if self.has_gate:                       # the gates' rows ride on the same product: [q | k | v | g]
            parts.append(source.get(self.tn["g"], device))
        dt = torch.float32 if any(t.dtype == torch.float32 for t in parts) else torch.bfloat16
        self.w_qkv = torch.cat([t.to(dt) for t in parts], dim=0).contiguous()    # [Q + 2 KV (+ heads), H]
        del parts
        self.w_o = source.get(o, device).contiguous()
        if self.bias:
            names = [("q_bias", self.nh)] + ([("k_bias", self.nkv)] if self.has_kv else [])
            bs = [by_map(source.get(self.tn[n], device).to(torch.float32), heads) for n, heads in names]
            if self.has_kv and not self.values_from_keys:
                bs.append(source.get(self.tn["v_bias"], device).to(torch.float32))
            self.b_qkv = torch.cat(bs).contiguous()
        if self.has_o_bias:
            self.b_o = source.get(self.tn["o_bias"], device).to(torch.float32).contiguous()
        if self.diff is not None:
            l = {n: source.get(self.tn[n], "cpu").to(torch.float64) for n in ("lq1", "lk1", "lq2", "lk2")}
            self.lam = (math.exp(float((l["lq1"] * l["lk1"]).sum())) - math.exp(float((l["lq2"] * l["lk2"]).sum()))
                        + self.diff)
        if self.qk_norm and self.norm_scope == "projection":
            self.w_qnorm = source.get(self.tn["q_norm"], device).to(torch.float32).contiguous()
            if self.has_kv:
                self.w_knorm = source.get(self.tn["k_norm"], device).to(torch.float32).contiguous()
        if self.norm_weight_shared:
            self.w_qnorm = source.get(self.tn["q_norm"], device).to(torch.float32).contiguous()
            if self.has_kv:
                self.w_knorm = source.get(self.tn["k_norm"], device).to(torch.float32).contiguous()
        if self.taps is not None:
            names = ["q_conv"] + (["k_conv", "v_conv"] if self.has_kv else [])
            self.w_conv = torch.cat([source.get(self.tn[n], device).to(torch.float32) for n in names], dim=0).contiguous()
        if self.value_mix is not None and self.value_mix[0] == "later":
            self.w_vmix = source.get(self.tn["v_mix"], device).to(torch.float32).reshape(1).contiguous()
        if self.has_sink:
            self.sink = source.get(self.tn["sink"], device).to(torch.float32).contiguous()
        self.position.prepare(device)
        # what the position part is to this mixer: a rotation of q and k (done with the head norm and the cache
        # write, in one kernel), a bias on the scores (taken by the general attention kernel only), or nothing
        enc = self.position.encoding()
        self.rotary = enc if isinstance(enc, RotaryEncoding) else None
        self.score_bias = enc.table if isinstance(enc, ScoreBias) else None
        if enc is not None and self.rotary is None and self.score_bias is None:
            raise TypeError(f"attention: the position part '{self.position.spec.kind}' describes itself as "
                            f"{type(enc).__name__}; this mixer's kernels take RotaryEncoding, ScoreBias or None")
        if self.score_bias is not None and (self.score_bias.dim() != 2 or self.score_bias.shape[0] != self.nh
                                            or self.score_bias.dtype != torch.float32):
            raise ValueError(f"attention: a score bias must be float32 [{self.nh} heads, distances], got "
                             f"{tuple(self.score_bias.shape)} {self.score_bias.dtype}")

    # ---- cache -----------------------------------------------------------------------------------
    def kv_requirement(self):
        if self.maps == 2:
            return KVRequirement(self.nkv, self.d, self.window_kind, self.window_size, keep_first=self.keep_first,
                                 streams=(("k", self.nkv, self.d), ("k2", self.nkv, self.d), ("v", self.nkv, self.dv)))
        if self.dv != self.d:
            return KVRequirement(self.nkv, self.d, self.window_kind, self.window_size,
                                 streams=(("k", self.nkv, self.d), ("v", self.nkv, self.dv)), keep_first=self.keep_first)
        return KVRequirement(self.nkv, self.d, self.window_kind, self.window_size, keep_first=self.keep_first)

    def state_requirements(self):
        if self.taps is None:
            return []
        return [StateRequirement("conv", (max(self.taps - 1, 0), self.w_rows()))]

    def w_rows(self) -> int:
        """Rows of the stacked q | k | v projection (what the convolution runs over)."""
        kv = self.nkv * (self.maps * self.d + (0 if self.values_from_keys else self.dv))
        return self.maps * self.nh * self.d + (kv if self.has_kv else 0)

    # ---- step ------------------------------------------------------------------------------------
    can_store = True          # forward(..., add=False) stores the mixer's output (float32) instead of adding it

    def forward(self, h, residual, batch, cache, add=True):
        T = h.shape[0]
        dt = h.dtype
        k_cache, v_cache, table, page_size = cache.kv()
        q = self.ws.get("attn_q", (T, self.nh * self.d), dt)
        if self.general:
            # float32 projection rows: bias, norm and rotation act on unrounded values
            qkv = self.ws.get("attn_qkv", (T, self.w_qkv.shape[0]), torch.float32)
            with phase("qkv"):
                project(h, self.w_qkv, qkv)
            if self.taps is not None:          # the last taps - 1 projected rows of each sequence are its state
                conv = self.ws.get("attn_qkv_conv", (T, self.w_qkv.shape[0]), torch.float32)
                with phase("conv"):
                    K.causal_conv(qkv, self.w_conv, None, cache.state("conv"), conv, batch, silu=False)
                qkv = conv
            v_first, mix_mode = None, 0
            if self.value_mix is not None and cache.owns:
                v_first = self.ws.get("attn_" + self.value_mix[1], (T, self.nkv * self.dv), torch.float32)
                mix_mode = 1 if self.value_mix[0] == "first" else 2
            head_norm = self.qk_norm and self.norm_scope == "head"
            q2 = k2_cache = None
            if self.maps == 2:
                q2 = self.ws.get("attn_q2", (T, self.nh * self.d), dt)
                k2_cache = cache.stream("k2")[0]
            with phase("kv_store"):
                K.qkv_prepare(qkv, q, k_cache, v_cache, table, page_size, batch.token_seq, batch.token_pos,
                              batch.seq_slot, n_heads=self.nh, n_kv_heads=self.nkv, head_dim=self.d,
                              value_dim=self.dv, bias=self.b_qkv, q_norm=self.w_qnorm, k_norm=self.w_knorm,
                              norm_whole=self.qk_norm and self.norm_scope == "projection",
                              head_norm=(2 if self.norm_weight_shared else 1) if head_norm else 0,
                              norm_eps=self.qk_norm_eps,
                              inv_freq=None if self.rotary is None else self.rotary.inv_freq,
                              rotary_dims=self.rot_dims if self.rotary is not None else 0,
                              interleaved=self.rotary is not None and self.rotary.interleaved,
                              write_kv=self.has_kv and cache.owns, v_first=v_first, v_mix=self.w_vmix,
                              v_mix_mode=mix_mode, q2_out=q2, k2_cache=k2_cache, values_from_keys=self.values_from_keys,
                              temperature=self.temperature,
                              rotary_amplitude=1.0 if self.rotary is None else self.rotary.amplitude)
        else:
            qkv = self.ws.get("attn_qkv", (T, self.w_qkv.shape[0]), dt)
            with phase("qkv"):
                project(h, self.w_qkv, qkv)
            with phase("kv_store"):          # head norm, rotation, temperature and the write into the cache: one kernel
                K.qkv_post(qkv, q, k_cache, v_cache, table, page_size, batch.token_seq, batch.token_pos,
                           batch.seq_slot, n_heads=self.nh, n_kv_heads=self.nkv, head_dim=self.d,
                           inv_freq=None if self.rotary is None else self.rotary.inv_freq,
                           interleaved=self.rotary is not None and self.rotary.interleaved,
                           qk_norm=self.qk_norm, norm_before_rope=self.norm_before_rope,
                           norm_eps=self.qk_norm_eps, temperature=self.temperature,
                           write_kv=self.has_kv and cache.owns)
        att = self.ws.get("attn_out", (T, self.nh * self.dv), dt)
        with phase("attention"):
            self.attend(q, att, k_cache, v_cache, table, page_size, batch)
            att2 = None
            if self.maps == 2:                  # the second map: its own queries and keys, the same values
                att2 = self.ws.get("attn_out2", (T, self.nh * self.dv), dt)
                self.attend(q2, att2, k2_cache, v_cache, table, page_size, batch)
        if att2 is not None or self.has_gate:
            with phase("head_post"):            # a1 - lambda a2, its norm, the gate: one pass over the heads' outputs
                K.head_post(att, att, n_heads=self.nh, value_dim=self.dv, a2=att2, lam=self.lam,
                            norm_eps=self.qk_norm_eps if att2 is not None else None,
                            norm_scale=1.0 if self.diff is None else 1.0 - self.diff,
                            gate=qkv[:, qkv.shape[1] - self.nh:] if self.has_gate else None)
        with phase("wo"):
            if self.b_o is not None:            # the product adds into rows that hold the bias
                K.bias_rows(residual, self.b_o, add=add)
                add = True
            project(att, self.w_o, residual, MODE_ADD if add else MODE_STORE)

    def attend(self, q, att, k_cache, v_cache, table, page_size, batch):
        attend(q, att, k_cache, v_cache, table, page_size, batch, n_heads=self.nh, n_kv_heads=self.nkv, head_dim=self.d,
               value_dim=self.dv, window_kind=self.window_kind, window_size=self.window_size, scale=self.scale,
               sink=self.sink, keep_first=self.keep_first, score_bias=self.score_bias, softcap=self.softcap)


def attend(q, att, k_cache, v_cache, table, page_size, batch, *, n_heads, n_kv_heads, head_dim, value_dim, window_kind,
           window_size, scale, sink=None, keep_first=0, score_bias=None, softcap=0.0):
    """Softmax attention of the step's prepared queries q [T, heads * head_dim] over a paged cache into att
    [T, heads * value_dim]: the tensor-core kernels where they apply (bfloat16, keys and values of one size 64 or 128,
    nothing added to the scores), the general kernel otherwise."""
    nh, nkv, d, dv = n_heads, n_kv_heads, head_dim, value_dim
    wk = K.WINDOW_KINDS[window_kind]
    # the tensor-core kernels add nothing to a score and take keys and values of one size
    tensor_cores = use_tensor_core_kernels and score_bias is None and dv == d
    if (tensor_cores and batch.is_decode and q.dtype == torch.bfloat16
            and K.attention_decode_supported(nh, nkv, d, page_size)):
        # keys per sequence that the window lets through, at most (a bucketed bound: the split count
        # then stays the same from step to step, which a captured graph needs)
        longest = batch.ctx_bucket
        if window_kind != "full":
            kept = -(-keep_first // page_size) * page_size       # the kept first positions, in whole pages
            longest = min(longest, window_size + page_size + kept)
        pages = -(-longest // page_size)
        base = batch.n_tokens * nkv
        slots = K.attention_decode_blocks_per_sm(d) * K.sm_count()     # blocks that run at once
        if base <= slots:
            want = slots // base                                # one full wave and no more
        else:
            want = -(-4 * slots // base)                        # several waves of smaller blocks
        n_splits = max(1, min(want, pages // 4, K.MAX_DECODE_SPLITS))    # a block takes four pages or more
        K.attention_decode(q, att, k_cache, v_cache, table, page_size, batch.token_seq, batch.token_pos,
                           batch.seq_slot, n_heads=nh, n_kv_heads=nkv, head_dim=d,
                           window_kind=wk, window_size=window_size, scale=scale, n_splits=n_splits,
                           sink=sink, keep_first=keep_first, softcap=softcap)
        return
    if (tensor_cores and not batch.is_decode and q.dtype == torch.bfloat16 and batch.n_q_tiles
            and K.attention_prefill_supported(nh, nkv, d, page_size)):
        K.attention_prefill(q, att, k_cache, v_cache, table, page_size, batch.token_seq, batch.token_pos,
                            batch.seq_slot, batch.tile_tok0, batch.tile_rows, n_heads=nh,
                            n_kv_heads=nkv, head_dim=d, window_kind=wk, window_size=window_size,
                            scale=scale, sink=sink, keep_first=keep_first, softcap=softcap)
        return
    K.attention_general(q, att, k_cache, v_cache, table, page_size, batch.token_seq, batch.token_pos,
                        batch.seq_slot, n_heads=nh, n_kv_heads=nkv, head_dim=d, window_kind=wk,
                        window_size=window_size, scale=scale, score_bias=score_bias, sink=sink, value_dim=dv,
                        keep_first=keep_first, softcap=softcap)
