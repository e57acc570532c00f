"""Recurrent mixers: what they remember is a fixed-size state per sequence, not a growing cache.

Both keep, per head, a matrix S [rows, columns] in float32 that is updated token by token,
    S_t = diag(a_t) S_{t-1} + k_t v_t^T,        o_t = S_t^T q_t,
and differ in where a, k, q and v come from (`csrc/recurrent.cu: linear_scan`).  The state lives in the cache
manager's per-slot state tensors, is zero when a slot is acquired and is carried across steps, so a prompt may
come whole, in pieces or token by token.  Decays, step sizes, gates of the recurrence and the state are float32
in both precisions; the projections feed them as float32 rows.

"mamba2"  selective state space, scalar decay per head:
          [z | x | B | C | dt] = W_in h;  (x, B, C) <- silu(causal conv over the last `conv` tokens, per channel);
          dt <- softplus(dt + dt_bias);  a = exp(-exp(A_log) dt);  k = B, q = C (shared by the heads of a group),
          v = dt x;  y = o + D x;  out = W_o (groupnorm(y * silu(z)) * norm)   -- the gate comes before the norm.
          params: hidden_size, heads, head_dim (columns), state (rows), groups, conv (taps), norm_groups, norm_eps,
          tensor_names {"in", "conv", "conv_bias", "dt_bias", "A_log", "D", "norm", "o"}.
          state: "ssm" [heads, state, head_dim], "conv" [conv - 1, channels] (the last inputs of the convolution).
"gla"     gated linear attention, a decay per key channel:
          q = W_q h / sqrt(key_dim), k = W_k h, v = W_v h;  a = sigmoid(W_a2 (W_a1 h) + b)^(1 / tau);
          out = W_o (concat_heads(rmsnorm(o_head) * norm) * silu(W_g h))   -- norm weight shared by the heads.
          params: hidden_size, heads, key_dim (rows), value_dim (columns), tau, decay_rank, norm_eps,
          tensor_names {"q", "k", "v", "g", "o", "norm", "a1", "a2", "a2_bias"}.
          state: "s" [heads, key_dim, value_dim].

"rglru" keeps a vector instead of a matrix: one state element per channel, see `RGLRUMixer`.
"""
from __future__ import annotations

import torch

from ..cache.manager import StateRequirement
from ..csrc import lib as K
from ..phases import phase
from ..weights.store import TensorReq
from .base import Mixer, register_mixer
from .linear import MODE_ADD, MODE_STORE, project

# steps whose longest portion has more tokens than this prepare the row decays with a kernel of their own
DECAY_PREPASS_FROM = 16


def _cat_rows(tensors):
    dt = torch.float32 if any(t.dtype == torch.float32 for t in tensors) else torch.bfloat16
    return torch.cat([t.to(dt) for t in tensors], dim=0).contiguous()


@register_mixer("mamba2")
class Mamba2Mixer(Mixer):
    graph_safe = True
    can_store = True

    def __init__(self, spec, prefix="", workspace=None, owns_cache=True):
        super().__init__(spec, prefix)
        p = spec.params
        self.hidden, self.nh, self.dv = int(p["hidden_size"]), int(p["heads"]), int(p["head_dim"])
        self.n, self.groups, self.taps = int(p["state"]), int(p["groups"]), int(p["conv"])
        self.norm_groups, self.eps = int(p.get("norm_groups", 1)), float(p["norm_eps"])
        self.inner = self.nh * self.dv
        if self.nh % self.groups:
            raise ValueError(f"mamba2: {self.nh} heads cannot share {self.groups} groups of B and C")
        if self.inner % self.norm_groups:
            raise ValueError(f"mamba2: {self.inner} channels cannot be normed in {self.norm_groups} equal parts")
        if not 1 <= self.taps <= 8:
            raise ValueError(f"mamba2: a convolution of {self.taps} taps (supported: 1 to 8)")
        if not owns_cache:
            raise ValueError("mamba2: a recurrent layer cannot read another run entry's state")
        self.channels = self.inner + 2 * self.groups * self.n          # what the convolution runs over
        self.proj = 2 * self.inner + 2 * self.groups * self.n + self.nh
        tn = {"in": "mixer.in_proj.weight", "conv": "mixer.conv1d.weight", "conv_bias": "mixer.conv1d.bias",
              "dt_bias": "mixer.dt_bias", "A_log": "mixer.A_log", "D": "mixer.D", "norm": "mixer.norm.weight",
              "o": "mixer.out_proj.weight"}
        tn.update(p.get("tensor_names") or {})
        self.tn = {k: prefix + v for k, v in tn.items()}
        self.ws = workspace
        self.w_in = self.w_conv = self.b_conv = self.dt_bias = self.a_log = self.d_skip = self.w_norm = self.w_o = None

    def requirements(self):
        t = self.tn
        return [TensorReq(t["in"], (self.proj, self.hidden)), TensorReq(t["conv"], (self.channels, self.taps)),
                TensorReq(t["conv_bias"], (self.channels,)), TensorReq(t["dt_bias"], (self.nh,)),
                TensorReq(t["A_log"], (self.nh,)), TensorReq(t["D"], (self.nh,), init="ones+normal"),
                TensorReq(t["norm"], (self.inner,), init="ones+normal"), TensorReq(t["o"], (self.hidden, self.inner))]

    def load(self, source, device):
        t = self.tn
        f32 = lambda name: source.get(t[name], device).to(torch.float32).contiguous()
        self.w_in = source.get(t["in"], device).contiguous()
        self.w_conv, self.b_conv = f32("conv"), f32("conv_bias")
        self.dt_bias, self.a_log, self.d_skip, self.w_norm = f32("dt_bias"), f32("A_log"), f32("D"), f32("norm")
        self.w_o = source.get(t["o"], device).contiguous()

    def state_requirements(self):
        return [StateRequirement("ssm", (self.nh, self.n, self.dv)),
                StateRequirement("conv", (max(self.taps - 1, 0), self.channels))]

    def forward(self, h, residual, batch, cache, add=True):
        T, f32 = h.shape[0], torch.float32
        inner, gn = self.inner, self.groups * self.n
        proj = self.ws.get("mamba_proj", (T, self.proj), f32)
        with phase("qkv"):
            project(h, self.w_in, proj)
        xbc = self.ws.get("mamba_xbc", (T, self.channels), f32)
        with phase("conv"):
            K.causal_conv(proj[:, inner:inner + self.channels], self.w_conv, self.b_conv, cache.state("conv"), xbc,
                          batch, silu=True)
        y = self.ws.get("mamba_y", (T, inner), f32)
        with phase("scan"):
            K.linear_scan(xbc[:, inner:inner + gn], xbc[:, inner + gn:], xbc[:, :inner], cache.state("ssm"), y, batch,
                          n_heads=self.nh, heads_per_group=self.nh // self.groups, n_rows=self.n, n_cols=self.dv,
                          dt=proj[:, inner + self.channels:], dt_bias=self.dt_bias, a_log=self.a_log,
                          skip=self.d_skip)
        with phase("gated_norm"):
            g = self.ws.get("mamba_gated", (T, inner), h.dtype)
            K.gated_norm(y, proj[:, :inner], self.w_norm, g, parts=self.norm_groups, gate_first=True, eps=self.eps)
        with phase("wo"):
            project(g, self.w_o, residual, MODE_ADD if add else MODE_STORE)


@register_mixer("gla")
class GLAMixer(Mixer):
    graph_safe = True
    can_store = True

    def __init__(self, spec, prefix="", workspace=None, owns_cache=True):
        super().__init__(spec, prefix)
        p = spec.params
        self.hidden, self.nh = int(p["hidden_size"]), int(p["heads"])
        self.dk, self.dv = int(p["key_dim"]), int(p["value_dim"])
        self.tau, self.rank, self.eps = float(p["tau"]), int(p["decay_rank"]), float(p["norm_eps"])
        if self.tau <= 0:
            raise ValueError(f"gla: tau must be positive, not {self.tau}")
        if not owns_cache:
            raise ValueError("gla: a recurrent layer cannot read another run entry's state")
        tn = {"q": "mixer.q_proj.weight", "k": "mixer.k_proj.weight", "v": "mixer.v_proj.weight",
              "g": "mixer.g_proj.weight", "o": "mixer.o_proj.weight", "norm": "mixer.g_norm.weight",
              "a1": "mixer.gk_proj.0.weight", "a2": "mixer.gk_proj.1.weight", "a2_bias": "mixer.gk_proj.1.bias"}
        tn.update(p.get("tensor_names") or {})
        self.tn = {k: prefix + v for k, v in tn.items()}
        self.ws = workspace
        self.w_qkvg = self.w_a1 = self.w_a2 = self.b_a2 = self.w_norm = self.w_o = None

    def requirements(self):
        t, H, nk, nv = self.tn, self.hidden, self.nh * self.dk, self.nh * self.dv
        return [TensorReq(t["q"], (nk, H)), TensorReq(t["k"], (nk, H)), TensorReq(t["v"], (nv, H)),
                TensorReq(t["g"], (nv, H)), TensorReq(t["o"], (H, nv)), TensorReq(t["norm"], (self.dv,), init="ones+normal"),
                TensorReq(t["a1"], (self.rank, H)), TensorReq(t["a2"], (nk, self.rank)), TensorReq(t["a2_bias"], (nk,))]

    def load(self, source, device):
        t = self.tn
        self.w_qkvg = _cat_rows([source.get(t[n], device) for n in ("q", "k", "v", "g")])
        self.w_a1 = source.get(t["a1"], device).contiguous()
        self.w_a2 = source.get(t["a2"], device).contiguous()
        self.b_a2 = source.get(t["a2_bias"], device).to(torch.float32).contiguous()
        self.w_norm = source.get(t["norm"], device).to(torch.float32).contiguous()
        self.w_o = source.get(t["o"], device).contiguous()

    def state_requirements(self):
        return [StateRequirement("s", (self.nh, self.dk, self.dv))]

    def forward(self, h, residual, batch, cache, add=True):
        T, f32 = h.shape[0], torch.float32
        nk, nv = self.nh * self.dk, self.nh * self.dv
        proj = self.ws.get("gla_proj", (T, 2 * nk + 2 * nv), f32)
        low = self.ws.get("gla_low", (T, self.rank), h.dtype)
        z = self.ws.get("gla_z", (T, nk), f32)
        with phase("qkv"):
            project(h, self.w_qkvg, proj)
            project(h, self.w_a1, low)
            project(low, self.w_a2, z)
        o = self.ws.get("gla_o", (T, nv), f32)
        with phase("scan"):
            # a step of many tokens prepares its decays once per element; a decode step leaves them to the
            # recurrence (one launch less), which computes the same expression
            ready = batch.max_new > DECAY_PREPASS_FROM
            if ready:
                K.row_decay(z, self.b_a2, self.tau)
            K.linear_scan(proj[:, nk:2 * nk], proj[:, :nk], proj[:, 2 * nk:2 * nk + nv], cache.state("s"), o, batch,
                          n_heads=self.nh, heads_per_group=1, n_rows=self.dk, n_cols=self.dv, z=z,
                          z_bias=None if ready else self.b_a2, tau=self.tau, q_scale=self.dk ** -0.5,
                          decay_ready=ready)
        with phase("gated_norm"):
            g = self.ws.get("gla_gated", (T, nv), h.dtype)
            K.gated_norm(o, proj[:, 2 * nk + nv:], self.w_norm, g, parts=self.nh, gate_first=False, eps=self.eps)
        with phase("wo"):
            project(g, self.w_o, residual, MODE_ADD if add else MODE_STORE)


@register_mixer("gated_delta")
class GatedDeltaMixer(Mixer):
    """The gated delta rule: a matrix state per head that forgets per key channel and is corrected, not just added to.

        q = W_q h, k = W_k h (kv_heads heads of key_dim), v = W_v h (heads of value_dim); each passes a short causal
        convolution per channel (no bias) and silu; q and k become unit vectors per head, x / sqrt(sum x^2 + unit_eps);
        beta = sigmoid(W_b h) per head;  a = exp(-exp(A_log[head]) softplus(W_a2 (W_a1 h) + dt_bias)) per head and key channel;
        S <- diag(a) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q / sqrt(key_dim)   (head h reads q/k head h // (heads / kv_heads));
        out = W_o concat_heads(rmsnorm(o_head) * norm * sigmoid(W_g2 (W_g1 h)))   -- norm weight shared by the heads.

    params: hidden_size, heads, kv_heads, key_dim, value_dim, conv (taps), decay_rank, gate_rank, norm_eps, unit_eps,
    tensor_names {"q", "k", "v", "q_conv", "k_conv", "v_conv", "b", "A_log", "dt_bias", "a1", "a2", "g1", "g2", "norm", "o"}.
    state: "s" [heads, key_dim, value_dim] float32, "conv" [conv - 1, channels] (the last inputs of the convolutions).
    Decays, beta, the unit vectors and the state are float32 in both precisions."""
    graph_safe = True
    can_store = True

    def __init__(self, spec, prefix="", workspace=None, owns_cache=True):
        super().__init__(spec, prefix)
        p = spec.params
        self.hidden, self.nh, self.nkv = int(p["hidden_size"]), int(p["heads"]), int(p.get("kv_heads") or p["heads"])
        self.dk, self.dv, self.taps = int(p["key_dim"]), int(p["value_dim"]), int(p.get("conv") or 1)
        self.rank_a, self.rank_g = int(p["decay_rank"]), int(p["gate_rank"])
        self.eps, self.unit_eps = float(p["norm_eps"]), float(p.get("unit_eps", 1e-6))
        if self.nh % self.nkv:
            raise ValueError(f"gated_delta: {self.nh} heads cannot share {self.nkv} heads of q and k")
        if not 1 <= self.taps <= 8:
            raise ValueError(f"gated_delta: a convolution of {self.taps} taps (supported: 1 to 8)")
        if not owns_cache:
            raise ValueError("gated_delta: a recurrent layer cannot read another run entry's state")
        self.nqk, self.nv = self.nkv * self.dk, self.nh * self.dv
        self.channels = 2 * self.nqk + self.nv                       # what the convolutions run over: q | k | v
        tn = {"q": "mixer.q_proj.weight", "k": "mixer.k_proj.weight", "v": "mixer.v_proj.weight",
              "q_conv": "mixer.q_conv.weight", "k_conv": "mixer.k_conv.weight", "v_conv": "mixer.v_conv.weight",
              "b": "mixer.b_proj.weight", "A_log": "mixer.A_log", "dt_bias": "mixer.dt_bias",
              "a1": "mixer.a_proj.0.weight", "a2": "mixer.a_proj.1.weight", "g1": "mixer.g_proj.0.weight",
              "g2": "mixer.g_proj.1.weight", "norm": "mixer.o_norm.weight", "o": "mixer.o_proj.weight"}
        tn.update(p.get("tensor_names") or {})
        self.tn = {k: prefix + v for k, v in tn.items()}
        self.ws = workspace
        self.w_in = self.w_conv = self.w_a2 = self.w_g2 = self.dt_bias = self.a_log = self.w_norm = self.w_o = None

    def requirements(self):
        t, H = self.tn, self.hidden
        return [TensorReq(t["q"], (self.nqk, H)), TensorReq(t["k"], (self.nqk, H)), TensorReq(t["v"], (self.nv, H)),
                TensorReq(t["q_conv"], (self.nqk, self.taps), init="const:0.3+normal"),
                TensorReq(t["k_conv"], (self.nqk, self.taps), init="const:0.3+normal"),
                TensorReq(t["v_conv"], (self.nv, self.taps), init="const:0.3+normal"),
                TensorReq(t["b"], (self.nh, H)), TensorReq(t["A_log"], (self.nh,)),
                TensorReq(t["dt_bias"], (self.nh * self.dk,)),
                TensorReq(t["a1"], (self.rank_a, H)), TensorReq(t["a2"], (self.nh * self.dk, self.rank_a)),
                TensorReq(t["g1"], (self.rank_g, H)), TensorReq(t["g2"], (self.nv, self.rank_g)),
                TensorReq(t["norm"], (self.dv,), init="ones+normal"), TensorReq(t["o"], (H, self.nv))]

    def load(self, source, device):
        t = self.tn
        f32 = lambda name: source.get(t[name], device).to(torch.float32).contiguous()
        self.w_in = _cat_rows([source.get(t[n], device) for n in ("q", "k", "v", "b", "a1", "g1")])
        self.w_conv = torch.cat([f32("q_conv"), f32("k_conv"), f32("v_conv")], dim=0).contiguous()
        self.w_a2 = source.get(t["a2"], device).contiguous()
        self.w_g2 = source.get(t["g2"], device).contiguous()
        self.dt_bias, self.a_log, self.w_norm = f32("dt_bias"), f32("A_log"), f32("norm")
        self.w_o = source.get(t["o"], device).contiguous()

    def state_requirements(self):
        return [StateRequirement("s", (self.nh, self.dk, self.dv)),
                StateRequirement("conv", (max(self.taps - 1, 0), self.channels))]

    def forward(self, h, residual, batch, cache, add=True):
        T, f32 = h.shape[0], torch.float32
        C, nqk, nv = self.channels, self.nqk, self.nv
        o_b, o_a, o_g = C, C + self.nh, C + self.nh + self.rank_a
        proj = self.ws.get("gdr_proj", (T, o_g + self.rank_g), f32)
        z = self.ws.get("gdr_z", (T, self.nh * self.dk), f32)
        gate = self.ws.get("gdr_gate", (T, nv), f32)
        with phase("qkv"):
            project(h, self.w_in, proj)
            project(proj[:, o_a:o_g], self.w_a2, z)
            project(proj[:, o_g:], self.w_g2, gate)
        qkv = self.ws.get("gdr_qkv", (T, C), f32)
        with phase("conv"):
            K.causal_conv(proj[:, :C], self.w_conv, None, cache.state("conv"), qkv, batch, silu=True)
            K.head_unit(qkv[:, :2 * nqk], heads=2 * self.nkv, dim=self.dk, eps=self.unit_eps)
        o = self.ws.get("gdr_o", (T, nv), f32)
        with phase("scan"):
            ready = batch.max_new > DECAY_PREPASS_FROM
            if ready:
                K.row_decay(z, self.dt_bias, 1.0, kind=1, a_log=self.a_log, rows_per_head=self.dk)
            K.linear_scan(qkv[:, nqk:2 * nqk], qkv[:, :nqk], qkv[:, 2 * nqk:], cache.state("s"), o, batch,
                          n_heads=self.nh, heads_per_group=self.nh // self.nkv, n_rows=self.dk, n_cols=self.dv, z=z,
                          z_bias=self.dt_bias, a_log=self.a_log, decay_kind=1, decay_ready=ready,
                          q_scale=self.dk ** -0.5, beta=proj[:, o_b:o_a])
        with phase("gated_norm"):
            g = self.ws.get("gdr_gated", (T, nv), h.dtype)
            K.gated_norm(o, gate, self.w_norm, g, parts=self.nh, gate_first=False, eps=self.eps, gate_act="sigmoid")
        with phase("wo"):
            project(g, self.w_o, residual, MODE_ADD if add else MODE_STORE)


@register_mixer("rglru")
class RGLRUMixer(Mixer):
    """A recurrent block around a real-gated linear recurrent unit: two branches of `width` channels,

        y = gelu_tanh(W_y h + b_y);   u = conv(W_x h + b_x)   (a causal convolution per channel with a bias, no activation);
        per block b of `blocks` equal parts of u:  r = sigmoid(A_b u_b + a_b),  i = sigmoid(I_b u_b + i_b);
        log a = -decay_scale * softplus(lam) * r;   S <- a S + sqrt(1 - a^2) (i u);   out = W_o (S y).

    params: hidden_size, width, blocks, conv (taps), decay_scale (8 by default),
    tensor_names {"y", "y_bias", "x", "x_bias", "conv", "conv_bias", "ra", "ra_bias", "ri", "ri_bias", "lam", "o"}
    (ra, ri: [blocks, n, n] as [out, in]; their biases [blocks, n]).
    state: "s" [width] float32, "conv" [conv - 1, width] (the last inputs of the convolution, biases included).
    The gates' products take u in the activation dtype; the gates themselves, the decay with its softplus and
    exponential, sqrt(1 - a^2), the state and the product S y are float32 in both precisions."""
    graph_safe = True
    can_store = True

    def __init__(self, spec, prefix="", workspace=None, owns_cache=True):
        super().__init__(spec, prefix)
        p = spec.params
        self.hidden, self.width, self.blocks = int(p["hidden_size"]), int(p["width"]), int(p["blocks"])
        self.taps, self.rate = int(p.get("conv") or 1), float(p.get("decay_scale", 8.0))
        if self.blocks < 1 or self.width % self.blocks:
            raise ValueError(f"rglru: {self.width} channels cannot be cut into {self.blocks} equal blocks")
        if not 1 <= self.taps <= 8:
            raise ValueError(f"rglru: a convolution of {self.taps} taps (supported: 1 to 8)")
        if not owns_cache:
            raise ValueError("rglru: a recurrent layer cannot read another run entry's state")
        self.n = self.width // self.blocks
        tn = {"y": "mixer.y_proj.weight", "y_bias": "mixer.y_proj.bias", "x": "mixer.x_proj.weight",
              "x_bias": "mixer.x_proj.bias", "conv": "mixer.conv1d.weight", "conv_bias": "mixer.conv1d.bias",
              "ra": "mixer.recurrent_gate.weight", "ra_bias": "mixer.recurrent_gate.bias",
              "ri": "mixer.input_gate.weight", "ri_bias": "mixer.input_gate.bias", "lam": "mixer.recurrent_param",
              "o": "mixer.out_proj.weight"}
        tn.update(p.get("tensor_names") or {})
        self.tn = {k: prefix + v for k, v in tn.items()}
        self.ws = workspace
        self.w_in = self.b_y = self.b_x = self.w_conv = self.b_conv = self.w_gates = self.b_r = self.b_i = None
        self.lam = self.w_o = None

    def requirements(self):
        t, H, W, B, n = self.tn, self.hidden, self.width, self.blocks, self.n
        return [TensorReq(t["y"], (W, H)), TensorReq(t["y_bias"], (W,)), TensorReq(t["x"], (W, H)),
                TensorReq(t["x_bias"], (W,)), TensorReq(t["conv"], (W, self.taps), init="const:0.3+normal"),
                TensorReq(t["conv_bias"], (W,)), TensorReq(t["ra"], (B, n, n)), TensorReq(t["ra_bias"], (B, n)),
                TensorReq(t["ri"], (B, n, n)), TensorReq(t["ri_bias"], (B, n)), TensorReq(t["lam"], (W,)),
                TensorReq(t["o"], (H, W))]

    def load(self, source, device):
        t = self.tn
        f32 = lambda name: source.get(t[name], device).to(torch.float32).reshape(-1).contiguous()
        self.w_in = _cat_rows([source.get(t["y"], device), source.get(t["x"], device)])          # [2 W, H]
        self.b_y, self.b_x, self.b_conv = f32("y_bias"), f32("x_bias"), f32("conv_bias")
        self.w_conv = source.get(t["conv"], device).to(torch.float32).contiguous()
        ra, ri = source.get(t["ra"], device), source.get(t["ri"], device)
        dt = torch.float32 if torch.float32 in (ra.dtype, ri.dtype) else torch.bfloat16
        self.w_gates = torch.cat([ra.to(dt), ri.to(dt)], dim=1).contiguous()                      # [blocks, 2 n, n]
        self.b_r, self.b_i, self.lam = f32("ra_bias"), f32("ri_bias"), f32("lam")
        self.w_o = source.get(t["o"], device).contiguous()

    def state_requirements(self):
        return [StateRequirement("s", (self.width,)), StateRequirement("conv", (max(self.taps - 1, 0), self.width))]

    def forward(self, h, residual, batch, cache, add=True):
        T, f32, W, B, n = h.shape[0], torch.float32, self.width, self.blocks, self.n
        proj = self.ws.get("rglru_proj", (T, 2 * W), f32)                  # [y | x] before their biases
        with phase("qkv"):
            project(h, self.w_in, proj)
        u = self.ws.get("rglru_u", (T, W), f32)
        with phase("conv"):
            K.causal_conv(proj[:, W:], self.w_conv, self.b_conv, cache.state("conv"), u, batch, silu=False,
                          in_bias=self.b_x)
        # the gates: a block-diagonal product, run as a grouped product with one group per block over u's blocks
        # laid out block by block
        ub = self.ws.get("rglru_ub", (B * T, n), h.dtype)
        offsets = self.ws.get("rglru_offsets", (B + 1,), torch.int32)
        gates = self.ws.get("rglru_gates", (B * T, 2 * n), f32)
        with phase("gates"):
            K.block_major_rows(u, ub, offsets, parts=B)
            project(ub, self.w_gates, gates, MODE_STORE, m_rows=B * T, group_offsets=offsets, n_groups=B,
                    rows_per_group_hint=T)
        out = self.ws.get("rglru_out", (T, W), h.dtype)
        with phase("scan"):
            K.rglru_scan(gates, u, proj[:, :W], cache.state("s"), out, batch, block=n, lam=self.lam, r_bias=self.b_r,
                         i_bias=self.b_i, y_bias=self.b_y, rate=self.rate)
        with phase("wo"):
            project(out, self.w_o, residual, MODE_ADD if add else MODE_STORE)
