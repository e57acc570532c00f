"""Attention over a cached latent: what a position keeps is one low-rank vector and one rotated key part.

"latent_attention"   c_q = rmsnorm(W_dq h) * dq_norm;  q = W_uq c_q, head by head [dim plain | rot_dim rotated];
                     [c' | r] = W_dkv h;  c = rmsnorm(c') * dkv_norm (kv_rank elements), r rotated (rot_dim elements,
                     one for all heads);  head n: key [W_uk,n c | r], value W_uv,n c;
                     score = (q . key) * scale over all earlier positions and the token's own, softmax with an optional
                     learned sink per head (its exponential joins the denominator, without a key or a value);
                     out = W_o concat_heads(sum_j p_j value_j).
                     params: hidden_size, heads, head_dim (plain), rot_dim, value_dim, q_rank, kv_rank, softmax_scale,
                     norm_eps, position (PartSpec; a rotation of rot_dim elements, or "none"), sink (bool),
                     tensor_names {"dq", "dq_norm", "uq", "dkv", "dkv_norm", "uk", "uv", "o", "sink"}.
                     cache: one stream "latent" of one head of kv_rank + rot_dim elements per position.

How it runs.  Only [c | r] is cached, and the keys and values of the heads are never formed: since
q_n . (W_uk,n c) = (W_uk,n^T q_n) . c, the plain part of a query is first taken through W_uk,n^T (a grouped product, one
group per head, over rows laid out head by head), and attention then runs over the cached rows themselves as ONE
key/value head of kv_rank + rot_dim elements that all query heads share, with the library's attention kernels.  Its
output per head is a weighted sum of rows [c | r]; the first kv_rank elements go through W_uv,n (the second grouped
product) and the result through W_o.  Norms, the rotation, scores and softmax are float32 in both precisions.
"""
from __future__ import annotations

import torch

from ..cache.manager import KVRequirement
from ..csrc import lib as K
from ..phases import phase
from ..weights.store import TensorReq
from . import attention as _attention
from .attention import attend
from .base import Mixer, RotaryEncoding, build_part, register_mixer
from .linear import MODE_ADD, MODE_STORE, project


def use_tensor_core_kernels() -> bool:
    """The switch of the attention part: off, every attention runs through the general kernel."""
    return _attention.use_tensor_core_kernels


@register_mixer("latent_attention")
class LatentAttentionMixer(Mixer):
    graph_safe = True
    can_store = True

    def __init__(self, spec, prefix="", workspace=None, owns_cache=True):
        super().__init__(spec, prefix)
        p = spec.params
        if not owns_cache:
            raise ValueError("latent_attention: reading another run entry's cache is not supported")
        self.hidden, self.nh = int(p["hidden_size"]), int(p["heads"])
        self.d, self.r, self.dv = int(p["head_dim"]), int(p["rot_dim"]), int(p["value_dim"])
        self.q_rank, self.kv_rank = int(p["q_rank"]), int(p["kv_rank"])
        self.scale, self.eps = float(p["softmax_scale"]), float(p["norm_eps"])
        self.has_sink = bool(p.get("sink", False))
        self.row = self.kv_rank + self.r              # what a position keeps, and the size of a query head
        if self.r % 2 or self.r < 0:
            raise ValueError(f"latent_attention: a rotated part of {self.r} elements (an even number)")
        if self.row > K.GENERAL_ATTENTION_MAX_DIM:
            raise ValueError(f"latent_attention: kv_rank + rot_dim = {self.row} exceeds the attention kernels' "
                             f"{K.GENERAL_ATTENTION_MAX_DIM}")
        self.position = build_part("position", p["position"])
        tn = {"dq": "mixer.q_a_proj.weight", "dq_norm": "mixer.q_a_norm.weight", "uq": "mixer.q_b_proj.weight",
              "dkv": "mixer.kv_a_proj.weight", "dkv_norm": "mixer.kv_a_norm.weight", "uk": "mixer.k_b_proj.weight",
              "uv": "mixer.v_b_proj.weight", "o": "mixer.o_proj.weight", "sink": "mixer.sinks"}
        tn.update(p.get("tensor_names") or {})
        self.tn = {k: prefix + v for k, v in tn.items()}
        self.ws = workspace
        self.w_down = self.w_uq = self.w_ukT = self.w_uv = self.w_o = None
        self.w_qnorm = self.w_cnorm = self.sink = self.rotary = None

    def requirements(self):
        t, H = self.tn, self.hidden
        reqs = [TensorReq(t["dq"], (self.q_rank, H)), TensorReq(t["dq_norm"], (self.q_rank,), init="ones+normal"),
                TensorReq(t["uq"], (self.nh * (self.d + self.r), self.q_rank)),
                TensorReq(t["dkv"], (self.row, H)), TensorReq(t["dkv_norm"], (self.kv_rank,), init="ones+normal"),
                TensorReq(t["uk"], (self.nh * self.d, self.kv_rank)), TensorReq(t["uv"], (self.nh * self.dv, self.kv_rank)),
                TensorReq(t["o"], (H, self.nh * self.dv))]
        if self.has_sink:
            reqs.append(TensorReq(t["sink"], (self.nh,)))
        return reqs

    def load(self, source, device):
        t = self.tn
        f32 = lambda name: source.get(t[name], device).to(torch.float32).contiguous()
        dq, dkv = source.get(t["dq"], device), source.get(t["dkv"], device)
        dt = torch.float32 if torch.float32 in (dq.dtype, dkv.dtype) else torch.bfloat16
        self.w_down = torch.cat([dq.to(dt), dkv.to(dt)], dim=0).contiguous()          # [q_rank + kv_rank + rot, H]
        self.w_uq = source.get(t["uq"], device).contiguous()
        uk = source.get(t["uk"], device).view(self.nh, self.d, self.kv_rank)
        self.w_ukT = uk.transpose(1, 2).contiguous()                                   # [heads, kv_rank, dim]
        self.w_uv = source.get(t["uv"], device).view(self.nh, self.dv, self.kv_rank).contiguous()
        self.w_o = source.get(t["o"], device).contiguous()
        self.w_qnorm, self.w_cnorm = f32("dq_norm"), f32("dkv_norm")
        if self.has_sink:
            self.sink = f32("sink")
        self.position.prepare(device)
        enc = self.position.encoding()
        if enc is not None and not isinstance(enc, RotaryEncoding):
            raise TypeError(f"latent_attention: the position part '{self.position.spec.kind}' describes itself as "
                            f"{type(enc).__name__}; this mixer takes a rotation or none")
        self.rotary = enc
        if enc is not None and enc.inv_freq.numel() != self.r // 2:
            raise ValueError(f"latent_attention: the rotation turns {2 * enc.inv_freq.numel()} elements, the rotated "
                             f"part has {self.r}")

    def kv_requirement(self):
        return KVRequirement(1, self.row, "full", 0, streams=(("latent", 1, self.row),))

    def forward(self, h, residual, batch, cache, add=True):
        T, f32, dt = h.shape[0], torch.float32, h.dtype
        H, D, R, rank, row = self.nh, self.d, self.r, self.kv_rank, self.row
        pages, table, page_size = cache.stream("latent")
        inv_freq = None if self.rotary is None else self.rotary.inv_freq
        inter = self.rotary is not None and self.rotary.interleaved
        down = self.ws.get("latent_down", (T, self.q_rank + row), f32)
        with phase("qkv"):
            project(h, self.w_down, down)
        with phase("kv_store"):          # the normed latent and the rotated key part of every token go into its page
            K.latent_kv_write(down[:, self.q_rank:], self.w_cnorm, self.eps, inv_freq, inter, pages, table, page_size,
                              batch.token_seq, batch.token_pos, batch.seq_slot, rank=rank, rot=R)
        cq = self.ws.get("latent_cq", (T, self.q_rank), dt)
        with phase("rmsnorm"):
            K.rmsnorm(down[:, :self.q_rank], self.w_qnorm, self.eps, cq)
        q = self.ws.get("latent_q", (T, H * (D + R)), f32)
        with phase("qkv"):
            project(cq, self.w_uq, q)
        plain = self.ws.get("latent_q_plain", (H * T, D), dt)               # head-major rows
        full = self.ws.get("latent_q_full", (T, H * row), dt)
        offsets = self.ws.get("latent_offsets", (H + 1,), torch.int32)
        rows = self.ws.get("latent_rows", (H * T,), torch.int32)
        with phase("kv_store"):
            K.latent_q_split(q, inv_freq, inter, plain, full, offsets, rows, batch.token_pos, n_heads=H, dim=D, rot=R,
                             rank=rank)
        with phase("qkv"):               # the plain part of every query through its head's W_uk^T, into full[t, head, :rank]
            project(plain, self.w_ukT, full.view(T * H, row)[:, :rank], MODE_STORE, out_rows=rows, group_offsets=offsets,
                    n_groups=H, rows_per_group_hint=T)
        lat = self.ws.get("latent_att_heads", (H * T, rank), dt)            # head-major, the latent part only
        out = self.ws.get("latent_values", (T, H * self.dv), dt)
        if use_tensor_core_kernels() and dt == torch.bfloat16 and K.latent_attention_supported(row, rank):
            with phase("latent_attention"):
                if batch.is_decode:
                    # key splits from a bucketed bound of the context, so that a captured graph keeps its shape
                    groups = -(-H // 64)
                    tiles = -(-batch.ctx_bucket // K.LATENT_KEY_TILE)
                    n_splits = max(1, min(K.sm_count() // max(1, T * groups), tiles // 2,
                                          K.latent_attention_max_splits()))
                    K.latent_attention(full, lat, pages, table, page_size, batch.token_seq, batch.token_pos,
                                       batch.seq_slot, n_heads=H, rank=rank, scale=self.scale, sink=self.sink,
                                       n_splits=n_splits)
                else:
                    K.latent_attention(full, lat, pages, table, page_size, batch.token_seq, batch.token_pos,
                                       batch.seq_slot, n_heads=H, rank=rank, scale=self.scale, sink=self.sink,
                                       tile_tok0=batch.tile_tok0, tile_rows=batch.tile_rows)
        else:
            att = self.ws.get("latent_att", (T, H * row), dt)
            with phase("latent_attention"):
                attend(full, att, pages, pages, table, page_size, batch, n_heads=H, n_kv_heads=1, head_dim=row,
                       value_dim=row, window_kind="full", window_size=0, scale=self.scale, sink=self.sink)
            with phase("wo"):
                K.head_major_rows(att, lat, n_heads=H, n=rank)
        with phase("wo"):
            project(lat, self.w_uv, out.view(T * H, self.dv), MODE_STORE, out_rows=rows, group_offsets=offsets,
                    n_groups=H, rows_per_group_hint=T)
            project(out, self.w_o, residual, MODE_ADD if add else MODE_STORE)
