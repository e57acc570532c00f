"""Kikerax through the engine against the plain implementation (`plain_kikerax.py`): every mechanism alone, whole
prompts, portions, token-by-token decoding, unequal batches, reused slots and pages, the edges of chunks, far keys,
the first tokens of a sequence, long decoding, other sizes, generation through the entry point, and the replay tool."""
from __future__ import annotations

import copy
import json
import math
import os
import subprocess
import sys

import pytest
import torch

import kikerax_tiny as V
import plain_kikerax as P

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TOL = {"float32": 2e-4, "bfloat16": 3e-2}
F64 = torch.float64
DEV = "cuda"


def err(got, want, rms=False):
    """Difference of logit rows, mean taken off, relative to the spread of the expected row: the largest element of the
    worst row (float32), or with `rms` (bfloat16) a row's root mean square: what nine rows in ten stay under, and a
    quarter of the worst row but the worst in fifty.  A sublayer's output enters the residual through a norm, so where
    that output happens to be far smaller than usual, bfloat16 rounding of what came before is magnified by as much,
    and a router's near-tie may fall the other way; neither is a fault.  The float32 measure leaves out nothing."""
    d = got.double() - want.double()
    d = d - d.mean(-1, keepdim=True)
    w = want.double() - want.double().mean(-1, keepdim=True)
    size = (d.pow(2).mean(-1).sqrt() if rms else d.abs().max(-1).values) / w.pow(2).mean(-1).sqrt().clamp_min(1e-6)
    if rms:
        n = size.numel()
        drop = max(1, math.ceil(0.02 * n)) if n >= 5 else 0
        kept = size.sort().values[:n - drop]
        return max(torch.quantile(size, 0.9).item(), kept.max().item() / 4)
    return size.max().item()


class Built:
    def __init__(self, cfg, seed, tmp, change=None):
        self.cfg, self.W = cfg, V.draw_weights(cfg, seed)
        if change is not None:
            change(self.W)
        self.dir = V.write_model(cfg, self.W, root=str(tmp))
        self._plain = {}

    def plain(self, toks):
        key = tuple(toks)
        if key not in self._plain:
            self._plain[key] = P.forward(self.cfg, self.W, list(toks))
        return self._plain[key]

    def engine(self, dtype, **kw):
        from cpi_b200.engine import Engine
        kw.setdefault("max_tokens", 4096)
        return Engine.from_model_dir(self.dir, dtype=dtype, **kw)


class Run:
    """Feeds requests to an engine step by step and keeps the logits by (request, position).  In bfloat16 it also
    records the experts every token chose: a router's near-tie may fall the other way than in double precision, and
    because the cache and the recurrent state carry that token on, every later position would differ too.  The plain
    implementation is then run with the engine's choices, and the choices themselves are compared apart: all but a few
    must be the plain router's own.  In float32 nothing is recorded or forced."""

    def __init__(self, engine, record=True):
        self.e, self.slots, self.logits = engine, {}, {}
        self.routing = {}          # rid -> {layer: {position: [experts]}}
        # (while choices are recorded the engine replays no graphs: `record=False` for a test of those)
        self.cap = engine.capture_routing(True) if record and engine.dtype == torch.bfloat16 else None

    def step(self, items):
        from cpi_b200.engine import StepEntry
        entries, layout = [], []
        for rid, toks, want in items:
            if rid not in self.slots:
                self.slots[rid] = self.e.acquire_slot()
            start = self.e.length(self.slots[rid])
            entries.append(StepEntry(self.slots[rid], list(toks), list(want)))
            layout.append((rid, start, list(want), len(entries[-1].tokens)))
        for lst in (self.cap or {}).values():
            lst.clear()
        out = self.e.step(entries).float().cpu()
        self.e.check_device_errors()
        r = 0
        for rid, start, want, n in layout:
            for w in want:
                self.logits.setdefault(rid, {})[start + w] = out[r]
                r += 1
        for layer, lst in (self.cap or {}).items():       # a step that ran as pieces recorded one tensor per piece
            idx, t = torch.cat([x.cpu() for x in lst]), 0
            for rid, start, want, n in layout:
                for i in range(n):
                    self.routing.setdefault(rid, {}).setdefault(layer, {})[start + i] = sorted(idx[t + i].tolist())
                t += n

    def end(self, rid):
        self.e.release_slot(self.slots.pop(rid))

    def check(self, built, requests, tol):
        for rid, got in self.logits.items():
            toks = requests[rid]
            forced = {}
            for layer, by_pos in self.routing.get(rid, {}).items():
                n = max(by_pos) + 1
                assert sorted(by_pos) == list(range(n)), f"the choices of {rid} in layer {layer} have gaps"
                forced[layer] = [by_pos[p] for p in range(n)]
            if forced:
                n = min(len(v) for v in forced.values())
                own = {}
                ref = P.forward(built.cfg, built.W, list(toks[:n]), forced={l: v[:n] for l, v in forced.items()}, own_choices=own)
                other = sum(a != b for l in forced for a, b in zip(forced[l][:n], own[l]))
                assert other <= max(2, 0.04 * n * len(forced)), f"request {rid}: {other} choices of {n * len(forced)} differ"
            else:
                ref = built.plain(toks)
            pos = sorted(got)
            e = err(torch.stack([got[p] for p in pos]), ref[pos], rms=tol > 1e-3)
            assert e < tol, f"request {rid}: error {e:.3g} (tolerance {tol}) over positions {pos[0]}..{pos[-1]}"


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("kikerax")
    return {"A": Built(V.MIXED_A, 11, tmp), "B": Built(V.MIXED_B, 12, tmp), "C": Built(V.MIXED_C, 13, tmp)}


def K():
    from cpi_b200.csrc import lib
    return lib


class FakeBatch:
    """The index arrays a kernel reads of a step: sequences of `n_new` tokens that start at `starts`."""

    def __init__(self, slots, starts, n_new, dev=DEV):
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
        self.n_seqs, self.max_new = len(slots), max(n_new)
        self.seq_slot, self.seq_start, self.seq_new = i32(slots), i32(starts), i32(n_new)
        tok0, seq, pos, base = [], [], [], 0
        for s, (st, n) in enumerate(zip(starts, n_new)):
            tok0.append(base); seq += [s] * n; pos += range(st, st + n); base += n
        self.seq_tok0, self.token_seq, self.token_pos = i32(tok0), i32(seq), i32(pos)


def rn(g, *shape, std=1.0, mean=0.0):
    return torch.randn(*shape, generator=g) * std + mean


# ---- mechanisms alone ------------------------------------------------------------------------------------
def test_scaled_frequency_rule_and_amplitude():
    """Kept, stretched and blended pairs all occur, and the amplitude is the rule's."""
    from cpi_b200.parts.positions import yarn_frequencies
    for dims, base, sc in ((6, 300.0, (4.0, 64, 8.0, 1.0)), (12, 50.0, (8.0, 32, 4.0, 0.5)), (32, 2.5e5, (2.0, 128, 16.0, 2.0)),
                           (64, 1e4, (16.0, 4096, 32.0, 1.0)), (2, 10.0, (3.0, 16, 2.0, 1.0))):
        rot = {"base": base, "dims": dims, "scaling": dict(zip(("factor", "original", "fast", "slow"), sc))}
        want, amp = P.rotary_frequencies(rot)
        got, got_amp = yarn_frequencies(dims, base, {"factor": sc[0], "original_max_position_embeddings": sc[1],
                                                     "beta_fast": sc[2], "beta_slow": sc[3]})
        assert (torch.from_numpy(got).double() / want - 1).abs().max() < 1e-6 and abs(got_amp - amp) < 1e-12
        if dims == 64:
            plain = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F64)
            ratio = want / plain
            kept, slowed = (ratio - 1).abs() < 1e-12, (ratio - 1 / sc[0]).abs() < 1e-12
            assert kept.any() and slowed.any() and (~kept & ~slowed).any()
            assert abs(amp - (0.1 * math.log(16.0) + 1.0)) < 1e-12


@pytest.mark.parametrize("H,G,D,Dv,dims", [(6, 2, 10, 14, 6), (2, 2, 4, 20, 4), (4, 1, 32, 32, 8), (1, 1, 8, 8, 0)])
def test_preparation_of_two_score_maps(H, G, D, Dv, dims):
    """Rows [q | k | v] whose q and k hold two maps (all first maps, then all second maps) get their biases, a norm per
    head and map with one weight for all, a rotation of the first `dims` elements in pairs (2i, 2i + 1) with scaled
    frequencies and an amplitude; the maps go to buffers and cache streams of their own, the values to one."""
    g = torch.Generator().manual_seed(H * 10 + D)
    T, page, eps = 7, 64, 1e-5
    rows, bias = rn(g, T, 2 * (H + G) * D + G * Dv + 3, std=2.0), rn(g, 2 * (H + G) * D + G * Dv, std=0.5)
    qw, kw = rn(g, D, std=0.3, mean=1.0), rn(g, D, std=0.3, mean=1.0)
    rot = {"base": 300.0, "dims": dims, "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}} if dims else None
    f, amp = P.rotary_frequencies(rot) if dims else (None, 1.0)
    b = FakeBatch([0], [60], [T])                           # positions 60..66: the write crosses a page border
    table = torch.tensor([[3, 1]], dtype=torch.int32, device=DEV)
    kc, k2c = torch.zeros(4, G, page, D, device=DEV), torch.zeros(4, G, page, D, device=DEV)
    vc = torch.zeros(4, G, page, Dv, device=DEV)
    q, q2 = torch.empty(T, H * D, device=DEV), torch.empty(T, H * D, device=DEV)
    K().qkv_prepare(rows.to(DEV), q, kc, vc, table, page, b.token_seq, b.token_pos, b.seq_slot, n_heads=H, n_kv_heads=G,
                    head_dim=D, value_dim=Dv, bias=bias.to(DEV), q_norm=qw.to(DEV), k_norm=kw.to(DEV), head_norm=2,
                    norm_eps=eps, inv_freq=None if f is None else f.float().to(DEV), rotary_dims=dims, interleaved=True,
                    q2_out=q2, k2_cache=k2c, rotary_amplitude=amp)
    pos = torch.arange(60, 60 + T)
    x = (rows[:, :bias.numel()] + bias).double()
    nq, nk = 2 * H * D, 2 * G * D
    want_q = P.rotate(P.rms(x[:, :nq].view(T, 2 * H, D), eps) * qw.double(), pos, rot)
    want_k = P.rotate(P.rms(x[:, nq:nq + nk].view(T, 2 * G, D), eps) * kw.double(), pos, rot)
    assert (q.cpu().double().view(T, H, D) - want_q[:, :H]).abs().max() < 3e-5
    assert (q2.cpu().double().view(T, H, D) - want_q[:, H:]).abs().max() < 3e-5
    for t in range(T):
        p = 60 + t
        pg = int(table[0, p // page])
        assert (kc[pg, :, p % page].cpu().double() - want_k[t, :G]).abs().max() < 3e-5
        assert (k2c[pg, :, p % page].cpu().double() - want_k[t, G:]).abs().max() < 3e-5
        assert (vc[pg, :, p % page].cpu().double().reshape(-1) - x[t, nq + nk:]).abs().max() < 1e-6


@pytest.mark.parametrize("H,G,D,every", [(4, 1, 12, 3.0), (2, 2, 64, 64.0), (3, 3, 4, 1.0)])
def test_preparation_with_values_from_keys_and_temperature(H, G, D, every):
    """Rows [q | k | gates]: the cached values are the keys as projected, before their norm; q is multiplied by
    1 + c ln(floor((p + 1) / every) + 1) after its norm."""
    g = torch.Generator().manual_seed(D)
    T, page, eps, coef = 9, 64, 1e-6, 0.5
    rows = rn(g, T, (H + G) * D + H, std=2.0)
    qw, kw = rn(g, D, std=0.3, mean=1.0), rn(g, D, std=0.3, mean=1.0)
    b = FakeBatch([1], [59], [T])
    table = torch.tensor([[0, 0], [2, 3]], dtype=torch.int32, device=DEV)
    kc, vc = torch.zeros(4, G, page, D, device=DEV), torch.zeros(4, G, page, D, device=DEV)
    q = torch.empty(T, H * D, device=DEV)
    K().qkv_prepare(rows.to(DEV), q, kc, vc, table, page, b.token_seq, b.token_pos, b.seq_slot, n_heads=H, n_kv_heads=G,
                    head_dim=D, value_dim=D, q_norm=qw.to(DEV), k_norm=kw.to(DEV), head_norm=2, norm_eps=eps,
                    values_from_keys=True, temperature=(every, coef))
    pos = torch.arange(59, 59 + T, dtype=F64)
    temp = 1.0 + coef * torch.log(torch.floor((pos + 1.0) / every) + 1.0)
    x = rows.double()
    want_q = P.rms(x[:, :H * D].view(T, H, D), eps) * qw.double() * temp[:, None, None]
    want_k = P.rms(x[:, H * D:(H + G) * D].view(T, G, D), eps) * kw.double()
    assert (q.cpu().double().view(T, H, D) - want_q).abs().max() < 3e-5
    for t in range(T):
        p = 59 + t
        pg = int(table[1, p // page])
        assert (kc[pg, :, p % page].cpu().double() - want_k[t]).abs().max() < 3e-5
        assert torch.equal(vc[pg, :, p % page].cpu().reshape(-1), rows[t, H * D:(H + G) * D])


@pytest.mark.parametrize("cap", [0.0, 2.0, 30.0])
def test_soft_capped_scores_in_the_general_attention_kernel(cap):
    g = torch.Generator().manual_seed(3)
    T, H, G, D, Dv, page = 70, 4, 2, 12, 10, 64
    q, k, v = rn(g, T, H, D, std=1.5), rn(g, T, G, D, std=1.5), rn(g, T, G, Dv)
    kc, vc = torch.zeros(3, G, page, D, device=DEV), torch.zeros(3, G, page, Dv, device=DEV)
    table = torch.tensor([[2, 0]], dtype=torch.int32, device=DEV)
    for t in range(T):
        kc[int(table[0, t // page]), :, t % page] = k[t].to(DEV)
        vc[int(table[0, t // page]), :, t % page] = v[t].to(DEV)
    b = FakeBatch([0], [0], [T])
    out = torch.empty(T, H * Dv, device=DEV)
    K().attention_general(q.reshape(T, H * D).to(DEV).contiguous(), out, kc, vc, table, page, b.token_seq, b.token_pos,
                          b.seq_slot, n_heads=H, n_kv_heads=G, head_dim=D, window_kind=0, window_size=0, scale=0.7,
                          value_dim=Dv, softcap=cap)
    want = P.softmax_attention(q.double(), k.double(), v.double(), 0.7, P.visible(T, None), cap or None)
    assert (out.cpu().double().view(T, H, Dv) - want).abs().max() < 2e-5
    if cap == 2.0:
        assert (want - P.softmax_attention(q.double(), k.double(), v.double(), 0.7, P.visible(T, None))).abs().max() > 1e-2


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_what_follows_attention_per_head(dt):
    """o = a1 - lambda a2, normed over the head's values without a weight, times a constant, times the head's gate."""
    g = torch.Generator().manual_seed(8)
    T, H, Dv, lam, eps, c = 11, 3, 14, 0.63, 1e-5, 0.6
    a1, a2 = rn(g, T, H * Dv).to(dt), rn(g, T, H * Dv).to(dt)
    gate = rn(g, T, H + 5, std=2.0)
    sg = torch.sigmoid(gate[:, 5:].double())[:, :, None]
    want = P.rms((a1.double() - lam * a2.double()).view(T, H, Dv), eps) * c * sg
    out = torch.empty(T, H * Dv, dtype=dt, device=DEV)
    K().head_post(a1.to(DEV), out, n_heads=H, value_dim=Dv, a2=a2.to(DEV), lam=lam, norm_eps=eps, norm_scale=c,
                  gate=gate.to(DEV)[:, 5:])
    tol = 2e-5 if dt == torch.float32 else 1e-2
    assert (out.cpu().double().view(T, H, Dv) - want).abs().max() < tol * want.abs().max()
    buf = a1.to(DEV).clone()                                  # the gate alone, in place
    K().head_post(buf, buf, n_heads=H, value_dim=Dv, gate=gate.to(DEV)[:, 5:])
    assert (buf.cpu().double().view(T, H, Dv) - a1.double().view(T, H, Dv) * sg).abs().max() < tol * 4


def _unit_weights(g, W, C, B, taps):
    n = C // B
    w = {"y": rn(g, C, W, std=W ** -0.5), "y.b": rn(g, C, std=0.3), "x": rn(g, C, W, std=W ** -0.5), "x.b": rn(g, C, std=0.3),
         "conv": rn(g, C, taps, std=0.5, mean=0.3), "conv.b": rn(g, C, std=0.2), "ra": rn(g, B, n, n, std=1.5 * n ** -0.5),
         "ra.b": rn(g, B, n, std=0.5), "ri": rn(g, B, n, n, std=1.5 * n ** -0.5), "ri.b": rn(g, B, n, std=0.5),
         "lam": rn(g, C, std=1.5, mean=-2.0), "o": rn(g, W, C, std=C ** -0.5)}
    return {"p." + k: v.to(torch.bfloat16) for k, v in w.items()}


@pytest.mark.parametrize("W,C,B,taps,dtype", [(24, 36, 3, 3, "float32"), (40, 16, 1, 1, "float32"), (64, 128, 2, 4, "bfloat16"),
                                              (128, 256, 8, 2, "bfloat16"), (52, 30, 5, 8, "bfloat16")])
def test_recurrent_unit_part_whole_in_pieces_beside_another_and_in_a_reused_slot(W, C, B, taps, dtype):
    """The part as the model runs it: a sequence of 300 tokens in one step (the recurrence cut into runs), in pieces
    down to one token and shorter than the convolution, sharing its first step with another sequence, in a slot whose
    states another sequence left and that was zeroed on acquisition."""
    from cpi_b200.config.spec import PartSpec
    from cpi_b200.parts.base import build_part
    from cpi_b200.parts.workspace import Workspace
    from cpi_b200.weights.store import DictSource
    dt = getattr(torch, dtype)
    g = torch.Generator().manual_seed(W + C)
    Wt = _unit_weights(g, W, C, B, taps)
    names = {k: "p." + v for k, v in {"y": "y", "y_bias": "y.b", "x": "x", "x_bias": "x.b", "conv": "conv", "conv_bias": "conv.b",
                                      "ra": "ra", "ra_bias": "ra.b", "ri": "ri", "ri_bias": "ri.b", "lam": "lam", "o": "o"}.items()}
    part = build_part("mixer", PartSpec("rglru", {"hidden_size": W, "width": C, "blocks": B, "conv": taps,
                                                  "tensor_names": names}), "", workspace=Workspace(torch.device(DEV)))
    part.load(DictSource(Wt), torch.device(DEV))
    T = 300
    h, h2 = rn(g, T, W).to(dt), rn(g, 9, W).to(dt)
    m = {"width": C, "blocks": B, "conv": taps}
    want, want2 = P.recurrent_block(h.double(), Wt, "p.", m), P.recurrent_block(h2.double(), Wt, "p.", m)
    tol = 3e-5 if dtype == "float32" else 2e-2

    class Cache:
        def __init__(self):
            self.s = {"s": torch.randn(4, C, device=DEV), "conv": torch.randn(4, max(taps - 1, 0), C, device=DEV)}
            for t in self.s.values():
                t[0].zero_(); t[2].zero_()                    # slots are zeroed when they are acquired

        def state(self, name):
            return self.s[name]

    for cuts in ([T], [1, 2, 1, 3, 40, 253], [150, 1, 1, 148]):
        cache, out, at = Cache(), torch.empty(T, W, device=DEV), 0
        for i, n in enumerate(cuts):
            if i == 0:
                b = FakeBatch([0, 2], [0, 0], [9, n])
                b.dtype = dt
                o = torch.zeros(9 + n, W, device=DEV)
                part.forward(torch.cat([h2, h[:n]]).to(DEV), o, b, cache, add=False)
                assert (o[:9].cpu().double() - want2).abs().max() < tol * want2.abs().max()
                out[:n] = o[9:]
            else:
                b = FakeBatch([2], [at], [n])
                b.dtype = dt
                part.forward(h[at:at + n].to(DEV), out[at:at + n], b, cache, add=False)
            at += n
        assert (out.cpu().double() - want).abs().max() < tol * want.abs().max(), cuts[:3]


def test_recurrence_keeps_a_token_for_hundreds_of_steps():
    """Decays close to one: what the first token writes is still most of the state 400 tokens later (a lost or reset
    state shows), and decays close to zero forget at once; sqrt(1 - a^2) keeps its digits either way."""
    g = torch.Generator().manual_seed(1)
    T, C = 400, 32
    gates = torch.cat([rn(g, T, C, std=0.3), rn(g, T, C, std=0.3)], dim=1)
    u, y = rn(g, T, C), rn(g, T, C)
    u[1:] *= 0.01
    lam = torch.cat([torch.full((C // 2,), -9.0), torch.full((C // 2,), 3.0)])
    r, i = torch.sigmoid(gates[:, :C].double()), torch.sigmoid(gates[:, C:].double())
    a = torch.exp(-8.0 * r * P.softplus(lam.double()))
    S, want = torch.zeros(C, dtype=F64), torch.zeros(T, C, dtype=F64)
    for t in range(T):
        S = a[t] * S + torch.sqrt(1 - a[t] * a[t]) * i[t] * u[t].double()
        want[t] = S * P.gelu_tanh(y[t].double())
    kept = a[1:].prod(0)                    # the share of the first token's write that is still there at the end
    assert (kept[:C // 2] > 0.5).all() and (kept[C // 2:] < 1e-30).all()
    for cuts in ([T], [1] * 40 + [360]):
        state, out, at = torch.zeros(2, C, device=DEV), torch.empty(T, C, device=DEV), 0
        for n in cuts:
            b = FakeBatch([1], [at], [n])
            K().rglru_scan(gates[at:at + n].to(DEV).contiguous(), u[at:at + n].to(DEV), y[at:at + n].to(DEV), state,
                           out[at:at + n], b, block=C, lam=lam.to(DEV))
            at += n
        assert (out.cpu().double() - want).abs().max() < 1e-5 * want.abs().max()
        assert (state[1].cpu().double() - S).abs().max() < 1e-5 * S.abs().max() and state[0].abs().max() == 0


@pytest.mark.parametrize("E,top,groups,keep,T", [(6, 2, 3, 2, 40), (16, 4, 4, 2, 300), (8, 3, 2, 1, 5), (5, 5, 1, 1, 9),
                                                 (3, 1, 1, 1, 70), (12, 2, 6, 1, 33), (64, 6, 8, 3, 20)])
def test_choice_of_experts_from_the_best_groups(E, top, groups, keep, T):
    """Scores sigmoid(z); the choice on score + correction inside the kept groups (a group's score: its two largest
    choice scores); weights from the scores without the correction, normed and scaled.  Corrections are drawn so
    that they change both the groups kept and the experts chosen, and so that choice scores are negative."""
    g = torch.Generator().manual_seed(E * 7 + top)
    z, corr, scale = rn(g, T, E, std=2.0), rn(g, E, std=0.6, mean=-0.8), 2.5
    idx = torch.empty(T, top, dtype=torch.int32, device=DEV)
    gate = torch.empty(T, top, device=DEV)
    K().router_select(z.to(DEV), idx, gate, top_k=top, sigmoid_gate="sigmoid_normed",
                      rule={"choice_bias": corr.to(DEV), "groups": groups, "keep": keep, "scale": scale})
    r = {"experts": E, "top": top, "scale": scale, "groups": {"count": groups, "keep": keep}}
    moved = 0
    for t in range(T):
        wi, ww = P.router_choice(z[t].double(), corr.double(), r)
        assert sorted(idx[t].tolist()) == sorted(wi.tolist()), t
        order = {e: k for k, e in enumerate(idx[t].tolist())}
        got = torch.tensor([gate[t, order[e]].item() for e in wi.tolist()], dtype=F64)
        assert (got - ww).abs().max() < 1e-5 * scale
        plain_top = torch.topk(z[t], top).indices.tolist()
        moved += sorted(plain_top) != sorted(wi.tolist())
    if E > top:
        assert moved > 0


@pytest.mark.parametrize("T,W,n,dt", [(5, 52, 2, torch.bfloat16), (3, 40, 1, torch.float32), (70, 256, 4, torch.bfloat16),
                                      (4, 37, 3, torch.bfloat16), (2, 8200, 2, torch.float32)])
def test_norm_of_a_weighted_sum_enters_the_residual(T, W, n, dt):
    g = torch.Generator().manual_seed(T)
    ys, sc = [rn(g, T, W, std=2.0) for _ in range(n)], [0.6, 1.3, -0.4, 2.0][:n]
    x, w = rn(g, T, W), rn(g, W, std=0.2, mean=0.8).to(torch.bfloat16)
    total = sum(s * y.double() for s, y in zip(sc, ys))
    want = x.double() + P.rms(total, 1e-5) * w.double()
    buf, h = x.to(DEV).clone(), torch.empty(T, W, dtype=dt, device=DEV)
    K().sum_norm_add([y.to(DEV) for y in ys], sc, w.to(DEV), buf, eps=1e-5, add=True, h_out=h)
    assert (buf.cpu().double() - want).abs().max() < 2e-5 * want.abs().max()
    assert torch.equal(h.cpu(), buf.cpu().to(dt))
    K().sum_norm_add([y.to(DEV) for y in ys], sc, None, buf, add=False, normalise=False)
    assert (buf.cpu().double() - total).abs().max() < 2e-5 * total.abs().max()
    bias = rn(g, W).to(torch.bfloat16)
    K().bias_rows(buf, bias.to(DEV))
    assert torch.equal(buf.cpu(), bias.float().expand(T, W))


@pytest.mark.parametrize("T,I,H,dtype", [(5, 44, 52, torch.float32), (40, 200, 136, torch.bfloat16),
                                         (600, 256, 128, torch.bfloat16), (8, 512, 4096, torch.bfloat16)])
def test_gelu_feed_forward_part(T, I, H, dtype):
    """down(gelu(up h)) on the float32 pipe, the tensor-core kernel (also with the contraction split over blocks: the
    activation acts on the whole sum) and the paired one."""
    from cpi_b200.config.spec import PartSpec
    from cpi_b200.parts.base import build_part
    from cpi_b200.parts.workspace import Workspace
    from cpi_b200.weights.store import DictSource
    g = torch.Generator().manual_seed(T)
    Wt = {"p.up": rn(g, I, H, std=1.5 * H ** -0.5).to(torch.bfloat16), "p.down": rn(g, H, I, std=I ** -0.5).to(torch.bfloat16)}
    h, res = rn(g, T, H).to(dtype), rn(g, T, H)
    part = build_part("feed_forward", PartSpec("dense_mlp", {"hidden_size": H, "intermediate_size": I, "activation": "gelu_tanh",
                                                             "tensor_names": {"up": "p.up", "down": "p.down"}}), "",
                      workspace=Workspace(torch.device(DEV)))
    part.load(DictSource(Wt), torch.device(DEV))
    buf = res.to(DEV).clone()

    class B:
        pass
    part.forward(h.to(DEV), buf, B())
    want = res.double() + P.dense_ff(h.double(), Wt, "p.")
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    assert (buf.cpu().double() - want).abs().max() < tol * want.abs().max()


# ---- the model -------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_whole_prompts_and_token_by_token(models, name, dtype):
    """A prompt in one step with logits everywhere, and the same tokens one by one from the first: both are the plain
    implementation's, which knows no cache and no state."""
    b = models[name]
    toks = V.tokens(150, b.cfg["vocab"], 5)
    r = Run(b.engine(dtype))
    r.step([("whole", toks, range(len(toks)))])
    r.end("whole")
    for i, t in enumerate(toks[:90]):
        r.step([("single", [t], [0])])
    r.check(b, {"whole": toks, "single": toks}, TOL[dtype])


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_portions_of_several_sizes(models, name):
    """A prompt cut into portions of 2, 3, 64, 1, 17, ... tokens, with cuts inside pages and chunks and portions shorter
    than the convolution; in float32 the logits are also those of the single step, to rounding."""
    b = models[name]
    toks = V.tokens(200, b.cfg["vocab"], 6)
    for dtype in ("float32", "bfloat16"):
        e = b.engine(dtype)
        r = Run(e)
        at = 0
        for n in (2, 3, 64, 1, 17, 2, 70, 5, 36):
            r.step([("p", toks[at:at + n], range(n))])
            at += n
        assert at == 200
        r.check(b, {"p": toks}, TOL[dtype])
        if dtype == "float32":
            one = Run(e)
            one.step([("w", toks, range(200))])
            d = err(torch.stack([r.logits["p"][i] for i in range(200)]), torch.stack([one.logits["w"][i] for i in range(200)]))
            assert d < 5e-5, d


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_unequal_batches_in_reused_slots(models, name, dtype):
    """Requests of 1 to 140 tokens start together, are decoded together, end at different steps; a second group then
    runs in the slots and pages the first gave back.  Every logit is the request's own: nothing of a slot's earlier
    recurrent state, convolution inputs or pages shows."""
    b = models[name]
    vocab = b.cfg["vocab"]
    reqs = {f"r{i}": V.tokens(n, vocab, 60 + i) for i, n in enumerate((1, 75, 130, 9, 66, 140))}
    e = b.engine(dtype, max_seqs=3, max_tokens=640)
    r = Run(e)
    for group in (("r0", "r1", "r2"), ("r3", "r4", "r5")):
        head = {i: max(1, len(reqs[i]) - 20) for i in group}
        r.step([(i, reqs[i][:head[i]], [0, head[i] - 1]) for i in group])
        live, k = [i for i in group if head[i] < len(reqs[i])], 0
        for i in group:
            if i not in live:
                r.end(i)
        while live:
            r.step([(i, [reqs[i][head[i] + k]], [0]) for i in live])
            k += 1
            for i in [i for i in live if head[i] + k == len(reqs[i])]:
                r.end(i)
                live.remove(i)
        e.cache.check_consistency()
    assert e.cache.free_slots == 3 and all(g.pages_held() == 0 for g in e.cache.groups)
    r.check(b, reqs, TOL[dtype])


@pytest.mark.parametrize("name", ["A", "B"])
def test_steps_larger_than_the_engine_takes_run_as_pieces(models, name):
    b = models[name]
    vocab = b.cfg["vocab"]
    reqs = {"x": V.tokens(123, vocab, 80), "y": V.tokens(8, vocab, 81), "z": V.tokens(66, vocab, 82)}
    for dtype in ("float32", "bfloat16"):
        r = Run(b.engine(dtype, max_step_tokens=50, max_seqs=3, max_tokens=512))
        r.step([("x", reqs["x"][:120], range(0, 120, 7)), ("y", reqs["y"][:7], [0, 6]), ("z", reqs["z"][:64], [1, 49, 50, 63])])
        r.step([("x", reqs["x"][120:121], [0]), ("y", reqs["y"][7:8], [0]), ("z", reqs["z"][64:65], [0])])
        r.end("y")
        r.step([("x", reqs["x"][121:123], [0, 1]), ("z", reqs["z"][65:66], [0])])
        r.check(b, reqs, TOL[dtype])


def _stand_out(W, pre, tokens, D):
    """Makes the keys of `tokens` stand out for every query that may see them.  Every token's embedding gets the same
    large element 1 and a small element 0, those of `tokens` a large element 0; the last row of every q head (and map) reads element
    1, the last row of every k head element 0, and the biases go.  After the per-head norm a query is then mostly its
    last element whatever its token, a key only when its token is one of `tokens` (the last element of a head is outside the
    rotated part in the configurations that use this)."""
    W["embed"][:, 0] = 0.05
    W["embed"][:, 1] = 3.0
    for token in tokens:
        W["embed"][token, 0] = 6.0
    for name, col in (("q", 1), ("k", 0)):
        w = W[pre + name].float()
        for r in range(D - 1, w.shape[0], D):
            w[r] = 0.0
            w[r, col] = 4.0
        W[pre + name] = w.to(torch.bfloat16)
        if pre + name + ".b" in W:
            W[pre + name + ".b"] = W[pre + name + ".b"] * 0


def test_chunk_edges_through_the_model(tmp_path):
    """One layer of two maps, one head: the keys at positions 0, 62 .. 65, 127 and 128 stand out.  A query in the same
    chunk gives such a key most of its weight, the first query of the next chunk cannot see it; in a prompt and token by
    token, with the chunk's edge on a page border, before it and after it, and for a chunk of one."""
    special = (7, 9, 11, 13, 15, 17, 19)
    toks = [t if t not in special else 8 for t in V.tokens(150, 50, 9)]
    for p, t in zip((0, 62, 63, 64, 65, 127, 128), special):
        toks[p] = t
    last = []
    for chunk in (64, 63, 65, 1, 128, None):
        cfg = V.model([V.layer(V.differential(1, 1, 16, 16, chunk=chunk, rot_dims=4, scale=1.0), None)], width=24, vocab=50)
        b = Built(cfg, 31, tmp_path, lambda W: _stand_out(W, "l0.mix.", special, 16))
        for dtype in ("float32", "bfloat16"):
            r = Run(b.engine(dtype))
            r.step([("x", toks[:126], range(126))])
            for i in range(126, 150):
                r.step([("x", toks[i:i + 1], [0])])
            r.check(b, {"x": toks}, TOL[dtype])
        last.append(b.plain(toks)[64:])
    for i in range(1, len(last)):                           # the variants do differ where the edge moved
        assert (last[i] - last[0]).abs().max() > 1e-3, i


def test_a_far_token_among_hundreds_and_long_decoding(models):
    """700 tokens: the pairs' left sides read every position back to the first across many pages, the recurrent state
    is carried through 120 decoded tokens past chunk edges and a page border."""
    b = models["A"]
    toks = V.tokens(700, b.cfg["vocab"], 17)
    for dtype in ("float32", "bfloat16"):
        e = b.engine(dtype, max_tokens=1024, max_seqs=2)
        r = Run(e)
        r.step([("far", toks[:580], [0, 1, 300, 579])])
        for i in range(580, 700):
            r.step([("far", toks[i:i + 1], [0])])
        r.check(b, {"far": toks}, TOL[dtype])


def test_one_position_that_stands_out_for_a_left_side(tmp_path):
    """A pair whose left side's queries and keys are dominated by one direction in which a token that occurs once, at
    position 2, is large: every later query gives that position most of its weight (under a soft cap that still lets it
    through), also hundreds of positions and several pages later; leaving it out would change every logit after it."""
    cfg = V.model([V.layer(V.pair(2, 1, 8, 16, 2, 2, softcap=12.0, q_temp=(0.3, 50), scale=1.0), V.dense(24))], width=32, vocab=40)
    b = Built(cfg, 3, tmp_path, lambda W: _stand_out(W, "l0.mix.left.", (7,), 8))
    toks = [t if t != 7 else 8 for t in V.tokens(330, 40, 1)]
    toks[2] = 7
    with_far = b.plain(toks)
    other = list(toks)
    other[2] = 9
    assert (b.plain(other)[300:] - with_far[300:]).abs().max() > 1e-2      # the far token does matter to late rows
    for dtype in ("float32", "bfloat16"):
        r = Run(b.engine(dtype, max_tokens=512, max_seqs=2))
        r.step([("x", toks[:290], [0, 1, 2, 3, 63, 64, 65, 128, 289])])
        for i in range(290, 330):
            r.step([("x", toks[i:i + 1], [0])])
        r.check(b, {"x": toks}, TOL[dtype])


def test_soft_cap_on_the_tensor_core_attention_kernels(tmp_path):
    """Left sides with heads of 64 and of 128 under a tight and a loose soft cap: in bfloat16 these run on the
    tensor-core attention kernels (a prompt of several query tiles, portions, decoding with key splits), and the result
    is that of the general kernel and of the plain implementation; without the cap it would be another."""
    from cpi_b200.parts import attention as A
    cfg = V.model([V.layer(V.pair(4, 2, 64, 64, 2, 2, softcap=3.0, scale=0.5), V.dense(64)),
                   V.layer(V.pair(2, 1, 128, 32, 1, 3, softcap=25.0, q_temp=(0.3, 100), scale=0.3), None)], width=128, vocab=60)
    b = Built(cfg, 5, tmp_path)
    toks = V.tokens(400, 60, 3)
    no_cap = copy.deepcopy(cfg)
    for L in no_cap["layers"]:
        L["mixer"]["left"].pop("softcap")
    assert (P.forward(no_cap, b.W, toks[:50]) - b.plain(toks[:50])).abs().max() > 1e-2
    logits = {}
    for tc in (True, False):
        A.use_tensor_core_kernels = tc
        try:
            r = Run(b.engine("bfloat16", max_tokens=1024, max_seqs=2), record=False)
            r.step([("x", toks[:300], range(0, 300, 7))])
            r.step([("x", toks[300:360], range(60))])
            for i in range(360, 400):
                r.step([("x", toks[i:i + 1], [0])])
            r.check(b, {"x": toks}, TOL["bfloat16"])
            logits[tc] = r.logits["x"]
        finally:
            A.use_tensor_core_kernels = True
    pos = sorted(logits[True])
    assert err(torch.stack([logits[True][p] for p in pos]), torch.stack([logits[False][p] for p in pos]), rms=True) < TOL["bfloat16"]


def test_other_constants_change_the_result_as_the_plain_implementation_says(tmp_path):
    base = V.model([V.layer(V.differential(4, 2, 8, 12, diff=0.4, chunk=9, rot_dims=4, base=100.0, scaling=(4.0, 16, 4.0, 0.5)),
                            V.moe(8, 2, 12, groups=(4, 2), shared=10)),
                    V.layer(V.pair(2, 1, 8, 24, 3, 3, softcap=3.0, q_temp=(0.5, 4)), V.dense(24)),
                    V.layer(V.differential(2, 2, 16, 12, diff=0.6, chunk=30, rot_dims=16), V.dense(16))],
                   width=32, vocab=70, logit_softcap=5.0)
    att, par, ff = (lambda c, i=0: c["layers"][i]["mixer"]), (lambda c: c["layers"][1]["mixer"]), (lambda c: c["layers"][0]["mlp"])
    changes = {
        "base": lambda c: None,
        "eps": lambda c: c["norm"].update(eps=1e-2),
        "no_logit_cap": lambda c: c.pop("logit_softcap"), "logit_cap": lambda c: c.update(logit_softcap=2.0),
        "factor": lambda c: att(c)["rot"]["scaling"].update(factor=1.0),
        "no_scaling": lambda c: att(c)["rot"].pop("scaling"),
        "original": lambda c: att(c)["rot"]["scaling"].update(original=64),
        "fast": lambda c: att(c)["rot"]["scaling"].update(fast=0.1),
        "rot_base": lambda c: att(c)["rot"].update(base=1000.0), "rot_dims": lambda c: att(c)["rot"].update(dims=8),
        "no_rot": lambda c: att(c, 2).pop("rot"),
        "scale": lambda c: att(c).update(scale=0.4), "chunk": lambda c: att(c)["mask"].update(size=8),
        "no_mask": lambda c: att(c).pop("mask"), "diff": lambda c: att(c).update(diff=0.1),
        "kv_heads": lambda c: att(c).update(kv_heads=4),
        "softcap": lambda c: par(c)["left"].update(softcap=30.0), "no_softcap": lambda c: par(c)["left"].pop("softcap"),
        "temp": lambda c: par(c)["left"]["q_temp"].update(every=5), "coef": lambda c: par(c)["left"]["q_temp"].update(coef=0.1),
        "no_temp": lambda c: par(c)["left"].pop("q_temp"), "left_scale": lambda c: par(c).update(left_scale=0.2),
        "right_scale": lambda c: par(c).update(right_scale=0.3), "left_attn_scale": lambda c: par(c)["left"].update(scale=0.1),
        "taps": lambda c: par(c)["right"].update(conv=2), "blocks": lambda c: par(c)["right"].update(blocks=2),
        "top": lambda c: ff(c)["router"].update(top=3), "keep": lambda c: ff(c)["router"]["groups"].update(keep=1),
        "groups": lambda c: ff(c)["router"]["groups"].update(count=2, keep=1),
        "no_groups": lambda c: ff(c)["router"].pop("groups"), "router_scale": lambda c: ff(c)["router"].update(scale=0.5),
        "no_shared": lambda c: ff(c).pop("shared"),
        "no_mlp": lambda c: c["layers"][0].update(mlp=None), "ff": lambda c: c["layers"][1]["mlp"].update(ff=9),
        "order": lambda c: c["layers"].reverse(),
    }
    toks = V.tokens(40, 70, 2)
    seen = {}
    for key, change in changes.items():
        cfg = copy.deepcopy(base)
        change(cfg)
        b = Built(cfg, 21, tmp_path)
        r = Run(b.engine("float32"))
        r.step([("x", toks[:25], range(25))])
        for i in range(25, 40):
            r.step([("x", toks[i:i + 1], [0])])
        r.check(b, {"x": toks}, TOL["float32"])
        seen[key] = b.plain(toks)
    for key in changes:
        if key not in ("base", "kv_heads", "blocks", "taps", "ff", "order", "factor"):
            assert (seen[key] - seen["base"]).abs().max() > 1e-3, key      # same weights, other constant


@pytest.mark.parametrize("seed", [1, 2, 3, 4, 5, 6, 7, 8, 9, 10])
def test_configurations_drawn_from_a_seed(seed, tmp_path):
    """Every size, option and constant drawn from a seed: a prompt with logits everywhere, a second request in a
    portion and then both decoded together, in float32 to rounding and in bfloat16."""
    cfg = V.draw_config(seed)
    b = Built(cfg, 40 + seed, tmp_path)
    vocab = cfg["vocab"]
    ta, tb = V.tokens(110, vocab, seed), V.tokens(75, vocab, seed + 100)
    for dtype in ("float32", "bfloat16"):
        r = Run(b.engine(dtype, max_tokens=1024, max_seqs=2))
        r.step([("a", ta[:90], range(90)), ("b", tb[:3], range(3))])
        r.step([("b", tb[3:70], range(67))])
        for i in range(5):
            r.step([("a", ta[90 + i:91 + i], [0]), ("b", tb[70 + i:71 + i], [0])])
        r.end("b")
        for i in range(95, 110):
            r.step([("a", ta[i:i + 1], [0])])
        r.check(b, {"a": ta, "b": tb}, TOL[dtype])


def test_layers_recorded_one_by_one(models):
    """The residual after every layer is the plain implementation's."""
    b = models["A"]
    toks = V.tokens(30, b.cfg["vocab"], 4)
    want = []
    P.forward(b.cfg, b.W, toks, want)
    for dtype, tol in (("float32", 2e-4), ("bfloat16", 5e-2)):
        e = b.engine(dtype)
        e.model.layer_capture = []
        Run(e).step([("x", toks, [29])])
        assert len(e.model.layer_capture) == len(want) == 4
        for got, w in zip(e.model.layer_capture, want):
            assert (got.cpu().double() - w).abs().max() < tol * w.abs().max()


def test_greedy_generation_through_the_entry_point(models):
    """`Model.generate` (scheduler, sampler, decode graphs) picks the plain implementation's tokens: unequal prompts,
    more requests than slots."""
    from cpi_b200.api import Model
    b = models["A"]
    vocab = b.cfg["vocab"]
    prompts = [V.tokens(n, vocab, 30 + n) for n in (5, 33, 1, 70, 12)]
    m = Model.load(b.dir, dtype="float32", max_batch=2, max_context=128)
    results = m.generate(prompts, max_new=12, temperature=0.0)
    for p, res in zip(prompts, results):
        seq = list(p)
        for tok in res.tokens:
            ref = b.plain(seq)[-1]
            best = int(ref.argmax())
            if tok != best:            # a near-tie may fall either way; anything else is a fault
                assert (ref[best] - ref[tok]).item() < 1e-3 * ref.abs().max().item(), (len(p), len(seq))
            seq.append(tok)
        assert len(res.tokens) == 12


def test_decode_steps_replayed_as_graphs_are_the_eager_ones(models):
    """Every part of the model says it is safe to capture; replayed decode steps give the eager steps' logits."""
    b = models["B"]
    toks = V.tokens(60, b.cfg["vocab"], 77)
    e = b.engine("bfloat16", max_seqs=2, max_tokens=256)
    assert e.use_graphs
    r = Run(e, record=False)
    r.step([("g", toks[:40], [39])])
    for i in range(40, 60):
        r.step([("g", toks[i:i + 1], [0])])
    assert e.graph_kernel_launches > 0
    e2 = b.engine("bfloat16", max_seqs=2, max_tokens=256)
    e2.use_graphs = False
    r2 = Run(e2, record=False)
    r2.step([("g", toks[:40], [39])])
    for i in range(40, 60):
        r2.step([("g", toks[i:i + 1], [0])])
    for p in range(39, 60):
        assert torch.equal(r.logits["g"][p], r2.logits["g"][p]), p


def test_random_weights_mode_and_command_line(models):
    """A folder drawn by the library's random mode loads and generates; bin/llama_infer knows the family by its
    config.json and its greedy tokens are the plain implementation's."""
    from cpi_b200.engine import Engine
    e = Engine.from_random(V.MIXED_B, seed=3, dtype="bfloat16", max_tokens=512)
    out = Run(e)
    out.step([("x", V.tokens(70, 384, 1), [69])])
    assert torch.isfinite(out.logits["x"][69]).all()
    b = models["C"]
    prompt = V.tokens(9, b.cfg["vocab"], 50)
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "llama_infer"), b.dir, "--tokens",
                        ",".join(map(str, prompt)), "--max-new", "6", "--temp", "0", "--dtype", "float32",
                        "--benchmark-phases", "--max-context", "64"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    line = next(l for l in r.stdout.splitlines() if l.startswith("Output tokens:"))
    got = [int(x) for x in line.split(":")[1].split()]
    assert got[:9] == prompt and len(got) == 15
    seq = list(prompt)
    for tok in got[9:]:
        ref = b.plain(seq)[-1]
        best = int(ref.argmax())
        assert tok == best or (ref[best] - ref[tok]).item() < 1e-3 * ref.abs().max().item()
        seq.append(tok)
    assert "Kikerax" in r.stdout and "attention" in r.stdout


def test_replay_tool_runs_a_kikerax_folder(models, tmp_path):
    """bin/trace_run in a process of its own: a request whole, and two requests batched then decoded."""
    import numpy as np
    b = models["B"]
    vocab = b.cfg["vocab"]
    ta, tb = V.tokens(80, vocab, 40), V.tokens(21, vocab, 41)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": ta, "want": list(range(80))}], "end": ["a"]},
             {"step": 1, "entries": [{"id": "b", "tokens": tb[:20], "want": []},
                                     {"id": "a2", "tokens": ta[:70], "want": [69]}], "end": []},
             {"step": 2, "entries": [{"id": "b", "tokens": tb[20:], "want": [0]},
                                     {"id": "a2", "tokens": ta[70:71], "want": [0]}], "end": ["b"]},
             {"step": 3, "entries": [{"id": "a2", "tokens": ta[71:72], "want": [0]}], "end": ["a2"]}]
    for dtype in ("float32", "bfloat16"):
        out = tmp_path / f"out_{dtype}"
        p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", b.dir, "--dtype", dtype,
                            "--out", str(out), "--max-tokens", "256"], input="\n".join(json.dumps(s) for s in steps),
                           capture_output=True, text=True, timeout=600)
        assert p.returncode == 0, p.stderr[-2000:]
        assert [l for l in p.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(4)]
        rd = lambda i: torch.from_numpy(np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, vocab).copy())
        ra, rb = b.plain(ta), b.plain(tb)
        got = torch.cat([rd(i) for i in range(4)])
        want = torch.cat([ra, torch.stack([ra[69], rb[20], ra[70], ra[71]])])
        assert got.shape == want.shape and err(got, want, dtype == "bfloat16") < TOL[dtype]
