"""Nogapel through the engine against the plain implementation (`plain_nogapel.py`): every mechanism alone, whole
prompts, portions, token-by-token decoding, unequal batches, reused slots and pages, the edges of windows, far keys,
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

import nogapel_tiny as V
import plain_nogapel as P

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TOL = {"float32": 2e-4, "bfloat16": 3e-2}
F64 = torch.float64
DEV = "cuda"


def err(got, want, rms=False):
    """Difference of logit rows, mean taken off, relative to the spread of the expected row: the largest element of the
    worst row (float32), or with `rms` (bfloat16) a row's root mean square: what nine rows in ten stay under, and a
    quarter of the worst row.  The per-token input enters the residual through a norm, so at a position where the gated
    vector happens to be hundreds of times smaller than usual, bfloat16 rounding of the layers before is magnified by as
    much, which is no fault: of five rows or more, the worst one in fifty (at least one) is left out of the second
    measure.  The float32 measure leaves out nothing."""
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
    """Feeds requests to an engine step by step and keeps the logits by (request, position)."""

    def __init__(self, engine):
        self.e, self.slots, self.logits = engine, {}, {}

    def step(self, items):
        from cpi_b200.engine import StepEntry
        entries, layout = [], []
        for rid, toks, want in items:
            if rid not in self.slots:
                self.slots[rid] = self.e.acquire_slot()
            start = self.e.length(self.slots[rid])
            entries.append(StepEntry(self.slots[rid], list(toks), list(want)))
            layout.append((rid, start, list(want)))
        out = self.e.step(entries).float().cpu()
        self.e.check_device_errors()
        r = 0
        for rid, start, want in layout:
            for w in want:
                self.logits.setdefault(rid, {})[start + w] = out[r]
                r += 1

    def end(self, rid):
        self.e.release_slot(self.slots.pop(rid))

    def check(self, built, requests, tol):
        for rid, got in self.logits.items():
            ref = built.plain(requests[rid])
            pos = sorted(got)
            e = err(torch.stack([got[p] for p in pos]), ref[pos], rms=tol > 1e-3)
            assert e < tol, f"request {rid}: error {e:.3g} (tolerance {tol}) over positions {pos[0]}..{pos[-1]}"


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("nogapel")
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
def test_frequency_rule_three_branches():
    """The scaled frequencies are the plain rule's: kept, divided, and blended ones all occur."""
    from cpi_b200.parts.positions import llama3_frequencies_f64
    for dims, base, sc in ((8, 200.0, (8.0, 1.0, 4.0, 64)), (40, 50.0, (0.5, 2.0, 3.0, 16)), (64, 2.5e5, (4.0, 1.0, 8.0, 256)),
                           (6, 300.0, None)):
        rot = {"base": base, "dims": dims}
        scaling = None
        if sc is not None:
            rot["scaling"] = dict(zip(("factor", "low", "high", "original"), sc))
            scaling = {"factor": sc[0], "low_freq_factor": sc[1], "high_freq_factor": sc[2],
                       "original_max_position_embeddings": sc[3]}
        want = P.frequencies(rot)
        got = torch.from_numpy(llama3_frequencies_f64(dims, base, scaling)).double()
        assert (got / want - 1).abs().max() < 1e-6
        if dims == 64:
            plain = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F64)
            ratio = want / plain
            kept, slowed = (ratio - 1).abs() < 1e-12, (ratio - 1 / sc[0]).abs() < 1e-12
            assert kept.any() and slowed.any() and (~kept & ~slowed).any()


@pytest.mark.parametrize("taps,C", [(1, 20), (2, 7), (4, 96), (5, 33), (8, 130)])
def test_short_convolution_whole_in_pieces_and_in_a_reused_slot(taps, C):
    """y_t = sum_j w[:, j] u_(t - taps + 1 + j) without activation or bias: a sequence in one launch, in pieces down
    to one token (pieces shorter than the taps), beside another sequence, in a slot whose state another left."""
    g = torch.Generator().manual_seed(taps * 100 + C)
    T = 23
    u, u2, w = rn(g, T, C), rn(g, 9, C), rn(g, C, taps, std=0.5, mean=0.3)
    want, want2 = P.short_conv(u.double(), w.double()), P.short_conv(u2.double(), w.double())
    for cuts in ([T], [1, 2, 1, 3, 16], [1] * T):
        carry = torch.randn(4, max(taps - 1, 0), C, device=DEV)           # what a finished sequence left behind
        carry[2].zero_()
        carry[0].zero_()                                                  # a slot is zeroed when it is acquired
        out = torch.empty(T, C, device=DEV)
        at = 0
        for i, n in enumerate(cuts):
            if i == 0:                                                    # the first piece shares its step with another
                b = FakeBatch([0, 2], [0, 0], [9, n])
                x = torch.cat([u2, u[:n]]).to(DEV)
                o = torch.empty(9 + n, C, device=DEV)
                K().causal_conv(x, w.to(DEV), None, carry, o, b, silu=False)
                assert (o[:9].cpu().double() - want2).abs().max() < 1e-5
                out[:n] = o[9:]
            else:
                b = FakeBatch([2], [at], [n])
                K().causal_conv(u[at:at + n].to(DEV), w.to(DEV), None, carry, out[at:at + n], b, silu=False)
            at += n
        assert (out.cpu().double() - want).abs().max() < 1e-5, cuts[:3]
        if taps > 1:
            assert torch.equal(carry[2].cpu(), u[T - taps + 1:])


@pytest.mark.parametrize("H,G,D,Dv,dims,mode", [(4, 2, 12, 10, 8, 2), (2, 2, 20, 10, 20, 1), (3, 1, 32, 48, 32, 2),
                                                (1, 1, 6, 20, 0, 0), (4, 2, 8, 8, 2, 1)])
def test_preparation_shared_norm_weight_interleaved_rotation_and_value_mixing(H, G, D, Dv, dims, mode):
    """Rows [q | k | v]: every q and k head normed with one weight [D] for all heads, then its first `dims` elements
    turned as pairs (2i, 2i + 1); values stored for later layers (mode 1) or mixed with stored ones (mode 2)."""
    g = torch.Generator().manual_seed(H * 10 + D)
    T, page, eps = 7, 64, 1e-5
    rows = rn(g, T, (H + G) * D + G * Dv, std=2.0)
    qw, kw = rn(g, D, std=0.3, mean=1.0), rn(g, D, std=0.3, mean=1.0)
    rot = {"base": 300.0, "dims": dims, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 32}}
    f = P.frequencies(rot).float() if dims else None
    lam, vf = torch.tensor([0.3]), rn(g, T, G * Dv)
    b = FakeBatch([0], [60], [T])                           # positions 60..66: the write crosses a page border
    table = torch.tensor([[3, 1]], dtype=torch.int32, device=DEV)
    kc, vc = torch.zeros(4, G, page, D, device=DEV), torch.zeros(4, G, page, Dv, device=DEV)
    q = torch.empty(T, H * D, device=DEV)
    v_first = vf.to(DEV).clone() if mode == 2 else (torch.zeros(T, G * Dv, device=DEV) if mode == 1 else None)
    K().qkv_prepare(rows.to(DEV), q, kc, vc, table, page, b.token_seq, b.token_pos, b.seq_slot, n_heads=H, n_kv_heads=G,
                    head_dim=D, value_dim=Dv, q_norm=qw.to(DEV), k_norm=kw.to(DEV), head_norm=2, norm_eps=eps,
                    inv_freq=None if f is None else f.to(DEV), rotary_dims=dims, interleaved=True, v_first=v_first,
                    v_mix=lam.to(DEV) if mode == 2 else None, v_mix_mode=mode)
    pos = torch.arange(60, 60 + T)
    want_q = P.rms_norm(rows[:, :H * D].double().view(T, H, D), qw.double(), eps)
    want_k = P.rms_norm(rows[:, H * D:(H + G) * D].double().view(T, G, D), kw.double(), eps)
    if dims:
        want_q, want_k = P.rotate_interleaved(want_q, pos, rot), P.rotate_interleaved(want_k, pos, rot)
    want_v = rows[:, (H + G) * D:].double()
    if mode == 2:
        want_v = 0.7 * want_v + 0.3 * vf.double()
    assert (q.cpu().double().view(T, H, D) - want_q).abs().max() < 2e-5
    for t in range(T):
        p = 60 + t
        pg = int(table[0, p // page])
        assert (kc[pg, :, p % page].cpu().double() - want_k[t]).abs().max() < 2e-5
        assert (vc[pg, :, p % page].cpu().double().reshape(-1) - want_v[t]).abs().max() < 1e-6
    if mode == 1:
        assert torch.equal(v_first.cpu(), rows[:, (H + G) * D:])


def test_latent_rows_queries_and_head_major_kernels():
    """What a position keeps: the normed latent and the rotated key part, written to its page; a query's plain parts
    head by head and its rotated parts placed behind the latent's columns; rows regrouped head by head."""
    g = torch.Generator().manual_seed(5)
    T, H, D, R, rank, page, eps = 6, 3, 10, 6, 14, 64, 1e-5
    rot = {"base": 300.0, "dims": R}
    f = P.frequencies(rot).float().to(DEV)
    x, w = rn(g, T, 5 + rank + R, std=2.0), rn(g, rank, std=0.3, mean=1.0)
    b = FakeBatch([1], [62], [T])
    table = torch.tensor([[0, 0], [2, 3]], dtype=torch.int32, device=DEV)
    cache = torch.zeros(4, 1, page, rank + R, device=DEV)
    K().latent_kv_write(x.to(DEV)[:, 5:], w.to(DEV), eps, f, True, cache, table, page, b.token_seq, b.token_pos, b.seq_slot,
                        rank=rank, rot=R)
    pos = torch.arange(62, 62 + T)
    want_c = P.rms_norm(x[:, 5:5 + rank].double(), w.double(), eps)
    want_r = P.rotate_interleaved(x[:, 5 + rank:].double().view(T, 1, R), pos, rot).view(T, R)
    for t in range(T):
        p = 62 + t
        row = cache[int(table[1, p // page]), 0, p % page].cpu().double()
        assert (row[:rank] - want_c[t]).abs().max() < 2e-5 and (row[rank:] - want_r[t]).abs().max() < 2e-5
    q = rn(g, T, H * (D + R))
    plain, full = torch.empty(H * T, D, device=DEV), torch.zeros(T, H * (rank + R), device=DEV)
    offsets, rows = torch.empty(H + 1, dtype=torch.int32, device=DEV), torch.empty(H * T, dtype=torch.int32, device=DEV)
    K().latent_q_split(q.to(DEV), f, True, plain, full, offsets, rows, b.token_pos, n_heads=H, dim=D, rot=R, rank=rank)
    qh = q.view(T, H, D + R)
    want_rot = P.rotate_interleaved(qh[..., D:].double(), pos, rot)
    assert torch.equal(plain.cpu().view(H, T, D), qh[..., :D].transpose(0, 1))
    assert (full.cpu().double().view(T, H, rank + R)[..., rank:] - want_rot).abs().max() < 2e-5
    assert full.view(T, H, rank + R)[..., :rank].abs().max() == 0
    assert offsets.tolist() == [h * T for h in range(H + 1)]
    assert rows.tolist() == [t * H + h for h in range(H) for t in range(T)]
    y = rn(g, T, H * (rank + R)).to(DEV)
    out = torch.empty(H * T, rank, device=DEV)
    K().head_major_rows(y, out, n_heads=H, n=rank)
    assert torch.equal(out.view(H, T, rank), y.view(T, H, rank + R)[..., :rank].transpose(0, 1))


@pytest.mark.parametrize("T,W,n,off,wdt", [(5, 52, 6, 12, torch.bfloat16), (3, 40, 1, 0, torch.float32),
                                           (70, 256, 40, 80, torch.bfloat16), (2, 24, 16, 16, torch.bfloat16)])
def test_gated_token_input_kernel(T, W, n, off, wdt):
    g = torch.Generator().manual_seed(T + W)
    vocab = 30
    x = rn(g, T, W, std=3.0)
    table = rn(g, vocab, off + n + 3).to(wdt)
    gate, proj = rn(g, n, W, std=1.5 * W ** -0.5).to(wdt), rn(g, W, n, std=n ** -0.5).to(wdt)
    nw = rn(g, W, std=0.3, mean=0.8)
    toks = torch.randint(0, vocab, (T,), generator=g)
    e = table[toks][:, off:off + n].double()
    y = (P.gelu_tanh(x.double() @ gate.double().T) * e) @ proj.double().T
    want = x.double() + P.rms_norm(y, nw.double(), 1e-5)
    buf = x.to(DEV).clone()
    K().gated_side_input(buf, toks.to(torch.int32).to(DEV), table.to(DEV), off, gate.to(DEV), proj.to(DEV), nw.to(DEV), 1e-5)
    assert (buf.cpu().double() - want).abs().max() < 2e-5 * want.abs().max()
    if off % n == 0:                               # the plain function's slicing by layer says the same
        layer = off // n
        pw = {"side.embed": table.double(), "p.gate": gate.double(), "p.proj": proj.double(), "p.norm": nw.double()}
        assert (P.token_side_input(x.double(), toks, pw, "p.", layer, n, 1e-5) - want).abs().max() < 1e-9


@pytest.mark.parametrize("T,W,n,layer,dtype", [(5, 52, 6, 2, "bfloat16"), (600, 256, 64, 1, "bfloat16"),
                                               (9, 128, 16, 0, "bfloat16"), (4, 40, 3, 1, "float32")])
def test_gated_token_input_part_in_both_precisions(T, W, n, layer, dtype):
    """The junction as the model runs it: float32 in one kernel, bfloat16 with its two products as matrix products
    (few and many tokens, sizes the tensor-core kernels take and sizes they do not); two parts share one table."""
    from cpi_b200.config.spec import PartSpec
    from cpi_b200.parts.base import build_part
    from cpi_b200.parts.workspace import Workspace
    from cpi_b200.weights.store import DictSource
    dt = getattr(torch, dtype)
    g = torch.Generator().manual_seed(T * W)
    vocab, n_layers = 30, 3
    x = rn(g, T, W, std=2.0)
    table = rn(g, vocab, n_layers * n).bfloat16()
    gate, proj = rn(g, n, W, std=1.5 * W ** -0.5).bfloat16(), rn(g, W, n, std=n ** -0.5).bfloat16()
    nw = rn(g, W, std=0.3, mean=0.8).bfloat16()
    toks = torch.randint(0, vocab, (T,), generator=g)
    src = DictSource({"side.embed": table, "p.gate": gate, "p.proj": proj, "p.norm": nw,
                      "o.gate": gate, "o.proj": proj, "o.norm": nw})
    ws = Workspace(torch.device(DEV))
    spec = {"hidden_size": W, "vocab_size": vocab, "dim": n, "table": "side.embed", "table_width": n_layers * n,
            "offset": layer * n, "gate": "p.gate", "proj": "p.proj", "norm": "p.norm", "eps": 1e-5}
    part = build_part("junction", PartSpec("token_gated_input", spec), "", workspace=ws)
    other = build_part("junction", PartSpec("token_gated_input", {**spec, "offset": 0, "gate": "o.gate", "proj": "o.proj",
                                                                  "norm": "o.norm"}), "", workspace=ws)
    part.load(src, torch.device(DEV))
    other.load(src, torch.device(DEV))
    assert part.table.data_ptr() == other.table.data_ptr()

    class B:
        tokens = toks.to(torch.int32).to(DEV)
    B.dtype = dt
    buf = x.to(DEV).clone()
    part.run(buf, None, B)
    pw = {"side.embed": table.double(), "p.gate": gate.double(), "p.proj": proj.double(), "p.norm": nw.double()}
    want = P.token_side_input(x.double(), toks, pw, "p.", layer, n, 1e-5)
    tol = 2e-5 if dtype == "float32" else 2e-2
    assert (buf.cpu().double() - want).abs().max() < tol * want.abs().max()


@pytest.mark.parametrize("T,I,H,dtype", [(5, 44, 52, torch.float32), (40, 200, 136, torch.bfloat16),
                                         (600, 256, 128, torch.bfloat16), (7, 96, 64, torch.bfloat16),
                                         (8, 512, 4096, torch.bfloat16), (1, 1024, 2048, torch.bfloat16)])
def test_squared_relu_feed_forward_part(T, I, H, dtype):
    """down(max(up h, 0)^2) added to the residual, on the float32 pipe, the tensor-core kernel (also with the
    contraction split over blocks: the activation acts on the whole sum) and the paired one."""
    from cpi_b200.config.spec import PartSpec
    from cpi_b200.parts.base import build_part
    from cpi_b200.parts.workspace import Workspace
    from cpi_b200.weights.store import DictSource
    g = torch.Generator().manual_seed(T)
    up, down = rn(g, I, H, std=1.5 * H ** -0.5).to(torch.bfloat16), rn(g, H, I, std=I ** -0.5).to(torch.bfloat16)
    h, res = rn(g, T, H).to(dtype), rn(g, T, H)
    ff = build_part("feed_forward", PartSpec("dense_mlp", {"hidden_size": H, "intermediate_size": I,
                                                           "activation": "relu_squared"}), prefix="x.",
                    workspace=Workspace(torch.device(DEV)))
    ff.load(DictSource({"x.feed_forward.up_proj.weight": up, "x.feed_forward.down_proj.weight": down}), torch.device(DEV))
    out = res.to(DEV).clone()
    ff.forward(h.to(DEV), out, None)
    want = res.double() + P.dense_feed_forward(h.double(), {"up": up.double(), "down": down.double()}, "")
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert (out.cpu().double() - want).abs().max() < tol * want.abs().max()


def test_window_edge_in_the_attention_kernel_with_values_of_another_size():
    """One key is made to carry the row: the output is that key's value exactly when the window lets it through -- the
    oldest key of the window and the one before it, the token itself, a window of one, across a page border, in a
    portion and for a single token."""
    D, Dv, page, n_pos = 12, 20, 64, 200
    kc, vc = torch.zeros(8, 1, page, D, device=DEV), torch.zeros(8, 1, page, Dv, device=DEV)
    table = torch.tensor([[5, 2, 7, 1, 0, 0, 0, 0]], dtype=torch.int32, device=DEV)
    pos_of = lambda p: (int(table[0, p // page]), p % page)
    for p in range(n_pos):
        pg, off = pos_of(p)
        kc[pg, 0, off, 1 + p % (D - 1)] = 1.0               # orthogonal to the query direction (element 0)
        vc[pg, 0, off] = float(p + 1)
    for window, target, qpos, seen in ((10, 181, 190, True), (10, 180, 190, False), (64, 64, 127, True), (64, 63, 127, False),
                                       (65, 63, 127, True), (1, 150, 150, True), (1, 149, 150, False), (130, 0, 129, True),
                                       (130, 0, 130, False), (3, 190, 190, True)):
        pg, off = pos_of(target)
        old = kc[pg, 0, off].clone()
        kc[pg, 0, off] = 0
        kc[pg, 0, off, 0] = 1.0
        for n_q in (1, 3):
            first = qpos - n_q + 1
            q = torch.zeros(n_q, D, device=DEV)
            q[:, 0] = 40.0
            b = FakeBatch([0], [first], [n_q])
            out = torch.empty(n_q, Dv, device=DEV)
            K().attention_general(q, out, kc, vc, table, page, b.token_seq, b.token_pos, b.seq_slot, n_heads=1,
                                  n_kv_heads=1, head_dim=D, window_kind=K().WINDOW_KINDS["sliding"], window_size=window,
                                  scale=1.0, value_dim=Dv)
            got = out[-1, 0].item()
            if seen:
                assert abs(got - (target + 1)) < 1e-3, (window, target, qpos, got)
            else:                                           # every visible key scores zero: the mean of their values
                vis = [p for p in range(max(0, qpos - window + 1), qpos + 1)]
                assert target not in vis and abs(got - sum(p + 1 for p in vis) / len(vis)) < 1e-2, (window, target, got)
        kc[pg, 0, off] = old


@pytest.mark.parametrize("row,heads,dtype", [(24, 3, torch.float32), (128, 4, torch.bfloat16), (64, 8, torch.bfloat16),
                                             (576, 2, torch.float32), (200, 5, torch.bfloat16)])
def test_a_far_row_and_the_sink_in_attention_over_shared_rows(row, heads, dtype):
    """All heads read one cached row per position (keys and values are the same rows): a row hundreds of positions
    back carries the softmax of one head; a sink as large as that score takes half of the weight and adds nothing."""
    page, n_pos, far = 64, 700, 3
    cache = torch.zeros(16, 1, page, row, dtype=dtype, device=DEV)
    table = torch.tensor([[0] * 12, [9, 4, 11, 2, 15, 7, 1, 8, 3, 13, 6, 0]], dtype=torch.int32, device=DEV)
    g = torch.Generator().manual_seed(row)
    rows = rn(g, n_pos, row, std=0.5)
    rows[:, 0] = 0
    rows[far, 0] = 1.0
    for p in range(n_pos):
        cache[int(table[1, p // page]), 0, p % page] = rows[p].to(dtype)
    q = torch.zeros(2, heads * row, dtype=dtype, device=DEV)
    q.view(2, heads, row)[:, 1, 0] = 30.0                   # head 1 looks for the far row; the others see a flat row
    sink = torch.full((heads,), -30.0, device=DEV)
    sink[1] = 30.0
    for n_q in (1, 2):
        b = FakeBatch([1], [n_pos - n_q], [n_q])
        out = torch.empty(n_q, heads * row, dtype=dtype, device=DEV)
        for use_sink in (False, True):
            from cpi_b200.parts.attention import attend
            class B:                                        # what `attend` reads of a step
                is_decode, n_tokens, ctx_bucket, n_q_tiles = n_q == 1, n_q, 1024, 0
                token_seq, token_pos, seq_slot = b.token_seq, b.token_pos, b.seq_slot
            attend(q[:n_q].contiguous(), out, cache, cache, table, page, B, n_heads=heads, n_kv_heads=1, head_dim=row,
                   value_dim=row, window_kind="full", window_size=0, scale=1.0, sink=sink if use_sink else None)
            got = out.float().cpu().view(n_q, heads, row)[-1]
            want = rows[far].to(dtype).float() * (0.5 if use_sink else 1.0)
            assert (got[1] - want).abs().max() < 2e-2, (n_q, use_sink)
            flat = rows.to(dtype).float().mean(0)
            assert (got[0] - flat).abs().max() < 2e-2


@pytest.mark.parametrize("H,row,rank", [(6, 128, 96), (16, 576, 512), (80, 48, 32), (5, 208, 192), (3, 16, 16),
                                        (4, 160, 128), (2, 256, 256), (7, 80, 48), (20, 64, 48), (40, 32, 16)])
def test_tensor_core_attention_over_shared_rows_against_plain_softmax(H, row, rank):
    """The kernel that stacks the heads of a few tokens into one tile, against softmax in float64 over the same
    rounded rows: sequences that start at zero and in the middle, at page and key-tile borders, in scattered pages; one
    token per sequence with the keys undivided and divided over blocks; with and without a sink; more heads than a tile
    has rows."""
    lib = K()
    assert lib.latent_attention_supported(row, rank)
    page, n_pages = 16, 64
    g = torch.Generator().manual_seed(H * row)
    perm = torch.randperm(n_pages, generator=g)
    table = torch.stack([perm[:20], perm[20:40], perm[40:60]]).to(torch.int32).to(DEV)       # slots 0, 1, 2
    lens = [257, 96, 320]
    seqs = [rn(g, n, row, std=0.7).bfloat16() for n in lens]
    cache = torch.full((n_pages, 1, page, row), float("nan"), dtype=torch.bfloat16, device=DEV)
    for s, rows in enumerate(seqs):
        for pos in range(rows.shape[0]):
            cache[int(table[s, pos // page]), 0, pos % page] = rows[pos]
    scale = 1.7 / row ** 0.5
    sink = rn(g, H).to(DEV)

    def want(q, slots, starts, n_new, snk):
        out, t = torch.zeros(H * q.shape[0], rank, dtype=F64), 0
        for s, st, n in zip(slots, starts, n_new):
            for i in range(n):
                keys = seqs[s][:st + i + 1].double()
                sc = q[t].double().view(H, row) @ keys.T * scale
                if snk is not None:
                    sc = torch.cat([sc, snk.double().cpu()[:, None]], 1)
                w = torch.softmax(sc, -1)[:, :keys.shape[0]]
                out[torch.arange(H) * q.shape[0] + t] = w @ keys[:, :rank]
                t += 1
        return out

    cases = [([0, 1, 2], [0, 33, 63], [250, 40, 1], None),          # runs: from zero, from the middle, a single token
             ([2, 0], [200, 31], [120, 2], None),
             ([0, 1, 2], [256, 0, 319], [1, 1, 1], 1),              # one token each, keys undivided
             ([0, 1, 2], [128, 95, 300], [1, 1, 1], 4),             # keys over four blocks (some get nothing)
             ([1], [31], [1], 7)]
    for slots, starts, n_new, splits in cases:
        b = FakeBatch(slots, starts, n_new)
        T = sum(n_new)
        q = rn(g, T, H * row).bfloat16()
        for snk in (None, sink):
            out = torch.full((H * T, rank), float("nan"), dtype=torch.bfloat16, device=DEV)
            kw = {}
            if splits is None:
                kw = {"tile_tok0": b.seq_tok0, "tile_rows": b.seq_new}
            else:
                kw = {"n_splits": splits}
            lib.latent_attention(q.to(DEV), out, cache, table, page, b.token_seq, b.token_pos, b.seq_slot, n_heads=H,
                                 rank=rank, scale=scale, sink=snk, **kw)
            ref = want(q, slots, starts, n_new, snk)
            assert (out.double().cpu() - ref).abs().max() < 2e-2, (slots, starts, n_new, splits, snk is not None)


# ---- the model -------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_whole_prompts_and_token_by_token(models, name, dtype):
    """A prompt in one step with logits everywhere, and the same tokens one by one from the first: both are the plain
    implementation's, which knows no cache."""
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
    """A prompt cut into portions of 2, 3, 64, 1, 17, ... tokens, with cuts inside pages and windows and portions
    shorter than the convolutions; in float32 the logits are also those of the single step, to rounding."""
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
            assert d < 2e-5, d


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_unequal_batches_in_reused_slots(models, name, dtype):
    """Requests of 1 to 140 tokens start together, are decoded together, end at different steps; a second group then
    runs in the slots and pages the first gave back.  Every logit is the request's own: nothing of a slot's earlier
    convolution state or pages shows."""
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
    """An engine that takes 50 tokens a step gets a step of 191 tokens: it runs as pieces against the cache, the
    convolution state and the stored first values that the pieces before left; same logits."""
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


def test_window_edges_through_the_model(tmp_path):
    """One attention layer, one head: moving the window by one changes the logits as the plain implementation says,
    in a prompt and token by token, with the edge on a page border, at it and beside it, and for a window of one."""
    toks = V.tokens(150, 50, 9)
    last = []
    for window in (64, 63, 65, 1, 128, None):
        cfg = V.model([V.layer(V.attention(1, 1, 16, 16, window=window, conv=2, rot_dims=16, scale=2.0), None)],
                      width=24, vocab=50)
        b = Built(cfg, 31, tmp_path)
        r = Run(b.engine("float32"))
        r.step([("x", toks[:126], range(126))])
        for i in range(126, 150):
            r.step([("x", toks[i:i + 1], [0])])
        r.check(b, {"x": toks}, TOL["float32"])
        last.append(b.plain(toks)[64:])
    for i in range(1, len(last)):                           # the variants do differ where the edge moved
        assert (last[i] - last[0]).abs().max() > 1e-3, i


def test_a_far_token_among_hundreds_and_long_decoding(models):
    """700 tokens: the latent layers read every position back to the first across many pages while the windowed
    layers give pages back; 120 tokens are decoded past several windows and a page border.  Then the same with
    one latent layer whose first position is made to stand out for every later query."""
    b = models["A"]
    toks = V.tokens(700, b.cfg["vocab"], 17)
    for dtype in ("float32", "bfloat16"):
        e = b.engine(dtype, max_tokens=1024, max_seqs=2)
        r = Run(e)
        r.step([("far", toks[:580], [0, 1, 300, 579])])
        for i in range(580, 700):
            r.step([("far", toks[i:i + 1], [0])])
        r.check(b, {"far": toks}, TOL[dtype])


def test_one_position_that_stands_out_for_a_latent_layer(tmp_path):
    """A latent layer whose queries and keys are dominated by the rotated part at frequency ~0 of a token that occurs
    once, at position 2: every later query gives that position most of its weight; leaving it out (or reading a
    neighbour) would change every logit after it."""
    cfg = V.model([V.layer(V.latent(2, 8, 4, 8, 6, 10, base=1e8, scale=1.0), 24)], width=32, vocab=40)

    def change(W):
        W["embed"][7] = W["embed"][7] * 0 + torch.linspace(-3, 3, 32).to(torch.bfloat16)
        # the shared rotated key part's last pair turns by position * 1e-4: nearly fixed; make token 7 large there
        W["l0.mix.dkv"][10 + 2] = (W["embed"][7].float() * 0.6).to(torch.bfloat16)
        W["l0.mix.sink"][:] = 0.0

    b = Built(cfg, 3, tmp_path, change)
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


def test_other_constants_change_the_result_as_the_plain_implementation_says(tmp_path):
    base = V.model([V.layer(V.attention(4, 2, 8, 12, window=9, conv=3, v_mix=True, rot_dims=4, base=100.0,
                                        scaling=(4.0, 1.0, 2.0, 16)), 40),
                    V.layer(V.latent(2, 8, 4, 6, 10, 12, base=100.0, scaling=(2.0, 1.0, 4.0, 32)), 24),
                    V.layer(V.attention(2, 2, 16, 12, window=30, conv=2, v_mix=True, rot_dims=16), 16)],
                   width=32, vocab=70, side=4)
    att, lat = (lambda c, i=0: c["layers"][i]["mixer"]), (lambda c: c["layers"][1]["mixer"])
    changes = {
        "base": lambda c: None,
        "eps": lambda c: c["norm"].update(eps=1e-2),
        "no_side": lambda c: c.pop("token_side"), "side": lambda c: c["token_side"].update(dim=7),
        "factor": lambda c: att(c)["rot"]["scaling"].update(factor=1.0),
        "no_scaling": lambda c: att(c)["rot"].pop("scaling"),
        "low": lambda c: att(c)["rot"]["scaling"].update(original=64),
        "rot_base": lambda c: att(c)["rot"].update(base=1000.0), "rot_dims": lambda c: att(c)["rot"].update(dims=8),
        "no_rot": lambda c: att(c, 2).pop("rot"),
        "scale": lambda c: att(c).update(scale=0.4), "window": lambda c: att(c)["mask"].update(size=8),
        "no_mask": lambda c: att(c).pop("mask"), "taps": lambda c: att(c).update(conv=4),
        "no_conv": lambda c: att(c, 2).pop("conv"),
        "no_mix": lambda c: (att(c).pop("v_mix"), att(c, 2).pop("v_mix")),
        "one_mix": lambda c: att(c).pop("v_mix"),
        "groups": lambda c: (att(c).update(kv_heads=4), att(c, 2).update(heads=4, kv_heads=4, vdim=12)),
        "lat_scale": lambda c: lat(c).update(scale=0.2), "lat_base": lambda c: lat(c)["rot"].update(base=10.0),
        "lat_scaling": lambda c: lat(c)["rot"].pop("scaling"),
        "lat_rank": lambda c: lat(c).update(kv_rank=5, q_rank=3), "lat_heads": lambda c: lat(c).update(heads=3, vdim=10),
        "lat_rot": lambda c: (lat(c).update(rot_dim=8), lat(c)["rot"].update(dims=8)),
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
    assert torch.equal(seen["factor"], seen["no_scaling"])
    for key in changes:
        if key not in ("base", "side", "groups", "lat_rank", "lat_heads", "lat_rot", "ff", "order", "no_side", "taps"):
            assert (seen[key] - seen["base"]).abs().max() > 1e-3, key      # same weights, other constant


@pytest.mark.parametrize("seed", [1, 2, 3, 4, 5, 6, 7, 8])
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
    """The residual after every layer (after its token input) is the plain implementation's."""
    b = models["A"]
    toks = V.tokens(30, b.cfg["vocab"], 4)
    want = []
    P.forward(b.cfg, b.W, toks, want)
    e = b.engine("float32")
    e.model.layer_capture = []
    Run(e).step([("x", toks, [29])])
    assert len(e.model.layer_capture) == len(want) == 6
    for got, w in zip(e.model.layer_capture, want):
        assert (got.cpu().double() - w).abs().max() < 2e-4 * w.abs().max()


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
    assert "Nogapel" in r.stdout and "attention" in r.stdout


def test_replay_tool_runs_a_nogapel_folder(models, tmp_path):
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
