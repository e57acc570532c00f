"""Arrangements of a layer's parts.

"pre_norm": x += mixer(norm1(x)); x += ffn(norm2(x))  (the order of src/engine/llama4_cpu_engine.cpp:300-329).

"parallel_residual": h = norm1(x); x += mixer(h) + ffn(h).  One norm, and both sublayers read its output; each adds
its result into the float32 residual.

"hyper_connections": the residual is S streams x_1 .. x_S (float32 [S, T, H], all equal to the embedding output
at the start; the final norm reads their sum).  Sublayer q (1: mixer, 2: feed-forward) reads a mixture of the
streams and writes to all of them:
    u = sum_s read_q[s] x_s;   y = sublayer_q(norm_q(u));   x_t <- sum_s mix_q[s, t] x_s + write_q[t] y
(every x_t from the old streams; mix indexed [from, to]).  One kernel per boundary applies the write-back of the
sublayer before and forms and normalises the next u; the write-back of a layer's last sublayer is left pending in
the workspace and done by the next layer's first kernel (or by `Workspace.settle()` when something else reads the
residual first), so a layer costs as many of these launches as it has sublayers.  A layer without a feed-forward
has the first sublayer only.

"post_norm": x += norm1(mixer(x)); x += norm2(ffn(x)).  The sublayers read the residual itself (in the activation
dtype); the norm acts on a sublayer's output, with the layer's norm weights.  One kernel per sublayer norms the output,
adds it into the float32 residual and writes the next sublayer's input; the copy a layer's last sublayer leaves is the
next layer's input when that layer is of this kind too.  A mixer that is a weighted sum of branches hands its branches
over (`branch_outputs`), so that the sum, the norm and the addition are one pass.

"scaled_pre_norm": x += m * mixer(norm1(x)); x += m * ffn(norm2(x)) with one constant m (`residual_scale`).  It is the
arrangement above with a single stream and constant coefficients (read 1, mix 1, write m), so the scaled addition of a
sublayer's output rides on the kernel that forms the next sublayer's normed input.
"""
from __future__ import annotations

import torch

from ..csrc import lib as K
from ..phases import phase
from ..weights.store import TensorReq
from .base import Block, register_block
from .linear import single_cta_products


@register_block("pre_norm")
class PreNormBlock(Block):
    graph_safe = True
    def __init__(self, spec, prefix="", **_):
        super().__init__(spec, prefix)

    def run(self, layer, residual, batch, cache):
        layer.mixer_norm.ws.settle()        # a block of another kind may have left its last write-back pending
        with phase("rmsnorm"):
            h = layer.mixer_norm(residual, batch.dtype)
        layer.mixer.forward(h, residual, batch, cache)
        if layer.feed_forward is None:
            return
        with phase("rmsnorm"):
            h2 = layer.feed_forward_norm(residual, batch.dtype)
        layer.feed_forward.forward(h2, residual, batch)


@register_block("parallel_residual")
class ParallelResidualBlock(Block):
    graph_safe = True

    def __init__(self, spec, prefix="", **_):
        super().__init__(spec, prefix)

    def run(self, layer, residual, batch, cache):
        layer.mixer_norm.ws.settle()
        with phase("rmsnorm"):
            h = layer.mixer_norm(residual, batch.dtype)
        layer.mixer.forward(h, residual, batch, cache)
        if layer.feed_forward is not None:
            layer.feed_forward.forward(h, residual, batch)


@register_block("hyper_connections")
class HyperConnectionsBlock(Block):
    """params: streams, sublayers (1 or 2), names: per sublayer a dict {"read", "write", "mix"} of tensor names
    under the layer's prefix, required (False: a missing tensor means ones / the identity, which makes the block
    the ordinary residual sum).  The layer's norms are the model's norm parts; the block reads their weight,
    offset and eps and fuses them into its kernel."""
    graph_safe = True

    def __init__(self, spec, prefix="", **_):
        super().__init__(spec, prefix)
        self.S = int(spec["streams"])
        if not 1 <= self.S <= 8:
            raise ValueError(f"hyper_connections: {self.S} streams (supported: 1 to 8)")
        self.names = [dict(n) for n in spec["names"]]
        self.required = bool(spec.get("required", True))
        self.coef = []                 # per sublayer (read, write, mix) float32 on the device

    def requirements(self):
        S, opt = self.S, not self.required
        reqs = []
        for n in self.names:
            reqs += [TensorReq(self.prefix + n["read"], (S,), init=f"const:{1.0 / S}+normal", optional=opt),
                     TensorReq(self.prefix + n["write"], (S,), init="ones+normal", optional=opt),
                     TensorReq(self.prefix + n["mix"], (S, S), init="eye+normal", optional=opt)]
        return reqs

    def load(self, source, device):
        S = self.S
        self.coef = []
        for n in self.names:
            def get(key, default):
                name = self.prefix + n[key]
                if source.has(name):
                    return source.get(name, device).to(torch.float32).contiguous()
                return default.to(device)
            self.coef.append((get("read", torch.ones(S)), get("write", torch.ones(S)), get("mix", torch.eye(S))))

    def _sublayer(self, x, norm, coef, pending, dtype, tag):
        """Applies the pending write-back (y, coef of the sublayer before) and returns this sublayer's input."""
        T, H = x.shape[1], x.shape[2]
        h = norm.ws.get(tag, (T, H), dtype)
        kw = {} if pending is None else {"y": pending[0], "write": pending[1][1], "mix": pending[1][2]}
        K.hc_step(x, read=coef[0], norm_weight=norm.weight, norm_offset=norm.weight_offset, eps=norm.eps,
                  h_out=h, **kw)
        return h

    @staticmethod
    def _run_part(part, h, y, *args):
        """y = part(h): parts that can store their output do; the others add into a zeroed buffer."""
        if getattr(part, "can_store", False):
            part.forward(h, y, *args, add=False)
        else:
            y.zero_()
            part.forward(h, y, *args)

    def run(self, layer, residual, batch, cache):
        x = residual if residual.dim() == 3 else residual.unsqueeze(0)
        T, H = x.shape[1], x.shape[2]
        ws = layer.mixer_norm.ws
        before, ws.pending_writeback = ws.pending_writeback, None
        if before is not None and before[0].data_ptr() != x.data_ptr():
            ws.pending_writeback = before          # another residual's: not ours to fuse
            ws.settle()
            before = None
        with phase("rmsnorm"):
            h = self._sublayer(x, layer.mixer_norm, self.coef[0], None if before is None else (before[1], (None, before[2], before[3])),
                               batch.dtype, "norm_mixer")
        y = ws.get("hc_y", (T, H), torch.float32)
        self._run_part(layer.mixer, h, y, batch, cache)
        pending = (y, self.coef[0])
        if layer.feed_forward is not None:
            with phase("rmsnorm"):
                h2 = self._sublayer(x, layer.feed_forward_norm, self.coef[1], pending, batch.dtype, "norm_ffn")
            y2 = ws.get("hc_y2", (T, H), torch.float32)
            self._run_part(layer.feed_forward, h2, y2, batch)
            pending = (y2, self.coef[1])
        ws.pending_writeback = (x, pending[0], pending[1][1], pending[1][2])


@register_block("scaled_pre_norm")
class ScaledPreNormBlock(HyperConnectionsBlock):
    """params: residual_scale (m).  No tensors of its own."""
    graph_safe = True

    def __init__(self, spec, prefix="", **_):
        Block.__init__(self, spec, prefix)
        self.S, self.names, self.required = 1, [], False
        self.scale = float(spec["residual_scale"])
        self.coef = []

    def requirements(self):
        return []

    def load(self, source, device):
        one = torch.ones(1, dtype=torch.float32, device=device)
        c = (one, torch.full((1,), self.scale, dtype=torch.float32, device=device), one.view(1, 1).clone())
        self.coef = [c, c]


@register_block("post_norm")
class PostNormBlock(Block):
    """No params and no tensors of its own: the layer's norm parts give weight and eps."""
    graph_safe = True

    def __init__(self, spec, prefix="", **_):
        super().__init__(spec, prefix)

    @staticmethod
    def _input(ws, x, dtype):
        """The residual in the activation dtype: x itself in float32, else the copy that the sublayer before left
        (or a fresh one)."""
        if dtype == torch.float32:
            return x
        T, H = x.shape
        h = ws.get("post_norm_h", (T, H), dtype)
        if ws.residual_copy != (x.data_ptr(), T, H, dtype):
            K.cast_rows(x, h)
        return h

    @staticmethod
    def _enter(ws, ys, scales, norm, x, dtype):
        """x += rmsnorm(sum_b scales[b] ys[b]) * w, and the new x in the activation dtype for whoever reads it next."""
        if norm.weight_offset:
            raise ValueError("post_norm: a norm weight stored as a distance from a constant is not supported here")
        h = None if dtype == torch.float32 else ws.get("post_norm_h", x.shape, dtype)
        with phase("rmsnorm"):
            K.sum_norm_add(ys, scales, norm.weight, x, eps=norm.eps, add=True, h_out=h)
        ws.residual_copy = None if h is None else (x.data_ptr(), x.shape[0], x.shape[1], dtype)

    def run(self, layer, residual, batch, cache):
        # The sublayers' products stay on the single-CTA tensor-core kernel.  With the two-SM kernel in these chains
        # (a storing up product directly followed by a storing down product, the launches of this block between
        # them and the next layer's) a prompt of 2,048 tokens at width 2,048 did not return in one run of a few;
        # reading the kernels did not show why, and the single-CTA kernel ran the same prompts at the same speed
        # (3.8 ms for four layers) every time, so that is what this block takes until the cause is known.
        with single_cta_products():
            self._run(layer, residual, batch, cache)

    def _run(self, layer, residual, batch, cache):
        ws, x = layer.mixer_norm.ws, residual
        if x.dim() != 2:
            raise ValueError("post_norm: the block keeps one residual stream")
        keep, ws.residual_copy = ws.residual_copy, None
        ws.settle()                         # (forgets the copy: whoever else settles has changed the residual)
        ws.residual_copy = keep
        T, H = x.shape
        h = self._input(ws, x, batch.dtype)
        outs = getattr(layer.mixer, "branch_outputs", lambda *a: None)(h, batch, cache)
        if outs is None:
            y = ws.get("post_norm_y", (T, H), torch.float32)
            HyperConnectionsBlock._run_part(layer.mixer, h, y, batch, cache)
            outs = ([y], [1.0])
        self._enter(ws, outs[0], outs[1], layer.mixer_norm, x, batch.dtype)
        if layer.feed_forward is None:
            return
        h = self._input(ws, x, batch.dtype)
        y = ws.get("post_norm_y", (T, H), torch.float32)
        HyperConnectionsBlock._run_part(layer.feed_forward, h, y, batch)
        self._enter(ws, [y], [1.0], layer.feed_forward_norm, x, batch.dtype)
