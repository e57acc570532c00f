"""Junctions: what a run order may place between two layers, acting on the residual itself.

"concat_linear"  x <- W [x ; x0]: the residual and the embedding output side by side (x first) through one matrix
                 W [width, 2 width].  params: hidden_size, weight (tensor name).  The operand row is formed in the
                 activation dtype; the product accumulates in float32 and writes the float32 residual.

"token_gated_input"  x <- x + rmsnorm(P (gelu_tanh(G x) * e)) * w: every token brings a small vector e of its own, the
                 columns [offset, offset + dim) of its row in a table indexed by token id (one table may serve many
                 layers, each with its own columns); a projection G [dim, width] of the residual gates it, P [width,
                 dim] takes it to the model width, and the result enters the residual through an RMS norm with a plain
                 weight w.  params: hidden_size, dim, table (tensor name), table_width, offset, gate, proj, norm
                 (tensor names), eps.  float32: one kernel, float32 throughout.  bfloat16: the two products run as
                 matrix products with bfloat16 operands (the residual row and the gated vector are rounded for them),
                 the activation, the norm and the sum stay float32.
"""
from __future__ import annotations

import torch

from ..csrc import lib as K
from ..phases import phase
from ..weights.store import TensorReq
from .base import Junction, register_junction
from .linear import project


@register_junction("concat_linear")
class ConcatLinear(Junction):
    graph_safe = True
    needs_embedding_output = True

    def __init__(self, spec, prefix="", workspace=None):
        super().__init__(spec, prefix)
        self.hidden = int(spec["hidden_size"])
        self.weight_name = prefix + spec["weight"]
        self.ws, self.weight = workspace, None

    def requirements(self):
        return [TensorReq(self.weight_name, (self.hidden, 2 * self.hidden))]

    def load(self, source, device):
        self.weight = source.get(self.weight_name, device).contiguous()

    def run(self, x, x0, batch) -> None:
        cat = self.ws.get("junction_cat", (x.shape[0], 2 * self.hidden), batch.dtype)
        with phase("junction"):
            K.concat_rows(x, x0, cat)
            project(cat, self.weight, x)


@register_junction("token_gated_input")
class TokenGatedInput(Junction):
    graph_safe = True

    def __init__(self, spec, prefix="", workspace=None):
        super().__init__(spec, prefix)
        self.hidden, self.dim = int(spec["hidden_size"]), int(spec["dim"])
        self.offset, self.table_width = int(spec.get("offset", 0)), int(spec["table_width"])
        self.vocab = int(spec["vocab_size"])
        if self.offset < 0 or self.offset + self.dim > self.table_width:
            raise ValueError(f"token_gated_input: columns {self.offset}..{self.offset + self.dim} of a table of "
                             f"{self.table_width}")
        self.eps = float(spec["eps"])
        self.names = {k: prefix + spec[k] for k in ("table", "gate", "proj", "norm")}
        self.ws = workspace
        self.table = self.w_gate = self.w_proj = self.w_norm = None

    def requirements(self):
        n = self.names
        return [TensorReq(n["table"], (self.vocab, self.table_width)), TensorReq(n["gate"], (self.dim, self.hidden)),
                TensorReq(n["proj"], (self.hidden, self.dim)), TensorReq(n["norm"], (self.hidden,), init="ones+normal")]

    def load(self, source, device):
        n = self.names
        shared = getattr(source, "_shared_tables", None)      # one copy on the device for the layers of one source
        if shared is None:
            shared = {}
            try:
                source._shared_tables = shared
            except AttributeError:
                pass
        key = (n["table"], str(device))
        if key not in shared:
            shared[key] = source.get(n["table"], device).contiguous()
        self.table = shared[key]
        gate, proj = source.get(n["gate"], device), source.get(n["proj"], device)
        dt = torch.float32 if torch.float32 in (gate.dtype, proj.dtype) else torch.bfloat16
        self.w_gate, self.w_proj = gate.to(dt).contiguous(), proj.to(dt).contiguous()
        self.w_norm = source.get(n["norm"], device).to(torch.float32).contiguous()

    def run(self, x, x0, batch) -> None:
        T = x.shape[0]
        with phase("side_input"):
            if batch.dtype != torch.bfloat16 or self.w_gate.dtype != torch.bfloat16:
                K.gated_side_input(x, batch.tokens, self.table, self.offset, self.w_gate, self.w_proj, self.w_norm,
                                   self.eps)
                return
            # bfloat16: the two products on the tensor cores, the gate's activation and the norm in float32 between
            xb = self.ws.get("side_x", (T, self.hidden), torch.bfloat16)
            z = self.ws.get("side_z", (T, self.dim), torch.float32)
            g = self.ws.get("side_g", (T, self.dim), torch.bfloat16)
            y = self.ws.get("side_y", (T, self.hidden), torch.float32)
            K.cast_rows(x, xb)
            project(xb, self.w_gate, z)
            K.side_gate_act(z, batch.tokens, self.table, self.offset, g)
            project(g, self.w_proj, y)
            K.branch_norm_sum([y], [self.w_norm], x, eps=self.eps, add=True)
