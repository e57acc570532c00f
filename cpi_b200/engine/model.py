"""A decoder built from a ModelSpec: layers of registered parts, run in the order the spec lists."""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..config.spec import ModelSpec
from ..csrc import lib as K
from ..parts import base as parts_base
from ..parts import Workspace, build_part
from ..parts.linear import project
from ..phases import phase
from ..weights.store import TensorReq, check_source


@dataclass
class Layer:
    block: object
    mixer: object
    feed_forward: object
    mixer_norm: object
    feed_forward_norm: object

    def parts(self):
        return tuple(p for p in (self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward)
                     if p is not None)

    def all_parts(self):
        """Every object whose code runs in a step of this layer (the mixer's position encoding included)."""
        out = [self.block, *self.parts()]
        pos = getattr(self.mixer, "position", None)
        if pos is not None:
            out.append(pos)
        return out


class DecoderModel:
    def __init__(self, spec: ModelSpec, dtype: torch.dtype, device, workspace: Workspace | None = None):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"activation dtype must be float32 or bfloat16, not {dtype}")
        spec.validate()
        self.spec, self.dtype, self.device = spec, dtype, torch.device(device)
        self.ws = workspace if workspace is not None else Workspace(self.device)
        owners = set()                      # layers that some run entry uses with a cache of its own
        for e in spec.run_order:
            if e.cache_of is None:
                owners.add(e.layer)
        self.layers = []
        for i, ls in enumerate(spec.layers):
            self.layers.append(Layer(
                block=build_part("block", ls.block, ls.prefix),
                mixer=build_part("mixer", ls.mixer, ls.prefix, workspace=self.ws, owns_cache=i in owners),
                feed_forward=None if ls.feed_forward is None else
                build_part("feed_forward", ls.feed_forward, ls.prefix, workspace=self.ws),
                mixer_norm=build_part("norm", ls.mixer_norm, ls.prefix, workspace=self.ws, tag="norm_mixer"),
                feed_forward_norm=None if ls.feed_forward is None or ls.feed_forward_norm is None else
                build_part("norm", ls.feed_forward_norm, ls.prefix, workspace=self.ws, tag="norm_ffn"),
            ))
        self.streams = int(spec.residual_streams)
        if self.streams < 1:
            raise ValueError(f"a model keeps at least one residual stream, not {self.streams}")
        self.logit_scale = float(spec.head.get("logit_scale", 1.0) or 1.0)
        self.logit_softcap = float(spec.head.get("logit_softcap", 0.0) or 0.0)
        self.layer_capture = None           # a list: every run appends the residual after each run entry [T, H]
        self.final_norm = build_part("norm", spec.final_norm, "", workspace=self.ws, tag="norm_final")
        en = spec.embedding.get("norm")
        self.embed_norm = None if en is None else build_part("norm", en, "", workspace=self.ws, tag="norm_embed")
        self.junctions = {name: build_part("junction", js, "", workspace=self.ws) for name, js in spec.junctions}
        self.keep_x0 = any(j.needs_embedding_output for j in self.junctions.values())
        if self.embed_norm is not None and self.streams != 1:
            raise ValueError("a norm on the embedding output does not combine with several residual streams")
        self.embed_name = spec.embedding["weight"]
        self.head_name = spec.head["weight"]
        self.embedding = self.head = None
        self.err_flag = None

    # ---- weights ---------------------------------------------------------------------------------
    def all_parts(self) -> list:
        """Every part object of the model (layers' blocks, norms, mixers with their position encodings,
        feed-forwards, the final norm)."""
        out = [self.final_norm, *self.junctions.values()]
        if self.embed_norm is not None:
            out.append(self.embed_norm)
        for layer in self.layers:
            out += layer.all_parts()
        return out

    def requirements(self) -> list:
        V, H = self.spec.vocab_size, self.spec.hidden_size
        reqs = [TensorReq(self.embed_name, (V, H))]
        if self.head_name != self.embed_name:
            reqs.append(TensorReq(self.head_name, (V, H)))
        reqs += self.final_norm.requirements()
        if self.embed_norm is not None:
            reqs += self.embed_norm.requirements()
        for j in self.junctions.values():
            reqs += j.requirements()
        for layer in self.layers:
            for p in (layer.block, *layer.parts()):
                reqs += p.requirements()
        return reqs

    def load(self, source) -> None:
        tolerated = ()
        if self.head_name == self.embed_name:      # a tied model may still store a head tensor
            tolerated = tuple(n for n in source.names() if n.endswith("lm_head.weight"))
        check_source(self.requirements(), source, self.spec.ignored_tensor_prefixes, tolerated)
        dev = self.device
        self.embedding = source.get(self.embed_name, dev).contiguous()
        self.head = self.embedding if self.head_name == self.embed_name else source.get(self.head_name, dev).contiguous()
        self.final_norm.load(source, dev)
        if self.embed_norm is not None:
            self.embed_norm.load(source, dev)
        for j in self.junctions.values():
            j.load(source, dev)
        for layer in self.layers:
            for p in (layer.block, *layer.parts()):
                p.load(source, dev)
        # the word of the device's error flags that the embedding kernel sets for a token outside the table
        self.err_flag = K.device_error_flags(dev)[1:2] if torch.device(dev).type == "cuda" \
            else torch.zeros(1, dtype=torch.int32, device=dev)

    # ---- cache needs -----------------------------------------------------------------------------
    def cache_requirements(self):
        """({run entry: KVRequirement}, {run entry: [StateRequirement]}) for entries that own a cache."""
        kv, state = {}, {}
        for i, e in enumerate(self.spec.run_order):
            if e.cache_of is not None:
                continue
            m = self.layers[e.layer].mixer
            r = m.kv_requirement()
            if r is not None:
                kv[i] = r
            s = m.state_requirements()
            if s:
                state[i] = list(s)
        return kv, state

    # ---- forward ---------------------------------------------------------------------------------
    def run(self, batch, cache_manager) -> torch.Tensor:
        """Runs the step's tokens through every run entry; returns float32 logits [n_want, vocab]."""
        T, H, S = batch.n_tokens, self.spec.hidden_size, self.streams
        # the residual: float32 [T, H], or [S, T, H] for blocks that keep S streams (each starts as the embedding)
        xs = self.ws.get("residual", (S, T, H), torch.float32)
        self.ws.pending_writeback = None
        self.ws.residual_copy = None
        with phase("embedding"):
            if self.embed_norm is not None:                 # the looked-up rows are normed into the residual
                raw = self.ws.get("embed_rows", (T, H), torch.float32)
                K.embedding(batch.tokens, self.embedding, raw, self.err_flag)
                self.embed_norm(raw, torch.float32, out=xs[0])
            else:
                for s in range(S):
                    K.embedding(batch.tokens, self.embedding, xs[s], self.err_flag)
        x = xs[0] if S == 1 else xs
        x0 = None
        if self.keep_x0:
            x0 = self.ws.get("embed_out", (T, H), torch.float32)
            x0.copy_(xs[0])
        for i, e in enumerate(self.spec.run_order):
            layer = self.layers[e.layer]
            if e.before is not None:
                self.ws.settle()                # a block may have left its last write-back to whoever reads x next
                self.junctions[e.before].run(x, x0, batch)
            owner = i if e.cache_of is None else e.cache_of
            view = parts_base.CacheView(cache_manager, owner, owns=e.cache_of is None)
            layer.block.run(layer, x, batch, view)
            if e.after is not None:
                self.ws.settle()
                self.junctions[e.after].run(x, x0, batch)
            if self.layer_capture is not None:
                self.ws.settle()
                self.layer_capture.append(xs.sum(0))
        self.ws.settle()                    # a write-back that the last block left to its successor
        R = batch.n_want
        logits = self.ws.get("logits", (R, self.spec.vocab_size), torch.float32)   # valid until the next step
        if R:
            with phase("rmsnorm"):
                if S == 1:
                    xn = self.final_norm(x, self.dtype, rows=batch.want_rows)
                else:                       # the norm of the streams' sum, one kernel
                    xn = self.ws.get("norm_final", (R, H), self.dtype)
                    K.hc_step(xs, rows=batch.want_rows, norm_weight=self.final_norm.weight,
                              norm_offset=self.final_norm.weight_offset, eps=self.final_norm.eps, h_out=xn)
            with phase("lm_head"):
                project(xn, self.head, logits)
                if self.logit_scale != 1.0 or self.logit_softcap > 0.0:
                    K.logit_post(logits, self.logit_scale, self.logit_softcap)
        return logits


def tensor_requirements(spec: ModelSpec) -> list:
    """The tensors a model of this spec needs (names, shapes, random-init rule), without a device."""
    return DecoderModel(spec, torch.float32, "cpu").requirements()
