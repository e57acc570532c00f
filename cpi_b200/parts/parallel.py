"""Mixers side by side: several mixers read the same normed input, and their outputs are summed.

"parallel"  params: branches (a list of {"name", "mixer": PartSpec}: tensors of a branch live under the mixer's prefix
            + name + "."), combine {"kind": "normed_mean", "eps", "weights": [tensor name per branch, under the mixer's
            prefix]}: out = (1 / n) sum_b rmsnorm(branch_b(h)) * weight_b, each branch divided by its own root mean
            square over the model width.  ("sum": the plain sum of the branches, no tensors.  {"kind": "weighted_sum",
            "scales": [a constant per branch]}: out = sum_b scale_b * branch_b(h), no tensors either.)

The branches do not depend on one another: in a step of few tokens the first runs on a second stream beside the
others (inside a captured graph this becomes two chains side by side), each into a buffer of its own, and the sum
waits for both.

What the branches keep lives in the one run entry of their layer: at most one branch may keep a paged cache (its
requirement becomes the layer's), and the branches' per-sequence state is held under names that carry the branch's
name, so two recurrent branches of one kind do not collide.
"""
from __future__ import annotations

import torch

from ..csrc import lib as K
from ..phases import active as phases_active, phase
from ..weights.store import TensorReq
from .base import Mixer, build_part, register_mixer


class _BranchCache:
    """A branch's view of its layer's cache: the paged streams as they are, state under the branch's name."""

    def __init__(self, cache, name: str):
        self._c, self._name = cache, name
        self.owns = cache.owns

    def kv(self):
        return self._c.kv()

    def stream(self, name):
        return self._c.stream(name)

    def state(self, name):
        return self._c.state(f"{self._name}.{name}")


@register_mixer("parallel")
class ParallelMixer(Mixer):
    can_store = True

    def __init__(self, spec, prefix="", workspace=None, owns_cache=True):
        super().__init__(spec, prefix)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.names = [str(b["name"]) for b in p["branches"]]
        if len(set(self.names)) != len(self.names) or not 1 <= len(self.names) <= 4:
            raise ValueError(f"parallel: one to four branches with names of their own, not {self.names}")
        self.branches = [build_part("mixer", b["mixer"], prefix, workspace=workspace, owns_cache=owns_cache)
                         for b in p["branches"]]
        c = p.get("combine") or {"kind": "sum"}
        if c["kind"] not in ("sum", "normed_mean", "weighted_sum"):
            raise ValueError(f"parallel: unknown way of combining the branches '{c['kind']}'")
        self.normed = c["kind"] == "normed_mean"
        self.scales = [float(x) for x in c["scales"]] if c["kind"] == "weighted_sum" else None
        if self.scales is not None and len(self.scales) != len(self.branches):
            raise ValueError("parallel: a weighted sum needs one constant per branch")
        self.eps = float(c.get("eps", 0.0))
        self.weight_names = [prefix + n for n in c.get("weights", [])] if self.normed else []
        if self.normed and len(self.weight_names) != len(self.branches):
            raise ValueError("parallel: a normed mean needs one weight per branch")
        if sum(b.kv_requirement() is not None for b in self.branches) > 1:
            raise ValueError("parallel: at most one branch may keep a paged cache")
        self.weights = []
        self.overlap_branches = True      # the first branch on a second stream (off while phases are timed)
        self.overlap_max_tokens = 16      # ... in steps whose longest portion has at most this many tokens
        self._side_stream = None
        self.ws = workspace
        self.graph_safe = all(getattr(b, "graph_safe", False) for b in self.branches)
        positions = [b.position for b in self.branches if getattr(b, "position", None) is not None]
        self.position = positions[0] if positions else None

    def requirements(self):
        reqs = [r for b in self.branches for r in b.requirements()]
        return reqs + [TensorReq(n, (self.hidden,), init="ones+normal") for n in self.weight_names]

    def load(self, source, device):
        for b in self.branches:
            b.load(source, device)
        self.weights = [source.get(n, device).to(torch.float32).contiguous() for n in self.weight_names]

    def kv_requirement(self):
        for b in self.branches:
            r = b.kv_requirement()
            if r is not None:
                return r
        return None

    def state_requirements(self):
        import dataclasses
        return [dataclasses.replace(r, name=f"{n}.{r.name}") for n, b in zip(self.names, self.branches)
                for r in b.state_requirements()]

    def forward(self, h, residual, batch, cache, add=True):
        T = h.shape[0]
        if self.scales is not None:
            ys, scales = self.branch_outputs(h, batch, cache)
            with phase("combine"):
                K.sum_norm_add(ys, scales, None, residual, add=add, normalise=False)
            return
        if not self.normed:
            for i, (n, b) in enumerate(zip(self.names, self.branches)):
                b.forward(h, residual, batch, _BranchCache(cache, n), add=add or i > 0)
            return
        ys = self._run_branches(h, batch, cache)
        with phase("combine"):
            K.branch_norm_sum(ys, self.weights, residual, eps=self.eps, scale=1.0 / len(ys), add=add)

    def branch_outputs(self, h, batch, cache):
        """(the branches' outputs, float32 [T, hidden] each, in workspace buffers; a constant per branch): the mixer's
        output is their weighted sum, which a block that does something to that sum anyway may form itself.  None
        unless the branches are combined by constants."""
        if self.scales is None:
            return None
        return self._run_branches(h, batch, cache), self.scales

    def _run_branches(self, h, batch, cache):
        T = h.shape[0]
        ys = [self.ws.get(f"parallel_y{i}", (T, self.hidden), torch.float32) for i in range(len(self.branches))]

        def run(i):
            n, b, y = self.names[i], self.branches[i], ys[i]
            if getattr(b, "can_store", False):
                b.forward(h, y, batch, _BranchCache(cache, n), add=False)
            else:
                y.zero_()
                b.forward(h, y, batch, _BranchCache(cache, n))

        joined = None
        # (a step of few tokens only: its kernels are short and leave most of the GPU idle.  In a prompt a branch's
        # kernels fill the GPU by themselves, and a recurrence that runs beside another branch's products was
        # measured slower than the two one after the other: 11.3 against 8.9 ms for 2,048 tokens)
        if (self.overlap_branches and len(self.branches) > 1 and h.is_cuda and phases_active() is None
                and batch.max_new <= self.overlap_max_tokens):
            if self._side_stream is None:
                self._side_stream = torch.cuda.Stream(device=h.device)
            fork = torch.cuda.Event()
            fork.record(torch.cuda.current_stream())
            self._side_stream.wait_event(fork)
            with torch.cuda.stream(self._side_stream):
                run(0)
                joined = torch.cuda.Event()
                joined.record(self._side_stream)
        else:
            run(0)
        for i in range(1, len(self.branches)):
            run(i)
        if joined is not None:
            torch.cuda.current_stream().wait_event(joined)
        return ys
