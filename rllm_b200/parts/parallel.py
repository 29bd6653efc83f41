"""``parallel``: two mixers side by side that read the same input; the result is
the mean of their outputs, each first divided by its root mean square over the
model width (eps inside the root) and multiplied by a weight of its own:

    y = 1/2 (rms(a(x)) * w_a + rms(b(x)) * w_b).

Each branch is a registered mixer with its own ``PartSpec``, tensors (below its
``tensor_prefix``) and cache: the part's cache need is the branches' needs one
after the other (pages for one, state for the other, whatever they declare),
and each branch gets its own views.

params: hidden_size, eps, branches (two mixer ``PartSpec``s), tensor_names (key
"out": the two weights' names below the part's prefix, in branch order).
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..kernels import ops
from .base import Mixer, StepContext
from .registry import build_part, register_part
from .spec import PartSpec, TensorSpec


def _needs(mixer: Mixer) -> tuple:
    need = mixer.cache_need()
    if need is None:
        return ()
    return tuple(need) if isinstance(need, (tuple, list)) else (need,)


@register_part("mixer", "parallel")
class ParallelMixer(Mixer):
    def __init__(self, spec: PartSpec, prefix: str = ""):
        super().__init__(spec, prefix)
        p = spec.get()
        self.hidden, self.eps = int(p["hidden_size"]), float(p["eps"])
        branches = tuple(p["branches"])
        if len(branches) != 2:
            raise ValueError("a parallel mixer has two branches")
        self.branches: List[Mixer] = [
            build_part("mixer", b, prefix=prefix + str(b.get().get("tensor_prefix") or "")) for b in branches]
        names = dict(p.get("tensor_names") or ())
        out = tuple(names.get("out") or ())
        if len(out) != 2:
            raise ValueError("a parallel spec names its two output weights: tensor_names with the key out")
        self.out_names = [prefix + str(n) for n in out]
        self.w_out: List[torch.Tensor] = []
        self.counts = [len(_needs(b)) for b in self.branches]
        self.several = [isinstance(b.cache_need(), (tuple, list)) for b in self.branches]

    @property
    def graph_safe(self) -> bool:
        return all(bool(b.graph_safe) for b in self.branches)

    def tensor_specs(self) -> List[TensorSpec]:
        specs = [ts for b in self.branches for ts in b.tensor_specs()]
        return specs + [TensorSpec(n, (self.hidden,), role="vector", init=("one_plus_normal", 0.1))
                        for n in self.out_names]

    def ignored_tensors(self) -> List[str]:
        return [n for b in self.branches for n in b.ignored_tensors()]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        for b in self.branches:
            b.load(tensors)
        self.w_out = [tensors[n].contiguous() for n in self.out_names]
        self.w_out[1] = self.w_out[1].to(self.w_out[0].dtype)

    def cache_need(self):
        return tuple(n for b in self.branches for n in _needs(b))

    def forward(self, x: torch.Tensor, ctx: StepContext, cache) -> torch.Tensor:
        views = tuple(cache) if isinstance(cache, (tuple, list)) else ((cache,) if cache is not None else ())
        outs, at = [], 0
        for b, n, several in zip(self.branches, self.counts, self.several):
            mine = views[at:at + n]
            at += n
            outs.append(b.forward(x, ctx, mine if several else (mine[0] if n else None)))
        return ops.rms_mean2(outs[0], outs[1], self.w_out[0], self.w_out[1], self.eps)
