"""A feed-forward of routed experts.

Router: z = W_r x in float32, s = softmax(z) over all experts; a token uses the
``top`` experts with the largest s (lowest index among equals), weighted by their
s as they are (not renormalised).  Expert
(no biases): y = W_down act(W_gate x, W_up x) with the gated activation

    act(g, u) = g' * sigmoid(alpha * g') * (u' + up_shift),
    g' = min(g, limit),  u' = clamp(u, -limit, limit)        (limit None: no clamp)

The tokens' (token, expert) pairs are ordered by expert on the device; the experts'
products run over row tiles of that order, one launch for all experts, with no size
read back to the host.  ``forward_slots`` returns the pairs' results [T * top, H]
and the weights [T, top] for a reader that takes the weighted sum itself;
``forward`` takes it.

params: hidden_size, inner_size, num_experts, top, limit, alpha, up_shift,
tensor_names (keys "router", "gate", "up", "down"; the last three with ``{e}`` where
the expert's number stands).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops
from .base import FeedForward
from .linear import linear
from .registry import register_part
from .spec import PartSpec, TensorSpec


@register_part("feed_forward", "routed_experts")
class RoutedExperts(FeedForward):
    graph_safe = True

    def __init__(self, spec: PartSpec, prefix: str = ""):
        super().__init__(spec, prefix)
        p = spec.get()
        self.hidden, self.inner = int(p["hidden_size"]), int(p["inner_size"])
        self.experts, self.top = int(p["num_experts"]), int(p["top"])
        if not 1 <= self.top <= self.experts:
            raise ValueError(f"top {self.top} of {self.experts} experts")
        self.limit = float(p["limit"]) if p.get("limit") is not None else float("inf")
        self.alpha = float(p.get("alpha", 1.0))
        self.up_shift = float(p.get("up_shift", 0.0))
        if self.up_shift != 1.0:
            raise ValueError("the expert kernel computes (u' + 1); another up_shift is not built")
        names = dict(p.get("tensor_names") or ())
        if sorted(names) != ["down", "gate", "router", "up"]:
            raise ValueError("a routed_experts spec names its tensors: tensor_names with the keys router, gate, up, down")
        self.names = {k: prefix + str(v) for k, v in names.items()}
        self.w_router = self.w_gate_up = self.w_down = None

    def _expert(self, key: str, e: int) -> str:
        return self.names[key].format(e=e)

    def tensor_specs(self) -> List[TensorSpec]:
        specs = [TensorSpec(self.names["router"], (self.experts, self.hidden), init=("normal", 0.3))]
        for e in range(self.experts):
            specs += [TensorSpec(self._expert("gate", e), (self.inner, self.hidden), init=("normal", 0.1)),
                      TensorSpec(self._expert("up", e), (self.inner, self.hidden), init=("normal", 0.1)),
                      TensorSpec(self._expert("down", e), (self.hidden, self.inner), init=("normal", 0.1))]
        return specs

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.w_router = tensors[self.names["router"]].contiguous()
        # [E, 2 F, H]: an expert's gate rows, then its up rows;  [E, H, F]
        self.w_gate_up = torch.stack([torch.cat([tensors[self._expert("gate", e)], tensors[self._expert("up", e)]], dim=0)
                                      for e in range(self.experts)]).contiguous()
        self.w_down = torch.stack([tensors[self._expert("down", e)] for e in range(self.experts)]).contiguous()

    def forward_slots(self, x: torch.Tensor):
        # the logits are one matrix product with a float32 result (float32 accumulation from the first term
        # on), softmax and choice a small kernel (``ops.moe_route`` is the same in one kernel, a warp a token:
        # the form the two are checked against)
        ids, scores = ops.moe_choose(linear(x, self.w_router, out_dtype=torch.float32), self.top)
        return ops.moe_experts(x, ids, self.w_gate_up, self.w_down, self.limit, self.alpha), scores

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y, scores = self.forward_slots(x)
        out = torch.empty_like(x)
        ops.weighted_slot_sum(y, scores, out)
        return out
