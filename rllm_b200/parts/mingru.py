"""minGRU: a recurrence whose gates read the current token only.

    z_t = sigmoid(W_z x_t + b_z),   u_t = W_x x_t + b_x,
    c_t = u_t + 1/2  where u_t >= 0,  sigmoid(u_t)  where u_t < 0,
    S_t = (1 - z_t) S_{t-1} + z_t c_t                  (element by element, S_{-1} = 0),
    y_t = W_o (S_t * silu(W_g x_t)).

The three input projections are one matrix product over the stacked weights
[W_z; W_x; W_g].  The state S is float32 [width] per request, kept in the
request's state slot from step to step; gates, candidate, recurrence and the
output gate are float32 arithmetic in one kernel that walks each sequence's
tokens of the step in order.

params: hidden_size, width, tensor_names (keys "z", "z_bias", "x", "x_bias",
"g", "o": names below the part's prefix).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops
from .base import Mixer, StateCacheView, StepContext
from .linear import linear
from .registry import register_part
from .spec import PartSpec, StateNeed, TensorSpec

_KEYS = ("z", "z_bias", "x", "x_bias", "g", "o")


@register_part("mixer", "mingru")
class MinGRU(Mixer):
    graph_safe = True

    def __init__(self, spec: PartSpec, prefix: str = ""):
        super().__init__(spec, prefix)
        p = spec.get()
        self.hidden = int(p["hidden_size"])
        self.width = int(p["width"])
        names = dict(p.get("tensor_names") or ())
        if sorted(names) != sorted(_KEYS):
            raise ValueError(f"a mingru spec names its tensors: tensor_names with the keys {_KEYS}")
        self.names = {k: prefix + str(v) for k, v in names.items()}
        self.w_in: Optional[torch.Tensor] = None
        self.w_o: Optional[torch.Tensor] = None
        self.b_z: Optional[torch.Tensor] = None
        self.b_x: Optional[torch.Tensor] = None

    def tensor_specs(self) -> List[TensorSpec]:
        n, W, H = self.names, self.width, self.hidden
        return [TensorSpec(n["z"], (W, H)), TensorSpec(n["z_bias"], (W,), role="vector", init=("normal", 0.5)),
                TensorSpec(n["x"], (W, H)), TensorSpec(n["x_bias"], (W,), role="vector", init=("normal", 0.5)),
                TensorSpec(n["g"], (W, H)), TensorSpec(n["o"], (H, W))]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        n = self.names
        self.w_in = torch.cat([tensors[n["z"]], tensors[n["x"]], tensors[n["g"]]], dim=0).contiguous()
        self.b_z, self.b_x = tensors[n["z_bias"]].contiguous(), tensors[n["x_bias"]].contiguous()
        self.w_o = tensors[n["o"]]

    def cache_need(self):
        return StateNeed((self.width,))

    def stack_input(self, weight: torch.Tensor) -> bool:
        self.w_in = torch.cat([self.w_in[: 3 * self.width], weight], dim=0).contiguous()
        return True

    def forward(self, x, ctx: StepContext, cache: StateCacheView, side: bool = False):
        a = linear(x, self.w_in)                                   # [T, 3 width (+ side rows)]: z | x | g | side
        out = torch.empty((x.shape[0], self.width), dtype=x.dtype, device=x.device)
        ops.mingru_scan(a, self.b_z, self.b_x, cache.state, ctx.q_start, ctx.state_slots, ctx.num_seqs, out, ctx.err,
                        max_q_len=ctx.max_q_len)
        y = linear(out, self.w_o)
        return (y, a[:, 3 * self.width:]) if side else y
