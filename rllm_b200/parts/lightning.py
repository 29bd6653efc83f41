"""``lightning_attention``: linear attention with a fixed decay per head.

    q = silu(W_q h), k = silu(W_k h)  [heads, head_dim],   v = silu(W_v h)  [heads, v_dim]
    S_t = decay[head] * S_{t-1} + k_t v_t^T,   o_t = S_t^T q_t            (no other scale)
    y = W_o (rms(o over all heads together) * w * sigmoid(W_g h))         (eps inside the root)

S is float32 [heads, head_dim, v_dim] per request, starts at zero and is carried
from step to step in the request's state slot.  The four input projections are
one matrix product over the stacked weights; the activations, the recurrence and
the norm are float32 arithmetic in the kernels.

params: hidden_size, num_heads, head_dim, v_dim, decay (one number a head), eps,
tensor_names (keys "q", "k", "v", "g", "o", "norm").
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops
from .base import Mixer, StateCacheView, StepContext
from .linear import linear
from .registry import register_part
from .spec import PartSpec, StateNeed, TensorSpec

_KEYS = ("q", "k", "v", "g", "o", "norm")


@register_part("mixer", "lightning_attention")
class LightningAttention(Mixer):
    graph_safe = True

    def __init__(self, spec: PartSpec, prefix: str = ""):
        super().__init__(spec, prefix)
        p = spec.get()
        self.hidden, self.heads = int(p["hidden_size"]), int(p["num_heads"])
        self.d, self.dv, self.eps = int(p["head_dim"]), int(p["v_dim"]), float(p["eps"])
        self.decay = tuple(float(v) for v in p["decay"])
        if len(self.decay) != self.heads:
            raise ValueError(f"lightning_attention: {len(self.decay)} decays for {self.heads} heads")
        if self.d > 256:
            raise ValueError(f"lightning_attention: head_dim {self.d}; the scan kernel takes up to 256")
        names = dict(p.get("tensor_names") or ())
        if sorted(names) != sorted(_KEYS):
            raise ValueError(f"a lightning_attention spec names its tensors: tensor_names with the keys {_KEYS}")
        self.names = {k: prefix + str(v) for k, v in names.items()}
        self.w_in: Optional[torch.Tensor] = None
        self.w_o: Optional[torch.Tensor] = None
        self.w_norm: Optional[torch.Tensor] = None
        self.decay_dev: Optional[torch.Tensor] = None

    def tensor_specs(self) -> List[TensorSpec]:
        n, H, qk, vv = self.names, self.hidden, self.heads * self.d, self.heads * self.dv
        return [TensorSpec(n["q"], (qk, H)), TensorSpec(n["k"], (qk, H)), TensorSpec(n["v"], (vv, H)),
                TensorSpec(n["g"], (vv, H)), TensorSpec(n["o"], (H, vv)),
                TensorSpec(n["norm"], (vv,), role="vector", init=("one_plus_normal", 0.1))]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        n = self.names
        self.w_in = torch.cat([tensors[n["q"]], tensors[n["k"]], tensors[n["v"]], tensors[n["g"]]], dim=0).contiguous()
        self.w_o, self.w_norm = tensors[n["o"]], tensors[n["norm"]].contiguous()
        self.decay_dev = torch.tensor(self.decay, dtype=torch.float32, device=self.w_in.device)

    def cache_need(self):
        return StateNeed((self.heads, self.d, self.dv))

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: StateCacheView) -> torch.Tensor:
        qk, vv = self.heads * self.d, self.heads * self.dv
        a = linear(x, self.w_in)                                     # [T, 2 qk + 2 vv]: q | k | v | g
        o = ops.lightning_scan(a[:, :qk], a[:, qk:2 * qk], a[:, 2 * qk:2 * qk + vv], self.decay_dev, cache.state,
                               ctx.q_start, ctx.state_slots, ctx.num_seqs, ctx.err, max_q_len=ctx.max_q_len)
        y = ops.gated_rmsnorm(o, a[:, 2 * qk + vv:], self.w_norm, self.eps, x.dtype)
        return linear(y, self.w_o)
