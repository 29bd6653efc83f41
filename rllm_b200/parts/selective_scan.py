"""``selective_scan``: the Mamba mixer.

    [x | z] = W_in h                                    (inner channels each)
    c_t = silu(conv_bias + sum_j conv[ch, j] x_{t - (taps - 1) + j})      (zeros before the start)
    [r | B | C] = W_x c_t                               (dt_rank, state, state values)
    dt = softplus(W_dt r + dt_bias)                     (one per channel)
    S[ch, n] <- exp(dt A[ch, n]) S[ch, n] + dt c_t[ch] B[n],   A = -exp(A_log)
    y[ch] = sum_n S[ch, n] C[n] + D[ch] c_t[ch],   out = W_o (y * silu(z))

Per request the part keeps two states, both float32: S (as [state, inner]) and
the convolution's last taps - 1 inputs ([taps - 1, inner]); both start at zero.
The projections are matrix products in the activation dtype (W_dt's result is
kept in float32); step sizes, decays, exponentials, the state and the sums are
float32 in the scan kernel.

params: hidden_size, inner, state, dt_rank, conv (taps), tensor_names (keys "in",
"conv", "conv_bias", "x", "dt", "dt_bias", "a_log", "d", "o").
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..kernels import ops
from .base import Mixer, StepContext
from .linear import linear
from .registry import register_part
from .spec import PartSpec, StateNeed, TensorSpec

_KEYS = ("in", "conv", "conv_bias", "x", "dt", "dt_bias", "a_log", "d", "o")


@register_part("mixer", "selective_scan")
class SelectiveScan(Mixer):
    graph_safe = True

    def __init__(self, spec: PartSpec, prefix: str = ""):
        super().__init__(spec, prefix)
        p = spec.get()
        self.hidden, self.inner = int(p["hidden_size"]), int(p["inner"])
        self.state, self.dt_rank, self.taps = int(p["state"]), int(p["dt_rank"]), int(p["conv"])
        if min(self.inner, self.state, self.dt_rank, self.taps) < 1:
            raise ValueError("selective_scan: inner, state, dt_rank and conv must be positive")
        if self.state > 128:
            raise ValueError(f"selective_scan: state {self.state}; the scan kernel keeps up to 128 a channel")
        names = dict(p.get("tensor_names") or ())
        if sorted(names) != sorted(_KEYS):
            raise ValueError(f"a selective_scan spec names its tensors: tensor_names with the keys {_KEYS}")
        self.names = {k: prefix + str(v) for k, v in names.items()}
        self.w: Dict[str, torch.Tensor] = {}

    def tensor_specs(self) -> List[TensorSpec]:
        n, E, N, R, H = self.names, self.inner, self.state, self.dt_rank, self.hidden
        return [TensorSpec(n["in"], (2 * E, H)),
                TensorSpec(n["conv"], (E, self.taps), role="vector", init=("normal", 0.4)),
                TensorSpec(n["conv_bias"], (E,), role="vector", init=("normal", 0.1)),
                TensorSpec(n["x"], (R + 2 * N, E), init=("normal", 0.05)),
                TensorSpec(n["dt"], (E, R), init=("normal", 0.3)),
                TensorSpec(n["dt_bias"], (E,), role="vector", init=("normal", 0.5)),
                TensorSpec(n["a_log"], (E, N), role="vector", init=("normal", 0.5)),
                TensorSpec(n["d"], (E,), role="vector", init=("one_plus_normal", 0.1)),
                TensorSpec(n["o"], (H, E))]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.w = {k: tensors[n].contiguous() for k, n in self.names.items()}
        small = self.w["a_log"].dtype                     # the small tensors go to the kernels in one dtype
        for k in ("conv", "conv_bias", "dt_bias", "d"):
            self.w[k] = self.w[k].to(small).contiguous()

    def cache_need(self):
        return (StateNeed((self.state, self.inner)), StateNeed((self.taps - 1, self.inner)))

    def forward(self, x: torch.Tensor, ctx: StepContext, cache) -> torch.Tensor:
        scan_state, tail = cache
        w, E, N, R = self.w, self.inner, self.state, self.dt_rank
        xz = linear(x, w["in"])                                            # [T, 2 E]: x | z
        c = ops.causal_conv(xz[:, :E], w["conv"], w["conv_bias"], tail.state, ctx.q_start, ctx.token_seq,
                            ctx.state_slots, ctx.num_seqs, ctx.num_tokens > ctx.num_decode, ctx.err)
        proj = linear(c, w["x"])                                           # [T, R + 2 N]: r | B | C
        dt_raw = linear(proj[:, :R], w["dt"], out_dtype=torch.float32)     # [T, E]
        y = ops.selective_scan(c, dt_raw, w["dt_bias"], proj, R, R + N, w["a_log"], w["d"], xz[:, E:],
                               scan_state.state, ctx.q_start, ctx.state_slots, ctx.num_seqs, ctx.err,
                               max_q_len=ctx.max_q_len)
        return linear(y, w["o"])
