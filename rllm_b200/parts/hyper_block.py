"""``hyper_connections``: a pre-norm layer over several residual streams.

Instead of one residual x there are S streams x_1 .. x_S (float32 [S, T, H]; the
model starts them all from the embedding's output and its head reads their sum).
Sublayer q (1: the mixer, 2: the feed-forward) with its learned a_q [S], M_q [S, S]
and b_q [S]:

    u   = sum_s a_q[s] x_s
    y   = sublayer(norm_q(u)) * g_q                 (g_q [H]: a per-channel scale, optional)
    x_t <- sum_s M_q[s, t] x_s + b_q[t] y           for all t at once, from the old streams

(M is indexed [from, to]).  A layer without a feed-forward has only the first
sublayer.  With S = 1, a = b = M = 1 this is the ordinary pre-norm layer.

The streams are read and written by element-wise kernels in float32; the
write-back of a sublayer, the read of the next one (this layer's feed-forward or
the next layer's mixer) and the norm on that read are one kernel where the norm
needs no statistics (``elementwise()`` of the norm part); another norm runs as a
kernel of its own on the float32 read.

A caller that puts a list under ``ctx.extras["residual_trace"]`` gets the sum of the streams after every
layer run appended to it (float32 [T, H], from the layer's last kernel): what the tests compare layer by layer.

norms: two (before the mixer, before the feed-forward).  params: hidden_size,
streams, tensor_names (keys "read1", "mix1", "write1", "read2", "mix2", "write2",
and optionally "scale1", "scale2": names below the layer's prefix).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops
from .base import FeedForward, Mixer, Norm, Part, PreparedInput, StepContext
from .registry import register_part
from .spec import PartSpec, TensorSpec

_KEYS = ("read1", "mix1", "write1", "read2", "mix2", "write2")


def _fused(norm: Norm):
    return norm.elementwise() if hasattr(norm, "elementwise") else None


@register_part("block", "hyper_connections")
class HyperConnectionsBlock(Part):
    takes_next_block = True

    def __init__(self, mixer: Mixer, ffn: Optional[FeedForward], norms: List[Norm], spec: PartSpec, prefix: str = ""):
        super().__init__(spec, prefix)
        if len(norms) != 2:
            raise ValueError("a hyper_connections block has two norms: before the mixer and before the feed-forward")
        self.mixer, self.ffn, self.norms = mixer, ffn, norms
        p = spec.get()
        self.hidden, self.streams = int(p["hidden_size"]), int(p["streams"])
        if not 1 <= self.streams <= ops.HS_MAX_STREAMS:
            raise ValueError(f"streams {self.streams}: the kernels take 1 to {ops.HS_MAX_STREAMS}")
        names = dict(p.get("tensor_names") or ())
        if not set(_KEYS) <= set(names) or set(names) - set(_KEYS) - {"scale1", "scale2"}:
            raise ValueError(f"a hyper_connections spec names its tensors: tensor_names with the keys {_KEYS} "
                             f"(and optionally scale1, scale2)")
        self.names = {k: prefix + str(v) for k, v in names.items()}
        self.read: List[Optional[torch.Tensor]] = [None, None]
        self.mix: List[Optional[torch.Tensor]] = [None, None]
        self.write: List[Optional[torch.Tensor]] = [None, None]
        self.scale: List[Optional[torch.Tensor]] = [None, None]

    @property
    def graph_safe(self) -> bool:
        return True

    def parts(self):
        return [self, self.norms[0], self.mixer] + ([self.norms[1], self.ffn] if self.ffn is not None else [])

    def _sublayers(self):
        return (1, 2) if self.ffn is not None else (1,)

    def tensor_specs(self) -> List[TensorSpec]:
        n, S, specs = self.names, self.streams, []
        for q in self._sublayers():
            specs += [TensorSpec(n[f"read{q}"], (S,), role="vector", init=("one_plus_normal", 0.2)),
                      TensorSpec(n[f"mix{q}"], (S, S), role="vector", init=("normal", 0.3)),
                      TensorSpec(n[f"write{q}"], (S,), role="vector", init=("one_plus_normal", 0.2))]
            if f"scale{q}" in n:
                specs.append(TensorSpec(n[f"scale{q}"], (self.hidden,), role="vector", init=("one_plus_normal", 0.2)))
        return specs

    def ignored_tensors(self) -> List[str]:
        """A layer without a feed-forward uses none of its second sublayer's tensors: a file that carries
        them all the same is no error."""
        if self.ffn is not None:
            return []
        out = [v for k, v in self.names.items() if k.endswith("2")]
        nrm = self.norms[1]
        return out + [getattr(nrm, a) for a in ("name", "alpha_name", "shift_name") if hasattr(nrm, a)]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        n = self.names
        for q in self._sublayers():
            # the streams' coefficients are float32 on the device whatever the run's dtype
            self.read[q - 1] = tensors[n[f"read{q}"]].float().contiguous()
            self.mix[q - 1] = tensors[n[f"mix{q}"]].float().contiguous()
            self.write[q - 1] = tensors[n[f"write{q}"]].float().contiguous()
            if f"scale{q}" in n:
                self.scale[q - 1] = tensors[n[f"scale{q}"]].contiguous()

    def _scale_for(self, q: int, norm_args):
        """The sublayer's channel scale in the dtype the write kernel reads its vectors in."""
        g = self.scale[q]
        if g is not None and norm_args is not None and g.dtype is not norm_args[1].dtype:
            g = self.scale[q] = g.to(norm_args[1].dtype).contiguous()
        return g

    def first_input(self, xs: torch.Tensor, act_dtype: torch.dtype) -> torch.Tensor:
        """The mixer's input from the streams: the read and the first norm."""
        fused = _fused(self.norms[0])
        u = ops.streams_read(xs, self.read[0], fused, act_dtype)
        return u if fused is not None else self.norms[0].forward(u, act_dtype)

    def _write(self, xs, y, q: int, nxt_read, nxt_norm: Optional[Norm], act_dtype, sum_out=None):
        """Sublayer q's write-back and, if a reader follows, its input."""
        fused = _fused(nxt_norm) if nxt_norm is not None else None
        u = ops.streams_write(xs, y, self._scale_for(q, fused), self.mix[q], self.write[q], next_read=nxt_read,
                              norm=fused, sum_out=sum_out)
        if u is not None and fused is None and nxt_norm is not None:
            u = nxt_norm.forward(u, act_dtype)
        return u

    def forward(self, xs: torch.Tensor, pending, ctx: StepContext, cache, next_block=None):
        if xs.dim() != 3 or xs.shape[0] != self.streams:
            raise RuntimeError(f"a hyper_connections block reads {self.streams} streams; the model keeps "
                               f"{tuple(xs.shape)}")
        if isinstance(pending, PreparedInput) and pending.key is self:
            a = pending.x
        else:
            a = self.first_input(xs, ctx.act_dtype)
        y = self.mixer.forward(a, ctx, cache)
        follows = isinstance(next_block, HyperConnectionsBlock) and next_block.streams == self.streams
        nxt_read = next_block.read[0] if follows else None
        nxt_norm = next_block.norms[0] if follows else None
        trace = ctx.extras.get("residual_trace")                  # a list: the sum of the streams after every layer
        sums = torch.empty(xs.shape[1:], dtype=torch.float32, device=xs.device) if trace is not None else None
        if self.ffn is None:
            u = self._write(xs, y, 0, nxt_read, nxt_norm, ctx.act_dtype, sum_out=sums)
        else:
            b = self._write(xs, y, 0, self.read[1], self.norms[1], ctx.act_dtype)
            u = self._write(xs, self.ffn.forward(b), 1, nxt_read, nxt_norm, ctx.act_dtype, sum_out=sums)
        if trace is not None:
            trace.append(sums)
        return xs, (PreparedInput(u, next_block) if u is not None else None)
