"""Typed configuration of the Fevolorn decoder, read from ``config.json``.

A Fevolorn model is a list of layers over several residual streams
(hyper-connections).  Each layer has a mixer of one of two kinds and a
feed-forward (dense, routed experts with a shared expert, or none); a range of
the layers may run several times in a row with the same weights.  Keys:

    architecture: "Fevolorn"     vocab, width, streams
    embedding: {scale}           norm: {eps}
    loop: {start, stop, times}   (optional: layers start .. stop-1 run `times` times)
    layers: [{type, mixer: {...}, mlp: {...} | null}, ...]
      type "lightning": mixer {heads, dim, vdim, decay: [one per head]}
      type "parallel":  mixer {left: {heads, kv_heads, dim, vdim, scale, mask: {size}},
                               right: {inner, state, dt_rank, conv}}
      mlp {kind: "dense", ff}
      mlp {kind: "moe", expert: {ff}, router: {experts, top, scale}, shared: {ff} | absent}

Every size and constant is taken from these keys; optional ``max_positions``
(default 131,072) bounds a request's length for the engine, which sizes its
cache pools by it (the design itself has no bound).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .model_config import ConfigError

MIXER_KINDS = ("lightning", "parallel")
MLP_KINDS = ("dense", "moe")


@dataclass(frozen=True)
class LightningMixer:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]


@dataclass(frozen=True)
class WindowAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int


@dataclass(frozen=True)
class ScanMixer:
    inner: int
    state: int
    dt_rank: int
    conv: int


@dataclass(frozen=True)
class ParallelMixer:
    left: WindowAttention
    right: ScanMixer


@dataclass(frozen=True)
class FevolornMlp:
    kind: str
    ff: int                           # dense: the inner size; moe: an expert's
    experts: int = 0
    top: int = 0
    route_scale: float = 1.0
    shared_ff: Optional[int] = None


@dataclass(frozen=True)
class FevolornLayer:
    kind: str
    mixer: object
    mlp: Optional[FevolornMlp]


@dataclass(frozen=True)
class FevolornConfig:
    vocab: int
    width: int
    streams: int
    eps: float
    embedding_scale: float
    layers: Tuple[FevolornLayer, ...]
    loop: Optional[Tuple[int, int, int]] = None        # (start, stop, times)
    max_positions: int = 1 << 17
    torch_dtype: str = "bfloat16"

    def order(self) -> Tuple[int, ...]:
        """The layers in the order they run."""
        n = len(self.layers)
        if self.loop is None:
            return tuple(range(n))
        a, b, times = self.loop
        return tuple(range(a)) + tuple(range(a, b)) * times + tuple(range(b, n))

    @staticmethod
    def from_json(raw: Mapping[str, Any]) -> "FevolornConfig":
        def need(d: Mapping[str, Any], key: str, where: str):
            if not isinstance(d, Mapping) or key not in d:
                raise ConfigError(f"config.json: {where} lacks {key!r}")
            return d[key]

        def positive(d, key, where) -> int:
            v = int(need(d, key, where))
            if v < 1:
                raise ConfigError(f"config.json: {where}.{key} must be positive")
            return v

        raw_layers = need(raw, "layers", "the configuration")
        if not isinstance(raw_layers, (list, tuple)) or not raw_layers:
            raise ConfigError("config.json: layers must be a non-empty list")
        layers = []
        for i, L in enumerate(raw_layers):
            where = f"layers[{i}]"
            kind = str(need(L, "type", where))
            if kind not in MIXER_KINDS:
                raise ConfigError(f"config.json: {where} has mixer type {kind!r}; known: {list(MIXER_KINDS)}")
            m, mw = need(L, "mixer", where), where + ".mixer"
            if kind == "lightning":
                heads = positive(m, "heads", mw)
                decay = tuple(float(v) for v in need(m, "decay", mw))
                if len(decay) != heads:
                    raise ConfigError(f"config.json: {mw}.decay has {len(decay)} numbers for {heads} heads")
                mixer = LightningMixer(heads, positive(m, "dim", mw), positive(m, "vdim", mw), decay)
            else:
                a, aw = need(m, "left", mw), mw + ".left"
                left = WindowAttention(positive(a, "heads", aw), positive(a, "kv_heads", aw), positive(a, "dim", aw),
                                       positive(a, "vdim", aw), float(need(a, "scale", aw)),
                                       positive(need(a, "mask", aw), "size", aw + ".mask"))
                if left.heads % left.kv_heads:
                    raise ConfigError(f"config.json: {aw}: heads {left.heads} is no multiple of kv_heads {left.kv_heads}")
                b, bw = need(m, "right", mw), mw + ".right"
                right = ScanMixer(positive(b, "inner", bw), positive(b, "state", bw), positive(b, "dt_rank", bw),
                                  positive(b, "conv", bw))
                mixer = ParallelMixer(left, right)
            mlp = L.get("mlp")
            ff = None
            if mlp is not None:
                fw = where + ".mlp"
                mk = str(need(mlp, "kind", fw))
                if mk not in MLP_KINDS:
                    raise ConfigError(f"config.json: {fw}.kind {mk!r}; known: {list(MLP_KINDS)}")
                if mk == "dense":
                    ff = FevolornMlp("dense", positive(mlp, "ff", fw))
                else:
                    ro = need(mlp, "router", fw)
                    shared = mlp.get("shared")
                    ff = FevolornMlp("moe", positive(need(mlp, "expert", fw), "ff", fw + ".expert"),
                                     experts=positive(ro, "experts", fw + ".router"),
                                     top=positive(ro, "top", fw + ".router"),
                                     route_scale=float(ro.get("scale", 1.0)),
                                     shared_ff=positive(shared, "ff", fw + ".shared") if shared is not None else None)
                    if ff.top > ff.experts:
                        raise ConfigError(f"config.json: {fw}.router: top {ff.top} of {ff.experts} experts")
            layers.append(FevolornLayer(kind, mixer, ff))
        loop = raw.get("loop")
        if loop is not None:
            a, b, times = int(need(loop, "start", "loop")), int(need(loop, "stop", "loop")), \
                int(need(loop, "times", "loop"))
            if not 0 <= a <= b <= len(layers) or times < 1:
                raise ConfigError(f"config.json: loop {dict(loop)} does not fit {len(layers)} layers")
            loop = (a, b, times) if b > a and times != 1 else None
        streams = int(raw.get("streams", 1))
        if streams < 1:
            raise ConfigError("config.json: streams must be positive")
        emb = raw.get("embedding") or {}
        return FevolornConfig(vocab=positive(raw, "vocab", "the configuration"),
                              width=positive(raw, "width", "the configuration"), streams=streams,
                              eps=float(need(need(raw, "norm", "the configuration"), "eps", "norm")),
                              embedding_scale=float(emb.get("scale", 1.0)), layers=tuple(layers), loop=loop,
                              max_positions=int(raw.get("max_positions", 1 << 17)),
                              torch_dtype=str(raw.get("torch_dtype", "bfloat16")))
