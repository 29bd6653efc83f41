"""Typed configuration of the Fasulix decoder, read from ``config.json``.

A Fasulix model is a list of layers, each with a mixer of one of three kinds
(``mingru``; ``latent_attention``: causal, softmax with a sink;
``latent_attention_2``: sliding window, plain softmax, optionally reading an
earlier layer's cached rows through ``kv_from``) and a feed-forward of routed
experts, or none.  Keys:

    architecture: "Fasulix"      vocab, width      norm: {eps}
    layers: [{type, mixer: {...}, mlp: {...} | null}, ...]
      mingru mixer:  {width}
      latent mixers: {heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, rot: {base, dims},
                      mask: {size} (latent_attention_2), kv_from (optional)}
      mlp:           {kind: "moe", expert: {ff, limit}, router: {experts, top}}

Every size and constant is taken from these keys; optional ``max_positions`` (default
131,072) bounds a request's length for the engine, which sizes its cache pools by it (the
design itself has no bound, and trace replay does not look at it).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .model_config import ConfigError

MIXER_KINDS = ("mingru", "latent_attention", "latent_attention_2")


@dataclass(frozen=True)
class FasulixMixer:
    kind: str
    width: int = 0                    # mingru
    heads: int = 0                    # latent attention
    dim: int = 0
    rot_dim: int = 0
    vdim: int = 0
    q_rank: int = 0
    kv_rank: int = 0
    scale: float = 0.0
    rot_base: float = 0.0
    rot_dims: int = 0
    window: Optional[int] = None
    kv_from: Optional[int] = None


@dataclass(frozen=True)
class FasulixExperts:
    ff: int
    limit: float
    experts: int
    top: int


@dataclass(frozen=True)
class FasulixLayer:
    mixer: FasulixMixer
    mlp: Optional[FasulixExperts]


@dataclass(frozen=True)
class FasulixConfig:
    vocab: int
    width: int
    eps: float
    layers: Tuple[FasulixLayer, ...]
    max_positions: int = 1 << 17
    torch_dtype: str = "bfloat16"

    @staticmethod
    def from_json(raw: Mapping[str, Any]) -> "FasulixConfig":
        def need(d: Mapping[str, Any], key: str, where: str):
            if not isinstance(d, Mapping) or key not in d:
                raise ConfigError(f"config.json: {where} lacks {key!r}")
            return d[key]

        layers = []
        raw_layers = need(raw, "layers", "the configuration")
        if not isinstance(raw_layers, (list, tuple)) or not raw_layers:
            raise ConfigError("config.json: layers must be a non-empty list")
        for i, L in enumerate(raw_layers):
            where = f"layers[{i}]"
            kind = str(need(L, "type", where))
            if kind not in MIXER_KINDS:
                raise ConfigError(f"config.json: {where} has mixer type {kind!r}; known: {list(MIXER_KINDS)}")
            m = need(L, "mixer", where)
            if kind == "mingru":
                mixer = FasulixMixer(kind, width=int(need(m, "width", where + ".mixer")))
            else:
                rot = m.get("rot") or {}
                rot_dim = int(need(m, "rot_dim", where + ".mixer"))
                window = None
                if kind == "latent_attention_2":
                    window = int(need(need(m, "mask", where + ".mixer"), "size", where + ".mixer.mask"))
                    if window < 1:
                        raise ConfigError(f"config.json: {where}.mixer.mask.size must be positive")
                kv_from = m.get("kv_from")
                if kv_from is not None:
                    kv_from = int(kv_from)
                    if not 0 <= kv_from < i:
                        raise ConfigError(f"config.json: {where}.mixer.kv_from names layer {kv_from}, not an earlier layer")
                mixer = FasulixMixer(
                    kind, heads=int(need(m, "heads", where + ".mixer")), dim=int(need(m, "dim", where + ".mixer")),
                    rot_dim=rot_dim, vdim=int(need(m, "vdim", where + ".mixer")),
                    q_rank=int(need(m, "q_rank", where + ".mixer")), kv_rank=int(need(m, "kv_rank", where + ".mixer")),
                    scale=float(need(m, "scale", where + ".mixer")),
                    rot_base=float(rot.get("base", 10000.0)) if rot_dim else 0.0,
                    rot_dims=int(rot.get("dims", rot_dim)) if rot_dim else 0, window=window, kv_from=kv_from)
                if mixer.rot_dim % 2 or mixer.rot_dims % 2 or mixer.rot_dims > mixer.rot_dim:
                    raise ConfigError(f"config.json: {where}.mixer: rot_dim and rot.dims must be even, rot.dims <= rot_dim")
            mlp = L.get("mlp")
            experts = None
            if mlp is not None:
                if mlp.get("kind", "moe") != "moe":
                    raise ConfigError(f"config.json: {where}.mlp.kind {mlp.get('kind')!r}; known: ['moe']")
                ex, ro = need(mlp, "expert", where + ".mlp"), need(mlp, "router", where + ".mlp")
                experts = FasulixExperts(ff=int(need(ex, "ff", where + ".mlp.expert")),
                                         limit=float(need(ex, "limit", where + ".mlp.expert")),
                                         experts=int(need(ro, "experts", where + ".mlp.router")),
                                         top=int(need(ro, "top", where + ".mlp.router")))
                if not 1 <= experts.top <= experts.experts:
                    raise ConfigError(f"config.json: {where}.mlp.router: top {experts.top} of {experts.experts} experts")
            layers.append(FasulixLayer(mixer, experts))
        for i, L in enumerate(layers):
            j = L.mixer.kv_from
            if j is not None:
                src = layers[j].mixer
                if src.kind == "mingru" or src.kv_from is not None:
                    raise ConfigError(f"config.json: layers[{i}].mixer.kv_from names layer {j}, which keeps no rows of its own")
                if (src.kv_rank, src.rot_dim, src.rot_dims, src.rot_base) != \
                        (L.mixer.kv_rank, L.mixer.rot_dim, L.mixer.rot_dims, L.mixer.rot_base):
                    raise ConfigError(f"config.json: layers[{i}] reads the rows of layer {j}: kv_rank, rot_dim and "
                                      f"rotation must be equal")
        return FasulixConfig(vocab=int(need(raw, "vocab", "the configuration")),
                             width=int(need(raw, "width", "the configuration")),
                             eps=float(need(need(raw, "norm", "the configuration"), "eps", "norm")),
                             layers=tuple(layers), max_positions=int(raw.get("max_positions", 1 << 17)),
                             torch_dtype=str(raw.get("torch_dtype", "bfloat16")))
