"""Fevolorn as a ``ModelSpec``: a decoder over several residual streams
(``hyper_connections`` blocks with a dynamic-tanh norm and a per-channel scale on
every sublayer's result) whose layers have one of two mixers: ``lightning_attention``
(linear attention with a fixed decay per head) or ``parallel`` (windowed
grouped-query attention with per-head query/key norms and no positions, beside a
Mamba ``selective_scan``; their outputs are normalised and averaged), each followed
by a dense feed-forward (tanh-gelu gate), routed experts with a shared expert, or
nothing.  A range of layers may run several times with the same weights; every run
has a cache slot of its own.  The embedding is scaled by a constant; the output is
the model's norm on the sum of the streams and the embedding table as the head.

Tensor names: ``embed``, ``final.norm`` (+ ``.alpha``, ``.b``), and per layer ``l<i>.`` +
``norm1|norm2`` (+ ``.alpha``, ``.b``), ``ls1|ls2``, ``hc1|hc2`` + ``.in|.mix|.out``,
``mix.*`` (lightning: q, k, v, g, o, norm; parallel: left.q|k|v|o, left.q.norm,
left.k.norm, left.out, right.in|conv|conv.b|x|dt|dt.b|A_log|D|o, right.out) and
``mlp.*`` (dense: gate, up, down; experts: router, correction, e<k>.gate|up|down,
shared.gate|up|down, shared.sg).
"""
from __future__ import annotations

from ..config.fevolorn_config import FevolornConfig
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, Run

_GUD = {"gate": "gate", "up": "up", "down": "down"}


def _tanh_norm(size: int, name: str) -> PartSpec:
    return PartSpec.of("dynamic_tanh", size=size, name=name, alpha_name=name + ".alpha", shift_name=name + ".b")


def fevolorn_spec(cfg: FevolornConfig) -> ModelSpec:
    H = cfg.width
    layers = []
    for i, L in enumerate(cfg.layers):
        m = L.mixer
        if L.kind == "lightning":
            mixer = PartSpec.of("lightning_attention", hidden_size=H, num_heads=m.heads, head_dim=m.dim, v_dim=m.vdim,
                                decay=m.decay, eps=cfg.eps, tensor_prefix="mix.",
                                tensor_names={"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "norm": "norm"})
        else:
            a, b = m.left, m.right
            left = PartSpec.of("attention", hidden_size=H, num_heads=a.heads, num_kv_heads=a.kv_heads, head_dim=a.dim,
                               v_dim=a.vdim, window=a.window, scale=a.scale, qk_norm=cfg.eps, position=None,
                               tensor_prefix="left.",
                               tensor_names={"q": "q", "k": "k", "v": "v", "o": "o", "q_norm": "q.norm",
                                             "k_norm": "k.norm"})
            right = PartSpec.of("selective_scan", hidden_size=H, inner=b.inner, state=b.state, dt_rank=b.dt_rank,
                                conv=b.conv, tensor_prefix="right.",
                                tensor_names={"in": "in", "conv": "conv", "conv_bias": "conv.b", "x": "x", "dt": "dt",
                                              "dt_bias": "dt.b", "a_log": "A_log", "d": "D", "o": "o"})
            mixer = PartSpec.of("parallel", hidden_size=H, eps=cfg.eps, branches=(left, right), tensor_prefix="mix.",
                                tensor_names={"out": ("left.out", "right.out")})
        ffn = None
        if L.mlp is not None and L.mlp.kind == "dense":
            ffn = PartSpec.of("gated_mlp", hidden_size=H, intermediate_size=L.mlp.ff, activation="gelu_tanh",
                              tensor_prefix="mlp.", tensor_names=_GUD)
        elif L.mlp is not None:
            f = L.mlp
            names = {"router": "router", "correction": "correction", "gate": "e{e}.gate", "up": "e{e}.up",
                     "down": "e{e}.down"}
            shared = None
            if f.shared_ff is not None:
                shared = PartSpec.of("gated_mlp", hidden_size=H, intermediate_size=f.shared_ff, activation="silu",
                                     tensor_prefix="shared.", tensor_names=_GUD)
                names["shared_gate"] = "shared.sg"
            ffn = PartSpec.of("routed_experts", hidden_size=H, inner_size=f.ff, num_experts=f.experts, top=f.top,
                              limit=None, alpha=1.0, up_shift=0.0, score="sigmoid", route_scale=f.route_scale,
                              shared=shared, tensor_prefix="mlp.", tensor_names=names)
        block = PartSpec.of("hyper_connections", hidden_size=H, streams=cfg.streams,
                            tensor_names={"read1": "hc1.in", "mix1": "hc1.mix", "write1": "hc1.out", "scale1": "ls1",
                                          "read2": "hc2.in", "mix2": "hc2.mix", "write2": "hc2.out", "scale2": "ls2"})
        layers.append(LayerSpec(block="hyper_connections", mixer=mixer, ffn=ffn,
                                norms=(_tanh_norm(H, "norm1"), _tanh_norm(H, "norm2")), prefix=f"l{i}.",
                                block_params=block))
    # every run of a layer, repeated or not, owns the cache slot of its place in the order
    order = tuple(Run(layer=layer, cache=at) for at, layer in enumerate(cfg.order()))
    return ModelSpec(
        hidden_size=H, vocab_size=cfg.vocab,
        embedding=PartSpec.of("token_embedding", vocab_size=cfg.vocab, hidden_size=H, name="embed",
                              scale=cfg.embedding_scale),
        layers=tuple(layers), order=order, final_norm=_tanh_norm(H, "final.norm"),
        head=PartSpec.of("lm_head", vocab_size=cfg.vocab, hidden_size=H, name="lm_head", tied_to="embed"),
        max_positions=cfg.max_positions, streams=cfg.streams)


register_architecture("Fevolorn", FevolornConfig.from_json, fevolorn_spec)
