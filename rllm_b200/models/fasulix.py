"""Fasulix as a ``ModelSpec``: a decoder whose layers mix three kinds of mixers
(a minGRU recurrence, latent attention with a softmax sink, windowed latent
attention that may read an earlier layer's cached rows), each followed by a
feed-forward of routed experts, in ``sandwich_gated`` blocks (norms on both sides
of a sublayer, a sigmoid gate from the sublayer's input) with a depth-weighted
stream: layer i averages the embedding's output and the results of layers 0 .. i
with its own i + 2 learned numbers.  The output is the model's norm and the
embedding table as the head.

Tensor names: ``embed``, ``final.norm``, and per layer ``l<i>.`` + ``norm1``,
``norm1b``, ``norm2``, ``norm2b``, ``rg1``, ``rg1.b``, ``rg2``, ``rg2.b``,
``dwa``, ``mix.*`` (mingru: z, z.b, x, x.b, g, o; latent: dq, dq.norm, uq, dkv,
dkv.norm, uk, uv, sink, o) and ``mlp.router``, ``mlp.e<k>.gate|up|down``.
"""
from __future__ import annotations

from ..config.fasulix_config import FasulixConfig
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, Run

EXPERT_ALPHA = 1.702          # the experts' activation: g * sigmoid(1.702 g) * (u + 1)


def fasulix_spec(cfg: FasulixConfig) -> ModelSpec:
    H = cfg.width
    layers, order = [], []
    for i, L in enumerate(cfg.layers):
        m = L.mixer
        if m.kind == "mingru":
            mixer = PartSpec.of("mingru", hidden_size=H, width=m.width, tensor_prefix="mix.",
                                tensor_names={"z": "z", "z_bias": "z.b", "x": "x", "x_bias": "x.b", "g": "g", "o": "o"})
        else:
            position = PartSpec.of("rotary", head_dim=m.rot_dim, rotary_dim=m.rot_dims, theta=m.rot_base,
                                   scaling=None, interleaved=True) if m.rot_dims else None
            mixer = PartSpec.of("latent_attention", hidden_size=H, num_heads=m.heads, nope_dim=m.dim,
                                rot_dim=m.rot_dim, v_dim=m.vdim, q_rank=m.q_rank, kv_rank=m.kv_rank, scale=m.scale,
                                eps=cfg.eps, window=m.window, sink=m.kind == "latent_attention",
                                shares_kv=m.kv_from is not None, position=position, tensor_prefix="mix.",
                                tensor_names={"dq": "dq", "dq_norm": "dq.norm", "uq": "uq", "dkv": "dkv",
                                              "dkv_norm": "dkv.norm", "uk": "uk", "uv": "uv", "sink": "sink",
                                              "o": "o"})
        ffn = None
        if L.mlp is not None:
            ffn = PartSpec.of("routed_experts", hidden_size=H, inner_size=L.mlp.ff, num_experts=L.mlp.experts,
                              top=L.mlp.top, limit=L.mlp.limit, alpha=EXPERT_ALPHA, up_shift=1.0,
                              tensor_prefix="mlp.",
                              tensor_names={"router": "router", "gate": "e{e}.gate", "up": "e{e}.up",
                                            "down": "e{e}.down"})
        norms = tuple(PartSpec.of("rmsnorm", size=H, eps=cfg.eps, name=n)
                      for n in ("norm1", "norm1b", "norm2", "norm2b"))
        block = PartSpec.of("sandwich_gated", hidden_size=H, depth_levels=i + 2,
                            tensor_names={"gate1": "rg1", "gate1_bias": "rg1.b", "gate2": "rg2",
                                          "gate2_bias": "rg2.b", "depth": "dwa"})
        layers.append(LayerSpec(block="sandwich_gated", mixer=mixer, ffn=ffn, norms=norms, prefix=f"l{i}.",
                                block_params=block))
        order.append(Run(layer=i, cache=i if m.kv_from is None else m.kv_from))
    return ModelSpec(
        hidden_size=H, vocab_size=cfg.vocab,
        embedding=PartSpec.of("token_embedding", vocab_size=cfg.vocab, hidden_size=H, name="embed"),
        layers=tuple(layers), order=tuple(order),
        final_norm=PartSpec.of("rmsnorm", size=H, eps=cfg.eps, name="final.norm"),
        head=PartSpec.of("lm_head", vocab_size=cfg.vocab, hidden_size=H, name="lm_head", tied_to="embed"),
        max_positions=cfg.max_positions)


register_architecture("Fasulix", FasulixConfig.from_json, fasulix_spec)
