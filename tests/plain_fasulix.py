"""A plain, slow Fasulix in float64, written from the design's equations: one
function per mechanism, whole sequences only, no cache, no batching.  It is what
the engine's Fasulix is compared with and shares no code with it.

Weights: a dict name -> float64 tensor.  Configuration: the dict of config.json.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional

import torch

F64 = torch.float64


def read_model_dir(model_dir: str, round_to: Optional[torch.dtype] = None):
    from safetensors import safe_open
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    w = {}
    with safe_open(os.path.join(model_dir, "model.safetensors"), framework="pt") as f:
        for n in f.keys():
            t = f.get_tensor(n)
            w[n] = (t.to(round_to) if round_to is not None else t).to(F64)
    return cfg, w


def unit_rms(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """x over its root mean square (eps under the root), times a weight."""
    return x / torch.sqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps) * weight


def rotate_pairs(x: torch.Tensor, positions: torch.Tensor, base: float, dims: int) -> torch.Tensor:
    """x [T, ..., d]: the first ``dims`` of the last axis are rotated, entry 2i with 2i+1, by the
    angle position * base^(-2i/dims); the rest passes."""
    out = x.clone()
    for i in range(dims // 2):
        ang = positions.to(F64) * (base ** (-2.0 * i / dims))
        shape = [x.shape[0]] + [1] * (x.dim() - 2)
        c, s = torch.cos(ang).view(shape), torch.sin(ang).view(shape)
        a, b = x[..., 2 * i], x[..., 2 * i + 1]
        out[..., 2 * i] = a * c - b * s
        out[..., 2 * i + 1] = b * c + a * s
    return out


def latent_rows(w: Dict[str, torch.Tensor], p: str, m: dict, x: torch.Tensor, eps: float):
    """What a latent-attention layer keeps per token: (normalised latent [T, kv_rank], rotated shared
    key part [T, rot_dim])."""
    T = x.shape[0]
    down = x @ w[p + "dkv"].t()
    c = unit_rms(down[:, : m["kv_rank"]], w[p + "dkv.norm"], eps)
    shared = down[:, m["kv_rank"]:]
    if m["rot_dim"]:
        shared = rotate_pairs(shared, torch.arange(T), m["rot"]["base"], m["rot"]["dims"])
    return c, shared


def latent_attention(w: Dict[str, torch.Tensor], p: str, m: dict, x: torch.Tensor, eps: float, rows,
                     window: Optional[int], sink: bool) -> torch.Tensor:
    """Token by token, head by head, with explicit loops over the visible keys."""
    T = x.shape[0]
    H, dn, dr, dv = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    c, shared = rows
    cq = unit_rms(x @ w[p + "dq"].t(), w[p + "dq.norm"], eps)
    q = (cq @ w[p + "uq"].t()).view(T, H, dn + dr)
    q_plain = q[:, :, :dn]
    q_rot = rotate_pairs(q[:, :, dn:], torch.arange(T), m["rot"]["base"], m["rot"]["dims"]) if dr else q[:, :, dn:]
    keys = (c @ w[p + "uk"].t()).view(T, H, dn)
    vals = (c @ w[p + "uv"].t()).view(T, H, dv)
    out = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        first = 0 if window is None else max(0, t - window + 1)
        for h in range(H):
            s = (keys[first:t + 1, h] @ q_plain[t, h] + shared[first:t + 1] @ q_rot[t, h]) * m["scale"]
            top = s.max()
            if sink:
                top = torch.maximum(top, w[p + "sink"][h])
            e = torch.exp(s - top)
            denom = e.sum() + (torch.exp(w[p + "sink"][h] - top) if sink else 0.0)
            out[t, h] = (e / denom) @ vals[first:t + 1, h]
    return out.reshape(T, H * dv) @ w[p + "o"].t()


def mingru(w: Dict[str, torch.Tensor], p: str, x: torch.Tensor) -> torch.Tensor:
    z = torch.sigmoid(x @ w[p + "z"].t() + w[p + "z.b"])
    u = x @ w[p + "x"].t() + w[p + "x.b"]
    cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    g = x @ w[p + "g"].t()
    state = torch.zeros(z.shape[1], dtype=F64)
    outs = []
    for t in range(x.shape[0]):
        state = (1.0 - z[t]) * state + z[t] * cand[t]
        outs.append(state * g[t] * torch.sigmoid(g[t]))
    return torch.stack(outs) @ w[p + "o"].t()


def expert(w: Dict[str, torch.Tensor], p: str, x: torch.Tensor, limit: float) -> torch.Tensor:
    g = torch.clamp(x @ w[p + "gate"].t(), max=limit)
    u = torch.clamp(x @ w[p + "up"].t(), min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].t()


def routed_experts(w: Dict[str, torch.Tensor], p: str, mlp: dict, x: torch.Tensor) -> torch.Tensor:
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    scores = torch.softmax(x @ w[p + "router"].t(), dim=-1)
    out = torch.zeros_like(x)
    for t in range(x.shape[0]):
        order = sorted(range(E), key=lambda e: (-float(scores[t, e]), e))[:top]
        for e in order:
            out[t] += scores[t, e] * expert(w, p + f"e{e}.", x[t:t + 1], mlp["expert"]["limit"])[0]
    return out


def gated(w: Dict[str, torch.Tensor], name: str, inp: torch.Tensor, result: torch.Tensor) -> torch.Tensor:
    return result * torch.sigmoid(inp @ w[name].t() + w[name + ".b"])


def streams(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int]) -> List[torch.Tensor]:
    """The stream after the embedding and after every layer (depth-averaged), [T, width] each."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(tokens, dtype=torch.long)]
    results = [x]
    kept = {}
    out = [x]
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        a = unit_rms(x, w[p + "norm1"], eps)
        if layer["type"] == "mingru":
            y = mingru(w, p + "mix.", a)
        else:
            if "kv_from" in m:
                rows = kept[m["kv_from"]]
            else:
                rows = kept[i] = latent_rows(w, p + "mix.", m, a, eps)
            window = m["mask"]["size"] if layer["type"] == "latent_attention_2" else None
            y = latent_attention(w, p + "mix.", m, a, eps, rows, window, sink=layer["type"] == "latent_attention")
        x = x + unit_rms(gated(w, p + "rg1", a, y), w[p + "norm1b"], eps)
        if layer.get("mlp") is not None:
            b = unit_rms(x, w[p + "norm2"], eps)
            x = x + unit_rms(gated(w, p + "rg2", b, routed_experts(w, p + "mlp.", layer["mlp"], b)),
                             w[p + "norm2b"], eps)
        results.append(x)
        x = sum(w[p + "dwa"][j] * results[j] for j in range(i + 2))
        out.append(x)
    return out


def logits(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int]) -> torch.Tensor:
    x = streams(cfg, w, tokens)[-1]
    return unit_rms(x, w["final.norm"], cfg["norm"]["eps"]) @ w["embed"].t()


def greedy(cfg: dict, w: Dict[str, torch.Tensor], prompt: List[int], n: int) -> List[int]:
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(torch.argmax(logits(cfg, w, toks)[-1])))
    return toks[len(prompt):]
