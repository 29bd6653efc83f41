"""A plain, slow Fevolorn in float64, written from the design's equations: one
function per mechanism, whole sequences only, no cache, no batching.  It is what
the engine's Fevolorn is compared with and shares no code with it.

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
            w[n] = (t.to(round_to) if round_to is not None and t.is_floating_point() else t).to(F64)
    return cfg, w


# ---------------------------------------------------------------------------
# small functions
# ---------------------------------------------------------------------------
def unit_rms(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """x over its root mean square (eps under the root), times a weight as it is."""
    return x / torch.sqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps) * weight


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z.pow(3))))


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def tanh_norm(w: Dict[str, torch.Tensor], name: str, x: torch.Tensor) -> torch.Tensor:
    """The design's norm has no statistics: tanh(alpha x) * weight + shift."""
    return torch.tanh(w[name + ".alpha"] * x) * w[name] + w[name + ".b"]


# ---------------------------------------------------------------------------
# mixers
# ---------------------------------------------------------------------------
def lightning_mixer(w: Dict[str, torch.Tensor], p: str, m: dict, h: torch.Tensor, eps: float) -> torch.Tensor:
    """Linear attention with a fixed decay per head, token by token."""
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w[p + "q"].t()).view(T, H, d)
    k = silu(h @ w[p + "k"].t()).view(T, H, d)
    v = silu(h @ w[p + "v"].t()).view(T, H, dv)
    out = torch.zeros(T, H, dv, dtype=F64)
    for hd in range(H):
        S = torch.zeros(d, dv, dtype=F64)
        lam = float(m["decay"][hd])
        for t in range(T):
            S = lam * S + torch.outer(k[t, hd], v[t, hd])
            out[t, hd] = S.t() @ q[t, hd]
    o = unit_rms(out.reshape(T, H * dv), w[p + "norm"], eps)
    o = o * torch.sigmoid(h @ w[p + "g"].t())
    return o @ w[p + "o"].t()


def windowed_attention(w: Dict[str, torch.Tensor], p: str, m: dict, h: torch.Tensor, eps: float) -> torch.Tensor:
    """Grouped-query attention without positions: per-head unit-rms queries and keys, a sliding window,
    an ordinary softmax."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = unit_rms((h @ w[p + "q"].t()).view(T, H, d), w[p + "q.norm"], eps)
    k = unit_rms((h @ w[p + "k"].t()).view(T, G, d), w[p + "k.norm"], eps)
    v = (h @ w[p + "v"].t()).view(T, G, dv)
    win = int(m["mask"]["size"])
    out = torch.zeros(T, H, dv, dtype=F64)
    for hd in range(H):
        g = hd // (H // G)
        for i in range(T):
            lo = max(0, i - win + 1)
            s = (k[lo:i + 1, g] @ q[i, hd]) * float(m["scale"])
            a = torch.softmax(s, dim=0)
            out[i, hd] = a @ v[lo:i + 1, g]
    return out.reshape(T, H * dv) @ w[p + "o"].t()


def selective_scan(w: Dict[str, torch.Tensor], p: str, m: dict, h: torch.Tensor) -> torch.Tensor:
    """The Mamba recurrence, token by token."""
    T = h.shape[0]
    E, N, R, taps = m["inner"], m["state"], m["dt_rank"], m["conv"]
    xz = h @ w[p + "in"].t()
    x, z = xz[:, :E], xz[:, E:]
    padded = torch.cat([torch.zeros(taps - 1, E, dtype=F64), x], dim=0)
    conv = torch.zeros(T, E, dtype=F64)
    for j in range(taps):                              # the last column is the current token's
        conv = conv + padded[j:j + T] * w[p + "conv"][:, j]
    x = silu(conv + w[p + "conv.b"])
    proj = x @ w[p + "x"].t()
    dt, B, C = proj[:, :R], proj[:, R:R + N], proj[:, R + N:]
    dt = softplus(dt @ w[p + "dt"].t() + w[p + "dt.b"])          # [T, E]
    A = -torch.exp(w[p + "A_log"])                               # [E, N]
    S = torch.zeros(E, N, dtype=F64)
    y = torch.zeros(T, E, dtype=F64)
    for t in range(T):
        S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * B[t][None, :]
        y[t] = S @ C[t] + w[p + "D"] * x[t]
    y = y * silu(z)
    return y @ w[p + "o"].t()


def parallel_mixer(w: Dict[str, torch.Tensor], p: str, m: dict, h: torch.Tensor, eps: float) -> torch.Tensor:
    a = windowed_attention(w, p + "left.", m["left"], h, eps)
    b = selective_scan(w, p + "right.", m["right"], h)
    return 0.5 * (unit_rms(a, w[p + "left.out"], eps) + unit_rms(b, w[p + "right.out"], eps))


# ---------------------------------------------------------------------------
# feed-forwards
# ---------------------------------------------------------------------------
def gated_ff(w: Dict[str, torch.Tensor], p: str, h: torch.Tensor, act) -> torch.Tensor:
    return (act(h @ w[p + "gate"].t()) * (h @ w[p + "up"].t())) @ w[p + "down"].t()


def route(w: Dict[str, torch.Tensor], p: str, mlp: dict, h: torch.Tensor):
    """(chosen experts [T, top], their weights [T, top])."""
    s = torch.sigmoid(h @ w[p + "router"].t())
    choice = s + w[p + "correction"]
    top = int(mlp["router"]["top"])
    # the largest first; among equals the lowest index
    ids = torch.sort(choice, dim=-1, descending=True, stable=True).indices[:, :top]
    return ids, torch.gather(s, 1, ids) * float(mlp["router"]["scale"])


def expert_ff(w: Dict[str, torch.Tensor], p: str, mlp: dict, h: torch.Tensor) -> torch.Tensor:
    ids, wt = route(w, p, mlp, h)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(ids.shape[1]):
            e = int(ids[t, j])
            out[t] += wt[t, j] * gated_ff(w, f"{p}e{e}.", h[t:t + 1], silu)[0]
    if mlp.get("shared") is not None:
        gate = torch.sigmoid(h @ w[p + "shared.sg"].t())           # [T, 1]
        out = out + gate * gated_ff(w, p + "shared.", h, silu)
    return out


def feed_forward(w: Dict[str, torch.Tensor], p: str, mlp: dict, h: torch.Tensor) -> torch.Tensor:
    if mlp["kind"] == "dense":
        return gated_ff(w, p, h, gelu_tanh)
    return expert_ff(w, p, mlp, h)


# ---------------------------------------------------------------------------
# the layer and the model
# ---------------------------------------------------------------------------
def layer_order(cfg: dict) -> List[int]:
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def sublayer(w, cfg, i: int, q: int, xs: torch.Tensor) -> torch.Tensor:
    """xs [streams, T, width] -> the same after sublayer q (1: mixer, 2: feed-forward) of layer i."""
    L, p, eps = cfg["layers"][i], f"l{i}.", float(cfg["norm"]["eps"])
    u = torch.einsum("s,std->td", w[f"{p}hc{q}.in"], xs)
    a = tanh_norm(w, f"{p}norm{q}", u)
    if q == 1:
        if L["type"] == "lightning":
            y = lightning_mixer(w, p + "mix.", L["mixer"], a, eps)
        elif L["type"] == "parallel":
            y = parallel_mixer(w, p + "mix.", L["mixer"], a, eps)
        else:
            raise ValueError(L["type"])
    else:
        y = feed_forward(w, p + "mlp.", L["mlp"], a)
    y = y * w[f"{p}ls{q}"]
    return torch.einsum("st,sxd->txd", w[f"{p}hc{q}.mix"], xs) + w[f"{p}hc{q}.out"][:, None, None] * y[None]


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens, layers_out: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence."""
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    x = w["embed"][tokens] * float(cfg["embedding"]["scale"])
    xs = x[None].repeat(int(cfg["streams"]), 1, 1)
    for i in layer_order(cfg):
        xs = sublayer(w, cfg, i, 1, xs)
        if cfg["layers"][i]["mlp"] is not None:
            xs = sublayer(w, cfg, i, 2, xs)
        if layers_out is not None:
            layers_out.append(xs.sum(dim=0))
    return tanh_norm(w, "final.norm", xs.sum(dim=0)) @ w["embed"].t()


logits = forward


def greedy(cfg: dict, w: Dict[str, torch.Tensor], prompt: List[int], n_new: int) -> List[int]:
    seq, out = list(prompt), []
    for _ in range(n_new):
        t = int(torch.argmax(forward(cfg, w, seq)[-1]))
        out.append(t)
        seq.append(t)
    return out
