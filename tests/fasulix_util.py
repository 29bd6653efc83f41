"""Small Fasulix configurations for the tests, none with a shipped model's sizes.

FX_A: every mixer kind; a window shorter than a page and one longer than two pages; a layer that
reads an earlier windowed layer's rows with ANOTHER window; a layer that reads a causal (sink)
layer's rows; rot.dims smaller than rot_dim; dim != vdim; q_rank != kv_rank; one head; top 1, top
== experts, an odd number of experts; a layer without a feed-forward; width and vocab no powers of two.
FX_B: three layers, sizes that are multiples of 16 and 64 (other tile paths), a window of one, no rotation in one layer.
FX_C: recurrences first, then one attention layer whose sizes are multiples of 2 only (width 52, rows of 26
values: none of the 16-byte paths applies), so a model may also keep no pages at all in its first layers.
FX_D: recurrences only (no paged cache at all).
"""
from __future__ import annotations

import json
import os


def _latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, base, rot_dims=None, window=None, kv_from=None, scale=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
         "rot": {"base": base, "dims": rot_dim if rot_dims is None else rot_dims},
         "scale": scale if scale is not None else (dim + rot_dim) ** -0.5}
    if window is not None:
        m["mask"] = {"size": window}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _moe(experts, top, ff, limit):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}


FX_A = {
    "architecture": "Fasulix", "vocab": 211, "width": 88, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "latent_attention", "mixer": _latent(3, 16, 8, 24, 40, 48, 10000.0), "mlp": _moe(5, 2, 24, 1.5)},
        {"type": "mingru", "mixer": {"width": 72}, "mlp": _moe(3, 1, 40, 0.75)},
        {"type": "latent_attention_2", "mixer": _latent(2, 24, 16, 8, 24, 40, 500.0, rot_dims=8, window=9),
         "mlp": None},
        {"type": "latent_attention_2", "mixer": _latent(1, 8, 16, 40, 56, 40, 500.0, rot_dims=8, window=37, kv_from=2),
         "mlp": _moe(4, 4, 16, 3.0)},
        {"type": "mingru", "mixer": {"width": 100}, "mlp": _moe(5, 2, 24, 1.5)},
        {"type": "latent_attention_2", "mixer": _latent(4, 8, 8, 8, 16, 48, 10000.0, window=20, kv_from=0),
         "mlp": _moe(6, 3, 8, 2.5)},
    ],
}
FX_B = {
    "architecture": "Fasulix", "vocab": 256, "width": 128, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "latent_attention_2", "mixer": _latent(4, 32, 32, 32, 64, 64, 100000.0, window=1),
         "mlp": _moe(8, 2, 64, 2.0)},
        {"type": "latent_attention", "mixer": _latent(2, 64, 0, 64, 128, 128, 100000.0), "mlp": _moe(2, 1, 128, 8.0)},
        {"type": "mingru", "mixer": {"width": 128}, "mlp": None},
    ],
}


FX_C = {
    "architecture": "Fasulix", "vocab": 97, "width": 52, "norm": {"eps": 1e-4},
    "layers": [
        {"type": "mingru", "mixer": {"width": 30}, "mlp": _moe(2, 2, 12, 1.0)},
        {"type": "mingru", "mixer": {"width": 66}, "mlp": None},
        {"type": "latent_attention", "mixer": _latent(5, 12, 6, 10, 22, 20, 3000.0, rot_dims=2), "mlp": _moe(7, 3, 10, 2.0)},
    ],
}
FX_D = {
    "architecture": "Fasulix", "vocab": 64, "width": 32, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "mingru", "mixer": {"width": 48}, "mlp": _moe(4, 2, 16, 2.0)},
        {"type": "mingru", "mixer": {"width": 16}, "mlp": _moe(4, 1, 16, 2.0)},
    ],
}


def write_model(folder: str, cfg: dict, seed: int, edit=None) -> str:
    """A model folder with random weights; ``edit(weights dict)`` may change tensors before they are
    written (float32 storage)."""
    from rllm_b200.engine.loading import write_random_model
    write_random_model(folder, dict(cfg, torch_dtype="float32"), seed, "float32")
    if edit is not None:
        from safetensors import safe_open
        from safetensors.torch import save_file
        path = os.path.join(folder, "model.safetensors")
        with safe_open(path, framework="pt") as f:
            w = {n: f.get_tensor(n).clone() for n in f.keys()}
        edit(w)
        save_file({n: t.contiguous() for n, t in w.items()}, path)
    return folder


def sharpen(w: dict) -> None:
    """Make the mechanisms show: queries 6 times larger (peaked attention, so a key that is wrongly seen
    or missed moves the result), sinks large enough to take a visible share, recurrence gates spread out."""
    for n, t in w.items():
        if n.endswith("mix.uq"):
            t.mul_(6.0)
        elif n.endswith("mix.sink"):
            t.add_(2.0)
        elif n.endswith("mix.z") or n.endswith("mix.x"):
            t.mul_(3.0)
        elif n.endswith("mlp.router"):
            t.mul_(2.0)
