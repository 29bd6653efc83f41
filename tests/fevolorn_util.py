"""Small Fevolorn configurations for the tests, none with a shipped model's sizes.

FV_A: three streams; a parallel layer whose attention has keys of 24 and values of 40 (no multiple of 16),
three query heads per kv head and a window shorter than a page, beside a scan with 10 states, 5 step
values and 3 taps; experts with a shared expert (top 2 of 5); a lightning layer with a dense feed-forward;
a lightning layer without a feed-forward; a parallel layer whose attention has as many kv heads as heads,
keys and values of 16 (the tensor-core kernels' sizes) and a window over two pages, a scan with 2 taps, and
experts without a shared one (top 3 of 3); layers 1 and 2 run three times.
FV_B: one stream, no repeat, sizes that are multiples of 16 and 64; a convolution of one tap (no tail at
all); a window of 5 and one of 64; one lightning head; top 1 of 2.
FV_C: lightning layers only (no pages at all), two streams, everything runs twice.
"""
from __future__ import annotations

import os


def _moe(experts, top, ff, scale, shared=None):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "scale": scale}}
    if shared is not None:
        m["shared"] = {"ff": shared}
    return m


def _par(heads, kv, dim, vdim, scale, window, inner, state, dt_rank, conv):
    return {"left": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": window}},
            "right": {"inner": inner, "state": state, "dt_rank": dt_rank, "conv": conv}}


FV_A = {
    "architecture": "Fevolorn", "vocab": 203, "width": 72, "streams": 3, "norm": {"eps": 1e-5},
    "embedding": {"scale": 2.0}, "loop": {"start": 1, "stop": 3, "times": 3},
    "layers": [
        {"type": "parallel", "mixer": _par(6, 2, 24, 40, 0.3, 11, 56, 10, 5, 3), "mlp": _moe(5, 2, 24, 1.7, shared=40)},
        {"type": "lightning", "mixer": {"heads": 3, "dim": 20, "vdim": 24, "decay": [0.5, 0.93, 0.999]},
         "mlp": {"kind": "dense", "ff": 100}},
        {"type": "lightning", "mixer": {"heads": 2, "dim": 16, "vdim": 48, "decay": [1.0, 0.8]}, "mlp": None},
        {"type": "parallel", "mixer": _par(4, 4, 16, 16, 0.25, 37, 40, 20, 8, 2), "mlp": _moe(3, 3, 16, 0.5)},
    ],
}
FV_B = {
    "architecture": "Fevolorn", "vocab": 256, "width": 128, "streams": 1, "norm": {"eps": 1e-6},
    "embedding": {"scale": 1.0},
    "layers": [
        {"type": "lightning", "mixer": {"heads": 1, "dim": 64, "vdim": 128, "decay": [0.97]},
         "mlp": _moe(2, 1, 64, 1.0, shared=64)},
        {"type": "parallel", "mixer": _par(4, 2, 64, 32, 0.11, 5, 128, 16, 16, 1), "mlp": {"kind": "dense", "ff": 192}},
        {"type": "parallel", "mixer": _par(2, 1, 32, 64, 0.2, 64, 64, 32, 8, 4), "mlp": _moe(8, 2, 32, 2.0)},
    ],
}
FV_C = {
    "architecture": "Fevolorn", "vocab": 97, "width": 40, "streams": 2, "norm": {"eps": 1e-4},
    "embedding": {"scale": 0.5}, "loop": {"start": 0, "stop": 2, "times": 2},
    "layers": [
        {"type": "lightning", "mixer": {"heads": 5, "dim": 8, "vdim": 12, "decay": [0.3, 0.6, 0.9, 0.99, 1.0]},
         "mlp": _moe(4, 2, 12, 1.0, shared=8)},
        {"type": "lightning", "mixer": {"heads": 2, "dim": 36, "vdim": 20, "decay": [0.95, 0.5]}, "mlp": None},
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
    """Make the mechanisms show: attention queries 8 times larger (peaked attention, so a key that is wrongly
    seen or missed moves the result), half the scan's channels with slow decays (far tokens stay in the state),
    routers spread out, the streams' mixing well away from the identity, and norms that do not saturate."""
    for n, t in w.items():
        if n.endswith("left.q"):
            t.mul_(8.0)
        elif n.endswith("A_log"):
            t[::2] -= 3.0
        elif n.endswith("mlp.router"):
            t.mul_(3.0)
        elif n.endswith(".alpha"):
            t.fill_(0.4)
        elif n.endswith("mix.q") or n.endswith("mix.k"):
            t.mul_(3.0)
