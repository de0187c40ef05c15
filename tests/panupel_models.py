"""Small Panupel models for the tests: configurations that differ in every size and option, random weights
whose scales make every mechanism matter, and model folders written from them.

The weights are drawn in float32 and rounded to bfloat16 values, so the engine in either compute type and
the plain implementation (tests/plain_panupel.py, in float64) start from the same numbers.
"""
from __future__ import annotations

import copy
import json
import math
import os
from typing import Dict, List

import numpy as np
import torch


def _left(heads, kv_heads, dim, vdim, rot=None, scale=None):
    d = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5}
    if rot is not None:
        d["rot"] = rot
    return d


def parallel(left, right, left_scale=0.7, right_scale=1.2, ff=None):
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": left_scale, "right_scale": right_scale},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def delta(heads, kv_heads, dim, vdim, conv, ff=None):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def _config(vocab, width, layers, loop=None, eps=1e-5, mult=0.5):
    c = {"architecture": "Panupel", "vocab": vocab, "width": width, "norm": {"eps": eps}, "residual_mult": mult, "layers": layers}
    if loop is not None:
        c["loop"] = loop
    return c


SCALING = {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}

# A: a looped span in the middle, partial rotary with rescaled frequencies, grouped heads, a layer without a feed-forward
CONFIG_A = _config(97, 64, [
    delta(4, 2, 16, 8, 4, ff=96),
    parallel(_left(4, 2, 16, 16, rot={"dims": 8, "base": 100.0, "scaling": SCALING}), {"heads": 2, "dim": 16, "vdim": 24, "gate_cap": 10.0}),
    delta(2, 2, 32, 16, 2, ff=80),
    parallel(_left(2, 1, 32, 32, rot={"dims": 32, "base": 10000.0}, scale=0.3), {"heads": 4, "dim": 8, "vdim": 16, "gate_cap": 14.0}, ff=64),
], loop={"start": 1, "stop": 3, "times": 3}, eps=1e-5, mult=0.5)

# B: key size and value size differ and neither is a multiple of 16 (the cache pads both to 48); one key/value head;
# the attention layer comes first; no loop; a multiplier of 1
CONFIG_B = _config(203, 96, [
    parallel(_left(3, 1, 24, 40, rot={"dims": 24, "base": 500.0}), {"heads": 3, "dim": 40, "vdim": 20, "gate_cap": 5.0},
             left_scale=1.0, right_scale=0.5, ff=136),
    delta(2, 2, 48, 36, 3, ff=None),
    delta(6, 3, 16, 16, 1, ff=72),
], eps=1e-6, mult=1.0)

# C: heads of 64 and 128 (the tensor-core attention kernels' sizes), no rotary positions, as many key/value heads as
# heads, the whole stack looped once (one pass, entered through the mix)
CONFIG_C = _config(311, 128, [
    parallel(_left(4, 4, 64, 64), {"heads": 1, "dim": 64, "vdim": 128, "gate_cap": 20.0}, ff=192),
    delta(2, 1, 128, 64, 4, ff=160),
    parallel(_left(2, 1, 128, 128, rot={"dims": 64, "base": 1000.0, "scaling": {"factor": 2.0, "low": 2.0, "high": 8.0, "original": 128}}),
             {"heads": 2, "dim": 96, "vdim": 32, "gate_cap": 8.0}, ff=None),
], loop={"start": 0, "stop": 3, "times": 1}, eps=1e-6, mult=0.25)

# D: a width that is no multiple of 8 (the bfloat16 products then take the kernel for odd sizes), two passes at the end
CONFIG_D = _config(64, 100, [
    delta(5, 5, 20, 12, 3, ff=60),
    parallel(_left(5, 5, 32, 16, rot={"dims": 16, "base": 50.0}), {"heads": 5, "dim": 20, "vdim": 20, "gate_cap": 12.0}, ff=52),
], loop={"start": 1, "stop": 2, "times": 2}, eps=1e-4, mult=0.8)

CONFIGS = {"A": CONFIG_A, "B": CONFIG_B, "C": CONFIG_C, "D": CONFIG_D}


def tensor_shapes(config: dict) -> Dict[str, List[int]]:
    """Every tensor of a model of this configuration, by its name in the weight file."""
    w = config["width"]
    out = {"embed": [config["vocab"], w], "head": [config["vocab"], w], "final.norm": [w]}
    if config.get("loop"):
        out["loop.in"] = [w, 2 * w]
    for i, l in enumerate(config["layers"]):
        p = f"l{i}."
        for n in ("norm1", "norm1b"):
            out[p + n] = [w]
        m = l["mixer"]
        if l["type"] == "delta":
            H, G, d, e, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            x = p + "mix."
            out.update({x + "q": [G * d, w], x + "k": [G * d, w], x + "v": [H * e, w], x + "g": [H * e, w], x + "o": [w, H * e],
                        x + "q.conv": [G * d, taps], x + "k.conv": [G * d, taps], x + "v.conv": [H * e, taps],
                        x + "b": [H, w], x + "a": [H, w], x + "A_log": [H], x + "dt_bias": [H], x + "norm": [e]})
        else:
            a, r = m["left"], m["right"]
            x = p + "mix.left."
            H, G, d, e = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            out.update({x + "q": [H * d, w], x + "k": [G * d, w], x + "v": [G * e, w], x + "o": [w, H * e], x + "g": [H, w],
                        x + "q.norm": [H * d], x + "k.norm": [G * d], x + "sink": [H]})
            x = p + "mix.right."
            H, d, e = r["heads"], r["dim"], r["vdim"]
            out.update({x + "q": [H * d, w], x + "k": [H * d, w], x + "v": [H * e, w], x + "g": [H * e, w], x + "o": [w, H * e],
                        x + "norm": [H * e], x + "i": [H, w], x + "i.b": [H], x + "f": [H, w], x + "f.b": [H]})
        if l.get("mlp"):
            ff = l["mlp"]["ff"]
            for n in ("norm2", "norm2b"):
                out[p + n] = [w]
            out.update({p + "mlp.gate": [ff, w], p + "mlp.up": [ff, w], p + "mlp.down": [w, ff]})
    return out


def make_weights(config: dict, seed: int) -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(config).items():
        last = name.split(".")[-1]
        n = lambda std=1.0, mean=0.0: mean + std * torch.randn(shape, generator=g)
        if name in ("embed",):
            t = n()
        elif last in ("norm1", "norm2", "norm1b", "norm2b") or name == "final.norm" or name.endswith((".q.norm", ".k.norm", ".norm")):
            t = n(0.2, 1.0)
        elif last == "sink":
            t = n(1.5)
        elif last == "conv":
            t = n(0.6)
        elif last == "A_log":
            t = torch.log(0.3 + 2.7 * torch.rand(shape, generator=g))
        elif last == "dt_bias":
            t = n(1.0)
        elif name.endswith(".i.b"):
            t = n(1.0)
        elif name.endswith(".f.b"):
            t = n(1.0, 2.0)
        elif len(shape) == 2:
            t = n(1.2 / math.sqrt(shape[1]))
        else:
            raise ValueError(name)
        out[name] = t.to(torch.bfloat16).to(torch.float32)
    return out


def write_model(config: dict, weights: Dict[str, torch.Tensor], path: str, store=torch.bfloat16) -> str:
    from sandyrt_b200.weights.safetensors import write_safetensors

    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(config, f, indent=1)
    write_safetensors(os.path.join(path, "model.safetensors"), {k: v.to(store) for k, v in weights.items()})
    return path


def variant(config: dict, **changes) -> dict:
    c = copy.deepcopy(config)
    c.update(changes)
    return c


def rel_error(got: np.ndarray, want: np.ndarray) -> float:
    """Largest over the rows of: RMS over the vocabulary of the difference (mean taken off) over the RMS of the
    wanted logits (mean taken off)."""
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    d = got - want
    d = d - d.mean(-1, keepdims=True)
    w = want - want.mean(-1, keepdims=True)
    return float((np.sqrt((d ** 2).mean(-1)) / np.sqrt((w ** 2).mean(-1))).max())
