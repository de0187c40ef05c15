"""Small Sovezen models for the tests: configurations that differ in every size and option, random weights whose
scales make every mechanism matter, and model folders written from them.

The weights are drawn in float32 and rounded to bfloat16 values, so the engine in either compute type and the
plain implementation (tests/plain_sovezen.py, in float64) start from the same numbers.

Routers.  A token's experts are the largest of a handful of logits, and two of them are now and then closer than
the rounding of a bfloat16 run moves them; the token then takes another expert and its logits land elsewhere,
which says nothing about the engine.  So `make_weights(..., decisive_router=True)` spreads the router's biases far
apart and shrinks its matrix: the choice is then the same with either rounding (the weights of the chosen experts
still depend on the token).  The float32 tests use ordinary routers, whose choices change from token to token.
"""
from __future__ import annotations

import copy
import json
import math
import os
from typing import Dict, List, Optional

import numpy as np
import torch


def rotated(heads, dim, rot_dim, vdim, kv_rank, base=10000.0, dims=None, scale=None):
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
                      "scale": scale if scale is not None else (dim + rot_dim) ** -0.5,
                      "rot": {"dims": rot_dim if dims is None else dims, "base": base}}}


def plain_queries(heads, dim, vdim, kv_rank, q_rank, scale=None):
    return {"type": "latent_attention_2",
            "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
                      "scale": scale if scale is not None else dim ** -0.5}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def layer(mixer: dict, mlp: Optional[dict], weights_of: Optional[int] = None) -> dict:
    out = copy.deepcopy(mixer)
    out["mlp"] = copy.deepcopy(mlp)
    if weights_of is not None:
        out["weights_of"] = weights_of
    return out


def _config(vocab, width, layers, eps=1e-5, logit_scale=1.0):
    return {"architecture": "Sovezen", "vocab": vocab, "width": width, "norm": {"eps": eps}, "logit_scale": logit_scale,
            "layers": layers}


_A0 = rotated(2, 16, 8, 24, 24)                 # cache rows of 32
_A1 = plain_queries(4, 16, 8, 32, 24)           # cache rows of 32
# A: both mixers, both feed-forwards, two layers on other layers' tensors, a layer without a feed-forward whose
# cache rows are 64 wide (the tensor-core attention kernels' size)
CONFIG_A = _config(101, 64, [
    layer(_A0, dense(96)),
    layer(_A1, moe(8, 2, 40)),
    layer(_A0, dense(96), weights_of=0),
    layer(_A1, moe(8, 2, 40), weights_of=1),
    layer(rotated(3, 8, 16, 16, 48, base=100.0), None),
], eps=1e-5, logit_scale=0.5)

# B: a width that is no multiple of 8 (the bfloat16 products then take the kernel for odd sizes), one head, a rotated
# part of which only four entries turn, every expert chosen, one expert chosen, sizes that divide by nothing
CONFIG_B = _config(77, 100, [
    layer(rotated(1, 20, 6, 12, 20, base=50.0, dims=4), moe(5, 5, 12)),
    layer(plain_queries(5, 12, 20, 36, 10), dense(52)),
    layer(plain_queries(2, 28, 4, 12, 44), moe(3, 1, 20)),
], eps=1e-6, logit_scale=1.75)

# C: wide latents: cache rows of 128 (the decode kernels' largest common size), of 192 (beyond the prompt kernels),
# many heads on one latent, many experts
CONFIG_C = _config(311, 128, [
    layer(rotated(8, 32, 16, 32, 112), moe(32, 4, 64)),
    layer(plain_queries(8, 16, 48, 128, 96), dense(256)),
    layer(rotated(2, 64, 32, 64, 160, base=1e6), dense(64)),
    layer(rotated(8, 32, 16, 32, 112), moe(32, 4, 64), weights_of=0),
], eps=1e-5, logit_scale=0.25)

CONFIGS = {"A": CONFIG_A, "B": CONFIG_B, "C": CONFIG_C}


def owner(config: dict, i: int) -> int:
    while config["layers"][i].get("weights_of") is not None:
        i = config["layers"][i]["weights_of"]
    return i


def tensor_shapes(config: dict) -> Dict[str, List[int]]:
    """Every tensor of a model of this configuration, by its name in the weight file."""
    w = config["width"]
    out = {"embed": [config["vocab"], w], "final.norm": [w]}
    for i, l in enumerate(config["layers"]):
        if owner(config, i) != i:
            continue
        p = f"l{i}."
        out[p + "norm1"] = [w]
        out[p + "ls1"] = [w]
        m, x = l["mixer"], p + "mix."
        H, d, e, c = m["heads"], m["dim"], m["vdim"], m["kv_rank"]
        if l["type"] == "latent_attention":
            r = m["rot_dim"]
            out.update({x + "q": [H * (d + r), w], x + "dkv": [c + r, w], x + "sink": [H]})
        else:
            out.update({x + "dq": [m["q_rank"], w], x + "dq.norm": [m["q_rank"]], x + "uq": [H * d, m["q_rank"]], x + "dkv": [c, w]})
        out.update({x + "dkv.norm": [c], x + "uk": [H * d, c], x + "uv": [H * e, c], x + "o": [w, H * e]})
        mlp = l.get("mlp")
        if mlp:
            out[p + "ls2"] = [w]
            if mlp["kind"] == "dense":
                out.update({p + "mlp.gate": [mlp["ff"], w], p + "mlp.up": [mlp["ff"], w], p + "mlp.down": [w, mlp["ff"]]})
            else:
                E, ff = mlp["router"]["experts"], mlp["expert"]["ff"]
                out.update({p + "mlp.router": [E, w], p + "mlp.router.b": [E]})
                for k in range(E):
                    out.update({f"{p}mlp.e{k}.up": [ff, w], f"{p}mlp.e{k}.down": [w, ff]})
    return out


def make_weights(config: dict, seed: int, decisive_router: bool = False) -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(config).items():
        last = name.split(".")[-1]
        n = lambda std=1.0, mean=0.0: mean + std * torch.randn(shape, generator=g)
        if name == "embed":
            t = n()
        elif last in ("norm1", "norm") or name == "final.norm":
            t = n(0.2, 1.0)
        elif last in ("ls1", "ls2"):
            t = n(0.3, 0.7)
        elif last == "sink":
            t = n(1.5)
        elif last == "b":                       # router bias
            if decisive_router:
                t = 3.0 * torch.randperm(shape[0], generator=g).to(torch.float32)
            else:
                t = n(1.0)
        elif last == "router":
            t = n((0.2 if decisive_router else 3.0) / math.sqrt(shape[1]))
        elif last == "down" and ".mlp.e" in name:
            t = n(2.5 / math.sqrt(shape[1]))    # relu squared of unit inputs is small
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


def rel_error(got: np.ndarray, want: np.ndarray) -> float:
    """Largest over the rows of: RMS over the vocabulary of the difference (mean taken off) over the RMS of the
    wanted logits (mean taken off)."""
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    d = got - want
    d = d - d.mean(-1, keepdims=True)
    w = want - want.mean(-1, keepdims=True)
    return float((np.sqrt((d ** 2).mean(-1)) / np.sqrt((w ** 2).mean(-1))).max())
