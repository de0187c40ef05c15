"""A plain, slow implementation of the Sovezen design: one function per mechanism, whole sequences at
once, no cache, no batching.  It shares nothing with the engine; the tests compare the engine with it.

Everything is computed in the dtype of the tensors handed in (float64 for an oracle).  A model is
`(config, weights)`: the parsed config.json and a dict name -> tensor.

The design: every layer norms the stream once, h = rmsnorm(x), and adds two branches that both read h:
x <- x + ls1 * mixer(h) + ls2 * ff(h).  The mixers are two kinds of attention over a low-rank latent of
keys and values; the feed-forward is gated and dense, or a routed mixture of small experts, or absent.  A
layer may use another layer's tensors.  The head is the embedding table, times a constant.

Notation: T tokens, H heads, d the unrotated query/key size of a head, r its rotated size, e its value
size, c the latent's size.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

Weights = Dict[str, torch.Tensor]

# With ROUND_PRODUCTS set, every matrix product rounds its input and its output to bfloat16 values (the sums
# stay exact): what an engine that multiplies in bfloat16 does.  Tests use it to learn how far rounding alone
# moves the logits of a given model.
ROUND_PRODUCTS = False


def _bf16(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.bfloat16).to(x.dtype)


def linear(w: torch.Tensor, h: torch.Tensor, keep32: bool = False) -> torch.Tensor:
    """Weights are stored [out, in]; rows of h are tokens."""
    if not ROUND_PRODUCTS:
        return h @ w.to(h.dtype).t()
    y = _bf16(h) @ w.to(h.dtype).t()
    return y if keep32 else _bf16(y)


def rms_norm(x: torch.Tensor, w: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y * w.to(x.dtype) if w is not None else y


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


# ---- rotary positions, neighbours paired -------------------------------------------------------------
def rotate_pairs(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x: [T, heads, n].  Of each head the first `dims` entries turn: entries 2i and 2i+1 are one pair,
    turned by the angle position * base^(-2i/dims)."""
    out = x.clone()
    for i in range(dims // 2):
        f = float(base) ** (-2.0 * i / dims)
        a = positions.to(x.dtype) * f
        cos, sin = torch.cos(a)[:, None], torch.sin(a)[:, None]
        u, v = x[..., 2 * i], x[..., 2 * i + 1]
        out[..., 2 * i] = u * cos - v * sin
        out[..., 2 * i + 1] = v * cos + u * sin
    return out


# ---- attention -------------------------------------------------------------------------------------------
def causal_softmax_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                             sink: Optional[torch.Tensor]) -> torch.Tensor:
    """q, k: [T, H, n]; v: [T, H, e].  Token i sees tokens j <= i.  With a sink, exp(sink_h) joins the
    denominator of head h's softmax (once, unscaled) and nothing else."""
    T, H, _ = q.shape
    out = torch.zeros(T, H, v.shape[-1], dtype=q.dtype)
    for h in range(H):
        s = (q[:, h] @ k[:, h].t()) * scale
        s = s.masked_fill(torch.ones(T, T, dtype=torch.bool).triu(1), -math.inf)
        m = s.max(-1, keepdim=True).values
        if sink is not None:
            m = torch.maximum(m, sink[h].to(q.dtype).expand_as(m))
        p = torch.exp(s - m)
        den = p.sum(-1, keepdim=True)
        if sink is not None:
            den = den + torch.exp(sink[h].to(q.dtype) - m)
        out[:, h] = (p / den) @ v[:, h]
    return out


def latent_attention(m: dict, w: Weights, pre: str, h: torch.Tensor, positions: torch.Tensor, eps: float) -> torch.Tensor:
    """Queries straight from h, each head [d unrotated | r rotated]; keys and values from a normed latent;
    one rotated key part shared by all heads; a sink in the softmax."""
    T = h.shape[0]
    H, d, r, e, c = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    q = linear(w[pre + "q"], h).view(T, H, d + r)
    down = linear(w[pre + "dkv"], h)
    latent = rms_norm(down[:, :c], w[pre + "dkv.norm"], eps)
    k_rot = down[:, c:].view(T, 1, r)
    if ROUND_PRODUCTS:
        latent = _bf16(latent)
    k_plain = linear(w[pre + "uk"], latent).view(T, H, d)
    v = linear(w[pre + "uv"], latent).view(T, H, e)
    rot = m["rot"]
    q_rot = rotate_pairs(q[..., d:], positions, rot["dims"], rot["base"])
    k_rot = rotate_pairs(k_rot, positions, rot["dims"], rot["base"]).expand(T, H, r)
    qq = torch.cat([q[..., :d], q_rot], -1)
    kk = torch.cat([k_plain, k_rot], -1)
    o = causal_softmax_attention(qq, kk, v, m["scale"], w[pre + "sink"])
    return linear(w[pre + "o"], o.reshape(T, H * e))


def latent_attention_2(m: dict, w: Weights, pre: str, h: torch.Tensor, eps: float) -> torch.Tensor:
    """No positions, no sink; the queries pass a normed latent of their own."""
    T = h.shape[0]
    H, d, e, c = m["heads"], m["dim"], m["vdim"], m["kv_rank"]
    q_latent = rms_norm(linear(w[pre + "dq"], h), w[pre + "dq.norm"], eps)
    latent = rms_norm(linear(w[pre + "dkv"], h), w[pre + "dkv.norm"], eps)
    if ROUND_PRODUCTS:
        q_latent, latent = _bf16(q_latent), _bf16(latent)
    q = linear(w[pre + "uq"], q_latent).view(T, H, d)
    k = linear(w[pre + "uk"], latent).view(T, H, d)
    v = linear(w[pre + "uv"], latent).view(T, H, e)
    o = causal_softmax_attention(q, k, v, m["scale"], None)
    return linear(w[pre + "o"], o.reshape(T, H * e))


# ---- feed-forwards ---------------------------------------------------------------------------------------
def dense_ff(w: Weights, pre: str, h: torch.Tensor) -> torch.Tensor:
    a = silu(linear(w[pre + "gate"], h)) * linear(w[pre + "up"], h)
    return linear(w[pre + "down"], a)


def routed_ff(mlp: dict, w: Weights, pre: str, h: torch.Tensor) -> torch.Tensor:
    """Each token goes to the `top` experts with the largest router logits; their weights are the softmax over
    those logits alone.  An expert is down(relu(up h)^2)."""
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    z = linear(w[pre + "router"], h, keep32=True) + w[pre + "router.b"].to(h.dtype)
    out = torch.zeros(h.shape[0], w[pre + "e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        order = sorted(range(E), key=lambda e: (-float(z[t, e]), e))[:top]
        weights = torch.softmax(z[t, order], -1)
        for e, g in zip(order, weights):
            a = torch.relu(linear(w[f"{pre}e{e}.up"], h[t:t + 1])) ** 2
            out[t] += g * linear(w[f"{pre}e{e}.down"], a)[0]
    return out


# ---- the model ---------------------------------------------------------------------------------------------
def layer(cfg: dict, w: Weights, i: int, x: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
    spec = cfg["layers"][i]
    src = spec.get("weights_of", i)
    pre = f"l{src}."
    eps = cfg["norm"]["eps"]
    h = rms_norm(x, w[pre + "norm1"], eps)
    if spec["type"] == "latent_attention":
        mixed = latent_attention(spec["mixer"], w, pre + "mix.", h, positions, eps)
    elif spec["type"] == "latent_attention_2":
        mixed = latent_attention_2(spec["mixer"], w, pre + "mix.", h, eps)
    else:
        raise ValueError(spec["type"])
    branch = mixed * w[pre + "ls1"].to(x.dtype)
    mlp = spec.get("mlp")
    if mlp is not None:
        f = dense_ff(w, pre + "mlp.", h) if mlp["kind"] == "dense" else routed_ff(mlp, w, pre + "mlp.", h)
        branch = branch + f * w[pre + "ls2"].to(x.dtype)
    return x + branch


def forward(cfg: dict, w: Weights, tokens: List[int], dtype=torch.float64, streams: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence; `streams`, if given, receives the stream after every layer."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}
    ids = torch.tensor(tokens, dtype=torch.long)
    positions = torch.arange(len(tokens))
    x = w["embed"][ids]
    for i in range(len(cfg["layers"])):
        x = layer(cfg, w, i, x, positions)
        if streams is not None:
            streams.append(x.clone())
    y = rms_norm(x, w["final.norm"], cfg["norm"]["eps"])
    return linear(w["embed"], y, keep32=True) * cfg["logit_scale"]


def forward_rounded(cfg: dict, w: Weights, tokens: List[int]) -> torch.Tensor:
    """The same with every product's operands and results rounded to bfloat16 values."""
    global ROUND_PRODUCTS
    ROUND_PRODUCTS = True
    try:
        return forward(cfg, w, tokens)
    finally:
        ROUND_PRODUCTS = False


def router_margin(cfg: dict, w: Weights, tokens: List[int]) -> float:
    """How close the closest call of any router is on this sequence: the smallest gap between the last logit chosen
    and the first one left out, over the spread of that router's logits."""
    w64 = {k: (v.to(torch.float64) if v.is_floating_point() else v) for k, v in w.items()}
    x = w64["embed"][torch.tensor(tokens, dtype=torch.long)]
    positions = torch.arange(len(tokens))
    worst = math.inf
    for i, spec in enumerate(cfg["layers"]):
        mlp = spec.get("mlp")
        if mlp is not None and mlp["kind"] == "moe" and mlp["router"]["top"] < mlp["router"]["experts"]:
            pre = f"l{spec.get('weights_of', i)}."
            h = rms_norm(x, w64[pre + "norm1"], cfg["norm"]["eps"])
            z = linear(w64[pre + "mlp.router"], h) + w64[pre + "mlp.router.b"]
            s = z.sort(-1, descending=True).values
            top = mlp["router"]["top"]
            worst = min(worst, float(((s[:, top - 1] - s[:, top]) / z.std()).min()))
        x = layer(cfg, w64, i, x, positions)
    return worst


def greedy(cfg: dict, w: Weights, prompt: List[int], n: int) -> List[int]:
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(forward(cfg, w, toks)[-1].argmax()))
    return toks[len(prompt):]
