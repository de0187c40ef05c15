"""A plain, slow implementation of the Panupel design: one function per mechanism, whole sequences at
once, no cache, no batching.  It shares nothing with the engine; the tests compare the engine with it.

Everything is computed in the dtype of the tensors handed in (float64 for an oracle, float32 to see what
rounding alone does).  A model is `(config, weights)`: the parsed config.json and a dict name -> tensor.

Notation: T tokens, H heads, G key/value heads, d the query/key size of a head, e its value size.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch

Weights = Dict[str, torch.Tensor]


# ---- small pieces ----------------------------------------------------------------------------------
def rms_norm(x: torch.Tensor, w: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis, times w if given."""
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y * w if w is not None else y


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def log_sigmoid(z: torch.Tensor) -> torch.Tensor:
    return -softplus(-z)


# With ROUND_PRODUCTS set, every matrix product rounds its input to bfloat16 values and, unless the caller keeps
# the result in 32-bit, its output too: what an engine that multiplies in bfloat16 with 32-bit sums does.  The
# tests use this to learn how far rounding alone moves the logits of a given model.
ROUND_PRODUCTS = False


def _bf16(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.bfloat16).to(x.dtype)


def linear(w: torch.Tensor, h: torch.Tensor, keep32: bool = False) -> torch.Tensor:
    """Weights are stored [out, in]; rows of h are tokens."""
    if not ROUND_PRODUCTS:
        return h @ w.to(h.dtype).t()
    y = _bf16(h) @ w.to(h.dtype).t()
    return y if keep32 else _bf16(y)


# ---- rotary positions ------------------------------------------------------------------------------
def rotary_frequencies(dims: int, base: float, scaling: Optional[dict]) -> List[float]:
    """f_i = base^(-2i/dims), i < dims/2, then the long-context rescaling: wavelengths shorter than
    original/high are kept, longer than original/low are divided by `factor`, and in between the two are
    blended linearly in original/wavelength."""
    out = []
    for i in range(dims // 2):
        f = float(base) ** (-2.0 * i / dims)
        if scaling:
            factor, low, high, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
            wavelength = 2.0 * math.pi / f
            if wavelength < orig / high:
                pass
            elif wavelength > orig / low:
                f = f / factor
            else:
                s = (orig / wavelength - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return out


def rotate(x: torch.Tensor, positions: torch.Tensor, freqs: List[float], dims: int) -> torch.Tensor:
    """x: [T, heads, d].  The first `dims` entries of each head turn; entry i pairs with entry i + dims/2."""
    half = dims // 2
    f = torch.tensor(freqs, dtype=x.dtype)
    a = positions.to(x.dtype)[:, None] * f[None, :]                      # [T, half]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


# ---- softmax attention with a sink -----------------------------------------------------------------
def sink_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                   sink: Optional[torch.Tensor]) -> torch.Tensor:
    """q [T, H, d], k [T, G, d], v [T, G, e] -> [T, H, e].  Causal.  The sink adds exp(sink_h) to the
    softmax's denominator and nothing to its numerator."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].t()) * scale                              # [T, T]
        s = s.masked_fill(torch.ones(T, T, dtype=torch.bool).triu(1), float("-inf"))
        m = s.max(-1, keepdim=True).values
        if sink is not None:
            m = torch.maximum(m, sink[h].to(q.dtype).reshape(1, 1))
        p = torch.exp(s - m)
        den = p.sum(-1, keepdim=True)
        if sink is not None:
            den = den + torch.exp(sink[h].to(q.dtype) - m)
        out[:, h] = (p / den) @ v[:, g]
    return out


def left_mixer(c: dict, w: Weights, pre: str, h: torch.Tensor, positions: torch.Tensor, eps: float) -> torch.Tensor:
    H, G, d, e = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    T = h.shape[0]
    q = rms_norm(linear(w[pre + "q"], h), w[pre + "q.norm"].to(h.dtype), eps).view(T, H, d)
    k = rms_norm(linear(w[pre + "k"], h), w[pre + "k.norm"].to(h.dtype), eps).view(T, G, d)
    v = linear(w[pre + "v"], h).view(T, G, e)
    rot = c.get("rot")
    if rot:
        freqs = rotary_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
        q, k = rotate(q, positions, freqs, rot["dims"]), rotate(k, positions, freqs, rot["dims"])
    o = sink_attention(q, k, v, float(c["scale"]), w.get(pre + "sink"))
    gate = torch.sigmoid(linear(w[pre + "g"], h, keep32=True))           # [T, H]
    o = o * gate[:, :, None]
    return linear(w[pre + "o"], o.reshape(T, H * e), keep32=True)


# ---- matrix memory (mLSTM) -------------------------------------------------------------------------
def matrix_memory(q, k, v, log_i, log_f, state=None):
    """One head.  q, k [T, d], v [T, e], log_i, log_f [T].  Token by token:
        m' = max(log_f + m, log_i);  S' = exp(log_f + m - m') S + exp(log_i - m') k v^T;  n' likewise with k;
        o = S'^T q / (max(|n' . q|, exp(-m')) + 1e-6)
    The state (S [d, e], n [d], m) starts as zeros, m included."""
    T, d = q.shape
    e = v.shape[1]
    if state is None:
        S, n, m = torch.zeros(d, e, dtype=q.dtype), torch.zeros(d, dtype=q.dtype), torch.zeros((), dtype=q.dtype)
    else:
        S, n, m = state
    out = torch.zeros(T, e, dtype=q.dtype)
    for t in range(T):
        m_new = torch.maximum(log_f[t] + m, log_i[t])
        a, b = torch.exp(log_f[t] + m - m_new), torch.exp(log_i[t] - m_new)
        S = a * S + b * torch.outer(k[t], v[t])
        n = a * n + b * k[t]
        m = m_new
        out[t] = (S.t() @ q[t]) / (torch.maximum((n * q[t]).sum().abs(), torch.exp(-m)) + 1e-6)
    return out, (S, n, m)


def right_mixer(c: dict, w: Weights, pre: str, h: torch.Tensor, eps: float) -> torch.Tensor:
    H, d, e, cap = c["heads"], c["dim"], c["vdim"], float(c["gate_cap"])
    T = h.shape[0]
    q = (linear(w[pre + "q"], h) * d ** -0.5).view(T, H, d)
    k = linear(w[pre + "k"], h).view(T, H, d)
    v = linear(w[pre + "v"], h).view(T, H, e)
    log_i = cap * torch.tanh((linear(w[pre + "i"], h, keep32=True) + w[pre + "i.b"].to(h.dtype)) / cap)
    log_f = log_sigmoid(cap * torch.tanh((linear(w[pre + "f"], h, keep32=True) + w[pre + "f.b"].to(h.dtype)) / cap))
    o = torch.stack([matrix_memory(q[:, j], k[:, j], v[:, j], log_i[:, j], log_f[:, j])[0] for j in range(H)], dim=1)
    o = rms_norm(o, None, eps).reshape(T, H * e) * w[pre + "norm"].to(h.dtype)
    o = o * torch.sigmoid(linear(w[pre + "g"], h))
    return linear(w[pre + "o"], o, keep32=True)


def parallel_mixer(c: dict, w: Weights, pre: str, h, positions, eps):
    return (float(c["left_scale"]) * left_mixer(c["left"], w, pre + "left.", h, positions, eps) +
            float(c["right_scale"]) * right_mixer(c["right"], w, pre + "right.", h, eps))


# ---- gated delta rule ------------------------------------------------------------------------------
def short_conv(x: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """x [T, C], taps [C, n]: y[t] = sum_j taps[:, j] * x[t - (n - 1) + j], zeros before the start."""
    T, C = x.shape
    n = taps.shape[1]
    padded = torch.cat([torch.zeros(n - 1, C, dtype=x.dtype), x], dim=0)
    y = torch.zeros_like(x)
    for j in range(n):
        y = y + padded[j:j + T] * taps[:, j].to(x.dtype)[None, :]
    return y


def unit(x: torch.Tensor) -> torch.Tensor:
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + 1e-6)


def delta_rule(q, k, v, beta, decay, S=None):
    """One head.  q, k [T, d] (already unit vectors, q scaled), v [T, e], beta, decay [T].  Token by token:
        S <- decay S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q."""
    T, d = q.shape
    e = v.shape[1]
    if S is None:
        S = torch.zeros(d, e, dtype=q.dtype)
    out = torch.zeros(T, e, dtype=q.dtype)
    for t in range(T):
        S = decay[t] * S
        u = beta[t] * (v[t] - S.t() @ k[t])
        S = S + torch.outer(k[t], u)
        out[t] = S.t() @ q[t]
    return out, S


def delta_mixer(c: dict, w: Weights, pre: str, h: torch.Tensor, eps: float) -> torch.Tensor:
    H, G, d, e = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    T = h.shape[0]
    q = silu(short_conv(linear(w[pre + "q"], h), w[pre + "q.conv"])).view(T, G, d)
    k = silu(short_conv(linear(w[pre + "k"], h), w[pre + "k.conv"])).view(T, G, d)
    v = silu(short_conv(linear(w[pre + "v"], h), w[pre + "v.conv"])).view(T, H, e)
    q, k = unit(q) * d ** -0.5, unit(k)
    beta = torch.sigmoid(linear(w[pre + "b"], h, keep32=True))                                         # [T, H]
    decay = torch.exp(-torch.exp(w[pre + "A_log"].to(h.dtype)) *
                      softplus(linear(w[pre + "a"], h, keep32=True) + w[pre + "dt_bias"].to(h.dtype)))  # [T, H]
    o = torch.stack([delta_rule(q[:, j // (H // G)], k[:, j // (H // G)], v[:, j], beta[:, j], decay[:, j])[0]
                     for j in range(H)], dim=1)                                           # [T, H, e]
    o = rms_norm(o, w[pre + "norm"].to(h.dtype), eps)
    o = o.reshape(T, H * e) * silu(linear(w[pre + "g"], h))
    return linear(w[pre + "o"], o, keep32=True)


# ---- feed-forward, layer, model --------------------------------------------------------------------
def gated_mlp(w: Weights, pre: str, h: torch.Tensor) -> torch.Tensor:
    return linear(w[pre + "down"], silu(linear(w[pre + "gate"], h)) * linear(w[pre + "up"], h), keep32=True)


def layer(config: dict, w: Weights, i: int, x: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
    spec = config["layers"][i]
    eps, mult = float(config["norm"]["eps"]), float(config["residual_mult"])
    p = f"l{i}."
    h = rms_norm(x, w[p + "norm1"].to(x.dtype), eps)
    if spec["type"] == "parallel":
        y = parallel_mixer(spec["mixer"], w, p + "mix.", h, positions, eps)
    elif spec["type"] == "delta":
        y = delta_mixer(spec["mixer"], w, p + "mix.", h, eps)
    else:
        raise ValueError(spec["type"])
    x = x + mult * rms_norm(y, w[p + "norm1b"].to(x.dtype), eps)
    if spec.get("mlp"):
        y = gated_mlp(w, p + "mlp.", rms_norm(x, w[p + "norm2"].to(x.dtype), eps))
        x = x + mult * rms_norm(y, w[p + "norm2b"].to(x.dtype), eps)
    return x


def run_order(config: dict) -> List[Tuple[int, bool]]:
    """(layer, whether the pass's input mix comes right before it), in the order the layers run."""
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    start, stop, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, False) for i in range(start)]
    for _ in range(times):
        order += [(i, i == start) for i in range(start, stop)]
    return order + [(i, False) for i in range(stop, n)]


def forward_rounded(config: dict, w: Weights, tokens: List[int], dtype=torch.float64):
    """`forward` with every product's operands (and results, where an engine keeps them in 16 bits) rounded to
    bfloat16 values."""
    global ROUND_PRODUCTS
    ROUND_PRODUCTS = True
    try:
        return forward(config, w, tokens, dtype)
    finally:
        ROUND_PRODUCTS = False


def forward(config: dict, w: Weights, tokens: List[int], dtype=torch.float64):
    """Logits [T, vocab] and the residual stream after every layer run [runs, T, width]."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}
    x = w["embed"][torch.tensor(tokens, dtype=torch.long)]
    x0 = x
    positions = torch.arange(len(tokens))
    streams = []
    for i, mix_in in run_order(config):
        if mix_in:
            x = linear(w["loop.in"], torch.cat([x, x0], dim=-1), keep32=True)
        x = layer(config, w, i, x, positions)
        streams.append(x)
    y = rms_norm(x, w["final.norm"], float(config["norm"]["eps"]))
    return linear(w["head"], y, keep32=True), torch.stack(streams)
