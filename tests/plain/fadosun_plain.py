"""Plain, slow Fadosun forward for whole sequences: no cache, no batching, no kernels.

One function per mechanism, written from the design's equations with torch on the CPU (float64 by default).  It
shares no code with ``ember_b200``: it takes the configuration as the dictionary config.json holds and the
weights as a name -> tensor dictionary.  Every recurrence is a loop over tokens that starts from a zero state.

Notation: x [T, width] is the residual stream, h a sublayer's input, W[name] a matrix stored [out, in].
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch
import torch.nn.functional as F


def lin(h: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor] = None) -> torch.Tensor:
    y = h @ w.to(h.dtype).T
    return y + b.to(h.dtype) if b is not None else y


def layer_norm(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, eps: float) -> torch.Tensor:
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w.to(x.dtype) + b.to(x.dtype)


def rms_div(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def short_conv(x: torch.Tensor, taps: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y[t, c] = sum_j taps[c, j] * x[t - (n - 1 - j), c]: the last tap meets the current token, inputs before the
    sequence are zero."""
    T, C = x.shape
    n = taps.shape[1]
    pad = torch.cat([torch.zeros(n - 1, C, dtype=x.dtype), x], 0)
    y = torch.zeros_like(x)
    for j in range(n):
        y = y + pad[j:j + T] * taps[:, j].to(x.dtype)
    return y + bias.to(x.dtype) if bias is not None else y


def silu(x):
    return x * torch.sigmoid(x)


def relu_glu(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    return lin(torch.relu(lin(h, W[p + "gate"])) * lin(h, W[p + "up"]), W[p + "down"])


# ------------------------------------------------------------------------------------------------ mixers
def channel_delta(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    """Delta rule with one decay per head and key channel."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_conv(lin(h, W[p + "q"]), W[p + "q.conv"])).view(T, G, D)
    k = silu(short_conv(lin(h, W[p + "k"]), W[p + "k.conv"])).view(T, G, D)
    v = silu(short_conv(lin(h, W[p + "v"]), W[p + "v.conv"])).view(T, H, V)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(lin(h, W[p + "b"]))                                              # [T, H]
    a = lin(lin(h, W[p + "a1"]), W[p + "a2"]) + W[p + "dt_bias"].to(h.dtype)
    rate = torch.exp(W[p + "A_log"].to(h.dtype))                                          # [H]
    g = torch.exp(-rate[None, :, None] * F.softplus(a).view(T, H, D))                     # [T, H, D]
    gate = torch.sigmoid(lin(lin(h, W[p + "g1"]), W[p + "g2"])).view(T, H, V)
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for hd in range(H):
        kv = hd // (H // G)
        S = torch.zeros(D, V, dtype=h.dtype)
        for t in range(T):
            S = g[t, hd][:, None] * S
            u = beta[t, hd] * (v[t, hd] - S.T @ k[t, kv])
            S = S + torch.outer(k[t, kv], u)
            out[t, hd] = S.T @ q[t, kv]
    out = rms_div(out, eps) * W[p + "norm"].to(h.dtype) * gate
    return lin(out.reshape(T, H * V), W[p + "o"])


def mlstm(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    """Matrix memory with exponential input gate, stabilised by a running maximum that starts at zero."""
    T = h.shape[0]
    H, D, V, cap = m["heads"], m["dim"], m["vdim"], float(m["gate_cap"])
    q = (lin(h, W[p + "q"]) * D ** -0.5).view(T, H, D)
    k = lin(h, W[p + "k"]).view(T, H, D)
    v = lin(h, W[p + "v"]).view(T, H, V)
    ig = cap * torch.tanh(lin(h, W[p + "i"], W[p + "i.b"]) / cap)                         # log input gate [T, H]
    fg = F.logsigmoid(cap * torch.tanh(lin(h, W[p + "f"], W[p + "f.b"]) / cap))           # log forget gate
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for hd in range(H):
        S = torch.zeros(D, V, dtype=h.dtype)
        n = torch.zeros(D, dtype=h.dtype)
        mx = torch.zeros((), dtype=h.dtype)
        for t in range(T):
            new = torch.maximum(fg[t, hd] + mx, ig[t, hd])
            keep, put = torch.exp(fg[t, hd] + mx - new), torch.exp(ig[t, hd] - new)
            S = keep * S + put * torch.outer(k[t, hd], v[t, hd])
            n = keep * n + put * k[t, hd]
            mx = new
            den = torch.maximum((n @ q[t, hd]).abs(), torch.exp(-mx)) + 1e-6
            out[t, hd] = (S.T @ q[t, hd]) / den
    out = rms_div(out, eps).reshape(T, H * V) * W[p + "norm"].to(h.dtype) * torch.sigmoid(lin(h, W[p + "g"]))
    return lin(out, W[p + "o"])


def rotate(x: torch.Tensor, pos: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x [T, heads, D]: rotates pairs (i, i + dims/2) of the first ``dims`` entries by pos * base^(-2i/dims)."""
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=x.dtype)
    a = pos.to(x.dtype)[:, None] * f[None, :]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, w = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - w * s, w * c + u * s, x[..., dims:]], -1)


def sigmoid_attention(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict) -> torch.Tensor:
    """Causal attention whose weights are sigmoid(score + per-head bias), not normalised over keys."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = rotate(lin(h, W[p + "q"]).view(T, H, D), pos, m["rot"]["dims"], m["rot"]["base"])
    k = rotate(lin(h, W[p + "k"]).view(T, G, D), pos, m["rot"]["dims"], m["rot"]["base"])
    v = lin(h, W[p + "v"]).view(T, G, V)
    out = torch.zeros(T, H, V, dtype=h.dtype)
    seen = torch.tril(torch.ones(T, T, dtype=torch.bool))
    for hd in range(H):
        kv = hd // (H // G)
        w = torch.sigmoid(q[:, hd] @ k[:, kv].T * m["scale"] + W[p + "pb"][hd].to(h.dtype))
        out[:, hd] = torch.where(seen, w, torch.zeros_like(w)) @ v[:, kv]
    return lin(out.reshape(T, H * V), W[p + "o"])


def mamba2(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    """Selective state space with a scalar decay per head."""
    T = h.shape[0]
    H, V, N, G, parts = m["heads"], m["vdim"], m["state"], m["groups"], m["norm_groups"]
    inner = H * V
    zxbcdt = lin(h, W[p + "in"])
    z, xbc, dt = zxbcdt[:, :inner], zxbcdt[:, inner:2 * inner + 2 * G * N], zxbcdt[:, 2 * inner + 2 * G * N:]
    xbc = silu(short_conv(xbc, W[p + "conv"], W[p + "conv.b"]))
    x = xbc[:, :inner].view(T, H, V)
    B = xbc[:, inner:inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N:].view(T, G, N)
    dt = F.softplus(dt + W[p + "dt_bias"].to(h.dtype))                                    # [T, H]
    rate = torch.exp(W[p + "A_log"].to(h.dtype))
    y = torch.zeros(T, H, V, dtype=h.dtype)
    for hd in range(H):
        g = hd // (H // G)
        S = torch.zeros(N, V, dtype=h.dtype)
        for t in range(T):
            S = torch.exp(-rate[hd] * dt[t, hd]) * S + dt[t, hd] * torch.outer(B[t, g], x[t, hd])
            y[t, hd] = S.T @ C[t, g] + W[p + "D"][hd].to(h.dtype) * x[t, hd]
    y = y.reshape(T, inner) * silu(z)
    y = rms_div(y.view(T, parts, inner // parts), eps).reshape(T, inner) * W[p + "norm"].to(h.dtype)
    return lin(y, W[p + "o"])


def parallel(h, W, p, m, eps):
    return m["left_scale"] * sigmoid_attention(h, W, p + "left.", m["left"]) + \
        m["right_scale"] * mamba2(h, W, p + "right.", m["right"], eps)


MIXERS = {"channel_delta": channel_delta, "mlstm": mlstm, "parallel": parallel}


# ------------------------------------------------------------------------------------------------- model
def layer(x: torch.Tensor, W: Dict[str, torch.Tensor], i: int, spec: dict, eps: float) -> torch.Tensor:
    p = f"l{i}."

    def norm(name, t):
        return layer_norm(t, W[p + name], W[p + name + ".b"], eps)

    h = norm("norm1", x)
    if spec["type"] == "parallel":
        y = parallel(h, W, p + "mix.", spec["mixer"], eps)
    else:
        y = MIXERS[spec["type"]](h, W, p + "mix.", spec["mixer"], eps)
    x = x + norm("norm1b", y * torch.sigmoid(lin(h, W[p + "rg1"], W[p + "rg1.b"])))
    if spec.get("mlp") is not None:
        h = norm("norm2", x)
        y = relu_glu(h, W, p + "mlp.")
        x = x + norm("norm2b", y * torch.sigmoid(lin(h, W[p + "rg2"], W[p + "rg2.b"])))
    return x


def forward(config: dict, W: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float64, residuals=None) -> torch.Tensor:
    """Logits [T, vocab] for one sequence; ``residuals`` (a list) receives the stream after every layer."""
    eps = float(config["norm"]["eps"])
    x = W["embed"].to(dtype)[torch.tensor(tokens, dtype=torch.long)]
    for i, spec in enumerate(config["layers"]):
        x = layer(x, W, i, spec, eps)
        if residuals is not None:
            residuals.append(x.clone())
    x = layer_norm(x, W["final.norm"], W["final.norm.b"], eps)
    return lin(x, W["head"])
