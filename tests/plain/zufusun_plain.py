"""Plain, slow Zufusun forward for whole sequences: no cache, no batching, no kernels.

One function per mechanism, written from the design's equations with torch on the CPU (float64 by default).  It
shares no code with ``ember_b200``: it takes the configuration as the dictionary config.json holds and the weights
as a name -> tensor dictionary.  Attention is a dense [T, T] score matrix under an explicit mask; the recurrence
is a loop over tokens from a zero state; the latent attention builds every head's keys and values from the
latent (no folding of the up-projections into the queries).

Notation: x [T, width] is the residual stream, h a sublayer's input, W[name] a matrix stored [out, in].
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def lin(h: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor] = None) -> torch.Tensor:
    y = h @ w.to(h.dtype).T
    return y + b.to(h.dtype) if b is not None else y


def rms_norm(x: torch.Tensor, w: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y * w.to(x.dtype) if w is not None else y


def visible(T: int, window: int = 0, keep_first: int = 0) -> torch.Tensor:
    """[T, T] bool: query i sees key j when j <= i and, under a window, i - j < window or j < keep_first."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if window > 0:
        ok = ok & ((i - j < window) | (j < keep_first))
    return ok


def sink_softmax(scores: torch.Tensor, mask: torch.Tensor, sink: torch.Tensor) -> torch.Tensor:
    """Weights over keys whose denominator also holds exp(sink) per head.  scores [H, T, T], sink [H]."""
    s = scores.masked_fill(~mask[None], -math.inf)
    m = torch.maximum(s.max(-1, keepdim=True).values, sink.to(s.dtype)[:, None, None])
    e = torch.exp(s - m)
    return e / (e.sum(-1, keepdim=True) + torch.exp(sink.to(s.dtype)[:, None, None] - m))


def interleaved_rotation(x: torch.Tensor, base: float, dims: int, first_position: int = 0) -> torch.Tensor:
    """x [T, ..., n]: elements 2i and 2i + 1 (i < dims / 2) of the token at position p turn by p * base^(-2i / dims)."""
    T = x.shape[0]
    pos = torch.arange(first_position, first_position + T, dtype=x.dtype)
    freq = torch.tensor(base, dtype=x.dtype) ** (-torch.arange(0, dims, 2, dtype=x.dtype) / dims)
    ang = pos[:, None] * freq[None, :]
    shape = (T,) + (1,) * (x.dim() - 2) + (dims // 2,)
    c, s = torch.cos(ang).view(shape), torch.sin(ang).view(shape)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


# ------------------------------------------------------------------------------------------------ mixers
def windowed_sink_attention(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    """Grouped-query attention with biased projections, one RMS norm over the whole query (key) projection, no
    rotation, a window that keeps the first tokens, and a sink in the softmax."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms_norm(lin(h, W[p + "q"], W[p + "q.b"]), W[p + "q.norm"], eps).view(T, H, D)
    k = rms_norm(lin(h, W[p + "k"], W[p + "k.b"]), W[p + "k.norm"], eps).view(T, G, D)
    v = lin(h, W[p + "v"], W[p + "v.b"]).view(T, G, V)
    rep = H // G
    k = k.repeat_interleave(rep, dim=1)
    v = v.repeat_interleave(rep, dim=1)
    scores = torch.einsum("ihd,jhd->hij", q, k) * m["scale"]
    mask = visible(T, int(m["mask"]["size"]), int(m["mask"].get("keep_first", 0))) if m.get("mask") else visible(T)
    w = sink_softmax(scores, mask, W[p + "sink"])
    o = torch.einsum("hij,jhd->ihd", w, v).reshape(T, H * V)
    return lin(o, W[p + "o"])


def latent_kv(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float):
    """(latent c [T, kv_rank], rotated shared key part [T, rot_dim]) of the layer that owns W_dkv."""
    r, R = m["kv_rank"], m["rot_dim"]
    d = lin(h, W[p + "dkv"])
    c = rms_norm(d[:, :r], W[p + "dkv.norm"], eps)
    kr = interleaved_rotation(d[:, r:r + R], m["rot"]["base"], m["rot"]["dims"])
    return c, kr


def latent_attention(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float, c: torch.Tensor,
                     kr: torch.Tensor) -> torch.Tensor:
    """Causal attention whose keys and values are up-projections of a shared latent, with a rotated key part shared
    by the heads, a sink, and a sigmoid gate on the concatenated heads."""
    T = h.shape[0]
    H, D, R, V = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    cq = rms_norm(lin(h, W[p + "dq"]), W[p + "dq.norm"], eps)
    q = lin(cq, W[p + "uq"]).view(T, H, D + R)
    qn = q[..., :D]
    qr = interleaved_rotation(q[..., D:].contiguous(), m["rot"]["base"], m["rot"]["dims"])
    kn = lin(c, W[p + "uk"]).view(T, H, D)
    v = lin(c, W[p + "uv"]).view(T, H, V)
    scores = (torch.einsum("ihd,jhd->hij", qn, kn) + torch.einsum("ihd,jd->hij", qr, kr)) * m["scale"]
    w = sink_softmax(scores, visible(T), W[p + "sink"])
    o = torch.einsum("hij,jhd->ihd", w, v).reshape(T, H * V)
    o = o * torch.sigmoid(lin(h, W[p + "g"]))
    return lin(o, W[p + "o"])


def gated_linear_attention(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    """S_t = diag(alpha_t) S_{t-1} + k_t v_t^T, o_t = S_t^T q_t per head, alpha = sigmoid(z)^(1 / tau) per key channel."""
    T = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    q = (lin(h, W[p + "q"]) * D ** -0.5).view(T, H, D)
    k = lin(h, W[p + "k"]).view(T, H, D)
    v = lin(h, W[p + "v"]).view(T, H, V)
    z = lin(lin(h, W[p + "a1"]), W[p + "a2"], W[p + "a2.b"]).view(T, H, D)
    alpha = torch.sigmoid(z) ** (1.0 / m["tau"])
    o = torch.zeros(T, H, V, dtype=h.dtype)
    for hd in range(H):
        S = torch.zeros(D, V, dtype=h.dtype)
        for t in range(T):
            S = alpha[t, hd][:, None] * S + torch.outer(k[t, hd], v[t, hd])
            o[t, hd] = S.T @ q[t, hd]
    o = rms_norm(o, W[p + "norm"], eps).reshape(T, H * V)
    g = lin(h, W[p + "g"])
    return lin(o * (g * torch.sigmoid(g)), W[p + "o"])


# ------------------------------------------------------------------------------------------ feed-forward
def clamped_expert(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, limit: float) -> torch.Tensor:
    g = torch.clamp(lin(h, W[p + "gate"]), max=limit)
    u = torch.clamp(lin(h, W[p + "up"]), min=-limit, max=limit)
    return lin(g * torch.sigmoid(1.702 * g) * (u + 1.0), W[p + "down"])


def routed_experts(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, mlp: dict) -> torch.Tensor:
    """Every token goes to its ``top`` experts by router logit; their weights are the softmax of those logits alone."""
    E, top, limit = mlp["router"]["experts"], mlp["router"]["top"], mlp["expert"]["limit"]
    z = lin(h, W[p + "router"])
    val, idx = torch.topk(z, top, dim=-1)
    wgt = torch.softmax(val, dim=-1)
    out = torch.zeros_like(h)
    for e in range(E):
        y = clamped_expert(h, W, f"{p}e{e}.", limit)
        share = (wgt * (idx == e)).sum(-1, keepdim=True)
        out = out + share * y
    return out


def router_choice(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, mlp: dict):
    """(indices [T, top] in descending order of logit, weights [T, top])."""
    val, idx = torch.topk(lin(h, W[p + "router"]), mlp["router"]["top"], dim=-1)
    return idx, torch.softmax(val, dim=-1)


# ------------------------------------------------------------------------------------------------- model
def forward(cfg: dict, W: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float64,
            layers_out: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence.  ``layers_out``: a list that receives the residual stream after every layer."""
    eps = cfg["norm"]["eps"]
    x = W["embed"].to(dtype)[torch.tensor(tokens, dtype=torch.long)]
    latents = {}
    for i, layer in enumerate(cfg["layers"]):
        p, m, kind = f"l{i}.", layer["mixer"], layer["type"]
        if kind == "attention":
            y = windowed_sink_attention(x, W, p + "mix.", m, eps)
        elif kind == "latent_attention":
            src = m.get("kv_from")
            if src is None:
                latents[i] = latent_kv(x, W, p + "mix.", m, eps)
                src = i
            y = latent_attention(x, W, p + "mix.", m, eps, *latents[src])
        elif kind == "gla":
            y = gated_linear_attention(x, W, p + "mix.", m, eps)
        else:
            raise ValueError(f"unknown mixer {kind!r}")
        x = x + rms_norm(y, W[p + "norm1"], eps)
        if layer.get("mlp") is not None:
            x = x + rms_norm(routed_experts(x, W, p + "mlp.", layer["mlp"]), W[p + "norm2"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    x = rms_norm(x, W["final.norm"], eps)
    return lin(x, W["embed"])
