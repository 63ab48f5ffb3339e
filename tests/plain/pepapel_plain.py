"""Plain, slow Pepapel forward for whole sequences: no cache, no batching, no kernels.

One function per mechanism, written from the design's equations with torch on the CPU (float64 by default).  It
shares no code with ``ember_b200``: it takes the configuration as the dictionary config.json holds and the weights
as a name -> tensor dictionary.  Attention is a dense [T, T] score matrix under a boolean mask; the recurrence is a
loop over tokens from a zero state; a short convolution is a sum of shifted copies.

Notation: x [T, width] the residual stream, h a sublayer's input, W[name] a matrix stored [out, in].
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


def layer_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """(x - mean) / sqrt(var + eps) * w with var the mean squared deviation; no bias."""
    d = x - x.mean(-1, keepdim=True)
    return d / torch.sqrt((d * d).mean(-1, keepdim=True) + eps) * w.to(x.dtype)


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def short_conv(u: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """y[t, c] = sum_j taps[c, j] u[t - (n - 1) + j, c], zeros before the start: the last column meets the current token."""
    T, n = u.shape[0], taps.shape[1]
    w = taps.to(u.dtype)
    y = torch.zeros_like(u)
    for j in range(n):
        back = n - 1 - j
        if back < T:
            y[back:] += u[:T - back] * w[:, j]
    return y


# --------------------------------------------------------------------------------------------- positions
def rotate_half(x: torch.Tensor, rot: dict) -> torch.Tensor:
    """x [T, heads, dim]: the first rot.dims elements of every head turn, element i with element i + dims/2, by
    the angle p * base^(-2i/dims) / factor; the rest passes."""
    dims, base = int(rot["dims"]), float(rot["base"])
    factor = float((rot.get("scaling") or {}).get("factor", 1.0))
    T, half = x.shape[0], dims // 2
    f = base ** (-2.0 * torch.arange(half, dtype=x.dtype) / dims) / factor
    a = torch.arange(T, dtype=x.dtype)[:, None] * f[None, :]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def query_temperature(T: int, q_temp: dict, dtype) -> torch.Tensor:
    """1 + coef * ln(floor((p + 1) / every) + 1) for p = 0 .. T-1."""
    p = torch.arange(T, dtype=torch.int64)
    steps = torch.div(p + 1, int(q_temp["every"]), rounding_mode="floor")
    return 1.0 + float(q_temp["coef"]) * torch.log(steps.to(dtype) + 1.0)


def visible(T: int, chunk: int = 0) -> torch.Tensor:
    """[T, T] mask: j <= i, and with ``chunk`` also floor(i / chunk) == floor(j / chunk)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    m = j <= i
    if chunk > 0:
        m = m & (torch.div(i, chunk, rounding_mode="floor") == torch.div(j, chunk, rounding_mode="floor"))
    return m


def softmax_attention(q, k, v, scale: float, mask: torch.Tensor, softcap: float = 0.0) -> torch.Tensor:
    """q [T, H, dim], k [T, G, dim], v [T, G, vdim] -> [T, H, vdim]; query head h reads key head h // (H / G)."""
    H, G = q.shape[1], k.shape[1]
    out = []
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        if softcap > 0:
            s = softcap * torch.tanh(s / softcap)
        s = s.masked_fill(~mask, float("-inf"))
        out.append(torch.softmax(s, dim=-1) @ v[:, g])
    return torch.stack(out, dim=1)


# ------------------------------------------------------------------------------------------------ mixers
def attention_mixer(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    """Softmax attention with a norm per head on queries and keys (one weight for all heads), no rotation, queries
    scaled with their position, capped scores."""
    T = h.shape[0]
    H, G, D, V = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = rms_norm(lin(h, W[p + "q"]).reshape(T, H, D), W[p + "q.norm"], eps)
    k = rms_norm(lin(h, W[p + "k"]).reshape(T, G, D), W[p + "k.norm"], eps)
    v = lin(h, W[p + "v"]).reshape(T, G, V)
    if m.get("q_temp"):
        q = q * query_temperature(T, m["q_temp"], h.dtype)[:, None, None]
    o = softmax_attention(q, k, v, float(m["scale"]), visible(T), float(m.get("softcap") or 0.0))
    return lin(o.reshape(T, H * V), W[p + "o"])


def chunked_attention_mixer(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    """Softmax attention inside chunks of positions: short convolutions on q, k, v, a norm over the whole query and
    key projections, a rotation, and a sigmoid gate per head on the result."""
    T = h.shape[0]
    H, G, D, V = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q, k, v = lin(h, W[p + "q"]), lin(h, W[p + "k"]), lin(h, W[p + "v"])
    if m.get("conv"):
        q, k, v = short_conv(q, W[p + "q.conv"]), short_conv(k, W[p + "k.conv"]), short_conv(v, W[p + "v.conv"])
    q = rms_norm(q, W[p + "q.norm"], eps).reshape(T, H, D)
    k = rms_norm(k, W[p + "k.norm"], eps).reshape(T, G, D)
    if m.get("rot"):
        q, k = rotate_half(q, m["rot"]), rotate_half(k, m["rot"])
    o = softmax_attention(q, k, v.reshape(T, G, V), float(m["scale"]), visible(T, int((m.get("mask") or {}).get("size", 0))))
    o = o * torch.sigmoid(lin(h, W[p + "g"]))[:, :, None]
    return lin(o.reshape(T, H * V), W[p + "o"])


def delta_rule_mixer(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    """Gated delta rule with one decay per head: S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q."""
    T, dt = h.shape[0], h.dtype
    H, G, D, V = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = silu(short_conv(lin(h, W[p + "q"]), W[p + "q.conv"])).reshape(T, G, D)
    k = silu(short_conv(lin(h, W[p + "k"]), W[p + "k.conv"])).reshape(T, G, D)
    v = silu(short_conv(lin(h, W[p + "v"]), W[p + "v.conv"])).reshape(T, H, V)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(lin(h, W[p + "b"]))                                             # [T, H]
    decay = torch.exp(-torch.exp(W[p + "A_log"].to(dt)) * torch.nn.functional.softplus(lin(h, W[p + "a"]) + W[p + "dt_bias"].to(dt)))
    o = torch.zeros(T, H, V, dtype=dt)
    for hd in range(H):
        g = hd // (H // G)
        S = torch.zeros(D, V, dtype=dt)
        for t in range(T):
            S = decay[t, hd] * S
            u = beta[t, hd] * (v[t, hd] - S.T @ k[t, g])
            S = S + torch.outer(k[t, g], u)
            o[t, hd] = S.T @ q[t, g]
    o = rms_norm(o, W[p + "norm"], eps) * silu(lin(h, W[p + "g"])).reshape(T, H, V)
    return lin(o.reshape(T, H * V), W[p + "o"])


def parallel_mixer(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    left = chunked_attention_mixer(h, W, p + "left.", m["left"], eps)
    right = delta_rule_mixer(h, W, p + "right.", m["right"], eps)
    return 0.5 * (rms_norm(left, W[p + "left.out"], eps) + rms_norm(right, W[p + "right.out"], eps))


# ----------------------------------------------------------------------------------------- feed-forwards
def dense_ff(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, mlp: dict) -> torch.Tensor:
    limit = float(mlp["limit"])
    g = torch.clamp(lin(h, W[p + "gate"], W[p + "gate.b"]), max=limit)
    u = torch.clamp(lin(h, W[p + "up"], W[p + "up.b"]), -limit, limit)
    return lin(g * torch.sigmoid(1.702 * g) * (u + 1.0), W[p + "down"], W[p + "down.b"])


def route(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, router: dict):
    """(chosen [T, top], weights [T, top]): softmax over all outputs; the choice is by score + correction among the
    outputs of the ``keep`` groups whose best such score is largest; the weights are the plain scores."""
    E, I, top = int(router["experts"]), int(router.get("identity") or 0), int(router["top"])
    n = E + I
    s = torch.softmax(lin(h, W[p + "router"]), dim=-1)
    c = s + W[p + "correction"].to(h.dtype)
    groups = router.get("groups")
    if groups:
        count, keep = int(groups["count"]), int(groups["keep"])
        per = n // count
        best = c.reshape(-1, count, per).max(-1).values
        kept = torch.zeros_like(best, dtype=torch.bool)
        kept.scatter_(1, torch.topk(best, keep, dim=-1).indices, True)
        c = c.masked_fill(~kept.repeat_interleave(per, dim=1), float("-inf"))
    chosen = torch.topk(c, top, dim=-1).indices
    return chosen, torch.gather(s, 1, chosen)


def moe_ff(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, mlp: dict) -> torch.Tensor:
    """Experts W_down relu(W_up h)^2; the outputs beyond the stored experts return h itself."""
    E = int(mlp["router"]["experts"])
    chosen, weights = route(h, W, p, mlp["router"])
    y = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, w in zip(chosen[t].tolist(), weights[t]):
            if e >= E:
                y[t] += w * h[t]
            else:
                y[t] += w * lin(torch.relu(lin(h[t:t + 1], W[f"{p}e{e}.up"])) ** 2, W[f"{p}e{e}.down"])[0]
    return y


# ------------------------------------------------------------------------------------------------- model
def forward(config: dict, W: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float64, layers_out: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence; ``layers_out`` (a list) receives the stream after every layer."""
    eps, alpha = float(config["norm"]["eps"]), float(config.get("postln_alpha", 1.0))
    x = W["embed"].to(dtype)[torch.tensor(tokens, dtype=torch.long)] * float((config.get("embedding") or {}).get("scale", 1.0))
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        if layer["type"] == "attention":
            y = attention_mixer(x, W, p + "mix.", layer["mixer"], eps)
        elif layer["type"] == "parallel":
            y = parallel_mixer(x, W, p + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        x = layer_norm(alpha * x + y, W[p + "norm1"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            y = dense_ff(x, W, p + "mlp.", mlp) if mlp["kind"] == "dense" else moe_ff(x, W, p + "mlp.", mlp)
            x = layer_norm(alpha * x + y, W[p + "norm2"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return lin(layer_norm(x, W["final.norm"], eps), W["head"])
