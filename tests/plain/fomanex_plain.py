"""Plain, slow Fomanex forward for whole sequences: no cache, no batching, no kernels.

One function per mechanism, written from the design's equations with torch on the CPU (float64 by default).  It
shares no code with ``ember_b200``: it takes the configuration as the dictionary config.json holds and the weights
as a name -> tensor dictionary.  Attention is a dense [T, T] score matrix under a causal mask with every head's keys
and values built from the latent; the recurrence is a loop over tokens from a zero state; the residual streams are a
[streams, T, width] tensor.

Notation: X [s, T, width] the residual streams, h a sublayer's input, W[name] a matrix stored [out, in].
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def lin(h: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    return h @ w.to(h.dtype).T


def rms_norm(x: torch.Tensor, w: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y * w.to(x.dtype) if w is not None else y


def dynamic_tanh(x: torch.Tensor, W: Dict[str, torch.Tensor], name: str) -> torch.Tensor:
    """tanh(alpha x) * w + b: an element-wise norm without statistics (scalar alpha, vectors w and b)."""
    dt = x.dtype
    return torch.tanh(W[name + ".alpha"].to(dt) * x) * W[name].to(dt) + W[name + ".b"].to(dt)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


# --------------------------------------------------------------------------------------------- rotation
def scaled_frequencies(rot: dict, dtype=torch.float64) -> (torch.Tensor, float):
    """The dims / 2 rotation frequencies f_i = base^(-2i / dims), stretched for long contexts where ``scaling`` is
    given: frequency i becomes f_i / factor * r_i + f_i (1 - r_i) with a ramp r over the pair index, and cos and sin
    are multiplied by 0.1 ln(factor) + 1.  Returns (frequencies, that multiplier)."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(dims // 2, dtype=dtype)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, original = float(sc["factor"]), float(sc["original"])

    def turn_dim(turns: float) -> float:            # the pair index whose wave turns ``turns`` times over the original length
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(turn_dim(float(sc["fast"]))), 0)
    hi = min(math.ceil(turn_dim(float(sc["slow"]))), dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_half(x: torch.Tensor, rot: dict, first_position: int = 0) -> torch.Tensor:
    """x [T, ..., n]: element i < dims / 2 pairs with element i + dims / 2; the pair (u, v) of the token at position p
    becomes (u c - v s, v c + u s) with c, s the (scaled) cosine and sine of p * frequency_i.  Elements from ``dims``
    on pass unchanged."""
    dims = int(rot["dims"])
    half = dims // 2
    T = x.shape[0]
    f, mult = scaled_frequencies(rot, x.dtype)
    pos = torch.arange(first_position, first_position + T, dtype=x.dtype)
    ang = pos[:, None] * f[None, :]
    shape = (T,) + (1,) * (x.dim() - 2) + (half,)
    c, s = (torch.cos(ang) * mult).view(shape), (torch.sin(ang) * mult).view(shape)
    u, v = x[..., :half], x[..., half:dims]
    out = x.clone()
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


# ----------------------------------------------------------------------------------------------- mixers
def latent_attention(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    """Causal attention whose keys and values are up-projections of a normed latent; the rotated key part is shared by
    the heads; a sink per head joins the softmax's denominator."""
    T = h.shape[0]
    H, D, R, V, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    q = lin(h, W[p + "q"]).view(T, H, D + R)
    q_plain, q_rot = q[..., :D], q[..., D:]
    dkv = lin(h, W[p + "dkv"])
    c = rms_norm(dkv[:, :r], W[p + "dkv.norm"], eps)
    k_rot = dkv[:, r:]                                                   # [T, R], one for all heads
    if R:
        q_rot = rotate_half(q_rot, m["rot"])
        k_rot = rotate_half(k_rot, m["rot"])
    k_plain = lin(c, W[p + "uk"]).view(T, H, D)
    v = lin(c, W[p + "uv"]).view(T, H, V)
    scores = (torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihd,jd->hij", q_rot, k_rot)) * m["scale"]
    causal = torch.arange(T)[None, :] <= torch.arange(T)[:, None]
    scores = scores.masked_fill(~causal[None], -math.inf)
    sink = W[p + "sink"].to(h.dtype)[:, None, None]
    top = torch.maximum(scores.max(-1, keepdim=True).values, sink)
    e = torch.exp(scores - top)
    w = e / (e.sum(-1, keepdim=True) + torch.exp(sink - top))
    o = torch.einsum("hij,jhd->ihd", w, v).reshape(T, H * V)
    return lin(o, W[p + "o"])


def wkv(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    """Time mixing with a matrix state per head: every projection reads its own blend of the token's input and the
    previous token's; the state decays per key channel by a data-dependent w; the current token reaches its own
    read-out only through the bonus u."""
    T = h.shape[0]
    H, D = m["heads"], m["dim"]
    dt = h.dtype
    before = torch.cat([torch.zeros_like(h[:1]), h[:-1]], dim=0)

    def blend(name):
        return h + (before - h) * W[p + "mu." + name].to(dt)

    r = lin(blend("r"), W[p + "r"]).view(T, H, D)
    k = lin(blend("k"), W[p + "k"]).view(T, H, D)
    v = lin(blend("v"), W[p + "v"]).view(T, H, D)
    gate = silu(lin(blend("g"), W[p + "g"]))
    decay = torch.exp(-torch.exp(lin(torch.tanh(lin(blend("w"), W[p + "w1"])), W[p + "w2"]) + W[p + "w0"].to(dt))).view(T, H, D)
    u = W[p + "u"].to(dt)                                                # [H, D]
    S = torch.zeros(H, D, D, dtype=dt)                                   # [head, key channel, value channel]
    out = torch.zeros(T, H, D, dtype=dt)
    for t in range(T):
        kv = k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hkv,hk->hv", S + u[:, :, None] * kv, r[t])
        S = decay[t][:, :, None] * S + kv
    out = out / torch.sqrt((out * out).mean(-1, keepdim=True) + eps)
    y = out.reshape(T, H * D) * W[p + "norm"].to(dt) * gate
    return lin(y, W[p + "o"])


# ------------------------------------------------------------------------------------------ feed-forwards
def dense_ff(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    return lin(gelu_tanh(lin(h, W[p + "gate"])) * lin(h, W[p + "up"]), W[p + "down"])


def routed_ff(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, mlp: dict) -> torch.Tensor:
    """Sigmoid scores; the choice adds a per-expert correction, the weights do not; weights are the chosen scores
    times a constant, not renormalised."""
    n, top, scale = mlp["router"]["experts"], mlp["router"]["top"], float(mlp["router"]["scale"])
    s = torch.sigmoid(lin(h, W[p + "router"]))
    pick = torch.topk(s + W[p + "correction"].to(h.dtype), top, dim=-1).indices          # [T, top]
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e in pick[t].tolist():
            q = f"{p}e{e}."
            y = lin(silu(lin(h[t], W[q + "gate"])) * lin(h[t], W[q + "up"]), W[q + "down"])
            out[t] += s[t, e] * scale * y
    return out


# ------------------------------------------------------------------------------------------------- model
def layer_order(cfg: dict) -> List[int]:
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def forward(cfg: dict, W: Dict[str, torch.Tensor], tokens, dtype=torch.float64, layers_out: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence from position 0.  ``layers_out`` (a list) receives the sum of the streams
    after every layer run."""
    W = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in W.items()}
    eps, mult = float(cfg["norm"]["eps"]), float(cfg.get("residual_mult", 1.0))
    streams = int(cfg.get("streams", 1))
    ids = torch.as_tensor(list(tokens), dtype=torch.long)
    x = dynamic_tanh(W["embed"][ids] * float((cfg.get("embedding") or {}).get("scale", 1.0)), W, "embed.norm")
    X = x[None].repeat(streams, 1, 1)
    for i in layer_order(cfg):
        L, p = cfg["layers"][i], f"l{i}."
        for q, kind in ((1, "mixer"), (2, "mlp")):
            if kind == "mlp" and L.get("mlp") is None:
                continue
            hc = f"{p}hc{q}."
            hyper = "streams" in cfg                 # without the key: one stream and the plain residual sum
            u = torch.einsum("s,std->td", W[hc + "in"], X) if hyper else X[0]
            hn = dynamic_tanh(u, W, f"{p}norm{q}")
            if kind == "mixer":
                y = {"latent_attention": latent_attention, "wkv": wkv}[L["type"]](hn, W, p + "mix.", L["mixer"], eps)
            elif L["mlp"]["kind"] == "dense":
                y = dense_ff(hn, W, p + "mlp.")
            else:
                y = routed_ff(hn, W, p + "mlp.", L["mlp"])
            y = y * W[f"{p}ls{q}"]
            if hyper:
                X = torch.einsum("sr,std->rtd", W[hc + "mix"], X) + mult * W[hc + "out"][:, None, None] * y[None]
            else:
                X = X + mult * y[None]
        if layers_out is not None:
            layers_out.append(X.sum(0))
    x = dynamic_tanh(X.sum(0), W, "final.norm")
    logits = lin(x, W["embed"]) * float(cfg.get("logit_scale", 1.0))
    cap = float(cfg.get("logit_softcap") or 0.0)
    return cap * torch.tanh(logits / cap) if cap > 0 else logits
