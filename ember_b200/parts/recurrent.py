"""Mixers whose memory is a fixed-size state per request (kept in the request's state slot, fp32):

* "channel_delta": delta-rule memory with a decay per head and key channel,
* "mlstm":         matrix memory with an exponential input gate and a running maximum,
* "mamba2":        selective state space with a scalar decay per head,
* "gla":           linear attention with a decay per head and key channel (no convolution, no delta correction),
* "wkv":           time mixing: blends with the previous token's input, a data-dependent decay per head and key channel,
                   a read-out of the state before its update plus a bonus for the current token.

All of them project their input with one fused product whose fp32 result the recurrence kernel reads in place (column
offsets, no copies), run the same kernels for prompt portions and single tokens (a block walks its run's tokens in
order, so the state after a step does not depend on how the tokens were cut), normalise each head's read-out in
fp32 and end in an output product that stores into, or adds into, an fp32 [T, hidden] buffer.  A short causal
convolution's last inputs are part of the state.
"""
from __future__ import annotations

from typing import List

import torch

from .. import ops
from ..config.spec import ConfigError
from .base import CacheNeed, Mixer, Runtime, WeightDecl
from .linear import Linear
from .registry import register_part


class _StateMixer(Mixer):
    graph_safe = True
    can_store = True

    def state_floats(self) -> int:
        raise NotImplementedError

    def cache_need(self) -> CacheNeed:
        return CacheNeed(kind="state", state_shape=(self.state_floats(),), state_dtype="float32")

    def _take_all(self, store):
        got = {d.name: store.take(d.name, d.shape) for d in self.weight_decls()}
        return None if any(v is None for v in got.values()) else got

    def _fused(self, tensors, rt: Runtime) -> Linear:
        """One matrix from several stored ones (rows concatenated), in the product's dtype."""
        wd = rt.weight_dtype(tensors[0].dtype)
        return Linear(torch.cat([rt.to_device(t, wd) for t in tensors], dim=0).contiguous())

    def _out(self, ctx, y, out, accumulate):
        self.o(ctx, y, out, ctx.T, ops.EPI_ADD_F32 if accumulate else ops.EPI_STORE_F32)


# --------------------------------------------------------------------------------------- channel_delta
class GatedDelta(_StateMixer):
    """Per value head h (query/key head h // (heads / kv_heads)), with unit vectors q (also times dim^-1/2) and k,
    beta = sigmoid(W_b x), and g = exp(-exp(A_log[h]) * softplus(W_a2 W_a1 x + dt_bias)) per key channel:

        S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q

    then o / rms(o) * norm * sigmoid(W_g2 W_g1 x) and the output product.  q, k, v each pass a short causal
    convolution and silu first.  Tensors under the prefix: q, k, v (+ ``.conv``), b, a1, a2, dt_bias, A_log, g1, g2,
    norm, o.

    ``decay`` "head": g = exp(-exp(A_log[h]) * softplus(W_a x + dt_bias[h])), one number per head (tensor ``a`` [heads,
    hidden] instead of a1 / a2, ``dt_bias`` [heads]).  ``gate`` "silu": o / rms(o) * norm * silu(W_g x) with a full-rank
    ``g`` [heads vdim, hidden] instead of g1 / g2."""

    def __init__(self, spec, prefix: str = ""):
        super().__init__(spec, prefix)
        s = spec
        if s.num_heads <= 0 or s.num_kv_heads <= 0 or s.num_heads % s.num_kv_heads:
            raise ConfigError(f"{s.num_heads} value heads do not divide into {s.num_kv_heads} query/key heads")
        if min(s.head_dim, s.value_dim, s.conv_taps) <= 0:
            raise ConfigError("channel_delta: head sizes and convolution taps must be positive")
        if s.decay not in ("channel", "head") or s.gate not in ("low_rank_sigmoid", "silu"):
            raise ConfigError(f"channel_delta: decay {s.decay!r} (channel, head), gate {s.gate!r} (low_rank_sigmoid, silu)")
        self.qk, self.vd = s.num_kv_heads * s.head_dim, s.num_heads * s.value_dim
        self.channels = 2 * self.qk + self.vd
        self.decay_rank, self.gate_rank = s.decay_rank, s.gate_rank
        self.per_head, self.full_gate = s.decay == "head", s.gate == "silu"
        self.decays = s.num_heads if self.per_head else s.num_heads * s.head_dim

    def state_floats(self) -> int:
        s = self.spec
        return s.num_heads * s.head_dim * s.value_dim + (s.conv_taps - 1) * self.channels

    def weight_decls(self) -> List[WeightDecl]:
        s, p = self.spec, self.prefix
        H, D, hid, ra, rg = s.num_heads, s.head_dim, s.hidden_size, self.decay_rank, self.gate_rank
        if (not self.per_head and ra <= 0) or (not self.full_gate and rg <= 0):
            raise ConfigError("channel_delta: the ranks of the decay and gate projections are read from the weights at "
                              "load; a configuration that lists tensors without a file must give them")
        d = [WeightDecl(p + "q", (self.qk, hid)), WeightDecl(p + "q.conv", (self.qk, s.conv_taps), init="uniform", lo=-0.5, hi=0.5),
             WeightDecl(p + "k", (self.qk, hid)), WeightDecl(p + "k.conv", (self.qk, s.conv_taps), init="uniform", lo=-0.5, hi=0.5),
             WeightDecl(p + "v", (self.vd, hid)), WeightDecl(p + "v.conv", (self.vd, s.conv_taps), init="uniform", lo=-0.5, hi=0.5),
             WeightDecl(p + "b", (H, hid)), WeightDecl(p + "A_log", (H,), init="uniform", lo=-1.0, hi=1.0),
             WeightDecl(p + "norm", (s.value_dim,), init="norm"),
             WeightDecl(p + "dt_bias", (self.decays,), init="uniform", lo=-3.0, hi=0.0), WeightDecl(p + "o", (hid, self.vd))]
        d += [WeightDecl(p + "a", (H, hid))] if self.per_head else [WeightDecl(p + "a1", (ra, hid)), WeightDecl(p + "a2", (H * D, ra))]
        d += [WeightDecl(p + "g", (self.vd, hid))] if self.full_gate else [WeightDecl(p + "g1", (rg, hid)), WeightDecl(p + "g2", (self.vd, rg))]
        return d

    def load(self, store, rt: Runtime) -> None:
        s, p = self.spec, self.prefix
        self.rt = rt
        for attr, name, unused in (("decay_rank", "a1", self.per_head), ("gate_rank", "g1", self.full_gate)):
            if getattr(self, attr) <= 0 and not unused:    # a size the configuration leaves to the weights
                shape = store.shape(p + name)
                setattr(self, attr, int(shape[0]) if shape and len(shape) == 2 else 1)
        w = self._take_all(store)
        if w is None:
            return
        ra, rg, HD = self.decay_rank, self.gate_rank, s.num_heads * s.head_dim
        # one product for everything that is a full-rank projection of the input: [q | k | v | beta (| decay) (| gate)]
        self.in_proj = self._fused([w[p + "q"], w[p + "k"], w[p + "v"], w[p + "b"]] + ([w[p + "a"]] if self.per_head else [])
                                   + ([w[p + "g"]] if self.full_gate else []), rt)
        lows = ([] if self.per_head else [("a1", "a2", HD, ra)]) + ([] if self.full_gate else [("g1", "g2", self.vd, rg)])
        self.low = self.up = None
        if lows:                                           # the low-rank pairs: [a1 | g1], then a block-diagonal [a2, g2]
            self.low = self._fused([w[p + first] for first, _, _, _ in lows], rt)
            wd = self.low.weight.dtype
            up = torch.zeros(sum(n for _, _, n, _ in lows), sum(r for _, _, _, r in lows), dtype=wd, device=rt.device)
            row = col = 0
            for _, second, n, r in lows:
                up[row:row + n, col:col + r] = rt.to_device(w[p + second], wd)
                row, col = row + n, col + r
            self.up = Linear(up)
        self.o = Linear.from_host(w[p + "o"], rt)
        self.taps = torch.cat([rt.to_device(w[p + n + ".conv"], torch.float32) for n in "qkv"], dim=0).contiguous()
        self.dt_bias, self.A_log, self.norm_w = (rt.to_device(w[p + n], torch.float32) for n in ("dt_bias", "A_log", "norm"))

    def forward(self, ctx, x, out, cache, owns_cache: bool = True, accumulate: bool = True) -> None:
        s, rt, T, mt = self.spec, self.rt, ctx.T, ctx.max_tokens
        H, D, V, C = s.num_heads, s.head_dim, s.value_dim, self.channels
        proj = ctx.buf("delta.proj", (mt, self.in_proj.n), torch.float32)
        conv = ctx.buf("delta.conv", (mt, C), torch.float32)
        o = ctx.buf("delta.read", (mt, self.vd), torch.float32)
        y = ctx.buf("delta.normed", (mt, self.vd), rt.dtype)
        self.in_proj(ctx, x, proj, T, ops.EPI_STORE_F32)
        ag = None
        if self.up is not None:
            low = ctx.buf("delta.low", (mt, self.low.n), rt.dtype)
            ag = ctx.buf("delta.decay_gate", (mt, self.up.n), torch.float32)
            self.low(ctx, x, low, T, ops.EPI_STORE)
            self.up(ctx, low, ag, T, ops.EPI_STORE_F32)
        # where the decay logits and the gate logits are: columns of the input product, or of the low-rank pairs' result
        a_src, a_col = (proj, C + H) if self.per_head else (ag, 0)
        g_src, g_col = (proj, C + H + (H if self.per_head else 0)) if self.full_gate else (ag, 0 if self.per_head else H * D)
        ops.conv_silu(proj, 0, self.taps, None, cache.state, H * D * V, ctx.seq_of, ctx.query_start, ctx.state_slots, conv,
                      T, ctx.S, stream=ctx.stream)
        ops.delta_scan(conv, proj, C, a_src, a_col, self.dt_bias, self.A_log, cache.state, o, ctx.query_start, ctx.state_slots,
                       T, ctx.S, H, s.num_kv_heads, D, V, s.key_eps, stream=ctx.stream, per_head_decay=self.per_head)
        ops.group_norm_gate(o, 0, g_src, g_col, self.norm_w, False, s.norm_eps,
                            ops.GATE_SILU_AFTER if self.full_gate else ops.GATE_SIGMOID_AFTER, y, T, H, V, stream=ctx.stream)
        self._out(ctx, y, out, accumulate)


# ----------------------------------------------------------------------------------------------- mlstm
class MatrixMemory(_StateMixer):
    """Per head, with q = W_q x * dim^-1/2, log gates i~ = cap tanh((W_i x + b_i) / cap) and
    f~ = logsigmoid(cap tanh((W_f x + b_f) / cap)) and a running maximum m that starts at 0:

        m' = max(f~ + m, i~);  S <- e^(f~ + m - m') S + e^(i~ - m') k v^T;  n likewise with k alone
        o = S^T q / (max(|n . q|, e^(-m')) + 1e-6)

    then o / rms(o) per head, times norm (all heads' size), times sigmoid(W_g x), and the output product.
    Tensors under the prefix: q, k, v, g, o, norm, i, i.b, f, f.b."""

    def __init__(self, spec, prefix: str = ""):
        super().__init__(spec, prefix)
        s = spec
        if min(s.num_heads, s.head_dim, s.value_dim) <= 0 or not s.gate_cap > 0:
            raise ConfigError("mlstm: head count, sizes and the gate cap must be positive")
        self.qk, self.vd = s.num_heads * s.head_dim, s.num_heads * s.value_dim

    def state_floats(self) -> int:
        s = self.spec
        return s.num_heads * (s.head_dim * s.value_dim + s.head_dim + 1)

    def weight_decls(self) -> List[WeightDecl]:
        s, p = self.spec, self.prefix
        H, hid = s.num_heads, s.hidden_size
        return [WeightDecl(p + "q", (self.qk, hid)), WeightDecl(p + "k", (self.qk, hid)), WeightDecl(p + "v", (self.vd, hid)),
                WeightDecl(p + "g", (self.vd, hid)), WeightDecl(p + "o", (hid, self.vd)),
                WeightDecl(p + "norm", (self.vd,), init="norm"),
                WeightDecl(p + "i", (H, hid)), WeightDecl(p + "i.b", (H,), init="uniform", lo=-1.0, hi=1.0),
                WeightDecl(p + "f", (H, hid)), WeightDecl(p + "f.b", (H,), init="uniform", lo=1.0, hi=4.0)]

    def load(self, store, rt: Runtime) -> None:
        p = self.prefix
        self.rt = rt
        w = self._take_all(store)
        if w is None:
            return
        self.in_proj = self._fused([w[p + n] for n in ("q", "k", "v", "g", "i", "f")], rt)
        self.o = Linear.from_host(w[p + "o"], rt)
        self.bias_i, self.bias_f, self.norm_w = (rt.to_device(w[p + n], torch.float32) for n in ("i.b", "f.b", "norm"))

    def forward(self, ctx, x, out, cache, owns_cache: bool = True, accumulate: bool = True) -> None:
        s, rt, T, mt = self.spec, self.rt, ctx.T, ctx.max_tokens
        H, D, V = s.num_heads, s.head_dim, s.value_dim
        off_k, off_v, off_g = self.qk, 2 * self.qk, 2 * self.qk + self.vd
        off_i = off_g + self.vd
        proj = ctx.buf("mlstm.proj", (mt, off_i + 2 * H), torch.float32)
        gates = ctx.buf("mlstm.gates", (mt, H, 4), torch.float32)
        o = ctx.buf("mlstm.read", (mt, self.vd), torch.float32)
        y = ctx.buf("mlstm.normed", (mt, self.vd), rt.dtype)
        self.in_proj(ctx, x, proj, T, ops.EPI_STORE_F32)
        ops.memory_scan(proj, 0, off_k, off_v, off_i, off_i + H, self.bias_i, self.bias_f, s.gate_cap, cache.state, gates, o,
                        ctx.query_start, ctx.state_slots, T, ctx.S, H, D, V, stream=ctx.stream)
        ops.group_norm_gate(o, 0, proj, off_g, self.norm_w, True, s.norm_eps, ops.GATE_SIGMOID_AFTER, y, T, H, V, den=gates,
                            stream=ctx.stream)
        self._out(ctx, y, out, accumulate)


# ---------------------------------------------------------------------------------------------- mamba2
class StateSpace(_StateMixer):
    """W_in x = [z | x | B | C | dt]; x, B, C pass a short causal convolution (with bias) and silu;
    dt = softplus(dt + dt_bias); per head h (B, C of group h // (heads / groups)):

        S <- exp(-exp(A_log[h]) dt) S + dt B x^T  (S is state x vdim);  y = S^T C + D[h] x

    then y * silu(z), an RMS norm in ``norm_groups`` equal parts times norm, and the output product.
    Tensors under the prefix: in, conv, conv.b, dt_bias, A_log, D, norm, o."""

    def __init__(self, spec, prefix: str = ""):
        super().__init__(spec, prefix)
        s = spec
        if min(s.num_heads, s.value_dim, s.state_size, s.num_groups, s.norm_groups, s.conv_taps) <= 0:
            raise ConfigError("mamba2: sizes must be positive")
        if s.num_heads % s.num_groups or s.inner % s.norm_groups:
            raise ConfigError(f"mamba2: {s.num_heads} heads in {s.num_groups} groups, {s.inner} channels in {s.norm_groups} norm groups")
        self.channels = s.inner + 2 * s.num_groups * s.state_size

    def state_floats(self) -> int:
        s = self.spec
        return s.num_heads * s.state_size * s.value_dim + (s.conv_taps - 1) * self.channels

    def weight_decls(self) -> List[WeightDecl]:
        s, p = self.spec, self.prefix
        H, hid = s.num_heads, s.hidden_size
        return [WeightDecl(p + "in", (s.inner + self.channels + H, hid)),
                WeightDecl(p + "conv", (self.channels, s.conv_taps), init="uniform", lo=-0.5, hi=0.5),
                WeightDecl(p + "conv.b", (self.channels,), init="zeros"),
                WeightDecl(p + "dt_bias", (H,), init="uniform", lo=-3.0, hi=-1.0),
                WeightDecl(p + "A_log", (H,), init="uniform", lo=0.0, hi=2.0), WeightDecl(p + "D", (H,), init="norm"),
                WeightDecl(p + "norm", (s.inner,), init="norm"), WeightDecl(p + "o", (hid, s.inner))]

    def load(self, store, rt: Runtime) -> None:
        p = self.prefix
        self.rt = rt
        w = self._take_all(store)
        if w is None:
            return
        self.in_proj = Linear.from_host(w[p + "in"], rt)
        self.o = Linear.from_host(w[p + "o"], rt)
        self.taps, self.conv_bias, self.dt_bias, self.A_log, self.skip, self.norm_w = (
            rt.to_device(w[p + n], torch.float32) for n in ("conv", "conv.b", "dt_bias", "A_log", "D", "norm"))

    def forward(self, ctx, x, out, cache, owns_cache: bool = True, accumulate: bool = True) -> None:
        s, rt, T, mt = self.spec, self.rt, ctx.T, ctx.max_tokens
        H, V, N, inner, C = s.num_heads, s.value_dim, s.state_size, s.inner, self.channels
        proj = ctx.buf("mamba2.proj", (mt, inner + C + H), torch.float32)
        conv = ctx.buf("mamba2.conv", (mt, C), torch.float32)
        o = ctx.buf("mamba2.read", (mt, inner), torch.float32)
        y = ctx.buf("mamba2.normed", (mt, inner), rt.dtype)
        self.in_proj(ctx, x, proj, T, ops.EPI_STORE_F32)
        ops.conv_silu(proj, inner, self.taps, self.conv_bias, cache.state, H * N * V, ctx.seq_of, ctx.query_start,
                      ctx.state_slots, conv, T, ctx.S, stream=ctx.stream)
        ops.ssm_scan(conv, proj, inner + C, self.dt_bias, self.A_log, self.skip, cache.state, o, ctx.query_start,
                     ctx.state_slots, T, ctx.S, H, s.num_groups, N, V, stream=ctx.stream)
        ops.group_norm_gate(o, 0, proj, 0, self.norm_w, True, s.norm_eps, ops.GATE_SILU_BEFORE, y, T, s.norm_groups,
                            inner // s.norm_groups, stream=ctx.stream)
        self._out(ctx, y, out, accumulate)


# ------------------------------------------------------------------------------------------------- gla
class GatedLinearAttention(_StateMixer):
    """Per head, with q = W_q x * dim^-1/2, k = W_k x, v = W_v x and one decay per key channel
    alpha = sigmoid(W_a2 (W_a1 x) + b)^(1 / tau) (computed as exp(logsigmoid(.) / tau) in fp32):

        S <- diag(alpha) S + k v^T;  o = S^T q

    then o / rms(o) per head times norm (size vdim, shared by the heads), times silu(W_g x), and the output product.
    The state starts at zero and is carried in the request's slot.  Tensors under the prefix: q, k, v, g, o, norm, a1,
    a2, a2.b."""

    def __init__(self, spec, prefix: str = ""):
        super().__init__(spec, prefix)
        s = spec
        if min(s.num_heads, s.head_dim, s.value_dim) <= 0 or not s.tau > 0:
            raise ConfigError("gla: head count, sizes and tau must be positive")
        self.qk, self.vd = s.num_heads * s.head_dim, s.num_heads * s.value_dim
        self.decay_rank = s.decay_rank

    def state_floats(self) -> int:
        s = self.spec
        return s.num_heads * s.head_dim * s.value_dim

    def weight_decls(self) -> List[WeightDecl]:
        s, p = self.spec, self.prefix
        hid, ra = s.hidden_size, self.decay_rank
        if ra <= 0:
            raise ConfigError("gla: the rank of the decay projection is read from the weights at load; a configuration "
                              "that lists tensors without a file must give it")
        return [WeightDecl(p + "q", (self.qk, hid)), WeightDecl(p + "k", (self.qk, hid)), WeightDecl(p + "v", (self.vd, hid)),
                WeightDecl(p + "g", (self.vd, hid)), WeightDecl(p + "o", (hid, self.vd)),
                WeightDecl(p + "norm", (s.value_dim,), init="norm"),
                WeightDecl(p + "a1", (ra, hid)), WeightDecl(p + "a2", (self.qk, ra)),
                WeightDecl(p + "a2.b", (self.qk,), init="uniform", lo=0.0, hi=4.0)]

    def load(self, store, rt: Runtime) -> None:
        p = self.prefix
        self.rt = rt
        if self.decay_rank <= 0:                       # a size the configuration leaves to the weights
            shape = store.shape(p + "a1")
            self.decay_rank = int(shape[0]) if shape and len(shape) == 2 else 1
        w = self._take_all(store)
        if w is None:
            return
        self.in_proj = self._fused([w[p + n] for n in ("q", "k", "v", "g")], rt)
        self.low = Linear.from_host(w[p + "a1"], rt)
        self.up = Linear.from_host(w[p + "a2"], rt)
        self.o = Linear.from_host(w[p + "o"], rt)
        self.decay_bias, self.norm_w = (rt.to_device(w[p + n], torch.float32) for n in ("a2.b", "norm"))

    def forward(self, ctx, x, out, cache, owns_cache: bool = True, accumulate: bool = True) -> None:
        s, rt, T, mt = self.spec, self.rt, ctx.T, ctx.max_tokens
        H, D, V = s.num_heads, s.head_dim, s.value_dim
        off_k, off_v, off_g = self.qk, 2 * self.qk, 2 * self.qk + self.vd
        proj = ctx.buf("gla.proj", (mt, off_g + self.vd), torch.float32)
        low = ctx.buf("gla.low", (mt, self.decay_rank), rt.dtype)
        z = ctx.buf("gla.decay", (mt, self.qk), torch.float32)
        o = ctx.buf("gla.read", (mt, self.vd), torch.float32)
        y = ctx.buf("gla.normed", (mt, self.vd), rt.dtype)
        self.in_proj(ctx, x, proj, T, ops.EPI_STORE_F32)
        self.low(ctx, x, low, T, ops.EPI_STORE)
        self.up(ctx, low, z, T, ops.EPI_STORE_F32)
        ops.gla_scan(proj, 0, off_k, off_v, z, 0, self.decay_bias, 1.0 / s.tau, cache.state, o, ctx.query_start, ctx.state_slots,
                     T, ctx.S, H, D, V, stream=ctx.stream)
        ops.group_norm_gate(o, 0, proj, off_g, self.norm_w, False, s.norm_eps, ops.GATE_SILU_AFTER, y, T, H, V, stream=ctx.stream)
        self._out(ctx, y, out, accumulate)


# ------------------------------------------------------------------------------------------------- wkv
class TimeMix(_StateMixer):
    """With x' the previous token's input (zeros before a request's first token), each of r, k, v, g, w reads its own
    blend x + (x' - x) mu: r, k, v = W_r, W_k, W_v of theirs (heads x dim), gate = silu(W_g .), and the decay
    w = exp(-exp(W_w2 tanh(W_w1 .) + w0)) per head and key channel.  Per head, with the bonus u:

        o = (S + diag(u) k v^T)^T r;   S <- diag(w) S + k v^T

    then o / rms(o) per head, times norm (all heads' size), times the gate, and the output product.  The state row of a
    request holds S [heads, dim, dim] and, behind it, the last input x' [hidden]; both start at zero.  Blends are made
    in fp32 from the input and rounded to the products' dtype; the decay's logits, both exponentials, the bonus and the
    state are fp32.  Tensors under the prefix: mu.r, mu.k, mu.v, mu.g, mu.w, r, k, v, g, w1, w2, w0, u, norm, o."""

    BLENDS = ("r", "k", "v", "g", "w")

    def __init__(self, spec, prefix: str = ""):
        super().__init__(spec, prefix)
        s = spec
        if min(s.hidden_size, s.num_heads, s.head_dim) <= 0:
            raise ConfigError("wkv: width, head count and head size must be positive")
        self.inner = s.num_heads * s.head_dim
        self.decay_rank = s.decay_rank

    def state_floats(self) -> int:
        s = self.spec
        return s.num_heads * s.head_dim * s.head_dim + s.hidden_size

    def weight_decls(self) -> List[WeightDecl]:
        s, p = self.spec, self.prefix
        hid, n, ra = s.hidden_size, self.inner, self.decay_rank
        if ra <= 0:
            raise ConfigError("wkv: the rank of the decay projection is read from the weights at load; a configuration "
                              "that lists tensors without a file must give it")
        d = [WeightDecl(p + "mu." + b, (hid,), init="uniform", lo=0.0, hi=1.0) for b in self.BLENDS]
        d += [WeightDecl(p + n_, (n, hid)) for n_ in ("r", "k", "v", "g")]
        d += [WeightDecl(p + "w1", (ra, hid)), WeightDecl(p + "w2", (n, ra)),
              WeightDecl(p + "w0", (n,), init="uniform", lo=-3.0, hi=0.5),
              WeightDecl(p + "u", (s.num_heads, s.head_dim), init="uniform", lo=-0.5, hi=1.0),
              WeightDecl(p + "norm", (n,), init="norm"), WeightDecl(p + "o", (hid, n))]
        return d

    def load(self, store, rt: Runtime) -> None:
        p = self.prefix
        self.rt = rt
        if self.decay_rank <= 0:                       # a size the configuration leaves to the weights
            shape = store.shape(p + "w1")
            self.decay_rank = int(shape[0]) if shape and len(shape) == 2 else 1
        w = self._take_all(store)
        if w is None:
            return
        f32 = lambda name: rt.to_device(w[p + name], torch.float32)          # noqa: E731
        self.mu = torch.stack([f32("mu." + b) for b in self.BLENDS]).contiguous()           # [5, hidden]
        self.proj = [Linear.from_host(w[p + n], rt) for n in ("r", "k", "v", "g")]
        self.w1, self.w2, self.o = (Linear.from_host(w[p + n], rt) for n in ("w1", "w2", "o"))
        self.w0, self.bonus, self.norm_w = f32("w0"), f32("u").reshape(-1).contiguous(), f32("norm")
        self.one = torch.ones(1, dtype=torch.float32, device=rt.device)
        self.ones = torch.ones(self.decay_rank, dtype=torch.float32, device=rt.device)

    def forward(self, ctx, x, out, cache, owns_cache: bool = True, accumulate: bool = True) -> None:
        s, rt, T, mt = self.spec, self.rt, ctx.T, ctx.max_tokens
        H, D, n, hid = s.num_heads, s.head_dim, self.inner, s.hidden_size
        blends = ctx.buf("wkv.blends", (len(self.BLENDS), mt, hid), rt.dtype)
        rkvg = ctx.buf("wkv.rkvg", (4, mt, n), torch.float32)
        low = ctx.buf("wkv.low", (mt, self.decay_rank), torch.float32)
        low_t = ctx.buf("wkv.low_tanh", (mt, self.decay_rank), rt.dtype)
        z = ctx.buf("wkv.decay", (mt, n), torch.float32)
        o = ctx.buf("wkv.read", (mt, n), torch.float32)
        y = ctx.buf("wkv.normed", (mt, n), rt.dtype)
        # the previous token's input is the last ``hidden`` floats of the request's state row
        ops.token_shift(x, self.mu, cache.state, H * D * D, ctx.seq_of, ctx.query_start, ctx.state_slots, blends, T, ctx.S,
                        stream=ctx.stream)
        for i, lin in enumerate(self.proj):
            lin(ctx, blends[i], rkvg[i], T, ops.EPI_STORE_F32)
        self.w1(ctx, blends[4], low, T, ops.EPI_STORE_F32)
        ops.dynamic_tanh(low, self.one, self.ones, None, low_t, T, stream=ctx.stream)       # tanh alone
        self.w2(ctx, low_t, z, T, ops.EPI_STORE_F32)
        ops.wkv_scan(rkvg, n, 0, mt * n, 2 * mt * n, z, 0, self.w0, self.bonus, cache.state, o, ctx.query_start, ctx.state_slots,
                     T, ctx.S, H, D, D, stream=ctx.stream)
        ops.group_norm_gate(o, 0, rkvg[3], 0, self.norm_w, True, s.norm_eps, ops.GATE_SILU_AFTER, y, T, H, D, stream=ctx.stream)
        self._out(ctx, y, out, accumulate)


register_part("mixer", "wkv", TimeMix)
register_part("mixer", "gla", GatedLinearAttention)
register_part("mixer", "channel_delta", GatedDelta)
register_part("mixer", "mlstm", MatrixMemory)
register_part("mixer", "mamba2", StateSpace)
