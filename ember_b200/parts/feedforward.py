"""Gated feed-forward: h += down( act(gate(x)) * up(x) ), no biases; act = silu (SwiGLU), relu or gelu (tanh form).
With ``activation`` "clamped_swish": g = min(gate(x), limit), u = clamp(up(x), -limit, limit), down(g sigmoid(alpha g) (u +
up_offset)); with ``bias`` all three projections have biases.

Formula: src/backend/cpu/cpu_backend.cpp:204-211 with silu(g) = g / (1 + exp(-g)).
Device layout: gate and up rows are interleaved (even rows gate, odd rows up) into one
[2 * intermediate, hidden] matrix, so one product yields adjacent (gate, up) pairs and the
activation is the product's epilogue.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .. import ops
from ..config.spec import ConfigError
from .base import FeedForward, Runtime, WeightDecl
from .linear import Linear
from .registry import register_part


class GatedMLP(FeedForward):
    graph_safe = True
    can_store = True

    def __init__(self, spec, prefix: str = ""):
        super().__init__(spec, prefix)
        if spec.activation not in ops.ACTIVATIONS + ("clamped_swish",):
            raise ConfigError(f"activation {spec.activation!r} is not supported ({', '.join(ops.ACTIVATIONS)}, clamped_swish)")
        self.clamped = spec.activation == "clamped_swish"
        if self.clamped and spec.limit < 0:
            raise ConfigError("gated feed-forward: the clamp limit must be positive (or 0 for none)")
        if spec.bias and not self.clamped:
            raise ConfigError("gated feed-forward: biases come with the clamped activation (a kernel of its own behind the product)")
        # the last product's bias, left for whoever adds the result to the stream (``forward(..., fold_bias=True)``)
        self.result_bias = None

    def weight_decls(self) -> List[WeightDecl]:
        s, p = self.spec, self.prefix
        g, u, d = s.names
        decls = [WeightDecl(p + g, (s.intermediate_size, s.hidden_size)),
                 WeightDecl(p + u, (s.intermediate_size, s.hidden_size)),
                 WeightDecl(p + d, (s.hidden_size, s.intermediate_size))]
        if s.bias:
            decls += [WeightDecl(p + g + s.bias_suffix, (s.intermediate_size,), init="zeros"),
                      WeightDecl(p + u + s.bias_suffix, (s.intermediate_size,), init="zeros"),
                      WeightDecl(p + d + s.bias_suffix, (s.hidden_size,), init="zeros")]
        return decls

    def load(self, store, rt: Runtime) -> None:
        s, p = self.spec, self.prefix
        self.rt = rt
        gate = store.take(p + s.names[0], (s.intermediate_size, s.hidden_size))
        up = store.take(p + s.names[1], (s.intermediate_size, s.hidden_size))
        down = store.take(p + s.names[2], (s.hidden_size, s.intermediate_size))
        biases = [store.take(p + n + s.bias_suffix, (size,)) for n, size in
                  zip(s.names, (s.intermediate_size, s.intermediate_size, s.hidden_size))] if s.bias else []
        if gate is None or up is None or down is None or any(b is None for b in biases):
            return
        self.gate_up_bias = None
        if s.bias:                                         # (gate, up) biases interleaved like the rows
            self.gate_up_bias = torch.stack([rt.to_device(biases[0], torch.float32), rt.to_device(biases[1], torch.float32)], dim=1).reshape(-1).contiguous()
            self.result_bias = rt.to_device(biases[2], torch.float32)
        wd = rt.weight_dtype(torch.result_type(gate, up))
        gu = torch.stack([rt.to_device(gate, wd), rt.to_device(up, wd)], dim=1)   # [I, 2, H]
        self.gate_up = Linear(gu.reshape(2 * s.intermediate_size, s.hidden_size).contiguous())
        self.down = Linear.from_host(down, rt)

    def forward(self, ctx, x: torch.Tensor, residual: torch.Tensor, accumulate: bool = True, fold_bias: bool = False) -> None:
        """``fold_bias``: the caller adds ``result_bias`` (the down projection's) itself, in the kernel that joins the
        result to the stream; otherwise it is added here."""
        s = self.spec
        act = ctx.buf("gated_mlp.act", (ctx.max_tokens, s.intermediate_size), self.rt.dtype)
        if self.clamped:
            gu = ctx.buf("gated_mlp.gate_up", (ctx.max_tokens, 2 * s.intermediate_size), torch.float32)
            self.gate_up(ctx, x, gu, ctx.T, ops.EPI_STORE_F32)
            ops.moe_activation(gu, act, ctx.T, float(s.limit) if s.limit > 0 else float("inf"), s.alpha, stream=ctx.stream,
                               up_offset=s.up_offset, bias=self.gate_up_bias)
        else:
            self.gate_up(ctx, x, act, ctx.T, ops.GATED_EPILOGUE_OF[s.activation])
        if self.result_bias is not None and not fold_bias:
            if accumulate:
                raise ops.KernelError("gated feed-forward: a biased result is stored, or its bias is folded by the caller")
            self.down(ctx, act, residual, ctx.T, ops.EPI_STORE_F32)
            ops.add_row_bias(residual, self.result_bias, ctx.T, stream=ctx.stream)
            return
        self.down(ctx, act, residual, ctx.T, ops.EPI_ADD_F32 if accumulate else ops.EPI_STORE_F32)


class RoutedMLP(FeedForward):
    """Mixture of experts: h += sum over the token's ``top`` experts of weight * W_down (g sigmoid(alpha g) (u + up_offset))
    with g = min(W_gate x, limit), u = clamp(W_up x, -limit, limit) (``limit`` 0: no clamps; alpha 1 and up_offset 0 then
    give silu(W_gate x) * W_up x).  The router's logits W_router x are fp32 (fp32 weights and accumulation).  Scoring
    "softmax_top": the chosen experts are the ``top`` largest logits (ties: the lower index) and their weights the
    softmax over the chosen logits alone.  Scoring "sigmoid": scores s = sigmoid(logits), the choice is by
    s + correction (a stored vector, if ``correction``), the weights are the chosen experts' s times ``route_scale``
    (divided by their sum first if ``renormalize``).

    Device layout: every expert's gate and up rows interleaved into one [experts, 2 ff, hidden] tensor (the activation
    is the first product's epilogue) and the down matrices as [experts, hidden, ff].  The step's (token, choice) pairs
    are ordered by expert on the device; both products walk row tiles of one expert each, so every expert's weights
    are read once per step however the tokens fall, and nothing comes back to the host (decode steps are captured
    into CUDA graphs like any other).

    A bfloat16 step of more tokens than any captured step has (a prompt portion) takes the tensor cores instead: the
    tokens' rows are gathered expert by expert, the host reads the experts' row counts (the step's one look at the
    device) and every expert with rows runs the tcgen05 product on its slice, first gate/up into fp32, an element-wise
    kernel for the clamped activation, then down; the weighted sum over a token's choices is the same kernel either way.
    Tensors under the prefix: router, correction (if any), e<i>.gate, e<i>.up, e<i>.down.

    Scoring "softmax": s = softmax over all router outputs, otherwise as "sigmoid".  ``groups``: the outputs form equal
    groups of neighbours, a group's score is its largest s + correction, and the choice is among the outputs of the
    ``keep_groups`` best groups.  ``identity``: the router has experts + identity outputs, the last ones experts without
    tensors whose output is the token's input itself (``forward(..., stream=)`` hands the fp32 input where the caller has
    it; else the product's input is used).  ``expert`` "square_relu": W_down relu(W_up h)^2, no gate matrix."""

    graph_safe = True
    can_store = True
    TC_MIN_TOKENS = 257          # more runs than a captured decode step can have: such a step is never inside a graph
    STREAM_MAX_TOKENS = 256      # up to here the products stream the weights past the few rows of a tile

    def __init__(self, spec, prefix: str = ""):
        super().__init__(spec, prefix)
        s = spec
        if min(s.hidden_size, s.intermediate_size, s.experts, s.top) <= 0 or s.top > s.experts + max(s.identity, 0):
            raise ConfigError(f"routed feed-forward: top {s.top} of {s.experts} experts of {s.intermediate_size}")
        if s.experts > ops.MOE_MAX_EXPERTS or s.top > ops.MOE_MAX_TOP:
            raise ConfigError(f"routed feed-forward: at most {ops.MOE_MAX_TOP} of {ops.MOE_MAX_EXPERTS} experts")
        if s.limit < 0:
            raise ConfigError("routed feed-forward: the clamp limit must be positive (or 0 for none)")
        if s.scoring not in ("softmax_top", "sigmoid", "softmax"):
            raise ConfigError(f"routed feed-forward: scoring {s.scoring!r} (softmax_top, sigmoid, softmax)")
        if s.scoring == "softmax_top" and (s.correction or s.renormalize or s.route_scale != 1.0 or s.groups):
            raise ConfigError("routed feed-forward: a correction, a scale, groups and renormalising belong to sigmoid or softmax scoring")
        if s.identity < 0 or s.expert not in ("gated", "square_relu"):
            raise ConfigError(f"routed feed-forward: {s.identity} identity experts, expert {s.expert!r} (gated, square_relu)")
        self.outputs = s.experts + s.identity              # what the router chooses among
        if self.outputs > ops.MOE_MAX_EXPERTS or s.top > self.outputs:
            raise ConfigError(f"routed feed-forward: top {s.top} of {self.outputs} router outputs (at most {ops.MOE_MAX_EXPERTS})")
        if s.groups and (s.groups > 32 or self.outputs % s.groups or not 1 <= s.keep_groups <= s.groups
                         or s.top > s.keep_groups * (self.outputs // s.groups)):
            raise ConfigError(f"routed feed-forward: {self.outputs} router outputs in {s.groups} groups (at most 32, equal) of "
                              f"which {s.keep_groups} are kept for top {s.top}")
        self.gated = s.expert == "gated"
        self.limit = float(s.limit) if s.limit > 0 else float("inf")

    def weight_decls(self) -> List[WeightDecl]:
        s, p = self.spec, self.prefix
        d = [WeightDecl(p + "router", (self.outputs, s.hidden_size))]
        if s.correction:
            d.append(WeightDecl(p + "correction", (self.outputs,), init="uniform", lo=-0.2, hi=0.2))
        for e in range(s.experts):
            if self.gated:
                d.append(WeightDecl(f"{p}e{e}.gate", (s.intermediate_size, s.hidden_size)))
            d += [WeightDecl(f"{p}e{e}.up", (s.intermediate_size, s.hidden_size)),
                  WeightDecl(f"{p}e{e}.down", (s.hidden_size, s.intermediate_size))]
        return d

    def load(self, store, rt: Runtime) -> None:
        s, p = self.spec, self.prefix
        self.rt = rt
        got = {d.name: store.take(d.name, d.shape) for d in self.weight_decls()}
        if any(v is None for v in got.values()):
            return
        wd = rt.weight_dtype(got[f"{p}e0.up"].dtype)
        if wd != rt.dtype:
            wd = torch.float32 if rt.dtype == torch.float32 else torch.bfloat16
        self.router = rt.to_device(got[p + "router"], torch.float32)
        self.rule = None
        if s.scoring != "softmax_top":
            self.rule = (rt.to_device(got[p + "correction"], torch.float32) if s.correction else None, float(s.route_scale),
                         bool(s.renormalize), s.scoring, int(s.groups), int(s.keep_groups))
        down = torch.empty((s.experts, s.hidden_size, s.intermediate_size), dtype=wd, device=rt.device)
        if self.gated:
            gu = torch.empty((s.experts, s.intermediate_size, 2, s.hidden_size), dtype=wd, device=rt.device)
            for e in range(s.experts):
                gu[e, :, 0] = rt.to_device(got[f"{p}e{e}.gate"], wd)
                gu[e, :, 1] = rt.to_device(got[f"{p}e{e}.up"], wd)
            self.gate_up = gu.view(s.experts, 2 * s.intermediate_size, s.hidden_size)
        else:
            self.gate_up = torch.empty((s.experts, s.intermediate_size, s.hidden_size), dtype=wd, device=rt.device)
            for e in range(s.experts):
                self.gate_up[e] = rt.to_device(got[f"{p}e{e}.up"], wd)
        for e in range(s.experts):
            down[e] = rt.to_device(got[f"{p}e{e}.down"], wd)
        self.down = down
        if wd == torch.bfloat16:
            ops.reserve_scratch(rt.device, 128 * max(self.gate_up.shape[1], s.hidden_size))    # (the small-M product's)

    def _on_tensor_cores(self, ctx, x) -> bool:
        s = self.spec
        return (ops.TC_ENABLED and x.dtype == torch.bfloat16 and ctx.T >= self.TC_MIN_TOKENS and s.hidden_size % 8 == 0
                and s.intermediate_size % 8 == 0)

    def forward(self, ctx, x: torch.Tensor, residual: torch.Tensor, accumulate: bool = True, stream: Optional[torch.Tensor] = None) -> None:
        s, rt, T, mt = self.spec, self.rt, ctx.T, ctx.max_tokens
        E, top, pairs = self.outputs, s.top, ctx.T * s.top      # (identity experts take slots like the others, and no tiles)
        if x.dtype != self.gate_up.dtype:
            raise ops.KernelError(f"routed feed-forward: input {x.dtype} against experts {self.gate_up.dtype}")
        sel = ctx.buf("routed_mlp.sel", (mt * top,), torch.int32)
        wgt = ctx.buf("routed_mlp.weights", (mt * top,), torch.float32)
        offsets = ctx.buf("routed_mlp.offsets", (E + 1,), torch.int32)
        pair_of_slot = ctx.buf("routed_mlp.pair_of_slot", (mt * top,), torch.int32)
        slot_of_pair = ctx.buf("routed_mlp.slot_of_pair", (mt * top,), torch.int32)
        tiles = ctx.buf("routed_mlp.tiles", (1 + 2 * ops.moe_max_tiles(mt * top, E, ops.MOE_STREAM_ROWS),), torch.int32)
        act = ctx.buf("routed_mlp.act", (mt * top, s.intermediate_size), rt.dtype)
        y = ctx.buf("routed_mlp.down", (mt * top, s.hidden_size), torch.float32)
        ops.moe_router(x, self.router, T, top, sel, wgt, stream=ctx.stream, rule=self.rule)
        streaming = (T <= self.STREAM_MAX_TOKENS and ops.moe_stream_usable(x, s.hidden_size)
                     and ops.moe_stream_usable(x, s.intermediate_size))
        max_tiles = ops.moe_group(sel, pairs, E, offsets, pair_of_slot, slot_of_pair, tiles,
                                  ops.MOE_STREAM_ROWS if streaming else ops.MOE_TILE_ROWS, stream=ctx.stream, tiled=s.experts)
        if self._on_tensor_cores(ctx, x):
            xs = ctx.buf("routed_mlp.gathered", (mt * top, s.hidden_size), rt.dtype)
            gu = ctx.buf("routed_mlp.gate_up", (mt * top, self.gate_up.shape[1]), torch.float32)
            ops.moe_gather(x, pair_of_slot, pairs, top, xs, stream=ctx.stream)
            bounds = offsets.tolist()                      # the experts' row ranges: the host waits for the grouping here
            for e in range(s.experts):
                lo, n = bounds[e], bounds[e + 1] - bounds[e]
                if n > 0:
                    ops.gemm_tc(xs[lo:lo + n], self.gate_up[e], gu[lo:lo + n], n, ops.EPI_STORE_F32, err=ctx.err, stream=ctx.stream)
            if self.gated:
                ops.moe_activation(gu, act, pairs, self.limit, s.alpha, stream=ctx.stream, up_offset=s.up_offset)
            else:
                ops.moe_square_relu(gu, act, pairs * s.intermediate_size, stream=ctx.stream)
            for e in range(s.experts):
                lo, n = bounds[e], bounds[e + 1] - bounds[e]
                if n > 0:
                    ops.gemm_tc(act[lo:lo + n], self.down[e], y[lo:lo + n], n, ops.EPI_STORE_F32, err=ctx.err, stream=ctx.stream)
        else:
            ops.moe_gemm(x, self.gate_up, act, offsets, pair_of_slot, tiles, max_tiles, top, self.gated, self.limit, s.alpha,
                         stream=ctx.stream, streaming=streaming, up_offset=s.up_offset, square_relu=not self.gated)
            ops.moe_gemm(act, self.down, y, offsets, pair_of_slot, tiles, max_tiles, 0, False, stream=ctx.stream, streaming=streaming)
        if s.identity:
            ops.moe_combine(y, wgt, slot_of_pair, T, top, residual, accumulate=accumulate, stream=ctx.stream, sel=sel,
                            experts=s.experts, same=stream if stream is not None else x)
        else:
            ops.moe_combine(y, wgt, slot_of_pair, T, top, residual, accumulate=accumulate, stream=ctx.stream)


register_part("feed_forward", "gated_mlp", GatedMLP)
register_part("feed_forward", "routed_mlp", RoutedMLP)
