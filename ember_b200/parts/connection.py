"""Connections between a sublayer and a residual stream kept in several copies (hyper-connections).

With copies x_1 .. x_s (all equal to the embedding's output before the first layer; the head reads their sum), a sublayer
reads u = sum_s in[s] x_s through its norm, and its result y changes every copy at once from the old ones:

    x_t <- sum_s mix[s, t] x_s + multiplier * out[t] * (scale * y)

with ``mix`` indexed [from, to] and ``scale`` an optional learned vector over the width (layer scale).  Everything is fp32.
Without learned tensors (``learned`` False) in = out = 1 and mix is the identity: with one copy that is the plain
residual sum x <- x + multiplier * scale * y, so the same arrangement serves a model without hyper-connections.
"""
from __future__ import annotations

from typing import List

import torch

from .. import ops
from ..config.spec import ConfigError
from .base import Connection, Runtime, WeightDecl
from .registry import register_part


class HyperConnection(Connection):
    graph_safe = True

    def __init__(self, spec, prefix: str = ""):
        super().__init__(spec, prefix)
        if spec.size <= 0 or not 1 <= spec.streams <= ops.STREAMS_MAX:
            raise ConfigError(f"hyper-connection: {spec.streams} copies (1 to {ops.STREAMS_MAX}) of width {spec.size}")
        self.in_w = self.out_w = self.mix = self.scale = None

    def weight_decls(self) -> List[WeightDecl]:
        s, p = self.spec, self.prefix
        d = []
        if s.learned:
            n = s.streams
            d += [WeightDecl(f"{p}{s.name}.in", (n,), init="uniform", lo=0.3, hi=0.9),
                  WeightDecl(f"{p}{s.name}.out", (n,), init="uniform", lo=0.5, hi=1.2),
                  WeightDecl(f"{p}{s.name}.mix", (n, n), init="uniform", lo=0.1, hi=0.8)]
        if s.layer_scale:
            d.append(WeightDecl(p + s.scale_name, (s.size,), init="norm"))
        return d

    def load(self, store, rt: Runtime) -> None:
        s, p = self.spec, self.prefix
        decls = self.weight_decls()
        if s.learned and s.streams == 1 and not any(store.has(f"{p}{s.name}.{n}") for n in ("in", "out", "mix")):
            decls = [d for d in decls if d.name == p + s.scale_name]       # one copy and nothing stored: the plain residual sum
        got = {d.name: store.take(d.name, d.shape) for d in decls}
        if any(v is None for v in got.values()):
            return
        f32 = lambda name: rt.to_device(got[name], torch.float32)          # noqa: E731
        if f"{p}{s.name}.in" in got:
            self.in_w, self.out_w, self.mix = f32(f"{p}{s.name}.in"), f32(f"{p}{s.name}.out"), f32(f"{p}{s.name}.mix")
        if s.layer_scale:
            self.scale = f32(p + s.scale_name)

    def read(self, ctx, streams: torch.Tensor, norm, out: torch.Tensor) -> None:
        s = self.spec
        fused = getattr(norm, "stream_norm", None)
        if fused is not None:                       # an element-wise norm rides on the kernel that sums the copies
            ops.stream_read(streams, s.streams, self.in_w, out, ctx.T, norm=fused(), stream=ctx.stream)
            return
        if s.streams == 1 and self.in_w is None:
            u = streams
        else:
            u = ctx.buf("connection.read", (ctx.max_tokens, s.size), torch.float32)
            ops.stream_read(streams, s.streams, self.in_w, u, ctx.T, stream=ctx.stream)
        norm.forward(ctx, u, out, ctx.T)

    def write(self, ctx, streams: torch.Tensor, y: torch.Tensor) -> None:
        s = self.spec
        ops.stream_write(streams, s.streams, self.mix, self.out_w, self.scale, float(s.multiplier), y, ctx.T, stream=ctx.stream)


register_part("connection", "hyper", HyperConnection)
