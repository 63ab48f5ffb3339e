"""Norms.  RMSNorm: out = weight * (x * rsqrt(mean(x^2) + eps)), statistics in fp32.

Formula: src/backend/cpu/cpu_backend.cpp:34-39 (the weight multiplies after the scaling; it
is the plain weight, not 1 + weight).
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .. import ops
from .base import Norm, Runtime, WeightDecl
from .registry import register_part


class RMSNorm(Norm):
    graph_safe = True

    def _name(self) -> str:
        return self.prefix + getattr(self.spec, "weight_suffix", "weight")

    def weight_decls(self) -> List[WeightDecl]:
        return [WeightDecl(self._name(), (self.spec.size,), init="norm")]

    def load(self, store, rt: Runtime) -> None:
        w = store.take(self._name(), (self.spec.size,))
        self.weight = rt.to_device(w, torch.float32) if w is not None else None

    def scale_output(self, scale: float) -> None:
        if self.weight is not None:
            self.weight = self.weight * scale

    def forward(self, ctx, x: torch.Tensor, out: torch.Tensor, n_rows: int, rows: Optional[torch.Tensor] = None) -> None:
        ops.rmsnorm(x, self.weight, self.spec.eps, out, n_rows, rows=rows, stream=ctx.stream)

    def gated_add(self, ctx, y: torch.Tensor, gate_logits: Optional[torch.Tensor], residual: torch.Tensor, n_rows: int,
                  gate_bias: Optional[torch.Tensor] = None, rounded: Optional[torch.Tensor] = None) -> None:
        """residual += norm(y * sigmoid(gate_logits + gate_bias)) in one kernel (no gate if ``gate_logits`` is None);
        ``rounded`` (bfloat16) also receives the new residual rows."""
        ops.gated_norm_add(y, gate_logits, self.weight, None, self.spec.eps, False, residual, n_rows, gate_bias=gate_bias,
                           rounded=rounded, stream=ctx.stream)

    def scaled_add(self, ctx, y: torch.Tensor, residual: torch.Tensor, n_rows: int, alpha: float,
                   y_bias: Optional[torch.Tensor] = None, rounded: Optional[torch.Tensor] = None) -> None:
        """residual = norm(alpha * residual + y + y_bias) in one kernel, in place: the norm after the residual sum;
        ``rounded`` (bfloat16) also receives the new rows."""
        ops.scaled_add_norm(y, y_bias, alpha, self.weight, None, self.spec.eps, False, residual, n_rows, rounded=rounded,
                            stream=ctx.stream)


class LayerNorm(Norm):
    """out = (x - mean) / sqrt(var + eps) * weight + bias, var = mean((x - mean)^2), statistics in fp32."""

    graph_safe = True

    def _names(self):
        return self.prefix + self.spec.weight_suffix, self.prefix + self.spec.bias_suffix

    def _has_bias(self) -> bool:
        return bool(getattr(self.spec, "bias", True))

    def weight_decls(self) -> List[WeightDecl]:
        w, b = self._names()
        return [WeightDecl(w, (self.spec.size,), init="norm")] + ([WeightDecl(b, (self.spec.size,), init="zeros")] if self._has_bias() else [])

    def load(self, store, rt: Runtime) -> None:
        names = self._names()
        w = store.take(names[0], (self.spec.size,))
        b = store.take(names[1], (self.spec.size,)) if self._has_bias() else None
        self.weight = rt.to_device(w, torch.float32) if w is not None else None
        self.bias = rt.to_device(b, torch.float32) if b is not None else None

    def scale_output(self, scale: float) -> None:
        if self.weight is not None:
            self.weight = self.weight * scale
            self.bias = self.bias * scale if self.bias is not None else None

    def scaled_add(self, ctx, y: torch.Tensor, residual: torch.Tensor, n_rows: int, alpha: float,
                   y_bias: Optional[torch.Tensor] = None, rounded: Optional[torch.Tensor] = None) -> None:
        """residual = norm(alpha * residual + y + y_bias) in one kernel, in place: the norm after the residual sum;
        ``rounded`` (bfloat16) also receives the new rows."""
        ops.scaled_add_norm(y, y_bias, alpha, self.weight, self.bias, self.spec.eps, True, residual, n_rows, rounded=rounded,
                            stream=ctx.stream)

    def forward(self, ctx, x: torch.Tensor, out: torch.Tensor, n_rows: int, rows: Optional[torch.Tensor] = None) -> None:
        ops.layer_norm(x, self.weight, self.bias, self.spec.eps, out, n_rows, rows=rows, stream=ctx.stream)

    def gated_add(self, ctx, y: torch.Tensor, gate_logits: Optional[torch.Tensor], residual: torch.Tensor, n_rows: int,
                  gate_bias: Optional[torch.Tensor] = None, rounded: Optional[torch.Tensor] = None) -> None:
        """residual += norm(y * sigmoid(gate_logits + gate_bias)) in one kernel (no gate if ``gate_logits`` is None);
        ``rounded`` (bfloat16) also receives the new residual rows."""
        ops.gated_norm_add(y, gate_logits, self.weight, self.bias, self.spec.eps, True, residual, n_rows, gate_bias=gate_bias,
                           rounded=rounded, stream=ctx.stream)


class DynamicTanh(Norm):
    """out = tanh(alpha * x) * weight + bias, element by element, fp32: a norm that computes no mean or variance
    (``alpha`` is a stored scalar).  Being element-wise it can ride on the kernel that sums the copies of a residual
    stream (``stream_norm``)."""

    graph_safe = True

    def _names(self):
        s = self.spec
        return self.prefix + s.weight_suffix, self.prefix + s.bias_suffix, self.prefix + s.alpha_suffix

    def weight_decls(self) -> List[WeightDecl]:
        w, b, a = self._names()
        return [WeightDecl(w, (self.spec.size,), init="norm"), WeightDecl(b, (self.spec.size,), init="zeros"),
                WeightDecl(a, (), init="uniform", lo=0.4, hi=1.2)]

    def load(self, store, rt: Runtime) -> None:
        w, b, a = self._names()
        w, b, a = store.take(w, (self.spec.size,)), store.take(b, (self.spec.size,)), store.take(a, ())
        self.weight = rt.to_device(w, torch.float32) if w is not None else None
        self.bias = rt.to_device(b, torch.float32) if b is not None else None
        self.alpha = rt.to_device(a, torch.float32).reshape(1) if a is not None else None

    def scale_output(self, scale: float) -> None:
        if self.weight is not None:
            self.weight, self.bias = self.weight * scale, self.bias * scale

    def forward(self, ctx, x: torch.Tensor, out: torch.Tensor, n_rows: int, rows: Optional[torch.Tensor] = None) -> None:
        ops.dynamic_tanh(x, self.alpha, self.weight, self.bias, out, n_rows, rows=rows, stream=ctx.stream)

    def stream_norm(self):
        """(alpha, weight, bias) for ``ops.stream_read``, which applies the norm to the sum it has just made."""
        return self.alpha, self.weight, self.bias


register_part("norm", "rmsnorm", RMSNorm)
register_part("norm", "dynamic_tanh", DynamicTanh)
register_part("norm", "layernorm", LayerNorm)
