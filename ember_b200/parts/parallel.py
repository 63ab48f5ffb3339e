"""Two mixers side by side on the same input: result = left_scale * left + right_scale * right.

Each inner mixer keeps a cache of its own (pages, a state slot, ...): ``cache_needs`` names them "left" and "right"
(an inner mixer with several caches contributes "left.<its name>" ...) and ``forward`` receives a mapping with those
names.  The inner mixers store their fp32 results in buffers (``can_store``) and one kernel forms the scaled sum.

With ``branch_norm`` each result is first divided by its root mean square over the model width and multiplied by a
weight of its own: result = left_scale * w_l * left / rms(left) + right_scale * w_r * right / rms(right), still one
kernel (the scales are folded into the weights when they are loaded).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import ops
from ..config.spec import ConfigError
from .base import CacheNeed, Mixer, Runtime, WeightDecl
from .registry import build_part, register_part


class ParallelMixer(Mixer):
    can_store = True

    def __init__(self, spec, prefix: str = ""):
        super().__init__(spec, prefix)
        self.left = build_part("mixer", spec.left, prefix + spec.left_prefix)
        self.right = build_part("mixer", spec.right, prefix + spec.right_prefix)
        for m in (self.left, self.right):
            if not getattr(m, "can_store", False):
                raise ConfigError(f"a parallel mixer needs inner mixers that can store their result; {type(m).__name__} cannot")
        self._inner = {"left": list(self.left.cache_needs()), "right": list(self.right.cache_needs())}

    @property
    def graph_safe(self) -> bool:
        return self.left.graph_safe and self.right.graph_safe

    def _norm_names(self):
        return self.prefix + self.spec.left_norm_name, self.prefix + self.spec.right_norm_name

    def weight_decls(self) -> List[WeightDecl]:
        d = self.left.weight_decls() + self.right.weight_decls()
        if self.spec.branch_norm:
            d += [WeightDecl(n, (self.spec.hidden_size,), init="norm") for n in self._norm_names()]
        return d

    def load(self, store, rt: Runtime) -> None:
        self.rt = rt
        self.left.load(store, rt)
        self.right.load(store, rt)
        self.norm_left = self.norm_right = None
        if self.spec.branch_norm:
            wl, wr = (store.take(n, (self.spec.hidden_size,)) for n in self._norm_names())
            if wl is not None and wr is not None:
                self.norm_left = rt.to_device(wl, torch.float32) * float(self.spec.left_scale)
                self.norm_right = rt.to_device(wr, torch.float32) * float(self.spec.right_scale)

    @staticmethod
    def _join(side: str, inner: str) -> str:
        return side if not inner else f"{side}.{inner}"

    def cache_needs(self) -> Dict[str, Optional[CacheNeed]]:
        return {self._join(side, name): need for side, m in (("left", self.left), ("right", self.right))
                for name, need in m.cache_needs().items()}

    def _cache_of(self, cache, side: str):
        names = self._inner[side]
        if names == [""]:
            return cache[side]
        return {name: cache[self._join(side, name)] for name in names}

    def tile_requests(self):
        keys = []
        for m in (self.left, self.right):
            fn = getattr(m, "tile_requests", None)
            keys += [k for k in (fn() if fn else ()) if k not in keys]
        return keys

    def forward(self, ctx, x, out, cache, owns_cache: bool = True, accumulate: bool = True) -> None:
        s, hidden = self.spec, self.spec.hidden_size
        a = ctx.buf("parallel.left", (ctx.max_tokens, hidden), torch.float32)
        b = ctx.buf("parallel.right", (ctx.max_tokens, hidden), torch.float32)
        self.left.forward(ctx, x, a, self._cache_of(cache, "left"), owns_cache, accumulate=False)
        self.right.forward(ctx, x, b, self._cache_of(cache, "right"), owns_cache, accumulate=False)
        if s.branch_norm:
            ops.pair_norm_sum(a, self.norm_left, b, self.norm_right, s.norm_eps, out, ctx.T, accumulate=accumulate, stream=ctx.stream)
        else:
            ops.scaled_sum(a, s.left_scale, b, s.right_scale, out, ctx.T * hidden, accumulate=accumulate, stream=ctx.stream)


register_part("mixer", "parallel", ParallelMixer)
