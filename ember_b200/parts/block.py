"""Arrangements: how a layer's parts are put around the residual stream.

An arrangement is a registered class (family "arrangement") built from a ``LayerSpec``.  It decides which *roles*
the layer's parts play, which family each role belongs to and in what order they run; the model above it only
asks it for its tensors, for what its mixers need of the cache, and to run.  ``Arrangement`` does the common work
(building the parts of the declared roles, declaring and loading their tensors, listing the mixers' cache needs); a
subclass states ``ROLES`` and ``forward``.

"prenorm" (src/backend/cpu/cpu_backend.cpp:139-213): h += mixer(norm_a(h)); h += ffn(norm_b(h)).
The residual stream is fp32; mixers and feed-forwards add into it through the epilogue of
their last product.
"""
from __future__ import annotations

from typing import Dict, List, Mapping, Optional

import torch

from .. import ops
from ..config.spec import ConfigError
from .base import CacheNeed, Runtime, WeightDecl
from .registry import build_part, register_part


class Arrangement:
    """Base of arrangements.  ``ROLES`` maps every role the arrangement understands to its part family, in the
    order the parts are listed; ``OPTIONAL`` names roles a layer may leave out.

    A mixer's cache is known to the model by a *sub-id*: "" if the arrangement has a single mixer role, else the
    role's name.  ``forward`` receives ``caches``, a mapping from sub-id to the ``LayerCache`` of this layer (or of
    the layer whose cache the schedule tells this run to use)."""

    ROLES: Mapping[str, str] = {}
    OPTIONAL: frozenset = frozenset()

    def __init__(self, layer_spec):
        self.spec = layer_spec
        self.parts: Dict[str, object] = {}
        for role, spec, prefix in layer_spec.parts:
            family = self.ROLES.get(role)
            if family is None:
                raise ConfigError(f"arrangement {layer_spec.arrangement!r} has no role {role!r} "
                                  f"(its roles: {', '.join(self.ROLES)})")
            self.parts[role] = build_part(family, spec, prefix)
        missing = [r for r in self.ROLES if r not in self.parts and r not in self.OPTIONAL]
        if missing:
            raise ConfigError(f"arrangement {layer_spec.arrangement!r} needs parts in the roles: {', '.join(missing)}")
        mixer_roles = [r for r, f in self.ROLES.items() if f == "mixer" and r in self.parts]
        self.mixers: Dict[str, object] = {("" if len(mixer_roles) == 1 else r): self.parts[r] for r in mixer_roles}

    @property
    def graph_safe(self) -> bool:
        """Whether a decode step through this block may be captured into a CUDA graph: every part must allow it
        (an arrangement whose own ``forward`` reads host views overrides this with False)."""
        return all(getattr(p, "graph_safe", False) for p in self.parts.values())

    def weight_decls(self) -> List[WeightDecl]:
        return [d for p in self.parts.values() for d in p.weight_decls()]

    def load(self, store, rt: Runtime) -> None:
        self.rt = rt
        for p in self.parts.values():
            p.load(store, rt)

    @staticmethod
    def _join(sub: str, inner: str) -> str:
        return inner if not sub else (sub if not inner else f"{sub}.{inner}")

    def cache_needs(self) -> Dict[str, Optional[CacheNeed]]:
        """What each mixer of the block asks of the cache manager, by sub-id.  A mixer made of several mixers
        (``Mixer.cache_needs`` with names of its own) contributes one entry per inner mixer."""
        return {self._join(sub, inner): need for sub, m in self.mixers.items() for inner, need in m.cache_needs().items()}

    def cache_of(self, caches: Mapping[str, object], sub: str = ""):
        """What ``forward`` hands to the mixer with sub-id ``sub``: its cache, or for a mixer made of several a
        mapping from its inner names to their caches."""
        inner = list(self.mixers[sub].cache_needs())
        if inner == [""]:
            return caches[sub]
        return {name: caches[self._join(sub, name)] for name in inner}

    def tile_requests(self):
        """Attention tile shapes the block's mixers will ask the step context for."""
        keys = []
        for m in self.mixers.values():
            fn = getattr(m, "tile_requests", None)
            for k in (fn() if fn else ()):
                if k not in keys:
                    keys.append(k)
        return keys

    def forward(self, ctx, h: torch.Tensor, caches: Mapping[str, object], owns_cache: bool = True) -> None:
        raise NotImplementedError


class PreNormBlock(Arrangement):
    ROLES = {"mixer_norm": "norm", "mixer": "mixer", "feed_forward_norm": "norm", "feed_forward": "feed_forward"}

    def __init__(self, layer_spec):
        super().__init__(layer_spec)
        self.mixer_norm, self.mixer = self.parts["mixer_norm"], self.parts["mixer"]
        self.feed_forward_norm, self.feed_forward = self.parts["feed_forward_norm"], self.parts["feed_forward"]

    def forward(self, ctx, h: torch.Tensor, caches, owns_cache: bool = True) -> None:
        x = ctx.buf("block.normed", (ctx.max_tokens, h.shape[-1]), self.rt.dtype)
        self.mixer_norm.forward(ctx, h, x, ctx.T)
        self.mixer.forward(ctx, x, h, self.cache_of(caches), owns_cache)
        self.feed_forward_norm.forward(ctx, h, x, ctx.T)
        self.feed_forward.forward(ctx, x, h)


class GatedSandwichBlock(Arrangement):
    """A norm before and after each sublayer, and a gate computed from the sublayer's input on its result:

        x = norm_in(h);  h += norm_out( sublayer(x) * sigmoid(gate(x)) )

    once for the mixer and once for the feed-forward (a layer may have no feed-forward, and either gate may be
    left out).  The sublayer stores its fp32 result in a buffer (``can_store``; others add into a zeroed one); gate,
    output norm and the addition to the residual stream are one kernel (the output norm's ``gated_add``).

    The input norms may be left out as well: the sublayer then reads the residual stream itself,
    ``h += norm_out(sublayer(h))``.  On the float32 path that is the stream's own buffer; on the bfloat16 path it is the
    stream rounded once, which the ``gated_add`` before it leaves beside the new residual rows (the first sublayer of
    a step, or one that follows another arrangement, rounds the stream in a kernel of its own)."""

    ROLES = {"mixer_norm": "norm", "mixer": "mixer", "mixer_gate": "gate", "mixer_out_norm": "norm",
             "feed_forward_norm": "norm", "feed_forward": "feed_forward", "feed_forward_gate": "gate",
             "feed_forward_out_norm": "norm"}
    OPTIONAL = frozenset({"mixer_norm", "mixer_gate", "feed_forward_norm", "feed_forward", "feed_forward_gate",
                          "feed_forward_out_norm"})

    def __init__(self, layer_spec):
        super().__init__(layer_spec)
        p = self.parts
        if ("feed_forward" in p) != ("feed_forward_out_norm" in p) or ("feed_forward_norm" in p and "feed_forward" not in p):
            raise ConfigError("a gated-sandwich layer has a feed-forward with its output norm (and maybe an input norm), or none")
        for role in ("mixer_out_norm", "feed_forward_out_norm"):
            if role in p and not hasattr(p[role], "gated_add"):
                raise ConfigError(f"the norm in the role {role!r} cannot gate, norm and add in one kernel (no gated_add)")

    def _stream(self, ctx, h):
        """What a sublayer without an input norm reads: the stream itself (float32), or its bfloat16 rounding, made
        here unless the kernel that last added to the stream left it (``ctx.memo`` says at which run of the schedule)."""
        if self.rt.dtype == torch.float32:
            return h, None
        r = ctx.buf("block.stream_rounded", (ctx.max_tokens, h.shape[-1]), torch.bfloat16)
        at = ctx.memo.get("schedule.index")
        made = ctx.memo.get("block.stream_rounded.at")
        if at is None or made is None or made not in (at, at - 1) or ctx.memo.get("block.stream_rounded.of") != h.data_ptr():
            ops.round_rows(h, r, ctx.T * h.shape[-1], stream=ctx.stream)
        return r, r

    def _sublayer(self, ctx, h, x, norm_in, run, gate, norm_out, can_store: bool) -> None:
        T, hidden = ctx.T, h.shape[-1]
        y = ctx.buf("block.sublayer", (ctx.max_tokens, hidden), torch.float32)
        rounded = None
        if norm_in is not None:
            norm_in.forward(ctx, h, x, T)
        else:
            x, rounded = self._stream(ctx, h)
        if not can_store:
            y[:T].zero_()
        run(x, y)
        logits = None
        if gate is not None:
            logits = ctx.buf("block.gate", (ctx.max_tokens, hidden), torch.float32)
            gate.forward(ctx, x, logits)
        if rounded is not None:
            norm_out.gated_add(ctx, y, logits, h, T, gate_bias=getattr(gate, "bias", None), rounded=rounded)
            ctx.memo["block.stream_rounded.at"] = ctx.memo.get("schedule.index")
            ctx.memo["block.stream_rounded.of"] = h.data_ptr()
        else:
            norm_out.gated_add(ctx, y, logits, h, T, gate_bias=getattr(gate, "bias", None))

    def forward(self, ctx, h: torch.Tensor, caches, owns_cache: bool = True) -> None:
        p = self.parts
        x = ctx.buf("block.normed", (ctx.max_tokens, h.shape[-1]), self.rt.dtype)
        mixer = p["mixer"]
        store = bool(getattr(mixer, "can_store", False))
        kw = {"accumulate": False} if store else {}
        self._sublayer(ctx, h, x, p.get("mixer_norm"), lambda x, y: mixer.forward(ctx, x, y, self.cache_of(caches), owns_cache, **kw),
                       p.get("mixer_gate"), p["mixer_out_norm"], store)
        ff = p.get("feed_forward")
        if ff is not None:
            store = bool(getattr(ff, "can_store", False))
            kw = {"accumulate": False} if store else {}
            self._sublayer(ctx, h, x, p.get("feed_forward_norm"), lambda x, y: ff.forward(ctx, x, y, **kw),
                           p.get("feed_forward_gate"), p["feed_forward_out_norm"], store)


class ConnectedPreNormBlock(Arrangement):
    """Pre-norm sublayers joined to the residual stream by *connections*:

        x = norm(connection.read(streams));  y = sublayer(x);  connection.write(streams, y)

    once for the mixer and once for the feed-forward (a layer may have none).  The model keeps the stream in
    ``ModelSpec.residual_streams`` copies, ``h`` is [tokens, copies * hidden]; the connection says how the copies are
    read and written (hyper-connections, a residual multiplier, layer scale).  The sublayer stores its fp32 result in a
    buffer (``can_store``; others add into a zeroed one)."""

    ROLES = {"mixer_norm": "norm", "mixer": "mixer", "mixer_connection": "connection",
             "feed_forward_norm": "norm", "feed_forward": "feed_forward", "feed_forward_connection": "connection"}
    OPTIONAL = frozenset({"feed_forward_norm", "feed_forward", "feed_forward_connection"})

    def __init__(self, layer_spec):
        super().__init__(layer_spec)
        p = self.parts
        have = [r in p for r in ("feed_forward_norm", "feed_forward", "feed_forward_connection")]
        if any(have) and not all(have):
            raise ConfigError("a connected layer has a feed-forward with its norm and its connection, or none of the three")
        sizes = {(c.spec.streams, c.spec.size) for r, c in p.items() if self.ROLES[r] == "connection"}
        if len(sizes) != 1:
            raise ConfigError("the connections of a layer must agree on the copies of the stream and on its width")
        self.streams, self.hidden = next(iter(sizes))

    def _sublayer(self, ctx, h, norm, run, connection, can_store: bool) -> None:
        x = ctx.buf("block.normed", (ctx.max_tokens, self.hidden), self.rt.dtype)
        y = ctx.buf("block.sublayer", (ctx.max_tokens, self.hidden), torch.float32)
        connection.read(ctx, h, norm, x)
        if not can_store:
            y[:ctx.T].zero_()
        run(x, y)
        connection.write(ctx, h, y)

    def forward(self, ctx, h: torch.Tensor, caches, owns_cache: bool = True) -> None:
        p = self.parts
        if h.shape[-1] != self.streams * self.hidden:
            raise ConfigError(f"the layer is connected to {self.streams} copies of width {self.hidden}; the model's stream has "
                              f"rows of {h.shape[-1]}")
        mixer = p["mixer"]
        store = bool(getattr(mixer, "can_store", False))
        kw = {"accumulate": False} if store else {}
        self._sublayer(ctx, h, p["mixer_norm"], lambda x, y: mixer.forward(ctx, x, y, self.cache_of(caches), owns_cache, **kw),
                       p["mixer_connection"], store)
        ff = p.get("feed_forward")
        if ff is not None:
            store = bool(getattr(ff, "can_store", False))
            kw = {"accumulate": False} if store else {}
            self._sublayer(ctx, h, p["feed_forward_norm"], lambda x, y: ff.forward(ctx, x, y, **kw),
                           p["feed_forward_connection"], store)


class PostNormBlock(Arrangement):
    """The norm after the sum, with a scaled stream:

        h = mixer_norm(alpha * h + mixer(h));  h = feed_forward_norm(alpha * h + feed_forward(h))

    The sublayers read the stream itself (float32: the stream's buffer; bfloat16: the stream rounded once, which the
    fused scale + add + norm of the sublayer before leaves beside the new rows).  A layer may have no feed-forward.
    ``alpha`` is the arrangement's one constant (``LayerSpec.constants``, name "alpha"; 1 if absent).  The sublayer stores its fp32 result in a buffer
    (``can_store``; others add into a zeroed one); scale, addition, norm and the rounded copy are one kernel (the norm's
    ``scaled_add``), which also adds the bias a feed-forward's last product left out (``result_bias``).  A feed-forward
    that wants the fp32 stream beside its rounded input (identity experts) gets it as ``stream=``."""

    ROLES = {"mixer": "mixer", "mixer_norm": "norm", "feed_forward": "feed_forward", "feed_forward_norm": "norm"}
    OPTIONAL = frozenset({"feed_forward", "feed_forward_norm"})

    def __init__(self, layer_spec):
        super().__init__(layer_spec)
        p = self.parts
        self.alpha = layer_spec.constant("alpha", 1.0)
        if ("feed_forward" in p) != ("feed_forward_norm" in p):
            raise ConfigError("a post-norm layer has a feed-forward with its norm, or neither")
        for role in ("mixer_norm", "feed_forward_norm"):
            if role in p and not hasattr(p[role], "scaled_add"):
                raise ConfigError(f"the norm in the role {role!r} cannot scale, add and norm in one kernel (no scaled_add)")

    def _input(self, ctx, h):
        """What a sublayer reads, and the bfloat16 buffer the next fused norm fills (None on the float32 path)."""
        if self.rt.dtype == torch.float32:
            return h, None
        r = ctx.buf("block.stream_rounded", (ctx.max_tokens, h.shape[-1]), torch.bfloat16)
        at = ctx.memo.get("schedule.index")
        made = ctx.memo.get("block.stream_rounded.at")
        if at is None or made is None or made not in (at, at - 1) or ctx.memo.get("block.stream_rounded.of") != h.data_ptr():
            ops.round_rows(h, r, ctx.T * h.shape[-1], stream=ctx.stream)
        return r, r

    def _sublayer(self, ctx, h, part, norm, run) -> None:
        T, hidden = ctx.T, h.shape[-1]
        y = ctx.buf("block.sublayer", (ctx.max_tokens, hidden), torch.float32)
        x, rounded = self._input(ctx, h)
        if not getattr(part, "can_store", False):
            y[:T].zero_()
        run(x, y)
        norm.scaled_add(ctx, y, h, T, self.alpha, y_bias=getattr(part, "result_bias", None), rounded=rounded)
        if rounded is not None:
            ctx.memo["block.stream_rounded.at"] = ctx.memo.get("schedule.index")
            ctx.memo["block.stream_rounded.of"] = h.data_ptr()

    def forward(self, ctx, h: torch.Tensor, caches, owns_cache: bool = True) -> None:
        p = self.parts
        mixer = p["mixer"]
        kw = {"accumulate": False} if getattr(mixer, "can_store", False) else {}
        self._sublayer(ctx, h, mixer, p["mixer_norm"], lambda x, y: mixer.forward(ctx, x, y, self.cache_of(caches), owns_cache, **kw))
        ff = p.get("feed_forward")
        if ff is not None:
            kw = {"accumulate": False} if getattr(ff, "can_store", False) else {}
            if getattr(ff, "result_bias", None) is not None:
                kw["fold_bias"] = True
            if getattr(getattr(ff, "spec", None), "identity", 0):
                kw["stream"] = h
            self._sublayer(ctx, h, ff, p["feed_forward_norm"], lambda x, y: ff.forward(ctx, x, y, **kw))


register_part("arrangement", "prenorm", PreNormBlock)
register_part("arrangement", "postnorm", PostNormBlock)
register_part("arrangement", "connected_prenorm", ConnectedPreNormBlock)
register_part("arrangement", "gated_sandwich", GatedSandwichBlock)
