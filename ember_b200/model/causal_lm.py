"""A causal language model assembled from a ``ModelSpec``: embedding, blocks in schedule
order, final norm, head.

The model holds no sizes of its own.  ``forward`` runs exactly the tokens of the step's
context against the cache and returns fp32 logits for the wanted rows (final norm and head run
only on those rows, as in src/backend/cpu/cpu_backend.cpp:215-224).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import ops
from ..config.spec import ModelSpec
from ..parts.base import CacheNeed, Runtime, WeightDecl
from ..parts.linear import Linear
from ..parts.registry import build_part, part_class
from ..weights.loader import WeightStore


class CausalLM:
    def __init__(self, spec: ModelSpec):
        self.spec = spec
        self.blocks = [part_class("arrangement", ls.arrangement)(ls) for ls in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm, spec.final_norm_prefix)
        self.embedding_position = build_part("position", spec.embedding_position, spec.embedding_position_prefix)
        self.embedding_norm = (build_part("norm", spec.embedding_norm, spec.embedding_norm_prefix)
                               if spec.embedding_norm is not None else None)
        self.rt: Optional[Runtime] = None
        self._cache_subs = [tuple(b.cache_needs()) for b in self.blocks]      # sub-ids of each block's caches

    # ------------------------------------------------------------------ weights
    def weight_decls(self) -> List[WeightDecl]:
        s = self.spec
        d = [WeightDecl(s.embedding_name, (s.vocab_size, s.hidden_size))]
        if not s.tie_embeddings:
            d.append(WeightDecl(s.head_name, (s.vocab_size, s.hidden_size), optional=s.head_optional))
        d += self.final_norm.weight_decls()
        d += self.embedding_position.weight_decls()
        if self.embedding_norm is not None:
            d += self.embedding_norm.weight_decls()
        for b in self.blocks:
            d += b.weight_decls()
        return d

    def load(self, store: WeightStore, rt: Runtime) -> "CausalLM":
        """Device copies of all weights; raises one ``WeightError`` listing every problem."""
        s = self.spec
        self.rt = rt
        emb = store.take(s.embedding_name, (s.vocab_size, s.hidden_size))
        self.embedding = rt.to_device(emb, rt.weight_dtype(emb.dtype)) if emb is not None else None
        if s.tie_embeddings:
            store.allow_unused(s.head_name)       # some files repeat the tied matrix
            head = None
        elif s.head_optional and not store.has(s.head_name):
            head = None
        else:
            head = store.take(s.head_name, (s.vocab_size, s.hidden_size))
        if self.embedding is not None:
            self.head = Linear.from_host(head, rt) if head is not None else Linear(self.embedding)
        self.final_norm.load(store, rt)
        if s.logit_scale != 1.0 and not s.logit_softcap > 0:
            # logits = scale * (norm(h) . head^T): the scale rides on the final norm's output (a model that caps its
            # logits scales them in the capping kernel instead, on the fp32 logits)
            self.final_norm.scale_output(float(s.logit_scale))
        self.embedding_position.load(store, rt)
        if self.embedding_norm is not None:
            self.embedding_norm.load(store, rt)
        for b in self.blocks:
            b.load(store, rt)
        store.finish()
        return self

    @property
    def graph_safe(self) -> bool:
        """Whether decode steps may be captured into CUDA graphs: every part of every block must allow it."""
        return (all(getattr(b, "graph_safe", False) for b in self.blocks) and self.final_norm.graph_safe
                and self.embedding_position.graph_safe
                and (self.embedding_norm is None or self.embedding_norm.graph_safe))

    # -------------------------------------------------------------------- cache
    @staticmethod
    def cache_id(layer: int, sub: str, instance: int = 0):
        """How the cache manager and the storage know one mixer's cache: the layer's index when the block has a
        single mixer (sub-id ""), else (layer, sub-id); a layer that runs several times with caches of its own has
        (layer, sub-id, instance) for every run after the first."""
        if instance:
            return (layer, sub, instance)
        return layer if sub == "" else (layer, sub)

    def cache_needs(self) -> Dict[object, Optional[CacheNeed]]:
        """Need of every mixer of every layer that owns a cache (a layer that only reads another's owns none),
        as the blocks report them."""
        owners = {((e.cache_of if e.cache_of >= 0 else e.layer), e.instance) for e in self.spec.schedule}
        return {self.cache_id(l, sub, inst): need for l, inst in sorted(owners)
                for sub, need in self.blocks[l].cache_needs().items()}

    def tile_requests(self):
        """Attention tile shapes the blocks' mixers will ask the step context for (sent with the step's upload)."""
        if not hasattr(self, "_tile_requests"):
            keys = []
            for b in self.blocks:
                for k in b.tile_requests():
                    if k not in keys:
                        keys.append(k)
            self._tile_requests = tuple(keys)
        return self._tile_requests

    # ------------------------------------------------------------------ forward
    def forward(self, ctx, storage) -> Optional[torch.Tensor]:
        s, rt = self.spec, self.rt
        copies, width = s.residual_streams, s.hidden_size
        h = ctx.buf("model.residual", (ctx.max_tokens, copies * width), torch.float32)
        staged = copies > 1 or self.embedding_norm is not None
        e = ctx.buf("model.embedded", (ctx.max_tokens, width), torch.float32) if staged else h
        ops.embed(ctx.tokens, self.embedding, e, err=ctx.err, stream=ctx.stream, prev_ids=ctx.prev_ids,
                  scale=s.embedding_multiplier)
        self.embedding_position.on_embedding(ctx, e)          # nothing for rotary or absent encodings
        if self.embedding_norm is not None:
            n = h if copies == 1 else ctx.buf("model.embedded_normed", (ctx.max_tokens, width), torch.float32)
            self.embedding_norm.forward(ctx, e, n, ctx.T)
            e = n
        if copies > 1:
            ops.stream_spread(e, h, copies, ctx.T, stream=ctx.stream)       # every copy starts as the embedding's output
        capture = getattr(ctx, "capture_hidden", None)        # (row, buffer [runs of the schedule + 1, hidden]) or None

        def record(i):
            capture[1][i].copy_(h[row].view(copies, width).sum(0) if copies > 1 else h[row])

        if capture is not None:
            row = capture[0] if capture[0] >= 0 else ctx.T + capture[0]
            record(0)
        for i, e in enumerate(s.schedule):
            owner = e.cache_of if e.cache_of >= 0 else e.layer
            block = self.blocks[e.layer]
            caches = {sub: storage.layer(self.cache_id(owner, sub, e.instance)) for sub in self._cache_subs[e.layer]}
            ctx.memo["schedule.index"] = i            # (a block may leave something for the run right after it)
            block.forward(ctx, h, caches, owns_cache=(owner == e.layer))
            if capture is not None:
                record(i + 1)
        if ctx.R == 0:
            return None
        xn = ctx.buf_dyn("model.final_normed", ctx.R * width, rt.dtype).view(-1, width)
        if copies > 1:                                # the stream the head reads is the sum of the copies
            total = ctx.buf_dyn("model.stream_sum", ctx.R * width, torch.float32).view(-1, width)
            ops.stream_sum(h, copies, total, ctx.R, rows=ctx.logit_rows, stream=ctx.stream)
            self.final_norm.forward(ctx, total, xn, ctx.R)
        else:
            self.final_norm.forward(ctx, h, xn, ctx.R, rows=ctx.logit_rows)
        logits = ctx.buf_dyn("model.logits", ctx.R * s.vocab_size, torch.float32).view(-1, s.vocab_size)
        self.head(ctx, xn, logits, ctx.R, ops.EPI_STORE_F32)
        if s.logit_softcap > 0:
            ops.logit_finish(logits, ctx.R * s.vocab_size, float(s.logit_scale), float(s.logit_softcap), stream=ctx.stream)
        return logits[:ctx.R]


def build_model(spec: ModelSpec) -> CausalLM:
    return CausalLM(spec)
