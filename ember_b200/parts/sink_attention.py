"""Softmax attention whose denominator also holds a learned sink per head, in two mixers:

* "sink_attention": grouped-query attention with optional biases on q, k, v, an optional RMS norm over the *whole*
  query projection and over the whole key projection (all heads at once, before the split into heads), no rotation,
  keys of ``head_dim`` and values of ``value_dim``, and a window that keeps the first tokens in sight: position i sees
  j <= i with i - j < window or j < keep_first.  Its cache group is of kind "window" with ``keep_first``: pages the
  window has passed go back while the request runs, those of the kept first tokens stay.  Further options of the spec
  (each a parameter, off by default): an RMS norm per head with one weight for all heads; a short causal convolution on
  q, k, v straight after the projection (its last inputs are a per-request state beside the pages, sub-id "conv"); a
  rotation of queries and keys after the norm; a query temperature that grows with the logarithm of the position; a
  tanh cap on the scaled scores; a chunked mask (i sees j only inside i's chunk of positions); a sigmoid gate per head on
  the attention's output, computed from the mixer's input.
* "latent_attention": queries through a low-rank latent (c_q = RMSNorm(W_dq h), q = W_uq c_q, per head
  [head_dim unrotated | rot_dim rotated]) or, with ``q_rank`` 0, straight from the input (q = W_q h); the rotated parts
  turn in neighbouring pairs or in the rotate-half layout, with the position part's frequencies (stretched for long
  contexts or not) and magnitude; W_dkv h = [kv_rank | rot_dim] gives the RMS-normed latent c and a rotated
  key part shared by the heads; a head's unrotated key is W_uk c and its value W_uv c.  Only [c | rotated part] is
  cached, one row per token (``keys_only``).  The up-projections never touch the cache: with
  q~_h = W_uk[h]^T q_h the score is (q~_h . c + q_rot . k_rot) * scale, and the head's output is W_uv[h] applied to the
  attended latent sum_j w_j c_j, so the attention runs over the cache rows themselves with every query head sharing the
  one row (keys [c | k_rot], values its first kv_rank elements) and the two per-head products are small batched
  products around it.  The concatenated heads are multiplied by sigmoid(W_g h) in the second product's epilogue.
  A layer without W_dkv (``own_kv`` False) reads another layer's cache rows as that layer left them.

The sink has no key and no value: it adds exp(sink[h]) to the softmax's denominator once, unscaled.  Scores, weights,
norms, angles and sums are fp32 in both dtypes.
"""
from __future__ import annotations

from typing import List

import torch

from .. import ops
from ..config.spec import ConfigError
from .base import CacheNeed, Mixer, Runtime, WeightDecl
from .linear import Linear
from .registry import build_part, register_part


class _SinkSoftmax(Mixer):
    """What the two mixers share: cutting long key ranges of small steps into splits, and the attention call."""

    graph_safe = True
    can_store = True

    SPLIT_KEYS = 256            # keys per split, and the most tokens in a step for which key ranges are split
    SPLIT_MAX_TOKENS = 64

    # From how many tokens on a bfloat16 step takes the tensor-core kernel.  Measured at 16 heads over latent rows of 576
    # and 16/8 heads of 128 (eight layers, context 1,024): a decode step at batch 8 takes 2.20 ms with it against 2.95 ms
    # with the general kernel, at batch 64 4.93 against 6.14 ms; tests set it higher to run the general kernel in bfloat16.
    TC_MIN_TOKENS = int(__import__("os").environ.get("EMBER_SINK_TC_MIN_TOKENS", "1"))

    def _attend(self, ctx, q, k_pool, v_pool, out, table, page, heads, kv_heads, dim, vdim, window, keep_first, sink, scale,
                chunk: int = 0, softcap: float = 0.0, head_gate=None, head_gate_col: int = 0):
        on_tc = ctx.T >= self.TC_MIN_TOKENS and ops.shared_row_attention_tc_usable(q, v_pool, dim, vdim)
        tile_q = (ops.shared_row_attention_tc_tile_queries if on_tc else ops.sink_attention_tile_queries)(heads // kv_heads)
        tiles, n_tiles = ctx.attention_tiles(tile_q, "all")
        # long key ranges of a small step are cut into fixed splits so that more SMs share them
        span = ctx.max_context if window <= 0 else min(ctx.max_context, window + keep_first + tile_q)
        if chunk > 0:
            span = min(span, chunk + tile_q)
        n_splits, part_o, part_ml = 1, None, None
        if ctx.T <= self.SPLIT_MAX_TOKENS and span > 2 * self.SPLIT_KEYS:
            n_splits = (ctx.max_context + self.SPLIT_KEYS - 1) // self.SPLIT_KEYS
            part_o = ctx.buf_dyn("sink_attention.part_o", ctx.T * heads * n_splits * vdim, torch.float32)
            part_ml = ctx.buf_dyn("sink_attention.part_ml", ctx.T * heads * n_splits * 2, torch.float32)
        if on_tc:           # scores and the weighted sum on mma.sync
            ops.shared_row_attention_tc(q, k_pool, v_pool, out, ctx.T, heads, kv_heads, dim, vdim, tiles, n_tiles, tile_q, table,
                                        page, window, keep_first, sink, scale, n_splits, self.SPLIT_KEYS, part_o, part_ml,
                                        err=ctx.err, stream=ctx.stream, chunk=chunk, softcap=softcap, head_gate=head_gate,
                                        head_gate_col=head_gate_col)
        else:
            ops.sink_attention(q, k_pool, v_pool, out, ctx.T, heads, kv_heads, dim, vdim, tiles, n_tiles, tile_q, table, page,
                               window, keep_first, sink, scale, n_splits, self.SPLIT_KEYS, part_o, part_ml, err=ctx.err,
                               stream=ctx.stream, chunk=chunk, softcap=softcap, head_gate=head_gate,
                                        head_gate_col=head_gate_col)


class SinkAttention(_SinkSoftmax):
    def __init__(self, spec, prefix: str = ""):
        super().__init__(spec, prefix)
        s = spec
        if s.num_heads <= 0 or s.num_kv_heads <= 0 or s.num_heads % s.num_kv_heads:
            raise ConfigError(f"{s.num_heads} heads do not divide into {s.num_kv_heads} key/value heads")
        if s.head_dim <= 0 or not 0 < s.value_dim <= 512:
            raise ConfigError(f"sink attention: heads of {s.head_dim} / {s.value_dim} (values up to 512)")
        if s.qk_norm not in ("none", "whole", "head"):
            raise ConfigError(f"sink attention: qk_norm {s.qk_norm!r} (none, whole, head)")
        if s.window < 0 or s.keep_first < 0:
            raise ConfigError("sink attention: window and keep_first must be >= 0")
        if s.conv_taps < 0 or s.conv_taps > 64 or s.chunk < 0 or s.q_temp_every < 0 or s.softcap < 0:
            raise ConfigError("sink attention: convolution taps (up to 64), chunk, temperature period and score cap must be >= 0")
        if s.chunk > 0 and s.window > 0:
            raise ConfigError("sink attention: a chunked mask and a window exclude one another")
        self.q_dim, self.k_dim, self.v_dim = s.num_heads * s.head_dim, s.num_kv_heads * s.head_dim, s.num_kv_heads * s.value_dim
        self.channels = self.q_dim + self.k_dim + self.v_dim
        self.position = build_part("position", s.position)
        # the general preparation kernel serves whatever the whole-projection one does not know
        self.general = (s.qk_norm == "head" or s.position.kind != "none" or s.q_temp_every > 0)
        # Causal softmax over keys and values of equal size (no sink, no window; a cap and chunks are parameters) is what
        # the engine's TMA-fed kernels compute (tcgen05 for prompt portions, mma.sync with key splits for single tokens):
        # where they take the geometry, a bfloat16 step goes to them (``load`` decides, once the dtype and the page size
        # are known); a gate per head then is a pass of its own behind them
        self.dense = None
        if (not s.sink and s.window == 0 and s.value_dim == s.head_dim
                and s.head_dim % 2 == 0 and s.num_heads // s.num_kv_heads <= ops.ATTENTION_MAX_GROUP):
            from ..config.spec import AttentionSpec
            from .attention import Attention
            self.dense = Attention(AttentionSpec(hidden_size=s.hidden_size, num_heads=s.num_heads, num_kv_heads=s.num_kv_heads,
                                                 head_dim=s.head_dim, softmax_scale=s.scale, softcap=s.softcap, chunk=s.chunk))

    def weight_decls(self) -> List[WeightDecl]:
        s, p = self.spec, self.prefix
        d = [WeightDecl(p + "q", (self.q_dim, s.hidden_size)), WeightDecl(p + "k", (self.k_dim, s.hidden_size)),
             WeightDecl(p + "v", (self.v_dim, s.hidden_size)), WeightDecl(p + "o", (s.hidden_size, s.num_heads * s.value_dim))]
        if s.bias:
            d += [WeightDecl(p + "q.b", (self.q_dim,), init="zeros"), WeightDecl(p + "k.b", (self.k_dim,), init="zeros"),
                  WeightDecl(p + "v.b", (self.v_dim,), init="zeros")]
        if s.qk_norm == "whole":
            d += [WeightDecl(p + "q.norm", (self.q_dim,), init="norm"), WeightDecl(p + "k.norm", (self.k_dim,), init="norm")]
        if s.qk_norm == "head":
            d += [WeightDecl(p + "q.norm", (s.head_dim,), init="norm"), WeightDecl(p + "k.norm", (s.head_dim,), init="norm")]
        if s.conv_taps > 0:
            d += [WeightDecl(p + n + ".conv", (size, s.conv_taps), init="uniform", lo=-0.5, hi=0.5)
                  for n, size in (("q", self.q_dim), ("k", self.k_dim), ("v", self.v_dim))]
        if s.head_gate:
            d.append(WeightDecl(p + "g", (s.num_heads, s.hidden_size)))
        if s.sink:
            d.append(WeightDecl(p + "sink", (s.num_heads,), init="uniform", lo=-1.0, hi=1.0))
        return d

    def load(self, store, rt: Runtime) -> None:
        s, p = self.spec, self.prefix
        self.rt = rt
        got = {d.name: store.take(d.name, d.shape) for d in self.weight_decls()}
        if any(v is None for v in got.values()):
            return
        wd = rt.weight_dtype(got[p + "q"].dtype)
        # one product for q, k, v and, behind them, the per-head gate's logits (same input)
        self.qkv = Linear(torch.cat([rt.to_device(got[p + n], wd) for n in ("q", "k", "v") + (("g",) if s.head_gate else ())], dim=0).contiguous())
        self.o = Linear.from_host(got[p + "o"], rt)
        f32 = lambda name: rt.to_device(got[p + name], torch.float32)          # noqa: E731
        self.bias = torch.cat([f32(n + ".b") for n in "qkv"]).contiguous() if s.bias else None
        self.q_norm_w = f32("q.norm") if s.qk_norm != "none" else None
        self.k_norm_w = f32("k.norm") if s.qk_norm != "none" else None
        self.sink = f32("sink") if s.sink else None
        self.taps = torch.cat([f32(n + ".conv") for n in "qkv"], dim=0).contiguous() if s.conv_taps > 0 else None
        self.inv_freq, self.rotary = self.position.rotary_table(rt)
        if self.dense is not None:
            self.dense.rt = rt
            multi, single = self.dense._tc_modes()
            if not (self.DENSE_KERNELS and single and (multi or self.dense._fa())):
                self.dense = None

    DENSE_KERNELS = True        # tests switch it off to run such layers on this file's own kernels

    def cache_need(self) -> CacheNeed:
        s = self.spec
        return CacheNeed(kind="window" if s.window > 0 else "full", num_kv_heads=s.num_kv_heads, head_dim=s.head_dim,
                         window=s.window, value_dim=s.value_dim if s.value_dim != s.head_dim else 0,
                         keep_first=s.keep_first if s.window > 0 else 0)

    def cache_needs(self):
        """The pages, and with a convolution a state slot for its last ``conv_taps`` - 1 projected rows (sub-id "conv")."""
        s = self.spec
        needs = {"": self.cache_need()}
        if s.conv_taps > 1:
            needs["conv"] = CacheNeed(kind="state", state_shape=((s.conv_taps - 1) * self.channels,), state_dtype="float32")
        return needs

    def tile_requests(self):
        group = self.spec.num_heads // self.spec.num_kv_heads
        keys = [(ops.sink_attention_tile_queries(group), "all")]
        tc = (ops.shared_row_attention_tc_tile_queries(group), "all")
        keys += [tc] if tc not in keys else []
        if self.dense is not None and getattr(self.dense, "rt", None) is not None:
            keys += [k for k in self.dense.tile_requests() if k not in keys]
        return keys

    def forward(self, ctx, x, out, cache, owns_cache: bool = True, accumulate: bool = True) -> None:
        s, rt, T, mt = self.spec, self.rt, ctx.T, ctx.max_tokens
        H, G, D, V = s.num_heads, s.num_kv_heads, s.head_dim, s.value_dim
        conv_state = None
        if isinstance(cache, dict):                        # pages under "", the convolution's carried rows under "conv"
            cache, conv_state = cache[""], cache.get("conv")
        proj = qkv = ctx.buf("sink_attention.qkv", (mt, self.qkv.n), torch.float32)      # [q | k | v (| gate logits)]
        q = ctx.buf("sink_attention.q", (mt, self.q_dim), rt.dtype)
        att = ctx.buf("sink_attention.out", (mt, H * V), rt.dtype)
        table = ctx.block_table(cache.group)
        self.qkv(ctx, x, qkv, T, ops.EPI_STORE_F32)
        if s.conv_taps > 0:
            # (a run that only reads another layer's cache would still move its own carried rows: such a layer has a
            # state of its own, so nothing is shared)
            mixed = ctx.buf("sink_attention.conv", (mt, self.channels), torch.float32)
            carry = conv_state.state if conv_state is not None else ctx.buf("sink_attention.no_carry", (1, 1), torch.float32)
            ops.conv_silu(qkv, 0, self.taps, None, carry, 0, ctx.seq_of, ctx.query_start, ctx.state_slots, mixed, T, ctx.S,
                          stream=ctx.stream, silu=False)
            qkv = mixed
        if self.general:
            ops.head_prepare_store(qkv, self.bias, s.qk_norm, self.q_norm_w, self.k_norm_w, s.qk_norm_eps,
                                   self.inv_freq if self.rotary else None, self.rotary, s.q_temp_coef, s.q_temp_every, T, H, G, D, V,
                                   ctx.positions, ctx.seq_of, table, cache.page_tokens, cache.k, cache.v, q, write_kv=owns_cache,
                                   err=ctx.err, stream=ctx.stream)
        else:
            ops.whole_norm_store(qkv, self.bias, self.q_norm_w, self.k_norm_w, s.qk_norm_eps, T, H, G, D, V, ctx.positions,
                                 ctx.seq_of, table, cache.page_tokens, cache.k, cache.v, q, write_kv=owns_cache, err=ctx.err,
                                 stream=ctx.stream)
        if self.dense is not None and getattr(self.dense, "rt", None) is not None and ops.TC_ENABLED:
            self.dense.attend(ctx, q, cache, table, att)
            if s.head_gate:
                ops.head_gate_apply(att, proj, self.channels, T, H, V, stream=ctx.stream)
        else:
            self._attend(ctx, q, cache.k, cache.v, att, table, cache.page_tokens, H, G, D, V, s.window, s.keep_first, self.sink,
                         s.scale, chunk=s.chunk, softcap=s.softcap, head_gate=proj if s.head_gate else None,
                         head_gate_col=self.channels)
        self.o(ctx, att, out, T, ops.EPI_ADD_F32 if accumulate else ops.EPI_STORE_F32)


class LatentAttention(_SinkSoftmax):
    def __init__(self, spec, prefix: str = ""):
        super().__init__(spec, prefix)
        s = spec
        if min(s.num_heads, s.head_dim, s.value_dim, s.kv_rank) <= 0 or s.rot_dim < 0 or s.q_rank < 0:
            raise ConfigError("latent attention: head count, sizes and ranks must be positive")
        if s.kv_rank > 512:
            raise ConfigError(f"latent attention: a latent of {s.kv_rank} (up to 512)")
        self.position = build_part("position", s.position)
        rotary = getattr(s.position, "rotary_dim", 0)
        if rotary and (getattr(s.position, "layout", "half") not in ("interleaved", "half") or rotary > s.rot_dim):
            raise ConfigError(f"latent attention rotates at most rot_dim = {s.rot_dim} elements of the rotated part, in the "
                              "layout 'interleaved' or 'half'")
        self.half_layout = bool(rotary) and getattr(s.position, "layout", "half") == "half"
        self.magnitude = float(self.position.magnitude()) if rotary and hasattr(self.position, "magnitude") else 1.0
        self.q_head = s.head_dim + s.rot_dim          # a query head as W_uq makes it
        self.row = s.kv_rank + s.rot_dim              # a cache row, and a query head as the attention reads it

    def weight_decls(self) -> List[WeightDecl]:
        s, p = self.spec, self.prefix
        H, hid = s.num_heads, s.hidden_size
        if s.q_rank:
            d = [WeightDecl(p + "dq", (s.q_rank, hid)), WeightDecl(p + "dq.norm", (s.q_rank,), init="norm"),
                 WeightDecl(p + "uq", (H * self.q_head, s.q_rank))]
        else:
            d = [WeightDecl(p + "q", (H * self.q_head, hid))]
        if s.own_kv:
            d += [WeightDecl(p + "dkv", (self.row, hid)), WeightDecl(p + "dkv.norm", (s.kv_rank,), init="norm")]
        d += [WeightDecl(p + "uk", (H * s.head_dim, s.kv_rank)), WeightDecl(p + "uv", (H * s.value_dim, s.kv_rank))]
        if s.sink:
            d.append(WeightDecl(p + "sink", (H,), init="uniform", lo=-1.0, hi=1.0))
        if s.gate:
            d.append(WeightDecl(p + "g", (H * s.value_dim, hid)))
        d.append(WeightDecl(p + "o", (hid, H * s.value_dim)))
        return d

    def load(self, store, rt: Runtime) -> None:
        s, p = self.spec, self.prefix
        self.rt = rt
        got = {d.name: store.take(d.name, d.shape) for d in self.weight_decls()}
        if any(v is None for v in got.values()):
            return
        first = got[p + ("dq" if s.q_rank else "q")]
        wd = rt.weight_dtype(first.dtype)
        H = s.num_heads
        # one product for everything that reads the layer's input: [query latent, or the queries themselves | key/value
        # latent, key part | gate]
        fused = [first] + ([got[p + "dkv"]] if s.own_kv else []) + ([got[p + "g"]] if s.gate else [])
        self.down = Linear(torch.cat([rt.to_device(t, wd) for t in fused], dim=0).contiguous())
        self.c_col = s.q_rank if s.q_rank else H * self.q_head
        self.g_col = self.c_col + (self.row if s.own_kv else 0)
        self.uq = Linear.from_host(got[p + "uq"], rt) if s.q_rank else None
        # per head: [kv_rank, head_dim] (the key up-projection transposed: it multiplies the query) and [value_dim, kv_rank];
        # in the run's dtype (the per-head product has no form for float32 weights between bfloat16 operands)
        self.uk_t = rt.to_device(got[p + "uk"], rt.dtype).view(H, s.head_dim, s.kv_rank).transpose(1, 2).contiguous()
        self.uv = rt.to_device(got[p + "uv"], rt.dtype).view(H, s.value_dim, s.kv_rank).contiguous()
        self.o = Linear.from_host(got[p + "o"], rt)
        f32 = lambda name: rt.to_device(got[p + name], torch.float32)          # noqa: E731
        self.dq_norm_w = f32("dq.norm") if s.q_rank else None
        self.dkv_norm_w = f32("dkv.norm") if s.own_kv else None
        self.sink = f32("sink") if s.sink else None
        self.inv_freq, self.rotary = self.position.rotary_table(rt)

    def cache_need(self) -> CacheNeed:
        return CacheNeed(kind="full", num_kv_heads=1, head_dim=self.row, keys_only=True)

    def tile_requests(self):
        keys = [(ops.sink_attention_tile_queries(self.spec.num_heads), "all")]
        tc = (ops.shared_row_attention_tc_tile_queries(self.spec.num_heads), "all")
        return keys + ([tc] if tc not in keys else [])

    def forward(self, ctx, x, out, cache, owns_cache: bool = True, accumulate: bool = True) -> None:
        s, rt, T, mt = self.spec, self.rt, ctx.T, ctx.max_tokens
        H, D, R, V, r = s.num_heads, s.head_dim, s.rot_dim, s.value_dim, s.kv_rank
        a = ctx.buf("latent_attention.down", (mt, self.down.n), torch.float32)
        cq = ctx.buf("latent_attention.cq", (mt, s.q_rank), rt.dtype) if s.q_rank else None
        q = ctx.buf("latent_attention.q_latent", (mt, H * self.row), rt.dtype)
        lat = ctx.buf("latent_attention.attended", (mt, H * r), torch.float32)
        og = ctx.buf("latent_attention.out", (mt, H * V), rt.dtype)
        table = ctx.block_table(cache.group)
        write = bool(owns_cache and s.own_kv)
        self.down(ctx, x, a, T, ops.EPI_STORE_F32)
        if s.q_rank or write:
            ops.latent_prepare(a, 0, s.q_rank, self.c_col, r, R, self.dq_norm_w, self.dkv_norm_w, s.norm_eps, self.inv_freq,
                               self.rotary, T, ctx.positions, ctx.seq_of, table, cache.page_tokens, cq, cache.k if write else None,
                               write_kv=write, err=ctx.err, stream=ctx.stream, half_layout=self.half_layout,
                               magnitude=self.magnitude)
        if s.q_rank:
            qf = ctx.buf("latent_attention.q", (mt, H * self.q_head), torch.float32)
            self.uq(ctx, cq, qf, T, ops.EPI_STORE_F32)
        else:
            qf = a                                  # the queries are the first columns of the fused product
        # a query head as the attention reads it: [W_uk[h]^T q_unrotated | q_rotated]
        ops.head_gemm(qf, self.q_head, 0, self.uk_t, q, self.row, 0, T, stream=ctx.stream)
        if R:
            ops.rotate_pairs(qf, self.q_head, D, q, self.row, r, T, H, R, self.rotary, self.inv_freq, ctx.positions,
                             stream=ctx.stream, half_layout=self.half_layout, magnitude=self.magnitude)
        self._attend(ctx, q, cache.k, None, lat, table, cache.page_tokens, H, 1, self.row, r, 0, 0, self.sink, s.scale)
        ops.head_gemm(lat, r, 0, self.uv, og, V, 0, T, gate=a if s.gate else None, gate_col=self.g_col, stream=ctx.stream)
        self.o(ctx, og, out, T, ops.EPI_ADD_F32 if accumulate else ops.EPI_STORE_F32)


register_part("mixer", "sink_attention", SinkAttention)
register_part("mixer", "latent_attention", LatentAttention)
