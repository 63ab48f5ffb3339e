"""Typed description of a model as data: parts, layers, and the order they run in.

An architecture's configuration class (for instance ``Qwen3Config``) turns the keys
of its ``config.json`` into a ``ModelSpec``.  Everything below the configuration
(weights, parts, cache manager, step function) reads only the ``ModelSpec``; no
size or constant of a model is written anywhere else.

A part spec is a frozen dataclass with a class attribute ``kind``; the part
registry (``ember_b200.parts.registry``) maps ``(family, kind)`` to the class that
implements it.  A test or a user can define a new spec + part pair and register it
without touching the framework's files.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import ClassVar, Optional, Tuple


class ConfigError(ValueError):
    """A configuration that cannot be built (missing key, bad value, unsupported option)."""


@dataclass(frozen=True)
class PartSpec:
    """Base of all part specs.  ``kind`` selects the implementation in the registry."""

    kind: ClassVar[str] = ""


# ----------------------------------------------------------------------------- norms
@dataclass(frozen=True)
class RMSNormSpec(PartSpec):
    """out = weight * (x * rsqrt(mean(x^2) + eps)); plain weight (not 1 + weight).  The tensor is named prefix +
    ``weight_suffix``."""

    kind: ClassVar[str] = "rmsnorm"
    size: int = 0
    eps: float = 1e-6
    weight_suffix: str = "weight"


@dataclass(frozen=True)
class LayerNormSpec(PartSpec):
    """out = (x - mean) / sqrt(var + eps) * weight + bias, var the mean of the squared deviations.  The tensors are
    named prefix + ``weight_suffix`` and prefix + ``bias_suffix``."""

    kind: ClassVar[str] = "layernorm"
    size: int = 0
    eps: float = 1e-5
    weight_suffix: str = "weight"
    bias_suffix: str = "bias"
    bias: bool = True             # False: a weight and no bias (no tensor under ``bias_suffix``)


@dataclass(frozen=True)
class DynamicTanhSpec(PartSpec):
    """out = tanh(alpha * x) * weight + bias, element by element: a norm that takes no mean or variance.  ``alpha`` is a
    stored scalar.  The tensors are named prefix + ``weight_suffix``, ``bias_suffix`` and ``alpha_suffix``."""

    kind: ClassVar[str] = "dynamic_tanh"
    size: int = 0
    weight_suffix: str = "weight"
    bias_suffix: str = "bias"
    alpha_suffix: str = "alpha"


# ---------------------------------------------------------------- position encodings
@dataclass(frozen=True)
class RotarySpec(PartSpec):
    """Rotary embedding over the first ``rotary_dim`` elements of a head.  ``layout`` "half" pairs element i with
    i + rotary_dim / 2, "interleaved" pairs element 2i with 2i + 1; the angle of pair i is position * theta^(-2i / rotary_dim)
    either way."""

    kind: ClassVar[str] = "rope"
    head_dim: int = 0
    rotary_dim: int = 0          # == head_dim for a full rotation
    theta: float = 10000.0
    # "float32": 1 / powf(theta, 2i / rotary_dim) as the Qwen3 reference computes it; "float64": theta^(-2i / rotary_dim)
    # in double precision, rounded once
    frequency_precision: str = "float32"
    layout: str = "half"
    # Stretching for contexts longer than the model was made for (YaRN): with d(t) = rotary_dim ln(original / (2 pi t)) /
    # (2 ln theta), lo = max(floor(d(fast)), 0), hi = min(ceil(d(slow)), rotary_dim - 1) and the ramp
    # r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), frequency i becomes f_i / factor * r_i + f_i (1 - r_i), and
    # cosines and sines are multiplied by 0.1 ln(factor) + 1.  ``scaling_factor`` 0: no stretching.
    scaling_factor: float = 0.0
    scaling_original: float = 0.0
    scaling_fast: float = 32.0
    scaling_slow: float = 1.0
    # Linear scaling (position interpolation): every frequency is divided by ``linear_factor``, nothing else changes.
    linear_factor: float = 1.0


@dataclass(frozen=True)
class NoPositionSpec(PartSpec):
    kind: ClassVar[str] = "none"


# ---------------------------------------------------------------------------- mixers
@dataclass(frozen=True)
class AttentionSpec(PartSpec):
    """Grouped-query causal attention over a paged key/value cache."""

    kind: ClassVar[str] = "attention"
    hidden_size: int = 0
    num_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0
    qk_norm: bool = False         # RMSNorm on each query/key head before the rotation
    qk_norm_eps: float = 1e-6
    bias: bool = False            # biases on the q/k/v projections
    window: int = 0               # 0 = all keys; w > 0 = the last w keys (self included)
    softmax_scale: Optional[float] = None   # None = 1/sqrt(head_dim)
    position: PartSpec = field(default_factory=NoPositionSpec)
    softcap: float = 0.0          # > 0: score <- softcap * tanh(score / softcap) after the scale (tensor-core kernels only)
    chunk: int = 0                # > 0: position i sees j <= i only if floor(i / chunk) == floor(j / chunk) (tensor-core kernels only)

    @property
    def q_dim(self) -> int:
        return self.num_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_kv_heads * self.head_dim

    @property
    def group(self) -> int:
        return self.num_heads // self.num_kv_heads


@dataclass(frozen=True)
class SigmoidAttentionSpec(PartSpec):
    """Grouped-query causal attention without softmax over a paged cache: a visible key's weight is
    sigmoid(scale * q . k + head_bias[head]), not normalised over keys.  Keys and values may differ in size; the
    first ``position.rotary_dim`` elements of query and key heads are rotated.  Tensors: q, k, v, o, pb."""

    kind: ClassVar[str] = "sigmoid_attention"
    hidden_size: int = 0
    num_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0             # queries and keys
    value_dim: int = 0
    scale: float = 1.0
    position: PartSpec = field(default_factory=NoPositionSpec)


@dataclass(frozen=True)
class SinkAttentionSpec(PartSpec):
    """Grouped-query softmax attention over a paged cache whose denominator also holds exp(sink[head]) (a learned
    number per head without key or value, tensor ``sink``).  Keys and values may differ in size.  ``qk_norm`` "whole":
    one RMS norm over the whole query projection and one over the whole key projection (tensors ``q.norm``, ``k.norm``
    of that size), "none": no norm.  ``window`` > 0: position i sees j <= i with i - j < window or j < keep_first.
    ``bias``: q, k and v have biases (``q.b`` ...).  Tensors: q, k, v, o.

    Options that other designs turn on, each alone or together: ``qk_norm`` "head" (an RMS norm per head, weights of
    ``head_dim`` shared by the heads); ``conv_taps`` > 0 (a short causal convolution over time on every channel of q,
    k and v, tensors ``q.conv`` ... [channels, taps], straight after the projection; the last taps - 1 projected rows
    are a per-request state); ``position`` (a rotation of queries and keys after the norm); ``q_temp_every`` > 0 (the
    query at position p is multiplied by 1 + q_temp_coef * ln(floor((p + 1) / q_temp_every) + 1)); ``softcap`` > 0
    (score <- softcap * tanh(score / softcap) after the scale); ``chunk`` > 0 (position i sees j <= i only if
    floor(i / chunk) == floor(j / chunk), chunks counted from the sequence's start); ``head_gate`` (head h's output is
    multiplied by sigmoid(W_g x)_h, tensor ``g`` [heads, hidden])."""

    kind: ClassVar[str] = "sink_attention"
    hidden_size: int = 0
    num_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0
    value_dim: int = 0
    scale: float = 1.0
    bias: bool = False
    qk_norm: str = "none"
    qk_norm_eps: float = 1e-6
    window: int = 0
    keep_first: int = 0
    sink: bool = True
    conv_taps: int = 0
    position: PartSpec = field(default_factory=NoPositionSpec)
    q_temp_coef: float = 0.0
    q_temp_every: int = 0
    softcap: float = 0.0
    chunk: int = 0
    head_gate: bool = False


@dataclass(frozen=True)
class LatentAttentionSpec(PartSpec):
    """Causal attention whose keys and values are up-projections of a low-rank latent.  Queries: c_q = RMSNorm(W_dq h),
    q = W_uq c_q, per head [head_dim unrotated | rot_dim rotated].  W_dkv h = [kv_rank | rot_dim]: the first part,
    RMS-normed, is the latent c; the rest, rotated, is a key part all heads share.  Per head the unrotated key is
    W_uk c and the value W_uv c; only [c | rotated part] is cached.  A sink per head joins the softmax's denominator,
    and the concatenated heads are multiplied by sigmoid(W_g h) before W_o.  ``own_kv`` False: the layer has no W_dkv
    and reads the cache of another layer (the schedule says whose).  ``q_rank`` 0: no query latent, q = W_q h (tensor
    ``q``).  The rotated parts follow ``position`` (its layout, frequencies and magnitude)."""

    kind: ClassVar[str] = "latent_attention"
    hidden_size: int = 0
    num_heads: int = 0
    head_dim: int = 0             # unrotated query/key elements per head
    rot_dim: int = 0              # rotated query/key elements per head (the key's are shared by the heads)
    value_dim: int = 0
    q_rank: int = 0
    kv_rank: int = 0
    scale: float = 1.0
    norm_eps: float = 1e-6
    sink: bool = True
    gate: bool = True
    own_kv: bool = True
    position: PartSpec = field(default_factory=NoPositionSpec)


@dataclass(frozen=True)
class GatedLinearAttentionSpec(PartSpec):
    """Linear attention with a decay per head and key channel: S <- diag(alpha) S + k v^T, o = S^T q with
    alpha = sigmoid(W_a2 W_a1 h + b)^(1 / tau) and q times head_dim^-1/2; per-head RMS norm with a weight shared by
    the heads, a silu gate, W_o.  ``decay_rank`` 0: read from the stored tensors' shapes."""

    kind: ClassVar[str] = "gla"
    hidden_size: int = 0
    num_heads: int = 0
    head_dim: int = 0
    value_dim: int = 0
    tau: float = 16.0
    decay_rank: int = 0
    norm_eps: float = 1e-6


@dataclass(frozen=True)
class TimeMixSpec(PartSpec):
    """Time mixing with a matrix state per head and a decay per head and key channel (RWKV style).  With h' the
    previous token's input (zeros before the first token; part of the state), each of r, k, v, g, w reads its own blend
    h + (h' - h) mu; r, k, v are heads x head_dim, the gate is silu(W_g .), the decay
    w = exp(-exp(W_w2 tanh(W_w1 .) + w0)).  Per head: o = (S + diag(u) k v^T)^T r, then S <- diag(w) S + k v^T; o is divided
    by its root mean square, times ``norm``, times the gate, W_o.  ``decay_rank`` 0: read from the stored tensors' shapes."""

    kind: ClassVar[str] = "wkv"
    hidden_size: int = 0
    num_heads: int = 0
    head_dim: int = 0
    decay_rank: int = 0
    norm_eps: float = 1e-5


@dataclass(frozen=True)
class GatedDeltaSpec(PartSpec):
    """Delta-rule memory with a decay per head and key channel: short convolutions + silu on q, k, v, unit-length
    q and k, a write strength per head, low-rank projections for the decay and for the output gate.
    ``decay_rank`` / ``gate_rank`` 0: read from the stored tensors' shapes.

    ``decay`` "head": one decay per head, g = exp(-exp(A_log[h]) softplus(W_a x + dt_bias[h])) with a full-rank
    projection ``a`` [heads, hidden] (no a1 / a2, ``dt_bias`` [heads]).  ``gate`` "silu": the normed read-out is
    multiplied by silu(W_g x) with a full-rank ``g`` [heads vdim, hidden] (no g1 / g2) instead of the low-rank sigmoid gate."""

    kind: ClassVar[str] = "channel_delta"
    hidden_size: int = 0
    num_heads: int = 0            # value heads
    num_kv_heads: int = 0         # query/key heads
    head_dim: int = 0
    value_dim: int = 0
    conv_taps: int = 4
    decay_rank: int = 0
    gate_rank: int = 0
    norm_eps: float = 1e-6
    key_eps: float = 1e-6         # inside the root of the unit norm of q and k
    decay: str = "channel"        # "channel" | "head"
    gate: str = "low_rank_sigmoid"   # "low_rank_sigmoid" | "silu"


@dataclass(frozen=True)
class MatrixMemorySpec(PartSpec):
    """Matrix memory with an exponential input gate (mLSTM): log gates capped by ``gate_cap * tanh(. / gate_cap)``,
    a running maximum that starts at zero, per-head RMS norm and a sigmoid output gate."""

    kind: ClassVar[str] = "mlstm"
    hidden_size: int = 0
    num_heads: int = 0
    head_dim: int = 0
    value_dim: int = 0
    gate_cap: float = 15.0
    norm_eps: float = 1e-6


@dataclass(frozen=True)
class StateSpaceSpec(PartSpec):
    """Selective state space with a scalar decay per head (Mamba-2): one input projection [z | x | B | C | dt], a
    short convolution + silu over x, B, C, a silu gate before an RMS norm in ``norm_groups`` equal parts."""

    kind: ClassVar[str] = "mamba2"
    hidden_size: int = 0
    num_heads: int = 0
    value_dim: int = 0
    state_size: int = 0
    num_groups: int = 1
    norm_groups: int = 1
    conv_taps: int = 4
    norm_eps: float = 1e-6

    @property
    def inner(self) -> int:
        return self.num_heads * self.value_dim


@dataclass(frozen=True)
class ParallelMixerSpec(PartSpec):
    """Two mixers that read the same input; the result is left_scale * left + right_scale * right.  ``branch_norm``:
    each result is first RMS-normed over the model width with a weight of its own (tensors ``left_norm_name`` and
    ``right_norm_name`` under the mixer's prefix, eps ``norm_eps``)."""

    kind: ClassVar[str] = "parallel"
    hidden_size: int = 0
    left: PartSpec = field(default_factory=PartSpec)
    right: PartSpec = field(default_factory=PartSpec)
    left_scale: float = 1.0
    right_scale: float = 1.0
    left_prefix: str = "left."
    right_prefix: str = "right."
    branch_norm: bool = False
    norm_eps: float = 1e-6
    left_norm_name: str = "left.out"
    right_norm_name: str = "right.out"


# ----------------------------------------------------------------------------- gates
@dataclass(frozen=True)
class SigmoidGateSpec(PartSpec):
    """An element-wise gate sigmoid(W h + b) on a sublayer's result.  Tensors: prefix + ``weight_suffix`` [size,
    size] and prefix + ``bias_suffix`` [size]."""

    kind: ClassVar[str] = "sigmoid_linear"
    size: int = 0
    weight_suffix: str = "weight"
    bias_suffix: str = "bias"


# --------------------------------------------------------------------- feed-forwards
@dataclass(frozen=True)
class GatedMLPSpec(PartSpec):
    """down( act(gate(x)) * up(x) ), no biases; act is "silu", "relu" or "gelu_tanh" (0.5 z (1 + tanh(sqrt(2 / pi)
    (z + 0.044715 z^3)))).  ``names``: the three tensors' names under the prefix (gate, up, down)."""

    kind: ClassVar[str] = "gated_mlp"
    hidden_size: int = 0
    intermediate_size: int = 0
    activation: str = "silu"
    names: Tuple[str, str, str] = ("gate_proj.weight", "up_proj.weight", "down_proj.weight")
    # ``activation`` "clamped_swish": g = min(gate, limit), u = clamp(up, -limit, limit), g sigmoid(alpha g) (u + up_offset).
    limit: float = 0.0
    alpha: float = 1.702
    up_offset: float = 1.0
    # ``bias``: the three projections have biases, named like the matrices with ``bias_suffix`` behind.
    bias: bool = False
    bias_suffix: str = ".b"


@dataclass(frozen=True)
class RoutedMLPSpec(PartSpec):
    """Mixture of ``experts`` gated feed-forwards (tensors e0.., each gate, up, down, no biases) of which a token uses
    the ``top`` with the largest router logits (tensor ``router``, fp32), weighted by the softmax over those logits
    alone.  An expert: g = min(W_gate h, limit), u = clamp(W_up h, -limit, limit), W_down (g sigmoid(alpha g) (u + 1))."""

    kind: ClassVar[str] = "routed_mlp"
    hidden_size: int = 0
    intermediate_size: int = 0
    experts: int = 0
    top: int = 0
    limit: float = 7.0
    alpha: float = 1.702
    # ``limit`` 0: no clamps.  ``up_offset``: what is added to the (clamped) up projection, so that limit 0, alpha 1
    # and up_offset 0 give silu(W_gate h) * W_up h.
    up_offset: float = 1.0
    # ``scoring`` "softmax_top" as above, or "sigmoid": scores s = sigmoid(logits); the choice is by s + correction
    # (tensor ``correction`` [experts], if ``correction``), the weights are the chosen experts' s times
    # ``route_scale``, divided by their sum if ``renormalize``.
    scoring: str = "softmax_top"
    correction: bool = False
    route_scale: float = 1.0
    renormalize: bool = False
    # ``scoring`` "softmax": s = softmax(logits) over all router outputs, otherwise like "sigmoid".
    # ``groups`` > 0: the router's outputs form that many equal groups of neighbours; a group's score is its largest
    # s + correction, and only outputs of the ``keep_groups`` best groups can be chosen.
    groups: int = 0
    keep_groups: int = 0
    # ``identity`` > 0: the router has ``experts`` + ``identity`` outputs; the last ``identity`` are experts without
    # tensors whose output is the token's input itself (times the weight).
    identity: int = 0
    # ``expert`` "gated" as above, or "square_relu": W_down relu(W_up h)^2, tensors e<i>.up and e<i>.down only.
    expert: str = "gated"


# ---------------------------------------------------------------------- connections
@dataclass(frozen=True)
class HyperConnectionSpec(PartSpec):
    """How a sublayer reads from and writes to ``streams`` copies x_1 .. x_s of the residual stream: its input is
    u = sum_s in[s] x_s, and with its result y all streams change at once from the old ones,
    x_t <- sum_s mix[s, t] x_s + multiplier * out[t] * (scale * y) (``mix`` is indexed [from, to]; ``scale`` a vector over
    the width, element by element, if ``layer_scale``).  Tensors: prefix + ``name`` + ".in" [s], ".out" [s], ".mix"
    [s, s], and prefix + ``scale_name`` [size].  ``learned`` False: no tensors, in = out = 1 and mix the identity (with
    one stream, the plain residual sum x <- x + multiplier * scale * y)."""

    kind: ClassVar[str] = "hyper"
    size: int = 0
    streams: int = 1
    multiplier: float = 1.0
    layer_scale: bool = False
    learned: bool = True
    name: str = "hc"
    scale_name: str = "ls"


# ---------------------------------------------------------------------------- layers
@dataclass(frozen=True)
class LayerSpec:
    """One block: the name of its arrangement (a registered class) and the parts that arrangement puts around the
    residual stream, each under a *role*: ``(role, part spec, weight-name prefix)``.  Which roles exist, which
    family each belongs to and in what order they run is the arrangement's business ("prenorm" knows
    ``mixer_norm``, ``mixer``, ``feed_forward_norm``, ``feed_forward``); a block with four norms, with two mixers
    or without a feed-forward is another arrangement over another set of roles, not another ``LayerSpec``."""

    arrangement: str = "prenorm"
    parts: Tuple[Tuple[str, PartSpec, str], ...] = ()
    # numbers that belong to the arrangement itself and to none of its parts, by name (a post-norm layer's multiplier
    # of the stream, for instance)
    constants: Tuple[Tuple[str, float], ...] = ()

    def __post_init__(self):
        roles = [r for r, _, _ in self.parts]
        if len(set(roles)) != len(roles):
            raise ConfigError(f"a layer names a role twice: {roles}")

    def roles(self) -> Tuple[str, ...]:
        return tuple(r for r, _, _ in self.parts)

    def constant(self, name: str, default: float) -> float:
        for n, v in self.constants:
            if n == name:
                return float(v)
        return float(default)

    def part(self, role: str) -> Tuple[PartSpec, str]:
        for r, spec, prefix in self.parts:
            if r == role:
                return spec, prefix
        raise ConfigError(f"the layer has no part in the role {role!r} (it has: {', '.join(self.roles()) or 'none'})")

    @classmethod
    def prenorm(cls, mixer: PartSpec, feed_forward: PartSpec, mixer_norm: PartSpec, feed_forward_norm: PartSpec,
                mixer_prefix: str, feed_forward_prefix: str, mixer_norm_prefix: str,
                feed_forward_norm_prefix: str) -> "LayerSpec":
        """h += mixer(norm(h)); h += feed_forward(norm(h)): prefixes are, for instance, "model.layers.3.self_attn.",
        "model.layers.3.mlp.", "model.layers.3.input_layernorm.", "model.layers.3.post_attention_layernorm."."""
        return cls("prenorm", (("mixer_norm", mixer_norm, mixer_norm_prefix), ("mixer", mixer, mixer_prefix),
                               ("feed_forward_norm", feed_forward_norm, feed_forward_norm_prefix),
                               ("feed_forward", feed_forward, feed_forward_prefix)))


@dataclass(frozen=True)
class ScheduleEntry:
    """One position in the run order.  ``layer`` indexes ``ModelSpec.layers``; a layer
    may appear more than once.  ``cache_of`` names the layer whose cache this run
    reads and writes; -1 means its own.  ``instance`` tells the caches of one layer apart: a layer
    that runs several times with the same weights (a loop) keeps one cache or state per pass."""

    layer: int
    cache_of: int = -1
    instance: int = 0


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    final_norm_prefix: str = "model.norm."
    embedding_name: str = "model.embed_tokens.weight"
    head_name: str = "lm_head.weight"
    tie_embeddings: bool = False
    head_optional: bool = True            # untied but absent in the file => use the embedding
    max_positions: int = 4096
    eos_ids: Tuple[int, ...] = ()
    init_std: float = 0.02                # random-weights mode: std of linear weights
    init_norm_std: float = 0.05           # random-weights mode: norm weights are 1 + N(0, this)
    # a position encoding that acts on the embedded tokens (learned or sinusoidal tables); rotary ones
    # belong to their mixer's spec instead
    embedding_position: PartSpec = field(default_factory=NoPositionSpec)
    embedding_position_prefix: str = "model.embed_positions."
    # h = embedding_multiplier * table[token] and logits = logit_scale * (norm(h) . head^T): 1.0 for Qwen3; other
    # decoders scale the embedded tokens by sqrt(hidden) or the logits by a constant
    embedding_multiplier: float = 1.0
    logit_scale: float = 1.0
    # a norm on the embedded (and scaled) tokens, before the first layer
    embedding_norm: Optional[PartSpec] = None
    embedding_norm_prefix: str = "model.embed_norm."
    # logits <- cap * tanh(logits / cap), after the logit scale (which is then applied to the fp32 logits themselves, not
    # folded into the final norm); 0: none
    logit_softcap: float = 0.0
    # the residual stream in ``residual_streams`` copies (hyper-connections): all equal to the embedding's output at the
    # start, read and written by the layers' connections, summed before the final norm
    residual_streams: int = 1

    def __post_init__(self):
        n = len(self.layers)
        if n == 0:
            raise ConfigError("a model needs at least one layer")
        if not self.schedule:
            raise ConfigError("the layer schedule is empty")
        for e in self.schedule:
            if not (0 <= e.layer < n):
                raise ConfigError(f"schedule names layer {e.layer}; the model has {n}")
            if not (-1 <= e.cache_of < n):
                raise ConfigError(f"schedule entry reads the cache of layer {e.cache_of}; the model has {n}")
            if e.instance < 0:
                raise ConfigError("a schedule entry's cache instance cannot be negative")
        if self.residual_streams < 1:
            raise ConfigError("a model has at least one residual stream")


def default_schedule(n_layers: int) -> Tuple[ScheduleEntry, ...]:
    return tuple(ScheduleEntry(i) for i in range(n_layers))
