"""Descriptions of a model as data: parts, layers, their order, and the head.

An architecture turns its typed configuration into one ``ModelSpec``.  Every
size and constant a part needs is a field of that part's spec; no part reads
the model's configuration or knows which model it is in.  Layers may differ
from one another (each ``LayerSpec`` names its own mixer and feed-forward),
and the order in which layers run is a list of ``ScheduleEntry`` which may
name a layer twice or let a layer read the cache another run wrote.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple


@dataclass(frozen=True)
class NormSpec:
    """RMSNorm: ``y = x / sqrt(mean(x^2) + eps) * weight`` (``src/layers/rmsnorm.cpp:63-97``)."""
    size: int
    eps: float
    weight: str                      # tensor name
    kind: str = "rmsnorm"
    # added to the stored weight when it is loaded: 1.0 for checkpoints that keep a norm's weight as its distance
    # from one (``y = x / rms * (1 + w)``)
    weight_offset: float = 0.0


@dataclass(frozen=True)
class RopeSpec:
    """Rotary position encoding with split-half pairing (``src/layers/attention.cpp:96-135``)."""
    head_dim: int
    theta: float
    kind: str = "rope_half"


@dataclass(frozen=True)
class YarnSpec:
    """Rotary frequencies stretched for contexts longer than the ``original`` one (YaRN).  With
    ``pair(t) = dims ln(original / (2 pi t)) / (2 ln base)``, ``lo = max(floor(pair(fast)), 0)``,
    ``hi = min(ceil(pair(slow)), dims - 1)`` and ``ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1)``, pair i turns
    at ``f_i / factor * ramp_i + f_i (1 - ramp_i)``, and cosines and sines are multiplied by ``0.1 ln(factor) + 1``."""
    factor: float
    original: int
    fast: float
    slow: float


@dataclass(frozen=True)
class RotarySpec:
    """Rotary positions on the first ``dims`` numbers of a vector (the rest pass), number i paired with number
    ``i + dims/2``: ``(u, v) -> (u cos a - v sin a, v cos a + u sin a)``, ``a = position * base^(-2i/dims)``;
    ``scaling`` changes the frequencies (``YarnSpec``).  ``interleaved``: pair i is numbers ``2i`` and ``2i + 1``
    instead (mixers whose kernels know both layouts read it; the table is the same)."""
    dims: int
    base: float
    scaling: Optional[YarnSpec] = None
    kind: str = "rotary_table"
    interleaved: bool = False


@dataclass(frozen=True)
class DistanceBiasSpec:
    """A bias on attention scores that grows with the logarithm of the distance: query i and key j score
    ``(q.k) * scale - r1[h] * ln(1 + r2[h] * (i - j))`` with two learned numbers per head."""
    r1: str                          # tensor names, each [num_heads]
    r2: str
    max_distance: int = 0            # the longest distance a model can reach (its positions); 0: unknown
    kind: str = "log_distance"


@dataclass(frozen=True)
class QueryTemperatureSpec:
    """Queries grow with the position: those at position p are multiplied by
    ``1 + coef * ln(floor((p + 1) / every) + 1)``."""
    coef: float
    every: int


@dataclass(frozen=True)
class AttentionSpec:
    """Causal grouped-query attention over a paged cache (``src/layers/attention.cpp:153-342``).

    The fields after ``window`` are mechanisms that a design may add, each off by default: a value head
    size of its own (``v_head_dim``), biases on the three projections, an RMS norm without weight on every
    value head before it is cached (``value_norm_eps``), a bias on the scores by distance, and a gate per
    head on the attention output, ``sigmoid(h . gate_weight[head])``, read from the mixer's own input
    (``gate_per_element``: a gate for every number of the output, ``gate_weight`` ``[heads * value size, hidden]``).
    ``qk_norm_eps``: every query and key head is divided by its root mean square (no weight) before the key is
    cached.  ``q_temperature``: see ``QueryTemperatureSpec``.  ``softcap`` c > 0: scores become
    ``c * tanh(score / c)`` before the softmax.  ``shares_kv``: the mixer has no key and value projections and
    attends over the cache entry that another layer's run wrote (its schedule entry names that entry and does
    not write it).  ``q_norm_weight`` / ``k_norm_weight`` (tensor names, ``[heads * head_dim]`` and
    ``[kv_heads * head_dim]``) with ``projection_norm_eps``: one RMS norm with that weight over ALL query heads
    together, and one over all key heads, after the biases and before the heads are split."""
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    scale: float                     # multiplies q.k after the dot product
    position: Optional[RopeSpec]
    q_weight: str
    k_weight: str
    v_weight: str
    o_weight: str
    window: int = 0                  # 0: every earlier key; w > 0: the last w keys only
    kind: str = "attention"
    v_head_dim: int = 0              # 0: values as wide as keys
    q_bias: Optional[str] = None     # tensor names
    k_bias: Optional[str] = None
    v_bias: Optional[str] = None
    value_norm_eps: Optional[float] = None
    distance_bias: Optional[DistanceBiasSpec] = None
    gate_weight: Optional[str] = None     # [num_heads, hidden_size]
    gate_per_element: bool = False
    qk_norm_eps: Optional[float] = None
    q_temperature: Optional[QueryTemperatureSpec] = None
    softcap: float = 0.0
    shares_kv: bool = False
    q_norm_weight: Optional[str] = None
    k_norm_weight: Optional[str] = None
    projection_norm_eps: float = 0.0

    @property
    def value_dim(self) -> int:
        return self.v_head_dim or self.head_dim

    @property
    def extended(self) -> bool:
        """True if any mechanism beyond rotated, unbiased queries, keys and values of one width is in use."""
        return bool(self.v_head_dim and self.v_head_dim != self.head_dim or self.q_bias or self.k_bias
                    or self.v_bias or self.value_norm_eps is not None or self.distance_bias or self.gate_weight
                    or self.qk_norm_eps is not None or self.q_temperature or self.softcap or self.shares_kv
                    or self.q_norm_weight or self.k_norm_weight)


@dataclass(frozen=True)
class LatentAttentionSpec:
    """Causal attention whose keys and values are up-projections of one compressed vector per position.

    ``c = rmsnorm(Wdkv h) * latent_norm`` (``latent_dim`` numbers) is all the cache keeps; head h has
    ``k = Wuk[h] c`` (``head_dim``) and ``v = Wuv[h] c`` (``v_head_dim``), ``score = (q . k) * scale``, no position
    encoding; ``x += Wo (heads' outputs)``.

    Mechanisms a design may add, each off by default.  ``rope_dim`` r > 0 with ``rope``: a query head is
    ``[head_dim unrotated | r rotated]`` numbers, the down projection has r more rows, which (not normed, rotated) are
    one key part that all heads share and that is cached behind the latent; the score adds the two parts' products.
    ``sink``: a learned number per head whose exponential counts once in the softmax's denominator (no key, no value,
    not scaled).  ``gate_weight`` ``[heads, hidden]``: a head's output times ``sigmoid(gate_weight[head] . h)``.
    ``shares_kv``: no down projection of its own; the layer attends over the cache entry another layer's run wrote
    (its schedule entry names that entry and does not write it)."""
    hidden_size: int
    num_heads: int
    head_dim: int
    v_head_dim: int
    latent_dim: int
    scale: float
    eps: float                       # of the latent's norm
    q_weight: str                    # [heads * head_dim, hidden]
    down_weight: str                 # [latent_dim, hidden]
    latent_norm: str                 # [latent_dim]
    k_up_weight: str                 # [heads * head_dim, latent_dim]
    v_up_weight: str                 # [heads * v_head_dim, latent_dim]
    o_weight: str                    # [hidden, heads * v_head_dim]
    kind: str = "latent_attention"
    rope_dim: int = 0
    rope: Optional[RotarySpec] = None
    sink: Optional[str] = None            # [heads]
    gate_weight: Optional[str] = None     # [heads, hidden]
    shares_kv: bool = False


@dataclass(frozen=True)
class RetentionSpec:
    """Linear attention with a fixed decay per head and no softmax: ``q, k = rot(Wq h), rot(Wk h) * head_dim^-1/2``,
    ``v = Wv h``; per head ``S_t = decay S_(t-1) + k_t v_t^T`` (``head_dim x v_head_dim`` floats a sequence keeps),
    ``o_t = S_t^T q_t``; every head of o divided by its root mean square (``eps``), the heads times
    ``silu(Wg h)``, then ``Wo``."""
    hidden_size: int
    num_heads: int
    head_dim: int
    v_head_dim: int
    decay: Tuple[float, ...]         # per head
    eps: float
    rope: Optional[RotarySpec]
    q_weight: str                    # [heads * head_dim, hidden]
    k_weight: str
    v_weight: str                    # [heads * v_head_dim, hidden]
    gate_weight: str                 # [heads * v_head_dim, hidden]
    o_weight: str                    # [hidden, heads * v_head_dim]
    kind: str = "retention"


@dataclass(frozen=True)
class ConvAttentionSpec:
    """Causal grouped-query attention whose queries and keys pass a short convolution over time before they are
    rotated: ``q, k = conv(Wq h + bq), conv(Wk h + bk)`` with ``conv(u)_p = sum_j w[:, j] u_(p - taps + 1 + j)`` per
    channel (zeros before the sequence; the biased projections of the last ``taps - 1`` positions are state a sequence
    keeps); rotary positions (``rope``) on queries and keys; ``values_are_keys``: there is no value projection and the
    values are the convolved keys before rotation; ``score = (q . k) scale`` over the last ``window`` keys (0: all);
    ``sink``: a learned number per head whose exponential counts once in the softmax's denominator; ``Wo`` on the
    heads.  ``taps`` 0: no convolution."""
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    scale: float
    q_weight: str                    # [heads * head_dim, hidden]
    k_weight: str                    # [kv_heads * head_dim, hidden]
    o_weight: str                    # [hidden, heads * head_dim]
    taps: int = 0
    q_conv: Optional[str] = None     # [heads * head_dim, taps], the last column weighs the current token
    k_conv: Optional[str] = None     # [kv_heads * head_dim, taps]
    q_bias: Optional[str] = None
    k_bias: Optional[str] = None
    rope: Optional[RotarySpec] = None
    window: int = 0
    sink: Optional[str] = None       # [heads]
    values_are_keys: bool = True
    kind: str = "conv_attention"


@dataclass(frozen=True)
class TimeMixSpec:
    """Time mixing with a matrix state per head and a decay per token and key channel (the RWKV family).  With h' the
    token before's input (zeros for the first), every projection s of r, k, v, g, w reads ``h + (h' - h) mu_s``;
    ``r, k, v = Wr., Wk., Wv.`` (heads x head_dim), ``gate = silu(Wg.)``, ``w = exp(-exp(W2 tanh(W1 .) + w0))`` per head
    and key channel; per head ``o_t = (S_(t-1) + diag(u) k_t v_t^T)^T r_t`` and ``S_t = diag(w_t) S_(t-1) + k_t v_t^T``
    (S float32, zero before the first token); every head of o divided by its root mean square (``eps``), times
    ``norm``, times the gate, then ``Wo``."""
    hidden_size: int
    num_heads: int
    head_dim: int
    decay_rank: int
    eps: float
    mix: Tuple[str, str, str, str, str]   # the mu tensors of r, k, v, g, w, each [hidden]
    r_weight: str                    # [heads * head_dim, hidden]
    k_weight: str
    v_weight: str
    g_weight: str
    w1_weight: str                   # [decay_rank, hidden]
    w2_weight: str                   # [heads * head_dim, decay_rank]
    w0: str                          # [heads * head_dim]
    bonus: str                       # u, [heads, head_dim]
    norm: str                        # [heads * head_dim]
    o_weight: str                    # [hidden, heads * head_dim]
    kind: str = "time_mix"


@dataclass(frozen=True)
class MixerPairSpec:
    """Two mixers side by side on the same input: ``left_scale * left(h) + right_scale * right(h)``.  Either side is
    any mixer's spec; one cache entry serves both (the left one's pages, and both sides' per-sequence state one after
    the other)."""
    left: Any
    right: Any
    left_scale: float = 1.0
    right_scale: float = 1.0
    kind: str = "mixer_pair"


@dataclass(frozen=True)
class RgLruSpec:
    """A recurrent block around a real-gated linear recurrent unit (the Griffin block): two branches of
    ``channels`` numbers, ``y = gelu_tanh(Wy h + by)`` and ``u = conv(Wx h + bx)`` (causal, per channel, ``taps``
    wide); per equal part of the channels ``r = sigmoid(Ra u + ba)``, ``i = sigmoid(Ri u + bi)``;
    ``a = exp(-8 r softplus(lam))``, ``S <- a S + sqrt(1 - a^2) i u``; ``x += Wo (S * y)``."""
    hidden_size: int
    channels: int
    parts: int                       # the gates' matrices are block-diagonal with this many blocks
    taps: int
    y_weight: str
    y_bias: str
    x_weight: str
    x_bias: str
    conv_weight: str                 # [channels, taps], the last column weighs the current token
    conv_bias: str
    r_weight: str                    # [parts, channels / parts, channels / parts], rows are outputs
    r_bias: str                      # [parts, channels / parts]
    i_weight: str
    i_bias: str
    decay: str                       # lam, [channels]
    o_weight: str
    kind: str = "rglru"


@dataclass(frozen=True)
class TokenSideSpec:
    """An input that depends on the token, added to the stream at the end of a layer:
    ``e = table[token, offset : offset + dim]``, ``g = gelu_tanh(gate x) * e``, ``y = proj g``,
    ``x += rmsnorm(y) * norm`` (a plain-weight RMS norm with ``eps``).  ``table`` is one tensor for all layers."""
    hidden_size: int
    vocab_size: int
    dim: int
    offset: int
    table_width: int
    eps: float
    table: str
    gate_weight: str                 # [dim, hidden]
    proj_weight: str                 # [hidden, dim]
    norm_weight: str                 # [hidden]
    kind: str = "token_side"


@dataclass(frozen=True)
class GatedMlpSpec:
    """``down(act(gate(x)) * up(x))`` (``src/models/transformer_block.cpp:312-325``)."""
    hidden_size: int
    intermediate_size: int
    activation: str                  # "silu", "gelu_tanh", or "swiglu_clamp" (takes ``activation_param``)
    gate_weight: str
    up_weight: str
    down_weight: str
    kind: str = "gated_mlp"
    activation_param: float = 0.0    # "swiglu_clamp": both branches are clamped to it (ops.PARAMETRIC_ACTIVATIONS)


@dataclass(frozen=True)
class MlpSpec:
    """A feed-forward without a gate: ``down(act(up(x)))``."""
    hidden_size: int
    intermediate_size: int
    activation: str                  # "relu2" (the square of relu), "gelu_tanh", "silu"
    up_weight: str
    down_weight: str
    kind: str = "mlp"


@dataclass(frozen=True)
class SharedExpertSpec:
    """An expert every token uses; ``gate_weight`` ``[1, hidden]``: its result times ``sigmoid(gate_weight . h)``."""
    intermediate_size: int
    up_weight: str
    down_weight: str
    gate_weight: Optional[str] = None


@dataclass(frozen=True)
class RoutedMlpSpec:
    """A mixture of ``experts`` feed-forwards ``down_e act(up_e h)`` of which a token uses ``top``: router scores
    ``s = sigmoid(router h)`` in float32; the ``top`` largest ``s + correction`` choose; the chosen experts' results
    are added with weights ``s * route_scale`` (``renormalize``: divided by their sum first).  ``up_weights`` and
    ``down_weights`` name one tensor per expert."""
    hidden_size: int
    intermediate_size: int
    experts: int
    top: int
    activation: str
    route_scale: float
    router_weight: str               # [experts, hidden]
    up_weights: Tuple[str, ...]      # each [intermediate, hidden]
    down_weights: Tuple[str, ...]    # each [hidden, intermediate]
    correction: Optional[str] = None # [experts], added to the scores that choose only
    renormalize: bool = False
    shared: Optional[SharedExpertSpec] = None
    kind: str = "routed_mlp"
    # gated experts: ``down_e (act(gate_e h) * (up_e h))``, one more tensor per expert
    gate_weights: Optional[Tuple[str, ...]] = None
    score: str = "sigmoid"           # or "softmax": the scores are a softmax over all experts
    # the experts form ``groups`` equal groups of neighbours; a group scores what its best expert does, and only
    # experts of the ``keep_groups`` best groups can be chosen (0: no groups)
    groups: int = 0
    keep_groups: int = 0
    renormalize_eps: float = 0.0     # added to the chosen scores' sum before ``renormalize`` divides by it


@dataclass(frozen=True)
class StreamMixSpec:
    """How one sublayer is connected to ``streams`` copies of the residual stream (hyper-connections): it reads
    ``sum_s read[s] x_s``, and every stream becomes ``x_t <- sum_s mix[s, t] x_s + write[t] * result``, all from the
    old ones.  Without tensor names the connection is the plain residual sum (read 1, mix 1, write 1)."""
    streams: int
    read: Optional[str] = None       # [streams]
    write: Optional[str] = None      # [streams]
    mix: Optional[str] = None        # [streams, streams], indexed [from, to]
    kind: str = "stream_mix"


@dataclass(frozen=True)
class LayerSpec:
    """One block: which norm, mixer and feed-forward, and how they are arranged.

    ``pre_norm``: ``x += mixer(norm1(x)); x += ffn(norm2(x))``
    (``src/models/transformer_block.cpp:301-331``).
    ``parallel``: ``h = norm1(x); x += mixer(h) + ffn(h)``: one norm (``mixer_norm``), both branches read its
    output; ``ffn`` may be ``None``.
    ``sandwich``: ``x += post1(mixer(norm1(x))); x += post2(ffn(norm2(x)))``, then ``token_input`` if the layer
    has one; the norms after the sublayers are the extras ``mixer_post_norm`` and ``ffn_post_norm``, ``ffn`` (with
    its two norms) may be ``None``.
    ``multi_stream``: the ``pre_norm`` block over several copies of the stream; the extras ``mixer_streams`` and
    ``ffn_streams`` (``StreamMixSpec``) say how each sublayer reads and writes them; ``ffn`` may be ``None``.
    ``parallel_pair``: ``x += mixer(norm1(x)) + ffn(norm2(x))``, both norms of the same x, then ``token_input`` if the
    layer has one; ``ffn`` (with its norm) may be ``None``.

    The four named places are what that arrangement uses; another arrangement may leave
    some of them ``None`` (a block without a feed-forward, one norm for two branches) and
    may name further parts in ``extras`` as ``(name, role, spec)``, which the layer builds
    and hands to the arrangement as ``layer.extra[name]``.
    """
    mixer_norm: Any
    mixer: Any
    ffn_norm: Any = None
    ffn: Any = None
    arrangement: str = "pre_norm"
    extras: Tuple[Tuple[str, str, Any], ...] = ()

    def named_parts(self):
        """``(name, role, spec)`` of every part this layer has, in a fixed order."""
        places = (("mixer_norm", "norm", self.mixer_norm), ("mixer", "mixer", self.mixer),
                  ("ffn_norm", "norm", self.ffn_norm), ("ffn", "ffn", self.ffn))
        return tuple(place for place in places if place[2] is not None) + tuple(self.extras)


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.  ``cache`` is the index of the cache entry the run's
    mixer uses; ``writes_cache`` false means it only reads what another run wrote.
    ``adds_embedding``: the embedding's output is added to the stream once more right before this run (a model that
    runs some of its layers several times in a row feeds its input to every pass)."""
    layer: int
    cache: int
    writes_cache: bool = True
    adds_embedding: bool = False


@dataclass(frozen=True)
class EmbeddingSpec:
    vocab_size: int
    hidden_size: int
    weight: str
    kind: str = "embedding"
    scale: float = 1.0               # the table's rows times this


@dataclass(frozen=True)
class HashedPairSpec:
    """A second embedding table indexed by a hash of two neighbouring tokens: row
    ``(previous * mul_prev + current * mul_cur) mod buckets``; a sequence's first token reads row ``buckets``,
    the table's last."""
    buckets: int
    mul_prev: int
    mul_cur: int
    weight: str                      # [buckets + 1, hidden_size]


@dataclass(frozen=True)
class LearnedPositionSpec:
    """A learned vector per position, added to the embedding times ``scale``."""
    max_positions: int
    weight: str                      # [max_positions, hidden_size]
    scale: float = 1.0


@dataclass(frozen=True)
class SummedEmbeddingSpec:
    """``x = table[token] (+ pair table row) (+ position vector)``, summed in float."""
    vocab_size: int
    hidden_size: int
    weight: str
    pair: Optional[HashedPairSpec] = None
    positions: Optional[LearnedPositionSpec] = None
    kind: str = "summed_embedding"


@dataclass(frozen=True)
class HeadSpec:
    """Final norm on the wanted rows, then ``logits = y . W^T`` (``src/generation/generator.cpp:773-774``)
    times ``logit_scale``.  ``weight`` may be the embedding table's name (tied)."""
    vocab_size: int
    hidden_size: int
    weight: str
    kind: str = "linear_head"
    logit_scale: float = 1.0


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    embedding: EmbeddingSpec
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: Any
    head: HeadSpec
    stop_token_ids: Tuple[int, ...] = ()
    max_positions: int = 0
    # True if a table holds the positions (learned vectors): no sequence may pass ``max_positions`` then,
    # whatever the engine is told.
    positions_are_tabled: bool = False
    # Tensor names a checkpoint may carry that the model does not use.
    ignorable: Tuple[str, ...] = ()

    def num_cache_entries(self) -> int:
        return 1 + max((e.cache for e in self.schedule), default=-1)
