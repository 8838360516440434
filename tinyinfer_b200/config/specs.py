"""Typed descriptions of the parts a decoder is put together from.

A *spec* is plain data: the sizes and constants of one part and a ``kind`` string that a
registry of ``tinyinfer_b200.parts`` maps to the class that runs it. An architecture's
configuration (``tinyinfer_b200.config.qwen3``) turns the keys of its ``config.json`` into one
``ModelSpec``; nothing downstream reads ``config.json`` again, and no part knows which
architecture asked for it.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple


@dataclass(frozen=True)
class NormSpec:
    """A normalisation over the last axis. ``kind='rmsnorm'``: w * x * rsqrt(mean(x^2) + eps)."""
    size: int
    eps: float
    kind: str = "rmsnorm"
    tensor: str = "weight"                  # local name of the weight behind the norm's prefix ('' : the prefix itself)
    offset: float = 0.0                     # the stored weight is added to this (1.0: a weight stored around zero)


@dataclass(frozen=True)
class FrequencyBlend:
    """Stretches a rotary encoding beyond the length it was made for (the YaRN recipe): with
    pair(t) = rotary_dim * ln(original / (2 pi t)) / (2 ln theta), the pair index that makes t full turns over
    ``original`` positions, lo = max(floor(pair(fast)), 0), hi = min(ceil(pair(slow)), rotary_dim - 1) and
    ramp_j = clamp((j - lo) / max(hi - lo, 0.001), 0, 1), pair j turns at f_j / factor * ramp_j + f_j * (1 - ramp_j),
    and every cosine and sine is multiplied by 0.1 * ln(factor) + 1."""
    factor: float
    original: int
    fast: float
    slow: float


@dataclass(frozen=True)
class PositionSpec:
    """How positions enter a mixer. ``kind='rope'``: rotation of the first ``rotary_dim`` features of every head
    with inv_freq[j] = theta ** (-2j / rotary_dim), in pairs (j, j + rotary_dim / 2) or, ``interleaved``,
    (2j, 2j + 1). ``kind='none'``: positions are not used."""
    kind: str = "rope"
    theta: float = 10000.0
    rotary_dim: int = 0
    exact_frequencies: bool = False         # inv_freq worked out in float64 and rounded once (default: in float32)
    interleaved: bool = False
    blend: Optional[FrequencyBlend] = None  # frequencies slowed down for lengths beyond the original one


@dataclass(frozen=True)
class AttentionSpec:
    """Grouped-query softmax attention over a paged key/value cache."""
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    scale: float
    position: PositionSpec
    qk_norm: Optional[NormSpec] = None      # per-head norm of q and k before the rotation
    bias: bool = False                      # bias on the q, k, v and o projections
    window: Optional[int] = None            # None: all keys; n: the last n keys (itself included)
    kind: str = "attention"
    v_dim: Optional[int] = None             # size of a value head (None: head_dim)
    head_sinks: bool = False                # a learned logit per query head joins the softmax denominator, without a value
    head_gate: bool = False                 # head h's output is multiplied by sigmoid(W_g x)_h, one number per head
    shares_cache: bool = False              # no key/value tensors: the layer reads the keys and values another layer caches
    short_names: bool = False               # tensors are 'q', 'k', 'v', 'o', 'q.norm', 'k.norm', 'sink', 'g'
    qkv_bias: bool = False                  # biases on q, k and v alone (the tensor's name with '.b' added), none on o
    softcap: Optional[float] = None         # a score s becomes softcap * tanh(s / softcap) before the softmax
    qk_unit_norm: Optional[float] = None    # eps: q and k are divided by their root mean square per head (no weight)
                                            # AFTER the rotation

    @property
    def q_size(self) -> int:
        return self.num_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_kv_heads * self.head_dim

    @property
    def value_dim(self) -> int:
        return self.head_dim if self.v_dim is None else self.v_dim


@dataclass(frozen=True)
class GatedMLPSpec:
    """Dense gated feed-forward: down(act(gate(x)) * up(x)), no bias."""
    hidden_size: int
    intermediate_size: int
    activation: str = "silu"
    kind: str = "gated_mlp"
    names: Tuple[str, str, str] = ("gate_proj.weight", "up_proj.weight", "down_proj.weight")    # gate, up, down


@dataclass(frozen=True)
class LatentAttentionSpec:
    """Softmax attention whose keys and values are linear maps of one cached low-rank latent per token, with the
    queries through a latent of their own. Per head ``head_dim`` unrotated and ``rot_dim`` rotated query/key
    features (the rotated key part is one vector shared by all heads) and ``v_dim`` value features.
    ``sink``: a learned number per head whose exponential joins the softmax denominator.
    ``shares_cache``: the layer has no key/value down projection and reads the rows another layer caches."""
    hidden_size: int
    num_heads: int
    head_dim: int
    rot_dim: int
    v_dim: int
    q_rank: int
    kv_rank: int
    scale: float
    position: PositionSpec
    norm_eps: float
    sink: bool = False
    shares_cache: bool = False
    window: Optional[int] = None
    kind: str = "latent_attention"
    output_gate: bool = False               # the heads side by side are multiplied by sigmoid(W_g h), feature by feature
    # q_rank 0: the queries have no latent: q = W_q h (tensor "q") in place of "dq", "dq.norm" and "uq"


@dataclass(frozen=True)
class GatedRecurrenceSpec:
    """Recurrent block: out = W_o (S * gelu_tanh(W_y h + b)), S the state of a real-gated diagonal linear
    recurrence a = exp(-decay * r * softplus(lam)) driven by a causal per-channel convolution of W_x h + b;
    the gates r and i are block-diagonal maps (``blocks`` square blocks) of the convolution's output."""
    hidden_size: int
    width: int
    blocks: int
    conv_taps: int
    decay: float = 8.0
    kind: str = "gated_recurrence"


@dataclass(frozen=True)
class ExpertsSpec:
    """Mixture of experts: every token runs the ``top`` experts with the largest softmax scores, weighted by
    those scores over their sum (+ ``weight_eps``); an expert is down(act(up h)) without biases.
    ``shared_size`` > 0: one more expert of that inner size runs for every token and is added."""
    hidden_size: int
    num_experts: int
    top: int
    expert_size: int
    shared_size: int = 0
    activation: str = "relu_squared"
    weight_eps: float = 1e-20
    kind: str = "experts"
    # activation 'clamped_glu': an expert is down(g * sigmoid(glu_alpha * g) * (u + 1)) with g = min(gate h, glu_limit)
    # and u = clamp(up h, -glu_limit, glu_limit)
    glu_limit: float = 0.0
    glu_alpha: float = 1.702
    identity_experts: int = 0               # the router has this many outputs more: experts whose output is their input
    score_correction: bool = False          # a learned number per router output is added to the scores for the CHOICE only
    renormalize: bool = True                # False: the weights are the chosen scores themselves, not divided by their sum
    router_input: str = "stream"            # 'stream': the router reads the float32 residual; 'input': the sublayer's input
    # activation 'silu_glu': an expert is down(silu(gate h) * (up h))
    scoring: str = "softmax"                # 'sigmoid': an expert's score is the sigmoid of its own router logit
    weight_input: bool = False              # the weight multiplies what the expert READS (expert(w h)), not its output


@dataclass(frozen=True)
class ConvAttentionSpec:
    """Grouped-query softmax attention without a rotation, whose q, k and v pass a short causal convolution over
    time (``conv_taps`` taps per channel; one tap is a weight per channel; 0: no convolution) right after their
    projections. Keys have ``head_dim`` features,
    values ``v_dim``. ``query_temperature`` (coef, every): the query at position p is multiplied by
    1 + coef * ln(floor((p + 1) / every) + 1). ``sink``: a logit whose exponential joins the softmax denominator
    without a value (0.0 adds one to the sum of exp(score)); None: the ordinary softmax."""
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    v_dim: int
    scale: float
    conv_taps: int = 0
    query_temperature: Optional[Tuple[float, int]] = None
    sink: Optional[float] = None
    bias: bool = True
    window: Optional[int] = None
    kind: str = "conv_attention"


@dataclass(frozen=True)
class GatedLinearAttentionSpec:
    """Linear attention with a matrix state per head and a decay per key channel: S <- diag(a) S + k v^T,
    o = S^T q, a = sigmoid(W_a2 W_a1 h + b)^(1 / tau); q is scaled by ``key_dim`` ** -0.5. Each head's o is divided
    by its root mean square, weighted by one weight shared by the heads, gated by silu(W_g h) and projected.
    ``gate_rank``: the inner size of the decay's two projections; 0: whatever the checkpoint's tensors have."""
    hidden_size: int
    num_heads: int
    key_dim: int
    value_dim: int
    tau: float
    norm_eps: float
    gate_rank: int = 0
    kind: str = "gated_linear_attention"


@dataclass(frozen=True)
class RetentionSpec:
    """Linear attention with a fixed decay per head and no softmax or denominator: S <- decays[h] S + k v^T,
    o = S^T q per head, q and k rotated by their positions (``position``), k scaled by ``key_dim`` ** -0.5 after the
    rotation. Each head's o is divided by its root mean square (no weight), the heads side by side are multiplied by
    silu(W_g h) and projected."""
    hidden_size: int
    num_heads: int
    key_dim: int
    value_dim: int
    decays: Tuple[float, ...]
    position: PositionSpec
    norm_eps: float
    kind: str = "retention"


@dataclass(frozen=True)
class ChannelDeltaSpec:
    """The gated delta rule with a decay per head and key channel. q and k (``num_kv_heads`` heads of ``key_dim``) and v
    (``num_heads`` heads of ``value_dim``) pass a causal convolution of ``conv_taps`` taps per channel and silu; q and
    k become unit vectors per head (x / sqrt(sum x^2 + ``unit_eps``)), q also times key_dim ** -0.5;
    beta = sigmoid(W_b h) per head; g = exp(-exp(A_log[h]) softplus(W_a2 W_a1 h + dt_bias)) per head and key channel;
    S <- diag(g) S, u = beta (v - S^T k), S <- S + k u^T, o = S^T q. Each head's o is divided by its root mean
    square, weighted (one weight of value_dim entries for all heads), gated by sigmoid(W_g2 W_g1 h) and projected.
    ``gate_rank``: the inner size of the two-step projections; 0: whatever the checkpoint's tensors have."""
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    key_dim: int
    value_dim: int
    conv_taps: int
    norm_eps: float
    unit_eps: float = 1e-6
    gate_rank: int = 0
    kind: str = "channel_delta"


@dataclass(frozen=True)
class StateSpaceSpec:
    """Selective state-space mixer with a scalar decay per head (state-space duality): the input projection
    gives [z | x | B | C | dt]; x, B and C pass a causal convolution with bias and silu; dt = softplus(dt + dt_bias);
    S <- exp(-exp(A_log) dt) S + dt B x^T (``state_dim`` x ``head_dim`` per head, B and C shared by the heads of a
    group), y = S^T C + D x; y * silu(z) is normed in ``norm_groups`` equal parts, weighted and projected."""
    hidden_size: int
    num_heads: int
    head_dim: int
    state_dim: int
    groups: int
    conv_taps: int
    norm_groups: int
    norm_eps: float
    kind: str = "state_space"

    @property
    def inner_size(self) -> int:
        return self.num_heads * self.head_dim

    @property
    def conv_size(self) -> int:
        return self.inner_size + 2 * self.groups * self.state_dim


@dataclass(frozen=True)
class ParallelMixerSpec:
    """Several mixers side by side on the same input: sum_i scales[i] * branch_i(h). ``prefixes[i]`` is put between
    the mixer's tensor prefix and branch i's local names."""
    branches: Tuple[object, ...]
    scales: Tuple[float, ...]
    prefixes: Tuple[str, ...]
    kind: str = "parallel"


@dataclass(frozen=True)
class DenseMLPSpec:
    """Dense feed-forward without a gate: down(act(up h + b_up)) + b_down. ``activation``: 'gelu' (the exact,
    erf form) or 'gelu_tanh'."""
    hidden_size: int
    intermediate_size: int
    activation: str = "gelu"
    bias: bool = True
    kind: str = "dense_mlp"


@dataclass(frozen=True)
class LayerSpec:
    """One block: which mixer, which feed-forward, their norms and how they are arranged.
    ``arrangement='pre_norm'``: x += mixer(norm1(x)); x += feed_forward(norm2(x)).
    ``arrangement='output_norm'``: x += norm1(mixer(x)); x += norm2(feed_forward(x)), the sums in a float32 stream.
    ``arrangement='multi_stream'``: the residual is ``streams`` float32 copies; a sublayer reads a mixture of them
    through its norm and writes back into all of them (``learned_mixing``: the block owns the coefficients
    ``hc1.*`` for the mixer and ``hc2.*`` for the feed-forward; otherwise all are 1, which with one stream is the
    pre-norm residual kept in float32).
    ``feed_forward`` None (with ``feed_forward_norm`` None): the block has a mixer only.
    ``mixer_out_norm`` / ``feed_forward_out_norm`` ('multi_stream' only): a second norm on the sublayer's OUTPUT
    before it is added, x += norm_b(sublayer(norm(x))); its ``tensor`` is the name behind the LAYER's prefix.
    ``index``: the number in this layer's checkpoint names where that is not its place in ``ModelSpec.layers`` (a model
    that lists, among its layers, some that run another layer's tensors has fewer layers with tensors than numbers)."""
    mixer: object
    feed_forward: object
    mixer_norm: NormSpec
    feed_forward_norm: Optional[NormSpec]
    arrangement: str = "pre_norm"
    streams: int = 1
    learned_mixing: bool = False
    mixer_out_norm: Optional[NormSpec] = None
    feed_forward_out_norm: Optional[NormSpec] = None
    index: Optional[int] = None


@dataclass(frozen=True)
class ExecStep:
    """One entry of the run order. ``layer`` indexes ``ModelSpec.layers`` (a layer may be named
    more than once). ``cache`` names the cache entry the mixer works on; ``writes_cache`` is
    False for an entry that only reads what an earlier entry wrote there."""
    layer: int
    cache: int
    writes_cache: bool = True


@dataclass(frozen=True)
class TensorNames:
    """Checkpoint names of an architecture, as patterns. ``{i}`` is the layer index."""
    embedding: str = "model.embed_tokens.weight"
    layer: str = "model.layers.{i}."
    mixer: str = "self_attn."
    feed_forward: str = "mlp."
    mixer_norm: str = "input_layernorm."
    feed_forward_norm: str = "post_attention_layernorm."
    final_norm: str = "model.norm."
    head: str = "lm_head.weight"


@dataclass(frozen=True)
class ModelSpec:
    """Everything the generic decoder needs: sizes, the layers, and the order they run in."""
    architecture: str
    vocab_size: int
    hidden_size: int
    layers: Tuple[LayerSpec, ...]
    execution: Tuple[ExecStep, ...]
    final_norm: NormSpec
    tie_embeddings: bool
    max_positions: int
    names: TensorNames = field(default_factory=TensorNames)

    def __post_init__(self):
        seen = set()
        for step in self.execution:
            if not 0 <= step.layer < len(self.layers):
                raise ValueError(f"execution names layer {step.layer}, the model has {len(self.layers)}")
            if step.writes_cache:
                if step.cache in seen:
                    raise ValueError(f"cache entry {step.cache} has two writers in the run order")
                seen.add(step.cache)
            elif step.cache not in seen:
                raise ValueError(f"cache entry {step.cache} is read before any entry writes it")

    @property
    def num_cache_entries(self) -> int:
        return 1 + max((s.cache for s in self.execution), default=-1)


def default_execution(num_layers: int) -> Tuple[ExecStep, ...]:
    """Every layer once, in order, each with a cache entry of its own."""
    return tuple(ExecStep(layer=i, cache=i, writes_cache=True) for i in range(num_layers))
