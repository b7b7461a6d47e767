"""Descriptions of a model as data: which parts, with which sizes and constants, in which order.

An architecture (models/opt.py) turns its typed configuration into a ``ModelSpec``.  Every part
is named by a ``kind`` that the registries of parts/registry.py resolve to a class, so a model may
use different mixers and feed-forwards in different layers, and a test may register a kind of its
own.  The order in which layers run is the ``schedule``: a list of (layer, cache) pairs that may
name a layer twice, or give two entries the same cache so that one layer reads what another wrote.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Optional, Tuple


@dataclass(frozen=True)
class LinearSpec:
    in_features: int
    out_features: int
    weight: str                      # tensor name, [out_features, in_features]
    bias: Optional[str] = None       # tensor name, [out_features]; None: no bias


@dataclass(frozen=True)
class NormSpec:
    kind: str                        # 'layer_norm' | 'rms_norm'
    size: int
    eps: float
    weight: Optional[str] = None     # None: no elementwise scale
    bias: Optional[str] = None
    weight_offset: float = 0.0       # 'rms_norm': the scale is weight + weight_offset (1.0: "one plus" weights)


@dataclass(frozen=True)
class FrequencyRampSpec:
    """Stretching of a rotation's frequencies for contexts longer than the `original` one ("YaRN"): with
    turns(t) = dims * ln(original / (2 pi t)) / (2 ln base), lo = max(floor(turns(fast)), 0),
    hi = min(ceil(turns(slow)), dims - 1) and ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), pair i turns by
    f_i / factor * ramp_i + f_i * (1 - ramp_i), and sines and cosines are multiplied by 0.1 ln(factor) + 1."""
    factor: float
    original: float
    fast: float
    slow: float


@dataclass(frozen=True)
class RotarySpec:
    """Rotation of pairs of dims by position over the first `dims` dims of a head: pair i turns by
    position * base^(-2i/dims).  Pair i is (dim i, dim i + dims/2), or with `interleaved` (dim 2i, dim 2i + 1)."""
    dims: int
    base: float
    interleaved: bool = False
    scaling: Optional[FrequencyRampSpec] = None


@dataclass(frozen=True)
class PositionSpec:
    kind: str                        # 'learned' | 'sinusoidal' | 'none' | a registered kind
    table: Optional[str] = None      # tensor name, [rows, dim]
    rows: int = 0
    dim: int = 0
    offset: int = 0                  # row = position + offset
    extra: Tuple = ()
    base: float = 10000.0            # 'sinusoidal': entry 2i = sin(p base^(-2i/dim)), entry 2i + 1 = cos of the same


@dataclass(frozen=True)
class AttentionSpec:
    kind: str                        # 'attention'
    hidden: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    scale: float
    q: LinearSpec = None
    k: LinearSpec = None
    v: LinearSpec = None
    out: LinearSpec = None
    window: Optional[int] = None     # None: every earlier position is read
    position: Optional[PositionSpec] = None   # an encoding applied to queries and keys, if any


@dataclass(frozen=True)
class RotaryAttentionSpec:
    """Softmax attention over the paged cache whose queries and keys may be normalised over the whole
    projection, are rotated by position, and whose score is multiplied by a number per head; the values
    may be rotated as well (and each head's output turned back by the query's position)."""
    kind: str                        # 'rotary_attention'
    hidden: int
    n_heads: int
    n_kv_heads: int
    k_dim: int                       # per-head size of queries and keys
    v_dim: int                       # per-head size of values
    scale: float
    q: LinearSpec = None
    k: LinearSpec = None
    v: LinearSpec = None
    out: LinearSpec = None
    rotary: Optional[RotarySpec] = None
    rotate_values: bool = False      # values turned by their position over all v_dim dims (base of `rotary`)
    q_norm: Optional[str] = None     # tensor [n_heads * k_dim]: RMS norm over the whole projection, before rotation
    k_norm: Optional[str] = None     # tensor [n_kv_heads * k_dim]
    norm_eps: float = 1e-6
    head_scale: Optional[str] = None  # tensor [n_heads]: the score of head h is multiplied by its entry
    window: Optional[int] = None
    # `v` None: there is no value projection; the values are the keys as projected (with bias), before normalisation
    # and rotation (v_dim = k_dim)


@dataclass(frozen=True)
class LatentAttentionSpec:
    """Softmax attention whose queries and whose keys and values pass through low-rank latents, with a sliding window:
      c_q = rms(W_dq h) * q_norm,  q = W_uq c_q, per head [k_dim unrotated, rot_dim rotated]
      W_dkv h = [kv_rank | rot_dim]: c = rms(first part) * kv_norm (the latent), the rest one rotated key part that all
      heads share;  per head  k = [W_uk c | rotated part],  v = W_uv c;  score = scale * <q, k>.
    The rotated parts turn by position in interleaved pairs (2i, 2i + 1) or halves.  Only c and the rotated key part are
    kept per position."""
    kind: str                        # 'latent_attention'
    hidden: int
    n_heads: int
    k_dim: int                       # unrotated query/key dims per head
    rot_dim: int                     # rotated query/key dims per head (0: none)
    v_dim: int
    q_rank: int
    kv_rank: int
    scale: float
    dq: LinearSpec = None            # [q_rank, hidden]
    uq: LinearSpec = None            # [n_heads * (k_dim + rot_dim), q_rank]
    dkv: LinearSpec = None           # [kv_rank + rot_dim, hidden]
    uk: str = None                   # tensor [n_heads * k_dim, kv_rank]
    uv: str = None                   # tensor [n_heads * v_dim, kv_rank]
    out: LinearSpec = None
    q_norm: Optional[str] = None     # tensor [q_rank]
    kv_norm: Optional[str] = None    # tensor [kv_rank]
    norm_eps: float = 1e-6
    rotary: Optional[RotarySpec] = None    # over the rot_dim part (rotary.dims = rot_dim)
    window: Optional[int] = None


@dataclass(frozen=True)
class DeltaRuleSpec:
    """A recurrence with an error-correcting write and a decay per key channel.  Per head, with S of k_dim x v_dim:
        S <- diag(g_t) S;  u = beta_t (v_t - S^T k_t);  S <- S + k_t u^T;  o_t = S^T q_t
    q, k (n_kv_heads x k_dim, shared by groups of heads) and v (n_heads x v_dim) pass a short causal convolution over
    time and an activation; q and k are made unit vectors (x / sqrt(sum x^2 + unit_eps)), q times q_scale;
    beta = sigmoid(W_b h); g = exp(-exp(A_log_h) softplus(W_a2 W_a1 h + dt_bias)) per head and key channel;
    each head's o is divided by its root mean square, times `out_norm` (one weight vector of v_dim), times
    sigmoid(W_g2 W_g1 h).  The inner sizes of a1/a2 and g1/g2 may be -1: they are then the stored tensors'."""
    kind: str                        # 'delta_rule'
    hidden: int
    n_heads: int
    n_kv_heads: int
    k_dim: int
    v_dim: int
    conv_taps: int
    q: LinearSpec = None
    k: LinearSpec = None
    v: LinearSpec = None
    beta: LinearSpec = None          # [n_heads, hidden]
    a1: LinearSpec = None            # [rank_a, hidden]
    a2: LinearSpec = None            # [n_heads * k_dim, rank_a]
    g1: LinearSpec = None            # [rank_g, hidden]
    g2: LinearSpec = None            # [n_heads * v_dim, rank_g]
    out: LinearSpec = None
    q_conv: Optional[str] = None     # tensors [channels, conv_taps]; the last column weighs the current token
    k_conv: Optional[str] = None
    v_conv: Optional[str] = None
    a_log: str = None                # tensor [n_heads]
    dt_bias: str = None              # tensor [n_heads * k_dim]
    out_norm: Optional[str] = None   # tensor [v_dim]
    norm_eps: float = 1e-6
    unit_eps: float = 1e-6
    q_scale: float = 1.0
    conv_activation: str = "silu"


@dataclass(frozen=True)
class ConvAttentionSpec:
    """Softmax attention over the paged cache whose projections (with bias) pass through a short causal convolution
    over time, channel by channel, before queries and keys are normalised per head (one weight vector of k_dim for
    all heads) and rotated.  The mask is causal, and a sliding window or chunked (a query reads the keys of its own
    block of `chunk` positions).  With `kv_source` the mixer has no keys and values of its own: it reads the pages
    of the mixer whose schedule entry has that cache number (which ran earlier in the step), with its own queries
    and mask."""
    kind: str                        # 'conv_attention'
    hidden: int
    n_heads: int
    n_kv_heads: int
    k_dim: int
    v_dim: int
    scale: float
    q: LinearSpec = None
    k: Optional[LinearSpec] = None
    v: Optional[LinearSpec] = None
    out: LinearSpec = None
    conv_taps: int = 0               # taps of the convolution; 0: none
    q_conv: Optional[str] = None     # tensor [n_heads * k_dim, conv_taps]; tap j weighs the value conv_taps - 1 - j back
    k_conv: Optional[str] = None
    v_conv: Optional[str] = None
    q_norm: Optional[str] = None     # tensor [k_dim]: RMS norm of every query head, before rotation
    k_norm: Optional[str] = None
    norm_eps: float = 1e-6
    rotary: Optional[RotarySpec] = None
    window: Optional[int] = None
    chunk: Optional[int] = None
    kv_source: Optional[int] = None
    keep_all_pages: bool = False     # another mixer reads these pages with another mask: none is given back early


@dataclass(frozen=True)
class DiffAttentionSpec:
    """Differential softmax attention over the paged cache: every head holds TWO maps of queries and keys (k_dim dims
    each, the projections' rows laid out head by head as [map 1, map 2]) over the same values,
        o = softmax(scale q1 k1^T) v - lambda softmax(scale q2 k2^T) v,   lambda = exp(<lq1, lk1>) - exp(<lq2, lk2>) + diff,
    then each head's o is divided by its root mean square (no weight), multiplied by out_mult and by the sigmoid of the
    head's entry of a gate projection, before the output projection.  Queries and keys are normalised per head and map
    (one weight vector of k_dim for all), and queries are multiplied by 1 + temp_coef ln(floor((p + 1) / temp_every) + 1)
    at position p (temp_every 0: not).  Positions enter in no other way.  With `kv_source` the mixer has no keys and
    values of its own: it reads the pages of the mixer whose schedule entry has that cache number."""
    kind: str                        # 'diff_attention'
    hidden: int
    n_heads: int
    n_kv_heads: int
    k_dim: int                       # per map
    v_dim: int
    scale: float
    diff: float                      # the constant of lambda
    out_mult: float                  # what the normalised head output is multiplied by
    q: LinearSpec = None             # [n_heads * 2 * k_dim, hidden]
    k: Optional[LinearSpec] = None   # [n_kv_heads * 2 * k_dim, hidden]
    v: Optional[LinearSpec] = None   # [n_kv_heads * v_dim, hidden]
    gate: Optional[LinearSpec] = None   # [n_heads, hidden]; None: no output gate
    out: LinearSpec = None
    q_norm: Optional[str] = None     # tensor [k_dim]
    k_norm: Optional[str] = None
    lambda_q1: str = None            # tensors [k_dim]
    lambda_k1: str = None
    lambda_q2: str = None
    lambda_k2: str = None
    norm_eps: float = 1e-6
    temp_coef: float = 0.0
    temp_every: int = 0
    window: Optional[int] = None
    kv_source: Optional[int] = None


@dataclass(frozen=True)
class SSDSpec:
    """A selective state-space recurrence with one decay per head and token ("state-space duality").  The input
    projection's rows are [z: inner | x: inner | B: groups * state | C: groups * state | dt: n_heads], inner = n_heads * v_dim.
    x, B and C pass one short causal convolution per channel (with bias) and an activation; dt <- softplus(dt + dt_bias);
    per head h (group h / (n_heads / groups)), with S of state x v_dim:
        S <- exp(-exp(A_log_h) dt) S + dt B x^T;   y = S^T C + D_h x
    y times act(z) (the gate comes first), then divided by its root mean square in `norm_groups` equal parts of the
    inner width, times a weight vector, then the output projection."""
    kind: str                        # 'ssd'
    hidden: int
    n_heads: int
    v_dim: int
    state: int
    groups: int
    norm_groups: int
    conv_taps: int
    in_proj: LinearSpec = None       # [2 inner + 2 groups state + n_heads, hidden]
    out: LinearSpec = None
    conv: str = None                 # tensor [inner + 2 groups state, conv_taps]; the last column weighs the current token
    conv_bias: Optional[str] = None  # tensor [inner + 2 groups state]
    dt_bias: str = None              # tensor [n_heads]
    a_log: str = None                # tensor [n_heads]
    skip: Optional[str] = None       # tensor [n_heads]: D
    out_norm: Optional[str] = None   # tensor [inner]
    norm_eps: float = 1e-6
    activation: str = "silu"         # of the convolution's output and of the gate


@dataclass(frozen=True)
class RetentionSpec:
    """Linear attention with a fixed decay per head: S <- decay S + k v^T, o = S^T q; each head's o divided by
    its root mean square, gated by silu of a projection, then the output projection."""
    kind: str                        # 'retention'
    hidden: int
    n_heads: int
    k_dim: int
    v_dim: int
    decay: Tuple[float, ...] = ()    # one per head
    q: LinearSpec = None
    k: LinearSpec = None
    v: LinearSpec = None
    gate: Optional[LinearSpec] = None
    out: LinearSpec = None
    rotary: Optional[RotarySpec] = None
    k_scale: float = 1.0             # keys are multiplied by it after rotation
    norm_eps: float = 1e-6


@dataclass(frozen=True)
class ParallelMixerSpec:
    """Several mixers side by side on the same input; the result is the sum of scale_i * branch_i."""
    kind: str                        # 'parallel'
    branches: Tuple[Any, ...] = ()
    scales: Tuple[float, ...] = ()


@dataclass(frozen=True)
class MinGRUSpec:
    """S <- (1 - z) S + z cand with gates that read the current token only; output W_o (S * silu(gate))."""
    kind: str                        # 'mingru'
    hidden: int
    width: int
    z: LinearSpec = None             # update gate (sigmoid)
    x: LinearSpec = None             # candidate
    gate: Optional[LinearSpec] = None
    out: LinearSpec = None


@dataclass(frozen=True)
class GatedFeedForwardSpec:
    kind: str                        # 'gated_dense'
    gate: LinearSpec = None
    up: LinearSpec = None
    down: LinearSpec = None
    activation: str = "silu"         # applied to the gate's product


@dataclass(frozen=True)
class ExpertSpec:
    gate: Optional[str]              # tensor names, [ff, hidden], [ff, hidden], [hidden, ff]; no biases
    up: str                          # (gate None: an expert without a gate, see RoutedFeedForwardSpec.expert_form)
    down: str


@dataclass(frozen=True)
class RoutedFeedForwardSpec:
    """Experts chosen per token by a router: scores = sigmoid (or softmax) of router(h) in 32-bit, the `top` largest
    choose, their scores are the weights (divided by their sum with `renormalize`).  An expert computes
    down(g * sigmoid(act_alpha g) * (u + up_shift)) with g = min(gate(x), gate_limit) and u = clamp(up(x), +-up_limit);
    the weight multiplies the expert's input x = w h (`weight_on_input`) or its output.
    With `expert_form` 'relu2' an expert has no gate: down(relu(up(x))^2).
    Routing options (sigmoid scores): `correction` names a tensor [n_experts] that is added to the scores for the CHOICE
    only (the weights stay the uncorrected scores); with `n_groups` > 1 the experts form equal groups of neighbours, a
    group's score is the sum of its `group_top` largest choice scores, and only experts of the `keep_groups` best groups
    can be chosen; the weights are divided by (their sum + renorm_eps) with `renormalize`, then multiplied by
    `weight_scale`."""
    kind: str                        # 'routed_experts'
    hidden: int
    ff: int
    n_experts: int
    top: int
    router: str = None               # tensor [n_experts, hidden]
    experts: Tuple[ExpertSpec, ...] = ()
    scores: str = "sigmoid"          # 'sigmoid' | 'softmax'
    renormalize: bool = False
    weight_on_input: bool = True
    gate_limit: Optional[float] = None
    up_limit: Optional[float] = None
    act_alpha: float = 1.702
    up_shift: float = 1.0
    expert_form: str = "gated_swish"  # 'gated_swish' | 'relu2'
    correction: Optional[str] = None
    n_groups: int = 1
    keep_groups: int = 1
    group_top: int = 2
    renorm_eps: float = 0.0
    weight_scale: float = 1.0


@dataclass(frozen=True)
class DenseFeedForwardSpec:
    kind: str                        # 'dense'
    fc1: LinearSpec = None
    fc2: LinearSpec = None
    activation: str = "relu"


@dataclass(frozen=True)
class LayerSpec:
    block: str                       # 'pre_norm' | 'post_norm' | 'post_norm_scaled' | 'output_norm' | 'sandwich_norm' | 'parallel_residual' | a registered kind
    norm1: Any = None
    mixer: Any = None
    norm2: Any = None
    feed_forward: Any = None         # None: the layer has no feed-forward (and no second norm)
    norm1_post: Any = None           # 'sandwich_norm': the norms on the sublayers' outputs,
    norm2_post: Any = None           #     x <- x + norm1_post(mixer(norm1(x))); x <- x + norm2_post(ff(norm2(x)))
    residual_scale: float = 1.0      # 'post_norm_scaled': x <- norm(residual_scale * x + sublayer(x));
                                     # 'output_norm': x <- x + residual_scale * norm(sublayer(x))
    scale1: Optional[str] = None     # 'parallel_residual': tensors [hidden] that multiply the mixer's and the
    scale2: Optional[str] = None     #     feed-forward's result, x <- x + scale1 * mixer(norm1(x)) + scale2 * ff(norm2(x))


@dataclass(frozen=True)
class EmbeddingSpec:
    table: str                       # tensor name, [vocab, dim]
    vocab: int = 0
    dim: int = 0
    project_in: Optional[LinearSpec] = None
    position: Optional[PositionSpec] = None   # an encoding added to the hidden state, if any
    scale: float = 1.0               # the token's row is multiplied by it (in 32-bit) as it enters the stream


@dataclass(frozen=True)
class HeadSpec:
    weight: str                      # tensor name of the output matrix [vocab, dim]
    vocab: int = 0
    dim: int = 0
    tied_to: Optional[str] = None    # used when the file does not store `weight`
    final_norm: Optional[NormSpec] = None
    project_out: Optional[LinearSpec] = None
    logit_scale: float = 1.0         # the logits are multiplied by it


@dataclass(frozen=True)
class ScheduleEntry:
    layer: int                       # index into ModelSpec.layers
    cache: int                       # which cache its mixer uses; entries may share one


@dataclass(frozen=True)
class ModelSpec:
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: EmbeddingSpec
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    head: HeadSpec
    eos_token_id: Optional[int] = None
    pad_token_id: Optional[int] = None
    bos_token_id: Optional[int] = None
