"""Descriptions of a model as data.

A configuration class turns config.json into a `ModelSpec`: one `BlockSpec`
for every layer (its norms, its mixer, its feed-forward, each with all
sizes and constants), a schedule that says in which order layers run and
whose cache each reads, and the names of the tensors that every part
binds. Parts are built from these records through the registries in
`llm_b200.parts`; nothing here knows an architecture.

Any object with a `kind` attribute can stand as a spec: a part registered
under that kind receives it unchanged.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional


@dataclass(frozen=True)
class NormSpec:
    size: int
    eps: float
    weight: str                      # tensor name
    kind: str = "rmsnorm"
    unit_offset: bool = False        # the stored weight lies around zero: the gain is 1 + weight


@dataclass(frozen=True)
class TanhNormSpec:
    """A norm without a statistic: y = tanh(alpha x) * weight + bias, element by element (alpha one number)."""
    size: int
    weight: str                      # tensor names
    bias: str
    alpha: str
    kind: str = "tanh_norm"


@dataclass(frozen=True)
class PositionSpec:
    """Rotary encoding: angle = position * inv_freq[pair]."""
    head_dim: int
    theta: float
    max_positions: int
    scaling: Optional[tuple] = None  # sorted (key, value) pairs of rope_scaling, or None
    pairing: str = "half"            # 'half': (p, p + n/2); 'interleaved': (2p, 2p + 1)
    kind: str = "rope"
    rotary_dim: Optional[int] = None # n: how many leading elements of a head rotate (None: all)

    @property
    def scaling_dict(self):
        return dict(self.scaling) if self.scaling is not None else None


@dataclass(frozen=True)
class AttentionSpec:
    hidden: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    scale: float                     # multiplies q.k
    bias: bool
    window: int                      # 0: every earlier key; w > 0: the last w keys
    position: Optional[PositionSpec]
    names: tuple                     # sorted (role, tensor name): q, k, v, o (+ q_bias, ...)
    kind: str = "attention"

    @property
    def tensor(self):
        return dict(self.names)


@dataclass(frozen=True)
class DiffAttentionSpec:
    """Differential attention: every query head has two maps, each a softmax attention of its own
    over the same values; a head's result is map 1 minus lambda times map 2, divided by its root
    mean square and multiplied by 1 - diff. lambda = e^<lq1, lk1> - e^<lq2, lk2> + diff."""
    hidden: int
    n_heads: int
    n_kv_heads: int
    head_dim: int                    # query / key size of ONE map
    value_dim: int
    scale: float                     # multiplies q.k
    window: int                      # 0: every earlier key; w > 0: keys less than w positions back ...
    keep_first: int                  # ... and the sequence's first keep_first keys
    conv_taps: int                   # taps of the causal convolution behind q, k, v (0: none)
    diff: float                      # lambda's constant term; the result is scaled by 1 - diff
    eps: float                       # of the head's norm
    position: Optional[PositionSpec]
    names: tuple                     # sorted (role, tensor name): q, k, v, o, lq1, lk1, lq2, lk2 (+ q_conv, k_conv, v_conv)
    kind: str = "diff_attention"

    @property
    def tensor(self):
        return dict(self.names)


@dataclass(frozen=True)
class LatentAttentionSpec:
    """Attention whose keys and values of every head are made from one normed latent row per
    position, and whose queries pass through a normed latent of their own: c_q = norm(W_dq h),
    q = W_uq c_q, c = norm(W_dkv h), k = W_uk c, v = W_uv c. Only c is cached. Softmax over the
    visible keys with, optionally, one learned term per head in the denominator (`sink`), and,
    optionally, a sigmoid gate per head read from the mixer's input (`gate`)."""
    hidden: int
    n_heads: int
    head_dim: int                    # query / key size of a head
    value_dim: int
    q_rank: int                      # size of the queries' latent
    kv_rank: int                     # size of the cached latent
    scale: float                     # multiplies q.k
    window: int                      # 0: every earlier key; w > 0: keys less than w positions back
    eps: float                       # of both latent norms
    sink: bool
    gate: bool
    names: tuple                     # sorted (role, tensor name): dq, dq_norm, uq, dkv, dkv_norm, uk, uv, o (+ sink, gate)
    out_scale: float = 1.0           # multiplies the mixer's result
    kind: str = "latent_attention"

    @property
    def tensor(self):
        return dict(self.names)


@dataclass(frozen=True)
class SigmoidAttentionSpec:
    """Grouped-query attention without a softmax: the weight of a visible key is
    sigmoid(score + bias[head]), not normalised over the keys. Before that, optionally, the heads'
    scores of one (query, key) pair are mixed by a matrix (`talk`: score_h <- sum_g T[h, g] score_g).
    With `qk_norm`, queries and keys are RMS-normed over their whole projection (all heads at
    once) before the rotation."""
    hidden: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    value_dim: int
    scale: float
    window: int
    qk_norm: bool
    eps: float                       # of the query / key norm
    talk: bool
    head_bias: bool
    position: Optional[PositionSpec]
    names: tuple                     # sorted (role, tensor name): q, k, v, o (+ q_norm, k_norm, talk, head_bias)
    out_scale: float = 1.0
    kind: str = "sigmoid_attention"

    @property
    def tensor(self):
        return dict(self.names)


@dataclass(frozen=True)
class GatedRecurrenceSpec:
    """A recurrent block with a real-gated linear recurrent unit (De et al., "Griffin"): two
    branches of `width` channels, y = gelu(W_y h + b_y) and u = conv(W_x h + b_x) (causal, per
    channel, `conv_taps` taps with a bias); the channels are cut into `blocks` equal parts, each
    with its own square matrices for the recurrence gate r and the input gate i;
    a = exp(-decay * r * softplus(lam)), S_t = a S_(t-1) + sqrt(1 - a^2) i u; result W_o (S * y)."""
    hidden: int
    width: int
    blocks: int
    conv_taps: int
    decay: float                     # 8 in the published block
    names: tuple                     # sorted (role, tensor name): y, y_bias, x, x_bias, conv, conv_bias, ra, ra_bias, ri, ri_bias, lam, o
    out_scale: float = 1.0
    kind: str = "gated_recurrence"

    @property
    def tensor(self):
        return dict(self.names)


@dataclass(frozen=True)
class GatedAttentionSpec:
    """Grouped-query softmax attention whose result is multiplied, element by element, by
    sigmoid(W_g h) before the output projection (`out_gate`; the gate reads the mixer's input). With
    `values_are_keys` there is no value projection: a key head's values are its keys as projected,
    before the rotation (so value_dim == head_dim).

    Switches that are off by default: `head_norm` (every head of the queries and of the keys is divided by its
    own root mean square over head_dim (eps `norm_eps`) and multiplied by a weight of head_dim elements that the
    heads share, before the rotation); `head_gate` (one gate number per head, sigmoid(W_g h)[head] with W_g
    [n_heads, hidden], instead of one per element); `softcap` (c > 0: score <- c tanh(score / c) behind the
    scale); `unit_sink` (the softmax's denominator holds one more term e^0 that has no value);
    `value_mix` (a name shared by the layers whose values are blended: in every such layer but the one with
    `value_mix_first`, v <- (1 - w) v + w v_first with w one stored number (role `value_mix`) and v_first the
    values that the first such layer computed for the same token; the blended values are what is cached);
    `out_scale` multiplies the mixer's result."""
    hidden: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    value_dim: int
    scale: float                     # multiplies q.k
    window: int                      # 0: every earlier key; w > 0: keys less than w positions back
    values_are_keys: bool
    out_gate: bool
    position: Optional[PositionSpec]
    names: tuple                     # sorted (role, tensor name): q, k, o (+ v, gate, q_norm, k_norm, value_mix)
    kind: str = "gated_attention"
    head_norm: bool = False
    norm_eps: float = 0.0
    head_gate: bool = False
    softcap: float = 0.0
    unit_sink: bool = False
    value_mix: Optional[str] = None
    value_mix_first: bool = False
    out_scale: float = 1.0

    @property
    def tensor(self):
        return dict(self.names)


@dataclass(frozen=True)
class DeltaRuleSpec:
    """The gated delta rule: per head a state matrix M [head_dim,
    value_dim] with M_t = a_t M_{t-1} + k_t w_t^T with w_t = b_t (v_t - a_t M_{t-1}^T k_t); o_t = M_t^T q_t. q, k (n_kv_heads heads,
    shared by groups of query heads) and v (n_heads heads) pass a causal convolution of `conv_taps` taps
    per channel and silu; q and k are divided by sqrt(sum of squares + unit_eps), q also by
    sqrt(head_dim); b_t = sigmoid(W_b h); a_t = exp(-exp(A_log) softplus(W_a h + dt_bias)); every head's o
    is divided by its root mean square (eps), multiplied by a weight of value_dim elements shared by
    the heads and by silu(W_g h)."""
    hidden: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    value_dim: int
    conv_taps: int
    eps: float                       # of the heads' norm
    names: tuple                     # sorted (role, tensor name): q, k, v, q_conv, k_conv, v_conv, beta, decay, a_log, dt_bias, gate, norm, o
    unit_eps: float = 1e-6
    kind: str = "delta_rule"

    @property
    def tensor(self):
        return dict(self.names)


@dataclass(frozen=True)
class StateSpaceSpec:
    """A state-space recurrence with one scalar decay per head (the layer of Dao and Gu's "Transformers are
    SSMs"): W_in h = [z | x | B | C | dt] with x of n_heads heads of value_dim, B and C of `groups` groups of
    `state` elements (a group serves n_heads / groups heads); x, B, C pass one causal convolution per channel
    (`conv_taps` taps, a bias) and silu; dt <- softplus(dt + dt_bias); per head S_t = exp(-exp(A_log) dt) S_(t-1)
    + dt B_t x_t^T, y_t = S_t^T C_t + D x_t; y silu(z) is divided by its root mean square in `norm_groups` equal
    parts (eps), multiplied by a weight per channel, then W_o. `out_scale` multiplies the result."""
    hidden: int
    n_heads: int
    value_dim: int
    state: int
    groups: int
    conv_taps: int
    norm_groups: int
    eps: float
    names: tuple                     # sorted (role, tensor name): in, conv, conv_bias, dt_bias, a_log, skip, norm, o
    out_scale: float = 1.0
    kind: str = "state_space"

    @property
    def tensor(self):
        return dict(self.names)


@dataclass(frozen=True)
class SideBySideSpec:
    """Two mixers that read the same input; their results (each times its own `out_scale`) are added."""
    left: object
    right: object
    kind: str = "side_by_side"


@dataclass(frozen=True)
class GatedMlpSpec:
    hidden: int
    intermediate: int
    activation: str                  # 'silu'
    names: tuple                     # sorted (role, tensor name): gate, up, down
    kind: str = "gated_mlp"

    @property
    def tensor(self):
        return dict(self.names)


@dataclass(frozen=True)
class MlpSpec:
    """down(act(up h)) with two matrices; `activation` 'gelu_tanh' (the tanh form of gelu)."""
    hidden: int
    intermediate: int
    activation: str
    names: tuple                     # sorted (role, tensor name): up, down
    kind: str = "mlp"

    @property
    def tensor(self):
        return dict(self.names)


@dataclass(frozen=True)
class RoutedExpertsSpec:
    """A mixture of `n_experts` gated feed-forwards of which a token uses `top`: router logits
    W_r h (+ bias) in 32-bit, the `top` largest chosen, their weights the softmax over the chosen
    logits; expert e is down_e(silu(gate_e h) * (up_e h)). `expert_names` holds the (role, name)
    pairs of one expert with '{e}' in place of its index.

    `scoring` 'all' instead: scores s = softmax over ALL router outputs, the `top` largest of s + correction
    (`correction`: a stored vector that takes part in the choice only) are chosen, and the weights are the
    chosen scores divided by their sum (+ 1e-20). `pass_through` > 0: the router has n_experts + pass_through
    outputs; the last ones are experts without tensors whose result is their input. `out_scale` multiplies
    the result."""
    hidden: int
    intermediate: int
    n_experts: int
    top: int
    router_bias: bool
    names: tuple                     # sorted (role, tensor name): router (+ router_bias, correction)
    expert_names: tuple              # sorted (role, pattern): gate, up, down
    activation: str = "silu"
    kind: str = "routed_experts"
    scoring: str = "chosen"          # 'chosen': softmax over the chosen logits; 'all': see above
    correction: bool = False
    pass_through: int = 0
    out_scale: float = 1.0

    @property
    def tensor(self):
        return dict(self.names)

    def expert_tensor(self, e: int) -> dict:
        return {role: pattern.format(e=e) for role, pattern in self.expert_names}


@dataclass(frozen=True)
class SandwichBlockSpec:
    """x += mixer_post_norm(mixer(mixer_norm(x))); x += ffn_post_norm(feed_forward(ffn_norm(x))): a norm
    in front of and behind each part. `feed_forward` (with its two norms) may be None."""
    mixer_norm: object
    mixer: object
    mixer_post_norm: object
    ffn_norm: object
    feed_forward: object
    ffn_post_norm: object
    kind: str = "sandwich"


@dataclass(frozen=True)
class BlockSpec:
    """x += mixer(mixer_norm(x)); x += feed_forward(ffn_norm(x))  ('pre_norm')."""
    mixer_norm: object
    mixer: object
    ffn_norm: object
    feed_forward: object
    kind: str = "pre_norm"


@dataclass(frozen=True)
class ParallelBlockSpec:
    """x += mixer(norm(x)) + feed_forward(norm(x)): one norm, both parts read its output.
    `feed_forward` may be None (a layer that only mixes). With `ffn_norm` the feed-forward reads a
    norm of its own, of the same x: x += mixer(norm(x)) + feed_forward(ffn_norm(x))."""
    norm: object
    mixer: object
    feed_forward: object
    kind: str = "parallel"
    ffn_norm: object = None


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer. `cache_of` names an earlier schedule entry whose
    keys and values this run reads instead of writing its own. With `add_embedding` the
    embedding output (the stream as it was before the first run) is added to the stream
    right before this run."""
    layer: int
    cache_of: Optional[int] = None
    add_embedding: bool = False


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab: int
    hidden: int
    max_positions: int
    embedding: str                   # tensor name of the [vocab, hidden] table
    blocks: tuple                    # BlockSpec per layer
    schedule: tuple                  # ScheduleEntry, in running order
    final_norm: object
    head: Optional[str]              # tensor name of the [vocab, hidden] head; None: tied to the embedding
    stop_tokens: tuple = field(default_factory=tuple)
    embedding_scale: float = 1.0     # multiplies the embedded tokens
    logit_scale: float = 1.0         # multiplies the logits
    logit_softcap: float = 0.0       # c > 0: logits <- c * tanh(logits / c), after the scale


def names(**roles) -> tuple:
    return tuple(sorted(roles.items()))
