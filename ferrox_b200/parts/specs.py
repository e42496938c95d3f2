"""Plain-data descriptions of the parts a decoder is put together from.

A *spec* carries every size and constant of one part and the name prefix of its
tensors in the checkpoint; it holds no tensors and knows nothing of the model it
ends up in.  An architecture turns its ``config.json`` into a :class:`ModelSpec`
(one :class:`BlockSpec` per layer, chosen layer by layer, plus the order in which
the layers run); ``parts.build`` turns specs into parts that own weights and run
kernels.  New kinds of part register a spec class of their own with the same
``kind`` string as their implementation (``parts.registry``).

The reference keeps the same facts in ``ModelConfig`` and asks them per layer
(``layer_is_dense``, ``layer_sliding_window``, ``layer_rope_theta``;
crates/ferrox-models/src/config.rs:247-277).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple


@dataclass(frozen=True)
class NormSpec:
    size: int
    eps: float
    prefix: str  # tensor: <prefix>weight
    kind: str = "rms_norm"
    name: Optional[str] = None  # the weight tensor's full name, where it is not <prefix>weight
    one_plus: bool = False  # the stored weight lies around zero: the norm multiplies by 1 + w


@dataclass(frozen=True)
class LayerNormSpec:
    """(x - mean) / sqrt(variance + eps) * w (+ b) over whole rows; a weight and, with ``bias_name``, a bias."""

    size: int
    eps: float
    name: str  # the weight tensor's full name
    kind: str = "layer_norm"
    bias_name: Optional[str] = None  # the bias tensor's full name (None: no bias)


@dataclass(frozen=True)
class PositionSpec:
    """Rotary position encoding, split-half pairing (i, i + rotary_dim/2)."""

    rotary_dim: int
    theta: float
    kind: str = "rope_neox"


@dataclass(frozen=True)
class AdjacentRotarySpec:
    """Rotary position encoding on pairs of neighbours (2i, 2i + 1) of the first ``rotary_dim`` elements of a
    head, pair i at frequency theta^(-2i / rotary_dim); the rest of the head passes unchanged."""

    rotary_dim: int
    theta: float
    kind: str = "rope_adjacent"


@dataclass(frozen=True)
class ScaledRotarySpec:
    """Rotary position encoding on pairs (i, i + rotary_dim/2) whose frequencies are stretched for contexts longer
    than the ``original`` one: with pair(t) = rotary_dim ln(original / (2 pi t)) / (2 ln theta), lo = max(floor(
    pair(fast)), 0), hi = min(ceil(pair(slow)), rotary_dim - 1) and ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1),
    pair i turns at f_i / factor * ramp_i + f_i (1 - ramp_i), f_i = theta^(-2i / rotary_dim); cos and sin are
    multiplied by 0.1 ln(factor) + 1.  ``factor`` None: plain frequencies, no factor on cos and sin."""

    rotary_dim: int
    theta: float
    factor: Optional[float] = None
    original: float = 0.0
    fast: float = 0.0
    slow: float = 0.0
    kind: str = "rope_scaled"


@dataclass(frozen=True)
class NoPositionSpec:
    """Queries and keys are used as projected."""

    kind: str = "no_position"


@dataclass(frozen=True)
class AttentionSpec:
    hidden: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    qkv_bias: bool
    position: Optional[object]  # the spec of a position-encoding part (None: no encoding)
    window: Optional[int]  # None = all earlier keys; W = the last W positions, the query's own included
    prefix: str  # tensors: <prefix>{q,k,v}_proj.{weight,bias}, <prefix>o_proj.weight
    softmax_scale: Optional[float] = None  # None = 1/sqrt(head_dim)
    softcap: Optional[float] = None  # c: the scaled scores pass through c * tanh(s / c) before the softmax
    tied_values: bool = False  # the values are the keys as projected (before the position encoding); no v tensor
    # names of the tensors after <prefix>, for checkpoints that spell them differently: keys q, k, v, o (weights)
    # and q_bias, k_bias, v_bias
    tensor_names: Optional[Tuple[Tuple[str, str], ...]] = None
    kind: str = "gqa_attention"
    value_dim: Optional[int] = None  # width of a value head where it differs from head_dim
    # queries and keys RMS-normed per head before anything else, with one weight vector [head_dim] each that all
    # heads share: (name of q's weight after <prefix>, name of k's, eps)
    qk_norm: Optional[Tuple[str, str, float]] = None
    # (coef, every): the query at position p is multiplied by 1 + coef * ln(floor((p + 1) / every) + 1)
    query_temperature: Optional[Tuple[float, int]] = None
    # one slope per head: slope * (i - j) is taken off the score of key j for the query at position i
    distance_slopes: Optional[Tuple[float, ...]] = None
    # every value head is divided by its root mean square, v / sqrt(mean(v^2) + eps), without a weight, and cached so
    value_norm_eps: Optional[float] = None
    # with a window: the first keep_first positions of a request stay visible beside the window
    keep_first: int = 0
    # name (after <prefix>) of a [n_heads * value_dim, hidden] matrix g: the concatenated heads are multiplied
    # element by element with sigmoid(g x) before the output projection
    output_gate: Optional[str] = None


@dataclass(frozen=True)
class LatentAttentionSpec:
    """Attention whose keys and values are read out of one latent vector a position.  Per head ``head_dim`` plain
    and ``rot_dim`` rotated query/key elements; a position stores the normed latent [kv_rank] and one rotated key
    part [rot_dim] that all heads share; per head the plain key is uk . c and the value uv . c.  ``q_rank``: the
    queries pass a normed latent of their own.  ``output_gate``: the heads' outputs are multiplied by sigmoid(g . x).
    Tensors after <prefix>: q (or dq, dq.norm, uq), dkv, dkv.norm, uk, uv, g, o."""

    hidden: int
    n_heads: int
    head_dim: int
    rot_dim: int
    value_dim: int
    kv_rank: int
    q_rank: Optional[int]
    rotary_dims: int  # the leading elements of the rot_dim part that are rotated, on neighbouring pairs
    rotary_base: float
    window: Optional[int]
    scale: float
    output_gate: bool
    norm_eps: float
    prefix: str
    kind: str = "latent_attention"
    rotary_pairing: str = "adjacent"  # which elements form pair i: "adjacent" (2i, 2i + 1) or "halves" (i, i + dims/2)
    rotary_scaling: Optional[Tuple[float, float, float, float]] = None  # (factor, original, fast, slow): see ScaledRotarySpec
    gate_per_head: bool = False  # the output gate is one number a head (g [n_heads, hidden]) instead of one an element
    sink: Optional[str] = None  # name after <prefix> of a [n_heads] vector: exp(sink_h) joins the softmax's denominator


@dataclass(frozen=True)
class DifferentialAttentionSpec:
    """Differential attention: every head has two attention maps with queries and keys of their own over the same
    values; o = rms(a1 - lambda a2) (1 - diff) per head, lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff one number
    for the layer.  q rows are laid out head by head as [map 1 | map 2] (H * 2 * head_dim), k likewise (G * 2 *
    head_dim); query head h reads kv head h // (H / G).  ``conv_taps``: a short causal convolution on every channel
    of q, k and v right behind the projections (None: none).  ``position``: the spec of a rotary part that turns the
    first rotary_dim elements of each map of each head (None: none).  ``softcap`` c: scaled scores pass through
    c tanh(s / c).  Tensors after <prefix>: q, k, v, (q.conv, k.conv, v.conv), lq1, lk1, lq2, lk2, o."""

    hidden: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    value_dim: int
    diff: float
    scale: float
    softcap: Optional[float]
    conv_taps: Optional[int]
    position: Optional[object]
    norm_eps: float
    prefix: str
    kind: str = "differential_attention"


@dataclass(frozen=True)
class MlstmSpec:
    """Matrix memory of an mLSTM: per head a state S [head_dim, value_dim], a normaliser and the running maximum of
    the gates' logarithms (``parts.linear_state.Mlstm``).  Tensors after <prefix>: q, k, v, g, o, norm [H * V],
    i [H, hidden], i.b, f [H, hidden], f.b."""

    hidden: int
    n_heads: int
    head_dim: int
    value_dim: int
    gate_cap: float
    norm_eps: float
    prefix: str
    kind: str = "mlstm"


@dataclass(frozen=True)
class GatedDeltaSpec:
    """Gated delta rule: a [head_dim, value_dim] state per head, short causal convolutions on q, k and v.
    Tensors: <prefix>{q,k,v}, <prefix>{q,k,v}.conv [channels, taps], <prefix>b, <prefix>a, <prefix>A_log,
    <prefix>dt_bias, <prefix>g, <prefix>norm [value_dim], <prefix>o."""

    hidden: int
    n_heads: int
    n_kv_heads: int  # heads of q and k; value head h reads q/k head h // (n_heads / n_kv_heads)
    head_dim: int
    value_dim: int
    conv_taps: int
    norm_eps: float
    prefix: str
    kind: str = "gated_delta_rule"


@dataclass(frozen=True)
class GeneralDeltaSpec:
    """Generalized delta rule: per head a [head_dim, head_dim] state S with a decay and a removal rate per key
    channel, S = diag(w) S - (a u)(u^T S) + k v^T with the unit key u, o = S^T r;
    w = exp(-decay_rate sigmoid(w2 tanh(w1 x) + w0)), a = sigmoid(a x + a.b); each head's o is RMS-normed, the
    concatenated heads are weighted by ``norm`` and gated by sigmoid(g x).
    Tensors: <prefix>{r,k,v,g,a,o}, <prefix>a.b, <prefix>w1 [rank, hidden], <prefix>w2 [H*D, rank], <prefix>w0,
    <prefix>norm [H*D]."""

    hidden: int
    n_heads: int
    head_dim: int
    decay_rank: int
    decay_rate: float
    norm_eps: float
    prefix: str
    kind: str = "general_delta_rule"


@dataclass(frozen=True)
class InputConvSpec:
    """A mixer that reads x + conv(x) instead of x: a causal convolution over time on every channel,
    conv(x)_t = sum_j w[:, j] x_(t - taps + 1 + j), zeros before the request's start; ``name``: the [channels, taps]
    weight tensor's full name.  The last taps - 1 inputs are part of the request's state."""

    mixer: object
    channels: int
    taps: int
    name: str
    kind: str = "input_conv"


@dataclass(frozen=True)
class DecayedLinearAttentionSpec:
    """Linear attention with one fixed decay per head: S = d S + k v^T, o = S^T q on SiLU(q, k, v); the heads'
    read-outs are RMS-normed together and gated by a sigmoid.  Tensors: <prefix>{q,k,v,g,o}, <prefix>norm."""

    hidden: int
    n_heads: int
    head_dim: int
    value_dim: int
    decay: Tuple[float, ...]
    norm_eps: float
    prefix: str
    kind: str = "decayed_linear_attention"


@dataclass(frozen=True)
class MixerSumSpec:
    """Several mixers read the same input; the result is sum_i scales[i] * mixers[i](x)."""

    mixers: Tuple[object, ...]
    scales: Tuple[float, ...]
    kind: str = "mixer_sum"


@dataclass(frozen=True)
class DenseMlpSpec:
    hidden: int
    intermediate: int
    prefix: str  # tensors: <prefix>{gate,up,down}_proj.weight
    kind: str = "swiglu_mlp"
    activation: str = "silu"  # what the gate passes through: silu or relu
    tensor_names: Optional[Tuple[str, str, str]] = None  # (gate, up, down) after <prefix>, if spelled differently
    bias_names: Optional[Tuple[str, str, str]] = None  # (gate, up, down) biases after <prefix>; None: no biases


@dataclass(frozen=True)
class PlainMlpSpec:
    """down(act(up x)) without a gate; act: relu_square (max(z, 0)^2).  Tensors <prefix>{up,down} unless
    ``tensor_names`` spells them differently."""

    hidden: int
    intermediate: int
    prefix: str
    activation: str = "relu_square"
    tensor_names: Optional[Tuple[str, str]] = None
    kind: str = "plain_mlp"


@dataclass(frozen=True)
class MoeSpec:
    hidden: int
    n_experts: int
    top_k: int
    expert_intermediate: int
    shared_intermediate: int  # 0 = no shared expert
    norm_topk_prob: bool
    shared_gate: bool  # sigmoid(w . x) scales the shared expert's output
    prefix: str  # tensors: <prefix>gate.weight, <prefix>experts.<e>.{gate,up,down}_proj.weight,
    #                       <prefix>shared_expert.{gate,up,down}_proj.weight, <prefix>shared_expert_gate.weight
    kind: str = "softmax_topk_moe"
    scores: str = "softmax"  # what the router's logits become: softmax over all experts, or sigmoid of each
    weight_on_input: bool = False  # the routing weight multiplies the expert's input instead of its output
    # what the gate passes through: a name the kernels know, or (name, limit, alpha) for the clamped unit
    activation: object = "silu"
    shared_activation: object = None  # the shared expert's, where it differs
    # names after <prefix> where a checkpoint spells them differently: (router, expert pattern with {e} and {part},
    # shared pattern with {part}), part being gate, up or down
    tensor_names: Optional[Tuple[str, str, str]] = None
    # experts without a gate: down(act(up x)) with act one of the plain products' activations (e.g. "relu_square");
    # None: gated experts.  The shared expert has the same form.
    plain_activation: Optional[str] = None
    choice_bias: Optional[str] = None  # name after <prefix> of a [n_experts] vector added to the scores for the CHOICE
    #                                    only (sigmoid scores); the weights use the scores without it
    weight_scale: float = 1.0  # the final weights are multiplied by this
    renorm_eps: float = 0.0  # added to the sum the kept scores are divided by (norm_topk_prob)
    shared_gate_name: Optional[str] = None  # name after <prefix> of the shared expert's [1, hidden] gate row


@dataclass(frozen=True)
class BlockSpec:
    """h += mixer(norm1(h)); h += ffn(norm2(h)).  ``ffn`` None: the layer ends after the mixer (and has no norm2);
    ``unused_tensors``: (name, shape) of tensors a checkpoint may carry for the layer all the same."""

    norm1: object
    mixer: object
    norm2: Optional[object]
    ffn: Optional[object]
    kind: str = "pre_norm"
    unused_tensors: Tuple[Tuple[str, Tuple[int, ...]], ...] = ()


@dataclass(frozen=True)
class ParallelBlockSpec:
    """One norm, both sublayers read its output: h += mixer(norm1(h)) + ffn(norm1(h)).  ``ffn`` None: no
    feed-forward."""

    norm1: object
    mixer: object
    ffn: Optional[object]
    kind: str = "parallel"
    # h += residual_mult * (mixer(norm1(h)) + ffn(norm1(h))): the sum of the sublayers is made in a 32-bit buffer,
    # multiplied and added (1.0: the sublayers add to the stream themselves)
    residual_mult: float = 1.0


@dataclass(frozen=True)
class SandwichBlockSpec:
    """A norm before and after each sublayer: h += post1(mixer(norm1(h))); h += post2(ffn(norm2(h))).
    ``ffn`` None: the layer has no feed-forward (and no norm2 / post2)."""

    norm1: object
    mixer: object
    post1: object
    norm2: Optional[object]
    ffn: Optional[object]
    post2: Optional[object]
    kind: str = "sandwich_norm"


@dataclass(frozen=True)
class ScheduleEntry:
    """One call in the order of execution: run ``layer`` against cache ``cache``.

    ``layer`` may appear in several entries (the same weights run twice) and two
    entries may name the same ``cache`` (the later one reads what the earlier one
    wrote, with ``writes_cache=False``)."""

    layer: int
    cache: int
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden: int
    max_positions: int
    layers: Tuple[BlockSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: object
    embedding_name: str = "model.embed_tokens.weight"
    head_name: Optional[str] = "lm_head.weight"  # None = tied to the embedding
    eos_token_ids: Tuple[int, ...] = field(default_factory=tuple)
    embedding_norm: Optional[object] = None  # a norm applied to the embedding rows (the stream stays 32-bit)
    logit_scale: float = 1.0  # the head's output is multiplied by this
    position_table: Optional[str] = None  # a learned [max_positions, hidden] table: row p is added to position p's embedding
    logit_softcap: Optional[float] = None  # c: the logits pass through c * tanh(z / c)
    embedding_scale: float = 1.0  # the embedding rows are multiplied by this

    @property
    def n_caches(self) -> int:
        return 1 + max((e.cache for e in self.schedule), default=-1)
