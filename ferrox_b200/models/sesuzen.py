"""Sesuzen as a description made of parts.

A decoder with a learned position vector added to every embedding row, pre-norm layers whose norms are layer norms
with weight and bias, and a short causal convolution in front of every mixer:

    x = norm1(h);  x <- x + conv(x);  h += mixer(x);  h += ffn(norm2(h))             (ffn may be absent)

* ``attention``: grouped-query attention without rotation; biased q, k, v projections; every value head divided by
  its root mean square (and cached so); score scale from the configuration; a sliding window that keeps the first
  positions of a request visible: query i sees key j when j <= i and (i - j < size or j < keep_first); softmax; the
  heads' outputs gated by sigmoid(g x) before the output projection.
* ``general_delta``: a generalized delta rule with a matrix state per head (``parts/linear_state.py``).
* feed-forward: ``dense`` = down(relu(up x)^2); ``moe`` = the ``top`` experts with the largest router logits, weighted
  by the softmax over the chosen logits, each down(silu(gate x) * (up x)).
* ``loop``: layers start .. stop - 1 run ``times`` times in a row with the same weights: one block, several schedule
  entries, every pass with a cache of its own.
* output: the model's layer norm, the embedding table as the head, then c tanh(z / c).

Tensor names: ``embed``, ``pos``, ``l<i>.{norm1,norm2}`` (+ ``.b``), ``l<i>.canon1``, ``l<i>.mix.*``,
``l<i>.mlp.{up,down}`` or ``l<i>.mlp.{router, e<k>.{gate,up,down}}``, ``final.norm`` (+ ``.b``).
"""
from __future__ import annotations

import math

from ..config.registry import register_architecture
from ..config.sesuzen import ARCHITECTURE, AttentionConfig, DeltaConfig, DenseConfig, MoeConfig, SesuzenConfig
from ..parts.specs import (
    AttentionSpec,
    BlockSpec,
    GeneralDeltaSpec,
    InputConvSpec,
    LayerNormSpec,
    ModelSpec,
    MoeSpec,
    PlainMlpSpec,
    ScheduleEntry,
)

DECAY_RATE = math.exp(-0.5)     # a key channel's decay is exp(-DECAY_RATE * sigmoid(.)): never below exp(-DECAY_RATE)


def _norm(cfg: SesuzenConfig, name: str) -> LayerNormSpec:
    return LayerNormSpec(cfg.width, cfg.norm_eps, name, bias_name=name + ".b")


def _mixer(cfg: SesuzenConfig, m, prefix: str, shapes: dict):
    W, eps = cfg.width, cfg.norm_eps
    if isinstance(m, AttentionConfig):
        return AttentionSpec(
            hidden=W, n_heads=m.heads, n_kv_heads=m.kv_heads, head_dim=m.dim, qkv_bias=True, position=None,
            window=m.window, prefix=prefix, softmax_scale=m.scale, value_dim=m.vdim,
            tensor_names=(("q", "q"), ("k", "k"), ("v", "v"), ("o", "o"), ("q_bias", "q.b"), ("k_bias", "k.b"),
                          ("v_bias", "v.b")),
            value_norm_eps=eps, keep_first=m.keep_first if m.window is not None else 0, output_gate="g",
        )
    assert isinstance(m, DeltaConfig)
    return GeneralDeltaSpec(hidden=W, n_heads=m.heads, head_dim=m.dim, decay_rank=shapes["decay_rank"],
                            decay_rate=DECAY_RATE, norm_eps=eps, prefix=prefix)


def _ffn(cfg: SesuzenConfig, f, prefix: str):
    if f is None:
        return None
    if isinstance(f, DenseConfig):
        return PlainMlpSpec(hidden=cfg.width, intermediate=f.ff, prefix=prefix, activation="relu_square")
    assert isinstance(f, MoeConfig)
    # softmax over the chosen logits only = the softmax over all experts, renormalised over the chosen ones
    return MoeSpec(hidden=cfg.width, n_experts=f.experts, top_k=f.top, expert_intermediate=f.ff, shared_intermediate=0,
                   norm_topk_prob=True, shared_gate=False, prefix=prefix,
                   tensor_names=("router", "e{e}.{part}", "shared.{part}"))


DEFAULT_DECAY_RANK = 16


def model_spec(cfg: SesuzenConfig, tensor_shapes=None) -> ModelSpec:
    """``tensor_shapes`` (name -> shape, optional): the checkpoint's, for the one size that ``config.json`` leaves to
    them (the inner width of a general_delta layer's decay, the rows of ``l<i>.mix.w1``); without a checkpoint the
    mixer's optional ``decay_rank`` key or DEFAULT_DECAY_RANK says it."""
    W = cfg.width
    blocks = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        rank = getattr(layer.mixer, "decay_rank", None) or DEFAULT_DECAY_RANK
        if tensor_shapes is not None and p + "mix.w1" in tensor_shapes:
            rank = int(tensor_shapes[p + "mix.w1"][0])
        mixer = _mixer(cfg, layer.mixer, p + "mix.", {"decay_rank": rank})
        ffn = _ffn(cfg, layer.mlp, p + "mlp.")
        blocks.append(BlockSpec(
            norm1=_norm(cfg, p + "norm1"),
            mixer=InputConvSpec(mixer=mixer, channels=W, taps=cfg.taps, name=p + "canon1"),
            norm2=_norm(cfg, p + "norm2") if ffn is not None else None,
            ffn=ffn,
            unused_tensors=() if ffn is not None else ((p + "norm2", (W,)), (p + "norm2.b", (W,))),
        ))
    return ModelSpec(
        architecture=ARCHITECTURE,
        vocab_size=cfg.vocab,
        hidden=W,
        max_positions=cfg.max_positions,
        layers=tuple(blocks),
        # every run of a layer has a cache of its own, also the passes of the loop over the same weights
        schedule=tuple(ScheduleEntry(layer=l, cache=run) for run, l in enumerate(cfg.layer_runs())),
        final_norm=_norm(cfg, "final.norm"),
        embedding_name="embed",
        head_name=None,
        position_table="pos",
        logit_softcap=cfg.logit_softcap,
    )


register_architecture(ARCHITECTURE, SesuzenConfig.from_json, model_spec, replace=True, reads_shapes=True)
