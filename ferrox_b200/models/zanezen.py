"""Zanezen as a description made of parts.

A decoder whose layers, in whatever order ``config.json`` lists them, run one RMS norm and add, times a constant,
a mixer and a feed-forward that both read it; the embedding rows are multiplied by a constant:

    x = norm1(h);   h += residual_mult (mixer(x) + ffn(x))

* ``mlstm``: a matrix memory per head with an input and a forget gate in the logarithm, both capped, and a running
  maximum that keeps the exponentials in range; the read-out is RMS-normed per head, weighted and gated.
* ``attention``: differential attention on grouped query heads: two maps a head over the same values, the second
  taken off the first times one number of the layer; a short causal convolution on q, k and v behind their
  projections; part of each map rotated on pairs (i, i + dims/2) at frequencies that may be stretched for long
  contexts; capped scores; the heads' results RMS-normed without a weight.
* ``latent_attention``: a position caches one normed latent vector and one rotated key part that all heads share; a
  learned number per head in the softmax's denominator; one output gate per head.
* feed-forward: gated with SiLU and biases on all three projections, or experts without a gate (the square of ReLU)
  chosen by the largest sigmoid score plus a correction per expert; the weights are the chosen scores without the
  correction, divided by their sum, times a constant; a shared expert of the same form, gated by a sigmoid, is added
  for every token.

Tensor names: ``embed``, ``l<i>.norm1``, ``l<i>.mix.*``, ``l<i>.mlp.{gate,up,down}(.b)`` or ``l<i>.mlp.{router,
correction, e<k>.{up,down}, shared.{up,down,sg}}``, ``final.norm``, ``head``.
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.zanezen import (
    ARCHITECTURE,
    AttentionConfig,
    DenseConfig,
    LatentAttentionConfig,
    MlstmConfig,
    ZanezenConfig,
)
from ..parts.specs import (
    DenseMlpSpec,
    DifferentialAttentionSpec,
    LatentAttentionSpec,
    MlstmSpec,
    ModelSpec,
    MoeSpec,
    NormSpec,
    ParallelBlockSpec,
    ScaledRotarySpec,
    ScheduleEntry,
)

RENORM_EPS = 1e-20          # added to the sum of the chosen experts' scores before they are divided by it
EXPERT_ACTIVATION = "relu_square"


def _scaled_rotary(rot):
    f, o, fa, sl = rot.scaling if rot.scaling is not None else (None, 0.0, 0.0, 0.0)
    return ScaledRotarySpec(rotary_dim=rot.dims, theta=rot.base, factor=f, original=o, fast=fa, slow=sl)


def _mixer(cfg: ZanezenConfig, m, prefix: str):
    W, eps = cfg.width, cfg.norm_eps
    if isinstance(m, MlstmConfig):
        return MlstmSpec(hidden=W, n_heads=m.heads, head_dim=m.dim, value_dim=m.vdim, gate_cap=m.gate_cap, norm_eps=eps,
                         prefix=prefix)
    if isinstance(m, AttentionConfig):
        return DifferentialAttentionSpec(
            hidden=W, n_heads=m.heads, n_kv_heads=m.kv_heads, head_dim=m.dim, value_dim=m.vdim, diff=m.diff,
            scale=m.scale, softcap=m.softcap, conv_taps=m.conv,
            position=_scaled_rotary(m.rot) if m.rot is not None else None, norm_eps=eps, prefix=prefix)
    assert isinstance(m, LatentAttentionConfig)
    return LatentAttentionSpec(
        hidden=W, n_heads=m.heads, head_dim=m.dim, rot_dim=m.rot_dim, value_dim=m.vdim, kv_rank=m.kv_rank, q_rank=None,
        rotary_dims=m.rot.dims, rotary_base=m.rot.base, window=None, scale=m.scale, output_gate=True, norm_eps=eps,
        prefix=prefix, rotary_pairing="halves", rotary_scaling=m.rot.scaling, gate_per_head=True, sink="sink")


def _ffn(cfg: ZanezenConfig, f, prefix: str):
    if f is None:
        return None
    if isinstance(f, DenseConfig):
        return DenseMlpSpec(hidden=cfg.width, intermediate=f.ff, prefix=prefix, activation="silu",
                            tensor_names=("gate", "up", "down"), bias_names=("gate.b", "up.b", "down.b"))
    return MoeSpec(
        hidden=cfg.width, n_experts=f.experts, top_k=f.top, expert_intermediate=f.ff, shared_intermediate=f.shared_ff,
        norm_topk_prob=True, shared_gate=f.shared_ff > 0, prefix=prefix, scores="sigmoid",
        tensor_names=("router", "e{e}.{part}", "shared.{part}"), plain_activation=EXPERT_ACTIVATION,
        choice_bias="correction", weight_scale=f.scale, renorm_eps=RENORM_EPS, shared_gate_name="shared.sg")


def model_spec(cfg: ZanezenConfig) -> ModelSpec:
    W, eps = cfg.width, cfg.norm_eps
    blocks = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        blocks.append(ParallelBlockSpec(
            norm1=NormSpec(W, eps, p, name=p + "norm1"),
            mixer=_mixer(cfg, layer.mixer, p + "mix."),
            ffn=_ffn(cfg, layer.mlp, p + "mlp."),
            residual_mult=cfg.residual_mult,
        ))
    return ModelSpec(
        architecture=ARCHITECTURE,
        vocab_size=cfg.vocab,
        hidden=W,
        max_positions=cfg.max_positions,
        layers=tuple(blocks),
        schedule=tuple(ScheduleEntry(layer=i, cache=i) for i in range(len(blocks))),
        final_norm=NormSpec(W, eps, "final.", name="final.norm"),
        embedding_name="embed",
        head_name="head",
        embedding_scale=cfg.embedding_scale,
    )


register_architecture(ARCHITECTURE, ZanezenConfig.from_json, model_spec, replace=True)
