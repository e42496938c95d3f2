"""Typed configuration of the Zanezen design, read from its own ``config.json``.

The file is nested like Safepel's, Bobepel's and Sesuzen's: ``layers`` lists the layers in order, each with its
``type`` (which mixer: ``mlstm``, ``attention`` or ``latent_attention``), the mixer's sizes and constants under
``mixer`` and its feed-forward under ``mlp`` (``kind`` ``dense`` or ``moe``; null: none).  ``embedding.scale``
multiplies the embedding rows, ``residual_mult`` the sum of a layer's two sublayers, ``norm.eps`` is the constant of
every norm.  Every size and every constant that differs between models of the design is read from the file; nothing
is assumed about how many layers of which type there are or in which order.  A key that is not listed is ignored; a
layer type, a feed-forward kind or a value that the engine does not implement is refused by name.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from .schema import ConfigError, Key, non_negative, positive, read_keys

ARCHITECTURE = "Zanezen"
DEFAULT_MAX_POSITIONS = 1 << 17   # the design has no position limit; the engine's block tables need one

_TOP = (
    Key("vocab", int, check=positive),
    Key("width", int, check=positive),
    Key("layers", list),
    Key("norm", object),
    Key("embedding", object, default=None, nullable=True),
    Key("residual_mult", float, default=1.0),
    Key("max_positions", int, default=DEFAULT_MAX_POSITIONS, check=positive),
)
_MLSTM = (
    Key("heads", int, check=positive), Key("dim", int, check=positive),
    Key("vdim", int, default=lambda v: v["dim"], check=positive), Key("gate_cap", float, check=positive),
)
_ATTENTION = (
    Key("heads", int, check=positive), Key("kv_heads", int, default=lambda v: v["heads"], check=positive),
    Key("dim", int, check=positive), Key("vdim", int, default=lambda v: v["dim"], check=positive), Key("scale", float),
    Key("diff", float), Key("softcap", float, default=None, nullable=True, check=positive),
    Key("conv", int, default=None, nullable=True, check=positive), Key("rot", object, default=None, nullable=True),
)
_LATENT = (
    Key("heads", int, check=positive), Key("dim", int, check=positive), Key("rot_dim", int, check=positive),
    Key("vdim", int, check=positive), Key("kv_rank", int, check=positive), Key("scale", float), Key("rot", object),
)
_ROT = (Key("dims", int, check=non_negative), Key("base", float, check=positive),
        Key("scaling", object, default=None, nullable=True))
_SCALING = (Key("factor", float, check=positive), Key("original", float, check=positive),
            Key("fast", float, check=positive), Key("slow", float, check=positive))
_MLP = (Key("kind", str), Key("ff", int, default=None, nullable=True, check=positive),
        Key("expert", object, default=None, nullable=True), Key("router", object, default=None, nullable=True),
        Key("shared", object, default=None, nullable=True))
_ROUTER = (Key("experts", int, check=positive), Key("top", int, check=positive), Key("scale", float, default=1.0))
_FF = (Key("ff", int, check=positive),)


@dataclass(frozen=True)
class RotaryConfig:
    dims: int
    base: float
    scaling: Optional[Tuple[float, float, float, float]]   # (factor, original, fast, slow); None: plain frequencies


@dataclass(frozen=True)
class MlstmConfig:
    heads: int
    dim: int
    vdim: int
    gate_cap: float


@dataclass(frozen=True)
class AttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    diff: float
    softcap: Optional[float]
    conv: Optional[int]            # taps of the convolution behind the projections; None: none
    rot: Optional[RotaryConfig]    # None (or dims 0): no rotation


@dataclass(frozen=True)
class LatentAttentionConfig:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot: RotaryConfig


@dataclass(frozen=True)
class DenseConfig:
    ff: int


@dataclass(frozen=True)
class MoeConfig:
    experts: int
    top: int
    scale: float
    ff: int
    shared_ff: int            # 0: no shared expert


@dataclass(frozen=True)
class LayerConfig:
    type: str                 # mlstm | attention | latent_attention
    mixer: object
    mlp: Optional[object]     # DenseConfig | MoeConfig | None


@dataclass(frozen=True)
class ZanezenConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    residual_mult: float
    max_positions: int
    layers: Tuple[LayerConfig, ...]

    @classmethod
    def from_json(cls, obj: dict) -> "ZanezenConfig":
        v = read_keys(obj, _TOP)
        if not isinstance(v["norm"], dict):
            raise ConfigError("config.json: norm must be an object with 'eps'")
        eps = read_keys(v["norm"], (Key("eps", float, check=positive),), where="config.json: norm")["eps"]
        scale = 1.0
        if v["embedding"] is not None:
            if not isinstance(v["embedding"], dict):
                raise ConfigError("config.json: embedding must be an object with 'scale'")
            scale = read_keys(v["embedding"], (Key("scale", float, default=1.0),), where="config.json: embedding")["scale"]
        layers = []
        for i, raw in enumerate(v["layers"]):
            where = f"config.json: layers[{i}]"
            if not isinstance(raw, dict):
                raise ConfigError(f"{where}: must be an object")
            lv = read_keys(raw, (Key("type", str), Key("mixer", object), Key("mlp", object, default=None, nullable=True)),
                           where=where)
            if not isinstance(lv["mixer"], dict):
                raise ConfigError(f"{where}: mixer must be an object")
            reader = _MIXERS.get(lv["type"])
            if reader is None:
                raise ConfigError(f"{where}: layer type {lv['type']!r} is not implemented ({', '.join(_MIXERS)})")
            mixer = reader(lv["mixer"], where + ".mixer")
            mlp = _mlp(lv["mlp"], where + ".mlp") if lv["mlp"] is not None else None
            layers.append(LayerConfig(lv["type"], mixer, mlp))
        if not layers:
            raise ConfigError("config.json: layers is empty")
        return cls(vocab=v["vocab"], width=v["width"], norm_eps=eps, embedding_scale=scale,
                   residual_mult=v["residual_mult"], max_positions=v["max_positions"], layers=tuple(layers))


def _rotary(raw, where: str, limit: int) -> RotaryConfig:
    if not isinstance(raw, dict):
        raise ConfigError(f"{where}: must be an object with 'dims' and 'base'")
    r = read_keys(raw, _ROT, where=where)
    if r["dims"] % 2 or r["dims"] > limit:
        raise ConfigError(f"{where}: dims must be even and at most {limit}")
    scaling = None
    if r["scaling"] is not None:
        if not isinstance(r["scaling"], dict):
            raise ConfigError(f"{where}.scaling: must be an object or null")
        s = read_keys(r["scaling"], _SCALING, where=where + ".scaling")
        if not r["base"] > 1.0:
            raise ConfigError(f"{where}: stretched frequencies need a base above 1")
        scaling = (s["factor"], s["original"], s["fast"], s["slow"])
    return RotaryConfig(dims=r["dims"], base=r["base"], scaling=scaling)


def _mlstm(raw: dict, where: str) -> MlstmConfig:
    m = read_keys(raw, _MLSTM, where=where)
    return MlstmConfig(heads=m["heads"], dim=m["dim"], vdim=m["vdim"], gate_cap=m["gate_cap"])


def _attention(raw: dict, where: str) -> AttentionConfig:
    m = read_keys(raw, _ATTENTION, where=where)
    if m["heads"] % m["kv_heads"]:
        raise ConfigError(f"{where}: heads must be a multiple of kv_heads")
    rot = _rotary(m["rot"], where + ".rot", m["dim"]) if m["rot"] is not None else None
    if rot is not None and rot.dims == 0:
        rot = None
    return AttentionConfig(heads=m["heads"], kv_heads=m["kv_heads"], dim=m["dim"], vdim=m["vdim"], scale=m["scale"],
                           diff=m["diff"], softcap=m["softcap"], conv=m["conv"], rot=rot)


def _latent(raw: dict, where: str) -> LatentAttentionConfig:
    m = read_keys(raw, _LATENT, where=where)
    rot = _rotary(m["rot"], where + ".rot", m["rot_dim"])
    return LatentAttentionConfig(heads=m["heads"], dim=m["dim"], rot_dim=m["rot_dim"], vdim=m["vdim"],
                                 kv_rank=m["kv_rank"], scale=m["scale"], rot=rot)


_MIXERS = {"mlstm": _mlstm, "attention": _attention, "latent_attention": _latent}


def _mlp(raw, where: str):
    if not isinstance(raw, dict):
        raise ConfigError(f"{where}: must be an object or null")
    m = read_keys(raw, _MLP, where=where)
    if m["kind"] == "dense":
        if m["ff"] is None:
            raise ConfigError(f"{where}: ff: required key is missing")
        return DenseConfig(ff=m["ff"])
    if m["kind"] != "moe":
        raise ConfigError(f"{where}: kind {m['kind']!r} is not implemented (dense, moe)")
    for key in ("expert", "router"):
        if not isinstance(m[key], dict):
            raise ConfigError(f"{where}.{key}: must be an object")
    e = read_keys(m["expert"], _FF, where=where + ".expert")
    r = read_keys(m["router"], _ROUTER, where=where + ".router")
    if r["top"] > r["experts"]:
        raise ConfigError(f"{where}.router: top={r['top']} exceeds experts={r['experts']}")
    shared_ff = 0
    if m["shared"] is not None:
        if not isinstance(m["shared"], dict):
            raise ConfigError(f"{where}.shared: must be an object or null")
        shared_ff = read_keys(m["shared"], _FF, where=where + ".shared")["ff"]
    return MoeConfig(experts=r["experts"], top=r["top"], scale=r["scale"], ff=e["ff"], shared_ff=shared_ff)
