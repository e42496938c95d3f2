"""Typed configuration of the Sesuzen design, read from its own ``config.json``.

The file is nested like Safepel's and Bobepel's: ``layers`` lists the layers in order, each with its ``type`` (which
mixer: ``attention`` or ``general_delta``), the mixer's sizes and constants under ``mixer`` and its feed-forward under
``mlp`` (``kind`` ``dense`` or ``moe``; null: none).  ``loop`` (optional) names a run of layers ``start .. stop - 1``
that runs ``times`` times in a row with the same weights.  ``canon.taps`` is the length of the causal convolution in
front of every mixer, ``norm.eps`` the constant of every norm, ``logit_softcap`` the cap of the logits (absent: none),
``max_positions`` the rows of the learned position table.  Every size and every constant that differs between models of
the design is read from the file; nothing is assumed about how many layers of which type there are or in which order.
A key that is not listed is ignored; a layer type, a feed-forward kind or a value that the engine does not implement is
refused by name.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from .schema import ConfigError, Key, non_negative, positive, read_keys

ARCHITECTURE = "Sesuzen"

_TOP = (
    Key("vocab", int, check=positive),
    Key("width", int, check=positive),
    Key("layers", list),
    Key("norm", object),
    Key("canon", object),
    Key("max_positions", int, check=positive),
    Key("loop", object, default=None, nullable=True),
    Key("logit_softcap", float, default=None, nullable=True, check=positive),
)
_ATTENTION = (
    Key("heads", int, check=positive), Key("kv_heads", int, default=lambda v: v["heads"], check=positive),
    Key("dim", int, check=positive), Key("vdim", int, default=lambda v: v["dim"], check=positive), Key("scale", float),
    Key("mask", object, default=None, nullable=True),
)
_DELTA = (Key("heads", int, check=positive), Key("dim", int, check=positive),
          Key("decay_rank", int, default=None, nullable=True, check=positive))
_MASK = (Key("size", int, check=positive), Key("keep_first", int, default=0, check=non_negative))
_LOOP = (Key("start", int, check=non_negative), Key("stop", int, check=non_negative), Key("times", int, check=positive))
_ROUTER = (Key("experts", int, check=positive), Key("top", int, check=positive))


@dataclass(frozen=True)
class AttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: Optional[int]     # None: every earlier position
    keep_first: int           # with a window: the first positions that stay visible


@dataclass(frozen=True)
class DeltaConfig:
    heads: int
    dim: int
    decay_rank: Optional[int] = None   # inner width of the decay's two matrices; a checkpoint's tensor shapes say it


@dataclass(frozen=True)
class DenseConfig:
    ff: int


@dataclass(frozen=True)
class MoeConfig:
    experts: int
    top: int
    ff: int


@dataclass(frozen=True)
class LayerConfig:
    type: str                 # attention | general_delta
    mixer: object             # AttentionConfig | DeltaConfig
    mlp: Optional[object]     # DenseConfig | MoeConfig | None


@dataclass(frozen=True)
class SesuzenConfig:
    vocab: int
    width: int
    norm_eps: float
    taps: int
    max_positions: int
    logit_softcap: Optional[float]
    loop: Optional[Tuple[int, int, int]]      # (start, stop, times)
    layers: Tuple[LayerConfig, ...]

    def layer_runs(self) -> Tuple[int, ...]:
        """The order in which the layers run: the looped run ``times`` times in a row, the rest once."""
        n = len(self.layers)
        if self.loop is None:
            return tuple(range(n))
        a, b, times = self.loop
        return tuple(range(a)) + tuple(range(a, b)) * times + tuple(range(b, n))

    @classmethod
    def from_json(cls, obj: dict) -> "SesuzenConfig":
        v = read_keys(obj, _TOP)
        if not isinstance(v["norm"], dict):
            raise ConfigError("config.json: norm must be an object with 'eps'")
        eps = read_keys(v["norm"], (Key("eps", float, check=positive),), where="config.json: norm")["eps"]
        if not isinstance(v["canon"], dict):
            raise ConfigError("config.json: canon must be an object with 'taps'")
        taps = read_keys(v["canon"], (Key("taps", int, check=positive),), where="config.json: canon")["taps"]
        layers = []
        for i, raw in enumerate(v["layers"]):
            where = f"config.json: layers[{i}]"
            if not isinstance(raw, dict):
                raise ConfigError(f"{where}: must be an object")
            lv = read_keys(raw, (Key("type", str), Key("mixer", object), Key("mlp", object, default=None, nullable=True)),
                           where=where)
            if not isinstance(lv["mixer"], dict):
                raise ConfigError(f"{where}: mixer must be an object")
            if lv["type"] == "attention":
                mixer = _attention(lv["mixer"], where + ".mixer")
            elif lv["type"] == "general_delta":
                m = read_keys(lv["mixer"], _DELTA, where=where + ".mixer")
                mixer = DeltaConfig(heads=m["heads"], dim=m["dim"], decay_rank=m["decay_rank"])
            else:
                raise ConfigError(f"{where}: layer type {lv['type']!r} is not implemented (attention, general_delta)")
            layers.append(LayerConfig(lv["type"], mixer, _mlp(lv["mlp"], where + ".mlp") if lv["mlp"] is not None else None))
        if not layers:
            raise ConfigError("config.json: layers is empty")
        loop = None
        if v["loop"] is not None:
            if not isinstance(v["loop"], dict):
                raise ConfigError("config.json: loop must be an object with 'start', 'stop' and 'times', or null")
            lp = read_keys(v["loop"], _LOOP, where="config.json: loop")
            if not lp["start"] <= lp["stop"] <= len(layers):
                raise ConfigError(f"config.json: loop: layers {lp['start']} .. {lp['stop']} - 1 of {len(layers)}")
            if lp["stop"] > lp["start"] and lp["times"] != 1:
                loop = (lp["start"], lp["stop"], lp["times"])
        return cls(vocab=v["vocab"], width=v["width"], norm_eps=eps, taps=taps, max_positions=v["max_positions"],
                   logit_softcap=v["logit_softcap"], loop=loop, layers=tuple(layers))


def _attention(raw: dict, where: str) -> AttentionConfig:
    m = read_keys(raw, _ATTENTION, where=where)
    if m["heads"] % m["kv_heads"]:
        raise ConfigError(f"{where}: heads must be a multiple of kv_heads")
    window, keep = None, 0
    if m["mask"] is not None:
        if not isinstance(m["mask"], dict):
            raise ConfigError(f"{where}: mask must be an object with 'size' (and 'keep_first'), or null")
        mk = read_keys(m["mask"], _MASK, where=where + ".mask")
        window, keep = mk["size"], mk["keep_first"]
    return AttentionConfig(heads=m["heads"], kv_heads=m["kv_heads"], dim=m["dim"], vdim=m["vdim"], scale=m["scale"],
                           window=window, keep_first=keep)


def _mlp(raw, where: str):
    if not isinstance(raw, dict):
        raise ConfigError(f"{where}: must be an object or null")
    kind = read_keys(raw, (Key("kind", str),), where=where)["kind"]
    if kind == "dense":
        return DenseConfig(ff=read_keys(raw, (Key("ff", int, check=positive),), where=where)["ff"])
    if kind != "moe":
        raise ConfigError(f"{where}: kind {kind!r} is not implemented (dense, moe)")
    m = read_keys(raw, (Key("expert", object), Key("router", object)), where=where)
    for key in ("expert", "router"):
        if not isinstance(m[key], dict):
            raise ConfigError(f"{where}.{key}: must be an object")
    e = read_keys(m["expert"], (Key("ff", int, check=positive),), where=where + ".expert")
    r = read_keys(m["router"], _ROUTER, where=where + ".router")
    if r["top"] > r["experts"]:
        raise ConfigError(f"{where}.router: top={r['top']} exceeds experts={r['experts']}")
    return MoeConfig(experts=r["experts"], top=r["top"], ff=e["ff"])
