"""Typed configuration of the Givirax decoder, read from its ``config.json``.

The file is nested: ``vocab``, ``width``, ``max_positions``, ``embedding.scale``, ``norm.eps``, an optional ``loop``
(``start``, ``stop``, ``times``: layers start..stop-1 run ``times`` times in a row) and ``layers``, a list with one
entry per layer: ``type`` (the mixer), ``mixer`` (its sizes and constants) and ``mlp`` (``null``, a dense one with
``ff``, or a routed one with ``expert.ff``, ``router.experts`` and ``router.top``).  Layers need not be alike.
Every size and constant is taken from the file; a missing required key or an unknown kind raises ``ConfigError``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .model_config import ConfigError


def _get(d: Mapping[str, Any], key: str, typ, where: str, default=None, required: bool = True):
    if not isinstance(d, Mapping) or key not in d or d[key] is None:
        if required:
            raise ConfigError(f"config.json: required key '{where}{key}' is missing")
        return default
    try:
        return typ(d[key])
    except (TypeError, ValueError) as e:
        raise ConfigError(f"config.json: key '{where}{key}' has a bad value {d[key]!r}") from e


@dataclass(frozen=True)
class AttentionMixerConfig:
    heads: int
    kv_heads: int
    dim: int                 # per-head size of queries and keys
    vdim: int                # per-head size of values
    scale: float
    window: int              # 0: every earlier position is visible
    keep_first: int          # with a window: the first positions that stay visible


@dataclass(frozen=True)
class MlpConfig:
    kind: str                # "dense" or "moe"
    ff: int                  # inner size (of one expert, for "moe")
    experts: int = 0
    top: int = 0


@dataclass(frozen=True)
class GiviraxLayerConfig:
    type: str
    mixer: AttentionMixerConfig
    mlp: Optional[MlpConfig]


@dataclass(frozen=True)
class GiviraxConfig:
    vocab: int
    width: int
    max_positions: int
    embedding_scale: float
    norm_eps: float
    layers: Tuple[GiviraxLayerConfig, ...]
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1
    eos_token_ids: tuple = ()
    architecture: str = "Givirax"

    @property
    def has_loop(self) -> bool:
        return self.loop_stop > self.loop_start

    @staticmethod
    def from_dict(d: Mapping[str, Any]) -> "GiviraxConfig":
        layers = d.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        parsed = []
        for i, entry in enumerate(layers):
            where = f"layers[{i}]."
            kind = _get(entry, "type", str, where)
            if kind != "attention":
                raise ConfigError(f"config.json: {where}type '{kind}' is not a mixer of this design; known: attention")
            m = entry.get("mixer")
            if not isinstance(m, Mapping):
                raise ConfigError(f"config.json: required key '{where}mixer' is missing")
            mask = m.get("mask") or {}
            heads = _get(m, "heads", int, where + "mixer.")
            dim = _get(m, "dim", int, where + "mixer.")
            mixer = AttentionMixerConfig(
                heads=heads, kv_heads=_get(m, "kv_heads", int, where + "mixer.", heads, required=False), dim=dim,
                vdim=_get(m, "vdim", int, where + "mixer.", dim, required=False),
                scale=_get(m, "scale", float, where + "mixer."),
                window=_get(mask, "size", int, where + "mixer.mask.", 0, required=False),
                keep_first=_get(mask, "keep_first", int, where + "mixer.mask.", 0, required=False))
            if mixer.heads <= 0 or mixer.kv_heads <= 0 or mixer.heads % mixer.kv_heads or mixer.dim <= 0:
                raise ConfigError(f"config.json: {where}mixer: {mixer.heads} heads over {mixer.kv_heads} key/value heads of size {mixer.dim}")
            if mixer.vdim != mixer.dim:
                raise ConfigError(f"config.json: {where}mixer: values are the keys, so vdim ({mixer.vdim}) must equal dim ({mixer.dim})")
            if mixer.window < 0 or mixer.keep_first < 0:
                raise ConfigError(f"config.json: {where}mixer.mask: sizes cannot be negative")
            f = entry.get("mlp")
            mlp = None
            if f is not None:
                fk = _get(f, "kind", str, where + "mlp.")
                if fk == "dense":
                    mlp = MlpConfig("dense", _get(f, "ff", int, where + "mlp."))
                elif fk == "moe":
                    mlp = MlpConfig("moe", _get(f.get("expert"), "ff", int, where + "mlp.expert."),
                                    experts=_get(f.get("router"), "experts", int, where + "mlp.router."),
                                    top=_get(f.get("router"), "top", int, where + "mlp.router."))
                    if not (0 < mlp.top <= mlp.experts):
                        raise ConfigError(f"config.json: {where}mlp.router: top {mlp.top} of {mlp.experts} experts")
                else:
                    raise ConfigError(f"config.json: {where}mlp.kind '{fk}' is unknown; known: dense, moe")
                if mlp.ff <= 0:
                    raise ConfigError(f"config.json: {where}mlp: inner size must be positive")
            parsed.append(GiviraxLayerConfig(kind, mixer, mlp))
        loop = d.get("loop") or {}
        start = _get(loop, "start", int, "loop.", 0, required=False)
        stop = _get(loop, "stop", int, "loop.", 0, required=False)
        times = _get(loop, "times", int, "loop.", 1, required=False)
        if loop and not (0 <= start <= stop <= len(parsed) and times >= 1):
            raise ConfigError(f"config.json: loop start {start}, stop {stop}, times {times} does not fit {len(parsed)} layers")
        eos = d.get("eos_token_id")
        eos = tuple(int(x) for x in eos) if isinstance(eos, (list, tuple)) else ((int(eos),) if eos is not None else ())
        return GiviraxConfig(
            vocab=_get(d, "vocab", int, ""), width=_get(d, "width", int, ""),
            max_positions=_get(d, "max_positions", int, ""),
            embedding_scale=_get(d.get("embedding") or {}, "scale", float, "embedding.", 1.0, required=False),
            norm_eps=_get(d.get("norm") or {}, "eps", float, "norm."),
            layers=tuple(parsed), loop_start=start, loop_stop=stop, loop_times=times, eos_token_ids=eos)
