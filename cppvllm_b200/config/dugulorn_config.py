"""Typed configuration of the Dugulorn decoder, read from its ``config.json``.

Top level: ``vocab``, ``width``, ``norm.eps`` and ``layers``, a list with one entry per layer: ``type`` (which mixer:
``latent_attention``, ``lightning`` or ``channel_delta``), ``mixer`` (its sizes and constants) and ``mlp`` (``null`` or a dense
one with ``ff``).  Layers need not be alike and come in any order.  A latent-attention mixer may name ``kv_from``: an earlier
latent-attention layer with a down-projection of its own whose cache entries it reads.  Every size and constant is taken
from the file; a missing required key, an unknown kind or sizes that contradict one another raise ``ConfigError``.
Optional keys that only the random-weights writer needs: ``mixer.a_rank`` and ``mixer.g_rank`` of a channel_delta mixer (the
inner sizes of its two low-rank projections, which a checkpoint's tensors fix otherwise), ``max_positions`` and
``eos_token_id``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple, Union

from .givirax_config import _get
from .model_config import ConfigError


@dataclass(frozen=True)
class RotationConfig:
    dims: int
    base: float
    factor: float = 1.0          # 1 with original == 0: no stretching
    original: float = 0.0
    fast: float = 0.0
    slow: float = 0.0


@dataclass(frozen=True)
class LatentAttentionConfig:
    heads: int
    dim: int                     # unrotated query/key elements per head
    rot_dim: int                 # rotated query/key elements per head (the key's are shared by the heads)
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    rot: RotationConfig
    kv_from: Optional[int] = None


@dataclass(frozen=True)
class LightningConfig:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]


@dataclass(frozen=True)
class ChannelDeltaConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    a_rank: Optional[int] = None
    g_rank: Optional[int] = None


@dataclass(frozen=True)
class DugulornLayerConfig:
    type: str
    mixer: Union[LatentAttentionConfig, LightningConfig, ChannelDeltaConfig]
    ff: int = 0                  # 0: the layer has no feed-forward


@dataclass(frozen=True)
class DugulornConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[DugulornLayerConfig, ...]
    max_positions: int = 0
    eos_token_ids: tuple = ()
    architecture: str = "Dugulorn"

    @staticmethod
    def from_dict(d: Mapping[str, Any]) -> "DugulornConfig":
        layers = d.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        parsed = []
        for i, entry in enumerate(layers):
            where = f"layers[{i}]."
            kind = _get(entry, "type", str, where)
            m = entry.get("mixer")
            if not isinstance(m, Mapping):
                raise ConfigError(f"config.json: required key '{where}mixer' is missing")
            w = where + "mixer."
            if kind == "latent_attention":
                r = m.get("rot")
                if not isinstance(r, Mapping):
                    raise ConfigError(f"config.json: required key '{w}rot' is missing")
                sc = r.get("scaling") or {}
                rot = RotationConfig(dims=_get(r, "dims", int, w + "rot."), base=_get(r, "base", float, w + "rot."),
                                     factor=_get(sc, "factor", float, w + "rot.scaling.", 1.0, required=bool(sc)),
                                     original=_get(sc, "original", float, w + "rot.scaling.", 0.0, required=bool(sc)),
                                     fast=_get(sc, "fast", float, w + "rot.scaling.", 0.0, required=bool(sc)),
                                     slow=_get(sc, "slow", float, w + "rot.scaling.", 0.0, required=bool(sc)))
                mixer = LatentAttentionConfig(
                    heads=_get(m, "heads", int, w), dim=_get(m, "dim", int, w), rot_dim=_get(m, "rot_dim", int, w),
                    vdim=_get(m, "vdim", int, w), q_rank=_get(m, "q_rank", int, w), kv_rank=_get(m, "kv_rank", int, w),
                    scale=_get(m, "scale", float, w), rot=rot, kv_from=_get(m, "kv_from", int, w, None, required=False))
                if min(mixer.heads, mixer.dim, mixer.rot_dim, mixer.vdim, mixer.q_rank, mixer.kv_rank) <= 0:
                    raise ConfigError(f"config.json: {w}: sizes must be positive")
                if rot.dims <= 0 or rot.dims % 2 or rot.dims > mixer.rot_dim or rot.base <= 1.0:
                    raise ConfigError(f"config.json: {w}rot: {rot.dims} rotated elements (even, at most rot_dim = {mixer.rot_dim}), base {rot.base}")
                if sc and (rot.factor <= 0 or rot.original <= 0 or rot.fast <= 0 or rot.slow <= 0):
                    raise ConfigError(f"config.json: {w}rot.scaling: factor, original, fast and slow must be positive")
                if mixer.kv_from is not None:
                    j = mixer.kv_from
                    src = parsed[j].mixer if 0 <= j < i else None
                    if not isinstance(src, LatentAttentionConfig) or src.kv_from is not None:
                        raise ConfigError(f"config.json: {w}kv_from = {j} must name an earlier latent_attention layer that has "
                                          "a down-projection of its own")
                    if (src.kv_rank, src.rot_dim, src.rot) != (mixer.kv_rank, mixer.rot_dim, mixer.rot):
                        raise ConfigError(f"config.json: {w}kv_from = {j}: kv_rank, rot_dim and rot must equal that layer's")
            elif kind == "lightning":
                decay = m.get("decay")
                if not isinstance(decay, (list, tuple)):
                    raise ConfigError(f"config.json: required key '{w}decay' is missing (one number per head)")
                mixer = LightningConfig(heads=_get(m, "heads", int, w), dim=_get(m, "dim", int, w), vdim=_get(m, "vdim", int, w),
                                        decay=tuple(float(x) for x in decay))
                if min(mixer.heads, mixer.dim, mixer.vdim) <= 0 or len(mixer.decay) != mixer.heads:
                    raise ConfigError(f"config.json: {w}: {mixer.heads} heads of {mixer.dim} x {mixer.vdim} with {len(mixer.decay)} decays")
            elif kind == "channel_delta":
                heads = _get(m, "heads", int, w)
                mixer = ChannelDeltaConfig(heads=heads, kv_heads=_get(m, "kv_heads", int, w, heads, required=False),
                                           dim=_get(m, "dim", int, w), vdim=_get(m, "vdim", int, w), conv=_get(m, "conv", int, w),
                                           a_rank=_get(m, "a_rank", int, w, None, required=False),
                                           g_rank=_get(m, "g_rank", int, w, None, required=False))
                if min(mixer.heads, mixer.kv_heads, mixer.dim, mixer.vdim, mixer.conv) <= 0 or mixer.heads % mixer.kv_heads:
                    raise ConfigError(f"config.json: {w}: {mixer.heads} heads over {mixer.kv_heads} query/key heads, "
                                      f"{mixer.dim} x {mixer.vdim}, {mixer.conv} taps")
            else:
                raise ConfigError(f"config.json: {where}type '{kind}' is not a mixer of this design; known: latent_attention, "
                                  "lightning, channel_delta")
            f = entry.get("mlp")
            ff = 0
            if f is not None:
                fk = _get(f, "kind", str, where + "mlp.")
                if fk != "dense":
                    raise ConfigError(f"config.json: {where}mlp.kind '{fk}' is unknown; known: dense")
                ff = _get(f, "ff", int, where + "mlp.")
                if ff <= 0:
                    raise ConfigError(f"config.json: {where}mlp: inner size must be positive")
            parsed.append(DugulornLayerConfig(kind, mixer, ff))
        eos = d.get("eos_token_id")
        eos = tuple(int(x) for x in eos) if isinstance(eos, (list, tuple)) else ((int(eos),) if eos is not None else ())
        cfg = DugulornConfig(vocab=_get(d, "vocab", int, ""), width=_get(d, "width", int, ""),
                             norm_eps=_get(d.get("norm") or {}, "eps", float, "norm."), layers=tuple(parsed),
                             max_positions=_get(d, "max_positions", int, "", 0, required=False), eos_token_ids=eos)
        if cfg.vocab <= 0 or cfg.width <= 0:
            raise ConfigError("config.json: vocab and width must be positive")
        return cfg
