"""Typed configuration of the Bidinex decoder, read from config.json.

config.json keys (nested objects, every size and every constant that differs between models):
    architecture            "Bidinex"
    vocab, width            vocabulary and residual width
    embedding.scale         factor on the embedding rows
    norm.eps                eps of the RMS norms inside mixers (the layers' own norms use none)
    residual_mult           factor on every mixer's and feed-forward's output before it is added
    logit_softcap           cap c of the logits: c * tanh(logits / c)
    layers[i].type          the layer's mixer: "latent_attention"
    layers[i].mixer         heads, dim, rot_dim, vdim, kv_rank, scale, rot.base, rot.dims
    layers[i].mlp           null, or kind "moe" with expert.ff and router.experts / top / groups.count / groups.keep
    loop                    null / absent, or start, stop, times: layers start .. stop-1 run `times` times in a row
A key that is missing, or a value that no part here computes, is a `ConfigError` naming key and value.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .errors import ConfigError

MIXER_TYPES = ("latent_attention",)
MLP_KINDS = ("moe",)


def _get(d: Mapping[str, Any], path: str, kind, *, minimum=None, optional: bool = False):
    cur: Any = d
    for key in path.split("."):
        if not isinstance(cur, Mapping) or key not in cur or cur[key] is None:
            if optional:
                return None
            raise ConfigError(f"config.json: required key '{path}' is missing")
        cur = cur[key]
    if kind is int:
        if isinstance(cur, bool) or not isinstance(cur, int):
            raise ConfigError(f"config.json: '{path}' must be an integer, got {cur!r}")
    elif kind is float:
        if isinstance(cur, bool) or not isinstance(cur, (int, float)):
            raise ConfigError(f"config.json: '{path}' must be a number, got {cur!r}")
        cur = float(cur)
    if minimum is not None and cur < minimum:
        raise ConfigError(f"config.json: '{path}' must be >= {minimum}, got {cur}")
    return cur


@dataclass(frozen=True)
class LatentMixerConfig:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot_base: float
    rot_dims: int


@dataclass(frozen=True)
class MoeConfig:
    ff: int
    experts: int
    top: int
    groups: int
    keep: int


@dataclass(frozen=True)
class BidinexLayerConfig:
    type: str
    mixer: LatentMixerConfig
    mlp: Optional[MoeConfig]


@dataclass(frozen=True)
class LoopConfig:
    start: int
    stop: int
    times: int


@dataclass(frozen=True)
class BidinexConfig:
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    residual_mult: float
    logit_softcap: Optional[float]
    layers: Tuple[BidinexLayerConfig, ...]
    loop: Optional[LoopConfig]
    max_position: int = 0
    eos_token_ids: Tuple[int, ...] = ()
    bos_token_id: Optional[int] = None

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "BidinexConfig":
        layers_in = d.get("layers")
        if not isinstance(layers_in, (list, tuple)) or not layers_in:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, L in enumerate(layers_in):
            at = f"layers[{i}]"
            if not isinstance(L, Mapping):
                raise ConfigError(f"config.json: '{at}' must be an object")
            kind = L.get("type")
            if kind not in MIXER_TYPES:
                raise ConfigError(f"config.json: '{at}.type' is {kind!r}; known mixers: {list(MIXER_TYPES)}")
            m = {"m": L.get("mixer")}
            rot_dim = _get(m, "m.rot_dim", int, minimum=0)
            rot_dims = _get(m, "m.rot.dims", int, minimum=0)
            if rot_dims % 2 or rot_dims > rot_dim:
                raise ConfigError(f"config.json: '{at}.mixer.rot.dims' is {rot_dims}; it must be even and at most "
                                  f"rot_dim = {rot_dim}")
            mixer = LatentMixerConfig(
                heads=_get(m, "m.heads", int, minimum=1), dim=_get(m, "m.dim", int, minimum=1), rot_dim=rot_dim,
                vdim=_get(m, "m.vdim", int, minimum=1), kv_rank=_get(m, "m.kv_rank", int, minimum=1),
                scale=_get(m, "m.scale", float), rot_base=_get(m, "m.rot.base", float), rot_dims=rot_dims)
            mlp = None
            if L.get("mlp") is not None:
                f = {"f": L["mlp"]}
                fk = _get(f, "f.kind", str)
                if fk not in MLP_KINDS:
                    raise ConfigError(f"config.json: '{at}.mlp.kind' is {fk!r}; known feed-forwards: {list(MLP_KINDS)}")
                experts = _get(f, "f.router.experts", int, minimum=1)
                groups = _get(f, "f.router.groups.count", int, minimum=1, optional=True) or 1
                keep = _get(f, "f.router.groups.keep", int, minimum=1, optional=True) or groups
                top = _get(f, "f.router.top", int, minimum=1)
                if experts % groups:
                    raise ConfigError(f"config.json: '{at}.mlp.router': {experts} experts do not form {groups} equal groups")
                if keep > groups or top > keep * (experts // groups):
                    raise ConfigError(f"config.json: '{at}.mlp.router': top {top} does not fit {keep} kept groups of "
                                      f"{experts // groups} experts (of {groups} groups)")
                mlp = MoeConfig(ff=_get(f, "f.expert.ff", int, minimum=1), experts=experts, top=top, groups=groups, keep=keep)
            layers.append(BidinexLayerConfig(kind, mixer, mlp))
        loop = None
        if d.get("loop") is not None:
            start = _get(d, "loop.start", int, minimum=0)
            stop = _get(d, "loop.stop", int, minimum=0)
            times = _get(d, "loop.times", int, minimum=1)
            if not (start < stop <= len(layers)):
                raise ConfigError(f"config.json: 'loop' runs layers {start} .. {stop} - 1 of {len(layers)}")
            loop = LoopConfig(start, stop, times)
        cap = _get(d, "logit_softcap", float, optional=True)
        if cap is not None and cap <= 0:
            raise ConfigError(f"config.json: 'logit_softcap' must be positive, got {cap}")
        eos = d.get("eos_token_id")
        eos_ids = tuple(eos) if isinstance(eos, (list, tuple)) else ((int(eos),) if isinstance(eos, int) else ())
        mult = _get(d, "residual_mult", float, optional=True)
        scale = _get(d, "embedding.scale", float, optional=True)
        return cls(vocab=_get(d, "vocab", int, minimum=1), width=_get(d, "width", int, minimum=1),
                   embedding_scale=1.0 if scale is None else scale, norm_eps=_get(d, "norm.eps", float),
                   residual_mult=1.0 if mult is None else mult, logit_softcap=cap,
                   layers=tuple(layers), loop=loop,
                   max_position=_get(d, "max_position", int, minimum=1, optional=True) or 0,
                   eos_token_ids=eos_ids, bos_token_id=d.get("bos_token_id"))

    def schedule(self):
        """The runs of layers in order, as (layer, first of a pass): the looped block `times` times, each pass
        opened by the injection; layers before and after it once."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, False) for i in range(n)]
        lp = self.loop
        runs = [(i, False) for i in range(lp.start)]
        for _ in range(lp.times):
            runs += [(i, i == lp.start) for i in range(lp.start, lp.stop)]
        runs += [(i, False) for i in range(lp.stop, n)]
        return runs
