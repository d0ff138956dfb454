"""Typed configuration of the Loduzen decoder, read from config.json.

config.json keys (nested objects; every size and every constant that differs between models):
    architecture            "Loduzen"
    vocab, width            vocabulary and residual width
    norm.eps                eps of every RMS norm
    token_side.dim          numbers a layer reads about each token from the side table (absent or null: none)
    layers[i].type          the layer's mixer: "parallel" (an attention beside a gated linear attention) or "mamba2"
    layers[i].mixer         "parallel": left {heads, kv_heads, dim, vdim, scale, mask.size, rot.base, rot.dims,
                                rot.scaling {factor, original, fast, slow}}, right {heads, dim, vdim, tau},
                                left_scale, right_scale
                            "mamba2": heads, vdim, state, groups, conv, norm_groups
    layers[i].mlp           null, or kind "dense" with ff
The inner size of the linear attention's decay map is given by a tensor's shape only (`l<i>.mix.right.a1` is
[gate_rank, width]): `sizes_from_shapes` writes it into the optional key `layers[i].mixer.right.gate_rank`
when a model folder is opened; without a folder (random weights) the key, or 32, is taken.
A key that is missing, or a value that no part here computes, is a `ConfigError` naming key and value.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .bidinex import _get
from .errors import ConfigError

MIXER_TYPES = ("parallel", "mamba2")
MLP_KINDS = ("dense",)
DEFAULT_GATE_RANK = 32


@dataclass(frozen=True)
class RotScalingConfig:
    factor: float
    original: float
    fast: float
    slow: float


@dataclass(frozen=True)
class WindowAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: Optional[int]
    rot_base: float
    rot_dims: int
    rot_scaling: Optional[RotScalingConfig]


@dataclass(frozen=True)
class LinearAttentionConfig:
    heads: int
    dim: int
    vdim: int
    tau: float
    gate_rank: int


@dataclass(frozen=True)
class ParallelMixerConfig:
    left: WindowAttentionConfig
    right: LinearAttentionConfig
    left_scale: float
    right_scale: float


@dataclass(frozen=True)
class Mamba2Config:
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int


@dataclass(frozen=True)
class LoduzenLayerConfig:
    type: str
    mixer: Any                       # ParallelMixerConfig | Mamba2Config
    ff: Optional[int]                # the dense feed-forward's inner size, or None for no feed-forward


@dataclass(frozen=True)
class LoduzenConfig:
    vocab: int
    width: int
    norm_eps: float
    side_dim: int                    # 0: layers have no token input of their own
    layers: Tuple[LoduzenLayerConfig, ...]
    max_position: int = 0
    eos_token_ids: Tuple[int, ...] = ()
    bos_token_id: Optional[int] = None

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "LoduzenConfig":
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
            if kind == "parallel":
                mixer = cls._parallel(m, at)
            else:
                mixer = Mamba2Config(
                    heads=_get(m, "m.heads", int, minimum=1), vdim=_get(m, "m.vdim", int, minimum=1),
                    state=_get(m, "m.state", int, minimum=1), groups=_get(m, "m.groups", int, minimum=1),
                    conv=_get(m, "m.conv", int, minimum=1), norm_groups=_get(m, "m.norm_groups", int, minimum=1))
                if mixer.heads % mixer.groups:
                    raise ConfigError(f"config.json: '{at}.mixer': {mixer.heads} heads do not form {mixer.groups} equal groups")
                if (mixer.heads * mixer.vdim) % mixer.norm_groups:
                    raise ConfigError(f"config.json: '{at}.mixer': {mixer.heads * mixer.vdim} channels do not form "
                                      f"{mixer.norm_groups} equal norm groups")
            ff = None
            if L.get("mlp") is not None:
                f = {"f": L["mlp"]}
                fk = _get(f, "f.kind", str)
                if fk not in MLP_KINDS:
                    raise ConfigError(f"config.json: '{at}.mlp.kind' is {fk!r}; known feed-forwards: {list(MLP_KINDS)}")
                ff = _get(f, "f.ff", int, minimum=1)
            layers.append(LoduzenLayerConfig(kind, mixer, ff))
        eos = d.get("eos_token_id")
        eos_ids = tuple(eos) if isinstance(eos, (list, tuple)) else ((int(eos),) if isinstance(eos, int) else ())
        side = _get(d, "token_side.dim", int, minimum=1, optional=True)
        return cls(vocab=_get(d, "vocab", int, minimum=1), width=_get(d, "width", int, minimum=1),
                   norm_eps=_get(d, "norm.eps", float), side_dim=side or 0, layers=tuple(layers),
                   max_position=_get(d, "max_position", int, minimum=1, optional=True) or 0,
                   eos_token_ids=eos_ids, bos_token_id=d.get("bos_token_id"))

    @staticmethod
    def _parallel(m, at: str) -> ParallelMixerConfig:
        dim = _get(m, "m.left.dim", int, minimum=2)
        vdim = _get(m, "m.left.vdim", int, minimum=1)
        if vdim != dim:
            raise ConfigError(f"config.json: '{at}.mixer.left': the values are the keys, so vdim = {vdim} must equal dim = {dim}")
        heads, kv = _get(m, "m.left.heads", int, minimum=1), _get(m, "m.left.kv_heads", int, minimum=1)
        if heads % kv:
            raise ConfigError(f"config.json: '{at}.mixer.left': {heads} heads do not form {kv} equal groups")
        rot_dims = _get(m, "m.left.rot.dims", int, minimum=0)
        if rot_dims % 2 or rot_dims > dim:
            raise ConfigError(f"config.json: '{at}.mixer.left.rot.dims' is {rot_dims}; it must be even and at most dim = {dim}")
        scaling = None
        if _get(m, "m.left.rot.scaling", None, optional=True) is not None:
            scaling = RotScalingConfig(*(_get(m, "m.left.rot.scaling." + k, float) for k in ("factor", "original", "fast", "slow")))
            if min(scaling.factor, scaling.original, scaling.fast, scaling.slow) <= 0:
                raise ConfigError(f"config.json: '{at}.mixer.left.rot.scaling' wants positive numbers, got {scaling}")
        left = WindowAttentionConfig(
            heads=heads, kv_heads=kv, dim=dim, vdim=vdim, scale=_get(m, "m.left.scale", float),
            window=_get(m, "m.left.mask.size", int, minimum=1, optional=True),
            rot_base=_get(m, "m.left.rot.base", float), rot_dims=rot_dims, rot_scaling=scaling)
        rank = _get(m, "m.right.gate_rank", int, minimum=1, optional=True)
        tau = _get(m, "m.right.tau", float)
        if tau <= 0:
            raise ConfigError(f"config.json: '{at}.mixer.right.tau' must be positive, got {tau}")
        right = LinearAttentionConfig(heads=_get(m, "m.right.heads", int, minimum=1), dim=_get(m, "m.right.dim", int, minimum=1),
                                      vdim=_get(m, "m.right.vdim", int, minimum=1), tau=tau, gate_rank=rank or DEFAULT_GATE_RANK)
        ls, rs = _get(m, "m.left_scale", float, optional=True), _get(m, "m.right_scale", float, optional=True)
        return ParallelMixerConfig(left, right, 1.0 if ls is None else ls, 1.0 if rs is None else rs)


def sizes_from_shapes(d: Mapping[str, Any], shapes: Mapping[str, Tuple[int, ...]]) -> Mapping[str, Any]:
    """config.json's content with `layers[i].mixer.right.gate_rank` taken from the shape of `l<i>.mix.right.a1`."""
    import copy
    out = copy.deepcopy(dict(d))
    for i, L in enumerate(out.get("layers") or []):
        name = f"l{i}.mix.right.a1"
        if isinstance(L, dict) and L.get("type") == "parallel" and name in shapes and isinstance(L.get("mixer"), dict) \
                and isinstance(L["mixer"].get("right"), dict):
            if len(shapes[name]) != 2:
                raise ConfigError(f"{name} must be a matrix [gate_rank, width], got shape {tuple(shapes[name])}")
            L["mixer"]["right"]["gate_rank"] = int(shapes[name][0])
    return out
