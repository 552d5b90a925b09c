"""Typed configuration of the Bozovik design, read from its config.json.

The file names the design with one string (`architecture`) and gives the vocabulary, the model's width, the embedding's
scale, the norms' eps, the factor with which a sublayer's result joins the stream (`residual_mult`), the width of a
layer's part of the per-token side table (`token_side.dim`), a loop over some of the layers (`loop`: start, stop, times)
and the list of layers. A layer has a `type` (its mixer), the mixer's sizes and constants (`mixer`) and its feed-forward
(`mlp`, or null for none).

Mixer types: `attention` (every earlier key, a temperature and a gate per head, one added to the softmax's denominator),
`parallel` (a windowed attention that keeps the first keys, with a sink and a gate per head, beside a generalized delta
rule; under `left` and `right`, joined by `left_scale` and `right_scale`) and `latent_attention` (keys and values from
one latent row per token, a window and a sink per head). Every size and constant that can differ between models comes
from the file; what the file leaves out does not exist (no `mask`: every earlier key; no `keep_first`: none kept; no
`rot`: no rotation; no `loop`: every layer once; no `token_side`: no side input)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from .errors import ConfigError
from .lfm2 import _get
from .padadra import _obj

MIXERS = ("attention", "parallel", "latent_attention")
MLP_KINDS = ("dense",)


@dataclass(frozen=True)
class Rot:
    base: float
    dims: int


def _rot(d: dict, where: str, limit: int) -> Optional[Rot]:
    r = _obj(d, "rot", where, required=False)
    if r is None:
        return None
    rot = Rot(_get(r, "base", float), _get(r, "dims", int))
    if rot.dims % 2 or not 0 <= rot.dims <= limit or rot.base <= 0:
        raise ConfigError(f"config.json: {where}.rot: dims must be even and at most {limit}, base positive")
    return rot if rot.dims else None


@dataclass(frozen=True)
class GroupedAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int             # 0: every earlier key
    keep_first: int         # with a window: the first keys that stay visible
    rot: Optional[Rot]

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "GroupedAttention":
        heads, dim = _get(d, "heads", int), _get(d, "dim", int)
        mask = _obj(d, "mask", where, required=False) or {}
        c = cls(heads, _get(d, "kv_heads", int, heads), dim, _get(d, "vdim", int, dim), _get(d, "scale", float),
                _get(mask, "size", int, 0), _get(mask, "keep_first", int, 0), _rot(d, where, dim))
        if min(c.heads, c.kv_heads, c.dim, c.vdim) < 1 or c.window < 0 or c.keep_first < 0:
            raise ConfigError(f"config.json: {where}: sizes must be positive")
        if c.heads % c.kv_heads:
            raise ConfigError(f"config.json: {where}: {c.heads} heads are not a multiple of {c.kv_heads} key/value heads")
        return c


@dataclass(frozen=True)
class DeltaRule:
    heads: int
    dim: int
    decay_rank: Optional[int]       # the file's tensors give it; the key exists for writing random weights

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "DeltaRule":
        c = cls(_get(d, "heads", int), _get(d, "dim", int), _get(d, "decay_rank", int, None))
        if min(c.heads, c.dim, c.decay_rank or 1) < 1:
            raise ConfigError(f"config.json: {where}: sizes must be positive")
        return c


@dataclass(frozen=True)
class ParallelPair:
    left: GroupedAttention
    right: DeltaRule
    left_scale: float
    right_scale: float


@dataclass(frozen=True)
class LatentAttention:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    window: int
    rot: Optional[Rot]

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "LatentAttention":
        mask = _obj(d, "mask", where, required=False) or {}
        rot_dim = _get(d, "rot_dim", int, 0)
        c = cls(_get(d, "heads", int), _get(d, "dim", int), rot_dim, _get(d, "vdim", int), _get(d, "kv_rank", int),
                _get(d, "scale", float), _get(mask, "size", int, 0), _rot(d, where, rot_dim))
        if min(c.heads, c.dim, c.vdim, c.kv_rank) < 1 or c.rot_dim < 0 or c.window < 0:
            raise ConfigError(f"config.json: {where}: sizes must be positive")
        return c


@dataclass(frozen=True)
class DenseMlp:
    ff: int


@dataclass(frozen=True)
class BozovikLayer:
    type: str
    mixer: object           # GroupedAttention | ParallelPair | LatentAttention
    mlp: Optional[DenseMlp]


@dataclass(frozen=True)
class Loop:
    start: int
    stop: int
    times: int


@dataclass(frozen=True)
class BozovikConfig:
    vocab: int
    width: int
    norm_eps: float
    residual_mult: float
    embedding_scale: float
    token_side_dim: int             # 0: no side input
    loop: Optional[Loop]
    layers: tuple
    eos_token_id: Optional[int] = None

    @classmethod
    def from_dict(cls, d: dict) -> "BozovikConfig":
        norm = _get(d, "norm", dict)
        emb = _get(d, "embedding", dict, {})
        layers = []
        for i, entry in enumerate(_get(d, "layers", list)):
            where = f"layers[{i}]"
            if not isinstance(entry, dict):
                raise ConfigError(f"config.json: {where} should be an object")
            kind = _get(entry, "type", str)
            if kind not in MIXERS:
                raise ConfigError(f"config.json: {where}: mixer type {kind!r}; known: {list(MIXERS)}")
            m = _get(entry, "mixer", dict)
            if kind == "attention":
                mixer = GroupedAttention.from_dict(m, where + ".mixer")
            elif kind == "parallel":
                mixer = ParallelPair(GroupedAttention.from_dict(_obj(m, "left", where + ".mixer"), where + ".mixer.left"),
                                     DeltaRule.from_dict(_obj(m, "right", where + ".mixer"), where + ".mixer.right"),
                                     _get(m, "left_scale", float, 1.0), _get(m, "right_scale", float, 1.0))
            else:
                mixer = LatentAttention.from_dict(m, where + ".mixer")
            mlp = entry.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict):
                    raise ConfigError(f"config.json: {where}.mlp should be an object or null")
                mk = _get(mlp, "kind", str)
                if mk not in MLP_KINDS:
                    raise ConfigError(f"config.json: {where}: feed-forward kind {mk!r}; known: {list(MLP_KINDS)}")
                mlp = DenseMlp(_get(mlp, "ff", int))
                if mlp.ff < 1:
                    raise ConfigError(f"config.json: {where}: ff must be positive")
            layers.append(BozovikLayer(kind, mixer, mlp))
        loop = _obj(d, "loop", "config", required=False)
        if loop is not None:
            loop = Loop(_get(loop, "start", int), _get(loop, "stop", int), _get(loop, "times", int))
            if not 0 <= loop.start <= loop.stop <= len(layers) or loop.times < 1:
                raise ConfigError(f"config.json: loop {loop} does not fit {len(layers)} layers (0 <= start <= stop, times >= 1)")
            if loop.stop == loop.start:
                loop = None
        side = _obj(d, "token_side", "config", required=False)
        c = cls(_get(d, "vocab", int), _get(d, "width", int), _get(norm, "eps", float), _get(d, "residual_mult", float, 1.0),
                _get(emb, "scale", float, 1.0), _get(side, "dim", int) if side is not None else 0, loop, tuple(layers),
                _get(d, "eos_token_id", int, None))
        if c.vocab < 1 or c.width < 1 or c.token_side_dim < 0:
            raise ConfigError("config.json: vocab and width must be positive")
        return c
