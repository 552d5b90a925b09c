"""Typed configuration of the Padadra design, read from its config.json.

The file names the design with one string (`architecture`) and gives the vocabulary, the model's width, the
embedding's scale and its table of token pairs (`embedding.bigram`: buckets and the two multipliers of the hash), the
norms' eps, the factor with which a layer's result joins the stream (`residual_mult`), and a list of layers. A layer
has a `type` (its mixer), the mixer's sizes and constants (`mixer`) and its feed-forward (`mlp`, or null for none).

Mixer types: `parallel` (a windowed attention with sinks beside an HGRN2 recurrence, under `left` and `right`) and
`channel_delta` (a gated delta rule with one decay per head and key channel). Every size and constant that can differ
between models comes from the file; what the file leaves out does not exist (no `scaling`: plain frequencies; no
`mask`: every earlier key is seen; no `bigram`: the token's own row only)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from .errors import ConfigError
from .lfm2 import _get

MIXERS = ("parallel", "channel_delta")
MLP_KINDS = ("dense",)


def _obj(d: dict, key: str, where: str, required: bool = True) -> Optional[dict]:
    v = d.get(key)
    if v is None:
        if required:
            raise ConfigError(f"config.json: {where}: required key {key!r} is missing")
        return None
    if not isinstance(v, dict):
        raise ConfigError(f"config.json: {where}.{key} should be an object")
    return v


@dataclass(frozen=True)
class FrequencyScaling:
    factor: float
    low: float
    high: float
    original: float

    def to_dict(self) -> dict:
        return {"factor": self.factor, "high": self.high, "low": self.low, "original": self.original}


@dataclass(frozen=True)
class Rotation:
    base: float
    dims: int
    scaling: Optional[FrequencyScaling]

    def to_dict(self) -> dict:
        d = {"base": self.base, "dims": self.dims}
        if self.scaling is not None:
            d["scaling"] = self.scaling.to_dict()
        return d


@dataclass(frozen=True)
class SinkAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    conv: int               # taps of the short convolutions on q, k and v (0: none)
    window: int             # 0: every earlier key
    rot: Optional[Rotation]

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "SinkAttention":
        rot = _obj(d, "rot", where, required=False)
        if rot is not None:
            sc = _obj(rot, "scaling", where + ".rot", required=False)
            if sc is not None:
                sc = FrequencyScaling(*(_get(sc, k, float) for k in ("factor", "low", "high", "original")))
                if sc.factor <= 0 or sc.high <= sc.low or sc.original <= 0:
                    raise ConfigError(f"config.json: {where}.rot.scaling needs factor > 0, high > low and original > 0")
            rot = Rotation(_get(rot, "base", float), _get(rot, "dims", int), sc)
        mask = _obj(d, "mask", where, required=False)
        c = cls(*(_get(d, k, int) for k in ("heads", "kv_heads", "dim", "vdim")), _get(d, "scale", float),
                _get(d, "conv", int, 0), _get(mask, "size", int) if mask is not None else 0, rot)
        if min(c.heads, c.kv_heads, c.dim, c.vdim) < 1 or c.conv < 0 or c.window < 0:
            raise ConfigError(f"config.json: {where}: sizes must be positive")
        if c.heads % c.kv_heads:
            raise ConfigError(f"config.json: {where}: {c.heads} heads are not a multiple of {c.kv_heads} key/value heads")
        if rot is not None and (rot.dims % 2 or not 0 <= rot.dims <= c.dim or c.vdim % 2 or rot.base <= 0):
            raise ConfigError(f"config.json: {where}: rot.dims must be even and at most dim, vdim even, base positive")
        return c

    def to_dict(self) -> dict:
        d = {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "scale": self.scale, "vdim": self.vdim}
        if self.conv:
            d["conv"] = self.conv
        if self.window:
            d["mask"] = {"size": self.window}
        if self.rot is not None:
            d["rot"] = self.rot.to_dict()
        return d


@dataclass(frozen=True)
class Hgrn2:
    heads: int
    dim: int
    vdim: int

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "Hgrn2":
        c = cls(*(_get(d, k, int) for k in ("heads", "dim", "vdim")))
        if min(c.heads, c.dim, c.vdim) < 1:
            raise ConfigError(f"config.json: {where}: sizes must be positive")
        return c

    def to_dict(self) -> dict:
        return {"dim": self.dim, "heads": self.heads, "vdim": self.vdim}


@dataclass(frozen=True)
class ParallelMixer:
    left: SinkAttention
    right: Hgrn2

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "ParallelMixer":
        return cls(SinkAttention.from_dict(_obj(d, "left", where), where + ".mixer.left"),
                   Hgrn2.from_dict(_obj(d, "right", where), where + ".mixer.right"))

    def to_dict(self) -> dict:
        return {"left": self.left.to_dict(), "right": self.right.to_dict()}


@dataclass(frozen=True)
class ChannelDelta:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    # ranks of the decay's and the gate's low-rank products: the file's tensors give them; the keys exist for
    # writing random weights
    decay_rank: Optional[int] = None
    gate_rank: Optional[int] = None

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "ChannelDelta":
        c = cls(*(_get(d, k, int) for k in ("heads", "kv_heads", "dim", "vdim", "conv")),
                _get(d, "decay_rank", int, None), _get(d, "gate_rank", int, None))
        if min(c.heads, c.kv_heads, c.dim, c.vdim, c.conv, c.decay_rank or 1, c.gate_rank or 1) < 1:
            raise ConfigError(f"config.json: {where}: sizes must be positive")
        if c.heads % c.kv_heads:
            raise ConfigError(f"config.json: {where}: {c.heads} heads are not a multiple of {c.kv_heads} query/key heads")
        return c

    def to_dict(self) -> dict:
        d = {"conv": self.conv, "dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "vdim": self.vdim}
        if self.decay_rank:
            d["decay_rank"] = self.decay_rank
        if self.gate_rank:
            d["gate_rank"] = self.gate_rank
        return d


@dataclass(frozen=True)
class DenseMlp:
    ff: int

    def to_dict(self) -> dict:
        return {"ff": self.ff, "kind": "dense"}


@dataclass(frozen=True)
class PadadraLayer:
    type: str
    mixer: object           # ParallelMixer | ChannelDelta
    mlp: Optional[DenseMlp]

    def to_dict(self) -> dict:
        return {"mixer": self.mixer.to_dict(), "mlp": self.mlp.to_dict() if self.mlp else None, "type": self.type}


@dataclass(frozen=True)
class PairTable:
    buckets: int
    mul_prev: int
    mul_cur: int


@dataclass(frozen=True)
class PadadraConfig:
    vocab: int
    width: int
    norm_eps: float
    residual_mult: float
    embedding_scale: float
    bigram: Optional[PairTable]
    layers: tuple[PadadraLayer, ...]
    eos_token_id: Optional[int] = None

    @classmethod
    def from_dict(cls, d: dict) -> "PadadraConfig":
        norm = _get(d, "norm", dict)
        emb = _get(d, "embedding", dict, {})
        big = _obj(emb, "bigram", "embedding", required=False)
        if big is not None:
            big = PairTable(_get(big, "buckets", int), _get(big, "mul_prev", int), _get(big, "mul_cur", int))
            if big.buckets < 1 or big.mul_prev < 0 or big.mul_cur < 0:
                raise ConfigError("config.json: embedding.bigram needs buckets > 0 and multipliers that are not negative")
        layers = []
        for i, entry in enumerate(_get(d, "layers", list)):
            where = f"layers[{i}]"
            if not isinstance(entry, dict):
                raise ConfigError(f"config.json: {where} should be an object")
            kind = _get(entry, "type", str)
            if kind not in MIXERS:
                raise ConfigError(f"config.json: {where}: mixer type {kind!r}; known: {list(MIXERS)}")
            m = _get(entry, "mixer", dict)
            mixer = ParallelMixer.from_dict(m, where) if kind == "parallel" else ChannelDelta.from_dict(m, where + ".mixer")
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
            layers.append(PadadraLayer(kind, mixer, mlp))
        c = cls(_get(d, "vocab", int), _get(d, "width", int), _get(norm, "eps", float), _get(d, "residual_mult", float, 1.0),
                _get(emb, "scale", float, 1.0), big, tuple(layers), _get(d, "eos_token_id", int, None))
        if c.vocab < 1 or c.width < 1:
            raise ConfigError("config.json: vocab and width must be positive")
        return c

    def to_dict(self) -> dict:
        emb = {"scale": self.embedding_scale}
        if self.bigram is not None:
            emb["bigram"] = {"buckets": self.bigram.buckets, "mul_cur": self.bigram.mul_cur, "mul_prev": self.bigram.mul_prev}
        d = {"architecture": "Padadra", "embedding": emb, "layers": [l.to_dict() for l in self.layers],
             "norm": {"eps": self.norm_eps}, "residual_mult": self.residual_mult, "vocab": self.vocab, "width": self.width}
        if self.eos_token_id is not None:
            d["eos_token_id"] = self.eos_token_id
        return d
