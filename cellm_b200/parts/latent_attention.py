"""Latent attention mixer: keys and values of all heads are made from one compressed row per token, and only that
row is cached.

    q = W_q h, head by head [dim unrotated | rot_dim rotated]
    W_dkv h = [kv_rank values -> RMS norm with a weight = the latent c | rot_dim values = one rotated key part for all heads]
    head h: key = [K_h c | rotated part], value = V_h c, score = q . key * scale, causal softmax, output W_o (heads side by side)

Since q_h . (K_h c) = (K_h^T q_h) . c, the attention runs over the cached rows themselves with one key/value "head":
the query of head h becomes [K_h^T q_h | rotated part], the weighted sum of the rows' first kv_rank values is formed,
and V_h turns it into the head's output. The rotation is a position part of its own (`position`), applied to the last
rot_dim values of each query head and to the shared key part, in pairs that lie side by side or half a rotation apart.
Optional: a sliding window (from position i the rows j with 0 <= i - j < window are visible; rows that no later token can read give
their pages back) and a learned sink per head (one more term exp(sink_h) in the softmax's denominator, with no key and
no value)."""
from __future__ import annotations

import torch

from ..config.errors import ConfigError
from ..config.plan import PartSpec
from .base import CacheBinding, Mixer, PagedKV, StepContext, TensorSpec
from .linear import Linear, stack_rows
from .registry import part_class, register_mixer


class LatentAttentionMixer(Mixer):
    graph_safe = True

    """params: hidden_size, heads, dim, rot_dim, vdim, kv_rank, scale, eps (of the latent's norm),
    position (PartSpec of a rotation over rot_dim values, or None), window (default 0: every earlier row), sinks (default
    False), out_dtype32 (default False).
    weights: q [heads*(dim+rot_dim), H], dkv [kv_rank+rot_dim, H], dkv_norm [kv_rank], uk [heads*dim, kv_rank],
    uv [heads*vdim, kv_rank], o [H, heads*vdim]; sinks [heads]."""

    @classmethod
    def weight_specs(cls, params):
        H, nh, d, r, vd, rank = (params[k] for k in ("hidden_size", "heads", "dim", "rot_dim", "vdim", "kv_rank"))
        specs = {"q": TensorSpec((nh * (d + r), H), "linear"), "dkv": TensorSpec((rank + r, H), "linear"),
                 "dkv_norm": TensorSpec((rank,), "norm"), "uk": TensorSpec((nh * d, rank), "linear"),
                 "uv": TensorSpec((nh * vd, rank), "linear"), "o": TensorSpec((H, nh * vd), "linear")}
        if params.get("sinks"):
            specs["sinks"] = TensorSpec((nh,), "sink")
        return specs

    @classmethod
    def cache_need(cls, params):
        return PagedKV(1, int(params["kv_rank"]) + int(params["rot_dim"]), int(params.get("window") or 0), values=False)

    def __init__(self, params: dict, weights: dict, dtype: torch.dtype):
        self.H, self.dtype = int(params["hidden_size"]), dtype
        self.nh, self.d, self.r = int(params["heads"]), int(params["dim"]), int(params["rot_dim"])
        self.vd, self.rank = int(params["vdim"]), int(params["kv_rank"])
        self.scale, self.eps = float(params["scale"]), float(params["eps"])
        self.in_proj = Linear(stack_rows(weights["q"], weights["dkv"]), dtype)
        self.out_proj = Linear(weights["o"], dtype)
        self.c_norm_w = weights["dkv_norm"].contiguous()
        # K_h transposed, [heads, kv_rank, dim]: turns a head's unrotated query into a query against the latent rows
        self.absorb_k = weights["uk"].reshape(self.nh, self.d, self.rank).transpose(1, 2).contiguous()
        self.expand_v = weights["uv"].reshape(self.nh, self.vd, self.rank).contiguous()
        pos: PartSpec | None = params.get("position")
        self.position = part_class("position", pos.kind)(pos.params, self.c_norm_w.device) if pos is not None else None
        rot = self.position.rotation() if self.position is not None else (0, True, None)
        if rot is None or rot[0] > self.r:
            raise ConfigError("latent_attention: the position encoding must be a rotation over at most rot_dim values")
        self.rot, self.interleaved, self.inv_freq = int(rot[0]), bool(rot[1]), rot[2]
        self.window = int(params.get("window") or 0)
        self.sinks = weights["sinks"].to(torch.float32).contiguous() if params.get("sinks") else None
        self.extra = 0
        self._record = None

    def stack_behind_input(self, weight: torch.Tensor) -> bool:
        if self._record is not None or self.extra or weight.dtype != self.in_proj.weight.dtype or weight.shape[1] != self.H:
            return False
        self.in_proj = Linear(stack_rows(self.in_proj.weight, weight), self.dtype)
        self.extra = int(weight.shape[0])
        return True

    def stacked_rows(self) -> torch.Tensor:
        return self.in_proj.weight[self.in_proj.weight.shape[0] - self.extra:]

    def record(self):
        from ..ops._lib import tag
        from ..runtime import records as R
        ws = (self.in_proj.weight, self.out_proj.weight, self.absorb_k, self.expand_v)
        if self._record is None and all(w.dtype == self.dtype for w in ws):
            p = R.LatentAttentionParams()
            p.in_proj, p.out_proj = R.linear(self.in_proj.weight), R.linear(self.out_proj.weight)
            p.absorb_k, p.expand_v = self.absorb_k.data_ptr(), self.expand_v.data_ptr()
            p.heads, p.dim, p.rot_dim, p.vdim, p.rank, p.scale = self.nh, self.d, self.r, self.vd, self.rank, self.scale
            p.c_norm_w, p.c_norm_dtype, p.eps = self.c_norm_w.data_ptr(), tag(self.c_norm_w), self.eps
            p.rot, p.inv_freq, p.extra = self.rot, R.ptr(self.inv_freq), self.extra
            p.interleaved, p.window, p.sinks = int(self.interleaved), self.window, R.ptr(self.sinks)
            self._record = R.Record(R.LATENT_ATTENTION, p, keep=[self.inv_freq, self.sinks], part=self)
        return self._record

    def emit(self, emitter) -> None:
        rec = self.record()
        if rec is None:
            raise ConfigError("latent_attention: matrices kept in another element type than the activations")
        emitter.records.append(rec)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheBinding) -> torch.Tensor:
        from ..runtime.program import part_program
        rec = self.record()
        if rec is None:
            raise ConfigError("latent_attention: matrices kept in another element type than the activations")
        return part_program(self.dtype, x.device, self.H).run_part(rec, x, ctx, cache)


register_mixer("latent_attention", LatentAttentionMixer)
