"""The two ends of the model: the token embedding that starts the residual
stream (crates/cellm-model/src/lfm.rs:817-890: a row of the table, no scaling)
and the output product that turns the last normed rows into logits
(:689-757; the reference always reads the embedding table for it)."""
from __future__ import annotations

import torch

from .. import ops
from .base import Embedding, Head, TensorSpec
from .linear import Linear
from .registry import register_embedding, register_head


class TokenEmbedding(Embedding):
    graph_safe = True

    """params: vocab_size, dim, scale (default 1: the row as it is), max_positions (default 0: none; else a table of
    learned position vectors is added, unscaled). weights: weight [vocab, dim], positions [max_positions, dim]."""

    @classmethod
    def weight_specs(cls, params):
        specs = {"weight": TensorSpec((params["vocab_size"], params["dim"]), "embedding")}
        if params.get("max_positions"):
            specs["positions"] = TensorSpec((params["max_positions"], params["dim"]), "embedding")
        return specs

    def __init__(self, params: dict, weights: dict, dtype: torch.dtype):
        self.weight = weights["weight"].contiguous()
        self.scale = float(params.get("scale", 1.0))
        self.positions = None
        if params.get("max_positions"):
            self.positions = weights["positions"].to(self.weight.dtype).contiguous()

    def emit(self, emitter) -> None:
        from ..ops._lib import tag
        from ..runtime import records as R
        n = 0 if self.positions is None else self.positions.shape[0]
        emitter.native(R.EMBED, R.EmbedParams(self.weight.data_ptr(), tag(self.weight), self.scale, R.ptr(self.positions), n), part=self)

    def forward(self, token_ids: torch.Tensor, ctx) -> torch.Tensor:
        return ops.embed(self.weight, token_ids, ctx.err, self.scale, self.positions, ctx.positions if self.positions is not None else None)


class PairHashEmbedding(Embedding):
    """The token's row times `scale`, plus a row of a second table chosen by a hash of the token and the one before it:
    row (previous * mul_prev + token * mul_cur) mod buckets, and the table's last row (number `buckets`) for a
    sequence's first token. The previous token of a portion's first token is the request's state (one int32 in its
    slot), so a sequence cut anywhere finds the same rows.

    params: vocab_size, dim, scale (default 1), buckets, mul_prev, mul_cur. weights: weight [vocab, dim],
    pairs [buckets + 1, dim]."""
    graph_safe = True

    @classmethod
    def weight_specs(cls, params):
        return {"weight": TensorSpec((params["vocab_size"], params["dim"]), "embedding"),
                "pairs": TensorSpec((params["buckets"] + 1, params["dim"]), "embedding")}

    @classmethod
    def cache_need(cls, params):
        from .base import FixedState
        return FixedState((1,), torch.int32)

    def __init__(self, params: dict, weights: dict, dtype: torch.dtype):
        self.weight = weights["weight"].contiguous()
        self.pairs = weights["pairs"].to(self.weight.dtype).contiguous()
        self.scale = float(params.get("scale", 1.0))
        self.buckets, self.mul_prev, self.mul_cur = int(params["buckets"]), int(params["mul_prev"]), int(params["mul_cur"])

    def forward(self, token_ids: torch.Tensor, ctx, cache=None) -> torch.Tensor:
        if cache is None or cache.state is None:
            raise ValueError("lookup_pairs: the embedding needs its state (every request's last token)")
        return ops.embed_pairs(self.weight, self.pairs, self.buckets, self.mul_prev, self.mul_cur, self.scale, cache.state, ctx)


class LinearHead(Head):
    graph_safe = True

    """params: vocab_size, dim. weights: weight [vocab, dim] (the embedding's tensor when the two are tied)."""

    @classmethod
    def weight_specs(cls, params):
        return {"weight": TensorSpec((params["vocab_size"], params["dim"]), "linear")}

    def __init__(self, params: dict, weights: dict, dtype: torch.dtype):
        self.linear = Linear(weights["weight"], dtype)
        self.weight = self.linear.weight

    def emit(self, emitter) -> None:
        from ..runtime import records as R
        if not emitter.fits(self.weight):
            return super().emit(emitter)
        emitter.native(R.HEAD, R.HeadParams(R.linear(self.weight)), part=self)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.linear(x, out_dtype=torch.float32)


register_embedding("lookup", TokenEmbedding)
register_embedding("lookup_pairs", PairHashEmbedding)
register_head("linear", LinearHead)
