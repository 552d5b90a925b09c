"""Plain two-matrix feed-forward: W_down act(W_up h), with act one of "relu2" (the square of relu), "relu", "silu",
"gelu", "gelu_tanh". The activation is formed on the first product's 32-bit sums: in that product's epilogue for prompt
portions under bfloat16, by a kernel of its own otherwise."""
from __future__ import annotations

import torch

from ..config.errors import ConfigError
from .base import FeedForward, StepContext, TensorSpec
from .linear import Linear
from .registry import register_feed_forward

ACTIVATIONS = ("relu2", "relu", "silu", "gelu", "gelu_tanh")


class DenseMLP(FeedForward):
    graph_safe = True

    """params: hidden_size, ff_dim, activation. weights: up [ff, H], down [H, ff]."""

    @classmethod
    def weight_specs(cls, params):
        H, ff = params["hidden_size"], params["ff_dim"]
        return {"up": TensorSpec((ff, H), "linear"), "down": TensorSpec((H, ff), "linear")}

    def __init__(self, params: dict, weights: dict, dtype: torch.dtype):
        self.H, self.ff, self.dtype = int(params["hidden_size"]), int(params["ff_dim"]), dtype
        self.activation = params.get("activation", "relu2")
        if self.activation not in ACTIVATIONS:
            raise ConfigError(f"dense_mlp: activation {self.activation!r}; known: {list(ACTIVATIONS)}")
        self.up, self.down = Linear(weights["up"], dtype), Linear(weights["down"], dtype)

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        from .. import ops
        if self.up.weight.dtype != x.dtype:          # a matrix kept in 32-bit under bfloat16 activations
            return self.down(ops.activation(self.up(x, out_dtype=torch.float32), self.activation, self.dtype))
        return self.down(ops.gemm_act(x, self.up.weight, self.activation, self.dtype))


register_feed_forward("dense_mlp", DenseMLP)
