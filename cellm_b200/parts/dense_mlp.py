"""Plain two-matrix feed-forward: W_down act(W_up h), with act one of "relu2" (the square of relu), "relu", "silu",
"gelu", "gelu_tanh", or "xielu": with two learned numbers p, q (the part's weight `act`), softplus(p) z^2 + z / 2 for
z > 0 and (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2 otherwise. The activation is formed on the first product's 32-bit
sums: in that product's epilogue for prompt portions under bfloat16 (the activations without learned numbers), by a
kernel of its own otherwise."""
from __future__ import annotations

import torch

from ..config.errors import ConfigError
from .base import FeedForward, StepContext, TensorSpec
from .linear import Linear
from .registry import register_feed_forward

ACTIVATIONS = ("relu2", "relu", "silu", "gelu", "gelu_tanh", "xielu")


class DenseMLP(FeedForward):
    graph_safe = True

    """params: hidden_size, ff_dim, activation, out_dtype32 (default False: the result in the activations' type).
    weights: up [ff, H], down [H, ff]; act [2] for "xielu"."""

    @classmethod
    def weight_specs(cls, params):
        H, ff = params["hidden_size"], params["ff_dim"]
        specs = {"up": TensorSpec((ff, H), "linear"), "down": TensorSpec((H, ff), "linear")}
        if params.get("activation") == "xielu":
            specs["act"] = TensorSpec((2,), "sink")
        return specs

    def __init__(self, params: dict, weights: dict, dtype: torch.dtype):
        self.H, self.ff, self.dtype = int(params["hidden_size"]), int(params["ff_dim"]), dtype
        self.activation = params.get("activation", "relu2")
        if self.activation not in ACTIVATIONS:
            raise ConfigError(f"dense_mlp: activation {self.activation!r}; known: {list(ACTIVATIONS)}")
        self.up, self.down = Linear(weights["up"], dtype), Linear(weights["down"], dtype)
        self.act_numbers = weights["act"].to(torch.float32).contiguous() if self.activation == "xielu" else None
        self.out_dtype = torch.float32 if params.get("out_dtype32") else None

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        from .. import ops
        if self.up.weight.dtype != x.dtype:          # a matrix kept in 32-bit under bfloat16 activations
            u = self.up(x, out_dtype=torch.float32)
            h = ops.xielu(u, self.act_numbers, self.dtype) if self.act_numbers is not None else ops.activation(u, self.activation, self.dtype)
            return self.down(h, out_dtype=self.out_dtype)
        return self.down(ops.gemm_act(x, self.up.weight, self.activation, self.dtype, self.act_numbers), out_dtype=self.out_dtype)


register_feed_forward("dense_mlp", DenseMLP)
