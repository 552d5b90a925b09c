"""RMSNorm (crates/cellm-kernels/src/cpu_kernels.rs:17-34): x / sqrt(mean(x^2) + eps) * w,
fused with the addition of whatever waits to be added to the residual stream. With `groups` > 1 the
vector is split into that many equal consecutive parts and each is divided by its own root mean square.
With `offset` c the stored weight lies around zero and the factor is c + w (formed once, in 32-bit, when the
part is built: c + w has more digits than the stored type keeps).
With `scalar` the stored weight is a single number that multiplies every coordinate."""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from ..config.errors import ConfigError
from .base import Norm, Residual, TensorSpec
from .registry import register_norm


class RMSNorm(Norm):
    graph_safe = True

    """params: dim, eps, groups (default 1), offset (default 0), scalar (default False). weights: weight [dim] ([] if scalar)."""

    @classmethod
    def weight_specs(cls, params):
        shape = () if params.get("scalar") else (params["dim"],)
        return {"weight": TensorSpec(shape, "norm_offset" if params.get("offset") else "norm")}

    def __init__(self, params: dict, weights: dict, dtype: torch.dtype):
        self.dim = int(params["dim"])
        self.eps = float(params["eps"])
        self.groups = int(params.get("groups", 1))
        if self.groups < 1 or self.dim % self.groups:
            raise ConfigError(f"rms_norm: {self.dim} values do not split into {self.groups} equal groups")
        self.offset = float(params.get("offset", 0.0))
        self.weight = weights["weight"].contiguous()
        if params.get("scalar"):        # one number for all coordinates: kept as a row of it, which the kernels read
            self.weight = self.weight.reshape(1).expand(self.dim).contiguous()
        if self.offset:
            self.weight = (self.weight.to(torch.float32) + self.offset).contiguous()
        self.dtype = dtype
        self._w32 = self.weight if self.weight.dtype == torch.float32 else None

    def emit(self, emitter) -> None:
        from ..ops._lib import tag
        from ..runtime import records as R
        emitter.native(R.RMS_NORM, R.RmsNormParams(self.weight.data_ptr(), tag(self.weight), self.eps, self.groups), part=self)

    def forward(self, residual: Residual, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        delta, residual.pending = residual.pending, None
        y = ops.add_rmsnorm(residual.x, delta, self.weight, self.eps, self.dtype, rows, self.groups)
        if rows is not None and delta is not None:
            residual.pending = delta      # the stream itself was not updated
        return y

    def add_and_norm(self, x: torch.Tensor, addend: Optional[torch.Tensor], mult: float) -> torch.Tensor:
        """x += mult * addend (in place, 32-bit; None: nothing is added), then the norm of the sum."""
        if self.groups != 1:
            raise ConfigError("rms_norm: an addend times a constant is not taken by a norm in groups")
        if self._w32 is None:       # made at the first use, which must not be a step that is being captured in a graph
            if torch.cuda.is_available() and torch.cuda.is_current_stream_capturing():
                raise ConfigError("rms_norm: the 32-bit copy of the weight is made outside a graph's capture")
            self._w32 = self.weight.to(torch.float32).contiguous()
        return ops.add_scaled_norm(x, addend, mult, None, 0.0, "rms", self._w32, None, self.eps, self.dtype)


register_norm("rms_norm", RMSNorm)


class LayerNorm(Norm):
    graph_safe = True

    """(x - mean) / sqrt(var + eps) * w + b over the last axis, var the mean of the squared deviations; all of it 32-bit.
    params: dim, eps, bias (default True). weights: weight [dim], bias [dim]."""

    @classmethod
    def weight_specs(cls, params):
        specs = {"weight": TensorSpec((params["dim"],), "norm")}
        if params.get("bias", True):
            specs["bias"] = TensorSpec((params["dim"],), "bias")
        return specs

    def __init__(self, params: dict, weights: dict, dtype: torch.dtype):
        self.dim, self.eps, self.dtype = int(params["dim"]), float(params["eps"]), dtype
        self.weight = weights["weight"].to(torch.float32).contiguous()
        self.bias = weights["bias"].to(torch.float32).contiguous() if params.get("bias", True) else None

    def forward(self, residual: Residual, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        delta, residual.pending = residual.pending, None
        y = ops.add_scaled_norm(residual.x, delta, 1.0, None, 0.0, "layer", self.weight, self.bias, self.eps, self.dtype, rows)
        if rows is not None and delta is not None:
            residual.pending = delta      # the stream itself was not updated
        return y

    def add_and_norm(self, x: torch.Tensor, addend: Optional[torch.Tensor], mult: float) -> torch.Tensor:
        """x += mult * addend (in place, 32-bit; None: nothing is added), then the norm of the sum."""
        return ops.add_scaled_norm(x, addend, mult, None, 0.0, "layer", self.weight, self.bias, self.eps, self.dtype)


register_norm("layer_norm", LayerNorm)
