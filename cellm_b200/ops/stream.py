"""Python entry points of the kernels around the 32-bit residual stream of layers that run their sublayers one after
the other and add each result times a constant (norms with a mean and a bias, the start of another pass over the same
layers, a token's own row gated by the stream), and of the activation with learned numbers."""
from __future__ import annotations

from typing import Optional

import torch

from ._lib import check, fn, ptr, require_cuda, stream_of, tag

_LIB = "kernels_common"
NORM_KINDS = {"rms": 0, "layer": 1, "none": 2}


def _f32(*tensors) -> None:
    for t in tensors:
        if t is not None and t.dtype != torch.float32:
            raise ValueError(f"a 32-bit tensor is wanted, not {t.dtype}")


def add_scaled_norm(x: torch.Tensor, a: Optional[torch.Tensor], ma: float, b: Optional[torch.Tensor], mb: float, kind: str,
                    w: Optional[torch.Tensor], bias: Optional[torch.Tensor], eps: float, act_dtype: torch.dtype,
                    rows: Optional[torch.Tensor] = None, want: bool = True) -> Optional[torch.Tensor]:
    """x [T, H] float32 += ma * a + mb * b (in place, unless `rows` is given), then the norm of the sum in `act_dtype`:
    kind "layer" ((x - mean) / sqrt(var + eps) * w + bias), "rms" (x / sqrt(mean(x^2) + eps) * w) or "none" (the sum
    itself). With `rows` (int32 row indices) only those rows are formed and the stream stays as it was. `want` False:
    the sum only, nothing is returned."""
    require_cuda(x, a, b, w, bias, rows)
    _f32(x, w, bias)
    T, H = x.shape
    for t in (a, b):
        if t is not None and (t.shape != x.shape or (a is not None and t.dtype != a.dtype)):
            raise ValueError("add_scaled_norm: addends of the stream's shape and of one element type")
    n = T if rows is None else int(rows.numel())
    y = torch.empty((n, H), dtype=act_dtype, device=x.device) if want else None
    add = a if a is not None else b
    check(fn(_LIB, "cellm_add_scaled_norm")(ptr(y), ptr(x), ptr(a), float(ma), ptr(b), float(mb), tag(add) if add is not None else 0, ptr(w),
                                            ptr(bias), ptr(rows), n, T, H, float(eps), NORM_KINDS[kind], tag(act_dtype), stream_of(x)),
          "add_scaled_norm")
    return y


def stream_add_rows(x: torch.Tensor, table: Optional[torch.Tensor], ids: Optional[torch.Tensor], scale: float,
                    vec: Optional[torch.Tensor], err: torch.Tensor) -> None:
    """x [T, H] float32 += scale * table[ids] + vec (each optional; vec [H] float32)."""
    require_cuda(x, table, ids, vec)
    _f32(x, vec)
    T, H = x.shape
    check(fn(_LIB, "cellm_stream_add_rows")(ptr(x), ptr(table), tag(table) if table is not None else 0, ptr(ids),
                                            table.shape[0] if table is not None else 0, float(scale), ptr(vec), T, H, ptr(err), stream_of(x)),
          "stream_add_rows")


def token_gate_mul(g: torch.Tensor, table: torch.Tensor, col0: int, ids: torch.Tensor, act: str, act_dtype: torch.dtype,
                   err: torch.Tensor) -> torch.Tensor:
    """act(g [T, n] float32) * table[ids][:, col0 : col0 + n] in `act_dtype`; act "gelu_tanh", "gelu", "silu", "relu", "relu2"."""
    from .gemm import ACTIVATION_CODES
    _f32(g)
    T, n = g.shape
    out = torch.empty((T, n), dtype=act_dtype, device=g.device)
    check(fn(_LIB, "cellm_token_gate_mul")(ptr(out), ptr(g), g.stride(0), ptr(table), table.stride(0), int(col0), tag(table), ptr(ids),
                                           table.shape[0], T, n, ACTIVATION_CODES[act], tag(act_dtype), ptr(err), stream_of(g)), "token_gate_mul")
    return out


def scaled_rms_add(x: torch.Tensor, y: torch.Tensor, w: torch.Tensor, m: float, eps: float) -> None:
    """x [T, H] float32 += m * y / sqrt(mean(y^2) + eps) * w; y float32 [T, H], w float32 [H]."""
    require_cuda(x, y, w)
    _f32(x, y, w)
    if y.shape != x.shape or w.numel() != x.shape[1]:
        raise ValueError("scaled_rms_add: y of the stream's shape and a weight of its width")
    check(fn(_LIB, "cellm_scaled_rms_add")(ptr(x), ptr(y), ptr(w), float(m), x.shape[0], x.shape[1], float(eps), stream_of(x)), "scaled_rms_add")


def weighted_sum2(a: torch.Tensor, ca: float, b: torch.Tensor, cb: float) -> torch.Tensor:
    """ca * a + cb * b as float32; a and b of one shape and element type."""
    require_cuda(a, b)
    if a.shape != b.shape or a.dtype != b.dtype:
        raise ValueError("weighted_sum2: two tensors of one shape and element type")
    out = torch.empty(a.shape, dtype=torch.float32, device=a.device)
    check(fn(_LIB, "cellm_weighted_sum2")(ptr(out), ptr(a), float(ca), ptr(b), float(cb), a.numel(), tag(a), stream_of(a)), "weighted_sum2")
    return out


def xielu(u: torch.Tensor, pq: torch.Tensor, act_dtype: torch.dtype) -> torch.Tensor:
    """xIELU of float32 u [T, n] (rows may be strided) with the two learned numbers pq = (p, q) (float32, on the device):
    z > 0: softplus(p) z^2 + z / 2; otherwise (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2."""
    _f32(u, pq)
    T, n = u.shape
    out = torch.empty((T, n), dtype=act_dtype, device=u.device)
    check(fn(_LIB, "cellm_xielu")(ptr(out), ptr(u), u.stride(0), T, n, ptr(pq), tag(act_dtype), stream_of(u)), "xielu")
    return out


def head_gate_mul(o: torch.Tensor, gate: torch.Tensor, heads: int) -> torch.Tensor:
    """o [T, heads * vd], in place: head h of token t times sigmoid(gate[t, h]); gate float32, rows may be strided."""
    _f32(gate)
    T = o.shape[0]
    check(fn(_LIB, "cellm_head_gate_mul")(ptr(o), ptr(gate), gate.stride(0), T, heads, o.shape[1] // heads, tag(o), stream_of(o)), "head_gate_mul")
    return o
