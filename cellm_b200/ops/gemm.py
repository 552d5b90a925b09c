from __future__ import annotations

import torch

from ._lib import check, fn, ptr, stream_of, tag


def gemm_plain(a: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """a [M, K] . w [N, K]^T on the CUDA cores with 32-bit sums; rows may be strided."""
    if not (a.is_cuda and w.is_cuda) or a.stride(-1) != 1 or w.stride(-1) != 1:
        raise ValueError("gemm_plain: operands must be CUDA tensors with unit inner stride")
    if a.dtype != w.dtype or a.shape[1] != w.shape[1]:
        raise ValueError(f"gemm_plain: a {tuple(a.shape)} {a.dtype} and w {tuple(w.shape)} {w.dtype} do not fit")
    out_dtype = out_dtype or a.dtype
    M, K = a.shape
    N = w.shape[0]
    c = torch.empty((M, N), dtype=out_dtype, device=a.device)
    check(fn("gemm_plain", "cellm_gemm_plain")(ptr(c), ptr(a), ptr(w), M, N, K, a.stride(0), w.stride(0),
                                               c.stride(0), tag(a), tag(out_dtype), stream_of(a)), "gemm_plain")
    return c


def gemm(a: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype | None = None, records: dict | None = None) -> torch.Tensor:
    """The product a [M, K] . w [N, K]^T by the kernel the native executor chooses for the operands: 32-bit
    operands run the plain 32-bit kernel; bfloat16 operands run the tensor-core kernel in the tile shape and K
    split that fit M, N and K (or the plain kernel where K or the rows' alignment do not fit it). `w` is taken
    for a weight that nothing on the stream writes. `records`: the caller's dictionary, in which the product's record is
    kept from call to call (a part that multiplies with the same weight every step)."""
    from ..runtime import records as R
    from ..runtime.program import part_program
    if a.dtype != w.dtype or a.dim() != 2 or w.dim() != 2 or a.shape[1] != w.shape[1] or a.stride(1) != 1 or w.stride(1) != 1:
        raise ValueError(f"gemm: a {tuple(a.shape)} {a.dtype} and w {tuple(w.shape)} {w.dtype} do not fit")
    out_dtype = out_dtype or a.dtype
    c = torch.empty((a.shape[0], w.shape[0]), dtype=out_dtype, device=a.device)
    if a.shape[0] == 0:
        return c
    key = (a.stride(0), out_dtype, a.data_ptr() % 16 == 0)
    rec = records.get(key) if records is not None else None
    if rec is None:
        rec = R.Record(R.LINEAR, R.LinearParams(R.linear(w), a.stride(0), tag(out_dtype)))
        if a.data_ptr() % 16:
            rec.params.w.tc_ok = 0
        if records is not None:
            records[key] = rec
    part_program(a.dtype, a.device, a.shape[1]).run_part(rec, a, None, out=c, rows=a.shape[0])
    return c


ACTIVATION_CODES = {"gelu": 0, "gelu_tanh": 1, "silu": 2, "relu": 3, "relu2": 4}


def gemm_act(a: torch.Tensor, w: torch.Tensor, act: str, out_dtype: torch.dtype, act_numbers: torch.Tensor | None = None) -> torch.Tensor:
    """act(a [M, K] . w [N, K]^T) with the activation formed on the 32-bit sums. bfloat16 operands of more than 16 rows:
    the persistent tensor-core product with the activation in its epilogue; otherwise the product with 32-bit output
    and the activation as a kernel of its own. act "xielu" reads its two learned numbers from `act_numbers` (float32,
    on the device)."""
    M, K = a.shape
    if act == "xielu" and (act_numbers is None or act_numbers.dtype != torch.float32 or act_numbers.numel() != 2):
        raise ValueError("gemm_act: xielu wants its two numbers as a float32 tensor")
    if (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and M > 16 and K % 8 == 0 and a.stride(1) == 1 and w.stride(1) == 1
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and out_dtype in (torch.bfloat16, torch.float32)):
        from ._state import error_word
        N = w.shape[0]
        c = torch.empty((M, N), dtype=out_dtype, device=a.device)
        if act == "xielu":
            check(fn("gemm_tcgen05", "cellm_gemm_xielu_tcgen05")(ptr(c), ptr(a), ptr(w), M, N, K, a.stride(0), w.stride(0), N, tag(out_dtype),
                                                                ptr(act_numbers), ptr(error_word(a.device)), stream_of(a)), "gemm_xielu_tcgen05")
            return c
        check(fn("gemm_tcgen05", "cellm_gemm_grouped_tcgen05")(ptr(c), ptr(a), ptr(w), M, N, K, 1, a.stride(0), w.stride(0), N, tag(out_dtype),
                                                              None, ACTIVATION_CODES[act], ptr(error_word(a.device)), stream_of(a)),
              "gemm_grouped_tcgen05")
        return c
    if act == "xielu":
        from .stream import xielu
        return xielu(gemm(a, w, torch.float32), act_numbers, out_dtype)
    from .recurrent import activation
    return activation(gemm(a, w, torch.float32), act, out_dtype)
