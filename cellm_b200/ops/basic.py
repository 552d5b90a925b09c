from __future__ import annotations

from typing import Optional

import torch

from ._lib import check, count_launch, fn, ptr, require_cuda, stream_of, tag

_LIB = "kernels_common"


def embed(table: torch.Tensor, ids: torch.Tensor, err: torch.Tensor, scale: float = 1.0,
          pos_table: Optional[torch.Tensor] = None, positions: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Rows of `table` [V, H] for int32 ids [T], times `scale`, as float32 [T, H]; with `pos_table` [P, H] (of the
    table's element type) and int32 `positions` [T], plus the rows of that table (unscaled)."""
    require_cuda(table, ids, err, pos_table, positions)
    T, (V, H) = ids.numel(), table.shape
    out = torch.empty((T, H), dtype=torch.float32, device=table.device)
    if pos_table is not None:
        if pos_table.dtype != table.dtype or pos_table.shape[1] != H or positions is None or positions.numel() != T:
            raise ValueError("embed: position vectors [P, H] of the table's element type and one position per token")
        check(fn(_LIB, "cellm_embed_pos")(ptr(out), ptr(table), tag(table), ptr(ids), ptr(pos_table), ptr(positions), pos_table.shape[0],
                                          T, H, V, float(scale), ptr(err), stream_of(table)), "embed_pos")
        return out
    check(fn(_LIB, "cellm_embed")(ptr(out), ptr(table), tag(table), ptr(ids), T, H, V, float(scale), ptr(err),
                                  stream_of(table)), "embed")
    return out


def add_rmsnorm(x: torch.Tensor, delta: Optional[torch.Tensor], w: torch.Tensor, eps: float,
                act_dtype: torch.dtype, rows: Optional[torch.Tensor] = None, groups: int = 1) -> torch.Tensor:
    """x [*, H] float32 (+= delta in place when rows is None); returns the normed
    rows in act_dtype: all of them, or those listed in `rows`. `groups` > 1: each of that
    many equal consecutive parts of a row is divided by its own root mean square."""
    require_cuda(x, delta, w, rows)
    H = x.shape[-1]
    if x.dtype != torch.float32 or w.numel() != H:
        raise ValueError("add_rmsnorm: x must be float32 [*, H] and w must have H values")
    if delta is not None and (delta.dtype != act_dtype or delta.shape != x.shape):
        raise ValueError(f"add_rmsnorm: delta {tuple(delta.shape)} {delta.dtype} does not match x {tuple(x.shape)} / {act_dtype}")
    n = x.shape[0] if rows is None else rows.numel()
    y = torch.empty((n, H), dtype=act_dtype, device=x.device)
    check(fn(_LIB, "cellm_add_rmsnorm")(ptr(x), ptr(delta), ptr(w), tag(w), ptr(y), ptr(rows), n, H,
                                        int(groups), float(eps), tag(act_dtype), stream_of(x)), "add_rmsnorm")
    return y


def upload(dst: torch.Tensor, pinned: torch.Tensor, n: int) -> None:
    """The first n elements of a pinned host tensor into a device tensor of the same
    element type, asynchronously on the current stream."""
    if not dst.is_cuda or not pinned.is_pinned() or dst.dtype != pinned.dtype or n > dst.numel() or n > pinned.numel():
        raise ValueError("upload: a pinned host tensor into a device tensor of the same element type")
    code = fn(_LIB, "cellm_upload")(dst.data_ptr(), pinned.data_ptr(), n * dst.element_size(), stream_of(dst))
    if code != 0:
        raise RuntimeError(f"upload: CUDA error {code}")


def residual_add(x: torch.Tensor, delta: torch.Tensor) -> None:
    require_cuda(x, delta)
    if x.dtype != torch.float32 or x.shape != delta.shape:
        raise ValueError("residual_add: x must be float32 and delta of the same shape")
    check(fn(_LIB, "cellm_residual_add")(ptr(x), ptr(delta), x.numel(), tag(delta), stream_of(x)), "residual_add")


def swiglu(gu: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """gu [T, 2*ff] = [gate | up] -> silu(gate) * up [T, ff] of `out_dtype` (default: gu's; float32 gate and up
    may give a bfloat16 result)."""
    require_cuda(gu)
    T, two_ff = gu.shape
    h = torch.empty((T, two_ff // 2), dtype=out_dtype or gu.dtype, device=gu.device)
    check(fn(_LIB, "cellm_swiglu")(ptr(h), ptr(gu), T, two_ff // 2, tag(h), tag(gu), stream_of(gu)), "swiglu")
    return h


def short_conv(bcx: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], state: torch.Tensor,
               slot_ids: torch.Tensor, seq_of_token: torch.Tensor, cu_seqlens: torch.Tensor,
               err: torch.Tensor, max_q_len: int = 0) -> torch.Tensor:
    """bcx [T, 3H]; w [H, taps]; bias [H] or None; state [slots, taps-1, H] float32
    (read, then updated in place). Returns y [T, H]. `max_q_len`: the longest
    portion of the batch if the host knows it (0: unknown); short portions run a
    single fused kernel."""
    require_cuda(bcx, w, bias, state, slot_ids, seq_of_token, cu_seqlens, err)
    T, H3 = bcx.shape
    H, taps = w.shape
    if H3 != 3 * H or state.dtype != torch.float32 or tuple(state.shape[1:]) != (max(taps - 1, 0), H):
        raise ValueError(f"short_conv: shapes do not fit (bcx {tuple(bcx.shape)}, w {tuple(w.shape)}, state {tuple(state.shape)})")
    if bias is not None and (bias.dtype != w.dtype or bias.numel() != H):
        raise ValueError("short_conv: bias must have the taps' element type and H values")
    y = torch.empty((T, H), dtype=bcx.dtype, device=bcx.device)
    B = cu_seqlens.numel() - 1
    check(fn(_LIB, "cellm_short_conv")(ptr(y), ptr(bcx), ptr(w), ptr(bias), tag(w), ptr(state),
                                       state.stride(0), ptr(slot_ids), ptr(seq_of_token), ptr(cu_seqlens),
                                       T, B, H, taps, state.shape[0], int(max_q_len), tag(bcx), ptr(err),
                                       stream_of(bcx)), "short_conv")
    if taps > 1 and not 0 < max_q_len <= 4:
        count_launch()          # the state update is a launch of its own
    return y


def qk_norm_rope(qkv: torch.Tensor, q_w: Optional[torch.Tensor], k_w: Optional[torch.Tensor], eps: float,
                 positions: torch.Tensor, seq_of_token: torch.Tensor, block_table: Optional[torch.Tensor],
                 k_pool: Optional[torch.Tensor], v_pool: Optional[torch.Tensor], page_size: int,
                 nh: int, nkv: int, hd: int, rot: int, interleaved: bool, inv_freq: Optional[torch.Tensor],
                 err: torch.Tensor) -> torch.Tensor:
    """qkv [T, (nh + 2*nkv)*hd] -> q [T, nh*hd] normed and rotated; keys (normed,
    rotated) and values written into the pools [pages, kv_heads, page_size, hd].
    nkv = 0: rows hold queries only and nothing is written."""
    require_cuda(q_w, k_w, positions, seq_of_token, block_table, k_pool, v_pool, inv_freq, err)
    if not qkv.is_cuda or qkv.stride(1) != 1:
        raise ValueError("qk_norm_rope: rows must lie on the GPU with unit inner stride")
    T = qkv.shape[0]
    if qkv.shape[1] != (nh + 2 * nkv) * hd:
        raise ValueError(f"qk_norm_rope: row of {qkv.shape[1]} values, expected {(nh + 2 * nkv) * hd}")
    if rot > 0 and (inv_freq is None or inv_freq.dtype != torch.float32 or tuple(inv_freq.shape) != (rot // 2, 2)):
        raise ValueError("qk_norm_rope: inv_freq must be float32 [rot/2, 2] (high part, remainder)")
    if nkv > 0 and (k_pool.dtype != qkv.dtype or tuple(k_pool.shape[1:]) != (nkv, page_size, hd) or k_pool.shape != v_pool.shape):
        raise ValueError(f"qk_norm_rope: pool {tuple(k_pool.shape)} {k_pool.dtype} does not fit [pages, {nkv}, {page_size}, {hd}] {qkv.dtype}")
    w_tag = tag(q_w) if q_w is not None else 0
    q = torch.empty((T, nh * hd), dtype=qkv.dtype, device=qkv.device)
    check(fn(_LIB, "cellm_qk_norm_rope")(
        ptr(q), ptr(qkv), qkv.stride(0), ptr(q_w), ptr(k_w), w_tag, float(eps), ptr(positions),
        ptr(seq_of_token), ptr(block_table), block_table.stride(0) if block_table is not None else 0,
        ptr(k_pool), ptr(v_pool), k_pool.shape[0] if k_pool is not None else 0, page_size, T, nh, nkv, hd,
        rot, 1 if interleaved else 0, ptr(inv_freq), tag(qkv), ptr(err), stream_of(qkv)), "qk_norm_rope")
    return q


def attention_plain(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, positions: torch.Tensor,
                    seq_of_token: torch.Tensor, block_table: torch.Tensor, nh: int, scale: float,
                    window: int, err: torch.Tensor, value_dim: Optional[int] = None) -> torch.Tensor:
    """q [T, nh*hd]; pools [pages, kv_heads, page_size, hd]; each token reads keys
    0..positions[t] (or the last `window`) of its request. `value_dim`: a value is the first
    that many entries of its row (default hd); `v_pool` may then be `k_pool` itself."""
    require_cuda(q, k_pool, v_pool, positions, seq_of_token, block_table, err)
    pages, nkv, page_size, hd = k_pool.shape
    T = q.shape[0]
    hdv = hd if value_dim is None else int(value_dim)
    if q.shape[1] != nh * hd or k_pool.dtype != q.dtype or v_pool.shape != k_pool.shape:
        raise ValueError("attention_plain: shapes or element types do not fit")
    out = torch.empty((T, nh * hdv), dtype=q.dtype, device=q.device)
    check(fn(_LIB, "cellm_attention_plain")(
        ptr(out), ptr(q), ptr(k_pool), ptr(v_pool), ptr(positions), ptr(seq_of_token), ptr(block_table),
        block_table.stride(0), pages, page_size, T, nh, nkv, hd, hdv, float(scale), int(window), tag(q),
        ptr(err), stream_of(q)), "attention_plain")
    return out


def take_pending_tokens(ids: torch.Tensor, seq_of_token: torch.Tensor, slot_ids: torch.Tensor, last: torch.Tensor,
                        err: torch.Tensor) -> None:
    """Token ids of -1 (decoded tokens the host has not read yet) are replaced, in place, by last[state slot of the
    token's request], where the step before left them."""
    require_cuda(ids, seq_of_token, slot_ids, last, err)
    check(fn(_LIB, "cellm_take_pending_tokens")(ptr(ids), ptr(seq_of_token), ptr(slot_ids), ptr(last), ids.numel(),
                                                last.numel(), ptr(err), stream_of(ids)), "take_pending_tokens")


def keep_last_tokens(last: torch.Tensor, slot_ids: torch.Tensor, tokens: torch.Tensor) -> None:
    """last[slot_ids[r]] = tokens[r]: the tokens a decode step chose stay on the device for the step after it."""
    require_cuda(last, slot_ids, tokens)
    check(fn(_LIB, "cellm_keep_last_tokens")(ptr(last), ptr(slot_ids), ptr(tokens), tokens.numel(), last.numel(),
                                             stream_of(tokens)), "keep_last_tokens")


def argmax(logits: torch.Tensor) -> torch.Tensor:
    """Row-wise arg-max of float32 logits [R, V] as int32 [R]; lowest id among equals."""
    require_cuda(logits)
    if logits.dtype != torch.float32 or logits.dim() != 2:
        raise ValueError("argmax: logits must be float32 [R, V]")
    R, V = logits.shape
    out = torch.empty((R,), dtype=torch.int32, device=logits.device)
    # long rows are searched by 32 blocks each, which leave their finds in `parts` for a second, tiny kernel
    parts = torch.empty((R, 32), dtype=torch.int64, device=logits.device) if V >= 8192 else None
    check(fn(_LIB, "cellm_argmax")(ptr(out), ptr(logits), R, V, ptr(parts), stream_of(logits)), "argmax")
    if parts is not None:
        count_launch()
    return out


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, u: torch.Tensor,
           penalty: Optional[torch.Tensor] = None, recent: Optional[torch.Tensor] = None,
           max_top_k: int = 0, prefilter: bool = True) -> torch.Tensor:
    """One token per row of float32 logits [R, V]: arg-max where temperature <= 0,
    else a draw from softmax(logits / temperature) over the top_k logits (0: all),
    decided by the uniform number u[r]. recent [R, W] int32 (-1 padded) and
    penalty [R] apply the repetition penalty. max_top_k is the host's bound of top_k.
    `prefilter`: a first kernel finds the maxima of groups of 128 logits, which lets the
    rows that take a top k skip most of the row (off: one block searches the whole row;
    the choice is the same). Returns int32 [R]."""
    require_cuda(logits, temperature, top_k, u, penalty, recent)
    if logits.dtype != torch.float32 or logits.dim() != 2:
        raise ValueError("sample: logits must be float32 [R, V]")
    R, V = logits.shape
    W = recent.shape[1] if recent is not None else 0
    out = torch.empty((R,), dtype=torch.int32, device=logits.device)
    group_max = None
    if prefilter and 2048 <= V <= 128 * 8192:
        group_max = torch.empty((R, (V + 127) // 128), dtype=torch.int32, device=logits.device)
        count_launch()
    check(fn(_LIB, "cellm_sample")(ptr(out), ptr(logits), R, V, ptr(temperature), ptr(top_k), ptr(u),
                                   ptr(penalty), ptr(recent), W, int(max_top_k), ptr(group_max),
                                   stream_of(logits)), "sample")
    return out


def stream_cast(x: torch.Tensor, act_dtype: torch.dtype) -> torch.Tensor:
    """The 32-bit stream in the activations' element type (the stream itself when that is float32)."""
    require_cuda(x)
    if x.dtype != torch.float32:
        raise ValueError("stream_cast: the stream is float32")
    if act_dtype == torch.float32:
        return x
    y = torch.empty_like(x, dtype=act_dtype)
    check(fn(_LIB, "cellm_stream_cast")(ptr(y), ptr(x), x.numel(), tag(act_dtype), stream_of(x)), "stream_cast")
    return y


def gated_norm_add(x: torch.Tensor, m: torch.Tensor, gate: Optional[torch.Tensor], gate_bias: Optional[torch.Tensor],
                   w: torch.Tensor, groups: int, eps: float, want_copy: bool = True,
                   m_bias: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """x [T, H] float32 += group_rms_norm((m + m_bias) * sigmoid(gate + gate_bias)) * w, in place (gate None: no gate;
    m_bias None: none). m is of the activations' type, gate too or float32 (it may be a view of columns of a wider matrix), the biases of w's. Returns the new stream in that type (x itself for float32), or None if not wanted."""
    require_cuda(x, m, gate_bias, w, m_bias)
    T, H = x.shape
    if x.dtype != torch.float32 or m.shape != x.shape or (gate is not None and (gate.shape != x.shape or gate.stride(1) != 1 or
                                                                              gate.dtype not in (m.dtype, torch.float32))):
        raise ValueError("gated_norm_add: x float32 [T, H]; m [T, H]; gate [T, H] of m's element type or float32, rows dense")
    if w.numel() != H or any(b is not None and (b.numel() != H or b.dtype != w.dtype) for b in (gate_bias, m_bias)):
        raise ValueError("gated_norm_add: w and gate_bias have H values of one element type")
    y = torch.empty_like(m) if (want_copy and m.dtype != torch.float32) else None
    check(fn(_LIB, "cellm_gated_norm_add")(ptr(x), ptr(m), ptr(m_bias), ptr(gate), gate.stride(0) if gate is not None else H,
                                           tag(gate) if gate is not None else tag(m), ptr(gate_bias), ptr(w), tag(w), ptr(y), T, H, int(groups),
                                           float(eps), tag(m), stream_of(x)), "gated_norm_add")
    return y if y is not None else (x if want_copy else None)


def mingru_scan(proj: torch.Tensor, bz: Optional[torch.Tensor], bx: Optional[torch.Tensor], state: torch.Tensor,
                slot_ids: torch.Tensor, cu_seqlens: torch.Tensor, act_dtype: torch.dtype, err: torch.Tensor,
                max_q_len: int = 0) -> torch.Tensor:
    """proj [T, 3W] = [z | candidate | output gate] pre-activations; state [slots, W] float32, read and updated in place.
    Returns S_t * silu(gate) [T, W] in act_dtype. `max_q_len`: the longest portion if the host knows it (long portions
    under bfloat16 are walked in runs side by side)."""
    require_cuda(proj, bz, bx, state, slot_ids, cu_seqlens, err)
    T, W3 = proj.shape
    W = W3 // 3
    if W * 3 != W3 or state.dtype != torch.float32 or state.shape[1] != W:
        raise ValueError(f"mingru_scan: shapes do not fit (proj {tuple(proj.shape)}, state {tuple(state.shape)})")
    wt = tag(bz) if bz is not None else tag(act_dtype)
    out = torch.empty((T, W), dtype=act_dtype, device=proj.device)
    check(fn(_LIB, "cellm_mingru_scan")(ptr(out), ptr(proj), proj.stride(0), tag(proj), ptr(bz), ptr(bx), wt, ptr(state), state.stride(0),
                                        ptr(slot_ids), ptr(cu_seqlens), T, cu_seqlens.numel() - 1, W, state.shape[0], int(max_q_len), tag(act_dtype),
                                        ptr(err), stream_of(proj)), "mingru_scan")
    return out


def head_product(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x [T, heads, K] (any row pitch, head pitch K or more) times per-head matrices w [heads, N, K] -> [T, heads, N];
    `out` may be a view with pitches of its own (last axis dense)."""
    heads, N, K = w.shape
    T = x.shape[0]
    if out is None:
        out = torch.empty((T, heads, N), dtype=x.dtype, device=x.device)
    if x.stride(2) != 1 or out.stride(2) != 1 or x.dtype != w.dtype or out.dtype != w.dtype or not w.is_contiguous():
        raise ValueError("head_product: dense last axes and one element type")
    check(fn(_LIB, "cellm_head_product")(out.data_ptr(), out.stride(0), out.stride(1), x.data_ptr(), x.stride(0), x.stride(1),
                                         ptr(w), T, heads, N, K, tag(w), stream_of(x)), "head_product")
    return out


def gated_act(gu: torch.Tensor, bg: Optional[torch.Tensor], bu: Optional[torch.Tensor], act: str,
              out_dtype: torch.dtype) -> torch.Tensor:
    """gu [T, 2 ff] = [gate | up] -> act(gate + bg) * (up + bu); act "silu" or "gelu_tanh"."""
    require_cuda(gu, bg, bu)
    T, two_ff = gu.shape
    h = torch.empty((T, two_ff // 2), dtype=out_dtype, device=gu.device)
    wt = tag(bg) if bg is not None else tag(out_dtype)
    check(fn(_LIB, "cellm_gated_act")(ptr(h), ptr(gu), gu.stride(0), ptr(bg), ptr(bu), wt, T, two_ff // 2, {"silu": 0, "gelu_tanh": 1}[act],
                                      tag(h), tag(gu), stream_of(gu)), "gated_act")
    return h


def attention_latent(q: torch.Tensor, pool: torch.Tensor, cu_seqlens: torch.Tensor, ctx_lens: torch.Tensor,
                     block_table: torch.Tensor, q_lens, nh: int, dv: int, scale: float, nsplit: int,
                     err: torch.Tensor, window: int = 0, sinks: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The tensor-core attention over a latent cache by itself: q [T, nh * kw] bfloat16, pool [pages, 1, page_size, kw];
    every head reads the same rows, a value is a row's first dv entries. `q_lens`: the host's copy of the portions'
    lengths; `nsplit`: pieces the keys are cut into; `window`: 0, or how many of its last rows a token reads; `sinks` [nh]
    float32: a sink per head in the denominator. Returns [T, nh * dv]."""
    require_cuda(q, pool, cu_seqlens, ctx_lens, block_table, err)
    pages, one, page_size, kw = pool.shape
    T = q.shape[0]
    if one != 1 or q.shape[1] != nh * kw or q.dtype != torch.bfloat16 or pool.dtype != torch.bfloat16:
        raise ValueError("attention_latent: bfloat16 queries [T, nh * kw] over a pool [pages, 1, page_size, kw]")
    n_tiles = sum((int(n) * nh + 63) // 64 for n in q_lens)
    out = torch.empty((T, nh * dv), dtype=q.dtype, device=q.device)
    part_o = part_ml = None
    if nsplit > 1:
        part_o = torch.empty((nsplit, T * nh, dv), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((nsplit, T * nh, 2), dtype=torch.float32, device=q.device)
        count_launch()
    check(fn("attention_latent", "cellm_attention_latent")(
        ptr(out), ptr(part_o), ptr(part_ml), ptr(q), ptr(pool), ptr(cu_seqlens), ptr(ctx_lens), ptr(block_table),
        block_table.stride(0), len(q_lens), T, n_tiles, pages, page_size, nh, kw, dv, float(scale), int(nsplit), int(window), ptr(sinks),
        ptr(err), stream_of(q)), "attention_latent")
    return out
