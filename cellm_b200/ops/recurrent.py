"""Python entry points of the kernels for layers with matrix-valued recurrent state, short convolutions over a
projection's channels, attention with sinks and rotated values, and the stream operations of layers whose two
sublayers have norms of their own. Small vectors (biases, taps, norm weights, sinks, decays' constants) are 32-bit."""
from __future__ import annotations

from typing import Optional

import torch

from ._lib import check, fn, ptr, require_cuda, stream_of, tag

_LIB = "kernels_common"


def _f32(*tensors) -> None:
    for t in tensors:
        if t is not None and t.dtype != torch.float32:
            raise ValueError(f"a 32-bit tensor is wanted, not {t.dtype}")


def embed_pairs(table: torch.Tensor, pair_table: torch.Tensor, buckets: int, mul_prev: int, mul_cur: int, scale: float,
                prev_state: torch.Tensor, ctx) -> torch.Tensor:
    """Rows of `table` [V, H] times `scale` plus the row (previous token * mul_prev + token * mul_cur) mod buckets of
    `pair_table` [buckets + 1, H] (its last row for a sequence's first token) as float32 [T, H]. `prev_state`
    [slots, 1] int32: every request's last token, read and moved on."""
    require_cuda(table, pair_table, prev_state)
    (V, H), T = table.shape, ctx.T
    if pair_table.shape != (buckets + 1, H) or pair_table.dtype != table.dtype or prev_state.dtype != torch.int32:
        raise ValueError("embed_pairs: a pair table [buckets + 1, H] of the table's element type and int32 state")
    out = torch.empty((T, H), dtype=torch.float32, device=table.device)
    check(fn(_LIB, "cellm_embed_pairs")(ptr(out), ptr(table), tag(table), ptr(ctx.token_ids), ptr(pair_table), int(buckets), int(mul_prev),
                                        int(mul_cur), ptr(prev_state), prev_state.stride(0), prev_state.shape[0], ptr(ctx.positions),
                                        ptr(ctx.seq_of_token), ptr(ctx.cu_seqlens), ptr(ctx.slot_ids), T, H, V, float(scale),
                                        ptr(ctx.err), stream_of(table)), "embed_pairs")
    return out


def norm_pair(x: torch.Tensor, w1: torch.Tensor, w2: Optional[torch.Tensor], eps: float, act_dtype: torch.dtype):
    """(x / rms(x) * w1, x / rms(x) * w2) in `act_dtype` from one read of the 32-bit stream x [T, H]; w2 None: the first only."""
    require_cuda(x, w1, w2)
    T, H = x.shape
    if x.dtype != torch.float32 or w1.numel() != H or (w2 is not None and (w2.numel() != H or w2.dtype != w1.dtype)):
        raise ValueError("norm_pair: a float32 stream [T, H] and weights of H values in one element type")
    y1 = torch.empty((T, H), dtype=act_dtype, device=x.device)
    y2 = torch.empty((T, H), dtype=act_dtype, device=x.device) if w2 is not None else None
    check(fn(_LIB, "cellm_norm_pair")(ptr(y1), ptr(y2), ptr(x), ptr(w1), ptr(w2), tag(w1), T, H, float(eps), tag(act_dtype), stream_of(x)),
          "norm_pair")
    return y1, y2


def scaled_add2(x: torch.Tensor, a: torch.Tensor, b: Optional[torch.Tensor], m: float) -> None:
    """x += m * (a + b) on the 32-bit stream; a and b (optional) in one element type."""
    require_cuda(x, a, b)
    if x.dtype != torch.float32 or a.shape != x.shape or (b is not None and (b.shape != x.shape or b.dtype != a.dtype)):
        raise ValueError("scaled_add2: a float32 stream and addends of its shape")
    check(fn(_LIB, "cellm_scaled_add2")(ptr(x), ptr(a), ptr(b), float(m), x.numel(), tag(a), stream_of(x)), "scaled_add2")


def pair_norm_mean(a: torch.Tensor, b: torch.Tensor, wa: torch.Tensor, wb: torch.Tensor, eps: float, act_dtype: torch.dtype) -> torch.Tensor:
    """(a / rms(a) * wa + b / rms(b) * wb) / 2 over the last axis of float32 a, b [T, H], in `act_dtype`."""
    require_cuda(a, b, wa, wb)
    _f32(a, b, wa, wb)
    T, H = a.shape
    if b.shape != a.shape or wa.numel() != H or wb.numel() != H or not a.is_contiguous() or not b.is_contiguous():
        raise ValueError("pair_norm_mean: two dense [T, H] tensors and weights of H values")
    out = torch.empty((T, H), dtype=act_dtype, device=a.device)
    check(fn(_LIB, "cellm_pair_norm_mean")(ptr(out), ptr(a), ptr(b), ptr(wa), ptr(wb), T, H, float(eps), tag(act_dtype), stream_of(a)), "pair_norm_mean")
    return out


def conv_state_update(state: torch.Tensor, proj: torch.Tensor, col0: int, bias: Optional[torch.Tensor], n_taps: int, ctx) -> None:
    """state [slots, n_taps - 1, C] float32 <- the last n_taps - 1 rows of (state ‖ the portion's projected values +
    bias) for every request of the step; the channels are columns col0 .. col0 + C of proj [T, ld] float32."""
    if n_taps <= 1:
        return
    require_cuda(state, bias)
    _f32(state, proj, bias)
    C = state.shape[2]
    check(fn(_LIB, "cellm_conv_state_update")(ptr(state), state.stride(0), state.shape[0], ptr(ctx.slot_ids), ptr(ctx.cu_seqlens),
                                              ptr(proj), proj.stride(0), int(col0), ptr(bias), int(n_taps), C, ctx.B, ptr(ctx.err),
                                              stream_of(proj)), "conv_state_update")


def sink_attn_prep(proj: torch.Tensor, col0: int, bias, taps, n_taps: int, conv_state, q_norm_w, k_norm_w, eps: float, qk_freq, rot: int,
                   v_freq, interleaved: bool, ctx, cache, nh: int, nkv: int, hd: int, vd: int, act_dtype: torch.dtype,
                   q_mult: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Bias, short convolution, norm over the projection, rotation of q, k (and v), and the write of k and v into the
    token's page; returns q [T, nh * hd] in `act_dtype`. proj [T, ld] float32 holds q | k | v from column col0 on.
    `q_mult` [nh]: a factor per query head."""
    _f32(proj, bias, taps, conv_state, q_norm_w, k_norm_w, qk_freq, v_freq, q_mult)
    T = ctx.T
    q = torch.empty((T, nh * hd), dtype=act_dtype, device=proj.device)
    k, v, bt = cache.k, cache.v, cache.block_table
    if k.dtype != act_dtype or v.dtype != act_dtype or k.shape[1:] != (nkv, cache.page_size, hd) or v.shape[1:] != (nkv, cache.page_size, vd):
        raise ValueError("sink_attn_prep: pools [pages, kv heads, page size, width] of the activations' element type")
    check(fn(_LIB, "cellm_sink_attn_prep")(
        ptr(q), ptr(k), ptr(v), ptr(proj), proj.stride(0), int(col0), ptr(bias), ptr(taps), int(n_taps), ptr(conv_state),
        conv_state.stride(0) if conv_state is not None else 0, conv_state.shape[0] if conv_state is not None else 1 << 30,
        ptr(q_norm_w), ptr(k_norm_w), float(eps), ptr(qk_freq), int(rot), ptr(v_freq), int(interleaved), ptr(ctx.positions),
        ptr(ctx.seq_of_token), ptr(ctx.cu_seqlens), ptr(ctx.slot_ids), ptr(bt), bt.stride(0), k.shape[0], cache.page_size, T, nh, nkv, hd, vd,
        ptr(q_mult), tag(act_dtype), ptr(ctx.err), stream_of(proj)), "sink_attn_prep")
    return q


def attention_plain_sink(q: torch.Tensor, cache, ctx, nh: int, nkv: int, hd: int, vd: int, scale: float, window: int,
                         sinks: Optional[torch.Tensor], unrot: Optional[torch.Tensor], interleaved: bool) -> torch.Tensor:
    """Attention of q [T, nh * hd] over the paged keys and values (rows of vd) with 32-bit scores; `sinks` [nh]: one more
    term exp(sink_h) in each head's denominator; `unrot` [vd/2, 2]: the output is turned back by the token's position."""
    _f32(sinks, unrot)
    k, v, bt = cache.k, cache.v, cache.block_table
    out = torch.empty((q.shape[0], nh * vd), dtype=q.dtype, device=q.device)
    check(fn(_LIB, "cellm_attention_plain_sink")(ptr(out), ptr(q), ptr(k), ptr(v), ptr(ctx.positions), ptr(ctx.seq_of_token), ptr(bt),
                                                 bt.stride(0), k.shape[0], cache.page_size, q.shape[0], nh, nkv, hd, vd, float(scale),
                                                 int(window), ptr(sinks), ptr(unrot), int(interleaved), tag(q), ptr(ctx.err), stream_of(q)),
          "attention_plain_sink")
    return out


def attention_plain_masked(q: torch.Tensor, cache, ctx, nh: int, nkv: int, hd: int, vd: int, scale: float, window: int = 0,
                           keep_first: int = 0, sinks: Optional[torch.Tensor] = None, fixed_sink: Optional[float] = None,
                           gate: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The plain attention in its general form: from position i a key j <= i is visible when i - j < window or j < keep_first (window 0:
    every earlier key); `sinks` [nh] float32 (a learned sink per head) or `fixed_sink` (one sink score for all heads) is
    one more term in the denominator; `gate` [T, >= nh] float32 (rows may be strided): head h's output times
    sigmoid(gate[t, h]). A cache without a pool of values gives its key rows' first vd entries as values."""
    _f32(sinks, gate)
    k, bt = cache.k, cache.block_table
    v = cache.v if cache.v is not None else k
    out = torch.empty((q.shape[0], nh * vd), dtype=q.dtype, device=q.device)
    check(fn(_LIB, "cellm_attention_plain_masked")(ptr(out), ptr(q), ptr(k), ptr(v), ptr(ctx.positions), ptr(ctx.seq_of_token), ptr(bt),
                                                   bt.stride(0), k.shape[0], cache.page_size, q.shape[0], nh, nkv, hd, vd, v.shape[-1],
                                                   float(scale), int(window), int(keep_first), ptr(sinks),
                                                   float(fixed_sink) if fixed_sink is not None else 0.0, int(fixed_sink is not None),
                                                   ptr(gate), gate.stride(0) if gate is not None else 0, tag(q), ptr(ctx.err), stream_of(q)),
          "attention_plain_masked")
    return out


def attention_flash_sink(q: torch.Tensor, cache, ctx, nh: int, nkv: int, hd: int, scale: float, window: int,
                         sinks: Optional[torch.Tensor], unrot: Optional[torch.Tensor], interleaved: bool) -> torch.Tensor:
    """The same attention on the tensor cores (bfloat16; keys and values of one width hd of 32, 64 or 128): tiles of
    64 (token, head) rows for prompt portions, of 16 for steps of single tokens, whose keys are cut into pieces when
    the tiles alone leave most of the GPU idle."""
    _f32(sinks, unrot)
    k, v, bt = cache.k, cache.v, cache.block_table
    if q.dtype != torch.bfloat16 or k.dtype != torch.bfloat16 or v.shape != k.shape or hd not in (32, 64, 128):
        raise ValueError("attention_flash_sink: bfloat16 and keys and values of one width of 32, 64 or 128")
    T, G = q.shape[0], nh // nkv
    wide = ctx.max_q_len * G > 16
    rows = 64 if wide else 16
    n_tiles = sum(-(-n * G // rows) for n in ctx.q_lens)
    # pieces of keys: only where a step's tiles are few; a piece is at least two blocks of 64 keys
    longest = ctx.max_total_len          # a captured step's bound: the width of its block tables
    span = min(longest, window + ctx.max_q_len) if window > 0 else longest
    nsplit = max(1, min(-(-span // 128), 296 // max(1, n_tiles * nkv), 32))
    out = torch.empty((T, nh * hd), dtype=q.dtype, device=q.device)
    part_o = part_ml = None
    if nsplit > 1:
        part_o = torch.empty((nsplit, T * nh, hd), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((nsplit, T * nh, 2), dtype=torch.float32, device=q.device)
    check(fn("attention_flash", "cellm_attention_flash_sink")(
        ptr(out), ptr(part_o), ptr(part_ml), ptr(q), ptr(k), ptr(v), ptr(ctx.cu_seqlens), ptr(ctx.ctx_lens), ptr(bt), bt.stride(0),
        ctx.B, T, n_tiles, k.shape[0], cache.page_size, nh, nkv, hd, float(scale), int(window), int(wide), nsplit, ptr(sinks), ptr(unrot),
        int(interleaved), ptr(ctx.positions), ptr(ctx.err), stream_of(q)), "attention_flash_sink")
    return out


def attention_flash_masked(q: torch.Tensor, cache, ctx, nh: int, nkv: int, hd: int, scale: float, window: int, keep_first: int,
                           sinks: Optional[torch.Tensor], gate: Optional[torch.Tensor]) -> torch.Tensor:
    """The tensor-core attention in its general form (bfloat16; keys and values of one width hd of 32, 64 or 128):
    from position i a key j <= i is visible when i - j < window or j < keep_first (window 0: every earlier key); `sinks` [nh] float32:
    one more term exp(sink_h) in a head's denominator; `gate` [T, >= nh] float32 (rows may be strided): head h's output
    times sigmoid(gate[t, h])."""
    _f32(sinks, gate)
    k, v, bt = cache.k, cache.v, cache.block_table
    if q.dtype != torch.bfloat16 or k.dtype != torch.bfloat16 or v.shape != k.shape or hd not in (32, 64, 128):
        raise ValueError("attention_flash_masked: bfloat16 and keys and values of one width of 32, 64 or 128")
    T, G = q.shape[0], nh // nkv
    wide = ctx.max_q_len * G > 16
    rows = 64 if wide else 16
    n_tiles = sum(-(-n * G // rows) for n in ctx.q_lens)
    longest = ctx.max_total_len
    span = min(longest, window + keep_first + ctx.max_q_len) if window > 0 else longest
    nsplit = max(1, min(-(-span // 128), 296 // max(1, n_tiles * nkv), 32))
    out = torch.empty((T, nh * hd), dtype=q.dtype, device=q.device)
    part_o = part_ml = None
    if nsplit > 1:
        part_o = torch.empty((nsplit, T * nh, hd), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((nsplit, T * nh, 2), dtype=torch.float32, device=q.device)
    check(fn("attention_flash", "cellm_attention_flash_masked")(
        ptr(out), ptr(part_o), ptr(part_ml), ptr(q), ptr(k), ptr(v), ptr(ctx.cu_seqlens), ptr(ctx.ctx_lens), ptr(bt), bt.stride(0),
        ctx.B, T, n_tiles, k.shape[0], cache.page_size, nh, nkv, hd, float(scale), int(window), int(keep_first), int(wide), nsplit,
        ptr(sinks), ptr(gate), gate.stride(0) if gate is not None else 0, ptr(ctx.err), stream_of(q)), "attention_flash_masked")
    return out


def hgrn2_scan(proj: torch.Tensor, col_q: int, col_f: int, col_v: int, f_bias: torch.Tensor, lower: torch.Tensor, state: torch.Tensor,
               ctx, heads: int, dim: int, vd: int) -> torch.Tensor:
    """The HGRN2 recurrence over every request's tokens of the step; state [slots, heads, dim, vd] float32 is moved on.
    Returns S^T q per token and head, float32 [T, heads * vd]. The q and f columns of `proj` are replaced by silu(q) and
    by the forget gate."""
    _f32(proj, f_bias, lower, state)
    o = torch.empty((ctx.T, heads * vd), dtype=torch.float32, device=proj.device)
    check(fn(_LIB, "cellm_hgrn2_scan")(ptr(o), ptr(state), state.stride(0), state.shape[0], ptr(proj), proj.stride(0), int(col_q), int(col_f),
                                       int(col_v), ptr(f_bias), ptr(lower), ptr(ctx.cu_seqlens), ptr(ctx.slot_ids), ctx.B, ctx.T, heads, dim, vd,
                                       ptr(ctx.err), stream_of(proj)), "hgrn2_scan")
    return o


def delta_prep(proj: torch.Tensor, col0: int, col_b: int, taps, n_taps: int, conv_state, a2: torch.Tensor, dt_bias, A_log, ctx,
               heads: int, kvh: int, dim: int, vd: int, l2_eps: float):
    """Inputs of the gated delta rule from the projections: (qk [T, 2 kvh dim], v [T, heads vd], beta [T, heads],
    decay [T, heads dim]), all float32."""
    _f32(proj, taps, conv_state, a2, dt_bias, A_log)
    T, dev = ctx.T, proj.device
    qk = torch.empty((T, 2 * kvh * dim), dtype=torch.float32, device=dev)
    v = torch.empty((T, heads * vd), dtype=torch.float32, device=dev)
    beta = torch.empty((T, heads), dtype=torch.float32, device=dev)
    decay = torch.empty((T, heads * dim), dtype=torch.float32, device=dev)
    if a2.stride(1) != 1 or a2.shape != (T, heads * dim):
        raise ValueError("delta_prep: the decay's pre-activation [T, heads * dim] (rows may be strided)")
    check(fn(_LIB, "cellm_delta_prep")(ptr(qk), ptr(v), ptr(beta), ptr(decay), ptr(proj), proj.stride(0), int(col0), int(col_b), ptr(taps),
                                       int(n_taps), ptr(conv_state), conv_state.stride(0) if conv_state is not None else 0,
                                       conv_state.shape[0] if conv_state is not None else 1 << 30, ptr(a2), a2.stride(0), ptr(dt_bias), ptr(A_log),
                                       ptr(ctx.seq_of_token), ptr(ctx.cu_seqlens), ptr(ctx.slot_ids), T, heads, kvh, dim, vd, float(l2_eps),
                                       ptr(ctx.err), stream_of(proj)), "delta_prep")
    return qk, v, beta, decay


def delta_scan(qk, v, beta, decay, state: torch.Tensor, ctx, heads: int, kvh: int, dim: int, vd: int) -> torch.Tensor:
    """The gated delta rule over every request's tokens of the step; state [slots, heads, dim, vd] float32 is moved on.
    Returns S^T q per token and head, float32 [T, heads * vd]."""
    _f32(qk, v, beta, decay, state)
    o = torch.empty((ctx.T, heads * vd), dtype=torch.float32, device=qk.device)
    check(fn(_LIB, "cellm_delta_scan")(ptr(o), ptr(state), state.stride(0), state.shape[0], ptr(qk), ptr(v), ptr(beta), ptr(decay),
                                       ptr(ctx.cu_seqlens), ptr(ctx.slot_ids), ctx.B, heads, kvh, dim, vd, ptr(ctx.err), stream_of(qk)),
          "delta_scan")
    return o


def gdelta_prep(proj: torch.Tensor, col_k: int, col_a: int, w_pre: torch.Tensor, w0: torch.Tensor, a_bias: torch.Tensor, rate: float,
                unit_eps: float, heads: int, dim: int) -> torch.Tensor:
    """Inputs of the generalized delta rule's walk, float32 [T, 3, heads * dim]: the decay exp(-rate * sigmoid(w_pre + w0)),
    the unit key k / sqrt(sum(k^2) + unit_eps) of each head, and sigmoid(a_pre + a_bias) times the unit key. proj [T, ld]
    float32 holds k at column col_k and a_pre at col_a; w_pre [T, heads * dim] float32 (rows may be strided)."""
    _f32(proj, w_pre, w0, a_bias)
    T = proj.shape[0]
    vecs = torch.empty((T, 3, heads * dim), dtype=torch.float32, device=proj.device)
    check(fn(_LIB, "cellm_gdelta_prep")(ptr(vecs), ptr(proj), proj.stride(0), int(col_k), int(col_a), ptr(w_pre), w_pre.stride(0), ptr(w0),
                                        ptr(a_bias), float(rate), float(unit_eps), T, heads, dim, stream_of(proj)), "gdelta_prep")
    return vecs


def gdelta_scan(proj: torch.Tensor, col_r: int, col_k: int, col_v: int, vecs: torch.Tensor, state: torch.Tensor, ctx, heads: int,
                dim: int, vd: int) -> torch.Tensor:
    """The generalized delta rule S <- diag(d) S - (a u)(u^T S) + k v^T over every request's tokens of the step (both
    terms read the old S); state [slots, heads, dim, vd] float32 is moved on. Returns S^T r per token and head, float32
    [T, heads * vd]."""
    _f32(proj, vecs, state)
    o = torch.empty((ctx.T, heads * vd), dtype=torch.float32, device=proj.device)
    check(fn(_LIB, "cellm_gdelta_scan")(ptr(o), ptr(state), state.stride(0), state.shape[0], ptr(proj), proj.stride(0), int(col_r), int(col_k),
                                        int(col_v), ptr(vecs), ptr(ctx.cu_seqlens), ptr(ctx.slot_ids), ctx.B, heads, dim, vd, ptr(ctx.err),
                                        stream_of(proj)), "gdelta_scan")
    return o


def head_norm_gate(o: torch.Tensor, w: torch.Tensor, gate: Optional[torch.Tensor], heads: int, vd: int, eps: float,
                   act_dtype: torch.dtype) -> torch.Tensor:
    """o [T, heads * vd] float32 -> o / rms over each head * w (* sigmoid(gate [T, heads * vd], rows may be strided));
    w [vd] serves every head, w [heads * vd] gives each head a row of its own."""
    _f32(o, w, gate)
    T = o.shape[0]
    if w.numel() not in (vd, heads * vd):
        raise ValueError("head_norm_gate: a weight of vd or of heads * vd values")
    per_head = int(w.numel() != vd)
    out = torch.empty((T, heads * vd), dtype=act_dtype, device=o.device)
    check(fn(_LIB, "cellm_head_norm_gate")(ptr(out), ptr(o), ptr(w), ptr(gate), gate.stride(0) if gate is not None else 0, T, heads, vd,
                                           float(eps), per_head, tag(act_dtype), stream_of(o)), "head_norm_gate")
    return out


def activation(u: torch.Tensor, act: str, act_dtype: torch.dtype) -> torch.Tensor:
    """act(u) for float32 u [T, n] (rows may be strided) in `act_dtype`; act: gelu, gelu_tanh, silu, relu, relu2, tanh."""
    _f32(u)
    T, n = u.shape
    h = torch.empty((T, n), dtype=act_dtype, device=u.device)
    check(fn(_LIB, "cellm_activation")(ptr(h), ptr(u), u.stride(0), T, n, {"gelu": 0, "gelu_tanh": 1, "silu": 2, "relu": 3, "relu2": 4, "tanh": 5}[act],
                                       tag(act_dtype), stream_of(u)), "activation")
    return h
