"""Windowed attention with a learned sink per head, short convolutions on its projections and rotated values.

    q, k, v = W h (+ b);   each channel then passes a short causal convolution over time (optional)
    q, k normed over the whole projection (all heads of a token by one root mean square, plain weights; optional)
    q, k: the first `rotary_dim` entries of every head turn by pos * f_i (the position part: a rotation, frequencies
          possibly stretched by wavelength)
    v:    every value head turns over all its entries by its own position j, pair m by j * theta^(-2m/vd), and is
          cached so; a head's output at position i (the weighted sum of values) is turned back by -i * theta^(-2m/vd)
    softmax over the keys j with 0 <= i - j < window (window 0: all earlier keys; with `keep_first` n the sequence's
          first n keys stay visible behind the window, at their true positions); the denominator also holds
          exp(sink_h): a learned number per head with no key and no value, not scaled, counted once (or, with
          `fixed_sink`, exp of one given score for every head: 0 adds one to the denominator)
    scores of head h times a learned number per head (`head_temperature`, optional)
    head h's output times sigmoid(G h)_h, one number per head from a product over the mixer's input (`head_gate`, optional)
    out = W_o (heads side by side)

Scores, softmax, norms, angles and the convolutions' sums are 32-bit. The request keeps pages of keys and values
(values with rows of their own width) and, beside them, the last taps - 1 projected rows (bias included) of q, k and v
in its state slot, so a sequence cut anywhere sees the same convolution inputs.

Kernels: one product for q | k | v with 32-bit sums, `sink_attn_prep` (bias, convolution, norm, rotations, cache
write), `conv_state_update`, the attention itself (32-bit, and heads whose key and value widths differ or are none
of 32, 64, 128: the plain kernel with sink and turn-back; bfloat16: the paged mma.sync flash kernel, which takes the
sink into a row's denominator and turns the row's sum back in its epilogue, or in the merge of its pieces), the
output product."""
from __future__ import annotations

import torch

from ..config.errors import ConfigError
from ..config.plan import PartSpec
from .base import CacheBinding, FixedState, Mixer, PagedKV, StepContext, TensorSpec
from .linear import Linear, stack_rows
from .registry import part_class, register_mixer
from .rope import split_inv_freq


# Tests turn the tensor-core attention off to compare it with the plain kernel on the same cache, and the tcgen05 kernel
# off to compare it with the mma.sync one.
OPTIONS = {"tensor_cores": True, "tcgen05": True}


def bindings_of(cache: CacheBinding, n: int) -> tuple:
    """The n bindings of a mixer that declared n needs (one need: the binding itself)."""
    if n == 1:
        return (cache.parts[0] if cache.parts else cache,)
    if len(cache.parts) != n:
        raise ValueError(f"a mixer with {n} cache needs was given {len(cache.parts)} bindings")
    return cache.parts


class SinkAttentionMixer(Mixer):
    graph_safe = True

    """params: hidden_size, num_heads, num_kv_heads, head_dim, value_dim (default head_dim), scale, window (default 0),
    bias (default False: q, k, v have none), conv_taps (default 0: no convolution), qk_norm_eps (None: no norm over the
    projection), position (PartSpec of a rotation, or None), value_theta (None: values are not rotated),
    sinks (default True), out_dtype32 (default False: out_proj's result in the activations' type), keep_first (default 0),
    fixed_sink (None, or the sink's score where it is no learned number; not beside sinks), head_gate, head_temperature
    (default False).
    weights: q_proj [nh*hd, H], k_proj [nkv*hd, H], v_proj [nkv*vd, H], out_proj [H, nh*vd]; q_bias, k_bias, v_bias;
    q_conv [nh*hd, taps], k_conv, v_conv; q_norm [nh*hd], k_norm [nkv*hd]; sinks [nh]; gate [nh, H]; temperature [nh]."""

    @classmethod
    def _sizes(cls, params):
        nh, nkv, hd = int(params["num_heads"]), int(params["num_kv_heads"]), int(params["head_dim"])
        return nh, nkv, hd, int(params.get("value_dim") or hd)

    @classmethod
    def weight_specs(cls, params):
        H = params["hidden_size"]
        nh, nkv, hd, vd = cls._sizes(params)
        taps = int(params.get("conv_taps") or 0)
        specs = {"q_proj": TensorSpec((nh * hd, H), "linear"), "k_proj": TensorSpec((nkv * hd, H), "linear"),
                 "v_proj": TensorSpec((nkv * vd, H), "linear"), "out_proj": TensorSpec((H, nh * vd), "linear")}
        if params.get("bias"):
            specs.update(q_bias=TensorSpec((nh * hd,), "bias"), k_bias=TensorSpec((nkv * hd,), "bias"), v_bias=TensorSpec((nkv * vd,), "bias"))
        if taps:
            specs.update(q_conv=TensorSpec((nh * hd, taps), "conv_tap_wide"), k_conv=TensorSpec((nkv * hd, taps), "conv_tap_wide"),
                         v_conv=TensorSpec((nkv * vd, taps), "conv_tap_wide"))
        if params.get("qk_norm_eps") is not None:
            specs.update(q_norm=TensorSpec((nh * hd,), "norm"), k_norm=TensorSpec((nkv * hd,), "norm"))
        if params.get("sinks", True):
            specs["sinks"] = TensorSpec((nh,), "sink")
        if params.get("head_gate"):
            specs["gate"] = TensorSpec((nh, H), "linear")
        if params.get("head_temperature"):
            specs["temperature"] = TensorSpec((nh,), "norm")
        return specs

    @classmethod
    def cache_need(cls, params):
        nh, nkv, hd, vd = cls._sizes(params)
        window = int(params.get("window") or 0)
        paged = PagedKV(nkv, hd, window, value_dim=vd if vd != hd else 0, keep_first=int(params.get("keep_first") or 0) if window else 0)
        taps = int(params.get("conv_taps") or 0)
        if taps > 1:
            return (paged, FixedState((taps - 1, nh * hd + nkv * hd + nkv * vd), torch.float32))
        return paged

    def __init__(self, params: dict, weights: dict, dtype: torch.dtype):
        self.H = int(params["hidden_size"])
        self.nh, self.nkv, self.hd, self.vd = self._sizes(params)
        if self.nh % self.nkv:
            raise ConfigError(f"sink_attention: {self.nh} heads are not a multiple of {self.nkv} key/value heads")
        self.scale, self.window = float(params["scale"]), int(params.get("window") or 0)
        self.taps = int(params.get("conv_taps") or 0)
        self.dtype = dtype
        f32 = lambda *names: torch.cat([weights[n].to(torch.float32).reshape(-1) for n in names]).contiguous()
        self.keep_first = int(params.get("keep_first") or 0) if self.window else 0
        self.fixed_sink = params.get("fixed_sink")
        if self.fixed_sink is not None and params.get("sinks", True):
            raise ConfigError("sink_attention: a fixed sink beside learned ones")
        # the gate's rows ride behind q | k | v: one product over the mixer's input forms all of them as 32-bit sums
        mats = [weights["q_proj"], weights["k_proj"], weights["v_proj"]] + ([weights["gate"]] if params.get("head_gate") else [])
        self.gated = bool(params.get("head_gate"))
        self.temperature = f32("temperature") if params.get("head_temperature") else None
        self.qkv = Linear(stack_rows(*mats), dtype)
        self.out_proj = Linear(weights["out_proj"], dtype)
        self.out32 = bool(params.get("out_dtype32", False))
        self.bias = f32("q_bias", "k_bias", "v_bias") if params.get("bias") else None
        self.conv_w = None
        if self.taps:
            self.conv_w = torch.cat([weights[n].to(torch.float32) for n in ("q_conv", "k_conv", "v_conv")], dim=0).contiguous()
        self.eps = params.get("qk_norm_eps")
        self.q_norm_w = self.k_norm_w = None
        if self.eps is not None:
            self.q_norm_w, self.k_norm_w = f32("q_norm"), f32("k_norm")
        self.sinks = f32("sinks") if params.get("sinks", True) else None
        # one sink score for every head: the tensor-core kernel takes it as a vector (made here, not in a step that may be
        # captured in a graph)
        self._fixed = None
        if self.fixed_sink is not None:
            self._fixed = torch.full((self.nh,), float(self.fixed_sink), dtype=torch.float32, device=weights["q_proj"].device)
        dev = weights["q_proj"].device
        pos: PartSpec | None = params.get("position")
        self.position = part_class("position", pos.kind)(pos.params, dev) if pos is not None else None
        self.rot, self.interleaved, self.qk_freq = 0, False, None
        if self.position is not None:
            r = self.position.rotation()
            if r is None:
                raise ConfigError("sink_attention: the position encoding must be a rotation")
            self.rot, self.interleaved, self.qk_freq = int(r[0]), bool(r[1]), r[2]
        self.v_freq = None
        if params.get("value_theta") is not None:
            if self.vd % 2:
                raise ConfigError(f"sink_attention: values of {self.vd} entries cannot be rotated in pairs")
            self.v_freq = split_inv_freq(float(params["value_theta"]), self.vd).to(dev)
        self.n_needs = 2 if self.taps > 1 else 1

    def _tcgen05(self, ctx: StepContext, pages: CacheBinding) -> bool:
        from ..ops._state import sm_count
        from ..ops.attention import attention_tc_fills, attention_tc_supports
        from ..runtime.program import OPTIONS as RUN
        if not OPTIONS["tcgen05"] or self.scale <= 0 or not attention_tc_supports(self.hd, self.nh, self.nkv, pages.page_size):
            return False
        return attention_tc_fills(ctx.q_lens, self.nh, self.nkv, sm_count(ctx.device), RUN["attention_tc_min_ctas"], RUN["attention_tc_min_fill"])

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheBinding) -> torch.Tensor:
        from .. import ops
        b = bindings_of(cache, self.n_needs)
        pages = b[0]
        conv_state = b[1].state if self.taps > 1 else None
        proj = self.qkv(x, out_dtype=torch.float32)
        q = ops.sink_attn_prep(proj, 0, self.bias, self.conv_w, self.taps, conv_state, self.q_norm_w, self.k_norm_w,
                               float(self.eps or 0.0), self.qk_freq, self.rot, self.v_freq, self.interleaved, ctx, pages,
                               self.nh, self.nkv, self.hd, self.vd, self.dtype, self.temperature)
        if conv_state is not None:
            ops.conv_state_update(conv_state, proj, 0, self.bias, self.taps, ctx)
        gate = proj[:, proj.shape[1] - self.nh:] if self.gated else None
        tc = self.dtype == torch.bfloat16 and self.hd == self.vd and self.hd in (32, 64, 128) and OPTIONS["tensor_cores"]
        general = bool(self.keep_first) or self.fixed_sink is not None or gate is not None
        if tc and (general or self.v_freq is None):
            sinks = self.sinks if self.fixed_sink is None else self._fixed
            if general and self.v_freq is not None:
                raise ConfigError("sink_attention: rotated values beside kept first keys, a fixed sink or a gate per head")
            if not self.keep_first and self._tcgen05(ctx, pages):
                # prompt portions that fill its tiles: scores and outputs in tensor memory (heads of 64)
                from ..ops.attention import attention_tc
                o = attention_tc(q, pages.k, pages.v, ctx.cu_seqlens, ctx.ctx_lens, pages.block_table, ctx.q_lens, self.nh, self.scale,
                                 self.window, ctx.err, sinks, gate)
            else:
                o = ops.attention_flash_masked(q, pages, ctx, self.nh, self.nkv, self.hd, self.scale, self.window, self.keep_first, sinks, gate)
        elif tc:
            o = ops.attention_flash_sink(q, pages, ctx, self.nh, self.nkv, self.hd, self.scale, self.window, self.sinks,
                                         self.v_freq, self.interleaved)
        elif self.keep_first or self.fixed_sink is not None or gate is not None:
            if self.v_freq is not None:
                raise ConfigError("sink_attention: rotated values beside kept first keys, a fixed sink or a gate per head")
            o = ops.attention_plain_masked(q, pages, ctx, self.nh, self.nkv, self.hd, self.vd, self.scale, self.window, self.keep_first,
                                           self.sinks, self.fixed_sink, gate)
        else:
            o = ops.attention_plain_sink(q, pages, ctx, self.nh, self.nkv, self.hd, self.vd, self.scale, self.window, self.sinks,
                                         self.v_freq, self.interleaved)
        return self.out_proj(o, out_dtype=torch.float32 if self.out32 else None)


register_mixer("sink_attention", SinkAttentionMixer)
