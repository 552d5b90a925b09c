"""Mixers whose state is a matrix per head, S [dim, value_dim] in 32-bit floats in the request's slot (zero at its start).

`hgrn2`: linear attention in which the forget gate also decides what is written.

    q = silu(W_q h)    v = W_v h    f = l + (1 - l) sigmoid(W_f h + b_f)      (l: a learned lower bound per channel)
    S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T        o_t = S_t^T q_t
    out = W_o (rms_norm(o_t per head) * w, heads side by side)

`gated_delta`: the gated delta rule with one decay per head and key channel.

    q, k, v = silu(conv(W h))   (a short causal convolution over time per channel)
    q, k unit vectors per head (x / sqrt(sum x^2 + 1e-6)), q also times dim^-1/2;   beta = sigmoid(W_b h)
    g = exp(-exp(A_log_h) * softplus(W_a2 (W_a1 h) + dt_bias))     per head and key channel
    S <- diag(g) S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q
    out = W_o (rms_norm(o per head) * w * sigmoid(W_g2 (W_g1 h)))
    Value head h reads the q and k of head floor(h / (heads / qk_heads)).

`general_delta`: the generalized delta rule, whose decay and removal both read the old state.

    r, k, v = W h   (heads x dim each)
    d = exp(-rate * sigmoid(W_w2 tanh(W_w1 h) + w0))    a decay per head and key channel (rate: a constant, exp(-1/2) by default)
    a = sigmoid(W_a h + a_bias)                         a removal rate per head and key channel
    u = k / sqrt(sum(k^2) + unit_eps)                   the unit key of each head
    S <- diag(d) S - (a * u)(u^T S) + k v^T (the old S on the right);   o = S^T r
    out = W_o (rms_norm(o per head) * w * sigmoid(W_g h))    (w: a row for every head)

`weighted_pair`: two mixers side by side over the same input, out = a * first(h) + b * second(h) with constants a, b.

Everything that enters a recurrence is 32-bit (the projections keep their 32-bit sums; gates, decays, unit vectors and
the state are computed in 32-bit), and a request's tokens are walked in order from the state the step before left, so
the state after a token does not depend on how the sequence was cut. The delta rule also keeps the convolution's last
taps - 1 projected rows in the slot."""
from __future__ import annotations

import torch

from ..config.errors import ConfigError
from .base import CacheBinding, FixedState, Mixer, StepContext, TensorSpec
from .linear import Linear, stack_rows
from .registry import register_mixer
from .sink_attention import bindings_of


def _f32(weights: dict, *names) -> torch.Tensor:
    return torch.cat([weights[n].to(torch.float32).reshape(-1) for n in names]).contiguous()


class Hgrn2Mixer(Mixer):
    graph_safe = True

    """params: hidden_size, heads, dim, value_dim, eps, out_dtype32 (default False).
    weights: q, f [heads*dim, H]; f_bias, lower [heads*dim]; v [heads*vd, H]; norm [vd]; o [H, heads*vd]."""

    @classmethod
    def weight_specs(cls, params):
        H, h, d, vd = (int(params[k]) for k in ("hidden_size", "heads", "dim", "value_dim"))
        return {"q": TensorSpec((h * d, H), "linear"), "f": TensorSpec((h * d, H), "linear"), "f_bias": TensorSpec((h * d,), "bias"),
                "lower": TensorSpec((h * d,), "unit_interval"), "v": TensorSpec((h * vd, H), "linear"),
                "norm": TensorSpec((vd,), "norm"), "o": TensorSpec((H, h * vd), "linear")}

    @classmethod
    def cache_need(cls, params):
        return FixedState((int(params["heads"]), int(params["dim"]), int(params["value_dim"])), torch.float32)

    def __init__(self, params: dict, weights: dict, dtype: torch.dtype):
        self.H, self.heads, self.dim, self.vd = (int(params[k]) for k in ("hidden_size", "heads", "dim", "value_dim"))
        self.eps, self.dtype = float(params["eps"]), dtype
        self.in_proj = Linear(stack_rows(weights["q"], weights["f"], weights["v"]), dtype)
        self.out_proj = Linear(weights["o"], dtype)
        self.out32 = bool(params.get("out_dtype32", False))
        self.f_bias, self.lower, self.norm_w = _f32(weights, "f_bias"), _f32(weights, "lower"), _f32(weights, "norm")

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheBinding) -> torch.Tensor:
        from .. import ops
        state = bindings_of(cache, 1)[0].state
        hd = self.heads * self.dim
        proj = self.in_proj(x, out_dtype=torch.float32)
        o = ops.hgrn2_scan(proj, 0, hd, 2 * hd, self.f_bias, self.lower, state, ctx, self.heads, self.dim, self.vd)
        y = ops.head_norm_gate(o, self.norm_w, None, self.heads, self.vd, self.eps, self.dtype)
        return self.out_proj(y, out_dtype=torch.float32 if self.out32 else None)


register_mixer("hgrn2", Hgrn2Mixer)


class GatedDeltaMixer(Mixer):
    graph_safe = True

    """params: hidden_size, heads, qk_heads, dim, value_dim, conv_taps, eps, decay_rank, gate_rank (-1: whatever the
    file's tensors have), unit_eps (default 1e-6).
    weights: q, k [qk_heads*dim, H]; v [heads*vd, H]; q_conv, k_conv [qk_heads*dim, taps]; v_conv [heads*vd, taps];
    beta [heads, H]; a1 [decay_rank, H], a2 [heads*dim, decay_rank], dt_bias [heads*dim], A_log [heads];
    g1 [gate_rank, H], g2 [heads*vd, gate_rank]; norm [vd]; o [H, heads*vd]."""

    @classmethod
    def weight_specs(cls, params):
        H, h, g, d, vd, taps = (int(params[k]) for k in ("hidden_size", "heads", "qk_heads", "dim", "value_dim", "conv_taps"))
        ra, rg = int(params.get("decay_rank", -1)), int(params.get("gate_rank", -1))
        return {"q": TensorSpec((g * d, H), "linear"), "k": TensorSpec((g * d, H), "linear"), "v": TensorSpec((h * vd, H), "linear"),
                "q_conv": TensorSpec((g * d, taps), "conv_tap_wide"), "k_conv": TensorSpec((g * d, taps), "conv_tap_wide"),
                "v_conv": TensorSpec((h * vd, taps), "conv_tap_wide"), "beta": TensorSpec((h, H), "linear"),
                "a1": TensorSpec((ra, H), "linear"), "a2": TensorSpec((h * d, ra), "linear_wide"), "dt_bias": TensorSpec((h * d,), "bias"),
                "A_log": TensorSpec((h,), "log_rate"), "g1": TensorSpec((rg, H), "linear"), "g2": TensorSpec((h * vd, rg), "linear_wide"),
                "norm": TensorSpec((vd,), "norm"), "o": TensorSpec((H, h * vd), "linear")}

    @classmethod
    def cache_need(cls, params):
        h, g, d, vd, taps = (int(params[k]) for k in ("heads", "qk_heads", "dim", "value_dim", "conv_taps"))
        state = FixedState((h, d, vd), torch.float32)
        if taps > 1:
            return (FixedState((taps - 1, 2 * g * d + h * vd), torch.float32), state)
        return state

    def __init__(self, params: dict, weights: dict, dtype: torch.dtype):
        self.H, self.heads, self.qkh, self.dim, self.vd, self.taps = (
            int(params[k]) for k in ("hidden_size", "heads", "qk_heads", "dim", "value_dim", "conv_taps"))
        if self.heads % self.qkh:
            raise ConfigError(f"gated_delta: {self.heads} heads are not a multiple of {self.qkh} query/key heads")
        self.eps, self.unit_eps, self.dtype = float(params["eps"]), float(params.get("unit_eps", 1e-6)), dtype
        self.ra, self.rg = int(weights["a1"].shape[0]), int(weights["g1"].shape[0])
        if weights["a2"].shape[1] != self.ra or weights["g2"].shape[1] != self.rg:
            raise ConfigError("gated_delta: the two matrices of a low-rank product do not fit each other")
        self.in_proj = Linear(stack_rows(weights["q"], weights["k"], weights["v"], weights["beta"]), dtype)
        self.low_proj = Linear(stack_rows(weights["a1"], weights["g1"]), dtype)
        # the two second halves as one product: a2 and g2 on the diagonal of one matrix over a1's and g1's outputs side by
        # side (the zeros add nothing to a sum), so the decays' and the gate's pre-activations come from one launch
        a2, g2 = weights["a2"], weights["g2"]
        both = torch.zeros((a2.shape[0] + g2.shape[0], self.ra + self.rg), dtype=a2.dtype if a2.dtype == g2.dtype else torch.float32,
                           device=a2.device)
        both[:a2.shape[0], :self.ra] = a2
        both[a2.shape[0]:, self.ra:] = g2
        self.second = Linear(both, dtype)
        self.out_proj = Linear(weights["o"], dtype)
        self.conv_w = torch.cat([weights[n].to(torch.float32) for n in ("q_conv", "k_conv", "v_conv")], dim=0).contiguous()
        self.dt_bias, self.A_log, self.norm_w = _f32(weights, "dt_bias"), _f32(weights, "A_log"), _f32(weights, "norm")
        self.n_needs = 2 if self.taps > 1 else 1

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheBinding) -> torch.Tensor:
        from .. import ops
        b = bindings_of(cache, self.n_needs)
        conv_state = b[0].state if self.taps > 1 else None
        state = b[-1].state
        proj = self.in_proj(x, out_dtype=torch.float32)
        low = self.low_proj(x)
        second = self.second(low, out_dtype=torch.float32)
        a, gate = second[:, :self.heads * self.dim], second[:, self.heads * self.dim:]
        C = 2 * self.qkh * self.dim + self.heads * self.vd
        qk, v, beta, decay = ops.delta_prep(proj, 0, C, self.conv_w, self.taps, conv_state, a, self.dt_bias, self.A_log, ctx,
                                            self.heads, self.qkh, self.dim, self.vd, self.unit_eps)
        if conv_state is not None:
            ops.conv_state_update(conv_state, proj, 0, None, self.taps, ctx)
        o = ops.delta_scan(qk, v, beta, decay, state, ctx, self.heads, self.qkh, self.dim, self.vd)
        y = ops.head_norm_gate(o, self.norm_w, gate, self.heads, self.vd, self.eps, self.dtype)
        return self.out_proj(y)


register_mixer("gated_delta", GatedDeltaMixer)


class GeneralDeltaMixer(Mixer):
    graph_safe = True

    """params: hidden_size, heads, dim, eps, rate (default exp(-1/2)), unit_eps (default 1e-6), decay_rank (-1: whatever the
    file's tensor has), out_dtype32 (default False).
    weights: r, k, v, g, a [heads*dim, H]; a_bias [heads*dim]; w1 [decay_rank, H], w2 [heads*dim, decay_rank], w0 [heads*dim];
    norm [heads*dim]; o [H, heads*dim]."""

    @classmethod
    def weight_specs(cls, params):
        H, h, d = (int(params[k]) for k in ("hidden_size", "heads", "dim"))
        rank = int(params.get("decay_rank", -1))
        n = h * d
        return {"r": TensorSpec((n, H), "linear"), "k": TensorSpec((n, H), "linear"), "v": TensorSpec((n, H), "linear"),
                "g": TensorSpec((n, H), "linear"), "a": TensorSpec((n, H), "linear"), "a_bias": TensorSpec((n,), "bias"),
                "w1": TensorSpec((rank, H), "linear"), "w2": TensorSpec((n, rank), "linear_wide"), "w0": TensorSpec((n,), "bias"),
                "norm": TensorSpec((n,), "norm"), "o": TensorSpec((H, n), "linear")}

    @classmethod
    def cache_need(cls, params):
        return FixedState((int(params["heads"]), int(params["dim"]), int(params["dim"])), torch.float32)

    def __init__(self, params: dict, weights: dict, dtype: torch.dtype):
        import math
        self.H, self.heads, self.dim = (int(params[k]) for k in ("hidden_size", "heads", "dim"))
        self.eps, self.unit_eps, self.dtype = float(params["eps"]), float(params.get("unit_eps", 1e-6)), dtype
        self.rate = float(params.get("rate", math.exp(-0.5)))
        if weights["w2"].shape[1] != weights["w1"].shape[0]:
            raise ConfigError("general_delta: the two matrices of the decay's low-rank product do not fit each other")
        self.rank = int(weights["w1"].shape[0])
        # one product over the mixer's input: r | k | v | a | g | the decay's first matrix, as 32-bit sums
        self.in_proj = Linear(stack_rows(weights["r"], weights["k"], weights["v"], weights["a"], weights["g"], weights["w1"]), dtype)
        self.w2 = Linear(weights["w2"], dtype)
        self.out_proj = Linear(weights["o"], dtype)
        self.out32 = bool(params.get("out_dtype32", False))
        self.a_bias, self.w0, self.norm_w = _f32(weights, "a_bias"), _f32(weights, "w0"), _f32(weights, "norm")

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheBinding) -> torch.Tensor:
        from .. import ops
        state = bindings_of(cache, 1)[0].state
        n = self.heads * self.dim
        proj = self.in_proj(x, out_dtype=torch.float32)
        low = ops.activation(proj[:, 5 * n:], "tanh", self.dtype)
        w_pre = self.w2(low, out_dtype=torch.float32)
        vecs = ops.gdelta_prep(proj, n, 3 * n, w_pre, self.w0, self.a_bias, self.rate, self.unit_eps, self.heads, self.dim)
        o = ops.gdelta_scan(proj, 0, n, 2 * n, vecs, state, ctx, self.heads, self.dim, self.dim)
        y = ops.head_norm_gate(o, self.norm_w, proj[:, 4 * n:5 * n], self.heads, self.dim, self.eps, self.dtype)
        return self.out_proj(y, out_dtype=torch.float32 if self.out32 else None)


register_mixer("general_delta", GeneralDeltaMixer)


class SideBySideMixer(Mixer):
    graph_safe = True

    """Two mixers that read the same input; the result is half the sum of their outputs, each first RMS-normed over the
    model's width with a plain weight of its own:  out = (rms_norm(A(h)) * w_a + rms_norm(B(h)) * w_b) / 2.
    Both keep their own caches: the item's needs are the first mixer's followed by the second's.

    params: hidden_size, eps, first, second (PartSpecs of registered mixers; their weights' names are prefixed
    `first.` and `second.` here). weights: first_out, second_out [H] and the two mixers' own."""

    @staticmethod
    def _subs(params):
        from .registry import part_class
        return [(name, params[name], part_class("mixer", params[name].kind)) for name in ("first", "second")]

    @classmethod
    def weight_specs(cls, params):
        H = int(params["hidden_size"])
        specs = {"first_out": TensorSpec((H,), "norm"), "second_out": TensorSpec((H,), "norm")}
        for name, spec, klass in cls._subs(params):
            for local, ts in klass.weight_specs(spec.params).items():
                specs[f"{name}.{local}"] = ts
        return specs

    @classmethod
    def cache_need(cls, params):
        needs = []
        for name, spec, klass in cls._subs(params):
            n = klass.cache_need(spec.params)
            needs += list(n) if isinstance(n, (tuple, list)) else ([n] if n is not None else [])
        return tuple(needs) if len(needs) != 1 else needs[0]

    def __init__(self, params: dict, weights: dict, dtype: torch.dtype):
        self.H, self.eps, self.dtype = int(params["hidden_size"]), float(params["eps"]), dtype
        self.parts, self.counts = [], []
        for name, spec, klass in self._subs(params):
            own = {k[len(name) + 1:]: v for k, v in weights.items() if k.startswith(name + ".")}
            sub_params = dict(spec.params)
            sub_params.setdefault("out_dtype32", True)      # the norm over the result reads the product's 32-bit sums
            self.parts.append(klass(sub_params, own, dtype))
            n = klass.cache_need(spec.params)
            self.counts.append(len(n) if isinstance(n, (tuple, list)) else (0 if n is None else 1))
        self.first, self.second = self.parts
        self.w_first, self.w_second = _f32(weights, "first_out"), _f32(weights, "second_out")

    def _binding(self, cache: CacheBinding, start: int, n: int) -> CacheBinding:
        every = cache.parts if cache.parts else (cache,)
        mine = every[start:start + n]
        if n == 1:
            return mine[0]
        return CacheBinding(need=tuple(p.need for p in mine), writes=cache.writes, parts=tuple(mine))

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheBinding) -> torch.Tensor:
        from .. import ops
        a = self.first.forward(x, ctx, self._binding(cache, 0, self.counts[0]))
        b = self.second.forward(x, ctx, self._binding(cache, self.counts[0], self.counts[1]))
        if a.dtype != torch.float32:
            a = a.to(torch.float32)
        if b.dtype != torch.float32:
            b = b.to(torch.float32)
        return ops.pair_norm_mean(a.contiguous(), b.contiguous(), self.w_first, self.w_second, self.eps, self.dtype)


register_mixer("side_by_side", SideBySideMixer)


class WeightedPairMixer(SideBySideMixer):
    graph_safe = True

    """Two mixers that read the same input; the result is first_scale * first(h) + second_scale * second(h), formed in
    32-bit from the two mixers' 32-bit results and returned so. Both keep their own caches: the item's needs are the first
    mixer's followed by the second's.

    params: hidden_size, first, second (PartSpecs of registered mixers; their weights' names are prefixed `first.` and
    `second.` here), first_scale, second_scale."""

    @classmethod
    def weight_specs(cls, params):
        specs = {}
        for name, spec, klass in cls._subs(params):
            for local, ts in klass.weight_specs(spec.params).items():
                specs[f"{name}.{local}"] = ts
        return specs

    def __init__(self, params: dict, weights: dict, dtype: torch.dtype):
        self.H, self.dtype = int(params["hidden_size"]), dtype
        self.scales = (float(params["first_scale"]), float(params["second_scale"]))
        self.parts, self.counts = [], []
        for name, spec, klass in self._subs(params):
            own = {k[len(name) + 1:]: v for k, v in weights.items() if k.startswith(name + ".")}
            sub_params = dict(spec.params)
            sub_params.setdefault("out_dtype32", True)
            self.parts.append(klass(sub_params, own, dtype))
            n = klass.cache_need(spec.params)
            self.counts.append(len(n) if isinstance(n, (tuple, list)) else (0 if n is None else 1))
        self.first, self.second = self.parts

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheBinding) -> torch.Tensor:
        from .. import ops
        a = self.first.forward(x, ctx, self._binding(cache, 0, self.counts[0]))
        b = self.second.forward(x, ctx, self._binding(cache, self.counts[0], self.counts[1]))
        if a.dtype != b.dtype:
            a, b = a.to(torch.float32), b.to(torch.float32)
        return ops.weighted_sum2(a.contiguous(), self.scales[0], b.contiguous(), self.scales[1])


register_mixer("weighted_pair", WeightedPairMixer)
