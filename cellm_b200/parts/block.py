"""Pre-norm arrangement of a layer (crates/cellm-model/src/lfm.rs:333-347,
:610-629, :665-667): x += mixer(norm(x)); x += feed_forward(norm(x))."""
from __future__ import annotations

from .base import Block, CacheBinding, Residual, StepContext
from .registry import register_block


class PreNormBlock(Block):
    graph_safe = True

    def __init__(self, mixer_norm, mixer, feed_forward_norm, feed_forward):
        self.mixer_norm, self.mixer = mixer_norm, mixer
        self.feed_forward_norm, self.feed_forward = feed_forward_norm, feed_forward

    def emit(self, emitter) -> None:
        """The layer as records: each of the four parts emits its own, in the order they run."""
        for part in (self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward):
            part.emit(emitter)

    def forward(self, residual: Residual, ctx: StepContext, cache: CacheBinding) -> None:
        residual.add(self.mixer.forward(self.mixer_norm.forward(residual), ctx, cache))
        residual.add(self.feed_forward.forward(self.feed_forward_norm.forward(residual), ctx))


register_block("pre_norm", PreNormBlock)


class ParallelBlock(Block):
    """A layer with one norm whose output both sublayers read: h = norm(x); x += mixer(h) + feed_forward(h).
    The layer may have no feed-forward. Both results wait as addends of the 32-bit stream; the next norm adds them."""
    graph_safe = True

    def __init__(self, mixer_norm, mixer, feed_forward_norm, feed_forward):
        from ..config.errors import ConfigError
        if feed_forward_norm is not None:
            raise ConfigError("parallel: the layer has one norm; its feed-forward reads the mixer's input")
        self.mixer_norm, self.mixer = mixer_norm, mixer
        self.feed_forward_norm, self.feed_forward = None, feed_forward

    def emit(self, emitter) -> None:
        self.mixer_norm.emit(emitter)
        self.mixer.emit(emitter)
        if self.feed_forward is not None:
            self.feed_forward.emit(emitter)

    def forward(self, residual: Residual, ctx: StepContext, cache: CacheBinding) -> None:
        h = self.mixer_norm.forward(residual)
        residual.add(self.mixer.forward(h, ctx, cache))
        if self.feed_forward is not None:
            residual.add(self.feed_forward.forward(h, ctx))


register_block("parallel", ParallelBlock)


class TwoNormParallelBlock(Block):
    """A layer whose mixer and feed-forward read the same stream through a norm each, and whose sum joins the stream
    times a constant:  x += mult * (mixer(norm1(x)) + feed_forward(norm2(x))). The layer may have no feed-forward.
    Both norms must be RMS norms with one eps and no groups: the stream is read once for both. The sum is 32-bit.

    params: residual_mult (default 1)."""
    graph_safe = True

    def __init__(self, mixer_norm, mixer, feed_forward_norm, feed_forward, params=None, weights=None, dtype=None):
        from ..config.errors import ConfigError
        self.mixer_norm, self.mixer = mixer_norm, mixer
        self.feed_forward_norm, self.feed_forward = feed_forward_norm, feed_forward
        self.mult = float((params or {}).get("residual_mult", 1.0))
        self.dtype = dtype
        if (feed_forward is None) != (feed_forward_norm is None):
            raise ConfigError("parallel_two_norms: a feed-forward and its norm come together")
        for n in (mixer_norm, feed_forward_norm):
            if n is not None and (not all(hasattr(n, a) for a in ("weight", "eps", "groups")) or n.groups != 1):
                raise ConfigError("parallel_two_norms: the norms must be RMS norms without groups")
        if feed_forward_norm is not None and (feed_forward_norm.eps != mixer_norm.eps or
                                              feed_forward_norm.weight.dtype != mixer_norm.weight.dtype):
            raise ConfigError("parallel_two_norms: the two norms must have one eps and one element type")

    def forward(self, residual: Residual, ctx: StepContext, cache: CacheBinding) -> None:
        from .. import ops
        x = residual.flush()
        n1, n2 = self.mixer_norm, self.feed_forward_norm
        y1, y2 = ops.norm_pair(x, n1.weight, n2.weight if n2 is not None else None, n1.eps, self.dtype)
        a = self.mixer.forward(y1, ctx, cache)
        b = self.feed_forward.forward(y2, ctx) if self.feed_forward is not None else None
        ops.scaled_add2(x, a, b, self.mult)


register_block("parallel_two_norms", TwoNormParallelBlock)


class GatedPostNormBlock(Block):
    """A layer whose sublayers read the residual stream itself and whose norm sits on the sublayer's result:

        x += norm1(mixer(x) * sigmoid(G1 x + g1));    x += norm2(feed_forward(x) * sigmoid(G2 x + g2))

    The gates (`gate`: True) are the block's own weights; a layer without a feed-forward has the first line only. The
    norms must be RMS norms (in groups or not): gate, norm and the sum into the stream are one kernel, which also
    leaves the stream in the activations' type for the next sublayer's products.

    params: hidden_size, gate (default False). weights: mixer_gate, feed_forward_gate [H, H] and mixer_gate_bias,
    feed_forward_gate_bias [H] if gate (the feed-forward's only if the layer has one)."""
    graph_safe = True

    @classmethod
    def weight_specs(cls, params):
        from .base import TensorSpec
        H = params["hidden_size"]
        specs = {}
        if params.get("gate"):
            specs["mixer_gate"] = TensorSpec((H, H), "linear")
            specs["mixer_gate_bias"] = TensorSpec((H,), "bias")
            if params.get("feed_forward", True):
                specs["feed_forward_gate"] = TensorSpec((H, H), "linear")
                specs["feed_forward_gate_bias"] = TensorSpec((H,), "bias")
        return specs

    def __init__(self, mixer_norm, mixer, feed_forward_norm, feed_forward, params=None, weights=None, dtype=None):
        from ..config.errors import ConfigError
        from .linear import Linear
        self.mixer_norm, self.mixer = mixer_norm, mixer
        self.feed_forward_norm, self.feed_forward = feed_forward_norm, feed_forward
        params, weights = params or {}, weights or {}
        self.dtype = dtype
        for n in (mixer_norm, feed_forward_norm):
            if n is not None and not all(hasattr(n, a) for a in ("weight", "eps", "groups")):
                raise ConfigError("gated_post_norm: the norms must be RMS norms (weight, eps, groups)")
        self.gates, self.stacked = {}, {}
        if params.get("gate"):
            for name in ("mixer", "feed_forward"):
                if name + "_gate" in weights:
                    self.gates[name] = (Linear(weights[name + "_gate"], dtype), weights[name + "_gate_bias"].contiguous())
                    # a sublayer that can form the gate with its own first product (both read the sublayer's input) is
                    # given the gate's rows; the gate-and-norm record then finds the gate where that product left it
                    part = getattr(self, name)
                    self.stacked[name] = bool(params.get("stack_gates", True)) and part.stack_behind_input(weights[name + "_gate"])
                    if self.stacked[name]:          # no second copy: the block's own matrix is those rows of the part's
                        self.gates[name] = (Linear(part.stacked_rows(), dtype), self.gates[name][1])
        self._keep = []

    def _join(self, emitter, name: str, norm) -> None:
        from ..ops._lib import tag
        from ..runtime import records as R
        p = R.GatedNormAddParams()
        if name in self.gates:
            lin, bias = self.gates[name]
            if not emitter.fits(lin.weight):
                from ..config.errors import ConfigError
                raise ConfigError("gated_post_norm: a gate kept in another element type than the activations")
            bias = bias.to(norm.weight.dtype).contiguous()      # the kernel reads bias and norm weight as one element type
            self._keep.append(bias)
            p.gate, p.gate_bias = R.linear(lin.weight), bias.data_ptr()
            p.stacked = int(self.stacked.get(name, False))
        p.w, p.w_dtype, p.groups, p.eps = norm.weight.data_ptr(), tag(norm.weight), norm.groups, norm.eps
        emitter.native(R.GATED_NORM_ADD, p, part=self)

    def emit(self, emitter) -> None:
        from ..runtime import records as R
        emitter.native(R.READ_STREAM, R.ReadStreamParams(0), part=self)
        self.mixer.emit(emitter)
        self._join(emitter, "mixer", self.mixer_norm)
        if self.feed_forward is not None:
            self.feed_forward.emit(emitter)
            self._join(emitter, "feed_forward", self.feed_forward_norm)

    def _sublayer(self, residual: Residual, name: str, norm, run) -> None:
        from .. import ops
        x = residual.flush()
        h = ops.stream_cast(x, self.dtype)
        m = run(h)
        g = b = None
        if name in self.gates:
            lin, b = self.gates[name]
            g = lin(h)
            b = b.to(norm.weight.dtype)
        ops.gated_norm_add(x, m.to(self.dtype).contiguous(), g, b, norm.weight, norm.groups, norm.eps, want_copy=False)

    def forward(self, residual: Residual, ctx: StepContext, cache: CacheBinding) -> None:
        self._sublayer(residual, "mixer", self.mixer_norm, lambda h: self.mixer.forward(h, ctx, cache))
        if self.feed_forward is not None:
            self._sublayer(residual, "feed_forward", self.feed_forward_norm, lambda h: self.feed_forward.forward(h, ctx))


register_block("gated_post_norm", GatedPostNormBlock)


class ScaledPreNormBlock(Block):
    """A pre-norm layer whose results join the 32-bit stream times a constant m, with two optional additions:

        [at the start of a pass over looped layers:  x += the embedding row once more (passes after the first);  x += step[t]]
        x += m * mixer(norm1(x));    x += m * feed_forward(norm2(x))        (the layer may have no feed-forward)
        [x += m * rms_norm(P (act(G x) * e)) * w:  e is the layer's own part of a second embedding row of the token]

    The norms may be layer norms or RMS norms (parts with `add_and_norm`): a sublayer's result is added and the next norm
    formed by one kernel. The token's own row is gated by the stream itself (not normed), in the activations' type.

    params: hidden_size, residual_mult (default 1);
      token_rows (optional): {dim, offset, eps, activation}: columns offset .. offset + dim of the second table;
      passes (optional): {order item: pass number} for the items at which this layer starts a pass, and
      embedding_scale (the factor of the embedding row that is added again).
    weights: token_table [vocab, >= offset + dim], token_gate [dim, H], token_proj [H, dim], token_norm [H] with token_rows;
      pass_steps [passes, H] and embedding [vocab, H] with passes."""
    graph_safe = True

    @classmethod
    def weight_specs(cls, params):
        from .base import TensorSpec
        H = int(params["hidden_size"])
        specs = {}
        tr = params.get("token_rows")
        if tr:
            specs["token_table"] = TensorSpec((int(tr["vocab"]), int(tr["table_width"])), "embedding")
            specs["token_gate"] = TensorSpec((int(tr["dim"]), H), "linear")
            specs["token_proj"] = TensorSpec((H, int(tr["dim"])), "linear")
            specs["token_norm"] = TensorSpec((H,), "norm")
        if params.get("passes"):
            specs["pass_steps"] = TensorSpec((int(params["n_passes"]), H), "bias")
            specs["embedding"] = TensorSpec((int(params["vocab"]), H), "embedding")
        return specs

    def __init__(self, mixer_norm, mixer, feed_forward_norm, feed_forward, params=None, weights=None, dtype=None):
        import torch
        from ..config.errors import ConfigError
        from .linear import Linear
        params, weights = params or {}, weights or {}
        self.mixer_norm, self.mixer = mixer_norm, mixer
        self.feed_forward_norm, self.feed_forward = feed_forward_norm, feed_forward
        self.H, self.mult, self.dtype = int(params["hidden_size"]), float(params.get("residual_mult", 1.0)), dtype
        if (feed_forward is None) != (feed_forward_norm is None):
            raise ConfigError("pre_norm_scaled: a feed-forward and its norm come together")
        for n in (mixer_norm, feed_forward_norm):
            if n is not None and not hasattr(n, "add_and_norm"):
                raise ConfigError("pre_norm_scaled: the norms must take an addend times a constant (layer_norm, rms_norm)")
        self.token_rows = params.get("token_rows")
        if self.token_rows:
            tr = self.token_rows
            self.token_table = weights["token_table"].contiguous()
            self.token_gate, self.token_proj = Linear(weights["token_gate"], dtype), Linear(weights["token_proj"], dtype)
            self.token_norm = weights["token_norm"].to(torch.float32).contiguous()
            self.token_offset, self.token_dim = int(tr["offset"]), int(tr["dim"])
            self.token_eps, self.token_act = float(tr["eps"]), tr.get("activation", "gelu_tanh")
            if self.token_offset + self.token_dim > self.token_table.shape[1]:
                raise ConfigError("pre_norm_scaled: the layer's part lies outside the token table's rows")
        self.passes = {int(k): int(v) for k, v in (params.get("passes") or {}).items()}
        if self.passes:
            self.pass_steps = weights["pass_steps"].to(torch.float32).contiguous()
            self.embedding = weights["embedding"].contiguous()
            self.embedding_scale = float(params.get("embedding_scale", 1.0))
            if max(self.passes.values()) >= self.pass_steps.shape[0]:
                raise ConfigError("pre_norm_scaled: more passes than step vectors")

    def forward(self, residual: Residual, ctx: StepContext, cache: CacheBinding) -> None:
        import torch
        from .. import ops
        x = residual.flush()
        if self.passes:
            t = self.passes.get(ctx.extras.get("order_item"))
            if t is not None:
                ops.stream_add_rows(x, self.embedding if t > 0 else None, ctx.token_ids, self.embedding_scale, self.pass_steps[t], ctx.err)
        m = self.mult
        a = self.mixer.forward(self.mixer_norm.add_and_norm(x, None, 0.0), ctx, cache)
        if self.feed_forward is not None:
            a = self.feed_forward.forward(self.feed_forward_norm.add_and_norm(x, a.contiguous(), m), ctx)
        if not self.token_rows:
            ops.add_scaled_norm(x, a.contiguous(), m, None, 0.0, "none", None, None, 0.0, self.dtype, want=False)
            return
        # x += m * a, and the sum in the activations' type for the gate's product
        xb = ops.add_scaled_norm(x, a.contiguous(), m, None, 0.0, "none", None, None, 0.0, self.dtype)
        g = self.token_gate(xb, out_dtype=torch.float32)
        e = ops.token_gate_mul(g, self.token_table, self.token_offset, ctx.token_ids, self.token_act, self.dtype, ctx.err)
        ops.scaled_rms_add(x, self.token_proj(e, out_dtype=torch.float32), self.token_norm, m, self.token_eps)


register_block("pre_norm_scaled", ScaledPreNormBlock)
