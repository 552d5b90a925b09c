"""Padadra as a plan: a decoder whose layers run a mixer and a feed-forward side by side, each behind an RMS norm of
its own with a single number as its weight, and whose sum joins the 32-bit stream times a constant:
x += m (mixer(norm1(x)) + ff(norm2(x))). The embedding adds a row of a second table chosen by a hash of the token and
the one before it.

Mixers, in the order the configuration lists them:

* `parallel`: two mixers read the same input, and the result is half the sum of their outputs, each RMS-normed over
  the model's width. The left one is a windowed attention with a learned sink per head, short convolutions on q, k
  and v, a norm over the whole projection, a rotation with stretched frequencies, and values that are rotated too
  (and the heads' sums turned back); the right one is an HGRN2 recurrence.
* `channel_delta`: the gated delta rule with a decay per head and key channel.

The feed-forward is two matrices around the square of relu. The ranks of the delta rule's two low-rank products are
no configuration keys: the file's tensors give them (the optional keys `decay_rank` and `gate_rank` name them where
random weights are to be written).

Tensor names: `embed`, `bigram`, `final.norm`, `head`, and for layer i `l<i>.norm1|norm2`, `l<i>.mlp.up|down`,
`l<i>.mix.left.q|k|v` (+ `.b`, `.conv`), `l<i>.mix.left.q.norm|k.norm|sink|o`, `l<i>.mix.right.q|f|f.b|lower|v|norm|o`,
`l<i>.mix.left.out|right.out`; `l<i>.mix.q|k|v` (+ `.conv`), `l<i>.mix.b|A_log|norm|a1|a2|dt_bias|g1|g2|o`."""
from __future__ import annotations

from ..config.padadra import ChannelDelta, PadadraConfig, ParallelMixer
from ..config.plan import LayerSpec, ModelPlan, OrderEntry, PartSpec
from ..config.registry import register_architecture

MAX_POSITIONS = 1 << 20      # the design has no limit of its own; angles are formed from 32-bit positions


def _norm(cfg: PadadraConfig, tensor: str) -> PartSpec:
    return PartSpec("rms_norm", {"dim": cfg.width, "eps": cfg.norm_eps, "scalar": True}, {"weight": tensor})


def _sink_attention(cfg: PadadraConfig, a, p: str) -> tuple[PartSpec, dict]:
    position = None
    if a.rot is not None:
        position = PartSpec("rope", {"head_dim": a.dim, "rotary_dim": a.rot.dims, "theta": a.rot.base, "layout": "interleaved",
                                     "scaling": a.rot.scaling.to_dict() if a.rot.scaling is not None else None})
    params = {"hidden_size": cfg.width, "num_heads": a.heads, "num_kv_heads": a.kv_heads, "head_dim": a.dim, "value_dim": a.vdim,
              "scale": a.scale, "window": a.window, "bias": True, "conv_taps": a.conv, "qk_norm_eps": cfg.norm_eps,
              "position": position, "value_theta": a.rot.base if a.rot is not None else None, "sinks": True}
    names = {"q_proj": p + "q", "k_proj": p + "k", "v_proj": p + "v", "out_proj": p + "o",
             "q_bias": p + "q.b", "k_bias": p + "k.b", "v_bias": p + "v.b",
             "q_norm": p + "q.norm", "k_norm": p + "k.norm", "sinks": p + "sink"}
    if a.conv:
        names.update(q_conv=p + "q.conv", k_conv=p + "k.conv", v_conv=p + "v.conv")
    return PartSpec("sink_attention", params, names), names


def _mixer(cfg: PadadraConfig, layer, p: str) -> PartSpec:
    H, m = cfg.width, layer.mixer
    if isinstance(m, ParallelMixer):
        left, left_names = _sink_attention(cfg, m.left, p + "mix.left.")
        r = p + "mix.right."
        right_names = {"q": r + "q", "f": r + "f", "f_bias": r + "f.b", "lower": r + "lower", "v": r + "v", "norm": r + "norm", "o": r + "o"}
        right = PartSpec("hgrn2", {"hidden_size": H, "heads": m.right.heads, "dim": m.right.dim, "value_dim": m.right.vdim,
                                   "eps": cfg.norm_eps}, right_names)
        names = {"first_out": p + "mix.left.out", "second_out": p + "mix.right.out"}
        names.update({"first." + k: v for k, v in left_names.items()})
        names.update({"second." + k: v for k, v in right_names.items()})
        return PartSpec("side_by_side", {"hidden_size": H, "eps": cfg.norm_eps, "first": left, "second": right}, names)
    assert isinstance(m, ChannelDelta)
    q = p + "mix."
    names = {"q": q + "q", "k": q + "k", "v": q + "v", "q_conv": q + "q.conv", "k_conv": q + "k.conv", "v_conv": q + "v.conv",
             "beta": q + "b", "a1": q + "a1", "a2": q + "a2", "dt_bias": q + "dt_bias", "A_log": q + "A_log",
             "g1": q + "g1", "g2": q + "g2", "norm": q + "norm", "o": q + "o"}
    return PartSpec("gated_delta", {"hidden_size": H, "heads": m.heads, "qk_heads": m.kv_heads, "dim": m.dim, "value_dim": m.vdim,
                                    "conv_taps": m.conv, "eps": cfg.norm_eps, "decay_rank": m.decay_rank or -1,
                                    "gate_rank": m.gate_rank or -1}, names)


def build_plan(cfg: PadadraConfig) -> ModelPlan:
    H = cfg.width
    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        ffn = ffn_norm = None
        if layer.mlp is not None:
            ffn = PartSpec("dense_mlp", {"hidden_size": H, "ff_dim": layer.mlp.ff, "activation": "relu2"},
                           {"up": p + "mlp.up", "down": p + "mlp.down"})
            ffn_norm = _norm(cfg, p + "norm2")
        layers.append(LayerSpec(PartSpec("parallel_two_norms", {"residual_mult": cfg.residual_mult}), _mixer(cfg, layer, p), ffn,
                                _norm(cfg, p + "norm1"), ffn_norm))
    if cfg.bigram is not None:
        b = cfg.bigram
        embedding = PartSpec("lookup_pairs", {"vocab_size": cfg.vocab, "dim": H, "scale": cfg.embedding_scale, "buckets": b.buckets,
                                              "mul_prev": b.mul_prev, "mul_cur": b.mul_cur}, {"weight": "embed", "pairs": "bigram"})
    else:
        embedding = PartSpec("lookup", {"vocab_size": cfg.vocab, "dim": H, "scale": cfg.embedding_scale}, {"weight": "embed"})
    return ModelPlan(hidden_size=H, vocab_size=cfg.vocab, max_positions=MAX_POSITIONS, embedding=embedding,
                     final_norm=_norm(cfg, "final.norm"), head="head", layers=tuple(layers),
                     order=tuple(OrderEntry(i) for i in range(len(layers))), eos_token_id=cfg.eos_token_id,
                     unread_tensors=tuple(f"l{i}.norm2" for i, layer in enumerate(cfg.layers) if layer.mlp is None))


register_architecture("Padadra", PadadraConfig, build_plan, model_types=("padadra",))
