"""Bozovik as a plan: a pre-norm decoder with layer norms (weight and bias), whose sublayers' results join the 32-bit
stream times a constant, x += m mixer(norm1(x)); x += m ff(norm2(x)), followed in every layer by a per-token side
input: the layer's own part e of a second embedding row, x += m rms_norm(P (gelu_tanh(G x) * e)) * w. A run of layers
may be looped: it runs several times with the same weights and a cache of its own each time; every pass after the
first starts by adding the embedding's output again, and every pass adds a learned vector of its own.

Mixers, in the order the configuration lists them:

* `attention`: grouped-query attention over every earlier key, rotation of the first `rot.dims` entries of a head in
  pairs half the rotation apart, scores times a learned temperature per head, one added to the softmax's denominator,
  every head's output times a sigmoid gate formed from the mixer's input.
* `parallel`: `left_scale` times such an attention with a sliding window that keeps the sequence's first keys, a learned
  sink per head and the gate, plus `right_scale` times a generalized delta rule (a decay and a removal rate per head and
  key channel, both reading the old state).
* `latent_attention`: keys and values of all heads from one cached latent row per token, a shared rotated key part, a
  sliding window and a learned sink per head.

The feed-forward is two matrices around xIELU with two learned numbers. The rank of the decay's low-rank product is no
configuration key: the file's tensors give it (the optional key `decay_rank` names it where random weights are written).

Tensor names: `embed`, `side.embed`, `loop.step`, `final.norm` (+ `.b`), `head`, and for layer i `l<i>.norm1|norm2` (+ `.b`),
`l<i>.mlp.up|down|act`, `l<i>.side.gate|proj|norm`, `l<i>.mix.q|k|v|g|temp|o`, `l<i>.mix.left.q|k|v|g|sink|o`,
`l<i>.mix.right.r|k|v|g|a|a.b|w1|w2|w0|norm|o`, `l<i>.mix.q|dkv|dkv.norm|uk|uv|sink|o`."""
from __future__ import annotations

from ..config.bozovik import BozovikConfig, GroupedAttention, LatentAttention, ParallelPair
from ..config.plan import LayerSpec, ModelPlan, OrderEntry, PartSpec
from ..config.registry import register_architecture

MAX_POSITIONS = 1 << 20      # the design has no limit of its own; angles are formed from 32-bit positions


def _norm(cfg: BozovikConfig, tensor: str) -> PartSpec:
    return PartSpec("layer_norm", {"dim": cfg.width, "eps": cfg.norm_eps}, {"weight": tensor, "bias": tensor + ".b"})


def _rope(width: int, rot) -> PartSpec | None:
    if rot is None:
        return None
    return PartSpec("rope", {"head_dim": width, "rotary_dim": rot.dims, "theta": rot.base, "layout": "half"})


def _grouped(cfg: BozovikConfig, a: GroupedAttention, p: str, full: bool) -> tuple[PartSpec, dict]:
    params = {"hidden_size": cfg.width, "num_heads": a.heads, "num_kv_heads": a.kv_heads, "head_dim": a.dim, "value_dim": a.vdim,
              "scale": a.scale, "window": a.window, "keep_first": a.keep_first, "position": _rope(a.dim, a.rot), "head_gate": True,
              "sinks": not full, "fixed_sink": 0.0 if full else None, "head_temperature": full}
    names = {"q_proj": p + "q", "k_proj": p + "k", "v_proj": p + "v", "out_proj": p + "o", "gate": p + "g"}
    names.update({"temperature": p + "temp"} if full else {"sinks": p + "sink"})
    return PartSpec("sink_attention", params, names), names


def _mixer(cfg: BozovikConfig, layer, p: str) -> PartSpec:
    H, m = cfg.width, layer.mixer
    if isinstance(m, GroupedAttention):
        return _grouped(cfg, m, p + "mix.", full=True)[0]
    if isinstance(m, ParallelPair):
        left, left_names = _grouped(cfg, m.left, p + "mix.left.", full=False)
        r = p + "mix.right."
        right_names = {k: r + k for k in ("r", "k", "v", "g", "a", "w1", "w2", "w0", "norm", "o")}
        right_names["a_bias"] = r + "a.b"
        right = PartSpec("general_delta", {"hidden_size": H, "heads": m.right.heads, "dim": m.right.dim, "eps": cfg.norm_eps,
                                           "decay_rank": m.right.decay_rank or -1}, right_names)
        names = {"first." + k: v for k, v in left_names.items()}
        names.update({"second." + k: v for k, v in right_names.items()})
        return PartSpec("weighted_pair", {"hidden_size": H, "first": left, "second": right, "first_scale": m.left_scale,
                                          "second_scale": m.right_scale}, names)
    assert isinstance(m, LatentAttention)
    q = p + "mix."
    return PartSpec("latent_attention", {"hidden_size": H, "heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "vdim": m.vdim,
                                         "kv_rank": m.kv_rank, "scale": m.scale, "eps": cfg.norm_eps, "window": m.window, "sinks": True,
                                         "position": _rope(m.rot_dim, m.rot)},
                    {"q": q + "q", "dkv": q + "dkv", "dkv_norm": q + "dkv.norm", "uk": q + "uk", "uv": q + "uv", "o": q + "o",
                     "sinks": q + "sink"})


def run_order(cfg: BozovikConfig) -> tuple[list, dict]:
    """The layers in the order they run (a looped run of layers `times` times), and for every item of that order at
    which a pass over the loop begins, the number of the pass."""
    n, loop = len(cfg.layers), cfg.loop
    order, passes = [], {}
    i = 0
    while i < n:
        if loop is not None and i == loop.start:
            for t in range(loop.times):
                passes[len(order)] = t
                order += list(range(loop.start, loop.stop))
            i = loop.stop
        else:
            order.append(i)
            i += 1
    return order, passes


def build_plan(cfg: BozovikConfig) -> ModelPlan:
    H = cfg.width
    order, passes = run_order(cfg)
    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        ffn = ffn_norm = None
        if layer.mlp is not None:
            ffn = PartSpec("dense_mlp", {"hidden_size": H, "ff_dim": layer.mlp.ff, "activation": "xielu", "out_dtype32": True},
                           {"up": p + "mlp.up", "down": p + "mlp.down", "act": p + "mlp.act"})
            ffn_norm = _norm(cfg, p + "norm2")
        params = {"hidden_size": H, "residual_mult": cfg.residual_mult}
        weights = {}
        if cfg.token_side_dim:
            d = cfg.token_side_dim
            params["token_rows"] = {"dim": d, "offset": i * d, "eps": cfg.norm_eps, "activation": "gelu_tanh", "vocab": cfg.vocab,
                                    "table_width": d * len(cfg.layers)}
            weights.update(token_table="side.embed", token_gate=p + "side.gate", token_proj=p + "side.proj", token_norm=p + "side.norm")
        if cfg.loop is not None and i == cfg.loop.start:
            params.update(passes={item: t for item, t in passes.items()}, n_passes=cfg.loop.times, vocab=cfg.vocab,
                          embedding_scale=cfg.embedding_scale)
            weights.update(pass_steps="loop.step", embedding="embed")
        layers.append(LayerSpec(PartSpec("pre_norm_scaled", params, weights), _mixer(cfg, layer, p), ffn, _norm(cfg, p + "norm1"), ffn_norm))
    embedding = PartSpec("lookup", {"vocab_size": cfg.vocab, "dim": H, "scale": cfg.embedding_scale}, {"weight": "embed"})
    unread = [f"l{i}.norm2{s}" for i, layer in enumerate(cfg.layers) if layer.mlp is None for s in ("", ".b")]
    return ModelPlan(hidden_size=H, vocab_size=cfg.vocab, max_positions=MAX_POSITIONS, embedding=embedding,
                     final_norm=_norm(cfg, "final.norm"), head="head", layers=tuple(layers),
                     order=tuple(OrderEntry(i) for i in order), eos_token_id=cfg.eos_token_id, unread_tensors=tuple(unread))


register_architecture("Bozovik", BozovikConfig, build_plan, model_types=("bozovik",))
