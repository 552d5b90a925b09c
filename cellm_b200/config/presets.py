"""Shapes of the LFM2 family as config.json dictionaries, for runs with random
weights (benchmarks and workloads; no checkpoint is read). The keys are the
architecture's own; the reference hard-codes the same attention layout for
LFM2-1.2B when a header lacks `layer_types`
(crates/cellm-model/src/lfm.rs:104-114)."""
from __future__ import annotations

_COMMON = {
    "architectures": ["Lfm2ForCausalLM"], "model_type": "lfm2",
    "vocab_size": 65536, "num_key_value_heads": 8, "head_dim": 64,
    "block_auto_adjust_ff_dim": True, "block_multiple_of": 256, "block_ffn_dim_multiplier": 1.0,
    "rope_theta": 1000000.0, "conv_L_cache": 3, "conv_bias": False, "norm_eps": 1e-5,
    "tie_embedding": True, "max_position_embeddings": 128000,
}

LFM2_SHAPES = {
    # 16 layers, feed-forward 12288 -> 8192
    "lfm2-1.2b": dict(_COMMON, hidden_size=2048, num_hidden_layers=16, full_attn_idxs=[2, 5, 8, 10, 12, 14],
                      num_attention_heads=32, intermediate_size=12288),
    # 30 layers, feed-forward 10752 -> 7168
    "lfm2-2.6b": dict(_COMMON, hidden_size=2048, num_hidden_layers=30, full_attn_idxs=[2, 6, 10, 14, 18, 21, 24, 27],
                      num_attention_heads=32, intermediate_size=10752),
    # 16 layers, width 1536, feed-forward 10240 -> 6912
    "lfm2-700m": dict(_COMMON, hidden_size=1536, num_hidden_layers=16, full_attn_idxs=[2, 5, 8, 10, 12, 14],
                      num_attention_heads=24, intermediate_size=10240),
}


def shape(name: str) -> dict:
    try:
        return dict(LFM2_SHAPES[name.lower()])
    except KeyError:
        raise ValueError(f"unknown shape {name!r}; known: {sorted(LFM2_SHAPES)}") from None


# ---- Vezalorn shapes beside LFM2's ---------------------------------------------------------------------------------
def _vezalorn(width: int, layers: int, attention_at, heads: int, ff: int, vocab: int = 65536) -> dict:
    """Layers of a width and count that an LFM2 shape has: recurrent layers of the model's width where LFM2 has its
    short convolutions, latent attention (heads of 128 + 64 rotated values, a latent of 512) where it has attention,
    and the same feed-forward width after every layer."""
    attn = {"heads": heads, "dim": 128, "rot_dim": 64, "vdim": 128, "kv_rank": 512, "scale": 192 ** -0.5,
            "rot": {"base": 1000000.0, "dims": 64}}
    mlp = {"kind": "dense", "ff": ff}
    return {"architecture": "Vezalorn", "vocab": vocab, "width": width, "embedding": {"scale": 1.0},
            "norm": {"eps": 1e-5, "groups": 2},
            "layers": [{"type": "latent_attention", "mixer": dict(attn), "mlp": dict(mlp)} if i in attention_at else
                       {"type": "mingru", "mixer": {"width": width}, "mlp": dict(mlp)} for i in range(layers)]}


# name -> (Vezalorn shape, the LFM2 shape of equal width, depth, feed-forward and attention places)
VEZALORN_SHAPES = {
    "1.2b": (_vezalorn(2048, 16, [2, 5, 8, 10, 12, 14], 16, 8192), "lfm2-1.2b"),
    "700m": (_vezalorn(1536, 16, [2, 5, 8, 10, 12, 14], 12, 6912), "lfm2-700m"),
}


# ---- Tufadra shapes beside LFM2's ----------------------------------------------------------------------------------
def _tufadra(width: int, layers: int, heads: int, kv_heads: int, experts: int, top: int, ff: int, shared_ff: int, vocab: int = 65536,
             dim: int = 64, vdim: int = 64) -> dict:
    """Layers of a width and count that an LFM2 shape has, every one an attention layer (the design has no other mixer)
    with LFM2's heads beside a mixture of experts whose chosen experts and shared expert together are as wide as LFM2's
    feed-forward."""
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": dim ** -0.5, "q_temp": {"coef": 0.1, "every": 1024}}
    mlp = {"kind": "moe", "expert": {"ff": ff}, "shared": {"ff": shared_ff},
           "router": {"experts": experts, "top": top, "scale": 1.0, "groups": {"count": 8, "keep": 4}}}
    return {"architecture": "Tufadra", "vocab": vocab, "width": width, "max_positions": 16384, "norm": {"eps": 1e-5},
            "layers": [{"type": "attention", "mixer": dict(mixer), "mlp": dict(mlp)} for _ in range(layers)]}


# name -> (Tufadra shape, the LFM2 shape of equal width and depth): 64 experts of which 6 are chosen, 6 x 1,024 + 2,048 = 8,192
# active feed-forward columns at the larger size (LFM2-1.2B's feed-forward), 6 x 896 + 1,536 = 6,912 at the smaller
TUFADRA_SHAPES = {
    "1.2b": (_tufadra(2048, 16, 32, 8, 64, 6, 1024, 2048), "lfm2-1.2b"),
    "700m": (_tufadra(1536, 16, 24, 8, 64, 6, 896, 1536), "lfm2-700m"),
}


# ---- Padadra shapes beside LFM2's ----------------------------------------------------------------------------------
def _padadra(width: int, layers: int, parallel_at, heads: int, kv_heads: int, rec_heads: int, ff: int, vocab: int = 65536) -> dict:
    """Layers of a width and count that an LFM2 shape has: the two mixers side by side (LFM2's attention heads of 64 with
    a window of 1,024 and convolutions of four taps, beside an HGRN2 recurrence with states of 64 x 128 a head) where
    LFM2 has attention, the gated delta rule with states of 128 x 128 a head where it has its short convolutions, and a
    feed-forward of LFM2's width beside every mixer."""
    left = {"heads": heads, "kv_heads": kv_heads, "dim": 64, "vdim": 64, "scale": 0.125, "conv": 4, "mask": {"size": 1024},
            "rot": {"base": 1000000.0, "dims": 64, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}}
    right = {"heads": rec_heads, "dim": 64, "vdim": 128}
    delta = {"heads": rec_heads, "kv_heads": rec_heads // 2, "dim": 128, "vdim": 128, "conv": 4, "decay_rank": 64, "gate_rank": 64}
    mlp = {"kind": "dense", "ff": ff}
    return {"architecture": "Padadra", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "residual_mult": 0.5,
            "embedding": {"scale": 1.0, "bigram": {"buckets": 100003, "mul_prev": 31, "mul_cur": 7}},
            "layers": [{"type": "parallel", "mixer": {"left": dict(left), "right": dict(right)}, "mlp": dict(mlp)} if i in parallel_at else
                       {"type": "channel_delta", "mixer": dict(delta), "mlp": dict(mlp)} for i in range(layers)]}


# name -> (Padadra shape, the LFM2 shape of equal width, depth, feed-forward and attention places)
PADADRA_SHAPES = {
    "1.2b": (_padadra(2048, 16, [2, 5, 8, 10, 12, 14], 32, 8, 16, 8192), "lfm2-1.2b"),
    "700m": (_padadra(1536, 16, [2, 5, 8, 10, 12, 14], 24, 8, 12, 6912), "lfm2-700m"),
}


# ---- Bozovik shapes beside Padadra's -------------------------------------------------------------------------------
def _bozovik(width: int, layers: int, parallel_at, attention_at, heads: int, kv_heads: int, rec_heads: int, latent_heads: int, ff: int,
             vocab: int = 65536) -> dict:
    """Layers of a width and count that a Padadra shape has: the windowed attention that keeps its first keys beside the
    generalized delta rule (states of 64 x 64 a head) where Padadra has its two mixers side by side, attention over every
    earlier key at a few places, latent attention (heads of 128 + 64, a latent of 512, a window of 1,024) elsewhere, a
    feed-forward of Padadra's width behind every mixer and a side input of 64 values a layer. No layers are looped, so
    that both models do a layer's work as often."""
    left = {"heads": heads, "kv_heads": kv_heads, "dim": 64, "vdim": 64, "scale": 0.125, "mask": {"size": 1024, "keep_first": 64},
            "rot": {"base": 1000000.0, "dims": 64}}
    right = {"heads": rec_heads, "dim": 64, "decay_rank": 64}
    full = {"heads": heads, "kv_heads": kv_heads, "dim": 64, "vdim": 64, "scale": 0.125, "rot": {"base": 1000000.0, "dims": 32}}
    lat = {"heads": latent_heads, "dim": 128, "rot_dim": 64, "vdim": 128, "kv_rank": 512, "scale": 192 ** -0.5, "mask": {"size": 1024},
           "rot": {"base": 500000.0, "dims": 64}}
    mlp = {"kind": "dense", "ff": ff}

    def layer(i):
        if i in parallel_at:
            return {"type": "parallel", "mixer": {"left": dict(left), "right": dict(right), "left_scale": 0.6, "right_scale": 0.5}, "mlp": dict(mlp)}
        if i in attention_at:
            return {"type": "attention", "mixer": dict(full), "mlp": dict(mlp)}
        return {"type": "latent_attention", "mixer": dict(lat), "mlp": dict(mlp)}
    return {"architecture": "Bozovik", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "residual_mult": 0.5,
            "embedding": {"scale": 1.0}, "token_side": {"dim": 64}, "layers": [layer(i) for i in range(layers)]}


# name -> (Bozovik shape, (the closest design's name, its shape of equal width, depth and feed-forward))
BOZOVIK_SHAPES = {
    "1.2b": (_bozovik(2048, 16, [2, 5, 8, 10, 12, 14], [0, 7, 15], 32, 8, 32, 16, 8192), ("padadra", PADADRA_SHAPES["1.2b"][0])),
    "700m": (_bozovik(1536, 16, [2, 5, 8, 10, 12, 14], [0, 7, 15], 24, 8, 24, 12, 6912), ("padadra", PADADRA_SHAPES["700m"][0])),
}
