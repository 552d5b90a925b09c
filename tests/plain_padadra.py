"""A plain, slow restatement of the Padadra design in 64-bit torch: whole sequences, no cache, no kernels.

One function per mechanism; nothing here is shared with the product path. `cfg` is the design's config.json as a
dictionary, `w` maps tensor names to 64-bit tensors."""
from __future__ import annotations

import math

import torch

F64 = torch.float64

# How sensitive a model's logits are to rounding differs from row to row (a head's read-out that nearly cancels is scaled
# up by the norm behind it). `perturbed` multiplies every intermediate result by 1 + rel * u, u uniform in [-1, 1) and
# drawn anew for every entry, which is what a 16-bit engine's roundings do to them; the difference from the exact run
# measures, row by row, what rounding alone causes.
_NOISE = None


class perturbed:
    def __init__(self, rel, seed):
        self.rel, self.gen = rel, torch.Generator().manual_seed(seed)

    def __enter__(self):
        global _NOISE
        _NOISE = self

    def __exit__(self, *a):
        global _NOISE
        _NOISE = None


def _p(x):
    if _NOISE is None:
        return x
    return x * (1 + _NOISE.rel * (2 * torch.rand(x.shape, generator=_NOISE.gen, dtype=F64) - 1))


def lin(h, W, b=None):
    y = h @ W.T
    return _p(y if b is None else y + b)


def rms(x, eps):
    return _p(x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps))


def gelu_tanh(z):
    return 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))


def bigram_rows(tokens, emb_cfg):
    """Row of the bigram table for every token: the last row for a sequence's first token."""
    b = emb_cfg["bigram"]
    rows = []
    for t, tok in enumerate(tokens):
        rows.append(b["buckets"] if t == 0 else (tokens[t - 1] * b["mul_prev"] + tok * b["mul_cur"]) % b["buckets"])
    return rows


def embedding(tokens, cfg, w):
    x = w["embed"][torch.tensor(tokens)] * cfg["embedding"]["scale"]
    if cfg["embedding"].get("bigram"):
        x = x + w["bigram"][torch.tensor(bigram_rows(tokens, cfg["embedding"]))]
    return x


def scalar_norm(x, g, eps):
    return rms(x, eps) * g


def causal_conv(u, taps_w):
    """u [T, C], taps_w [C, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros before the start."""
    T, C = u.shape
    taps = taps_w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=u.dtype), u], dim=0)
    y = torch.zeros_like(u)
    for j in range(taps):
        y = y + padded[j:j + T] * taps_w[:, j]
    return _p(y)


def scaled_frequencies(base, dims, scaling):
    """f_i = base^(-2i/dims), then the wavelength-dependent scaling."""
    out = []
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        if scaling is not None:
            factor, low, high, orig = scaling["factor"], scaling["low"], scaling["high"], scaling["original"]
            wl = 2 * math.pi / f
            if wl < orig / high:
                pass
            elif wl > orig / low:
                f = f / factor
            else:
                s = (orig / wl - low) / (high - low)
                f = (1 - s) * f / factor + s * f
        out.append(f)
    return torch.tensor(out, dtype=F64)


def rotate_interleaved(x, positions, freqs, sign=1.0):
    """x [T, heads, d]: pairs (2i, 2i+1) of the first 2*len(freqs) entries turn by sign * p * f_i."""
    n = freqs.shape[0]
    ang = sign * positions.to(F64)[:, None] * freqs[None, :]          # [T, n]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    out = x.clone()
    u, v = x[..., 0:2 * n:2], x[..., 1:2 * n:2]
    out[..., 0:2 * n:2] = u * c - v * s
    out[..., 1:2 * n:2] = v * c + u * s
    return _p(out)


def sink_window_attention(q, k, v, scale, window, sinks, weights_out=None):
    """q [T, H, d], k [T, G, d], v [T, G, dv]; position i sees j with 0 <= i - j < window (None: every j <= i); the
    softmax's denominator also holds exp(sink_h). `weights_out`, a list, receives every head's weights [T, T]."""
    T, H, d = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        i = torch.arange(T)[:, None]
        j = torch.arange(T)[None, :]
        ok = (i - j >= 0) & ((i - j < window) if window else (i >= j))
        s = s.masked_fill(~ok, -math.inf)
        m = torch.maximum(s.max(dim=1, keepdim=True).values, sinks[h].reshape(1, 1))
        e = torch.exp(s - m)
        den = e.sum(dim=1, keepdim=True) + torch.exp(sinks[h] - m)
        out[:, h] = (e / den) @ v[:, g]
        if weights_out is not None:
            weights_out.append(e / den)
    return _p(out)


def left_mixer(h, m, w, p, eps, weights_out=None):
    """The windowed attention with sinks, short convolutions, a norm over the projection, rotated keys and values."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q, k, v = lin(h, w[p + "q"], w[p + "q.b"]), lin(h, w[p + "k"], w[p + "k.b"]), lin(h, w[p + "v"], w[p + "v.b"])
    if m.get("conv"):
        q, k, v = causal_conv(q, w[p + "q.conv"]), causal_conv(k, w[p + "k.conv"]), causal_conv(v, w[p + "v.conv"])
    q = rms(q, eps) * w[p + "q.norm"]
    k = rms(k, eps) * w[p + "k.norm"]
    q, k, v = q.reshape(T, H, d), k.reshape(T, G, d), v.reshape(T, G, dv)
    rot = m.get("rot")
    if rot is not None:
        fr = scaled_frequencies(rot["base"], rot["dims"], rot.get("scaling"))
        q, k = rotate_interleaved(q, pos, fr), rotate_interleaved(k, pos, fr)
        fv = scaled_frequencies(rot["base"], dv, None)
        v = rotate_interleaved(v, pos, fv)
    o = sink_window_attention(q, k, v, m["scale"], (m.get("mask") or {}).get("size"), w[p + "sink"], weights_out)
    if rot is not None:
        o = rotate_interleaved(o, pos, fv, sign=-1.0)
    return lin(o.reshape(T, H * dv), w[p + "o"])


def hgrn2(h, m, w, p, eps):
    """Linear attention whose forget gate also decides what is written."""
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = torch.nn.functional.silu(lin(h, w[p + "q"])).reshape(T, H, d)
    v = lin(h, w[p + "v"]).reshape(T, H, dv)
    low = w[p + "lower"]
    f = (low + (1 - low) * torch.sigmoid(lin(h, w[p + "f"]) + w[p + "f.b"])).reshape(T, H, d)
    S = torch.zeros(H, d, dv, dtype=h.dtype)
    o = torch.zeros(T, H, dv, dtype=h.dtype)
    for t in range(T):
        S = f[t][:, :, None] * S + (1 - f[t])[:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = rms(_p(o), eps) * w[p + "norm"]
    return lin(o.reshape(T, H * dv), w[p + "o"])


def parallel_mixer(h, m, w, p, eps):
    a = left_mixer(h, m["left"], w, p + "left.", eps)
    b = hgrn2(h, m["right"], w, p + "right.", eps)
    return _p(0.5 * (rms(a, eps) * w[p + "left.out"] + rms(b, eps) * w[p + "right.out"]))


def channel_delta(h, m, w, p, eps):
    """Gated delta rule with one decay per head and key channel."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    silu = torch.nn.functional.silu
    q = silu(causal_conv(lin(h, w[p + "q"]), w[p + "q.conv"])).reshape(T, G, d)
    k = silu(causal_conv(lin(h, w[p + "k"]), w[p + "k.conv"])).reshape(T, G, d)
    v = silu(causal_conv(lin(h, w[p + "v"]), w[p + "v.conv"])).reshape(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(lin(h, w[p + "b"]))                                      # [T, H]
    a = lin(lin(h, w[p + "a1"]), w[p + "a2"]) + w[p + "dt_bias"]
    g = torch.exp(-torch.exp(w[p + "A_log"])[None, :, None] * torch.nn.functional.softplus(a).reshape(T, H, d))
    gate = torch.sigmoid(lin(lin(h, w[p + "g1"]), w[p + "g2"])).reshape(T, H, dv)
    S = torch.zeros(H, d, dv, dtype=h.dtype)
    o = torch.zeros(T, H, dv, dtype=h.dtype)
    rep = H // G
    for t in range(T):
        qt, kt = q[t].repeat_interleave(rep, dim=0), k[t].repeat_interleave(rep, dim=0)   # [H, d]
        S = g[t][:, :, None] * S
        u = beta[t][:, None] * (v[t] - torch.einsum("hdv,hd->hv", S, kt))
        S = S + kt[:, :, None] * u[:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, qt)
    o = _p(rms(_p(o), eps) * w[p + "norm"] * gate)
    return lin(o.reshape(T, H * dv), w[p + "o"])


def dense_mlp(h, w, p):
    return lin(_p(torch.relu(lin(h, w[p + "up"])) ** 2), w[p + "down"])


MIXERS = {"parallel": parallel_mixer, "channel_delta": channel_delta}


def forward(tokens, cfg, w, return_layers=False):
    """Logits [T, vocab] of one whole sequence (and the stream after every layer)."""
    eps = cfg["norm"]["eps"]
    mult = cfg["residual_mult"]
    x = embedding(list(tokens), cfg, w)
    layers = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        y = MIXERS[layer["type"]](scalar_norm(x, w[p + "norm1"], eps), layer["mixer"], w, p + "mix.", eps)
        if layer.get("mlp") is not None:
            y = y + dense_mlp(scalar_norm(x, w[p + "norm2"], eps), w, p + "mlp.")
        x = x + mult * y
        layers.append(x)
    logits = lin(scalar_norm(x, w["final.norm"], eps), w["head"])
    return (logits, torch.stack(layers)) if return_layers else logits
