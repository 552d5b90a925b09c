"""A plain, slow restatement of the Bozovik design in 64-bit torch: whole sequences, no cache, no kernels.

One function per mechanism; nothing here is shared with the product path. `cfg` is the design's config.json as a
dictionary, `w` maps tensor names to 64-bit tensors. `forward` returns the logits of every position and, if asked,
the stream after every layer that ran (a looped layer once for every pass)."""
from __future__ import annotations

import math

import torch

F64 = torch.float64

# How far rounding alone moves a row's logits differs from row to row (a recurrence's read-out that nearly cancels is
# scaled up by the norm behind it). Inside `disturbed(rel, seed)` every product and every norm is multiplied by
# 1 + rel * u, u uniform in [-1, 1) and drawn anew for every entry, which is what a 16-bit engine's roundings do; the
# difference from the exact run measures, row by row, what rounding alone causes.
_NOISE = []


class disturbed:
    def __init__(self, rel, seed):
        self.rel, self.gen = rel, torch.Generator().manual_seed(seed)

    def __enter__(self):
        _NOISE.append(self)

    def __exit__(self, *a):
        _NOISE.pop()


def _d(x):
    if not _NOISE:
        return x
    n = _NOISE[-1]
    return x * (1 + n.rel * (2 * torch.rand(x.shape, generator=n.gen, dtype=F64) - 1))


def lin(h, W):
    return _d(h @ W.T)


def gelu_tanh(z):
    return 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))


def softplus(x):
    return torch.log1p(torch.exp(-x.abs())) + x.clamp(min=0)


def rms(x, eps):
    return _d(x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps))


def layer_norm(x, weight, bias, eps):
    mu = x.mean(dim=-1, keepdim=True)
    d = x - mu
    return _d(d / torch.sqrt((d * d).mean(dim=-1, keepdim=True) + eps) * weight + bias)


def xielu(z, p, q):
    """Positive side: softplus(p) z^2 + z/2. Other side: (1/2 + softplus(q)) (exp(z) - 1 - z) + z/2."""
    ap, aq = softplus(p), 0.5 + softplus(q)
    return torch.where(z > 0, ap * z * z + 0.5 * z, aq * (torch.expm1(torch.clamp(z, max=0.0)) - z) + 0.5 * z)


def rotate_half(x, positions, base, dims):
    """x [T, heads, d]: entries i and i + dims/2 (i < dims/2) of every head turn by p * base^(-2i/dims); the rest stay."""
    if not dims:
        return x
    half = dims // 2
    i = torch.arange(half, dtype=F64)
    ang = positions.to(F64)[:, None] * base ** (-2.0 * i / dims)[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def visible(T, size=None, keep_first=0):
    """[T, T] mask: entry [i, j] is true when j <= i and (size is None, or i - j < size, or j < keep_first)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    m = j <= i
    if size is not None:
        m = m & ((i - j < size) | (j < keep_first))
    return m


def softmax_with_sink(scores, mask, sink):
    """scores [H, T, T]; sink [H]: one more term exp(sink_h) in every row's denominator, with no value."""
    s = scores.masked_fill(~mask[None], -math.inf)
    top = torch.maximum(s.max(dim=-1, keepdim=True).values, sink[:, None, None])
    e = torch.exp(s - top)
    return e / (e.sum(dim=-1, keepdim=True) + torch.exp(sink[:, None, None] - top))


def grouped_attention(h, w, p, m, positions, sink, temp=None, size=None, keep_first=0, weights_out=None):
    """Attention with fewer key/value heads than query heads, rotation of part of a head, a sink, a gate per head."""
    T = h.shape[0]
    H, d = m["heads"], m["dim"]
    G, vd = m.get("kv_heads", H), m.get("vdim", d)
    q = lin(h, w[p + "q"]).view(T, H, d)
    k = lin(h, w[p + "k"]).view(T, G, d)
    v = lin(h, w[p + "v"]).view(T, G, vd)
    rot = m.get("rot")
    if rot:
        q = rotate_half(q, positions, rot["base"], rot["dims"])
        k = rotate_half(k, positions, rot["base"], rot["dims"])
    rep = H // G
    k = k.repeat_interleave(rep, dim=1)
    v = v.repeat_interleave(rep, dim=1)
    s = torch.einsum("ihd,jhd->hij", q, k) * m["scale"]
    if temp is not None:
        s = s * temp[:, None, None]
    pr = softmax_with_sink(s, visible(T, size, keep_first), sink)
    if weights_out is not None:
        weights_out.append(pr)
    o = torch.einsum("hij,jhd->ihd", pr, v)
    o = o * torch.sigmoid(lin(h, w[p + "g"]))[:, :, None]
    return lin(o.reshape(T, H * vd), w[p + "o"])


def full_attention(h, w, p, m, positions):
    H = m["heads"]
    return grouped_attention(h, w, p, m, positions, torch.zeros(H, dtype=F64), temp=w[p + "temp"])


def windowed_sink_attention(h, w, p, m, positions, weights_out=None):
    mask = m.get("mask") or {}
    return grouped_attention(h, w, p, m, positions, w[p + "sink"], size=mask.get("size"), keep_first=mask.get("keep_first", 0),
                             weights_out=weights_out)


def delta_rule(h, w, p, m, eps):
    """S <- diag(d) S - (a * u)(u^T S) + k v^T (both read the old S); o = S^T r; per head RMS norm, weight, gate, W_o."""
    T = h.shape[0]
    H, d = m["heads"], m["dim"]
    r = lin(h, w[p + "r"]).view(T, H, d)
    k = lin(h, w[p + "k"]).view(T, H, d)
    v = lin(h, w[p + "v"]).view(T, H, d)
    decay = torch.exp(-math.exp(-0.5) * torch.sigmoid(lin(torch.tanh(lin(h, w[p + "w1"])), w[p + "w2"]) + w[p + "w0"])).view(T, H, d)
    a = torch.sigmoid(lin(h, w[p + "a"]) + w[p + "a.b"]).view(T, H, d)
    u = k / torch.sqrt((k * k).sum(dim=-1, keepdim=True) + 1e-6)
    S = torch.zeros(H, d, d, dtype=F64)
    out = []
    for t in range(T):
        uS = torch.einsum("hi,hij->hj", u[t], S)
        S = decay[t][:, :, None] * S - (a[t] * u[t])[:, :, None] * uS[:, None, :] + k[t][:, :, None] * v[t][:, None, :]
        out.append(torch.einsum("hij,hi->hj", S, r[t]))
    o = rms(torch.stack(out), eps).reshape(T, H * d) * w[p + "norm"] * torch.sigmoid(lin(h, w[p + "g"]))
    return lin(o, w[p + "o"])


def parallel_mixer(h, w, p, m, positions, eps):
    return m["left_scale"] * windowed_sink_attention(h, w, p + "left.", m["left"], positions) + \
        m["right_scale"] * delta_rule(h, w, p + "right.", m["right"], eps)


def latent_attention(h, w, p, m, positions, eps, weights_out=None):
    """Keys and values of all heads from one latent row per token; one rotated key part for all heads."""
    T = h.shape[0]
    H, d, rd, vd, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    q = lin(h, w[p + "q"]).view(T, H, d + rd)
    q_plain, q_rot = q[..., :d], q[..., d:]
    down = lin(h, w[p + "dkv"])
    c = rms(down[:, :rank], eps) * w[p + "dkv.norm"]
    k_rot = down[:, rank:].view(T, 1, rd)
    rot = m.get("rot")
    if rot:
        q_rot = rotate_half(q_rot, positions, rot["base"], rot["dims"])
        k_rot = rotate_half(k_rot, positions, rot["base"], rot["dims"])
    k_plain = lin(c, w[p + "uk"]).view(T, H, d)
    v = lin(c, w[p + "uv"]).view(T, H, vd)
    s = (torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihd,jd->hij", q_rot, k_rot[:, 0])) * m["scale"]
    mask = m.get("mask") or {}
    pr = softmax_with_sink(s, visible(T, mask.get("size")), w[p + "sink"])
    if weights_out is not None:
        weights_out.append(pr)
    o = torch.einsum("hij,jhd->ihd", pr, v).reshape(T, H * vd)
    return lin(o, w[p + "o"])


def dense_mlp(h, w, p):
    act = w[p + "act"]
    return lin(xielu(lin(h, w[p + "up"]), act[0], act[1]), w[p + "down"])


def token_side(x, tokens, w, p, layer, dim, eps):
    """The layer's own part of a second embedding row, gated by the stream: RMS-normed proj(gelu(gate x) * e)."""
    e = w["side.embed"][tokens][:, layer * dim:(layer + 1) * dim]
    y = lin(gelu_tanh(lin(x, w[p + "gate"])) * e, w[p + "proj"])
    return rms(y, eps) * w[p + "norm"]


def run_layer(x, i, cfg, w, tokens, positions):
    L, eps, mult, p = cfg["layers"][i], cfg["norm"]["eps"], cfg.get("residual_mult", 1.0), f"l{i}."
    h = layer_norm(x, w[p + "norm1"], w[p + "norm1.b"], eps)
    kind = L["type"]
    if kind == "parallel":
        y = parallel_mixer(h, w, p + "mix.", L["mixer"], positions, eps)
    elif kind == "attention":
        y = full_attention(h, w, p + "mix.", L["mixer"], positions)
    elif kind == "latent_attention":
        y = latent_attention(h, w, p + "mix.", L["mixer"], positions, eps)
    else:
        raise ValueError(kind)
    x = x + mult * y
    if L.get("mlp") is not None:
        x = x + mult * dense_mlp(layer_norm(x, w[p + "norm2"], w[p + "norm2.b"], eps), w, p + "mlp.")
    if cfg.get("token_side"):
        x = x + mult * token_side(x, tokens, w, p + "side.", i, cfg["token_side"]["dim"], eps)
    return x


def forward_until(tokens, cfg, w, n_runs):
    """The stream after the first n_runs layer runs (0: the embedding's output with the first pass' vector, if a loop
    starts there, not yet added)."""
    if n_runs == 0:
        return w["embed"][torch.as_tensor(tokens, dtype=torch.long)] * cfg.get("embedding", {}).get("scale", 1.0)
    out = []
    forward(tokens, cfg, w, out)
    return out[n_runs - 1]


def forward(tokens, cfg, w, layers_out=None):
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    T = tokens.shape[0]
    positions = torch.arange(T)
    x0 = w["embed"][tokens] * cfg.get("embedding", {}).get("scale", 1.0)
    x = x0
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    start, stop, times = (loop["start"], loop["stop"], loop["times"]) if loop else (0, 0, 0)

    def run(i, x):
        x = run_layer(x, i, cfg, w, tokens, positions)
        if layers_out is not None:
            layers_out.append(x)
        return x
    i = 0
    while i < n:
        if loop and i == start and stop > start:
            for t in range(times):
                if t > 0:
                    x = x + x0
                x = x + w["loop.step"][t]
                for k in range(start, stop):
                    x = run(k, x)
            i = stop
            continue
        x = run(i, x)
        i += 1
    eps = cfg["norm"]["eps"]
    return lin(layer_norm(x, w["final.norm"], w["final.norm.b"], eps), w["head"])
