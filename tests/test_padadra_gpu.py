"""The Padadra design against its plain restatement (tests/plain_padadra.py): the kernels of each mechanism alone, whole
models in every cutting of the requests, pages and slots that are used again, keys at the edges of a window and far
away, the sink, the first tokens of a sequence, long decoding through windows and pages, sizes that differ in
everything, and greedy generation through the engine and its command line."""
import json
import math
import os
import re
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_padadra as plain
import traces
from tolerances import K, K_SELF, check_close

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def left(heads, kv_heads, dim, vdim, scale=None, conv=0, window=0, rot=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5}
    if conv:
        m["conv"] = conv
    if window:
        m["mask"] = {"size": window}
    if rot is not None:
        base, dims, scaling = rot
        m["rot"] = {"base": base, "dims": dims}
        if scaling is not None:
            m["rot"]["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return m


def right(heads, dim, vdim):
    return {"heads": heads, "dim": dim, "vdim": vdim}


def par(l, r, ff=None):
    return {"type": "parallel", "mixer": {"left": l, "right": r}, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def delta(heads, kv_heads, dim, vdim, conv, ranks=(6, 5), ff=None):
    return {"type": "channel_delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv,
                                               "decay_rank": ranks[0], "gate_rank": ranks[1]},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def model_config(vocab, width, layers, eps=1e-5, mult=1.0, scale=1.0, bigram=(97, 31, 5)):
    return {"architecture": "Padadra", "vocab": vocab, "width": width, "norm": {"eps": eps}, "residual_mult": mult,
            "embedding": {"scale": scale, "bigram": {"buckets": bigram[0], "mul_prev": bigram[1], "mul_cur": bigram[2]}}, "layers": layers}


# A: key and value widths differ both ways, windows shorter and longer than a page, a layer without a feed-forward, stretched
# and plain frequencies, all and some of a head's entries rotated, groups of query heads and of value heads
CONFIG_A = model_config(300, 96, [
    par(left(4, 2, 16, 24, conv=2, window=40, rot=(10000.0, 8, (4.0, 1.0, 4.0, 64))), right(3, 8, 16), ff=144),
    delta(4, 2, 16, 8, 3),
    par(left(2, 2, 32, 12, conv=4, window=7, rot=(500.0, 32, None)), right(1, 32, 32), ff=64),
    delta(2, 2, 8, 24, 2, ranks=(3, 9), ff=80),
], mult=0.7, scale=2.0)
# B: sizes that are multiples of nothing, a convolution of one tap, a window longer than every sequence, one query/key head
# for three value heads, a factor of one into the stream and an embedding scale of one
CONFIG_B = model_config(211, 54, [
    par(left(3, 3, 10, 14, conv=1, window=1000, rot=(77.0, 4, (2.0, 0.5, 3.0, 16))), right(2, 5, 6), ff=33),
    delta(3, 1, 6, 10, 2, ranks=(2, 7), ff=21),
    par(left(2, 1, 6, 6, scale=0.9), right(3, 3, 2)),
], eps=1e-6, bigram=(13, 1, 1))
# C: heads of 64 and 32 with values as wide (bfloat16 runs the tensor-core attention), no window in one layer, no
# convolution in another, recurrences whose columns live in registers
CONFIG_C = model_config(512, 128, [
    par(left(4, 2, 64, 64, conv=3, window=50, rot=(20000.0, 16, (8.0, 1.0, 4.0, 32))), right(2, 16, 64), ff=192),
    delta(2, 2, 64, 64, 4, ranks=(8, 8), ff=128),
    par(left(8, 1, 32, 32, window=130, rot=(10000.0, 32, None)), right(4, 32, 32), ff=128),
    par(left(2, 2, 64, 64, conv=2, rot=(3000.0, 64, (2.0, 1.0, 2.0, 100))), right(1, 64, 128)),
    delta(4, 1, 32, 16, 2, ranks=(4, 4)),
], mult=0.5, scale=0.5, bigram=(1021, 1, 1))
# D: heads of 128, recurrences whose rows number 128 (registers) and 48 (shared memory), value columns that are no
# multiple of 32, a window of one token
CONFIG_D = model_config(157, 100, [
    par(left(2, 1, 128, 128, conv=2, window=64, rot=(10000.0, 64, None)), right(1, 128, 40), ff=100),
    delta(2, 1, 48, 33, 3, ranks=(5, 5), ff=60),
    par(left(2, 2, 20, 10, conv=3, window=1, rot=(100.0, 20, None)), right(2, 48, 20)),
], mult=1.3, scale=3.0)
CONFIGS = {"a": CONFIG_A, "b": CONFIG_B, "c": CONFIG_C, "d": CONFIG_D}
LENGTHS = {"a": [1, 9, 40, 64, 131, 77, 2], "b": [3, 55, 150, 18, 97], "c": [200, 1, 65, 129, 30, 260], "d": [70, 2, 33, 140, 17]}
PAGE = {"a": 8, "b": 16, "c": 16, "d": 4}


def write_model(folder, config, seed, dtype="bfloat16", init=None):
    from cellm_b200.weights import InitSpec, write_random_model
    init = init or InitSpec(linear_std=0.1, embedding_std=0.08, bias_std=0.1, norm_jitter=0.2)
    return write_random_model(str(folder), config, seed, dtype, init)


def load_plain(folder):
    from cellm_b200.weights.safetensors_io import SafetensorsFile
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    sf = SafetensorsFile(os.path.join(folder, "model.safetensors"))
    return cfg, {n: sf.tensor(n).to(torch.float64) for n in sf.names()}


def run_trace(folder, dtype, steps, page, use_graphs=True, max_tokens=None):
    from cellm_b200.replay import Replayer
    rp = Replayer(folder, dtype, max_tokens or traces.max_live_tokens(steps), page, 4, use_graphs=use_graphs)
    outs = [rp.step(s["entries"], s["end"]) for s in steps]
    assert rp.cache.live == 0
    assert all(rp.cache.free_pages(g) == rp.cache.group_pages[g] for g in range(len(rp.cache.group_pages)))
    return traces.collect(steps, outs)


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """name -> (folder, requests, plain logits)."""
    d = tmp_path_factory.mktemp("pd")
    out = {}
    for i, (name, config) in enumerate(CONFIGS.items()):
        rng = np.random.default_rng(23 + i)
        reqs = {f"r{j}": rng.integers(0, config["vocab"], n).tolist() for j, n in enumerate(LENGTHS[name])}
        folder = write_model(d / name, config, 41 + i)
        cfg, w = load_plain(folder)
        ref = {rid: Ref(toks, cfg, w) for rid, toks in reqs.items()}
        out[name] = (folder, reqs, ref)
    return out


# Against the plain restatement in 64-bit. The recurrent states carry their 32-bit rounding from token to token, every
# head's read-out is divided by its root mean square, and unit vectors of a handful of entries are formed: a rounding
# is passed on and scaled where an attention would average it away, so the 32-bit bound is 1e-5 of the logits' size
# (a few dozen units of rounding more than a sum of products needs); bfloat16 keeps the engine's bound.
KP = {"float32": 1e-5, "bfloat16": K["bfloat16"]}


class Ref(np.ndarray):
    """A request's plain logits [T, vocab] and, as `.spread` [T], how far three runs whose every intermediate result
    was disturbed by a 16-bit rounding's worth (1 + 2^-9 u, u uniform in [-1, 1)) moved each row."""
    def __new__(cls, toks, cfg, w):
        exact = plain.forward(toks, cfg, w)
        self = np.asarray(exact.numpy()).view(cls)
        spread = torch.zeros(len(toks), dtype=torch.float64)
        for seed in range(3):
            with plain.perturbed(2.0 ** -9, seed):
                spread = torch.maximum(spread, (plain.forward(toks, cfg, w) - exact).abs().amax(dim=1))
        self.spread = spread.numpy()
        return self


def against_plain(got, ref, dtype, what):
    """32-bit: one bound for all rows. bfloat16: a row whose logits rounding alone moves further than the engine's bound
    (a read-out of a recurrence that nearly cancels, scaled up by the norm behind it; common in models of a few
    channels) is held to four times that movement instead."""
    if dtype == "float32":
        return check_close(got, ref, dtype, what, k=KP[dtype])
    got, exact = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    assert got.shape == exact.shape and np.isfinite(got).all(), what
    tol = np.maximum(KP[dtype] * (1.0 + np.abs(exact).max()), 4.0 * ref.spread)
    err = np.abs(got - exact).max(axis=1)
    bad = np.nonzero(err > tol)[0]
    assert bad.size == 0, f"{what}: row {bad[0]} is off by {err[bad[0]]:.3e} > {tol[bad[0]]:.3e} ({bad.size} rows of {len(err)})"
FAMILIES = {"whole": traces.whole, "tail": traces.tail_one_by_one, "portions": traces.portions, "mixed": traces.mixed}


# ---------------------------------------------------------------------------------------------- whole models
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_every_cutting_matches_plain(models, name, dtype):
    folder, reqs, ref = models[name]
    results = {}
    for fam, make in FAMILIES.items():
        got = results[fam] = run_trace(folder, dtype, make(reqs), PAGE[name])
        for rid, toks in reqs.items():
            against_plain(traces.as_matrix(got[rid], len(toks)), ref[rid], dtype, f"{name} {dtype} {fam} {rid}")
    for fam in ("tail", "portions", "mixed"):
        for rid, toks in reqs.items():
            check_close(traces.as_matrix(results[fam][rid], len(toks)), traces.as_matrix(results["whole"][rid], len(toks)),
                        dtype, f"{name} {dtype} {fam} vs whole {rid}", k=K_SELF[dtype])
    got = run_trace(folder, dtype, traces.mixed(reqs), PAGE[name], use_graphs=False)
    for rid, toks in reqs.items():
        check_close(traces.as_matrix(got[rid], len(toks)), traces.as_matrix(results["mixed"][rid], len(toks)), dtype,
                    f"{name} {dtype} mixed: kernel by kernel vs graphs {rid}", k=K_SELF[dtype])


def test_mixed_trace_reuses_pages_and_slots(models):
    folder, reqs, _ = models["a"]
    steps = traces.mixed(reqs)
    assert len(reqs) > 4                                     # more requests than state slots
    assert traces.max_live_tokens(steps) < sum(-(-len(t) // 64) * 64 for t in reqs.values())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["b", "c"])
def test_portions_of_two_and_odd_sizes(models, name, dtype):
    folder, reqs, ref = models[name]
    for sizes in ((2,), (3, 2, 5), (17, 2, 2, 31), (1, 1, 2)):
        got = run_trace(folder, dtype, traces.portions(reqs, sizes), PAGE[name])
        for rid, toks in reqs.items():
            against_plain(traces.as_matrix(got[rid], len(toks)), ref[rid], dtype, f"{name} {dtype} portions {sizes} {rid}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "c"])
def test_long_decoding_through_windows_and_pages(models, name, dtype):
    """Most of the sequence decoded token by token: the windows (7 and 40, 50 and 130 keys) pass wholly over decoded tokens,
    pages are given back while the request lives, and the recurrent states walk a hundred and more single steps."""
    folder, reqs, ref = models[name]
    some = {rid: reqs[rid] for rid in (("r4", "r5") if name == "a" else ("r0", "r5"))}
    got = run_trace(folder, dtype, traces.tail_one_by_one(some, tail=190), 8)
    for rid, toks in some.items():
        against_plain(traces.as_matrix(got[rid], len(toks)), ref[rid], dtype, f"{name} {dtype} long tail {rid}")


def test_a_windowed_request_holds_its_window_only(models):
    """A request longer than the pool of its windowed layers runs through: pages behind the window go back at once."""
    from cellm_b200.replay import Replayer
    folder, reqs, ref = models["a"]
    toks = reqs["r4"]                                        # 131 tokens; windows of 40 and 7
    rp = Replayer(folder, "float32", 64, 8, 4)               # 8 pages of 8 tokens a group
    rows = []
    for i in range(0, len(toks), 5):
        part = toks[i:i + 5]
        rows.append(rp.step([{"id": "x", "tokens": part, "want": list(range(len(part)))}], []))
    check_close(np.concatenate(rows), ref["r4"], "float32", "a request longer than its pools", k=KP["float32"])
    rp.step([], ["x"])
    assert rp.cache.live == 0


# ------------------------------------------------------------------------- window edges, far keys, the sink
def sharp_config(scale, window):
    # one layer of attention beside a small recurrence, then one with every earlier key in sight
    return model_config(128, 64, [
        par(left(4, 2, 16, 16, scale=scale, conv=2, window=window, rot=(10000.0, 8, (4.0, 1.0, 4.0, 32))), right(1, 4, 8)),
        par(left(2, 1, 32, 16, scale=scale * 0.7, rot=(1000.0, 16, None)), right(1, 4, 8)),
    ], mult=1.0, scale=1.0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sharp_attention_at_the_window_edges_and_far_back(tmp_path, dtype):
    """A softmax so peaked (a large score scale; q and k leave their norm with a root mean square of one) that a row's
    output is a few single keys wherever they lie: a key lost at a page border or at the window's far edge, one seen
    beyond it, or a forgotten sink changes the logits outright."""
    from cellm_b200.weights import InitSpec
    window = 37
    scale = 1.5 if dtype == "float32" else 0.6
    folder = write_model(tmp_path / "sharp", sharp_config(scale, window), 9,
                         init=InitSpec(linear_std=0.25, embedding_std=0.1, bias_std=0.05, norm_jitter=0.1, conv_tap_wide_std=0.5))
    cfg, w = load_plain(folder)
    rng = np.random.default_rng(4)
    toks = rng.integers(0, cfg["vocab"], 600).tolist()
    reqs = {"long": toks, "short": toks[:45]}
    ref = {rid: Ref(t, cfg, w) for rid, t in reqs.items()}
    # the first layer's attention really is peaked, and its heaviest key often is the window's last or the row itself
    eps = cfg["norm"]["eps"]
    x0 = plain.embedding(toks, cfg, w)
    weights = []
    plain.left_mixer(plain.scalar_norm(x0, w["l0.norm1"], eps), cfg["layers"][0]["mixer"]["left"], w, "l0.mix.left.", eps, weights)
    W = torch.stack(weights)                                  # [heads, T, T]
    top, where = W[:, 100:].max(-1)
    assert float(top.median()) > (0.3 if dtype == "float32" else 0.12)
    dist = torch.arange(100, 600)[None] - where
    assert int((dist == window - 1).sum()) >= 5 and int(dist.max()) == window - 1
    assert float(W.sum(-1).min()) < 0.9                       # the sink takes a share somewhere
    # the second layer reaches keys hundreds back
    x1 = x0 + plain.parallel_mixer(plain.scalar_norm(x0, w["l0.norm1"], eps), cfg["layers"][0]["mixer"], w, "l0.mix.", eps)
    weights = []
    plain.left_mixer(plain.scalar_norm(x1, w["l1.norm1"], eps), cfg["layers"][1]["mixer"]["left"], w, "l1.mix.left.", eps, weights)
    top, where = torch.stack(weights)[:, 500:].max(-1)
    assert float((torch.arange(500, 600)[None] - where).float().median()) > 60
    for fam in ("whole", "tail", "portions", "mixed"):
        for page in (8, 32):
            got = run_trace(folder, dtype, FAMILIES[fam](reqs), page)
            for rid, t in reqs.items():
                against_plain(traces.as_matrix(got[rid], len(t)), ref[rid], dtype, f"sharp {dtype} {fam} page {page} {rid}")


@pytest.mark.parametrize("heads", [16, 32])
def test_many_channels_a_token(tmp_path, heads):
    """Projections of 2,560 and 4,608 channels: steps of few tokens spread a token's channels over more threads (and the
    delta rule's over several blocks) than prompt portions do."""
    config = model_config(96, 64, [par(left(heads, 2, 128, 128, conv=3, window=20, rot=(10000.0, 64, (2.0, 1.0, 4.0, 16))), right(1, 8, 8)),
                                   delta(heads, 2, 64, 64, 3, ranks=(4, 4))])
    folder = write_model(tmp_path / "m", config, 12, init=InitSpec_small())
    cfg, w = load_plain(folder)
    rng = np.random.default_rng(2)
    reqs = {"x": rng.integers(0, 96, 530).tolist(), "y": rng.integers(0, 96, 9).tolist()}
    ref = {rid: Ref(t, cfg, w) for rid, t in reqs.items()}
    for dtype in ("float32", "bfloat16"):
        for fam in ("whole", "tail", "mixed"):
            got = run_trace(folder, dtype, FAMILIES[fam](reqs), 16)
            for rid, t in reqs.items():
                against_plain(traces.as_matrix(got[rid], len(t)), ref[rid], dtype, f"wide {heads} {dtype} {fam} {rid}")


def InitSpec_small():
    from cellm_b200.weights import InitSpec
    return InitSpec(linear_std=0.05, embedding_std=0.08, bias_std=0.1, norm_jitter=0.2)


# ------------------------------------------------------------------------------------------ generation
def check_greedy_tokens(cfg, w, prompt, out, dtype):
    seq = list(prompt) + list(out[:-1])
    ref = plain.forward(seq, cfg, w)[len(prompt) - 1:].numpy()
    tol = 2 * KP[dtype] * (1 + np.abs(ref).max())
    for j, t in enumerate(out):
        best = int(ref[j].argmax())
        assert t == best or ref[j][best] - ref[j][t] <= tol, f"token {j}: {t} where the plain model has {best}"


@pytest.mark.parametrize("name,dtype", [("a", "float32"), ("d", "float32"), ("c", "bfloat16")])
def test_greedy_generation_through_the_engine(models, name, dtype):
    from cellm_b200 import Engine, SamplingParams
    folder, reqs, _ = models[name]
    cfg, w = load_plain(folder)
    prompts = [t for t in reqs.values() if len(t) < 140][:5]
    eng = Engine(folder, dtype=dtype, tokens_per_block=8, total_blocks=96, max_num_seqs=3, max_batch_tokens=48, prefill_chunk=24)
    outs = eng.generate(prompts, SamplingParams.greedy(14, stop_eos=False))
    for prompt, out in zip(prompts, outs):
        assert len(out) == 14
        check_greedy_tokens(cfg, w, prompt, out, dtype)
    again = eng.generate(prompts[:2], SamplingParams.greedy(14, stop_eos=False))      # slots and pages used again
    for prompt, out in zip(prompts[:2], again):
        check_greedy_tokens(cfg, w, prompt, out, dtype)
    s = eng.stats()
    assert s["idle"] and s["free_pages"] == s["total_pages"] and s["free_slots"] == 3


def test_the_command_lines_run_the_design(models, tmp_path):
    folder, reqs, ref = models["b"]
    env = {**os.environ, "PYTHONPATH": ROOT}
    prompt = reqs["r3"]
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "infer"), "--model", folder, "--tokens", ",".join(map(str, prompt)),
                        "--gen", "6", "--temperature", "0", "--dtype", "float32", "--stop-eos", "false"], capture_output=True, text=True,
                       env=env, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    cfg, w = load_plain(folder)
    out = [int(t) for t in re.search(r"^tokens: ([\d,]+)$", p.stdout, re.M).group(1).split(",")]
    assert len(out) == 6
    check_greedy_tokens(cfg, w, prompt, out, "float32")
    steps = traces.portions({"r3": prompt}, (7, 2, 4))
    q = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", "float32", "--out",
                        str(tmp_path / "o"), "--max-tokens", "64"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                       capture_output=True, text=True, env=env, timeout=600)
    assert q.returncode == 0, q.stderr[-2000:]
    assert [l for l in q.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(len(steps))]
    rows = np.concatenate([np.fromfile(tmp_path / "o" / f"{i}.f32", dtype="<f4").reshape(-1, cfg["vocab"]) for i in range(len(steps))])
    check_close(rows, ref["r3"], "float32", "trace_run", k=KP["float32"])


# ------------------------------------------------------------------------------------- the mechanisms by themselves
def step_ctx(q_lens, ctx_lens, slots, tokens=None):
    """A step's index arrays for requests that bring q_lens[b] tokens after ctx_lens[b] earlier ones."""
    from cellm_b200.ops._state import error_word
    from cellm_b200.parts.base import StepContext
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    T, B = sum(q_lens), len(q_lens)
    pos = [c + i for c, n in zip(ctx_lens, q_lens) for i in range(n)]
    seq = [b for b, n in enumerate(q_lens) for _ in range(n)]
    cu = [0] + list(np.cumsum(q_lens))
    return StepContext(T=T, B=B, dtype=torch.float32, device=torch.device(DEV), token_ids=i32(tokens if tokens is not None else [0] * T),
                       positions=i32(pos), seq_of_token=i32(seq), cu_seqlens=i32(cu), ctx_lens=i32(ctx_lens), slot_ids=i32(slots),
                       err=error_word(torch.device(DEV)), q_lens=list(q_lens), ctx_lens_host=list(ctx_lens), max_q_len=max(q_lens),
                       max_total_len=max(c + n for c, n in zip(ctx_lens, q_lens)))


def cuts_of(T, sizes):
    out, i, k = [], 0, 0
    while i < T:
        n = min(sizes[k % len(sizes)], T - i)
        out.append((i, n))
        i, k = i + n, k + 1
    return out


@pytest.mark.parametrize("heads,dim,vd", [(2, 16, 24), (1, 32, 32), (3, 5, 6), (1, 128, 40), (2, 48, 70), (1, 64, 128), (2, 17, 3), (1, 160, 20)])
def test_hgrn2_recurrence_alone(heads, dim, vd):
    """Two sequences side by side in slots 3 and 1, fed whole and in portions down to one token: the walk against the
    plain recurrence in 64-bit, and the cuttings against each other bit for bit."""
    from cellm_b200 import ops
    g = torch.Generator().manual_seed(heads * 1000 + dim)
    lens, slots = [37, 23], [3, 1]
    C = 2 * heads * dim + heads * vd
    proj = [torch.randn(n, C, generator=g) * 1.5 for n in lens]
    fb, lower = torch.randn(heads * dim, generator=g), torch.rand(heads * dim, generator=g) * 0.9
    want = []
    for p in proj:
        p = p.double()
        q = torch.nn.functional.silu(p[:, :heads * dim]).reshape(-1, heads, dim)
        f = (lower.double() + (1 - lower.double()) * torch.sigmoid(p[:, heads * dim:2 * heads * dim] + fb.double())).reshape(-1, heads, dim)
        v = p[:, 2 * heads * dim:].reshape(-1, heads, vd)
        S = torch.zeros(heads, dim, vd, dtype=torch.float64)
        o = []
        for t in range(p.shape[0]):
            S = f[t][:, :, None] * S + (1 - f[t])[:, :, None] * v[t][:, None, :]
            o.append(torch.einsum("hdv,hd->hv", S, q[t]).reshape(-1))
        want.append(torch.stack(o))
    outs = {}
    for name, sizes in (("whole", (64,)), ("portions", (5, 1, 2, 11)), ("single", (1,))):
        state = torch.full((4, heads, dim, vd), 7.0, device=DEV)
        state[slots] = 0
        got = [[] for _ in lens]
        cuts = [cuts_of(n, sizes) for n in lens]
        for step in range(max(len(c) for c in cuts)):
            live = [b for b in range(len(lens)) if step < len(cuts[b])]
            rows = torch.cat([proj[b][cuts[b][step][0]:cuts[b][step][0] + cuts[b][step][1]] for b in live]).to(DEV).contiguous()
            ctx = step_ctx([cuts[b][step][1] for b in live], [cuts[b][step][0] for b in live], [slots[b] for b in live])
            o = ops.hgrn2_scan(rows, 0, heads * dim, 2 * heads * dim, fb.to(DEV), lower.to(DEV), state, ctx, heads, dim, vd).cpu()
            at = 0
            for b in live:
                got[b].append(o[at:at + cuts[b][step][1]])
                at += cuts[b][step][1]
        outs[name] = [torch.cat(g_) for g_ in got]
        assert float(state[0].min()) == 7.0 and float(state[2].max()) == 7.0       # other requests' slots are untouched
        for b in range(len(lens)):
            torch.testing.assert_close(outs[name][b].double(), want[b], rtol=2e-5, atol=2e-5 * float(want[b].abs().max()))
    for b in range(len(lens)):
        assert torch.equal(outs["whole"][b], outs["portions"][b]) and torch.equal(outs["whole"][b], outs["single"][b])


@pytest.mark.parametrize("heads,kvh,dim,vd", [(4, 2, 16, 8), (2, 2, 64, 64), (3, 1, 6, 10), (2, 1, 48, 33), (1, 1, 128, 32), (2, 1, 33, 5), (1, 1, 136, 12)])
def test_delta_rule_alone(heads, kvh, dim, vd):
    """The walk of the gated delta rule given its inputs (unit q and k, values, beta, decays), against 64-bit."""
    from cellm_b200 import ops
    g = torch.Generator().manual_seed(heads * 100 + dim)
    lens, slots = [41, 19], [0, 2]
    mk = lambda n: dict(qk=torch.nn.functional.normalize(torch.randn(n, 2 * kvh, dim, generator=g), dim=-1).reshape(n, -1),
                        v=torch.randn(n, heads * vd, generator=g), beta=torch.rand(n, heads, generator=g),
                        decay=0.3 + 0.7 * torch.rand(n, heads * dim, generator=g))
    data = [mk(n) for n in lens]
    want = []
    for d in data:
        n = d["v"].shape[0]
        qk = d["qk"].double().reshape(n, 2, kvh, dim)
        S = torch.zeros(heads, dim, vd, dtype=torch.float64)
        o = []
        for t in range(n):
            q = qk[t, 0].repeat_interleave(heads // kvh, dim=0)
            k = qk[t, 1].repeat_interleave(heads // kvh, dim=0)
            S = d["decay"][t].double().reshape(heads, dim)[:, :, None] * S
            u = d["beta"][t].double()[:, None] * (d["v"][t].double().reshape(heads, vd) - torch.einsum("hdv,hd->hv", S, k))
            S = S + k[:, :, None] * u[:, None, :]
            o.append(torch.einsum("hdv,hd->hv", S, q).reshape(-1))
        want.append(torch.stack(o))
    outs = {}
    for name, sizes in (("whole", (64,)), ("portions", (3, 1, 2, 9))):
        state = torch.zeros((3, heads, dim, vd), device=DEV)
        got = [[] for _ in lens]
        cuts = [cuts_of(n, sizes) for n in lens]
        for step in range(max(len(c) for c in cuts)):
            live = [b for b in range(len(lens)) if step < len(cuts[b])]
            part = lambda key: torch.cat([data[b][key][cuts[b][step][0]:cuts[b][step][0] + cuts[b][step][1]] for b in live]).to(DEV).contiguous()
            ctx = step_ctx([cuts[b][step][1] for b in live], [cuts[b][step][0] for b in live], [slots[b] for b in live])
            o = ops.delta_scan(part("qk"), part("v"), part("beta"), part("decay"), state, ctx, heads, kvh, dim, vd).cpu()
            at = 0
            for b in live:
                got[b].append(o[at:at + cuts[b][step][1]])
                at += cuts[b][step][1]
        outs[name] = [torch.cat(g_) for g_ in got]
        for b in range(len(lens)):
            torch.testing.assert_close(outs[name][b].double(), want[b], rtol=2e-5, atol=2e-5 * float(want[b].abs().max()))
    for b in range(len(lens)):
        assert torch.equal(outs["whole"][b], outs["portions"][b])


def test_delta_rule_inputs_and_the_convolutions_state():
    """Convolution + silu, unit vectors, beta and decays from the projections, with the convolution's last inputs carried
    from portion to portion (a portion shorter than the taps included)."""
    from cellm_b200 import ops
    heads, kvh, dim, vd, taps, n = 3, 1, 6, 10, 4, 29
    g = torch.Generator().manual_seed(8)
    C = 2 * kvh * dim + heads * vd
    proj = torch.randn(n, C + heads, generator=g)
    w_taps, a2 = torch.randn(C, taps, generator=g) * 0.5, torch.randn(n, heads * dim, generator=g) * 3
    a2[0, 0], a2[1, 1] = 30.0, -30.0                          # softplus far out on both sides
    dt, A = torch.randn(heads * dim, generator=g), torch.randn(heads, generator=g) * 0.5
    y = torch.nn.functional.silu(plain.causal_conv(proj[:, :C].double(), w_taps.double()))
    q, k = y[:, :kvh * dim].reshape(n, kvh, dim), y[:, kvh * dim:2 * kvh * dim].reshape(n, kvh, dim)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dim ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    want = dict(qk=torch.cat([q.reshape(n, -1), k.reshape(n, -1)], 1), v=y[:, 2 * kvh * dim:], beta=torch.sigmoid(proj[:, C:].double()),
                decay=torch.exp(-torch.exp(A.double()).repeat_interleave(dim)[None] * torch.nn.functional.softplus(a2.double() + dt.double())))
    state = torch.zeros((2, taps - 1, C), device=DEV)
    got = {k_: [] for k_ in want}
    for start, m in cuts_of(n, (5, 1, 2, 9)):
        ctx = step_ctx([m], [start], [1])
        rows = proj[start:start + m].to(DEV).contiguous()
        outs = ops.delta_prep(rows, 0, C, w_taps.to(DEV), taps, state, a2[start:start + m].to(DEV).contiguous(), dt.to(DEV), A.to(DEV), ctx,
                              heads, kvh, dim, vd, 1e-6)
        ops.conv_state_update(state, rows, 0, None, taps, ctx)
        for key, o in zip(("qk", "v", "beta", "decay"), outs):
            got[key].append(o.cpu())
    for key in want:
        torch.testing.assert_close(torch.cat(got[key]).double(), want[key], rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(state[1].cpu(), proj[n - taps + 1:, :C])
    assert float(state[0].abs().max()) == 0.0


def test_pair_hash_embedding_and_the_first_token():
    from cellm_b200 import ops
    V, H, buckets, mp, mc = 50, 24, 13, 31, 5
    g = torch.Generator().manual_seed(2)
    table, pairs = torch.randn(V, H, generator=g), torch.randn(buckets + 1, H, generator=g)
    toks = torch.randint(0, V, (23,), generator=g).tolist()
    cfg = {"embedding": {"scale": 0.25, "bigram": {"buckets": buckets, "mul_prev": mp, "mul_cur": mc}}}
    want = plain.embedding(toks, cfg, {"embed": table.double(), "bigram": pairs.double()})
    assert plain.bigram_rows(toks, cfg["embedding"])[0] == buckets
    state = torch.zeros((3, 1), dtype=torch.int32, device=DEV)
    rows = []
    for start, m in cuts_of(len(toks), (4, 1, 2, 7)):
        ctx = step_ctx([m], [start], [2], toks[start:start + m])
        rows.append(ops.embed_pairs(table.to(DEV), pairs.to(DEV), buckets, mp, mc, 0.25, state, ctx).cpu())
    torch.testing.assert_close(torch.cat(rows).double(), want, rtol=1e-6, atol=1e-6)
    assert int(state[2, 0]) == toks[-1]


@pytest.mark.parametrize("T,H", [(9, 54), (5, 56), (3, 2048), (70, 1100)])
def test_stream_kernels_and_activation(T, H):
    """Rows of a width that is and is not a multiple of four (the kernels move four values at a time where they can)."""
    from cellm_b200 import ops
    g = torch.Generator().manual_seed(3)
    x, a, b = (torch.randn(T, H, generator=g) * 3 for _ in range(3))
    w1, w2 = torch.randn(H, generator=g), torch.randn(H, generator=g)
    y1, y2 = ops.norm_pair(x.to(DEV), w1.to(DEV), w2.to(DEV), 1e-5, torch.float32)
    torch.testing.assert_close(y1.cpu().double(), plain.rms(x.double(), 1e-5) * w1.double(), rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(y2.cpu().double(), plain.rms(x.double(), 1e-5) * w2.double(), rtol=1e-5, atol=1e-5)
    out = ops.pair_norm_mean(a.to(DEV), b.to(DEV), w1.to(DEV), w2.to(DEV), 1e-5, torch.float32)
    want = 0.5 * (plain.rms(a.double(), 1e-5) * w1.double() + plain.rms(b.double(), 1e-5) * w2.double())
    torch.testing.assert_close(out.cpu().double(), want, rtol=1e-5, atol=1e-5)
    xs = x.to(DEV).clone()
    ops.scaled_add2(xs, a.to(DEV), b.to(DEV), 0.3)
    torch.testing.assert_close(xs.cpu().double(), x.double() + 0.3 * (a.double() + b.double()), rtol=1e-6, atol=1e-6)
    u = ops.activation(a.to(DEV), "relu2", torch.float32)
    torch.testing.assert_close(u.cpu().double(), torch.relu(a.double()) ** 2, rtol=1e-6, atol=1e-6)
    # 16-bit activations and weights
    b1, b2, ab, bb = w1.bfloat16(), w2.bfloat16(), a.bfloat16(), b.bfloat16()
    y1, y2 = ops.norm_pair(x.to(DEV), b1.to(DEV), b2.to(DEV), 1e-5, torch.bfloat16)
    torch.testing.assert_close(y1.cpu().double(), plain.rms(x.double(), 1e-5) * b1.double(), rtol=2 ** -7, atol=1e-3)
    torch.testing.assert_close(y2.cpu().double(), plain.rms(x.double(), 1e-5) * b2.double(), rtol=2 ** -7, atol=1e-3)
    only, none = ops.norm_pair(x.to(DEV), b1.to(DEV), None, 1e-5, torch.bfloat16)
    assert none is None and torch.equal(only, y1)
    out = ops.pair_norm_mean(a.to(DEV), b.to(DEV), w1.to(DEV), w2.to(DEV), 1e-5, torch.bfloat16)
    torch.testing.assert_close(out.cpu().double(), want, rtol=2 ** -7, atol=1e-3)
    xs = x.to(DEV).clone()
    ops.scaled_add2(xs, ab.to(DEV), bb.to(DEV), 0.3)
    torch.testing.assert_close(xs.cpu().double(), x.double() + 0.3 * (ab.double() + bb.double()), rtol=1e-6, atol=1e-6)
    xs = x.to(DEV).clone()
    ops.scaled_add2(xs, ab.to(DEV), None, -1.5)
    torch.testing.assert_close(xs.cpu().double(), x.double() - 1.5 * ab.double(), rtol=1e-6, atol=1e-6)


@pytest.mark.parametrize("M,K,N", [(300, 64, 200), (17, 128, 96), (8, 64, 80), (2048, 256, 1000), (40, 64, 33), (100, 72, 7), (129, 40, 129)])
def test_product_with_the_activation_in_its_epilogue(M, K, N):
    """Prompt portions under bfloat16 form the feed-forward's activation on the 32-bit sums in the product itself."""
    from cellm_b200 import ops
    g = torch.Generator().manual_seed(M)
    a, w = torch.randn(M, K, generator=g).bfloat16(), (torch.randn(N, K, generator=g) * 0.2).bfloat16()
    want = torch.relu(a.double() @ w.double().T) ** 2
    got = ops.gemm_act(a.to(DEV), w.to(DEV), "relu2", torch.bfloat16).cpu().double()
    torch.testing.assert_close(got, want, rtol=2 ** -7, atol=1e-3)
    got32 = ops.gemm_act(a.to(DEV).float(), w.to(DEV).float(), "relu2", torch.float32).cpu().double()
    torch.testing.assert_close(got32, want, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("hd,window", [(64, 50), (32, 0), (128, 7)])
def test_tensor_core_attention_against_the_plain_kernel(tmp_path, hd, window):
    """One layer under bfloat16, once with the flash kernel and once with the plain kernel on the same rounded inputs:
    prompts, portions and single tokens (whose keys are cut into pieces)."""
    from cellm_b200.parts import sink_attention
    config = model_config(64, 64, [par(left(4, 2, hd, hd, conv=2, window=window, rot=(10000.0, hd // 2, None)), right(1, 4, 8))])
    folder = write_model(tmp_path / "m", config, 6)
    rng = np.random.default_rng(1)
    reqs = {"x": rng.integers(0, 64, 300).tolist(), "y": rng.integers(0, 64, 70).tolist()}
    got = {}
    for tc in (True, False):
        sink_attention.OPTIONS["tensor_cores"] = tc
        try:
            got[tc] = {fam: run_trace(folder, "bfloat16", FAMILIES[fam](reqs), 16) for fam in ("whole", "tail", "mixed")}
        finally:
            sink_attention.OPTIONS["tensor_cores"] = True
    for fam in got[True]:
        for rid, t in reqs.items():
            check_close(traces.as_matrix(got[True][fam][rid], len(t)), traces.as_matrix(got[False][fam][rid], len(t)), "bfloat16",
                        f"flash vs plain {fam} {rid}", k=K_SELF["bfloat16"])
