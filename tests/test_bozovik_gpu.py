"""The Bozovik design against its plain restatement (tests/plain_bozovik.py): the kernels of each mechanism alone, whole
models in every cutting of the requests, pages and slots that are used again, keys at the edges of a window, among the
kept first keys and far away, the sinks, the first tokens of a sequence, long decoding through windows and pages, the
loop over layers, sizes that differ in everything, and greedy generation through the engine and its command lines."""
import json
import math
import os
import re
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_bozovik as plain
import traces
from tolerances import K, K_SELF, check_close

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def grouped(heads, kv_heads, dim, vdim, scale=None, window=0, keep=0, rot=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5}
    if window:
        m["mask"] = {"size": window}
        if keep:
            m["mask"]["keep_first"] = keep
    if rot is not None:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
    return m


def attn(heads, kv_heads, dim, vdim, ff=None, **kw):
    return {"type": "attention", "mixer": grouped(heads, kv_heads, dim, vdim, **kw), "mlp": {"kind": "dense", "ff": ff} if ff else None}


def par(l, heads, dim, scales=(1.0, 1.0), rank=5, ff=None):
    return {"type": "parallel", "mixer": {"left": l, "right": {"heads": heads, "dim": dim, "decay_rank": rank}, "left_scale": scales[0],
                                          "right_scale": scales[1]}, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def latent(heads, dim, rot_dim, vdim, rank, scale=None, window=0, base=10000.0, ff=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank,
         "scale": scale if scale is not None else (dim + rot_dim) ** -0.5, "rot": {"base": base, "dims": rot_dim}}
    if window:
        m["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": m, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def model_config(vocab, width, layers, eps=1e-5, mult=1.0, scale=1.0, side=0, loop=None):
    c = {"architecture": "Bozovik", "vocab": vocab, "width": width, "norm": {"eps": eps}, "residual_mult": mult,
         "embedding": {"scale": scale}, "layers": layers}
    if side:
        c["token_side"] = {"dim": side}
    if loop:
        c["loop"] = dict(zip(("start", "stop", "times"), loop))
    return c


# A: every mixer; key and value widths differ both ways; windows shorter than a page and longer; kept first keys fewer and
# more than a page; a layer without a feed-forward; a loop over the two middle layers; one key/value head and several
CONFIG_A = model_config(300, 96, [
    latent(4, 16, 8, 12, 24, window=40, ff=144),
    par(grouped(4, 2, 16, 24, window=30, keep=5, rot=(10000.0, 8)), 3, 8, scales=(0.7, 0.4), ff=80),
    attn(4, 1, 24, 16, rot=(500.0, 24)),
    latent(2, 8, 4, 20, 16, window=7, base=77.0, ff=64),
], mult=0.6, scale=4.0, side=8, loop=(1, 3, 2))
# B: sizes that are multiples of nothing; no loop and no side input; a factor of one into the stream and an embedding scale
# of one; as many key/value heads as heads; a window longer than every sequence; more kept keys than the window is long;
# no rotation in one attention; a window of one row
CONFIG_B = model_config(211, 54, [
    par(grouped(3, 3, 10, 14, window=1000, keep=3, rot=(77.0, 4)), 2, 5, rank=3, ff=33),
    attn(2, 1, 6, 6, scale=0.9, ff=21),
    latent(3, 5, 6, 7, 9, window=1),
    par(grouped(2, 1, 6, 10, window=9, keep=21), 3, 3, scales=(1.0, 0.5), rank=2),
    latent(1, 7, 2, 3, 11, ff=17),
], eps=1e-6)
# C: heads of 64 and 32 with values as wide (bfloat16 runs the tensor-core attention), the whole model looped three times,
# a delta rule with heads of 64 rows, a latent of 64, a side input wider than a page of keys is long
CONFIG_C = model_config(512, 128, [
    attn(4, 2, 64, 64, rot=(20000.0, 16), ff=192),
    par(grouped(8, 1, 32, 32, window=50, keep=17, rot=(10000.0, 32)), 2, 64, scales=(0.5, 0.5), rank=8, ff=128),
    latent(4, 32, 16, 32, 64, window=130, ff=128),
    par(grouped(2, 2, 64, 64, window=33), 1, 32, rank=4),
], mult=0.5, scale=0.5, side=24, loop=(0, 4, 3))
# D: heads of 128; a loop that starts after the first layer, runs one layer and is followed by others; one pass only
CONFIG_D = model_config(157, 100, [
    par(grouped(2, 1, 128, 128, window=64, keep=1, rot=(10000.0, 64)), 1, 128, rank=6, ff=100),
    attn(2, 2, 20, 10, rot=(100.0, 20), ff=60),
    latent(2, 48, 16, 33, 40, window=20),
    attn(5, 1, 12, 12, ff=40),
], mult=1.3, scale=3.0, side=5, loop=(1, 2, 1))
CONFIGS = {"a": CONFIG_A, "b": CONFIG_B, "c": CONFIG_C, "d": CONFIG_D}
LENGTHS = {"a": [1, 9, 40, 64, 131, 77, 2], "b": [3, 55, 150, 18, 97], "c": [200, 1, 65, 129, 30, 260], "d": [70, 2, 33, 140, 17]}
PAGE = {"a": 8, "b": 16, "c": 16, "d": 4}


def write_model(folder, config, seed, dtype="bfloat16", init=None):
    from cellm_b200.weights import InitSpec, write_random_model
    init = init or InitSpec(linear_std=0.1, embedding_std=0.08, bias_std=0.3, norm_jitter=0.2)
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


class Ref(np.ndarray):
    """A request's plain logits [T, vocab] and, as `.spread` [T], how far `runs` runs whose every product and norm was
    disturbed by a 16-bit rounding's worth (1 + 2^-9 u, u uniform in [-1, 1)) moved each row."""
    def __new__(cls, toks, cfg, w, runs=3):
        exact = plain.forward(toks, cfg, w)
        self = np.asarray(exact.numpy()).view(cls)
        spread = torch.zeros(len(toks), dtype=torch.float64)
        for seed in range(runs):
            with plain.disturbed(2.0 ** -9, seed):
                spread = torch.maximum(spread, (plain.forward(toks, cfg, w) - exact).abs().amax(dim=1))
        self.spread = spread.numpy()
        return self


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """name -> (folder, requests, plain logits)."""
    d = tmp_path_factory.mktemp("bz")
    out = {}
    for i, (name, config) in enumerate(CONFIGS.items()):
        rng = np.random.default_rng(61 + i)
        reqs = {f"r{j}": rng.integers(0, config["vocab"], n).tolist() for j, n in enumerate(LENGTHS[name])}
        folder = write_model(d / name, config, 17 + i)
        cfg, w = load_plain(folder)
        out[name] = (folder, reqs, {rid: Ref(toks, cfg, w) for rid, toks in reqs.items()})
    return out


# Against the plain restatement in 64-bit. The recurrent state carries its 32-bit rounding from token to token, every
# head's read-out is divided by its root mean square and unit vectors of a handful of entries are formed, so the 32-bit
# bound is 1e-5 of the logits' size; bfloat16 keeps the engine's bound, except for rows that rounding alone moves further.
KP = {"float32": 1e-5, "bfloat16": K["bfloat16"]}


def against_plain(got, ref, dtype, what, k32=None):
    """32-bit: one bound for all rows (`k32`: another than the usual one). bfloat16: a row that rounding alone moves further
    than the engine's bound (measured on the plain model) is held to four times that movement instead."""
    if dtype == "float32":
        return check_close(got, ref, dtype, what, k=k32 or KP[dtype])
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
                        dtype, f"{name} {dtype} {fam} vs whole {rid}", k=K_SELF[dtype] if dtype == "bfloat16" else 4e-6)
    got = run_trace(folder, dtype, traces.mixed(reqs), PAGE[name], use_graphs=False)
    for rid, toks in reqs.items():
        check_close(traces.as_matrix(got[rid], len(toks)), traces.as_matrix(results["mixed"][rid], len(toks)), dtype,
                    f"{name} {dtype} mixed: kernel by kernel vs graphs {rid}", k=K_SELF[dtype])


def test_the_stream_after_every_layer_run(models):
    """The 32-bit stream after each run of a layer (a looped layer once for every pass) against the plain model's."""
    from cellm_b200.parts import block as B
    from cellm_b200.replay import Replayer
    folder, reqs, _ = models["a"]
    cfg, w = load_plain(folder)
    toks = reqs["r3"]
    want = []
    plain.forward(toks, cfg, w, want)
    seen = []
    original = B.ScaledPreNormBlock.forward

    def recording(self, residual, ctx, cache):
        original(self, residual, ctx, cache)
        seen.append(residual.x.clone())
    B.ScaledPreNormBlock.forward = recording
    try:
        rp = Replayer(folder, "float32", 64, 8, 4, use_graphs=False)
        rp.step([{"id": "x", "tokens": toks, "want": [0]}], ["x"])
    finally:
        B.ScaledPreNormBlock.forward = original
    assert len(seen) == len(want) == 6                    # layers 0, 1, 2, 1, 2, 3
    for i, (x, ref) in enumerate(zip(seen, want)):
        check_close(x.cpu().numpy(), ref.numpy(), "float32", f"stream after layer run {i}", k=KP["float32"])


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
    """Most of the sequence decoded token by token: the windows pass wholly over decoded tokens, pages behind them are
    given back while the request lives (the kept first keys' pages stay), and the recurrent state walks a hundred and more
    single steps."""
    folder, reqs, ref = models[name]
    some = {rid: reqs[rid] for rid in (("r4", "r5") if name == "a" else ("r0", "r5"))}
    got = run_trace(folder, dtype, traces.tail_one_by_one(some, tail=190), 8)
    for rid, toks in some.items():
        against_plain(traces.as_matrix(got[rid], len(toks)), ref[rid], dtype, f"{name} {dtype} long tail {rid}")


def test_a_windowed_request_holds_its_windows_and_its_first_keys_only(tmp_path):
    """A request longer than the pools of its layers runs through: pages behind a window go back at once, those of the
    kept first keys never, and the logits are the plain model's."""
    from cellm_b200.replay import Replayer
    config = model_config(120, 48, [latent(2, 8, 4, 8, 12, window=20), par(grouped(2, 1, 8, 8, window=14, keep=11, rot=(100.0, 4)), 1, 4, rank=2)])
    folder = write_model(tmp_path / "w", config, 3)
    cfg, w = load_plain(folder)
    toks = np.random.default_rng(0).integers(0, 120, 210).tolist()
    ref = plain.forward(toks, cfg, w).numpy()
    rp = Replayer(folder, "float32", 64, 8, 4)               # 8 pages of 8 tokens a group: 64 keys for 210 tokens
    rows = []
    for i in range(0, len(toks), 5):
        part = toks[i:i + 5]
        rows.append(rp.step([{"id": "x", "tokens": part, "want": list(range(len(part)))}], []))
    check_close(np.concatenate(rows), ref, "float32", "a request longer than its pools", k=KP["float32"])
    kept = [g for g, key in enumerate(rp.cache.paged_keys) if key.keep_first]
    assert len(kept) == 1
    table = rp.cache.block_table(0, kept[0], np.full((64,), -1, dtype=np.int32))
    assert (table[:2] >= 0).all() and (table[2:20] < 0).all()            # 11 kept keys lie in the first two pages
    rp.step([], ["x"])
    assert rp.cache.live == 0 and all(rp.cache.free_pages(g) == rp.cache.group_pages[g] for g in range(len(rp.cache.group_pages)))


# ------------------------------------------------------------------------- window edges, kept keys, far keys, the sinks
def sharp_config(scale, window, keep):
    return model_config(128, 64, [
        par(grouped(4, 2, 16, 16, scale=scale, window=window, keep=keep, rot=(10000.0, 8)), 1, 4, scales=(1.0, 0.2), rank=2),
        latent(2, 16, 8, 16, 24, scale=scale, window=window + 6),
        attn(2, 1, 32, 16, scale=scale * 0.7, rot=(1000.0, 16)),
    ], mult=1.0, scale=1.0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sharp_attention_at_the_edges_and_far_back(tmp_path, dtype):
    """A softmax so peaked (a large score scale on wide projections) that a row's output is a few single keys wherever they
    lie: a key lost at a page border, at a window's far edge or among the kept first keys, one seen beyond the window, or
    a forgotten sink changes the logits outright. The test first asserts, on the plain model, that such rows exist."""
    from cellm_b200.weights import InitSpec
    window, keep = 37, 6
    scale = 0.6 if dtype == "float32" else 0.2
    folder = write_model(tmp_path / "sharp", sharp_config(scale, window, keep), 9,
                         init=InitSpec(linear_std=0.25, embedding_std=0.1, bias_std=0.05, norm_jitter=0.1))
    cfg, w = load_plain(folder)
    rng = np.random.default_rng(4)
    toks = rng.integers(0, cfg["vocab"], 500).tolist()
    reqs = {"long": toks, "short": toks[:45]}
    ref = {rid: Ref(t, cfg, w, runs=6) for rid, t in reqs.items()}
    eps, pos = cfg["norm"]["eps"], torch.arange(len(toks))
    x0 = plain.forward_until(toks, cfg, w, 0)
    h0 = plain.layer_norm(x0, w["l0.norm1"], w["l0.norm1.b"], eps)
    seen = []
    plain.windowed_sink_attention(h0, w, "l0.mix.left.", cfg["layers"][0]["mixer"]["left"], pos, seen)
    W = seen[0]                                                 # [heads, T, T]
    top, where = W[:, 100:].max(-1)
    assert float(top.median()) > (0.5 if dtype == "float32" else 0.25)
    dist = torch.arange(100, 500)[None] - where
    assert int((dist == window - 1).sum()) >= 3                  # the heaviest key is the window's last
    assert int((where < keep).sum()) >= 3                        # or one of the kept first keys, hundreds of tokens back
    assert float(W[:, 100:, :keep].sum(-1).max()) > 0.2 and float(W[:, 100:, keep:60].max()) == 0.0
    assert float(W.sum(-1).min()) < 0.9                          # the sink takes a share somewhere
    x2 = plain.forward_until(toks, cfg, w, 2)
    seen = []
    plain.grouped_attention(plain.layer_norm(x2, w["l2.norm1"], w["l2.norm1.b"], eps), w, "l2.mix.", cfg["layers"][2]["mixer"], pos,
                            torch.zeros(2, dtype=torch.float64), temp=w["l2.mix.temp"], weights_out=seen)
    top, where = seen[0][:, 400:].max(-1)
    assert float((torch.arange(400, 500)[None] - where).float().median()) > 40      # the last layer reaches far back
    for fam in ("whole", "tail", "portions", "mixed"):
        for page in (8, 32):
            got = run_trace(folder, dtype, FAMILIES[fam](reqs), page)
            for rid, t in reqs.items():
                # so peaked a softmax passes a score's last bits on: the plain model itself, run in 32-bit, is 4e-5 of the
                # logits' size away from its 64-bit run; a lost or surplus key moves a row by a tenth of that size and more
                against_plain(traces.as_matrix(got[rid], len(t)), ref[rid], dtype, f"sharp {dtype} {fam} page {page} {rid}", k32=1e-4)


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


@pytest.mark.parametrize("heads,dim", [(4, 16), (2, 64), (3, 5), (1, 128), (2, 48), (2, 33), (1, 136)])
def test_generalized_delta_rule_alone(heads, dim):
    """Two sequences side by side in slots 3 and 1, fed whole and in portions down to one token: the inputs' kernel and the
    walk against the plain recurrence in 64-bit, the cuttings against each other bit for bit, other slots untouched."""
    from cellm_b200 import ops
    g = torch.Generator().manual_seed(heads * 100 + dim)
    n, lens, slots = heads * dim, [41, 19], [3, 1]
    rate = math.exp(-0.5)
    proj = [torch.randn(L, 4 * n, generator=g) for L in lens]          # r | k | v | a_pre
    w_pre = [torch.randn(L, n, generator=g) * 2 for L in lens]
    w0, a_bias = torch.randn(n, generator=g), torch.randn(n, generator=g)
    want = []
    for p, wp in zip(proj, w_pre):
        p, wp = p.double(), wp.double()
        L = p.shape[0]
        r, k, v, a = (p[:, i * n:(i + 1) * n].reshape(L, heads, dim) for i in range(4))
        d = torch.exp(-rate * torch.sigmoid(wp + w0.double())).reshape(L, heads, dim)
        a = torch.sigmoid(a + a_bias.double().reshape(heads, dim))
        u = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
        S = torch.zeros(heads, dim, dim, dtype=torch.float64)
        o = []
        for t in range(L):
            uS = torch.einsum("hi,hij->hj", u[t], S)
            S = d[t][:, :, None] * S - (a[t] * u[t])[:, :, None] * uS[:, None, :] + k[t][:, :, None] * v[t][:, None, :]
            o.append(torch.einsum("hij,hi->hj", S, r[t]).reshape(-1))
        want.append(torch.stack(o))
    outs = {}
    for name, sizes in (("whole", (64,)), ("portions", (5, 1, 2, 11)), ("single", (1,))):
        state = torch.full((4, heads, dim, dim), 7.0, device=DEV)
        state[slots] = 0
        got = [[] for _ in lens]
        cuts = [cuts_of(L, sizes) for L in lens]
        for step in range(max(len(c) for c in cuts)):
            live = [b for b in range(len(lens)) if step < len(cuts[b])]
            rows = lambda src: torch.cat([src[b][cuts[b][step][0]:cuts[b][step][0] + cuts[b][step][1]] for b in live]).to(DEV).contiguous()
            ctx = step_ctx([cuts[b][step][1] for b in live], [cuts[b][step][0] for b in live], [slots[b] for b in live])
            pr = rows(proj)
            vecs = ops.gdelta_prep(pr, n, 3 * n, rows(w_pre), w0.to(DEV), a_bias.to(DEV), rate, 1e-6, heads, dim)
            o = ops.gdelta_scan(pr, 0, n, 2 * n, vecs, state, ctx, heads, dim, dim).cpu()
            at = 0
            for b in live:
                got[b].append(o[at:at + cuts[b][step][1]])
                at += cuts[b][step][1]
        outs[name] = [torch.cat(g_) for g_ in got]
        assert float(state[0].min()) == 7.0 and float(state[2].max()) == 7.0
        for b in range(len(lens)):
            torch.testing.assert_close(outs[name][b].double(), want[b], rtol=3e-5, atol=3e-5 * float(want[b].abs().max()))
    for b in range(len(lens)):
        assert torch.equal(outs["whole"][b], outs["portions"][b]) and torch.equal(outs["whole"][b], outs["single"][b])


@pytest.mark.parametrize("T,H", [(9, 54), (5, 56), (3, 2048), (70, 1100)])
def test_stream_kernels(T, H):
    """Addend times a constant + layer norm / RMS norm / no norm (all rows and chosen rows), the start of another pass, a
    token's own row gated by the stream, the RMS-normed addition, the weighted sum of two mixers, xIELU, the per-head gate
    and the per-head norm with a row of weights for every head: each against 64-bit torch."""
    from cellm_b200 import ops
    g = torch.Generator().manual_seed(T * 7 + H)
    rnd = lambda *s: torch.randn(*s, generator=g)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    x, a, w, b = rnd(T, H) * 3 + 0.5, rnd(T, H), 1 + 0.2 * rnd(H), 0.3 * rnd(H)
    for add_dtype in (torch.float32, torch.bfloat16):
        ad = a.to(add_dtype)
        s = x.double() + 0.7 * ad.double()
        mu = s.mean(-1, keepdim=True)
        want = {"layer": (s - mu) / torch.sqrt(((s - mu) ** 2).mean(-1, keepdim=True) + 1e-5) * w.double() + b.double(),
                "rms": s / torch.sqrt((s * s).mean(-1, keepdim=True) + 1e-5) * w.double(), "none": s}
        for kind in ("layer", "rms", "none"):
            xd = x.to(DEV).clone()
            y = ops.add_scaled_norm(xd, ad.to(DEV), 0.7, None, 0.0, kind, w.to(DEV), b.to(DEV) if kind == "layer" else None, 1e-5, torch.float32)
            torch.testing.assert_close(xd.cpu().double(), s, rtol=1e-6, atol=1e-6)
            torch.testing.assert_close(y.cpu().double(), want[kind], rtol=2e-5, atol=2e-5)
            rows = torch.tensor([T - 1, 0, T // 2], dtype=torch.int32, device=DEV)
            xd = x.to(DEV).clone()
            y = ops.add_scaled_norm(xd, ad.to(DEV), 0.7, None, 0.0, kind, w.to(DEV), b.to(DEV) if kind == "layer" else None, 1e-5, torch.float32, rows)
            assert torch.equal(xd.cpu(), x)                                        # chosen rows leave the stream as it was
            torch.testing.assert_close(y.cpu().double(), want[kind][rows.cpu().long()], rtol=2e-5, atol=2e-5)
    # a row far from zero: the variance is that of the deviations, not a difference of large squares
    far = (100.0 + 0.1 * rnd(T, H)).to(DEV)
    y = ops.add_scaled_norm(far.clone(), None, 0.0, None, 0.0, "layer", torch.ones(H, device=DEV), None, 1e-5, torch.float32).cpu().double()
    fd = far.cpu().double()
    mu = fd.mean(-1, keepdim=True)
    torch.testing.assert_close(y, (fd - mu) / torch.sqrt(((fd - mu) ** 2).mean(-1, keepdim=True) + 1e-5), rtol=3e-3, atol=3e-3)
    # the start of another pass
    V = 23
    table, ids, vec = rnd(V, H).to(torch.bfloat16), torch.randint(0, V, (T,), generator=g), rnd(H)
    xd = x.to(DEV).clone()
    ops.stream_add_rows(xd, table.to(DEV), ids.to(torch.int32).to(DEV), 1.7, vec.to(DEV), err)
    torch.testing.assert_close(xd.cpu().double(), x.double() + 1.7 * table.double()[ids] + vec.double(), rtol=1e-6, atol=1e-5)
    xd = x.to(DEV).clone()
    ops.stream_add_rows(xd, None, None, 1.0, vec.to(DEV), err)
    torch.testing.assert_close(xd.cpu().double(), x.double() + vec.double(), rtol=1e-6, atol=1e-5)
    # a token's own row gated by the stream; the RMS-normed addition
    n, col0 = 7, 5
    wide, gpre = rnd(V, 19), rnd(T, n) * 2
    e = ops.token_gate_mul(gpre.to(DEV), wide.to(DEV), col0, ids.to(torch.int32).to(DEV), "gelu_tanh", torch.float32, err).cpu().double()
    torch.testing.assert_close(e, plain.gelu_tanh(gpre.double()) * wide.double()[ids][:, col0:col0 + n], rtol=1e-5, atol=1e-6)
    yv = rnd(T, H)
    xd = x.to(DEV).clone()
    ops.scaled_rms_add(xd, yv.to(DEV), w.to(DEV), 0.3, 1e-5)
    torch.testing.assert_close(xd.cpu().double(), x.double() + 0.3 * plain.rms(yv.double(), 1e-5) * w.double(), rtol=1e-5, atol=1e-5)
    # two mixers' weighted sum; xIELU on both sides of zero, with softplus far out on both sides
    torch.testing.assert_close(ops.weighted_sum2(a.to(DEV), 0.6, yv.to(DEV), -0.5).cpu().double(), 0.6 * a.double() - 0.5 * yv.double(), rtol=1e-6, atol=1e-6)
    for p, q in ((0.3, -0.2), (25.0, -30.0), (-30.0, 25.0)):
        pq = torch.tensor([p, q])
        z = rnd(T, H) * 3
        torch.testing.assert_close(ops.xielu(z.to(DEV), pq.to(DEV), torch.float32).cpu().double(),
                                   plain.xielu(z.double(), pq[0].double(), pq[1].double()), rtol=2e-5, atol=1e-5)
    assert int(err.item()) == 0
    # the per-head gate and the per-head norm with a row of weights for every head
    heads = 2 if H % 2 == 0 else 1
    vd = H // heads
    gate = rnd(T, heads + 3)
    o = ops.head_gate_mul(a.to(DEV).clone(), gate.to(DEV)[:, 3:], heads).cpu().double()
    torch.testing.assert_close(o, (a.double().reshape(T, heads, vd) * torch.sigmoid(gate.double()[:, 3:, None])).reshape(T, H), rtol=1e-5, atol=1e-6)
    gw = rnd(T, H)
    o = ops.head_norm_gate(a.to(DEV), w.to(DEV), gw.to(DEV), heads, vd, 1e-5, torch.float32).cpu().double()
    want = (plain.rms(a.double().reshape(T, heads, vd), 1e-5).reshape(T, H) * w.double()) * torch.sigmoid(gw.double())
    torch.testing.assert_close(o, want, rtol=2e-5, atol=2e-5)


@pytest.mark.parametrize("M,K,N", [(300, 64, 200), (17, 128, 96), (8, 64, 80), (2048, 256, 1000), (40, 64, 33), (129, 40, 129)])
def test_product_with_xielu_in_its_epilogue(M, K, N):
    """The feed-forward's first product with xIELU formed on its 32-bit sums (the tensor-core product's epilogue for prompt
    portions, a kernel of its own for few rows), against 64-bit torch, in both output types."""
    from cellm_b200 import ops
    g = torch.Generator().manual_seed(M + K + N)
    a = (torch.randn(M, K, generator=g) * 0.7).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) * 0.3).to(torch.bfloat16)
    pq = torch.tensor([0.4, -0.7])
    want = plain.xielu(a.double() @ w.double().T, pq[0].double(), pq[1].double())
    for out_dtype, tol in ((torch.float32, 2e-5), (torch.bfloat16, 8e-3)):
        got = ops.gemm_act(a.to(DEV), w.to(DEV), "xielu", out_dtype, pq.to(DEV)).cpu().double()
        torch.testing.assert_close(got, want, rtol=tol, atol=tol * float(want.abs().max()))


class _Pages:
    """A pool of keys and values with one request's pages in an order of their own."""
    def __init__(self, n_tokens, nkv, hd, vd, page, dtype, g, values=True):
        n_pages = -(-n_tokens // page) + 3
        self.k = torch.zeros(n_pages, nkv, page, hd, dtype=dtype, device=DEV)
        self.v = torch.zeros(n_pages, nkv, page, vd, dtype=dtype, device=DEV) if values else None
        order = torch.randperm(n_pages, generator=g)[: -(-n_tokens // page)]
        self.block_table = order.to(torch.int32).reshape(1, -1).to(DEV)
        self.page_size, self.order = page, order

    def put(self, keys, vals):
        for j in range(keys.shape[0]):
            p, s = int(self.order[j // self.page_size]), j % self.page_size
            self.k[p, :, s] = keys[j].to(self.k.dtype)
            if self.v is not None:
                self.v[p, :, s] = vals[j].to(self.v.dtype)


@pytest.mark.parametrize("window,keep,page", [(16, 0, 8), (16, 5, 8), (33, 9, 16), (5, 40, 4), (0, 0, 8), (1, 1, 8), (130, 3, 32)])
def test_masked_attention_sees_exactly_the_window_and_the_kept_keys(window, keep, page):
    """One key at a time carries a value that stands out; a query scores every key alike. The output tells which keys the
    row summed: those inside the window or among the kept first ones, and no key beyond either edge; with the sink's share
    and the gate on top. Prompt rows and single decoded rows, keys at page borders included."""
    from cellm_b200 import ops
    g = torch.Generator().manual_seed(window * 100 + keep)
    T, nh, nkv, hd, vd = 150, 2, 1, 8, 6
    keys = torch.zeros(T, nkv, hd)
    keys[:, :, 0] = 1.0
    vals = torch.zeros(T, nkv, vd)
    vals[:, 0, 0] = torch.arange(T, dtype=torch.float32) + 1          # the sum over a row's keys names them
    vals[:, 0, 1] = 1.0                                                # their number
    pool = _Pages(T, nkv, hd, vd, page, torch.float32, g)
    pool.put(keys, vals)
    q = torch.zeros(T, nh, hd)
    q[:, :, 0] = 0.5
    sinks = torch.tensor([math.log(3.0) + 0.5, -1e4])                  # head 0: a sink worth three keys (a key scores 0.5); head 1: none to speak of
    gate = torch.randn(T, nh, generator=g)
    for rows in (list(range(T)), [T - 1], [keep], [max(keep, 1) + window], [page - 1], [page], [0]):
        rows = [r for r in rows if 0 <= r < T]
        if len(rows) == T:
            ctx = step_ctx([T], [0], [0])
        else:
            ctx = step_ctx([1], [rows[0]], [0])
        out = ops.attention_plain_masked(q[rows].reshape(len(rows), -1).to(DEV).contiguous(), pool, ctx, nh, nkv, hd, vd, 1.0, window, keep,
                                         sinks.to(DEV), None, gate[rows].to(DEV).contiguous()).cpu().double().reshape(len(rows), nh, vd)
        for n, i in enumerate(rows):
            seen = [j for j in range(i + 1) if window == 0 or i - j < window or j < keep]
            for h in range(nh):
                denom = len(seen) + (3.0 if h == 0 else 0.0)
                gt = 1 / (1 + math.exp(-float(gate[i, h])))
                assert abs(float(out[n, h, 1]) - gt * len(seen) / denom) < 1e-5, (i, h, "how many keys")
                assert abs(float(out[n, h, 0]) - gt * sum(j + 1 for j in seen) / denom) < 1e-3, (i, h, "which keys")
    # a fixed sink of score 0 adds one to the denominator
    ctx = step_ctx([T], [0], [0])
    out = ops.attention_plain_masked(q.reshape(T, -1).to(DEV).contiguous(), pool, ctx, nh, nkv, hd, vd, 1.0, window, keep, None, 0.0, None)
    out = out.cpu().double().reshape(T, nh, vd)
    for i in (0, 1, T - 1):
        seen = [j for j in range(i + 1) if window == 0 or i - j < window or j < keep]
        assert abs(float(out[i, 0, 1]) - len(seen) * math.exp(0.5) / (len(seen) * math.exp(0.5) + 1.0)) < 1e-5


@pytest.mark.parametrize("hd,window,keep", [(64, 50, 0), (32, 0, 0), (128, 7, 0), (64, 40, 9), (32, 20, 70), (64, 0, 0), (64, 200, 30), (128, 150, 70)])
def test_tensor_core_attention_against_the_plain_kernel(tmp_path, hd, window, keep):
    """The bfloat16 mixer (paged mma.sync attention with sink, gate and kept first keys) against the plain kernel on the
    same cache, for a prompt, portions and single tokens (windows of 150 and more: a single token's keys are cut into
    pieces, whose list of blocks starts with the kept keys' blocks)."""
    from cellm_b200.parts import sink_attention as SA
    config = model_config(64, 64, [par(grouped(4, 2, hd, hd, window=window, keep=keep, rot=(10000.0, hd // 2)), 1, 4, rank=2),
                                   attn(4, 1, hd, hd, rot=(10000.0, hd))])
    folder = write_model(tmp_path / "t", config, 5)
    toks = np.random.default_rng(1).integers(0, 64, 300).tolist()
    reqs = {"x": toks, "y": toks[:33]}
    outs = {}
    for tc in (True, False):
        SA.OPTIONS["tensor_cores"] = tc
        try:
            outs[tc] = {fam: run_trace(folder, "bfloat16", FAMILIES[fam](reqs), 16) for fam in ("whole", "tail", "portions")}
        finally:
            SA.OPTIONS["tensor_cores"] = True
    for fam in outs[True]:
        for rid, t in reqs.items():
            check_close(traces.as_matrix(outs[True][fam][rid], len(t)), traces.as_matrix(outs[False][fam][rid], len(t)), "bfloat16",
                        f"tensor cores vs plain, {fam} {rid}", k=K_SELF["bfloat16"])


def test_tcgen05_attention_with_sinks_and_gate_against_the_mma_kernel(tmp_path):
    """Prompt portions that fill its tiles run the attention of heads of 64 on tcgen05 (scores and outputs in tensor
    memory), with the sink in a row's denominator and the gate in its normalisation: against the mma.sync kernel on the same
    requests, for a windowed attention with learned sinks and for one over every key with a temperature and the fixed sink."""
    import importlib
    from cellm_b200.parts import sink_attention as SA
    from cellm_b200.runtime import program
    A = importlib.import_module("cellm_b200.ops.attention")      # (the package exports a function of this name)
    config = model_config(80, 128, [par(grouped(8, 2, 64, 64, window=70, rot=(10000.0, 32)), 1, 8, rank=2, ff=64),
                                   attn(4, 1, 64, 64, rot=(5000.0, 64), ff=64)], mult=0.7, side=8)
    folder = write_model(tmp_path / "t", config, 8)
    cfg, w = load_plain(folder)
    toks = np.random.default_rng(2).integers(0, 80, 700).tolist()
    reqs = {"x": toks, "y": toks[100:333]}
    ref = {rid: Ref(t, cfg, w) for rid, t in reqs.items()}
    calls = []
    original = A.attention_tc

    def counting(*a, **k):
        calls.append(1)
        return original(*a, **k)
    A.attention_tc = counting
    old = program.OPTIONS["attention_tc_min_ctas"]
    program.OPTIONS["attention_tc_min_ctas"] = 1
    outs = {}
    try:
        for on in (True, False):
            SA.OPTIONS["tcgen05"] = on
            n = len(calls)
            outs[on] = {fam: run_trace(folder, "bfloat16", make(reqs), 16) for fam, make in
                        (("whole", traces.whole), ("portions", lambda r: traces.portions(r, (300, 64, 130, 2))))}
            assert (len(calls) > n) == on
    finally:
        SA.OPTIONS["tcgen05"] = True
        program.OPTIONS["attention_tc_min_ctas"] = old
        A.attention_tc = original
    for fam in outs[True]:
        for rid, t in reqs.items():
            against_plain(traces.as_matrix(outs[True][fam][rid], len(t)), ref[rid], "bfloat16", f"tcgen05 {fam} {rid}")
            check_close(traces.as_matrix(outs[True][fam][rid], len(t)), traces.as_matrix(outs[False][fam][rid], len(t)), "bfloat16",
                        f"tcgen05 vs mma.sync, {fam} {rid}", k=K_SELF["bfloat16"])


def test_config_reader_takes_what_the_file_leaves_out(tmp_path):
    """No loop, no side input, no mask, no rotation, no kv_heads: none of them exists then."""
    from cellm_b200.config import config_from_dict
    d = {"architecture": "Bozovik", "vocab": 50, "width": 32, "norm": {"eps": 1e-5}, "layers": [
        {"type": "attention", "mixer": {"heads": 2, "dim": 8, "vdim": 8, "scale": 0.3}, "mlp": None}]}
    cfg, plan = config_from_dict(d)
    assert cfg.loop is None and cfg.token_side_dim == 0 and cfg.residual_mult == 1.0 and cfg.embedding_scale == 1.0
    m = cfg.layers[0].mixer
    assert m.kv_heads == 2 and m.window == 0 and m.keep_first == 0 and m.rot is None
    assert [e.layer for e in plan.order] == [0]
    folder = write_model(tmp_path / "m", d, 1)
    c, w = load_plain(folder)
    toks = list(range(20))
    got = run_trace(folder, "float32", traces.portions({"r": toks}, (3, 2)), 8)
    check_close(traces.as_matrix(got["r"], 20), plain.forward(toks, c, w).numpy(), "float32", "bare model", k=KP["float32"])
