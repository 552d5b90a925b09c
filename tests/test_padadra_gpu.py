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
        out[name] = (folder, reqs, {rid: plain.forward(toks, cfg, w).numpy() for rid, toks in reqs.items()})
    return out


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
            check_close(traces.as_matrix(got[rid], len(toks)), ref[rid], dtype, f"{name} {dtype} {fam} {rid}")
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
            check_close(traces.as_matrix(got[rid], len(toks)), ref[rid], dtype, f"{name} {dtype} portions {sizes} {rid}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "c"])
def test_long_decoding_through_windows_and_pages(models, name, dtype):
    """Most of the sequence decoded token by token: the windows (7 and 40, 50 and 130 keys) pass wholly over decoded tokens,
    pages are given back while the request lives, and the recurrent states walk a hundred and more single steps."""
    folder, reqs, ref = models[name]
    some = {rid: reqs[rid] for rid in (("r4", "r5") if name == "a" else ("r0", "r5"))}
    got = run_trace(folder, dtype, traces.tail_one_by_one(some, tail=190), 8)
    for rid, toks in some.items():
        check_close(traces.as_matrix(got[rid], len(toks)), ref[rid], dtype, f"{name} {dtype} long tail {rid}")


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
    check_close(np.concatenate(rows), ref["r4"], "float32", "a request longer than its pools")
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
    ref = {rid: plain.forward(t, cfg, w) for rid, t in reqs.items()}
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
                check_close(traces.as_matrix(got[rid], len(t)), ref[rid].numpy(), dtype, f"sharp {dtype} {fam} page {page} {rid}")


# ------------------------------------------------------------------------------------------ generation
def check_greedy_tokens(cfg, w, prompt, out, dtype):
    seq = list(prompt) + list(out[:-1])
    ref = plain.forward(seq, cfg, w)[len(prompt) - 1:].numpy()
    tol = 2 * K[dtype] * (1 + np.abs(ref).max())
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
    check_close(rows, ref["r3"], "float32", "trace_run")
