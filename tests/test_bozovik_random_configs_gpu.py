"""Random Bozovik configurations (fixed seeds): widths that are and are not multiples of 8, the three mixers in any order
and number, head sizes of every relation to the fast kernels' (32, 64, 128 and others), key and value widths equal or
not, one to four key/value heads with one to eight query heads each, windows from one key to longer than the requests,
kept first keys from none to more than the window, rotations of none, some and all of a head's entries, latents whose
widths are and are not multiples of 16, delta rules with heads of 3 to 136 rows, layers without a feed-forward, with and
without the side input, and loops over any run of layers one to three times. Each is replayed whole and as a mixed trace
in both element types against the plain restatement, and some generate through the engine."""
import numpy as np
import pytest

import plain_bozovik as plain
import traces
from test_bozovik_gpu import KP, Ref, against_plain, attn, check_greedy_tokens, grouped, latent, load_plain, model_config, par, run_trace, write_model

pytestmark = pytest.mark.gpu

SEEDS = list(range(16))


def random_config(seed):
    rng = np.random.default_rng(3000 + seed)
    pick = lambda xs: xs[int(rng.integers(0, len(xs)))]
    width = pick([40, 54, 64, 96, 100, 128, 160])

    def rot(dim):
        if rng.random() < 0.2:
            return None
        return (pick([100.0, 10000.0, 1e6]), pick([d for d in (2, 4, 8, 16, 32, 64, dim) if d <= dim and d % 2 == 0]))

    def group(windowed):
        kv = pick([1, 2, 3, 4])
        heads = kv * pick([1, 2, 4, 8])
        dim = pick([6, 8, 16, 20, 32, 48, 64, 72, 128])
        vdim = pick([dim, dim, dim, 8, 24, 40])
        window = pick([1, 3, 7, 16, 33, 64, 500]) if windowed else 0
        keep = pick([0, 1, 2, 5, 17, 40]) if windowed else 0
        return grouped(heads, kv, dim, vdim, scale=round(dim ** -0.5 * float(rng.uniform(0.5, 1.5)), 4), window=window, keep=keep, rot=rot(dim))
    layers = []
    for _ in range(int(rng.integers(1, 5))):
        ff = pick([None, 24, 33, 64, 100])
        kind = pick(["attention", "parallel", "latent"])
        if kind == "attention":
            m = group(False)
            layers.append(attn(m["heads"], m["kv_heads"], m["dim"], m["vdim"], ff=ff, scale=m["scale"],
                               rot=(m["rot"]["base"], m["rot"]["dims"]) if "rot" in m else None))
        elif kind == "parallel":
            layers.append(par(group(rng.random() < 0.85), pick([1, 2, 3]), pick([3, 4, 8, 16, 32, 33, 64, 136]),
                              scales=(round(float(rng.uniform(0.3, 1.2)), 3), round(float(rng.uniform(0.2, 1.0)), 3)), rank=pick([1, 3, 8, 16]), ff=ff))
        else:
            dim, rd = pick([3, 4, 8, 16, 24, 64]), pick([2, 4, 8, 16, 32])
            layers.append(latent(pick([1, 2, 3, 4, 8]), dim, rd, pick([4, 8, 16, 40, 64]), pick([8, 12, 16, 24, 48, 64, 80]),
                                 window=pick([0, 1, 5, 16, 40, 300]), base=pick([50.0, 10000.0, 5e5]), ff=ff))
    n = len(layers)
    loop = None
    if rng.random() < 0.7:
        start = int(rng.integers(0, n))
        loop = (start, int(rng.integers(start + 1, n + 1)), int(rng.integers(1, 4)))
    return model_config(int(rng.integers(50, 400)), width, layers, eps=pick([1e-5, 1e-6]), mult=pick([1.0, 0.5, 0.8, 1.4]),
                        scale=pick([1.0, 2.0, 5.5]), side=pick([0, 0, 3, 8, 16]), loop=loop)


@pytest.mark.parametrize("seed", SEEDS)
def test_random_configuration(tmp_path, seed):
    config = random_config(seed)
    rng = np.random.default_rng(seed)
    reqs = {f"r{j}": rng.integers(0, config["vocab"], int(n)).tolist() for j, n in enumerate(rng.integers(1, 90, 3))}
    page = [4, 8, 16, 32][seed % 4]
    folder = write_model(tmp_path / "m", config, 77 + seed)
    cfg, w = load_plain(folder)
    ref = {rid: Ref(toks, cfg, w) for rid, toks in reqs.items()}
    for dtype in ("float32", "bfloat16"):
        for fam, make in (("whole", traces.whole), ("mixed", traces.mixed)):
            got = run_trace(folder, dtype, make(reqs), page)
            for rid, toks in reqs.items():
                against_plain(traces.as_matrix(got[rid], len(toks)), ref[rid], dtype, f"seed {seed} {dtype} {fam} {rid}")


@pytest.mark.parametrize("seed", SEEDS[:4])
def test_random_configuration_generates(tmp_path, seed):
    from cellm_b200 import Engine, SamplingParams
    config = random_config(seed)
    folder = write_model(tmp_path / "m", config, 5 + seed)
    cfg, w = load_plain(folder)
    rng = np.random.default_rng(seed)
    prompts = [rng.integers(0, config["vocab"], int(n)).tolist() for n in (3, 40, 17)]
    eng = Engine(folder, dtype="float32", tokens_per_block=8, total_blocks=64, max_num_seqs=2, max_batch_tokens=32, prefill_chunk=16)
    outs = eng.generate(prompts, SamplingParams.greedy(8, stop_eos=False))
    for prompt, out in zip(prompts, outs):
        check_greedy_tokens(cfg, w, prompt, out, "float32")
    s = eng.stats()
    assert s["idle"] and s["free_pages"] == s["total_pages"]
