"""What the Bozovik design adds that needs no GPU: its configuration reader (what the file leaves out does not exist;
faults name their key), the run order of looped layers with the items at which a pass begins, the tensors its plan
expects, and the cache manager's pages for a window that keeps the sequence's first keys."""
import numpy as np
import pytest
import torch

from cellm_b200 import models, parts  # noqa: F401  (register architectures and parts)
from cellm_b200.cache import CacheManager
from cellm_b200.config import ConfigError, config_from_dict
from cellm_b200.parts import PagedKV
from cellm_b200.weights.loader import expected_tensors


def grouped(**kw):
    return {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 12, "scale": 0.3, **kw}


def config(layers, **top):
    return {"architecture": "Bozovik", "vocab": 90, "width": 40, "norm": {"eps": 1e-5}, "layers": layers, **top}


ATT = {"type": "attention", "mixer": grouped(rot={"base": 100.0, "dims": 4}), "mlp": {"kind": "dense", "ff": 24}}
PAR = {"type": "parallel", "mixer": {"left": grouped(mask={"size": 9, "keep_first": 3}), "right": {"heads": 2, "dim": 4}, "left_scale": 0.7,
                                     "right_scale": 0.2}, "mlp": None}
LAT = {"type": "latent_attention", "mixer": {"heads": 2, "dim": 8, "rot_dim": 4, "vdim": 6, "kv_rank": 10, "scale": 0.2, "mask": {"size": 5},
                                             "rot": {"base": 50.0, "dims": 4}}, "mlp": {"kind": "dense", "ff": 16}}


def test_the_reader_takes_every_constant_from_the_file():
    cfg, plan = config_from_dict(config([ATT, PAR, LAT], residual_mult=0.4, embedding={"scale": 3.0}, token_side={"dim": 5},
                                        loop={"start": 1, "stop": 3, "times": 3}))
    assert (cfg.residual_mult, cfg.embedding_scale, cfg.token_side_dim) == (0.4, 3.0, 5)
    left = cfg.layers[1].mixer.left
    assert (left.window, left.keep_first, left.kv_heads, left.vdim) == (9, 3, 2, 12) and cfg.layers[1].mixer.right_scale == 0.2
    assert cfg.layers[2].mixer.window == 5 and cfg.layers[0].mixer.window == 0 and cfg.layers[0].mixer.rot.dims == 4
    assert [e.layer for e in plan.order] == [0, 1, 2, 1, 2, 1, 2]
    block = plan.layers[1].block
    assert block.params["passes"] == {1: 0, 3: 1, 5: 2} and block.params["n_passes"] == 3 and block.params["embedding_scale"] == 3.0
    assert "passes" not in plan.layers[0].block.params and "passes" not in plan.layers[2].block.params
    assert [plan.layers[i].block.params["token_rows"]["offset"] for i in range(3)] == [0, 5, 10]
    assert plan.layers[1].mixer.kind == "weighted_pair" and plan.layers[1].mixer.params["first"].params["keep_first"] == 3
    assert plan.layers[0].mixer.params["fixed_sink"] == 0.0 and not plan.layers[0].mixer.params["sinks"]
    names = expected_tensors(plan)
    assert names["side.embed"].shape == (90, 15) and names["loop.step"].shape == (3, 40) and names["l1.mix.right.w1"].shape == (-1, 40)
    assert {"l0.mix.temp", "l0.mix.g", "l1.mix.left.sink", "l1.mix.right.a.b", "l2.mix.dkv.norm", "l2.mix.sink", "l0.norm1.b", "final.norm.b",
            "l0.mlp.act", "l2.side.gate"} <= set(names)
    assert "l1.mlp.up" not in names and "l0.mix.sink" not in names


def test_what_the_file_leaves_out_does_not_exist():
    cfg, plan = config_from_dict(config([ATT, LAT]))
    assert cfg.loop is None and cfg.token_side_dim == 0 and cfg.residual_mult == 1.0 and cfg.embedding_scale == 1.0
    assert [e.layer for e in plan.order] == [0, 1]
    names = expected_tensors(plan)
    assert "side.embed" not in names and "loop.step" not in names and "l0.side.gate" not in names
    # a loop over no layers is no loop; one pass still adds its vector
    assert config_from_dict(config([ATT, LAT], loop={"start": 1, "stop": 1, "times": 4}))[0].loop is None
    cfg, plan = config_from_dict(config([ATT, LAT], loop={"start": 0, "stop": 1, "times": 1}))
    assert [e.layer for e in plan.order] == [0, 1] and plan.layers[0].block.params["passes"] == {0: 0}


@pytest.mark.parametrize("change,key", [
    (lambda c: c["layers"][0].update(type="conv"), "mixer type"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=10), "rot"),
    (lambda c: c.update(loop={"start": 1, "stop": 5, "times": 2}), "loop"),
    (lambda c: c.update(loop={"start": 0, "stop": 1, "times": 0}), "loop"),
    (lambda c: c["layers"][0].update(mlp={"kind": "gated", "ff": 8}), "feed-forward kind"),
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["layers"][1]["mixer"].pop("kv_rank"), "kv_rank"),
])
def test_faults_name_their_key(change, key):
    import copy
    c = copy.deepcopy(config([ATT, LAT]))
    change(c)
    with pytest.raises(ConfigError, match=key):
        config_from_dict(c)


def test_a_window_that_keeps_first_keys_keeps_their_pages():
    page = 4
    needs = [PagedKV(1, 8, 6, keep_first=5), PagedKV(1, 8, 6), PagedKV(1, 8, 0)]
    cm = CacheManager(needs, [None] * 3, page, 64, 2, torch.float32, "cpu")
    assert len(cm.paged_keys) == 3                                   # kept keys make a group of their own
    cm.add(1)
    total = 0
    for step in (3, 1, 7, 1, 1, 20, 2, 1):
        assert cm.reserve(1, total + step)
        total += step
        cm.commit(1, total)
        tables = [cm.block_table(1, g, np.full((64,), -1, dtype=np.int32)) for g in range(3)]
        first_key = total - 6 + 1                                    # the next token reads keys from here on
        for blk in range(-(-total // page)):
            behind = (blk + 1) * page <= first_key
            assert (tables[0][blk] >= 0) == (not behind or blk * page < 5), (total, blk)     # pages of keys 0..4 never go back
            assert (tables[1][blk] >= 0) == (not behind), (total, blk)
            assert tables[2][blk] >= 0
    assert cm.free_pages(0) == 64 - sum(1 for p in tables[0] if p >= 0)
    # the most pages a lone request holds at any time: the kept ones beside the window and one portion
    assert cm.pages_for(0, 1000, 8) == cm.pages_for(1, 1000, 8) + 2 and cm.pages_for(0, 3, 8) == 1
    cm.release(1)
    assert all(cm.free_pages(g) == 64 for g in range(3)) and cm.live == 0
