"""Manapel on a machine without a GPU: configuration and plan, and the engine's host side (batching, shared caches,
pages) with the torch stand-in for the CUDA library against the plain implementation."""
import copy

import pytest
import torch

import traces
from manapel_util import BLOCKS, CONFIGS, make_folder, plain_logits, requests


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {n: make_folder(c, str(tmp_path_factory.mktemp(f"manapel_{n}")), 5 + i) for i, (n, c) in enumerate(CONFIGS.items())}


def test_plan_follows_the_layer_list():
    from hfcpu_b200.config import config_from_dict, ManapelConfig
    cfg = config_from_dict(CONFIGS["odd"])
    assert isinstance(cfg, ManapelConfig)
    plan = cfg.plan()
    assert [e.cache_of for e in plan.schedule] == [None, 0, None, 0]
    assert [l.ffn.kind if l.ffn else None for l in plan.layers] == ["moe", None, "gated", "moe"]
    assert plan.layers[0].mixer.args["own_kv"] and not plan.layers[3].mixer.args["own_kv"]
    assert plan.layers[0].mixer.args["v_head_dim"] == 40 and plan.layers[2].mixer.args["scale"] == 1.0
    assert len(plan.positions) == 2                      # two different rotations, the equal ones share a table
    assert plan.head.args["scale"] == 1.7
    again = config_from_dict(cfg.to_dict())
    assert again.to_dict() == cfg.to_dict()


def test_tensor_names():
    from hfcpu_b200.config import config_from_dict
    from hfcpu_b200.models import build_model_specs
    specs = {s.name: s for s in build_model_specs(config_from_dict(CONFIGS["odd"]))}
    assert specs["l0.mix.v"].shape == (3 * 40, 72) and specs["l0.mix.o"].shape == (72, 6 * 40) and specs["l0.mix.k.b"].shape == (72,)
    assert "l1.mix.k" not in specs and "l3.mix.v.b" not in specs and "l1.mix.q.b" in specs
    assert specs["l0.norm1.alpha"].shape == () and specs["final.norm.b"].shape == (72,)
    assert specs["l1.norm2"].optional and not specs["l0.norm2"].optional       # layer 1 has no feed-forward
    assert "l1.mlp.up" not in specs and specs["l2.mlp.gate"].shape == (100, 72)
    assert specs["l3.mlp.e4.down"].shape == (72, 24) and specs["l3.mlp.shared.up"].shape == (56, 72) and "l0.mlp.shared.up" not in specs
    assert specs["l3.mlp.router.b"].shape == (5,) and specs["head"].shape == (300, 72)


@pytest.mark.parametrize("edit,word", [
    (lambda c: c["layers"][1]["mixer"].update(kv_from=2), "kv_from"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=1), "kv_from"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=6), "top"),
    (lambda c: c["layers"][0].update(type="recurrent"), "not supported"),
    (lambda c: c["layers"][2]["mlp"].update(kind="glu"), "not supported"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=26), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"].update(heads=7), "geometry"),
    (lambda c: c.pop("width"), "width"),
])
def test_bad_configurations_are_refused(edit, word):
    from hfcpu_b200.config import ConfigError, config_from_dict
    c = copy.deepcopy(CONFIGS["odd"])
    edit(c)
    with pytest.raises(ConfigError, match=word):
        config_from_dict(c)


@pytest.mark.parametrize("family", ["whole", "portions", "mixed"])
@pytest.mark.parametrize("name", ["odd", "thin"])
def test_engine_host_side_matches_plain(emu, folders, name, family):
    import hfcpu_b200
    reqs = requests(CONFIGS[name]["vocab"], [1, 9, 37, 20], seed=1)
    steps = {"whole": traces.whole, "portions": traces.portions, "mixed": traces.mixed}[family](reqs)
    model = hfcpu_b200.load_model(folders[name], torch.float32, "cpu")
    eng = hfcpu_b200.Engine(model, block_size=BLOCKS[name], max_tokens=traces.peak_tokens(steps), max_requests=4, ctx_max=256)
    got = traces.run_in_process(eng, steps, check=eng.cache.check)
    assert eng.cache.pages_in_use() == 0
    ref = {r: plain_logits(folders[name], ids) for r, ids in reqs.items()}
    bad = traces.first_bad(got, ref, 1e-4)
    assert bad is None, f"first wrong row: request {bad[0]} position {bad[1]} (error {bad[2]:.3g})"


def test_shared_cache_entries_own_no_pages(emu, folders):
    import hfcpu_b200
    model = hfcpu_b200.load_model(folders["odd"], torch.float32, "cpu")
    eng = hfcpu_b200.Engine(model, block_size=8, max_tokens=64, max_requests=2, ctx_max=64)
    # layers 0 and 2 keep keys and values (of different geometry: two groups), layers 1 and 3 read layer 0's
    assert sorted(e for g in eng.cache.groups for e in g.entries) == [0, 2]
    assert eng.cache.entry_cache(1) is None and eng.cache.entry_cache(3) is None
    g0 = next(g for g in eng.cache.groups if 0 in g.entries)
    assert g0.keys.shape[-1] == 24 and g0.values.shape[-1] == 40
