"""Peludra on a machine without a GPU: configuration and plan, the pieces that are computed on the host (rotation table,
page bookkeeping of chunked and windowed groups), and the engine's host side (batching, the previous token carried
from step to step, values handed from layer to layer) with the torch stand-in for the CUDA library against the plain
implementation."""
import copy

import numpy as np
import pytest
import torch

import plain_peludra as plain
import traces
from peludra_util import BLOCKS, CONFIGS, make_folder, plain_logits, requests


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {n: make_folder(c, str(tmp_path_factory.mktemp(f"peludra_{n}")), 5 + i) for i, (n, c) in enumerate(CONFIGS.items())}


def test_plan_follows_the_layer_list():
    from hfcpu_b200.config import config_from_dict, PeludraConfig
    cfg = config_from_dict(CONFIGS["odd"])
    assert isinstance(cfg, PeludraConfig)
    plan = cfg.plan()
    assert [l.mixer.kind for l in plan.layers] == ["paged_attention", "latent_attention", "paged_attention", "paged_attention",
                                                   "latent_attention", "paged_attention"]
    assert [l.mixer.args.get("v_mix") for l in plan.layers] == ["first", None, None, "later", None, "later"]
    assert [l.mixer.args.get("chunk") for l in plan.layers] == [12, None, 50, 7, None, 30]
    assert [l.mixer.args.get("window") for l in plan.layers] == [0, 9, 0, 0, 33, 0]
    assert [l.ffn.kind if l.ffn else None for l in plan.layers] == ["mlp", None, "mlp", "mlp", "mlp", None]
    assert all(l.norm1.args["offset"] == 1.0 for l in plan.layers) and plan.final_norm.args["offset"] == 1.0
    assert plan.layers[1].norm2 is None and plan.layers[0].norm2 is not None
    assert len(plan.positions) == 2 and all(p.args["pairing"] == "interleaved" for p in plan.positions.values())
    assert plan.embedding.kind == "hashed_pair_embedding" and plan.embedding.args["buckets"] == 53
    again = config_from_dict(cfg.to_dict())
    assert again.to_dict() == cfg.to_dict()
    thin = config_from_dict(CONFIGS["thin"]).plan()
    assert thin.embedding.args["pair_tensor"] is None and len(thin.positions) == 2
    twice = copy.deepcopy(CONFIGS["odd"])
    twice["layers"].append(copy.deepcopy(twice["layers"][1]))
    assert len(config_from_dict(twice).plan().positions) == 2                           # equal rotations share a table


def test_tensor_names():
    from hfcpu_b200.config import config_from_dict
    from hfcpu_b200.models import build_model_specs
    specs = {s.name: s for s in build_model_specs(config_from_dict(CONFIGS["odd"]))}
    assert specs["embed"].shape == (211, 72) and specs["bigram"].shape == (54, 72)
    assert specs["l0.mix.q"].shape == (144, 72) and specs["l0.mix.k"].shape == (72, 72) and specs["l0.mix.v"].shape == (120, 72)
    assert specs["l0.mix.o"].shape == (72, 240) and specs["l0.mix.q.norm"].shape == (24,) and specs["l0.mix.k.norm"].shape == (24,)
    assert specs["l0.mix.vmix"].shape == () and specs["l3.mix.vmix"].shape == () and "l2.mix.vmix" not in specs
    assert specs["l1.mix.dq"].shape == (40, 72) and specs["l1.mix.dq.norm"].shape == (40,) and specs["l1.mix.uq"].shape == (72, 40)
    assert specs["l1.mix.dkv"].shape == (32, 72) and specs["l1.mix.dkv.norm"].shape == (24,)
    assert specs["l1.mix.uk"].shape == (48, 24) and specs["l1.mix.uv"].shape == (72, 24) and specs["l1.mix.o"].shape == (72, 72)
    assert "l1.norm2" not in specs and "l1.mlp.up" not in specs and specs["l0.mlp.up"].shape == (100, 72)
    assert specs["final.norm"].shape == (72,) and specs["head"].shape == (211, 72)
    assert "bigram" not in {s.name for s in build_model_specs(config_from_dict(CONFIGS["thin"]))}


@pytest.mark.parametrize("edit,word", [
    (lambda c: c["layers"][0].update(type="recurrent"), "not supported"),
    (lambda c: c["layers"][0]["mlp"].update(kind="moe"), "not supported"),
    (lambda c: c["layers"][0]["mixer"].update(heads=7), "geometry"),
    (lambda c: c["layers"][3]["mixer"].update(vdim=24), "v_mix"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=6), "rot.dims"),
    (lambda c: c["layers"][1]["mixer"].update(rot_dim=7), "even"),
    (lambda c: c["layers"][1]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][4]["mixer"]["rot"]["scaling"].pop("slow"), "slow"),
    (lambda c: c["embedding"]["bigram"].pop("mul_cur"), "mul_cur"),
    (lambda c: c.pop("width"), "width"),
])
def test_bad_configurations_are_refused(edit, word):
    from hfcpu_b200.config import ConfigError, config_from_dict
    c = copy.deepcopy(CONFIGS["odd"])
    edit(c)
    with pytest.raises(ConfigError, match=word):
        config_from_dict(c)


@pytest.mark.parametrize("rot", [{"dims": 8, "base": 500.0}, {"dims": 32, "base": 15000.0},
                                 {"dims": 12, "base": 3000.0, "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 2.0}},
                                 {"dims": 64, "base": 1e6, "scaling": {"factor": 40.0, "original": 4096, "fast": 32.0, "slow": 1.0}},
                                 {"dims": 6, "base": 10.0, "scaling": {"factor": 2.0, "original": 5, "fast": 0.5, "slow": 0.25}}])
def test_rotation_table_matches_the_plain_frequencies(rot):
    from hfcpu_b200.config import PartSpec
    from hfcpu_b200.parts import make_part
    part = make_part("position", PartSpec("rotary", {"head_dim": rot["dims"], "n_rot": rot["dims"], "theta": rot["base"],
                                                     "pairing": "interleaved", "scaling": rot.get("scaling")}))
    part.prepare(700, torch.device("cpu"))
    f, m = plain.rotary_frequencies(rot)
    ang = np.arange(700)[:, None] * f[None, :]
    assert np.abs(part.cos_sin[..., 0].numpy() - np.cos(ang) * m).max() < 2e-7 * max(m, 1)
    assert np.abs(part.cos_sin[..., 1].numpy() - np.sin(ang) * m).max() < 2e-7 * max(m, 1)
    if "scaling" in rot:
        plain_f, _ = plain.rotary_frequencies({"dims": rot["dims"], "base": rot["base"]})
        assert f[0] == plain_f[0] or rot["dims"] == 6                        # the fastest pair keeps its frequency
        assert abs(f[-1] - plain_f[-1] / rot["scaling"]["factor"]) < 1e-12 * plain_f[-1] + 1e-18   # the slowest is stretched


def test_pages_of_passed_chunks_and_windows_go_back(emu, folders):
    import hfcpu_b200
    model = hfcpu_b200.load_model(folders["odd"], torch.float32, "cpu")
    eng = hfcpu_b200.Engine(model, block_size=8, max_tokens=128, max_requests=2, ctx_max=128)
    by_spec = {(g.spec.chunk, g.spec.window): g for g in eng.cache.groups}
    assert sorted(by_spec) == [(0, 9), (0, 33), (7, 0), (12, 0), (30, 0), (50, 0)]
    assert by_spec[(0, 9)].values is None and by_spec[(0, 9)].keys.shape[-2:] == (1, 32)     # a latent row, no values
    assert by_spec[(12, 0)].keys.shape[-1] == 24 and by_spec[(12, 0)].values.shape[-1] == 40
    eng.add_request("a")
    ids = requests(211, [100], seed=1)["r0"]
    eng.step([hfcpu_b200.StepEntry("a", ids[:61], [])])
    held = lambda g: [b for b, p in enumerate(g.tables["a"]) if p >= 0]
    # 61 tokens held; the next query is at 61: chunk 12 -> first key 60, chunk 50 -> 50, window 9 -> 53, window 33 -> 29
    assert held(by_spec[(12, 0)]) == [7] and held(by_spec[(50, 0)]) == [6, 7] and held(by_spec[(7, 0)]) == [7]
    assert held(by_spec[(0, 9)]) == [6, 7] and held(by_spec[(0, 33)]) == [3, 4, 5, 6, 7]
    eng.step([hfcpu_b200.StepEntry("a", ids[61:100], [38])])
    assert held(by_spec[(50, 0)]) == [12] and held(by_spec[(12, 0)]) == [12]
    eng.cache.check()
    eng.finish_request("a")
    assert eng.cache.pages_in_use() == 0


def test_previous_token_is_carried_in_the_request_slot(emu, folders):
    """The pair term of a step's first token comes from the request's state; a slot that is handed out again starts empty."""
    import hfcpu_b200
    from hfcpu_b200.models import EMBEDDING_STATE
    model = hfcpu_b200.load_model(folders["odd"], torch.float32, "cpu")
    eng = hfcpu_b200.Engine(model, block_size=8, max_tokens=128, max_requests=2, ctx_max=64)
    state = eng.slots.entry_state(EMBEDDING_STATE)
    assert state.dtype == torch.int32 and state.shape == (2,)
    assert not eng.can_fork                                   # a request cannot start on another's pages: its state is its own
    cfg, W = plain.read_folder(folders["odd"])
    ids = requests(211, [9, 6], seed=3)
    ref = {r: plain_logits(folders["odd"], v) for r, v in ids.items()}
    eng.add_request("r0"), eng.add_request("r1")
    a = eng.step([hfcpu_b200.StepEntry("r0", ids["r0"][:4], [3]), hfcpu_b200.StepEntry("r1", ids["r1"][:1], [0])]).clone()
    assert sorted(state.tolist()) == sorted([ids["r0"][3] + 1, ids["r1"][0] + 1])
    b = eng.step([hfcpu_b200.StepEntry("r1", ids["r1"][1:], [4]), hfcpu_b200.StepEntry("r0", ids["r0"][4:5], [0])]).clone()
    for got, (r, p) in ((a[0], ("r0", 3)), (a[1], ("r1", 0)), (b[0], ("r1", 5)), (b[1], ("r0", 4))):
        assert float((got.double() - ref[r][p]).abs().max() / ref[r][p].abs().max()) < 1e-4
    eng.finish_request("r1")
    eng.add_request("again")                                   # takes r1's slot
    c = eng.step([hfcpu_b200.StepEntry("again", ids["r1"][:3], [2])])[0]
    assert float((c.double() - ref["r1"][2]).abs().max() / ref["r1"][2].abs().max()) < 1e-4


@pytest.mark.parametrize("family", ["whole", "portions", "mixed"])
@pytest.mark.parametrize("name", ["odd", "thin"])
def test_engine_host_side_matches_plain(emu, folders, name, family):
    import hfcpu_b200
    reqs = requests(CONFIGS[name]["vocab"], [1, 9, 37, 20, 2], seed=1)
    steps = {"whole": traces.whole, "portions": traces.portions, "mixed": traces.mixed}[family](reqs)
    model = hfcpu_b200.load_model(folders[name], torch.float32, "cpu")
    eng = hfcpu_b200.Engine(model, block_size=BLOCKS[name], max_tokens=traces.peak_tokens(steps), max_requests=4, ctx_max=256)
    got = traces.run_in_process(eng, steps, check=eng.cache.check)
    assert eng.cache.pages_in_use() == 0 and eng.slots.free_count == 4
    ref = {r: plain_logits(folders[name], ids) for r, ids in reqs.items()}
    bad = traces.first_bad(got, ref, 1e-4)
    assert bad is None, f"first wrong row: request {bad[0]} position {bad[1]} (error {bad[2]:.3g})"


def test_plain_masks():
    w, c = plain.window_mask(9, 3), plain.chunk_mask(9, 4)
    assert w[5].tolist() == [False, False, False, True, True, True, False, False, False]
    assert c[5].tolist() == [False, False, False, False, True, True, False, False, False]
    assert c[4].tolist() == [False] * 4 + [True] + [False] * 4 and c[3].tolist() == [True] * 4 + [False] * 5
    assert plain.bigram_rows([5, 6, 5], {"buckets": 7, "mul_prev": 3, "mul_cur": 2}) == [7, (15 + 12) % 7, (18 + 10) % 7]
