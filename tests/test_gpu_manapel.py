"""Manapel on the GPU: each mechanism's kernels alone against the plain implementation's functions, then the engine
under every way of cutting the work, pages and slots used again, planted far keys at page borders, long decoding, and
greedy generation through the entry point and the trace program."""
import json
import os

import numpy as np
import pytest
import torch

import plain_manapel as plain
import traces
from manapel_util import BLOCKS, CONFIGS, make_folder, plain_logits, requests

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 2e-4, "bfloat16": 3e-2}
SELF_TOL = {"float32": 4e-5, "bfloat16": 1.5e-2}


def K():
    from hfcpu_b200 import kernels
    return kernels


def dev(a, dtype=torch.float32):
    return torch.as_tensor(np.asarray(a), dtype=torch.float64).to(dtype).to(DEV).contiguous()


def rel(a, b):
    b = torch.as_tensor(np.asarray(b), dtype=torch.float64)
    return float((a.double().cpu() - b).abs().max() / b.abs().max().clamp_min(1e-30))


def rng(seed):
    return np.random.default_rng(seed)


# ---- each mechanism alone ---------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("E", [40, 72, 1000])
def test_dynamic_tanh_forms(dtype, E):
    r = rng(E)
    dt = DT[dtype]
    W = {}
    for n in ("a", "b"):
        W[n], W[n + ".b"], W[n + ".alpha"] = (dev(x, dt).double().cpu().numpy() for x in
                                                (1 + 0.3 * r.standard_normal(E), 0.2 * r.standard_normal(E), np.asarray(0.4 + r.random())))
    P = {n: (dev(W[n + ".alpha"], dt).reshape(1), dev(W[n], dt), dev(W[n + ".b"], dt)) for n in ("a", "b")}
    x = 3 * r.standard_normal((37, E))
    xd = dev(x)
    out = torch.empty(37, E, dtype=dt, device=DEV)
    K().dyt(xd, P["a"], out)
    assert rel(out, plain.dynamic_tanh(xd.double().cpu().numpy(), W, "a")) < (2e-6 if dtype == "float32" else 5e-3)
    rows = torch.tensor([36, 0, 5, 5], dtype=torch.int32, device=DEV)
    out4 = torch.empty(4, E, dtype=dt, device=DEV)
    K().dyt(xd, P["a"], out4, rows)
    assert torch.equal(out4, out[rows.long()])
    # a sublayer's output through its norm into the stream, and the next norm of the new stream, in one pass
    y = dev(2 * r.standard_normal((37, E)))
    res = xd.clone()
    nxt = torch.empty(37, E, dtype=dt, device=DEV)
    K().dyt_residual(y, P["b"], res, P["a"], nxt)
    want = xd.double().cpu().numpy() + plain.dynamic_tanh(y.double().cpu().numpy(), W, "b")
    assert rel(res, want) < 2e-6
    assert rel(nxt, plain.dynamic_tanh(res.double().cpu().numpy(), W, "a")) < (2e-6 if dtype == "float32" else 5e-3)
    res2 = xd.clone()
    K().dyt_residual(y, P["b"], res2)
    assert torch.equal(res, res2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("geom", [(6, 3, 24, 40, 8), (4, 4, 16, 16, 16), (2, 1, 20, 12, 4), (8, 2, 64, 64, 32), (3, 0, 48, 48, 0),
                                  (2, 2, 256, 128, 256)])
def test_rotation_unit_rms_and_cache_write(dtype, geom):
    """Queries and keys rotated over their first dimensions only, then divided by their root mean square; values as they
    are; positions include the first ones (no rotation at 0) and far ones; tokens without a slot are not cached."""
    H, G, d, dv, n_rot = geom
    dt, eps, T, bs, pages = DT[dtype], 1e-3, 9, 4, 7
    r = rng(sum(geom))
    C = H * d + G * (d + dv)
    a, w, b = dev(r.standard_normal((T, 56)), dt), dev(0.3 * r.standard_normal((C, 56)), dt), dev(r.standard_normal(C), dt)
    positions = torch.tensor([0, 1, 2, 3, 500, 501, 63, 64, 4095], dtype=torch.int32, device=DEV)
    slots = torch.tensor([0, 5, 6, 7, -1, 27, 8, 9, 1], dtype=torch.int32, device=DEV)
    rot = {"dims": n_rot, "base": 300.0}
    cos_sin = None
    if n_rot:
        f = 300.0 ** (-2.0 * np.arange(n_rot // 2) / n_rot)
        ang = np.arange(4096)[:, None] * f[None, :]
        cos_sin = dev(np.stack([np.cos(ang), np.sin(ang)], -1))
    q = torch.zeros(T, H * d, dtype=dt, device=DEV)
    kc = torch.zeros(pages, bs, max(G, 1), d, dtype=dt, device=DEV)
    vc = torch.zeros(pages, bs, max(G, 1), dv, dtype=dt, device=DEV)
    buf = torch.empty(T, C, dtype=torch.float32, device=DEV)
    K().linear_rope_norm_kv(a, w, b, buf, cos_sin, n_rot, positions, slots if G else None, q, kc[:, :, :G], vc[:, :, :G], H, G, d, dv, eps) \
        if G else K().linear_rope_norm_kv(a, w, b, buf, cos_sin, n_rot, positions, None, q, None, None, H, 0, d, dv, eps)
    row = a.double().cpu().numpy() @ w.double().cpu().numpy().T + b.double().cpu().numpy()
    pos = positions.cpu().numpy()
    tol = 3e-6 if dtype == "float32" else 8e-3
    want_q = plain.unit_rms(plain.rotate_half(row[:, :H * d].reshape(T, H, d), pos, rot), eps)
    assert rel(q.view(T, H, d), want_q) < tol
    if G:
        want_k = plain.unit_rms(plain.rotate_half(row[:, H * d:(H + G) * d].reshape(T, G, d), pos, rot), eps)
        want_v = row[:, (H + G) * d:].reshape(T, G, dv)
        kf, vf = kc.view(-1, G, d), vc.view(-1, G, dv)
        for t, s in enumerate(slots.tolist()):
            if s >= 0:
                assert rel(kf[s], want_k[t]) < tol and rel(vf[s], want_v[t]) < tol
        untouched = [s for s in range(pages * bs) if s not in slots.tolist()]
        assert float(kf[untouched].abs().max()) == 0 and float(vf[untouched].abs().max()) == 0
    K().check_device_errors()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("geom", [(5, 7, 3, 40), (130, 12, 2, 192), (64, 40, 40, 72), (3, 2, 1, 1000)])
def test_router_top_k_and_softmax_over_the_chosen(dtype, geom):
    T, E, top, Kd = geom
    r = rng(T + E)
    dt = DT[dtype]
    h, w, b = dev(r.standard_normal((T, Kd)), dt), dev(r.standard_normal((E, Kd)), dt), dev(2 * r.standard_normal(E), dt)
    ids = torch.empty(T, top, dtype=torch.int32, device=DEV)
    wts = torch.empty(T, top, dtype=torch.float32, device=DEV)
    K().moe_route(h, w, b, top, ids, wts, torch.empty(T, E, dtype=torch.float32, device=DEV))
    W = {"m.router": w.double().cpu().numpy(), "m.router.b": b.double().cpu().numpy()}
    want_ids, want_w = plain.route(h.double().cpu().numpy(), W, "m", top)
    assert np.array_equal(ids.cpu().numpy(), want_ids)
    assert rel(wts, want_w) < 1e-5 and float((wts.sum(-1) - 1).abs().max()) < 1e-6


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("geom", [(1, 5, 1, 72, 40, 0), (70, 5, 3, 72, 24, 56), (300, 16, 4, 256, 64, 128), (9, 2, 2, 40, 16, 8),
                                  (200, 3, 1, 64, 200, 0)])
def test_routed_experts_part(dtype, geom):
    """The feed-forward part as the engine runs it (router, grouping on the device, grouped products, weighted sum, shared
    expert) against a loop over tokens and their experts."""
    from types import SimpleNamespace
    from hfcpu_b200.parts import make_part
    from hfcpu_b200.config import PartSpec
    from hfcpu_b200.engine.step import Workspace
    T, E, top, width, ff, shared = geom
    r = rng(sum(geom))
    dt = DT[dtype]
    part = make_part("ffn", PartSpec("moe", {"hidden_size": width, "experts": E, "top": top, "expert_size": ff, "activation": "relu2",
                                             "router_bias": True, "shared_size": shared, "prefix": "m"}))
    tensors = {s.name: dev(r.standard_normal(s.shape) * (2.0 if "router" in s.name else 0.2), dt) for s in part.tensor_specs()}
    part.bind(tensors, dt, torch.device(DEV))
    ws = Workspace(torch.device(DEV))
    ctx = SimpleNamespace(buf=ws.get, run_dtype=dt)
    xn = dev(r.standard_normal((T, width)), dt)
    out = torch.full((T, width), 7.0, dtype=torch.float32, device=DEV)
    part.forward(ctx, xn, out, accumulate=False)
    W = {k: v.double().cpu().numpy() for k, v in tensors.items()}
    mlp = {"router": {"top": top}, "shared": {"ff": shared} if shared else None}
    want = plain.moe_ff(xn.double().cpu().numpy(), W, "m", mlp)
    assert rel(out, want) < (2e-5 if dtype == "float32" else 2e-2)
    # the same tokens in another order and company: every token's row is the same (to the bit where no tensor-core
    # product changes its tiling with the number of rows)
    perm = torch.randperm(T, device=DEV)
    more = torch.cat([xn[perm], xn[:3]]).contiguous()
    out2 = torch.empty(more.shape[0], width, dtype=torch.float32, device=DEV)
    part.forward(ctx, more, out2, accumulate=False)
    if dtype == "float32":
        assert torch.equal(out2[:T], out[perm])
    else:
        assert rel(out2[:T], out[perm].double().cpu().numpy()) < 1e-2
    K().check_device_errors()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", [(5, 72, 100), (130, 256, 512), (1, 40, 24)])
def test_gated_relu_feed_forward(dtype, shape):
    from types import SimpleNamespace
    from hfcpu_b200.parts import make_part
    from hfcpu_b200.config import PartSpec
    from hfcpu_b200.engine.step import Workspace
    T, width, ff = shape
    r = rng(sum(shape))
    dt = DT[dtype]
    part = make_part("ffn", PartSpec("gated", {"hidden_size": width, "intermediate_size": ff, "prefix": "m", "activation": "relu",
                                               "names": {"gate": "gate", "up": "up", "down": "down"}}))
    tensors = {s.name: dev(0.3 * r.standard_normal(s.shape), dt) for s in part.tensor_specs()}
    part.bind(tensors, dt, torch.device(DEV))
    ctx = SimpleNamespace(buf=Workspace(torch.device(DEV)).get, run_dtype=dt)
    xn = dev(r.standard_normal((T, width)), dt)
    out = torch.full((T, width), -3.0, dtype=torch.float32, device=DEV)
    part.forward(ctx, xn, out, accumulate=False)
    want = plain.dense_ff(xn.double().cpu().numpy(), {k: v.double().cpu().numpy() for k, v in tensors.items()}, "m")
    assert rel(out, want) < (2e-5 if dtype == "float32" else 2e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_with_value_heads_of_another_size(dtype):
    """Keys of 24, values of 40 dimensions, a given factor on the scores, scattered pages; one far key, at a page's last
    slot, carries most of the weight for the last query."""
    from types import SimpleNamespace
    H, G, d, dv, bs, n, scale = 6, 3, 24, 40, 8, 203, 0.6
    dt = DT[dtype]
    r = rng(3)
    k, v = r.standard_normal((n, G, d)), r.standard_normal((n, G, dv))
    q = r.standard_normal((2, H, d))                     # the queries of positions n-2 and n-1
    far = 47                                             # last slot of its page
    k[far] = 2.5
    q[1] = 2.5
    pages = (n + bs - 1) // bs
    perm = torch.randperm(pages + 3).tolist()[:pages]
    kc = torch.zeros(pages + 3, bs, G, d, dtype=dt, device=DEV)
    vc = torch.zeros(pages + 3, bs, G, dv, dtype=dt, device=DEV)
    kd, vd = dev(k, dt), dev(v, dt)
    for j in range(n):
        kc[perm[j // bs], j % bs], vc[perm[j // bs], j % bs] = kd[j], vd[j]
    meta = SimpleNamespace(block_table=torch.tensor([perm], dtype=torch.int32, device=DEV), block_size=bs, max_blocks=pages)
    ctx = SimpleNamespace(token_seq=torch.zeros(2, dtype=torch.int32, device=DEV),
                          positions=torch.tensor([n - 2, n - 1], dtype=torch.int32, device=DEV))
    qd = dev(q, dt).view(2, H * d)
    out = torch.empty(2, H * dv, dtype=dt, device=DEV)
    K().paged_attention(qd, kc, vc, meta, ctx, H, G, d, 0, scale, out, dv=dv)
    kk, vv, qq = kd.double().cpu().numpy(), vd.double().cpu().numpy(), qd.double().cpu().numpy().reshape(2, H, d)
    want = np.zeros((2, H, dv))
    for t, last in enumerate((n - 2, n - 1)):
        for h in range(H):
            g = h // (H // G)
            s = kk[:last + 1, g] @ qq[t, h] * scale
            p = np.exp(s - s.max())
            want[t, h] = (p / p.sum()) @ vv[:last + 1, g]
    assert rel(out.view(2, H, dv), want) < (2e-5 if dtype == "float32" else 2e-2)
    assert rel(out.view(2, H, dv)[1, 0], vv[far, 0]) < 0.05          # the planted key took the weight


# ---- the engine -------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for i, (n, c) in enumerate(CONFIGS.items()):
        out[n] = make_folder(c, str(tmp_path_factory.mktemp(f"manapel_{n}")), 5 + i)
        out[n + "16"] = make_folder(c, str(tmp_path_factory.mktemp(f"manapel_{n}16")), 5 + i, torch.bfloat16)
    return out


LENGTHS = {"odd": [1, 19, 70, 130, 33], "wide": [3, 150, 64, 129, 260], "thin": [2, 9, 41]}
FAMILIES = {"whole": traces.whole, "tail": traces.tail_one_by_one, "portions": traces.portions, "mixed": traces.mixed}


def assert_rows(got, ref, dtype, tol, what="the plain implementation"):
    """Every row within ``tol``; in bfloat16 a few rows may rest on a close call (a router's choice between two nearly
    equal logits flips with the rounding of its input and changes the row by more than rounding does): up to 3 %."""
    keys = sorted(got, key=lambda k: (str(k[0]), k[1]))
    errs = [float((got[k].double() - ref[k[0]][k[1]].double()).abs().max() / ref[k[0]][k[1]].double().abs().max()) for k in keys]
    over = [(k, e) for k, e in zip(keys, errs) if e > tol]
    allowed = 0 if dtype == "float32" else max(1, int(0.03 * len(keys)))
    assert len(over) <= allowed, (f"{len(over)} of {len(keys)} rows differ from {what}; first: request {over[0][0][0]} "
                                  f"position {over[0][0][1]} (error {over[0][1]:.3g})")


def engine_for(folder, name, dtype, max_tokens, max_requests=4):
    import hfcpu_b200
    model = hfcpu_b200.load_model(folder, DT[dtype], DEV)
    return hfcpu_b200.Engine(model, block_size=BLOCKS[name], max_tokens=max_tokens, max_requests=max_requests, ctx_max=4096)


def check_clean(eng):
    K().check_device_errors()
    eng.cache.check()
    assert eng.cache.pages_in_use() == 0 and eng.slots.free_count == eng.max_requests


_WHOLE = {}


@pytest.mark.parametrize("family", list(FAMILIES))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_cuttings_match_plain(folders, name, dtype, family):
    """Whole prompts, a tail decoded token by token, portions down to two tokens, and mixed batches of up to four
    requests in a pool sized for the peak, so that pages and slots are used again."""
    folder = folders[name if dtype == "float32" else name + "16"]
    reqs = requests(CONFIGS[name]["vocab"], LENGTHS[name], seed=3)
    steps = FAMILIES[family](reqs)
    eng = engine_for(folder, name, dtype, traces.peak_tokens(steps, round_to=BLOCKS[name]))
    got = traces.run_in_process(eng, steps, check=eng.cache.check)
    check_clean(eng)
    ref = {r: plain_logits(folder, ids) for r, ids in reqs.items()}
    assert len(got) == sum(len(v) for v in reqs.values())
    assert_rows(got, ref, dtype, TOL[dtype])
    if family == "whole":
        _WHOLE[(name, dtype)] = got
    elif (name, dtype) in _WHOLE:
        base = _WHOLE[(name, dtype)]
        assert_rows(got, {r: torch.stack([base[(r, p)] for p in range(len(ids))]) for r, ids in reqs.items()}, dtype,
                    SELF_TOL[dtype], "the whole-prompt run")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["odd", "wide"])
def test_long_decoding(folders, name, dtype):
    """Every token a step of its own, two requests side by side, far past several pages."""
    folder = folders[name if dtype == "float32" else name + "16"]
    reqs = requests(CONFIGS[name]["vocab"], [90, 75], seed=8)
    n = max(len(v) for v in reqs.values())
    steps = []
    for p in range(n):
        entries = [{"id": r, "tokens": [ids[p]], "want": [0], "_pos": p} for r, ids in reqs.items() if p < len(ids)]
        steps.append({"step": p, "entries": entries, "end": [r for r, ids in reqs.items() if p == len(ids) - 1]})
    eng = engine_for(folder, name, dtype, 192)
    got = traces.run_in_process(eng, steps)
    check_clean(eng)
    assert_rows(got, {r: plain_logits(folder, ids) for r, ids in reqs.items()}, dtype, TOL[dtype])


def planted(cfg, dtype, tmp, seed):
    """A model whose first layer makes the token MARK's query find the token MARK's key wherever it is: feature 0 of the
    embedding is set for MARK only and drives the unrotated dimensions of every query and key head."""
    m = cfg["layers"][0]["mixer"]
    nr = (m.get("rot") or {"dims": 0})["dims"]

    def edit(W):
        W["embed"][:, 0] = 0
        W["embed"][7, 0] = 30.0
        W["l0.norm1"][0], W["l0.norm1.b"][0] = 1.0, 0.0
        for t, heads in (("q", m["heads"]), ("k", m["kv_heads"])):
            W[f"l0.mix.{t}"].view(heads, m["dim"], -1)[:, nr:, 0] = 25.0
        W["l0.mix.v"] *= 8                                 # what the found key carries weighs in the output
        W["l0.mix.o"] *= 4
    return make_folder(cfg, str(tmp), seed, DT[dtype], edit=edit)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["odd", "wide"])
def test_planted_far_key_at_page_borders(folders, tmp_path, name, dtype):
    """The marked token sits at one far position; the last token is marked too and must find it.  The position runs
    over the first tokens and both sides of page borders; the last token comes in a portion and as a single token."""
    cfg, bs = CONFIGS[name], BLOCKS[name]
    folder = planted(cfg, dtype, tmp_path, 21)
    C, W = plain.read_folder(folder)
    n = 300
    base = [int(t) for t in requests(cfg["vocab"], [n], seed=4)["r0"]]
    base = [t if t != 7 else 8 for t in base]
    tol, told = TOL[dtype], 0
    for far in (0, 1, bs - 1, bs, bs + 1, 2 * bs - 1, 5 * bs, n - 2 * bs - 1):
        ids = list(base)
        ids[far] = ids[-1] = 7
        want = plain.forward(C, W, ids)[-1]
        without = list(ids)
        without[far] = 8
        miss = plain.forward(C, W, without)[-1]
        matters = np.abs(want - miss).max() / np.abs(want).max()
        if dtype == "bfloat16":
            if matters < 0.02:                             # (with the smaller weights some places weigh too little to tell)
                continue
            tol = 0.3 * matters                            # far closer to the right answer than to the one without the key
        else:
            assert matters > 10 * tol, f"the planted key does not matter enough ({matters:.3g})"
        told += 1
        for tail in (5, 1):
            eng = engine_for(folder, name, dtype, 320, max_requests=1)
            eng.add_request("a")
            from hfcpu_b200 import StepEntry
            eng.step([StepEntry("a", ids[:n - tail], [])])
            got = eng.step([StepEntry("a", ids[n - tail:], [tail - 1])])[0].double().cpu().numpy()
            eng.finish_request("a")
            check_clean(eng)
            err = np.abs(got - want).max() / np.abs(want).max()
            assert err < tol, f"far key at {far}, last {tail} tokens in their own step: error {err:.3g}"
    assert told >= 4


def test_greedy_generation_through_the_entry_point(folders):
    import hfcpu_b200
    for name in ("odd", "wide"):
        folder = folders[name]
        sess = hfcpu_b200.Session(folder, dtype="float32", kv_block=BLOCKS[name], kv_pages=96, max_seqs=4,
                                  max_batched_tokens=48, batch=32, ctx_max=512)
        prompts = list(requests(CONFIGS[name]["vocab"], [7, 33, 1, 60], seed=2).values())
        out = sess.generate(prompts, temp=0, max_tokens=10)
        cfg, W = plain.read_folder(folder)
        for p, comps in zip(prompts, out):
            assert comps[0].tokens == plain.greedy(cfg, W, p, 10)
        assert sess.engine.cache.pages_in_use() == 0


def test_bfloat16_generation_replays_graphs(folders):
    """Steady decoding in bfloat16 goes through captured graphs (router and experts included) and repeats itself."""
    import hfcpu_b200
    sess = hfcpu_b200.Session(folders["wide16"], dtype="bfloat16", kv_block=16, kv_pages=128, max_seqs=4, ctx_max=512)
    prompts = list(requests(1032, [19, 130, 64], seed=2).values())
    a = sess.generate(prompts, temp=0, max_tokens=24)
    assert sess.engine.use_graphs and any(s[0] == "ready" for s in sess.engine._graphs.values())
    b = sess.generate(prompts, temp=0, max_tokens=24)
    assert [c[0].tokens for c in a] == [c[0].tokens for c in b] and all(len(c[0].tokens) == 24 for c in a)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_program(folders, tmp_path, dtype):
    folder = folders["odd" if dtype == "float32" else "odd16"]
    reqs = requests(300, [5, 40, 77], seed=9)
    steps = traces.mixed(reqs, max_live=2)
    got = traces.run_trace_program(folder, dtype, steps, str(tmp_path), traces.peak_tokens(steps), 300, block_size=8)
    assert_rows(got, {r: plain_logits(folder, ids) for r, ids in reqs.items()}, dtype, TOL[dtype])


def test_command_line_generates(folders):
    import subprocess
    import sys
    from conftest import ROOT
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "hfb200"), "--model", folders["wide16"], "--op", "generate",
                        "--stdin-mode", "none", "--prompt-ids", "5,17,3,900", "--temp", "0", "--max-tokens", "6", "--ctx-max", "256",
                        "--kv-pages", "32"],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert "stop=length" in r.stdout or "length" in r.stdout
