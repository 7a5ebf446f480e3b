"""Peludra on the GPU: each mechanism's kernels alone against the plain implementation's functions, then the engine under
every way of cutting the work, pages and slots used again, keys just inside and just outside every window and chunk in
prompts and in decoding, long decoding, and greedy generation through the entry point and the trace program."""
import copy
import os
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_peludra as plain
import traces
from peludra_util import BLOCKS, CONFIGS, att, lat, layer, make_folder, model, plain_logits, requests

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 2e-4, "bfloat16": 3e-2}
SELF_TOL = {"float32": 4e-5, "bfloat16": 1.5e-2}
KTOL = {"float32": 3e-6, "bfloat16": 8e-3}          # one kernel's output against float64


def K():
    from hfcpu_b200 import kernels
    return kernels


def dev(a, dtype=torch.float32):
    return torch.as_tensor(np.asarray(a), dtype=torch.float64).to(dtype).to(DEV).contiguous()


def f64(t):
    return t.double().cpu().numpy()


def rel(a, b):
    b = torch.as_tensor(np.asarray(b), dtype=torch.float64)
    return float((a.double().cpu() - b).abs().max() / b.abs().max().clamp_min(1e-30))


def rng(seed):
    return np.random.default_rng(seed)


def table(rot, n):
    f, m = plain.rotary_frequencies(rot)
    ang = np.arange(n)[:, None] * f[None, :]
    return dev(np.stack([np.cos(ang) * m, np.sin(ang) * m], -1))


# ---- each mechanism alone ---------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("pair", [(53, 31, 7), (1, 5, 3), (499, 100003, 99991), None])
def test_embedding_with_scale_and_pair_term(dtype, pair):
    """Three steps over two slots: a first step with a whole prompt beside a single first token, a step of single tokens,
    and a request that takes over a freed slot and must start without a previous token."""
    dt, V, E, scale = DT[dtype], 300, 72, 2.5
    r = rng(V)
    W = {"embed": f64(dev(r.standard_normal((V, E)), dt))}
    cfg = {"embedding": {"scale": scale}}
    pt = None
    if pair:
        W["bigram"] = f64(dev(r.standard_normal((pair[0] + 1, E)), dt))
        cfg["embedding"]["bigram"] = dict(zip(("buckets", "mul_prev", "mul_cur"), pair))
        pt = dev(W["bigram"], dt)
    tab = dev(W["embed"], dt)
    state = torch.zeros(3, dtype=torch.int32, device=DEV)
    a, b, c = [5, 299, 0, 17, 17], [200, 3], [9, 8, 7]

    def step(parts):                          # parts: [(slot, tokens)]
        ids = torch.tensor([t for _, ts in parts for t in ts], dtype=torch.int32, device=DEV)
        cu = np.cumsum([0] + [len(ts) for _, ts in parts])
        ctx = SimpleNamespace(token_seq=torch.tensor(np.repeat(np.arange(len(parts)), [len(ts) for _, ts in parts]), dtype=torch.int32, device=DEV),
                              cu_tokens=torch.tensor(cu, dtype=torch.int32, device=DEV),
                              seq_slots=torch.tensor([s for s, _ in parts], dtype=torch.int32, device=DEV))
        out = torch.empty(len(ids), E, dtype=torch.float32, device=DEV)
        K().embed_pair(ids, tab, scale, pt, pair[0] if pair else 0, pair[1] if pair else 0, pair[2] if pair else 0, ctx,
                       state if pair else None, out)
        return out
    wa, wb, wc = (plain.embed(cfg, W, x) for x in (a, b, c))
    o1 = step([(2, a[:4]), (0, b[:1])])
    assert rel(o1[:4], wa[:4]) < 1e-6 and rel(o1[4:], wb[:1]) < 1e-6
    o2 = step([(0, b[1:]), (2, a[4:])])
    assert rel(o2[:1], wb[1:]) < 1e-6 and rel(o2[1:], wa[4:]) < 1e-6
    if pair:
        assert state.tolist() == [b[-1] + 1, 0, a[-1] + 1]
        state[0] = 0                                        # the slot is handed out again
    o3 = step([(0, c)])
    assert rel(o3, wc) < 1e-6
    K().check_device_errors()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_norm_with_weight_stored_around_zero(dtype):
    from hfcpu_b200.config import PartSpec
    from hfcpu_b200.parts import make_part
    E, dt = 200, DT[dtype]
    r = rng(1)
    norm = make_part("norm", PartSpec("rmsnorm", {"size": E, "eps": 3e-5, "tensor": "n", "offset": 1.0}))
    assert norm.tensor_specs()[0].init == "normal"
    w = dev(0.4 * r.standard_normal(E), dt)
    norm.bind({"n": w}, dt, torch.device(DEV))
    x = dev(3 * r.standard_normal((70, E)))
    out = torch.empty(70, E, dtype=dt, device=DEV)
    norm.forward(x, out)
    assert rel(out, plain.norm_one_plus(f64(x), f64(w), 3e-5)) < KTOL[dtype]
    assert norm.fused_args()[0].dtype == torch.float32            # 1 + w does not fit the storage type


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("geom", [(6, 3, 24, 40), (5, 5, 48, 56), (2, 1, 20, 12), (8, 2, 64, 64), (4, 1, 128, 128), (1, 1, 256, 8)])
def test_head_norms_with_weights_and_value_mixing(dtype, geom):
    """The q|k|v tail without rotation: queries and keys normed per head with a weight shared by the heads; the first mixing
    layer leaves its values behind, a later one stores the mixture."""
    H, G, d, dv = geom
    dt, eps, T, bs, pages, lam = DT[dtype], 1e-4, 9, 4, 7, 0.37
    r = rng(sum(geom))
    C = H * d + G * (d + dv)
    a, w = dev(r.standard_normal((T, 56)), dt), dev(0.3 * r.standard_normal((C, 56)), dt)
    qw, kw = dev(0.5 + r.random(d)), dev(0.5 + r.random(d))
    positions = torch.tensor([0, 1, 2, 3, 500, 501, 63, 64, 4095], dtype=torch.int32, device=DEV)
    slots = torch.tensor([0, 5, 6, 7, 11, 27, 8, 9, 1], dtype=torch.int32, device=DEV)
    row = f64(a) @ f64(w).T
    want_q = plain.norm_plain(row[:, :H * d].reshape(T, H, d), f64(qw), eps)
    want_k = plain.norm_plain(row[:, H * d:(H + G) * d].reshape(T, G, d), f64(kw), eps)
    own_v = row[:, (H + G) * d:].reshape(T, G, dv)
    first = torch.full((T, G * dv), 9.0, dtype=torch.float32, device=DEV)
    for mode in (1, 2):
        q = torch.zeros(T, H * d, dtype=dt, device=DEV)
        kc, vc = torch.zeros(pages, bs, G, d, dtype=dt, device=DEV), torch.zeros(pages, bs, G, dv, dtype=dt, device=DEV)
        buf = torch.empty(T, C, dtype=torch.float32, device=DEV)
        if mode == 2:
            first.copy_(dev(r.standard_normal((T, G * dv))))
        given = f64(first).reshape(T, G, dv)
        K().linear_rope_norm_kv(a, w, None, buf, None, 0, positions, slots, q, kc, vc, H, G, d, dv, eps, norm_weights=(qw, kw),
                                value_mix=(first, mode, lam))
        assert rel(q.view(T, H, d), want_q) < KTOL[dtype]
        want_v = own_v if mode == 1 else (1 - lam) * own_v + lam * given
        for t, s in enumerate(slots.tolist()):
            assert rel(kc.view(-1, G, d)[s], want_k[t]) < KTOL[dtype] and rel(vc.view(-1, G, dv)[s], want_v[t]) < KTOL[dtype]
        if mode == 1:
            assert rel(first.view(T, G, dv), own_v) < 3e-6        # float32 whatever the run type
    K().check_device_errors()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("geom", [(3, 16, 8, 24, 40, 24), (4, 32, 16, 72, 112, 64), (5, 8, 12, 20, 16, 36), (1, 6, 2, 10, 12, 10),
                                  (4, 64, 32, 64, 128, 96), (2, 128, 64, 128, 1536, 512)])
def test_latent_tails_and_per_head_products(dtype, geom):
    """Down product -> two norms, rotation in pairs (2i, 2i+1), cache row; query product -> plain parts and rotated parts;
    the per-head product in both of its uses.  Positions include 0 and far ones; a token without a slot is not cached."""
    H, d, dr, dv, Qr, R = geom
    dt, eps, T, bs, pages, E = DT[dtype], 1e-5, 9, 4, 7, 56
    r = rng(sum(geom))
    rot = {"dims": dr, "base": 300.0, "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 2.0}}
    cs = table(rot, 4096)
    positions = torch.tensor([0, 1, 2, 3, 500, 501, 63, 64, 4095], dtype=torch.int32, device=DEV)
    pos = positions.cpu().numpy()
    slots = torch.tensor([0, 5, 6, 7, -1, 27, 8, 9, 1], dtype=torch.int32, device=DEV)
    a = dev(r.standard_normal((T, E)), dt)
    w_down = dev(0.3 * r.standard_normal((Qr + R + dr, E)), dt)
    qn, kn = dev(0.5 + r.random(Qr)), dev(0.5 + r.random(R))
    cq = torch.zeros(T, Qr, dtype=dt, device=DEV)
    cache = torch.zeros(pages, bs, 1, R + dr, dtype=dt, device=DEV)
    K().linear_latent_split(a, w_down, torch.empty(T, Qr + R + dr, dtype=torch.float32, device=DEV), qn, kn, eps, cs, positions,
                            slots, cq, cache, Qr, R, dr)
    row = f64(a) @ f64(w_down).T
    assert rel(cq, plain.norm_plain(row[:, :Qr], f64(qn), eps)) < KTOL[dtype]
    want_c = plain.norm_plain(row[:, Qr:Qr + R], f64(kn), eps)
    want_r = plain.rotate_interleaved(row[:, Qr + R:], pos, rot)
    flat = cache.view(-1, R + dr)
    for t, s in enumerate(slots.tolist()):
        if s >= 0:
            assert rel(flat[s, :R], want_c[t]) < KTOL[dtype] and rel(flat[s, R:], want_r[t]) < KTOL[dtype]
    untouched = [s for s in range(pages * bs) if s not in slots.tolist()]
    assert float(flat[untouched].abs().max()) == 0
    # the query product's tail
    w_uq = dev(0.3 * r.standard_normal((H * (d + dr), Qr)), dt)
    q_plain = torch.zeros(T, H * d, dtype=dt, device=DEV)
    q_att = torch.zeros(T, H * (R + dr), dtype=dt, device=DEV)
    K().linear_latent_query(cq, w_uq, torch.empty(T, H * (d + dr), dtype=torch.float32, device=DEV), cs, positions, q_plain, q_att,
                            H, d, dr, R)
    q = (f64(cq) @ f64(w_uq).T).reshape(T, H, d + dr)
    assert rel(q_plain.view(T, H, d), q[..., :d]) < KTOL[dtype]
    assert rel(q_att.view(T, H, R + dr)[..., R:], plain.rotate_interleaved(q[..., d:], pos, rot)) < KTOL[dtype]
    assert float(q_att.view(T, H, R + dr)[..., :R].abs().max()) == 0
    # a head's query carried into the latent space lands beside its rotated part; scores over cached rows are the scores
    # over expanded keys
    w_uk = dev(0.3 * r.standard_normal((H * d, R)), dt)
    ukt = w_uk.view(H, d, R).transpose(1, 2).contiguous()
    before = q_att.clone()
    K().headwise_linear(q_plain, ukt, q_att, H, d, R + dr)
    got = q_att.view(T, H, R + dr)
    assert torch.equal(got[..., R:], before.view(T, H, R + dr)[..., R:])
    want_lat = np.einsum("thd,hdr->thr", f64(q_plain).reshape(T, H, d), f64(w_uk).reshape(H, d, R))
    assert rel(got[..., :R], want_lat) < KTOL[dtype] * 2
    k_plain = (want_c @ f64(w_uk).T).reshape(T, H, d)
    s_expanded = np.einsum("thd,jhd->htj", f64(q_plain).reshape(T, H, d), k_plain)
    s_latent = np.einsum("thr,jr->htj", want_lat, want_c)
    assert np.abs(s_expanded - s_latent).max() < 1e-9 * np.abs(s_expanded).max()
    # the query product, the rotation and the per-head product behind one call (one kernel in bfloat16)
    fused = torch.zeros(T, H * (R + dr), dtype=dt, device=DEV)
    K().linear_latent_query_absorb(cq, w_uq, torch.empty(T, H * (d + dr), dtype=torch.float32, device=DEV), cs, positions, ukt,
                                   torch.empty(T, H * d, dtype=dt, device=DEV), fused, H, d, dr)
    assert rel(fused, q_att.double().cpu()) < (1e-6 if dtype == "float32" else 4e-3)
    # many tokens: every tile of the tensor-core form, tokens beyond a tile's end
    for many in (70, 130):
        xin = dev(r.standard_normal((many, H * (R + dr))), dt)
        wide = torch.zeros(many, H * dv, dtype=dt, device=DEV)
        w_uv_m = dev(0.3 * r.standard_normal((H, dv, R)), dt)
        K().headwise_linear(xin, w_uv_m, wide, H, R + dr, dv)
        assert rel(wide.view(many, H, dv), np.einsum("thr,hvr->thv", f64(xin).reshape(many, H, R + dr)[..., :R], f64(w_uv_m))) < KTOL[dtype] * 2
    # the value expansion reads the first R columns of a wider row
    w_uv = dev(0.3 * r.standard_normal((H * dv, R)), dt).view(H, dv, R)
    heads = torch.zeros(T, H * dv, dtype=dt, device=DEV)
    K().headwise_linear(q_att, w_uv, heads, H, R + dr, dv)
    assert rel(heads.view(T, H, dv), np.einsum("thr,hvr->thv", f64(got[..., :R]), f64(w_uv))) < KTOL[dtype] * 2
    K().check_device_errors()


def paged(k, v, bs, dt, extra=3, seed=0):
    """Keys [n, G, d] (and values) scattered over pages in a shuffled order; returns caches and the block table."""
    n = k.shape[0]
    pages = (n + bs - 1) // bs
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(pages + extra, generator=g).tolist()[:pages]
    kc = torch.zeros(pages + extra, bs, *k.shape[1:], dtype=dt, device=DEV)
    kd = dev(k, dt)
    vc = vd = None
    if v is not None:
        vc = torch.zeros(pages + extra, bs, *v.shape[1:], dtype=dt, device=DEV)
        vd = dev(v, dt)
    for j in range(n):
        kc[perm[j // bs], j % bs] = kd[j]
        if v is not None:
            vc[perm[j // bs], j % bs] = vd[j]
    return kc, vc, kd, vd, torch.tensor([perm], dtype=torch.int32, device=DEV), pages


def plain_attend(q, k, v, positions, lo_of, scale, H, G):
    out = np.zeros((len(positions), H, v.shape[-1]))
    for t, pos in enumerate(positions):
        lo = lo_of(pos)
        for h in range(H):
            g = h // (H // G)
            s = k[lo:pos + 1, g] @ q[t, h] * scale
            p = np.exp(s - s.max())
            out[t, h] = (p / p.sum()) @ v[lo:pos + 1, g]
    return out


MASKS = {"window": lambda size: (size, lambda pos: max(0, pos - size + 1)),
         "chunk": lambda size: (-size, lambda pos: pos // size * size)}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind,size", [("window", 44), ("window", 1), ("chunk", 208), ("chunk", 16), ("chunk", 1), ("window", 7), ("chunk", 1000),
                                       ("window", 400)])
@pytest.mark.parametrize("geom", [(6, 3, 24, 40, False), (4, 1, 96, 64, True), (3, 1, 32, 24, True), (2, 1, 576, 512, True)])
def test_edges_of_windows_and_chunks_plain_kernel(dtype, kind, size, geom):
    """One key carries a score far above the rest; it is placed just inside and just outside the mask of the last query
    (which comes in a portion of three and as a single token), and the output must follow it or ignore it."""
    H, G, d, dv, inside_keys = geom
    dt, bs, n, scale = DT[dtype], 8, 431, 0.5
    code, lo_of = MASKS[kind](size)
    last = n - 1
    lo = lo_of(last)
    # around the mask's edge, and far keys on both sides of page borders (inside or outside the mask as it falls)
    for planted in sorted({lo, lo - 1, max(lo - 2, 0), last, min(lo + 1, last), 0, bs - 1, bs, 7 * bs - 1, 7 * bs, 40 * bs - 1}):
        if planted < 0:
            continue
        r = rng(planted + size)
        k = 0.3 * r.standard_normal((n, G, d))
        q = 0.3 * r.standard_normal((3, H, d))
        if inside_keys:
            # a value is the first dv elements of its key: the mark sits in the elements behind them
            v = None
            k[planted, :, dv:] = 3.0
            q[..., dv:] = 4.0
        else:
            v = r.standard_normal((n, G, dv))
            k[planted] = 3.0
            q[:] = 12.0 / np.sqrt(d)
        kc, vc, kd, vd, bt, pages = paged(k, v, bs, dt, seed=planted)
        meta = SimpleNamespace(block_table=bt, block_size=bs, max_blocks=pages)
        kk = f64(kd)
        vv = kk[..., :dv] if inside_keys else f64(vd)
        for positions in ([n - 3, n - 2, n - 1], [n - 1]):
            qd = dev(q[-len(positions):], dt).reshape(len(positions), H * d).contiguous()
            ctx = SimpleNamespace(token_seq=torch.zeros(len(positions), dtype=torch.int32, device=DEV),
                                  positions=torch.tensor(positions, dtype=torch.int32, device=DEV), max_q_len=len(positions))
            out = torch.empty(len(positions), H * dv, dtype=dt, device=DEV)
            if inside_keys:
                K().paged_attention(qd, kc, None, meta, ctx, H, G, d, code, scale, out, dv=dv, values_in_keys=True)
            else:
                K().paged_attention(qd, kc, vc, meta, ctx, H, G, d, code, scale, out, dv=dv)
            want = plain_attend(f64(qd).reshape(-1, H, d), kk, vv, positions, lo_of, scale, H, G)
            assert rel(out.view(-1, H, dv), want) < (2e-5 if dtype == "float32" else 2e-2), (planted, positions)
            seen = lo <= planted
            took = rel(out.view(-1, H, dv)[-1, 0], vv[planted, 0]) < 0.05
            assert took == seen, f"key {planted} ({'inside' if seen else 'outside'} [{lo}, {last}]) took={took}"
    K().check_device_errors()


@pytest.mark.parametrize("kind,size", [("window", 44), ("window", 100), ("chunk", 48), ("chunk", 208), ("chunk", 64), ("chunk", 1), ("chunk", 1000),
                                       ("window", 400)])
@pytest.mark.parametrize("geom", [(8, 2, 64), (4, 1, 128), (4, 4, 64), (16, 1, 128)])
def test_edges_of_windows_and_chunks_tiled_kernels(kind, size, geom):
    """The same for the tensor-core kernels (bfloat16, head sizes 64 and 128): a prompt portion of 70 tokens (tcgen05
    tiles), a short portion of 3 (mma.sync tiles) and a single token (the decode kernel), each with the engine's own tile
    lists; with one key/value head the keys also serve as values (a latent row)."""
    from hfcpu_b200.kernels import attention_step_arrays
    H, G, d = geom
    dt, bs, n, scale = torch.bfloat16, 16, 431, 0.5
    code, lo_of = MASKS[kind](size)
    last = n - 1
    lo = lo_of(last)
    for planted in sorted({lo, lo - 1, last, 0, bs - 1, bs, 9 * bs - 1, 9 * bs}):
        if planted < 0:
            continue
        r = rng(planted + size + d)
        k = 0.3 * r.standard_normal((n, G, d))
        v = r.standard_normal((n, G, d))
        k[planted] = 3.0
        kc, vc, kd, vd, bt, pages = paged(k, v, bs, dt, seed=planted)
        same = G == 1                                   # keys as values
        meta = SimpleNamespace(block_table=bt, block_size=bs, max_blocks=pages, group=0)
        for count in (70, 3, 1):
            positions = list(range(n - count, n))
            q = 0.3 * r.standard_normal((count, H, d))
            q[-1] = 1.5
            qd = dev(q, dt).reshape(count, H * d).contiguous()
            tiles = {kk: torch.tensor(vv, dtype=torch.int32, device=DEV) for kk, vv in attention_step_arrays([count], H // G).items()}
            ctx = SimpleNamespace(token_seq=torch.zeros(count, dtype=torch.int32, device=DEV), max_q_len=count, max_kv_len=n,
                                  positions=torch.tensor(positions, dtype=torch.int32, device=DEV),
                                  buf=lambda name, shape, dtype: torch.empty(shape, dtype=dtype, device=DEV))
            out = torch.empty(count, H * d, dtype=dt, device=DEV)
            K().paged_attention(qd, kc, kc if same else vc, meta, ctx, H, G, d, code, scale, out, tiles=tiles)
            vv = f64(kd) if same else f64(vd)
            want = plain_attend(f64(qd).reshape(-1, H, d), f64(kd), vv, positions, lo_of, scale, H, G)
            assert rel(out.view(-1, H, d), want) < 2e-2, (planted, count)
            seen = lo <= planted
            took = rel(out.view(-1, H, d)[-1, 0], vv[planted, 0]) < 0.05
            assert took == seen, f"{count} tokens: key {planted} ({'inside' if seen else 'outside'} [{lo}, {last}]) took={took}"
    K().check_device_errors()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", [(5, 72, 100), (130, 256, 512), (1, 44, 24), (300, 328, 392)])
def test_feed_forward_with_squared_relu(dtype, shape):
    from hfcpu_b200.config import PartSpec
    from hfcpu_b200.engine.step import Workspace
    from hfcpu_b200.parts import make_part
    T, width, ff = shape
    r = rng(sum(shape))
    dt = DT[dtype]
    part = make_part("ffn", PartSpec("mlp", {"hidden_size": width, "intermediate_size": ff, "prefix": "m.mlp", "activation": "relu2"}))
    tensors = {s.name: dev(0.3 * r.standard_normal(s.shape), dt) for s in part.tensor_specs()}
    assert sorted(tensors) == ["m.mlp.down", "m.mlp.up"]
    part.bind(tensors, dt, torch.device(DEV))
    ctx = SimpleNamespace(buf=Workspace(torch.device(DEV)).get, run_dtype=dt)
    xn = dev(r.standard_normal((T, width)), dt)
    res = dev(r.standard_normal((T, width)))
    want = f64(res) + plain.feed_forward(f64(xn), {k: f64(v) for k, v in tensors.items()}, "m")
    out = res.clone()
    part.forward(ctx, xn, out)
    assert rel(out, want) < (2e-5 if dtype == "float32" else 2e-2)
    norm = make_part("norm", PartSpec("rmsnorm", {"size": width, "eps": 1e-6, "tensor": "n", "offset": 1.0}))
    nw = dev(0.3 * r.standard_normal(width), dt)
    norm.bind({"n": nw}, dt, torch.device(DEV))
    out2, xn2 = res.clone(), torch.empty(T, width, dtype=dt, device=DEV)
    assert part.forward_then_norm(ctx, xn, out2, norm, xn2) is True
    assert rel(out2, want) < (2e-5 if dtype == "float32" else 2e-2)
    assert rel(xn2, plain.norm_one_plus(f64(out2), f64(nw), 1e-6)) < KTOL[dtype]
    K().check_device_errors()


# ---- the engine -------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for i, (n, c) in enumerate(CONFIGS.items()):
        out[n] = make_folder(c, str(tmp_path_factory.mktemp(f"peludra_{n}")), 5 + i)
        out[n + "16"] = make_folder(c, str(tmp_path_factory.mktemp(f"peludra_{n}16")), 5 + i, torch.bfloat16)
    return out


LENGTHS = {"odd": [1, 19, 70, 130, 33], "wide": [3, 150, 64, 129, 260], "thin": [2, 9, 41]}
FAMILIES = {"whole": traces.whole, "tail": traces.tail_one_by_one, "portions": traces.portions, "mixed": traces.mixed}


def assert_rows(got, ref, tol, what="the plain implementation"):
    keys = sorted(got, key=lambda k: (str(k[0]), k[1]))
    errs = [float((got[k].double() - ref[k[0]][k[1]].double()).abs().max() / ref[k[0]][k[1]].double().abs().max()) for k in keys]
    over = [(k, e) for k, e in zip(keys, errs) if e > tol]
    assert not over, (f"{len(over)} of {len(keys)} rows differ from {what}; first: request {over[0][0][0]} position {over[0][0][1]} "
                      f"(error {over[0][1]:.3g})")


def engine_for(folder, block, dtype, max_tokens, max_requests=4):
    import hfcpu_b200
    m = hfcpu_b200.load_model(folder, DT[dtype], DEV)
    return hfcpu_b200.Engine(m, block_size=block, max_tokens=max_tokens, max_requests=max_requests, ctx_max=4096)


def check_clean(eng):
    K().check_device_errors()
    eng.cache.check()
    assert eng.cache.pages_in_use() == 0 and eng.slots.free_count == eng.max_requests


_WHOLE = {}


@pytest.mark.parametrize("family", list(FAMILIES))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_cuttings_match_plain(folders, name, dtype, family):
    """Whole prompts, a tail decoded token by token, portions down to two tokens, and mixed batches of up to four requests
    in a pool sized for the peak, so that pages and slots are used again."""
    folder = folders[name if dtype == "float32" else name + "16"]
    reqs = requests(CONFIGS[name]["vocab"], LENGTHS[name], seed=3)
    steps = FAMILIES[family](reqs)
    eng = engine_for(folder, BLOCKS[name], dtype, traces.peak_tokens(steps, round_to=BLOCKS[name]))
    got = traces.run_in_process(eng, steps, check=eng.cache.check)
    check_clean(eng)
    ref = {r: plain_logits(folder, ids) for r, ids in reqs.items()}
    assert len(got) == sum(len(v) for v in reqs.values())
    assert_rows(got, ref, TOL[dtype])
    if family == "whole":
        _WHOLE[(name, dtype)] = got
    elif (name, dtype) in _WHOLE:
        base = _WHOLE[(name, dtype)]
        assert_rows(got, {r: torch.stack([base[(r, p)] for p in range(len(ids))]) for r, ids in reqs.items()}, SELF_TOL[dtype],
                    "the whole-prompt run")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["odd", "wide"])
def test_long_decoding(folders, name, dtype):
    """Every token a step of its own (from the second bfloat16 step on a replayed graph), two requests side by side, past
    several pages, windows and chunks."""
    folder = folders[name if dtype == "float32" else name + "16"]
    reqs = requests(CONFIGS[name]["vocab"], [230, 75], seed=8)
    n = max(len(v) for v in reqs.values())
    steps = []
    for p in range(n):
        entries = [{"id": r, "tokens": [ids[p]], "want": [0], "_pos": p} for r, ids in reqs.items() if p < len(ids)]
        steps.append({"step": p, "entries": entries, "end": [r for r, ids in reqs.items() if p == len(ids) - 1]})
    eng = engine_for(folder, BLOCKS[name], dtype, 384)
    got = traces.run_in_process(eng, steps)
    check_clean(eng)
    assert_rows(got, {r: plain_logits(folder, ids) for r, ids in reqs.items()}, TOL[dtype])


ONE_LAYER = {
    "chunk": lambda: model(150, 64, 1e-5, 4.0, (31, 5, 3), [layer(att(4, 2, 16, 24, 0.5, 24, v_mix=True), 48)]),
    "window": lambda: model(150, 64, 1e-5, 4.0, (31, 5, 3), [layer(lat(4, 16, 8, 24, 32, 24, 0.4, 19, 100.0), 48)]),
    "window_tiled": lambda: model(150, 64, 1e-5, 4.0, (31, 5, 3), [layer(lat(4, 16, 16, 24, 32, 48, 0.4, 37, 100.0), 48)]),
    "chunk_tiled": lambda: model(150, 64, 1e-5, 4.0, (31, 5, 3), [layer(att(4, 2, 64, 64, 0.3, 40), 48)]),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", list(ONE_LAYER))
def test_a_changed_token_shows_exactly_inside_the_mask(tmp_path, which, dtype):
    """A model of one layer sees, from its last position, exactly the tokens inside that layer's window or chunk (and the one
    before the first of them, through the pair term of the embedding).  One token is changed at places around the edge:
    inside, the logits must move as the plain implementation's do; outside, they must not move at all.  The last tokens come
    in a portion and one by one."""
    cfg = ONE_LAYER[which]()
    folder = make_folder(cfg, str(tmp_path), 31, DT[dtype], sharp=4.0)
    C, W = plain.read_folder(folder)
    m = cfg["layers"][0]["mixer"]
    size, n, bs = m["mask"]["size"], 131, 8
    last = n - 1
    lo = last // size * size if "chunk" in which else last - size + 1
    base = requests(150, [n], seed=4)["r0"]
    from hfcpu_b200 import StepEntry

    def engine_last(ids, tail):
        eng = engine_for(folder, bs, dtype, 192, max_requests=1)
        eng.add_request("a")
        eng.step([StepEntry("a", ids[:n - tail], [])])
        for p in range(n - tail, n - 1):
            eng.step([StepEntry("a", ids[p:p + 1], [])])
        got = eng.step([StepEntry("a", ids[n - 1:], [0])])[0].double().cpu().numpy()
        eng.finish_request("a")
        check_clean(eng)
        return got

    def engine_portion(ids, tail):
        eng = engine_for(folder, bs, dtype, 192, max_requests=1)
        eng.add_request("a")
        eng.step([StepEntry("a", ids[:n - tail], [])])
        got = eng.step([StepEntry("a", ids[n - tail:], [tail - 1])])[0].double().cpu().numpy()
        eng.finish_request("a")
        check_clean(eng)
        return got
    ref = plain.forward(C, W, base)[-1]
    runs = {"portion": lambda ids: engine_portion(ids, 5), "decoded": lambda ids: engine_last(ids, 3)}
    same = {k: f(base) for k, f in runs.items()}
    for k in runs:
        assert np.abs(same[k] - ref).max() / np.abs(ref).max() < TOL[dtype]
    moved = 0
    for place in (lo - 3, lo - 2, lo - 1, lo, lo + 1, last - 1):
        if place < 0:
            continue
        ids = list(base)
        ids[place] = (ids[place] + 71) % 150
        want = plain.forward(C, W, ids)[-1]
        matters = np.abs(want - ref).max() / np.abs(ref).max()
        # the token at lo - 1 enters through the pair term of the token at lo; lo - 2 and earlier cannot be seen
        assert (matters > 0) == (place >= lo - 1)
        for k, f in runs.items():
            got = f(ids)
            if place < lo - 1:
                assert np.array_equal(got, same[k]), f"{k}: a token outside the mask (place {place}, first seen {lo}) changed the logits"
            else:
                err = np.abs(got - want).max() / np.abs(want).max()
                assert err < TOL[dtype], f"{k}: token changed at {place}: error {err:.3g}"
                if matters > 1e-2:
                    moved += 1
    assert moved >= 2 or dtype == "bfloat16", "no change inside the mask moved the logits enough to tell"


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
    """Steady decoding in bfloat16 goes through captured graphs (the previous token's state included) and repeats itself;
    more requests than slots, so that slots are used again."""
    import hfcpu_b200
    sess = hfcpu_b200.Session(folders["wide16"], dtype="bfloat16", kv_block=16, kv_pages=128, max_seqs=2, ctx_max=512)
    prompts = list(requests(1032, [19, 130, 64, 5], seed=2).values())
    a = sess.generate(prompts, temp=0, max_tokens=24)
    assert sess.engine.use_graphs and any(s[0] == "ready" for s in sess.engine._graphs.values())
    b = sess.generate(prompts, temp=0, max_tokens=24)
    assert [c[0].tokens for c in a] == [c[0].tokens for c in b] and all(len(c[0].tokens) == 24 for c in a)
    # and they are the tokens of the float32 run's first steps where the two agree on a clear winner
    cfg, W = plain.read_folder(folders["wide16"])
    for got, p in zip(a, prompts):
        row = np.sort(plain.forward(cfg, W, p)[-1])
        if row[-1] - row[-2] > 0.5:
            assert got[0].tokens[0] == int(np.argmax(plain.forward(cfg, W, p)[-1]))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_program(folders, tmp_path, dtype):
    folder = folders["odd" if dtype == "float32" else "odd16"]
    reqs = requests(211, [5, 40, 77, 12, 30], seed=9)
    steps = traces.mixed(reqs, max_live=4)
    got = traces.run_trace_program(folder, dtype, steps, str(tmp_path), traces.peak_tokens(steps), 211, block_size=8)
    assert_rows(got, {r: plain_logits(folder, ids) for r, ids in reqs.items()}, TOL[dtype])


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
