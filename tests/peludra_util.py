"""Small Peludra configurations, model folders with random weights, and the plain implementation's logits."""
import numpy as np
import torch

import plain_peludra as plain


def att(heads, kv_heads, dim, vdim, scale, chunk, v_mix=False):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": chunk}}
    if v_mix:
        m["v_mix"] = True
    return {"type": "attention", "mixer": m}


def lat(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, window, base, scaling=None):
    rot = {"dims": rot_dim, "base": base}
    if scaling:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank,
                                                  "kv_rank": kv_rank, "scale": scale, "mask": {"size": window}, "rot": rot}}


def layer(mixer, ff):
    return dict(mixer, mlp={"kind": "dense", "ff": ff} if ff else None)


def model(vocab, width, eps, scale, bigram, layers):
    emb = {"scale": scale}
    if bigram:
        emb["bigram"] = dict(zip(("buckets", "mul_prev", "mul_cur"), bigram))
    return {"architecture": "Peludra", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": emb, "layers": layers}


# Odd sizes throughout: fewer key/value heads than heads, value heads wider than key heads, a chunk shorter than a page
# and one longer than the prompts' portions, a latent layer without a feed-forward, plain and rotated parts of different
# sizes, one rotation scaled and one not, an attention layer that stays out of the value mixing between two that mix.
ODD = model(211, 72, 1e-5, 3.0, (53, 31, 7), [
    layer(att(6, 3, 24, 40, 0.3, 12, v_mix=True), 100),
    layer(lat(3, 16, 8, 24, 40, 24, 0.25, 9, 500.0), None),
    layer(att(4, 4, 16, 16, 0.35, 50), 64),
    layer(att(6, 3, 24, 40, 0.3, 7, v_mix=True), 40),
    layer(lat(5, 8, 12, 20, 16, 36, 0.3, 33, 3000.0, scaling=(4.0, 64, 8.0, 2.0)), 56),
    layer(att(3, 3, 32, 40, 0.25, 30, v_mix=True), None),
])
# Sizes the tensor-core kernels take: head sizes 64 and 128 with equal value heads, a latent row of 128 and one of 64,
# widths that are multiples of 8.
WIDE = model(1032, 256, 1e-6, 8.0, (499, 131, 19), [
    layer(lat(4, 64, 32, 64, 128, 96, 0.12, 44, 25000.0, scaling=(6.0, 128, 16.0, 1.0)), 512),
    layer(att(8, 2, 64, 64, 0.15, 48, v_mix=True), 256),
    layer(att(4, 1, 128, 128, 0.1, 208), 512),
    layer(lat(8, 32, 16, 48, 64, 48, 0.15, 100, 10000.0), 256),
    layer(att(8, 2, 64, 64, 0.15, 150, v_mix=True), 256),
])
# A width that is no multiple of 8 (no tensor-core product takes it), no pair term in the embedding, one key/value head,
# a chunk of one position (a query sees itself only), a window of one, a window longer than any request.
THIN = model(97, 44, 1e-4, 1.0, None, [
    layer(att(2, 1, 20, 12, 0.4, 1), 24),
    layer(lat(2, 12, 4, 8, 10, 6, 0.5, 200, 77.0), 20),
    layer(lat(1, 6, 2, 10, 12, 10, 0.5, 1, 77.0), None),
])
CONFIGS = {"odd": ODD, "wide": WIDE, "thin": THIN}
BLOCKS = {"odd": 8, "wide": 16, "thin": 4}


def make_folder(cfg_dict, folder, seed, dtype=torch.float32, edit=None, sharp=3.0):
    """A model folder with random weights whose attention is far from uniform (query and key projections scaled up), norm
    weights well away from their neutral values and a value-mixing weight well inside (0, 1).  Stored in bfloat16 the
    weights are smaller, so that the rounding of large intermediate values does not swamp the comparison."""
    from hfcpu_b200.config import config_from_dict
    from hfcpu_b200.models import build_model_specs
    from hfcpu_b200.weights import random_tensors, write_safetensors, weights_path
    cfg = config_from_dict(cfg_dict)
    cfg.save(folder)
    soft = dtype == torch.bfloat16
    tensors = random_tensors(build_model_specs(cfg), seed, torch.float32, std=0.05 if soft else 0.09)
    g = torch.Generator().manual_seed(seed)
    for name in tensors:
        t = tensors[name]
        if name in ("embed", "bigram"):
            tensors[name] = t * (6 if soft else 8)
        elif name.endswith(".vmix"):
            tensors[name] = torch.empty(()).uniform_(0.25, 0.75, generator=g)
        elif name.endswith(("norm1", "norm2", "final.norm")):
            tensors[name] = torch.empty(t.shape).uniform_(-0.4, 0.4, generator=g)
        elif name.endswith(".norm"):
            tensors[name] = torch.empty(t.shape).uniform_(0.5, 1.6, generator=g)
        elif name.endswith((".mix.q", ".mix.k", ".mix.uq", ".mix.uk", ".mix.dkv")):
            tensors[name] = t * sharp
        elif ".mix.o" in name or name.endswith(".down"):
            tensors[name] = t * 2
    if edit:
        edit(tensors)
    # what is stored is what both sides read: round once to the storage type
    write_safetensors(weights_path(folder), {k: v.to(dtype) for k, v in tensors.items()})
    return folder


_PLAIN = {}


def plain_logits(folder, ids):
    key = (folder, tuple(ids))
    if key not in _PLAIN:
        cfg, W = plain.read_folder(folder)
        _PLAIN[key] = torch.from_numpy(plain.forward(cfg, W, list(ids)))
    return _PLAIN[key]


def requests(vocab, lengths, seed=0):
    g = torch.Generator().manual_seed(seed)
    return {f"r{i}": torch.randint(0, vocab, (n,), generator=g).tolist() for i, n in enumerate(lengths)}
