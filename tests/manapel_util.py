"""Small Manapel configurations, model folders with random weights, and the plain implementation's logits."""
import os

import numpy as np
import torch

import plain_manapel as plain


def att(heads, kv_heads, dim, vdim, rot_dims, base, scale, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if rot_dims is not None:
        m["rot"] = {"dims": rot_dims, "base": base}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def moe(experts, top, ff, shared=None):
    d = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared:
        d["shared"] = {"ff": shared}
    return d


def layer(mixer, mlp):
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


# Odd sizes throughout: value heads wider than key heads, one expert per token, a layer without a feed-forward, keys and
# values borrowed from a layer that is not the neighbour, a head that is rotated whole, no shared expert in one layer.
ODD = {"architecture": "Manapel", "vocab": 300, "width": 72, "logit_scale": 1.7, "norm": {"eps": 1e-3}, "layers": [
    layer(att(6, 3, 24, 40, 8, 500.0, 0.6), moe(5, 1, 40)),
    layer(att(6, 3, 24, 40, 8, 500.0, 0.6, kv_from=0), None),
    layer(att(4, 4, 16, 16, 16, 10000.0, 1.0), {"kind": "dense", "ff": 100}),
    layer(att(6, 3, 24, 40, 8, 500.0, 0.6, kv_from=0), moe(5, 3, 24, shared=56)),
]}
# Sizes the tensor-core kernels take (head sizes 64 and 128, widths that are multiples of 8), many experts.
WIDE = {"architecture": "Manapel", "vocab": 1032, "width": 256, "logit_scale": 0.25, "norm": {"eps": 1e-6}, "layers": [
    layer(att(8, 2, 64, 64, 32, 10000.0, 0.3), moe(16, 4, 64, shared=128)),
    layer(att(8, 2, 64, 64, 32, 10000.0, 0.3, kv_from=0), {"kind": "dense", "ff": 512}),
    layer(att(4, 1, 128, 128, 64, 50000.0, 0.2), moe(3, 2, 128)),
    layer(att(4, 1, 128, 128, 64, 50000.0, 0.2, kv_from=2), moe(16, 1, 64, shared=64)),
]}
# One key/value head per query head, no rotation in one layer, a value head narrower than the key head, a width that is
# no multiple of 8 (no tensor-core product takes it).
THIN = {"architecture": "Manapel", "vocab": 97, "width": 44, "logit_scale": 1.0, "norm": {"eps": 1e-5}, "layers": [
    layer(att(2, 2, 32, 8, None, 0.0, 0.4), {"kind": "dense", "ff": 24}),
    layer(att(2, 1, 20, 12, 4, 77.0, 0.9), moe(2, 2, 16, shared=8)),
]}
CONFIGS = {"odd": ODD, "wide": WIDE, "thin": THIN}
BLOCKS = {"odd": 8, "wide": 16, "thin": 4}


def make_folder(cfg_dict, folder, seed, dtype=torch.float32, edit=None):
    """A model folder whose values leave the linear part of tanh, with routers that decide clearly.  Stored in bfloat16
    the weights are smaller, so that the rounding of large intermediate values does not swamp the comparison."""
    from hfcpu_b200.config import config_from_dict
    from hfcpu_b200.models import build_model_specs
    from hfcpu_b200.weights import random_tensors, write_safetensors, weights_path
    cfg = config_from_dict(cfg_dict)
    cfg.save(folder)
    soft = dtype == torch.bfloat16
    tensors = random_tensors(build_model_specs(cfg), seed, torch.float32, std=0.04 if soft else 0.08)
    g = torch.Generator().manual_seed(seed)
    for name in tensors:
        if name == "embed":
            tensors[name] = tensors[name] * (10 if soft else 12)
        elif name.endswith(".alpha"):
            tensors[name] = torch.empty(()).uniform_(0.4, 1.6, generator=g)
        elif name.endswith(".router"):
            tensors[name] = tensors[name] * 6
        elif ".mix.o" in name or name.endswith(".down"):
            tensors[name] = tensors[name] * 2
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
