"""Plain, slow implementation of the Manapel decoder in float64, whole sequences, no cache.

One function per mechanism, written from the design's equations and sharing no code with the
package.  A model is (config dict, {tensor name: float64 numpy array}).

Notation: x is the residual stream [T, width]; a layer is
    x += post1(mixer(pre1(x)));  x += post2(ff(pre2(x)))
with every norm a Dynamic Tanh  y = tanh(alpha * x) * w + b  (no statistics of x).
"""
import json
import os
import struct

import numpy as np


# ---- files ---------------------------------------------------------------------------------------
def read_safetensors(path):
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        head = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, m in head.items():
        if name == "__metadata__":
            continue
        a, b = m["data_offsets"]
        raw = data[a:b]
        if m["dtype"] == "BF16":
            v = (np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16).view(np.float32)
        elif m["dtype"] == "F32":
            v = np.frombuffer(raw, dtype="<f4")
        elif m["dtype"] == "I32":
            v = np.frombuffer(raw, dtype="<i4")
        else:
            raise ValueError(m["dtype"])
        out[name] = v.astype(np.float64).reshape(m["shape"])
    return out


def read_folder(folder):
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_safetensors(os.path.join(folder, "model.safetensors"))


# ---- mechanisms ----------------------------------------------------------------------------------
def dynamic_tanh(x, W, name):
    return np.tanh(W[name + ".alpha"] * x) * W[name] + W[name + ".b"]


def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def rotate_half(x, positions, rot):
    """x [T, heads, dim]: dimension i < dims/2 pairs with i + dims/2; angle = position * base^(-2i/dims)."""
    if not rot or not rot["dims"]:
        return x
    dims, base = rot["dims"], rot["base"]
    half = dims // 2
    f = base ** (-2.0 * np.arange(half) / dims)
    a = np.asarray(positions, dtype=np.float64)[:, None, None] * f[None, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return np.concatenate([u * np.cos(a) - v * np.sin(a), v * np.cos(a) + u * np.sin(a), x[..., dims:]], -1)


def keys_values(h, W, p, m, eps):
    """Keys (rotated, then unit rms per head) and values of a layer that projects its own: [T, G, dim], [T, G, vdim]."""
    T = h.shape[0]
    G, d, dv = m["kv_heads"], m["dim"], m["vdim"]
    k = (h @ W[p + ".mix.k"].T + W[p + ".mix.k.b"]).reshape(T, G, d)
    v = (h @ W[p + ".mix.v"].T + W[p + ".mix.v.b"]).reshape(T, G, dv)
    k = unit_rms(rotate_half(k, np.arange(T), m.get("rot")), eps)
    return k, v


def attention(h, W, p, m, eps, kv):
    """Causal softmax attention with grouped heads; ``kv`` = (keys, values) as the owning layer made them."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ W[p + ".mix.q"].T + W[p + ".mix.q.b"]).reshape(T, H, d)
    q = unit_rms(rotate_half(q, np.arange(T), m.get("rot")), eps)
    k, v = kv
    out = np.zeros((T, H, dv))
    mask = np.tril(np.ones((T, T), dtype=bool))
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * m["scale"]
        s = np.where(mask, s, -np.inf)
        s = s - s.max(-1, keepdims=True)
        w = np.exp(s)
        w = w / w.sum(-1, keepdims=True)
        out[:, hd] = w @ v[:, g]
    return out.reshape(T, H * dv) @ W[p + ".mix.o"].T


def dense_ff(h, W, p):
    return (np.maximum(h @ W[p + ".gate"].T, 0.0) * (h @ W[p + ".up"].T)) @ W[p + ".down"].T


def expert_ff(h, W, p):
    a = np.maximum(h @ W[p + ".up"].T, 0.0)
    return (a * a) @ W[p + ".down"].T


def route(h, W, p, top):
    """Chosen experts [T, top] (largest logits first) and their weights: softmax over the chosen logits only."""
    z = h @ W[p + ".router"].T + W[p + ".router.b"]
    idx = np.argsort(-z, axis=-1, kind="stable")[:, :top]
    zc = np.take_along_axis(z, idx, -1)
    e = np.exp(zc - zc.max(-1, keepdims=True))
    return idx, e / e.sum(-1, keepdims=True)


def moe_ff(h, W, p, mlp):
    idx, w = route(h, W, p, mlp["router"]["top"])
    out = np.zeros((h.shape[0], W[p + ".e0.down"].shape[0]))
    for t in range(h.shape[0]):
        for j in range(idx.shape[1]):
            out[t] += w[t, j] * expert_ff(h[t:t + 1], W, f"{p}.e{idx[t, j]}")[0]
    if mlp.get("shared"):
        out += expert_ff(h, W, p + ".shared")
    return out


def forward(cfg, W, ids, layers_out=None):
    """Logits [T, vocab] of every position of ``ids``; ``layers_out`` (a list) receives x after every layer."""
    eps = cfg["norm"]["eps"]
    x = W["embed"][np.asarray(ids)]
    kv = {}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}", L["mixer"]
        assert L["type"] == "attention"
        h = dynamic_tanh(x, W, p + ".norm1")
        if m.get("kv_from") is None:
            kv[i] = keys_values(h, W, p, m, eps)
            mine = kv[i]
        else:
            mine = kv[m["kv_from"]]
        x = x + dynamic_tanh(attention(h, W, p, m, eps, mine), W, p + ".norm1b")
        mlp = L.get("mlp")
        if mlp:
            h = dynamic_tanh(x, W, p + ".norm2")
            y = dense_ff(h, W, p + ".mlp") if mlp["kind"] == "dense" else moe_ff(h, W, p + ".mlp", mlp)
            x = x + dynamic_tanh(y, W, p + ".norm2b")
        if layers_out is not None:
            layers_out.append(x.copy())
    return (dynamic_tanh(x, W, "final.norm") @ W["head"].T) * cfg["logit_scale"]


def greedy(cfg, W, prompt, n_new):
    ids, out = list(prompt), []
    for _ in range(n_new):
        out.append(int(np.argmax(forward(cfg, W, ids)[-1])))
        ids.append(out[-1])
    return out
