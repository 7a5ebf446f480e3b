"""Plain, slow implementation of the Peludra decoder in float64, whole sequences, no cache.

One function per mechanism, written from the design's equations and sharing no code with the
package.  A model is (config dict, {tensor name: float64 numpy array}).

Notation: x is the residual stream [T, width]; a layer is
    x += mixer(norm1(x));  x += ff(norm2(x))
with norm(x) = x / sqrt(mean(x^2) + eps) * (1 + w).
"""
import json
import math
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


# ---- norms ---------------------------------------------------------------------------------------
def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def norm_plain(x, w, eps):
    return unit_rms(x, eps) * w


def norm_one_plus(x, w, eps):
    """The weight is stored around zero."""
    return unit_rms(x, eps) * (1.0 + w)


# ---- embedding -----------------------------------------------------------------------------------
def bigram_rows(ids, b):
    """Row of the pair table for every token: hashed (previous, current); the last row for a first token."""
    rows = []
    for i, t in enumerate(ids):
        rows.append(b["buckets"] if i == 0 else (ids[i - 1] * b["mul_prev"] + t * b["mul_cur"]) % b["buckets"])
    return rows


def embed(cfg, W, ids):
    e = cfg["embedding"]
    x = W["embed"][ids] * e["scale"]
    if e.get("bigram"):
        x = x + W["bigram"][bigram_rows(ids, e["bigram"])]
    return x


# ---- rotation ------------------------------------------------------------------------------------
def rotary_frequencies(rot):
    """(frequency per pair, factor on cos and sin).  With ``scaling``: low frequencies are divided by ``factor``, high
    ones kept, with a linear ramp over the pair index between the two; cos and sin grow by 0.1 ln(factor) + 1."""
    dims, base = rot["dims"], rot["base"]
    i = np.arange(dims // 2, dtype=np.float64)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, original = sc["factor"], sc["original"]

    def pair_of(turns):                  # the pair index whose wavelength makes ``turns`` turns over the original length
        return dims * math.log(original / (2 * math.pi * turns)) / (2 * math.log(base))
    lo = max(math.floor(pair_of(sc["fast"])), 0)
    hi = min(math.ceil(pair_of(sc["slow"])), dims - 1)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_interleaved(x, positions, rot):
    """x [T, ..., n]: dimensions 2i and 2i+1 of the first rot.dims form a pair; the rest pass unchanged."""
    dims = rot["dims"]
    f, m = rotary_frequencies(rot)
    a = np.asarray(positions, dtype=np.float64).reshape((-1,) + (1,) * (x.ndim - 1)) * f
    c, s = np.cos(a) * m, np.sin(a) * m
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.copy()
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


# ---- masks ---------------------------------------------------------------------------------------
def chunk_mask(T, size):
    """i sees j <= i of its own chunk of ``size`` positions, counted from position 0."""
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    return (j <= i) & (i // size == j // size)


def window_mask(T, size):
    """i sees itself and the size - 1 positions before it."""
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    return (j <= i) & (i - j < size)


def softmax_mix(scores, mask, v):
    """scores [H, T, T], v [T, H, dv] -> [T, H, dv]."""
    s = np.where(mask[None], scores, -np.inf)
    s = s - s.max(-1, keepdims=True)
    p = np.exp(s)
    p = p / p.sum(-1, keepdims=True)
    return np.einsum("hij,jhd->ihd", p, v)


# ---- mixers --------------------------------------------------------------------------------------
def attention(h, W, p, m, eps, v_first):
    """Grouped heads, per-head norm of queries and keys with a shared weight, no positions in the scores, chunked.
    ``v_first``: the values of the first value-mixing layer (None in that layer and in layers that do not mix).
    Returns (output, this layer's values before mixing)."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ W[p + ".mix.q"].T).reshape(T, H, d)
    k = (h @ W[p + ".mix.k"].T).reshape(T, G, d)
    v = (h @ W[p + ".mix.v"].T).reshape(T, G, dv)
    q = norm_plain(q, W[p + ".mix.q.norm"], eps)
    k = norm_plain(k, W[p + ".mix.k.norm"], eps)
    own_v = v
    if v_first is not None:
        lam = float(W[p + ".mix.vmix"])
        v = (1.0 - lam) * v + lam * v_first
    k = np.repeat(k, H // G, axis=1)
    v = np.repeat(v, H // G, axis=1)
    scores = np.einsum("ihd,jhd->hij", q, k) * m["scale"]
    o = softmax_mix(scores, chunk_mask(T, m["mask"]["size"]), v)
    return o.reshape(T, H * dv) @ W[p + ".mix.o"].T, own_v


def latent_attention(h, W, p, m, eps):
    """Queries through a normed latent; keys and values expanded from a normed latent of ``kv_rank``; one rotated key part
    shared by all heads; sliding window."""
    T = h.shape[0]
    H, d, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = np.arange(T)
    cq = norm_plain(h @ W[p + ".mix.dq"].T, W[p + ".mix.dq.norm"], eps)
    q = (cq @ W[p + ".mix.uq"].T).reshape(T, H, d + dr)
    q_plain, q_rot = q[..., :d], rotate_interleaved(q[..., d:], pos, m["rot"])
    ckv = h @ W[p + ".mix.dkv"].T
    c = norm_plain(ckv[:, :R], W[p + ".mix.dkv.norm"], eps)
    k_rot = rotate_interleaved(ckv[:, R:], pos, m["rot"])                    # [T, dr], shared by the heads
    k_plain = (c @ W[p + ".mix.uk"].T).reshape(T, H, d)
    v = (c @ W[p + ".mix.uv"].T).reshape(T, H, dv)
    scores = (np.einsum("ihd,jhd->hij", q_plain, k_plain) + np.einsum("ihd,jd->hij", q_rot, k_rot)) * m["scale"]
    o = softmax_mix(scores, window_mask(T, m["mask"]["size"]), v)
    return o.reshape(T, H * dv) @ W[p + ".mix.o"].T


# ---- feed-forward --------------------------------------------------------------------------------
def feed_forward(h, W, p):
    u = np.maximum(h @ W[p + ".mlp.up"].T, 0.0)
    return (u * u) @ W[p + ".mlp.down"].T


# ---- the model -----------------------------------------------------------------------------------
def forward(cfg, W, ids, layers_out=None):
    """Logits [T, vocab] of one whole sequence.  ``layers_out``: a list that receives the stream after every layer."""
    eps = cfg["norm"]["eps"]
    ids = list(ids)
    x = embed(cfg, W, ids)
    v_first = None
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}"
        h = norm_one_plus(x, W[p + ".norm1"], eps)
        if L["type"] == "attention":
            mixes = bool(L["mixer"].get("v_mix"))
            y, own_v = attention(h, W, p, L["mixer"], eps, v_first if mixes else None)
            if mixes and v_first is None:
                v_first = own_v
        elif L["type"] == "latent_attention":
            y = latent_attention(h, W, p, L["mixer"], eps)
        else:
            raise ValueError(L["type"])
        x = x + y
        if L.get("mlp"):
            x = x + feed_forward(norm_one_plus(x, W[p + ".norm2"], eps), W, p)
        if layers_out is not None:
            layers_out.append(x.copy())
    return norm_one_plus(x, W["final.norm"], eps) @ W["head"].T


def greedy(cfg, W, prompt, n):
    """n tokens by arg-max, the whole sequence computed anew for each."""
    ids, out = list(prompt), []
    for _ in range(n):
        t = int(np.argmax(forward(cfg, W, ids)[-1]))
        out.append(t)
        ids.append(t)
    return out
