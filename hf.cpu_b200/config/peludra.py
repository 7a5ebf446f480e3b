"""Peludra: a pre-norm decoder whose config.json lists its layers one by one, with two kinds of mixer.

Top-level keys: ``architecture`` ("Peludra"), ``vocab``, ``width``, ``norm`` ({``eps``}), ``embedding`` ({``scale``,
optionally ``bigram``: {``buckets``, ``mul_prev``, ``mul_cur``}}) and ``layers``.  A layer entry has ``type`` (the kind of
mixer), ``mixer`` (its sizes) and ``mlp`` (its feed-forward, or null for none):

* mixer "attention": ``heads``, ``kv_heads`` (default: ``heads``), ``dim`` (query/key head), ``vdim`` (value head;
  default: ``dim``), ``scale`` (factor on the
  scores), ``mask`` ({``size``}: chunks of that many positions; a query sees the earlier keys of its own chunk),
  optionally ``v_mix`` (true: from the second such layer on, the values are mixed with the first such layer's).  No
  biases, no rotation; queries and keys are normed per head (rms, one weight vector shared by the heads).
* mixer "latent_attention": ``heads``, ``dim`` (plain) and ``rot_dim`` (rotated) dimensions per query/key head, ``vdim``,
  ``q_rank`` and ``kv_rank`` (the latents), ``scale``, ``mask`` ({``size``}: a sliding window), ``rot`` ({``dims``,
  ``base``, optionally ``scaling``: {``factor``, ``original``, ``fast``, ``slow``}}).
* mlp ``kind`` "dense": ``ff``; ``down(relu(up x)^2)``.

Every norm of the stream is an rms norm whose weight is stored around zero (applied as 1 + w).  Tensor names: ``embed``,
``bigram``, ``l<i>.norm1`` / ``norm2``, ``l<i>.mix.{q,k,v,o}`` with ``q.norm`` / ``k.norm`` / ``vmix``, or
``l<i>.mix.{dq,uq,dkv,uk,uv,o}`` with ``dq.norm`` / ``dkv.norm``, ``l<i>.mlp.{up,down}``, ``final.norm``, ``head``.

config.json gives no context length: ``max_positions`` (optional key, default below) bounds the rotary tables and a
request's length in this engine.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Dict, List

from .base import (ConfigError, LayerSpec, ModelConfig, ModelPlan, PartSpec, ScheduleEntry, UnsupportedError,
                   take_float, take_int)
from .manapel import _obj
from .registry import register_architecture

DEFAULT_MAX_POSITIONS = 1 << 16


def _mask_size(m: Dict[str, Any], w: str) -> int:
    mask = _obj(m, "mask", w, required=False)
    return take_int(mask, "size", lo=1) if mask is not None else 0


@dataclass
class PeludraConfig(ModelConfig):
    vocab: int = 0
    width: int = 0
    norm_eps: float = 1e-6
    embedding_scale: float = 1.0
    bigram: Dict[str, int] = field(default_factory=dict)        # buckets, mul_prev, mul_cur; empty: no pair term
    max_positions: int = DEFAULT_MAX_POSITIONS
    layers: List[Dict[str, Any]] = field(default_factory=list)
    eos_token_id: List[int] = field(default_factory=list)

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "PeludraConfig":
        V = take_int(d, "vocab", lo=1)
        E = take_int(d, "width", lo=1, hi=1_000_000)
        norm = _obj(d, "norm", "")
        emb = _obj(d, "embedding", "", required=False) or {}
        big = _obj(emb, "bigram", "embedding: ", required=False)
        bigram = {}
        if big is not None:
            bigram = {"buckets": take_int(big, "buckets", lo=1), "mul_prev": take_int(big, "mul_prev", lo=0),
                      "mul_cur": take_int(big, "mul_cur", lo=0)}
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        out = []
        first_mix = None            # sizes of the first value-mixing layer's value heads
        for i, L in enumerate(layers):
            w = f"layers[{i}]: "
            if not isinstance(L, dict):
                raise ConfigError(f"config.json: {w}must be an object")
            kind = L.get("type")
            m = _obj(L, "mixer", w)
            H = take_int(m, "heads", lo=1)
            dim = take_int(m, "dim", lo=1)
            vdim = take_int(m, "vdim", default=dim, lo=1)
            take_float(m, "scale")
            _mask_size(m, w)
            if kind == "attention":
                G = take_int(m, "kv_heads", default=H, lo=1)
                if H % G:
                    raise UnsupportedError(f"config.json: {w}unsupported attention geometry: {H} heads over {G} key/value heads")
                mixes = m.get("v_mix", False)
                if not isinstance(mixes, bool):
                    raise ConfigError(f"config.json: {w}'v_mix' must be true or false")
                if mixes:
                    if first_mix is None:
                        first_mix = (G, vdim)
                    elif first_mix != (G, vdim):
                        raise ConfigError(f"config.json: {w}v_mix: the first such layer's value heads have other sizes")
            elif kind == "latent_attention":
                rd = take_int(m, "rot_dim", lo=0)
                take_int(m, "q_rank", lo=1), take_int(m, "kv_rank", lo=1)
                if rd % 2:
                    raise UnsupportedError(f"config.json: {w}rot_dim {rd} must be even")
                if rd:
                    rot = _obj(m, "rot", w)
                    if take_int(rot, "dims", lo=2) != rd:
                        raise UnsupportedError(f"config.json: {w}rot.dims must equal rot_dim (the rotated part is rotated whole)")
                    take_float(rot, "base", lo=0.0)
                    sc = _obj(rot, "scaling", w, required=False)
                    if sc is not None:
                        for k in ("factor", "original", "fast", "slow"):
                            take_float(sc, k, lo=0.0)
            else:
                raise UnsupportedError(f"config.json: {w}mixer type '{kind}' is not supported (known: attention, latent_attention)")
            mlp = _obj(L, "mlp", w, required=False)
            if mlp is not None:
                if mlp.get("kind") != "dense":
                    raise UnsupportedError(f"config.json: {w}mlp kind '{mlp.get('kind')}' is not supported (known: dense)")
                take_int(mlp, "ff", lo=1)
            out.append(copy.deepcopy(L))
        eos = d.get("eos_token_id", [])
        eos = [] if eos is None else ([eos] if isinstance(eos, int) else list(eos))
        return cls(vocab=V, width=E, norm_eps=take_float(norm, "eps", 1e-6, lo=0.0),
                   embedding_scale=take_float(emb, "scale", 1.0), bigram=bigram,
                   max_positions=take_int(d, "max_positions", default=DEFAULT_MAX_POSITIONS, lo=1), layers=out, eos_token_id=eos)

    def to_dict(self) -> Dict[str, Any]:
        emb: Dict[str, Any] = {"scale": self.embedding_scale}
        if self.bigram:
            emb["bigram"] = dict(self.bigram)
        d = {"architecture": self.architecture or "Peludra", "vocab": self.vocab, "width": self.width,
             "norm": {"eps": self.norm_eps}, "embedding": emb, "layers": copy.deepcopy(self.layers)}
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            d["max_positions"] = self.max_positions
        if self.eos_token_id:
            d["eos_token_id"] = list(self.eos_token_id)
        return d

    def plan(self) -> ModelPlan:
        E = self.width
        norm = lambda name: PartSpec("rmsnorm", {"size": E, "eps": self.norm_eps, "tensor": name, "offset": 1.0})
        positions: Dict[str, PartSpec] = {}
        layers, schedule = [], []
        mixing_seen = False
        for i, L in enumerate(self.layers):
            p, m, mlp = f"l{i}", L["mixer"], L.get("mlp")
            size = (m.get("mask") or {}).get("size", 0)
            if L["type"] == "attention":
                v_mix = None
                if m.get("v_mix"):
                    v_mix, mixing_seen = ("later" if mixing_seen else "first"), True
                mixer = PartSpec("paged_attention", {
                    "hidden_size": E, "num_heads": m["heads"], "num_kv_heads": m.get("kv_heads", m["heads"]), "head_dim": m["dim"],
                    "v_head_dim": m.get("vdim", m["dim"]), "scale": float(m["scale"]), "qk_norm_eps": self.norm_eps,
                    "qk_norm_weights": {"q": "q.norm", "k": "k.norm"}, "qkv_bias": False, "out_bias": False, "window": 0,
                    "chunk": size, "v_mix": v_mix, "v_mix_tensor": "vmix", "position": None, "prefix": f"{p}.mix",
                    "names": {"q": "q", "k": "k", "v": "v", "o": "o"}, "weight_suffix": "", "bias_suffix": ".b"})
            else:
                pos_name = None
                if m["rot_dim"]:
                    rot = m["rot"]
                    sc = rot.get("scaling")
                    # layers with the same rotation share one table
                    pos_name = f"rot{rot['dims']}_{float(rot['base'])!r}_{sorted(sc.items()) if sc else None!r}"
                    positions.setdefault(pos_name, PartSpec("rotary", {
                        "head_dim": m["rot_dim"], "n_rot": rot["dims"], "theta": float(rot["base"]), "pairing": "interleaved",
                        "scaling": dict(sc) if sc else None}))
                mixer = PartSpec("latent_attention", {
                    "hidden_size": E, "num_heads": m["heads"], "head_dim": m["dim"], "rot_dim": m["rot_dim"],
                    "v_head_dim": m.get("vdim", m["dim"]), "q_rank": m["q_rank"], "kv_rank": m["kv_rank"], "scale": float(m["scale"]),
                    "norm_eps": self.norm_eps, "window": size, "position": pos_name, "prefix": f"{p}.mix"})
            ffn = None
            if mlp is not None:
                ffn = PartSpec("mlp", {"hidden_size": E, "intermediate_size": mlp["ff"], "prefix": f"{p}.mlp",
                                       "activation": "relu2", "names": {"up": "up", "down": "down"}})
            layers.append(LayerSpec(prefix=p, block=PartSpec("prenorm_residual"), norm1=norm(f"{p}.norm1"), mixer=mixer,
                                    norm2=norm(f"{p}.norm2") if ffn is not None else None, ffn=ffn))
            schedule.append(ScheduleEntry(i))
        b = self.bigram
        plan = ModelPlan(
            hidden_size=E, vocab_size=self.vocab, max_positions=self.max_positions,
            embedding=PartSpec("hashed_pair_embedding", {
                "vocab_size": self.vocab, "hidden_size": E, "tensor": "embed", "scale": self.embedding_scale,
                "pair_tensor": "bigram" if b else None, "buckets": b.get("buckets", 0), "mul_prev": b.get("mul_prev", 0),
                "mul_cur": b.get("mul_cur", 0)}),
            positions=positions, layers=layers, schedule=schedule, final_norm=norm("final.norm"),
            head=PartSpec("linear_head", {"vocab_size": self.vocab, "hidden_size": E, "tensor": "head"}),
            eos_token_ids=list(self.eos_token_id))
        plan.validate()
        return plan


register_architecture("Peludra", PeludraConfig)
register_architecture("peludra", PeludraConfig)
