"""Manapel: a decoder whose config.json lists its layers one by one.

Top-level keys: ``architecture`` ("Manapel"), ``vocab``, ``width``, ``logit_scale``, ``norm`` ({``eps``}) and
``layers``.  A layer entry has ``type`` (the kind of mixer; "attention"), ``mixer`` (its sizes) and ``mlp`` (its
feed-forward, or null for none):

* mixer "attention": ``heads``, ``kv_heads``, ``dim`` (query/key head), ``vdim`` (value head), ``scale`` (factor on the
  scores), ``rot`` ({``dims``, ``base``}: rotation of the first ``dims`` dimensions of each head, half-split pairs) and
  optionally ``kv_from`` (the index of an earlier layer whose keys and values this layer attends over; it then has no
  key and value projections).  Projections carry biases; queries and keys are divided by their root mean square per
  head after the rotation, with ``norm.eps``.
* mlp ``kind`` "dense": ``ff``; gated, ``down(relu(gate x) * up x)``.
* mlp ``kind`` "moe": ``router`` ({``experts``, ``top``}), ``expert`` ({``ff``}) and optionally ``shared`` ({``ff``});
  experts are ``down(relu(up x)^2)``; the router has a bias.

Every norm is a Dynamic Tanh and stands on both sides of each sublayer.  Tensor names: ``embed``, ``l<i>.norm1`` /
``norm1b`` / ``norm2`` / ``norm2b`` (with ``.b`` and ``.alpha``), ``l<i>.mix.{q,k,v,o}`` (biases ``.b``),
``l<i>.mlp.{gate,up,down}`` or ``l<i>.mlp.router`` (``.b``), ``l<i>.mlp.e<j>.{up,down}``, ``l<i>.mlp.shared.{up,down}``,
``final.norm``, ``head``.

config.json gives no context length: ``max_positions`` (optional key, default below) bounds the rotary table and a
request's length in this engine.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Dict, List

from .base import (ConfigError, LayerSpec, ModelConfig, ModelPlan, PartSpec, ScheduleEntry, UnsupportedError,
                   take_float, take_int)
from .registry import register_architecture

DEFAULT_MAX_POSITIONS = 1 << 16


def _obj(d: Dict[str, Any], key: str, where: str, required: bool = True):
    v = d.get(key)
    if v is None:
        if required:
            raise ConfigError(f"config.json: {where}'{key}' is missing")
        return None
    if not isinstance(v, dict):
        raise ConfigError(f"config.json: {where}'{key}' must be an object")
    return v


@dataclass
class ManapelConfig(ModelConfig):
    vocab: int = 0
    width: int = 0
    logit_scale: float = 1.0
    norm_eps: float = 1e-5
    max_positions: int = DEFAULT_MAX_POSITIONS
    layers: List[Dict[str, Any]] = field(default_factory=list)
    eos_token_id: List[int] = field(default_factory=list)

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "ManapelConfig":
        V = take_int(d, "vocab", lo=1)
        E = take_int(d, "width", lo=1, hi=1_000_000)
        norm = _obj(d, "norm", "")
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        out = []
        for i, L in enumerate(layers):
            w = f"layers[{i}]: "
            if not isinstance(L, dict):
                raise ConfigError(f"config.json: {w}must be an object")
            kind = L.get("type")
            if kind != "attention":
                raise UnsupportedError(f"config.json: {w}mixer type '{kind}' is not supported (known: attention)")
            m = _obj(L, "mixer", w)
            H, G = take_int(m, "heads", lo=1), take_int(m, "kv_heads", lo=1)
            if H % G:
                raise UnsupportedError(f"config.json: {w}unsupported attention geometry: {H} heads over {G} key/value heads")
            dim, vdim = take_int(m, "dim", lo=1), take_int(m, "vdim", lo=1)
            take_float(m, "scale")
            rot = _obj(m, "rot", w, required=False)
            if rot is not None:
                rd = take_int(rot, "dims", lo=0)
                if rd % 2 or rd > dim:
                    raise UnsupportedError(f"config.json: {w}rot.dims {rd} must be even and at most dim {dim}")
                take_float(rot, "base", lo=0.0)
            src = m.get("kv_from")
            if src is not None:
                src = take_int(m, "kv_from", lo=0)
                if src >= i or out[src]["mixer"].get("kv_from") is not None:
                    raise ConfigError(f"config.json: {w}kv_from {src} must name an earlier layer with keys and values of its own")
                o = out[src]["mixer"]
                if (o["kv_heads"], o["dim"], o["vdim"]) != (G, dim, vdim):
                    raise ConfigError(f"config.json: {w}kv_from {src}: that layer's key/value heads have other sizes")
            mlp = _obj(L, "mlp", w, required=False)
            if mlp is not None:
                mk = mlp.get("kind")
                if mk == "dense":
                    take_int(mlp, "ff", lo=1)
                elif mk == "moe":
                    r = _obj(mlp, "router", w)
                    n, top = take_int(r, "experts", lo=1), take_int(r, "top", lo=1)
                    if top > n:
                        raise ConfigError(f"config.json: {w}router.top {top} exceeds router.experts {n}")
                    take_int(_obj(mlp, "expert", w), "ff", lo=1)
                    sh = _obj(mlp, "shared", w, required=False)
                    if sh is not None:
                        take_int(sh, "ff", lo=1)
                else:
                    raise UnsupportedError(f"config.json: {w}mlp kind '{mk}' is not supported (known: dense, moe)")
            out.append(copy.deepcopy(L))
        eos = d.get("eos_token_id", [])
        eos = [] if eos is None else ([eos] if isinstance(eos, int) else list(eos))
        return cls(vocab=V, width=E, logit_scale=take_float(d, "logit_scale", 1.0),
                   norm_eps=take_float(norm, "eps", 1e-5, lo=0.0),
                   max_positions=take_int(d, "max_positions", default=DEFAULT_MAX_POSITIONS, lo=1), layers=out, eos_token_id=eos)

    def to_dict(self) -> Dict[str, Any]:
        d = {"architecture": self.architecture or "Manapel", "vocab": self.vocab, "width": self.width,
             "logit_scale": self.logit_scale, "norm": {"eps": self.norm_eps}, "layers": copy.deepcopy(self.layers)}
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            d["max_positions"] = self.max_positions
        if self.eos_token_id:
            d["eos_token_id"] = list(self.eos_token_id)
        return d

    def plan(self) -> ModelPlan:
        E = self.width
        dyt = lambda name, optional=False: PartSpec("dynamic_tanh", {"size": E, "tensor": name, "optional": optional})
        positions: Dict[str, PartSpec] = {}
        layers, schedule = [], []
        for i, L in enumerate(self.layers):
            p, m, mlp = f"l{i}", L["mixer"], L.get("mlp")
            rot = m.get("rot")
            pos_name = None
            if rot and rot["dims"] > 0:
                # layers with the same rotation share one table
                pos_name = f"rot{rot['dims']}_{rot['base']!r}"
                positions.setdefault(pos_name, PartSpec("rotary", {"head_dim": m["dim"], "n_rot": rot["dims"],
                                                                   "theta": float(rot["base"]), "pairing": "half"}))
            shared_from = m.get("kv_from")
            mixer = PartSpec("paged_attention", {
                "hidden_size": E, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
                "v_head_dim": m["vdim"], "scale": float(m["scale"]), "qk_norm_eps": self.norm_eps,
                "own_kv": shared_from is None, "qkv_bias": True, "out_bias": False, "window": 0, "position": pos_name,
                "prefix": f"{p}.mix", "names": {"q": "q", "k": "k", "v": "v", "o": "o"}, "weight_suffix": "", "bias_suffix": ".b"})
            if mlp is None:
                ffn = None
            elif mlp["kind"] == "dense":
                ffn = PartSpec("gated", {"hidden_size": E, "intermediate_size": mlp["ff"], "prefix": f"{p}.mlp",
                                         "activation": "relu", "names": {"gate": "gate", "up": "up", "down": "down"}})
            else:
                ffn = PartSpec("moe", {"hidden_size": E, "experts": mlp["router"]["experts"], "top": mlp["router"]["top"],
                                       "expert_size": mlp["expert"]["ff"], "activation": "relu2", "router_bias": True,
                                       "shared_size": (mlp.get("shared") or {}).get("ff", 0), "prefix": f"{p}.mlp"})
            layers.append(LayerSpec(
                prefix=p, block=PartSpec("sandwich_residual"), norm1=dyt(f"{p}.norm1"), mixer=mixer,
                post_norm1=dyt(f"{p}.norm1b"),
                # a layer without a feed-forward needs no norms around one; a file that carries them anyway is accepted
                norm2=dyt(f"{p}.norm2", optional=ffn is None), ffn=ffn, post_norm2=dyt(f"{p}.norm2b", optional=ffn is None)))
            schedule.append(ScheduleEntry(i, cache_of=shared_from))
        plan = ModelPlan(
            hidden_size=E, vocab_size=self.vocab, max_positions=self.max_positions,
            embedding=PartSpec("embedding", {"vocab_size": self.vocab, "hidden_size": E, "tensor": "embed"}),
            positions=positions, layers=layers, schedule=schedule, final_norm=dyt("final.norm"),
            head=PartSpec("linear_head", {"vocab_size": self.vocab, "hidden_size": E, "tensor": "head",
                                          "scale": self.logit_scale}),
            eos_token_ids=list(self.eos_token_id))
        plan.validate()
        return plan


register_architecture("Manapel", ManapelConfig)
register_architecture("manapel", ManapelConfig)
