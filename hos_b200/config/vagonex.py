"""Typed configuration of Vagonex: a decoder-only model with the norm after the residual sum, whose layers are
listed one by one in config.json, each with its kind of mixer, the mixer's sizes and its feed-forward.

    {"architecture": "Vagonex", "vocab": V, "width": D, "postln_alpha": a, "norm": {"eps": e},
     "embedding": {"scale": s},
     "layers": [{"type": "attention",
                 "mixer": {"heads": H, "kv_heads": G, "dim": d, "vdim": v, "scale": s, "mask": {"size": C},
                           "rot": {"base": b, "dims": r, "scaling": {"factor": f, "original": n, "fast": x, "slow": y}},
                           "kv_from": j},
                 "mlp": MLP or null},
                {"type": "lightning", "mixer": {"heads": H, "dim": d, "vdim": v, "decay": [one per head]}, "mlp": ...},
                {"type": "delta", "mixer": {"heads": H, "kv_heads": G, "dim": d, "vdim": v, "conv": taps}, "mlp": ...}]}
    MLP = {"kind": "dense", "ff": F}

`mask`, `rot`, `rot.scaling` and `kv_from` may be absent (no chunks, no rotation, unscaled frequencies, keys and
values of the layer's own).  A layer with "kv_from": j has no key or value tensors and reads layer j's.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, Mapping, Tuple

from ..errors import MissingMetaError
from .base import ConfigReader, ModelConfig

MIXER_TYPES = ("attention", "lightning", "delta")


def _section(raw: Mapping[str, Any], key: str, where: str) -> Mapping[str, Any]:
    v = raw.get(key)
    if not isinstance(v, dict):
        raise MissingMetaError(f"missing model metadata: {where}{key} (an object is required)")
    return v


def _bad(msg: str):
    raise MissingMetaError("model metadata invalid: " + msg)


@dataclass(frozen=True)
class VagonexConfig(ModelConfig):
    vocab: int
    width: int
    postln_alpha: float
    norm_eps: float
    embedding_scale: float
    layers: Tuple[Mapping[str, Any], ...]      # the entries as config.json has them, checked

    architecture = "Vagonex"

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "VagonexConfig":
        r = ConfigReader(raw)
        norm = ConfigReader(_section(raw, "norm", ""))
        emb = ConfigReader(raw.get("embedding") if isinstance(raw.get("embedding"), dict) else {})
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise MissingMetaError("missing model metadata: layers (a list of layers is required)")
        eps = norm.opt_float("eps", None)
        if eps is None:
            raise MissingMetaError("missing model metadata: norm.eps")
        cfg = cls(vocab=r.need_int("vocab"), width=r.need_int("width"), postln_alpha=r.opt_float("postln_alpha", 1.0),
                  norm_eps=eps, embedding_scale=emb.opt_float("scale", 1.0),
                  layers=tuple(copy.deepcopy(l) for l in layers))
        cfg.check()
        return cfg

    def check(self) -> None:
        for key in ("vocab", "width"):
            if getattr(self, key) <= 0:
                _bad(f"{key} must be positive")
        if not self.norm_eps > 0.0:
            _bad("norm.eps must be positive")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]."
            if not isinstance(layer, dict):
                _bad(f"layers[{i}] must be an object")
            kind = layer.get("type")
            if kind not in MIXER_TYPES:
                _bad(f"{where}type must be one of {MIXER_TYPES}, found {kind!r}")
            m = ConfigReader(_section(layer, "mixer", where))
            for key in ("heads", "dim", "vdim"):
                if m.need_int(key) <= 0:
                    _bad(f"{where}mixer.{key} must be positive")
            if kind in ("attention", "delta"):
                g = m.need_int("kv_heads")
                if g <= 0 or m.need_int("heads") % g != 0:
                    _bad(f"{where}mixer.heads must be a multiple of mixer.kv_heads")
            if kind == "attention":
                self._check_attention(i, layer["mixer"], m, where)
            elif kind == "lightning":
                decay = layer["mixer"].get("decay")
                if not isinstance(decay, list) or len(decay) != m.need_int("heads") \
                        or not all(isinstance(d, (int, float)) and not isinstance(d, bool) for d in decay):
                    _bad(f"{where}mixer.decay must list one number per head")
            else:
                if m.need_int("conv") <= 0:
                    _bad(f"{where}mixer.conv must be positive")
            mlp = layer.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
                    _bad(f"{where}mlp.kind must be 'dense' (or mlp null)")
                if ConfigReader(mlp).need_int("ff") <= 0:
                    _bad(f"{where}mlp.ff must be positive")

    def _check_attention(self, i: int, mixer, m: ConfigReader, where: str) -> None:
        if m.opt_float("scale", None) is None:
            _bad(f"{where}mixer.scale is required")
        rot = mixer.get("rot")
        if rot is not None:
            rr = ConfigReader(rot)
            dims = rr.need_int("dims")
            if dims <= 0 or dims % 2 or dims > m.need_int("dim") or not rr.opt_float("base", 0.0) > 1.0:
                _bad(f"{where}mixer.rot needs a base above 1 and an even dims of at most dim")
            sc = rot.get("scaling")
            if sc is not None:
                s = ConfigReader(sc)
                if not all((s.opt_float(k, 0.0) or 0.0) > 0.0 for k in ("factor", "original", "fast", "slow")):
                    _bad(f"{where}mixer.rot.scaling needs positive factor, original, fast and slow")
        mask = mixer.get("mask")
        if mask is not None and ConfigReader(mask).need_int("size") <= 0:
            _bad(f"{where}mixer.mask.size must be positive")
        j = mixer.get("kv_from")
        if j is not None:
            if isinstance(j, bool) or not isinstance(j, int) or not 0 <= j < i:
                _bad(f"{where}mixer.kv_from must name an earlier layer")
            other = self.layers[j]
            if other.get("type") != "attention" or other["mixer"].get("kv_from") is not None:
                _bad(f"{where}mixer.kv_from names layer {j}, which keeps no keys and values of its own")
            for key in ("kv_heads", "dim", "vdim"):
                if other["mixer"].get(key) != mixer.get(key):
                    _bad(f"{where}mixer.{key} differs from layer {j}'s, whose keys and values it reads")

    def to_dict(self) -> Dict[str, Any]:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "postln_alpha": self.postln_alpha, "norm": {"eps": self.norm_eps},
                "embedding": {"scale": self.embedding_scale},
                "layers": [copy.deepcopy(dict(l)) for l in self.layers]}
