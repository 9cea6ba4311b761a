"""Typed configuration of Satapel: a decoder-only model whose layers are listed one by one in
config.json, each with its kind of mixer, the mixer's sizes and its feed-forward.

    {"architecture": "Satapel", "vocab": V, "width": D, "residual_mult": m, "norm": {"eps": e},
     "embedding": {"bigram": {"buckets": B, "mul_prev": a, "mul_cur": b}},
     "layers": [{"type": "wkv", "mixer": {"heads": H, "dim": d}, "mlp": MLP or null},
                {"type": "latent_attention",
                 "mixer": {"heads": H, "dim": d, "rot_dim": r, "vdim": v, "kv_rank": R, "scale": s,
                           "mask": {"size": W}, "rot": {"base": b, "dims": r}}, "mlp": MLP or null},
                {... , "weights_of": j}, ...]}
    MLP = {"kind": "moe", "expert": {"ff": F, "limit": L}, "router": {"experts": E, "identity": I, "top": K}}

A layer with "weights_of": j has no tensors of its own: it runs layer j's mixer, feed-forward and
norms with a cache or state of its own.  The rank of the wkv decay's low-rank projection is not a
key of the format: it is the shape of the layer's `mix.w1` tensor; `decay_rank` may be given beside
`heads` and `dim` (the random-weights mode writes it, since it has no tensor to read it from).
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, List, Mapping, Optional, Tuple

from ..errors import MissingMetaError
from .base import ConfigReader, ModelConfig

MIXER_TYPES = ("wkv", "latent_attention")


def _section(raw: Mapping[str, Any], key: str, where: str) -> Mapping[str, Any]:
    v = raw.get(key)
    if not isinstance(v, dict):
        raise MissingMetaError(f"missing model metadata: {where}{key} (an object is required)")
    return v


@dataclass(frozen=True)
class SatapelConfig(ModelConfig):
    vocab: int
    width: int
    residual_mult: float
    norm_eps: float
    bigram_buckets: int
    bigram_mul_prev: int
    bigram_mul_cur: int
    layers: Tuple[Mapping[str, Any], ...]      # the entries as config.json has them, checked

    architecture = "Satapel"

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "SatapelConfig":
        r = ConfigReader(raw)
        big = ConfigReader(_section(_section(raw, "embedding", ""), "bigram", "embedding."))
        norm = ConfigReader(_section(raw, "norm", ""))
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise MissingMetaError("missing model metadata: layers (a list of layers is required)")
        eps = norm.opt_float("eps", None)
        if eps is None:
            raise MissingMetaError("missing model metadata: norm.eps")
        cfg = cls(vocab=r.need_int("vocab"), width=r.need_int("width"),
                  residual_mult=r.opt_float("residual_mult", 1.0), norm_eps=eps,
                  bigram_buckets=big.need_int("buckets"), bigram_mul_prev=big.need_int("mul_prev"),
                  bigram_mul_cur=big.need_int("mul_cur"), layers=tuple(copy.deepcopy(l) for l in layers))
        cfg.check()
        return cfg

    def check(self) -> None:
        def bad(msg: str):
            raise MissingMetaError("model metadata invalid: " + msg)
        for key in ("vocab", "width", "bigram_buckets"):
            if getattr(self, key) <= 0:
                bad(f"{key} must be positive")
        if not self.norm_eps > 0.0:
            bad("norm.eps must be positive")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]."
            if not isinstance(layer, dict):
                bad(f"layers[{i}] must be an object")
            if layer.get("type") not in MIXER_TYPES:
                bad(f"{where}type must be one of {MIXER_TYPES}, found {layer.get('type')!r}")
            m = ConfigReader(_section(layer, "mixer", where))
            for key in ("heads", "dim"):
                if m.need_int(key) <= 0:
                    bad(f"{where}mixer.{key} must be positive")
            if layer["type"] == "latent_attention":
                for key in ("rot_dim", "vdim", "kv_rank"):
                    if m.need_int(key) <= 0:
                        bad(f"{where}mixer.{key} must be positive")
                if m.opt_float("scale", None) is None:
                    bad(f"{where}mixer.scale is required")
                rot = layer["mixer"].get("rot")
                if rot is not None:
                    rr = ConfigReader(rot)
                    dims = rr.need_int("dims")
                    if dims <= 0 or dims % 2 or dims > m.need_int("rot_dim") or not rr.opt_float("base", 0.0) > 0.0:
                        bad(f"{where}mixer.rot needs a positive base and an even dims of at most rot_dim")
                mask = layer["mixer"].get("mask")
                if mask is not None and ConfigReader(mask).need_int("size") <= 0:
                    bad(f"{where}mixer.mask.size must be positive")
            mlp = layer.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") != "moe":
                    bad(f"{where}mlp.kind must be 'moe' (or mlp null)")
                ex, ro = ConfigReader(_section(mlp, "expert", where + "mlp.")), ConfigReader(_section(mlp, "router", where + "mlp."))
                n_all = ro.need_int("experts") + ro.opt_int("identity", 0)
                if ex.need_int("ff") <= 0 or ro.need_int("experts") < 0 or not 0 < ro.need_int("top") <= n_all:
                    bad(f"{where}mlp sizes are inconsistent")
            j = layer.get("weights_of")
            if j is not None:
                if isinstance(j, bool) or not isinstance(j, int) or not 0 <= j < len(self.layers) or j == i:
                    bad(f"{where}weights_of must name another layer")
                if self.layers[j].get("weights_of") is not None:
                    bad(f"{where}weights_of names layer {j}, which has no tensors of its own")
                if self.layers[j].get("type") != layer["type"]:
                    bad(f"{where}weights_of names a layer of another type")

    def owner_of(self, i: int) -> int:
        """The layer whose tensors layer i uses (itself unless it has `weights_of`)."""
        j = self.layers[i].get("weights_of")
        return i if j is None else int(j)

    def to_dict(self) -> Dict[str, Any]:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "residual_mult": self.residual_mult, "norm": {"eps": self.norm_eps},
                "embedding": {"bigram": {"buckets": self.bigram_buckets, "mul_prev": self.bigram_mul_prev,
                                         "mul_cur": self.bigram_mul_cur}},
                "layers": [copy.deepcopy(dict(l)) for l in self.layers]}
