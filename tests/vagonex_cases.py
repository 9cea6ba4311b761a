"""Shared by the Vagonex tests: small configurations that differ from one another in every size and constant,
model folders with random weights scaled so that every mechanism matters to the logits (sharp attention, sinks of
the scores' size, norms around one, decays between nothing and everything), and the comparison rules.  The scales are small enough that 32-bit rounding alone (the oracle run in 32-bit against itself
in 64-bit) stays below 4e-6 of the logits' size, and large enough that a chunk that is off by one, a sink that is
left out or a state that is lost moves the logits by more than 2e-3 of it.

Tolerances, fixed before the first run: 32-bit: every row's error (root mean square over the vocabulary) at most
2e-5 of the logits' root mean square; bfloat16: at most 4e-2 of it for at least nine rows in ten."""
from __future__ import annotations

import json
import os
from typing import Callable, Dict, Optional

import torch

from satapel_cases import assert_rows, oracle_view, row_errors, tokens  # noqa: F401  (the rules are the same)


def attention(heads, kv_heads, dim, vdim, scale, chunk=None, rot_dims=None, base=10000.0, scaling=None, kv_from=None,
              mlp="dense"):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if rot_dims:
        m["rot"] = {"base": base, "dims": rot_dims}
        if scaling:
            m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    if chunk:
        m["mask"] = {"size": chunk}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m, "mlp": mlp}


def lightning(heads, dim, vdim, decay, mlp="dense"):
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}, "mlp": mlp}


def delta(heads, kv_heads, dim, vdim, conv, mlp="dense"):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}, "mlp": mlp}


def model(width, vocab, layers, ff=48, alpha=1.0, eps=1e-6, emb_scale=1.0):
    out = []
    for layer in layers:
        layer = json.loads(json.dumps(layer))
        if layer["mlp"] == "dense":
            layer["mlp"] = {"kind": "dense", "ff": ff}
        out.append(layer)
    return {"architecture": "Vagonex", "vocab": vocab, "width": width, "postln_alpha": alpha, "norm": {"eps": eps},
            "embedding": {"scale": emb_scale}, "layers": out}


# attention first: one kv head for three query heads, values wider than keys, chunks of 70 (no multiple of a page),
# 8 of 16 numbers rotated with a ramp that is cut at both ends; a delta layer with two key heads for four; a decay
# layer; a layer that reads layer 0's keys and values; a delta layer without a feed-forward
CASE_A = model(72, 211, [attention(3, 1, 16, 24, 0.8, chunk=70, rot_dims=8, scaling=(8.0, 64, 16.0, 2.0)),
                         delta(4, 2, 16, 8, 3),
                         lightning(3, 8, 16, (0.5, 0.9, 0.99)),
                         attention(3, 1, 16, 24, 0.6, chunk=70, rot_dims=8, scaling=(8.0, 64, 16.0, 2.0), kv_from=0),
                         delta(2, 2, 24, 12, 2, mlp=None)], ff=56, alpha=1.7, emb_scale=3.0)
# a decay layer first with one head; nine heads over three kv heads with chunks of 5 and unscaled frequencies; a layer
# that sees all keys without any rotation, read by two later layers with layers in between
CASE_B = model(64, 150, [lightning(1, 32, 32, (0.97,)),
                         attention(9, 3, 8, 8, 1.2, chunk=5, rot_dims=8, base=500.0),
                         attention(2, 2, 32, 16, 0.4, mlp=None),
                         delta(1, 1, 32, 48, 1),
                         attention(2, 2, 32, 16, 0.5, kv_from=2),
                         attention(2, 2, 32, 16, 0.3, chunk=33, kv_from=2, mlp=None)], ff=40, alpha=1.0, eps=1e-5)
# chunks of exactly one page and of exactly one key; a delta layer first; seven taps; keys wider than values
CASE_C = model(80, 90, [delta(3, 3, 8, 16, 7),
                        attention(2, 1, 40, 16, 0.3, chunk=64, rot_dims=40, base=30000.0, scaling=(3.0, 96, 24.0, 1.5)),
                        attention(4, 4, 8, 8, 1.5, chunk=1, rot_dims=2),
                        lightning(4, 16, 8, (0.2, 0.7, 1.0, 0.999))], ff=24, alpha=0.6, emb_scale=0.5)
# sizes that are multiples of nothing (a width of 100 is no multiple of 8: the tensor-core products step aside)
CASE_D = model(100, 77, [attention(5, 5, 12, 20, 0.7, chunk=33, rot_dims=6, scaling=(2.0, 40, 4.0, 1.0)),
                         delta(6, 2, 20, 12, 4),
                         lightning(5, 12, 20, (0.6, 0.8, 0.9, 0.95, 0.99)),
                         attention(5, 5, 12, 20, 0.7, chunk=33, rot_dims=6, scaling=(2.0, 40, 4.0, 1.0), kv_from=0)],
               ff=36, alpha=2.2, eps=3e-5, emb_scale=10.0)
# wider layers: chunks longer than four pages (decoding cuts a row's keys into shares), heads of 64/128 numbers,
# state rows cut over 8 and 16 threads, value columns over several blocks
CASE_E = model(256, 500, [attention(16, 4, 64, 128, 0.25, chunk=300, rot_dims=32, scaling=(4.0, 256, 32.0, 1.0)),
                          delta(8, 4, 128, 64, 4),
                          lightning(4, 96, 160, (0.9, 0.99, 0.995, 0.999)),
                          attention(16, 4, 64, 128, 0.25, kv_from=0, rot_dims=32, scaling=(4.0, 256, 32.0, 1.0))],
               ff=264, alpha=2.5, emb_scale=16.0)
CASES = {"A": (CASE_A, 21), "B": (CASE_B, 22), "C": (CASE_C, 23), "D": (CASE_D, 24), "E": (CASE_E, 25)}


def _scaled(name: str, t: torch.Tensor) -> torch.Tensor:
    t = t.float()
    if name.endswith(("norm1", "norm2", "final.norm", "q.norm", "k.norm", "mix.norm")):
        return 1.0 + t
    if name == "embed":
        return t * 25.0
    if name.endswith(("mix.o", "mlp.down")):
        return t * 8.0
    if name.endswith(("mix.q", "mix.k", "mix.v", "mix.g", "mlp.gate", "mlp.up", "mix.b", "mix.a")):
        return t * 3.0
    if name.endswith("sink"):
        return t * 3.0
    return t


def make_folder(tmp_path, raw: dict, seed: int, name: str = "m",
                edit: Optional[Callable[[Dict[str, torch.Tensor]], None]] = None) -> str:
    from hos_b200.model import weight_specs_for
    from hos_b200.registry import config_from_dict
    from hos_b200.weights import RandomSource
    from hos_b200.weights.safetensors import SINGLE_FILE, write_safetensors
    cfg = config_from_dict(raw)
    src = RandomSource(weight_specs_for(cfg), seed)
    tensors = {n: _scaled(n, src.read(n)) for n in src.names()}
    if edit is not None:
        edit(tensors)
    d = os.path.join(str(tmp_path), name)
    os.makedirs(d, exist_ok=True)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg.to_dict(), f)
    write_safetensors(os.path.join(d, SINGLE_FILE), ((n, t.to(torch.bfloat16)) for n, t in tensors.items()),
                      metadata={"format": "pt"})
    return d
