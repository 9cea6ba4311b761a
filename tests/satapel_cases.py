"""Shared by the Satapel tests: small configurations that differ from one another in every size and
constant, model folders with random weights scaled so that every mechanism matters to the logits
(sharp attention, norms around one, a router whose correction changes choices), the oracle's view of
a folder, and the comparison rules.

Tolerances, fixed before the first run: 32-bit: every row's error (root mean square over the
vocabulary) at most 2e-5 of the logits' root mean square; bfloat16: at most 4e-2 of it for at least
nine rows in ten (a router choice that bfloat16 rounding flips at one token is not a fault of a
mechanism; a wrong window, state or sink moves every row)."""
from __future__ import annotations

import json
import os
import random
from typing import Callable, Dict, Optional

import torch


def attention(heads, dim, rot_dim, vdim, rank, scale, window=None, rot_dims=None, base=10000.0, mlp="moe", **extra):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale,
         "rot": {"base": base, "dims": rot_dims or rot_dim}}
    if window:
        m["mask"] = {"size": window}
    return dict({"type": "latent_attention", "mixer": m, "mlp": mlp}, **extra)


def recurrence(heads, dim, decay_rank, mlp="moe", **extra):
    return dict({"type": "wkv", "mixer": {"heads": heads, "dim": dim, "decay_rank": decay_rank}, "mlp": mlp}, **extra)


def model(width, vocab, layers, moe=None, mult=0.7, eps=1e-5, buckets=97, mul_prev=31, mul_cur=7):
    out = []
    for layer in layers:
        layer = dict(layer)
        if layer["mlp"] == "moe":
            layer["mlp"] = moe
        out.append(layer)
    return {"architecture": "Satapel", "vocab": vocab, "width": width, "residual_mult": mult, "norm": {"eps": eps},
            "embedding": {"bigram": {"buckets": buckets, "mul_prev": mul_prev, "mul_cur": mul_cur}}, "layers": out}


def experts(n, identity, top, ff, limit=1.5):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": n, "identity": identity, "top": top}}


# attention first, a window shorter than two pages that is no multiple of anything, fewer rotated numbers than
# the rotated part holds, a shared layer in the middle, one layer without a feed-forward, an identity expert
CASE_A = model(72, 211, [attention(3, 16, 8, 24, 40, 2.5, window=70, rot_dims=4),
                         recurrence(3, 16, 12),
                         attention(3, 16, 8, 24, 40, 2.5, window=70, rot_dims=4, weights_of=0),
                         recurrence(2, 24, 5, mlp=None)],
               moe=experts(5, 1, 3, 56))
# recurrence first with one head, more heads than one block of the attention kernel takes, a window of 5,
# a layer that sees all keys, top-1 routing without identity experts, no clamp
CASE_B = model(64, 150, [recurrence(1, 32, 8),
                         attention(9, 8, 16, 8, 24, 3.0, window=5, base=500.0),
                         attention(2, 32, 4, 16, 48, 2.0, window=None, mlp=None),
                         recurrence(1, 32, 8, weights_of=0)],
               moe=experts(3, 0, 1, 40, limit=None), mult=1.0, eps=1e-6, buckets=13, mul_prev=5, mul_cur=3)
# a window of exactly one page and of exactly one key, a latent wider than a block's threads
CASE_C = model(80, 90, [attention(2, 16, 8, 16, 272, 0.15, window=64),
                        attention(4, 8, 8, 8, 16, 4.0, window=1),
                        recurrence(4, 8, 3)],
               moe=experts(2, 2, 2, 24, limit=0.8), mult=0.4)
# sizes that are multiples of nothing: no kernel that wants 16-byte rows can take them (width 100 is no multiple of
# 8, rows of 36 latent numbers, experts of 36, heads of 20), more identity experts than one, top 4 of 10
CASE_D = model(100, 77, [attention(5, 12, 6, 20, 30, 0.4, window=33),
                         recurrence(5, 20, 7),
                         recurrence(5, 20, 7, weights_of=1),
                         attention(5, 12, 6, 20, 30, 0.4, window=33, weights_of=0, mlp="moe")],
               moe=experts(7, 3, 4, 36, limit=1.1), mult=0.55, eps=3e-5, buckets=10, mul_prev=3, mul_cur=1)
# wider layers: two head groups, latents of 200 and 520 numbers (the attention kernel's other column counts), a
# window longer than four pages, recurrence heads of 64 and 128, experts of several feature tiles
CASE_E = model(256, 500, [attention(16, 16, 16, 24, 200, 0.3, window=300),
                          recurrence(2, 64, 16),
                          attention(4, 32, 8, 40, 520, 0.25, window=None),
                          recurrence(1, 128, 8, mlp=None)],
               moe=experts(6, 1, 2, 264, limit=2.5), mult=0.5)
CASES = {"A": (CASE_A, 11), "B": (CASE_B, 12), "C": (CASE_C, 13), "D": (CASE_D, 14), "E": (CASE_E, 15)}


def _scaled(name: str, t: torch.Tensor) -> torch.Tensor:
    t = t.float()
    if name.endswith(("norm1", "norm2", "final.norm", "dkv.norm", "mix.norm")):
        return 1.0 + t
    if name in ("embed", "bigram"):
        return t * 25.0
    if name == "head":
        return t * 10.0
    if name.endswith(("mix.q", "mix.dkv")):
        return t * 6.0
    if name.endswith("mix.o"):
        return t * 5.0
    if name.endswith((".gate", ".up", ".down", "mix.uk", "mix.uv", "mix.r", "mix.k", "mix.v", "mix.g")):
        return t * 3.0
    if name.endswith("correction"):
        return t * 4.0
    return t


def make_folder(tmp_path, raw: dict, seed: int, name: str = "m", edit: Optional[Callable[[Dict[str, torch.Tensor]], None]] = None) -> str:
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


def oracle_view(folder: str):
    """(config dict, weights as float64 CPU tensors), read with the safetensors package."""
    import safetensors.torch as st
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    w = {k: v.to(torch.float64) for k, v in st.load_file(os.path.join(folder, "model.safetensors")).items()}
    return cfg, w


def tokens(seed: int, n: int, vocab: int):
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(n)]


def row_errors(got: torch.Tensor, want: torch.Tensor) -> torch.Tensor:
    got, want = got.detach().double().cpu(), want.detach().double().cpu()
    assert got.shape == want.shape, f"shape {tuple(got.shape)} vs {tuple(want.shape)}"
    return (got - want).pow(2).mean(-1).sqrt() / want.pow(2).mean().sqrt()


def assert_rows(got, want, dtype: str, what: str = ""):
    e = row_errors(got, want)
    if dtype == "float32":
        assert float(e.max()) <= 2e-5, f"{what}: row {int(e.argmax())} is off by {float(e.max()):.2e} of the logits' size"
    else:
        ok = (e <= 4e-2).double().mean()
        assert float(ok) >= 0.9, f"{what}: only {float(ok):.2f} of the rows are within 4e-2 (worst {float(e.max()):.2e})"
