"""Vagonex in plain, slow PyTorch (float64, whole sequences, loops): the oracle of the tests.

One function per mechanism, written from the design's equations; nothing here is shared with the
library.  A model is (cfg, w): cfg the dict that config.json holds, w a dict of float64 tensors by
checkpoint name.

  rms                 x / sqrt(mean(x^2) + eps)
  rotary_table        per-pair frequencies with the long-context ramp, and the factor on cos and sin
  rotate_pairs        (u, v) -> (u cos - v sin, v cos + u sin) on pairs (2i, 2i+1)
  softmax_mixer       biased q/k/v, per-head q/k norm, rotation, chunk mask, sink, per-head gate
  lightning_mixer     S <- decay S + k v^T;  o = S^T q;  norm over all heads, sigmoid gate
  delta_mixer         short convolutions, unit q/k, S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q
  dense_ff            down(gelu_tanh(gate h) * up h)
  forward_logits      x <- norm1(alpha x + mixer(x)); x <- norm2(alpha x + ff(x)) per layer
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F = torch.float64


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(x):
    return x / (1.0 + torch.exp(-x))


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rotary_table(rot):
    """(frequency per pair, factor on cos and sin)."""
    dims, base = rot["dims"], rot["base"]
    freqs = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if not sc:
        return freqs, 1.0

    def turn_dim(t):
        return dims * math.log(sc["original"] / (2.0 * math.pi * t)) / (2.0 * math.log(base))
    lo = max(math.floor(turn_dim(sc["fast"])), 0)
    hi = min(math.ceil(turn_dim(sc["slow"])), dims - 1)
    out = []
    for i, f in enumerate(freqs):
        ramp = min(1.0, max(0.0, (i - lo) / max(hi - lo, 0.001)))
        out.append(f / sc["factor"] * ramp + f * (1.0 - ramp))
    return out, 0.1 * math.log(sc["factor"]) + 1.0


def rotate_pairs(v, positions, rot):
    """v: [T, heads, n]; the first rot.dims of the last axis are rotated, the rest pass."""
    if not rot:
        return v
    freqs, mult = rotary_table(rot)
    out = v.clone()
    for t, p in enumerate(positions):
        for i, f in enumerate(freqs):
            c, s = math.cos(p * f) * mult, math.sin(p * f) * mult
            x, y = v[t, :, 2 * i], v[t, :, 2 * i + 1]
            out[t, :, 2 * i] = x * c - y * s
            out[t, :, 2 * i + 1] = y * c + x * s
    return out


def softmax_keys_values(m, eps, w, p, h):
    """The keys (normed, rotated) and values that a layer with projections of its own makes: [T, G, dim], [T, G, vdim]."""
    T, G, d, vd = h.shape[0], m["kv_heads"], m["dim"], m["vdim"]
    k = (h @ w[p + "k"].T + w[p + "k.b"]).view(T, G, d)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).view(T, G, vd)
    k = rms(k, eps) * w[p + "k.norm"]
    return rotate_pairs(k, range(T), m.get("rot")), v


def softmax_mixer(m, eps, w, p, h, keys, values, use_sink=True, chunk_override=None, drop_far=None):
    """keys, values: this layer's own or the ones of the layer it reads.  `chunk_override`, `use_sink`, `drop_far`
    (keys more than that many positions back are left out) let a test show that a mechanism matters."""
    T, H, G, d, vd = h.shape[0], m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T + w[p + "q.b"]).view(T, H, d)
    q = rotate_pairs(rms(q, eps) * w[p + "q.norm"], range(T), m.get("rot"))
    gate = torch.sigmoid(h @ w[p + "g"].T)                      # [T, H]
    size = chunk_override if chunk_override is not None else (m["mask"]["size"] if m.get("mask") else None)
    out = torch.zeros(T, H, vd, dtype=F)
    for t in range(T):
        first = (t // size) * size if size else 0
        if drop_far is not None:
            first = max(first, t - drop_far)
        for hd in range(H):
            g = hd // (H // G)
            s = (keys[first:t + 1, g] @ q[t, hd]) * m["scale"]
            top = max(float(s.max()), float(w[p + "sink"][hd])) if use_sink else float(s.max())
            e = torch.exp(s - top)
            den = e.sum() + (math.exp(float(w[p + "sink"][hd]) - top) if use_sink else 0.0)
            out[t, hd] = (e / den) @ values[first:t + 1, g] * gate[t, hd]
    return out.reshape(T, H * vd) @ w[p + "o"].T


def lightning_mixer(m, eps, w, p, h):
    T, H, d, vd = h.shape[0], m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w[p + "q"].T).view(T, H, d)
    k = silu(h @ w[p + "k"].T).view(T, H, d)
    v = silu(h @ w[p + "v"].T).view(T, H, vd)
    S = torch.zeros(H, d, vd, dtype=F)
    o = torch.zeros(T, H, vd, dtype=F)
    for t in range(T):
        for hd in range(H):
            S[hd] = m["decay"][hd] * S[hd] + torch.outer(k[t, hd], v[t, hd])
            o[t, hd] = S[hd].T @ q[t, hd]
    y = rms(o.reshape(T, H * vd), eps) * w[p + "norm"] * torch.sigmoid(h @ w[p + "g"].T)
    return y @ w[p + "o"].T


def short_conv(x, taps_w):
    """x: [T, C]; taps_w: [C, taps], the last column is the current token's; zeros before the start."""
    T, taps = x.shape[0], taps_w.shape[1]
    y = torch.zeros_like(x)
    for t in range(T):
        for j in range(taps):
            src = t - (taps - 1) + j
            if src >= 0:
                y[t] += taps_w[:, j] * x[src]
    return y


def delta_mixer(m, eps, w, p, h):
    T, H, G, d, vd = h.shape[0], m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_conv(h @ w[p + "q"].T, w[p + "q.conv"])).view(T, G, d)
    k = silu(short_conv(h @ w[p + "k"].T, w[p + "k.conv"])).view(T, G, d)
    v = silu(short_conv(h @ w[p + "v"].T, w[p + "v.conv"])).view(T, H, vd)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[p + "b"].T)                                                    # [T, H]
    decay = torch.exp(-torch.exp(w[p + "A_log"]) * torch.nn.functional.softplus(h @ w[p + "a"].T + w[p + "dt_bias"]))
    S = torch.zeros(H, d, vd, dtype=F)
    o = torch.zeros(T, H, vd, dtype=F)
    for t in range(T):
        for hd in range(H):
            g = hd // (H // G)
            S[hd] = decay[t, hd] * S[hd]
            u = beta[t, hd] * (v[t, hd] - S[hd].T @ k[t, g])
            S[hd] = S[hd] + torch.outer(k[t, g], u)
            o[t, hd] = S[hd].T @ q[t, g]
    y = rms(o, eps) * w[p + "norm"] * silu(h @ w[p + "g"].T).view(T, H, vd)
    return y.reshape(T, H * vd) @ w[p + "o"].T


def dense_ff(w, p, h):
    return (gelu_tanh(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def forward_hidden(cfg, w, tokens: List[int], taps: Optional[list] = None, **attn_kw):
    """The residual stream after the last layer, [T, width]; `taps` collects it after every layer."""
    eps, alpha = cfg["norm"]["eps"], cfg["postln_alpha"]
    x = w["embed"][tokens] * cfg["embedding"]["scale"]
    kept: Dict[int, tuple] = {}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.mix.", layer["mixer"]
        if layer["type"] == "attention":
            src = m.get("kv_from")
            if src is None:
                kept[i] = softmax_keys_values(m, eps, w, p, x)
            a = softmax_mixer(m, eps, w, p, x, *kept[i if src is None else src], **attn_kw)
        elif layer["type"] == "lightning":
            a = lightning_mixer(m, eps, w, p, x)
        elif layer["type"] == "delta":
            a = delta_mixer(m, eps, w, p, x)
        else:
            raise ValueError(layer["type"])
        x = rms(alpha * x + a, eps) * w[f"l{i}.norm1"]
        if layer.get("mlp") is not None:
            x = rms(alpha * x + dense_ff(w, f"l{i}.mlp.", x), eps) * w[f"l{i}.norm2"]
        if taps is not None:
            taps.append(x.clone())
    return x


def forward_logits(cfg, w, tokens: List[int], **kw):
    x = forward_hidden(cfg, w, tokens, **kw)
    return (rms(x, cfg["norm"]["eps"]) * w["final.norm"]) @ w["embed"].T
