"""Satapel in plain, slow PyTorch (float64, whole sequences, loops): the oracle of the tests.

One function per mechanism, written from the design's equations; nothing here is shared with the
library.  A model is (cfg, w): cfg the dict that config.json holds, w a dict of float64 tensors by
checkpoint name.

  pair_embedding      x_t = E[tok_t] + B[(tok_{t-1} * a + tok_t * b) mod n],  B[n] for t = 0
  rms                 x / sqrt(mean(x^2) + eps)
  rotate_pairs        (u, v) -> (u cos - v sin, v cos + u sin) on pairs (2i, 2i+1), angle t * base^(-2i/dims)
  latent_attention    keys [W_uk c | rotated part], values W_uv c, window, sink in the denominator
  wkv                 o_t = (S + diag(u) k v^T)^T r;  S <- diag(w) S + k v^T;  head norm, gate
  routed_experts      softmax router, choice by score + correction, weights the plain scores
  forward_logits      all of it, x <- x + m (mixer(n1 x) + ff(n2 x)) per layer
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F = torch.float64


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def pair_embedding(cfg, w, tokens: List[int]):
    b = cfg["embedding"]["bigram"]
    rows = []
    for t, tok in enumerate(tokens):
        rows.append(b["buckets"] if t == 0 else (tokens[t - 1] * b["mul_prev"] + tok * b["mul_cur"]) % b["buckets"])
    return w["embed"][tokens] + w["bigram"][rows]


def rotate_pairs(v, positions, base: float, dims: int):
    """v: [T, ..., n]; the first `dims` of the last axis are rotated, the rest pass."""
    out = v.clone()
    for t, p in enumerate(positions):
        for i in range(dims // 2):
            a = p * base ** (-2.0 * i / dims)
            c, s = math.cos(a), math.sin(a)
            x, y = v[t, ..., 2 * i], v[t, ..., 2 * i + 1]
            out[t, ..., 2 * i] = x * c - y * s
            out[t, ..., 2 * i + 1] = y * c + x * s
    return out


def latent_attention(m, eps, w, p, h, use_sink=True, window_override=None):
    T = h.shape[0]
    H, d, r, vd, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    q = (h @ w[p + "q"].T).view(T, H, d + r)
    down = h @ w[p + "dkv"].T
    c = rms(down[:, :R], eps) * w[p + "dkv.norm"]
    key_rot = down[:, R:]
    if m.get("rot"):
        q_rot = rotate_pairs(q[..., d:], range(T), m["rot"]["base"], m["rot"]["dims"])
        key_rot = rotate_pairs(key_rot, range(T), m["rot"]["base"], m["rot"]["dims"])
    else:
        q_rot = q[..., d:]
    k_un = (c @ w[p + "uk"].T).view(T, H, d)
    val = (c @ w[p + "uv"].T).view(T, H, vd)
    window = window_override if window_override is not None else (m["mask"]["size"] if m.get("mask") else None)
    out = torch.zeros(T, H, vd, dtype=F)
    for i in range(T):
        lo = 0 if window is None else max(0, i - window + 1)
        for hh in range(H):
            s = (k_un[lo:i + 1, hh] @ q[i, hh, :d] + key_rot[lo:i + 1] @ q_rot[i, hh]) * m["scale"]
            mx = max(float(s.max()), float(w[p + "sink"][hh])) if use_sink else float(s.max())
            e = torch.exp(s - mx)
            den = e.sum() + (math.exp(float(w[p + "sink"][hh]) - mx) if use_sink else 0.0)
            out[i, hh] = (e / den) @ val[lo:i + 1, hh]
    return out.reshape(T, H * vd) @ w[p + "o"].T


def wkv(m, eps, w, p, h):
    T, H, d = h.shape[0], m["heads"], m["dim"]
    prev = torch.cat([torch.zeros(1, h.shape[1], dtype=F), h[:-1]])

    def mix(s):
        return h + (prev - h) * w[p + "mu." + s]
    r = (mix("r") @ w[p + "r"].T).view(T, H, d)
    k = (mix("k") @ w[p + "k"].T).view(T, H, d)
    v = (mix("v") @ w[p + "v"].T).view(T, H, d)
    g = mix("g") @ w[p + "g"].T
    gate = g / (1 + torch.exp(-g))
    decay = torch.exp(-torch.exp(torch.tanh(mix("w") @ w[p + "w1"].T) @ w[p + "w2"].T + w[p + "w0"])).view(T, H, d)
    out = torch.zeros(T, H, d, dtype=F)
    for hh in range(H):
        S = torch.zeros(d, d, dtype=F)
        for t in range(T):
            kv = torch.outer(k[t, hh], v[t, hh])
            out[t, hh] = (S + w[p + "u"][hh][:, None] * kv).T @ r[t, hh]
            S = decay[t, hh][:, None] * S + kv
    out = rms(out, eps).reshape(T, H * d)
    return (out * w[p + "norm"] * gate) @ w[p + "o"].T


def routed_experts(ff, w, p, h, alpha=1.702):
    E, I, top = ff["router"]["experts"], ff["router"].get("identity", 0), ff["router"]["top"]
    limit = ff["expert"].get("limit")
    z = h @ w[p + "router"].T
    s = torch.softmax(z, -1)
    pick = s + w[p + "correction"]
    out = torch.zeros_like(h)
    chosen = []
    for t in range(h.shape[0]):
        order = sorted(range(E + I), key=lambda e: (-float(pick[t, e]), e))[:top]
        chosen.append(order)
        for e in order:
            if e >= E:
                y = h[t]
            else:
                g, u = h[t] @ w[f"{p}e{e}.gate"].T, h[t] @ w[f"{p}e{e}.up"].T
                if limit:
                    g, u = torch.clamp(g, max=limit), torch.clamp(u, -limit, limit)
                y = (g / (1 + torch.exp(-alpha * g)) * (u + 1)) @ w[f"{p}e{e}.down"].T
            out[t] += s[t, e] * y
    return out, chosen, pick


def layer_states(cfg, w, tokens: List[int], **attn_kw):
    """The residual stream after the embedding and after every layer: [layers + 1] of [T, width]."""
    eps, mult = cfg["norm"]["eps"], cfg.get("residual_mult", 1.0)
    x = pair_embedding(cfg, w, tokens)
    states = [x]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{layer.get('weights_of', i)}."
        h1, h2 = rms(x, eps) * w[p + "norm1"], rms(x, eps) * w[p + "norm2"]
        if layer["type"] == "latent_attention":
            a = latent_attention(layer["mixer"], eps, w, p + "mix.", h1, **attn_kw)
        else:
            a = wkv(layer["mixer"], eps, w, p + "mix.", h1)
        f = routed_experts(layer["mlp"], w, p + "mlp.", h2)[0] if layer.get("mlp") else torch.zeros_like(x)
        x = x + mult * (a + f)
        states.append(x)
    return states


def forward_logits(cfg, w, tokens: List[int], **attn_kw):
    x = layer_states(cfg, w, tokens, **attn_kw)[-1]
    return (rms(x, cfg["norm"]["eps"]) * w["final.norm"]) @ w["head"].T


def greedy(cfg, w, prompt: List[int], n_new: int) -> List[int]:
    seq, out = list(prompt), []
    for _ in range(n_new):
        t = int(forward_logits(cfg, w, seq)[-1].argmax())
        out.append(t)
        seq.append(t)
    return out
