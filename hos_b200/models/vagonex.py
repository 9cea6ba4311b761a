"""Vagonex as data: the function from a `VagonexConfig` to a `ModelPlan`.

Embedding: the token table times a constant.  Every layer has the norm after the sum,
x <- norm1(alpha x + mixer(x)); x <- norm2(alpha x + ff(x)), the branches reading x itself.  The mixer is one of:
softmax attention (biased projections, per-head query/key norms, a partial rotation of neighbouring pairs with
ramped frequencies, a mask of chunks, a sink, a gate per head; `kv_from` makes the layer a call that reads an
earlier call's cache), a matrix-state recurrence with a constant decay per head, or the gated delta rule with short
convolutions.  The feed-forward is a gated dense one with the tanh form of GELU, or absent.  The model ends with an
RMS norm and a head that is the embedding table itself (without the constant).  Tensor names: `embed`,
`l<i>.norm1`, `l<i>.norm2`, `l<i>.mix.*`, `l<i>.mlp.*`, `final.norm`.
"""
from __future__ import annotations

from ..config.base import LayerCall, LayerSpec, ModelPlan, PartSpec
from ..config.vagonex import VagonexConfig
from ..registry import register_architecture

MAX_POSITIONS = 1 << 20        # the format names no limit: the cache alone bounds a sequence


def _mixer(cfg: VagonexConfig, layer, p: str) -> PartSpec:
    m, kind = layer["mixer"], layer["type"]
    if kind == "attention":
        rot, mask, shares = m.get("rot"), m.get("mask"), m.get("kv_from") is not None
        position = None
        if rot:
            position = PartSpec("rotary", {"theta": float(rot["base"]), "rotary_dim": int(rot["dims"]),
                                           "style": "interleaved", "table": "float64",
                                           "scaling": dict(rot["scaling"]) if rot.get("scaling") else None})
        names = {"q": p + "q", "q_bias": p + "q.b", "q_norm": p + "q.norm", "sink": p + "sink", "gate": p + "g", "o": p + "o"}
        if not shares:
            names.update({"k": p + "k", "k_bias": p + "k.b", "k_norm": p + "k.norm", "v": p + "v", "v_bias": p + "v.b"})
        return PartSpec(
            "gated_softmax_attention",
            {"width": cfg.width, "n_heads": m["heads"], "n_kv_heads": m["kv_heads"], "dim": m["dim"], "vdim": m["vdim"],
             "scale": float(m["scale"]), "eps": cfg.norm_eps, "chunk": int(mask["size"]) if mask else None,
             "bias": True, "qk_norm": True, "sink": True, "head_gate": True, "shares_kv": shares, "position": position},
            names)
    if kind == "lightning":
        return PartSpec("decay_linear_attention",
                        {"width": cfg.width, "n_heads": m["heads"], "dim": m["dim"], "vdim": m["vdim"],
                         "decay": tuple(float(d) for d in m["decay"]), "eps": cfg.norm_eps},
                        {"q": p + "q", "k": p + "k", "v": p + "v", "gate": p + "g", "norm": p + "norm", "o": p + "o"})
    return PartSpec("gated_delta_rule",
                    {"width": cfg.width, "n_heads": m["heads"], "n_kv_heads": m["kv_heads"], "dim": m["dim"],
                     "vdim": m["vdim"], "taps": m["conv"], "eps": cfg.norm_eps},
                    {"q": p + "q", "q_conv": p + "q.conv", "k": p + "k", "k_conv": p + "k.conv", "v": p + "v",
                     "v_conv": p + "v.conv", "beta": p + "b", "a": p + "a", "A_log": p + "A_log", "dt_bias": p + "dt_bias",
                     "gate": p + "g", "norm": p + "norm", "o": p + "o"})


def vagonex_plan(cfg: VagonexConfig) -> ModelPlan:
    def norm(name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"width": cfg.width, "eps": cfg.norm_eps, "add_one": False}, {"weight": name})

    layers, schedule = [], []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        mlp = layer.get("mlp")
        norms = {"post_mixer": norm(p + "norm1")}
        if mlp is None:
            ffn = PartSpec("none")
        else:
            ffn = PartSpec("gated_mlp", {"width": cfg.width, "inner": mlp["ff"], "activation": "gelu_tanh"},
                           {"gate": p + "mlp.gate", "up": p + "mlp.up", "down": p + "mlp.down"})
            norms["post_ffn"] = norm(p + "norm2")
        layers.append(LayerSpec("postnorm", _mixer(cfg, layer, p + "mix."), ffn, norms, {"alpha": cfg.postln_alpha}))
        schedule.append(LayerCall(i, layer["mixer"].get("kv_from") if layer["type"] == "attention" else None))
    return ModelPlan(
        width=cfg.width, vocab_size=cfg.vocab, max_positions=MAX_POSITIONS,
        embedding=PartSpec("scaled_embedding", {"vocab": cfg.vocab, "width": cfg.width, "scale": cfg.embedding_scale},
                           {"table": "embed"}),
        layers=layers, schedule=schedule, final_norm=norm("final.norm"),
        head=PartSpec("linear_head", {"vocab": cfg.vocab, "width": cfg.width, "softcap": 0.0}, {"table": "embed"}),
    )


register_architecture("Vagonex", VagonexConfig, vagonex_plan)
