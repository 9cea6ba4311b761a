"""Satapel as data: the function from a `SatapelConfig` to a `ModelPlan`.

Embedding: token table plus a hashed token-pair table.  Every layer is a parallel block,
x += residual_mult * (mixer(norm1(x)) + ff(norm2(x))), whose mixer is either attention over a
latent cache (rotary on neighbouring pairs, a window, a sink per head) or a matrix-state
recurrence, and whose feed-forward is a routed set of experts (or none).  A layer with
`weights_of` appears in the run order as another call of the layer it names: same parts, a cache
or state of its own.  The model ends with an RMS norm and an untied head.  Tensor names:
`embed`, `bigram`, `l<i>.norm1`, `l<i>.norm2`, `l<i>.mix.*`, `l<i>.mlp.*`, `final.norm`, `head`.
"""
from __future__ import annotations

from ..config.base import LayerCall, LayerSpec, ModelPlan, PartSpec
from ..config.satapel import SatapelConfig
from ..registry import register_architecture

MAX_POSITIONS = 1 << 20        # the format names no limit: the cache alone bounds a sequence


def _mixer(cfg: SatapelConfig, layer, p: str) -> PartSpec:
    m = layer["mixer"]
    if layer["type"] == "latent_attention":
        rot, mask = m.get("rot"), m.get("mask")
        position = PartSpec("rotary", {"theta": float(rot["base"]), "rotary_dim": int(rot["dims"]),
                                       "style": "interleaved"}) if rot else None
        return PartSpec(
            "latent_attention",
            {"width": cfg.width, "n_heads": m["heads"], "dim": m["dim"], "rot_dim": m["rot_dim"], "vdim": m["vdim"],
             "kv_rank": m["kv_rank"], "scale": float(m["scale"]), "eps": cfg.norm_eps,
             "window": int(mask["size"]) if mask else None, "sink": True, "position": position},
            {"q": p + "mix.q", "dkv": p + "mix.dkv", "dkv_norm": p + "mix.dkv.norm", "uk": p + "mix.uk",
             "uv": p + "mix.uv", "sink": p + "mix.sink", "o": p + "mix.o"})
    names = {s: p + "mix." + s for s in ("r", "k", "v", "g", "w1", "w2", "w0", "u", "norm", "o")}
    names.update({"mu_" + s: p + "mix.mu." + s for s in ("r", "k", "v", "g", "w")})
    return PartSpec("matrix_state_recurrence",
                    {"width": cfg.width, "n_heads": m["heads"], "dim": m["dim"], "eps": cfg.norm_eps,
                     "decay_rank": m.get("decay_rank")}, names)


def _feed_forward(cfg: SatapelConfig, layer, p: str) -> PartSpec:
    mlp = layer.get("mlp")
    if mlp is None:
        return PartSpec("none")
    return PartSpec("routed_experts",
                    {"width": cfg.width, "inner": mlp["expert"]["ff"], "limit": mlp["expert"].get("limit"),
                     "alpha": 1.702, "experts": mlp["router"]["experts"], "identity": mlp["router"].get("identity", 0),
                     "top": mlp["router"]["top"], "correction": True},
                    {"router": p + "mlp.router", "correction": p + "mlp.correction", "expert": p + "mlp.e{}.",
                     "gate": "gate", "up": "up", "down": "down"})


def satapel_plan(cfg: SatapelConfig) -> ModelPlan:
    def norm(name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"width": cfg.width, "eps": cfg.norm_eps, "add_one": False}, {"weight": name})

    layers, index = [], {}
    for i, layer in enumerate(cfg.layers):
        if cfg.owner_of(i) != i:
            continue
        p = f"l{i}."
        index[i] = len(layers)
        layers.append(LayerSpec("parallel", _mixer(cfg, layer, p), _feed_forward(cfg, layer, p),
                                {"pre_mixer": norm(p + "norm1"), "pre_ffn": norm(p + "norm2")},
                                {"residual_mult": cfg.residual_mult}))
    return ModelPlan(
        width=cfg.width, vocab_size=cfg.vocab, max_positions=MAX_POSITIONS,
        embedding=PartSpec("pair_hash_embedding",
                           {"vocab": cfg.vocab, "width": cfg.width, "buckets": cfg.bigram_buckets,
                            "mul_prev": cfg.bigram_mul_prev, "mul_cur": cfg.bigram_mul_cur},
                           {"table": "embed", "pair_table": "bigram"}),
        layers=layers,
        schedule=[LayerCall(index[cfg.owner_of(i)]) for i in range(len(cfg.layers))],
        final_norm=norm("final.norm"),
        head=PartSpec("linear_head", {"vocab": cfg.vocab, "width": cfg.width, "softcap": 0.0}, {"table": "head"}),
    )


register_architecture("Satapel", SatapelConfig, satapel_plan)
