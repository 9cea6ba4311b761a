"""Vagonex without a GPU: the configuration's checks, the plan (layers, calls that read another call's cache, tensor
names and shapes), the rotary table with the long-context ramp against the oracle's, and properties of the oracle
itself that the GPU tests rely on."""
import copy

import pytest
import torch

from vagonex_cases import CASES, attention, delta, lightning, make_folder, model, oracle_view, row_errors, tokens


def test_the_plan_names_every_tensor_once_and_shares_caches():
    from hos_b200.model import weight_specs_for
    from hos_b200.registry import config_from_dict, plan_for
    cfg = config_from_dict(CASES["B"][0])
    plan = plan_for(cfg)
    assert [c.cache_from for c in plan.schedule] == [None, None, None, None, 2, 2]
    assert [l.arrangement for l in plan.layers] == ["postnorm"] * 6
    names = {s.name: tuple(s.shape) for s in weight_specs_for(cfg)}
    assert names["embed"] == (150, 64) and "head" not in names
    assert "l4.mix.k" not in names and "l4.mix.v.b" not in names and "l4.mix.k.norm" not in names
    assert names["l4.mix.q"] == (64, 64) and names["l4.mix.q.norm"] == (32,) and names["l4.mix.g"] == (2, 64)
    assert names["l2.mix.v"] == (32, 64) and names["l2.mix.k.b"] == (64,) and names["l2.mix.sink"] == (2,)
    assert "l2.norm2" not in names and "l2.mlp.gate" not in names            # a layer without a feed-forward
    assert names["l3.mix.q.conv"] == (32, 1) and names["l3.mix.v"] == (48, 64) and names["l3.mix.norm"] == (48,)
    assert names["l0.mix.norm"] == (32,) and names["l0.mix.g"] == (32, 64)
    assert config_from_dict(cfg.to_dict()) == cfg


@pytest.mark.parametrize("edit, word", [
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=2), "multiple"),
    (lambda c: c["layers"][4]["mixer"].update(kv_from=4), "earlier"),
    (lambda c: c["layers"][4]["mixer"].update(kv_from=3), "keeps no keys"),
    (lambda c: c["layers"][5]["mixer"].update(kv_from=4), "keeps no keys"),
    (lambda c: c["layers"][4]["mixer"].update(vdim=8), "differs"),
    (lambda c: c["layers"][0]["mixer"].update(decay=[0.5, 0.5]), "one number per head"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7), "even"),
    (lambda c: c["layers"][3]["mixer"].pop("conv"), "conv"),
    (lambda c: c["layers"][0].update(type="conv"), "type"),
    (lambda c: c["layers"][0]["mlp"].update(kind="moe"), "dense"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_a_wrong_configuration_is_refused_with_the_key_named(edit, word):
    from hos_b200.errors import MissingMetaError
    from hos_b200.registry import config_from_dict
    raw = copy.deepcopy(CASES["B"][0])
    edit(raw)
    with pytest.raises(MissingMetaError) as e:
        config_from_dict(raw)
    assert word in str(e.value)


def test_the_rotary_table_with_the_ramp():
    from plain import vagonex_plain as P
    from hos_b200.config.base import PartSpec
    from hos_b200.parts.base import Runtime
    from hos_b200.parts.rope import Rotary
    rt = Runtime(torch.device("cpu"), torch.float32)
    for rot in ({"base": 30000.0, "dims": 40, "scaling": {"factor": 3.0, "original": 96, "fast": 24.0, "slow": 1.5}},
                {"base": 100.0, "dims": 16, "scaling": {"factor": 16.0, "original": 32, "fast": 3.0, "slow": 1.5}},
                {"base": 10000.0, "dims": 8, "scaling": {"factor": 8.0, "original": 64, "fast": 16.0, "slow": 2.0}},
                {"base": 500.0, "dims": 6}):
        part = Rotary(PartSpec("rotary", {"theta": rot["base"], "rotary_dim": rot["dims"], "style": "interleaved",
                                          "table": "float64", "scaling": rot.get("scaling")}), rt)
        freqs, mult = P.rotary_table(rot)
        assert abs(part.magnitude - mult) < 1e-12
        assert torch.allclose(part.inv_freq.double(), torch.tensor(freqs, dtype=torch.float64), rtol=1e-7, atol=0)
    ramped, _ = P.rotary_table({"base": 30000.0, "dims": 40, "scaling": {"factor": 3.0, "original": 96, "fast": 24.0, "slow": 1.5}})
    plain, _ = P.rotary_table({"base": 30000.0, "dims": 40})
    assert ramped[0] == plain[0] and abs(ramped[-1] - plain[-1] / 3.0) < 1e-15 and any(
        p / 3.0 * 1.0001 < r < p * 0.9999 for r, p in zip(ramped, plain))          # untouched, fully scaled, and in between


def test_the_oracle_feels_every_mechanism(tmp_path):
    """What the GPU tests compare with must move when a mechanism is taken away: the sink, the chunk's edge, the state
    and the convolution's memory (a sequence cut in two), the key/value source of a sharing layer."""
    from plain import vagonex_plain as P
    folder = make_folder(tmp_path, CASES["A"][0], CASES["A"][1], "A")
    cfg, w = oracle_view(folder)
    seq = tokens(1, 100, cfg["vocab"])
    want = P.forward_logits(cfg, w, seq)
    assert float(row_errors(P.forward_logits(cfg, w, seq, use_sink=False), want).median()) > 2e-3
    assert float(row_errors(P.forward_logits(cfg, w, seq, chunk_override=69)[70:], want[70:]).median()) > 2e-3
    assert float(row_errors(P.forward_logits(cfg, w, seq[40:]), want[40:]).median()) > 2e-3
    own = copy.deepcopy(cfg)
    own["layers"][3]["mixer"].pop("kv_from")
    w2 = dict(w)
    for name in ("k", "k.b", "k.norm", "v", "v.b"):
        w2["l3.mix." + name] = w["l0.mix." + name]              # the same tensors, but fed with layer 3's input
    assert float(row_errors(P.forward_logits(own, w2, seq), want).median()) > 2e-3
    # prefix property: a position's logits do not depend on later tokens
    assert float(row_errors(P.forward_logits(cfg, w, seq[:60]), want[:60]).max()) < 1e-12
