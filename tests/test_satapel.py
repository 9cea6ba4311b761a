"""Satapel without a GPU: the configuration reader, the plan (shared layers, tensor names, sizes that
only a checkpoint gives), the cache's groups and state for it, and the oracle against itself."""
import copy

import pytest
import torch

from satapel_cases import CASE_A, CASE_B, CASES, attention, experts, make_folder, model, oracle_view, recurrence, tokens


def test_the_architecture_is_found_by_its_single_string_key():
    from hos_b200.config.satapel import SatapelConfig
    from hos_b200.registry import config_from_dict, registered_architectures
    cfg = config_from_dict(CASE_A)
    assert isinstance(cfg, SatapelConfig) and "Satapel" in registered_architectures()
    assert config_from_dict(cfg.to_dict()) == cfg or config_from_dict(cfg.to_dict()).to_dict() == cfg.to_dict()


@pytest.mark.parametrize("breaker, word", [
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["norm"].pop("eps"), "norm.eps"),
    (lambda c: c["layers"][0].update(type="conv"), "type"),
    (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][2].update(weights_of=1), "another type"),
    (lambda c: c["layers"][2].update(weights_of=2), "another layer"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=5), "rot"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=9), "mlp"),
    (lambda c: c["embedding"].pop("bigram"), "bigram"),
])
def test_bad_configurations_are_refused_with_the_key_named(breaker, word):
    from hos_b200.errors import MissingMetaError
    from hos_b200.registry import config_from_dict
    raw = copy.deepcopy(CASE_A)
    breaker(raw)
    with pytest.raises(MissingMetaError, match=word):
        config_from_dict(raw)


def test_a_shared_layer_is_another_call_of_the_same_parts():
    from hos_b200.model import weight_specs_for
    from hos_b200.registry import config_from_dict, plan_for
    cfg = config_from_dict(CASE_A)
    plan = plan_for(cfg)
    assert [c.layer for c in plan.schedule] == [0, 1, 0, 2] and len(plan.layers) == 3
    assert plan.layers[0].params["residual_mult"] == 0.7
    names = {s.name: s.shape for s in weight_specs_for(cfg)}
    assert not any(n.startswith("l2.") for n in names)                 # the shared layer has no tensors
    assert names["l0.mix.dkv"] == (40 + 8, 72) and names["l0.mix.q"] == (3 * 24, 72) and names["l0.mix.sink"] == (3,)
    assert names["bigram"] == (98, 72) and names["l1.mlp.router"] == (6, 72) and names["l1.mix.u"] == (3, 16)
    assert "l3.mlp.router" not in names and names["l3.mix.w1"] == (5, 72)
    assert "l0.mlp.e4.down" in names and "l0.mlp.e5.down" not in names  # the identity expert has none


def test_the_decay_rank_may_come_from_the_checkpoint_alone(tmp_path):
    from hos_b200.errors import MissingMetaError, WeightMismatchError
    from hos_b200.model import weight_specs_for
    from hos_b200.registry import config_from_dict
    from hos_b200.weights import RandomSource, SafetensorsFolder
    from hos_b200.weights.loader import check_against
    folder = make_folder(tmp_path, CASE_A, 3)
    raw = copy.deepcopy(CASE_A)
    for layer in raw["layers"]:
        layer["mixer"].pop("decay_rank", None)
    specs = weight_specs_for(config_from_dict(raw))
    assert {s.name: s.shape for s in specs}["l1.mix.w1"] == (-1, 72)
    src = SafetensorsFolder(folder)
    try:
        check_against(specs, src)                                       # any rank fits
    finally:
        src.close()
    with pytest.raises(MissingMetaError, match="l1.mix.w1"):
        RandomSource(specs, 0)
    raw["layers"][1]["mixer"]["heads"] = 4                               # a size that does not fit is still refused
    src = SafetensorsFolder(folder)
    try:
        with pytest.raises(WeightMismatchError, match="l1.mix.r"):
            check_against(weight_specs_for(config_from_dict(raw)), src)
    finally:
        src.close()


def test_the_cache_gives_latent_layers_one_keys_only_group_and_every_part_its_state():
    from hos_b200.model import Model
    from hos_b200.parts.base import Runtime
    from hos_b200.registry import config_from_dict, plan_for
    m = Model(plan_for(config_from_dict(CASE_A)), Runtime(torch.device("cpu"), torch.float32))
    cache = m.new_cache(max_tokens=640, chunk_tokens=16)
    assert len(cache.groups) == 1
    g = cache.groups[0]
    assert g.need.keys_only and g.need.window == 70 and g.need.head_dim == 48 and g.n_entries == 2
    assert all(v is None for v in g.v) and g.k[0].shape == (10, 1, 64, 48)
    assert g.ring_pages == (70 + 16 - 1 + 63) // 64
    assert set(cache.stores[1].state) == {"S", "last_row"} and cache.stores[1].state["S"].shape[1:] == (3, 16, 16)
    assert cache.stores[3].state["S"].shape[1:] == (2, 24, 24) and not cache.stores[0].state
    assert cache.embedding_store.state["prev_token"].dtype == torch.int32
    # a slot's state is zeroed when it is taken, and a snapshot puts rows back
    for t in cache.state_tensors():
        t.fill_(7)
    s = cache.admit([0, 0])
    assert all(float(t[s[0]].double().abs().sum()) == 0 for t in cache.state_tensors())
    snap = cache.snapshot_state(torch.tensor(s, dtype=torch.int32))
    for t in cache.state_tensors():
        t[s[1]] = 3
    cache.restore_state(snap)
    assert all(float(t[s[1]].double().abs().sum()) == 0 for t in cache.state_tensors())
    cache.release(s[0]); cache.release(s[1]); cache.check()


def test_the_oracle_sees_what_it_should(tmp_path):
    """The oracle's own mechanisms: a key outside the window, the sink and the pair table all move its logits;
    the logits of a prefix do not depend on what follows."""
    from plain import satapel_plain as P
    folder = make_folder(tmp_path, CASE_B, 12)
    cfg, w = oracle_view(folder)
    toks = tokens(1, 40, cfg["vocab"])
    full = P.forward_logits(cfg, w, toks)
    assert torch.allclose(P.forward_logits(cfg, w, toks[:17]), full[:17], atol=1e-12)
    assert (P.forward_logits(cfg, w, toks, use_sink=False) - full).abs().max() > 1e-3
    wide = copy.deepcopy(cfg)
    wide["layers"][1]["mixer"]["mask"]["size"] = 6
    assert (P.forward_logits(wide, w, toks)[6:] - full[6:]).abs().max() > 1e-3
    assert torch.allclose(P.forward_logits(wide, w, toks)[:5], full[:5], atol=1e-12)
    other = dict(w, bigram=w["bigram"].flip(0))
    assert (P.forward_logits(cfg, other, toks) - full).abs().max() > 1e-3
    _, chosen, _ = P.routed_experts(cfg["layers"][0]["mlp"], w, "l0.mlp.", torch.randn(9, 64, dtype=torch.float64))
    assert all(len(c) == 1 and 0 <= c[0] < 3 for c in chosen)
