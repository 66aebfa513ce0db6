"""Sevipel without a device: configuration, the model as data, tensor names, the loader's
treatment of open ranks and optional tensors, the cache needs, and the plain implementation's
own properties (the tests on the device compare the engine with it)."""

from __future__ import annotations

import copy
import json

import pytest
import torch

import sevipel_models as M
from plain import sevipel_plain as plain


def spec_of(config):
    from lockstep_b200.config import config_from_dict

    return config_from_dict(config).model_spec()


def test_architecture_is_found_by_its_plain_name_key():
    from lockstep_b200.config import SevipelConfig, architecture_name, config_from_dict

    assert architecture_name({"architecture": "Sevipel"}) == "Sevipel"
    assert isinstance(config_from_dict(M.MODEL_P), SevipelConfig)
    assert config_from_dict(M.MODEL_P).to_dict() == M.MODEL_P


def test_model_spec_names_parts_and_schedule():
    spec = spec_of(M.MODEL_P)
    kinds = [layer.mixer.kind for layer in spec.layers]
    assert kinds == ["gqa_attention", "gated_delta", "wkv", "gated_delta", "gqa_attention"]
    assert [layer.feed_forward.kind for layer in spec.layers] == ["routed_experts", "routed_experts", "none",
                                                                  "routed_experts", "routed_experts"]
    # the layer that borrows keys and values reads the entry of the layer it names and writes none
    runs = [(r.layer, r.cache, r.writes_cache) for r in spec.schedule]
    assert runs == [(0, 0, True), (1, 1, True), (2, 2, True), (3, 3, True), (4, 0, False)]
    a0, a4 = spec.layers[0].mixer, spec.layers[4].mixer
    assert (a0["window"], a4["window"], a0["scale"], a4["scale"]) == (24, 40, 0.21, 0.3)
    assert a0["value_dim"] == 16 and a0["head_dim"] == 32 and a4["borrows_kv"] and not a0["borrows_kv"]
    assert spec.layers[0].position.kind == "rotary" and spec.layers[0].position["dim"] == 16
    assert spec.layers[1].position.kind == "none"
    assert spec.optional_tensors == ("l2.norm2",)


def test_tensor_names_and_shapes():
    from lockstep_b200.engine.model import expected_weights

    w = expected_weights(spec_of(M.MODEL_P))
    assert w["embed"].shape == (211, 64) and w["final.norm"].shape == (64,) and w["l0.norm1"].shape == (64,)
    assert w["l0.mix.q"].shape == (128, 64) and w["l0.mix.k"].shape == (64, 64) and w["l0.mix.v"].shape == (32, 64)
    assert w["l0.mix.q.norm"].shape == (128,) and w["l0.mix.k.norm"].shape == (64,) and w["l0.mix.o"].shape == (64, 64)
    # no key or value tensors where they are borrowed, no feed-forward tensors where there is none
    assert not any(n.startswith(("l4.mix.k", "l4.mix.v")) for n in w) and "l4.mix.q.norm" in w
    assert not any(n.startswith(("l2.mlp", "l2.norm2")) for n in w)
    assert w["l1.mix.q"].shape == (32, 64) and w["l1.mix.v"].shape == (128, 64) and w["l1.mix.q.conv"].shape == (32, 4)
    assert w["l1.mix.a1"].shape == (6, 64) and w["l1.mix.a2"].shape == (64, 6) and w["l1.mix.g2"].shape == (128, 5)
    assert w["l1.mix.A_log"].shape == (4,) and w["l1.mix.norm"].shape == (32,) and w["l1.mix.dt_bias"].shape == (64,)
    assert w["l2.mix.mu.w"].shape == (64,) and w["l2.mix.u"].shape == (2, 32) and w["l2.mix.w2"].shape == (64, 7)
    assert w["l0.mlp.router"].shape == (6, 64) and w["l0.mlp.e5.up"].shape == (48, 64) and w["l0.mlp.e5.down"].shape == (64, 48)
    assert "head.weight" not in w          # the head is the embedding table


def test_cache_needs_follow_the_longest_reader():
    from lockstep_b200.engine.model import Model
    from lockstep_b200.parts import Runtime

    def needs(config):
        rt = Runtime(device=torch.device("cpu"), dtype=torch.float32, page_size=8, max_positions=64,
                     err=torch.zeros(2, dtype=torch.int32))
        return Model(spec_of(config), rt).cache_needs()

    p = needs(M.MODEL_P)
    # keys padded to the larger of the key and value sizes; layer 4 reads entry 0 with window 40
    assert (p[0].kind, p[0].kv_heads, p[0].head_dim, p[0].window) == ("paged_kv", 2, 32, 40)
    assert p[1].kind == "state" and p[1].state_shape == (4 * 16 * 32 + 3 * (2 * 32 + 128),)
    assert p[2].state_shape == (2 * 32 * 32 + 64,)
    assert len(p) == 4
    q = needs(M.MODEL_Q)
    assert (q[1].head_dim, q[1].window) == (48, 50)      # a shorter reader changes nothing
    assert (q[2].head_dim, q[2].window) == (48, 0)
    unbounded = copy.deepcopy(M.MODEL_P)
    del unbounded["layers"][4]["mixer"]["mask"]            # a reader that sees every key keeps them all
    assert needs(unbounded)[0].window == 0


@pytest.mark.parametrize("change, message", [
    (lambda c: c["layers"][0].update(type="conv"), "not one of"),
    (lambda c: c["layers"][4]["mixer"].update(kv_from=1), "kv_from"),
    (lambda c: c["layers"][4]["mixer"].update(vdim=32), "differs from layer 0"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "multiple of kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=34), "rot.dims"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=7), "top exceeds"),
    (lambda c: c.pop("norm"), "norm.eps"),
    (lambda c: c["layers"][1]["mixer"].pop("conv"), "lacks 'conv'"),
])
def test_configuration_errors_are_named(change, message):
    from lockstep_b200.config import ConfigError, config_from_dict

    raw = copy.deepcopy(M.MODEL_P)
    change(raw)
    with pytest.raises(ConfigError, match=message):
        config_from_dict(raw)


def test_loader_reads_open_ranks_from_the_tensors_and_tolerates_named_extras(tmp_path):
    from safetensors.torch import load_file, save_file

    from lockstep_b200.config import load_config
    from lockstep_b200.engine.model import expected_weights
    from lockstep_b200.weights import load_weights
    from lockstep_b200.weights.loader import WeightError
    from lockstep_b200.weights.random_init import random_tensors

    folder = M.make_folder(tmp_path, M.MODEL_P, seed=3, dtype="bfloat16")
    # a configuration that does not name the ranks: they are the stored tensors' own
    raw = json.loads((folder / "config.json").read_text())
    for layer in raw["layers"]:
        for key in ("decay_rank", "gate_rank"):
            layer["mixer"].pop(key, None)
    (folder / "config.json").write_text(json.dumps(raw))
    spec = load_config(folder).model_spec()
    expected = expected_weights(spec)
    assert expected["l1.mix.a1"].shape == (-1, 64)
    with pytest.raises(ValueError, match="leaves an extent open"):
        random_tensors(expected, 0, "bfloat16")
    got = load_weights(folder, expected, torch.float32, "cpu", optional=spec.optional_tensors)
    assert got["l1.mix.a1"].shape == (6, 64) and got["l3.mix.g2"].shape == (32, 9) and got["l2.mix.w1"].shape == (7, 64)
    # a norm in front of a feed-forward that the layer does not have may be stored; anything else may not
    tensors = load_file(str(folder / "model.safetensors"))
    tensors["l2.norm2"] = torch.zeros(64, dtype=torch.bfloat16)
    save_file(tensors, str(folder / "model.safetensors"))
    load_weights(folder, expected, torch.float32, "cpu", optional=spec.optional_tensors)
    tensors["l2.mlp.router"] = torch.zeros(6, 64, dtype=torch.bfloat16)
    save_file(tensors, str(folder / "model.safetensors"))
    with pytest.raises(WeightError, match="unexpected"):
        load_weights(folder, expected, torch.float32, "cpu", optional=spec.optional_tensors)


def test_random_weights_use_the_parts_own_distributions(tmp_path):
    from safetensors.torch import load_file

    w = load_file(str(M.make_folder(tmp_path, M.MODEL_P, seed=4, dtype="float32") / "model.safetensors"))
    assert abs(float(w["l0.norm1"].mean())) < 0.1                   # the tensors hold gains minus one
    assert 0.0 <= float(w["l2.mix.mu.r"].min()) and float(w["l2.mix.mu.r"].max()) <= 1.0
    assert float(w["l2.mix.w0"].mean()) < -1.5


def test_state_slots_are_cleared_when_taken_again():
    from lockstep_b200.cache import CacheManager
    from lockstep_b200.parts import CacheNeed

    cm = CacheManager([CacheNeed("state", state_shape=(5,)), CacheNeed("paged_kv", kv_heads=1, head_dim=16, window=8)],
                      num_pages=4, page_size=8, max_live=2, max_seq_len=64)
    a = cm.create("a")
    cm.states[0].state[0, a].fill_(3.0)
    cm.release("a")
    b = cm.create("b")
    assert b == a and float(cm.states[0].state[0, b].abs().sum()) == 0.0


# -- the plain implementation's own properties ---------------------------------------------

def _one(layer, n=40, seed=0, tmp=None):
    config = M.one_layer(M.with_mlp(layer))
    folder = M.make_folder(tmp, config, seed=seed, dtype="float32")
    cfg, w = plain.read_model_folder(folder)
    return cfg, w


def test_plain_is_causal_and_its_window_has_the_stated_edges(tmp_path):
    cfg, w = _one(M.attention(2, 1, 16, 16, window=6, rot=(8, 100.0)), tmp=tmp_path)
    tokens = [5, 9, 1, 33, 7, 20, 4, 8, 15, 60, 2, 11, 30]
    base = plain.forward(cfg, w, tokens)
    assert torch.allclose(plain.forward(cfg, w, tokens[:7]), base[:7], atol=1e-12)
    changed = list(tokens)
    changed[4] = 77
    other = plain.forward(cfg, w, changed)
    # position i sees j with 0 <= i - j < 6: token 4 is seen by positions 4..9 and by no other
    differs = [bool((other[i] - base[i]).abs().max() > 1e-9) for i in range(len(tokens))]
    assert differs == [False] * 4 + [True] * 6 + [False] * 3


def test_plain_recurrences_carry_the_first_token_to_the_last(tmp_path):
    for layer in (M.delta(2, 1, 8, 16, conv=3), M.wkv(2, 8)):
        cfg, w = _one(layer, tmp=tmp_path)
        tokens = list(range(3, 60))
        base = plain.forward(cfg, w, tokens)
        other = plain.forward(cfg, w, [90] + tokens[1:])
        assert float((other[-1] - base[-1]).abs().max()) > 1e-9
        assert torch.allclose(plain.forward(cfg, w, tokens[:20]), base[:20], atol=1e-12)


def test_plain_delta_rule_with_full_write_reads_back_the_value():
    # one key, beta 1, no decay: after the write the state returns v for the query k
    k = torch.nn.functional.normalize(torch.randn(1, 1, 8, dtype=torch.float64), dim=-1)
    v = torch.randn(1, 1, 4, dtype=torch.float64)
    o = plain.delta_rule(k, k, v, torch.ones(1, 1, 8, dtype=torch.float64), torch.ones(1, 1, dtype=torch.float64))
    assert torch.allclose(o, v, atol=1e-12)


def test_plain_routing_scales_the_input_and_keeps_scores_unnormalised():
    x = torch.randn(3, 6, dtype=torch.float64)
    w = {"m.router": torch.randn(4, 6, dtype=torch.float64)}
    for e in range(4):
        w[f"m.e{e}.up"] = torch.randn(5, 6, dtype=torch.float64)
        w[f"m.e{e}.down"] = torch.randn(6, 5, dtype=torch.float64)
    out = plain.routed_experts(x, w, "m", {"router": {"experts": 4, "top": 2}})
    scores = torch.sigmoid(x @ w["m.router"].T)
    for t in range(3):
        want = torch.zeros(6, dtype=torch.float64)
        for e in scores[t].topk(2).indices.tolist():
            want += torch.relu((scores[t, e] * x[t]) @ w[f"m.e{e}.up"].T) ** 2 @ w[f"m.e{e}.down"].T
        assert torch.allclose(out[t], want, atol=1e-12)
