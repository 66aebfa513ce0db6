"""Malazen without a device: the configuration class and its errors, the schedule of a loop, tensor
names and shapes, the cache needs of mixers side by side and what the cache manager makes of them,
the stretched rotary tables, and properties of the plain implementation itself."""

from __future__ import annotations

import copy
import math

import pytest
import torch

import malazen_models as M
from plain import malazen_plain as plain

from lockstep_b200.cache import CacheManager
from lockstep_b200.config import ConfigError, MalazenConfig, config_from_dict
from lockstep_b200.engine.model import Model, expected_weights
from lockstep_b200.parts import CacheNeed, Runtime


def cpu_runtime(max_positions=64):
    return Runtime(device=torch.device("cpu"), dtype=torch.float32, page_size=8, max_positions=max_positions,
                   err=torch.zeros(2, dtype=torch.int32))


def test_registry_picks_the_class_by_the_architecture_key():
    cfg = config_from_dict(M.MODEL_S)
    assert isinstance(cfg, MalazenConfig) and cfg.to_dict() == M.MODEL_S
    assert (cfg.width, cfg.vocab, cfg.groups) == (72, 193, 3)


def test_a_loop_repeats_its_layers_with_caches_of_their_own():
    spec = config_from_dict(M.MODEL_S).model_spec()
    runs = [(r.layer, r.cache, r.add_embedding) for r in spec.schedule]
    assert runs == [(0, 0, False), (1, 1, False), (2, 2, False), (1, 3, True), (2, 4, False), (3, 5, False)]
    assert spec.cache_entries == 6
    # from the first layer, three times over one layer; and a loop of one pass changes nothing
    runs = [(r.layer, r.add_embedding) for r in config_from_dict(M.MODEL_U).model_spec().schedule]
    assert runs == [(0, False), (0, True), (0, True), (1, False), (2, False)]
    assert [(r.layer, r.add_embedding) for r in config_from_dict(M.MODEL_V).model_spec().schedule] == [(0, False), (1, False)]
    assert [r.layer for r in config_from_dict(M.MODEL_T).model_spec().schedule] == [0, 1, 2]


def test_tensor_names_and_shapes():
    w = expected_weights(config_from_dict(M.MODEL_S).model_spec())
    assert w["embed"].shape == (193, 72) and w["final.norm"].shape == (72,)
    assert w["l0.mix.q"].shape == (3 * (16 + 8), 72) and w["l0.mix.dkv"].shape == (40 + 8, 72)
    assert w["l0.mix.dkv.norm"].shape == (40,) and w["l0.mix.uk"].shape == (3 * 16, 40)
    assert w["l0.mix.uv"].shape == (3 * 24, 40) and w["l0.mix.sink"].shape == (3,) and w["l0.mix.o"].shape == (72, 72)
    assert w["l1.mix.left.q"].shape == (128, 72) and w["l1.mix.left.k"].shape == (32, 72)
    assert w["l1.mix.left.v.b"].shape == (16,) and w["l1.mix.left.o"].shape == (72, 64) and w["l1.mix.left.o.b"].shape == (72,)
    assert w["l1.mix.left.r1"].shape == (4,) and w["l1.mix.left.r2"].shape == (4,)
    assert w["l1.mix.right.q"].shape == (48, 72) and w["l1.mix.right.v"].shape == (80, 72)
    assert w["l1.mix.right.a1"].shape == (5, 72) and w["l1.mix.right.a2"].shape == (48, 5)
    assert w["l1.mix.right.a2.b"].shape == (48,) and w["l1.mix.right.norm"].shape == (40,)
    assert w["l1.mlp.gate"].shape == (56, 72) and w["l1.mlp.down.b"].shape == (72,)
    assert "l3.mlp.gate" not in w and "l3.norm2" not in w        # the last layer has no feed-forward
    # a rank the configuration does not name is whatever the stored tensors have
    raw = copy.deepcopy(M.MODEL_S)
    del raw["layers"][1]["mixer"]["right"]["decay_rank"]
    w = expected_weights(config_from_dict(raw).model_spec())
    assert w["l1.mix.right.a1"].shape == (-1, 72) and w["l1.mix.right.a1"].fits((9, 72))


@pytest.mark.parametrize("edit, message", [
    (lambda c: c.update(width=70), "groups"),
    (lambda c: c["layers"][0].update(type="attention"), "not one of"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=6), "rot_dim"),
    (lambda c: c["layers"][1]["mixer"]["left"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][1]["mixer"]["right"].update(tau=0.0), "tau"),
    (lambda c: c["layers"][1]["mixer"].pop("left_scale"), "left_scale"),
    (lambda c: c["layers"][1]["mlp"].update(kind="moe"), "dense"),
    (lambda c: c["loop"].update(stop=9), "loop"),
    (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
])
def test_configuration_errors_name_the_key(edit, message):
    raw = copy.deepcopy(M.MODEL_S)
    edit(raw)
    with pytest.raises(ConfigError, match=message):
        config_from_dict(raw)


def test_mixers_side_by_side_keep_a_cache_each():
    spec = config_from_dict(M.MODEL_S).model_spec()
    model = Model(spec, cpu_runtime())
    needs = model.cache_needs()
    assert [n.kind for n in needs] == ["paged_kv", "several", "paged_kv", "several", "paged_kv", "several"]
    assert needs[0] == CacheNeed("paged_kv", kv_heads=1, head_dim=48, window=21)
    left, right = needs[1].parts
    assert left == CacheNeed("paged_kv", kv_heads=1, head_dim=32, window=0)
    assert right.kind == "state" and right.state_shape == (2 * 24 * 40,)
    cache = CacheManager(needs, num_pages=8, page_size=16, max_live=2, max_seq_len=128, allocate=False)
    # both passes of the loop's parallel layer share a group of pages and a group of slots, with an entry each
    assert len(cache.paged) == 4 and len(cache.states) == 2
    view = cache.view(3)
    assert view.kind == "several" and [p.kind for p in view.parts] == ["paged_kv", "state"]
    assert cache.view(1).parts[0].group is view.parts[0].group
    cache.create("a")
    cache.reserve("a", 100)
    cache.advance("a", 100)
    cache.audit()
    # the window of 21 has given back what lies behind it, the layers that see every key nothing
    held = {g.window: sum(p >= 0 for p in g.seqs["a"].pages) for g in cache.paged}
    assert held[0] == 7 and held[21] == 2 and held[70] == 6
    cache.release("a")
    cache.audit()


@pytest.mark.parametrize("dims, base, scaling", [(16, 40000.0, (3.0, 1024, 16.0, 2.0)), (8, 100.0, (4.0, 64, 8.0, 1.0)),
                                                  (32, 10000.0, None), (4, 1000.0, (8.0, 16, 2.0, 1.0))])
def test_stretched_rotary_tables(dims, base, scaling):
    from lockstep_b200.parts.position import ScaledRotary

    s = dict(zip(("factor", "original", "fast", "slow"), scaling)) if scaling else None
    part = ScaledRotary(dims, base, cpu_runtime(300), scaling=s, interleaved=True)
    cos, sin, rot = part.rotary()
    want_cos, want_sin = plain.scaled_rotary_tables(300, dims, base, s)
    assert rot == dims and part.rotary_interleaved
    assert float((cos.double() - want_cos).abs().max()) < 1e-6 and float((sin.double() - want_sin).abs().max()) < 1e-6
    if scaling:
        # written out once more: slow dimensions turn factor times slower, and the tables are longer than one
        mag = 0.1 * math.log(scaling[0]) + 1.0
        assert abs(float(cos[0, 0]) - mag) < 1e-6
        f_last = base ** (-2.0 * (dims // 2 - 1) / dims)
        ratio = math.atan2(float(sin[1, -1]), float(cos[1, -1])) / f_last
        assert 1.0 / scaling[0] - 1e-4 <= ratio <= 1.0 + 1e-4


def test_plain_rule_continues_from_a_state_and_plain_sink_is_one_more_key():
    g = torch.Generator().manual_seed(3)
    n, H, dk, dv = 23, 2, 5, 7
    q, k = torch.randn(n, H, dk, generator=g, dtype=torch.float64), torch.randn(n, H, dk, generator=g, dtype=torch.float64)
    v, a = torch.randn(n, H, dv, generator=g, dtype=torch.float64), torch.rand(n, H, dk, generator=g, dtype=torch.float64)
    whole, S = plain.decayed_outer_product_rule(q, k, v, a)
    first, S1 = plain.decayed_outer_product_rule(q[:9], k[:9], v[:9], a[:9])
    rest, S2 = plain.decayed_outer_product_rule(q[9:], k[9:], v[9:], a[9:], state=S1)
    assert torch.allclose(torch.cat([first, rest]), whole) and torch.allclose(S2, S)
    # closed form of the last read-out: sum over tokens of (prod of later decays) k v^T
    want = torch.zeros(H, dv, dtype=torch.float64)
    for t in range(n):
        keep = a[t + 1:].prod(0)
        want += torch.einsum("hk,hk,hv->hv", q[-1] * keep, k[t], v[t])
    assert torch.allclose(whole[-1], want)
    # a sink is a key with a zero value whose score is the sink itself
    qq, kk = torch.randn(6, 1, 4, generator=g, dtype=torch.float64), torch.randn(6, 1, 4, generator=g, dtype=torch.float64)
    vv = torch.randn(6, 1, 3, generator=g, dtype=torch.float64)
    sink = torch.tensor([0.7], dtype=torch.float64)
    got = plain.sink_window_attention(qq, kk, vv, 0.5, 3, sink)
    for i in range(6):
        js = [j for j in range(6) if 0 <= i - j < 3]
        s = torch.tensor([float(qq[i, 0] @ kk[j, 0]) * 0.5 for j in js] + [0.7], dtype=torch.float64)
        p = torch.softmax(s, 0)
        assert torch.allclose(got[i, 0], sum(p[x] * vv[j, 0] for x, j in enumerate(js)))
