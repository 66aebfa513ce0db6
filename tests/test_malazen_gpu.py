"""Malazen on the device against the plain implementation: every mechanism's kernels alone,
one-layer models of each mixer, and whole models cut in four ways (whole prompts; a prompt and
then token by token; portions down to two tokens; up to three live requests with portions of
some beside single tokens of others, on so few pages and slots that they are used again), in
float32 and bfloat16; weights made so that a window's edge, a far key, a sink or a lost state
shows; greedy generation through the entry point and the scheduler; the trace runner."""

from __future__ import annotations

import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import helpers as H
import malazen_models as M
from plain import malazen_plain as plain

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
DEV = "cuda:0"
F32, BF16 = torch.float32, torch.bfloat16


def make_runner(folder, dtype, page, steps=None, max_live=3, num_pages=None, **kw):
    from lockstep_b200.engine import ModelRunner

    if num_pages is None:
        num_pages = H.max_live_tokens(steps, round_to=page) // page
    return ModelRunner(folder, dtype=dtype, num_pages=num_pages, page_size=page, max_live=max_live,
                       max_seq_len=1024, **kw)


PLANS = {
    "whole": H.plan_whole,
    "then_single": lambda r: H.plan_bulk_then_single(r, tail=70),
    "portions": lambda r: H.plan_portions(r, sizes=(7, 2, 17, 3, 33, 2, 5, 64, 1, 2, 150)),
    "mixed": lambda r: H.plan_mixed(r, max_live=3),
}


# ---------------------------------------------------------------------------
# kernels alone
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("out_dtype", [F32, BF16])
@pytest.mark.parametrize("width, groups", [(72, 3), (100, 2), (64, 1), (320, 5), (18, 9)])
def test_norm_in_groups(width, groups, out_dtype):
    from lockstep_b200 import kernels as K

    g = torch.Generator().manual_seed(width)
    x = torch.randn(13, width, generator=g) * torch.linspace(0.1, 30.0, width)       # parts of very different size
    gain = (1 + 0.3 * torch.randn(width, generator=g)).to(out_dtype)
    rows = torch.tensor([12, 0, 5, 5, 7], dtype=torch.int32)
    err = K.new_error_word(DEV)
    for index in (None, rows):
        out = torch.empty((13 if index is None else 5, width), dtype=out_dtype, device=DEV)
        K.rmsnorm(x.to(DEV), gain.to(DEV), out, 1e-5, err, None if index is None else index.to(DEV), groups)
        src = x if index is None else x[index.long()]
        want = plain.grouped_rms_norm(src.double(), gain.double(), 1e-5, groups)
        tol = 2e-6 if out_dtype == F32 else 8e-3
        assert float(((out.cpu().double() - want).abs() / (1 + want.abs())).max()) < tol
    K.raise_on_fault(err)
    if groups > 1:      # the parts are not the whole: one norm over the row gives something else
        whole = plain.grouped_rms_norm(x.double(), gain.double(), 1e-5, 1)
        assert float((whole - plain.grouped_rms_norm(x.double(), gain.double(), 1e-5, groups)).abs().max()) > 0.1


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("rows, ff, width, limit", [(9, 40, 24, 0.5), (70, 56, 100, 2.5), (1, 8, 8, 7.0)])
def test_clamped_gated_activation(dtype, rows, ff, width, limit):
    from lockstep_b200 import kernels as K

    g = torch.Generator().manual_seed(ff)
    gate_up = torch.randn(rows, 2 * ff, generator=g) * 3
    bias = torch.randn(2 * ff, generator=g)
    res_bias = torch.randn(width, generator=g)
    residual = torch.randn(rows, width, generator=g)
    out = torch.empty(rows, ff, dtype=dtype, device=DEV)
    res = residual.to(DEV)
    K.clamped_glu(gate_up.to(DEV), bias.to(DEV), out, limit, 1.702, res, res_bias.to(DEV))
    z = gate_up.double() + bias.double()
    gg, uu = z[:, :ff].clamp(max=limit), z[:, ff:].clamp(-limit, limit)
    want = gg * torch.sigmoid(1.702 * gg) * (uu + 1)
    assert float((out.cpu().double() - want).abs().max()) < (1e-5 if dtype == F32 else 3e-2) * (1 + float(want.abs().max()))
    assert float((res.cpu().double() - residual.double() - res_bias.double()).abs().max()) < 1e-6
    if limit < 5:
        # a gate above the limit is clamped, one far below is not; an up value is clamped on both sides
        assert float(gg.max()) == limit and float(gg.min()) < -limit and float(uu.min()) == -limit and float(uu.max()) == limit


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("nq, nkv, d, dv, every", [(4, 1, 32, 16, 7), (2, 2, 16, 48, 1), (6, 3, 24, 24, 128)])
def test_projection_finish_adds_biases_and_a_query_temperature(dtype, nq, nkv, d, dv, every):
    from lockstep_b200 import kernels as K

    g = torch.Generator().manual_seed(nq * 10 + d)
    tokens, page, pad = 12, 8, -(-max(d, dv) // 16) * 16
    cols = nq * d + nkv * (d + dv)
    qkv = torch.randn(tokens, cols, generator=g).to(dtype)
    bias = torch.randn(cols, generator=g)
    # the first positions, and those around the steps of the temperature; two requests, the second on far pages
    positions = torch.tensor([0, 1, 2, 3, 4, 5, 6, 7, every - 1, every, 2 * every + 1, 3 * every + 2], dtype=torch.int32)
    slot = torch.tensor([1] * 8 + [0] * 4, dtype=torch.int32)
    n_pages = (3 * every + 2) // page + 2
    # (each request's logical pages scattered over physical pages of its own: the even ones, the odd ones)
    table = torch.stack([2 * ((torch.arange(n_pages) * 7 + 3) % n_pages),
                         2 * ((torch.arange(n_pages) * 3 + 1) % n_pages) + 1]).to(torch.int32)
    pages = torch.full((2 * n_pages, 2, nkv, page, pad), 9.0, dtype=dtype, device=DEV)
    q_out = torch.full((tokens, nq * pad), 9.0, dtype=dtype, device=DEV)
    err = K.new_error_word(DEV)
    pos = positions
    K.qkv_finish(qkv.to(DEV), q_out, pages, None, None, None, None, pos.to(DEV), slot.to(DEV), table.to(DEV), nq, nkv, d, dv,
                 pad, 0, 0.0, False, True, True, err, bias=bias.to(DEV), q_temp=(0.4, every))
    K.raise_on_fault(err)
    x = qkv.double() + bias.double()
    temp = 1.0 + 0.4 * torch.log(torch.div(pos.long() + 1, every, rounding_mode="floor").double() + 1.0)
    assert len(set(temp.tolist())) > 1
    q = x[:, :nq * d].view(tokens, nq, d) * temp[:, None, None]
    k = x[:, nq * d:(nq + nkv) * d].view(tokens, nkv, d)
    v = x[:, (nq + nkv) * d:].view(tokens, nkv, dv)
    tol = 3e-6 if dtype == F32 else 3e-2
    got_q = q_out.double().cpu().view(tokens, nq, pad)
    assert float((got_q[..., :d] - q).abs().max()) < tol * 4 and float(got_q[..., d:].abs().sum()) == 0.0
    for t in range(tokens):
        pg = int(table[slot[t], pos[t] // page])
        row = pages[pg, :, :, int(pos[t]) % page].double().cpu()
        assert float((row[0, :, :d] - k[t]).abs().max()) < tol * 4 and float(row[0, :, d:].abs().sum()) == 0.0
        assert float((row[1, :, :dv] - v[t]).abs().max()) < tol * 4 and float(row[1, :, dv:].abs().sum()) == 0.0


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("H_, dk, dv", [(2, 16, 32), (3, 40, 24), (2, 72, 8), (1, 128, 64), (1, 5, 3)])
def test_decayed_outer_product_rule_walks_portions_and_carries_its_state(dtype, H_, dk, dv):
    """Three requests in one call, then the rest of two of them in later calls (one token by
    token): the outputs are the plain recurrence over each whole sequence.  q, k and v are columns
    of one wider tensor, as the mixer hands them over."""
    from lockstep_b200 import kernels as K

    g = torch.Generator().manual_seed(dk + dv)
    lengths = {0: 37, 2: 9, 1: 21}
    Kd, Vd = H_ * dk, H_ * dv
    pitch = 2 * Kd + Vd + 11
    seqs, want = {}, {}
    for slot, n in lengths.items():
        rows = (torch.randn(n, pitch, generator=g) * 0.5).to(dtype)
        decay = torch.rand(n, H_, dk, generator=g) * 0.3 + 0.7
        seqs[slot] = (rows, decay)
        q, k, v = (rows[:, 3:3 + Kd], rows[:, 3 + Kd:3 + 2 * Kd], rows[:, 8 + 2 * Kd:8 + 2 * Kd + Vd])
        want[slot] = plain.decayed_outer_product_rule(q.double().view(n, H_, dk), k.double().view(n, H_, dk),
                                                      v.double().view(n, H_, dv), decay.double())[0] * 0.37
    state = torch.zeros(4, H_ * dk * dv, device=DEV)
    state[3] = 5.0                                      # a slot nobody uses stays as it is
    err = K.new_error_word(DEV)

    def call(pieces):
        """pieces: [(slot, first, count)] packed one after the other."""
        rows = torch.cat([seqs[s][0][a:a + c] for s, a, c in pieces]).to(DEV)
        decay = torch.cat([seqs[s][1][a:a + c] for s, a, c in pieces]).reshape(-1, Kd).contiguous().to(DEV)
        token_slot = torch.tensor(sum(([s] * c for s, a, c in pieces), []), dtype=torch.int32, device=DEV)
        portions = torch.empty(1 + 3 * 4, dtype=torch.int32, device=DEV)
        K.find_portions(token_slot, portions, 4, err)
        out = torch.empty(rows.shape[0], Vd, device=DEV)
        K.state_rule(K.RULE_GLA, dtype, portions, 4, state, rows[:, 3:3 + Kd], rows[:, 3 + Kd:3 + 2 * Kd],
                     rows[:, 8 + 2 * Kd:8 + 2 * Kd + Vd], decay, None, None, out, None, 0, 0, H_, H_, dk, dv,
                     out_scale=0.37)
        got, at = {}, 0
        for s, a, c in pieces:
            got[(s, a)] = out[at:at + c].cpu().double().view(c, H_, dv)
            at += c
        return got

    got = call([(0, 0, 20), (2, 0, 9), (1, 0, 2)])
    got.update(call([(1, 2, 19), (0, 20, 1)]))
    for i in range(21, 37):
        got.update(call([(0, i, 1)]))
    K.raise_on_fault(err)
    tol = 2e-5 if dtype == F32 else 1e-5        # (the inputs are exact in either type: the walk is float32)
    for (s, a), rows in got.items():
        ref = want[s][a:a + rows.shape[0]]
        assert float((rows - ref).abs().max()) < tol * (1 + float(want[s].abs().max())), (s, a)
    assert float(state[3].min()) == 5.0 and float(state[3].max()) == 5.0
    assert K.kernel_counts()["gla_rule"] > 0


def test_decay_is_a_power_of_a_sigmoid():
    from lockstep_b200 import kernels as K

    z = torch.linspace(-30, 30, 7 * 12).view(7, 12)
    bias = torch.linspace(-1, 1, 12)
    for tau in (1.0, 16.0, 0.5):
        got = z.to(DEV).clone()
        K.sigmoid_power_decay(got, bias.to(DEV), tau)
        want = torch.sigmoid(z.double() + bias.double()) ** (1.0 / tau)
        assert float((got.cpu().double() - want).abs().max()) < 2e-6
        assert float(((got.cpu().double().log() - want.log()).abs() / (1 + want.log().abs())).max()) < 1e-5   # small decays keep their digits


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("heads, d, dr, dv, rank, interleaved", [(3, 16, 8, 24, 40, True), (1, 48, 2, 64, 30, True),
                                                                  (8, 8, 4, 8, 12, False), (2, 32, 32, 40, 64, True)])
def test_latent_finish_and_per_head_products(dtype, heads, d, dr, dv, rank, interleaved):
    from lockstep_b200 import kernels as K

    g = torch.Generator().manual_seed(heads + rank)
    tokens, page, pad = 11, 8, -(-(rank + dr) // 16) * 16
    cols = heads * (d + dr) + rank + dr + 5
    proj = (torch.randn(tokens, cols, generator=g)).to(dtype)
    gain = (1 + 0.3 * torch.randn(rank, generator=g)).to(dtype)
    positions = torch.tensor([3, 4, 5, 6, 7, 8, 9, 10, 0, 1, 2], dtype=torch.int32)
    slot = torch.tensor([1] * 8 + [0] * 3, dtype=torch.int32)
    table = torch.tensor([[4, -1], [2, 0]], dtype=torch.int32)
    scaling = {"factor": 4.0, "original": 8.0, "fast": 4.0, "slow": 0.5}
    cos, sin = plain.scaled_rotary_tables(16, dr, 100.0, scaling)
    pages = torch.full((5, 2, 1, page, pad), 9.0, dtype=dtype, device=DEV)
    q_out = torch.full((tokens, heads * pad), 9.0, dtype=dtype, device=DEV)
    err = K.new_error_word(DEV)
    dev_proj = proj.to(DEV)
    K.latent_finish(dev_proj, q_out, pages, gain.to(DEV), cos.float().to(DEV), sin.float().to(DEV), positions.to(DEV),
                    slot.to(DEV), table.to(DEV), heads, d, dr, rank, pad, 1e-5, interleaved, True, err)
    w_fold = (torch.randn(heads, rank, d, generator=g) * 0.3).to(dtype)
    K.heads_product(dev_proj, d + dr, w_fold.to(DEV), q_out, pad)
    K.raise_on_fault(err)
    x = proj.double()
    q = x[:, :heads * (d + dr)].view(tokens, heads, d + dr)
    c = x[:, heads * (d + dr):heads * (d + dr) + rank]
    c = c / torch.sqrt((c * c).mean(-1, keepdim=True) + 1e-5) * gain.double()
    k_rot = x[:, heads * (d + dr) + rank:heads * (d + dr) + rank + dr]
    pc, ps = cos[positions.long()], sin[positions.long()]

    def turn(v):                       # v [tokens, n, dr]
        if interleaved:
            return plain.rotate_pairs(v, pc, ps)
        half = dr // 2
        a, b = v[..., :half], v[..., half:]
        return torch.cat([a * pc[:, None] - b * ps[:, None], b * pc[:, None] + a * ps[:, None]], -1)

    tol = 4e-6 if dtype == F32 else 3e-2
    got_q = q_out.double().cpu().view(tokens, heads, pad)
    folded = torch.einsum("thd,hrd->thr", q[..., :d], w_fold.double())
    assert float((got_q[..., :rank] - folded).abs().max()) < tol * (1 + float(folded.abs().max()))
    assert float((got_q[..., rank:rank + dr] - turn(q[..., d:])).abs().max()) < tol * 4
    assert float(got_q[..., rank + dr:].abs().sum()) == 0.0
    for t in range(tokens):
        pg = int(table[slot[t], positions[t] // page])
        row = pages[pg, :, 0, int(positions[t]) % page].double().cpu()
        assert float((row[0, :rank] - c[t]).abs().max()) < tol * 4 and float((row[1, :rank] - c[t]).abs().max()) < tol * 4
        assert float((row[0, rank:rank + dr] - turn(k_rot[:, None])[t, 0]).abs().max()) < tol * 4
        assert float(row[0, rank + dr:].abs().sum()) == 0.0 and float(row[1, rank:].abs().sum()) == 0.0
    # the second per-head product reads heads of the padded size and writes heads of the value size
    attn = (torch.randn(tokens, heads * pad, generator=g)).to(dtype)
    w_up = (torch.randn(heads, dv, rank, generator=g) * 0.3).to(dtype)
    y = torch.empty(tokens, heads * dv, dtype=dtype, device=DEV)
    K.heads_product(attn.to(DEV), pad, w_up.to(DEV), y, dv)
    want = torch.einsum("thr,hvr->thv", attn.double().view(tokens, heads, pad)[..., :rank], w_up.double())
    assert float((y.double().cpu().view(tokens, heads, dv) - want).abs().max()) < tol * (1 + float(want.abs().max()))


def test_embedding_added_again_and_weighted_branches():
    from lockstep_b200 import kernels as K

    g = torch.Generator().manual_seed(1)
    table = torch.randn(50, 24, generator=g).to(BF16)
    ids = torch.tensor([3, 49, 0, 3], dtype=torch.int32)
    h = torch.randn(4, 24, generator=g)
    out = h.to(DEV)
    err = K.new_error_word(DEV)
    K.embed_gather(ids.to(DEV), table.to(DEV), out, err, accumulate=True)
    assert torch.equal(out.cpu(), h + table.float()[ids.long()])
    branches = torch.randn(3, 4, 24, generator=g)
    K.weighted_sum(out, branches.to(DEV), [0.8, -0.9, 2.0])
    want = (h + table.float()[ids.long()]).double() + 0.8 * branches[0].double() - 0.9 * branches[1].double() + 2 * branches[2].double()
    assert float((out.cpu().double() - want).abs().max()) < 1e-5
    x = torch.full((5, 24), 7.0, device=DEV)
    K.row_bias(x, None)
    assert float(x.abs().sum()) == 0.0
    bias = torch.randn(24, generator=g).to(DEV)
    K.row_bias(x, bias)
    K.row_bias(x, bias, add=True)
    assert torch.equal(x.cpu(), (2 * bias).cpu().expand(5, 24))
    K.raise_on_fault(err)


# ---------------------------------------------------------------------------
# models: one layer of each mixer, then whole models, in four cuttings
# ---------------------------------------------------------------------------

ONE_LAYER = {
    "parallel": (M.with_mlp(M.parallel(4, 2, 32, 16, 2, 24, 40, temp=(0.5, 5)), 40), None),
    "parallel_one_key_head": (M.with_mlp(M.parallel(6, 1, 16, 48, 1, 40, 8, temp=None, tau=2.0)), None),
    "parallel_looped": (M.with_mlp(M.parallel(2, 2, 48, 48, 3, 16, 16, temp=(0.5, 1), left_scale=1.3, right_scale=0.2), 24), (0, 1, 3)),
    "latent": (M.with_mlp(M.latent(3, 16, 8, 24, 40, window=20, scaling=(4.0, 32, 8.0, 1.0)), 40), None),
    "latent_sees_all": (M.with_mlp(M.latent(5, 8, 16, 8, 16, base=50.0)), None),
    "latent_looped": (M.with_mlp(M.latent(2, 24, 4, 40, 60, window=64, scaling=(2.0, 16, 2.0, 0.5)), 56), (0, 1, 2)),
}


@pytest.fixture(scope="module")
def zoo(tmp_path_factory):
    cache = {}

    def get(config, dtype, lengths, seed=7, edit=None, key=None):
        key = (key or str(config), dtype, tuple(lengths))
        if key not in cache:
            folder = M.make_folder(tmp_path_factory.mktemp("malazen"), config, seed=seed, dtype=dtype, edit=edit)
            requests = {f"r{i}": H.random_tokens(n, config["vocab"], seed=50 + i) for i, n in enumerate(lengths)}
            cache[key] = (folder, requests, {u: M.plain_logits(folder, t).float() for u, t in requests.items()})
        return cache[key]

    return get


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(ONE_LAYER))
def test_one_layer_models_in_every_cutting(zoo, name, dtype):
    layer, loop = ONE_LAYER[name]
    folder, requests, want = zoo(M.one_layer(layer, loop=loop), dtype, [45, 130, 9, 77])
    rows = {}
    for plan_name, plan in PLANS.items():
        steps = plan(requests)
        runner = make_runner(folder, dtype, 8, steps)
        rows[plan_name] = H.run_plan(runner, steps)
        M.assert_close(rows[plan_name], want, dtype, f"{name}, {plan_name}")
        runner.cache.audit()
    if dtype == "float32":
        # a row's arithmetic does not depend on how its request was cut or on the batch
        for plan_name in PLANS:
            for key, row in rows["whole"].items():
                assert torch.equal(row, rows[plan_name][key]), (name, plan_name, key)


LENGTHS = {"S": [70, 300, 37, 150, 129], "T": [45, 210, 90, 33, 260], "U": [40, 190, 75, 131], "V": [30, 100, 2, 61],
           "W": [50, 140, 3, 99]}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("plan_name", sorted(PLANS))
@pytest.mark.parametrize("model", sorted(M.MODELS))
def test_whole_models_in_every_cutting(zoo, model, plan_name, dtype):
    config, page = M.MODELS[model]
    folder, requests, want = zoo(config, dtype, LENGTHS[model])
    steps = PLANS[plan_name](requests)
    runner = make_runner(folder, dtype, page, steps)
    rows = H.run_plan(runner, steps)
    M.assert_close(rows, want, dtype, f"model {model}, {plan_name}")
    runner.cache.audit()
    if plan_name == "mixed":
        assert runner.cache.reused_pages() > 0           # more requests than slots, on few pages
    if plan_name == "then_single" and runner.graphs is not None:
        assert runner.graphs.replays > 100               # decoded tokens ran as recorded steps


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_branches_on_streams_of_their_own_give_the_bits_of_branches_in_turn(zoo, dtype):
    """In steps of few tokens the second mixer of a parallel layer runs on a stream of its own (recorded: a branch
    of the graph).  The logits are those of a runner that takes the mixers one after the other, bit for bit, in
    decoding (recorded steps), in portions of a few tokens and in mixed batches."""
    config, page = M.MODELS["S"]
    folder, requests, want = zoo(config, dtype, LENGTHS["S"])
    for plan_name in ("then_single", "portions", "mixed"):
        steps = PLANS[plan_name](requests)
        rows = {}
        for streams in (True, False):
            runner = make_runner(folder, dtype, page, steps)
            runner.rt.options["branch_streams"] = streams
            rows[streams] = H.run_plan(runner, steps)
            if plan_name == "then_single" and runner.graphs is not None:
                assert runner.graphs.replays > 100
        for key, row in rows[True].items():
            assert torch.equal(row, rows[False][key]), (plan_name, key)


def _sharpen(tensors):
    # large query weights make every row of a softmax pick one or two keys: a key that is wrongly
    # seen or not seen at a window's edge, a far key that is lost or a sink that is left out then
    # changes the output by as much as a value.  A weak distance bias keeps far keys in play.
    for name in tensors:
        if name.endswith(("mix.q", "left.q")):
            tensors[name] = (tensors[name].float() * (4.0 if name.endswith("mix.q") else 3.0)).to(tensors[name].dtype)
        if name.endswith(".r1"):
            tensors[name] = torch.full_like(tensors[name], 0.05)
        if name.endswith(".sink"):
            tensors[name] = torch.full_like(tensors[name], 3.0)


def _softmax_weights(folder, tokens, at=0):
    """The softmax's weights [heads, n, n] of layer ``at`` of the plain model."""
    cfg, w = plain.read_model_folder(folder)
    x = w["embed"][torch.tensor(tokens)]
    for i in range(at):
        x = plain.layer_forward(x, w, i, cfg["layers"][i], cfg)
    x = plain.grouped_rms_norm(x, w[f"l{at}.norm1"], cfg["norm"]["eps"], cfg["norm"]["groups"])
    layer = cfg["layers"][at]
    if layer["type"] == "latent_attention":
        return plain.latent_attention_mixer(x, w, f"l{at}.mix", layer["mixer"], cfg["norm"]["eps"], weights=True)
    return plain.biased_attention_mixer(x, w, f"l{at}.mix.left", layer["mixer"]["left"], weights=True)


def _tensor_core_attention_launches():
    from lockstep_b200 import kernels as K

    counts = K.kernel_counts()
    return counts.get("attention_prefill_tc", 0), counts.get("attention_decode_mma", 0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window, rank", [(1, 24), (37, 24), (37, 56), (64, 24), (256, 24), (None, 24), (None, 56)])
def test_sharp_latent_attention_shows_window_edges_far_keys_and_sinks(zoo, window, rank, dtype):
    # (a latent of 56 and a rotated part of 8 make a head of 64: in bfloat16 the tensor-core kernels)
    config = M.model(48, 97, 1e-5, 2, [M.with_mlp(M.latent(4, 16, 8, 16, rank, window=window, scale=0.5), 32),
                                       M.with_mlp(M.latent(2, 8, 8, 24, 40, window=(window + 5) if window else 40, scale=0.5))])
    folder, requests, want = zoo(config, dtype, [620, 300], edit=_sharpen, key=f"sharp-latent{window}-{rank}")
    before = _tensor_core_attention_launches()
    p = _softmax_weights(folder, requests["r0"])                      # [heads, n, n]
    n = p.shape[-1]
    rows = torch.arange(n)[None, :]
    best = p.argmax(-1)
    sink_share = 1.0 - p.sum(-1)
    assert float(sink_share.max()) > 0.5 and float(sink_share.min()) < 0.1     # rows the sink takes, and rows it does not
    if window and window > 1:
        assert float(p.max(-1).values.median()) > 0.3
        assert int(((best == rows - (window - 1)) & (rows >= window)).sum()) >= 3      # largest key the last one inside
    if not window:
        assert int((best < rows - 200).sum()) >= 20                                    # largest key more than 200 back
    for plan_name in ("whole", "then_single", "portions", "mixed"):
        steps = PLANS[plan_name](requests)
        runner = make_runner(folder, dtype, 16, steps)
        M.assert_close(H.run_plan(runner, steps), want, dtype, f"sharp latent attention, window {window}, {plan_name}",
                       slack=3.0)      # (scores are large: their rounding shows)
    after = _tensor_core_attention_launches()
    if rank == 56 and dtype == "bfloat16":
        assert after[0] > before[0] and after[1] > before[1]       # both tensor-core attention kernels ran
    else:
        assert after == before


def _sharpen_more_bias(tensors):
    _sharpen(tensors)
    for name in tensors:
        if name.endswith(".r1"):
            tensors[name] = torch.full_like(tensors[name], 0.4)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("dim", [32, 64])
def test_sharp_biased_attention_reaches_far_keys(zoo, dim, dtype):
    # (behind a layer that rotates: the stream then tells a token's repeats apart; heads of 64: in
    # bfloat16 the tensor-core kernels)
    config = M.model(48, 97, 1e-5, 1, [M.with_mlp(M.latent(2, 16, 8, 16, 24, window=50), 32),
                                       M.with_mlp(M.parallel(4, 2, dim, 16, 1, 16, 16, scale=0.5, temp=(0.3, 100)), 32)])
    folder, requests, want = zoo(config, dtype, [700, 280], edit=_sharpen_more_bias, key=f"sharp-left{dim}")
    before = _tensor_core_attention_launches()
    p = _softmax_weights(folder, requests["r0"], at=1)
    n = p.shape[-1]
    rows = torch.arange(n)[None, :]
    assert float(p.max(-1).values.median()) > 0.3
    assert int((p.argmax(-1) < rows - 256).sum()) >= 20               # largest key beyond a split of keys, pages away
    # and the bias matters: without it other keys win
    cfg, w = plain.read_model_folder(folder)
    w = dict(w, **{"l1.mix.left.r1": torch.zeros(4, dtype=torch.float64)})
    moved = plain.forward(cfg, w, requests["r0"])[-1]
    assert float((moved - want["r0"][-1].double()).abs().max()) > 1e-2
    for plan_name in ("whole", "then_single", "portions", "mixed"):
        steps = PLANS[plan_name](requests)
        runner = make_runner(folder, dtype, 16, steps)
        M.assert_close(H.run_plan(runner, steps), want, dtype, f"sharp biased attention, {plan_name}", slack=3.0)
    after = _tensor_core_attention_launches()
    assert (after[0] > before[0] and after[1] > before[1]) == (dim == 64 and dtype == "bfloat16")


def _remember(tensors):
    # decays close to one: what the first tokens wrote into the state still weighs in the last
    # token's read-out, so a state that is lost, cleared or mixed up between slots shows
    for name in tensors:
        if name.endswith("a2.b"):
            tensors[name] = torch.full_like(tensors[name], 6.0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_slow_decays_carry_the_first_tokens_through_long_decoding(zoo, dtype):
    config = M.model(64, 131, 1e-5, 2, [M.with_mlp(M.parallel(2, 1, 16, 16, 2, 32, 48, tau=16.0, left_scale=0.1, right_scale=1.5), 32),
                                        M.with_mlp(M.parallel(2, 2, 16, 16, 1, 24, 24, tau=8.0, left_scale=0.1, right_scale=1.5))],
                     loop=(0, 2, 2))
    folder, requests, want = zoo(config, dtype, [420, 150, 260, 90], edit=_remember, key="remember")
    cfg, w = plain.read_model_folder(folder)
    tokens = requests["r0"]
    moved = plain.forward(cfg, w, [(tokens[0] + 1) % 131] + tokens[1:])[-1]
    assert float((moved - want["r0"][-1].double()).abs().max()) > 1e-3      # the plain model itself remembers
    plans = dict(PLANS, long_decoding=lambda r: H.plan_bulk_then_single(r, tail=200))
    for plan_name, plan in plans.items():
        steps = plan(requests)
        runner = make_runner(folder, dtype, 16, steps)
        M.assert_close(H.run_plan(runner, steps), want, dtype, f"slow decays, {plan_name}")


# ---------------------------------------------------------------------------
# the entry point, the scheduler, the trace runner
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine(tmp_path, dtype):
    from lockstep_b200 import Engine, Request

    config, page = M.MODELS["S"]
    folder = M.make_folder(tmp_path, config, seed=21, dtype=dtype)
    engine = Engine(folder, dtype=dtype, num_pages=64, page_size=page, max_running=12, max_step_tokens=96,
                    max_seq_len=512)
    prompts = {f"g{i}": H.random_tokens(n, config["vocab"], seed=300 + i)
               for i, n in enumerate([33, 7, 120, 1, 64, 18, 45, 2, 90, 11])}
    got = engine.generate([Request(uid=u, prompt=p, max_new_tokens=8) for u, p in prompts.items()])
    cfg, w = plain.read_model_folder(folder)
    for uid, prompt in prompts.items():
        assert len(got[uid]) == 8
        rows = plain.forward(cfg, w, list(prompt) + got[uid])     # causal: one pass gives every step's logits
        for i, tok in enumerate(got[uid]):
            row = rows[len(prompt) + i - 1]
            margin = 2 * M.TOLERANCE[dtype] * (1 + float(row.abs().max()))
            assert float(row[tok]) >= float(row.max()) - margin, (dtype, uid, i, tok)
    # ten requests decode as recorded steps of sixteen rows: the padding rows share the padding slot
    assert engine.runner.graphs is not None and engine.runner.graphs.replays > 0
    engine.cache.audit()
    assert engine.cache.live == 0


def test_the_command_line_writes_a_random_model_and_runs_a_workload(tmp_path):
    """``bin/lockstep random-model`` from a configuration, then ``bin/lockstep run``: greedy tokens are the plain
    model's, and sampled requests (temperature, top-p) come out whole."""
    import json

    config, page = M.MODELS["V"]
    (tmp_path / "config.json").write_text(json.dumps(config))
    folder = tmp_path / "model"
    lockstep = [sys.executable, str(ROOT / "bin" / "lockstep")]
    proc = subprocess.run(lockstep + ["random-model", "--config", str(tmp_path / "config.json"), "--out", str(folder),
                                      "--seed", "5", "--init-std", "0.15", "--gain-std", "0.1"],
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    prompts = {f"c{i}": H.random_tokens(n, config["vocab"], 95 + i) for i, n in enumerate([4, 23, 50])}
    workload = tmp_path / "workload.json"
    requests = [{"uid": u, "prompt": p, "max_new_tokens": 10} for u, p in prompts.items()]
    requests += [{"uid": "s0", "prompt": prompts["c1"], "max_new_tokens": 12, "temperature": 0.8, "top_p": 0.9, "seed": 3},
                 {"uid": "s1", "prompt": prompts["c1"], "max_new_tokens": 12, "temperature": 0.8, "top_p": 0.9, "seed": 3}]
    workload.write_text(json.dumps(requests))
    proc = subprocess.run(lockstep + ["run", "--model", str(folder), "--dtype", "float32", "--workload", str(workload),
                                      "--policy", "fixed-chunk:16", "--num-blocks", "40", "--block-size", str(page),
                                      "--max-running", "3"], capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = {l["uid"]: l for l in (json.loads(x) for x in proc.stdout.splitlines() if x.startswith("{"))}
    assert set(lines) == set(prompts) | {"s0", "s1"}
    cfg, w = plain.read_model_folder(folder)
    for uid, prompt in prompts.items():
        got = lines[uid]["generated"]
        assert len(got) == 10
        rows = plain.forward(cfg, w, list(prompt) + got)
        for i, tok in enumerate(got):
            row = rows[len(prompt) + i - 1]
            assert float(row[tok]) >= float(row.max()) - 2 * M.TOLERANCE["float32"] * (1 + float(row.abs().max()))
    assert len(lines["s0"]["generated"]) == 12 and all(0 <= t < config["vocab"] for t in lines["s0"]["generated"])


def test_trace_runner_replays_a_trace(tmp_path):
    config, page = M.MODELS["T"]
    folder = M.make_folder(tmp_path, config, seed=9, dtype="bfloat16")
    requests = {f"t{i}": H.random_tokens(n, config["vocab"], seed=70 + i) for i, n in enumerate([40, 130, 25, 61, 90])}
    steps = H.plan_mixed(requests, max_live=4)
    out = tmp_path / "out"
    for dtype in ("bfloat16", "float32"):
        proc = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype,
                               "--out", str(out / dtype), "--max-tokens", str(H.max_live_tokens(steps, 64))],
                              input=H.plan_to_jsonl(steps), capture_output=True, text=True, timeout=900)
        assert proc.returncode == 0, proc.stderr[-2000:]
        assert [l for l in proc.stdout.splitlines() if l.startswith("done ")] == [f"done {i}" for i in range(len(steps))]
        want = {u: M.plain_logits(folder, t).float() for u, t in requests.items()}
        at = {u: 0 for u in requests}
        rows = {}
        for i, step in enumerate(steps):
            got = np.fromfile(out / dtype / f"{i}.f32", dtype="<f4").reshape(-1, config["vocab"])
            r = 0
            for uid, toks, wanted in step["entries"]:
                for wpos in wanted:
                    rows[(uid, at[uid] + wpos)] = torch.from_numpy(got[r].copy())
                    r += 1
                at[uid] += len(toks)
            assert r == got.shape[0]
        M.assert_close(rows, want, dtype, f"trace runner, {dtype}")
