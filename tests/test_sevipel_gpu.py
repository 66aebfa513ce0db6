"""Sevipel on the device against the plain implementation: every mechanism's kernels alone,
one-layer models of each mixer, and whole models cut in four ways (whole prompts; a prompt and
then token by token; portions down to two tokens; up to three live requests with portions of
some beside single tokens of others, on so few pages and slots that they are used again), in
float32 and bfloat16; weights made so that a window's edge, a far key or a lost state shows;
greedy generation through the entry point and the scheduler; the trace runner."""

from __future__ import annotations

import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import helpers as H
import sevipel_models as M
from plain import sevipel_plain as plain

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
DEV = "cuda:0"


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

def test_find_portions_lists_runs_of_equal_slots():
    from lockstep_b200 import kernels as K

    slots = [2] * 5 + [0] + [3] * 1100 + [1] * 2 + [4, 4, 4]
    out = torch.full((1 + 3 * 6,), -7, dtype=torch.int32, device=DEV)
    K.find_portions(torch.tensor(slots, dtype=torch.int32, device=DEV), out, 6, K.new_error_word(DEV))
    got = out.tolist()
    assert got[0] == 5
    assert [tuple(got[1 + 3 * p:4 + 3 * p]) for p in range(5)] == [(0, 5, 2), (5, 1, 0), (6, 1100, 3), (1106, 2, 1),
                                                                  (1108, 3, 4)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq, nkv, d, dv, rot, whole", [(4, 2, 32, 16, 16, True), (6, 3, 24, 40, 24, True),
                                                         (3, 3, 40, 24, 0, True), (2, 1, 16, 16, 8, False)])
def test_projection_finish_norms_rotates_and_pads(dtype, nq, nkv, d, dv, rot, whole):
    from lockstep_b200 import kernels as K

    g = torch.Generator().manual_seed(nq * 100 + d)
    tokens, page, pad = 11, 8, -(-max(d, dv) // 16) * 16
    qkv = torch.randn(tokens, nq * d + nkv * (d + dv), generator=g).to(dtype)
    q_gain = (1 + 0.3 * torch.randn(nq * d if whole else d, generator=g)).to(dtype)
    k_gain = (1 + 0.3 * torch.randn(nkv * d if whole else d, generator=g)).to(dtype)
    positions = torch.tensor([3, 4, 5, 6, 7, 8, 9, 10, 0, 1, 2], dtype=torch.int32)
    slot = torch.tensor([1] * 8 + [0] * 3, dtype=torch.int32)
    table = torch.tensor([[4, -1], [2, 0]], dtype=torch.int32)
    base, eps = 1000.0, 1e-5
    ang = torch.arange(16, dtype=torch.float64)[:, None] * base ** (-2.0 * torch.arange(max(rot, 2) // 2, dtype=torch.float64) / max(rot, 2))
    cos, sin = ang.cos().float().to(DEV), ang.sin().float().to(DEV)
    pages = torch.full((5, 2, nkv, page, pad), 9.0, dtype=dtype, device=DEV)
    q_out = torch.full((tokens, nq * pad), 9.0, dtype=dtype, device=DEV)
    err = K.new_error_word(DEV)
    K.qkv_finish(qkv.to(DEV), q_out, pages, q_gain.to(DEV), k_gain.to(DEV), cos, sin, positions.to(DEV), slot.to(DEV),
                 table.to(DEV), nq, nkv, d, dv, pad, rot, eps, whole, True, True, err)
    K.raise_on_fault(err)
    x = qkv.double()
    q, k, v = x[:, :nq * d], x[:, nq * d:(nq + nkv) * d], x[:, (nq + nkv) * d:]
    if whole:
        q, k = plain.rms(q, eps) * q_gain.double(), plain.rms(k, eps) * k_gain.double()
        q, k = q.view(tokens, nq, d), k.view(tokens, nkv, d)
    else:
        q = plain.rms(q.view(tokens, nq, d), eps) * q_gain.double()
        k = plain.rms(k.view(tokens, nkv, d), eps) * k_gain.double()
    q = plain.rotate_halves(q, positions.tolist(), rot, base)
    k = plain.rotate_halves(k, positions.tolist(), rot, base)
    tol = 2e-6 if dtype == torch.float32 else 2e-2
    got_q = q_out.double().cpu().view(tokens, nq, pad)
    assert float((got_q[..., :d] - q).abs().max()) < tol * 4 and float(got_q[..., d:].abs().sum()) == 0.0
    for t in range(tokens):
        pg = int(table[slot[t], positions[t] // page])
        row = pages[pg, :, :, int(positions[t]) % page].double().cpu()
        assert float((row[0, :, :d] - k[t]).abs().max()) < tol * 4 and float(row[0, :, d:].abs().sum()) == 0.0
        assert float((row[1, :, :dv] - v[t].view(nkv, dv)).abs().max()) == 0.0 and float(row[1, :, dv:].abs().sum()) == 0.0


@pytest.mark.parametrize("rule", ["delta", "wkv"])
@pytest.mark.parametrize("H_, G, dk, dv", [(2, 1, 16, 32), (3, 3, 40, 24), (2, 2, 72, 8), (1, 1, 128, 64)])
def test_state_rules_walk_portions_and_carry_their_state(rule, H_, G, dk, dv):
    """Three requests in one call, then the rest of two of them in a second call (one as single
    tokens): the outputs are the plain recurrence over each whole sequence."""
    from lockstep_b200 import kernels as K

    if rule == "wkv":
        G, dv = H_, dk
    g = torch.Generator().manual_seed(dk + dv)
    lengths = {0: 37, 2: 9, 1: 21}
    seqs = {}
    for slot, n in lengths.items():
        q = torch.nn.functional.normalize(torch.randn(n, G, dk, generator=g), dim=-1)
        k = torch.nn.functional.normalize(torch.randn(n, G, dk, generator=g), dim=-1)
        v = torch.randn(n, H_, dv, generator=g)
        decay = torch.rand(n, H_, dk, generator=g) * 0.3 + 0.7
        beta = torch.rand(n, H_, generator=g)
        seqs[slot] = (q, k, v, decay, beta)
    bonus = torch.randn(H_, dk, generator=g)
    rep = H_ // G
    want = {}
    for slot, (q, k, v, decay, beta) in seqs.items():
        qq, kk = q.double().repeat_interleave(rep, 1), k.double().repeat_interleave(rep, 1)
        want[slot] = plain.delta_rule(qq, kk, v.double(), decay.double(), beta.double()) if rule == "delta" \
            else plain.wkv_rule(qq, kk, v.double(), decay.double(), bonus.double())
    state = torch.zeros(4, H_ * dk * dv + 5, dtype=torch.float32, device=DEV)
    err = K.new_error_word(DEV)
    got = {slot: [] for slot in lengths}

    def call(pieces):
        """pieces: [(slot, first, count)] packed into one token axis."""
        cat = lambda i: torch.cat([seqs[s][i][a:a + n] for s, a, n in pieces]).contiguous()
        q, k, v, decay, beta = (cat(i) for i in range(5))
        tokens = q.shape[0]
        slots = torch.tensor(sum(([s] * n for s, _, n in pieces), []), dtype=torch.int32, device=DEV)
        portions = torch.empty(1 + 3 * 4, dtype=torch.int32, device=DEV)
        K.find_portions(slots, portions, 4, err)
        out = torch.empty(tokens, H_ * dv, dtype=torch.float32, device=DEV)
        carry = torch.zeros(tokens, 5, dtype=torch.float32, device=DEV)
        if rule == "delta":
            qkv = torch.cat([q.reshape(tokens, -1), k.reshape(tokens, -1), v.reshape(tokens, -1)], dim=1).to(DEV)
            K.state_rule(K.RULE_DELTA, torch.float32, portions, 4, state, qkv.contiguous(), None, None,
                         decay.reshape(tokens, -1).to(DEV), beta.to(DEV), None, out, carry, 5, 1, H_, G, dk, dv)
        else:
            K.state_rule(K.RULE_WKV, torch.float32, portions, 4, state, q.reshape(tokens, -1).to(DEV),
                         k.reshape(tokens, -1).to(DEV), v.reshape(tokens, -1).to(DEV),
                         decay.reshape(tokens, -1).to(DEV), None, bonus.reshape(-1).to(DEV), out, carry, 5, 1, H_, G, dk, dv)
        at = 0
        for s, _, n in pieces:
            got[s].append(out[at:at + n].cpu())
            at += n

    call([(0, 0, 20), (2, 0, 9), (1, 0, 2)])
    call([(1, 2, 18), (0, 20, 1)])
    for i in range(21, 37):
        call([(0, i, 1)] + ([(1, 20, 1)] if i == 21 else []))
    K.raise_on_fault(err)
    for slot in lengths:
        out = torch.cat(got[slot]).double().view(-1, H_, dv)
        assert out.shape == want[slot].shape
        assert float((out - want[slot]).abs().max()) < 2e-5 * (1 + float(want[slot].abs().max())), (rule, slot)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tokens, experts, top, width, ff", [(1, 5, 3, 48, 40), (70, 6, 2, 64, 48), (300, 40, 4, 32, 24),
                                                              (9, 3, 1, 96, 72)])
def test_routed_experts_part_matches_plain(dtype, tokens, experts, top, width, ff):
    from lockstep_b200 import kernels as K
    from lockstep_b200.parts import Runtime, build_part
    from lockstep_b200.config import PartSpec

    g = torch.Generator().manual_seed(tokens + experts)
    rt = Runtime(device=torch.device(DEV), dtype=dtype, page_size=16, max_positions=8, err=K.new_error_word(DEV))
    part = build_part("feed_forward", PartSpec("routed_experts", {"hidden_size": width, "expert_size": ff,
                                                                   "experts": experts, "top": top}), rt)
    w = {name: (0.4 * torch.randn(spec.shape, generator=g)).to(dtype) for name, spec in part.weight_specs().items()}
    part.bind({k: v.to(DEV) for k, v in w.items()})
    x = torch.randn(tokens, width, generator=g).to(dtype)
    residual = torch.randn(tokens, width, generator=g)
    out = residual.clone().to(DEV)
    part.forward(x.to(DEV), None, out)
    K.raise_on_fault(rt.err)
    want = plain.routed_experts(x.double(), {"m." + k: v.double() for k, v in w.items()}, "m",
                                {"router": {"experts": experts, "top": top}})
    tol = 1e-5 if dtype == torch.float32 else 3e-2
    assert float((out.cpu().double() - residual.double() - want).abs().max()) < tol * (1 + float(want.abs().max()))
    counts = K.kernel_counts()
    assert counts["experts_up"] and counts["experts_down"] and counts["experts_route"]


# ---------------------------------------------------------------------------
# models: one layer of each mixer, then whole models, in four cuttings
# ---------------------------------------------------------------------------

ONE_LAYER = {
    "attention": M.with_mlp(M.attention(4, 2, 32, 16, window=20, rot=(16, 10000.0), scale=0.25)),
    "attention_wide_values": M.with_mlp(M.attention(2, 2, 24, 40, rot=(24, 300.0))),
    # heads of a size the tensor-core attention kernels take (bfloat16)
    "attention_tensor_cores": M.with_mlp(M.attention(4, 2, 64, 48, window=100, rot=(32, 10000.0))),
    "delta": M.with_mlp(M.delta(4, 2, 16, 32, conv=4)),
    "delta_odd": M.with_mlp(M.delta(3, 1, 40, 24, conv=2, decay_rank=2, gate_rank=11)),
    "wkv": M.with_mlp(M.wkv(3, 24)),
    "experts": M.with_mlp(M.wkv(1, 16), 40, 7, 3),
}


@pytest.fixture(scope="module")
def zoo(tmp_path_factory):
    cache = {}

    def get(config, dtype, lengths, seed=7, edit=None, key=None):
        key = (key or str(config), dtype, tuple(lengths))
        if key not in cache:
            folder = M.make_folder(tmp_path_factory.mktemp("sevipel"), config, seed=seed, dtype=dtype, edit=edit)
            requests = {f"r{i}": H.random_tokens(n, config["vocab"], seed=50 + i) for i, n in enumerate(lengths)}
            cache[key] = (folder, requests, {u: M.plain_logits(folder, t).float() for u, t in requests.items()})
        return cache[key]

    return get


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(ONE_LAYER))
def test_one_layer_models_in_every_cutting(zoo, name, dtype):
    folder, requests, want = zoo(M.one_layer(ONE_LAYER[name]), dtype, [45, 130, 9, 77])
    rows = {}
    for plan_name, plan in PLANS.items():
        steps = plan(requests)
        runner = make_runner(folder, dtype, 8, steps)
        rows[plan_name] = H.run_plan(runner, steps)
        # (a one-layer model without experts has no close calls: every row is held to its bound)
        M.assert_close(rows[plan_name], want, dtype, f"{name}, {plan_name}", None if name == "experts" else 0.0)
        runner.cache.audit()
    if dtype == "float32":
        # a row's arithmetic does not depend on how its request was cut or on the batch
        for plan_name in PLANS:
            for key, row in rows["whole"].items():
                assert torch.equal(row, rows[plan_name][key]), (name, plan_name, key)


LENGTHS = {"P": [70, 300, 37, 150, 129], "Q": [45, 210, 90, 33, 260], "R": [40, 190, 75, 131]}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("plan_name", sorted(PLANS))
@pytest.mark.parametrize("model", ["P", "Q", "R"])
def test_whole_models_in_every_cutting(zoo, model, plan_name, dtype):
    config, page = M.MODELS[model]
    folder, requests, want = zoo(config, dtype, LENGTHS[model])
    steps = PLANS[plan_name](requests)
    runner = make_runner(folder, dtype, page, steps)
    rows = H.run_plan(runner, steps)
    M.assert_close(rows, want, dtype, f"model {model}, {plan_name}")
    runner.cache.audit()
    if plan_name == "mixed":
        assert runner.cache.reused_pages() > 0           # five requests on three slots and few pages
    if plan_name == "then_single" and runner.graphs is not None:
        assert runner.graphs.replays > 100               # decoded tokens ran as recorded steps


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_steps_of_a_repeating_shape_are_recorded_and_replayed(zoo, dtype):
    """Portions of 300 tokens with one wanted row: the shape comes again and again, so from its
    third occurrence the step is a recorded one (the portion list, the experts' work lists and
    the states' slots are all read on the device at replay)."""
    config, page = M.MODELS["P"]
    folder, requests, want = zoo(config, dtype, [900, 900, 601], key="recorded")
    steps = []
    for uid, toks in requests.items():
        for i in range(0, len(toks) - 1, 300):
            n = min(300, len(toks) - i)
            steps.append({"entries": [(uid, toks[i:i + n], [n - 1, 0])], "end": [uid] if i + n == len(toks) else []})
    steps.append({"entries": [("r2", requests["r2"][600:601], [0])], "end": ["r2"]})   # the last request ends on a single token
    runner = make_runner(folder, dtype, page, steps, max_live=2)
    rows = H.run_plan(runner, steps)
    assert runner.graphs is not None and runner.graphs.mixed_replays >= 4
    M.assert_close(rows, want, dtype, "recorded steps of 300 tokens")
    fresh = make_runner(folder, dtype, page, steps, max_live=2, use_graphs=False)
    plain_rows = H.run_plan(fresh, steps)
    for key, row in rows.items():
        assert torch.equal(row, plain_rows[key]), key      # a replayed step gives the bits of an unrecorded one


def _sharpen(tensors):
    # a large gain on the keys' and queries' norm makes every row of the softmax pick one or two
    # keys: a key that is wrongly seen or not seen at a window's edge, or a far key that is lost,
    # changes the output by as much as a value
    for name in tensors:
        if name.endswith(("q.norm", "k.norm")):
            tensors[name] = (tensors[name].float() * 3.0).to(tensors[name].dtype)


def sharpness(folder, tokens, window):
    """Of the first layer's softmax rows in the plain model: the median largest weight, how many
    rows have their largest key at the window's far edge, how many more than 200 tokens back."""
    cfg, w = plain.read_model_folder(folder)
    n = len(tokens)
    x = plain.offset_norm(w["embed"][torch.tensor(tokens)], w["l0.norm1"], 1e-5)
    m = cfg["layers"][0]["mixer"]
    k, _ = plain.attention_keys_values(x, w, "l0.mix", m, 1e-5)
    q = plain.rotate_halves((plain.rms(x @ w["l0.mix.q"].T, 1e-5) * w["l0.mix.q.norm"]).view(n, 4, 32), range(n), 16, 10000.0)
    s = torch.einsum("ihd,jhd->hij", q, k.repeat_interleave(2, 1)) * m["scale"]
    i, j = torch.arange(n)[:, None], torch.arange(n)[None, :]
    seen = (j <= i) & ((i - j < window) if window else (j <= i))
    p = torch.softmax(s.masked_fill(~seen[None], float("-inf")), -1)
    best = p.argmax(-1)                                                   # [heads, n]
    rows = torch.arange(n)[None, :]
    at_edge = int(((best == rows - (window - 1)) & (rows >= window)).sum()) if window else 0
    return float(p.max(-1).values.median()), at_edge, int((best < rows - 200).sum())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window", [37, 64, 256, None])
def test_sharp_attention_shows_window_edges_and_far_keys(zoo, window, dtype):
    layer = M.with_mlp(M.attention(4, 2, 32, 16, window=window, rot=(16, 10000.0), scale=0.6))
    config = M.model(48, 97, 1e-5, [layer, M.with_mlp(M.attention(4, 2, 32, 16, window=(window or 0) + 5 if window else 40,
                                                                   rot=(16, 10000.0), scale=0.6, kv_from=0))])
    folder, requests, want = zoo(config, dtype, [620, 300], edit=_sharpen, key=f"sharp{window}")
    sharp, at_edge, far = sharpness(folder, requests["r0"], window)
    assert sharp > 0.5                           # most of a row's weight lies on its largest key
    if window:
        assert at_edge >= 3                      # rows whose largest key is the last one inside the window
    else:
        assert far >= 20                         # rows whose largest key lies more than 200 tokens back
    for plan_name in ("whole", "then_single", "portions", "mixed"):
        steps = PLANS[plan_name](requests)
        runner = make_runner(folder, dtype, 16, steps)
        M.assert_close(H.run_plan(runner, steps), want, dtype, f"sharp attention, window {window}, {plan_name}",
                       close_calls=0.0 if dtype == "float32" else 0.05, slack=3.0)   # (scores are large: their rounding shows)


def _remember(tensors):
    # decays close to one: what the first tokens wrote into the state still weighs in the last
    # token's read-out, so a state that is lost, cleared or mixed up between slots shows
    for name in tensors:
        if name.endswith("A_log"):
            tensors[name] = torch.full_like(tensors[name], -5.0)
        if name.endswith("mix.w0"):
            tensors[name] = torch.full_like(tensors[name], -5.0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_slow_decays_carry_the_first_tokens_through_long_decoding(zoo, dtype):
    config = M.model(64, 131, 1e-5, [M.with_mlp(M.delta(2, 1, 32, 48, conv=3)), M.with_mlp(M.wkv(2, 32), 32, 4, 2)])
    folder, requests, want = zoo(config, dtype, [420, 150, 260, 90], edit=_remember, key="remember")
    # the plain model itself depends on the first token at the last position
    cfg, w = plain.read_model_folder(folder)
    tokens = requests["r0"]
    moved = plain.forward(cfg, w, [(tokens[0] + 1) % 131] + tokens[1:])[-1]
    assert float((moved - want["r0"][-1].double()).abs().max()) > 1e-3
    plans = dict(PLANS, long_decoding=lambda r: H.plan_bulk_then_single(r, tail=200))
    for plan_name, plan in plans.items():
        steps = plan(requests)
        runner = make_runner(folder, dtype, 16, steps, num_pages=4)
        M.assert_close(H.run_plan(runner, steps), want, dtype, f"slow decays, {plan_name}")


# ---------------------------------------------------------------------------
# the entry point, the scheduler, the trace runner
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine(tmp_path, dtype):
    from lockstep_b200 import Engine, Request

    config, page = M.MODELS["P"]
    folder = M.make_folder(tmp_path, config, seed=21, dtype=dtype)
    engine = Engine(folder, dtype=dtype, num_pages=64, page_size=page, max_running=12, max_step_tokens=96,
                    max_seq_len=512)
    prompts = {f"g{i}": H.random_tokens(n, config["vocab"], seed=300 + i)
               for i, n in enumerate([33, 7, 120, 1, 64, 18, 45, 2, 90, 11])}
    got = engine.generate([Request(uid=u, prompt=p, max_new_tokens=8) for u, p in prompts.items()])
    cfg, w = plain.read_model_folder(folder)
    wrong = []
    for uid, prompt in prompts.items():
        assert len(got[uid]) == 8
        rows = plain.forward(cfg, w, list(prompt) + got[uid])     # causal: one pass gives every step's logits
        for i, tok in enumerate(got[uid]):
            row = rows[len(prompt) + i - 1]
            margin = 2 * M.TOLERANCE[dtype] * (1 + float(row.abs().max()))
            if not float(row[tok]) >= float(row.max()) - margin:
                wrong.append((uid, i, tok))
    # (in bfloat16 a router's close call may change a row: see sevipel_models.CLOSE_CALLS)
    assert len(wrong) <= int(M.CLOSE_CALLS[dtype] * 80), (dtype, wrong)
    # ten requests decode as recorded steps of sixteen rows: the padding rows share the padding slot
    assert engine.runner.graphs is not None and engine.runner.graphs.replays > 0
    engine.cache.audit()
    assert engine.cache.live == 0


def test_trace_runner_replays_a_trace(tmp_path):
    config, page = M.MODELS["Q"]
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
