"""Small Sevipel configurations for the tests, and what the tests share.

The configurations differ from each other in every size and option: heads and groups, key and
value sizes (values smaller and larger than keys, sizes that are no multiple of 16 or 32),
windows (also none, and a reader with a longer window than the layer whose keys it reads),
rotated part (part of a head, a whole head, none), convolution taps, ranks, experts and how
many are chosen, layers without a feed-forward, eps, vocabulary, width, page size.
"""

from __future__ import annotations

import json
from pathlib import Path

import torch


def attention(heads, kv_heads, dim, vdim, window=None, rot=None, scale=None, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
         "scale": float(scale if scale is not None else dim ** -0.5)}
    if window is not None:
        m["mask"] = {"size": window}
    if rot is not None:
        m["rot"] = {"dims": rot[0], "base": float(rot[1])}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m}


def delta(heads, kv_heads, dim, vdim, conv, decay_rank=6, gate_rank=5):
    return {"type": "channel_delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
                                               "conv": conv, "decay_rank": decay_rank, "gate_rank": gate_rank}}


def wkv(heads, dim, decay_rank=7):
    return {"type": "wkv", "mixer": {"heads": heads, "dim": dim, "decay_rank": decay_rank}}


def with_mlp(layer, ff=None, experts=None, top=None):
    layer = dict(layer)
    layer["mlp"] = None if ff is None else {"kind": "moe", "expert": {"ff": ff},
                                            "router": {"experts": experts, "top": top}}
    return layer


def model(width, vocab, eps, layers):
    return {"architecture": "Sevipel", "width": width, "vocab": vocab, "norm": {"eps": eps}, "layers": layers}


# P: groups of two query heads, values smaller than keys, a reader (layer 4) with a longer window
# than the layer it reads, a layer without a feed-forward, two experts chosen of six
MODEL_P = model(64, 211, 1e-5, [
    with_mlp(attention(4, 2, 32, 16, window=24, rot=(16, 10000.0), scale=0.21), 48, 6, 2),
    with_mlp(delta(4, 2, 16, 32, conv=4), 48, 6, 2),
    with_mlp(wkv(2, 32)),
    with_mlp(delta(2, 2, 48, 16, conv=2, decay_rank=3, gate_rank=9), 40, 6, 2),
    with_mlp(attention(4, 2, 32, 16, window=40, rot=(16, 10000.0), scale=0.3, kv_from=0), 48, 6, 2),
])
PAGE_P = 16

# Q: values larger than keys, sizes that are no multiples of 16 or 32, a whole head rotated, a
# layer that sees every key, a reader with a shorter window, three experts of five, one of three
MODEL_Q = model(96, 157, 3e-6, [
    with_mlp(wkv(3, 24, decay_rank=4), 72, 5, 3),
    with_mlp(attention(6, 3, 24, 40, window=50, rot=(24, 500000.0)), 72, 5, 3),
    with_mlp(attention(3, 3, 40, 24), 56, 3, 1),
    with_mlp(delta(3, 1, 40, 24, conv=3), 72, 5, 3),
    with_mlp(attention(6, 3, 24, 40, window=9, rot=(24, 500000.0), kv_from=1)),
])
PAGE_Q = 8

# R: extremes.  A width that is no multiple of 8 (no row pitch of 16 bytes: the CUDA-core products also in
# bfloat16), a single expert, all experts chosen, convolutions of one tap and of eight, eight query heads on
# one key head at the size the tensor-core attention takes with values half as large, two readers of one
# layer's keys (one without a window, so every key is kept), heads of 8
MODEL_R = model(100, 300, 1e-6, [
    with_mlp(wkv(5, 20, decay_rank=3), 36, 1, 1),
    with_mlp(attention(8, 1, 128, 64, window=1000, rot=(128, 10000.0)), 36, 4, 4),
    with_mlp(delta(2, 2, 64, 64, conv=1, decay_rank=8, gate_rank=8), 50, 9, 2),
    with_mlp(attention(8, 1, 128, 64, window=17, rot=(128, 10000.0), kv_from=1), 36, 4, 4),
    with_mlp(attention(8, 1, 128, 64, rot=(128, 10000.0), kv_from=1)),
    with_mlp(delta(4, 1, 8, 8, conv=8), 36, 4, 1),
])
PAGE_R = 16

MODELS = {"P": (MODEL_P, PAGE_P), "Q": (MODEL_Q, PAGE_Q), "R": (MODEL_R, PAGE_R)}


def one_layer(layer, width=48, vocab=97, eps=1e-5):
    return model(width, vocab, eps, [layer])


def make_folder(tmp_path, config, seed: int, dtype: str, init_std: float = 0.3, edit=None) -> Path:
    """A model folder of random weights; ``edit(tensors)`` may change them before they are
    written (a test that needs weights which make a fault show)."""
    from safetensors.torch import save_file

    from lockstep_b200.config import config_from_dict
    from lockstep_b200.engine.model import expected_weights
    from lockstep_b200.weights.random_init import random_tensors

    folder = Path(tmp_path) / f"sevipel-{seed}-{dtype}"
    folder.mkdir(parents=True, exist_ok=True)
    cfg = config_from_dict(config)
    tensors = random_tensors(expected_weights(cfg.model_spec()), seed, dtype, init_std, 0.1)
    if edit is not None:
        edit(tensors)
    (folder / "config.json").write_text(json.dumps(cfg.to_dict(), indent=1))
    save_file({k: v.contiguous() for k, v in tensors.items()}, str(folder / "model.safetensors"))
    return folder


def plain_logits(folder, tokens) -> torch.Tensor:
    from plain import sevipel_plain as plain

    return plain.model_logits(folder, tokens, torch.float64)


# Error bounds relative to 1 + the request's largest plain logit: in float32 the rounding of sums
# a few hundred terms long and of a state carried over a few hundred tokens (a product or a state
# that lost mantissa bits would be a hundred times above it); in bfloat16 the rounding of every
# product's output to 8 bits of mantissa.
TOLERANCE = {"float32": 4e-5, "bfloat16": 5e-2}
# In bfloat16 a router's input carries the rounding of everything before it, and where two experts'
# scores lie closer than that, the engine and the plain run choose differently: the row then
# differs by a whole expert's output, rightly.  So a few rows of a bfloat16 run may be off; float32
# has no such rows, and it is the float32 run that holds every row to its bound.
CLOSE_CALLS = {"float32": 0.0, "bfloat16": 0.10}


def assert_close(rows, plain_by_uid, dtype, what, close_calls=None, slack=1.0):
    """``slack``: a factor on the bound, for weights that amplify rounding on purpose."""
    worst, bad = 0.0, []
    for (uid, pos), got in sorted(rows.items()):
        want = plain_by_uid[uid][pos].float()
        err = float((got - want).abs().max()) / (1.0 + float(plain_by_uid[uid].abs().max()))
        worst = max(worst, err)
        if not err <= slack * TOLERANCE[dtype]:
            bad.append((uid, pos, err))
    allowed = int((CLOSE_CALLS[dtype] if close_calls is None else close_calls) * len(rows))
    assert len(bad) <= allowed, (
        f"{what}: {len(bad)} of {len(rows)} rows are off ({allowed} allowed); the first is request {bad[0][0]} "
        f"position {bad[0][1]}: relative error {bad[0][2]:.3e} > {TOLERANCE[dtype]:.1e}")
    return worst
