"""Small Malazen configurations for the tests, and what the tests share.

The configurations differ from each other in every size and option: heads and groups of the
softmax side (one key head, as many key heads as query heads), key and value sizes (values
smaller and larger than keys, sizes that are no multiple of 16), heads and sizes of the linear
side, scales of the two sides, the query temperature's step, latent ranks and rotated parts,
windows (also none), frequency stretching (also none), norm groups (one, two, three), loops (none,
from the first layer, over layers of either kind, once), layers without a feed-forward, eps,
vocabulary, width, page size.
"""

from __future__ import annotations

import json
from pathlib import Path

import torch


def parallel(heads, kv_heads, dim, vdim, r_heads, r_dim, r_vdim, tau=8.0, scale=None, temp=(0.3, 16), left_scale=0.7,
             right_scale=1.1, decay_rank=5):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
            "scale": float(scale if scale is not None else dim ** -0.5)}
    if temp is not None:
        left["q_temp"] = {"coef": float(temp[0]), "every": int(temp[1])}
    right = {"heads": r_heads, "dim": r_dim, "vdim": r_vdim, "tau": float(tau), "decay_rank": decay_rank}
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": float(left_scale),
                                          "right_scale": float(right_scale)}}


def latent(heads, dim, rot_dim, vdim, kv_rank, window=None, base=10000.0, scaling=None, scale=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
         "scale": float(scale if scale is not None else (dim + rot_dim) ** -0.5),
         "rot": {"dims": rot_dim, "base": float(base)}}
    if scaling is not None:
        m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), map(float, scaling)))
    if window is not None:
        m["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": m}


def with_mlp(layer, ff=None, limit=1.5):
    layer = dict(layer)
    layer["mlp"] = None if ff is None else {"kind": "dense", "ff": ff, "limit": float(limit)}
    return layer


def model(width, vocab, eps, groups, layers, loop=None):
    cfg = {"architecture": "Malazen", "width": width, "vocab": vocab, "norm": {"eps": eps, "groups": groups},
           "layers": layers}
    if loop is not None:
        cfg["loop"] = dict(zip(("start", "stop", "times"), loop))
    return cfg


# S: a loop over one layer of each kind, twice; one key head for four query heads; values smaller
# than keys on the softmax side and larger on the linear side; a window shorter than a page run; a
# last layer without a feed-forward; three norm groups
MODEL_S = model(72, 193, 1e-5, 3, [
    with_mlp(latent(3, 16, 8, 24, 40, window=21, scaling=(4.0, 64, 8.0, 1.0)), 88),
    with_mlp(parallel(4, 1, 32, 16, 2, 24, 40, tau=4.0, temp=(0.5, 7)), 56, limit=0.8),
    with_mlp(latent(2, 24, 16, 8, 24, window=70, base=500.0), 40),
    with_mlp(parallel(2, 2, 16, 48, 3, 8, 16, temp=None, left_scale=1.0, right_scale=0.5, decay_rank=2)),
], loop=(1, 3, 2))
PAGE_S = 16

# T: no loop; a latent layer that sees every key; one norm group; sizes that are no multiples of
# 8 on the linear side; many query heads on the latent side; a latent and a rotated part that
# together make a head of 128, which the tensor-core attention takes (bfloat16)
MODEL_T = model(64, 211, 3e-6, 1, [
    with_mlp(parallel(6, 3, 16, 16, 1, 40, 24, tau=16.0, temp=(0.2, 64), left_scale=0.4, right_scale=0.9), 96, limit=3.0),
    with_mlp(latent(8, 8, 4, 8, 12, scaling=(2.0, 32, 4.0, 0.5)), 48),
    with_mlp(latent(2, 32, 32, 40, 96, window=33, base=1000.0), 72, limit=1.0),
])
PAGE_T = 8

# U: extremes.  The loop starts at the first layer and runs three times over a single layer; a
# loop of one pass in the other model below; a window of one token (a row sees itself and the
# sink only); a width that is no multiple of 8 (no row pitch of 16 bytes: the CUDA-core
# products also in bfloat16); heads of 64 on the softmax side with eight query heads on one key head
MODEL_U = model(100, 150, 1e-6, 2, [
    with_mlp(parallel(8, 1, 64, 64, 2, 64, 64, tau=2.0, temp=(0.4, 1), left_scale=0.6, right_scale=1.2, decay_rank=8), 36),
    with_mlp(latent(1, 48, 2, 64, 30, window=1), 50),
    with_mlp(latent(4, 16, 16, 16, 48, window=300, scaling=(8.0, 16, 2.0, 1.0))),
], loop=(0, 1, 3))
PAGE_U = 16

MODEL_V = model(48, 97, 1e-5, 2, [
    with_mlp(latent(2, 16, 8, 16, 24, window=12), 32),
    with_mlp(parallel(2, 1, 16, 32, 1, 16, 16), 32),
], loop=(0, 2, 1))

# W: odd sizes everywhere: projections with an odd number of rows, heads of 10 and 6, a latent of 21, a
# rank of 1, a feed-forward of 27, a vocabulary and a width that are no multiples of 8
MODEL_W = model(52, 101, 2e-6, 4, [
    with_mlp(latent(3, 10, 6, 14, 21, window=9, base=77.0, scaling=(1.5, 40, 6.0, 0.7)), 27, limit=0.9),
    with_mlp(parallel(3, 3, 10, 6, 3, 6, 10, tau=3.0, temp=(0.7, 3), left_scale=1.4, right_scale=0.3, decay_rank=1), 30),
    with_mlp(parallel(5, 1, 24, 40, 1, 10, 6, tau=1.0, temp=(0.1, 50), left_scale=0.2, right_scale=1.0, decay_rank=3)),
    with_mlp(latent(1, 6, 10, 22, 5), 14),
], loop=(1, 4, 2))

MODELS = {"S": (MODEL_S, PAGE_S), "T": (MODEL_T, PAGE_T), "U": (MODEL_U, PAGE_U), "V": (MODEL_V, 8), "W": (MODEL_W, 32)}


def one_layer(layer, width=48, vocab=97, eps=1e-5, groups=2, loop=None):
    return model(width, vocab, eps, groups, [layer], loop)


# standard deviation of the random matrices: with unit-size normed rows and no norm on queries and
# keys, larger weights make every softmax a choice of one key (the tests that want that ask for it)
INIT_STD = 0.15


def make_folder(tmp_path, config, seed: int, dtype: str, init_std: float = INIT_STD, edit=None) -> Path:
    """A model folder of random weights; ``edit(tensors)`` may change them before they are
    written (a test that needs weights which make a fault show)."""
    from safetensors.torch import save_file

    from lockstep_b200.config import config_from_dict
    from lockstep_b200.engine.model import expected_weights
    from lockstep_b200.weights.random_init import random_tensors

    folder = Path(tmp_path) / f"malazen-{seed}-{dtype}"
    folder.mkdir(parents=True, exist_ok=True)
    cfg = config_from_dict(config)
    tensors = random_tensors(expected_weights(cfg.model_spec()), seed, dtype, init_std, 0.1)
    if edit is not None:
        edit(tensors)
    (folder / "config.json").write_text(json.dumps(cfg.to_dict(), indent=1))
    save_file({k: v.contiguous() for k, v in tensors.items()}, str(folder / "model.safetensors"))
    return folder


def plain_logits(folder, tokens) -> torch.Tensor:
    from plain import malazen_plain as plain

    return plain.model_logits(folder, tokens, torch.float64)


# Error bounds relative to 1 + the request's largest plain logit: in float32 the rounding of sums
# a few hundred terms long and of a state carried over a few hundred tokens (a product or a state
# that lost mantissa bits would be a hundred times above it); in bfloat16 the rounding of every
# product's output to 8 bits of mantissa.
# (Measured on these models: float32 up to 6e-6; bfloat16 up to 6e-2, where loops that feed the
# embedding in again and queries without a norm make logits and scores large.)
TOLERANCE = {"float32": 4e-5, "bfloat16": 8e-2}


# In bfloat16 a row now and then sits where a softmax is undecided between two keys and the rounding
# of a score tips it: up to one row in a hundred may exceed the bound, none may exceed twice the bound.
TAIL = {"float32": 0.0, "bfloat16": 0.01}


def assert_close(rows, plain_by_uid, dtype, what, slack=1.0):
    """``slack``: a factor on the bound, for weights that amplify rounding on purpose."""
    worst, bad = 0.0, []
    bound = slack * TOLERANCE[dtype]
    for (uid, pos), got in sorted(rows.items()):
        want = plain_by_uid[uid][pos].float()
        err = float((got - want).abs().max()) / (1.0 + float(plain_by_uid[uid].abs().max()))
        worst = max(worst, err)
        if not err <= bound:
            bad.append((uid, pos, err))
    allowed = int(TAIL[dtype] * len(rows))
    assert len(bad) <= allowed and all(e <= 2 * bound for _, _, e in bad), (
        f"{what}: {len(bad)} of {len(rows)} rows are off ({allowed} allowed below twice the bound); the first is "
        f"request {bad[0][0]} position {bad[0][1]}: relative error {bad[0][2]:.3e} > {bound:.1e}")
    return worst
