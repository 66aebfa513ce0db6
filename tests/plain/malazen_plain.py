"""The Malazen design written out plainly, one function per mechanism, in float64 by default,
whole sequences at a time and without a cache.  It shares no code with the engine: tests compare
the engine's kernels, cache and step function with it.

Notation: ``x`` [n, width] is a sequence of n tokens at positions 0 .. n-1; linear weights are
[out, in] and applied as ``x @ W.T``; a "mixer" maps the normed residual stream to what is added
to it.  ``w`` is the dictionary of the model's tensors by name, ``p`` a tensor-name prefix.
"""

from __future__ import annotations

import math

import torch


def grouped_rms_norm(x, gain, eps, groups):
    """The vector is cut into ``groups`` equal consecutive parts, each scaled to unit root mean
    square of its own (eps inside the root); the whole is then multiplied by ``gain``."""
    n, width = x.shape
    parts = x.view(n, groups, width // groups)
    parts = parts / torch.sqrt((parts * parts).mean(-1, keepdim=True) + eps)
    return parts.reshape(n, width) * gain


# ---------------------------------------------------------------------------
# the "parallel" mixer: softmax attention with a distance bias beside gated linear attention
# ---------------------------------------------------------------------------

def query_temperature(n, coef, every, dtype=torch.float64):
    """Factor on the query at each position: 1 + coef ln(floor((p + 1) / every) + 1)."""
    p = torch.arange(n, dtype=torch.int64)
    return 1.0 + coef * torch.log((torch.div(p + 1, every, rounding_mode="floor") + 1).to(dtype))


def log_distance_attention(q, k, v, scale, r1, r2, weights=False):
    """q [n, H, d], k [n, G, d], v [n, G, dv], r1 and r2 [H].  Causal softmax attention whose
    score for query i and key j <= i is q.k scale - r1 ln(1 + r2 (i - j))."""
    n, H, _ = q.shape
    rep = H // k.shape[1]
    kk, vv = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
    scores = torch.einsum("ihd,jhd->hij", q, kk) * scale
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    dist = (i - j).clamp(min=0).to(q.dtype)
    scores = scores - r1[:, None, None] * torch.log1p(r2[:, None, None] * dist[None])
    scores = scores.masked_fill((j > i)[None], float("-inf"))
    if weights:
        return torch.softmax(scores, dim=-1)
    return torch.einsum("hij,jhd->ihd", torch.softmax(scores, dim=-1), vv)


def biased_attention_mixer(x, w, p, m, weights=False):
    n = x.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (x @ w[p + ".q"].T + w[p + ".q.b"]).view(n, H, d)
    k = (x @ w[p + ".k"].T + w[p + ".k.b"]).view(n, G, d)
    v = (x @ w[p + ".v"].T + w[p + ".v.b"]).view(n, G, dv)
    t = m.get("q_temp")
    if t:
        q = q * query_temperature(n, t["coef"], t["every"], x.dtype)[:, None, None]
    o = log_distance_attention(q, k, v, m["scale"], w[p + ".r1"], w[p + ".r2"], weights)
    if weights:
        return o
    return o.reshape(n, H * dv) @ w[p + ".o"].T + w[p + ".o.b"]


def channel_decay(x, w, p, tau):
    """alpha = sigmoid(z)^(1/tau) with z from the low-rank map, through its logarithm."""
    z = (x @ w[p + ".a1"].T) @ w[p + ".a2"].T + w[p + ".a2.b"]
    return torch.exp(torch.nn.functional.logsigmoid(z) / tau)


def decayed_outer_product_rule(q, k, v, alpha, state=None):
    """q, k, alpha [n, H, dk], v [n, H, dv].  S [H, dk, dv] from zero (or ``state``):
    S <- diag(alpha_t) S + k_t v_t^T, o_t = S^T q_t.  Returns (o [n, H, dv], S)."""
    n, H, dk = q.shape
    S = torch.zeros(H, dk, v.shape[-1], dtype=q.dtype) if state is None else state.clone()
    out = []
    for t in range(n):
        S = S * alpha[t][:, :, None] + k[t][:, :, None] * v[t][:, None, :]
        out.append(torch.einsum("hkv,hk->hv", S, q[t]))
    return torch.stack(out), S


def gated_linear_mixer(x, w, p, m, eps):
    n = x.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = (x @ w[p + ".q"].T).view(n, H, d) * d ** -0.5
    k = (x @ w[p + ".k"].T).view(n, H, d)
    v = (x @ w[p + ".v"].T).view(n, H, dv)
    alpha = channel_decay(x, w, p, m["tau"]).view(n, H, d)
    o, _ = decayed_outer_product_rule(q, k, v, alpha)
    o = o / torch.sqrt((o * o).mean(-1, keepdim=True) + eps) * w[p + ".norm"]
    gate = x @ w[p + ".g"].T
    return (o.reshape(n, H * dv) * torch.nn.functional.silu(gate)) @ w[p + ".o"].T


def parallel_mixer(x, w, p, m, eps):
    left = biased_attention_mixer(x, w, p + ".left", m["left"])
    right = gated_linear_mixer(x, w, p + ".right", m["right"], eps)
    return m["left_scale"] * left + m["right_scale"] * right


# ---------------------------------------------------------------------------
# latent attention
# ---------------------------------------------------------------------------

def scaled_rotary_tables(n, dims, base, scaling=None, dtype=torch.float64):
    """cos, sin [n, dims/2] of the angles p f_i.  With ``scaling`` (factor, original, fast, slow)
    frequencies below a ramp are divided by ``factor`` and both tables are multiplied by
    0.1 ln(factor) + 1."""
    i = torch.arange(dims // 2, dtype=dtype)
    f = base ** (-2.0 * i / dims)
    mag = 1.0
    if scaling:
        factor, original = float(scaling["factor"]), float(scaling["original"])

        def turn_dim(turns):
            return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

        lo = max(math.floor(turn_dim(float(scaling["fast"]))), 0)
        hi = min(math.ceil(turn_dim(float(scaling["slow"]))), dims - 1)
        ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
        f = f / factor * ramp + f * (1.0 - ramp)
        mag = 0.1 * math.log(factor) + 1.0
    ang = torch.arange(n, dtype=dtype)[:, None] * f[None, :]
    return ang.cos() * mag, ang.sin() * mag


def rotate_pairs(x, cos, sin):
    """x [n, heads, dims]: elements (2i, 2i+1) of every head turned by the angle of column i."""
    u, v = x[..., 0::2], x[..., 1::2]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.stack([u * c - v * s, v * c + u * s], dim=-1).flatten(-2)


def sink_window_attention(q, k, v, scale, window, sink, weights=False):
    """q [n, H, d], k [n, H, d], v [n, H, dv], sink [H].  Query i sees keys j with
    0 <= i - j < window (all j <= i for window 0); the softmax's denominator also holds
    exp(sink) of the head, which has no value.  ``weights``: return the softmax's weights
    [H, n, n] instead."""
    n = q.shape[0]
    scores = torch.einsum("ihd,jhd->hij", q, k) * scale
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    seen = (j <= i) & ((i - j < window) if window else torch.ones_like(j, dtype=torch.bool))
    scores = scores.masked_fill(~seen[None], float("-inf"))
    top = torch.maximum(scores.max(-1, keepdim=True).values, sink[:, None, None])
    e = torch.exp(scores - top)
    p = e / (e.sum(-1, keepdim=True) + torch.exp(sink[:, None, None] - top))
    if weights:
        return p
    return torch.einsum("hij,jhd->ihd", p, v)


def latent_attention_mixer(x, w, p, m, eps, weights=False):
    n = x.shape[0]
    H, d, dr, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    rot = m["rot"]
    cos, sin = scaled_rotary_tables(n, rot["dims"], rot["base"], rot.get("scaling"), x.dtype)
    q = (x @ w[p + ".q"].T).view(n, H, d + dr)
    q_plain, q_rot = q[..., :d], rotate_pairs(q[..., d:], cos, sin)
    down = x @ w[p + ".dkv"].T
    c = down[:, :rank]
    c = c / torch.sqrt((c * c).mean(-1, keepdim=True) + eps) * w[p + ".dkv.norm"]
    k_rot = rotate_pairs(down[:, None, rank:], cos, sin).expand(n, H, dr)
    k_plain = (c @ w[p + ".uk"].T).view(n, H, d)
    v = (c @ w[p + ".uv"].T).view(n, H, dv)
    o = sink_window_attention(torch.cat([q_plain, q_rot], -1), torch.cat([k_plain, k_rot], -1), v,
                              m["scale"], (m.get("mask") or {}).get("size", 0), w[p + ".sink"], weights)
    if weights:
        return o
    return o.reshape(n, H * dv) @ w[p + ".o"].T


# ---------------------------------------------------------------------------
# feed-forward, layers, model
# ---------------------------------------------------------------------------

def clamped_glu(x, w, p, f):
    limit = f["limit"]
    g = (x @ w[p + ".gate"].T + w[p + ".gate.b"]).clamp(max=limit)
    u = (x @ w[p + ".up"].T + w[p + ".up.b"]).clamp(-limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[p + ".down"].T + w[p + ".down.b"]


def layer_forward(x, w, i, layer, cfg):
    eps, groups = cfg["norm"]["eps"], cfg["norm"].get("groups", 1)
    p = f"l{i}"
    h = grouped_rms_norm(x, w[p + ".norm1"], eps, groups)
    if layer["type"] == "parallel":
        x = x + parallel_mixer(h, w, p + ".mix", layer["mixer"], eps)
    elif layer["type"] == "latent_attention":
        x = x + latent_attention_mixer(h, w, p + ".mix", layer["mixer"], eps)
    else:
        raise ValueError(layer["type"])
    if layer.get("mlp"):
        x = x + clamped_glu(grouped_rms_norm(x, w[p + ".norm2"], eps, groups), w, p + ".mlp", layer["mlp"])
    return x


def layer_order(cfg):
    """The layers in the order they run: those of the loop ``times`` times in a row.  Yields
    (layer, True where the embedding output is added before it)."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    start, stop, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, False) for i in range(start)]
    for t in range(times):
        order += [(i, t > 0 and i == start) for i in range(start, stop)]
    return order + [(i, False) for i in range(stop, n)]


def forward(cfg, w, tokens, dtype=torch.float64, trace=None):
    """Logits [n, vocab] of one sequence.  ``trace``: a list that receives the residual stream
    after every layer run."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}
    x0 = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    x = x0
    for i, add_embedding in layer_order(cfg):
        if add_embedding:
            x = x + x0
        x = layer_forward(x, w, i, cfg["layers"][i], cfg)
        if trace is not None:
            trace.append(x.clone())
    x = grouped_rms_norm(x, w["final.norm"], cfg["norm"]["eps"], cfg["norm"].get("groups", 1))
    return x @ w["embed"].T


def read_model_folder(folder):
    """(config dictionary, tensors by name in float64) of a model folder."""
    import json
    from pathlib import Path

    from safetensors.torch import load_file

    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    w = {k: (v.double() if v.is_floating_point() else v) for k, v in load_file(str(folder / "model.safetensors")).items()}
    return cfg, w


def model_logits(folder, tokens, dtype=torch.float64):
    cfg, w = read_model_folder(folder)
    return forward(cfg, w, tokens, dtype)
