"""The Sevipel design written out plainly, one function per mechanism, in any float type
(float64 by default), whole sequences at a time and without a cache.  It shares no code with
the engine: tests compare the engine's kernels, cache and step function with it.

Notation: ``x`` [n, width] is a sequence of n tokens; linear weights are [out, in] and applied
as ``x @ W.T``; a "mixer" maps the normed residual stream to what is added to it.
"""

from __future__ import annotations

import json
import math
from pathlib import Path

import torch
import torch.nn.functional as F


def rms(x, eps):
    """x scaled to unit root mean square over its last axis (eps inside the root)."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def offset_norm(x, w, eps):
    """The layer norm of the design: the tensor holds the gain minus one."""
    return rms(x, eps) * (1.0 + w)


def rotate_halves(x, positions, dims, base):
    """x [n, heads, d]: the first ``dims`` elements of every head are rotated, element i paired
    with element i + dims/2, by the angle position * base^(-2i/dims)."""
    if not dims:
        return x
    half = dims // 2
    i = torch.arange(half, dtype=x.dtype)
    freq = base ** (-2.0 * i / dims)
    ang = torch.as_tensor(positions, dtype=x.dtype)[:, None] * freq[None, :]
    c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., dims:]], dim=-1)


def window_attention(q, k, v, scale, window):
    """q [n, H, d], k [n, G, d], v [n, G, dv]; query i sees keys j with 0 <= i - j < window
    (every j <= i when window is 0).  Returns [n, H, dv]."""
    n, H, _ = q.shape
    G = k.shape[1]
    rep = H // G
    kk = k.repeat_interleave(rep, dim=1)
    vv = v.repeat_interleave(rep, dim=1)
    scores = torch.einsum("ihd,jhd->hij", q, kk) * scale
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    seen = (j <= i) & ((i - j < window) if window else torch.ones_like(j, dtype=torch.bool))
    scores = scores.masked_fill(~seen[None], float("-inf"))
    p = torch.softmax(scores, dim=-1)
    return torch.einsum("hij,jhd->ihd", p, vv)


def attention_keys_values(x, w, p, m, eps):
    """Keys (after the norm over the whole projection and the rotation) and values of a layer."""
    n = x.shape[0]
    G, d, dv = m["kv_heads"], m["dim"], m["vdim"]
    k = rms(x @ w[p + ".k"].T, eps) * w[p + ".k.norm"]
    rot = m.get("rot") or {}
    k = rotate_halves(k.view(n, G, d), range(n), rot.get("dims", 0), rot.get("base", 1.0))
    v = (x @ w[p + ".v"].T).view(n, G, dv)
    return k, v


def attention_mixer(x, w, p, m, eps, kv=None):
    """``kv``: (keys, values) of the layer this one borrows them from, else its own."""
    n = x.shape[0]
    H, d = m["heads"], m["dim"]
    q = rms(x @ w[p + ".q"].T, eps) * w[p + ".q.norm"]
    rot = m.get("rot") or {}
    q = rotate_halves(q.view(n, H, d), range(n), rot.get("dims", 0), rot.get("base", 1.0))
    k, v = kv if kv is not None else attention_keys_values(x, w, p, m, eps)
    window = (m.get("mask") or {}).get("size", 0)
    o = window_attention(q, k, v, m["scale"], window)
    return o.reshape(n, -1) @ w[p + ".o"].T


def causal_conv(x, taps):
    """x [n, channels], taps [channels, t]: y[i] = sum_j taps[:, j] * x[i - (t - 1 - j)], zeros
    before the start."""
    n, t = x.shape[0], taps.shape[1]
    padded = torch.cat([torch.zeros(t - 1, x.shape[1], dtype=x.dtype), x], dim=0)
    y = torch.zeros_like(x)
    for j in range(t):
        y = y + padded[j:j + n] * taps[:, j][None, :]
    return y


def unit(x):
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + 1e-6)


def delta_rule(q, k, v, g, beta):
    """q, k, g [n, H, dk], v [n, H, dv], beta [n, H].  State S [H, dk, dv] from zero:
    S <- g S (rows); u = beta (v - S^T k); S <- S + k u^T; o = S^T q."""
    n, H, dk = q.shape
    dv = v.shape[-1]
    S = torch.zeros(H, dk, dv, dtype=q.dtype)
    out = []
    for t in range(n):
        S = S * g[t][:, :, None]
        u = beta[t][:, None] * (v[t] - torch.einsum("hkv,hk->hv", S, k[t]))
        S = S + k[t][:, :, None] * u[:, None, :]
        out.append(torch.einsum("hkv,hk->hv", S, q[t]))
    return torch.stack(out)


def channel_delta_mixer(x, w, p, m, eps):
    n = x.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = F.silu(causal_conv(x @ w[p + ".q"].T, w[p + ".q.conv"])).view(n, G, d)
    k = F.silu(causal_conv(x @ w[p + ".k"].T, w[p + ".k.conv"])).view(n, G, d)
    v = F.silu(causal_conv(x @ w[p + ".v"].T, w[p + ".v.conv"])).view(n, H, dv)
    q = unit(q) * d ** -0.5
    k = unit(k)
    rep = H // G
    q, k = q.repeat_interleave(rep, dim=1), k.repeat_interleave(rep, dim=1)
    beta = torch.sigmoid(x @ w[p + ".b"].T)
    z = (x @ w[p + ".a1"].T) @ w[p + ".a2"].T + w[p + ".dt_bias"]
    g = torch.exp(-torch.exp(w[p + ".A_log"])[None, :, None] * F.softplus(z).view(n, H, d))
    o = delta_rule(q, k, v, g, beta)
    o = rms(o, eps) * w[p + ".norm"]
    gate = torch.sigmoid((x @ w[p + ".g1"].T) @ w[p + ".g2"].T).view(n, H, dv)
    return (o * gate).reshape(n, H * dv) @ w[p + ".o"].T


def wkv_rule(r, k, v, decay, bonus):
    """r, k, v, decay [n, H, d], bonus [H, d].  o_t = (S + diag(bonus) k_t v_t^T)^T r_t with
    the state before the token, then S <- diag(decay_t) S + k_t v_t^T."""
    n, H, d = r.shape
    S = torch.zeros(H, d, d, dtype=r.dtype)
    out = []
    for t in range(n):
        kv = k[t][:, :, None] * v[t][:, None, :]
        out.append(torch.einsum("hkv,hk->hv", S + bonus[:, :, None] * kv, r[t]))
        S = decay[t][:, :, None] * S + kv
    return torch.stack(out)


def wkv_mixer(x, w, p, m, eps):
    n = x.shape[0]
    H, d = m["heads"], m["dim"]
    prev = torch.cat([torch.zeros(1, x.shape[1], dtype=x.dtype), x[:-1]], dim=0)
    mix = {s: x + (prev - x) * w[f"{p}.mu.{s}"] for s in "rkvgw"}
    r = (mix["r"] @ w[p + ".r"].T).view(n, H, d)
    k = (mix["k"] @ w[p + ".k"].T).view(n, H, d)
    v = (mix["v"] @ w[p + ".v"].T).view(n, H, d)
    gate = F.silu(mix["g"] @ w[p + ".g"].T)
    decay = torch.exp(-torch.exp(torch.tanh(mix["w"] @ w[p + ".w1"].T) @ w[p + ".w2"].T + w[p + ".w0"]))
    o = wkv_rule(r, k, v, decay.view(n, H, d), w[p + ".u"])
    o = rms(o, eps).reshape(n, H * d) * w[p + ".norm"]
    return (o * gate) @ w[p + ".o"].T


def routed_experts(x, w, p, f):
    """Sigmoid scores, the ``top`` largest chosen, each chosen expert run on score * x:
    down(relu(up(score x))^2), summed."""
    E, top = f["router"]["experts"], f["router"]["top"]
    scores = torch.sigmoid(x @ w[p + ".router"].T)
    # ties go to the lower expert index
    order = torch.sort(scores, dim=-1, descending=True, stable=True).indices[:, :top]
    out = torch.zeros_like(x)
    for e in range(E):
        chosen = (order == e).any(-1)
        if not bool(chosen.any()):
            continue
        xe = x[chosen] * scores[chosen, e][:, None]
        out[chosen] = out[chosen] + torch.relu(xe @ w[f"{p}.e{e}.up"].T) ** 2 @ w[f"{p}.e{e}.down"].T
    return out


def forward(config: dict, w: dict, tokens, layers_out: list | None = None):
    """Logits [n, vocab] of one sequence; ``layers_out`` receives the residual stream after
    every layer."""
    eps = config["norm"]["eps"]
    x = w["embed"][torch.as_tensor(tokens)]
    kept = {}
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}.mix", layer["mixer"]
        y = offset_norm(x, w[f"l{i}.norm1"], eps)
        if layer["type"] == "attention":
            src = m.get("kv_from")
            if src is None:
                kept[i] = attention_keys_values(y, w, p, m, eps)
                x = x + attention_mixer(y, w, p, m, eps, kept[i])
            else:
                x = x + attention_mixer(y, w, p, m, eps, kept[src])
        elif layer["type"] == "channel_delta":
            x = x + channel_delta_mixer(y, w, p, m, eps)
        elif layer["type"] == "wkv":
            x = x + wkv_mixer(y, w, p, m, eps)
        else:
            raise ValueError(layer["type"])
        if layer.get("mlp") is not None:
            y = offset_norm(x, w[f"l{i}.norm2"], eps)
            x = x + routed_experts(y, w, f"l{i}.mlp", layer["mlp"])
        if layers_out is not None:
            layers_out.append(x.clone())
    return offset_norm(x, w["final.norm"], eps) @ w["embed"].T


def read_model_folder(folder, dtype=torch.float64):
    from safetensors.torch import load_file

    folder = Path(folder)
    config = json.loads((folder / "config.json").read_text())
    w = {k: (v.to(dtype) if v.dtype.is_floating_point else v) for k, v in
         load_file(str(folder / "model.safetensors")).items()}
    return config, w


def model_logits(folder, tokens, dtype=torch.float64):
    config, w = read_model_folder(folder, dtype)
    return forward(config, w, tokens)
