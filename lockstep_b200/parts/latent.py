"""Attention over a cached latent.

Per token the layer caches one small vector c (``kv_rank`` elements, RMS-normed with a gain of its
own) and one rotated key part (``rot_dim`` elements) that all heads share, instead of keys and
values per head.  With q_h = [q_plain,h (``head_dim``) ; q_rot,h (``rot_dim``)] per query head:

    key of head h = [W_uk,h c ; k_rot],   value of head h = W_uv,h c,
    score = (q_plain,h . W_uk,h c + q_rot,h . k_rot) * scale.

Since q_plain,h . (W_uk,h c) = (W_uk,h^T q_plain,h) . c, the attention kernels are given one key head
[c ; k_rot] (padded to a multiple of 16) that every query head reads, queries
[W_uk,h^T q_plain,h ; q_rot,h], and values [c ; 0]; the head's output, a weighted sum of latents, then
goes through W_uv,h.  A prompt's tokens and a decoded token take the same path, so a row does not
depend on how its request was cut.  Rotation is the position encoding's (its tables; neighbouring
pairs or halves), a window and a sink per head are optional.

Kernels: one product for the queries' and the latent's projections, ``latent_finish`` (norm,
rotation, cache write), ``heads_product`` (the two per-head products), the engine's attention
kernels over the paged cache, the output product (csrc/latent.cu, csrc/attention_simt.cu).
"""

from __future__ import annotations

import torch

from .. import kernels as K
from .attention import ScoreExtras, attend
from .base import CacheNeed, Mixer, PositionEncoding, Runtime, WeightSpec, register_part
from .norm import NormedRows

_DEFAULT_NAMES = {"q": "q", "down": "dkv", "down_norm": "dkv.norm", "up_k": "uk", "up_v": "uv", "o": "o",
                  "sink": "sink"}


class LatentAttention(Mixer):
    graph_safe = True
    accepts_normed_rows = True

    def __init__(self, hidden_size, num_heads, head_dim, rot_dim, value_dim, kv_rank, scale, window, norm_eps,
                 position: PositionEncoding, runtime: Runtime, sink=False, names=None):
        self.w, self.H, self.d, self.dr = int(hidden_size), int(num_heads), int(head_dim), int(rot_dim)
        self.dv, self.rank = int(value_dim), int(kv_rank)
        self.scale, self.window, self.eps = float(scale), int(window or 0), float(norm_eps)
        self.sink, self.position, self.rt = bool(sink), position, runtime
        self.pad = -(-(self.rank + self.dr) // 16) * 16          # the one head size the attention kernels see
        if not 16 <= self.pad <= 256:
            raise ValueError(f"kv_rank + rot_dim = {self.rank + self.dr} is not supported: the attention kernels "
                             "take heads of up to 256 elements")
        rot = position.rotary() if position is not None else None
        if self.dr and (rot is None or rot[2] != self.dr):
            raise ValueError("the position encoding must rotate exactly the rot_dim part of a head")
        self.names = dict(_DEFAULT_NAMES)
        self.names.update(names or {})
        self.exact = runtime.dtype == torch.float32
        self.extras = ScoreExtras()

    def cache_need(self):
        return CacheNeed("paged_kv", kv_heads=1, head_dim=self.pad, window=self.window)

    def attention_windows(self):
        return {self.window}

    def weight_specs(self):
        n, H = self.names, self.H
        specs = {n["q"]: WeightSpec((H * (self.d + self.dr), self.w)),
                 n["down"]: WeightSpec((self.rank + self.dr, self.w)),
                 n["down_norm"]: WeightSpec((self.rank,), "gain"),
                 n["up_k"]: WeightSpec((H * self.d, self.rank)),
                 n["up_v"]: WeightSpec((H * self.dv, self.rank)),
                 n["o"]: WeightSpec((self.w, H * self.dv))}
        if self.sink:
            specs[n["sink"]] = WeightSpec((H,), "gain", ("normal", 0.0, 1.0))
        return specs

    def bind(self, t):
        n, H = self.names, self.H
        self.w_in = torch.cat([t[n["q"]], t[n["down"]]], dim=0).contiguous()
        self.gain = t[n["down_norm"]]
        # W_uk per head, transposed: [H, rank, d], so that the fold is a product with rows of weights
        self.w_fold = t[n["up_k"]].view(H, self.d, self.rank).transpose(1, 2).contiguous()
        self.w_up_v = t[n["up_v"]].view(H, self.dv, self.rank).contiguous()
        self.w_o = t[n["o"]]
        if self.sink:
            self.extras = ScoreExtras(sinks=t[n["sink"]].to(torch.float32).contiguous())

    def forward(self, x, ctx, cache, residual):
        rt, t, H = self.rt, residual.shape[0], self.H
        proj = rt.rows(t, self.w_in.shape[0])
        if isinstance(x, NormedRows):
            x.linear(self.w_in, proj, K.EPILOGUE_STORE, rt.err)
        else:
            K.gemm_nt(x, self.w_in, proj, err=rt.err)
        rot = self.position.rotary() if self.dr else None
        cos, sin, _ = rot if rot is not None else (None, None, 0)
        q = rt.rows(t, H * self.pad)
        # few tokens: the finishing kernel folds W_uk into the queries itself (the same bits, a launch fewer)
        few = t <= K.FEW_TOKENS and H * self.d * 4 <= 40 * 1024
        K.latent_finish(proj, q, cache.pages, self.gain, cos, sin, ctx.positions, ctx.token_slot, cache.block_table,
                        H, self.d, self.dr, self.rank, self.pad, self.eps,
                        bool(self.dr and self.position.rotary_interleaved), bool(cache.writes), rt.err,
                        w_fold=self.w_fold if few else None)
        if not few:
            K.heads_product(proj, self.d + self.dr, self.w_fold, q, self.pad)
        attn = attend(rt, q, ctx, cache, H, 1, self.pad, self.window, self.scale, self.exact, self.extras)
        y = rt.rows(t, H * self.dv)
        K.heads_product(attn, self.pad, self.w_up_v, y, self.dv)
        K.gemm_nt(y, self.w_o, residual, K.EPILOGUE_RESIDUAL, err=rt.err)


@register_part("mixer", "latent_attention")
def _build(spec, runtime, position=None, **_):
    return LatentAttention(spec["hidden_size"], spec["num_heads"], spec["head_dim"], spec["rot_dim"],
                           spec["value_dim"], spec["kv_rank"], spec["scale"], spec.get("window", 0), spec["norm_eps"],
                           position, runtime, sink=spec.get("sink", False), names=spec.get("names"))
