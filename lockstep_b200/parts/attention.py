"""Grouped-query attention over the paged cache.

q, k, v projections without bias as one product over the row-concatenated
weights (a row of the product is the same dot product as in three separate
ones), optional per-head RMSNorm of q and k before the rotation, rotation by
the position encoding, write of k and v into the cache pages, causal softmax
attention with an optional window, output projection added into the residual
stream (LockStep: engine/model/qwen3.py:246-277, engine/kernels/attention.py).

Further parameters, for designs that differ from that one:
- ``value_dim``: the size of a value head where it is not the size of a key head.  The cache
  and the attention kernels then work on heads of one padded size D (the larger of the two,
  rounded up to 16): queries and keys are padded with zeros (no score changes), values too
  (the padded outputs are zero and meet zero columns of the output projection).
- ``qk_norm_scope`` "projection": one RMSNorm over the whole query projection and one over
  the whole key projection, with gains of those sizes, before the heads are split ("head":
  one norm per head with a gain of the head's size).
- ``borrows_kv``: the layer has no key or value tensors; the schedule gives it the cache
  entry of another layer, which it reads with its own queries, window and scale.
- ``names``: the local names of its tensors.
"""

from __future__ import annotations

import torch

from .. import kernels as K
from .base import CacheNeed, Mixer, PositionEncoding, Runtime, WeightSpec, register_part
from .norm import NormedRows


_DEFAULT_NAMES = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "o": "o_proj.weight",
                  "q_norm": "q_norm.weight", "k_norm": "k_norm.weight"}


class GQAttention(Mixer):
    graph_safe = True
    accepts_normed_rows = True

    def __init__(self, hidden_size, num_heads, num_kv_heads, head_dim, scale, window, qk_norm_eps,
                 position: PositionEncoding, runtime: Runtime, value_dim=None, qk_norm_scope="head",
                 borrows_kv=False, names=None):
        if num_heads % num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if qk_norm_scope not in ("head", "projection"):
            raise ValueError(f"qk_norm_scope must be head or projection, got {qk_norm_scope!r}")
        self.h, self.nq, self.nkv, self.d = int(hidden_size), int(num_heads), int(num_kv_heads), int(head_dim)
        self.dv = int(value_dim or head_dim)
        self.scope, self.borrows = qk_norm_scope, bool(borrows_kv)
        # the general finishing kernel (norm over the projection, heads padded to one size) where
        # the design asks for any of this; else the per-head kernels and the fused products
        self.wide = self.scope == "projection" or self.dv != self.d or self.borrows or self.d % 16 != 0
        self.pad = -(-max(self.d, self.dv) // 16) * 16 if self.wide else self.d
        if self.pad % 16 or not 16 <= self.pad <= 256:
            raise ValueError(
                f"head size {self.pad} is not supported: the attention kernels take multiples of 16 up to 256")
        self.names = dict(_DEFAULT_NAMES)
        self.names.update(names or {})
        self.scale, self.window = float(scale), int(window or 0)
        self.qk_norm_eps = qk_norm_eps
        self.position, self.rt = position, runtime
        self.w_qkv = self.w_o = self.q_gain = self.k_gain = self.slopes = None
        # in float32 every row takes the tile kernel, so that a row's bits do not
        # depend on whether it was decoded or part of a prompt
        self.exact = runtime.dtype == torch.float32

    def cache_need(self):
        return CacheNeed("paged_kv", kv_heads=self.nkv, head_dim=self.pad, window=self.window)

    def attention_windows(self):
        return {self.window}

    def weight_specs(self):
        n = self.names
        whole = self.scope == "projection"
        specs = {n["q"]: WeightSpec((self.nq * self.d, self.h)),
                 n["o"]: WeightSpec((self.h, self.nq * self.dv))}
        if not self.borrows:
            specs[n["k"]] = WeightSpec((self.nkv * self.d, self.h))
            specs[n["v"]] = WeightSpec((self.nkv * self.dv, self.h))
        if self.qk_norm_eps is not None:
            specs[n["q_norm"]] = WeightSpec((self.nq * self.d if whole else self.d,), "gain")
            if not self.borrows:
                specs[n["k_norm"]] = WeightSpec((self.nkv * self.d if whole else self.d,), "gain")
        return specs

    def bind(self, tensors):
        n = self.names
        parts = [tensors[n["q"]]] if self.borrows else [tensors[n["q"]], tensors[n["k"]], tensors[n["v"]]]
        self.w_qkv = torch.cat(parts, dim=0).contiguous()
        self.w_o = tensors[n["o"]]
        if self.pad != self.dv:
            # the attention's output has heads of the padded size: zero columns meet the padding
            w = torch.zeros((self.h, self.nq, self.pad), dtype=self.w_o.dtype, device=self.w_o.device)
            w[:, :, :self.dv] = self.w_o.view(self.h, self.nq, self.dv)
            self.w_o = w.view(self.h, self.nq * self.pad).contiguous()
        self.slopes = self.position.score_slopes(self.nq)      # asked once: a step allocates nothing for it
        if self.qk_norm_eps is not None:
            self.q_gain = tensors[n["q_norm"]]
            self.k_gain = None if self.borrows else tensors[n["k_norm"]]

    def _project_wide(self, x, ctx, cache, t, cos, sin, rot_dim):
        """q (and k, v) through memory, then the finishing kernel that takes any head sizes."""
        qkv = self.rt.rows(t, self.w_qkv.shape[0])
        if isinstance(x, NormedRows):
            x.linear(self.w_qkv, qkv, K.EPILOGUE_STORE, self.rt.err)
        else:
            K.gemm_nt(x, self.w_qkv, qkv, err=self.rt.err)
        q = self.rt.rows(t, self.nq * self.pad)
        K.qkv_finish(qkv, q, cache.pages, self.q_gain, self.k_gain, cos, sin, ctx.positions, ctx.token_slot,
                     cache.block_table, self.nq, self.nkv, self.d, self.dv, self.pad, rot_dim,
                     self.qk_norm_eps or 0.0, self.scope == "projection", not self.borrows,
                     bool(cache.writes) and not self.borrows, self.rt.err)
        return q

    def forward(self, x, ctx, cache, residual):
        nq, nkv, d = self.nq, self.nkv, self.pad
        t = residual.shape[0]
        rot = self.position.rotary()
        cos, sin, rot_dim = rot if rot is not None else (None, None, 0)
        if self.wide:
            if rot_dim and self.position.rotary_interleaved:
                raise ValueError("rotation of neighbouring pairs is not available with padded heads")
            q = self._project_wide(x, ctx, cache, t, cos, sin, rot_dim)
            return self._attend(q, ctx, cache, residual, t)
        q = self.rt.rows(t, nq * d)
        heads = (q, cache.pages, self.q_gain, self.k_gain, cos, sin, ctx.positions, ctx.token_slot,
                 cache.block_table, nq, nkv, d, rot_dim, self.qk_norm_eps or 0.0, cache.writes, self.rt.err)
        interleaved = bool(rot_dim and self.position.rotary_interleaved)
        # a bias on the scores is known to the CUDA-core attention kernels only
        slopes = self.slopes
        tensor_core_attention = not self.exact and slopes is None
        # few tokens: the product finishes its heads itself (norm, rotation, cache write); else
        # the projection goes through memory and a second kernel does that
        fused = False
        if t <= K.FEW_TOKENS and not self.exact and not interleaved:
            pending = isinstance(x, NormedRows) and x.pending()
            fused = K.gemm_nt_tc_qkv_heads(None if pending else (x.materialize() if isinstance(x, NormedRows) else x),
                                           self.w_qkv, *heads,
                                           normed=(x.h, x.gain, x.eps, x.row_index) if pending else None)
        if not fused:
            qkv = self.rt.rows(t, (nq + 2 * nkv) * d)
            if isinstance(x, NormedRows):
                x.linear(self.w_qkv, qkv, K.EPILOGUE_STORE, self.rt.err)
            else:
                K.gemm_nt(x, self.w_qkv, qkv, err=self.rt.err)
            K.qk_norm_rope_store(qkv, *heads, interleaved=interleaved)
        self._attend(q, ctx, cache, residual, t)

    def _attend(self, q, ctx, cache, residual, t):
        nq, nkv, d = self.nq, self.nkv, self.pad
        slopes = self.slopes
        tensor_core_attention = not self.exact and slopes is None
        attn = self.rt.rows(t, nq * d)
        plan, done = None, False
        if tensor_core_attention and d in (64, 128):
            plan = ctx.attention_plan(self.window, K.attention_prefill_tc_tile_tokens())
            done = not plan.n_tile or K.attention_prefill_tc(
                q, cache.pages, attn, plan.tile_work, plan.n_tile, cache.block_table, nq, nkv, d,
                self.window, self.scale, self.rt.err)
        if not done:
            plan = ctx.attention_plan(self.window)
            if plan.n_tile:
                K.attention_tile(q, cache.pages, attn, None, None, plan.tile_work, plan.n_tile,
                                 cache.block_table, nq, nkv, d, self.window, self.scale, self.rt.err, slopes)
        if plan.n_split:
            part_acc = self.rt.rows(plan.n_slots, nq, d, dtype=torch.float32)
            part_ml = self.rt.rows(plan.n_slots, nq, 2, dtype=torch.float32)
            done = False
            if tensor_core_attention:
                done = K.attention_decode_mma(q, cache.pages, part_acc, part_ml, plan.split_work,
                                              plan.n_split, cache.block_table, nq, nkv, d, self.window,
                                              self.scale, self.rt.err)
            if not done and not self.exact:
                done = K.attention_decode(q, cache.pages, part_acc, part_ml, plan.split_work,
                                          plan.n_split, cache.block_table, nq, nkv, d, self.window,
                                          self.scale, self.rt.err, slopes)
            if not done:
                K.attention_tile(q, cache.pages, None, part_acc, part_ml, plan.split_work,
                                 plan.n_split, cache.block_table, nq, nkv, d, self.window,
                                 self.scale, self.rt.err, slopes)
            K.attention_combine(part_acc, part_ml, attn, plan.combine_items, plan.n_combine, nq, d)
        K.gemm_nt(attn, self.w_o, residual, K.EPILOGUE_RESIDUAL, err=self.rt.err)


@register_part("mixer", "gqa_attention")
def _build(spec, runtime, position=None, **_):
    return GQAttention(spec["hidden_size"], spec["num_heads"], spec["num_kv_heads"], spec["head_dim"],
                       spec["scale"], spec.get("window", 0), spec.get("qk_norm_eps"), position, runtime,
                       value_dim=spec.get("value_dim"), qk_norm_scope=spec.get("qk_norm_scope", "head"),
                       borrows_kv=spec.get("borrows_kv", False), names=spec.get("names"))
