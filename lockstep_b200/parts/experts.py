"""A feed-forward of routed experts.

Router logits z = W_router x in float32, scores from ``score`` of z ("sigmoid"), the ``top``
largest scores chosen (ties to the lower index).  Each chosen expert runs on the token's row
times its score (``scale`` "input": the score multiplies what goes into the expert; scores are
not renormalised), an expert being down(act(up(.))) with act the square of relu and no biases;
the token's chosen experts are summed in order of rank and added into the residual stream.

On the device: the router's product, the choice, a sort of the step's (token, choice) pairs by
expert (a counting sort made by one block), the two products over the sorted rows tile by tile
(a tile belongs to one expert), and the sum (csrc/experts.cu).  Nothing goes through the host,
so the part can be recorded in a graph; the work lists are sized for the worst case, every
expert holding a partly filled last tile.
"""

from __future__ import annotations

import torch

from .. import kernels as K
from .base import FeedForward, Runtime, WeightSpec, register_part


class RoutedExperts(FeedForward):
    graph_safe = True

    def __init__(self, hidden_size: int, expert_size: int, experts: int, top: int, runtime: Runtime,
                 score: str = "sigmoid", activation: str = "relu2", scale: str = "input"):
        if (score, activation, scale) != ("sigmoid", "relu2", "input"):
            raise ValueError("routed_experts takes sigmoid scores, squared-relu experts and scores on the input")
        if not 1 <= top <= experts or experts > 512:
            raise ValueError(f"top {top} of {experts} experts is not supported (up to 512 experts)")
        self.h, self.f, self.E, self.top, self.rt = int(hidden_size), int(expert_size), int(experts), int(top), runtime
        self.w_router = self.w_up = self.w_down = None

    def weight_specs(self):
        specs = {"router": WeightSpec((self.E, self.h))}
        for e in range(self.E):
            specs[f"e{e}.up"] = WeightSpec((self.f, self.h))
            specs[f"e{e}.down"] = WeightSpec((self.h, self.f))
        return specs

    def bind(self, t):
        self.w_router = t["router"]
        self.w_up = torch.stack([t[f"e{e}.up"] for e in range(self.E)]).contiguous()       # [E, f, h]
        self.w_down = torch.stack([t[f"e{e}.down"] for e in range(self.E)]).contiguous()   # [E, h, f]

    def forward(self, x, ctx, residual):
        rt, tokens = self.rt, residual.shape[0]
        f32, i32 = torch.float32, torch.int32
        pairs = tokens * self.top
        logits = rt.rows(tokens, self.E, dtype=f32)
        K.gemm_nt(x, self.w_router, logits, err=rt.err)
        ids = rt.rows(tokens, self.top, dtype=i32)
        weights = rt.rows(tokens, self.top, dtype=f32)
        K.experts_route(logits, self.top, ids, weights)
        # bfloat16 products go to the tensor cores where TMA can address the rows (16-byte pitches)
        tensor_cores = (rt.dtype == torch.bfloat16 and K.USE_TENSOR_CORES[0] and self.h % 8 == 0 and self.f % 8 == 0)
        tile = K.experts_tile_rows(tensor_cores)
        max_tiles = min(pairs, pairs // tile + self.E)
        plan = rt.rows(1 + 3 * max_tiles, dtype=i32)
        row_token = rt.rows(pairs, dtype=i32)
        row_weight = rt.rows(pairs, dtype=f32)
        pair_row = rt.rows(pairs, dtype=i32)
        K.experts_plan(ids, weights, self.E, tile, plan, max_tiles, row_token, row_weight, pair_row, rt.err)
        act = rt.rows(pairs, self.f)
        # one expert a token: the second product adds into the residual stream itself (an element has
        # one writer); more: its rows go through memory and are added in order of rank
        alone = self.top == 1
        y = residual if alone else rt.rows(pairs, self.h, dtype=f32)
        down = 2 if alone else 1
        if tensor_cores:
            scaled = rt.rows(pairs, self.h)
            K.experts_gather(x, row_token, row_weight, scaled)
            if not (K.experts_product_tc(0, plan, max_tiles, scaled, self.w_up, act, rt.err)
                    and K.experts_product_tc(down, plan, max_tiles, act, self.w_down, y, rt.err, row_token)):
                raise K.KernelError("routed_experts: the tensor-core product refused shapes it was chosen for")
        else:
            K.experts_product(0, plan, max_tiles, x, row_token, row_weight, self.w_up, act)
            K.experts_product(down, plan, max_tiles, act, row_token, row_weight, self.w_down, y)
        if not alone:
            K.experts_combine(y, pair_row, residual, self.top)


@register_part("feed_forward", "routed_experts")
def _build(spec, runtime, **_):
    return RoutedExperts(spec["hidden_size"], spec["expert_size"], spec["experts"], spec["top"], runtime,
                         score=spec.get("score", "sigmoid"), activation=spec.get("activation", "relu2"),
                         scale=spec.get("scale", "input"))
