"""minGRU: a gated recurrence whose gates read only the current token.

    z = sigmoid(W_z h + b_z)        u = W_x h + b_x        c = u + 1/2 (u >= 0),  sigmoid(u) (u < 0)
    S_t = (1 - z) S_(t-1) + z c     per channel, S = 0 before a sequence's first token
    out = W_o ( S_t * silu(W_g h) )

The three input projections are one packed product with float32 results; gates, candidate and state
are float32.  The state of a request is a row of the engine's per-request state table, carried from
step to step.  A portion's tokens are scanned serially per channel, or in chunks (three short
kernels) where a step brings long portions.
"""
from __future__ import annotations

from typing import List

import torch

from .. import kernels
from ..config.plan import GatedRecurrenceSpec
from ..weights.loader import WeightSpec
from .base import Mixer, StepContext, register_mixer
from .linear import linear

# from this many tokens in a step on, the scan runs in chunks
CHUNKED_FROM = 256


class MinGRU(Mixer):
    kind = "min_gru"
    graph_safe = True

    def __init__(self, spec: GatedRecurrenceSpec, prefix: str, dtype, device):
        super().__init__(spec, prefix, dtype, device)
        self.w_zxg = self.w_o = self.b_z = self.b_x = None

    @classmethod
    def weight_specs(cls, spec: GatedRecurrenceSpec, prefix: str) -> List[WeightSpec]:
        W, H = spec.width, spec.hidden
        return [WeightSpec(prefix + "z", (W, H)), WeightSpec(prefix + "z.b", (W,), "unit"),
                WeightSpec(prefix + "x", (W, H)), WeightSpec(prefix + "x.b", (W,), "unit"),
                WeightSpec(prefix + "g", (W, H)), WeightSpec(prefix + "o", (H, W))]

    def load(self, store) -> None:
        p = self.prefix
        parts = [store.get(p + n, self.device, self.dtype, operand=True) for n in ("z", "x", "g")]
        self.w_zxg = torch.cat(parts, dim=0).contiguous()
        del parts
        self.w_o = store.get(p + "o", self.device, self.dtype, operand=True)
        self.b_z = store.get(p + "z.b", self.device, torch.float32).float().contiguous()
        self.b_x = store.get(p + "x.b", self.device, torch.float32).float().contiguous()

    def state_need(self):
        return {"S": ((self.spec.width,), torch.float32)}

    def inner_width(self) -> int:
        return self.spec.width

    def output_weight(self) -> torch.Tensor:
        return self.w_o

    def forward_inner(self, x, ctx: StepContext, cache, state, writes_cache, out, out_scale) -> None:
        T, W = x.shape[0], self.spec.width
        ws = ctx.workspace
        zxg = ws.get("mingru.zxg", (T, 3 * W), torch.float32)
        linear(zxg, x, self.w_zxg, ctx.err)
        scratch = None
        if T >= CHUNKED_FROM and not ctx.fixed_shapes:
            scratch = ws.get("mingru.scan", (3 * T * W,), torch.float32)
        kernels.gated_scan(out, zxg, self.b_z, self.b_x, state["S"], ctx.q_start, ctx.slots, ctx.req_of_token,
                           ctx.num_entries, out_scale, scratch)

    def forward(self, x, ctx: StepContext, cache=None, state=None, writes_cache: bool = True):
        T = x.shape[0]
        inner = ctx.workspace.get("mingru.inner", (T, self.spec.width), self.dtype)
        self.forward_inner(x, ctx, cache, state, writes_cache, inner, 1.0)
        out = ctx.workspace.get("mingru.out", (T, self.spec.hidden), ctx.branch_dtype or self.dtype)
        linear(out, inner, self.w_o, ctx.err)
        return out


register_mixer("min_gru", MinGRU)
