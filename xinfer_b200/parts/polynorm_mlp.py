"""Dense feed-forward with a polynomial activation whose powers are normed:

    out = W_down act(W_up h),    act(z) = a N(z) + b N(z^2) + c N(z^3) + e

Powers are taken element by element; N divides a token's vector by its root mean square (eps under the
root).  The four numbers are a tensor of the layer.  The up projection's results and the activation's
arithmetic are float32.
"""
from __future__ import annotations

from typing import List

import torch

from .. import kernels
from ..config.plan import FeedForwardSpec
from ..weights.loader import WeightSpec
from .base import FeedForward, StepContext, register_feed_forward
from .linear import linear


class PolyNormMLP(FeedForward):
    kind = "polynorm_mlp"
    graph_safe = True

    def __init__(self, spec: FeedForwardSpec, prefix: str, dtype, device):
        super().__init__(spec, prefix, dtype, device)
        if spec.activation != "polynorm":
            raise ValueError(f"this feed-forward has the 'polynorm' activation, not '{spec.activation}'")
        self.w_up = self.w_down = self.coef = None

    @classmethod
    def weight_specs(cls, spec: FeedForwardSpec, prefix: str) -> List[WeightSpec]:
        return [WeightSpec(prefix + "up", (spec.intermediate, spec.hidden)),
                WeightSpec(prefix + "down", (spec.hidden, spec.intermediate)),
                WeightSpec(prefix + "act", (4,), "unit")]

    def load(self, store) -> None:
        p = self.prefix
        self.w_up = store.get(p + "up", self.device, self.dtype, operand=True)
        self.w_down = store.get(p + "down", self.device, self.dtype, operand=True)
        self.coef = store.get(p + "act", self.device, torch.float32).float().contiguous()

    def forward(self, x, ctx: StepContext):
        s = self.spec
        T = x.shape[0]
        ws = ctx.workspace
        z = ws.get("polyff.z", (T, s.intermediate), torch.float32)
        linear(z, x, self.w_up, ctx.err)
        act = ws.get("polyff.act", (T, s.intermediate), self.dtype)
        kernels.polynorm(act, z, self.coef, s.eps)
        out = ws.get("polyff.out", (T, s.hidden), ctx.branch_dtype or self.dtype)
        linear(out, act, self.w_down, ctx.err)
        return out


register_feed_forward("polynorm_mlp", PolyNormMLP)
