"""Mixture of small SiLU-gated experts chosen by a table over token ids.

    experts of a token: table[token id, 0 .. top)  (the entries of a row differ), each with weight 1 / top
    expert e:           W_down_e ( silu(W_gate_e h) * (W_up_e h) ),  no biases
    out = (1 / top) * sum over the token's experts

There is no router: which experts run depends on the token's id alone.  Two forms:

* many tokens: the step's (token, choice) pairs are grouped by expert on the device, two grouped products run
  (gate/up with the gate applied in the same kernel, then down), and a last kernel sums a token's experts in
  the order of its table row;
* few tokens in bfloat16 (a decode step): once most experts are in use their matrices are read anyway, and
  reading them is all the step costs.  ONE dense product with the gate/up matrices stacked gives every expert's
  values for every token, a small kernel keeps a token's own experts (times 1 / top) and zeroes the others, and
  ONE product with the down matrices side by side along K sums them: three launches on the weight-streaming
  product, no grouping.

The down matrices are held side by side, ``[hidden, experts * ff]``, for both forms.
"""
from __future__ import annotations

from typing import List

import torch

from .. import kernels
from ..config.plan import ExpertTableSpec
from ..weights.loader import WeightSpec
from .base import FeedForward, StepContext, register_feed_forward
from .linear import linear

# up to this many tokens a bfloat16 step takes the dense form
DENSE_MAX_TOKENS = 32


class TableExperts(FeedForward):
    kind = "table_experts"
    graph_safe = True

    def __init__(self, spec: ExpertTableSpec, prefix: str, dtype, device):
        super().__init__(spec, prefix, dtype, device)
        if not (0 < spec.top <= spec.experts):
            raise ValueError(f"a token cannot use {spec.top} of {spec.experts} experts")
        self.w_gate_up = self.w_down = self.table = None

    @classmethod
    def weight_specs(cls, spec: ExpertTableSpec, prefix: str) -> List[WeightSpec]:
        out = []
        for e in range(spec.experts):
            p = f"{prefix}e{e}."
            out += [WeightSpec(p + "gate", (spec.intermediate, spec.hidden)),
                    WeightSpec(p + "up", (spec.intermediate, spec.hidden)),
                    WeightSpec(p + "down", (spec.hidden, spec.intermediate))]
        out.append(WeightSpec(prefix + "table", (spec.vocab, spec.top), "choice", spec.experts))
        return out

    def load(self, store) -> None:
        s, p = self.spec, self.prefix
        gu, dn = [], []
        for e in range(s.experts):
            q = f"{p}e{e}."
            gu.append(torch.cat([store.get(q + "gate", self.device, self.dtype, operand=True),
                                 store.get(q + "up", self.device, self.dtype, operand=True)], dim=0))
            dn.append(store.get(q + "down", self.device, self.dtype, operand=True))
        self.w_gate_up = torch.stack(gu).contiguous()      # [experts, 2 ff, hidden]
        self.w_down = torch.cat(dn, dim=1).contiguous()    # [hidden, experts * ff]: side by side along K
        self.table = store.get(p + "table", self.device, self.dtype).to(torch.int32).contiguous()

    def forward(self, x, ctx: StepContext):
        s = self.spec
        T = x.shape[0]
        ws = ctx.workspace
        if self.dtype == torch.bfloat16 and T <= DENSE_MAX_TOKENS:
            gu = ws.get("experts.gu_all", (T, s.experts * 2 * s.intermediate), self.dtype)
            linear(gu, x, self.w_gate_up.view(s.experts * 2 * s.intermediate, s.hidden), ctx.err)
            act = ws.get("experts.act_all", (T, s.experts * s.intermediate), self.dtype)
            kernels.expert_select_gate(act, gu, self.table, ctx.token_ids, ctx.sampled, ctx.req_of_token, s.top, s.experts,
                                       ctx.err)
            out = ws.get("experts.out", (T, s.hidden), ctx.branch_dtype or self.dtype)
            linear(out, act, self.w_down, ctx.err)
            return out
        n = T * s.top
        offsets = ws.get("experts.offsets", (s.experts + 1,), torch.int32)
        perm = ws.get("experts.perm", (n,), torch.int32)
        inv = ws.get("experts.inv", (n,), torch.int32)
        kernels.expert_route(offsets, perm, inv, self.table, ctx.token_ids, ctx.sampled, ctx.req_of_token, T, s.top,
                             s.experts, ctx.err)
        act = ws.get("experts.act", (n, s.intermediate), self.dtype)
        kernels.expert_gemm(act, x, self.w_gate_up, offsets, perm, True, s.top, True)
        y = ws.get("experts.y", (n, s.hidden), torch.float32)
        kernels.expert_gemm(y, act, self.w_down, offsets, perm, False, s.top, False, side_by_side=True)
        out = ws.get("experts.out", (T, s.hidden), ctx.branch_dtype or self.dtype)
        kernels.expert_combine(out, y, inv, s.top)
        return out


register_feed_forward("table_experts", TableExperts)
