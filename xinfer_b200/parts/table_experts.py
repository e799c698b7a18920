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

* many tokens in bfloat16 whose ids the host knows (a prompt step): the host looks the ids up in its copy of
  the table and so knows how many rows every expert gets; the device groups the rows as before, and each
  expert's contiguous rows go through the library's matrix product (gate/up, the SiLU gate kernel, down).

The down matrices are held side by side, ``[hidden, experts * ff]``, for all forms.
"""
from __future__ import annotations

from typing import List

import numpy as np
import torch

from .. import kernels
from ..config.plan import ExpertTableSpec
from ..weights.loader import WeightSpec
from .base import FeedForward, StepContext, register_feed_forward
from .linear import linear

# up to this many tokens a bfloat16 step takes the dense form
DENSE_MAX_TOKENS = 32
# bfloat16 steps of more tokens whose ids the host knows: per-expert library products (tests switch it off to
# reach the grouped kernels)
PER_EXPERT_LIBRARY_PRODUCTS = True
ROW_STEP = 128
# ... and only where a call is large enough: the form is bound by the host (three launches per expert, about
# 20 us each), the grouped kernels by the device (about 200 TFLOP/s).  Measured on a B200 with 2,048 tokens, 2 of 8
# experts: 0.53 against 1.53 ms at width 4,096, 0.46 against 0.44 ms at 2,048, 0.62 against 0.17 ms at 1,024.
LIBRARY_FROM_FLOP_PER_CALL = 8e9


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
        self.table_host = self.table.cpu().numpy()

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
        ids = ctx.h_token_ids
        by_library = (PER_EXPERT_LIBRARY_PRODUCTS and self.dtype == torch.bfloat16 and not ctx.fixed_shapes and ids is not None
                      and ctx.real_tokens == T and len(ids) == T and int(ids.min()) >= 0
                      and int(ids.max()) < self.table_host.shape[0]
                      and 6.0 * n * s.hidden * s.intermediate > LIBRARY_FROM_FLOP_PER_CALL * 3 * s.experts)
        offsets = ws.get("experts.offsets", (s.experts + 1,), torch.int32)
        perm = ws.get("experts.perm", (n,), torch.int32)
        inv = ws.get("experts.inv", (n,), torch.int32)
        kernels.expert_route(offsets, perm, inv, self.table, ctx.token_ids, ctx.sampled, ctx.req_of_token, T, s.top,
                             s.experts, ctx.err)
        if by_library:
            # Each expert's rows are rounded up to a multiple of ROW_STEP, so that the library meets few distinct
            # shapes (it chooses its kernel anew, on the host, for every shape it has not seen).  The extra rows
            # are the next expert's: what is computed for them here is overwritten when that expert's turn comes,
            # and past the last expert lies spare room that nobody reads.
            counts = np.bincount(self.table_host[ids].ravel(), minlength=s.experts)
            room = n + ROW_STEP
            act = ws.get("experts.act", (room, s.intermediate), self.dtype)
            y = ws.get("experts.y", (room, s.hidden), torch.float32)
            xp = ws.get("experts.x_grouped", (room, s.hidden), self.dtype)
            kernels.expert_gather(xp[:n], x, perm, offsets, s.top)
            gu = ws.get("experts.gate_up", (room, 2 * s.intermediate), self.dtype)
            at = 0
            for e in range(s.experts):
                c = int(counts[e])
                if c == 0:
                    continue
                m = min((c + ROW_STEP - 1) // ROW_STEP * ROW_STEP, room - at)
                torch.mm(xp[at:at + m], self.w_gate_up[e].t(), out=gu[at:at + m])
                kernels.swiglu(act[at:at + m], gu[at:at + m])
                torch.mm(act[at:at + m], self.w_down[:, e * s.intermediate:(e + 1) * s.intermediate].t(),
                         out_dtype=torch.float32, out=y[at:at + m])
                at += c
            y = y[:n]
        else:
            act = ws.get("experts.act", (n, s.intermediate), self.dtype)
            y = ws.get("experts.y", (n, s.hidden), torch.float32)
            kernels.expert_gemm(act, x, self.w_gate_up, offsets, perm, True, s.top, True)
            kernels.expert_gemm(y, act, self.w_down, offsets, perm, False, s.top, False, side_by_side=True)
        out = ws.get("experts.out", (T, s.hidden), ctx.branch_dtype or self.dtype)
        kernels.expert_combine(out, y, inv, s.top)
        return out


register_feed_forward("table_experts", TableExperts)
