"""Attention whose keys and values are linear maps of one cached latent vector per token.

    q_h = [q_h,plain | q_h,rot] = W_q h            head_dim plain and rope_dim rotated channels per head
    [c' | k_r'] = W_dkv h                          kv_rank + rope_dim channels
    c = c' / rms(c') * w_norm,   k_r = rotate(k_r'),   q_h,rot <- rotate(q_h,rot)
    k_h[j] = [W_uk,h c_j | k_r,j],   v_h[j] = W_uv,h c_j
    s_h[i, j] = scale * q_h[i] . k_h[j]            causal, optionally within a window
    p_h[i, j] = exp(s_h[i, j]) / (exp(sink_h) + sum_j' exp(s_h[i, j']))     (``sink``; without: the plain softmax)
    out = W_o ( concat_h(sum_j p_h[i, j] v_h[j]) * sigmoid(W_g h) )          (``gate``; without: no factor)

Only the row ``[c | k_r]`` is cached.  Because ``q_h,plain . (W_uk,h c) = (W_uk,h^T q_h,plain) . c`` and
``sum_j p_j W_uv,h c_j = W_uv,h sum_j p_j c_j``, the step carries each head's plain query part into the latent space
(a batch of small products, one per head), runs attention with ONE key/value head over the cached rows themselves
(kv_rank + rope_dim key channels, the first kv_rank of them the value) and maps the result through ``W_uv,h``
afterwards: no key or value is ever formed per head, for prompts or for single tokens.  A layer with
``shares_cache`` has no ``W_dkv``: it reads the rows another layer wrote, with its own maps, queries, window and sink.
"""
from __future__ import annotations

from typing import List

import torch

from .. import kernels
from ..config.plan import LatentAttentionSpec
from ..weights.loader import WeightSpec
from .base import CacheTensor, LayerCache, Mixer, PagedCacheNeed, StepContext, build_part, register_mixer
from .linear import linear


def batched_product(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor) -> None:
    """out[b] = a[b] . w[b]^T for every b (``a`` [B, M, K], ``w`` [B, N, K], views allowed): the library's batched
    product in bfloat16, the engine's FMA kernel in float32 (true 32-bit)."""
    if a.dtype == torch.bfloat16:
        torch.bmm(a, w.transpose(1, 2), out=out)
    else:
        kernels.gemm_batched_plain(out, a, w)


# bfloat16: both products of the attention on tensor cores where the sizes allow; tests switch it off to compare
USE_TENSOR_CORES = True
# a step of single tokens deals every token's key tiles out to several blocks so that about one block per SM runs
_DECODE_BLOCKS = 148
_DECODE_MIN_TILES = 2


def latent_attend(out, q, pages, ctx: StepContext, table, stride, page_size, window, scale, sink) -> None:
    """Attention of ``q`` ``[T, heads, dk]`` over the cached rows ``pages`` ``[page, slot, dk]`` into ``out``
    ``[T, heads, rank]``: on tensor cores in bfloat16 where the sizes fit, else one warp per (token, head)."""
    T, H, dk = q.shape
    rank = out.shape[-1]
    if USE_TENSOR_CORES and q.dtype == torch.bfloat16 and kernels.attn_latent_mma_takes(dk, rank):
        single = ctx.all_single or ctx.fixed_shapes
        rg = 1 if (single and H <= 16) else 2
        parts, part_o, part_ml = 1, None, None
        if single:
            # key ranges: a replayed step must not look at its actual lengths
            bound = stride * page_size if ctx.fixed_shapes else ctx.max_context
            if window:
                bound = min(bound, window + 63)
            tiles = (max(bound, 1) + 63) // 64
            blocks = max(T, 1) * ((H + 16 * rg - 1) // (16 * rg))
            parts = max(1, min(_DECODE_BLOCKS // blocks, tiles // _DECODE_MIN_TILES, 64))
            if parts > 1:
                part_o = ctx.workspace.get("latent.part_o", (T * H * parts * rank,), torch.float32)
                part_ml = ctx.workspace.get("latent.part_ml", (T * H * parts * 2,), torch.float32)
        kernels.attn_latent_mma(out, q, pages, ctx.q_start, ctx.start_pos, ctx.num_entries, table, stride, window, scale,
                                sink, ctx.err, row_groups=rg, parts=parts, part_o=part_o, part_ml=part_ml)
        return
    kernels.attention_plain(out, q, pages.view(pages.shape[0], 1, pages.shape[1], dk), None, ctx.positions,
                            ctx.req_of_token, table, stride, window, scale, ctx.err, sink=sink, value_dim=rank)


class LatentAttention(Mixer):
    kind = "latent_attention"
    graph_safe = True

    def __init__(self, spec: LatentAttentionSpec, prefix: str, dtype, device):
        super().__init__(spec, prefix, dtype, device)
        if spec.rope is None or not (0 < spec.rope.rotary_dim <= spec.rope_dim):
            raise ValueError("latent attention needs a rotary encoding over at most its rope_dim channels")
        if spec.rope.layout != "interleaved":
            raise ValueError("latent attention rotates pairs of neighbouring channels (layout 'interleaved')")
        self.position = build_part("position", spec.rope, prefix, dtype, device)
        if not hasattr(self.position, "frequencies"):
            raise ValueError("latent attention needs a rotary position encoding that offers its frequencies")
        self.w_in = self.w_uk = self.w_uv = self.w_o = self.norm_w = self.sink = None

    @classmethod
    def weight_specs(cls, spec: LatentAttentionSpec, prefix: str) -> List[WeightSpec]:
        n, H = spec.names, spec.num_heads
        out = [WeightSpec(prefix + n[0], (H * (spec.head_dim + spec.rope_dim), spec.hidden))]
        if not spec.shares_cache:
            out += [WeightSpec(prefix + n[1], (spec.kv_rank + spec.rope_dim, spec.hidden)),
                    WeightSpec(prefix + n[2], (spec.kv_rank,), "norm")]
        out += [WeightSpec(prefix + n[3], (H * spec.head_dim, spec.kv_rank)),
                WeightSpec(prefix + n[4], (H * spec.v_head_dim, spec.kv_rank))]
        if spec.sink:
            out.append(WeightSpec(prefix + n[5], (H,), "unit"))
        if spec.gate:
            out.append(WeightSpec(prefix + n[6], (H * spec.v_head_dim, spec.hidden)))
        out.append(WeightSpec(prefix + n[7], (spec.hidden, H * spec.v_head_dim)))
        return out

    def load(self, store) -> None:
        p, n, s = self.prefix, self.spec.names, self.spec

        def operand(name):
            return store.get(p + name, self.device, self.dtype, operand=True)
        # one projection for everything that reads the layer's input: queries, gate, latent
        parts = [operand(n[0])]
        if s.gate:
            parts.append(operand(n[6]))
        if not s.shares_cache:
            parts.append(operand(n[1]))
            self.norm_w = store.get(p + n[2], self.device, torch.float32).float().contiguous()
        self.w_in = torch.cat(parts, dim=0).contiguous()
        del parts
        H = s.num_heads
        self.w_uk = operand(n[3]).view(H, s.head_dim, s.kv_rank)      # [head, plain channel, latent channel]
        self.w_uv = operand(n[4]).view(H, s.v_head_dim, s.kv_rank)    # [head, value channel, latent channel]
        self.w_o = operand(n[7])
        if s.sink:
            self.sink = store.get(p + n[5], self.device, torch.float32).float().contiguous()

    def cache_need(self) -> PagedCacheNeed:
        s = self.spec
        return PagedCacheNeed((("latent", CacheTensor((s.kv_rank + s.rope_dim,), None, 0)),), s.cache_window)

    def forward(self, x, ctx: StepContext, cache: LayerCache, state=None, writes_cache: bool = True):
        s = self.spec
        if writes_cache == s.shares_cache:
            raise ValueError("a latent attention layer writes the cache exactly when it has a latent projection of its own")
        T = x.shape[0]
        H, d, rd, dv, r = s.num_heads, s.head_dim, s.rope_dim, s.v_head_dim, s.kv_rank
        ws = ctx.workspace
        nq, ng = H * (d + rd), (H * dv if s.gate else 0)
        width = self.w_in.shape[0]
        proj = ws.get("latent.proj", (T, width), self.dtype)
        linear(proj, x, self.w_in, ctx.err)
        # every head's plain query part carried into the latent space, q_lat[h] = q_plain[h] . W_uk,h, written
        # straight into the front of the head's query row
        q_plain = proj[:, :nq].view(T, H, d + rd)[:, :, :d].transpose(0, 1)          # [H, T, d] view
        q_abs = ws.get("latent.q", (T, H, r + rd), self.dtype)
        batched_product(q_abs[:, :, :r].transpose(0, 1), q_plain, self.w_uk.transpose(1, 2))
        pages = cache["latent"]
        table, stride = ctx.tables[cache.group], ctx.strides[cache.group]
        rope = self.position.spec
        kernels.latent_prepare(q_abs, pages, proj, 0, -1 if s.shares_cache else nq + ng, None, self.norm_w,
                               self.position.frequencies(), ctx.positions, ctx.req_of_token, table, stride, H, d, rd, r,
                               rope.rotary_dim, s.norm_eps, rope.magnitude, ctx.err)
        # one key/value head over the cached rows: keys are the whole row, values its first kv_rank channels
        o_lat = ws.get("latent.o_lat", (T, H, r), self.dtype)
        latent_attend(o_lat, q_abs, pages, ctx, table, stride, cache.page_size, s.window, s.scale, self.sink)
        # back out of the latent space, head by head: o[h] = o_lat[h] . W_uv,h^T, written where the output
        # projection reads it; the gate then works in place
        inner = ws.get("latent.inner", (T, H * dv), self.dtype)
        o_heads = inner.view(T, H, dv).transpose(0, 1)                                # [H, T, dv] view
        batched_product(o_heads, o_lat.transpose(0, 1), self.w_uv)
        if s.gate:
            kernels.gate_sigmoid(inner, o_heads, proj[:, nq:nq + ng])
        out = ws.get("latent.out", (T, s.hidden), ctx.branch_dtype or self.dtype)
        linear(out, inner, self.w_o, ctx.err)
        return out


register_mixer("latent_attention", LatentAttention)
