"""The Dufitar decoder on the GPU against the plain implementation (plain_dufitar.py): every mechanism alone
through its kernel, then whole models through the step function, the replay program and the generation entry
point - whole prompts, token-by-token decoding, portions down to two tokens, unequal batches, pages that are
used again, planted far keys, window and page edges, the first tokens of a sequence."""
import math

import numpy as np
import pytest
import torch

import plain_dufitar as plain
from dufitar_models import TINY_D, make_folder, prompts
from helpers import build_all_modes, replay_in_process, run_trace

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
F64 = torch.float64


def _k():
    from xinfer_b200 import kernels
    return kernels


def _err():
    return torch.zeros(1, dtype=torch.int32, device=DEV)


def _i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


def _rand(*shape, seed=0, scale=1.0):
    return torch.randn(tuple(shape), generator=torch.Generator().manual_seed(seed), dtype=F64) * scale


# ---------------------------------------------------------------------------------------------
# the norm and the residual arithmetic it takes in
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("x_dtype,branch_dtype,out_dtype", [
    (torch.float32, None, torch.bfloat16), (torch.float32, torch.float32, torch.bfloat16),
    (torch.float32, torch.bfloat16, torch.float32), (torch.bfloat16, torch.bfloat16, torch.bfloat16),
    (torch.float32, torch.float32, torch.float32)])
@pytest.mark.parametrize("branch_norm", [False, True])
@pytest.mark.parametrize("rows,dim", [(37, 48), (5, 1030), (300, 256)])
def test_dynamic_tanh_with_scaled_and_normed_branch(x_dtype, branch_dtype, out_dtype, branch_norm, rows, dim):
    if branch_dtype is None and branch_norm:
        pytest.skip("no branch")
    k = _k()
    x = _rand(rows, dim, seed=1, scale=2.0).to(x_dtype)
    br = _rand(rows, dim, seed=2, scale=3.0).to(branch_dtype) if branch_dtype is not None else None
    alpha, w, b = _rand(seed=3).abs().float() + 0.3, _rand(dim, seed=4).float(), _rand(dim, seed=5).float()
    ba, bw, bb = _rand(seed=6).abs().float() + 0.2, _rand(dim, seed=7).float(), _rand(dim, seed=8).float()
    scale = 0.55
    s = x.double()
    if br is not None:
        v = br.double()
        if branch_norm:
            v = plain.dynamic_tanh(v, ba.double(), bw.double(), bb.double())
        s = s + scale * v
    want_sum = s.to(x_dtype).double()
    want = plain.dynamic_tanh(s, alpha.double(), w.double(), b.double())
    out = torch.full((rows, dim), float("nan"), dtype=out_dtype, device=DEV)
    xd = x.to(DEV)
    err = _err()
    k.dyt_norm(out, xd, alpha.to(DEV), w.to(DEV), b.to(DEV), err, branch=br.to(DEV) if br is not None else None,
               branch_scale=scale, branch_norm=(ba.to(DEV), bw.to(DEV), bb.to(DEV)) if branch_norm else None,
               sum_out=xd if br is not None else None)
    tol = 1e-5 if out_dtype == torch.float32 and x_dtype == torch.float32 else 2e-2
    assert int(err.item()) == 0
    assert (out.double().cpu() - want).abs().max() <= tol * (1 + want.abs().max())
    if br is not None:
        assert (xd.double().cpu() - want_sum).abs().max() <= (1e-5 if x_dtype == torch.float32 else 3e-2) * (1 + want_sum.abs().max())


def test_dynamic_tanh_gathers_rows_and_flags_a_bad_one():
    k = _k()
    x = _rand(9, 40, seed=1).float()
    alpha, w, b = torch.tensor(0.8), _rand(40, seed=2).float(), _rand(40, seed=3).float()
    out = torch.zeros(3, 40, device=DEV)
    err = _err()
    k.dyt_norm(out, x.to(DEV), alpha.to(DEV), w.to(DEV), b.to(DEV), err, rows=_i32([7, 0, 4]))
    want = plain.dynamic_tanh(x.double()[[7, 0, 4]], 0.8, w.double(), b.double())
    assert int(err.item()) == 0 and (out.double().cpu() - want).abs().max() < 1e-5
    k.dyt_norm(out, x.to(DEV), alpha.to(DEV), w.to(DEV), b.to(DEV), err, rows=_i32([7, 9, 4]))
    assert int(err.item()) != 0


@pytest.mark.parametrize("scale", [1.0, 0.35])
@pytest.mark.parametrize("x_dtype,b_dtype", [(torch.float32, torch.float32), (torch.float32, torch.bfloat16),
                                             (torch.bfloat16, torch.bfloat16)])
def test_scaled_addition(scale, x_dtype, b_dtype):
    k = _k()
    x, br = _rand(33, 20, seed=1).to(x_dtype), _rand(33, 20, seed=2).to(b_dtype)
    xd = x.to(DEV)
    k.add(xd, xd, br.to(DEV), scale)
    want = x.double() + scale * br.double()
    assert (xd.double().cpu() - want).abs().max() <= (1e-6 if x_dtype == torch.float32 else 2e-2) * (1 + want.abs().max())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,inter", [(3, 40), (70, 136), (600, 64)])
def test_gelu_gate_equals_plain(dtype, T, inter):
    k = _k()
    gu = _rand(T, 2 * inter, seed=T, scale=2.0).to(dtype)
    out = torch.empty(T, inter, dtype=dtype, device=DEV)
    k.swiglu(out, gu.to(DEV), "gelu_tanh")
    want = plain.gelu_tanh(gu.double()[:, :inter]) * gu.double()[:, inter:]
    assert (out.double().cpu() - want).abs().max() <= (1e-5 if dtype == torch.float32 else 1e-2) * (1 + want.abs().max())
    silu = torch.empty(T, inter, dtype=dtype, device=DEV)
    k.swiglu(silu, gu.to(DEV))
    assert (silu.double().cpu() - want).abs().max() > 1e-2          # the other activation is another function


# ---------------------------------------------------------------------------------------------
# rotation with scaled frequencies and a magnitude, through the kernel that prepares q, k, v
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,d,dv,rot", [
    (4, 2, 16, 24, dict(dims=8, base=1000.0, scaling=dict(factor=8.0, original=64, fast=16.0, slow=2.0))),
    (3, 1, 10, 6, dict(dims=6, base=3000.0, scaling=dict(factor=5.0, original=40, fast=10.0, slow=3.0))),
    (2, 2, 32, 32, dict(dims=32, base=500.0))])
def test_prepare_rotates_neighbours_with_magnitude_and_writes_pages(dtype, nh, nkv, d, dv, rot):
    from xinfer_b200.config.plan import YarnScaling
    from xinfer_b200.parts.rope import inv_frequencies
    k = _k()
    ps, T = 8, 21
    positions = torch.tensor([5, 6, 7, 0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 200, 201, 202, 203, 204, 205, 206])
    req = torch.tensor([0] * 3 + [1] * 11 + [2] * 7)
    qkv = _rand(T, (nh + nkv) * d + nkv * dv, seed=d).to(dtype)
    sc = rot.get("scaling")
    freq = torch.from_numpy(inv_frequencies(rot["base"], rot["dims"], YarnScaling(sc["factor"], sc["original"], sc["fast"], sc["slow"]) if sc else None, True))
    mag = plain.rotary_frequencies(rot)[1]
    pages = 3 * 130
    table = torch.arange(pages, dtype=torch.int32).view(3, 130).flip(1).contiguous()
    kc = torch.zeros(pages, nkv, ps, d, dtype=dtype, device=DEV)
    vc = torch.zeros(pages, nkv, ps, dv, dtype=dtype, device=DEV)
    q = torch.zeros(T, nh, d, dtype=dtype, device=DEV)
    err = _err()
    k.qkv_prepare(q, kc, vc, qkv.to(DEV), None, None, freq.to(DEV), _i32(positions.tolist()), _i32(req.tolist()),
                  table.to(DEV), 130, nh, nkv, d, dv, rot["dims"], True, 0, 1e-6, True, err, rot_magnitude=mag)
    assert int(err.item()) == 0
    x = qkv.double()
    want_q = plain.rotate(x[:, : nh * d].reshape(T, nh, d), positions, rot)
    want_k = plain.rotate(x[:, nh * d:(nh + nkv) * d].reshape(T, nkv, d), positions, rot)
    want_v = x[:, (nh + nkv) * d:].reshape(T, nkv, dv)
    # float32 angles: position * frequency carries the frequency's rounding, 200 * 6e-8 radians here
    tol = 5e-5 if dtype == torch.float32 else 2e-2
    assert (q.double().cpu() - want_q).abs().max() <= tol * (1 + want_q.abs().max())
    for t in range(T):
        page = int(table[req[t], positions[t] // ps])
        slot = int(positions[t]) % ps
        assert (kc[page, :, slot].double().cpu() - want_k[t]).abs().max() <= tol * (1 + want_k.abs().max()), t
        assert (vc[page, :, slot].double().cpu() - want_v[t]).abs().max() <= tol * (1 + want_v.abs().max()), t


# ---------------------------------------------------------------------------------------------
# the latent path: per-head maps as batched products, the prepare kernel, the gate
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_batched_product_takes_views_in_both_weight_orders(dtype):
    k = _k()
    B, M, K, N = 3, 37, 20, 45
    wide = _rand(M, B, K + 5, seed=1).to(dtype).to(DEV)
    a = wide[:, :, :K].transpose(0, 1)                      # [B, M, K] view, rows far apart
    w_nk = _rand(B, N, K, seed=2).to(dtype).to(DEV)
    w_kn = _rand(B, K, N, seed=3).to(dtype).to(DEV)
    out = torch.zeros(B, M, N, dtype=dtype, device=DEV)
    tol = 1e-5 if dtype == torch.float32 else 3e-2
    k.gemm_batched_plain(out, a, w_nk)
    want = torch.einsum("bmk,bnk->bmn", a.double().cpu(), w_nk.double().cpu())
    assert (out.double().cpu() - want).abs().max() <= tol * (1 + want.abs().max())
    k.gemm_batched_plain(out, a, w_kn.transpose(1, 2))
    want = torch.einsum("bmk,bkn->bmn", a.double().cpu(), w_kn.double().cpu())
    assert (out.double().cpu() - want).abs().max() <= tol * (1 + want.abs().max())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("given", [True, False])
@pytest.mark.parametrize("H,d,rd,rank,shares", [(3, 8, 4, 20, False), (5, 16, 8, 24, True), (2, 6, 2, 14, False)])
def test_latent_prepare_norms_rotates_and_writes_rows(dtype, H, d, rd, rank, shares, given):
    """``given``: the queries' latent parts come as a tensor of their own and are copied; otherwise they lie in the
    query rows already (the product that forms them writes them there) and must stay as they are."""
    k = _k()
    ps, T, eps = 8, 14, 1e-5
    rot = dict(dims=rd, base=300.0)
    positions = torch.tensor([0, 1, 2, 3, 4, 5, 6, 7, 8, 77, 78, 79, 80, 81])
    req = torch.tensor([0] * 9 + [1] * 5)
    nq, extra = H * (d + rd), 13
    proj = _rand(T, nq + extra + rank + rd, seed=H, scale=1.5).to(dtype)
    q_lat = _rand(H, T, rank, seed=H + 1).to(dtype)
    norm_w = (_rand(rank, seed=9) * 0.2 + 1).float()
    freq = plain.rotary_frequencies(rot)[0].float()
    table = torch.arange(2 * 16, dtype=torch.int32).view(2, 16).flip(0).contiguous()
    cache = torch.zeros(32, ps, rank + rd, dtype=dtype, device=DEV)
    q_abs = torch.zeros(T, H, rank + rd, dtype=dtype, device=DEV)
    if not given:
        q_abs[:, :, :rank] = q_lat.transpose(0, 1).to(DEV)
    err = _err()
    k.latent_prepare(q_abs, cache, proj.to(DEV), 0, -1 if shares else nq + extra, q_lat.to(DEV) if given else None,
                     None if shares else norm_w.to(DEV),
                     freq.to(DEV), _i32(positions.tolist()), _i32(req.tolist()), table.to(DEV), 16, H, d, rd, rank, rd, eps, 1.0, err)
    assert int(err.item()) == 0
    x = proj.double()
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    want_rot = plain.rotate(x[:, :nq].reshape(T, H, d + rd)[..., d:], positions, rot)
    got = q_abs.double().cpu()
    assert (got[..., rank:] - want_rot).abs().max() <= tol * (1 + want_rot.abs().max())
    assert (got[..., :rank] - q_lat.double().transpose(0, 1)).abs().max() <= tol
    if shares:
        assert not cache.any()
        return
    c = x[:, nq + extra: nq + extra + rank]
    c = c / torch.sqrt((c * c).mean(dim=1, keepdim=True) + eps) * norm_w.double()
    kr = plain.rotate(x[:, None, nq + extra + rank:], positions, rot)[:, 0]
    for t in range(T):
        row = cache[int(table[req[t], positions[t] // ps]), int(positions[t]) % ps].double().cpu()
        assert (row[:rank] - c[t]).abs().max() <= tol * (1 + c.abs().max()), t
        assert (row[rank:] - kr[t]).abs().max() <= tol * (1 + kr.abs().max()), t


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,T,dv,lead", [(3, 11, 10, 7), (4, 70, 16, 8), (2, 5, 24, 16)])
def test_gate_multiplies_heads_by_a_sigmoid(dtype, H, T, dv, lead):
    """Heads laid out head by head into a fresh tensor, and in place on heads that lie token by token (the second and
    third sizes take 16-byte accesses in bfloat16)."""
    k = _k()
    heads = _rand(H, T, dv, seed=1).to(dtype)
    wide = _rand(T, lead + H * dv + 8, seed=2, scale=3.0).to(dtype).to(DEV)
    gate = wide[:, lead:lead + H * dv]
    want = heads.double().transpose(0, 1).reshape(T, H * dv) * torch.sigmoid(gate.double().cpu())
    tol = (1e-6 if dtype == torch.float32 else 2e-2) * (1 + want.abs().max())
    out = torch.zeros(T, H * dv, dtype=dtype, device=DEV)
    k.gate_sigmoid(out, heads.to(DEV), gate)
    assert (out.double().cpu() - want).abs().max() <= tol
    inner = heads.transpose(0, 1).reshape(T, H * dv).contiguous().to(DEV)
    k.gate_sigmoid(inner, inner.view(T, H, dv).transpose(0, 1), gate)
    assert (inner.double().cpu() - want).abs().max() <= tol


# ---------------------------------------------------------------------------------------------
# attention over cached latent rows: the plain kernel and the tensor-core kernel against the oracle
# ---------------------------------------------------------------------------------------------
def _latent_oracle(q, rows, rank, scale, sink, window):
    """q [n, H, dk], rows [n, dk] -> [n, H, rank]: one key/value head, values are the rows' first channels."""
    n, H, dk = q.shape
    mask = plain.visible(n, window)
    out = torch.zeros(n, H, rank, dtype=F64)
    for h in range(H):
        out[:, h] = plain.softmax_rows((q[:, h] @ rows.T) * scale, mask, sink=None if sink is None else sink[h]) @ rows[:, :rank]
    return out


class _Ctx:
    """The few fields of a step context that the latent attention's dispatcher reads."""

    def __init__(self, seqs, starts, ps, dtype, seed, fixed=False):
        from xinfer_b200.parts import Workspace
        need = [(r.shape[0] + ps - 1) // ps for _, r in seqs]
        total = sum(need) + 3
        order = torch.randperm(total, generator=torch.Generator().manual_seed(seed)).tolist()
        dk = seqs[0][1].shape[1]
        pages = torch.full((total, ps, dk), float("nan"), dtype=dtype)
        self.stride = max(need) + 2
        table = torch.full((len(seqs), self.stride), -1, dtype=torch.int32)
        at = 0
        for b, (_, rows) in enumerate(seqs):
            for p in range(need[b]):
                page = order[at]
                at += 1
                table[b, p] = page
                n = min(ps, rows.shape[0] - p * ps)
                pages[page, :n] = rows[p * ps:p * ps + n].to(dtype)
        counts = [q.shape[0] - s for (q, _), s in zip(seqs, starts)]
        self.pages, self.table = pages.to(DEV), table.to(DEV)
        self.q = torch.cat([q[s:] for (q, _), s in zip(seqs, starts)]).to(dtype).to(DEV).contiguous()
        self.bounds = np.concatenate([[0], np.cumsum(counts)]).tolist()
        self.q_start, self.start_pos, self.num_entries = _i32(self.bounds), _i32(starts), len(seqs)
        self.positions = _i32([s + i for s, c in zip(starts, counts) for i in range(c)])
        self.req_of_token = _i32([b for b, c in enumerate(counts) for _ in range(c)])
        self.all_single = all(c == 1 for c in counts)
        self.fixed_shapes = fixed
        self.max_context = max(q.shape[0] for q, _ in seqs)
        self.workspace = Workspace(DEV)
        self.err = _err()


def _latent_attend(seqs, starts, rank, scale, sink, window, ps, dtype, tensor_cores=True, seed=0, fixed=False):
    from xinfer_b200.parts import latent_attention as part
    ctx = _Ctx(seqs, starts, ps, dtype, seed, fixed)
    T, H, _ = ctx.q.shape
    out = torch.full((T, H, rank), float("nan"), dtype=dtype, device=DEV)
    keep = part.USE_TENSOR_CORES
    part.USE_TENSOR_CORES = tensor_cores
    try:
        part.latent_attend(out, ctx.q, ctx.pages, ctx, ctx.table, ctx.stride, ps, window, scale,
                           sink.float().to(DEV) if sink is not None else None)
    finally:
        part.USE_TENSOR_CORES = keep
    assert int(ctx.err.item()) == 0
    res = out.double().cpu()
    return [res[a:b] for a, b in zip(ctx.bounds[:-1], ctx.bounds[1:])]


def _latent_qr(n, H, dk, seed, sharp=1.0):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(n, H, dk, generator=g, dtype=F64) / math.sqrt(dk) * sharp
    rows = torch.randn(n, dk, generator=g, dtype=F64)
    return q, rows


@pytest.mark.parametrize("dtype,tensor_cores", [(torch.float32, False), (torch.bfloat16, False), (torch.bfloat16, True)])
@pytest.mark.parametrize("H,dk,rank", [(3, 24, 20), (4, 32, 16), (5, 96, 72), (16, 48, 40), (2, 576, 512), (40, 32, 24),
                                       (4, 160, 128), (3, 272, 256), (1, 144, 136)])
@pytest.mark.parametrize("sink,window", [(True, None), (False, 19), (True, 70)])
def test_latent_attention_equals_plain_for_unequal_entries(dtype, tensor_cores, H, dk, rank, sink, window):
    """Prompt portions of several lengths and starts beside single tokens, pages in a shuffled order."""
    k = _k()
    if tensor_cores and not k.attn_latent_mma_takes(dk, rank):
        pytest.skip("sizes of the plain kernel only")
    lens, starts = [150, 1, 41, 97, 64, 33], [0, 0, 40, 95, 17, 32]
    scale = 2.5
    seqs = [tuple(t.to(dtype).double() for t in _latent_qr(n, H, dk, 11 * n + H, sharp=2.0)) for n in lens]
    sk = _rand(H, seed=5) if sink else None
    got = _latent_attend(seqs, starts, rank, scale, sk, window, 16, dtype, tensor_cores)
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    for (q, rows), s, o in zip(seqs, starts, got):
        ref = _latent_oracle(q, rows, rank, scale, sk, window)[s:]
        assert (o - ref).abs().max() <= tol * (1 + ref.abs().max())


@pytest.mark.parametrize("fixed", [False, True])
@pytest.mark.parametrize("window", [None, 300])
def test_latent_single_tokens_in_key_ranges(fixed, window):
    """Long contexts, one token each: the key tiles are dealt out to several blocks and merged."""
    H, dk, rank = 6, 48, 32
    lens = [900, 1, 70, 513, 64]
    seqs = [tuple(t.to(torch.bfloat16).double() for t in _latent_qr(n, H, dk, n, sharp=2.0)) for n in lens]
    sk = _rand(H, seed=3)
    got = _latent_attend(seqs, [n - 1 for n in lens], rank, 2.0, sk, window, 16, torch.bfloat16, True, fixed=fixed)
    for (q, rows), o in zip(seqs, got):
        ref = _latent_oracle(q, rows, rank, 2.0, sk, window)[-1:]
        assert (o - ref).abs().max() <= 3e-2 * (1 + ref.abs().max())


@pytest.mark.parametrize("dtype,tensor_cores", [(torch.float32, False), (torch.bfloat16, True)])
@pytest.mark.parametrize("where", ["first", "second", "page_end", "page_start", "tile_end", "tile_start", "far", "previous", "self"])
@pytest.mark.parametrize("decode", [False, True])
def test_one_planted_latent_row_decides_the_output(dtype, tensor_cores, where, decode):
    """Among hundreds of rows one is made to stand out for the last query of every head, so the output is that
    row's value part: a kernel that skips it, or reads a neighbour, is far off."""
    H, dk, rank, ps, n = 4, 32, 16, 16, 600
    j = {"first": 0, "second": 1, "page_end": 31, "page_start": 32, "tile_end": 63, "tile_start": 64, "far": n - 517,
         "previous": n - 2, "self": n - 1}[where]
    q, rows = _latent_qr(n, H, dk, 99)
    for h in range(H):
        q[-1, h] = rows[j] * 0.6
    q, rows = q.to(dtype).double(), rows.to(dtype).double()
    start = n - 1 if decode else n - 37
    got = _latent_attend([(q, rows)], [start], rank, 1.0, torch.zeros(H, dtype=F64), None, ps, dtype, tensor_cores)[0]
    ref = _latent_oracle(q, rows, rank, 1.0, torch.zeros(H, dtype=F64), None)[start:]
    assert (got - ref).abs().max() <= (2e-5 if dtype == torch.float32 else 3e-2) * (1 + ref.abs().max())
    assert (got[-1] - rows[j, :rank]).abs().max() < 5e-2 * (1 + rows[j].abs().max()), "the planted row must carry the output"


@pytest.mark.parametrize("dtype,tensor_cores", [(torch.float32, False), (torch.bfloat16, True)])
@pytest.mark.parametrize("decode", [False, True])
@pytest.mark.parametrize("window", [48, 64, 1, 200])
def test_latent_window_edges(dtype, tensor_cores, decode, window):
    """A row just inside the window decides the output, the same row just outside must not be seen."""
    H, dk, rank, ps, n = 2, 32, 16, 8, 200
    for j, inside in [(n - window, True), (n - window - 1, False), (n - 1, True)]:
        if j < 0:
            continue
        q, rows = _latent_qr(n, H, dk, 5)
        for h in range(H):
            q[-1, h] = rows[j] * 0.6
        q, rows = q.to(dtype).double(), rows.to(dtype).double()
        start = n - 1 if decode else n - 9
        got = _latent_attend([(q, rows)], [start], rank, 1.0, None, window, ps, dtype, tensor_cores)[0]
        ref = _latent_oracle(q, rows, rank, 1.0, None, window)[start:]
        assert (got - ref).abs().max() <= (2e-5 if dtype == torch.float32 else 3e-2) * (1 + ref.abs().max())
        carried = (got[-1] - rows[j, :rank]).abs().max() < 5e-2 * (1 + rows[j].abs().max())
        assert bool(carried) == inside, (j, inside)


@pytest.mark.parametrize("dtype,tensor_cores", [(torch.float32, False), (torch.bfloat16, True)])
def test_a_large_sink_takes_the_weight_of_one_head_only(dtype, tensor_cores):
    H, dk, rank = 3, 32, 16
    q, rows = (t.to(dtype).double() for t in _latent_qr(40, H, dk, 2))
    sink = torch.tensor([-30.0, 30.0, 0.0], dtype=F64)
    got = _latent_attend([(q, rows)], [0], rank, 1.0, sink, None, 8, dtype, tensor_cores)[0]
    free = _latent_attend([(q, rows)], [0], rank, 1.0, None, None, 8, dtype, tensor_cores)[0]
    assert got[:, 1].abs().max() < 1e-6                                       # exp(30) in the denominator
    assert (got[:, 0] - free[:, 0]).abs().max() < 1e-3                        # exp(-30) changes nothing
    assert (got[0, 2] - rows[0, :rank] * (1 / (1 + math.exp(-float(q[0, 2] @ rows[0]))))).abs().max() < 2e-2


# ---------------------------------------------------------------------------------------------
# the grouped-query layers: the engine's attention backend against the kernels that take any size
# ---------------------------------------------------------------------------------------------
def test_window_attention_runs_on_the_attention_backend_and_equals_the_general_kernels(tmp_path):
    """D3's grouped-query layers have key and value heads of one size in steps of 16: in bfloat16 they go to the
    tcgen05 kernels; switched off, the same layers run on the kernels that take any sizes.  Same logits."""
    from xinfer_b200.engine.runner import ModelRunner, StepInput
    from xinfer_b200.parts import talking_attention as ta
    folder = make_folder(str(tmp_path / "model"), "D3", torch.bfloat16)
    ps = prompts("D3", [150, 61])
    outs = []
    keep = ta.USE_ATTENTION_BACKEND
    try:
        for flag in (True, False):
            ta.USE_ATTENTION_BACKEND = flag
            runner = ModelRunner(folder, "bfloat16", block_size=TINY_D["D3"][2], num_blocks=32, max_num_seqs=2)
            assert runner.model.blocks[0].mixer._plain_softmax() == flag
            slots = [runner.open_request() for _ in ps]
            a = runner.step([StepInput(s, p[:-7], list(range(len(p) - 7))) for s, p in zip(slots, ps)]).float().cpu()
            tail = []
            for i in range(7):
                tail.append(runner.step([StepInput(s, p[len(p) - 7 + i:len(p) - 6 + i], [0]) for s, p in zip(slots, ps)]).float().cpu())
            runner.check_errors()
            outs.append(torch.cat([a] + tail))
    finally:
        ta.USE_ATTENTION_BACKEND = keep
    spread = float(outs[0].std())
    assert (outs[0] - outs[1]).abs().max() < 0.1 * spread


# ---------------------------------------------------------------------------------------------
# whole models: every way of cutting, pages used again, layer by layer, generation
# ---------------------------------------------------------------------------------------------
LENGTHS = {"D1": [70, 45, 130, 33], "D2": [97, 41, 260, 150], "D3": [170, 1, 75, 58], "D4": [90, 2, 51, 140],
           "D5": [200, 37, 3, 111]}


def _row_error(got, want):
    """Root mean square over the vocabulary of the difference, its mean taken off."""
    d = got.astype(np.float64) - want
    d = d - d.mean()
    return float(np.sqrt((d * d).mean()))


def _tolerance(dtype, ref, cfg=None, w=None, p=None):
    """float32: a small share of the logits' spread (the engine's float32 against float64).  bfloat16: three
    times what rounding alone causes - the largest row error of the plain run that rounds activations to
    bfloat16 where an engine stores them."""
    spread = max(float(np.std(ref)), 1e-3)
    if dtype == "float32":
        return 3e-5 * spread
    rounded = plain.forward(cfg, w, p, round_to=torch.bfloat16).numpy()
    return max(3.0 * max(_row_error(rounded[i], ref[i]) for i in range(len(p))), 1e-3 * spread)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["D1", "D2", "D3", "D4", "D5"])
def test_every_way_of_cutting_gives_the_plain_logits(name, dtype, tmp_path):
    folder = make_folder(str(tmp_path / "model"), name, torch.float32 if dtype == "float32" else torch.bfloat16)
    ps = prompts(name, LENGTHS[name])
    tb = build_all_modes(ps, seed=len(name))
    out = run_trace(folder, dtype, tb.steps, str(tmp_path / "out"), max_tokens=tb.peak, page_size=TINY_D[name][2],
                    max_num_seqs=4)
    cfg, w = plain.load_folder(folder)
    ref = [plain.forward(cfg, w, p).numpy() for p in ps]
    tol = [_tolerance(dtype, r, cfg, w, p) for r, p in zip(ref, ps)]
    seen, worst = {}, {}
    for step, rows in tb.rows.items():
        got = out[step]
        assert got.shape[0] == len(rows)
        for r, ((mode, i), pos) in enumerate(rows):
            e = _row_error(got[r], ref[i][pos])
            worst[mode] = max(worst.get(mode, 0.0), e / tol[i])
            assert e <= tol[i], (f"{name} {dtype} {mode}: request {i} position {pos} (step {step}) differs by {e:.3g} "
                                 f"> {tol[i]:.3g}: the first wrong token of this mode")
            seen.setdefault((mode, i), set()).add(pos)
    for mode in ("whole", "tail", "portions", "mixed"):
        for i, p in enumerate(ps):
            assert sorted(seen[(mode, i)]) == list(range(len(p))), (mode, i)
    print(name, dtype, "worst error / tolerance per mode:", {k: f"{v:.3g}" for k, v in worst.items()})


@pytest.mark.parametrize("name,dtype", [("D1", "float32"), ("D3", "bfloat16"), ("D2", "bfloat16")])
def test_freed_pages_are_used_again_and_nothing_stale_is_read(name, dtype, tmp_path):
    """Pages that go back to the pool - at a request's end, and behind a window while it runs - are filled with
    NaN before the next step: the logits stay the plain ones and stay finite."""
    from xinfer_b200.engine.runner import ModelRunner
    folder = make_folder(str(tmp_path / "model"), name, torch.float32 if dtype == "float32" else torch.bfloat16)
    ps = prompts(name, LENGTHS[name])
    tb = build_all_modes(ps, seed=3)
    page = TINY_D[name][2]
    runner = ModelRunner(folder, dtype, block_size=page, num_blocks=(tb.peak + page - 1) // page, max_num_seqs=4,
                         poison_freed_pages=True)
    out = replay_in_process(runner, tb.steps)
    assert runner.pages_poisoned > runner.num_blocks
    cfg, w = plain.load_folder(folder)
    ref = [plain.forward(cfg, w, p).numpy() for p in ps]
    tol = [_tolerance(dtype, r, cfg, w, p) for r, p in zip(ref, ps)]
    for step, rows in tb.rows.items():
        assert np.isfinite(out[step]).all(), f"step {step} read a poisoned page"
        for r, ((mode, i), pos) in enumerate(rows):
            assert _row_error(out[step][r], ref[i][pos]) <= tol[i], (mode, i, pos)


def test_cache_groups_follow_the_windows_of_the_layers_that_read_them(tmp_path):
    from xinfer_b200.engine.runner import ModelRunner
    folder = make_folder(str(tmp_path / "model"), "D3", torch.bfloat16)
    runner = ModelRunner(folder, "bfloat16", block_size=32, num_blocks=16, max_num_seqs=2)
    windows = sorted(g.window for g in runner.cache.groups)
    assert windows == [9, 23, 50, 120]          # layer 1's rows are kept for its widest reader (120), not its own 70
    assert runner.layer_caches[3] is None and runner.layer_caches[4] is None and runner.layer_caches[1] is not None
    assert runner.layer_caches[1]["latent"].shape[1:] == (32, 48 + 16)


def test_layers_one_by_one_in_float32(tmp_path):
    """The residual stream after every layer (with its waiting additions) against the plain one."""
    from xinfer_b200.engine.runner import ModelRunner, StepInput
    from xinfer_b200.parts.block import Block
    folder = make_folder(str(tmp_path / "model"), "D1", torch.float32)
    cfg, w = plain.load_folder(folder)
    p = prompts("D1", [29])[0]
    want = []
    plain.forward(cfg, w, p, layers_out=want)
    rec, orig = [], Block.forward

    def spy(self, stream, ctx, cache, state, writes_cache):
        out = orig(self, stream, ctx, cache, state, writes_cache)
        x = out.x.double().clone()
        for a in out.pending:
            t = a.t.double()
            if a.norm is not None:
                alpha, weight, bias = (v.double() for v in a.norm.params())
                t = plain.dynamic_tanh(t, alpha, weight, bias)
            x += a.scale * t
        rec.append(x.cpu())
        return out

    Block.forward = spy
    try:
        runner = ModelRunner(folder, "float32", block_size=8, num_blocks=16, max_num_seqs=2)
        slot = runner.open_request()
        runner.step([StepInput(slot, p[:11], []), ])
        first = [r.clone() for r in rec]
        rec.clear()
        runner.step([StepInput(slot, p[11:], [])])
        runner.check_errors()
    finally:
        Block.forward = orig
    assert len(rec) == len(cfg["layers"])
    for i, (a, b, ref) in enumerate(zip(first, rec, want)):
        got = torch.cat([a, b])
        assert (got - ref).abs().max() <= 2e-5 * (1 + ref.abs().max()), f"layer {i}"


def test_a_step_of_a_sandwich_block_launches_one_norm_kernel_per_sublayer(tmp_path):
    """The norm of a sublayer's output, the scaled addition and the next norm are one kernel."""
    from xinfer_b200 import kernels
    from xinfer_b200.engine.runner import ModelRunner, StepInput
    folder = make_folder(str(tmp_path / "model"), "D1", torch.bfloat16)
    runner = ModelRunner(folder, "bfloat16", block_size=8, num_blocks=16, max_num_seqs=2)
    slot = runner.open_request()
    before = dict(kernels.launch_counts())
    runner.step([StepInput(slot, [1, 2, 3, 4, 5], [4])])
    runner.check_errors()
    after = kernels.launch_counts()
    norms = after.get("dyt_norm", 0) - before.get("dyt_norm", 0)
    adds = sum(after.get(n, 0) - before.get(n, 0) for n in ("add", "add_f32"))
    sublayers = sum(1 + (layer["mlp"] is not None) for layer in TINY_D["D1"][0]["layers"])
    assert norms == sublayers + 1 and adds == 0


def _engine(folder, dtype, page, **kw):
    from xinfer_b200 import Engine, EngineConfig
    opts = dict(weight_path=folder, block_size=page, num_blocks=96, max_num_seqs=4, max_num_batched_tokens=64,
                prefill_chunk_size=16, disable_cuda_graph=True, max_model_len=1024)
    opts.update(kw)
    return Engine(EngineConfig(**opts), dtype)


def _quiet_table(name, t):
    """The head is the embedding table: a smaller table lets the layers decide the next token, so that a
    generated sequence shows a wrong step instead of repeating its last token."""
    return t.float() * 0.15 if name == "embed" else None


def test_greedy_generation_in_float32_equals_plain(tmp_path):
    from xinfer_b200 import SamplingParams
    folder = make_folder(str(tmp_path / "model"), "D1", torch.float32, override=_quiet_table)
    cfg, w = plain.load_folder(folder)
    ps = prompts("D1", [1, 5, 23, 40, 9, 17])       # six requests over four slots, prompts in portions of 16
    eng = _engine(folder, "f32", TINY_D["D1"][2])
    outs = eng.generate_sync(SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True), ps)
    for p, o in zip(ps, outs):
        assert o.decode_output == plain.generate(cfg, w, p, 12)


@pytest.mark.parametrize("graphs", [False, True], ids=["launched", "cuda_graph"])
def test_long_greedy_decoding_in_bfloat16_follows_the_plain_logits(graphs, tmp_path):
    """Each generated token is checked against the plain logits of the sequence the engine produced (bfloat16
    may flip a near-tie): it must be the best token up to the drift.  Long enough for several pages per request,
    for every window to pass over decoded tokens and for pages behind the windows to go back to their pools."""
    from xinfer_b200 import SamplingParams
    folder = make_folder(str(tmp_path / "model"), "D3", torch.bfloat16, override=_quiet_table)
    cfg, w = plain.load_folder(folder)
    ps = prompts("D3", [3, 30, 61])
    eng = _engine(folder, "bf16", TINY_D["D3"][2], disable_cuda_graph=not graphs)
    outs = eng.generate_sync(SamplingParams(max_tokens=200, ignore_eos=True), ps)
    assert eng.runner.last_used_graph == graphs
    for p, o in zip(ps, outs):
        assert o.decoded_length == 200
        seq = p + o.decode_output
        ref = plain.forward(cfg, w, seq)
        slack = 2 * 3.0 * float((plain.forward(cfg, w, seq, round_to=torch.bfloat16) - ref).abs().max())
        for i, tok in enumerate(o.decode_output):
            row = ref[len(p) + i - 1]
            assert row[tok] >= row.max() - slack, (i, tok)


def test_command_line_writes_a_random_folder_and_generates_from_it(tmp_path, capsys):
    """The command line end to end: a folder from a configuration and a seed, then generation from given ids (equal
    to the plain continuation in float32) and from a seeded prompt of a given length."""
    import json
    from xinfer_b200.cli import main
    config = tmp_path / "config.json"
    config.write_text(json.dumps(TINY_D["D4"][0]))
    folder = str(tmp_path / "model")
    assert main(["--random", str(config), "--seed", "4", "--m", folder, "--store-dtype", "f32"]) == 0
    cfg, w = plain.load_folder(folder)
    capsys.readouterr()
    assert main(["--m", folder, "--dtype", "f32", "--prompts", "5,6,7|9,10", "--max-tokens", "4", "--ignore-eos",
                 "--disable-cuda-graph", "--num-blocks", "16"]) == 0
    out = capsys.readouterr().out
    assert ",".join(str(t) for t in plain.generate(cfg, w, [5, 6, 7], 4)) in out and "Decoded tokens: 8" in out
    assert main(["--m", folder, "--prompt-len", "21", "--batch", "3", "--max-tokens", "5", "--ignore-eos", "--num-blocks", "16",
                 "--seed", "1"]) == 0
    assert "Decoded tokens: 15" in capsys.readouterr().out
