"""The Tidarax decoder on the GPU against the plain implementation (plain_tidarax.py): every
mechanism alone through its kernel, then whole models through the step function, the replay program and
the generation entry point - whole prompts, token-by-token decoding, portions down to two tokens,
unequal batches, pages and state slots that are used again, planted far keys, window and page edges."""
import math

import numpy as np
import pytest
import torch

import plain_tidarax as plain
from helpers import build_all_modes, replay_in_process, run_trace
from tidarax_models import TINY_T, make_folder, prompts

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _k():
    from xinfer_b200 import kernels
    return kernels


def _err():
    return torch.zeros(1, dtype=torch.int32, device=DEV)


def _i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


# ---------------------------------------------------------------------------------------------
# the float32 stream's kernels
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("branch_dtype", [None, torch.float32, torch.bfloat16])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_norm_over_a_float32_stream(branch_dtype, out_dtype):
    if out_dtype == torch.float32 and branch_dtype in (None, torch.float32):
        pytest.skip("all-float32 goes through the generic kernel, tested elsewhere")
    k = _k()
    g = torch.Generator().manual_seed(3)
    T, dim, eps = 7, 88, 3e-6
    x = torch.randn(T, dim, generator=g) * 5
    w = torch.randn(dim, generator=g) * 0.3
    br = torch.randn(T, dim, generator=g).to(branch_dtype) if branch_dtype else None
    xd = x.to(DEV)
    out = torch.empty(T, dim, dtype=out_dtype, device=DEV)
    k.rmsnorm(out, xd, w.to(DEV), eps, _err(), branch=br.to(DEV) if br is not None else None,
              sum_out=xd if br is not None else None, weight_offset=1.0)
    s = x.double() + (br.double() if br is not None else 0)
    ref = plain.norm_around_zero(s, w.double(), eps)
    tol = 1e-5 if out_dtype == torch.float32 else 2 ** -8
    assert ((out.double().cpu() - ref).abs() <= tol * ref.abs() + 1e-6).all()
    if br is not None:
        assert torch.allclose(xd.cpu().double(), s, atol=1e-6)       # the float32 sum is stored
    rows = _i32([5, 0, 5])
    out2 = torch.empty(3, dim, dtype=out_dtype, device=DEV)
    k.rmsnorm(out2, xd, w.to(DEV), eps, _err(), rows=rows, weight_offset=1.0)
    assert torch.equal(out2[0], out2[2])
    ref2 = plain.norm_around_zero(xd.cpu().double()[[5, 0, 5]], w.double(), eps)
    assert ((out2.double().cpu() - ref2).abs() <= tol * ref2.abs() + 1e-6).all()


def test_embedding_widens_and_addition_keeps_float32():
    k = _k()
    g = torch.Generator().manual_seed(4)
    table = torch.randn(50, 24, generator=g).to(torch.bfloat16).to(DEV)
    ids = _i32([3, 49, 0, -2])
    sampled = _i32([7, 11, 13])
    out = torch.empty(4, 24, dtype=torch.float32, device=DEV)
    k.embedding(out, table, ids, _err(), sampled)
    assert torch.equal(out.cpu(), table.float().cpu()[[3, 49, 0, 11]])
    x = torch.randn(4, 24, generator=g).to(DEV)
    b = torch.randn(4, 24, generator=g).to(torch.bfloat16).to(DEV)
    want = x + b.float()
    k.add(x, x, b)
    assert torch.equal(x, want)


# ---------------------------------------------------------------------------------------------
# rotation with scaled frequencies, unit norm after it, page write
# ---------------------------------------------------------------------------------------------
def test_scaled_frequencies_equal_the_plain_rule():
    from xinfer_b200.config.plan import RopeScaling
    from xinfer_b200.parts.rope import inv_frequencies
    for dims, base, sc in [(8, 1000.0, dict(factor=8.0, low=1.0, high=4.0, original=64)),
                           (64, 500000.0, dict(factor=32.0, low=1.0, high=4.0, original=8192)),
                           (24, 10000.0, dict(factor=3.0, low=2.0, high=16.0, original=300)), (16, 300.0, None)]:
        got = inv_frequencies(base, dims, RopeScaling(**sc) if sc else None, True)
        ref = np.array(plain.rotary_frequencies(dict(dims=dims, base=base, scaling=sc)))
        assert np.allclose(got, ref, rtol=1e-7, atol=0)
        if sc:   # all three regimes occur in at least one of the cases
            wl = 2 * math.pi / np.array(plain.rotary_frequencies(dict(dims=dims, base=base)))
            assert (wl < sc["original"] / sc["high"]).any()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,d,dv,rot", [(4, 2, 16, 24, 8), (3, 3, 40, 8, 40), (2, 1, 32, 16, 0), (6, 2, 96, 64, 64)])
def test_prepare_rotates_then_norms_and_writes_pages(dtype, nh, nkv, d, dv, rot):
    k = _k()
    g = torch.Generator().manual_seed(nh * 100 + d)
    eps, ps, pages = 1e-5, 8, 9
    # two requests: one continues at position 13 with 6 tokens, one starts at 0 with 3 tokens
    starts, counts = [13, 0], [6, 3]
    T = sum(counts)
    qkv = (torch.randn(T, (nh + nkv) * d + nkv * dv, generator=g) * 2).to(dtype)
    positions = [s + i for s, c in zip(starts, counts) for i in range(c)]
    req = [b for b, c in enumerate(counts) for _ in range(c)]
    table = _i32([[4, 7, 1, -1], [6, -1, -1, -1]])
    rope = dict(dims=rot, base=777.0, scaling=dict(factor=4.0, low=1.0, high=4.0, original=32)) if rot else None
    inv = torch.tensor(plain.rotary_frequencies(rope), dtype=torch.float32, device=DEV) if rot else None
    q_out = torch.zeros(T, nh, d, dtype=dtype, device=DEV)
    kc = torch.zeros(pages, nkv, ps, d, dtype=dtype, device=DEV)
    vc = torch.zeros(pages, nkv, ps, dv, dtype=dtype, device=DEV)
    err = _err()
    k.qkv_prepare(q_out, kc, vc, qkv.to(DEV), None, None, inv, _i32(positions), _i32(req), table, 4, nh, nkv, d, dv, rot,
                  False, 2, eps, True, err)
    assert int(err.item()) == 0
    x = qkv.double()
    pos = torch.tensor(positions)
    q = plain.unit_rms(plain.rotate(x[:, : nh * d].view(T, nh, d), pos, rope), eps)
    kk = plain.unit_rms(plain.rotate(x[:, nh * d:(nh + nkv) * d].view(T, nkv, d), pos, rope), eps)
    vv = x[:, (nh + nkv) * d:].view(T, nkv, dv)
    tol = 2e-6 if dtype == torch.float32 else 2 ** -7
    assert (q_out.double().cpu() - q).abs().max() <= tol * 4
    tab = table.cpu().tolist()
    for t in range(T):
        page, off = tab[req[t]][positions[t] // ps], positions[t] % ps
        assert (kc[page, :, off].double().cpu() - kk[t]).abs().max() <= tol * 4
        assert torch.equal(vc[page, :, off].cpu(), qkv[t, (nh + nkv) * d:].view(nkv, dv))
    written = {(tab[req[t]][positions[t] // ps], positions[t] % ps) for t in range(T)}
    for page in range(pages):
        for off in range(ps):
            if (page, off) not in written:
                assert not kc[page, :, off].any() and not vc[page, :, off].any()


# ---------------------------------------------------------------------------------------------
# the attention kernel
# ---------------------------------------------------------------------------------------------
def _paged(seqs, nkv, d, dv, ps, dtype, seed):
    """Pages in a shuffled order for sequences of (k [n, G, d], v [n, G, dv]); returns caches and tables."""
    need = [(k.shape[0] + ps - 1) // ps for k, _ in seqs]
    total = sum(need) + 3
    order = torch.randperm(total, generator=torch.Generator().manual_seed(seed)).tolist()
    kc = torch.full((total, nkv, ps, d), float("nan"), dtype=dtype)
    vc = torch.full((total, nkv, ps, dv), float("nan"), dtype=dtype)
    stride = max(need) + 2
    table = torch.full((len(seqs), stride), -1, dtype=torch.int32)
    at = 0
    for b, (k, v) in enumerate(seqs):
        for p in range(need[b]):
            page = order[at]
            at += 1
            table[b, p] = page
            n = min(ps, k.shape[0] - p * ps)
            kc[page, :, :n] = k[p * ps:p * ps + n].transpose(0, 1).to(dtype)
            vc[page, :, :n] = v[p * ps:p * ps + n].transpose(0, 1).to(dtype)
    return kc.to(DEV), vc.to(DEV), table.to(DEV), stride


def _plain_attention(q, k, v, talk, scale, sink, window):
    """The oracle with the two switches the kernel has beyond the model (no sink, a window)."""
    n, H, d = q.shape
    rep = H // k.shape[1]
    kk, vv = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
    s = torch.einsum("ihd,jhd->hij", q, kk) * scale
    if talk is not None:
        s = torch.einsum("hg,gij->hij", talk, s)
    i, j = torch.arange(n)[:, None], torch.arange(n)[None, :]
    seen = (j <= i) & ((j > i - window) if window else True)
    s = s.masked_fill(~seen[None], float("-inf"))
    m = s.max(dim=-1, keepdim=True).values
    m = torch.clamp(m, min=0.0) if sink else m
    e = torch.exp(s - m)
    p = e / ((torch.exp(-m) if sink else 0.0) + e.sum(dim=-1, keepdim=True))
    return torch.einsum("hij,jhd->ihd", p, vv)


def _attend(seqs, starts, talk, scale, sink, window, ps, dtype, bq=None, parts=1, out_scale=1.0, seed=0, mma=False):
    """seqs: (q, k, v) whole sequences; entry b brings the tokens from starts[b] on.  Returns per-entry outputs."""
    k_ = _k()
    H, d = seqs[0][0].shape[1:]
    G, dv = seqs[0][2].shape[1:]
    kc, vc, table, stride = _paged([(k, v) for _, k, v in seqs], G, d, dv, ps, dtype, seed)
    counts = [q.shape[0] - s for (q, _, _), s in zip(seqs, starts)]
    T = sum(counts)
    qs = torch.cat([q[s:] for (q, _, _), s in zip(seqs, starts)]).to(dtype).to(DEV).contiguous()
    q_start = _i32(np.concatenate([[0], np.cumsum(counts)]).tolist())
    pad = 6 if mma else 5                                         # the output sits inside a wider buffer
    buf = torch.zeros(T, H * dv + pad, dtype=dtype, device=DEV)
    out = buf[:, 2:2 + H * dv]
    if bq is None:
        bq = k_.attn_talking_mma_tile(H, G, d, dv, max(counts)) if mma else k_.attn_talking_tile(H, d, dv, max(counts))
        assert bq > 0
    po = pml = None
    if parts > 1:
        po = torch.zeros(T * parts * H * dv, dtype=torch.float32, device=DEV)
        pml = torch.zeros(T * parts * H * 2, dtype=torch.float32, device=DEV)
    err = _err()
    (k_.attn_talking_mma if mma else k_.attn_talking)(out, qs, kc, vc, talk.float().to(DEV) if talk is not None else None, q_start, _i32(starts), len(seqs),
                    table, stride, window, scale, sink, out_scale, bq, err, parts, po, pml)
    assert int(err.item()) == 0
    assert not buf[:, :2].any() and not buf[:, 2 + H * dv:].any()
    res = out.double().cpu().view(T, H, dv)
    return [res[a:b] for a, b in zip(q_start.tolist()[:-1], q_start.tolist()[1:])]


def _random_qkv(n, H, G, d, dv, seed, sharp=1.0):
    g = torch.Generator().manual_seed(seed)
    q = plain.unit_rms(torch.randn(n, H, d, generator=g, dtype=torch.float64), 1e-6) * sharp
    k = plain.unit_rms(torch.randn(n, G, d, generator=g, dtype=torch.float64), 1e-6)
    v = torch.randn(n, G, dv, generator=g, dtype=torch.float64)
    return q, k, v


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,d,dv", [(4, 2, 16, 24), (6, 6, 24, 8), (2, 1, 32, 16), (5, 1, 8, 40), (16, 4, 64, 64)])
@pytest.mark.parametrize("sink,talks,window", [(True, True, None), (False, True, None), (True, False, 19), (False, False, None)])
def test_attention_equals_plain_for_unequal_entries(dtype, H, G, d, dv, sink, talks, window):
    ps, scale = 8, 1.7 / math.sqrt(d)
    g = torch.Generator().manual_seed(H + d)
    talk = (torch.randn(H, H, generator=g, dtype=torch.float64) * 0.8 + torch.eye(H)) if talks else None
    # a whole prompt, a long continuation, a portion of two tokens, single decoded tokens at several places
    plan = [(70, 0), (131, 90), (45, 43), (33, 32), (64, 63), (17, 16), (1, 0)]
    seqs = [_random_qkv(n, H, G, d, dv, 10 * i + H) for i, (n, _) in enumerate(plan)]
    if dtype == torch.bfloat16:   # the kernel reads rounded operands: give the oracle the same
        seqs = [tuple(t.to(torch.bfloat16).double() for t in s) for s in seqs]
    starts = [s for _, s in plan]
    got = _attend(seqs, starts, talk, scale, sink, window, ps, dtype)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    for (q, k, v), s, o in zip(seqs, starts, got):
        ref = _plain_attention(q, k, v, talk, scale, sink, window)[s:]
        assert (o - ref).abs().max() <= tol, (q.shape[0], s, float((o - ref).abs().max()))


@pytest.mark.parametrize("H,G,d,dv", [(2, 1, 32, 16), (16, 4, 64, 64), (6, 2, 96, 64), (32, 8, 128, 128), (8, 8, 16, 16),
                                      (12, 4, 48, 80), (3, 1, 32, 128), (64, 8, 64, 32), (10, 5, 16, 48)])
@pytest.mark.parametrize("sink,talks,window", [(True, True, None), (False, True, 40), (True, False, None)])
def test_tensor_core_attention_equals_plain(H, G, d, dv, sink, talks, window):
    """The bfloat16 form whose two products run on tensor cores: whole prompts, continuations, a portion of two
    tokens, single tokens (also cut into key ranges), against the plain implementation on the rounded operands."""
    ps, scale = 16, 1.7 / math.sqrt(d)
    g = torch.Generator().manual_seed(H * 7 + d)
    talk = (torch.randn(H, H, generator=g, dtype=torch.float64) * (0.8 / math.sqrt(H)) + torch.eye(H)) if talks else None
    plan = [(70, 0), (131, 90), (45, 43), (33, 32), (64, 63), (17, 16), (1, 0), (300, 281)]
    seqs = [tuple(t.to(torch.bfloat16).double() for t in _random_qkv(n, H, G, d, dv, 10 * i + H)) for i, (n, _) in enumerate(plan)]
    starts = [s for _, s in plan]
    got = _attend(seqs, starts, talk, scale, sink, window, ps, torch.bfloat16, mma=True)
    for (q, k, v), s, o in zip(seqs, starts, got):
        ref = _plain_attention(q, k, v, talk, scale, sink, window)[s:]
        assert (o - ref).abs().max() <= 2e-2, (q.shape[0], s, float((o - ref).abs().max()))
    # single tokens, keys in ranges
    singles = [(q, k, v) for (q, k, v) in seqs]
    for parts in (1, 3):
        got = _attend(singles, [q.shape[0] - 1 for q, _, _ in singles], talk, scale, sink, window, ps, torch.bfloat16, bq=1,
                      parts=parts, out_scale=0.75, mma=True)
        for (q, k, v), o in zip(singles, got):
            ref = 0.75 * _plain_attention(q, k, v, talk, scale, sink, window)[-1:]
            assert (o - ref).abs().max() <= 2e-2


@pytest.mark.parametrize("where", ["first", "page_end", "page_start", "far", "self"])
def test_tensor_core_attention_finds_a_planted_key(where):
    H, G, d, dv, ps, n = 4, 2, 16, 16, 16, 600
    j = {"first": 0, "page_end": 31, "page_start": 32, "far": n - 517, "self": n - 1}[where]
    q, k, v = (t.to(torch.bfloat16).double() for t in _random_qkv(n, H, G, d, dv, 99))
    for h in range(H):
        q[-1, h] = k[j, h // (H // G)] * 3.0
    for start, parts in ((n - 37, 1), (n - 1, 1), (n - 1, 4)):
        got = _attend([(q, k, v)], [start], None, 1.0, True, None, ps, torch.bfloat16, parts=parts,
                      bq=1 if start == n - 1 else None, mma=True)[0]
        want = v[j].repeat_interleave(H // G, dim=0)
        assert (got[-1] - want).abs().max() < 2e-2 * (1 + want.abs().max()), "the planted key must carry the output"


@pytest.mark.parametrize("parts", [1, 2, 5, 16])
def test_decode_in_key_ranges_equals_plain(parts):
    H, G, d, dv, ps = 6, 2, 32, 24, 16
    scale = 2.0 / math.sqrt(d)
    talk = torch.randn(H, H, generator=torch.Generator().manual_seed(1), dtype=torch.float64)
    lens = [700, 1, 33, 257, 64]
    seqs = [_random_qkv(n, H, G, d, dv, 7 + n) for n in lens]
    got = _attend(seqs, [n - 1 for n in lens], talk, scale, True, None, ps, torch.float32, bq=1, parts=parts, out_scale=1.25)
    for (q, k, v), o in zip(seqs, got):
        ref = 1.25 * plain.talking_sink_attention(q, k, v, talk, scale)[-1:]
        assert (o - ref).abs().max() <= 2e-5


@pytest.mark.parametrize("where", ["first", "second", "page_end", "page_start", "far", "previous", "self"])
@pytest.mark.parametrize("decode", [False, True])
def test_one_planted_key_decides_the_output(where, decode):
    """Among hundreds of keys one is made to stand out for the last query (its score is far above the
    others'), so the output is that key's value: a kernel that skips it, or reads a neighbour, is far off."""
    H, G, d, dv, ps, n = 4, 2, 16, 8, 16, 600
    j = {"first": 0, "second": 1, "page_end": 31, "page_start": 32, "far": n - 517, "previous": n - 2, "self": n - 1}[where]
    q, k, v = _random_qkv(n, H, G, d, dv, 99)
    q[-1] = q[-1] * 0.05
    for h in range(H):                      # every head's last query points at key j of its kv head
        q[-1, h] = k[j, h // (H // G)] * 3.0
    scale = 1.0
    start = n - 1 if decode else n - 37
    got = _attend([(q, k, v)], [start], None, scale, True, None, ps, torch.float32, parts=4 if decode else 1,
                  bq=1 if decode else None)[0]
    ref = plain.talking_sink_attention(q, k, v, torch.eye(H, dtype=torch.float64), scale)[start:]
    assert (got - ref).abs().max() <= 2e-5
    want = v[j].repeat_interleave(H // G, dim=0)
    assert (got[-1] - want).abs().max() < 1e-3 * want.abs().max() + 1e-3, "the planted key must carry the output"


@pytest.mark.parametrize("decode", [False, True])
def test_window_edges(decode):
    """A key just inside the window decides the output, the same key just outside must not be seen."""
    H, G, d, dv, ps, n, window = 2, 1, 16, 8, 8, 200, 48
    for j, inside in [(n - window, True), (n - window - 1, False), (n - 1, True)]:
        q, k, v = _random_qkv(n, H, G, d, dv, 5)
        for h in range(H):
            q[-1, h] = k[j, 0] * 3.0
        start = n - 1 if decode else n - 9
        got = _attend([(q, k, v)], [start], None, 1.0, True, window, ps, torch.float32, bq=1 if decode else None)[0]
        ref = _plain_attention(q, k, v, None, 1.0, True, window)[start:]
        assert (got - ref).abs().max() <= 2e-5
        carried = (got[-1] - v[j].repeat_interleave(H, dim=0)).abs().max() < 1e-2
        assert bool(carried) == inside


def test_a_sink_lets_a_query_attend_to_nothing():
    H, G, d, dv = 2, 2, 8, 8
    q, k, v = _random_qkv(5, H, G, d, dv, 1)
    q = -k.clone() * 4.0          # every score is strongly negative: the weights all but vanish
    with_sink = _attend([(q, k, v)], [0], None, 1.0, True, None, 8, torch.float32)[0]
    without = _attend([(q, k, v)], [0], None, 1.0, False, None, 8, torch.float32)[0]
    assert with_sink[0].abs().max() < 1e-4 * without[0].abs().max()
    assert (without[0] - v[0]).abs().max() < 1e-5       # the first token sees itself alone: weight one


# ---------------------------------------------------------------------------------------------
# the recurrence
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("chunked", [False, True])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_scan_equals_plain_and_carries_state(chunked, out_dtype):
    k = _k()
    g = torch.Generator().manual_seed(8)
    W, hid, slots = 72, 40, 6
    w = {"z": torch.randn(W, hid, generator=g).double(), "z.b": torch.randn(W, generator=g).double(),
         "x": torch.randn(W, hid, generator=g).double() * 2, "x.b": torch.randn(W, generator=g).double(),
         "g": torch.randn(W, hid, generator=g).double(), "o": torch.eye(W).double()}
    lens = [150, 3, 1, 67]
    hs = [torch.randn(n, hid, generator=g).double() * 0.7 for n in lens]
    refs = [plain.mingru_branch(h, w, "")[1] * torch.nn.functional.silu(h @ w["g"].T) for h in hs]
    state = torch.full((slots, W), float("nan"), device=DEV)
    use = [4, 0, 5, 2]
    for s in use:
        state[s].zero_()
    done = [0] * len(lens)
    # three steps with unequal portions (a chunk border inside a portion, an entry that sits one step out)
    for portions in ([70, 2, 1, 64], [79, 0, 0, 2], [1, 1, 0, 1]):
        ent = [i for i, c in enumerate(portions) if c]
        rows = torch.cat([hs[i][done[i]:done[i] + portions[i]] for i in ent])
        T = rows.shape[0]
        zxg = torch.cat([rows @ w["z"].T, rows @ w["x"].T, rows @ w["g"].T], dim=1).float().to(DEV).contiguous()
        cnt = [portions[i] for i in ent]
        q_start = _i32(np.concatenate([[0], np.cumsum(cnt)]).tolist() + [sum(cnt)])     # one padding entry
        slot_ids = _i32([use[i] for i in ent] + [-1])
        req = _i32([b for b, c in enumerate(cnt) for _ in range(c)])
        buf = torch.zeros(T, W + 3, dtype=out_dtype, device=DEV)
        scratch = torch.empty(3 * T * W, dtype=torch.float32, device=DEV) if chunked else None
        k.gated_scan(buf[:, 3:], zxg, w["z.b"].float().to(DEV), w["x.b"].float().to(DEV), state, q_start, slot_ids, req,
                     len(ent) + 1, 0.5, scratch)
        at = 0
        tol = 3e-5 if out_dtype == torch.float32 else 2e-2
        for i in ent:
            ref = 0.5 * refs[i][done[i]:done[i] + portions[i]]
            got = buf[at:at + portions[i], 3:].double().cpu()
            assert (got - ref).abs().max() <= tol * (1 + ref.abs().max()), (i, done[i])
            at += portions[i]
            done[i] += portions[i]
        assert not buf[:, :3].any()
    assert done == lens
    assert torch.isnan(state[1]).all() and torch.isnan(state[3]).all(), "slots of other requests are untouched"


def test_candidate_is_continuous_and_positive():
    u = torch.tensor([-30.0, -1e-7, 0.0, 1e-7, 4.0], dtype=torch.float64)
    c = plain.mingru_candidate(u)
    assert (c > 0).all() and abs(float(c[1] - c[2])) < 1e-6 and float(c[4]) == 4.5


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_polynorm_equals_plain(out_dtype):
    k = _k()
    g = torch.Generator().manual_seed(2)
    for F in (56, 300, 2050):
        z = torch.randn(9, F, generator=g) * 3
        coef = torch.tensor([0.7, -0.4, 0.25, 0.1])
        out = torch.empty(9, F, dtype=out_dtype, device=DEV)
        k.polynorm(out, z.to(DEV), coef.to(DEV), 1e-5)
        ref = plain.polynorm(z.double(), coef.double(), 1e-5)
        tol = 1e-5 if out_dtype == torch.float32 else 2 ** -7
        assert ((out.double().cpu() - ref).abs() <= tol * (ref.abs() + 1)).all()


# ---------------------------------------------------------------------------------------------
# experts by table
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype,tensor_cores,dense_up_to,library", [
    (torch.float32, False, 32, False), (torch.bfloat16, False, 0, False), (torch.bfloat16, True, 0, False),
    (torch.bfloat16, True, 32, False), (torch.bfloat16, True, 32, True), (torch.bfloat16, True, 0, True)])
@pytest.mark.parametrize("E,top,ff,hid,T", [(5, 2, 24, 48, 77), (8, 1, 40, 64, 3), (3, 3, 16, 32, 130), (16, 4, 72, 96, 1),
                                            (4, 2, 200, 136, 300), (2, 1, 60, 44, 9)])
def test_table_experts_equal_plain(dtype, tensor_cores, dense_up_to, library, E, top, ff, hid, T, monkeypatch):
    """The grouped form on FMA units and on tensor cores, the dense form that steps of few tokens take, and the
    form that gives each expert's rows to the library's product when the host knows the ids."""
    from xinfer_b200.config.plan import ExpertTableSpec
    from xinfer_b200.parts import table_experts
    monkeypatch.setattr(_k(), "expert_tensor_cores", tensor_cores)
    monkeypatch.setattr(table_experts, "DENSE_MAX_TOKENS", dense_up_to)
    monkeypatch.setattr(table_experts, "PER_EXPERT_LIBRARY_PRODUCTS", library)
    monkeypatch.setattr(table_experts, "LIBRARY_FROM_FLOP_PER_CALL", 0.0)     # the test's sizes are tiny
    from xinfer_b200.parts import StepContext, Workspace, build_part
    vocab = 41
    g = torch.Generator().manual_seed(E * 10 + top)
    w = {}
    for e in range(E):
        w[f"m.e{e}.gate"] = torch.randn(ff, hid, generator=g) * 0.3
        w[f"m.e{e}.up"] = torch.randn(ff, hid, generator=g) * 0.3
        w[f"m.e{e}.down"] = torch.randn(hid, ff, generator=g) * 0.3
    w["m.table"] = torch.rand(vocab, E, generator=g).argsort(dim=1)[:, :top].to(torch.int32)
    if dtype == torch.bfloat16:
        w = {n: (t.to(dtype).float() if t.is_floating_point() else t) for n, t in w.items()}

    class Store:
        def get(self, name, device, dt, operand=False):
            t = w[name]
            return t.to(device) if not t.is_floating_point() else t.to(device).to(dt if operand else torch.float32)

    part = build_part("feed_forward", ExpertTableSpec(kind="table_experts", hidden=hid, intermediate=ff, experts=E, top=top,
                                                       vocab=vocab), "m.", dtype, DEV)
    part.load(Store())
    ids = torch.randint(0, vocab, (T,), generator=g)
    ids_dev = ids.to(torch.int32)
    sampled = _i32([int(ids[0]), 5])
    if not library:
        ids_dev[0] = -1                               # the first token's id waits on the device
    x = (torch.randn(T, hid, generator=g)).to(dtype)
    pad = 2                                           # two padding rows at the end
    xd = torch.cat([x, torch.zeros(pad, hid, dtype=dtype)]).to(DEV)
    req = _i32([0] * T + [-1] * pad)
    tok = torch.cat([ids_dev, torch.zeros(pad, dtype=torch.int32)]).to(DEV)
    err = _err()
    ctx = StepContext(dtype=dtype, device=torch.device(DEV), num_tokens=T + pad, num_entries=1, token_ids=tok,
                      positions=tok, req_of_token=req, q_start=_i32([0, T]), start_pos=_i32([0]), slots=_i32([0]),
                      logit_rows=_i32([0]), num_logit_rows=1, tables=[], strides=[], err=err, workspace=Workspace(DEV),
                      sampled=sampled, branch_dtype=torch.float32, real_tokens=T + pad,
                      h_token_ids=np.concatenate([ids_dev.numpy(), np.zeros(pad, dtype=np.int32)]))
    if library:     # the library form wants a step without padding rows
        xd, req, tok = xd[:T].contiguous(), req[:T].contiguous(), tok[:T].contiguous()
        ctx = StepContext(dtype=dtype, device=torch.device(DEV), num_tokens=T, num_entries=1, token_ids=tok, positions=tok,
                          req_of_token=req, q_start=_i32([0, T]), start_pos=_i32([0]), slots=_i32([0]), logit_rows=_i32([0]),
                          num_logit_rows=1, tables=[], strides=[], err=err, workspace=Workspace(DEV), sampled=sampled,
                          branch_dtype=torch.float32, real_tokens=T, h_token_ids=ids_dev.numpy())
    out = part.forward(xd, ctx)
    assert int(err.item()) == 0 and out.dtype == torch.float32
    ref = plain.table_moe(x.double(), ids, {n: t.double() if t.is_floating_point() else t for n, t in w.items()}, "m.")
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    assert (out[:T].double().cpu() - ref).abs().max() <= tol * (1 + ref.abs().max())
    assert not out[T:].any()
    # a token's result does not depend on its company: run three tokens alone
    for t in (0, T // 2, T - 1):
        ctx1 = StepContext(dtype=dtype, device=torch.device(DEV), num_tokens=1, num_entries=1,
                           token_ids=_i32([int(ids[t])]), positions=_i32([0]), req_of_token=_i32([0]), q_start=_i32([0, 1]),
                           start_pos=_i32([0]), slots=_i32([0]), logit_rows=_i32([0]), num_logit_rows=1, tables=[],
                           strides=[], err=err, workspace=Workspace(DEV), branch_dtype=torch.float32)
        alone = part.forward(xd[t:t + 1].contiguous(), ctx1).clone()
        if dtype == torch.float32 or (not library and (dense_up_to == 0 or T <= dense_up_to)):
            assert torch.equal(alone[0], out[t])        # the same form took both: a row's sum has one order
        else:                                           # one token takes the dense form, the batch the grouped one
            assert (alone[0].double().cpu() - ref[t]).abs().max() <= tol * (1 + ref.abs().max())


# ---------------------------------------------------------------------------------------------
# whole models
# ---------------------------------------------------------------------------------------------
# one prompt of T2 is long enough for the recurrence's chunked form and for several attention query tiles
LENGTHS = {"T1": [70, 45, 130, 33], "T2": [97, 41, 300, 150], "T3": [120, 1, 75, 58], "T4": [90, 2, 51, 140]}


def _tolerance(dtype, ref, cfg=None, w=None, p=None):
    """float32: a small share of the logits' spread (the engine's float32 against float64).  bfloat16: three
    times what rounding alone causes - the largest row error of the plain run that rounds activations to
    bfloat16 where an engine stores them."""
    spread = max(float(np.std(ref)), 1e-3)
    if dtype == "float32":
        return 3e-5 * spread
    rounded = plain.forward(cfg, w, p, round_to=torch.bfloat16).numpy()
    return max(3.0 * max(_row_error(rounded[i], ref[i]) for i in range(len(p))), 1e-3 * spread)


def _row_error(got, want):
    """Root mean square over the vocabulary of the difference, its mean taken off."""
    d = got.astype(np.float64) - want
    d = d - d.mean()
    return float(np.sqrt((d * d).mean()))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["T1", "T2", "T3", "T4"])
def test_every_way_of_cutting_gives_the_plain_logits(name, dtype, tmp_path):
    folder = make_folder(str(tmp_path / "model"), name, torch.float32 if dtype == "float32" else torch.bfloat16)
    ps = prompts(name, LENGTHS[name])
    tb = build_all_modes(ps, seed=len(name))
    out = run_trace(folder, dtype, tb.steps, str(tmp_path / "out"), max_tokens=tb.peak, page_size=TINY_T[name][2],
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


@pytest.mark.parametrize("name,dtype", [("T1", "float32"), ("T2", "bfloat16")])
def test_freed_pages_and_slots_are_used_again_and_nothing_stale_is_read(name, dtype, tmp_path):
    """Pages that go back to the pool are filled with NaN before the next step, and a state slot that a
    request leaves is taken by the next one: the logits stay the plain ones."""
    from xinfer_b200.engine.runner import ModelRunner
    folder = make_folder(str(tmp_path / "model"), name, torch.float32 if dtype == "float32" else torch.bfloat16)
    ps = prompts(name, LENGTHS[name])
    tb = build_all_modes(ps, seed=3)
    page = TINY_T[name][2]
    runner = ModelRunner(folder, dtype, block_size=page, num_blocks=(tb.peak + page - 1) // page, max_num_seqs=4,
                         poison_freed_pages=True)
    # what a request leaves in its state slot must not reach the next one: fill every slot with junk first
    for t in runner.state.tables.values():
        t.fill_(1e6)
    out = replay_in_process(runner, tb.steps)
    assert runner.pages_poisoned > runner.num_blocks
    cfg, w = plain.load_folder(folder)
    ref = [plain.forward(cfg, w, p).numpy() for p in ps]
    tol = [_tolerance(dtype, r, cfg, w, p) for r, p in zip(ref, ps)]
    for step, rows in tb.rows.items():
        assert np.isfinite(out[step]).all(), f"step {step} read a poisoned page"
        for r, ((mode, i), pos) in enumerate(rows):
            assert _row_error(out[step][r], ref[i][pos]) <= tol[i], (mode, i, pos)


def test_layers_one_by_one_in_float32(tmp_path):
    """The residual stream after every layer (with its waiting additions) against the plain one."""
    from xinfer_b200.engine.runner import ModelRunner, StepInput
    from xinfer_b200.parts.block import Block
    folder = make_folder(str(tmp_path / "model"), "T1", torch.float32)
    cfg, w = plain.load_folder(folder)
    p = prompts("T1", [29])[0]
    want = []
    plain.forward(cfg, w, p, layers_out=want)
    rec, orig = [], Block.forward

    def spy(self, stream, ctx, cache, state, writes_cache):
        out = orig(self, stream, ctx, cache, state, writes_cache)
        x = out.x.double().clone()
        for b in out.pending:
            x += b.scale * b.plain(ctx).double()
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


# ---------------------------------------------------------------------------------------------
# generation through the entry point and the scheduler
# ---------------------------------------------------------------------------------------------
def _engine(folder, dtype, page, **kw):
    from xinfer_b200 import Engine, EngineConfig
    opts = dict(weight_path=folder, block_size=page, num_blocks=96, max_num_seqs=4, max_num_batched_tokens=64,
                prefill_chunk_size=16, disable_cuda_graph=True, max_model_len=1024)
    opts.update(kw)
    return Engine(EngineConfig(**opts), dtype)


def test_greedy_generation_in_float32_equals_plain(tmp_path):
    from xinfer_b200 import SamplingParams
    folder = make_folder(str(tmp_path / "model"), "T1", torch.float32)
    cfg, w = plain.load_folder(folder)
    ps = prompts("T1", [1, 5, 23, 40, 9, 17])       # six requests over four slots, prompts in portions of 16
    eng = _engine(folder, "f32", TINY_T["T1"][2])
    outs = eng.generate_sync(SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True), ps)
    for p, o in zip(ps, outs):
        assert o.decode_output == plain.generate(cfg, w, p, 12)


@pytest.mark.parametrize("graphs", [False, True], ids=["launched", "cuda_graph"])
def test_long_greedy_decoding_in_bfloat16_follows_the_plain_logits(graphs, tmp_path):
    """Each generated token is checked against the plain logits of the sequence the engine produced (bfloat16
    may flip a near-tie): it must be the best token up to the drift.  Long enough for several pages per
    request and for every decode kernel's key ranges; launched kernel by kernel and replayed from graphs."""
    from xinfer_b200 import SamplingParams
    folder = make_folder(str(tmp_path / "model"), "T2", torch.bfloat16)
    cfg, w = plain.load_folder(folder)
    ps = prompts("T2", [3, 30, 61])
    eng = _engine(folder, "bf16", TINY_T["T2"][2], disable_cuda_graph=not graphs)
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
