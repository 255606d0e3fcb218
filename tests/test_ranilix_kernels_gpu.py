"""Each Ranilix mechanism alone: the CUDA kernel against the plain fp32 functions of oracle/ranilix_oracle.py, in both
storage formats (bf16 serving, fp32 exact)."""
import importlib
import math

import pytest
import torch

from oracle import ranilix_oracle as R

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTS = [torch.float32, torch.bfloat16]


@pytest.fixture(scope="module")
def ops():
    return importlib.import_module("nano-vllm-candle_b200.ops")


def tol(dt):
    return dict(rtol=2e-5, atol=2e-5) if dt == torch.float32 else dict(rtol=2e-2, atol=2e-2)


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


def test_embedding_rows_times_a_constant(ctx, ops):
    g = torch.Generator().manual_seed(1)
    for dt in DTS:
        table = torch.randn(41, 56, generator=g).to(dt).to(DEV)
        ids = i32([0, 40, 7, 7, 19])
        out = ops.embed_gather_scaled_f32(ctx, ids, table, 2.75)
        assert torch.equal(out.cpu(), table.float().cpu()[ids.cpu().long()] * 2.75)


@pytest.mark.parametrize("dt", DTS)
@pytest.mark.parametrize("H", [24, 200, 1100])
def test_two_norms_of_one_residual_sum(ctx, ops, dt, H):
    g = torch.Generator().manual_seed(2)
    N, eps = 7, 1e-3
    res, a0, a1 = (torch.randn(N, H, generator=g) * 3 for _ in range(3))
    w0, w1 = 1 + 0.2 * torch.randn(H, generator=g), 1 + 0.2 * torch.randn(H, generator=g)
    d = [t.to(DEV) for t in (res, a0, a1, w0, w1)]
    s = res + a0 + a1
    ro, o0, o1 = ops.rms_norm_pair(ctx, d[0], d[1:3], d[3], d[4], eps=eps, out_dtype=dt)
    assert torch.allclose(ro.cpu(), s, rtol=1e-6, atol=1e-6)
    assert torch.allclose(o0.float().cpu(), R.rms_norm(s, w0, eps), **tol(dt))
    assert torch.allclose(o1.float().cpu(), R.rms_norm(s, w1, eps), **tol(dt))
    # one norm, one addend, gathered rows: nothing is written back
    rows = i32([6, 0, 3])
    before = d[0].clone()
    ro2, o2, none = ops.rms_norm_pair(ctx, d[0], [d[1]], d[3], None, eps=eps, out_dtype=dt, rows=rows)
    assert ro2 is None and none is None and torch.equal(before, d[0])
    assert torch.allclose(o2.float().cpu(), R.rms_norm(res + a0, w0, eps)[rows.cpu().long()], **tol(dt))
    # accumulation alone
    ro3, _, _ = ops.rms_norm_pair(ctx, d[0], d[1:3], None, None)
    assert torch.allclose(ro3.cpu(), s, rtol=1e-6, atol=1e-6)


def test_the_norm_keeps_eps_inside_the_root(ctx, ops):
    """A row of tiny numbers: x / sqrt(mean(x^2) + eps) is about x / sqrt(eps), far from x / rms(x)."""
    x = torch.full((2, 48), 1e-4)
    w = torch.ones(48)
    _, o, _ = ops.rms_norm_pair(ctx, x.to(DEV), [], w.to(DEV), None, eps=1e-2, write_back=False)
    assert torch.allclose(o.cpu(), x / math.sqrt(1e-8 + 1e-2), rtol=1e-5, atol=0)


@pytest.mark.parametrize("dt", DTS)
@pytest.mark.parametrize("norm,act", [(True, "silu"), (False, "sigmoid"), (True, "sigmoid")])
def test_head_output_stage(ctx, ops, dt, norm, act):
    g = torch.Generator().manual_seed(3)
    N, H, vd, eps = 11, 3, 40, 1e-4
    o, z = torch.randn(N, H * vd, generator=g) * 5, torch.randn(N, H * vd + 8, generator=g) * 2
    y = R.rms_norm(o.view(N, H, vd), None, eps).reshape(N, H * vd) if norm else o
    zz = z[:, 8:]
    want = y * (zz * torch.sigmoid(zz) if act == "silu" else torch.sigmoid(zz)) * 0.6
    got = ops.head_gate(ctx, o.to(DEV), z.to(DEV)[:, 8:], H, vd, norm, eps, act, 0.6, out_dtype=dt)
    assert torch.allclose(got.float().cpu(), want, **tol(dt))


# ---------------------------------------------------------------------------------------------------------------- q / k / v preparation
@pytest.mark.parametrize("dt", DTS)
@pytest.mark.parametrize("H,G,d,vd,rot,half,normed", [(4, 2, 32, 24, 16, False, True), (3, 3, 40, 40, 40, False, False),
                                                     (2, 1, 16, 72, 0, False, True), (3, 3, 24, 8, 24, True, False),
                                                     (5, 5, 48, 16, 20, True, False)])
def test_bias_norm_rotation_and_cache_store(ctx, ops, dt, H, G, d, vd, rot, half, normed):
    g = torch.Generator().manual_seed(4)
    N, eps, base, slots = 13, 1e-5, 5000.0, 40
    qw, kw, vw = H * d, G * d, G * vd
    ld = qw + kw + vw + 16
    x = torch.randn(N, ld, generator=g)
    bias = torch.randn(ld, generator=g) * 0.3 if normed else None
    qn, kn = (1 + 0.3 * torch.randn(d, generator=g), 1 + 0.3 * torch.randn(d, generator=g)) if normed else (None, None)
    pos = torch.tensor([0, 1, 2, 3, 100, 101, 7, 8, 9, 511, 0, 1, 2])
    slot = torch.tensor([5, 6, 7, 39, 0, 1, 20, -1, 22, 23, 30, 31, 32])
    xb = x + (bias if bias is not None else 0)
    q = xb[:, :qw].view(N, H, d)
    k = xb[:, qw:qw + kw].view(N, G, d)
    v = xb[:, qw + kw:qw + kw + vw]
    if normed:
        q, k = R.rms_norm(q, qn, eps), R.rms_norm(k, kn, eps)
    rf = R.rotary_half if half else R.rotary_interleaved
    q, k = rf(q, pos, rot, base), rf(k, pos, rot, base) * 0.5
    table = ops.rotary_table(ctx, base, rot, 512) if rot else None
    q_out = torch.zeros(N, qw, dtype=dt, device=DEV)
    kc = torch.full((slots, kw), 9.0, dtype=dt, device=DEV)
    vc = torch.full((slots, vw), 9.0, dtype=dt, device=DEV)
    dv = lambda t: None if t is None else t.to(DEV)
    ops.qkv_prep(ctx, x.to(DEV), 0, qw, qw + kw, H, G, d, vd, q_out, kc, vc, bias=dv(bias), q_norm=dv(qn), k_norm=dv(kn), eps=eps,
                 rot_dims=rot, rot_half=half, rot_table=table, positions=i32(pos.tolist()), k_scale=0.5, slot_mapping=i32(slot.tolist()))
    assert torch.allclose(q_out.float().cpu(), q.reshape(N, qw), **tol(dt))
    ok = slot >= 0
    assert torch.allclose(kc.float().cpu()[slot[ok]], k.reshape(N, kw)[ok], **tol(dt))
    assert torch.allclose(vc.float().cpu()[slot[ok]], v[ok], **tol(dt))
    untouched = torch.ones(slots, dtype=torch.bool)
    untouched[slot[ok]] = False
    assert (kc.float().cpu()[untouched] == 9.0).all() and (vc.float().cpu()[untouched] == 9.0).all()


@pytest.mark.parametrize("dt", DTS)
def test_value_blending_provider_and_user(ctx, ops, dt):
    g = torch.Generator().manual_seed(5)
    N, H, G, d, vd = 9, 2, 2, 8, 24
    ld = H * d + G * d + G * vd
    x1, x2 = torch.randn(N, ld, generator=g), torch.randn(N, ld, generator=g)
    b1 = torch.randn(ld, generator=g)
    lam = torch.tensor([0.3])
    vf = torch.zeros(N, G * vd, device=DEV)
    outs = [torch.zeros(N, w, dtype=dt, device=DEV) for w in (H * d, G * d, G * vd)]
    ops.qkv_prep(ctx, x1.to(DEV), 0, H * d, H * d + G * d, H, G, d, vd, *outs, bias=b1.to(DEV), blend=1, v_first=vf)
    v1 = (x1 + b1)[:, -G * vd:]
    assert torch.allclose(vf.cpu(), v1, rtol=1e-6, atol=1e-6)            # the provider's own values, unblended, in fp32
    assert torch.allclose(outs[2].float().cpu(), v1, **tol(dt))
    ops.qkv_prep(ctx, x2.to(DEV), 0, H * d, H * d + G * d, H, G, d, vd, *outs, blend=2, lam=lam.to(DEV), v_first=vf)
    assert torch.allclose(outs[2].float().cpu(), 0.7 * x2[:, -G * vd:] + 0.3 * v1, **tol(dt))
    ops.qkv_prep(ctx, x2.to(DEV), 0, H * d, H * d + G * d, H, G, d, vd, *outs, blend=2, lam=lam.to(DEV), v_first=vf, v_scale=1.5)
    assert torch.allclose(outs[2].float().cpu(), 1.5 * (0.7 * x2[:, -G * vd:] + 0.3 * v1), **tol(dt))      # the factor comes last
    assert torch.allclose(vf.cpu(), v1, rtol=1e-6, atol=1e-6)            # a user does not change what the provider left


def test_rotation_angles_stay_exact_far_from_the_start(ctx, ops):
    tab = ops.rotary_table(ctx, 1e6, 64, 40000).cpu()
    for p in (1, 4097, 39999):
        a = R.rotary_angles(torch.tensor([p]), 64, 1e6)[0]
        assert torch.allclose(tab[p, :, 0].double(), a.cos(), atol=1e-7) and torch.allclose(tab[p, :, 1].double(), a.sin(), atol=1e-7)


# ---------------------------------------------------------------------------------------------------------------- attention
def paged(k, v, bs, nblocks, g):
    """Scatters per-sequence k / v rows [T, kw] into pools through a shuffled block table; returns (kc, vc, table rows)."""
    order = torch.randperm(nblocks, generator=g).tolist()
    kc = torch.zeros(nblocks * bs, k[0].shape[1])
    vc = torch.zeros(nblocks * bs, v[0].shape[1])
    tables, at = [], 0
    for kk, vv in zip(k, v):
        nb = (kk.shape[0] + bs - 1) // bs
        bl = order[at:at + nb]
        at += nb
        for j in range(kk.shape[0]):
            kc[bl[j // bs] * bs + j % bs] = kk[j]
            vc[bl[j // bs] * bs + j % bs] = vv[j]
        tables.append(bl)
    width = max(len(t) for t in tables)
    return kc, vc, [t + [-1] * (width - len(t)) for t in tables]


def run_attention(ctx, ops, dt, H, G, d, vd, lens, qlens, bs, window, sink, gate, scale, seed=0, boost=None):
    """Sequences of lens[b] tokens whose last qlens[b] are queried.  boost = (b, query row, key position, factor) makes one
    score stand out.  Returns (got, want)."""
    g = torch.Generator().manual_seed(seed)
    ks = [torch.randn(n, G, d, generator=g) for n in lens]
    vs = [torch.randn(n, G, vd, generator=g) for n in lens]
    qs = [torch.randn(m, H, d, generator=g) for m in qlens]
    if boost:
        b, i, j, f = boost
        qs[b][i, :] = qs[b][i, 0]          # every head of the row asks the same question, every key head answers it
        ks[b][j, :] = qs[b][i, 0] * f / (qs[b][i, 0] @ qs[b][i, 0])
    if dt == torch.bfloat16:
        ks, vs, qs = ([t.bfloat16().float() for t in x] for x in (ks, vs, qs))
    sk = torch.randn(H, generator=g) * 2 if sink else None
    rows = sum(qlens)
    gt = torch.randn(rows, H * vd + 4, generator=g) if gate else None
    want, r0 = [], 0
    for b, (n, m) in enumerate(zip(lens, qlens)):
        o = R.softmax_attention(qs[b], ks[b], vs[b], scale, torch.arange(n - m, n), window or None, sk)
        if gate:
            o = o * torch.sigmoid(gt[r0:r0 + m, 4:])
        want.append(o * 1.25)
        r0 += m
    nblocks = sum((n + bs - 1) // bs for n in lens) + 3
    kc, vc, tables = paged([k.reshape(k.shape[0], -1) for k in ks], [v.reshape(v.shape[0], -1) for v in vs], bs, nblocks, g)
    cu = [0]
    for m in qlens:
        cu.append(cu[-1] + m)
    decode = all(m == 1 for m in qlens)
    got = ops.attn_paged_wide(ctx, torch.cat(qs).reshape(rows, H * d).to(dt).to(DEV), kc.to(dt).to(DEV), vc.to(dt).to(DEV), i32(tables), i32(lens),
                              None if decode else i32(cu), max(qlens), bs, H, G, d, vd, scale, window, None if sk is None else sk.to(DEV),
                              None if gt is None else gt.to(DEV)[:, 4:], 1.25)
    return got.float().cpu(), torch.cat(want)


SHAPES = [(4, 2, 32, 48), (3, 3, 40, 24), (6, 1, 16, 80), (2, 2, 64, 128), (8, 4, 128, 64)]


@pytest.mark.parametrize("dt", DTS)
@pytest.mark.parametrize("H,G,d,vd", SHAPES)
@pytest.mark.parametrize("window", [0, 13])
def test_attention_over_a_mixed_batch(ctx, ops, dt, H, G, d, vd, window):
    got, want = run_attention(ctx, ops, dt, H, G, d, vd, lens=[70, 1, 33, 129, 16], qlens=[70, 1, 2, 40, 1], bs=16, window=window,
                              sink=window > 0, gate=window > 0, scale=0.2, seed=H)
    assert torch.allclose(got, want, **tol(dt))


@pytest.mark.parametrize("dt", DTS)
@pytest.mark.parametrize("bs", [16, 64])
def test_attention_decode_rows_without_cu_seqlens(ctx, ops, dt, bs):
    got, want = run_attention(ctx, ops, dt, 4, 2, 32, 48, lens=[300, 1, 64, 65, 17], qlens=[1] * 5, bs=bs, window=0, sink=False, gate=False,
                              scale=0.15, seed=9)
    assert torch.allclose(got, want, **tol(dt))


@pytest.mark.parametrize("dt", DTS)
@pytest.mark.parametrize("H,G,d,vd", [(4, 2, 32, 48), (2, 2, 64, 128)])
@pytest.mark.parametrize("qlen", [1, 37])
@pytest.mark.parametrize("back,seen", [(0, True), (19, True), (20, False), (21, False), (300, False)])
def test_the_window_edge_is_where_it_belongs(ctx, ops, dt, H, G, d, vd, qlen, back, seen):
    """One key gets a score far above the rest, `back` tokens behind the last query row; a window of 20 holds the row
    itself and the 19 before it.  Seen, it takes nearly all the weight; one token outside, it takes none."""
    n, window = 420, 20
    j = n - 1 - back
    got, want = run_attention(ctx, ops, dt, H, G, d, vd, lens=[n], qlens=[qlen], bs=16, window=window, sink=False, gate=False, scale=1.0,
                              seed=11, boost=(0, qlen - 1, j, 60.0))
    assert torch.allclose(got, want, **tol(dt))
    g = torch.Generator().manual_seed(11)     # the same draws as run_attention: the value row of key j
    _ks = [torch.randn(n, G, d, generator=g)]
    vs = torch.randn(n, G, vd, generator=g)
    if dt == torch.bfloat16:
        vs = vs.bfloat16().float()
    vj = torch.cat([vs[j, h // (H // G)] for h in range(H)]) * 1.25
    close = torch.allclose(got[-1], vj, rtol=0.05, atol=0.05)
    assert close == seen


@pytest.mark.parametrize("dt", DTS)
@pytest.mark.parametrize("where", [0, 1, 15, 16, 17, 500, 1023, 1024])
@pytest.mark.parametrize("qlens", [[3, 40], [1, 1]])
def test_full_attention_finds_one_far_key(ctx, ops, dt, where, qlens):
    """One key among 1 100 takes nearly all the weight of the last row - in a prompt portion and in a decode step (keys split over
    warps) - wherever it lies: the first tokens, either side of a page border, far back."""
    n = 1100
    got, want = run_attention(ctx, ops, dt, 4, 2, 32, 48, lens=[n, 40], qlens=qlens, bs=16, window=0, sink=False, gate=False, scale=1.0,
                              seed=12, boost=(0, qlens[0] - 1, where, 60.0))
    assert torch.allclose(got, want, **tol(dt))


@pytest.mark.parametrize("dt", DTS)
def test_a_large_sink_takes_the_weight_and_a_small_one_does_not(ctx, ops, dt):
    g = torch.Generator().manual_seed(13)
    H, G, d, vd, n, bs = 2, 1, 16, 24, 50, 16
    q = torch.randn(1, H * d, generator=g).to(dt)
    k, v = torch.randn(n, G * d, generator=g).to(dt), torch.randn(n, G * vd, generator=g).to(dt)
    kc, vc, tab = paged([k.float()], [v.float()], bs, 6, g)
    for s0, s1 in ((40.0, -40.0), (-40.0, 40.0)):
        sink = torch.tensor([s0, s1])
        got = ops.attn_paged_wide(ctx, q.to(DEV), kc.to(dt).to(DEV), vc.to(dt).to(DEV), i32(tab), i32([n]), None, 1, bs, H, G, d, vd, 0.25, 0,
                                  sink.to(DEV)).float().cpu()
        want = R.softmax_attention(q.float().view(1, H, d), k.float().view(n, G, d), v.float().view(n, G, vd), 0.25, torch.tensor([n - 1]), None, sink)
        assert torch.allclose(got, want, **tol(dt))
        big = 0 if s0 > 0 else 1
        assert got[0, big * vd:(big + 1) * vd].abs().max() < 1e-6 and got[0, (1 - big) * vd:(2 - big) * vd].abs().max() > 1e-2


def test_paged_prefill_kernel_writes_into_wider_rows(ctx, ops):
    """The tcgen05 paged-prefill kernel with a caller's output row stride: its heads land in the left columns of wider rows and
    the columns to their right stay as they were."""
    g = torch.Generator().manual_seed(16)
    H, G, d, bs, lens, qlens = 4, 2, 128, 16, [200, 90], [130, 90]
    ks = [torch.randn(n, G, d, generator=g).bfloat16().float() for n in lens]
    vs = [torch.randn(n, G, d, generator=g).bfloat16().float() for n in lens]
    qs = [torch.randn(m, H, d, generator=g).bfloat16().float() for m in qlens]
    want = torch.cat([R.softmax_attention(qs[b], ks[b], vs[b], 0.09, torch.arange(lens[b] - qlens[b], lens[b])) for b in range(2)])
    nblocks = sum((n + bs - 1) // bs for n in lens) + 2
    kc, vc, tables = paged([k.reshape(k.shape[0], -1) for k in ks], [v.reshape(v.shape[0], -1) for v in vs], bs, nblocks, g)
    rows = sum(qlens)
    out = torch.full((rows, H * d + 72), 7.0, dtype=torch.bfloat16, device=DEV)
    ctx.prefill_attn_paged_ld(torch.cat(qs).reshape(rows, H * d).bfloat16().to(DEV), kc.view(nblocks, bs, G, d).bfloat16().to(DEV),
                              vc.view(nblocks, bs, G, d).bfloat16().to(DEV), i32(tables), i32(lens), i32([0, 130, 220]), 130, H, G, d, bs, 0.09, out)
    assert torch.allclose(out[:, :H * d].float().cpu(), want, rtol=2e-2, atol=2e-2)
    assert (out[:, H * d:].float() == 7.0).all()


# ---------------------------------------------------------------------------------------------------------------- retention
def plain_retention(q, k, v, decay, S):
    """q, k: [T, H, d]; v: [T, H, vd]; S: [H, d, vd].  Returns (o [T, H, vd], S after)."""
    o = torch.zeros(q.shape[0], q.shape[1], v.shape[2])
    S = S.clone()
    for t in range(q.shape[0]):
        S = decay.view(-1, 1, 1) * S + k[t].unsqueeze(-1) * v[t].unsqueeze(-2)
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    return o, S


@pytest.mark.parametrize("form", ["token by token", "32 tokens at a time"])
@pytest.mark.parametrize("H,d,vd", [(3, 16, 24), (2, 32, 64), (1, 8, 1), (4, 64, 40), (2, 128, 96), (2, 200, 72), (1, 300, 33)])
def test_retention_carries_state_between_portions_and_slots(ctx, ops, H, d, vd, form):
    max_qlen = 1 if form == "token by token" else 64
    g = torch.Generator().manual_seed(14)
    slots = 4
    decay = torch.tensor([0.5, 1.0, 0.99, 0.0])[:H].contiguous()
    state = torch.randn(slots, H, d, vd, generator=g)        # whatever an earlier owner left behind
    state_d = state.to(DEV)
    ref = {}
    lens = {"a": 37, "b": 5, "c": 97}
    data = {n: (torch.randn(T, H, d, generator=g), torch.randn(T, H, d, generator=g) * d ** -0.5, torch.randn(T, H, vd, generator=g)) for n, T in lens.items()}
    want = {n: plain_retention(*data[n], decay, torch.zeros(H, d, vd))[0] for n in lens}
    got = {n: torch.zeros(T, H * vd) for n, T in lens.items()}
    at = {n: 0 for n in lens}
    slot_of = {"a": 2, "b": 0, "c": 3}
    # steps of (name, count): portions beside single tokens, in changing batch order
    sched = [[("a", 20), ("b", 1)], [("b", 1), ("a", 1), ("c", 33)], [("c", 1), ("b", 3), ("a", 16)], [("c", 63)]]
    for step in sched:
        cu, pos, q, k, v = [0], [], [], [], []
        for n, c in step:
            lo = at[n]
            q.append(data[n][0][lo:lo + c]); k.append(data[n][1][lo:lo + c]); v.append(data[n][2][lo:lo + c])
            pos += list(range(lo, lo + c))
            cu.append(cu[-1] + c)
        N = cu[-1]
        o = ops.retention_scan(ctx, torch.cat(q).reshape(N, H * d).to(DEV), torch.cat(k).reshape(N, H * d).to(DEV), torch.cat(v).reshape(N, H * vd).to(DEV),
                               state_d, i32([slot_of[n] for n, _ in step]), i32(cu), i32(pos), decay.to(DEV), H, d, vd, max_qlen).cpu()
        for b, (n, c) in enumerate(step):
            got[n][at[n]:at[n] + c] = o[cu[b]:cu[b + 1]]
            at[n] += c
    for n in lens:
        assert at[n] == lens[n]
        assert torch.allclose(got[n], want[n].reshape(lens[n], H * vd), rtol=2e-5, atol=2e-5), n
    assert torch.equal(state_d[1].cpu(), state[1])           # a slot nobody owns is not touched
    # decode form (no cu_seqlens): sequence "b" goes on, a new owner of slot 3 starts at position 0 over the old state
    qb, kb, vb = (torch.randn(1, H, x, generator=g) for x in (d, d, vd))
    qn, kn, vn = (torch.randn(1, H, x, generator=g) for x in (d, d, vd))
    Sb = plain_retention(*data["b"], decay, torch.zeros(H, d, vd))[1]
    o = ops.retention_scan(ctx, torch.cat([qb, qn]).reshape(2, H * d).to(DEV), torch.cat([kb, kn]).reshape(2, H * d).to(DEV),
                           torch.cat([vb, vn]).reshape(2, H * vd).to(DEV), state_d, i32([0, 3]), None, i32([5, 0]), decay.to(DEV), H, d, vd).cpu()
    assert torch.allclose(o[0], plain_retention(qb, kb, vb, decay, Sb)[0].reshape(-1), rtol=2e-5, atol=2e-5)
    assert torch.allclose(o[1], plain_retention(qn, kn, vn, decay, torch.zeros(H, d, vd))[0].reshape(-1), rtol=2e-5, atol=2e-5)


def test_retention_remembers_a_far_token_by_its_decay(ctx, ops):
    """One early key matches the last query; everything between is orthogonal to it.  The output is decay^(distance) v."""
    H, d, vd, T = 2, 16, 8, 600
    decay = torch.tensor([0.99, 0.999])
    q, k, v = torch.zeros(T, H, d), torch.zeros(T, H, d), torch.randn(T, H, vd, generator=torch.Generator().manual_seed(15))
    k[:, :, 1] = 1.0           # every other token writes along axis 1
    k[3, :, :] = 0.0
    k[3, :, 0] = 1.0           # token 3 writes along axis 0
    q[T - 1, :, 0] = 1.0       # the last token reads axis 0
    for max_qlen in (1, T):
        state = torch.zeros(1, H, d, vd, device=DEV)
        o = ops.retention_scan(ctx, q.reshape(T, -1).to(DEV), k.reshape(T, -1).to(DEV), v.reshape(T, -1).to(DEV), state, i32([0]), i32([0, T]),
                               i32(list(range(T))), decay.to(DEV), H, d, vd, max_qlen).cpu().view(T, H, vd)
        for h in range(H):
            assert torch.allclose(o[T - 1, h], float(decay[h]) ** (T - 1 - 3) * v[3, h], rtol=1e-4, atol=1e-6)
