"""Each Karuzen mechanism alone: the CUDA kernel against the plain fp32 functions of oracle/karuzen_oracle.py,
in both storage formats (bf16 serving, fp32 exact)."""
import importlib
import math

import pytest
import torch

from oracle import karuzen_oracle as K

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTS = [torch.float32, torch.bfloat16]


@pytest.fixture(scope="module")
def ops():
    return importlib.import_module("nano-vllm-candle_b200.ops")


def tol(dt):
    return dict(rtol=2e-5, atol=2e-5) if dt == torch.float32 else dict(rtol=2e-2, atol=2e-2)


def test_embed_gather_f32(ctx, ops):
    g = torch.Generator().manual_seed(1)
    for dt in DTS:
        table = torch.randn(37, 72, generator=g).to(dt).to(DEV)
        ids = torch.tensor([0, 36, 5, 5, 17], dtype=torch.int32, device=DEV)
        out = ops.embed_gather_f32(ctx, ids, table)
        assert torch.equal(out.cpu(), table.float().cpu()[ids.cpu().long()])


@pytest.mark.parametrize("dt", DTS)
@pytest.mark.parametrize("H", [24, 200, 1100])
def test_dyt_norm_accumulates_and_norms(ctx, ops, dt, H):
    g = torch.Generator().manual_seed(2)
    N = 7
    res, a0, a1, a2 = (torch.randn(N, H, generator=g) * 3 for _ in range(4))
    w, b, alpha = 1 + 0.2 * torch.randn(H, generator=g), 0.1 * torch.randn(H, generator=g), torch.tensor(0.37)
    want_res = res + a0 + a1 + a2
    want = K.dyt(want_res, w, b, alpha)
    d = [t.to(DEV) for t in (res, a0, a1, a2, w, b, alpha.view(1))]
    ro, out = ops.dyt_norm(ctx, d[0], d[1:4], d[4], d[5], d[6], out_dtype=dt)
    assert torch.allclose(ro.cpu(), want_res, rtol=1e-6, atol=1e-6)
    assert torch.allclose(out.float().cpu(), want, **tol(dt))
    # gathered rows, nothing written back; one addend only
    rows = torch.tensor([6, 0, 3], dtype=torch.int32, device=DEV)
    before = d[0].clone()
    _, out2 = ops.dyt_norm(ctx, d[0], [d[1]], d[4], d[5], d[6], out_dtype=dt, rows=rows)
    assert torch.equal(before, d[0])
    assert torch.allclose(out2.float().cpu(), K.dyt(want_res + a0, w, b, alpha)[rows.cpu().long()], **tol(dt))


@pytest.mark.parametrize("dt", DTS)
def test_latent_norm_store_divides_by_the_logical_width(ctx, ops, dt):
    g = torch.Generator().manual_seed(3)
    N, n0, n1, off1, ld = 9, 40, 72, 64, 160     # neither width is a multiple of 32 or of the padding
    x = torch.randn(N, ld, generator=g) * 2
    x[:, n0:off1] = 0
    w0, w1 = 1 + 0.2 * torch.randn(n0, generator=g), 1 + 0.2 * torch.randn(n1, generator=g)
    slots = torch.tensor([5, 0, -1, 17, 3, 4, 30, 31, 8], dtype=torch.int32)
    cache = torch.zeros(32, 128, dtype=dt, device=DEV)
    cq = ops.latent_norm_store(ctx, x.to(DEV), n0, off1, n1, w0.to(DEV), w1.to(DEV), 1e-5, cache, slots.to(DEV), dt)
    assert torch.allclose(cq.float().cpu(), K.rms_norm(x[:, :n0], w0, 1e-5), **tol(dt))
    want_c = K.rms_norm(x[:, off1:off1 + n1], w1, 1e-5)
    for i, s in enumerate(slots.tolist()):
        if s >= 0:
            assert torch.allclose(cache[s, :n1].float().cpu(), want_c[i], **tol(dt))
    untouched = [s for s in range(32) if s not in slots.tolist()]
    assert float(cache[untouched].float().abs().max()) == 0 and float(cache[:, n1:].float().abs().max()) == 0


@pytest.mark.parametrize("dt", DTS)
def test_activations(ctx, ops, dt):
    g = torch.Generator().manual_seed(4)
    x = (torch.randn(11, 2 * 56, generator=g) * 2).to(dt)
    xf = x.float()
    out = ops.act_mul(ctx, x.to(DEV), 56, ops.ACT_GELU_TANH_MUL)
    assert torch.allclose(out.float().cpu(), K.gelu_tanh(xf[:, :56]) * xf[:, 56:], **tol(dt))
    out = ops.act_mul(ctx, x.to(DEV), 112, ops.ACT_RELU2)
    assert torch.allclose(out.float().cpu(), torch.relu(xf) ** 2, **tol(dt))


@pytest.mark.parametrize("M,I,Kd", [(1, 64, 64), (64, 192, 128), (300, 320, 192), (2100, 1024, 256)])
def test_gate_up_projection_with_gelu_in_the_epilogue(ctx, ops, M, I, Kd):
    """Both tcgen05 schedules (1-CTA tiles up to 128 rows, CTA pairs above) against gelu_tanh(gate) * up in fp32."""
    g = torch.Generator().manual_seed(21)
    a = torch.randn(M, Kd, generator=g).bfloat16()
    w = (torch.randn(2 * I, Kd, generator=g) * Kd ** -0.5 * 2).bfloat16()
    out = ctx.gemm_gelu_mul(a.to(DEV), ctx.interleave_gate_up(w.to(DEV)))
    z = a.float() @ w.float().T
    want = K.gelu_tanh(z[:, :I]) * z[:, I:]
    assert torch.allclose(out.float().cpu(), want, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("dt", DTS)
@pytest.mark.parametrize("shape", [(1, 16, 8), (70, 130, 100), (5, 257, 33), (200, 64, 64), (130, 72, 40), (64, 200, 264)])
def test_linear_any_shape(ctx, ops, dt, shape):
    M, N, Kd = shape
    g = torch.Generator().manual_seed(5)
    A, W = torch.randn(M, Kd, generator=g).to(dt), torch.randn(N, Kd, generator=g).to(dt) * Kd ** -0.5
    want = A.float() @ W.float().T
    out = ops.linear(ctx, A.to(DEV), W.to(DEV))
    assert torch.allclose(out.float().cpu(), want, **tol(dt))
    out = ops.linear(ctx, A.to(DEV), W.to(DEV), out_dtype=torch.float32, act=ops.ACT_RELU2)
    assert torch.allclose(out.cpu(), torch.relu(want) ** 2, rtol=2e-5, atol=2e-5)


def test_linear_large_shapes_take_the_wide_tiles(ctx, ops):
    """Enough rows and columns for one 128 x 128 tile per SM: plain, batched and grouped, with ragged edges."""
    g = torch.Generator().manual_seed(23)
    dt = torch.bfloat16
    A, W = torch.randn(5000, 72, generator=g).to(dt), (torch.randn(520, 72, generator=g) * 0.1).to(dt)
    out = ops.linear(ctx, A.to(DEV), W.to(DEV), out_dtype=torch.float32)
    assert torch.allclose(out.cpu(), A.float() @ W.float().T, rtol=2e-3, atol=2e-3)
    A3, W3 = torch.randn(5, 4000, 40, generator=g).to(dt), (torch.randn(5, 136, 40, generator=g) * 0.2).to(dt)
    out = ops.linear(ctx, A3.to(DEV), W3.to(DEV))
    assert torch.allclose(out.float().cpu(), torch.einsum("bmk,bnk->bmn", A3.float(), W3.float()), **tol(dt))
    sizes = [3000, 0, 129, 9000, 7871]
    offsets = torch.tensor([0] + list(torch.tensor(sizes).cumsum(0)), dtype=torch.int32)
    rows = int(offsets[-1])
    Ag, Wg = torch.randn(700, 48, generator=g).to(dt), (torch.randn(5, 130, 48, generator=g) * 0.2).to(dt)
    a_rows = torch.randint(0, 700, (rows,), generator=g, dtype=torch.int32)
    out = ops.linear_grouped(ctx, Ag.to(DEV), a_rows.to(DEV), Wg.to(DEV), offsets.to(DEV), rows, out_dtype=torch.float32, act=ops.ACT_RELU2)
    want = torch.zeros(rows, 130)
    for e in range(5):
        lo, hi = int(offsets[e]), int(offsets[e + 1])
        want[lo:hi] = torch.relu(Ag.float()[a_rows[lo:hi].long()] @ Wg[e].float().T) ** 2
    assert torch.allclose(out.cpu(), want, rtol=2e-3, atol=2e-3)


@pytest.mark.parametrize("dt", DTS)
def test_linear_batched_per_head(ctx, ops, dt):
    g = torch.Generator().manual_seed(6)
    A, W = torch.randn(5, 33, 40, generator=g).to(dt), torch.randn(5, 72, 40, generator=g).to(dt) * 0.2
    out = ops.linear(ctx, A.to(DEV), W.to(DEV))
    assert torch.allclose(out.float().cpu(), torch.einsum("bmk,bnk->bmn", A.float(), W.float()), **tol(dt))


@pytest.mark.parametrize("dt", DTS)
def test_linear_grouped_with_empty_and_ragged_groups(ctx, ops, dt):
    g = torch.Generator().manual_seed(7)
    G, N, Kd, T = 5, 48, 40, 30
    sizes = [0, 70, 1, 0, 129]
    offsets = torch.tensor([0] + list(torch.tensor(sizes).cumsum(0)), dtype=torch.int32)
    rows = int(offsets[-1])
    A, W = torch.randn(T, Kd, generator=g).to(dt), torch.randn(G, N, Kd, generator=g).to(dt) * 0.2
    a_rows = torch.randint(0, T, (rows,), generator=g, dtype=torch.int32)
    out = ops.linear_grouped(ctx, A.to(DEV), a_rows.to(DEV), W.to(DEV), offsets.to(DEV), rows, act=ops.ACT_RELU2)
    want = torch.zeros(rows, N)
    for e in range(G):
        lo, hi = int(offsets[e]), int(offsets[e + 1])
        want[lo:hi] = torch.relu(A.float()[a_rows[lo:hi].long()] @ W[e].float().T) ** 2
    assert torch.allclose(out.float().cpu(), want, **tol(dt))


@pytest.mark.parametrize("E,top,N", [(6, 2, 700), (16, 3, 45), (1, 1, 130), (70, 8, 33), (5, 5, 128), (9, 1, 1)])
def test_padded_sort_gather_and_grouped_tensor_core_product(ctx, ops, E, top, N):
    """Groups padded to the 128-row tile: offsets, padding rows, positions and the tile table of the sort; the gather; the
    grouped tcgen05 product (squared relu in the epilogue, fp32 and bf16 outputs) against a loop over the experts.  Expert
    choices are skewed so that some experts get nothing and one gets several tiles."""
    g = torch.Generator().manual_seed(100 + E + N)
    Kd, F = 192, 80
    score = torch.randn(N, E, generator=g) + torch.linspace(2.0, -2.0, E)
    if E > 2:
        score[:, 1] = -1e9                                        # an expert that nobody chooses
    idx = score.topk(top, dim=-1).indices.to(torch.int32)
    offsets, src, pos, tile_group = ops.moe_sort_padded(ctx, idx.to(DEV), E)
    offsets, src, pos, tile_group = offsets.cpu().long(), src.cpu().long(), pos.cpu().long(), tile_group.cpu().long()
    counts = torch.bincount(idx.flatten().long(), minlength=E)
    starts = torch.zeros(E + 1, dtype=torch.long)
    starts[1:] = ((counts + 127) // 128 * 128).cumsum(0)
    assert torch.equal(offsets, starts)
    used = int(starts[-1]) // 128
    for e in range(E):
        lo, n = int(starts[e]), int(counts[e])
        pairs = (idx.flatten().long() == e).nonzero().flatten()  # in token order: the sort is stable
        assert torch.equal(src[lo:lo + n], pairs // top)
        assert torch.equal(pos[pairs], torch.arange(lo, lo + n))
        assert (src[lo + n:int(starts[e + 1])] == -1).all()
        assert (tile_group[lo // 128:int(starts[e + 1]) // 128] == e).all()
    assert (tile_group[used:] == -1).all() and tile_group.numel() >= used
    x = torch.randn(N, Kd, generator=g).bfloat16()
    xs = ops.gather_rows(ctx, x.to(DEV), src.to(torch.int32).to(DEV), offsets[-1:].to(torch.int32).to(DEV))
    live = src[:used * 128]
    want_xs = torch.where((live >= 0).unsqueeze(1), x.float()[live.clamp(min=0)], torch.zeros(1))
    assert torch.equal(xs[:used * 128].float().cpu(), want_xs)
    assert (xs[used * 128:] == 3.0).all()                        # rows behind the device count are not touched
    W = (torch.randn(E, F, Kd, generator=g) * 0.1).bfloat16()
    for act, odt in ((ops.ACT_RELU2, torch.bfloat16), (ops.ACT_NONE, torch.float32)):
        out = ops.gemm_grouped(ctx, xs, W.to(DEV), tile_group.to(torch.int32).to(DEV), act=act, out_dtype=odt).float().cpu()
        for e in range(E):
            lo, n = int(starts[e]), int(counts[e])
            ref = want_xs[lo:lo + n] @ W[e].float().T
            if act == ops.ACT_RELU2:
                ref = torch.relu(ref) ** 2
            assert torch.allclose(out[lo:lo + n], ref, **(tol(odt) if odt == torch.bfloat16 else dict(rtol=1e-4, atol=1e-4))), f"expert {e}"
        assert (out[used * 128:] == 0).all()                     # tiles behind the last group are skipped


@pytest.mark.parametrize("M", [1, 77, 128, 300, 1100])
def test_squared_relu_in_the_product_epilogue(ctx, ops, M):
    g = torch.Generator().manual_seed(M)
    A, W = torch.randn(M, 128, generator=g).bfloat16(), (torch.randn(208, 128, generator=g) * 0.2).bfloat16()
    want = torch.relu(A.float() @ W.float().T) ** 2
    for odt in (torch.bfloat16, torch.float32):
        out = ops.gemm_act(ctx, A.to(DEV), W.to(DEV), ops.ACT_RELU2, odt)
        assert torch.allclose(out.float().cpu(), want, **(tol(odt) if odt == torch.bfloat16 else dict(rtol=1e-4, atol=1e-4)))
    plain = ops.gemm_act(ctx, A.to(DEV), W.to(DEV), ops.ACT_NONE, torch.float32)
    assert torch.allclose(plain.cpu(), A.float() @ W.float().T, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("E,top", [(6, 2), (16, 3), (1, 1), (70, 8), (5, 5)])
def test_moe_route_sort_combine(ctx, ops, E, top):
    g = torch.Generator().manual_seed(8 + E)
    N, H = 45, 88
    h = torch.randn(N, H, generator=g)
    router, corr, sg = torch.randn(E, H, generator=g) * 0.3, torch.randn(E, generator=g) * 0.5, torch.randn(H, generator=g) * 0.2
    idx, w, gate = ops.moe_route(ctx, h.to(DEV), router.to(DEV), corr.to(DEV), sg.to(DEV), top, 2.5)
    widx, ww = K.route(h, router, corr, top, 2.5)
    assert torch.equal(idx.cpu().long().sort(-1).values, widx.sort(-1).values)
    # weights follow the chosen experts whatever their order
    dense = torch.zeros(N, E).scatter(1, idx.cpu().long(), w.cpu())
    assert torch.allclose(dense, torch.zeros(N, E).scatter(1, widx, ww), rtol=1e-5, atol=1e-6)
    assert torch.allclose(gate.cpu(), torch.sigmoid(h @ sg), rtol=1e-5, atol=1e-6)
    # the same choice from logits taken by a matrix product (one more column: the shared gate)
    z = torch.cat([h @ router.T, (h @ sg).unsqueeze(1), torch.full((N, 3), float("nan"))], 1)
    idx2, w2, gate2 = ops.moe_route_logits(ctx, z.to(DEV), corr.to(DEV), E, top, 2.5, gate_col=E)
    assert torch.equal(idx2.cpu().long().sort(-1).values, widx.sort(-1).values)
    assert torch.allclose(torch.zeros(N, E).scatter(1, idx2.cpu().long(), w2.cpu()), torch.zeros(N, E).scatter(1, widx, ww), rtol=1e-5, atol=1e-6)
    assert torch.allclose(gate2.cpu(), torch.sigmoid(h @ sg), rtol=1e-5, atol=1e-6)
    offsets, src, pos = ops.moe_sort(ctx, idx, E)
    o, s, p = offsets.cpu().tolist(), src.cpu().tolist(), pos.cpu().tolist()
    assert o[0] == 0 and o[-1] == N * top
    flat = idx.cpu().flatten().tolist()
    for e in range(E):
        assert o[e + 1] - o[e] == flat.count(e)
    for pair, at in enumerate(p):
        assert o[flat[pair]] <= at < o[flat[pair] + 1] and s[at] == pair // top
    for e in range(E):          # stable: inside an expert's group the tokens ascend
        assert s[o[e]:o[e + 1]] == sorted(s[o[e]:o[e + 1]])
    assert sorted(p) == list(range(N * top))
    y = torch.randn(N * top, H, generator=g)
    shared = torch.randn(N, H, generator=g)
    out = ops.moe_combine(ctx, y.to(DEV), pos, w, shared.to(DEV), gate)
    want = (w.cpu().unsqueeze(-1) * y[pos.cpu().long().view(N, top)]).sum(1) + shared * gate.cpu().unsqueeze(-1)
    assert torch.allclose(out.cpu(), want, rtol=1e-5, atol=1e-5)


def test_moe_correction_changes_the_choice_but_not_the_weights(ctx, ops):
    """A large correction forces an expert in; its weight still comes from its unbiased score."""
    N, H, E = 3, 16, 4
    h = torch.ones(N, H)
    router = torch.zeros(E, H)
    router[0] = 0.5     # s0 = sigmoid(8) ~ 1
    router[1] = -0.5    # s1 ~ 0
    corr = torch.tensor([0.0, 5.0, 0.0, 0.0])
    idx, w, _ = ops.moe_route(ctx, h.to(DEV), router.to(DEV), corr.to(DEV), None, 2, 1.0)
    assert sorted(idx[0].cpu().tolist()) == [0, 1]
    s = torch.sigmoid(h @ router.T)[0]
    dense = torch.zeros(E).scatter(0, idx[0].cpu().long(), w[0].cpu())
    assert torch.allclose(dense[:2], s[:2] / (s[0] + s[1]), rtol=1e-5)


def paged(c_seqs, block_size, num_blocks, dt, seed):
    """Scatters per-sequence latents into a shuffled paged pool; returns (cache, block_tables, context_lens)."""
    g = torch.Generator().manual_seed(seed)
    D = c_seqs[0].shape[1]
    perm = torch.randperm(num_blocks, generator=g).tolist()
    cache = torch.full((num_blocks * block_size, D + 8), float("nan"))
    cache[:, D:] = 0
    bts, maxb = [], max((c.shape[0] + block_size - 1) // block_size for c in c_seqs)
    for c in c_seqs:
        nb = (c.shape[0] + block_size - 1) // block_size
        blocks = [perm.pop() for _ in range(nb)]
        for j in range(c.shape[0]):
            cache[blocks[j // block_size] * block_size + j % block_size, :D] = c[j]
        bts.append(blocks + [-1] * (maxb - nb))
    return (cache.to(dt).to(DEV), torch.tensor(bts, dtype=torch.int32, device=DEV),
            torch.tensor([c.shape[0] for c in c_seqs], dtype=torch.int32, device=DEV))


def attn_want(q, c, scale):
    """q [Tq, heads, D] are the last Tq positions of c [Tk, D]."""
    Tq, Tk = q.shape[0], c.shape[0]
    s = torch.einsum("ihd,jd->hij", q, c) * scale
    s = s.masked_fill(torch.arange(Tk).view(1, 1, Tk) > torch.arange(Tk - Tq, Tk).view(1, Tq, 1), float("-inf"))
    return torch.einsum("hij,jd->ihd", torch.softmax(s, -1), c)


@pytest.mark.parametrize("dt", DTS)
@pytest.mark.parametrize("heads,D,bs", [(3, 40, 16), (7, 64, 64), (1, 8, 32), (5, 96, 16), (16, 128, 64)])
def test_latent_attention_mixed_batch(ctx, ops, dt, heads, D, bs):
    """Portions behind cached prefixes, whole prompts and single decode rows in one launch, unwritten slots poisoned."""
    g = torch.Generator().manual_seed(11)
    ctx_lens, q_lens = [1, 130, 65, 64, 200, 17], [1, 1, 65, 2, 37, 17]
    cs = [(torch.randn(n, D, generator=g)).to(dt).float() for n in ctx_lens]
    cache, bt, cl = paged(cs, bs, 64, dt, 12)
    qs = [(torch.randn(n, heads, D, generator=g)).to(dt).float() for n in q_lens]
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device=DEV)
    out = ops.latent_attn_paged(ctx, torch.cat(qs).to(dt).to(DEV), cache, bt, cl, cu, max(q_lens), bs, 0.3)
    want = torch.cat([attn_want(q, c, 0.3) for q, c in zip(qs, cs)])
    assert torch.allclose(out.float().cpu(), want, **tol(dt))


@pytest.mark.parametrize("heads,D", [(5, 64), (16, 128), (40, 128), (70, 64)])
def test_latent_attention_decode_with_keys_split_over_ctas(ctx, ops, heads, D):
    """A small decode batch with a workspace: the keys of a sequence are walked by several CTAs and merged."""
    g = torch.Generator().manual_seed(17)
    bs, dt = 32, torch.bfloat16
    ctx_lens = [1, 63, 64, 65, 700, 129]
    cs = [torch.randn(n, D, generator=g).to(dt).float() for n in ctx_lens]
    cache, bt, cl = paged(cs, bs, 48, dt, 18)
    q = torch.randn(len(ctx_lens), heads, D, generator=g).to(dt).float()
    ws = torch.full((4 << 20,), float("nan"), dtype=torch.float32, device=DEV)
    out = ops.latent_attn_paged(ctx, q.to(dt).to(DEV), cache, bt, cl, None, 1, bs, 0.2, workspace=ws)
    plain = ops.latent_attn_paged(ctx, q.to(dt).to(DEV), cache, bt, cl, None, 1, bs, 0.2)
    want = torch.cat([attn_want(q[i:i + 1], c, 0.2) for i, c in enumerate(cs)])
    assert torch.allclose(out.float().cpu(), want, **tol(dt))
    assert torch.allclose(out.float(), plain.float(), rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("dt", DTS)
def test_latent_attention_decode_rows_without_cu_seqlens(ctx, ops, dt):
    g = torch.Generator().manual_seed(13)
    heads, D, bs = 4, 72, 16
    ctx_lens = [1, 16, 17, 300]
    cs = [torch.randn(n, D, generator=g).to(dt).float() for n in ctx_lens]
    cache, bt, cl = paged(cs, bs, 32, dt, 14)
    q = torch.randn(len(ctx_lens), heads, D, generator=g).to(dt).float()
    out = ops.latent_attn_paged(ctx, q.to(dt).to(DEV), cache, bt, cl, None, 1, bs, 0.25)
    want = torch.cat([attn_want(q[i:i + 1], c, 0.25) for i, c in enumerate(cs)])
    assert torch.allclose(out.float().cpu(), want, **tol(dt))


@pytest.mark.parametrize("dt,D", [(torch.float32, 32), (torch.bfloat16, 64), (torch.bfloat16, 128), (torch.bfloat16, 24)])
@pytest.mark.parametrize("where", [0, 1, 15, 16, 63, 64, 255, 256, 699, 700])
def test_latent_attention_finds_one_far_key(ctx, ops, where, dt, D):
    """One key among hundreds carries the whole weight: a lost page or tile, or an off-by-one in the causal bound, shows."""
    g = torch.Generator().manual_seed(15)
    heads, bs, Tk = 2, 64, 701
    c = torch.randn(Tk, D, generator=g) * 0.1
    q = torch.randn(1, heads, D, generator=g) * 0.1
    c[where] = 4.0 * q[0, 0] / q[0, 0].norm()
    q[0, 0] = 40.0 * q[0, 0] / q[0, 0].norm()
    c, q = c.to(dt).float(), q.to(dt).float()
    t = dict(rtol=1e-4, atol=1e-5) if dt == torch.float32 else dict(rtol=2e-2, atol=2e-2)
    cache, bt, cl = paged([c], bs, 16, dt, 16)
    out = ops.latent_attn_paged(ctx, q.to(dt).to(DEV), cache, bt, cl, None, 1, bs, 1.0)
    assert torch.allclose(out[0, 0].float().cpu(), c[where], atol=1e-3 if dt == torch.float32 else 3e-2)
    assert torch.allclose(out.float().cpu(), attn_want(q, c, 1.0), **t)
    # a portion of 40 tokens ends the sequence: row i sees the key iff where <= 661 + i
    q40 = q.repeat(40, 1, 1)
    cu = torch.tensor([0, 40], dtype=torch.int32, device=DEV)
    out40 = ops.latent_attn_paged(ctx, q40.to(dt).to(DEV), cache, bt, cl, cu, 40, bs, 1.0)
    assert torch.allclose(out40.float().cpu(), attn_want(q40, c, 1.0), **t)
    for i in (0, 38, 39):
        sees = where <= Tk - 40 + i
        assert torch.allclose(out40[i, 0].float().cpu(), c[where], atol=1e-1) == sees
