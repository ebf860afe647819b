"""The kernels of the Sukalorn mixers, each alone, against the plain implementation's functions (float64), in
float32 and bfloat16 storage: the row-wise kernel between the attention mixer's product and its attention, the
latent mixer's, the pair rotation, the activations, and the attention with reshaped scores over paged keys and
values of different widths (prompt tiles and single decoded tokens, one split and several, inputs built so that a
key just inside or just outside a block, a key hundreds of positions back, the cap or the distance bias decides
the result)."""

import math

import pytest
import torch

from plain import sukalorn_plain as plain

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]
TOL = {torch.float32: dict(atol=2e-5, rtol=2e-5), torch.bfloat16: dict(atol=2e-2, rtol=2e-2)}


def _ops():
    from ampere_kv_engine_b200.kernels import ops
    return ops


def _pages(seed, pages, heads, page_size, width, dtype):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return torch.randn((pages, heads, page_size, width), generator=g, device="cuda", dtype=torch.float32).to(dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,dim,vdim,gated,blend", [(4, 2, 8, 24, True, "reader"), (3, 3, 16, 8, True, "source"),
                                                                  (6, 1, 12, 20, False, None), (40, 8, 64, 128, True, "reader")])
def test_head_prep(dtype, heads, kv_heads, dim, vdim, gated, blend):
    ops = _ops()
    n, page_size, pages, eps = 37, 8, 9, 1e-5
    g = torch.Generator(device="cuda").manual_seed(5)
    width = heads * dim + kv_heads * (dim + vdim) + (heads if gated else 0)
    x = (3.0 * torch.randn((n, width), generator=g, device="cuda")).to(dtype)
    other = torch.randn((n, kv_heads * vdim), generator=g, device="cuda").to(dtype) if blend == "reader" else None
    keep = torch.full((n, kv_heads * vdim), float("nan"), device="cuda", dtype=dtype) if blend == "source" else None
    lam = torch.tensor([0.3], device="cuda")
    slots = torch.randperm(pages * page_size, generator=g, device="cuda")[:n].to(torch.int32)
    slots[5] = -1
    k_cache = torch.zeros((pages, kv_heads, page_size, dim), device="cuda", dtype=dtype)
    v_cache = torch.zeros((pages, kv_heads, page_size, vdim), device="cuda", dtype=dtype)
    q, gate = ops.head_prep(x, slots, k_cache, v_cache, num_heads=heads, num_kv_heads=kv_heads, head_dim=dim, v_dim=vdim,
                            unit_norm=True, eps=eps, gated=gated, v_keep=keep, v_other=other,
                            blend_weight=lam if other is not None else None)
    xd = x.double().cpu()
    a, b = heads * dim, kv_heads * dim
    want_q = plain.rms_unit(xd[:, :a].view(n, heads, dim), eps)
    want_k = plain.rms_unit(xd[:, a:a + b].view(n, kv_heads, dim), eps)
    own = xd[:, a + b:a + b + kv_heads * vdim].view(n, kv_heads, vdim)
    want_v = own if other is None else 0.7 * own + 0.3 * other.double().cpu().view(n, kv_heads, vdim)
    torch.testing.assert_close(q.double().cpu().view(n, heads, dim), want_q, **TOL[dtype])
    if gated:
        torch.testing.assert_close(gate.double().cpu(), torch.sigmoid(xd[:, a + b + kv_heads * vdim:]), atol=1e-6, rtol=1e-5)
    else:
        assert gate is None
    if keep is not None:
        torch.testing.assert_close(keep.double().cpu().view(n, kv_heads, vdim), own, atol=0, rtol=0)
    s = slots.cpu().long()
    for t in range(n):
        if s[t] < 0:
            continue
        torch.testing.assert_close(k_cache[s[t] // page_size, :, s[t] % page_size].double().cpu(), want_k[t], **TOL[dtype])
        torch.testing.assert_close(v_cache[s[t] // page_size, :, s[t] % page_size].double().cpu(), want_v[t], **TOL[dtype])
    written = torch.zeros(pages * page_size, dtype=torch.bool)
    written[s[s >= 0]] = True
    assert float(k_cache.view(pages, kv_heads, page_size, dim).permute(0, 2, 1, 3).reshape(pages * page_size, -1)[~written].abs().max()) == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("q_rank,kv_rank,rot_dim,dims,heads,dim", [(40, 24, 8, 8, 3, 8), (16, 36, 12, 4, 2, 12),
                                                                    (96, 128, 32, 32, 4, 64), (7, 5, 6, 2, 1, 3)])
def test_latent_prep_and_pair_rotation(dtype, q_rank, kv_rank, rot_dim, dims, heads, dim):
    ops = _ops()
    n, page_size, pages, eps, base = 29, 4, 11, 1e-6, 500.0
    g = torch.Generator(device="cuda").manual_seed(9)
    x = (2.0 * torch.randn((n, q_rank + kv_rank + rot_dim), generator=g, device="cuda")).to(dtype)
    positions = torch.randint(0, 3000, (n,), generator=g, device="cuda").to(torch.int32)
    wq = 1 + 0.1 * torch.randn(q_rank, generator=g, device="cuda")
    wkv = 1 + 0.1 * torch.randn(kv_rank, generator=g, device="cuda")
    i = torch.arange(dims // 2, dtype=torch.float64)
    inv_freq = (base ** (-2.0 * i / dims)).float().cuda()
    slots = torch.randperm(pages * page_size, generator=g, device="cuda")[:n].to(torch.int32)
    cache = torch.zeros((pages, 1, page_size, kv_rank + rot_dim), device="cuda", dtype=dtype)
    q_latent = ops.latent_prep(x, positions, slots, wq, wkv, inv_freq, cache, q_rank=q_rank, kv_rank=kv_rank,
                               rot_dim=rot_dim, rotary_dims=dims, eps=eps)
    xd, pos = x.double().cpu(), positions.cpu().long()
    tol = dict(TOL[dtype])
    if dtype == torch.float32:
        tol = dict(atol=3e-4, rtol=1e-4)      # float32 angles of positions in the thousands
    torch.testing.assert_close(q_latent.double().cpu(), plain.norm_plain(xd[:, :q_rank], wq.double().cpu(), eps), **TOL[dtype])
    want = torch.cat((plain.norm_plain(xd[:, q_rank:q_rank + kv_rank], wkv.double().cpu(), eps),
                      plain.rotate_interleaved(xd[:, q_rank + kv_rank:], pos, base, dims)), dim=-1)
    s = slots.cpu().long()
    torch.testing.assert_close(cache[s // page_size, 0, s % page_size].double().cpu(), want, **tol)
    # the queries' rotated part: columns [dim, dim + rot_dim) of every head go to [kv_rank, kv_rank + rot_dim)
    q = torch.randn((n, heads * (dim + rot_dim)), generator=g, device="cuda").to(dtype)
    out = torch.full((n, heads * (kv_rank + rot_dim)), 7.0, device="cuda", dtype=dtype)
    ops.rotate_pairs(q, out, positions, inv_freq, heads=heads, cols=rot_dim, rotary_dims=dims, in_offset=dim, out_offset=kv_rank)
    want_q = plain.rotate_interleaved(q.double().cpu().view(n, heads, dim + rot_dim)[..., dim:], pos, base, dims)
    got = out.double().cpu().view(n, heads, kv_rank + rot_dim)
    torch.testing.assert_close(got[..., kv_rank:], want_q, **tol)
    assert bool((got[..., :kv_rank] == 7.0).all())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("count", [1, 7, 8 * 300 + 3])
def test_activations(dtype, count):
    ops = _ops()
    x = (3 * torch.randn(count, device="cuda", generator=torch.Generator(device="cuda").manual_seed(count))).to(dtype)
    z = x.double().cpu()
    gelu = 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))
    for kind, want in (("relu2", plain.relu_squared(z)), ("gelu_tanh", gelu), ("silu", z * torch.sigmoid(z))):
        torch.testing.assert_close(ops.activation(x, kind).double().cpu(), want, **TOL[dtype])


def _dense_attention(q, k, v, *, first_pos, scale, softcap, slopes, chunk, window, gate):
    """q [n, H, D] at positions first_pos.., k [ctx, G, D], v [ctx, G, Dv], all float64 on the CPU."""
    n, H, _ = q.shape
    ctx, G, _ = k.shape
    kh, vh = k.repeat_interleave(H // G, dim=1), v.repeat_interleave(H // G, dim=1)
    s = torch.einsum("ihd,jhd->hij", q, kh) * scale
    if softcap:
        s = softcap * torch.tanh(s / softcap)
    pos = torch.arange(first_pos, first_pos + n)[:, None]
    keys = torch.arange(ctx)[None, :]
    if slopes is not None:
        s = s - slopes[:, None, None] * (pos - keys).double()[None]
    visible = keys <= pos
    if chunk:
        visible &= (keys // chunk) == (pos // chunk)
    if window:
        visible &= keys > pos - window
    out = torch.einsum("hij,jhd->ihd", plain.masked_softmax(s, visible[None]), vh)
    return out if gate is None else out * gate[:, :, None]


def _run_scored(ops, dtype, q, keys, values, tables, seq_q, *, heads, kv_heads, v_dim, page_size, q_tile, splits, **score):
    """One call over sequences given as (context length, new tokens): q rows are the new tokens of all sequences."""
    cu = [0]
    for _, n in seq_q:
        cu.append(cu[-1] + n)
    tiles = [(s, cu[s] + t0, min(q_tile, n - t0)) for s, (_, n) in enumerate(seq_q) for t0 in range(0, n, q_tile)]
    dev = lambda values_: torch.tensor(values_, dtype=torch.int32, device="cuda")
    out = torch.full((q.shape[0], heads * v_dim), float("nan"), device="cuda", dtype=dtype)
    ops.scored_attention(q, keys, values, tables, dev(cu), dev([c for c, _ in seq_q]), dev([t[0] for t in tiles]),
                         dev([t[1] for t in tiles]), dev([t[2] for t in tiles]), num_tiles=len(tiles), q_tile=q_tile,
                         num_splits=splits, num_heads=heads, num_kv_heads=kv_heads, v_dim=v_dim, out=out, **score)
    return out


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,dim,v_dim,chunk,softcap,biased,gated", [
    (4, 2, 8, 24, 20, 2.0, True, True), (3, 3, 16, 8, 7, 30.0, True, True), (6, 1, 12, 20, 0, 0.0, False, False),
    (8, 2, 128, 64, 96, 10.0, True, True), (5, 5, 36, 36, 33, 0.0, True, False)])
@pytest.mark.parametrize("splits", [1, 3])
def test_scored_attention_prompts_and_decoded_tokens(dtype, heads, kv_heads, dim, v_dim, chunk, softcap, biased, gated, splits):
    """Three sequences in one call: a whole prompt from position 0, a portion that starts in the middle of a block
    and crosses two block edges, and, in a second call with one-token tiles, single decoded tokens whose position is
    the last of a block, the first of a block, and one in between."""
    ops = _ops()
    page_size, scale = 16, 0.4
    g = torch.Generator(device="cuda").manual_seed(31)
    slopes = plain.distance_slopes(heads) if biased else None
    for seq_q, q_tile in (([(70, 70), (150, 61), (3, 2)], 32), ([(chunk * 3 or 40, 1), (chunk * 3 + 1 or 41, 1), (131, 1), (1, 1)], 1)):
        num_pages = sum((c + page_size - 1) // page_size for c, _ in seq_q) + 3
        k_pages, v_pages = _pages(1, num_pages, kv_heads, page_size, dim, dtype), _pages(2, num_pages, kv_heads, page_size, v_dim, dtype)
        order = torch.randperm(num_pages, generator=torch.Generator().manual_seed(4)).tolist()
        width = max((c + page_size - 1) // page_size for c, _ in seq_q)
        table = torch.full((len(seq_q), width), -1, dtype=torch.int32)
        for s, (c, _) in enumerate(seq_q):
            for j in range((c + page_size - 1) // page_size):
                table[s, j] = order.pop()
        total = sum(n for _, n in seq_q)
        q = torch.randn((total, heads * dim), generator=g, device="cuda").to(dtype)
        gate = torch.rand((total, heads), generator=g, device="cuda") if gated else None
        out = _run_scored(ops, dtype, q, k_pages, v_pages, table.cuda(), seq_q, heads=heads, kv_heads=kv_heads, v_dim=v_dim,
                          page_size=page_size, q_tile=q_tile, splits=splits, scale=scale, chunk=chunk, softcap=softcap,
                          slopes=None if slopes is None else slopes.float().cuda(), gate=gate)
        row = 0
        for s, (c, n) in enumerate(seq_q):
            pages = table[s].long()[torch.arange(c) // page_size]
            k = k_pages.cpu()[pages, :, torch.arange(c) % page_size].double()
            v = v_pages.cpu()[pages, :, torch.arange(c) % page_size].double()
            want = _dense_attention(q[row:row + n].double().cpu().view(n, heads, dim), k, v, first_pos=c - n, scale=scale,
                                    softcap=softcap, slopes=slopes, chunk=chunk, window=0,
                                    gate=None if gate is None else gate[row:row + n].double().cpu())
            torch.testing.assert_close(out[row:row + n].double().cpu().view(n, heads, v_dim), want, **TOL[dtype])
            row += n


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("splits", [1, 4])
def test_one_key_decides_far_back_and_at_a_block_edge(dtype, splits):
    """All keys but one are orthogonal to the query; the one that is not has a value of its own.  Far back in a long
    context (no blocks) it must own the output; as the first key of the query's block it must own it too; as the last
    key of the block before, it must not show at all."""
    ops = _ops()
    heads, dim, v_dim, page_size, ctx = 2, 16, 8, 16, 700
    num_pages = (ctx + page_size - 1) // page_size
    table = torch.arange(num_pages - 1, -1, -1, dtype=torch.int32)[None].cuda()         # pages in reverse order
    for chunk, special, shows in ((0, 3, True), (128, 640, True), (128, 639, False), (0, 699, True)):
        k = torch.zeros((ctx, 1, dim))
        k[:, 0, 1] = 1.0
        k[special, 0, 0] = 1.0
        v = torch.ones((ctx, 1, v_dim))
        v[special] = -50.0
        k_pages = torch.zeros((num_pages, 1, page_size, dim))
        v_pages = torch.zeros((num_pages, 1, page_size, v_dim))
        pages = table[0].cpu().long()[torch.arange(ctx) // page_size]
        k_pages[pages, :, torch.arange(ctx) % page_size] = k
        v_pages[pages, :, torch.arange(ctx) % page_size] = v
        q = torch.zeros((1, heads * dim))
        q[0, 0], q[0, dim] = 30.0, 30.0                      # both heads look along dimension 0
        out = _run_scored(ops, dtype, q.cuda().to(dtype), k_pages.cuda().to(dtype), v_pages.cuda().to(dtype), table,
                          [(ctx, 1)], heads=heads, kv_heads=1, v_dim=v_dim, page_size=page_size, q_tile=1, splits=splits,
                          scale=1.0, chunk=chunk)
        want = -50.0 if shows else 1.0
        assert torch.allclose(out.float().cpu(), torch.full((1, heads * v_dim), want), atol=1e-3), (chunk, special, out)


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_latent_row_read_as_key_and_value(dtype):
    """One paged tensor, read whole as the key and in its first v_dim elements as the value, one kv head for all
    query heads: what the latent mixer asks of the kernel."""
    ops = _ops()
    heads, row, v_dim, page_size = 5, 40, 24, 8
    seq_q = [(50, 50), (77, 1), (9, 2)]
    num_pages = 20
    rows = _pages(8, num_pages, 1, page_size, row, dtype)
    table = torch.full((3, 10), -1, dtype=torch.int32)
    order = list(range(num_pages))[::-1]
    for s, (c, _) in enumerate(seq_q):
        for j in range((c + page_size - 1) // page_size):
            table[s, j] = order.pop()
    q = torch.randn((53, heads * row), device="cuda", generator=torch.Generator(device="cuda").manual_seed(1)).to(dtype)
    out = _run_scored(ops, dtype, q, rows, rows, table.cuda(), seq_q, heads=heads, kv_heads=1, v_dim=v_dim, page_size=page_size,
                      q_tile=32, splits=1, scale=0.2)
    at = 0
    for s, (c, n) in enumerate(seq_q):
        pages = table[s].long()[torch.arange(c) // page_size]
        k = rows.cpu()[pages, :, torch.arange(c) % page_size].double()
        want = _dense_attention(q[at:at + n].double().cpu().view(n, heads, row), k, k[..., :v_dim], first_pos=c - n, scale=0.2,
                                softcap=0.0, slopes=None, chunk=0, window=0, gate=None)
        torch.testing.assert_close(out[at:at + n].double().cpu().view(n, heads, v_dim), want, **TOL[dtype])
        at += n


@pytest.mark.parametrize("heads,kv_heads,dim,chunk,softcap,biased,gated", [
    (8, 2, 128, 96, 10.0, True, True), (4, 4, 128, 0, 0.0, True, False), (6, 2, 128, 50, 3.0, False, True),
    (8, 1, 64, 40, 3.0, True, True), (5, 1, 128, 200, 30.0, True, True)])
def test_tensor_core_forms_match_the_plain_formula_and_the_general_kernel(heads, kv_heads, dim, chunk, softcap, biased, gated):
    """bfloat16 keys and values of the same 64 or 128 dims: prompt tiles on the tcgen05 kernel's scored form (128
    dims), single tokens on the decode kernel's (1, 2, 4 and 8 key splits), against the float64 formula and, more
    tightly, against the general kernel on the same inputs.  Positions are chosen at block edges; pages of blocks the
    sequence has left are not held (-1 in the table) and hold NaN."""
    ops = _ops()
    dtype, page_size, scale = torch.bfloat16, 16, 0.1
    g = torch.Generator(device="cuda").manual_seed(77)
    slopes = plain.distance_slopes(heads) if biased else None
    c3 = chunk * 3 or 300
    group = heads // kv_heads
    q_tile = ops.attention_q_tile(dim, group)
    cases = [([(c3, 1), (c3 + 1, 1), (c3 - 1, 1), (700, 1), (1, 1)], 1, (1, 2, 4, 8))]
    if dim == 128:
        cases.append(([(300, 300), (c3 + 37, 90), (3, 2), (c3, 1)], q_tile, (1,)))
    for seq_q, tile, split_counts in cases:
        num_pages = sum((c + page_size - 1) // page_size for c, _ in seq_q) + 2
        k_pages, v_pages = _pages(1, num_pages, kv_heads, page_size, dim, dtype), _pages(2, num_pages, kv_heads, page_size, dim, dtype)
        order = torch.randperm(num_pages, generator=torch.Generator().manual_seed(4)).tolist()
        width = max((c + page_size - 1) // page_size for c, _ in seq_q)
        table = torch.full((len(seq_q), width), -1, dtype=torch.int32)
        for s, (c, n) in enumerate(seq_q):
            first_needed = ((c - n) // chunk * chunk) if chunk else 0
            for j in range((c + page_size - 1) // page_size):
                page = order.pop()
                if (j + 1) * page_size <= first_needed:          # a page the sequence has given back
                    k_pages[page], v_pages[page] = float("nan"), float("nan")
                else:
                    table[s, j] = page
        total = sum(n for _, n in seq_q)
        q = (3 * torch.randn((total, heads * dim), generator=g, device="cuda")).to(dtype)
        gate = torch.rand((total, heads), generator=g, device="cuda") if gated else None
        score = dict(scale=scale, chunk=chunk, softcap=softcap, slopes=None if slopes is None else slopes.float().cuda(), gate=gate)
        common = dict(heads=heads, kv_heads=kv_heads, v_dim=dim, page_size=page_size, q_tile=tile)
        general = _run_scored(ops, dtype, q, k_pages, v_pages, table.cuda(), seq_q, splits=1, kernel="general", **common, **score)
        for splits in split_counts:
            out = _run_scored(ops, dtype, q, k_pages, v_pages, table.cuda(), seq_q, splits=splits, **common, **score)
            torch.testing.assert_close(out.float(), general.float(), atol=6e-3, rtol=2e-2)
            row = 0
            for s, (c, n) in enumerate(seq_q):
                first_needed = ((c - n) // chunk * chunk) if chunk else 0
                keys = torch.arange(c)
                pages = table[s].long()[keys // page_size].clamp(min=0)
                k = k_pages.cpu()[pages, :, keys % page_size].double()
                v = v_pages.cpu()[pages, :, keys % page_size].double()
                k[:first_needed // page_size * page_size] = 0
                v[:first_needed // page_size * page_size] = 0
                want = _dense_attention(q[row:row + n].double().cpu().view(n, heads, dim), k, v, first_pos=c - n, scale=scale,
                                        softcap=softcap, slopes=slopes, chunk=chunk, window=0,
                                        gate=None if gate is None else gate[row:row + n].double().cpu())
                torch.testing.assert_close(out[row:row + n].double().cpu().view(n, heads, dim), want, **TOL[dtype])
                row += n


@pytest.mark.parametrize("heads,row,v_dim,window", [(5, 160, 128, 0), (16, 576, 512, 0), (3, 96, 64, 70), (20, 272, 256, 0)])
@pytest.mark.parametrize("splits", [1, 3, 8])
def test_shared_rows_on_tensor_cores(heads, row, v_dim, window, splits):
    """bfloat16 rows read as key and value on the mma.sync kernel: prompt tiles (a whole prompt, a portion behind a long
    context, a short one) and single tokens, one split and several, against the float64 formula and the general
    kernel."""
    ops = _ops()
    dtype, page_size, scale = torch.bfloat16, 16, 0.05
    g = torch.Generator(device="cuda").manual_seed(13)
    for seq_q, q_tile in (([(130, 130), (400, 45), (3, 2), (65, 1)], 32), ([(257, 1), (32, 1), (1, 1), (700, 1)], 1)):
        num_pages = sum((c + page_size - 1) // page_size for c, _ in seq_q) + 2
        rows = _pages(5, num_pages, 1, page_size, row, dtype)
        order = torch.randperm(num_pages, generator=torch.Generator().manual_seed(6)).tolist()
        width = max((c + page_size - 1) // page_size for c, _ in seq_q)
        table = torch.full((len(seq_q), width), -1, dtype=torch.int32)
        for s, (c, _) in enumerate(seq_q):
            for j in range((c + page_size - 1) // page_size):
                table[s, j] = order.pop()
        total = sum(n for _, n in seq_q)
        q = torch.randn((total, heads * row), generator=g, device="cuda").to(dtype)
        common = dict(heads=heads, kv_heads=1, v_dim=v_dim, page_size=page_size, q_tile=q_tile, scale=scale, window=window)
        general = _run_scored(ops, dtype, q, rows, rows, table.cuda(), seq_q, splits=1, kernel="general", **common)
        out = _run_scored(ops, dtype, q, rows, rows, table.cuda(), seq_q, splits=splits, **common)
        torch.testing.assert_close(out.float(), general.float(), atol=6e-3, rtol=2e-2)
        at = 0
        for s, (c, n) in enumerate(seq_q):
            pages = table[s].long()[torch.arange(c) // page_size]
            k = rows.cpu()[pages, :, torch.arange(c) % page_size].double()
            want = _dense_attention(q[at:at + n].double().cpu().view(n, heads, row), k, k[..., :v_dim], first_pos=c - n,
                                    scale=scale, softcap=0.0, slopes=None, chunk=0, window=window, gate=None)
            torch.testing.assert_close(out[at:at + n].double().cpu().view(n, heads, v_dim), want, **TOL[dtype])
            at += n


@pytest.mark.parametrize("tokens,features,k", [(1, 384, 192), (8, 512, 256), (33, 200, 72), (64, 1024, 512)])
@pytest.mark.parametrize("kind", ["relu2", "gelu_tanh", "silu"])
def test_product_with_the_activation_on_its_output_tile(tokens, features, k, kind):
    """The small-batch product kernel's activation against the product followed by the activation kernel: both round
    the product to bfloat16 first, so they agree to the last bit but for the sums' order."""
    ops = _ops()
    g = torch.Generator(device="cuda").manual_seed(tokens)
    x = torch.randn((tokens, k), generator=g, device="cuda").bfloat16()
    w = (torch.randn((features, k), generator=g, device="cuda") / k ** 0.5).bfloat16()
    fused = ops.linear_activation(x, w, kind)
    plain_product = (x.double() @ w.double().T).float().bfloat16()
    want = ops.activation(plain_product, kind)
    torch.testing.assert_close(fused.float(), want.float(), atol=2e-2, rtol=2e-2)
    assert float((fused.float() - want.float()).abs().mean()) < 2e-3
