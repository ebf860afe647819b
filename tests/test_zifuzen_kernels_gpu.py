"""Each kernel of the Zifuzen path alone, against the plain functions: the embedding with a scale and position rows,
both LayerNorm forms, the gated activations, the logit cap, the q/k norm with learned weights, the delta rule's two
kernels (prompts against token-by-token, portions, slots that are used again, padding, a key far back that alone
decides the output), and the routed experts' five kernels (groups, negative scores, ties, empty experts, experts with
more rows than a tile)."""

import math

import pytest
import torch

from plain import zifuzen_plain as plain

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def _ops():
    from ampere_kv_engine_b200.kernels import ops
    return ops


def _tol(dtype):
    return dict(atol=2e-5, rtol=2e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)


def _gen(seed):
    return torch.Generator(device="cuda").manual_seed(seed)


def _randn(*shape, seed=0, dtype=torch.float32, scale=1.0):
    return (torch.randn(*shape, generator=_gen(seed), device="cuda") * scale).to(dtype)


def _i32(values):
    return torch.tensor(values, dtype=torch.int32, device="cuda")


# ----------------------------------------------------------------------------- row-wise kernels


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_scales_the_row_and_adds_the_position_row(dtype):
    ops = _ops()
    table, rows = _randn(37, 50, seed=1, dtype=dtype), _randn(64, 50, seed=2, dtype=dtype)
    ids, positions = _i32([3, 36, 0, 3, 9]), _i32([0, 63, 5, 6, 1])
    got = ops.embedding(ids, table, scale=2.5, positions=positions, position_rows=rows)
    want = table.float()[ids.long()] * 2.5 + rows.float()[positions.long()]
    torch.testing.assert_close(got, want, atol=1e-6, rtol=1e-6)
    torch.testing.assert_close(ops.embedding(ids, table, scale=0.5), table.float()[ids.long()] * 0.5, atol=0, rtol=0)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops.embedding(ids, table, status=status, scale=1.0, positions=_i32([0, 64, 0, 0, 0]), position_rows=rows)
    assert int(status.item()) != 0        # a position beyond the table is reported, not read


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [72, 256, 1000])
def test_layernorm_forms(dtype, width):
    ops = _ops()
    eps = 1e-5
    weight = 1.0 + 0.1 * _randn(width, seed=3)
    hidden = _randn(9, width, seed=4) * 3.0 + 40.0          # a mean far from zero: the variance is about deviations
    want = plain.layer_norm(hidden.double(), weight.double(), eps)
    got = ops.add_layernorm(hidden.clone(), None, weight, eps, dtype)
    torch.testing.assert_close(got.double(), want, **(_tol(dtype) if dtype != torch.float32 else dict(atol=5e-5, rtol=5e-5)))
    rows = _i32([8, 0, 3])
    got = ops.add_layernorm(hidden.clone(), None, weight, eps, dtype, rows=rows)
    torch.testing.assert_close(got.double(), want[rows.long()], **(_tol(dtype) if dtype != torch.float32 else dict(atol=5e-5, rtol=5e-5)))
    delta = _randn(9, width, seed=5, dtype=dtype)
    stream = hidden.clone()
    got = ops.add_layernorm(stream, delta, weight, eps, dtype)
    torch.testing.assert_close(stream, hidden + delta.float(), atol=1e-6, rtol=1e-6)
    torch.testing.assert_close(got.double(), plain.layer_norm((hidden + delta.float()).double(), weight.double(), eps),
                               **(_tol(dtype) if dtype != torch.float32 else dict(atol=5e-5, rtol=5e-5)))
    # the norm on a branch's output: what joins the stream is the normed branch
    for branch in (_randn(9, width, seed=6, dtype=dtype) * 5 + 2, _randn(9, width, seed=7) * 0.01):
        stream = hidden.clone()
        copy = ops.branch_layernorm(stream, branch, weight, eps, dtype)
        want_stream = hidden.double() + plain.layer_norm(branch.double(), weight.double(), eps)
        torch.testing.assert_close(stream.double(), want_stream, atol=2e-5, rtol=2e-6)
        if dtype == torch.float32:
            assert copy is stream
        else:
            torch.testing.assert_close(copy, stream.to(dtype), atol=0, rtol=0)
    if dtype == torch.bfloat16:
        torch.testing.assert_close(ops.stream_copy(hidden, dtype), hidden.to(dtype), atol=0, rtol=0)
    else:
        assert ops.stream_copy(hidden, dtype) is hidden


@pytest.mark.parametrize("dtype", DTYPES)
def test_gated_activations(dtype):
    ops = _ops()
    both = _randn(7, 2 * 48, seed=8, dtype=dtype) * 4.0           # beyond the clamps below
    g, u = both.double()[:, :48], both.double()[:, 48:]
    want = plain.gelu_tanh(g) * u
    torch.testing.assert_close(ops.glu(both, "gelu_tanh").double(), want, **_tol(dtype))
    limit = 1.25
    gc, uc = g.clamp(max=limit), u.clamp(min=-limit, max=limit)
    want = gc * torch.sigmoid(1.702 * gc) * (uc + 1.0)
    torch.testing.assert_close(ops.glu(both, "clamped_swish", 0, limit, 1.702).double(), want, **_tol(dtype))
    # gate and up columns in alternating runs of 16
    pairs = both.view(7, 3, 2, 16)
    g, u = pairs[:, :, 0].reshape(7, 48).double(), pairs[:, :, 1].reshape(7, 48).double()
    torch.testing.assert_close(ops.glu(both, "gelu_tanh", 16).double(), plain.gelu_tanh(g) * u, **_tol(dtype))
    torch.testing.assert_close(ops.glu(both, "silu", 16).double(), plain.silu(g) * u, **_tol(dtype))


def test_logit_cap():
    ops = _ops()
    logits = _randn(5, 333, seed=9) * 40.0
    want = 30.0 * torch.tanh(logits.double() / 30.0)
    torch.testing.assert_close(ops.softcap_(logits.clone(), 30.0).double(), want, atol=1e-5, rtol=1e-6)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("has_kv", [True, False])
def test_head_prep_with_learned_norm_weights(dtype, has_kv):
    ops = _ops()
    H, G, D, V, n, page = 4, 2, 48, 24, 6, 4
    eps = 1e-6
    width = H * D + (G * (D + V) if has_kv else 0)
    x = _randn(n, width, seed=10, dtype=dtype)
    qw, kw = 1.0 + 0.3 * _randn(D, seed=11), 1.0 + 0.3 * _randn(D, seed=12)
    k_cache = torch.zeros(5, G, page, D, dtype=dtype, device="cuda") if has_kv else None
    v_cache = torch.zeros(5, G, page, V, dtype=dtype, device="cuda") if has_kv else None
    slots = _i32([4, 5, 6, 7, 17, 0]) if has_kv else None
    q, gate = ops.head_prep(x, slots, k_cache, v_cache, num_heads=H, num_kv_heads=G, head_dim=D, v_dim=V,
                            unit_norm=True, eps=eps, gated=False, q_weight=qw, k_weight=kw if has_kv else None,
                            has_kv=has_kv)
    assert gate is None
    xd = x.double()
    want_q = plain.rms_unit(xd[:, :H * D].view(n, H, D), eps) * qw.double()
    torch.testing.assert_close(q.double().view(n, H, D), want_q, **_tol(dtype))
    if has_kv:
        want_k = plain.rms_unit(xd[:, H * D:H * D + G * D].view(n, G, D), eps) * kw.double()
        want_v = xd[:, H * D + G * D:].view(n, G, V)
        s = slots.long()
        torch.testing.assert_close(k_cache[s // page, :, s % page].double(), want_k, **_tol(dtype))
        torch.testing.assert_close(v_cache[s // page, :, s % page].double(), want_v, **_tol(dtype))


# ----------------------------------------------------------------------------- the delta rule


def _delta_inputs(H, G, D, V, taps, tokens, dtype, seed):
    channels = 2 * G * D + H * V
    x = _randn(tokens, channels + H * V + 2 * H, seed=seed, dtype=dtype)
    conv = _randn(channels, taps, seed=seed + 1) * 0.5
    rate_log = torch.empty(H, device="cuda").uniform_(-4.0, -0.5, generator=_gen(seed + 2))
    step_bias = _randn(H, seed=seed + 3) * 0.3
    norm_w = 1.0 + 0.2 * _randn(V, seed=seed + 4)
    return x, conv, rate_log, step_bias, norm_w


def _delta_plain(x, conv, rate_log, step_bias, norm_w, H, G, D, V, eps):
    """The mixer between its two products, one whole sequence, float64."""
    xd = x.double().cpu()
    conv, rate_log, step_bias, norm_w = conv.double().cpu(), rate_log.double().cpu(), step_bias.double().cpu(), norm_w.double().cpu()
    T = xd.shape[0]
    c = 2 * G * D + H * V
    y = plain.silu(plain.short_conv(xd[:, :c], conv))
    q, k, v = y[:, :G * D].view(T, G, D), y[:, G * D:2 * G * D].view(T, G, D), y[:, 2 * G * D:].view(T, H, V)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    gate = plain.silu(xd[:, c:c + H * V]).view(T, H, V)
    beta = torch.sigmoid(xd[:, c + H * V:c + H * V + H])
    decay = torch.exp(-torch.exp(rate_log) * torch.nn.functional.softplus(xd[:, c + H * V + H:] + step_bias))
    heads = []
    for h in range(H):
        o = plain.delta_rule(q[:, h // (H // G)], k[:, h // (H // G)], v[:, h], beta[:, h], decay[:, h])
        heads.append(plain.rms_unit(o, eps) * norm_w * gate[:, h])
    return torch.cat(heads, dim=-1)


def _delta_run(ops, x, conv, rate_log, step_bias, norm_w, state, cuts, slot, sizes, eps, others=()):
    """Feed x in portions of the given sizes for the sequence in ``slot``; ``others`` are (rows, slot) of further
    sequences that share every step (their outputs are dropped).  Returns the outputs of all portions."""
    outs, p = [], 0
    for n in cuts:
        rows = [x[p:p + n]] + [o[0] for o in others]
        slots = [slot] + [o[1] for o in others]
        batch = torch.cat(rows, dim=0)
        cu = [0]
        for r in rows:
            cu.append(cu[-1] + r.shape[0])
        qkv, coef = ops.delta_prep(batch, conv, rate_log, step_bias, state, _i32(cu), _i32(slots), unit_eps=1e-6, **sizes)
        out = ops.delta_scan(qkv, coef, batch, norm_w, state, _i32(cu), _i32(slots), norm_eps=eps, **sizes)
        outs.append(out[:n])
        p += n
    return torch.cat(outs, dim=0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,D,V,taps", [(2, 1, 64, 32, 4), (6, 6, 64, 32, 3), (3, 3, 16, 20, 2), (4, 2, 128, 128, 4),
                                          (2, 1, 24, 8, 1), (2, 2, 256, 64, 2), (4, 1, 40, 256, 5), (1, 1, 8, 1, 8),
                                          (2, 1, 32, 16, 12)])
def test_delta_rule_prompt_portions_and_single_tokens_agree_with_the_plain_recurrence(dtype, H, G, D, V, taps):
    ops = _ops()
    eps, T = 1e-6, 45
    sizes = dict(num_heads=H, num_kv_heads=G, head_dim=D, v_dim=V, taps=taps)
    x, conv, rate_log, step_bias, norm_w = _delta_inputs(H, G, D, V, taps, T, dtype, seed=20)
    want = _delta_plain(x, conv, rate_log, step_bias, norm_w, H, G, D, V, eps)
    width = ops.delta_state_floats(H, G, D, V, taps)[1]
    tol = dict(atol=3e-5, rtol=3e-4) if dtype == torch.float32 else dict(atol=3e-2, rtol=3e-2)
    results = []
    for cuts, slot in (((T,), 2), ((1,) * T, 0), ((7, 2, 1, 13, 2, 1, 1, 16, 2), 1), ((44, 1), 2)):
        state = torch.full((3, width), float("nan"), device="cuda")
        state[slot] = 0.0                                   # a slot is zeroed when a request opens; the others are not its business
        got = _delta_run(ops, x, conv, rate_log, step_bias, norm_w, state, cuts, slot, sizes, eps)
        torch.testing.assert_close(got.double().cpu(), want, **tol)
        results.append((got, state[slot].clone()))
    # however the tokens were cut, the memory after the last one is the same up to rounding
    for got, memory in results[1:]:
        torch.testing.assert_close(memory, results[0][1], atol=2e-5, rtol=1e-4)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("lens", [[1, 19, 6, 4], [1, 5, 1, 1], [2, 3, 1, 2]])
def test_delta_rule_in_a_batch_of_unequal_sequences_with_padding(dtype, lens):
    """Three sequences (of 1, 19 and 6 rows; or of so few rows that the step counts as decoding and is staged two
    tokens at a time) and a padded one share a step; each result equals the sequence alone, the padded sequence's rows
    are zero and no slot but the three is written."""
    ops = _ops()
    H, G, D, V, taps, eps = 4, 2, 32, 16, 3, 1e-5
    sizes = dict(num_heads=H, num_kv_heads=G, head_dim=D, v_dim=V, taps=taps)
    width = ops.delta_state_floats(H, G, D, V, taps)[1]
    inputs = _delta_inputs(H, G, D, V, taps, 30, dtype, seed=30)
    x, rest = inputs[0], inputs[1:]
    slots = [3, 0, 2, -1]
    state = torch.zeros(5, width, device="cuda")
    state[1] = 5.0
    state[4] = -3.0
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    x = x[:cu[-1]].contiguous()
    qkv, coef = ops.delta_prep(x, rest[0], rest[1], rest[2], state, _i32(cu), _i32(slots), unit_eps=1e-6, **sizes)
    out = ops.delta_scan(qkv, coef, x, rest[3], state, _i32(cu), _i32(slots), norm_eps=eps, **sizes)
    tol = dict(atol=3e-5, rtol=3e-4) if dtype == torch.float32 else dict(atol=3e-2, rtol=3e-2)
    for i in range(3):
        want = _delta_plain(x[cu[i]:cu[i + 1]], *rest, H, G, D, V, eps)
        torch.testing.assert_close(out[cu[i]:cu[i + 1]].double().cpu(), want, **tol)
    assert float(out[cu[3]:].float().abs().max()) == 0.0
    assert bool((state[1] == 5.0).all()) and bool((state[4] == -3.0).all())


def test_delta_rule_keeps_a_key_from_far_back():
    """Decay one, beta one: a value written under a key at token 5 comes back whole 600 tokens later when the query
    is that key, while all keys in between are orthogonal to it; and with a decay below one it has faded by exactly
    the product of the decays."""
    ops = _ops()
    H = G = 1
    D, V, T = 64, 32, 606
    sizes = dict(num_heads=H, num_kv_heads=G, head_dim=D, v_dim=V, taps=1)
    g = _gen(40)
    k = torch.randn(T, D, generator=g, device="cuda")
    k[:, 0] = 0.0
    k = k / k.norm(dim=-1, keepdim=True)
    k[5] = 0.0
    k[5, 0] = 1.0
    q = k.clone() * D ** -0.5
    q[-1] = 0.0
    q[-1, 0] = D ** -0.5
    v = torch.randn(T, V, generator=g, device="cuda")
    qkv = torch.cat((q, k, v), dim=1).contiguous()
    x = torch.zeros(T, 2 * D + V + V + 2, device="cuda")         # gate columns zero: silu(0) = 0 would hide the output
    x[:, 2 * D + V:2 * D + 2 * V] = 4.0
    norm_w = torch.ones(V, device="cuda")
    for decay in (1.0, 0.995):
        coef = torch.tensor([[1.0, decay]], device="cuda").repeat(T, 1).contiguous()
        state = torch.zeros(1, ops.delta_state_floats(H, G, D, V, 1)[1], device="cuda")
        out = ops.delta_scan(qkv, coef, x, norm_w, state, _i32([0, T]), _i32([0]), norm_eps=1e-12, **sizes)
        raw_want = v[5].double() * D ** -0.5 * decay ** (T - 1 - 5)
        want = plain.rms_unit(raw_want, 1e-12) * plain.silu(torch.tensor(4.0, dtype=torch.float64))
        torch.testing.assert_close(out[-1].double(), want.cuda(), atol=1e-4, rtol=1e-4)
    # the same in two steps: the memory carried in the state slot holds the far key
    state = torch.zeros(2, ops.delta_state_floats(H, G, D, V, 1)[1], device="cuda")
    coef = torch.tensor([[1.0, 1.0]], device="cuda").repeat(T, 1).contiguous()
    ops.delta_scan(qkv[:300].contiguous(), coef[:300].contiguous(), x[:300].contiguous(), norm_w, state, _i32([0, 300]),
                   _i32([1]), norm_eps=1e-12, **sizes)
    out = ops.delta_scan(qkv[300:].contiguous(), coef[300:].contiguous(), x[300:].contiguous(), norm_w, state,
                         _i32([0, T - 300]), _i32([1]), norm_eps=1e-12, **sizes)
    want = plain.rms_unit(v[5].double() * D ** -0.5, 1e-12) * plain.silu(torch.tensor(4.0, dtype=torch.float64))
    torch.testing.assert_close(out[-1].double(), want.cuda(), atol=1e-4, rtol=1e-4)


def test_convolution_sees_exactly_its_taps_across_a_step_border():
    """An impulse in one channel reaches exactly the next taps - 1 tokens, whether or not a step ends in between."""
    ops = _ops()
    H, G, D, V, taps = 1, 1, 8, 8, 4
    sizes = dict(num_heads=H, num_kv_heads=G, head_dim=D, v_dim=V, taps=taps)
    channels = 2 * D + V
    T = 12
    x = torch.zeros(T, channels + V + 2, device="cuda")
    x[3, 2 * D + 1] = 2.0                                         # a value channel at token 3
    conv = torch.zeros(channels, taps, device="cuda")
    conv[2 * D + 1] = torch.tensor([0.5, -1.0, 2.0, 1.0])         # last tap: the current token
    zeros = torch.zeros(H, device="cuda")
    for cuts in ((T,), (4, 8), (5, 1, 6), (3, 1, 1, 1, 1, 5)):
        state = torch.zeros(1, ops.delta_state_floats(H, G, D, V, taps)[1], device="cuda")
        got, p = [], 0
        for n in cuts:
            qkv, _ = ops.delta_prep(x[p:p + n].contiguous(), conv, zeros, zeros, state, _i32([0, n]), _i32([0]),
                                    unit_eps=1e-6, **sizes)
            out = ops.delta_scan(qkv, torch.zeros(n, 2, device="cuda"), x[p:p + n].contiguous(),
                                 torch.ones(V, device="cuda"), state, _i32([0, n]), _i32([0]), norm_eps=1e-6, **sizes)
            got.append(qkv[:, 2 * D + 1])
            p += n
        got = torch.cat(got).cpu()
        pre = torch.tensor([0, 0, 0, 2.0 * 1.0, 2.0 * 2.0, 2.0 * -1.0, 2.0 * 0.5, 0, 0, 0, 0, 0], dtype=torch.float64)
        torch.testing.assert_close(got.double(), plain.silu(pre), atol=1e-6, rtol=1e-6)


# ----------------------------------------------------------------------------- routed experts


def _route_plain(logits, correction, top, groups, keep, scale):
    w = {"p.router": torch.eye(logits.shape[1], dtype=torch.float64), "p.correction": correction.double().cpu()}
    router = {"experts": logits.shape[1], "top": top, "scale": scale, "groups": {"count": groups, "keep": keep}}
    # the plain router sees logits as W h with W the identity
    return plain.route(logits.double().cpu(), w, "p", router)


@pytest.mark.parametrize("experts,top,groups,keep", [(12, 2, 3, 2), (8, 4, 2, 1), (5, 1, 1, 1), (64, 6, 8, 3),
                                                     (256, 8, 8, 4), (6, 6, 1, 1), (48, 3, 48, 5)])
def test_route_follows_the_plain_router(experts, top, groups, keep):
    ops = _ops()
    logits = _randn(301, experts, seed=50) * 2.0
    correction = _randn(experts, seed=51) * 0.4
    chosen, weights = ops.moe_route(logits, correction, top=top, groups=groups, keep_groups=keep, group_top=2,
                                    scale=1.7, weight_eps=1e-20)
    want_ids, want_w = _route_plain(logits, correction, top, groups, keep, 1.7)
    assert chosen.cpu().long().tolist() == want_ids.tolist()
    torch.testing.assert_close(weights.double().cpu(), want_w, atol=1e-6, rtol=1e-5)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tokens,experts,width", [(1, 12, 256), (8, 64, 1000), (64, 5, 72), (3, 7, 33), (70, 6, 48)])
def test_router_logits(dtype, tokens, experts, width):
    ops = _ops()
    x, w = _randn(tokens, width, seed=55, dtype=dtype), _randn(experts, width, seed=56, dtype=dtype)
    got = ops.moe_router_logits(x, w)
    assert got.dtype == torch.float32
    torch.testing.assert_close(got.double(), x.double() @ w.double().T, atol=2e-4, rtol=1e-5)


def test_route_engineered_cases():
    ops = _ops()
    kw = dict(group_top=2, scale=1.0, weight_eps=1e-20)
    # every choice score is negative: an expert of a dropped group must count as minus infinity, not as zero
    logits = torch.tensor([[-3.0, -2.0, -1.0, -2.5, 0.5, 0.4]], device="cuda")
    correction = torch.full((6,), -2.0, device="cuda")
    chosen, weights = ops.moe_route(logits, correction, top=2, groups=3, keep_groups=1, **kw)
    assert sorted(chosen[0].tolist()) == [4, 5]
    chosen, _ = ops.moe_route(torch.tensor([[-3.0, -2.0, -1.0, -2.5, -9.0, -9.0]], device="cuda"), correction, top=2,
                              groups=3, keep_groups=1, **kw)
    assert sorted(chosen[0].tolist()) == [2, 3]
    # a group's score is the sum of its two best: one very large expert does not beat two good ones
    sig = lambda p: math.log(p / (1 - p))
    logits = torch.tensor([[sig(0.95), sig(0.05), sig(0.05), sig(0.6), sig(0.6), sig(0.05)]], device="cuda")
    chosen, weights = ops.moe_route(logits, None, top=1, groups=2, keep_groups=1, **kw)
    assert chosen[0].tolist() == [3]                          # 0.6 + 0.6 beats 0.95 + 0.05; ties go to the lower index
    assert abs(float(weights[0, 0]) - 1.0) < 1e-6
    # the correction decides the choice but not the weight
    logits = torch.tensor([[sig(0.2), sig(0.7), sig(0.6)]], device="cuda")
    correction = torch.tensor([0.9, 0.0, 0.2], device="cuda")
    chosen, weights = ops.moe_route(logits, correction, top=2, groups=1, keep_groups=1, group_top=2, scale=3.0,
                                    weight_eps=1e-20)
    assert chosen[0].tolist() == [0, 2]
    torch.testing.assert_close(weights[0].cpu(), torch.tensor([0.2, 0.6]) / 0.8 * 3.0, atol=1e-6, rtol=1e-6)
    # rows that hold anything at all (padding of a captured step) still choose experts that exist
    logits = torch.full((3, 12), float("nan"), device="cuda")
    logits[1] = float("inf")
    chosen, _ = ops.moe_route(logits, torch.zeros(12, device="cuda"), top=2, groups=3, keep_groups=2, **kw)
    assert bool(((chosen >= 0) & (chosen < 12)).all())


def test_sort_by_expert():
    ops = _ops()
    experts, top = 7, 3
    chosen = torch.randint(0, experts, (250, top), generator=_gen(60), device="cuda", dtype=torch.int32)
    chosen[chosen == 4] = 5                                   # an expert nobody chose
    order, offsets = ops.moe_sort(chosen, experts)
    flat, order, offsets = chosen.reshape(-1).cpu(), order.cpu().long(), offsets.cpu().tolist()
    assert sorted(order.tolist()) == list(range(250 * top))
    assert offsets[0] == 0 and offsets[-1] == 250 * top and offsets[4] == offsets[5]
    for e in range(experts):
        assert bool((flat[order[offsets[e]:offsets[e + 1]]] == e).all())


@pytest.mark.parametrize("dtype,kernel", [(torch.float32, "auto"), (torch.bfloat16, "auto"), (torch.bfloat16, "plain"),
                                          (torch.bfloat16, "mma"), (torch.bfloat16, "few")])
@pytest.mark.parametrize("tokens,width,inter,experts,top", [(70, 72, 40, 6, 2), (3, 48, 16, 8, 4), (150, 256, 64, 3, 1),
                                                            (1, 100, 33, 5, 2), (450, 136, 200, 2, 2)])
def test_expert_products_and_sum(dtype, kernel, tokens, width, inter, experts, top):
    ops = _ops()
    if kernel in ("mma", "few") and width % 8:
        pytest.skip("the tensor-core and few-rows forms take hidden sizes that are multiples of eight")
    limit, slope = 1.5, 1.702
    x = _randn(tokens, width, seed=70, dtype=dtype)
    w_gu = _randn(experts, 2 * inter, width, seed=71, dtype=dtype, scale=0.3)
    w_d = _randn(experts, width, inter, seed=72, dtype=dtype, scale=0.3)
    chosen = torch.stack([torch.randperm(experts, generator=_gen(73 + t), device="cuda")[:top] for t in range(tokens)]
                         ).to(torch.int32)
    if experts > 2:
        chosen[chosen == 1] = 0 if top == 1 else chosen[chosen == 1]          # top 1: expert 1 stays empty
    weights = torch.rand(tokens, top, generator=_gen(74), device="cuda") + 0.1
    shared = _randn(tokens, width, seed=75, dtype=dtype)
    order, offsets = ops.moe_sort(chosen, experts)
    act = ops.moe_gate_up(x, w_gu, order, offsets, top=top, limit=limit, slope=slope, kernel=kernel)
    parts = ops.moe_down(act, w_d, order, offsets, weights, kernel=kernel)
    got = ops.moe_combine(parts, shared, top=top)
    xd, wg, wd = x.double().cpu(), w_gu.double().cpu(), w_d.double().cpu()
    want = shared.double().cpu().clone()
    acts = {}
    for t in range(tokens):
        for s in range(top):
            e = int(chosen[t, s])
            g = (xd[t] @ wg[e, :inter].T).clamp(max=limit)
            u = (xd[t] @ wg[e, inter:].T).clamp(min=-limit, max=limit)
            a = g * torch.sigmoid(slope * g) * (u + 1.0)
            acts[t * top + s] = a
            if dtype == torch.bfloat16:
                a = a.to(torch.bfloat16).double()              # the activations are stored in the compute dtype
            want[t] += float(weights[t, s]) * (a @ wd[e].T)
    tol = dict(atol=1e-4, rtol=1e-4) if dtype == torch.float32 else dict(atol=3e-2, rtol=2e-2)
    order = order.cpu().tolist()
    got_act = act.double().cpu()
    for r, pair in enumerate(order):
        torch.testing.assert_close(got_act[r], acts[pair], **tol)
    torch.testing.assert_close(got.double().cpu(), want, **(tol if dtype == torch.float32 else dict(atol=8e-2, rtol=3e-2)))
    torch.testing.assert_close(ops.moe_combine(parts, None, top=top).double().cpu(), want - shared.double().cpu(),
                               **(tol if dtype == torch.float32 else dict(atol=8e-2, rtol=3e-2)))


@pytest.mark.parametrize("kernel", ["mma", "few", "plain"])
def test_a_row_of_the_expert_products_does_not_depend_on_the_rest_of_the_batch(kernel):
    """The same token alone and among 99 others: bit-equal results within each form of the products (its dot products
    are accumulated in one order whatever tile or row group it falls in), and equal up to the order of the sums
    between the forms, which the size of a step chooses."""
    ops = _ops()
    width, inter, experts, top = 96, 48, 4, 2
    x = _randn(100, width, seed=80, dtype=torch.bfloat16)
    w_gu = _randn(experts, 2 * inter, width, seed=81, dtype=torch.bfloat16, scale=0.3)
    w_d = _randn(experts, width, inter, seed=82, dtype=torch.bfloat16, scale=0.3)
    chosen = torch.stack([torch.randperm(experts, generator=_gen(83 + t), device="cuda")[:top] for t in range(100)]
                         ).to(torch.int32)
    weights = torch.rand(100, top, generator=_gen(84), device="cuda")

    def run(rows, form):
        order, offsets = ops.moe_sort(chosen[rows].contiguous(), experts)
        act = ops.moe_gate_up(x[rows].contiguous(), w_gu, order, offsets, top=top, limit=2.0, slope=1.702, kernel=form)
        return ops.moe_combine(ops.moe_down(act, w_d, order, offsets, weights[rows].contiguous(), kernel=form), None,
                               top=top)

    everyone = run(slice(0, 100), kernel)
    by_size = run(slice(0, 100), "auto")
    for t in (0, 37, 99):
        torch.testing.assert_close(run(slice(t, t + 1), kernel)[0], everyone[t], atol=0, rtol=0)
        torch.testing.assert_close(run(slice(t, t + 1), "auto")[0], by_size[t], atol=2e-6, rtol=2e-5)
