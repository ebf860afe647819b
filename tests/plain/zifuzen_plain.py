"""The Zifuzen decoder written out plainly: whole sequences, dense score matrices, Python loops over time and over
experts, one function per mechanism.  It shares nothing with the package; the tests run it in float64 (or float32)
on the weights the engine was given.

    x_0      = embed[token] * scale + pos[p]
    x       <- x + LN_1(mixer(x));   x <- x + LN_2(ff(x))          (the norm sits on each branch's output)
    logits   = cap * tanh(head(LN(x)) / cap)

``raw`` is the configuration as config.json holds it; ``w`` maps tensor names to tensors.
"""

from __future__ import annotations

import math

import torch


def layer_norm(x, weight, eps):
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * weight


def rms_unit(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def embed(tokens, w, raw):
    ids = torch.as_tensor(tokens, dtype=torch.long)
    return w["embed"][ids] * float(raw["embedding"]["scale"]) + w["pos"][: len(ids)]


def short_conv(x, taps):
    """x [T, C], taps [C, n]: y[t, c] = sum_j taps[c, j] * x[t - (n - 1) + j, c], zeros before the start."""
    T, C = x.shape
    n = taps.shape[1]
    padded = torch.cat((x.new_zeros(n - 1, C), x), dim=0)
    y = x.new_zeros(T, C)
    for j in range(n):
        y = y + padded[j:j + T] * taps[:, j]
    return y


def delta_rule(q, k, v, beta, decay):
    """One head.  q, k [T, D], v [T, V], beta, decay [T].  S starts at zero; per token: S *= decay;
    u = beta (v - S^T k); S += k u^T; o = S^T q."""
    T, D = q.shape
    S = q.new_zeros(D, v.shape[1])
    out = []
    for t in range(T):
        S = S * decay[t]
        u = beta[t] * (v[t] - S.T @ k[t])
        S = S + torch.outer(k[t], u)
        out.append(S.T @ q[t])
    return torch.stack(out)


def delta_mixer(h, w, prefix, m, eps):
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = silu(short_conv(h @ w[f"{prefix}.q"].T, w[f"{prefix}.q.conv"])).view(T, G, D)
    k = silu(short_conv(h @ w[f"{prefix}.k"].T, w[f"{prefix}.k.conv"])).view(T, G, D)
    v = silu(short_conv(h @ w[f"{prefix}.v"].T, w[f"{prefix}.v.conv"])).view(T, H, V)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[f"{prefix}.b"].T)                                      # [T, H]
    rate = torch.exp(w[f"{prefix}.A_log"])
    decay = torch.exp(-rate * torch.nn.functional.softplus(h @ w[f"{prefix}.a"].T + w[f"{prefix}.dt_bias"]))
    gate = silu(h @ w[f"{prefix}.g"].T).view(T, H, V)
    heads = []
    for i in range(H):
        j = i // (H // G)
        o = delta_rule(q[:, j], k[:, j], v[:, i], beta[:, i], decay[:, i])
        heads.append(rms_unit(o, eps) * w[f"{prefix}.norm"] * gate[:, i])
    return torch.cat(heads, dim=-1) @ w[f"{prefix}.o"].T


def attention_keys_values(h, w, prefix, m, eps):
    """What an attention layer leaves for itself and for layers that borrow from it: normed keys and values."""
    T = h.shape[0]
    G, D, V = m["kv_heads"], m["dim"], m["vdim"]
    k = rms_unit((h @ w[f"{prefix}.k"].T).view(T, G, D), eps) * w[f"{prefix}.k.norm"]
    v = (h @ w[f"{prefix}.v"].T).view(T, G, V)
    return k, v


def attention_mixer(h, w, prefix, m, eps, keys, values):
    T = h.shape[0]
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    q = rms_unit((h @ w[f"{prefix}.q"].T).view(T, H, D), eps) * w[f"{prefix}.q.norm"]
    mask = torch.ones(T, T, dtype=torch.bool).tril()
    heads = []
    for i in range(H):
        j = i // (H // G)
        s = (q[:, i] @ keys[:, j].T) * float(m["scale"])
        s = s.masked_fill(~mask, float("-inf"))
        heads.append(torch.softmax(s, dim=-1) @ values[:, j])
    return torch.cat(heads, dim=-1) @ w[f"{prefix}.o"].T


def dense_ff(h, w, prefix):
    g = h @ w[f"{prefix}.gate"].T + w[f"{prefix}.gate.b"]
    u = h @ w[f"{prefix}.up"].T + w[f"{prefix}.up.b"]
    return (gelu_tanh(g) * u) @ w[f"{prefix}.down"].T + w[f"{prefix}.down.b"]


def clamped_expert(h, w, prefix, limit):
    g = torch.clamp(h @ w[f"{prefix}.gate"].T, max=limit)
    u = torch.clamp(h @ w[f"{prefix}.up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[f"{prefix}.down"].T


def route(h, w, prefix, router, margins=None):
    """(chosen experts [T, top], their weights [T, top]).  ``margins`` (a list) receives, per token, how far the
    decision was from another one: the gap between the last kept and the first dropped group score, and between the
    last chosen and the first unchosen choice score."""
    E, top = router["experts"], router["top"]
    groups = router.get("groups") or {"count": 1, "keep": 1}
    s = torch.sigmoid(h @ w[f"{prefix}.router"].T)
    choice = s + w[f"{prefix}.correction"]
    per = E // groups["count"]
    grouped = choice.view(-1, groups["count"], per)
    group_score = grouped.topk(min(2, per), dim=-1).values.sum(-1)
    kept = group_score.topk(groups["keep"], dim=-1).indices
    allowed = torch.zeros_like(group_score, dtype=torch.bool).scatter_(1, kept, True)
    masked = torch.where(allowed.unsqueeze(-1).expand_as(grouped), grouped, torch.full_like(grouped, float("-inf")))
    ranked = masked.reshape(-1, E).sort(dim=-1, descending=True)
    chosen = ranked.indices[:, :top]
    if margins is not None:
        gap = torch.full((h.shape[0],), float("inf"), dtype=h.dtype)
        if groups["keep"] < groups["count"]:
            by_group = group_score.sort(dim=-1, descending=True).values
            gap = torch.minimum(gap, by_group[:, groups["keep"] - 1] - by_group[:, groups["keep"]])
        if top < E:
            gap = torch.minimum(gap, ranked.values[:, top - 1] - ranked.values[:, top])
        margins.append(gap)
    picked = s.gather(1, chosen)
    weights = picked / (picked.sum(-1, keepdim=True) + 1e-20) * float(router["scale"])
    return chosen, weights


def moe_ff(h, w, prefix, mlp, margins=None):
    chosen, weights = route(h, w, prefix, mlp["router"], margins)
    out = torch.zeros(h.shape[0], w[f"{prefix}.e0.down"].shape[0], dtype=h.dtype)
    limit = float(mlp["expert"]["limit"])
    for slot in range(chosen.shape[1]):             # a token's choices are added in their order
        for e in range(mlp["router"]["experts"]):
            rows = (chosen[:, slot] == e).nonzero().flatten()
            if len(rows):
                out[rows] = out[rows] + weights[rows, slot, None] * clamped_expert(h[rows], w, f"{prefix}.e{e}", limit)
    if mlp.get("shared"):
        out = out + clamped_expert(h, w, f"{prefix}.shared", float(mlp["shared"]["limit"]))
    return out


def forward(raw, w, tokens, return_layers=False, margins=None):
    """Logits [T, vocab] of one whole sequence (and the residual stream after every layer).  ``margins``: see
    :func:`route`; one entry per routed layer."""
    eps = float(raw["norm"]["eps"])
    x = embed(tokens, w, raw)
    kept = {}
    after = []
    for i, layer in enumerate(raw["layers"]):
        m, p = layer["mixer"], f"l{i}.mix"
        if layer["type"] == "attention":
            if m.get("kv_from") is None:
                kept[i] = attention_keys_values(x, w, p, m, eps)
            keys, values = kept[m["kv_from"] if m.get("kv_from") is not None else i]
            branch = attention_mixer(x, w, p, m, eps, keys, values)
        else:
            branch = delta_mixer(x, w, p, m, eps)
        x = x + layer_norm(branch, w[f"l{i}.norm1"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            branch = dense_ff(x, w, f"l{i}.mlp") if mlp.get("kind", "dense") == "dense" else \
                moe_ff(x, w, f"l{i}.mlp", mlp, margins)
            x = x + layer_norm(branch, w[f"l{i}.norm2"], eps)
        after.append(x)
    logits = layer_norm(x, w["final.norm"], eps) @ w["head"].T
    cap = raw.get("logit_softcap")
    if cap:
        logits = float(cap) * torch.tanh(logits / float(cap))
    return (logits, torch.stack(after)) if return_layers else logits


def greedy_generate(raw, w, prompt, new_tokens):
    ids = list(prompt)
    for _ in range(new_tokens):
        ids.append(int(forward(raw, w, ids)[-1].argmax()))
    return ids[len(prompt):]
