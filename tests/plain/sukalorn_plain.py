"""Plain, slow Sukalorn decoder: whole sequences, no cache, one function per mechanism.

The oracle of the Sukalorn tests.  It shares no code with the package: it reads a ``dict`` of
tensors keyed by checkpoint name and the ``dict`` of config.json, works on one whole sequence
at a time with dense [T, T] score matrices, and runs in the dtype of the tensors it is given
(the tests hand it float64 or float32 copies).

The design in short.  The stream starts as the normed embedding row.  A layer is
``x += mixer(norm(x)); x += ff(norm(x))`` (the feed-forward may be absent); norms are RMS
norms whose stored weight w stands for ``1 + w``.  Two mixers:

* ``attention``: grouped queries over keys and values of different widths; q and k are scaled
  to unit RMS per head (no weight); scores are scaled, squashed by ``cap * tanh(s / cap)``
  and lowered by ``slope_h * (i - j)``; token i sees j <= i inside its own block of
  ``mask.size`` positions; values may be blended with the values the first blending layer
  computed for the same token; each head's output is scaled by a sigmoid gate read from the
  mixer's input.
* ``latent_attention``: queries through a normed low-rank latent; keys and values from a
  normed low-rank latent c (the only thing a cache would keep, beside one rotated key part
  shared by all heads); interleaved rotary positions on the rotated parts; causal softmax.
"""

from __future__ import annotations

import math

import torch


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last dim."""
    return x / torch.sqrt(x.square().mean(dim=-1, keepdim=True) + eps)


def norm_around_zero(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """RMS norm whose weight is stored around zero: unit RMS times (1 + w)."""
    return rms_unit(x, eps) * (1.0 + w)


def norm_plain(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """RMS norm with a plain weight."""
    return rms_unit(x, eps) * w


def relu_squared(z: torch.Tensor) -> torch.Tensor:
    return torch.relu(z).square()


def dense_feed_forward(h: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    return relu_squared(h @ up.T) @ down.T


def rotate_interleaved(x: torch.Tensor, positions: torch.Tensor, base: float, dims: int) -> torch.Tensor:
    """Rotary positions on the first ``dims`` dims of the last axis, dimension 2i paired with 2i + 1.
    x: [T, ..., D]; positions: [T]."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    freq = torch.tensor(base, dtype=torch.float64) ** (-2.0 * i / dims)
    angle = positions.to(torch.float64)[:, None] * freq[None, :]                 # [T, dims / 2]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [dims // 2]
    cos, sin = angle.cos().to(x.dtype).view(shape), angle.sin().to(x.dtype).view(shape)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


def distance_slopes(heads: int) -> torch.Tensor:
    """slope_h = 2 ** (-8 (h + 1) / H)."""
    return torch.tensor([2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads)], dtype=torch.float64)


def block_causal_mask(length: int, block: int | None) -> torch.Tensor:
    """[T, T] bool: i sees j iff j <= i and (no block size, or both lie in the same block of positions)."""
    i = torch.arange(length)[:, None]
    j = torch.arange(length)[None, :]
    mask = j <= i
    if block:
        mask &= (i // block) == (j // block)
    return mask


def masked_softmax(scores: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    return torch.softmax(scores.masked_fill(~mask, -math.inf), dim=-1)


def gated_capped_attention(h: torch.Tensor, w: dict, cfg: dict, eps: float, v_first: torch.Tensor | None):
    """Mixer ``attention``.  h: [T, width]; w: local tensor names ('q', 'k', 'v', 'vmix', 'g', 'o').
    Returns (output [T, width], this layer's own unblended values [T, G, vdim])."""
    T = h.shape[0]
    H, G, D, Dv = cfg["heads"], cfg["kv_heads"], cfg["dim"], cfg["vdim"]
    q = rms_unit((h @ w["q"].T).view(T, H, D), eps)
    k = rms_unit((h @ w["k"].T).view(T, G, D), eps)
    v_own = (h @ w["v"].T).view(T, G, Dv)
    v = v_own
    if cfg.get("v_mix") and v_first is not None:
        lam = w["vmix"]
        v = (1.0 - lam) * v_own + lam * v_first
    per = H // G
    kh = k.repeat_interleave(per, dim=1)                       # query head h reads key/value head h // per
    vh = v.repeat_interleave(per, dim=1)
    s = torch.einsum("ihd,jhd->hij", q, kh) * cfg["scale"]
    cap = cfg.get("softcap")
    if cap:
        s = cap * torch.tanh(s / cap)
    dist = (torch.arange(T)[:, None] - torch.arange(T)[None, :]).to(h.dtype)
    s = s - distance_slopes(H).to(h.dtype)[:, None, None] * dist[None]
    size = (cfg.get("mask") or {}).get("size")
    p = masked_softmax(s, block_causal_mask(T, size)[None])
    out = torch.einsum("hij,jhd->ihd", p, vh)
    gate = torch.sigmoid(h @ w["g"].T)                         # [T, H]
    out = out * gate[:, :, None]
    return out.reshape(T, H * Dv) @ w["o"].T, v_own


def latent_attention(h: torch.Tensor, w: dict, cfg: dict, eps: float) -> torch.Tensor:
    """Mixer ``latent_attention``.  w: 'dq', 'dq.norm', 'uq', 'dkv', 'dkv.norm', 'uk', 'uv', 'o'."""
    T = h.shape[0]
    H, D, R, Dv, rank = cfg["heads"], cfg["dim"], cfg["rot_dim"], cfg["vdim"], cfg["kv_rank"]
    pos = torch.arange(T)
    rot = cfg["rot"]
    q = (norm_plain(h @ w["dq"].T, w["dq.norm"], eps) @ w["uq"].T).view(T, H, D + R)
    q_plain, q_rot = q[..., :D], rotate_interleaved(q[..., D:], pos, rot["base"], rot["dims"])
    down = h @ w["dkv"].T
    c = norm_plain(down[:, :rank], w["dkv.norm"], eps)
    k_rot = rotate_interleaved(down[:, rank:], pos, rot["base"], rot["dims"])          # [T, R], shared by the heads
    k_plain = (c @ w["uk"].T).view(T, H, D)
    v = (c @ w["uv"].T).view(T, H, Dv)
    s = (torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihr,jr->hij", q_rot, k_rot)) * cfg["scale"]
    p = masked_softmax(s, block_causal_mask(T, None)[None])
    out = torch.einsum("hij,jhd->ihd", p, v)
    return out.reshape(T, H * Dv) @ w["o"].T


def local(weights: dict, prefix: str) -> dict:
    """Tensors under ``prefix.`` by the rest of their name."""
    return {k[len(prefix) + 1:]: v for k, v in weights.items() if k.startswith(prefix + ".")}


def forward(weights: dict, config: dict, tokens: list[int], return_layers: bool = False):
    """Logits [T, vocab] of one whole sequence (and the stream after every layer, if asked)."""
    eps = config["norm"]["eps"]
    x = norm_around_zero(weights["embed"][torch.tensor(tokens)], weights["embed.norm"], eps)
    v_first = None
    after = []
    for i, layer in enumerate(config["layers"]):
        pre = f"l{i}"
        h = norm_around_zero(x, weights[f"{pre}.norm1"], eps)
        mix = local(weights, f"{pre}.mix")
        if layer["type"] == "attention":
            blends = bool(layer["mixer"].get("v_mix"))
            out, v_own = gated_capped_attention(h, mix, layer["mixer"], eps, v_first if blends else None)
            if blends and v_first is None:
                v_first = v_own
        elif layer["type"] == "latent_attention":
            out = latent_attention(h, mix, layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        x = x + out
        if layer.get("mlp") is not None:
            h = norm_around_zero(x, weights[f"{pre}.norm2"], eps)
            x = x + dense_feed_forward(h, weights[f"{pre}.mlp.up"], weights[f"{pre}.mlp.down"])
        after.append(x)
    logits = norm_around_zero(x, weights["final.norm"], eps) @ weights["head"].T
    return (logits, torch.stack(after)) if return_layers else logits


def greedy_generate(weights: dict, config: dict, prompt: list[int], new_tokens: int) -> list[int]:
    ids, out = list(prompt), []
    for _ in range(new_tokens):
        token = int(forward(weights, config, ids)[-1].argmax())
        out.append(token)
        ids.append(token)
    return out
