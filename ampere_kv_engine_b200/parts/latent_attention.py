"""Attention through low-rank latents: the cache keeps one compressed row per token.

    (a | b | r) = (W_dq | W_dkv) x                 one product: query latent, key/value latent, rotated key part
    c_q = rmsnorm(a) * w_q;   c = rmsnorm(b) * w_kv;   r <- rotary(r)      (pairs of neighbouring dims)
    q   = W_uq c_q, per head [head_dim unrotated | rot_dim rotated];  the rotated part <- rotary(.)
    per head: k = W_uk c (unrotated) beside the shared r, v = W_uv c
    s(i, j) = (q_unrot . k_j + q_rot . r_j) * scale,  causal softmax,  y = W_o concat_h(sum_j p_j v_j)

Only ``c`` and ``r`` are kept per token, side by side in one cache row ``[kv_rank + rot_dim]``.  Keys and values
are never expanded: since ``q_unrot . (W_uk c) = (W_uk^T q_unrot) . c``, the query is carried into the latent space
(one batched product per step) and attention runs over the rows as they are stored, every head reading the same
row as its key and the row's first ``kv_rank`` elements as its value; the result per head is a mix of latents,
which ``W_uv`` turns into the head's output (one more batched product).  Between the products stand two row-wise
kernels (``ops.latent_prep``, ``ops.rotate_pairs``) and ``ops.scored_attention``.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import CacheSpec, CacheTensor, Mixer, ParamSpec, register_mixer
from .scored_attention import run_attention


@register_mixer("latent_attention")
class LatentAttention(Mixer):
    """params: ``num_heads``, ``head_dim`` (unrotated query / key dims per head), ``rot_dim`` (rotated dims per head,
    and the width of the shared rotated key part), ``v_dim``, ``q_rank``, ``kv_rank``, ``scale``, ``norm_eps``,
    ``rotary_base``, ``rotary_dims`` (how many of the ``rot_dim`` dims turn; default all), ``window`` (None: all
    keys), ``names`` (local tensor names)."""

    graph_safe = True
    takes_lazy_norm = True
    adds_residual = True

    NAMES = {"dq": "q_a_proj.weight", "dq_norm": "q_a_norm.weight", "uq": "q_b_proj.weight",
             "dkv": "kv_a_proj.weight", "dkv_norm": "kv_a_norm.weight", "uk": "k_b_proj.weight",
             "uv": "v_b_proj.weight", "out": "o_proj.weight"}

    def __init__(self, spec, **kw):
        super().__init__(spec, **kw)
        p = spec.params
        self.num_heads, self.head_dim, self.rot_dim = int(p["num_heads"]), int(p["head_dim"]), int(p["rot_dim"])
        self.v_dim, self.q_rank, self.kv_rank = int(p["v_dim"]), int(p["q_rank"]), int(p["kv_rank"])
        self.rotary_dims = int(p.get("rotary_dims", self.rot_dim))
        self.rotary_base = float(p.get("rotary_base", 10000.0))
        if min(self.num_heads, self.head_dim, self.v_dim, self.q_rank, self.kv_rank) <= 0 or self.rot_dim < 0:
            raise ValueError("latent_attention: sizes must be positive")
        if self.rotary_dims % 2 or not 0 <= self.rotary_dims <= self.rot_dim:
            raise ValueError(f"latent_attention: rotary_dims must be even and at most rot_dim ({self.rot_dim}), "
                             f"got {self.rotary_dims}")
        if self.kv_rank > 512 or self.kv_rank + self.rot_dim > 1024:
            raise ValueError(f"latent_attention: a latent of {self.kv_rank} + {self.rot_dim} is wider than the "
                             f"attention kernel takes (512 + rotated part up to 1024)")
        self.scale = float(p["scale"]) if p.get("scale") is not None else (self.head_dim + self.rot_dim) ** -0.5
        self.norm_eps = float(p.get("norm_eps", 1e-6))
        self.window = int(p["window"]) if p.get("window") else 0
        self.names = dict(self.NAMES, **(p.get("names") or {}))
        i = torch.arange(self.rotary_dims // 2, dtype=torch.float64)
        self.inv_freq = (self.rotary_base ** (-2.0 * i / max(self.rotary_dims, 1))).to(torch.float32).to(self.device)
        self.w_down = self.w_uq = self.w_uk = self.w_uv = self.w_o = self.q_norm = self.kv_norm = None

    @property
    def row(self) -> int:
        return self.kv_rank + self.rot_dim

    def cache_spec(self) -> CacheSpec:
        return CacheSpec(kind="window" if self.window else "full", num_kv_heads=1, head_dim=self.row,
                         window=self.window or None, tensors=(CacheTensor("latent", 1, self.row),))

    def param_specs(self):
        h, n, H = self.hidden_size, self.names, self.num_heads
        return {
            n["dq"]: ParamSpec((self.q_rank, h)),
            n["dq_norm"]: ParamSpec((self.q_rank,), kind="vector", init="norm"),
            n["uq"]: ParamSpec((H * (self.head_dim + self.rot_dim), self.q_rank)),
            n["dkv"]: ParamSpec((self.row, h)),
            n["dkv_norm"]: ParamSpec((self.kv_rank,), kind="vector", init="norm"),
            n["uk"]: ParamSpec((H * self.head_dim, self.kv_rank)),
            n["uv"]: ParamSpec((H * self.v_dim, self.kv_rank)),
            n["out"]: ParamSpec((h, H * self.v_dim)),
        }

    def load(self, tensors):
        n, H = self.names, self.num_heads
        self.w_down = torch.cat((tensors[n["dq"]], tensors[n["dkv"]]), dim=0).contiguous()
        self.q_norm, self.kv_norm = tensors[n["dq_norm"]], tensors[n["dkv_norm"]]
        self.w_uq = tensors[n["uq"]].contiguous()
        # per head: [head_dim, kv_rank] carries a query into the latent space, [kv_rank, v_dim] a latent mix out of it
        self.w_uk = tensors[n["uk"]].view(H, self.head_dim, self.kv_rank).contiguous()
        self.w_uv = tensors[n["uv"]].view(H, self.v_dim, self.kv_rank).transpose(1, 2).contiguous()
        self.w_o = tensors[n["out"]].contiguous()

    def forward(self, x, ctx, cache, residual=None):
        group = ctx.groups[cache.group]
        rows = cache.tensors["latent"]
        H, D, R, rank = self.num_heads, self.head_dim, self.rot_dim, self.kv_rank
        down = ops.linear(x, self.w_down, status=ctx.status)
        tokens = down.shape[0]
        writes = cache.writes
        q_latent = ops.latent_prep(down, ctx.positions, group.slot_mapping if writes else None, self.q_norm,
                                   self.kv_norm, self.inv_freq, rows if writes else None, q_rank=self.q_rank,
                                   kv_rank=rank, rot_dim=R, rotary_dims=self.rotary_dims, eps=self.norm_eps,
                                   status=ctx.status)
        q = ops.linear(q_latent, self.w_uq, status=ctx.status)                      # [tokens, H * (D + R)]
        q_row = torch.empty((tokens, H * self.row), dtype=q.dtype, device=q.device)
        if R:
            ops.rotate_pairs(q, q_row, ctx.positions, self.inv_freq, heads=H, cols=R, rotary_dims=self.rotary_dims,
                             in_offset=D, out_offset=rank)
        # the unrotated part of every head's query, carried into the latent space: [H, tokens, D] x [H, D, rank]
        torch.bmm(q.view(tokens, H, D + R)[:, :, :D].transpose(0, 1), self.w_uk,
                  out=q_row.view(tokens, H, self.row)[:, :, :rank].transpose(0, 1))
        mixed = torch.empty((tokens, H * rank), dtype=q.dtype, device=q.device)
        run_attention(ctx, group, q_row, rows, rows, mixed, num_heads=H, num_kv_heads=1, v_dim=rank, scale=self.scale,
                      window=self.window)
        out = torch.empty((tokens, H * self.v_dim), dtype=q.dtype, device=q.device)
        torch.bmm(mixed.view(tokens, H, rank).transpose(0, 1), self.w_uv,
                  out=out.view(tokens, H, self.v_dim).transpose(0, 1))              # [H, tokens, v_dim]
        if residual is not None:
            summed = ops.linear_into_residual(out, self.w_o, residual, status=ctx.status)
            if summed is not None:
                return summed
        return ops.linear(out, self.w_o, partial_ok=True, status=ctx.status)
