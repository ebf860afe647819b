"""The gated delta rule: a linear-attention mixer whose memory is one matrix per head, carried from token to token.

    q, k, v   = silu(conv(W_q x)), silu(conv(W_k x)), silu(conv(W_v x))     short causal convolutions over time, per
                                                                            channel, zeros before the sequence's start
    q, k     <- q / sqrt(|q|^2 + unit_eps) * dim^-1/2,  k / sqrt(|k|^2 + unit_eps)          per head
    beta      = sigmoid(W_b x);   decay = exp(-exp(rate_log) * softplus(W_a x + step_bias))  one of each per head
    S        <- decay * S;   u = beta * (v - S^T k);   S <- S + k u^T;   o = S^T q           per head, S: [dim, vdim]
    y         = W_o concat_h( o_h / sqrt(mean(o_h^2) + norm_eps) * norm * silu(W_g x)_h )

``num_kv_heads`` heads of q and k serve ``num_heads`` heads of v in groups.  What a request carries from step to
step is float32 and lives in its state slot: every head's S and the last ``taps - 1`` inputs of the three
convolutions.  One product makes all projections of a token; a row-wise kernel (``ops.delta_prep``) turns them into
float32 q, k, v, beta and decay; one block per (sequence, head) walks the step's tokens of that sequence in order
(``ops.delta_scan``), so the state after a token is the same however the tokens were cut into steps.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import CacheSpec, Mixer, ParamSpec, register_mixer


@register_mixer("gated_delta")
class GatedDelta(Mixer):
    """params: ``num_heads``, ``num_kv_heads``, ``head_dim`` (q / k width), ``v_dim``, ``taps`` (of the convolutions;
    1: none), ``unit_eps``, ``norm_eps``, ``names`` (local tensor names of q, k, v, their convolutions, beta, step,
    rate_log, step_bias, gate, norm, out)."""

    graph_safe = True

    NAMES = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "q_conv": "q_conv.weight",
             "k_conv": "k_conv.weight", "v_conv": "v_conv.weight", "beta": "b_proj.weight", "step": "a_proj.weight",
             "rate_log": "A_log", "step_bias": "dt_bias", "gate": "g_proj.weight", "norm": "o_norm.weight",
             "out": "o_proj.weight"}

    def __init__(self, spec, **kw):
        super().__init__(spec, **kw)
        p = spec.params
        self.num_heads, self.num_kv_heads = int(p["num_heads"]), int(p["num_kv_heads"])
        self.head_dim, self.v_dim, self.taps = int(p["head_dim"]), int(p["v_dim"]), int(p["taps"])
        if self.num_heads <= 0 or self.num_kv_heads <= 0 or self.num_heads % self.num_kv_heads:
            raise ValueError(f"gated_delta: {self.num_heads} heads are not a multiple of {self.num_kv_heads} q/k heads")
        if ops.delta_shape(self.head_dim, self.v_dim) is None:
            raise ValueError(f"gated_delta: q/k width {self.head_dim} with value width {self.v_dim} is outside what "
                             f"the kernel takes (each up to {ops.DELTA_MAX_DIM})")
        if not 1 <= self.taps <= ops.DELTA_MAX_TAPS:
            raise ValueError(f"gated_delta: {self.taps} taps outside what the kernel takes (1 to {ops.DELTA_MAX_TAPS})")
        self.unit_eps = float(p.get("unit_eps", 1e-6))
        self.norm_eps = float(p.get("norm_eps", 1e-6))
        self.names = dict(self.NAMES, **(p.get("names") or {}))
        self.qk_width = self.num_kv_heads * self.head_dim
        self.v_width = self.num_heads * self.v_dim
        self.channels = 2 * self.qk_width + self.v_width            # what the convolutions run over
        # floats of all heads' S per request, and of the whole state with the convolutions' inputs behind it
        self.memory, self.state_floats = ops.delta_state_floats(self.num_heads, self.num_kv_heads, self.head_dim,
                                                                self.v_dim, self.taps)
        self.w_in = self.w_o = self.conv = self.rate_log = self.step_bias = self.norm_weight = None

    def cache_spec(self) -> CacheSpec:
        return CacheSpec(kind="none", state_shape=(self.state_floats,))

    def param_specs(self):
        h, n = self.hidden_size, self.names
        return {
            n["q"]: ParamSpec((self.qk_width, h)), n["q_conv"]: ParamSpec((self.qk_width, self.taps), kind="vector", init="unit_interval"),
            n["k"]: ParamSpec((self.qk_width, h)), n["k_conv"]: ParamSpec((self.qk_width, self.taps), kind="vector", init="unit_interval"),
            n["v"]: ParamSpec((self.v_width, h)), n["v_conv"]: ParamSpec((self.v_width, self.taps), kind="vector", init="unit_interval"),
            n["beta"]: ParamSpec((self.num_heads, h)),
            n["rate_log"]: ParamSpec((self.num_heads,), kind="vector", init="around_zero"),
            n["norm"]: ParamSpec((self.v_dim,), kind="vector", init="norm"),
            n["step"]: ParamSpec((self.num_heads, h)),
            n["step_bias"]: ParamSpec((self.num_heads,), kind="vector", init="around_zero"),
            n["gate"]: ParamSpec((self.v_width, h)),
            n["out"]: ParamSpec((h, self.v_width)),
        }

    def load(self, tensors):
        n = self.names
        # one product: [q | k | v | gate | beta | step]
        self.w_in = torch.cat([tensors[n[k]] for k in ("q", "k", "v", "gate", "beta", "step")], dim=0).contiguous()
        self.conv = torch.cat([tensors[n[k]] for k in ("q_conv", "k_conv", "v_conv")], dim=0).float().contiguous()
        self.rate_log = tensors[n["rate_log"]].float().contiguous()
        self.step_bias = tensors[n["step_bias"]].float().contiguous()
        self.norm_weight = tensors[n["norm"]].float().contiguous()
        self.w_o = tensors[n["out"]].contiguous()

    def forward(self, x, ctx, cache):
        if cache.state is None:
            raise ValueError("gated_delta: the cache manager gave this position no state")
        sizes = dict(num_heads=self.num_heads, num_kv_heads=self.num_kv_heads, head_dim=self.head_dim,
                     v_dim=self.v_dim, taps=self.taps)
        x = ops.linear(x, self.w_in, status=ctx.status)
        qkv, coef = ops.delta_prep(x, self.conv, self.rate_log, self.step_bias, cache.state, ctx.cu_q,
                                   ctx.state_slots, unit_eps=self.unit_eps, **sizes)
        out = ops.delta_scan(qkv, coef, x, self.norm_weight, cache.state, ctx.cu_q, ctx.state_slots,
                             norm_eps=self.norm_eps, **sizes)
        return ops.linear(out, self.w_o, status=ctx.status)
