"""Dense gated feed-forward: ``down(act(gate(x)) * up(x))``.

The reference's form (ampere_kv/runner.py:172-177) with SiLU; the tanh form of GELU and biases on all three
projections are options.  gate and up are stored as one
matrix, so one product feeds the activation; each output element keeps its own row's
accumulation order.  Where the intermediate size allows it the rows alternate in runs of 64
gate rows and the 64 up rows of the same outputs: a 128-row tile of the decode GEMM then holds
both and applies the activation itself, and the prompt path's activation kernel reads the same
layout.  Otherwise all gate rows come first.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import FeedForward, ParamSpec, register_feed_forward


@register_feed_forward("gated_mlp")
class GatedMLP(FeedForward):
    """params: ``intermediate_size``, ``activation`` (``"silu"`` or ``"gelu_tanh"``), ``bias`` (all three projections
    carry one), ``names`` (local tensor names of ``gate``, ``up``, ``down`` and, with biases, ``gate_bias``,
    ``up_bias``, ``down_bias``)."""

    graph_safe = True
    takes_lazy_norm = True
    adds_residual = True
    takes_stream_norm = True

    NAMES = {"gate": "gate_proj.weight", "up": "up_proj.weight", "down": "down_proj.weight",
             "gate_bias": "gate_proj.bias", "up_bias": "up_proj.bias", "down_bias": "down_proj.bias"}

    def __init__(self, spec, **kw):
        super().__init__(spec, **kw)
        self.intermediate_size = int(spec.params["intermediate_size"])
        self.activation = spec.params.get("activation", "silu")
        if self.activation not in ("silu", "gelu_tanh"):
            raise ValueError(f"gated_mlp: activation {self.activation!r} is not supported ('silu', 'gelu_tanh')")
        self.bias = bool(spec.params.get("bias", False))
        self.names = dict(self.NAMES, **(spec.params.get("names") or {}))
        #: the fused small-batch kernels carry SiLU and no bias
        self.plain = self.activation == "silu" and not self.bias
        self.gate_up: torch.Tensor | None = None
        self.run = ops.GATE_UP_RUN if self.intermediate_size % ops.GATE_UP_RUN == 0 else 0
        self.down: torch.Tensor | None = None
        self.gate_up_bias = self.down_bias = None

    def param_specs(self):
        i, h, n = self.intermediate_size, self.hidden_size, self.names
        specs = {n["gate"]: ParamSpec((i, h)), n["up"]: ParamSpec((i, h)), n["down"]: ParamSpec((h, i))}
        if self.bias:
            specs.update({n["gate_bias"]: ParamSpec((i,), kind="bias"), n["up_bias"]: ParamSpec((i,), kind="bias"),
                          n["down_bias"]: ParamSpec((h,), kind="bias")})
        return specs

    def load(self, tensors):
        n = self.names
        gate, up = tensors[n["gate"]], tensors[n["up"]]
        if self.run:
            self.gate_up = ops.interleave_gate_up(gate, up, self.run).contiguous()
        else:
            self.gate_up = torch.cat((gate, up), dim=0).contiguous()
        self.down = tensors[n["down"]].contiguous()
        if self.bias:
            gb, ub = tensors[n["gate_bias"]].unsqueeze(1), tensors[n["up_bias"]].unsqueeze(1)
            both = ops.interleave_gate_up(gb, ub, self.run) if self.run else torch.cat((gb, ub), dim=0)
            self.gate_up_bias = both.reshape(-1).contiguous()
            self.down_bias = tensors[n["down_bias"]].contiguous()

    def forward(self, x, ctx, residual=None):
        status = getattr(ctx, "status", None)
        if not self.plain:
            if not isinstance(x, torch.Tensor):
                x = x.materialize()
            both = ops.linear(x, self.gate_up, self.gate_up_bias, status=status)
            act = ops.glu(both, self.activation, self.run)
            return ops.linear(act, self.down, self.down_bias, status=status)
        if isinstance(x, ops.StreamNorm):
            # a few decoded tokens: both products go behind the output projection that is still queued; whoever
            # comes next (the next layer's q/k/v projection, or the final norm) launches them
            if (residual is x.hidden and self.run == ops.GATE_UP_RUN and self.gate_up.shape[0] % 128 == 0
                    and ops.stream_takes(x.shape[0], self.gate_up, self.down)):
                act = torch.empty((x.shape[0], self.intermediate_size), dtype=torch.bfloat16,
                                  device=self.gate_up.device)
                x.pending.add(x.normed_phase(self.gate_up, epilogue="gated", out=act))
                x.pending.add(dict(w=self.down, x=act, epilogue="residual"))
                return x.pending
            x = x.materialize()
        act = ops.gated_linear(x, self.gate_up, self.run, status=status)
        if residual is not None:
            summed = ops.linear_into_residual(act, self.down, residual, status=status)
            if summed is not None:
                return summed
        return ops.linear(act, self.down, partial_ok=True, status=status)


@register_feed_forward("dense_mlp")
class DenseMLP(FeedForward):
    """``down(act(up(x)))`` without a gate.  params: ``intermediate_size``, ``activation`` (``"relu2"``: the square
    of relu; ``"gelu_tanh"``; ``"silu"``), ``up`` / ``down`` (the matrices' names under the prefix, defaults
    ``up_proj.weight`` / ``down_proj.weight``)."""

    graph_safe = True
    takes_lazy_norm = True
    adds_residual = True

    def __init__(self, spec, **kw):
        super().__init__(spec, **kw)
        self.intermediate_size = int(spec.params["intermediate_size"])
        self.activation = str(spec.params.get("activation", "relu2"))
        if self.activation not in ops.ACTIVATIONS:
            raise ValueError(f"dense_mlp: activation {self.activation!r} is not one of {sorted(ops.ACTIVATIONS)}")
        self.up_name = str(spec.params.get("up", "up_proj.weight"))
        self.down_name = str(spec.params.get("down", "down_proj.weight"))
        self.up: torch.Tensor | None = None
        self.down: torch.Tensor | None = None

    def param_specs(self):
        i, h = self.intermediate_size, self.hidden_size
        return {self.up_name: ParamSpec((i, h)), self.down_name: ParamSpec((h, i))}

    def load(self, tensors):
        self.up = tensors[self.up_name].contiguous()
        self.down = tensors[self.down_name].contiguous()

    def forward(self, x, ctx, residual=None):
        status = getattr(ctx, "status", None)
        act = ops.linear_activation(x, self.up, self.activation, status=status)
        if residual is not None:
            summed = ops.linear_into_residual(act, self.down, residual, status=status)
            if summed is not None:
                return summed
        return ops.linear(act, self.down, partial_ok=True, status=status)
