"""RMSNorm fused with the residual sum.

Formula of the reference (ampere_kv/runner.py:48-57): float32 mean of squares over the last
dim, ``x * rsqrt(ms + eps)``, times a plain weight (not ``1 + w``).  The reference rounds to
the activation dtype before the weight multiply; here the product is formed in float32 and
rounded once.  The residual sums of runner.py:167 and :179 are folded into the same kernel and
kept in float32.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import Norm, ParamSpec, register_norm


@register_norm("rmsnorm")
class RMSNorm(Norm):
    """params: ``size`` (defaults to the hidden size), ``eps``, ``tensor`` (the weight's name under the prefix,
    default ``weight``), ``unit_offset`` (the stored weight w is kept around zero and stands for ``1 + w``)."""

    graph_safe = True


    def __init__(self, spec, **kw):
        super().__init__(spec, **kw)
        self.size = int(spec.params.get("size", self.hidden_size))
        self.eps = float(spec.params["eps"])
        self.tensor = str(spec.params.get("tensor", "weight"))
        self.unit_offset = bool(spec.params.get("unit_offset", False))
        self.weight: torch.Tensor | None = None

    def param_specs(self):
        return {self.tensor: ParamSpec((self.size,), kind="vector", init="around_zero" if self.unit_offset else "norm")}

    def load(self, tensors):
        # the factor the kernels multiply by: the stored weight, or one more than it (formed once, in float32)
        self.weight = tensors[self.tensor] + 1.0 if self.unit_offset else tensors[self.tensor]

    takes_summed = True
    takes_pending = True

    def forward(self, hidden, delta, ctx, rows=None, lazy=False):
        status = getattr(ctx, "status", None)
        if isinstance(delta, ops.PendingPhases):
            if lazy and rows is None and self.size == hidden.shape[1] and self.weight.data_ptr() % 16 == 0:
                return ops.StreamNorm(delta, self.weight, self.eps, self.dtype)
            return None
        if isinstance(delta, ops.Summed):
            if lazy and rows is None and self.size == hidden.shape[1]:
                return ops.LazyNorm(delta, self.weight, self.eps, self.dtype, status)
            delta = None      # hidden holds the sum already
        return ops.add_rmsnorm(hidden, delta, self.weight, self.eps, self.dtype, rows=rows, status=status)


@register_norm("layernorm")
class LayerNorm(Norm):
    """``(x - mean) / sqrt(var + eps) * weight`` with the variance as the mean of squared deviations and no bias.
    params: ``size`` (defaults to the hidden size), ``eps``, ``tensor`` (the weight's name under the prefix, default
    ``weight``).  Beside the usual form (:meth:`forward`: sum into the stream, then norm what a branch reads) it has
    the form a layer with normed branch *outputs* needs (:meth:`add_normed`): the norm of the branch's result is what
    is added to the stream.  Mean, variance, the scale and the sum are float32."""

    graph_safe = True
    #: ``add_normed`` takes an ``ops.ExpertParts`` as the branch and adds its rows up in the same kernel
    takes_parts = True

    def __init__(self, spec, **kw):
        super().__init__(spec, **kw)
        self.size = int(spec.params.get("size", self.hidden_size))
        self.eps = float(spec.params["eps"])
        self.tensor = str(spec.params.get("tensor", "weight"))
        self.weight: torch.Tensor | None = None

    def param_specs(self):
        return {self.tensor: ParamSpec((self.size,), kind="vector", init="norm")}

    def load(self, tensors):
        self.weight = tensors[self.tensor].contiguous()

    def forward(self, hidden, delta, ctx, rows=None):
        return ops.add_layernorm(hidden, delta, self.weight, self.eps, self.dtype, rows=rows,
                                 status=getattr(ctx, "status", None))

    def add_normed(self, hidden, branch, ctx):
        """``hidden += LN(branch)`` in place; returns the new stream in the compute dtype (the stream itself when
        that is float32), which is what the next branch reads."""
        return ops.branch_layernorm(hidden, branch, self.weight, self.eps, self.dtype)
