"""RMSNorm, fused with the residual sum that precedes it."""

from __future__ import annotations

from typing import List

import torch

from .base import Norm, ScaledSum, StreamUpdate, WeightSpec, register_norm
from .params import DynamicTanhParams, LayerNormParams, RMSNormParams


class RMSNorm(Norm):
    """``x * rsqrt(mean(x^2) + eps) * w`` in float32 (fastgen/kernels/rmsnorm.py:33-60).

    The weight keeps the dtype it was stored in (a 32-bit weight stays 32-bit);
    the float32 path upcasts it.
    """

    params: RMSNormParams

    def weight_specs(self) -> List[WeightSpec]:
        init = ("normal", 0.1) if self.params.one_plus else ("ones",)
        return [WeightSpec(self.names["weight"], (self.params.dim,), init)]

    def bind(self, tensors, ops) -> None:
        self.ops = ops
        w = tensors["weight"]
        if ops.act_dtype == torch.float32:
            w = w.float()
        self.weight = w.contiguous()

    def forward(self, x, out_dtype=None, rows=None):
        n = x.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, x.shape[1]), dtype=out_dtype or self.ops.act_dtype, device=x.device)
        if self.params.one_plus:
            # the factor 1 + w is formed in float32 by the kernel that also takes sums of summands
            return self.ops.rmsnorm_sum(x, (), self.weight, self.params.eps, out=out, rows=rows, one_plus=True)
        return self.ops.rmsnorm(x, self.weight, self.params.eps, out=out, rows=rows)

    def add_forward(self, h, delta, rows=None, delta_norm=None):
        """``h += delta`` in float32 (stored back unless ``rows`` gathers), then the norm.  ``delta``
        may be a :class:`ScaledSum`: all of its summands join in the same kernel."""
        if delta_norm is not None:
            return super().add_forward(h, delta, rows=rows, delta_norm=delta_norm)
        n = h.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, h.shape[1]), dtype=self.ops.act_dtype, device=h.device)
        if isinstance(delta, ScaledSum) or self.params.one_plus:
            total = ScaledSum.of(delta)
            if len(total.terms) > 4 or len({t.dtype for t, _ in total.terms}) > 1:
                total.add_into(h, self.ops)
                total = ScaledSum([])
            return self.ops.rmsnorm_sum(h, total.terms, self.weight, self.params.eps, out=out, row=total.row,
                                        rows=rows, one_plus=self.params.one_plus)
        return self.ops.rmsnorm(h, self.weight, self.params.eps, out=out, delta=delta, rows=rows)


class DynamicTanh(Norm):
    """``tanh(alpha * x) * w + b`` in float32, with a scalar ``alpha`` and vectors ``w``, ``b``
    (tensors ``weight``, ``bias``, ``alpha``): elementwise, no mean and no variance.

    The sum that precedes the norm is fused into its kernel, and so is the norm of the
    summand when that is a Dynamic Tanh too: ``h += tanh(a' d) w' + b'; out = tanh(a h) w + b``
    is one launch.
    """

    params: DynamicTanhParams

    def weight_specs(self) -> List[WeightSpec]:
        d = self.params.dim
        return [
            WeightSpec(self.names["weight"], (d,), ("ones",)),
            WeightSpec(self.names["bias"], (d,), ("normal", 0.02)),
            WeightSpec(self.names["alpha"], (), ("ones",)),
        ]

    def bind(self, tensors, ops) -> None:
        self.ops = ops
        # small vectors: float32 whatever they were stored in (the arithmetic is float32)
        self.weight = tensors["weight"].float().contiguous()
        self.bias = tensors["bias"].float().contiguous()
        self.alpha = tensors["alpha"].float().reshape(1).contiguous()

    def triple(self):
        return (self.alpha, self.weight, self.bias)

    def forward(self, x, out_dtype=None, rows=None):
        n = x.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, x.shape[1]), dtype=out_dtype or self.ops.act_dtype, device=x.device)
        if x.dtype != torch.float32:
            x = x.float()
        return self.ops.dyt(x, self.triple(), out, rows=rows)

    def add_forward(self, h, delta, rows=None, delta_norm=None):
        if isinstance(delta, ScaledSum):
            delta = self._joined(h, delta, rows)
        if delta is not None and delta_norm is not None and not isinstance(delta_norm, DynamicTanh):
            delta, delta_norm = delta_norm.forward(delta, out_dtype=torch.float32), None
        n = h.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, h.shape[1]), dtype=self.ops.act_dtype, device=h.device)
        post = delta_norm.triple() if delta is not None and delta_norm is not None else None
        return self.ops.dyt(h, self.triple(), out, delta=delta, post=post, rows=rows)


class LayerNorm(Norm):
    """``(x - mean) / sqrt(var + eps) * w + b`` in float32; the variance is the mean of the squared
    deviations.  Tensors ``weight`` and, with ``params.bias``, ``bias``.

    The residual stream may be several streams ``h`` [T, S, dim] that are mixed on the way
    (``streams_forward``): the update a sub-layer left pending, the weighted sum of the streams
    and the norm are one kernel.  The plain ``h += delta; norm(h)`` is its case ``S = 1``."""

    params: LayerNormParams
    kind = 0  # the kernel's code for "with mean and variance"

    def weight_specs(self) -> List[WeightSpec]:
        d = self.params.dim
        specs = [WeightSpec(self.names["weight"], (d,), ("ones",))]
        if self.params.bias:
            specs.append(WeightSpec(self.names["bias"], (d,), ("normal", 0.02)))
        return specs

    def bind(self, tensors, ops) -> None:
        self.ops = ops
        self.weight = tensors["weight"].float().contiguous()
        self.bias = tensors["bias"].float().contiguous() if self.params.bias else None

    def streams_forward(self, h, update=None, in_coef=None, rows=None, out_dtype=None):
        """``h`` [T, S, dim] (or [T, dim]): apply ``update`` (a :class:`StreamUpdate` or ``None``),
        then norm ``sum_s in_coef[s] x_s`` (``in_coef`` ``None``: the plain sum)."""
        n = h.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, h.shape[-1]), dtype=out_dtype or self.ops.act_dtype, device=h.device)
        return self.ops.stream_norm(h, self.weight, self.bias, self.params.eps, out, kind=self.kind, update=update,
                                    in_coef=in_coef, rows=rows)

    def forward(self, x, out_dtype=None, rows=None):
        if x.dtype != torch.float32:
            x = x.float()
        return self.streams_forward(x, rows=rows, out_dtype=out_dtype)

    def add_forward(self, h, delta, rows=None, delta_norm=None):
        if isinstance(delta, ScaledSum):
            delta = self._joined(h, delta, rows)
        if delta is not None and delta_norm is not None:
            delta = delta_norm.forward(delta, out_dtype=torch.float32)
        update = StreamUpdate(delta) if delta is not None else None
        return self.streams_forward(h, update=update, rows=rows)


register_norm("rmsnorm", RMSNorm)
register_norm("layernorm", LayerNorm)
register_norm("dynamic_tanh", DynamicTanh)
