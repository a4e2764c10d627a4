"""Feed-forward with routed experts (a mixture of experts)."""

from __future__ import annotations

from typing import List

import torch

from .base import FeedForward, WeightSpec, register_feed_forward
from .params import RoutedExpertsParams


class RoutedExperts(FeedForward):
    """``sum over a token's top experts of weight_e * w2_e(silu(w1_e x) * w3_e x)``.

    The router's logits ``router x`` are float32 sums (of the activations as the compute dtype holds
    them) and so is their softmax ``s`` over all experts.  A token's experts are the ``top`` largest
    ``s + correction`` (the lower index among equal ones); their weights are their ``s``, divided
    by the sum of the chosen ones only with ``renormalize``.  The experts' matrices are stacked at
    bind time ([experts, 2 ffn, dim]: gate rows then up rows; [experts, dim, ffn]) and the (token, expert) pairs are
    sorted by expert on the device, so the step launches a fixed number of kernels whatever the
    router says.
    """

    params: RoutedExpertsParams

    @property
    def names(self):
        """Local name -> checkpoint name; an expert's tensors are ``w1.<e>`` and so on (the
        templates given in the spec are filled with the expert's number)."""
        return self._flat

    @names.setter
    def names(self, value) -> None:
        self._templates = dict(value)
        flat = {}
        for local, name in self._templates.items():
            if local in ("w1", "w2", "w3"):
                for e in range(self.params.n_experts):
                    flat[f"{local}.{e}"] = name.format(e)
            elif local != "correction" or self.params.correction:
                flat[local] = name
        self._flat = flat

    def weight_specs(self) -> List[WeightSpec]:
        p, n = self.params, self._templates
        specs = [WeightSpec(n["router"], (p.n_experts, p.dim), ("normal", 0.5))]
        if p.correction:
            specs.append(WeightSpec(n["correction"], (p.n_experts,), ("normal", 0.05)))
        for e in range(p.n_experts):
            specs += [
                WeightSpec(n["w1"].format(e), (p.ffn_dim, p.dim)),
                WeightSpec(n["w3"].format(e), (p.ffn_dim, p.dim)),
                WeightSpec(n["w2"].format(e), (p.dim, p.ffn_dim)),
            ]
        return specs

    def bind(self, tensors, ops) -> None:
        p = self.params
        self.ops = ops
        dt = ops.act_dtype
        stack = lambda local: torch.stack([tensors[f"{local}.{e}"] for e in range(p.n_experts)]).to(dt).contiguous()
        # an expert's gate rows, then its up rows: one product gives both, and each is a view
        self.w13 = torch.cat([stack("w1"), stack("w3")], dim=1).contiguous()
        self.w1, self.w3, self.w2 = self.w13[:, : p.ffn_dim], self.w13[:, p.ffn_dim :], stack("w2")
        self.router = tensors["router"].float().contiguous()
        self.correction = tensors["correction"].float().contiguous() if p.correction else None

    def forward(self, x, ctx):
        p, ops = self.params, self.ops
        logits = ops.moe_logits(x, self.router, ctx)
        ids, weights = ops.moe_route(logits, self.correction, p.top, ctx, renormalize=p.renormalize)
        return ops.moe_experts(x, ids, weights, self.w1, self.w3, self.w2, self.w13)


register_feed_forward("routed_experts", RoutedExperts)
