"""Feed-forward with routed experts (a mixture of experts)."""

from __future__ import annotations

from typing import List

import torch

from .base import FeedForward, ScaledSum, WeightSpec, make_feed_forward, register_feed_forward
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

    Options of the parameters: sigmoid scores instead of a softmax; a choice that is limited to the
    experts of the best groups of neighbours; a small number added to the sum that renormalises; a
    factor on the weights; experts without a gate, ``w2_e(act(w3_e x))``; a shared feed-forward that every
    token passes and whose output is added (the result is then a sum that the next norm's kernel forms).
    """

    params: RoutedExpertsParams

    def __init__(self, spec) -> None:
        super().__init__(spec)
        p = self.params
        self.gated = p.act == "silu_gate"
        self.shared = make_feed_forward(p.shared) if p.shared is not None else None

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
            if local == "w1" and self.params.act != "silu_gate":
                continue  # experts without a gate
            if local in ("w1", "w2", "w3"):
                for e in range(self.params.n_experts):
                    flat[f"{local}.{e}"] = name.format(e)
            elif local != "correction" or self.params.correction:
                flat[local] = name
        if self.params.shared is not None:
            for local, name in dict(self.params.shared.names).items():
                flat["shared." + local] = name
        self._flat = flat

    def weight_specs(self) -> List[WeightSpec]:
        p, n = self.params, self._templates
        specs = [WeightSpec(n["router"], (p.n_experts, p.dim), ("normal", 0.5))]
        if p.correction:
            specs.append(WeightSpec(n["correction"], (p.n_experts,), ("normal", 0.05)))
        for e in range(p.n_experts):
            if self.gated:
                specs.append(WeightSpec(n["w1"].format(e), (p.ffn_dim, p.dim)))
            specs += [
                WeightSpec(n["w3"].format(e), (p.ffn_dim, p.dim)),
                WeightSpec(n["w2"].format(e), (p.dim, p.ffn_dim)),
            ]
        if self.shared is not None:
            specs += self.shared.weight_specs()
        return specs

    def bind(self, tensors, ops) -> None:
        p = self.params
        self.ops = ops
        dt = ops.act_dtype
        stack = lambda local: torch.stack([tensors[f"{local}.{e}"] for e in range(p.n_experts)]).to(dt).contiguous()
        if self.gated:
            # an expert's gate rows, then its up rows: one product gives both, and each is a view
            self.w13 = torch.cat([stack("w1"), stack("w3")], dim=1).contiguous()
            self.w1, self.w3, self.w2 = self.w13[:, : p.ffn_dim], self.w13[:, p.ffn_dim :], stack("w2")
        else:
            # no gate: the one stack of up matrices takes the first product's place
            self.w13 = self.w1 = stack("w3")
            self.w3, self.w2 = None, stack("w2")
        if self.shared is not None:
            self.shared.bind({local: tensors["shared." + local] for local in self.shared.names}, ops)
        self.router = tensors["router"].float().contiguous()
        self.correction = tensors["correction"].float().contiguous() if p.correction else None

    def forward(self, x, ctx):
        p, ops = self.params, self.ops
        logits = ops.moe_logits(x, self.router, ctx)
        groups = (*p.groups, p.group_top) if p.groups is not None else None
        ids, weights = ops.moe_route(logits, self.correction, p.top, ctx, renormalize=p.renormalize, score=p.score,
                                     groups=groups, renorm_eps=p.renorm_eps, weight_scale=p.weight_scale)
        out = ops.moe_experts(x, ids, weights, self.w1, self.w3, self.w2, self.w13,
                              act=None if self.gated else p.act)
        if self.shared is None:
            return out
        return ScaledSum([(out, 1.0), (self.shared.forward(x, ctx), 1.0)])


register_feed_forward("routed_experts", RoutedExperts)
