"""Griffin's recurrent block: a gated branch beside a convolved branch that feeds the real-gated
linear recurrent unit."""

from __future__ import annotations

from typing import List, Optional

import torch

from .base import Mixer, StateSpec, WeightSpec, register_mixer
from .params import GatedLinearRecurrenceParams


class GatedLinearRecurrence(Mixer):
    """``wo(S * y)`` with two branches of ``width`` channels:

        y = gelu_tanh(wy x + by)
        u = conv(wx x + bx)          (causal, per channel, ``conv`` taps, bias, no activation)
        r = sigmoid(ra[b] u_b + ra_b),  i = sigmoid(ri[b] u_b + ri_b)      (u in ``blocks`` equal parts)
        a = exp(-decay * r * softplus(lam));   S <- a S + sqrt(1 - a^2) * i * u       (float32, S starts at 0)

    The two gate maps of a block run as one product against ``[ra[b]; ri[b]]`` with float32 results.
    The request's state is one float32 row per slot, zeroed on admission: S, then the convolution's
    last ``conv - 1`` inputs.  The recurrence runs token by token in float32, so prompt portions, single
    tokens and mixed batches take the same kernels and give the same numbers however a prompt is cut.
    """

    params: GatedLinearRecurrenceParams
    graph_safe = True

    def weight_specs(self) -> List[WeightSpec]:
        p, n = self.params, self.names
        bw = p.width // p.blocks
        return [
            WeightSpec(n["wy"], (p.width, p.dim)),
            WeightSpec(n["by"], (p.width,)),
            WeightSpec(n["wx"], (p.width, p.dim)),
            WeightSpec(n["bx"], (p.width,)),
            WeightSpec(n["conv"], (p.width, p.conv), ("normal", 0.3)),
            WeightSpec(n["conv_b"], (p.width,)),
            WeightSpec(n["ra"], (p.blocks, bw, bw), ("normal", 0.1)),
            WeightSpec(n["ra_b"], (p.blocks, bw), ("normal", 0.5)),
            WeightSpec(n["ri"], (p.blocks, bw, bw), ("normal", 0.1)),
            WeightSpec(n["ri_b"], (p.blocks, bw), ("normal", 0.5)),
            WeightSpec(n["lam"], (p.width,), ("uniform", -4.0, 0.0)),
            WeightSpec(n["wo"], (p.dim, p.width)),
        ]

    def state_spec(self) -> Optional[StateSpec]:
        p = self.params
        return StateSpec((p.width + max(1, p.conv - 1) * p.width,))

    def bind(self, tensors, ops) -> None:
        p = self.params
        self.ops = ops
        dt = ops.act_dtype
        self.wy, self.by = tensors["wy"].to(dt).contiguous(), tensors["by"].to(dt).contiguous()
        self.wx, self.bx = tensors["wx"].to(dt).contiguous(), tensors["bx"].to(dt).contiguous()
        self.wo = tensors["wo"].to(dt).contiguous()
        # a block's two gate maps as one matrix [2 bw, bw]; the batched library product wants [bw, 2 bw]
        self.w_gates = torch.cat([tensors["ra"], tensors["ri"]], dim=1).to(dt).contiguous()
        self.w_gates_t = self.w_gates.transpose(1, 2).contiguous()
        # what enters float32 arithmetic is float32 whatever it was stored in
        self.conv_w = tensors["conv"].float().contiguous()
        self.conv_b = tensors["conv_b"].float().contiguous()
        self.bias_r = tensors["ra_b"].float().reshape(-1).contiguous()
        self.bias_i = tensors["ri_b"].float().reshape(-1).contiguous()
        lam = tensors["lam"].float()
        softplus = torch.where(lam > 20.0, lam, torch.log1p(torch.exp(torch.clamp(lam, max=20.0))))
        self.neg_rate = (-float(p.decay) * softplus).contiguous()

    def forward(self, x, ctx, memory):
        p, ops = self.params, self.ops
        state = memory.state
        y = ops.linear(x, self.wy, bias=self.by, act="gelu_tanh")
        xb = ops.linear(x, self.wx, bias=self.bx)
        u = ops.time_conv(xb, 0, p.width, self.conv_w, self.conv_b, state, p.width, p.conv, ctx, out_dtype=x.dtype)
        gates = ops.block_products(u.view(u.shape[0], p.blocks, p.width // p.blocks), self.w_gates_t, self.w_gates)
        out = ops.rglru_scan(gates, u, self.bias_r, self.bias_i, self.neg_rate, y, state, 0, ctx, p.blocks)
        return ops.linear(out, self.wo)


register_mixer("gated_linear_recurrence", GatedLinearRecurrence)
