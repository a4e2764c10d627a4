"""The matrix memory with exponential gates (the mLSTM of xLSTM): a linear-time mixer with a matrix
state, a normaliser vector and a running maximum per head."""

from __future__ import annotations

from typing import List, Optional

import torch

from .base import Mixer, StateSpec, WeightSpec, register_mixer
from .params import MatrixMemoryParams


def _pad8(n: int) -> int:
    return -(-n // 8) * 8


class MatrixMemory(Mixer):
    """``wo(norm_h(o) * w * sigmoid(wg x))`` with ``o`` read from a matrix state per head.

    Per token and head (``head_dim`` = d, ``v_head_dim`` = dv), in float32:

        q = wq x * d^-1/2,  k = wk x,  v = wv x
        i = cap tanh((wi x + bi) / cap),   f = logsigmoid(cap tanh((wf x + bf) / cap))
        m' = max(f + m, i)                                   (m starts at 0, not at minus infinity)
        S <- exp(f + m - m') S + exp(i - m') k v^T;   n <- exp(f + m - m') n + exp(i - m') k
        o = S^T q / (max(|n . q|, exp(-m')) + 1e-6)

    ``o`` is divided by its root mean square per head (eps of the parameters), multiplied by ``norm``
    (a weight over all heads' columns) and by ``sigmoid(wg x)``.

    q, k, v and the output gate run as one product against ``[wq; wk; wv; wg]``.  The two gates' sums
    are float32 sums of their own (everything that enters the recurrence besides the projections is
    32-bit), from a kernel that keeps a token's sums independent of the batch.  The request's state is
    fixed-size, one float32 row per slot that the cache manager zeroes on admission: S with n as one
    more column, and the running maxima.  The recurrence runs token by token, so prompt portions,
    single tokens and mixed batches take the same kernels and give the same numbers however a prompt
    is cut.
    """

    params: MatrixMemoryParams
    graph_safe = True

    def __init__(self, spec) -> None:
        super().__init__(spec)
        p = self.params
        self.qk_width = p.n_heads * p.head_dim
        self.v_width = p.n_heads * p.v_head_dim

    def weight_specs(self) -> List[WeightSpec]:
        p, n = self.params, self.names
        return [
            WeightSpec(n["wq"], (self.qk_width, p.dim)),
            WeightSpec(n["wk"], (self.qk_width, p.dim)),
            WeightSpec(n["wv"], (self.v_width, p.dim)),
            WeightSpec(n["wg"], (self.v_width, p.dim)),
            WeightSpec(n["wo"], (p.dim, self.v_width)),
            WeightSpec(n["norm"], (self.v_width,), ("ones",)),
            WeightSpec(n["wi"], (p.n_heads, p.dim), ("normal", 0.1)),
            WeightSpec(n["bi"], (p.n_heads,), ("normal", 1.0)),
            WeightSpec(n["wf"], (p.n_heads, p.dim), ("normal", 0.1)),
            WeightSpec(n["bf"], (p.n_heads,), ("uniform", 1.0, 4.0)),
        ]

    def state_spec(self) -> Optional[StateSpec]:
        p = self.params
        # [heads][dv + 1][d] (column dv: the normaliser), then the heads' running maxima
        return StateSpec((p.n_heads * (p.v_head_dim + 1) * p.head_dim + p.n_heads,))

    def bind(self, tensors, ops) -> None:
        p = self.params
        self.ops = ops
        dt = ops.act_dtype
        rows, self.offsets, at = [], {}, 0
        for name in ("wq", "wk", "wv", "wg"):
            w = tensors[name]
            self.offsets[name] = at
            pad = _pad8(w.shape[0]) - w.shape[0]  # so that the views handed on are aligned
            rows.append(w)
            if pad:
                rows.append(w.new_zeros((pad, w.shape[1])))
            at += w.shape[0] + pad
        self.w_in = torch.cat(rows, dim=0).to(dt).contiguous()
        self.wo = tensors["wo"].to(dt).contiguous()
        # what enters float32 arithmetic is float32 whatever it was stored in
        self.w_gates = torch.cat([tensors["wi"], tensors["wf"]], dim=0).float().contiguous()
        self.b_gates = torch.cat([tensors["bi"], tensors["bf"]], dim=0).float().contiguous()
        self.norm_w = tensors["norm"].float().contiguous()

    def forward(self, x, ctx, memory):
        p, ops = self.params, self.ops
        proj = ops.linear(x, self.w_in)  # [T, q | k | v | g]
        o = self.offsets
        q = proj[:, o["wq"] : o["wq"] + self.qk_width]
        k = proj[:, o["wk"] : o["wk"] + self.qk_width]
        v = proj[:, o["wv"] : o["wv"] + self.v_width]
        z = proj[:, o["wg"] : o["wg"] + self.v_width]
        gates = ops.moe_logits(x, self.w_gates, ctx)  # float32 [T, 2 heads]: input gates, forget gates
        y, coef = ops.mlstm_scan(gates, self.b_gates, p.gate_cap, q, k, v, memory.state, ctx, p.n_heads, p.head_dim,
                                 p.v_head_dim, p.head_dim ** -0.5)
        g = ops.mlstm_out(y, coef, z, self.norm_w, p.n_heads, p.v_head_dim, p.eps, ctx)
        return ops.linear(g, self.wo)


register_mixer("matrix_memory", MatrixMemory)
