"""The gated delta rule: a linear-time mixer with a matrix state per head."""

from __future__ import annotations

from typing import List, Optional

import torch

from .base import Mixer, StateSpec, WeightSpec, register_mixer
from .params import GatedDeltaParams


def _pad8(n: int) -> int:
    return -(-n // 8) * 8


class GatedDeltaRule(Mixer):
    """``wo(norm(o) * sigmoid(gate))`` with ``o`` read from a state that forgets per key channel and
    is corrected towards each new value.

    Per token: q and k (``n_kv_heads`` heads of ``head_dim``) and v (``n_heads`` heads of
    ``v_head_dim``) are projections that pass a causal convolution per channel (``conv`` taps, the
    last one on the current token, no bias) and SiLU; q and k are then made unit vectors per head
    (``x / sqrt(sum x^2 + 1e-6)``) and q is multiplied by ``head_dim ** -0.5``.  Head ``h`` uses the
    q/k head ``h // (n_heads / n_kv_heads)``.  In float32, per head:

        g = exp(-exp(A_log[h]) softplus(a2 (a1 x) + dt_bias))      (one decay per key channel)
        S <- diag(g) S;  u = sigmoid(b x) (v - S^T k);  S <- S + k u^T;  o = S^T q

    so the read-out sees the token's own write.  ``o`` is divided by its root mean square per head
    (eps of the parameters), multiplied by ``norm`` (shared by the heads) and by
    ``sigmoid(g2 (g1 x))``.

    All small projections run as one product against ``[q; k; v; a1; g1; b]`` (every part padded to
    a multiple of 8 rows, so that the views handed on are aligned).  The request's state is
    fixed-size: S of every head ([heads][v_head_dim][head_dim]) and the convolutions' last
    ``conv - 1`` inputs, one float32 row per slot that the cache manager zeroes on admission.  The
    recurrence runs token by token in float32, so prompt portions, single tokens and mixed batches
    take the same kernels and give the same numbers however a prompt is cut.
    """

    params: GatedDeltaParams
    graph_safe = True

    def __init__(self, spec) -> None:
        super().__init__(spec)
        p = self.params
        self.qk_width = p.n_kv_heads * p.head_dim
        self.v_width = p.n_heads * p.v_head_dim
        self.decay_width = p.n_heads * p.head_dim
        self.state_floats = p.n_heads * p.v_head_dim * p.head_dim
        self.conv_floats = (p.conv - 1) * p.channels

    def weight_specs(self) -> List[WeightSpec]:
        p, n = self.params, self.names
        ra = p.decay_rank if p.decay_rank is not None else -1
        rg = p.gate_rank if p.gate_rank is not None else -1
        return [
            WeightSpec(n["wq"], (self.qk_width, p.dim)),
            WeightSpec(n["wk"], (self.qk_width, p.dim)),
            WeightSpec(n["wv"], (self.v_width, p.dim)),
            WeightSpec(n["conv_q"], (self.qk_width, p.conv), ("normal", 0.3)),
            WeightSpec(n["conv_k"], (self.qk_width, p.conv), ("normal", 0.3)),
            WeightSpec(n["conv_v"], (self.v_width, p.conv), ("normal", 0.3)),
            WeightSpec(n["wb"], (p.n_heads, p.dim)),
            WeightSpec(n["a_log"], (p.n_heads,), ("uniform", -2.0, 0.5)),
            WeightSpec(n["norm"], (p.v_head_dim,), ("ones",)),
            WeightSpec(n["wa1"], (ra, p.dim)),
            WeightSpec(n["wa2"], (self.decay_width, ra)),
            WeightSpec(n["dt_bias"], (self.decay_width,), ("uniform", -3.0, 0.5)),
            WeightSpec(n["wg1"], (rg, p.dim)),
            WeightSpec(n["wg2"], (self.v_width, rg)),
            WeightSpec(n["wo"], (p.dim, self.v_width)),
        ]

    def state_spec(self) -> Optional[StateSpec]:
        return StateSpec((self.state_floats + self.conv_floats,))

    def bind(self, tensors, ops) -> None:
        p = self.params
        self.ops = ops
        dt = ops.act_dtype
        parts = [tensors[n] for n in ("wq", "wk", "wv")]
        # q, k and v are read by the convolution as one run of channels: no padding between them
        qkv = torch.cat(parts, dim=0)
        self.ra, self.rg = tensors["wa1"].shape[0], tensors["wg1"].shape[0]
        if tensors["wa2"].shape[1] != self.ra or tensors["wg2"].shape[1] != self.rg:
            raise ValueError("the two maps of a low-rank projection disagree on the inner size")
        rows, self.offsets = [], {}
        at = 0
        for name, w in (("qkv", qkv), ("a1", tensors["wa1"]), ("g1", tensors["wg1"]), ("b", tensors["wb"])):
            self.offsets[name] = at
            pad = _pad8(w.shape[0]) - w.shape[0]
            rows.append(w)
            if pad:
                rows.append(w.new_zeros((pad, w.shape[1])))
            at += w.shape[0] + pad
        self.w_in = torch.cat(rows, dim=0).to(dt).contiguous()
        # the second maps read the padded inner columns too: zero columns for them
        self.wa2 = self._pad_cols(tensors["wa2"], _pad8(self.ra)).to(dt).contiguous()
        self.wg2 = self._pad_cols(tensors["wg2"], _pad8(self.rg)).to(dt).contiguous()
        self.wo = tensors["wo"].to(dt).contiguous()
        # what enters float32 arithmetic is float32 whatever it was stored in
        self.conv_w = torch.cat([tensors["conv_q"], tensors["conv_k"], tensors["conv_v"]], dim=0).float().contiguous()
        self.a_log = tensors["a_log"].float().contiguous()
        self.dt_bias = tensors["dt_bias"].float().contiguous()
        self.norm_w = tensors["norm"].float().contiguous()

    @staticmethod
    def _pad_cols(w: torch.Tensor, cols: int) -> torch.Tensor:
        if w.shape[1] == cols:
            return w
        out = w.new_zeros((w.shape[0], cols))
        out[:, : w.shape[1]] = w
        return out

    def forward(self, x, ctx, memory):
        p, ops = self.params, self.ops
        state = memory.state
        proj = ops.linear(x, self.w_in)  # [T, q k v | a1 | g1 | b]
        o = self.offsets
        qkv = ops.conv_silu(proj, o["qkv"], p.channels, self.conv_w, state, self.state_floats, p.conv, ctx)
        a = ops.linear(proj[:, o["a1"] : o["a1"] + _pad8(self.ra)], self.wa2)
        z = ops.linear(proj[:, o["g1"] : o["g1"] + _pad8(self.rg)], self.wg2)
        b = proj[:, o["b"] : o["b"] + p.n_heads]
        y = ops.delta_scan(qkv, a, b, self.dt_bias, self.a_log, state, ctx, p.n_heads, p.n_kv_heads, p.head_dim,
                           p.v_head_dim)
        g = ops.head_norm_gate(y, z, self.norm_w, p.n_heads, p.v_head_dim, p.eps, ctx)
        return ops.linear(g, self.wo)


register_mixer("gated_delta", GatedDeltaRule)
