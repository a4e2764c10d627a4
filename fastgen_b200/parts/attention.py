"""Grouped-query causal attention over the paged cache."""

from __future__ import annotations

from typing import List, Optional

import torch

from .base import CacheSpec, Mixer, StateSpec, WeightSpec, make_position, register_mixer
from .params import AttentionParams, SigmoidAttentionParams


def interleave_rope_rows(w: torch.Tensor, n_heads: int) -> torch.Tensor:
    """Reorder the rows of a q/k projection from the checkpoint's half-split
    rotary order to adjacent pairs: within a head, row ``2j`` <- row ``j`` and
    row ``2j+1`` <- row ``j + head_dim/2`` (the permutation the reference
    applies at load time, fastgen/utils/loading.py:296-305).  Scores are
    unchanged because queries and keys get the same permutation."""
    rows, cols = w.shape
    half = rows // n_heads // 2
    idx = torch.arange(rows, device=w.device).view(n_heads, 2, half)
    return w[idx.permute(0, 2, 1).reshape(-1)]


def pair_rows_adjacent(w: torch.Tensor, n_heads: int, rot_dims: int) -> torch.Tensor:
    """Reorder the rows of each head of ``w`` [heads * size, ...] so that the rotated pairs of the
    half-split layout, ``(i, i + rot_dims/2)`` among a head's first ``rot_dims`` rows, become the
    adjacent pairs ``(2i, 2i + 1)``; a head's other rows stay where they are."""
    size = w.shape[0] // n_heads
    half = rot_dims // 2
    within = torch.arange(size)
    within[: rot_dims : 2] = torch.arange(half)
    within[1 : rot_dims : 2] = torch.arange(half) + half
    idx = (torch.arange(n_heads)[:, None] * size + within[None, :]).reshape(-1)
    return w[idx.to(w.device)]


def pad_heads(w: torch.Tensor, n_heads: int, size: int) -> torch.Tensor:
    """Zero rows after each head of ``w`` [heads * s, ...] so that a head has ``size`` rows."""
    s = w.shape[0] // n_heads
    if s == size:
        return w
    out = w.new_zeros((n_heads, size, *w.shape[1:]))
    out[:, :s] = w.reshape(n_heads, s, *w.shape[1:])
    return out.reshape(n_heads * size, *w.shape[1:])


class GQAAttention(Mixer):
    """``wo(attention(rope(wq x), rope(wk x), wv x))`` (fastgen/forward.py:438-472).

    The three projections run as one product against ``[wq; wk; wv]`` built at
    bind time.  Keys and values of the step's tokens are written to this run's
    cache pages before attention reads them back, so a prompt portion attends to
    itself through the cache exactly as a decoded token does.

    Options of the parameters: biases on the four projections; an RMS norm of queries and of keys
    over their whole projection before the rotation; a cap on the scores; a value head size of its own
    (heads are padded with zero rows to one kernel head size, see
    ``AttentionParams.kernel_head_dim``); rotary encodings that turn a part of the head, in
    either pairing (half-split rows are reordered at bind time, which changes no score);
    values turned by their position on their way into the cache and outputs turned back by
    the query's position.  Further options: an RMS norm of queries and keys per head; values that are
    the keys as projected (no value projection); a query temperature that grows with the position; a
    sink per head in the softmax's denominator; a sigmoid gate per head on the output; a short causal
    convolution over time on q, k and v directly after the projection, whose last inputs are the
    request's fixed-size state beside its pages.
    """

    params: AttentionParams
    graph_safe = True

    def __init__(self, spec) -> None:
        super().__init__(spec)
        p = self.params
        self.position = make_position(p.position)
        self.value_position = make_position(p.value_position) if p.value_position is not None else None
        self.scale = p.softmax_scale if p.softmax_scale is not None else p.head_dim ** -0.5
        self.v_head_dim = p.v_head_dim or p.head_dim
        self.hd = p.kernel_head_dim
        self.q_width = p.n_heads * self.hd
        self.kv_width = p.n_kv_heads * self.hd
        self.o_bias = p.bias if p.o_bias is None else p.o_bias
        #: channels that pass the convolution: q, k and v as the kernels hold them (padded heads)
        self.conv_channels = self.q_width + 2 * self.kv_width
        #: the fused few-token kernel (projection, rotation, page write) knows none of these
        self.plain = not (p.qk_norm or p.q_temp or p.conv or p.head_gate)
        if p.q_temp and p.qk_norm == "projection":
            raise ValueError("a query temperature joins the per-head factors: not with a norm over the projection")

    def weight_specs(self) -> List[WeightSpec]:
        p = self.params
        q, k, v = p.n_heads * p.head_dim, p.n_kv_heads * p.head_dim, p.n_kv_heads * self.v_head_dim
        o = p.n_heads * self.v_head_dim
        specs = [
            WeightSpec(self.names["wq"], (q, p.dim)),
            WeightSpec(self.names["wk"], (k, p.dim)),
        ]
        if not p.shared_kv:
            specs.append(WeightSpec(self.names["wv"], (v, p.dim)))
        specs.append(WeightSpec(self.names["wo"], (p.dim, o)))
        if p.bias:
            specs += [
                WeightSpec(self.names["bq"], (q,)),
                WeightSpec(self.names["bk"], (k,)),
            ]
            if not p.shared_kv:
                specs.append(WeightSpec(self.names["bv"], (v,)))
            if self.o_bias:
                specs.append(WeightSpec(self.names["bo"], (p.dim,)))
        if p.qk_norm == "projection":
            specs += [
                WeightSpec(self.names["q_norm"], (q,), ("ones",)),
                WeightSpec(self.names["k_norm"], (k,), ("ones",)),
            ]
        elif p.qk_norm == "head":
            specs += [
                WeightSpec(self.names["q_norm"], (p.head_dim,), ("ones",)),
                WeightSpec(self.names["k_norm"], (p.head_dim,), ("ones",)),
            ]
        if p.sink:
            specs.append(WeightSpec(self.names["sink"], (p.n_heads,), ("normal", 1.0)))
        if p.head_gate:
            specs.append(WeightSpec(self.names["wg"], (p.n_heads, p.dim)))
        if p.conv:
            specs += [
                WeightSpec(self.names["conv_q"], (q, p.conv), ("normal", 0.3)),
                WeightSpec(self.names["conv_k"], (k, p.conv), ("normal", 0.3)),
                WeightSpec(self.names["conv_v"], (v, p.conv), ("normal", 0.3)),
            ]
        return specs

    def cache_spec(self) -> Optional[CacheSpec]:
        p = self.params
        return CacheSpec(p.n_kv_heads, self.hd, p.window, keep_first=p.keep_first if p.window else 0)

    def state_spec(self) -> Optional[StateSpec]:
        p = self.params
        if not p.conv:
            return None
        # the convolution's last inputs: conv - 1 rows of the projected q, k and v
        return StateSpec((max(1, p.conv - 1) * self.conv_channels,))

    def _rot_dims(self, position, size: int) -> int:
        params = getattr(position, "params", None)
        return getattr(params, "rot_dims", None) or size

    def _rows(self, t: torch.Tensor, n_heads: int, size: int, layout: str, position) -> torch.Tensor:
        """A projection's rows (or its bias) as the kernels want them: rotated pairs adjacent,
        heads padded to the kernel head size."""
        if layout == "half_split" and position is not None:
            t = pair_rows_adjacent(t, n_heads, self._rot_dims(position, size))
        return pad_heads(t, n_heads, self.hd)

    def bind(self, tensors, ops) -> None:
        p = self.params
        self.ops = ops
        dt = ops.act_dtype
        vd = self.v_head_dim
        rotates = not isinstance(self.position.table(ops.device), type(None))
        qk_pos = self.position if rotates else None
        if p.shared_kv:
            # the values are the keys as projected: the key rows once more, in the values' place
            tensors = dict(tensors, wv=tensors["wk"])
            if p.bias:
                tensors["bv"] = tensors["bk"]
        wq = self._rows(tensors["wq"], p.n_heads, p.head_dim, p.qk_layout, qk_pos)
        wk = self._rows(tensors["wk"], p.n_kv_heads, p.head_dim, p.qk_layout, qk_pos)
        wv = self._rows(tensors["wv"], p.n_kv_heads, vd, p.v_layout, self.value_position)
        parts = [wq, wk, wv]
        self.gate_rows = 0
        if p.head_gate:
            # the gate's rows ride in the same product (padded to whole groups of 8 rows)
            self.gate_rows = -(-p.n_heads // 8) * 8
            wg = tensors["wg"].new_zeros((self.gate_rows, p.dim))
            wg[: p.n_heads] = tensors["wg"]
            parts.append(wg)
        self.wqkv = torch.cat(parts, dim=0).to(dt).contiguous()
        # the output projection's columns follow the value heads' rows
        wo_t = self._rows(tensors["wo"].t(), p.n_heads, vd, p.v_layout, self.value_position)
        self.wo = wo_t.t().to(dt).contiguous()
        self.bqkv = self.bo = None
        if p.bias:
            bq = self._rows(tensors["bq"], p.n_heads, p.head_dim, p.qk_layout, qk_pos)
            bk = self._rows(tensors["bk"], p.n_kv_heads, p.head_dim, p.qk_layout, qk_pos)
            bv = self._rows(tensors["bv"], p.n_kv_heads, vd, p.v_layout, self.value_position)
            self.bqkv = torch.cat([bq, bk, bv, bq.new_zeros(self.gate_rows)], dim=0).to(dt).contiguous()
            self.bo = tensors["bo"].to(dt).contiguous() if self.o_bias else None
        self.q_norm = self.k_norm = None
        if p.qk_norm:
            # the norm's weights follow their projection's rows (a head's padding has weight zero);
            # they enter float32 arithmetic.  Weights of one head's size are shared by the heads.
            qn, kn = tensors["q_norm"], tensors["k_norm"]
            if p.qk_norm == "head":
                qn, kn = qn.repeat(p.n_heads), kn.repeat(p.n_kv_heads)
            self.q_norm = self._rows(qn, p.n_heads, p.head_dim, p.qk_layout, qk_pos).float().contiguous()
            self.k_norm = self._rows(kn, p.n_kv_heads, p.head_dim, p.qk_layout, qk_pos).float().contiguous()
        self.sinks = tensors["sink"].float().contiguous() if p.sink else None
        self.conv_w = None
        if p.conv:
            self.conv_w = torch.cat([
                self._rows(tensors["conv_q"], p.n_heads, p.head_dim, p.qk_layout, qk_pos),
                self._rows(tensors["conv_k"], p.n_kv_heads, p.head_dim, p.qk_layout, qk_pos),
                self._rows(tensors["conv_v"], p.n_kv_heads, vd, p.v_layout, self.value_position),
            ], dim=0).float().contiguous()
        self.freqs = self._table(self.position)
        self.v_freqs = self.v_unfreqs = None
        if self.value_position is not None:
            self.v_freqs = self._table(self.value_position)
            if self.v_freqs is not None:
                self.v_unfreqs = (-self.v_freqs).contiguous()

    def _table(self, position) -> Optional[torch.Tensor]:
        """A position encoding's frequency table over the kernel head size: the pairs of a
        head's padding have frequency zero."""
        table = position.table(self.ops.device)
        if table is not None and table.numel() < self.hd // 2:
            table = torch.cat([table, table.new_zeros(self.hd // 2 - table.numel())]).contiguous()
        return table

    def _attend(self, q, o, ctx, memory) -> bool:
        """Attention of the step's tokens into ``o``.  Returns whether the outputs have been turned
        back already (values cached turned by their positions): the kernels do it where they can."""
        p = self.params
        return self.ops.attention(q, o, memory, ctx, p.n_heads, p.n_kv_heads, self.hd, p.window, self.scale,
                                  out_freqs=self.v_unfreqs, keep_first=p.keep_first, softcap=p.softcap,
                                  sinks=self.sinks)

    def forward(self, x, ctx, memory):
        p, ops = self.params, self.ops
        t = x.shape[0]
        q = None
        gate = None
        if memory.writes and x.dtype == torch.bfloat16 and self.plain:
            # a few tokens: projection, rotation and page write in one kernel
            q = ops.qkv_rope_write(x, self.wqkv, ctx.pos, ctx.req, self.freqs, memory,
                                   p.n_heads, p.n_kv_heads, self.hd, bias=self.bqkv, v_freqs=self.v_freqs)
        if q is None:
            if memory.writes:
                qkv = ops.linear(x, self.wqkv, bias=self.bqkv)
                if p.head_gate:
                    gate = qkv[:, self.conv_channels : self.conv_channels + p.n_heads]
                if p.conv:
                    # the convolution reads the projected rows (and the state's last ones) and gives
                    # q, k and v in the compute type
                    qkv = ops.time_conv(qkv, 0, self.conv_channels, self.conv_w, None, memory.state, 0, p.conv, ctx,
                                        out_dtype=x.dtype)
                q = qkv[:, : self.q_width]
                k = qkv[:, self.q_width : self.q_width + self.kv_width]
                v = qkv[:, self.q_width + self.kv_width : self.q_width + 2 * self.kv_width]
            else:
                # this run reads another run's cache: only queries are needed
                if p.conv or p.head_gate or p.qk_norm == "head" or p.q_temp:
                    raise NotImplementedError("a run that reads another run's cache takes plain queries")
                bq = self.bqkv[: self.q_width] if self.bqkv is not None else None
                q = ops.linear(x, self.wqkv[: self.q_width], bias=bq)
                k = v = None
            qk_norm = None
            if p.qk_norm == "head" or p.q_temp:
                # a factor per (token, head): the head's RMS norm and, for queries, the temperature of
                # the token's position; the kernel that rotates multiplies by them and by the weights
                factors = ops.qk_head_factors(q, k, ctx.pos, ctx.req, p.n_heads, p.n_kv_heads, self.hd, p.head_dim,
                                              norm_eps=p.qk_norm_eps if p.qk_norm else None, temp=p.q_temp)
                qk_norm = (factors, self.q_norm, self.k_norm)
            elif p.qk_norm:
                # a norm over the whole projection: the token's two factors first, then the kernel
                # that rotates multiplies by them and by the weights
                rstd = ops.qk_rstd(q, k, p.n_heads * p.head_dim, p.n_kv_heads * p.head_dim, p.qk_norm_eps, ctx.req)
                qk_norm = (rstd, self.q_norm, self.k_norm)
            ops.rope_kv_write(
                q, k, v, ctx.pos, ctx.req, self.freqs, memory.k_pages, memory.v_pages,
                memory.block_table, memory.page_size, p.n_heads, p.n_kv_heads, self.hd, v_freqs=self.v_freqs,
                qk_norm=qk_norm,
            )
        o = torch.empty((t, self.q_width), dtype=x.dtype, device=x.device)
        turned = self._attend(q, o, ctx, memory)
        if self.v_unfreqs is not None and not turned:
            # the sum over values that were turned by their own positions is turned back by the query's
            ops.rotate_heads(o, ctx.pos, ctx.req, self.v_unfreqs, p.n_heads, self.hd)
        if gate is not None:
            ops.head_gate(o, gate, ctx.req, p.n_heads, self.hd)
        return ops.linear(o, self.wo, bias=self.bo)


class SigmoidAttention(GQAAttention):
    """Attention with sigmoid weights that are not normalised over the keys:
    ``sum_j sigmoid(q.k_j * scale + gate_h - r1_h ln(1 + r2_h (i - j))) v_j`` over the visible
    keys (causal, with the window of the parameters).  Projections, cache and options are
    those of :class:`GQAAttention`; the per-head numbers are the tensors ``gate``, ``r1``, ``r2``."""

    params: SigmoidAttentionParams

    def weight_specs(self) -> List[WeightSpec]:
        p = self.params
        specs = super().weight_specs()
        if p.distance_bias:
            specs += [
                WeightSpec(self.names["r1"], (p.n_heads,), ("ones",)),
                WeightSpec(self.names["r2"], (p.n_heads,), ("ones",)),
            ]
        if p.gate:
            specs.append(WeightSpec(self.names["gate"], (p.n_heads,), ("normal", 0.5)))
        return specs

    def bind(self, tensors, ops) -> None:
        super().bind(tensors, ops)
        p = self.params
        self.r1 = tensors["r1"].float().contiguous() if p.distance_bias else None
        self.r2 = tensors["r2"].float().contiguous() if p.distance_bias else None
        self.gate = tensors["gate"].float().contiguous() if p.gate else None

    def _attend(self, q, o, ctx, memory) -> bool:
        p = self.params
        self.ops.attention_sigmoid(q, o, memory, ctx, p.n_heads, p.n_kv_heads, self.hd, p.window, self.scale,
                                   gate=self.gate, r1=self.r1, r2=self.r2)
        return False


register_mixer("gqa_attention", GQAAttention)
register_mixer("sigmoid_attention", SigmoidAttention)
