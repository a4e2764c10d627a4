"""Two mixers that read the same input side by side."""

from __future__ import annotations

from typing import List, Optional

import torch

from .base import CacheSpec, Mixer, ScaledSum, StateSpec, WeightSpec, make_mixer, make_norm, register_mixer
from .params import SideBySideParams


class SideBySide(Mixer):
    """``left_scale * left(x) + right_scale * right(x)`` for two mixers of any registered kinds.

    The layer has one cache and one state, so at most one of the two may cache per-token entries
    and at most one may keep a fixed-size state: both are handed the layer's memory and each takes
    from it what it asked for.  The result is returned as a sum that has not been formed (a
    :class:`~fastgen_b200.parts.base.ScaledSum`): the kernel that adds it to the residual stream
    multiplies the two outputs by their scales in float32.  With ``left_norm`` / ``right_norm`` an
    output passes a norm of its own first (its result stays float32 on its way into the sum).
    """

    params: SideBySideParams

    def __init__(self, spec) -> None:
        super().__init__(spec)
        p = self.params
        self.left = make_mixer(p.left)
        self.right = make_mixer(p.right)
        self.left_norm = make_norm(p.left_norm) if p.left_norm is not None else None
        self.right_norm = make_norm(p.right_norm) if p.right_norm is not None else None
        for what in ("cache_spec", "state_spec"):
            if getattr(self.left, what)() is not None and getattr(self.right, what)() is not None:
                raise ValueError(f"both mixers of a side-by-side pair ask for a {what.split('_')[0]}: a layer has one")
        self.graph_safe = self.left.graph_safe and self.right.graph_safe

    def weight_specs(self) -> List[WeightSpec]:
        specs = self.left.weight_specs() + self.right.weight_specs()
        for norm in (self.left_norm, self.right_norm):
            if norm is not None:
                specs += norm.weight_specs()
        return specs

    def cache_spec(self) -> Optional[CacheSpec]:
        return self.left.cache_spec() or self.right.cache_spec()

    def state_spec(self) -> Optional[StateSpec]:
        return self.left.state_spec() or self.right.state_spec()

    def bind(self, tensors, ops) -> None:
        # the two mixers' tensors arrive under their checkpoint names (see ``names`` below)
        self.left.bind({local: tensors["left." + local] for local in self.left.names}, ops)
        self.right.bind({local: tensors["right." + local] for local in self.right.names}, ops)
        if self.left_norm is not None:
            self.left_norm.bind({local: tensors["left_norm." + local] for local in self.left_norm.names}, ops)
        if self.right_norm is not None:
            self.right_norm.bind({local: tensors["right_norm." + local] for local in self.right_norm.names}, ops)

    @property
    def names(self):
        out = {"left." + k: v for k, v in self.left.names.items()}
        out.update({"right." + k: v for k, v in self.right.names.items()})
        if self.left_norm is not None:
            out.update({"left_norm." + k: v for k, v in self.left_norm.names.items()})
        if self.right_norm is not None:
            out.update({"right_norm." + k: v for k, v in self.right_norm.names.items()})
        return out

    @names.setter
    def names(self, value) -> None:  # the pair has no tensors of its own
        pass

    def forward(self, x, ctx, memory):
        p = self.params
        left = self.left.forward(x, ctx, memory)
        right = self.right.forward(x, ctx, memory)
        if self.left_norm is not None:
            left = self.left_norm.forward(left, out_dtype=torch.float32)
        if self.right_norm is not None:
            right = self.right_norm.forward(right, out_dtype=torch.float32)
        return ScaledSum.of(left, p.left_scale).plus(ScaledSum.of(right, p.right_scale))


register_mixer("side_by_side", SideBySide)
