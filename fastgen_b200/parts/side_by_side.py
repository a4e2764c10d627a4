"""Two mixers that read the same input side by side."""

from __future__ import annotations

from typing import List, Optional

from .base import CacheSpec, Mixer, ScaledSum, StateSpec, WeightSpec, make_mixer, register_mixer
from .params import SideBySideParams


class SideBySide(Mixer):
    """``left_scale * left(x) + right_scale * right(x)`` for two mixers of any registered kinds.

    The layer has one cache and one state, so at most one of the two may cache per-token entries
    and at most one may keep a fixed-size state: both are handed the layer's memory and each takes
    from it what it asked for.  The result is returned as a sum that has not been formed (a
    :class:`~fastgen_b200.parts.base.ScaledSum`): the kernel that adds it to the residual stream
    multiplies the two outputs by their scales in float32.
    """

    params: SideBySideParams

    def __init__(self, spec) -> None:
        super().__init__(spec)
        p = self.params
        self.left = make_mixer(p.left)
        self.right = make_mixer(p.right)
        for what in ("cache_spec", "state_spec"):
            if getattr(self.left, what)() is not None and getattr(self.right, what)() is not None:
                raise ValueError(f"both mixers of a side-by-side pair ask for a {what.split('_')[0]}: a layer has one")
        self.graph_safe = self.left.graph_safe and self.right.graph_safe

    def weight_specs(self) -> List[WeightSpec]:
        return self.left.weight_specs() + self.right.weight_specs()

    def cache_spec(self) -> Optional[CacheSpec]:
        return self.left.cache_spec() or self.right.cache_spec()

    def state_spec(self) -> Optional[StateSpec]:
        return self.left.state_spec() or self.right.state_spec()

    def bind(self, tensors, ops) -> None:
        # the two mixers' tensors arrive under their checkpoint names (see ``names`` below)
        self.left.bind({local: tensors["left." + local] for local in self.left.names}, ops)
        self.right.bind({local: tensors["right." + local] for local in self.right.names}, ops)

    @property
    def names(self):
        out = {"left." + k: v for k, v in self.left.names.items()}
        out.update({"right." + k: v for k, v in self.right.names.items()})
        return out

    @names.setter
    def names(self, value) -> None:  # the pair has no tensors of its own
        pass

    def forward(self, x, ctx, memory):
        p = self.params
        left = ScaledSum.of(self.left.forward(x, ctx, memory), p.left_scale)
        return left.plus(ScaledSum.of(self.right.forward(x, ctx, memory), p.right_scale))


register_mixer("side_by_side", SideBySide)
