"""Interfaces of the parts a layer is put together from, and their registries.

A part is built from a :class:`~fastgen_b200.config.PartSpec` alone: it knows
its own sizes, constants and tensor names and nothing about the model around it.
Parts are looked up by ``spec.kind`` in one registry per role, so a new mixer,
feed-forward, norm, position encoding or block arrangement is one ``register_*``
call and needs no change to the files of this package.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, List, Mapping, Optional, Sequence, Tuple

import torch

from ..config.model_args import PartSpec


@dataclass(frozen=True)
class WeightSpec:
    """One checkpoint tensor a part needs.

    ``init`` is the law the random-weights writer draws it from:
    ``("normal", std)``, ``("ones",)``, ``("ones_jitter", half_width)`` for
    ``1 + U(-w, w)``, or ``("randint", high)`` for integer tables.
    ``integer`` tensors are kept as int32; others follow the compute dtype
    unless the file stores them in 32-bit (see ``weights.loader``).  A size of -1 in
    ``shape`` stands for "whatever the checkpoint has" (the part reads it when it binds);
    the random-weights writer needs every size.
    """

    name: str
    shape: Tuple[int, ...]
    init: tuple = ("normal", 0.02)
    integer: bool = False


@dataclass(frozen=True)
class CacheSpec:
    """What a mixer that caches per-token entries needs per token.

    The usual case is keys and values: two pools of ``[pages, n_kv_heads, page, head_dim]``.
    ``n_pools = 1`` asks for one pool only (a mixer that keeps one entry per token, say a
    compressed one from which it makes keys and values itself); ``page_size`` asks for pages
    of that many tokens instead of the engine's.  Runs with equal specs share a group of
    pages; every group has its own pool of page ids and its own block table per request.
    """

    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None  # keys a query may see, itself included
    n_pools: int = 2  # 2: keys and values; 1: one entry per token
    page_size: Optional[int] = None  # tokens per page; None: the engine's page size
    keep_first: int = 0  # with a window: a sequence's first positions that stay visible for good

    def __post_init__(self) -> None:
        if self.n_pools not in (1, 2):
            raise ValueError(f"a cache spec asks for 1 or 2 pools, got {self.n_pools}")
        if self.page_size is not None and self.page_size <= 0:
            raise ValueError(f"page size must be positive, got {self.page_size}")


@dataclass(frozen=True)
class StateSpec:
    """Fixed-size per-request state of a mixer or of the embedder (zeroed on admission;
    float32 unless ``dtype`` says otherwise)."""

    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


class Part:
    """Common base: weights are declared, then bound once they are on device."""

    def __init__(self, spec: PartSpec) -> None:
        self.spec = spec
        self.params = spec.params
        self.names = dict(spec.names)

    def weight_specs(self) -> List[WeightSpec]:
        return []

    def bind(self, tensors: Mapping[str, torch.Tensor], ops) -> None:
        """Receive the loaded tensors, keyed by local name, and the kernel set
        (``ops``) of the compute dtype.  Fused buffers are built here."""

    def tied_name(self, local: str) -> str:
        return self.names[local]


class Norm(Part):
    def _joined(self, h, total, rows):
        """For norms whose kernel does not take a :class:`ScaledSum`: add it to ``h`` with the kernel
        that does (needs ``self.ops``) and return ``None``; with ``rows`` (``h`` must stay as it
        was) the sum is formed beside ``h`` and returned as the one summand."""
        if rows is None:
            total.add_into(h, self.ops)
            return None
        delta = torch.zeros_like(h)
        total.add_into(delta, self.ops)
        return delta

    def forward(self, x: torch.Tensor, out_dtype=None, rows=None) -> torch.Tensor:
        """Normalise rows of ``x`` [T, dim] (only the rows indexed by the int32
        tensor ``rows`` when it is given)."""
        raise NotImplementedError

    def add_forward(self, h: torch.Tensor, delta: Optional[torch.Tensor], rows=None,
                    delta_norm: Optional["Norm"] = None) -> torch.Tensor:
        """``h += delta`` (32-bit sum; ``delta`` may be ``None``) and return
        ``norm(h)``.  With ``delta_norm`` the summand is ``delta_norm(delta)``: the
        norm that closes a sub-layer whose output is normed before it joins the
        residual stream.  With ``rows`` only those rows are computed and ``h`` may
        be left as it was.

        The default composes the steps; implementations may fuse them."""
        if isinstance(delta, ScaledSum):
            delta = self._joined(h, delta, rows)
        if delta is not None:
            if delta_norm is not None:
                delta = delta_norm.forward(delta, out_dtype=torch.float32)
            if rows is not None:
                h = h.index_select(0, rows.long()) + delta.index_select(0, rows.long()).to(h.dtype)
                return self.forward(h)
            h.add_(delta.to(h.dtype))
        return self.forward(h, rows=rows)


@dataclass
class ScaledSum:
    """A sum that has not been formed yet: ``row + sum_i coef_i * term_i`` with ``terms`` a list of
    ``(tensor [T, dim], coef)`` and ``row`` a float32 [dim] vector that joins every token (or
    ``None``).  Blocks whose sub-layers read one norm side by side hand it on as ``pending``, so
    that one kernel adds everything to the residual stream and norms the result."""

    terms: list
    row: Optional[torch.Tensor] = None

    @staticmethod
    def of(pending, coef: float = 1.0) -> "ScaledSum":
        """``coef * pending`` as a sum: a tensor becomes its one term, a sum is multiplied through."""
        if pending is None:
            return ScaledSum([])
        if isinstance(pending, ScaledSum):
            if pending.row is not None and coef != 1.0:
                raise ValueError("a sum with a row vector cannot be multiplied")
            return ScaledSum([(t, c * coef) for t, c in pending.terms], pending.row)
        if isinstance(pending, torch.Tensor):
            return ScaledSum([(pending, coef)])
        raise TypeError(f"{type(pending).__name__} cannot join a scaled sum")

    def plus(self, other: "ScaledSum") -> "ScaledSum":
        if self.row is not None and other.row is not None:
            raise ValueError("two row vectors in one sum")
        return ScaledSum(self.terms + other.terms, self.row if self.row is not None else other.row)

    def add_into(self, h: torch.Tensor, ops) -> None:
        """``h += the sum`` (no norm): for norms whose own kernel does not take such a sum."""
        terms = list(self.terms)
        row = self.row
        while terms or row is not None:
            ops.rmsnorm_sum(h, terms[:4], None, 0.0, row=row)
            terms, row = terms[4:], None


@dataclass
class NormedDelta:
    """A summand that has not joined the residual stream yet, with the norm it passes
    through on its way (``None``: none).  Blocks hand it on as ``pending`` so that the sum
    can be fused with the next norm."""

    delta: torch.Tensor
    norm: Optional[Norm] = None


@dataclass
class StreamUpdate:
    """A sub-layer's output on its way into several residual streams: every stream becomes a
    mix of the old streams plus its own multiple of ``delta``
    (``x_t <- sum_s mix[s, t] x_s + out[t] delta``; ``None`` stands for the identity mix and for
    ones).  Handed on as ``pending`` so that the update is fused with the next read."""

    delta: torch.Tensor
    mix: Optional[torch.Tensor] = None
    out: Optional[torch.Tensor] = None


def split_pending(pending):
    """``(delta, its norm)`` of what a block handed on: a tensor, a :class:`NormedDelta` or ``None``."""
    if isinstance(pending, NormedDelta):
        return pending.delta, pending.norm
    return pending, None


class PositionEncoding(Part):
    """Position encoding of queries and keys.

    ``table()`` returns what the mixer's kernels need (for rotary encodings a
    float32 frequency table of ``head_dim/2`` entries, or ``None`` for no
    rotation)."""

    def table(self, device) -> Optional[torch.Tensor]:
        raise NotImplementedError


class Embedder(Part):
    """From token ids to the first residual stream.  ``forward`` fills ``out`` [T, dim]
    (float32) for the step's tokens; an embedder that keeps something per request between
    steps says so with ``state_spec`` and finds it in ``state`` (indexed by slot)."""

    def state_spec(self) -> Optional[StateSpec]:
        return None

    def table(self) -> torch.Tensor:
        """The token table [vocab, dim] (what a tied output projection uses)."""
        raise NotImplementedError

    def forward(self, ctx, state: Optional[torch.Tensor], out: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class Mixer(Part):
    #: whether ``forward`` only launches work that a CUDA graph may capture and
    #: copes with padding lanes (slot -1).  Steps of a model with a mixer that
    #: does not say so are never captured.
    graph_safe = False

    def cache_spec(self) -> Optional[CacheSpec]:
        return None

    def state_spec(self) -> Optional[StateSpec]:
        return None

    def forward(self, x: torch.Tensor, ctx, memory) -> torch.Tensor:
        """Mix tokens.  ``x`` is [T, dim] (normed), ``ctx`` the step's
        :class:`~fastgen_b200.engine.step.StepContext` and ``memory`` this
        run's :class:`~fastgen_b200.cache.LayerMemory`."""
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        raise NotImplementedError


class Connection(Part):
    """How a sub-layer is wired to the residual stream(s) ``h`` [T, streams, dim].

    ``read`` applies what the sub-layer before left pending, forms this sub-layer's input from
    the streams and returns its norm; ``write`` wraps the sub-layer's output as the pending
    update of the streams."""

    def read(self, h: torch.Tensor, pending, norm: "Norm") -> torch.Tensor:
        raise NotImplementedError

    def write(self, delta: torch.Tensor):
        raise NotImplementedError


class Block:
    """Arrangement of a layer's parts around the residual stream."""

    def __init__(self, mixer: Mixer, mixer_norm: Norm, ffn: Optional[FeedForward], ffn_norm: Optional[Norm],
                 params=None, **extra: Part):
        #: the arrangement's own constants (``LayerSpec.block_params``), or ``None``
        self.params = params
        self.mixer = mixer
        self.mixer_norm = mixer_norm
        self.ffn = ffn
        self.ffn_norm = ffn_norm
        #: further parts by name (``LayerSpec.extra``), for arrangements with more than four
        self.extra: Dict[str, Part] = dict(extra)

    def parts(self) -> Sequence[Part]:
        parts = (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn, *self.extra.values())
        return tuple(p for p in parts if p is not None)

    def forward(self, h, pending, ctx, memory):
        """Run the layer.  ``h`` is the residual stream [T, dim] (float32) and
        ``pending`` a delta not yet added to it (or ``None``); returns the new
        ``(h, pending)`` so that the sum can be fused with the next norm."""
        raise NotImplementedError


_MIXERS: Dict[str, Callable[[PartSpec], Mixer]] = {}
_FEED_FORWARDS: Dict[str, Callable[[PartSpec], FeedForward]] = {}
_NORMS: Dict[str, Callable[[PartSpec], Norm]] = {}
_POSITIONS: Dict[str, Callable[[PartSpec], PositionEncoding]] = {}
_BLOCKS: Dict[str, Callable[..., Block]] = {}
_EMBEDDERS: Dict[str, Callable[[PartSpec], Embedder]] = {}
_CONNECTIONS: Dict[str, Callable[[PartSpec], Connection]] = {}


def register_connection(kind: str, factory) -> None:
    _CONNECTIONS[kind] = factory


def make_connection(spec: PartSpec) -> Connection:
    return _make(_CONNECTIONS, "connection", spec)


def register_embedder(kind: str, factory) -> None:
    _EMBEDDERS[kind] = factory


def make_embedder(spec: PartSpec) -> Embedder:
    return _make(_EMBEDDERS, "embedder", spec)


def register_mixer(kind: str, factory) -> None:
    _MIXERS[kind] = factory


def register_feed_forward(kind: str, factory) -> None:
    _FEED_FORWARDS[kind] = factory


def register_norm(kind: str, factory) -> None:
    _NORMS[kind] = factory


def register_position(kind: str, factory) -> None:
    _POSITIONS[kind] = factory


def register_block(kind: str, factory) -> None:
    _BLOCKS[kind] = factory


def _make(table, role: str, spec: PartSpec):
    factory = table.get(spec.kind)
    if factory is None:
        raise KeyError(
            f"no {role} of kind {spec.kind!r} is registered; known: {sorted(table)}"
        )
    return factory(spec)


def make_mixer(spec: PartSpec) -> Mixer:
    return _make(_MIXERS, "mixer", spec)


def make_feed_forward(spec: PartSpec) -> FeedForward:
    return _make(_FEED_FORWARDS, "feed-forward", spec)


def make_norm(spec: PartSpec) -> Norm:
    return _make(_NORMS, "norm", spec)


def make_position(spec: PartSpec) -> PositionEncoding:
    return _make(_POSITIONS, "position encoding", spec)


def make_block(kind: str, mixer, mixer_norm, ffn, ffn_norm, params=None, **extra) -> Block:
    factory = _BLOCKS.get(kind)
    if factory is None:
        raise KeyError(f"no block of kind {kind!r} is registered; known: {sorted(_BLOCKS)}")
    if params is not None:
        extra["params"] = params
    return factory(mixer, mixer_norm, ffn, ffn_norm, **extra)
