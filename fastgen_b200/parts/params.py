"""Parameter dataclasses of the built-in parts.

Every size and constant a part needs is a field here; the parts read nothing
from the model they are in.  The architecture code fills these from the keys of
``config.json``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple


@dataclass(frozen=True)
class Llama3Scaling:
    """Frequency rescaling of fastgen/forward.py:616-633."""

    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_positions: int


@dataclass(frozen=True)
class YarnScaling:
    """Frequency interpolation by parts with a ramp between two pair indices ("YaRN").

    With ``dim(t) = dims * ln(original / (2 pi t)) / (2 ln theta)`` the ramp runs from
    ``lo = max(floor(dim(fast)), 0)`` to ``hi = min(ceil(dim(slow)), dims - 1)``:
    ``ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1)`` and pair ``i`` turns with
    ``f_i / factor * ramp_i + f_i * (1 - ramp_i)``.  Cosine and sine are both multiplied by
    ``0.1 * ln(factor) + 1`` (the encoding's ``magnitude``)."""

    factor: float
    original_max_positions: float
    fast: float
    slow: float


@dataclass(frozen=True)
class RopeParams:
    """Rotary position encoding over adjacent pairs (fastgen/kernels/rope.py:77-89).

    ``rot_dims`` (even, at most ``head_dim``): only that many dimensions of a head turn, pair
    ``i`` by ``pos * theta^(-2i / rot_dims)``; the rest pass unchanged (``None``: all of them).
    ``linear_factor`` divides every frequency (positions stretched linearly).  The table's
    entries beyond the rotated pairs are zero, which turns nothing.
    """

    head_dim: int
    theta: float
    scaling: Optional[object] = None  # a Llama3Scaling or a YarnScaling
    rot_dims: Optional[int] = None
    linear_factor: Optional[float] = None

    def __post_init__(self) -> None:
        if self.rot_dims is not None and (self.rot_dims <= 0 or self.rot_dims % 2 or self.rot_dims > self.head_dim):
            raise ValueError(f"{self.rot_dims} rotated dimensions do not fit a head of {self.head_dim}")
        if self.linear_factor is not None and self.linear_factor <= 0:
            raise ValueError(f"a linear scaling factor must be positive, got {self.linear_factor}")


@dataclass(frozen=True)
class NoPositionParams:
    """No position encoding: queries and keys are used as projected."""


@dataclass(frozen=True)
class AttentionParams:
    """Grouped-query causal attention (fastgen/model.py:50-80, forward.py:438-472).

    ``window`` is the number of most recent keys a query may see (itself
    included); ``None`` means all of them.  ``position`` is a ``PartSpec`` of a
    position encoding applied to queries and keys.  ``qk_layout`` says how the
    checkpoint orders the rows of a head in its query and key projections:
    ``"half_split"`` (the rotated pair of row ``j`` is row ``j + head_dim/2``, as
    Hugging Face Llama checkpoints store them; the rows are reordered at bind time,
    fastgen/utils/loading.py:296-305) or ``"adjacent"`` (pairs ``(2j, 2j+1)``, what the
    kernels rotate: taken as stored).
    """

    dim: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    position: object
    window: Optional[int] = None
    softmax_scale: Optional[float] = None  # None: head_dim ** -0.5 (forward.py:221)
    qk_layout: str = "adjacent"
    #: size of a value head when it differs from the query/key size (``None``: ``head_dim``)
    v_head_dim: Optional[int] = None
    #: the four projections carry biases (tensors ``bq``, ``bk``, ``bv``, ``bo``)
    bias: bool = False
    #: a ``PartSpec`` of a position encoding for the values: the value of position j is turned by
    #: j before it is cached and a head's output at position i is turned back by i, so that the
    #: output sees values turned by j - i.  ``v_layout`` is the checkpoint's pairing of a value
    #: head's dimensions, as ``qk_layout`` is for queries and keys.
    value_position: Optional[object] = None
    v_layout: str = "adjacent"
    #: with a window: so many of a sequence's first positions stay visible to every later
    #: query, at their true positions
    keep_first: int = 0
    #: ``"projection"``: queries and keys pass an RMS norm over their whole projection (all heads of
    #: a token at once, eps ``qk_norm_eps``, plain weights ``q_norm`` / ``k_norm`` of that size) before
    #: they are rotated; ``"head"``: an RMS norm per head, weights of ``head_dim`` numbers shared by the
    #: heads; ``None``: none
    qk_norm: Optional[str] = None
    qk_norm_eps: float = 1e-6
    #: a scaled score ``s`` enters the softmax as ``softcap * tanh(s / softcap)`` (``None``: as it is)
    softcap: Optional[float] = None
    #: whether the output projection has a bias when ``bias`` is set (``None``: as the others)
    o_bias: Optional[bool] = None
    #: the values are the keys as projected: the model has no value projection (tensor ``wv``), and
    #: ``v_head_dim`` equals ``head_dim``
    shared_kv: bool = False
    #: ``(coef, every)``: the query at position ``p`` is multiplied by
    #: ``1 + coef * ln(floor((p + 1) / every) + 1)``, a temperature that grows in steps
    q_temp: Optional[Tuple[float, int]] = None
    #: the softmax's denominator also holds ``exp(sink[h])`` for query head ``h`` (tensor ``sink``): a score
    #: without a key or a value, not scaled, counted once
    sink: bool = False
    #: head ``h``'s output is multiplied by ``sigmoid(wg x)[h]`` before the output projection (tensor
    #: ``wg`` [heads, dim]; ``x`` is the mixer's input)
    head_gate: bool = False
    #: taps of a causal convolution over time on every channel of q, k and v, directly after the
    #: projection (tensors ``conv_q``, ``conv_k``, ``conv_v`` [channels, taps], no bias; 0: none).  The
    #: last ``conv - 1`` projected rows of a sequence are its state
    conv: int = 0

    def __post_init__(self) -> None:
        if self.qk_norm not in (None, "projection", "head"):
            raise ValueError(f"qk_norm must be None, 'projection' or 'head', got {self.qk_norm!r}")
        if self.shared_kv and (self.v_head_dim or self.head_dim) != self.head_dim:
            raise ValueError("values that are the keys have the keys' size")
        if self.q_temp is not None and (len(self.q_temp) != 2 or int(self.q_temp[1]) < 1):
            raise ValueError(f"a query temperature is (coef, every >= 1), got {self.q_temp!r}")
        if not 0 <= self.conv <= 8:
            raise ValueError(f"the convolution takes up to 8 taps, got {self.conv}")
        if self.softcap is not None and self.softcap <= 0:
            raise ValueError(f"a cap on the scores must be positive, got {self.softcap}")
        for name, layout in (("qk_layout", self.qk_layout), ("v_layout", self.v_layout)):
            if layout not in ("adjacent", "half_split"):
                raise ValueError(f"{name} must be 'adjacent' or 'half_split', got {layout!r}")
        if self.n_heads % self.n_kv_heads != 0:
            raise ValueError(
                f"{self.n_heads} query heads cannot be grouped over "
                f"{self.n_kv_heads} key/value heads"
            )
        for size, position in ((self.head_dim, self.position), (self.v_head_dim or self.head_dim, self.value_position)):
            if not 1 <= size <= 256:
                raise ValueError(
                    f"head size {size} is not supported: the attention kernels take sizes up to 256 "
                    "(padded to a multiple of 16)"
                )
            turns = position is not None and getattr(position, "kind", "none") != "none"
            if turns and size % 2 != 0 and getattr(position.params, "rot_dims", None) is None:
                raise ValueError(f"head size {size} is odd: a rotation needs pairs of dimensions")
        if self.window is not None and self.window <= 0:
            raise ValueError(f"attention window must be positive, got {self.window}")
        if self.keep_first < 0:
            raise ValueError(f"the number of first positions kept visible cannot be negative, got {self.keep_first}")

    @property
    def kernel_head_dim(self) -> int:
        """The head size the kernels and the cache run with: the larger of the query/key and
        the value size, rounded up to a multiple of 16.  Heads are padded with zero rows of
        the projections, which changes no score and no output."""
        return -(-max(self.head_dim, self.v_head_dim or self.head_dim) // 16) * 16


@dataclass(frozen=True)
class SigmoidAttentionParams(AttentionParams):
    """Attention whose weights are ``sigmoid(score + gate_h - r1_h ln(1 + r2_h distance))``,
    not normalised over the keys.  ``gate`` (tensor ``gate``, a number per query head) and
    ``distance_bias`` (tensors ``r1``, ``r2``) say which of the terms the model has."""

    gate: bool = True
    distance_bias: bool = True


@dataclass(frozen=True)
class SwiGLUParams:
    """Dense gated feed-forward ``w2(silu(w1 x) * w3 x)`` (forward.py:491-496)."""

    dim: int
    ffn_dim: int


@dataclass(frozen=True)
class RMSNormParams:
    """``x * rsqrt(mean(x^2) + eps) * w`` (fastgen/kernels/rmsnorm.py:33-60); with ``one_plus`` the
    weight is stored around zero and the factor is ``1 + w``."""

    dim: int
    eps: float
    one_plus: bool = False


@dataclass(frozen=True)
class DenseMLPParams:
    """Dense feed-forward ``down(act(up x))`` without a gate; ``act`` is ``"gelu_erf"`` (the
    exact GELU), ``"gelu_tanh"`` or ``"relu2"`` (the square of ReLU)."""

    dim: int
    ffn_dim: int
    act: str = "gelu_erf"

    def __post_init__(self) -> None:
        if self.act not in ("gelu_erf", "gelu_tanh", "relu2"):
            raise ValueError(f"unknown activation {self.act!r}")


@dataclass(frozen=True)
class DynamicTanhParams:
    """``tanh(alpha x) * w + b`` with a scalar ``alpha``: a norm that computes no statistics."""

    dim: int


@dataclass(frozen=True)
class TableEmbeddingParams:
    """``x = table[token] * scale``."""

    vocab_size: int
    dim: int
    scale: float = 1.0


@dataclass(frozen=True)
class BigramHashParams:
    """``x = table[token] + bigram[(previous * mul_prev + token * mul_cur) mod buckets]``; the
    bigram table has ``buckets + 1`` rows and a sequence's first token takes the last one."""

    vocab_size: int
    dim: int
    buckets: int
    mul_prev: int
    mul_cur: int

    def __post_init__(self) -> None:
        if self.buckets <= 0:
            raise ValueError(f"a bigram table needs at least one bucket, got {self.buckets}")


@dataclass(frozen=True)
class LayerNormParams:
    """``(x - mean) / sqrt(var + eps) * w + b`` with the variance the mean of the squared
    deviations; ``bias`` says whether the norm has a ``b``."""

    dim: int
    eps: float
    bias: bool = True


@dataclass(frozen=True)
class HyperConnectionParams:
    """How a sub-layer reads from and writes to ``streams`` residual streams: its input is
    ``sum_s in[s] x_s`` and, with its output ``y``, ``x_t <- sum_s mix[s, t] x_s + out[t] y``."""

    streams: int

    def __post_init__(self) -> None:
        if not 1 <= self.streams <= 8:
            raise ValueError(f"1 to 8 residual streams are supported, got {self.streams}")


@dataclass(frozen=True)
class Mamba2Params:
    """State-space mixer in the Mamba-2 form: ``n_heads`` heads of ``head_dim`` values, a state of
    ``state`` rows per head, ``groups`` groups of heads that share B and C, a causal convolution
    of ``conv`` taps over x, B and C, and a gated RMS norm in ``norm_groups`` equal parts."""

    dim: int
    n_heads: int
    head_dim: int
    state: int
    groups: int
    conv: int
    norm_groups: int
    eps: float

    def __post_init__(self) -> None:
        if self.n_heads % self.groups:
            raise ValueError(f"{self.n_heads} heads cannot be split into {self.groups} groups")
        if (self.n_heads * self.head_dim) % self.norm_groups:
            raise ValueError(f"{self.n_heads * self.head_dim} columns cannot be normed in {self.norm_groups} equal parts")
        if not 1 <= self.conv <= 8:
            raise ValueError(f"the convolution takes 1 to 8 taps, got {self.conv}")
        if not 1 <= self.state <= 256:
            raise ValueError(f"the state takes 1 to 256 rows, got {self.state}")

    @property
    def inner(self) -> int:
        return self.n_heads * self.head_dim

    @property
    def channels(self) -> int:
        """Columns that pass the convolution: x, B and C."""
        return self.inner + 2 * self.groups * self.state


@dataclass(frozen=True)
class LatentAttentionParams:
    """Causal softmax attention whose keys and values are linear maps of a cached latent.

    Queries come through a latent of ``q_rank`` numbers (RMS-normed); a head's query and key have
    ``head_dim`` unrotated and ``rot_dim`` rotated dimensions (``position`` is the ``PartSpec`` of
    the rotation of those), its value ``v_head_dim``.  A token caches ``kv_rank`` latent numbers
    (RMS-normed) and one rotated key part that all heads share.  ``own_cache`` false: the layer
    has no latent projection and reads the entries another layer caches.  ``gate``: every head's
    output is multiplied by the sigmoid of a projection of the mixer's input."""

    dim: int
    n_heads: int
    head_dim: int
    rot_dim: int
    v_head_dim: int
    q_rank: int
    kv_rank: int
    softmax_scale: float
    eps: float
    position: object
    own_cache: bool = True
    gate: bool = True

    def __post_init__(self) -> None:
        if self.rot_dim % 2:
            raise ValueError(f"the rotated part has {self.rot_dim} dimensions: a rotation needs pairs")
        if not 1 <= self.kv_rank <= 512:
            raise ValueError(f"the attention kernels take latents of 1 to 512 numbers, got {self.kv_rank}")


@dataclass(frozen=True)
class GatedDeltaParams:
    """The gated delta rule: ``n_heads`` heads with a state of ``head_dim`` x ``v_head_dim`` each;
    queries and keys have ``n_kv_heads`` heads (head ``h`` uses ``h // (n_heads / n_kv_heads)``).
    q, k and v pass a causal convolution of ``conv`` taps per channel and SiLU.  The decay per head
    and key channel and the gate of the output come through two low-rank maps whose inner sizes are
    ``decay_rank`` and ``gate_rank`` (``None``: whatever the checkpoint's tensors have)."""

    dim: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    v_head_dim: int
    conv: int
    eps: float
    decay_rank: Optional[int] = None
    gate_rank: Optional[int] = None

    def __post_init__(self) -> None:
        if self.n_heads % self.n_kv_heads:
            raise ValueError(f"{self.n_heads} heads cannot share {self.n_kv_heads} query/key heads")
        if not 1 <= self.conv <= 8:
            raise ValueError(f"the convolution takes 1 to 8 taps, got {self.conv}")
        if not 1 <= self.head_dim <= 256:
            raise ValueError(f"the state takes 1 to 256 rows a head, got {self.head_dim}")

    @property
    def channels(self) -> int:
        """Columns that pass the convolution: q, k and v."""
        return 2 * self.n_kv_heads * self.head_dim + self.n_heads * self.v_head_dim


@dataclass(frozen=True)
class SideBySideParams:
    """Two mixers that read the same input; the result is ``left_scale * left + right_scale * right``.
    ``left`` and ``right`` are ``PartSpec``s of mixers; at most one of them caches per-token entries
    and at most one keeps a fixed-size state (the layer's cache and state are theirs)."""

    left: object
    right: object
    left_scale: float = 1.0
    right_scale: float = 1.0
    #: ``PartSpec``s of norms that the two outputs pass before they are multiplied and added
    #: (``None``: none)
    left_norm: Optional[object] = None
    right_norm: Optional[object] = None


@dataclass(frozen=True)
class RoutedExpertsParams:
    """``n_experts`` gated feed-forwards ``down(silu(gate x) * up x)`` of inner width ``ffn_dim``, of
    which a token uses ``top``: the experts with the largest ``softmax(router x) + correction``
    (``correction``: whether the model has that tensor), weighted by their softmax scores as they are
    (``renormalize``: divided by their sum).  The router runs in float32."""

    dim: int
    ffn_dim: int
    n_experts: int
    top: int
    correction: bool = True
    renormalize: bool = False
    #: the experts' scores: ``"softmax"`` over all experts or ``"sigmoid"`` of each logit
    score: str = "softmax"
    #: ``(count, keep)``: the experts form ``count`` equal groups of neighbours; a group's score is the
    #: sum of its ``group_top`` largest scores and only experts of the ``keep`` best groups can be chosen
    groups: Optional[Tuple[int, int]] = None
    group_top: int = 2
    #: added to the chosen scores' sum before ``renormalize`` divides by it
    renorm_eps: float = 0.0
    #: the weights are multiplied by it at the end
    weight_scale: float = 1.0
    #: ``"silu_gate"``: experts ``down(silu(gate x) * up x)``; an activation of the dense feed-forward
    #: (``"relu2"``, ...): experts ``down(act(up x))`` without a gate (no tensors ``w1``; ``w3`` is up)
    act: str = "silu_gate"
    #: a ``PartSpec`` of a feed-forward that every token also passes and whose output is added
    shared: Optional[object] = None

    def __post_init__(self) -> None:
        if not 1 <= self.top <= self.n_experts:
            raise ValueError(f"a token cannot use {self.top} of {self.n_experts} experts")
        if self.n_experts > 256:
            raise ValueError(f"the router takes up to 256 experts, got {self.n_experts}")
        if self.score not in ("softmax", "sigmoid"):
            raise ValueError(f"unknown kind of score {self.score!r}")
        if self.groups is not None:
            count, keep = self.groups
            if count < 1 or self.n_experts % count or not 1 <= keep <= count:
                raise ValueError(f"{self.n_experts} experts cannot form {count} equal groups of which {keep} are kept")
            if keep * (self.n_experts // count) < self.top:
                raise ValueError(f"{keep} groups of {self.n_experts // count} experts cannot hold {self.top} choices")


@dataclass(frozen=True)
class ParallelBlockParams:
    """A layer whose sub-layers all read one norm: ``x <- x + residual_mult * (mixer(h) + ffn(h))``
    with ``h = norm(x)``."""

    residual_mult: float = 1.0


@dataclass(frozen=True)
class MatrixMemoryParams:
    """The matrix memory with exponential gates (the mLSTM of xLSTM): ``n_heads`` heads with a state
    of ``head_dim`` x ``v_head_dim`` each, a normaliser vector and a running maximum that starts at
    zero.  The log gates are ``cap * tanh(x / cap)`` of their sums plus biases (the forget gate then
    passes ``logsigmoid``); the read-out is divided by ``max(|n . q|, exp(-m)) + 1e-6``, by its root mean
    square per head (``eps``), multiplied by a weight over all heads and by a sigmoid gate."""

    dim: int
    n_heads: int
    head_dim: int
    v_head_dim: int
    gate_cap: float
    eps: float

    def __post_init__(self) -> None:
        if not 1 <= self.head_dim <= 256:
            raise ValueError(f"the state takes 1 to 256 rows a head, got {self.head_dim}")
        if self.gate_cap <= 0:
            raise ValueError(f"the cap of the gates must be positive, got {self.gate_cap}")


@dataclass(frozen=True)
class GatedLinearRecurrenceParams:
    """Griffin's recurrent block: two branches of ``width`` channels, ``gelu_tanh(W_y x + b)`` and a
    causal convolution (``conv`` taps, with bias) of ``W_x x + b`` that feeds the real-gated linear
    recurrent unit ``S <- a S + sqrt(1 - a^2) i u`` with ``a = exp(-decay r softplus(lam))``; the gates
    ``r`` and ``i`` are sigmoids of block-diagonal maps (``blocks`` equal blocks) of ``u``."""

    dim: int
    width: int
    blocks: int
    conv: int
    decay: float = 8.0

    def __post_init__(self) -> None:
        if self.width % self.blocks:
            raise ValueError(f"{self.width} channels cannot form {self.blocks} equal blocks")
        if not 1 <= self.conv <= 8:
            raise ValueError(f"the convolution takes 1 to 8 taps, got {self.conv}")
