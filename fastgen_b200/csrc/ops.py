"""Python face of the CUDA kernels: one :class:`Ops` per compute dtype.

Every method launches hand-written kernels on the current CUDA stream through
the C interface of the in-tree libraries.  The only library call is the bfloat16
matrix product (cuBLAS through ``torch.mm``), where the reference calls
``F.linear``; the float32 path uses this package's own float32 GEMM.  Nothing
here falls back to the CPU or to eager PyTorch.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_ulonglong, c_void_p
from typing import Optional

import torch

from . import build

FG_F32, FG_BF16 = 0, 1

STATUS_BAD_PAGE = 1
STATUS_BAD_TOKEN = 2
STATUS_WAIT_TIMEOUT = 4
STATUS_BAD_SPLITS = 8


def _code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return FG_F32
    if dtype == torch.bfloat16:
        return FG_BF16
    raise TypeError(f"unsupported dtype {dtype}; the kernels take float32 and bfloat16")


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


_P, _I, _F = c_void_p, c_int, c_float
#: (token, expert) pairs from which the experts' products go to the vendor's grouped product
MOE_GROUPED_PAIRS = 512
_L = ctypes.c_long

_CORE_SIGNATURES = {
    "fg_embedding": [_P, _I, _P, _P, _I, _I, _I, _I, _F, _I, _P, _P],
    "fg_stream_norm": [_P, _I, _P, _I, _P, _P, _P, _P, _P, _P, _I, _P, _I, _I, _F, _I, _P],
    "fg_mamba2_conv": [_P, _L, _L, _I, _P, _L, _P, _P, _P, _L, _L, _P, _P, _P, _I, _I, _I, _I, _P],
    "fg_time_conv": [_P, _L, _L, _I, _P, _L, _I, _P, _P, _P, _L, _L, _P, _P, _P, _I, _I, _I, _I, _I, _P],
    "fg_head_gate": [_P, _L, _P, _L, _I, _P, _I, _I, _I, _P],
    "fg_qk_head_factors": [_P, _L, _P, _L, _I, _I, _I, _I, _I, _I, _F, _F, _I, _P, _P, _P, _I, _P],
    "fg_mamba2_scan": [_P, _L, _P, _L, _L, _I, _P, _P, _P, _P, _L, _P, _L, _P, _P, _I, _I, _I, _I, _I, _P],
    "fg_gated_part_norm": [_P, _L, _P, _L, _I, _P, _P, _L, _P, _I, _I, _I, _F, _P],
    "fg_rms_rows": [_P, _L, _I, _P, _F, _P, _L, _I, _I, _P],
    "fg_rotate_part": [_P, _L, _I, _P, _P, _P, _F, _I, _I, _I, _I, _I, _P],
    "fg_latent_entry_write": [_P, _L, _I, _P, _F, _P, _F, _P, _P, _I, _I, _I, _P, _P, _I, _I, _I, _I, _P, _P],
    "fg_latent_attention_simt": [_P, _I, _L, _L, _P, _L, _L, _P, _L, _L, _I, _P, _L, _P, _P, _I, _I, _I, _P, _P, _P,
                                 _P, _I, _I, _I, _I, _I, _F, _P, _P],
    "fg_rmsnorm": [_P, _I, _P, _I, _P, _I, _P, _I, _P, _I, _I, _F, _P],
    "fg_silu_gate": [_P, _P, _I, _I, _I, _I, _P],
    "fg_embedding_bigram": [_P, _P, _I, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P, _P],
    "fg_dyt": [_P, _P, _I, _P, _P, _P, _P, _P, _P, _P, _I, _P, _I, _I, _P],
    "fg_bias_act": [_P, _P, _I, _I, _I, _I, _P],
    "fg_scale_softcap": [_P, _I, _I, _F, _F, _P],
    "fg_rope_kv_write": [_P, _I, _P, _I, _P, _I, _I, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P, _P, _P,
                         _P, _I, _P],
    "fg_qk_rstd": [_P, _L, _I, _I, _P, _L, _I, _I, _I, _P, _F, _P, _I, _P],
    "fg_rmsnorm_sum": [_P, _P, _P, _I, _I, _P, _P, _I, _I, _P, _I, _P, _I, _I, _F, _P],
    "fg_gemm_f32_nt_from": [_P, _I, _I, _P, _I, _P, _I, _I, _I, _I, _P],
    "fg_gemm_f32_nt": [_P, _I, _P, _I, _P, _I, _I, _I, _I, _P, _P],
    "fg_gemm_skinny_bf16": [_P, _I, _P, _I, _P, _I, _I, _I, _I, _I, _P, _I, _P],
    "fg_gemm_skinny_swiglu_bf16": [_P, _I, _P, _I, _P, _I, _I, _I, _I, _P],
    "fg_gemm_skinny_qkv_bf16": [_P, _I, _P, _I, _P, _I, _I, _I, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I,
                                _I, _I, _P, _P],
    "fg_sample": [_P, _I, _I, _I, _P, _F, c_ulonglong, _P, _P, _P, _P, _P, _P, _P],
    "fg_selftest_wait_timeout": [_I, _P, _P, _P],
    "fg_sample_uniform": [c_ulonglong, _P, _P, _P, _I, _P],
    "fg_make_kv_tensor_map": [_P, _P, _I, _I, _I, _I, _I, _I],
}

_ATTN_SIGNATURES = {
    "fg_attention_simt": [_P, _I, _P, _I, _I, _P, _P, _P, _I, _I, _I, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _F,
                          _P, _P, _P],
    "fg_attention_sigmoid": [_P, _I, _P, _I, _I, _P, _P, _P, _I, _I, _I, _P, _P, _P, _P, _I, _I, _I, _I, _I, _F,
                             _P, _P, _P, _P, _P],
    "fg_attention_sigmoid_prefill_tc5_bf16": [_P, _I, _P, _I, _P, _P, _I, _P, _I, _I, _I, _P, _P, _P, _P, _I, _I, _I,
                                              _I, _I, _F, _P, _P, _P, _P, _P, _P, _P],
    "fg_attention_sigmoid_decode_bf16": [_P, _I, _P, _I, _P, _P, _P, _I, _I, _I, _P, _P, _P, _I, _I, _I, _I, _I, _F,
                                         _P, _P, _P, _P, ctypes.c_longlong, _I, _P, _P],
    "fg_attention_sigmoid_prefill_bf16": [_P, _I, _P, _I, _P, _P, _P, _I, _I, _I, _P, _P, _P, _P, _I, _I, _I, _I, _I,
                                          _F, _P, _P, _P, _P, _P],
    "fg_attention_prefill_bf16": [_P, _I, _P, _I, _P, _P, _P, _I, _I, _I, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _F,
                                  _P, _P, _P],
    "fg_attention_decode_bf16": [_P, _I, _P, _I, _P, _P, _P, _I, _I, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _P,
                                 ctypes.c_longlong, _I, _P, _F, _P, _P, _P],
    "fg_attention_prefill_tma_bf16": [_P, _I, _P, _I, _P, _P, _I, _P, _I, _I, _I, _P, _P, _P, _P, _I, _I, _I, _I,
                                      _I, _F, _I, _P, _P],
    "fg_attention_prefill_tc5_bf16": [_P, _I, _P, _I, _P, _P, _I, _P, _I, _I, _I, _P, _P, _P, _P, _I, _I, _I, _I,
                                      _I, _F, _P, _P, _P, _I, _I, _P, _I, _F, _P, _P, _P],
    "fg_attention_prefill_tc5_split_slots": [_I, _I, _I, _I, _I],
    "fg_attention_decode_tma_bf16": [_P, _I, _P, _I, _P, _P, _I, _P, _I, _I, _I, _P, _P, _P, _I, _I, _I, _I, _I,
                                     _F, _P, ctypes.c_longlong, _I, ctypes.c_longlong, _P, _P, _P, _P],
    "fg_attention_decode_is_persistent": [_I, _I, _I, _I],
}

SKINNY_MAX_M = int(os.environ.get("FG_SKINNY_MAX_M", "8"))      # most tokens the weight-streaming product is used for (it takes up to 32)
SIMT_ROWS = 16       # query rows per block of the float32 attention kernel
PREFILL_ROWS = 64    # ... of the bfloat16 prompt kernel
PREFILL_TMA_ROWS = 128  # ... of the bfloat16 prompt kernel with tiled TMA loads
PREFILL_TMA_KEYS = 64   # key positions per tile of that kernel
DECODE_SPLIT = 128   # key positions per split of the bfloat16 single-token kernel
SIGMOID_DECODE_KEYS = 256  # key positions per stretch of the sigmoid attention's single-token kernel

#: activations the products' epilogues and ``bias_act`` know
ACTIVATIONS = {None: 0, "none": 0, "gelu_erf": 1, "gelu_tanh": 2, "relu2": 3}


def _declare(lib: ctypes.CDLL, signatures) -> None:
    lib.fg_last_error.restype = ctypes.c_char_p
    for name, argtypes in signatures.items():
        fn = getattr(lib, name, None)
        if fn is None:
            continue
        fn.argtypes = argtypes
        fn.restype = c_int


class KernelError(RuntimeError):
    pass


def describe_status(word: int) -> str:
    """The faults that the bits of a status word stand for, in words."""
    faults = []
    if word & STATUS_BAD_PAGE:
        faults.append("a block-table entry was missing or out of range")
    if word & STATUS_BAD_TOKEN:
        faults.append("a token id was outside the vocabulary")
    if word & STATUS_WAIT_TIMEOUT:
        faults.append("a bounded wait inside a kernel gave up")
    if word & STATUS_BAD_SPLITS:
        faults.append("decode attention was launched with too few splits")
    if word & ~(STATUS_BAD_PAGE | STATUS_BAD_TOKEN | STATUS_WAIT_TIMEOUT | STATUS_BAD_SPLITS):
        faults.append(f"unknown bits {word:#x}")
    return "kernel status: " + "; ".join(faults)


class TensorMap:
    """A 128-byte TMA descriptor kept on the host (64-byte aligned)."""

    def __init__(self) -> None:
        self._raw = ctypes.create_string_buffer(128 + 64)
        addr = ctypes.addressof(self._raw)
        self.ptr = (addr + 63) & ~63


def _check(lib: ctypes.CDLL, rc: int) -> None:
    if rc != 0:
        raise KernelError(lib.fg_last_error().decode())
    Ops.launches += 1


_core = None
_attn = {}
_latent = {}

_LATENT_SIGNATURES = {
    "fg_latent_attention_mma": [_P, _L, _L, _P, _L, _L, _P, _L, _L, _P, _L, _P, _P, _I, _I, _I, _P, _P, _P, _P, _I, _I,
                                _I, _I, _I, _F, _I, _I, _P, ctypes.c_longlong, _P, _P],
}


def latent(rank: int, rot_dim: int):
    """The tensor-core library of the attention over a cached latent of these sizes."""
    key = (rank, rot_dim)
    lib = _latent.get(key)
    if lib is None:
        lib = build.latent_library(rank, rot_dim)
        _declare(lib, _LATENT_SIGNATURES)
        lib.fg_latent_mma_scratch_floats.argtypes = [_I, _I, _I]
        lib.fg_latent_mma_scratch_floats.restype = ctypes.c_longlong
        _latent[key] = lib
    return lib


_DELTA_SIGNATURES = {
    "fg_delta_scan": [_P, _L, _P, _L, _P, _L, _I, _P, _P, _P, _L, _P, _L, _P, _P, _I, _P, _I, _P, _I, _I, _I, _I, _P],
    "fg_delta_scan_scratch_floats": [_I, _I, _I, _I, _I],
    "fg_head_norm_gate": [_P, _L, _P, _L, _I, _P, _P, _L, _P, _I, _I, _I, _F, _P],
}
_MOE_SIGNATURES = {
    "fg_moe_logits": [_P, _I, _L, _P, _L, _P, _P, _I, _I, _I, _P],
    "fg_moe_route": [_P, _P, _P, _P, _P, _I, _I, _I, _I, _P],
    "fg_moe_route_groups": [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _F, _F, _P],
    "fg_moe_plan": [_P, _I, _I, _I, _P, _P, _P, _P, _P, _P, _I, _P, _P],
    "fg_moe_gather": [_P, _L, _P, _L, _I, _P, _P, _I, _I, _I, _I, _P],
    "fg_moe_gemm": [_P, _L, _P, _P, _L, _P, _L, _I, _I, _I, _P, _I, _P, _P, _P, _P, _I, _P],
    "fg_moe_gemm_mma": [_P, _L, _P, _P, _L, _P, _L, _I, _I, _P, _I, _P, _P, _P, _P, _I, _P],
    "fg_moe_combine": [_P, _L, _P, _P, _P, _L, _I, _I, _I, _I, _P],
}
_RECUR_SIGNATURES = {
    "fg_mlstm_scan": [_P, _P, _F, _P, _L, _P, _L, _P, _L, _I, _P, _P, _L, _P, _L, _P, _P, _P, _I, _I, _I, _I, _I, _F,
                      _P],
    "fg_mlstm_out": [_P, _L, _P, _P, _L, _I, _P, _P, _L, _P, _I, _I, _I, _F, _P],
    "fg_rglru_scan": [_P, _I, _P, _L, _I, _P, _P, _P, _P, _P, _L, _P, _L, _I, _P, _L, _L, _P, _P, _P, _I, _I, _I, _I,
                      _P],
}
_delta = None
_moe = None
_recur = None


def recurrent():
    """The library of the matrix memory with exponential gates and of the gated linear recurrent unit."""
    global _recur
    if _recur is None:
        lib = build.recurrent_library()
        _declare(lib, _RECUR_SIGNATURES)
        lib.fg_mlstm_state_floats.argtypes = [_I, _I, _I]
        lib.fg_mlstm_state_floats.restype = ctypes.c_longlong
        _recur = lib
    return _recur


def delta_rule():
    """The library of the gated delta rule."""
    global _delta
    if _delta is None:
        lib = build.delta_rule_library()
        _declare(lib, _DELTA_SIGNATURES)
        _delta = lib
    return _delta


def moe():
    """The library of the feed-forward with routed experts."""
    global _moe
    if _moe is None:
        lib = build.moe_library()
        _declare(lib, _MOE_SIGNATURES)
        _moe = lib
    return _moe


def core():
    global _core
    if _core is None:
        lib = build.core_library()
        _declare(lib, _CORE_SIGNATURES)
        _core = lib
    return _core


def attn(head_dim: int):
    lib = _attn.get(head_dim)
    if lib is None:
        lib = build.attention_library(head_dim)
        _declare(lib, _ATTN_SIGNATURES)
        lib.fg_attention_decode_scratch_floats.argtypes = [_I, _I, _I, ctypes.c_longlong]
        lib.fg_attention_decode_scratch_floats.restype = ctypes.c_longlong
        assert lib.fg_attention_rows_per_block() == SIMT_ROWS
        assert lib.fg_attention_prefill_rows() == PREFILL_ROWS
        assert lib.fg_attention_decode_split() == DECODE_SPLIT
        assert lib.fg_attention_sigmoid_decode_keys() == SIGMOID_DECODE_KEYS
        _attn[head_dim] = lib
    return lib


def require_cuda(device) -> torch.device:
    device = torch.device(device)
    if device.type != "cuda":
        raise RuntimeError(
            f"fastgen_b200 runs on a CUDA device only (got {device}); there is no CPU path"
        )
    if not torch.cuda.is_available():
        raise RuntimeError("no CUDA device is available; fastgen_b200 has no CPU path")
    return device


_device_index = 0  # set by Ops: the engine runs on one device
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current stream's handle.  Asked for at every launch, so through torch's
    direct call where it has one (the public way costs several microseconds)."""
    if _raw_stream is not None:
        return _raw_stream(_device_index)
    return torch.cuda.current_stream().cuda_stream


def attention_tiling(n_heads: int, n_kv_heads: int, rows: int = SIMT_ROWS) -> int:
    """Tokens per attention tile for a head grouping and a block of ``rows``
    query rows (see attention.cu)."""
    group = n_heads // n_kv_heads
    return max(1, rows // min(group, rows))


class Ops:
    """Kernels bound to one compute dtype (``torch.float32`` or ``torch.bfloat16``).

    ``act_dtype`` is the type of activations, weights' matrices and the cache;
    the residual stream, norms' arithmetic, softmax and rotation angles are
    float32 in both modes.
    """

    launches = 0  # kernels of this package launched (graph replays add their kernels)

    def __init__(self, dtype: torch.dtype, device) -> None:
        self.device = require_cuda(device)
        global _device_index
        _device_index = self.device.index if self.device.index is not None else torch.cuda.current_device()
        self.act_dtype = dtype
        self.code = _code(dtype)
        self.lib = core()
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._scratch = {}
        # the prompt attention kernel's blocks draw their work from it; zero between launches
        self._work_counter = torch.zeros(1, dtype=torch.int32, device=self.device)
        # head size -> (partials, flags, (item, part) pairs they hold) of prompt-attention launches
        # that work on their long items in several parts; buffers that were outgrown stay alive, since
        # captured graphs may hold their addresses
        self._split = {}
        self._split_retired = []
        self.use_tcgen05 = not bool(os.environ.get("FG_NO_TCGEN05"))
        # library products accumulate and reduce in float32 (no bfloat16 split-K sums)
        torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False

    # -- status word ---------------------------------------------------------
    def clear_status(self) -> None:
        """Zero the status word after a recorded fault, and with it what a kernel whose wait
        ran out may have left behind between launches: the prompt attention's work counter
        and the flags of its split items."""
        self.status.zero_()
        self._work_counter.zero_()
        for _scratch, flags, _room in self._split.values():
            flags.zero_()
        for _scratch, flags in self._split_retired:
            flags.zero_()

    def check_status(self) -> None:
        """Read the device status word (synchronises) and raise if a kernel
        recorded a fault instead of performing a bad access."""
        word = int(self.status.item())
        if word:
            self.status.zero_()
            raise KernelError(describe_status(word))

    def wait_timeout_selftest(self, limit: int = 1024):
        """Run a bounded wait on a barrier nobody arrives at (``limit`` polls) and return
        what the kernel saw: (first wait returned, second wait returned, cycles of the
        first, cycles of the second, wait on a completed phase returned).  The status word
        then holds the time-out bit."""
        out = torch.zeros(5, dtype=torch.int64, device=self.device)
        _check(self.lib, self.lib.fg_selftest_wait_timeout(int(limit), _ptr(self.status), _ptr(out), _stream()))
        return out.tolist()

    # -- kernels ---------------------------------------------------------------
    def embedding(self, table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
        """``out[t] = table[tokens[t]] * scale``; an ``out`` of [T, S, dim] receives the row S times."""
        assert table.is_contiguous() and out.is_contiguous() and tokens.dtype == torch.int32
        n, dim = out.shape[0], out.shape[-1]
        copies = out.shape[1] if out.dim() == 3 else 1
        _check(self.lib, self.lib.fg_embedding(
            _ptr(table), _code(table.dtype), _ptr(tokens), _ptr(out), _code(out.dtype),
            n, dim, table.shape[0], float(scale), copies, _ptr(self.status), _stream()))
        return out

    def stream_norm(self, h, weight, bias, eps: float, out, kind: int = 0, update=None, in_coef=None, rows=None):
        """Norm over one or several residual streams ``h`` [T, S, dim] or [T, dim] (float32), fused
        with the update that precedes it: with ``update`` (``delta`` [T, dim], ``mix`` [S, S] or
        ``None`` for the identity, ``out`` [S] or ``None`` for ones) every stream becomes
        ``sum_s mix[s, t] x_s + out[t] delta``; then ``out = norm(sum_s in_coef[s] x_s)`` (``in_coef``
        ``None``: the plain sum).  ``kind`` 0 is the layer norm (``bias`` may be ``None``), 1 the RMS
        norm.  With ``rows`` only those rows are computed and ``h`` stays as it was."""
        assert h.is_contiguous() and h.dtype == torch.float32
        dim = h.shape[-1]
        streams = h.shape[1] if h.dim() == 3 else 1
        n = h.shape[0] if rows is None else rows.numel()
        delta = mix = out_coef = None
        if update is not None:
            delta, mix, out_coef = update.delta, update.mix, update.out
            assert delta.is_contiguous() and delta.shape == (h.shape[0], dim)
        for t, shape in ((mix, (streams, streams)), (out_coef, (streams,)), (in_coef, (streams,)),
                         (weight, (dim,)), (bias, (dim,))):
            assert t is None or (t.dtype == torch.float32 and t.is_contiguous() and tuple(t.shape) == shape)
        assert out.is_contiguous() and out.shape == (n, dim)
        assert rows is None or rows.dtype == torch.int32
        _check(self.lib, self.lib.fg_stream_norm(
            _ptr(h), streams, _ptr(delta), _code(delta.dtype) if delta is not None else 0, _ptr(mix), _ptr(out_coef),
            _ptr(in_coef), _ptr(weight), _ptr(bias), _ptr(out), _code(out.dtype), _ptr(rows), n, dim, float(eps),
            int(kind), _stream()))
        return out

    # -- the state-space mixer --------------------------------------------------------------------
    def mamba2_conv(self, proj, xbc_offset: int, channels: int, weight, bias, state, conv_offset: int, taps: int,
                    ctx) -> torch.Tensor:
        """Causal convolution per channel with SiLU over the columns ``xbc_offset .. + channels`` of
        ``proj`` [T, .]; the inputs before the step's tokens come from ``state`` [slots, .] (float32,
        ``taps - 1`` rows of ``channels`` from ``conv_offset``), which is advanced.  Returns float32
        [T, channels]."""
        t = proj.shape[0]
        assert proj.stride(1) == 1 and state.dtype == torch.float32 and state.is_contiguous()
        assert weight.dtype == torch.float32 and weight.shape == (channels, taps) and weight.is_contiguous()
        out = torch.empty((t, channels), dtype=torch.float32, device=proj.device)
        _check(self.lib, self.lib.fg_mamba2_conv(
            _ptr(proj), proj.stride(0), int(xbc_offset), _code(proj.dtype), _ptr(out), out.stride(0), _ptr(weight),
            _ptr(bias), _ptr(state), state.stride(0), int(conv_offset), _ptr(ctx.req), _ptr(ctx.seq_slot),
            _ptr(ctx.seq_start), t, ctx.n_seqs, channels, taps, _stream()))
        Ops.launches += int(taps > 1)
        return out

    def mamba2_scan(self, xbc, proj, dt_offset: int, dt_bias, a_log, d_skip, state, ctx, heads: int, groups: int,
                    n_state: int, head_dim: int) -> torch.Tensor:
        """The recurrence ``S <- exp(-exp(A) dt) S + dt B x^T; y = S^T C + D x`` per (sequence, head),
        token by token in float32, from and into ``state`` [slots, .] (its first
        ``heads * n_state * head_dim`` numbers).  ``xbc`` [T, x | B | C] float32; the raw step sizes are
        the columns ``dt_offset .. + heads`` of ``proj``.  Returns y [T, heads * head_dim] float32."""
        t = xbc.shape[0]
        assert xbc.dtype == torch.float32 and xbc.stride(1) == 1 and proj.stride(1) == 1
        for v in (dt_bias, a_log, d_skip):
            assert v.dtype == torch.float32 and v.numel() == heads and v.is_contiguous()
        y = torch.empty((t, heads * head_dim), dtype=torch.float32, device=xbc.device)
        _check(self.lib, self.lib.fg_mamba2_scan(
            _ptr(xbc), xbc.stride(0), _ptr(proj), proj.stride(0), int(dt_offset), _code(proj.dtype), _ptr(dt_bias),
            _ptr(a_log), _ptr(d_skip), _ptr(y), y.stride(0), _ptr(state), state.stride(0), _ptr(ctx.seq_slot),
            _ptr(ctx.seq_start), ctx.n_seqs, heads, groups, n_state, head_dim, _stream()))
        return y

    def gated_part_norm(self, y, z, weight, parts: int, eps: float, ctx) -> torch.Tensor:
        """``v = y * silu(z)``, RMS-normed in ``parts`` equal parts of the columns, times ``weight``;
        ``y`` float32, ``z`` a (strided) view of the compute dtype, which the result has."""
        t, width = y.shape
        assert y.dtype == torch.float32 and y.stride(1) == 1 and z.stride(1) == 1 and z.shape == (t, width)
        assert weight.dtype == torch.float32 and weight.numel() == width and weight.is_contiguous()
        out = torch.empty((t, width), dtype=z.dtype, device=y.device)
        _check(self.lib, self.lib.fg_gated_part_norm(
            _ptr(y), y.stride(0), _ptr(z), z.stride(0), _code(z.dtype), _ptr(weight), _ptr(out), out.stride(0),
            _ptr(ctx.req), t, width, parts, float(eps), _stream()))
        return out

    # -- latent attention ---------------------------------------------------------------------------
    def rms_rows(self, x, weight, eps: float) -> torch.Tensor:
        """``x * rsqrt(mean(x^2) + eps) * weight`` per row of ``x`` [T, dim], which may be a column
        range of a wider tensor; float32 arithmetic, the result has ``x``'s type."""
        assert x.stride(1) == 1 and weight.dtype == torch.float32 and weight.numel() == x.shape[1]
        out = torch.empty(x.shape, dtype=x.dtype, device=x.device)
        _check(self.lib, self.lib.fg_rms_rows(_ptr(x), x.stride(0), _code(x.dtype), _ptr(weight), float(eps),
                                              _ptr(out), out.stride(0), x.shape[0], x.shape[1], _stream()))
        return out

    def head_products(self, x, w, w_t=None, out=None) -> torch.Tensor:
        """One product per head: ``out[h] = x[:, h, :] @ w[h]`` for ``x`` [T, H, a] (a strided view),
        ``w`` [H, a, b]; returns [H, T, b].  bfloat16 is the library's batched product; float32 runs
        this package's float32 product head by head and wants ``w_t`` [H, b, a]."""
        t, H, a = x.shape
        b = w.shape[2]
        if out is None:
            out = torch.empty((H, t, b), dtype=x.dtype, device=x.device)
        if x.dtype == torch.bfloat16:
            torch.bmm(x.permute(1, 0, 2), w, out=out)
            return out
        assert w_t is not None and w_t.shape == (H, b, a) and x.stride(2) == 1
        for h in range(H):
            self.linear(x[:, h, :], w_t[h], out=out[h])
        return out

    def head_products_out(self, x, w, w_t, out) -> torch.Tensor:
        """``out[:, h, :] = x[h] @ w[h].T`` for ``x`` [H, T, a], ``w`` [H, b, a] (``w_t`` [H, a, b] for
        the library's batched product in bfloat16), ``out`` [T, H, b]: heads side by side."""
        H = x.shape[0]
        if x.dtype == torch.bfloat16:
            torch.bmm(x, w_t, out=out.permute(1, 0, 2))
            return out
        for h in range(H):
            self.linear(x[h], w[h], out=out[:, h, :])
        return out

    def rotate_part(self, x, ctx, freqs, magnitude: float, n_heads: int, head_size: int, offset: int,
                    rot_dims: int) -> torch.Tensor:
        """Turn, in place, the adjacent pairs of the dimensions ``offset .. + rot_dims`` of every head of
        ``x`` [T, heads * head_size] by ``pos * freqs``; cosine and sine are multiplied by ``magnitude``."""
        assert x.stride(1) == 1 and freqs.dtype == torch.float32 and freqs.numel() >= rot_dims // 2
        _check(self.lib, self.lib.fg_rotate_part(
            _ptr(x), x.stride(0), _code(x.dtype), _ptr(ctx.pos), _ptr(ctx.req), _ptr(freqs), float(magnitude),
            x.shape[0], n_heads, head_size, offset, rot_dims, _stream()))
        return x

    def latent_entry_write(self, src, norm_weight, eps: float, freqs, magnitude: float, memory, ctx, rank: int,
                           rot_dim: int) -> None:
        """The cache entries of the step's tokens: ``[rmsnorm(src[:, :rank]) * w | src[:, rank:] turned]``
        into the pages of ``memory`` (one pool, one head, entries of ``head_dim`` numbers)."""
        pages = memory.k_pages
        assert src.stride(1) == 1 and src.shape[1] == rank + rot_dim and pages.is_contiguous()
        assert norm_weight.dtype == torch.float32 and norm_weight.numel() == rank
        _check(self.lib, self.lib.fg_latent_entry_write(
            _ptr(src), src.stride(0), _code(src.dtype), _ptr(norm_weight), float(eps), _ptr(freqs), float(magnitude),
            _ptr(pages), _ptr(memory.block_table), memory.block_table.shape[1], memory.page_size, pages.shape[0],
            _ptr(ctx.pos), _ptr(ctx.req), src.shape[0], rank, rot_dim, pages.shape[-1], _ptr(self.status),
            _stream()))

    def latent_attention(self, qa, qt, out, gate, memory, ctx, n_heads: int, rank: int, rot_dim: int,
                         scale: float) -> torch.Tensor:
        """Causal softmax attention of ``n_heads`` query heads on the one cached entry per token:
        score ``(qa_h . c + qt_h . k_t) * scale``, output the weighted sum of the latents ``c``, times
        ``sigmoid(gate[t, h])`` when a gate is given.  ``qa`` [heads, T, rank] (folded queries),
        ``qt`` [T, heads, rot_dim] (a strided view), ``out`` [heads, T, rank], ``gate`` [T, heads]
        (a strided view) or ``None``."""
        pages = memory.k_pages
        assert qa.stride(2) == 1 and qt.stride(2) == 1 and out.stride(2) == 1 and pages.is_contiguous()
        assert gate is None or gate.stride(1) == 1
        even = all(v % 2 == 0 for v in (*qa.stride()[:2], *qt.stride()[:2], *out.stride()[:2], qt.storage_offset()))
        if (qa.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and even
                and build.latent_mma_supported(rank, rot_dim) and pages.shape[-1] == -(-(rank + rot_dim) // 8) * 8):
            # bfloat16: the tensor cores; few tiles (single tokens) are cut into stretches of keys
            lib = latent(rank, rot_dim)
            rows, keys = lib.fg_latent_mma_rows(), lib.fg_latent_mma_keys()
            tiles = ctx.attention_tiles(attention_tiling(n_heads, 1, rows), 1)
            max_keys = tiles.max_keys or memory.block_table.shape[1] * memory.page_size
            blocks = tiles.n * -(-n_heads // min(n_heads, rows))
            n_splits = 1
            if blocks < 96:
                # few blocks: stretches of key tiles, as many as give every SM one block (the large
                # latents' blocks are alone on their SM, so more would be a second wave)
                n_splits = max(1, min(-(-max_keys // keys), 148 // blocks, 64))
            per = -(-(-(-max_keys // n_splits)) // keys) * keys
            n_splits = -(-max_keys // per)
            floats = lib.fg_latent_mma_scratch_floats(tiles.n, n_heads, n_splits)
            scratch = self._decode_scratch(floats) if floats else None
            _check(lib, lib.fg_latent_attention_mma(
                _ptr(qa), qa.stride(1), qa.stride(0), _ptr(qt), qt.stride(0), qt.stride(1), _ptr(out), out.stride(1),
                out.stride(0), _ptr(gate), gate.stride(0) if gate is not None else 0, _ptr(pages),
                _ptr(memory.block_table), memory.block_table.shape[1], memory.page_size, pages.shape[0], _ptr(ctx.pos),
                _ptr(tiles.req), _ptr(tiles.tok0), _ptr(tiles.ntok), tiles.n, n_heads, rank, rot_dim, pages.shape[-1],
                float(scale), n_splits, per, _ptr(scratch), scratch.numel() if scratch is not None else 0,
                _ptr(self.status), _stream()))
            Ops.launches += int(n_splits > 1)  # the merge of the stretches
            return out
        tiles = ctx.attention_tiles(attention_tiling(n_heads, 1, SIMT_ROWS), 1)
        _check(self.lib, self.lib.fg_latent_attention_simt(
            _ptr(qa), _code(qa.dtype), qa.stride(1), qa.stride(0), _ptr(qt), qt.stride(0), qt.stride(1), _ptr(out),
            out.stride(1), out.stride(0), _code(out.dtype), _ptr(gate), gate.stride(0) if gate is not None else 0,
            _ptr(pages), _ptr(memory.block_table), memory.block_table.shape[1], memory.page_size, pages.shape[0],
            _ptr(ctx.pos), _ptr(tiles.req), _ptr(tiles.tok0), _ptr(tiles.ntok), tiles.n, n_heads, rank, rot_dim,
            pages.shape[-1], float(scale), _ptr(self.status), _stream()))
        return out

    def embedding_bigram(self, table, bigram, tokens, pos, req, last_token, out, buckets: int, mul_prev: int,
                         mul_cur: int) -> torch.Tensor:
        """``out[t] = table[token] + bigram[hash(previous token, token)]`` (the table's last row for
        a sequence's first token); ``last_token`` [slots] int32 is the sequences' state: read for a
        token that opens its sequence's part of the step, then set to the last token brought."""
        assert table.is_contiguous() and bigram.is_contiguous() and out.is_contiguous()
        assert table.dtype == bigram.dtype and out.dtype == torch.float32
        assert tokens.dtype == torch.int32 and last_token.dtype == torch.int32
        assert bigram.shape == (buckets + 1, table.shape[1])
        n, dim = out.shape
        _check(self.lib, self.lib.fg_embedding_bigram(
            _ptr(table), _ptr(bigram), _code(table.dtype), _ptr(tokens), _ptr(pos), _ptr(req), _ptr(last_token),
            _ptr(out), n, dim, table.shape[0], int(buckets), int(mul_prev), int(mul_cur), _ptr(self.status),
            _stream()))
        Ops.launches += 1  # the state's own launch
        return out

    def dyt(self, h, pre=None, out=None, delta=None, post=None, rows=None):
        """Dynamic Tanh around the residual stream ``h`` (float32): ``h += post(delta)`` (``post``
        and ``delta`` optional), then ``out = pre(h)``.  ``pre`` / ``post`` are ``(alpha, weight,
        bias)`` float32 device tensors.  With ``rows`` only those rows are computed and ``h`` stays."""
        assert h.is_contiguous() and h.dtype == torch.float32
        dim = h.shape[1]
        n = h.shape[0] if rows is None else rows.numel()
        if delta is not None:
            assert delta.is_contiguous() and delta.shape == h.shape
        if out is not None:
            assert out.is_contiguous() and out.shape == (n, dim) and pre is not None
        for params in (pre, post):
            if params is not None:
                assert all(t.dtype == torch.float32 and t.is_contiguous() for t in params)
        pa, pw, pb = post if post is not None else (None, None, None)
        ra, rw, rb = pre if pre is not None else (None, None, None)
        _check(self.lib, self.lib.fg_dyt(
            _ptr(h), _ptr(delta), _code(delta.dtype) if delta is not None else 0, _ptr(pa), _ptr(pw), _ptr(pb),
            _ptr(ra), _ptr(rw), _ptr(rb), _ptr(out), _code(out.dtype) if out is not None else 0, _ptr(rows),
            n, dim, _stream()))
        return out

    def bias_act(self, x: torch.Tensor, act: Optional[str], bias: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``x = act(x + bias)`` in place (float32 arithmetic, one rounding)."""
        assert x.is_contiguous() and (bias is None or (bias.dtype == x.dtype and bias.is_contiguous()))
        _check(self.lib, self.lib.fg_bias_act(_ptr(x), _ptr(bias), _code(x.dtype), x.shape[0], x.shape[1],
                                              ACTIVATIONS[act], _stream()))
        return x

    def scale_softcap(self, logits: torch.Tensor, scale: float, cap: Optional[float]) -> torch.Tensor:
        """``logits = cap * tanh(logits * scale / cap)`` in place (only the scaling without a cap)."""
        assert logits.is_contiguous() and logits.dtype == torch.float32
        _check(self.lib, self.lib.fg_scale_softcap(_ptr(logits), logits.shape[0], logits.shape[1], float(scale),
                                                   float(cap or 0.0), _stream()))
        return logits

    def rmsnorm(self, h, weight, eps: float, out=None, delta=None, rows=None):
        """``h += delta`` (if given), then ``out = rmsnorm(h) * weight``.
        With ``out=None`` and a delta only the sum is done.  With ``rows``
        (int32 indices) only those rows are summed and normed into ``out``
        [len(rows), dim] and ``h`` is left as it was."""
        assert h.is_contiguous() and weight.is_contiguous()
        dim = h.shape[1]
        n = h.shape[0] if rows is None else rows.numel()
        if delta is not None:
            assert delta.is_contiguous() and delta.shape == h.shape
        if out is not None:
            assert out.is_contiguous() and out.shape == (n, dim)
        if rows is not None:
            assert rows.dtype == torch.int32 and out is not None
        _check(self.lib, self.lib.fg_rmsnorm(
            _ptr(h), _code(h.dtype), _ptr(delta), _code(delta.dtype) if delta is not None else 0,
            _ptr(weight), _code(weight.dtype), _ptr(out), _code(out.dtype) if out is not None else 0,
            _ptr(rows), n, dim, float(eps), _stream()))
        return out

    def rmsnorm_sum(self, h, terms, weight, eps: float, out=None, row=None, rows=None, one_plus: bool = False):
        """``h += row + sum_i coef_i * delta_i`` (float32), then ``out = rmsnorm(h) * weight`` (times
        ``1 + weight`` with ``one_plus``).  ``terms`` is a sequence of ``(delta [T, dim], coef)`` of one
        dtype (at most four); ``row`` a float32 [dim] vector or ``None``.  With ``out=None`` only the sum
        is done; with ``rows`` only those rows are summed and normed and ``h`` stays as it was.  With ``out``
        and no ``weight`` the summed rows are stored in ``out`` as they are (no norm)."""
        assert h.is_contiguous() and h.dtype == torch.float32
        dim = h.shape[1]
        n = h.shape[0] if rows is None else rows.numel()
        terms = list(terms)
        dtypes = {d.dtype for d, _ in terms}
        assert len(dtypes) <= 1, "the summands of one sum have one type"
        for d, _ in terms:
            assert d.is_contiguous() and d.shape == h.shape
        if row is not None:
            assert row.dtype == torch.float32 and row.is_contiguous() and row.numel() == dim
        if out is not None:
            assert out.is_contiguous() and out.shape == (n, dim) and (weight is None or weight.is_contiguous())
        assert rows is None or (rows.dtype == torch.int32 and out is not None)
        ptrs = (c_void_p * max(1, len(terms)))(*[d.data_ptr() for d, _ in terms])
        coefs = (c_float * max(1, len(terms)))(*[float(c) for _, c in terms])
        _check(self.lib, self.lib.fg_rmsnorm_sum(
            _ptr(h), ptrs, coefs, len(terms), _code(terms[0][0].dtype) if terms else 0, _ptr(row), _ptr(weight),
            _code(weight.dtype) if weight is not None else 0, int(one_plus), _ptr(out),
            _code(out.dtype) if out is not None else 0, _ptr(rows), n, dim, float(eps), _stream()))
        return out

    def linear_f32(self, x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        """``x @ w.T`` in float32 whatever the serving type: ``w`` [N, K] float32, ``x`` [M, K] of either
        type (16-bit activations are widened as they are read); IEEE sums in ascending k."""
        m, k = x.shape
        n = w.shape[0]
        assert w.dtype == torch.float32 and w.shape[1] == k and x.stride(1) == 1 and w.stride(1) == 1
        out = torch.empty((m, n), dtype=torch.float32, device=x.device)
        _check(self.lib, self.lib.fg_gemm_f32_nt_from(_ptr(x), _code(x.dtype), x.stride(0), _ptr(w), w.stride(0),
                                                      _ptr(out), out.stride(0), m, n, k, _stream()))
        return out

    # -- the gated delta rule ---------------------------------------------------------------------
    def conv_silu(self, proj, offset: int, channels: int, weight, state, conv_offset: int, taps: int, ctx):
        """Causal convolution per channel with SiLU, without a bias, over the columns
        ``offset .. + channels`` of ``proj`` (see ``mamba2_conv``): float32 [T, channels]."""
        return self.mamba2_conv(proj, offset, channels, weight, None, state, conv_offset, taps, ctx)

    def delta_scan(self, qkv, a, b, dt_bias, a_log, state, ctx, heads: int, kv_heads: int, d: int, dv: int):
        """The gated delta rule per (sequence, head), token by token in float32, from and into ``state``
        [slots, .] (a slot's first ``heads * dv * d`` numbers, laid out [heads][dv][d]):
        ``S <- diag(g) S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q`` with q, k made unit vectors
        (q also times ``d ** -0.5``), ``g = exp(-exp(a_log) softplus(a + dt_bias))``, ``beta =
        sigmoid(b)``.  ``qkv`` float32 [T, q | k | v] (``kv_heads * d`` twice, ``heads * dv``); ``a``
        [T, heads * d] and ``b`` [T, heads] strided views of the compute dtype.  Returns o float32
        [T, heads * dv]."""
        lib = delta_rule()
        t = qkv.shape[0]
        assert qkv.dtype == torch.float32 and qkv.stride(1) == 1 and qkv.shape[1] == 2 * kv_heads * d + heads * dv
        assert a.stride(1) == 1 and b.stride(1) == 1 and a.dtype == b.dtype and a.shape == (t, heads * d)
        assert b.shape == (t, heads) and state.dtype == torch.float32 and state.is_contiguous()
        assert dt_bias.dtype == torch.float32 and dt_bias.numel() == heads * d and dt_bias.is_contiguous()
        assert a_log.dtype == torch.float32 and a_log.numel() == heads and a_log.is_contiguous()
        out = torch.empty((t, heads * dv), dtype=torch.float32, device=qkv.device)
        # the tokens as the recurrence reads them (unit vectors, decays, step sizes; padded rows)
        scratch = torch.empty(lib.fg_delta_scan_scratch_floats(t, heads, kv_heads, d, dv), dtype=torch.float32,
                              device=qkv.device)
        _check(lib, lib.fg_delta_scan(
            _ptr(qkv), qkv.stride(0), _ptr(a), a.stride(0), _ptr(b), b.stride(0), _code(a.dtype), _ptr(dt_bias),
            _ptr(a_log), _ptr(out), out.stride(0), _ptr(state), state.stride(0), _ptr(ctx.seq_slot),
            _ptr(ctx.seq_start), ctx.n_seqs, _ptr(ctx.req), t, _ptr(scratch), heads, kv_heads, d, dv, _stream()))
        Ops.launches += 1  # the kernel that prepares the tokens
        return out

    def head_norm_gate(self, o, z, weight, heads: int, dv: int, eps: float, ctx) -> torch.Tensor:
        """Per head ``o * rsqrt(mean(o^2) + eps) * weight * sigmoid(z)``: ``o`` float32 [T, heads * dv],
        ``z`` of the compute dtype (which the result has), ``weight`` float32 [dv] shared by the heads."""
        lib = delta_rule()
        t = o.shape[0]
        assert o.dtype == torch.float32 and o.stride(1) == 1 and z.stride(1) == 1 and z.shape == o.shape
        assert weight.dtype == torch.float32 and weight.numel() == dv and weight.is_contiguous()
        out = torch.empty((t, heads * dv), dtype=z.dtype, device=o.device)
        _check(lib, lib.fg_head_norm_gate(
            _ptr(o), o.stride(0), _ptr(z), z.stride(0), _code(z.dtype), _ptr(weight), _ptr(out), out.stride(0),
            _ptr(ctx.req), t, heads, dv, float(eps), _stream()))
        return out

    # -- routed experts -----------------------------------------------------------------------------
    def moe_logits(self, x: torch.Tensor, w: torch.Tensor, ctx=None) -> torch.Tensor:
        """The router's logits ``x @ w.T`` in float32 whatever the serving type: ``w`` [E, K] float32,
        ``x`` [T, K] of either type (16-bit activations are widened as they are read).  A warp a
        token, sums in a fixed order: a token's logits do not depend on its batch.  Rows of padding
        tokens (with ``ctx``) are left unwritten."""
        lib = moe()
        t, k = x.shape
        n = w.shape[0]
        assert w.dtype == torch.float32 and w.shape[1] == k and x.stride(1) == 1 and w.stride(1) == 1
        out = torch.empty((t, n), dtype=torch.float32, device=x.device)
        _check(lib, lib.fg_moe_logits(_ptr(x), _code(x.dtype), x.stride(0), _ptr(w), w.stride(0), _ptr(out),
                                      _ptr(ctx.req) if ctx is not None else None, t, n, k, _stream()))
        return out

    def moe_route(self, logits, correction, top: int, ctx, renormalize: bool = False, score: str = "softmax",
                  groups=None, renorm_eps: float = 0.0, weight_scale: float = 1.0):
        """Scores over the experts (float32; ``score``: ``"softmax"`` or ``"sigmoid"``), choice of the
        ``top`` largest ``score + correction`` (equal ones: the lower index), weights = the chosen
        experts' scores (with ``renormalize``: divided by their sum plus ``renorm_eps``), times
        ``weight_scale``.  ``groups = (count, keep, group_top)``: the experts form ``count`` equal groups of
        neighbours, a group's score is the sum of its ``group_top`` largest scores, and only experts of
        the ``keep`` best groups can be chosen.  Returns (ids int32
        [T, top], weights float32 [T, top]); padding tokens get expert -1."""
        lib = moe()
        t, n = logits.shape
        assert logits.dtype == torch.float32 and logits.is_contiguous()
        assert correction is None or (correction.dtype == torch.float32 and correction.numel() == n)
        ids = torch.empty((t, top), dtype=torch.int32, device=logits.device)
        weights = torch.empty((t, top), dtype=torch.float32, device=logits.device)
        if score != "softmax" or groups is not None or renorm_eps or weight_scale != 1.0:
            count, keep, group_top = groups if groups is not None else (0, 0, 0)
            _check(lib, lib.fg_moe_route_groups(
                _ptr(logits), _ptr(correction), _ptr(ids), _ptr(weights), _ptr(ctx.req), t, n, int(top),
                {"softmax": 0, "sigmoid": 1}[score], int(count), int(keep), int(group_top), int(renormalize),
                float(renorm_eps), float(weight_scale), _stream()))
            return ids, weights
        _check(lib, lib.fg_moe_route(_ptr(logits), _ptr(correction), _ptr(ids), _ptr(weights), _ptr(ctx.req), t, n,
                                     int(top), int(renormalize), _stream()))
        return ids, weights

    def moe_experts(self, x, ids, weights, w1, w3, w2, w13=None, act: Optional[str] = None) -> torch.Tensor:
        """``sum_k weights[t, k] * expert_{ids[t, k]}(x[t])`` with expert ``e`` the gated feed-forward
        ``w2[e] (silu(w1[e] x) * (w3[e] x))``; ``w1``, ``w3`` [E, F, K] (each expert's matrix contiguous,
        the experts a fixed stride apart: they may be the halves of ``w13`` [E, 2F, K]) and ``w2``
        [E, K, F].  The (token, choice) pairs are sorted by expert on the device.  Few pairs: the
        products run over tiles of one expert's rows, on the tensor cores in bfloat16 where the sizes
        allow, else (and in float32) with float32 sums in ascending order.  Many pairs in bfloat16 (a
        prompt portion), given ``w13``: the sorted rows are gathered and the two products are the
        vendor library's grouped product over the experts' row ranges, as a dense layer's large
        products are the vendor's; gate and combine stay these kernels.

        ``w3 = None``: the experts have no gate, ``w2[e] act(w1[e] x)`` with ``act`` a key of
        ``ACTIVATIONS`` (``w13`` is then ``w1`` itself, for the grouped product)."""
        lib = moe()
        t, k = x.shape
        n_experts, f, _ = w1.shape
        top = ids.shape[1]
        pairs = t * top
        gated = w3 is not None
        assert x.stride(1) == 1 and w2.is_contiguous() and w1.stride(1) == k
        assert w2.shape == (n_experts, k, f) and w1.dtype == x.dtype == w2.dtype
        assert not gated or (w1.shape == w3.shape and w1.stride() == w3.stride())
        assert gated or ACTIVATIONS[act] >= 0
        w_stride = w1.stride(0)
        grouped = (w13 is not None and x.dtype == torch.bfloat16 and pairs >= MOE_GROUPED_PAIRS and k % 8 == 0
                   and f % 8 == 0 and hasattr(torch, "_grouped_mm") and not os.environ.get("FG_NO_GROUPED_MM"))
        mma = (not grouped and x.dtype == torch.bfloat16 and k % 8 == 0 and f % 8 == 0 and x.stride(0) % 8 == 0
               and w_stride % 8 == 0 and x.data_ptr() % 16 == 0 and w1.data_ptr() % 16 == 0
               and (not gated or w3.data_ptr() % 16 == 0) and hasattr(lib, "fg_moe_gemm_mma") and not os.environ.get("FG_NO_MOE_MMA"))
        tile_rows = lib.fg_moe_mma_tile_rows() if mma else lib.fg_moe_gemm_tile_rows()
        max_tiles = -(-pairs // tile_rows) + n_experts - 1
        plan = torch.empty(2 * pairs + 3 * max_tiles + 1 + n_experts, dtype=torch.int32, device=x.device)
        row_pair, pair_row = plan[:pairs], plan[pairs : 2 * pairs]
        o = 2 * pairs
        tile_expert, tile_row0, tile_n = plan[o : o + max_tiles], plan[o + max_tiles : o + 2 * max_tiles], \
            plan[o + 2 * max_tiles : o + 3 * max_tiles]
        n_tiles = plan[o + 3 * max_tiles : o + 3 * max_tiles + 1]
        expert_end = plan[o + 3 * max_tiles + 1 :]
        _check(lib, lib.fg_moe_plan(_ptr(ids), pairs, n_experts, tile_rows, _ptr(row_pair), _ptr(pair_row),
                                    _ptr(tile_expert), _ptr(tile_row0), _ptr(tile_n), _ptr(n_tiles), max_tiles,
                                    _ptr(expert_end), _stream()))
        if grouped:
            xs = torch.empty((pairs, k), dtype=x.dtype, device=x.device)
            _check(lib, lib.fg_moe_gather(_ptr(x), x.stride(0), _ptr(xs), xs.stride(0), _code(x.dtype), _ptr(row_pair),
                                          _ptr(expert_end), n_experts, top, pairs, k, _stream()))
            # rows beyond the last expert's end are never written and never read by the combine
            h = torch._grouped_mm(xs, w13.transpose(1, 2), offs=expert_end)
            if gated:
                mid = torch.empty((pairs, f), dtype=x.dtype, device=x.device)
                self.silu_gate(h, mid, 0)
            else:
                mid = self.bias_act(h, act)
            y = torch._grouped_mm(mid, w2.transpose(1, 2), offs=expert_end)
        else:
            # (rows beyond the plan's last tile are never written; zeroed where a kernel reads them all)
            mid = (torch.empty if gated else torch.zeros)((pairs, f), dtype=x.dtype, device=x.device)
            y = torch.empty((pairs, k), dtype=x.dtype, device=x.device)
            tiles = (_ptr(tile_expert), _ptr(tile_row0), _ptr(tile_n), _ptr(n_tiles), max_tiles, _stream())
            if mma:
                _check(lib, lib.fg_moe_gemm_mma(_ptr(x), x.stride(0), _ptr(w1), _ptr(w3), w_stride, _ptr(mid),
                                                mid.stride(0), f, k, _ptr(row_pair), top, *tiles))
                if not gated:
                    self.bias_act(mid, act)
                _check(lib, lib.fg_moe_gemm_mma(_ptr(mid), mid.stride(0), _ptr(w2), None, w2.stride(0), _ptr(y),
                                                y.stride(0), k, f, None, top, *tiles))
            else:
                code = _code(x.dtype)
                _check(lib, lib.fg_moe_gemm(_ptr(x), x.stride(0), _ptr(w1), _ptr(w3), w_stride, _ptr(mid), mid.stride(0),
                                            code, f, k, _ptr(row_pair), top, *tiles))
                if not gated:
                    self.bias_act(mid, act)
                _check(lib, lib.fg_moe_gemm(_ptr(mid), mid.stride(0), _ptr(w2), None, w2.stride(0), _ptr(y), y.stride(0),
                                            code, k, f, None, top, *tiles))
        out = torch.empty((t, k), dtype=x.dtype, device=x.device)
        _check(lib, lib.fg_moe_combine(_ptr(y), y.stride(0), _ptr(weights), _ptr(pair_row), _ptr(out), out.stride(0),
                                       _code(x.dtype), t, k, top, _stream()))
        return out

    def linear(self, x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None,
               out_dtype: Optional[torch.dtype] = None, bias: Optional[torch.Tensor] = None,
               act: Optional[str] = None) -> torch.Tensor:
        """``act(x @ w.T + bias)`` for ``x`` [M, K] and ``w`` [N, K] (fastgen/forward.py:438-440);
        ``bias`` [N] of the compute dtype and ``act`` (a key of ``ACTIVATIONS``) are optional.  The
        bias is added to the float32 sums; the activation sees the rounded result."""
        m, k = x.shape
        n = w.shape[0]
        assert w.shape[1] == k and x.stride(1) == 1 and w.stride(1) == 1
        assert bias is None or (bias.shape == (n,) and bias.dtype == w.dtype and bias.is_contiguous())
        code = ACTIVATIONS[act]
        if self.act_dtype == torch.float32:
            assert x.dtype == torch.float32 and w.dtype == torch.float32
            if out is None:
                out = torch.empty((m, n), dtype=torch.float32, device=x.device)
            assert out.dtype == torch.float32 and out.stride(1) == 1
            _check(self.lib, self.lib.fg_gemm_f32_nt(
                _ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(out), out.stride(0),
                m, n, k, _ptr(bias), _stream()))
            if code:
                assert out.is_contiguous()
                self.bias_act(out, act)
            return out
        assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
        want = out.dtype if out is not None else (out_dtype or torch.bfloat16)
        if (m <= SKINNY_MAX_M and k % 8 == 0 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
                and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0):
            # few tokens: this package's weight-streaming kernel
            if out is None:
                out = torch.empty((m, n), dtype=want, device=x.device)
            assert out.stride(1) == 1
            _check(self.lib, self.lib.fg_gemm_skinny_bf16(
                _ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(out), out.stride(0), _code(out.dtype),
                m, n, k, _ptr(bias), code, _stream()))
            return out
        if want == torch.bfloat16:
            # the library adds the bias to its float32 sums: one rounding, as in the kernel above
            if bias is not None:
                res = torch.addmm(bias, x, w.t(), out=out) if out is not None else torch.addmm(bias, x, w.t())
            else:
                res = torch.mm(x, w.t(), out=out) if out is not None else torch.mm(x, w.t())
            if code:
                self.bias_act(res, act)
            return res
        assert bias is None and not code, "a float32 result of a bfloat16 product takes no bias or activation"
        # float32 result of a bfloat16 product (logits)
        res = torch.mm(x, w.t(), out_dtype=torch.float32)
        if out is not None:
            out.copy_(res)
            return out
        return res

    def _skinny_ok(self, x: torch.Tensor, w: torch.Tensor, k: int) -> bool:
        return (x.dtype == torch.bfloat16 and x.shape[0] <= SKINNY_MAX_M and k % 8 == 0
                and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and x.stride(1) == 1 and w.stride(1) == 1
                and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)

    def linear_swiglu(self, x: torch.Tensor, w13: torch.Tensor) -> Optional[torch.Tensor]:
        """``silu(x @ w1.T) * (x @ w3.T)`` in one kernel for a few tokens, for
        ``w13`` that holds w1 and w3 interleaved in blocks of 8 rows; ``None``
        when the shapes do not allow it (the caller then runs the product and
        the gate separately)."""
        m, k = x.shape
        f = w13.shape[0] // 2
        if f % 8 or not self._skinny_ok(x, w13, k):
            return None
        out = torch.empty((m, f), dtype=torch.bfloat16, device=x.device)
        _check(self.lib, self.lib.fg_gemm_skinny_swiglu_bf16(
            _ptr(x), x.stride(0), _ptr(w13), w13.stride(0), _ptr(out), out.stride(0), m, f, k, _stream()))
        return out

    def qkv_rope_write(self, x, wqkv, pos, req, freqs, memory, n_heads: int, n_kv_heads: int,
                       head_dim: int, bias=None, v_freqs=None) -> Optional[torch.Tensor]:
        """Queries, keys and values of a few tokens in one kernel: the product
        against ``[wq; wk; wv]``, the rotation, and the write of keys and
        values into their pages.  ``bias`` (over the fused rows) is added before the
        rounding; ``v_freqs`` turns the values by their own position too.  Returns the
        rotated queries [T, heads*head_dim], or ``None`` when the shapes do not allow it."""
        m, k = x.shape
        if not self._skinny_ok(x, wqkv, k) or head_dim % 16:
            return None
        q = torch.empty((m, n_heads * head_dim), dtype=torch.bfloat16, device=x.device)
        _check(self.lib, self.lib.fg_gemm_skinny_qkv_bf16(
            _ptr(x), x.stride(0), _ptr(wqkv), wqkv.stride(0), _ptr(q), q.stride(0), m, k, _ptr(bias),
            _ptr(pos), _ptr(req), _ptr(freqs), _ptr(v_freqs), _ptr(memory.k_pages), _ptr(memory.v_pages),
            _ptr(memory.block_table), memory.block_table.shape[1], memory.page_size,
            memory.k_pages.shape[0], n_heads, n_kv_heads, head_dim, _ptr(self.status), _stream()))
        return q

    def silu_gate(self, x13: torch.Tensor, out: torch.Tensor, interleave: int = 0) -> torch.Tensor:
        """``silu(gate) * up`` for ``x13`` holding gate and up as halves
        (``interleave=0``) or interleaved in blocks of 8 columns (``8``)."""
        n, two_f = x13.shape
        assert x13.is_contiguous() and out.is_contiguous() and out.shape == (n, two_f // 2)
        _check(self.lib, self.lib.fg_silu_gate(_ptr(x13), _ptr(out), _code(x13.dtype), n, two_f // 2,
                                               interleave, _stream()))
        return out

    def rope_kv_write(self, q, k, v, pos, req, freqs, k_pages, v_pages, block_table,
                      page_size: int, n_heads: int, n_kv_heads: int, head_dim: int, v_freqs=None, qk_norm=None) -> None:
        """Rotate ``q`` in place; rotate ``k`` and copy ``v`` into their pages (``v`` is
        rotated too, by the table ``v_freqs``, when that is given).
        ``q``/``k``/``v`` are row-strided views [T, heads*head_dim]; ``k``/``v``
        may both be ``None`` (queries only).  ``qk_norm`` = (rstd [T, 2], query weights, key
        weights), all float32: queries and keys are multiplied by their token's factor (see
        ``qk_rstd``) and their weights before they turn.  An ``rstd`` of [T, heads + kv heads] holds a
        factor per head instead (see ``qk_head_factors``); the weights may then be ``None`` (ones)."""
        rstd, qn_w, kn_w = qk_norm if qk_norm is not None else (None, None, None)
        rstd_heads = 0
        if rstd is not None:
            assert rstd.dtype == torch.float32 and rstd.is_contiguous() and rstd.shape[0] == q.shape[0]
            # (with one query head and one key head the two layouts are the same)
            rstd_heads = 0 if rstd.shape[1] == 2 else rstd.shape[1]
            assert rstd_heads in (0, n_heads + n_kv_heads)
            assert qn_w is None or (qn_w.dtype == torch.float32 and qn_w.numel() == n_heads * head_dim and qn_w.is_contiguous())
            assert k is None or kn_w is None or (kn_w.dtype == torch.float32 and kn_w.numel() == n_kv_heads * head_dim)
        t = q.shape[0]
        assert q.stride(1) == 1 and pos.dtype == torch.int32 and req.dtype == torch.int32
        if k is not None:
            assert k.stride(1) == 1 and v.stride(1) == 1
            assert k_pages.is_contiguous() and v_pages.is_contiguous()
            assert block_table.dtype == torch.int32 and block_table.is_contiguous()
            n_pages = k_pages.shape[0]
            width = block_table.shape[1]
        else:
            n_pages = width = 0
        _check(self.lib, self.lib.fg_rope_kv_write(
            _ptr(q), q.stride(0), _ptr(k), k.stride(0) if k is not None else 0,
            _ptr(v), v.stride(0) if v is not None else 0, _code(q.dtype), _ptr(pos), _ptr(req),
            _ptr(freqs), _ptr(v_freqs) if k is not None else None, _ptr(k_pages) if k is not None else None,
            _ptr(v_pages) if k is not None else None,
            _ptr(block_table) if k is not None else None, width, page_size, n_pages,
            t, n_heads, n_kv_heads, head_dim, _ptr(self.status), _ptr(rstd), _ptr(qn_w), _ptr(kn_w), rstd_heads,
            _stream()))

    def qk_head_factors(self, q, k, pos, req, n_heads: int, n_kv_heads: int, head_dim: int, real_dim: int,
                        norm_eps: Optional[float] = None, temp=None) -> torch.Tensor:
        """Per-head factors of queries and keys, float32 [T, heads + kv heads]: with ``norm_eps`` a
        head's ``rsqrt(mean(x^2) + eps)`` over its first ``real_dim`` columns (an RMS norm per head; the
        columns up to ``head_dim`` are padding and hold zeros); with ``temp = (coef, every)`` a query
        head's factor is also multiplied by ``1 + coef * ln(floor((pos + 1) / every) + 1)``.  ``q`` /
        ``k`` are row-strided views."""
        t = q.shape[0]
        assert q.stride(1) == 1 and k.stride(1) == 1 and k.dtype == q.dtype
        coef, every = temp if temp is not None else (0.0, 0)
        out = torch.empty((t, n_heads + n_kv_heads), dtype=torch.float32, device=q.device)
        _check(self.lib, self.lib.fg_qk_head_factors(
            _ptr(q), q.stride(0), _ptr(k), k.stride(0), _code(q.dtype), n_heads, n_kv_heads, head_dim, real_dim,
            int(norm_eps is not None), float(norm_eps or 0.0), float(coef), int(every), _ptr(pos), _ptr(req), _ptr(out),
            t, _stream()))
        return out

    def head_gate(self, x, gate, req, heads: int, head_dim: int) -> torch.Tensor:
        """``x[t, h, :] *= sigmoid(gate[t, h])`` in place (float32 arithmetic): ``x`` [T, heads * head_dim],
        ``gate`` a row-strided view [T, heads] of the same type."""
        assert x.stride(1) == 1 and gate.stride(1) == 1 and x.dtype == gate.dtype and x.shape[1] == heads * head_dim
        _check(self.lib, self.lib.fg_head_gate(_ptr(x), x.stride(0), _ptr(gate), gate.stride(0), _code(x.dtype),
                                               _ptr(req), x.shape[0], heads, head_dim, _stream()))
        return x

    def time_conv(self, proj, offset: int, channels: int, weight, bias, state, conv_offset: int, taps: int, ctx,
                  act: Optional[str] = None, out_dtype=None) -> torch.Tensor:
        """Causal convolution over time per channel over the columns ``offset .. + channels`` of ``proj``
        [T, .] (the last tap meets the current token; zeros before a sequence's start).  The inputs before
        the step's tokens come from ``state`` [slots, .] (float32, ``taps - 1`` rows of ``channels`` from
        ``conv_offset``), which is advanced.  ``act``: ``None`` or ``"silu"``; the result [T, channels] is
        float32 or, with ``out_dtype``, of ``proj``'s type."""
        t = proj.shape[0]
        assert proj.stride(1) == 1 and state.dtype == torch.float32 and state.is_contiguous()
        assert weight.dtype == torch.float32 and weight.shape == (channels, taps) and weight.is_contiguous()
        assert act in (None, "silu") and out_dtype in (None, torch.float32, proj.dtype)
        out = torch.empty((t, channels), dtype=out_dtype or torch.float32, device=proj.device)
        _check(self.lib, self.lib.fg_time_conv(
            _ptr(proj), proj.stride(0), int(offset), _code(proj.dtype), _ptr(out), out.stride(0), _code(out.dtype),
            _ptr(weight), _ptr(bias), _ptr(state), state.stride(0), int(conv_offset), _ptr(ctx.req), _ptr(ctx.seq_slot),
            _ptr(ctx.seq_start), t, ctx.n_seqs, channels, taps, int(act == "silu"), _stream()))
        Ops.launches += int(taps > 1)
        return out

    # -- the matrix memory with exponential gates ------------------------------------------------------
    def mlstm_state_floats(self, heads: int, d: int, dv: int) -> int:
        return int(recurrent().fg_mlstm_state_floats(heads, d, dv))

    def mlstm_scan(self, gates, gate_bias, cap: float, q, k, v, state, ctx, heads: int, d: int, dv: int,
                   q_scale: float):
        """The matrix memory per (sequence, head), token by token in float32, from and into ``state``
        [slots, .] (``[heads][dv + 1][d]``, column ``dv`` being n, then the heads' running maxima):
        ``m' = max(f + m, i); S <- exp(f + m - m') S + exp(i - m') k v^T`` and n likewise with k alone, with
        ``i = cap tanh((gates_i + bias) / cap)``, ``f = logsigmoid(cap tanh((gates_f + bias) / cap))``.
        ``gates`` float32 [T, 2 heads] raw sums (overwritten); ``q``, ``k`` [T, heads * d] and ``v``
        [T, heads * dv] row-strided views of the compute type; q is multiplied by ``q_scale``.  Returns
        ``(y, coef)``: y float32 [T, heads * (dv + 1)] (a head's ``S^T q``, then ``n . q``) and the
        tokens' log coefficients [T, heads, 3] whose last is ``-m'``."""
        lib = recurrent()
        t = q.shape[0]
        assert gates.dtype == torch.float32 and gates.is_contiguous() and gates.shape == (t, 2 * heads)
        assert gate_bias.dtype == torch.float32 and gate_bias.numel() == 2 * heads and gate_bias.is_contiguous()
        assert q.stride(1) == 1 and k.stride(1) == 1 and v.stride(1) == 1 and q.dtype == k.dtype == v.dtype
        assert q.shape[1] == heads * d and k.shape[1] == heads * d and v.shape[1] == heads * dv
        assert state.dtype == torch.float32 and state.is_contiguous()
        coef = torch.empty((t, heads, 3), dtype=torch.float32, device=q.device)
        y = torch.empty((t, heads * (dv + 1)), dtype=torch.float32, device=q.device)
        _check(lib, lib.fg_mlstm_scan(
            _ptr(gates), _ptr(gate_bias), float(cap), _ptr(q), q.stride(0), _ptr(k), k.stride(0), _ptr(v), v.stride(0),
            _code(q.dtype), _ptr(coef), _ptr(y), y.stride(0), _ptr(state), state.stride(0), _ptr(ctx.req),
            _ptr(ctx.seq_slot), _ptr(ctx.seq_start), t, ctx.n_seqs, heads, d, dv, float(q_scale), _stream()))
        Ops.launches += 1 if t <= 4 * ctx.n_seqs else 2  # the chain of running maxima; the gates of many tokens
        return y, coef

    def mlstm_out(self, y, coef, z, weight, heads: int, dv: int, eps: float, ctx) -> torch.Tensor:
        """``o = y / (max(|n . q|, exp(-m')) + 1e-6)`` per head, divided by its root mean square (``eps``),
        times ``weight`` [heads * dv] and ``sigmoid(z)``; ``z`` a row-strided view of the compute type,
        which the result has."""
        lib = recurrent()
        t = y.shape[0]
        assert y.dtype == torch.float32 and y.stride(1) == 1 and z.stride(1) == 1 and z.shape == (t, heads * dv)
        assert weight.dtype == torch.float32 and weight.numel() == heads * dv and weight.is_contiguous()
        out = torch.empty((t, heads * dv), dtype=z.dtype, device=y.device)
        _check(lib, lib.fg_mlstm_out(_ptr(y), y.stride(0), _ptr(coef), _ptr(z), z.stride(0), _code(z.dtype),
                                     _ptr(weight), _ptr(out), out.stride(0), _ptr(ctx.req), t, heads, dv, float(eps),
                                     _stream()))
        return out

    # -- the gated linear recurrent unit ---------------------------------------------------------------
    def rglru_scan(self, gates, u, bias_r, bias_i, neg_rate, y, state, state_offset: int, ctx, blocks: int):
        """``S <- a S + sqrt(1 - a^2) i u; out = S y`` per (sequence, channel), token by token in float32,
        with ``r = sigmoid(gates_r + bias_r)``, ``i = sigmoid(gates_i + bias_i)``, ``a = exp(neg_rate r)``.
        ``gates`` [blocks, T, 2 bw] (a block's r sums, then its i sums), ``u`` and ``y`` [T, width]
        row-strided; ``state`` [slots, .] float32 holds S at ``state_offset``.  The result has ``y``'s
        type."""
        lib = recurrent()
        t, width = y.shape
        bw = width // blocks
        assert gates.is_contiguous() and gates.shape == (blocks, t, 2 * bw)
        assert u.stride(1) == 1 and y.stride(1) == 1 and u.shape == (t, width)
        for vec in (bias_r, bias_i, neg_rate):
            assert vec.dtype == torch.float32 and vec.numel() == width and vec.is_contiguous()
        assert state.dtype == torch.float32 and state.is_contiguous()
        coef = torch.empty((t, 2, width), dtype=torch.float32, device=y.device)
        out = torch.empty((t, width), dtype=y.dtype, device=y.device)
        _check(lib, lib.fg_rglru_scan(
            _ptr(gates), _code(gates.dtype), _ptr(u), u.stride(0), _code(u.dtype), _ptr(bias_r), _ptr(bias_i),
            _ptr(neg_rate), _ptr(coef), _ptr(y), y.stride(0), _ptr(out), out.stride(0), _code(y.dtype), _ptr(state),
            state.stride(0), int(state_offset), _ptr(ctx.req), _ptr(ctx.seq_slot), _ptr(ctx.seq_start), t, ctx.n_seqs,
            width, blocks, _stream()))
        Ops.launches += 1  # the coefficients' kernel
        return out

    def block_products(self, x, w_t, w) -> torch.Tensor:
        """A block-diagonal map: ``out[b] = x[:, b, :] @ w[b].T`` for ``x`` [T, blocks, a] (a strided
        view), ``w`` [blocks, n, a]; returns float32 [blocks, T, n].  bfloat16 inputs go through the
        library's batched product with float32 results (``w_t`` [blocks, a, n]); float32 runs this
        package's float32 product block by block."""
        t, blocks, a = x.shape
        if x.dtype == torch.bfloat16:
            return torch.bmm(x.permute(1, 0, 2), w_t, out_dtype=torch.float32)
        n = w.shape[1]
        out = torch.empty((blocks, t, n), dtype=torch.float32, device=x.device)
        for b in range(blocks):
            self.linear(x[:, b, :], w[b], out=out[b])
        return out

    def qk_rstd(self, q, k, count_q: int, count_k: int, eps: float, req) -> torch.Tensor:
        """For every token the factors of an RMS norm over its whole query projection and over its
        whole key projection: ``rsqrt(sum(x^2) / count + eps)`` as float32 [T, 2].  ``q`` / ``k`` are
        row-strided views whose padding columns hold zeros; ``count`` is the number of real ones.
        ``k`` may be ``None``."""
        t = q.shape[0]
        assert q.stride(1) == 1 and (k is None or (k.stride(1) == 1 and k.dtype == q.dtype))
        out = torch.empty((t, 2), dtype=torch.float32, device=q.device)
        _check(self.lib, self.lib.fg_qk_rstd(
            _ptr(q), q.stride(0), q.shape[1], int(count_q), _ptr(k), k.stride(0) if k is not None else 0,
            k.shape[1] if k is not None else 0, int(count_k), _code(q.dtype), _ptr(req), float(eps), _ptr(out), t,
            _stream()))
        return out

    def _decode_scratch(self, floats: int) -> torch.Tensor:
        """Scratch for the split partials.  Buffers are kept for good (captured
        graphs hold their addresses) and come in power-of-two sizes."""
        size = 1 << max(16, (floats - 1).bit_length())
        buf = self._scratch.get(size)
        if buf is None:
            buf = self._scratch[size] = torch.empty(size, dtype=torch.float32, device=self.device)
        return buf

    def make_kv_tensor_maps(self, k_pool, v_pool, page_size: int):
        """Tensor maps of a key and a value pool [layers, pages, kv heads, page,
        head size], or ``None`` where the tiled-load kernels do not apply."""
        n_layers, n_pages, n_kv_heads, page, head_dim = k_pool.shape
        if (k_pool.dtype != torch.bfloat16 or head_dim % 64 != 0 or page_size < 8
                or page_size & (page_size - 1)):
            return None
        # the box (rows a TMA instruction brings) is part of the map: one pair of maps
        # for the single-token kernel (128 positions a split), one for the prompt
        # kernel (64 positions a tile)
        maps = []
        for box_rows in (min(page_size, DECODE_SPLIT), min(page_size, PREFILL_TMA_KEYS)):
            for pool in (k_pool, v_pool):
                tm = TensorMap()
                _check(self.lib, self.lib.fg_make_kv_tensor_map(
                    tm.ptr, _ptr(pool), n_layers, n_pages, n_kv_heads, page_size, head_dim, box_rows))
                Ops.launches -= 1  # not a kernel
                maps.append(tm)
        return tuple(maps)

    def _split_buffers(self, head_dim: int, items: int):
        """Partials and flags for a prompt-attention launch that wants to work on its long
        items in parts, ``items`` (item, part) pairs in all (0: it does not).  They grow to the largest launch seen, outside
        graph captures only: a capture that finds them too small records a launch that does
        not split."""
        scratch, flags, room = self._split.get(head_dim, (None, None, 0))
        if items > room and not torch.cuda.is_current_stream_capturing():
            if room:
                self._split_retired.append((scratch, flags))
            room = max(items, 2 * room)
            scratch = torch.empty(room * PREFILL_TMA_ROWS * (head_dim + 2), dtype=torch.float32, device=self.device)
            flags = torch.zeros(2 * room, dtype=torch.int32, device=self.device)
            self._split[head_dim] = (scratch, flags, room)
        return scratch, flags, room

    def attention(self, q, out, memory, ctx, n_heads: int, n_kv_heads: int, head_dim: int,
                  window: Optional[int], scale: float, out_freqs: Optional[torch.Tensor] = None,
                  keep_first: int = 0, softcap: Optional[float] = None,
                  sinks: Optional[torch.Tensor] = None) -> bool:
        """Paged causal attention of the step's query tokens; ``memory`` is the
        run's :class:`~fastgen_b200.cache.LayerMemory`, ``ctx`` the step's
        context.  bfloat16 runs on the tensor cores: prompt portions in one
        kernel, single tokens in a split-and-combine pair (with tiled TMA loads
        where the shapes allow); float32 runs one CUDA-core kernel for all.

        ``out_freqs`` (a frequency table, or ``None``): the caller wants the outputs' adjacent
        pairs turned by ``position * frequency``.  Returns ``True`` if the kernels did that for
        every token of the step (a bfloat16 step of single tokens only: the merge of the splits
        turns what it stores), ``False`` if the caller still has to (``rotate_heads``).

        ``softcap``: a scaled score ``s`` enters the softmax as ``softcap * tanh(s / softcap)``.

        ``sinks`` (float32 [heads] or ``None``): ``exp(sinks[h])`` joins the softmax's denominator of head
        ``h`` once; it has no key and no value and is not scaled."""
        lib = attn(head_dim)
        assert sinks is None or (sinks.dtype == torch.float32 and sinks.numel() == n_heads and sinks.is_contiguous())
        k_pages, v_pages, block_table, page_size = (
            memory.k_pages, memory.v_pages, memory.block_table, memory.page_size)
        assert q.stride(1) == 1 and out.stride(1) == 1
        common = (_ptr(k_pages), _ptr(v_pages), _ptr(block_table), block_table.shape[1], page_size,
                  k_pages.shape[0], _ptr(ctx.pos))
        keep_first = int(keep_first) if window else 0
        if q.dtype == torch.float32:
            tiles = ctx.attention_tiles(attention_tiling(n_heads, n_kv_heads, SIMT_ROWS), 1)
            _check(lib, lib.fg_attention_simt(
                _ptr(q), q.stride(0), _ptr(out), out.stride(0), _code(q.dtype), *common,
                _ptr(tiles.req), _ptr(tiles.tok0), _ptr(tiles.ntok), tiles.n,
                n_heads, n_kv_heads, head_dim, int(window or 0), keep_first, float(scale), float(softcap or 0.0),
                _ptr(sinks), _ptr(self.status), _stream()))
            return False
        # windows that keep a sequence's first positions visible run on the mma.sync kernels (on TMA
        # tiles for prompts where the pools have tensor maps), which walk the tiles of the kept
        # positions before those of the window
        # capped scores: the cap lives in the tcgen05 kernel (head sizes 64 and 128) and in the
        # mma.sync kernels on cp.async tiles
        # sinks: in prompt portions a row starts its running maximum and sum from the sink, in the
        # tcgen05 kernel (head sizes 64 and 128) and in the mma.sync kernel on cp.async tiles; single
        # tokens keep their kernels (the sink joins where the splits are merged)
        tc5 = head_dim in (64, 128) and self.use_tcgen05 and not keep_first
        use_tma = memory.tensor_maps is not None and (not softcap or tc5)
        prompt_tma = use_tma and (sinks is None or tc5)
        rows = PREFILL_TMA_ROWS if prompt_tma else PREFILL_ROWS
        tiling = attention_tiling(n_heads, n_kv_heads, rows)
        tiles = ctx.attention_tiles(tiling, 2)
        if tiles.n and prompt_tma:
            # head sizes 64 and 128: tcgen05.mma with S and O in tensor memory; other
            # multiples of 64: mma.sync on the same TMA tiles (FG_NO_TCGEN05=1 forces that)
            args = (_ptr(q), q.stride(0), _ptr(out), out.stride(0), memory.tensor_maps[2].ptr,
                    memory.tensor_maps[3].ptr, memory.layer_index, _ptr(block_table), block_table.shape[1],
                    page_size, k_pages.shape[0], _ptr(ctx.pos), _ptr(tiles.req), _ptr(tiles.tok0),
                    _ptr(tiles.ntok), tiles.n, n_heads, n_kv_heads, head_dim, int(window or 0), float(scale))
            if tc5:
                max_keys = -1 if tiles.max_keys is None else tiles.max_keys
                # a captured list has padding: what a step of prompt tokens only would hold
                nominal = 0 if tiles.count is None else max(1, -(-q.shape[0] // tiling))
                want = lib.fg_attention_prefill_tc5_split_slots(tiles.n, n_heads, n_kv_heads, max_keys, nominal)
                scratch, flags, room = self._split_buffers(head_dim, want)
                _check(lib, lib.fg_attention_prefill_tc5_bf16(
                    *args, _ptr(self._work_counter), _ptr(scratch), _ptr(flags), room, max_keys,
                    _ptr(tiles.count), nominal, float(softcap or 0.0), _ptr(sinks), _ptr(self.status), _stream()))
            else:
                _check(lib, lib.fg_attention_prefill_tma_bf16(*args, keep_first, _ptr(self.status), _stream()))
        elif tiles.n:
            _check(lib, lib.fg_attention_prefill_bf16(
                _ptr(q), q.stride(0), _ptr(out), out.stride(0), *common,
                _ptr(tiles.req), _ptr(tiles.tok0), _ptr(tiles.ntok), tiles.n,
                n_heads, n_kv_heads, head_dim, int(window or 0), keep_first, float(scale), float(softcap or 0.0),
                _ptr(sinks), _ptr(self.status), _stream()))
        singles = ctx.single_tokens()
        fused = out_freqs is not None and tiles.n == 0 and singles.n > 0
        turn = _ptr(out_freqs) if fused else None
        if singles.n:
            max_splits = max(1, -(-singles.max_len // DECODE_SPLIT))
            # (capped scores: single tokens stay on the kernel that knows the cap)
            tma = use_tma and not softcap and n_heads // n_kv_heads <= 16 and not keep_first
            # the persistent kernel numbers its partials by the (request, split) pairs that
            # exist: the scratch follows the keys in the cache, not requests x longest request
            pairs = 0
            if tma and lib.fg_attention_decode_is_persistent(singles.n, n_heads, n_kv_heads, page_size):
                pairs = min(singles.n * max_splits, singles.stretches(DECODE_SPLIT))
            floats = lib.fg_attention_decode_scratch_floats(singles.n, max_splits, n_heads, pairs)
            scratch = self._decode_scratch(floats)
            head = (_ptr(singles.req), _ptr(singles.tok), singles.n, n_heads, n_kv_heads, head_dim,
                    int(window or 0), float(scale), _ptr(scratch), scratch.numel(), max_splits)
            if not tma:
                head = head[:7] + (keep_first,) + head[7:]
            if tma:
                _check(lib, lib.fg_attention_decode_tma_bf16(
                    _ptr(q), q.stride(0), _ptr(out), out.stride(0), memory.tensor_maps[0].ptr,
                    memory.tensor_maps[1].ptr, memory.layer_index, _ptr(block_table),
                    block_table.shape[1], page_size, k_pages.shape[0], _ptr(ctx.pos), *head, pairs, turn,
                    _ptr(sinks), _ptr(self.status), _stream()))
            else:
                _check(lib, lib.fg_attention_decode_bf16(
                    _ptr(q), q.stride(0), _ptr(out), out.stride(0), *common, *head, turn, float(softcap or 0.0),
                    _ptr(sinks), _ptr(self.status), _stream()))
            Ops.launches += 1  # the combine kernel
        return fused

    def rotate_heads(self, x, pos, req, freqs, n_heads: int, head_dim: int) -> torch.Tensor:
        """Rotate the adjacent pairs of every head of ``x`` [T, heads*head_dim] in place by
        ``pos * freqs`` (a table of negated frequencies turns them back)."""
        self.rope_kv_write(x, None, None, pos, req, freqs, None, None, None, 0, n_heads, 0, head_dim)
        return x

    def attention_sigmoid(self, q, out, memory, ctx, n_heads: int, n_kv_heads: int, head_dim: int,
                          window: Optional[int], scale: float, gate=None, r1=None, r2=None) -> None:
        """Paged attention with sigmoid weights, not normalised over the keys:
        ``sum_j sigmoid(q.k_j * scale + gate[h] - r1[h] * ln(1 + r2[h] * distance)) v_j`` over the
        visible keys; ``gate``, ``r1``, ``r2`` are float32 [heads] or ``None``.  float32: one
        CUDA-core kernel for all tokens.  bfloat16: prompt portions on the tensor cores
        (``tcgen05.mma`` at head sizes 64 and 128 on pages the TMA can tile, else ``mma.sync``;
        the weights rounded to bfloat16 for the second product), single tokens in a
        kernel of their own, a block per (token, key/value head), which reads a window's keys once."""
        lib = attn(head_dim)
        k_pages, v_pages, block_table = memory.k_pages, memory.v_pages, memory.block_table
        assert q.stride(1) == 1 and out.stride(1) == 1
        for t in (gate, r1, r2):
            assert t is None or (t.dtype == torch.float32 and t.numel() == n_heads and t.is_contiguous())
        head = (_ptr(k_pages), _ptr(v_pages), _ptr(block_table), block_table.shape[1], memory.page_size,
                k_pages.shape[0], _ptr(ctx.pos))
        tail = (n_heads, n_kv_heads, head_dim, int(window or 0), float(scale), _ptr(gate), _ptr(r1), _ptr(r2),
                _ptr(self.status), _stream())
        if q.dtype == torch.float32:
            tiles = ctx.attention_tiles(attention_tiling(n_heads, n_kv_heads, SIMT_ROWS), 1)
            _check(lib, lib.fg_attention_sigmoid(
                _ptr(q), q.stride(0), _ptr(out), out.stride(0), FG_F32, *head,
                _ptr(tiles.req), _ptr(tiles.tok0), _ptr(tiles.ntok), tiles.n, *tail))
            return
        tc5 = memory.tensor_maps is not None and head_dim in (64, 128) and self.use_tcgen05
        rows = PREFILL_TMA_ROWS if tc5 else PREFILL_ROWS
        tiles = ctx.attention_tiles(attention_tiling(n_heads, n_kv_heads, rows), 2)
        if tiles.n and tc5:
            # head sizes 64 and 128 on pages the TMA can tile: tcgen05.mma with the scores and the
            # output in tensor memory, the weights computed by the kernel's softmax warps
            _check(lib, lib.fg_attention_sigmoid_prefill_tc5_bf16(
                _ptr(q), q.stride(0), _ptr(out), out.stride(0), memory.tensor_maps[2].ptr, memory.tensor_maps[3].ptr,
                memory.layer_index, _ptr(block_table), block_table.shape[1], memory.page_size, k_pages.shape[0],
                _ptr(ctx.pos), _ptr(tiles.req), _ptr(tiles.tok0), _ptr(tiles.ntok), tiles.n, n_heads, n_kv_heads,
                head_dim, int(window or 0), float(scale), _ptr(gate), _ptr(r1), _ptr(r2), _ptr(self._work_counter),
                _ptr(tiles.count), _ptr(self.status), _stream()))
        elif tiles.n:
            _check(lib, lib.fg_attention_sigmoid_prefill_bf16(
                _ptr(q), q.stride(0), _ptr(out), out.stride(0), *head,
                _ptr(tiles.req), _ptr(tiles.tok0), _ptr(tiles.ntok), tiles.n, *tail))
        singles = ctx.single_tokens()
        if singles.n:
            # a token's keys reach into so many stretches at most: its window's, or all it can hold
            keys = SIGMOID_DECODE_KEYS
            stretches = -(-singles.max_len // keys)
            if window:
                stretches = min(stretches, -(-int(window) // keys) + 1)
            stretches = max(1, stretches)
            scratch = self._decode_scratch(singles.n * n_heads * stretches * head_dim) if stretches > 1 else None
            _check(lib, lib.fg_attention_sigmoid_decode_bf16(
                _ptr(q), q.stride(0), _ptr(out), out.stride(0), *head,
                _ptr(singles.req), _ptr(singles.tok), singles.n, *tail[:-2], _ptr(scratch),
                scratch.numel() if scratch is not None else 0, stretches, *tail[-2:]))
            Ops.launches += int(stretches > 1)  # the sum of the stretches

    def sample(self, logits, temps, top_p: float, seed: int, req_keys, positions,
               out_tokens, out_logprobs=None, scratch=None, with_status: bool = False) -> torch.Tensor:
        """One token per row of ``logits`` into ``out_tokens``.  ``with_status``: the
        device status word is copied to ``out_tokens[rows]`` (one more entry), so that the
        host's read of the tokens also tells it whether a kernel of the step recorded a fault."""
        rows, vocab = logits.shape
        assert logits.dtype == torch.float32 and logits.stride(1) == 1
        assert out_tokens.dtype == torch.int32 and out_tokens.numel() >= rows + int(with_status)
        if temps is not None:
            assert temps.dtype == torch.float32 and scratch is not None
            assert scratch.numel() >= rows * vocab and scratch.dtype == torch.float32
        if req_keys is not None:
            assert req_keys.dtype == torch.int64 and positions.dtype == torch.int32
        _check(self.lib, self.lib.fg_sample(
            _ptr(logits), logits.stride(0), rows, vocab, _ptr(temps), float(top_p),
            int(seed) & 0xFFFFFFFFFFFFFFFF, _ptr(req_keys), _ptr(positions), _ptr(out_tokens),
            _ptr(out_logprobs), _ptr(scratch), _ptr(self.status) if with_status else None, _stream()))
        return out_tokens

    def sample_uniform(self, seed: int, req_keys, positions) -> torch.Tensor:
        n = req_keys.numel()
        out = torch.empty(n, dtype=torch.float32, device=self.device)
        _check(self.lib, self.lib.fg_sample_uniform(
            int(seed) & 0xFFFFFFFFFFFFFFFF, _ptr(req_keys), _ptr(positions), _ptr(out), n, _stream()))
        return out
