"""``Tanupel``: config.json keys -> model description.

A decoder whose layers are listed one by one under ``layers``.  Every layer is a *parallel* block:
one RMS norm (weight stored around zero, factor ``1 + w``) whose output the mixer and the
feed-forward both read, ``x <- x + residual_mult * (mixer(h) + ff(h))``.  A run of layers
(``loop{start, stop, times}``) is passed several times with the same weights; every pass has a cache
and a state of its own and starts by adding row ``t`` of the tensor ``loop.step`` to the residual
stream.

Keys read: ``architecture``, ``vocab``, ``width``, ``norm.eps``, ``residual_mult``,
``embedding.scale`` (optional), ``loop{start, stop, times}`` (optional) and per layer ``type``,
``mixer`` and ``mlp`` (or null):

* ``attention``: ``heads, kv_heads, dim, vdim, scale, rot{dims, base, scaling}``, optionally
  ``softcap``: grouped-query causal softmax attention; queries and keys pass an RMS norm over their
  whole projection (plain weights ``q.norm``, ``k.norm``) and then turn on a head's first
  ``rot.dims`` dimensions, dimension ``i`` paired with ``i + dims/2``.  ``rot.scaling`` with
  ``{factor, low, high, original}`` rescales the frequencies by wavelength (the Llama 3.1 law), with
  ``{factor}`` alone it divides them all;
* ``parallel``: ``left`` (an attention as above), ``right{heads, kv_heads, dim, vdim, conv}`` (the
  gated delta rule, see ``parts/gated_delta.py``), ``left_scale``, ``right_scale``;
* ``mlp{kind: dense, ff}`` or ``mlp{kind: moe, expert{ff}, router{experts, top}}``.

Tensors: ``embed``, ``loop.step``, ``l<i>.norm1``, ``l<i>.mix.*`` (``.left.*`` / ``.right.*``),
``l<i>.mlp.gate|up|down`` or ``l<i>.mlp.router|correction|e<j>.gate|up|down``, ``final.norm``,
``head``.
"""

from __future__ import annotations

from typing import Any, Mapping, Optional

from ..parts.params import (
    AttentionParams,
    GatedDeltaParams,
    Llama3Scaling,
    NoPositionParams,
    ParallelBlockParams,
    RMSNormParams,
    RopeParams,
    RoutedExpertsParams,
    SideBySideParams,
    SwiGLUParams,
    TableEmbeddingParams,
)
from .model_args import ConfigError, LayerSpec, ModelArgs, PartSpec, ScheduleEntry, positive_int, require
from .registry import register_architecture

#: the design sets no limit on positions; the engine's own limits (cache size) apply
MAX_POSITIONS = 1 << 30

STEP_TABLE = "loop.step"


def _norm(dim: int, eps: float, name: str) -> PartSpec:
    return PartSpec("rmsnorm", RMSNormParams(dim, eps, one_plus=True), {"weight": name})


def _rope(rot: Optional[Mapping[str, Any]], head_dim: int, where: str, by_wavelength: bool = True) -> PartSpec:
    """``by_wavelength``: a scaling that names ``low``/``high``/``original`` bends the frequencies by
    wavelength; without them, or with ``by_wavelength`` off, ``factor`` divides every frequency."""
    if not rot:
        return PartSpec("none", NoPositionParams())
    require(rot, ("dims", "base"), f"{where}.rot")
    scaling = None
    linear = None
    sc = rot.get("scaling")
    if sc:
        require(sc, ("factor",), f"{where}.rot.scaling")
        if by_wavelength and any(k in sc for k in ("low", "high", "original")):
            require(sc, ("low", "high", "original"), f"{where}.rot.scaling")
            scaling = Llama3Scaling(float(sc["factor"]), float(sc["low"]), float(sc["high"]), sc["original"])
        else:
            linear = float(sc["factor"])
    return PartSpec("rope", RopeParams(head_dim=head_dim, theta=float(rot["base"]), scaling=scaling,
                                       rot_dims=positive_int(rot, "dims"), linear_factor=linear))


def _attention(dim: int, eps: float, m: Mapping[str, Any], prefix: str, where: str,
               by_wavelength: bool = True) -> PartSpec:
    require(m, ("heads", "kv_heads", "dim", "vdim", "scale"), where)
    head_dim = positive_int(m, "dim")
    softcap = m.get("softcap")
    params = AttentionParams(
        dim=dim,
        n_heads=positive_int(m, "heads"),
        n_kv_heads=positive_int(m, "kv_heads"),
        head_dim=head_dim,
        v_head_dim=positive_int(m, "vdim"),
        position=_rope(m.get("rot"), head_dim, where, by_wavelength),
        softmax_scale=float(m["scale"]),
        qk_layout="half_split",
        qk_norm="projection",
        qk_norm_eps=eps,
        softcap=float(softcap) if softcap is not None else None,
    )
    names = {"wq": "q", "wk": "k", "wv": "v", "wo": "o", "q_norm": "q.norm", "k_norm": "k.norm"}
    return PartSpec("gqa_attention", params, {k: prefix + v for k, v in names.items()})


def _gated_delta(dim: int, eps: float, m: Mapping[str, Any], prefix: str, where: str) -> PartSpec:
    require(m, ("heads", "kv_heads", "dim", "vdim", "conv"), where)
    params = GatedDeltaParams(
        dim=dim,
        n_heads=positive_int(m, "heads"),
        n_kv_heads=positive_int(m, "kv_heads"),
        head_dim=positive_int(m, "dim"),
        v_head_dim=positive_int(m, "vdim"),
        conv=positive_int(m, "conv"),
        eps=eps,
        # the inner sizes of the two low-rank maps are the checkpoint's; a config may name them
        decay_rank=int(m["decay_rank"]) if m.get("decay_rank") else None,
        gate_rank=int(m["gate_rank"]) if m.get("gate_rank") else None,
    )
    names = {"wq": "q", "wk": "k", "wv": "v", "conv_q": "q.conv", "conv_k": "k.conv", "conv_v": "v.conv", "wb": "b",
             "a_log": "A_log", "norm": "norm", "wa1": "a1", "wa2": "a2", "dt_bias": "dt_bias", "wg1": "g1", "wg2": "g2",
             "wo": "o"}
    return PartSpec("gated_delta", params, {k: prefix + v for k, v in names.items()})


def _side_by_side(dim: int, eps: float, m: Mapping[str, Any], prefix: str, where: str) -> PartSpec:
    require(m, ("left", "right"), where)
    params = SideBySideParams(
        # the attention of a pair divides its frequencies by the factor, whatever else the scaling names
        left=_attention(dim, eps, m["left"], prefix + "left.", f"{where}.left", by_wavelength=False),
        right=_gated_delta(dim, eps, m["right"], prefix + "right.", f"{where}.right"),
        left_scale=float(m.get("left_scale", 1.0)),
        right_scale=float(m.get("right_scale", 1.0)),
    )
    return PartSpec("side_by_side", params, {})


_MIXERS = {"attention": _attention, "parallel": _side_by_side}


def _feed_forward(dim: int, mlp: Mapping[str, Any], prefix: str, where: str) -> PartSpec:
    require(mlp, ("kind",), where)
    kind = mlp["kind"]
    if kind == "dense":
        require(mlp, ("ff",), where)
        return PartSpec("swiglu", SwiGLUParams(dim, positive_int(mlp, "ff")),
                        {"w1": prefix + "gate", "w3": prefix + "up", "w2": prefix + "down"})
    if kind == "moe":
        require(mlp, ("expert", "router"), where)
        require(mlp["expert"], ("ff",), f"{where}.expert")
        require(mlp["router"], ("experts", "top"), f"{where}.router")
        params = RoutedExpertsParams(dim, positive_int(mlp["expert"], "ff"), positive_int(mlp["router"], "experts"),
                                     positive_int(mlp["router"], "top"), correction=True, renormalize=False)
        return PartSpec("routed_experts", params,
                        {"router": prefix + "router", "correction": prefix + "correction",
                         "w1": prefix + "e{}.gate", "w3": prefix + "e{}.up", "w2": prefix + "e{}.down"})
    raise ConfigError(f"{where}: unknown kind {kind!r}; known: dense, moe")


def tanupel_model_args(config: Mapping[str, Any]) -> ModelArgs:
    require(config, ("vocab", "width", "layers", "norm"), "Tanupel config.json")
    require(config["norm"], ("eps",), "Tanupel config.json: norm")
    dim = positive_int(config, "width")
    vocab = positive_int(config, "vocab")
    eps = float(config["norm"]["eps"])
    mult = float(config.get("residual_mult", 1.0))
    if not isinstance(config["layers"], (list, tuple)) or not config["layers"]:
        raise ConfigError("Tanupel config.json: 'layers' must be a non-empty list")

    layers = []
    for i, layer in enumerate(config["layers"]):
        where = f"layers[{i}]"
        require(layer, ("type", "mixer"), where)
        kind = layer["type"]
        if kind not in _MIXERS:
            raise ConfigError(f"{where}: unknown mixer type {kind!r}; known: {', '.join(sorted(_MIXERS))}")
        p = f"l{i}."
        try:
            mixer = _MIXERS[kind](dim, eps, layer["mixer"], p + "mix.", f"{where}.mixer")
            mlp = layer.get("mlp")
            ffn = _feed_forward(dim, mlp, p + "mlp.", f"{where}.mlp") if mlp is not None else None
        except ValueError as e:
            raise ConfigError(f"{where}: {e}") from None
        layers.append(LayerSpec(block="parallel", mixer=mixer, mixer_norm=_norm(dim, eps, p + "norm1"), ffn=ffn,
                                ffn_norm=None, block_params=ParallelBlockParams(mult)))

    n = len(layers)
    loop = config.get("loop")
    schedule = []
    times = 0
    if loop:
        require(loop, ("start", "stop", "times"), "Tanupel config.json: loop")
        start, stop, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
        if not (0 <= start < stop <= n) or times < 1:
            raise ConfigError(f"loop: layers {start}..{stop - 1} passed {times} times do not fit {n} layers")
        schedule += [ScheduleEntry(i) for i in range(start)]
        for t in range(times):
            # a pass has caches and states of its own (no kv_from) and opens with its step vector
            schedule += [ScheduleEntry(i, step_row=t if i == start else None) for i in range(start, stop)]
        schedule += [ScheduleEntry(i) for i in range(stop, n)]
    else:
        schedule = [ScheduleEntry(i) for i in range(n)]

    scale = float((config.get("embedding") or {}).get("scale", 1.0))
    return ModelArgs(
        architecture="Tanupel",
        dim=dim,
        vocab_size=vocab,
        max_positions=MAX_POSITIONS,
        tie_embeddings=False,
        embedding_name="embed",
        output_name="head",
        layers=tuple(layers),
        schedule=tuple(schedule),
        final_norm=_norm(dim, eps, "final.norm"),
        embedder=PartSpec("table", TableEmbeddingParams(vocab, dim, scale), {"table": "embed"}),
        step_table_name=STEP_TABLE if loop else None,
        step_table_rows=times,
    )


register_architecture("Tanupel", tanupel_model_args)
