"""``Palulorn``: config.json keys -> model description.

A decoder whose layers are listed one by one under ``layers``.  Every layer is a pre-norm block with RMS
norms (plain weights): ``x <- x + mixer(norm1(x)); x <- x + ff(norm2(x))``.  A run of layers
(``loop{start, stop, times}``) is passed several times with the same weights; every pass has a cache and
a state of its own and opens with ``x <- W_in [x; x0] + step[t]`` (``x0``: the embedding output, ``W_in``
the tensor ``loop.in``, ``step`` the tensor ``loop.step``).

Keys read: ``architecture``, ``vocab``, ``width``, ``norm.eps``, ``embedding.scale`` (optional),
``loop{start, stop, times}`` (optional) and per layer ``type``, ``mixer`` and ``mlp`` (or null):

* ``parallel``: ``left{heads, kv_heads, dim, vdim, scale, q_temp{coef, every}}``: causal attention without
  a rotation whose values are its keys, with biases on q, k and o, a query temperature, a sink per head
  and a sigmoid gate per head; ``right{heads, dim, vdim, gate_cap}``: the matrix memory with exponential
  gates (``parts/matrix_memory.py``).  The result is half the sum of the two outputs, each RMS-normed
  over the model width first;
* ``rglru``: ``width, blocks, conv``: Griffin's recurrent block (``parts/gated_linear_recurrence.py``);
* ``attention``: ``heads, kv_heads, dim, vdim, scale, conv, rot{dims, base, scaling.factor}, mask.size``:
  grouped-query attention over a sliding window with biases on q, k and v, a short causal convolution
  on q, k and v, an RMS norm of q and k per head and a rotation of a head's first ``rot.dims`` dimensions
  (dimension ``i`` with ``i + dims/2``, every frequency divided by ``scaling.factor``);
* ``mlp{kind: moe, expert{ff}, router{experts, top, scale, groups{count, keep}}, shared{ff}}``: experts
  ``down(relu(up x)^2)`` chosen by sigmoid scores among the best groups, a shared expert beside them.

Tensors: ``embed``, ``loop.in``, ``loop.step``, ``l<i>.norm1|norm2``, ``l<i>.mix.*``,
``l<i>.mlp.router|e<j>.up|e<j>.down|shared.up|shared.down``, ``final.norm``, ``head``.
"""

from __future__ import annotations

from typing import Any, Mapping, Optional

from ..parts.params import (
    AttentionParams,
    DenseMLPParams,
    GatedLinearRecurrenceParams,
    MatrixMemoryParams,
    NoPositionParams,
    RMSNormParams,
    RopeParams,
    RoutedExpertsParams,
    SideBySideParams,
    TableEmbeddingParams,
)
from .model_args import ConfigError, LayerSpec, ModelArgs, PartSpec, ScheduleEntry, positive_int, require
from .registry import register_architecture

#: the design sets no limit on positions; the engine's own limits (cache size) apply
MAX_POSITIONS = 1 << 30

STEP_TABLE = "loop.step"
PASS_INPUT = "loop.in"

#: constants the design fixes
EXPERT_ACT = "relu2"
GROUP_TOP = 2
RENORM_EPS = 1e-20
DECAY = 8.0


def _norm(dim: int, eps: float, name: str) -> PartSpec:
    return PartSpec("rmsnorm", RMSNormParams(dim, eps), {"weight": name})


def _rope(rot: Optional[Mapping[str, Any]], head_dim: int, where: str) -> PartSpec:
    if not rot:
        return PartSpec("none", NoPositionParams())
    require(rot, ("dims", "base"), f"{where}.rot")
    linear = None
    sc = rot.get("scaling")
    if sc:
        require(sc, ("factor",), f"{where}.rot.scaling")
        linear = float(sc["factor"])
    return PartSpec("rope", RopeParams(head_dim=head_dim, theta=float(rot["base"]), rot_dims=positive_int(rot, "dims"),
                                       linear_factor=linear))


def _sink_attention(dim: int, eps: float, m: Mapping[str, Any], prefix: str, where: str) -> PartSpec:
    require(m, ("heads", "kv_heads", "dim", "vdim", "scale"), where)
    head_dim = positive_int(m, "dim")
    if positive_int(m, "vdim") != head_dim:
        raise ConfigError(f"{where}: the values are the keys, so vdim must equal dim")
    qt = m.get("q_temp")
    if qt:
        require(qt, ("coef", "every"), f"{where}.q_temp")
    params = AttentionParams(
        dim=dim,
        n_heads=positive_int(m, "heads"),
        n_kv_heads=positive_int(m, "kv_heads"),
        head_dim=head_dim,
        position=PartSpec("none", NoPositionParams()),
        softmax_scale=float(m["scale"]),
        bias=True,
        o_bias=True,
        shared_kv=True,
        q_temp=(float(qt["coef"]), positive_int(qt, "every")) if qt else None,
        sink=True,
        head_gate=True,
    )
    names = {"wq": "q", "wk": "k", "wo": "o", "bq": "q.b", "bk": "k.b", "bo": "o.b", "sink": "sink", "wg": "g"}
    return PartSpec("gqa_attention", params, {k: prefix + v for k, v in names.items()})


def _matrix_memory(dim: int, eps: float, m: Mapping[str, Any], prefix: str, where: str) -> PartSpec:
    require(m, ("heads", "dim", "vdim", "gate_cap"), where)
    params = MatrixMemoryParams(dim=dim, n_heads=positive_int(m, "heads"), head_dim=positive_int(m, "dim"),
                                v_head_dim=positive_int(m, "vdim"), gate_cap=float(m["gate_cap"]), eps=eps)
    names = {"wq": "q", "wk": "k", "wv": "v", "wg": "g", "wo": "o", "norm": "norm", "wi": "i", "bi": "i.b", "wf": "f",
             "bf": "f.b"}
    return PartSpec("matrix_memory", params, {k: prefix + v for k, v in names.items()})


def _pair(dim: int, eps: float, m: Mapping[str, Any], prefix: str, where: str) -> PartSpec:
    require(m, ("left", "right"), where)
    params = SideBySideParams(
        left=_sink_attention(dim, eps, m["left"], prefix + "left.", f"{where}.left"),
        right=_matrix_memory(dim, eps, m["right"], prefix + "right.", f"{where}.right"),
        # half the sum of the two outputs, each normed over the model width first
        left_scale=0.5,
        right_scale=0.5,
        left_norm=_norm(dim, eps, prefix + "left.out"),
        right_norm=_norm(dim, eps, prefix + "right.out"),
    )
    return PartSpec("side_by_side", params, {})


def _recurrent(dim: int, eps: float, m: Mapping[str, Any], prefix: str, where: str) -> PartSpec:
    require(m, ("width", "blocks", "conv"), where)
    params = GatedLinearRecurrenceParams(dim=dim, width=positive_int(m, "width"), blocks=positive_int(m, "blocks"),
                                         conv=positive_int(m, "conv"), decay=DECAY)
    names = {"wy": "y", "by": "y.b", "wx": "x", "bx": "x.b", "conv": "conv", "conv_b": "conv.b", "ra": "ra",
             "ra_b": "ra.b", "ri": "ri", "ri_b": "ri.b", "lam": "lam", "wo": "o"}
    return PartSpec("gated_linear_recurrence", params, {k: prefix + v for k, v in names.items()})


def _window_attention(dim: int, eps: float, m: Mapping[str, Any], prefix: str, where: str) -> PartSpec:
    require(m, ("heads", "kv_heads", "dim", "vdim", "scale"), where)
    head_dim = positive_int(m, "dim")
    mask = m.get("mask")
    if mask:
        require(mask, ("size",), f"{where}.mask")
    params = AttentionParams(
        dim=dim,
        n_heads=positive_int(m, "heads"),
        n_kv_heads=positive_int(m, "kv_heads"),
        head_dim=head_dim,
        v_head_dim=positive_int(m, "vdim"),
        position=_rope(m.get("rot"), head_dim, where),
        window=positive_int(mask, "size") if mask else None,
        softmax_scale=float(m["scale"]),
        qk_layout="half_split",
        bias=True,
        o_bias=False,
        qk_norm="head",
        qk_norm_eps=eps,
        conv=int(m.get("conv") or 0),
    )
    names = {"wq": "q", "wk": "k", "wv": "v", "wo": "o", "bq": "q.b", "bk": "k.b", "bv": "v.b", "q_norm": "q.norm",
             "k_norm": "k.norm"}
    if params.conv:
        names.update({"conv_q": "q.conv", "conv_k": "k.conv", "conv_v": "v.conv"})
    return PartSpec("gqa_attention", params, {k: prefix + v for k, v in names.items()})


_MIXERS = {"parallel": _pair, "rglru": _recurrent, "attention": _window_attention}


def _feed_forward(dim: int, mlp: Mapping[str, Any], prefix: str, where: str) -> PartSpec:
    require(mlp, ("kind",), where)
    if mlp["kind"] != "moe":
        raise ConfigError(f"{where}: unknown kind {mlp['kind']!r}; known: moe")
    require(mlp, ("expert", "router"), where)
    require(mlp["expert"], ("ff",), f"{where}.expert")
    router = mlp["router"]
    require(router, ("experts", "top"), f"{where}.router")
    groups = router.get("groups")
    if groups:
        require(groups, ("count", "keep"), f"{where}.router.groups")
    shared = mlp.get("shared")
    if shared:
        require(shared, ("ff",), f"{where}.shared")
        shared = PartSpec("dense_mlp", DenseMLPParams(dim, positive_int(shared, "ff"), act=EXPERT_ACT),
                          {"up": prefix + "shared.up", "down": prefix + "shared.down"})
    params = RoutedExpertsParams(
        dim, positive_int(mlp["expert"], "ff"), positive_int(router, "experts"), positive_int(router, "top"),
        correction=False, renormalize=True, score="sigmoid",
        groups=(positive_int(groups, "count"), positive_int(groups, "keep")) if groups else None,
        group_top=GROUP_TOP, renorm_eps=RENORM_EPS, weight_scale=float(router.get("scale", 1.0)), act=EXPERT_ACT,
        shared=shared or None)
    return PartSpec("routed_experts", params,
                    {"router": prefix + "router", "w3": prefix + "e{}.up", "w2": prefix + "e{}.down"})


def palulorn_model_args(config: Mapping[str, Any]) -> ModelArgs:
    require(config, ("vocab", "width", "layers", "norm"), "Palulorn config.json")
    require(config["norm"], ("eps",), "Palulorn config.json: norm")
    dim = positive_int(config, "width")
    vocab = positive_int(config, "vocab")
    eps = float(config["norm"]["eps"])
    if not isinstance(config["layers"], (list, tuple)) or not config["layers"]:
        raise ConfigError("Palulorn config.json: 'layers' must be a non-empty list")

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
        layers.append(LayerSpec(block="prenorm", mixer=mixer, mixer_norm=_norm(dim, eps, p + "norm1"), ffn=ffn,
                                ffn_norm=_norm(dim, eps, p + "norm2") if ffn is not None else None))

    n = len(layers)
    loop = config.get("loop")
    times = 0
    if loop:
        require(loop, ("start", "stop", "times"), "Palulorn config.json: loop")
        start, stop, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
        if not (0 <= start < stop <= n) or times < 1:
            raise ConfigError(f"loop: layers {start}..{stop - 1} passed {times} times do not fit {n} layers")
        schedule = [ScheduleEntry(i) for i in range(start)]
        for t in range(times):
            # a pass has caches and states of its own (no kv_from); it opens by mixing the embedding
            # output into the stream, then adds its step vector
            schedule += [ScheduleEntry(i, step_row=t if i == start else None, mix_input=i == start)
                         for i in range(start, stop)]
        schedule += [ScheduleEntry(i) for i in range(stop, n)]
    else:
        schedule = [ScheduleEntry(i) for i in range(n)]

    scale = float((config.get("embedding") or {}).get("scale", 1.0))
    return ModelArgs(
        architecture="Palulorn",
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
        pass_input_name=PASS_INPUT if loop else None,
        optional_tensors=tuple(f"l{i}.norm2" for i, layer in enumerate(config["layers"]) if layer.get("mlp") is None),
    )


register_architecture("Palulorn", palulorn_model_args)
