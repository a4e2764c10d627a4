"""The model: parts put together as the description says, and its forward pass.

The reference's ``Transformer`` only holds weights and its forward is one
function written for one architecture (fastgen/model.py:151-202,
fastgen/forward.py:347-515).  Here the model is generic: it builds one block
per :class:`~fastgen_b200.config.LayerSpec` from the part registries and runs
the schedule; nothing in this file knows what a mixer or feed-forward does.
"""

from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

from ..config import ModelArgs, PartSpec, load_model_args
from ..parts.base import (
    Block,
    CacheSpec,
    Embedder,
    Part,
    StateSpec,
    WeightSpec,
    ScaledSum,
    StreamUpdate,
    make_block,
    make_connection,
    make_embedder,
    make_feed_forward,
    make_mixer,
    make_norm,
    split_pending,
)
from ..parts.params import TableEmbeddingParams
from ..weights.loader import load_weights


_MAKERS = {"mixer": make_mixer, "norm": make_norm, "feed_forward": make_feed_forward, "connection": make_connection}


def _build_blocks(args: ModelArgs) -> List[Block]:
    blocks = []
    for layer in args.layers:
        extra = {}
        for name, role, spec in layer.extra:
            if role not in _MAKERS:
                raise ValueError(f"part {name!r} of a layer has role {role!r}; known: {sorted(_MAKERS)}")
            extra[name] = _MAKERS[role](spec)
        blocks.append(
            make_block(
                layer.block,
                make_mixer(layer.mixer),
                make_norm(layer.mixer_norm),
                make_feed_forward(layer.ffn) if layer.ffn is not None else None,
                make_norm(layer.ffn_norm) if layer.ffn_norm is not None else None,
                params=layer.block_params,
                **extra,
            )
        )
    return blocks


def _build_embedder(args: ModelArgs) -> Embedder:
    spec = args.embedder
    if spec is None:
        spec = PartSpec("table", TableEmbeddingParams(args.vocab_size, args.dim), {"table": args.embedding_name})
    return make_embedder(spec)


def _collect_specs(args: ModelArgs, blocks: Sequence[Block], final_norm, embedder: Embedder) -> List[WeightSpec]:
    specs: Dict[str, WeightSpec] = {}
    ordered = list(embedder.weight_specs())
    for block in blocks:
        for part in block.parts():
            ordered.extend(part.weight_specs())
    ordered.extend(final_norm.weight_specs())
    if args.step_table_name is not None:
        ordered.append(WeightSpec(args.step_table_name, (args.step_table_rows, args.dim), ("normal", 0.1)))
    if args.pass_input_name is not None:
        ordered.append(WeightSpec(args.pass_input_name, (args.dim, 2 * args.dim), ("normal", (2 * args.dim) ** -0.5)))
    if not args.tie_embeddings:
        ordered.append(WeightSpec(args.output_name, (args.vocab_size, args.dim)))
    for s in ordered:
        if s.name in specs and specs[s.name].shape != s.shape:
            raise ValueError(f"tensor {s.name} is asked for with two shapes")
        specs.setdefault(s.name, s)
    return list(specs.values())


def model_weight_specs(args: ModelArgs) -> List[WeightSpec]:
    """Every checkpoint tensor a model of this description needs, in a fixed order."""
    return _collect_specs(args, _build_blocks(args), make_norm(args.final_norm), _build_embedder(args))


class Model:
    """Blocks, embedding and output of one model on one device."""

    def __init__(self, args: ModelArgs, ops) -> None:
        self.args = args
        self.ops = ops
        self.blocks = _build_blocks(args)
        self.final_norm = make_norm(args.final_norm)
        self.embedder = _build_embedder(args)
        self.embedding: Optional[torch.Tensor] = None
        self.output: Optional[torch.Tensor] = None
        self.step_table: Optional[torch.Tensor] = None  # float32 [rows, dim]
        # the two halves of the map that opens a pass: what meets the stream, what meets the embedder's output
        self.pass_stream: Optional[torch.Tensor] = None
        self.pass_embed: Optional[torch.Tensor] = None

    # -- description -----------------------------------------------------------
    def weight_specs(self) -> List[WeightSpec]:
        return _collect_specs(self.args, self.blocks, self.final_norm, self.embedder)

    def cache_specs(self) -> List[Optional[CacheSpec]]:
        return [self.blocks[e.layer].mixer.cache_spec() for e in self.args.schedule]

    def state_specs(self) -> List[Optional[StateSpec]]:
        return [self.blocks[e.layer].mixer.state_spec() for e in self.args.schedule]

    def embedder_state_spec(self) -> Optional[StateSpec]:
        return self.embedder.state_spec()

    def kv_from(self) -> List[Optional[int]]:
        return [e.kv_from for e in self.args.schedule]

    def cache_bytes_per_token(self, elt_size: int) -> int:
        """Bytes of keys and values one token adds over all runs that own a cache."""
        total = 0
        for spec, src in zip(self.cache_specs(), self.kv_from()):
            if spec is not None and src is None:
                total += spec.n_pools * spec.n_kv_heads * spec.head_dim * elt_size
        return total

    def weight_bytes(self) -> int:
        """Bytes of every tensor a step reads (fused buffers, embedding once if tied)."""
        seen, total = set(), 0
        def add(t):
            nonlocal total
            # (a view into a tensor that is counted whole, such as one half of a stacked pair, is skipped)
            if t is not None and t.data_ptr() not in seen and (t._base is None or t._base.data_ptr() not in seen):
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()
        def add_part(part):
            for v in vars(part).values():
                if isinstance(v, torch.Tensor):
                    add(v)
                elif isinstance(v, Part):  # a part made of parts (two mixers side by side)
                    add_part(v)
        add(self.output)
        add(self.step_table)
        add(self.pass_stream)
        add(self.pass_embed)
        for block in self.blocks:
            for part in block.parts():
                add_part(part)
        add_part(self.final_norm)
        return total

    # -- weights -----------------------------------------------------------------
    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        dt = self.ops.act_dtype
        self.embedder.bind({local: tensors[name] for local, name in self.embedder.names.items()}, self.ops)
        self.embedding = self.embedder.table()
        if self.args.tie_embeddings:
            self.output = self.embedding
        else:
            self.output = tensors[self.args.output_name].to(dt).contiguous()
        for block in self.blocks:
            for part in block.parts():
                part.bind({local: tensors[name] for local, name in part.names.items()}, self.ops)
        self.final_norm.bind(
            {local: tensors[name] for local, name in self.final_norm.names.items()}, self.ops
        )
        if self.args.step_table_name is not None:
            # the vectors join the float32 residual sum: float32 whatever they were stored in
            self.step_table = tensors[self.args.step_table_name].float().contiguous()
        if self.args.pass_input_name is not None:
            w = tensors[self.args.pass_input_name].to(dt)
            self.pass_stream = w[:, : self.args.dim].contiguous()
            self.pass_embed = w[:, self.args.dim :].contiguous()

    @staticmethod
    def load(model_dir, dtype: torch.dtype, device) -> "Model":
        """Read ``config.json`` and the safetensors of ``model_dir``."""
        from ..csrc.ops import Ops

        args = load_model_args(model_dir)
        model = Model(args, Ops(dtype, device))
        ignore = [args.output_name or "lm_head.weight"] if args.tie_embeddings else []
        ignore += list(args.optional_tensors)
        tensors = load_weights(model_dir, model.weight_specs(), device, ignore=ignore)
        model.bind(tensors)
        del tensors
        return model

    @staticmethod
    def random(args: ModelArgs, dtype: torch.dtype, device, seed: int = 0) -> "Model":
        """A model with seeded random weights drawn on the device (no files):
        matrices N(0, 0.02), norm weights 1, as the random-weights writer does."""
        from ..csrc.ops import Ops

        model = Model(args, Ops(dtype, device))
        gen = torch.Generator(device=device).manual_seed(int(seed))
        tensors = {}
        for spec in model.weight_specs():
            if spec.init[0] == "normal":
                t = torch.empty(spec.shape, dtype=torch.bfloat16, device=device)
                t.normal_(0.0, spec.init[1], generator=gen)
            elif spec.init[0] == "uniform":
                t = torch.empty(spec.shape, dtype=torch.float32, device=device)
                t.uniform_(spec.init[1], spec.init[2], generator=gen)
                t = t.to(torch.bfloat16)
            elif spec.init[0] == "constant":
                t = torch.full(spec.shape, spec.init[1], dtype=torch.bfloat16, device=device)
            elif spec.init[0] in ("ones", "ones_jitter"):
                t = torch.ones(spec.shape, dtype=torch.bfloat16, device=device)
            else:
                t = torch.randint(0, spec.init[1], spec.shape, generator=gen, device=device, dtype=torch.int32)
            tensors[spec.name] = t
        model.bind(tensors)
        return model

    # -- forward -----------------------------------------------------------------
    def _mix_input(self, h, pending, embed_part):
        """``x <- W [x; x0]``: what is pending joins the stream (float32), the stream meets its half of
        the map, and the embedder's half (``embed_part``, float32) is left pending: the next norm's
        kernel adds it."""
        ops = self.ops
        delta, delta_norm = split_pending(pending)
        if delta is not None and delta_norm is not None:
            delta = delta_norm.forward(delta, out_dtype=torch.float32)
        total = ScaledSum.of(delta)
        if len(total.terms) > 4 or len({term.dtype for term, _ in total.terms}) > 1:
            total.add_into(h, ops)
            total = ScaledSum([])
        x = torch.empty(h.shape, dtype=ops.act_dtype, device=h.device)
        ops.rmsnorm_sum(h, total.terms, None, 0.0, out=x, row=total.row)
        return ops.linear(x, self.pass_stream, out_dtype=torch.float32), ScaledSum([(embed_part, 1.0)])

    def forward(self, ctx, memories) -> Optional[torch.Tensor]:
        """Run the step's tokens through the schedule.  Returns float32 logits
        ``[len(ctx.want_rows), vocab]`` (``None`` when no logits are wanted).
        ``memories`` is the cache's :class:`~fastgen_b200.cache.StepMemories`: one
        ``LayerMemory`` per schedule entry, and the state of an embedder that keeps one."""
        ops = self.ops
        t = ctx.n_tokens
        # one residual stream [T, dim], or several side by side [T, streams, dim] that start equal
        shape = (t, self.args.dim) if self.args.streams is None else (t, self.args.streams, self.args.dim)
        h = torch.empty(shape, dtype=torch.float32, device=ops.device)
        self.embedder.forward(ctx, getattr(memories, "embedder_state", None), h)
        pending = None
        embed_part = None
        if self.pass_embed is not None:
            # the embedder's output meets its half of the map once a step: that product is the same
            # before every pass
            x0 = torch.empty((t, self.args.dim), dtype=ops.act_dtype, device=ops.device)
            ops.rmsnorm_sum(h, (), None, 0.0, out=x0)
            embed_part = ops.linear(x0, self.pass_embed, out_dtype=torch.float32)
        for e, entry in enumerate(self.args.schedule):
            if entry.mix_input:
                h, pending = self._mix_input(h, pending, embed_part)
            if entry.step_row is not None:
                # the pass's step vector joins whatever the layer before left pending
                pending = ScaledSum.of(pending).plus(ScaledSum([], row=self.step_table[entry.step_row]))
            h, pending = self.blocks[entry.layer].forward(h, pending, ctx, memories[e])
        if ctx.n_want == 0:
            return None
        if self.args.streams is not None:
            # the last update of the streams, their sum and the norm in one kernel
            x = self.final_norm.streams_forward(h, update=pending, rows=ctx.want_rows)
        else:
            delta, delta_norm = split_pending(pending)
            if delta is None:
                x = self.final_norm.forward(h, rows=ctx.want_rows)
            else:
                x = self.final_norm.add_forward(h, delta, rows=ctx.want_rows, delta_norm=delta_norm)
        logits = ops.linear(x, self.output, out_dtype=torch.float32)
        if self.args.logit_scale != 1.0 or self.args.logit_softcap:
            ops.scale_softcap(logits, self.args.logit_scale, self.args.logit_softcap)
        return logits
