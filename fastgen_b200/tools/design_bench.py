"""Throughput of one design beside another at equal size, step by step and kernel by kernel.

``bench.py --design sinorax|zeladra|tanupel|palulorn`` runs this: prefill and decode throughput of a model of that
design at a few sizes that resemble a real model's layers (random weights), beside a Llama-shaped model of
the same width, heads, head size, number of layers and number of parameters a layer, and the
time of each kernel family of the two designs at those sizes with its fraction of the roofline
(HBM bandwidth for the elementwise kernels and single-token attention, tensor throughput for
prompt attention).  Timed with CUDA events, L2 flushed before every timed launch; the Tanupel
table times its few-token rows as captured launches.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Callable, Dict, List

import torch

PAGE = 64
PREFILL_TOKENS = 2048
DECODE_BATCH = 8
DECODE_CONTEXT = 2048
SEED = 4

#: name -> (width, layers, query heads, key/value heads, head size, SwiGLU width, vocabulary, window)
SIZES = {
    "1b-like": (2048, 6, 32, 8, 64, 8192, 128256, 1024),
    "3b-like": (3072, 6, 24, 8, 128, 8192, 128256, 1024),
}


def llama_config(width, layers, heads, kv, head_dim, ffn, vocab, window=None) -> dict:
    cfg = dict(architectures=["LlamaForCausalLM"], hidden_size=width, intermediate_size=ffn, num_hidden_layers=layers,
               num_attention_heads=heads, num_key_value_heads=kv, head_dim=head_dim, rms_norm_eps=1e-5, vocab_size=vocab,
               tie_word_embeddings=False, rope_theta=500000.0, max_position_embeddings=131072)
    if window:
        cfg["sliding_window"] = window
    return cfg


def sinorax_config(width, layers, heads, kv, head_dim, ffn, vocab, window, kinds=("attention", "attention", "attention_2")) -> dict:
    """Two softmax layers, then one with sigmoid weights and a window, and so on; the dense
    feed-forward is half as wide again as the gated one, which gives a layer the same number
    of parameters."""
    out = []
    for i in range(layers):
        kind = kinds[i % len(kinds)]
        mixer = dict(heads=heads, kv_heads=kv, dim=head_dim, vdim=head_dim, scale=head_dim ** -0.5)
        if kind == "attention":
            mixer["rot"] = dict(dims=head_dim, base=500000.0, scaling=dict(factor=2.0))
        else:
            mixer["mask"] = dict(size=window)
        out.append(dict(type=kind, mixer=mixer, mlp=dict(kind="dense", ff=ffn * 3 // 2)))
    return dict(architecture="Sinorax", vocab=vocab, width=width, norm=dict(eps=1e-5), logit_scale=1.0, logit_softcap=30.0,
                embedding=dict(bigram=dict(buckets=65521, mul_prev=1000003, mul_cur=31)), layers=out)


def zeladra_config(width, layers, heads, kv, head_dim, ffn, vocab, window) -> dict:
    """Latent attention, the state-space mixer and windowed attention that keeps the first four
    positions, in turn (every second latent layer reads the first one's cache), on two residual
    streams; every layer has the gated feed-forward of the Llama shape."""
    latent = dict(heads=heads, dim=head_dim, rot_dim=head_dim // 2, vdim=head_dim, q_rank=width * 3 // 4,
                  kv_rank=4 * head_dim, scale=(head_dim * 3 // 2) ** -0.5,
                  rot=dict(dims=head_dim // 2, base=500000.0, scaling=dict(factor=4.0, original=8192, fast=32.0, slow=1.0)))
    ssm = dict(heads=2 * width // 64, vdim=64, state=128, groups=8, conv=4, norm_groups=8)
    att = dict(heads=heads, kv_heads=kv, dim=head_dim, vdim=head_dim, scale=head_dim ** -0.5,
               rot=dict(dims=head_dim, base=500000.0), mask=dict(size=window, keep_first=4))
    out, first_latent = [], None
    for i in range(layers):
        kind = ("latent_attention", "mamba2", "attention")[i % 3]
        mixer = dict({"latent_attention": latent, "mamba2": ssm, "attention": att}[kind])
        if kind == "latent_attention":
            if first_latent is None:
                first_latent = i
            elif (i // 3) % 2 == 1:
                mixer["kv_from"] = first_latent
        out.append(dict(type=kind, mixer=mixer, mlp=dict(kind="dense", ff=ffn)))
    return dict(architecture="Zeladra", vocab=vocab, width=width, norm=dict(eps=1e-5), embedding=dict(scale=1.0),
                streams=2, layers=out)


def tanupel_config(width, layers, heads, kv, head_dim, ffn, vocab, window=None, experts=8, top=2) -> dict:
    """A pair of mixers (capped attention with half the heads beside a gated delta rule with the
    other half) and plain attention with the whole projection's query/key norm, in turn; the
    feed-forwards are dense and routed in turn, the routed one with ``experts`` experts of
    ``ffn / experts`` rows (as many parameters as the dense one, ``top`` of them a token).  All
    layers are one run that is passed once, so the pass's step vector is added.  A layer has the
    parameters of the Llama shape's layer, up to the small low-rank maps of the delta rule."""
    rot = dict(dims=head_dim // 2, base=500000.0)
    att = dict(heads=heads, kv_heads=kv, dim=head_dim, vdim=head_dim, scale=head_dim ** -0.5,
               rot=dict(rot, scaling=dict(factor=8.0, low=1.0, high=4.0, original=8192)))
    left = dict(heads=heads // 2, kv_heads=max(1, kv // 2), dim=head_dim, vdim=head_dim, scale=head_dim ** -0.5, softcap=50.0,
                rot=dict(rot, scaling=dict(factor=2.0)))
    right = dict(heads=heads // 2, kv_heads=max(1, kv // 2), dim=head_dim, vdim=head_dim, conv=4, decay_rank=32, gate_rank=32)
    pair = dict(left=left, right=right, left_scale=0.5, right_scale=1.0)
    dense = dict(kind="dense", ff=ffn)
    routed = dict(kind="moe", expert=dict(ff=ffn // experts), router=dict(experts=experts, top=top))
    out = []
    for i in range(layers):
        kind = ("parallel", "attention")[i % 2]
        out.append(dict(type=kind, mixer=dict(pair if kind == "parallel" else att), mlp=dict(dense if (i // 2) % 2 == 0 else routed)))
    return dict(architecture="Tanupel", vocab=vocab, width=width, norm=dict(eps=1e-5), embedding=dict(scale=1.0),
                residual_mult=0.5, loop=dict(start=0, stop=layers, times=1), layers=out)


def palulorn_config(width, layers, heads, kv, head_dim, ffn, vocab, window=1024, experts=8, top=2) -> dict:
    """A pair of mixers (attention with a sink, whose values are its keys, with half the heads beside a
    matrix memory with the other half), windowed attention with a short convolution and a norm per head,
    and the gated linear recurrent unit, in turn; every feed-forward is routed: ``experts`` ungated
    experts of ``3 ffn / (2 experts)`` rows with a squared ReLU (together the parameters of the Llama
    shape's gated feed-forward, ``top`` of them a token, chosen among the best half of four groups) and a
    shared expert of that size.  All layers are one run that is passed once, so the pass opens by mixing
    the embedding output in and adding its step vector."""
    left = dict(heads=heads // 2, kv_heads=max(1, kv // 2), dim=head_dim, vdim=head_dim, scale=head_dim ** -0.5,
                q_temp=dict(coef=0.1, every=512))
    right = dict(heads=heads // 2, dim=head_dim, vdim=head_dim, gate_cap=15.0)
    att = dict(heads=heads, kv_heads=kv, dim=head_dim, vdim=head_dim, scale=head_dim ** -0.5, conv=4,
               rot=dict(dims=head_dim // 2, base=500000.0, scaling=dict(factor=4.0)), mask=dict(size=window))
    lru = dict(width=width, blocks=16, conv=4)
    f = ffn * 3 // 2 // experts
    routed = dict(kind="moe", expert=dict(ff=f), router=dict(experts=experts, top=top, scale=1.0, groups=dict(count=4, keep=2)),
                  shared=dict(ff=f))
    mixers = (("parallel", dict(left=left, right=right)), ("attention", att), ("rglru", lru))
    out = [dict(type=mixers[i % 3][0], mixer=dict(mixers[i % 3][1]), mlp=dict(routed)) for i in range(layers)]
    return dict(architecture="Palulorn", vocab=vocab, width=width, norm=dict(eps=1e-5), embedding=dict(scale=1.0),
                loop=dict(start=0, stop=layers, times=1), layers=out)


class Timer:
    """CUDA-event times of single launches, each after a write larger than L2."""

    def __init__(self, device) -> None:
        self.flush = torch.empty(64 * 1024 * 1024, dtype=torch.float32, device=device)  # 256 MB

    def us(self, fn: Callable[[], None], reps: int = 7, graph: bool = False) -> float:
        """``graph``: the launches of ``fn`` are captured once and the replay is timed, so that an
        operation of several small launches shows its time on the device and not the host's."""
        for _ in range(3):
            fn()
        if graph:
            torch.cuda.synchronize()
            side = torch.cuda.Stream()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.stream(side):
                fn()
                torch.cuda.synchronize()
                with torch.cuda.graph(g, stream=side):
                    fn()
            torch.cuda.synchronize()
            fn = g.replay
            fn()
        times = []
        for _ in range(reps):
            self.flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b) * 1e3)
        times.sort()
        return times[len(times) // 2]


def _engine(cfg, device, max_requests, tokens):
    from ..config import model_args_from_config
    from ..engine import Engine, Model

    model = Model.random(model_args_from_config(cfg), torch.bfloat16, device, seed=SEED)
    n_pages = max_requests * (-(-(tokens + 1) // PAGE)) + 2
    return Engine(model, page_size=PAGE, n_pages=n_pages, max_requests=max_requests, max_length=tokens + PAGE,
                  num_cuda_graphs=max_requests, max_step_tokens=PREFILL_TOKENS)


def _fill(engine) -> None:
    for grp in engine.cache.groups:
        grp.k_pages.normal_(0.0, 1.0)
        if grp.v_pages is not None:
            grp.v_pages.normal_(0.0, 1.0)


def model_throughput(cfg, device) -> Dict[str, float]:
    """Prefill tokens/s of one 2,048-token prompt and decode tokens/s at batch 8 around position
    2,048, through the engine's step function (graphs included), device-timed."""
    from ..csrc.ops import Ops
    from ..engine import StepEntry
    from ..sampling import Sampler

    engine = _engine(cfg, device, DECODE_BATCH, max(PREFILL_TOKENS, DECODE_CONTEXT))
    vocab = engine.model.args.vocab_size
    gen = torch.Generator().manual_seed(SEED)
    toks = torch.randint(0, vocab, (PREFILL_TOKENS,), generator=gen).tolist()

    def prefill_once():
        engine.admit("p")
        engine.step([StepEntry("p", toks, [PREFILL_TOKENS - 1])])
        engine.release("p")

    for _ in range(3):
        prefill_once()
    times = []
    for _ in range(5):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        prefill_once()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
    pre_ms = min(times)

    steps, warm = 64, 5
    ids = [f"d{i}" for i in range(DECODE_BATCH)]
    for rid in ids:
        r = engine.admit(rid)
        engine.cache.reserve(r, DECODE_CONTEXT - steps - warm)
        engine.cache.advance(r, DECODE_CONTEXT - steps - warm)
    _fill(engine)
    reqs = [engine.cache.get(rid) for rid in ids]
    slots = [r.slot for r in reqs]
    sampler = Sampler(engine.ops, vocab, DECODE_BATCH, use_sampling=False)
    tokens = torch.randint(0, vocab, (DECODE_BATCH,), generator=gen).to(device, torch.int32)

    def one_step():
        nonlocal tokens
        for r in reqs:
            engine.cache.reserve(r, r.length + 1)
        engine.cache.flush_tables()
        logits = engine.graphs.run(tokens, [r.length for r in reqs], slots)
        tokens, _ = sampler.sample(logits, [0.0] * DECODE_BATCH, [0] * DECODE_BATCH, [0] * DECODE_BATCH)
        for r in reqs:
            engine.cache.advance(r, r.length + 1)

    for _ in range(warm):
        one_step()
    torch.cuda.synchronize()
    launches = Ops.launches
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        one_step()
    b.record()
    torch.cuda.synchronize()
    dec_ms = a.elapsed_time(b) / steps
    launches = (Ops.launches - launches) // steps
    engine.ops.check_status()
    weight_bytes = engine.model.weight_bytes()
    out = dict(prefill_tok_s=round(PREFILL_TOKENS / pre_ms * 1e3, 1), prefill_ms=round(pre_ms, 3),
               decode_tok_s=round(DECODE_BATCH / dec_ms * 1e3, 1), decode_ms_per_step=round(dec_ms, 4),
               decode_launches_per_step=int(launches), weight_gb=round(weight_bytes / 1e9, 3),
               decode_weight_stream_gbs=round(weight_bytes / (dec_ms * 1e-3) / 1e9, 1))
    for rid in ids:
        engine.release(rid)
    del engine
    torch.cuda.empty_cache()
    return out


def _attention_times(cfg, device, timer: Timer, layer: int, flops_window, heads, kv, head_dim, pick=None) -> Dict[str, float]:
    """The attention launches of one layer alone: a 2,048-token prompt, and 8 single tokens at
    position 2,048, with what the mixer adds around them (turning the outputs back)."""
    from ..engine import StepEntry

    engine = _engine(cfg, device, DECODE_BATCH, DECODE_CONTEXT)
    _fill(engine)
    mixer = engine.model.blocks[layer].mixer
    if pick is not None:
        mixer = pick(mixer)
    memory = engine.memories[layer]
    out = {}
    gen = torch.Generator().manual_seed(SEED)

    def context(entries):
        reqs = engine._validate(entries)
        for e, r in zip(entries, reqs):
            engine.cache.reserve(r, r.length + len(e.tokens))
        engine.cache.flush_tables()
        return engine.build_context(entries, reqs)

    # the prompt
    engine.admit("p")
    ctx = context([StepEntry("p", [1] * PREFILL_TOKENS, [])])
    q = torch.randn(PREFILL_TOKENS, mixer.q_width, generator=gen).to(device, torch.bfloat16)
    o = torch.empty_like(q)
    us = timer.us(lambda: mixer._attend(q, o, ctx, memory))
    w = flops_window or PREFILL_TOKENS
    keys = sum(min(i + 1, w) for i in range(PREFILL_TOKENS))
    out["prefill_us"] = round(us, 1)
    out["prefill_tflops"] = round(4 * head_dim * heads * keys / (us * 1e-6) / 1e12, 1)
    if getattr(mixer, "v_unfreqs", None) is not None:
        out["prefill_unrotate_us"] = round(timer.us(lambda: engine.ops.rotate_heads(
            o, ctx.pos, ctx.req, mixer.v_unfreqs, heads, head_dim)), 1)
    engine.release("p")
    # single tokens
    ids = [f"d{i}" for i in range(DECODE_BATCH)]
    for rid in ids:
        r = engine.admit(rid)
        engine.cache.reserve(r, DECODE_CONTEXT - 1)
        engine.cache.advance(r, DECODE_CONTEXT - 1)
    ctx = context([StepEntry(rid, [1], []) for rid in ids])
    q = torch.randn(DECODE_BATCH, mixer.q_width, generator=gen).to(device, torch.bfloat16)
    o = torch.empty_like(q)
    us = timer.us(lambda: mixer._attend(q, o, ctx, memory))
    keys = min(DECODE_CONTEXT, flops_window or DECODE_CONTEXT)
    out["decode_us"] = round(us, 1)
    out["decode_gbs"] = round(DECODE_BATCH * keys * 2 * kv * head_dim * 2 / (us * 1e-6) / 1e9, 1)
    if getattr(mixer, "v_unfreqs", None) is not None:
        out["decode_unrotate_us"] = round(timer.us(lambda: engine.ops.rotate_heads(
            o, ctx.pos, ctx.req, mixer.v_unfreqs, heads, head_dim)), 1)
    engine.ops.check_status()
    del engine
    torch.cuda.empty_cache()
    return out


def kernel_table(size, device, peaks) -> Dict[str, dict]:
    """Every kernel family of the two designs alone at one size: microseconds and the fraction
    of the roofline (bytes or FLOPs that the operation needs over the measured peak)."""
    from ..csrc.ops import Ops

    width, _layers, heads, kv, head_dim, ffn, vocab, window = size
    ops = Ops(torch.bfloat16, device)
    timer = Timer(device)
    gen = torch.Generator().manual_seed(SEED)
    hbm, tensor = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12
    table: Dict[str, dict] = {}

    def bw(name, us, nbytes):
        table[name] = dict(us=round(us, 1), gbs=round(nbytes / (us * 1e-6) / 1e9, 1), hbm_frac=round(nbytes / (us * 1e-6) / hbm, 3))

    def rand(*shape, dtype=torch.bfloat16):
        return torch.randn(*shape, generator=gen).to(device, dtype)

    for t in (PREFILL_TOKENS, DECODE_BATCH):
        h, delta = rand(t, width, dtype=torch.float32), rand(t, width)
        out = torch.empty(t, width, dtype=torch.bfloat16, device=device)
        w32 = [rand(1, dtype=torch.float32), rand(width, dtype=torch.float32), rand(width, dtype=torch.float32)]
        nbytes = t * width * (4 + 4 + 2 + 2)
        bw(f"norm+sum t={t}: dynamic tanh (post, sum, pre)", timer.us(lambda: ops.dyt(h, w32, out, delta=delta, post=w32)), nbytes)
        wb = rand(width)
        bw(f"norm+sum t={t}: rmsnorm (sum, norm)", timer.us(lambda: ops.rmsnorm(h, wb, 1e-5, out=out, delta=delta)), nbytes)
    t = PREFILL_TOKENS
    x = rand(t, ffn * 3 // 2)
    bw(f"activation t={t}: gelu in place [t, 1.5 f]", timer.us(lambda: ops.bias_act(x, "gelu_erf")), t * (ffn * 3 // 2) * 4)
    x13, g = rand(t, 2 * ffn), torch.empty(t, ffn, dtype=torch.bfloat16, device=device)
    bw(f"activation t={t}: silu gate [t, 2 f] -> [t, f]", timer.us(lambda: ops.silu_gate(x13, g, 8)), t * ffn * 6)
    logits = rand(DECODE_BATCH, vocab, dtype=torch.float32)
    bw("logits scale and cap, 8 rows", timer.us(lambda: ops.scale_softcap(logits, 1.0, 30.0)), DECODE_BATCH * vocab * 8)

    geometry = (heads, kv, head_dim)
    small = (width, 3, heads, kv, head_dim, ffn, 1024)  # the attention launches do not depend on depth or vocabulary
    sx = sinorax_config(*small, window)
    table["attention softmax (sinorax 'attention', causal)"] = _attention_times(sx, device, timer, 0, None, *geometry)
    table["attention softmax (llama, causal)"] = _attention_times(llama_config(*small), device, timer, 0, None, *geometry)
    table[f"attention sigmoid (sinorax 'attention_2', window {window})"] = _attention_times(sx, device, timer, 2, window, *geometry)
    table[f"attention softmax (llama, window {window})"] = _attention_times(llama_config(*small, window=window), device, timer, 0,
                                                                          window, *geometry)
    for name, row in table.items():
        if "prefill_tflops" in row:
            row["prefill_tensor_frac"] = round(row["prefill_tflops"] * 1e12 / tensor, 3)
            row["decode_hbm_frac"] = round(row["decode_gbs"] * 1e9 / hbm, 3)
    return table


def _mixer_times(cfg, device, timer: Timer, layer: int, pick=None) -> Dict[str, float]:
    """A whole mixer of one layer alone (its projections included): a 2,048-token prompt, and 8
    single tokens at position 2,048."""
    from ..engine import StepEntry

    engine = _engine(cfg, device, DECODE_BATCH, DECODE_CONTEXT)
    _fill(engine)
    mixer = engine.model.blocks[layer].mixer
    if pick is not None:
        mixer = pick(engine.model.blocks[layer])
    memory = engine.memories[layer]
    width = engine.model.args.dim
    gen = torch.Generator().manual_seed(SEED)
    out = {}

    def context(entries):
        reqs = engine._validate(entries)
        for e, r in zip(entries, reqs):
            engine.cache.reserve(r, r.length + len(e.tokens))
        engine.cache.flush_tables()
        return engine.build_context(entries, reqs)

    engine.admit("p")
    ctx = context([StepEntry("p", [1] * PREFILL_TOKENS, [])])
    x = torch.randn(PREFILL_TOKENS, width, generator=gen).to(device, torch.bfloat16)
    run = (lambda x, ctx: mixer.forward(x, ctx, memory)) if hasattr(mixer, "cache_spec") else (lambda x, ctx: mixer.forward(x, ctx))
    out["prefill_us"] = round(timer.us(lambda: run(x, ctx)), 1)
    engine.release("p")
    ids = [f"d{i}" for i in range(DECODE_BATCH)]
    for rid in ids:
        r = engine.admit(rid)
        engine.cache.reserve(r, DECODE_CONTEXT - 1)
        engine.cache.advance(r, DECODE_CONTEXT - 1)
    ctx = context([StepEntry(rid, [1], []) for rid in ids])
    x = torch.randn(DECODE_BATCH, width, generator=gen).to(device, torch.bfloat16)
    out["decode_us"] = round(timer.us(lambda: run(x, ctx)), 1)
    engine.ops.check_status()
    del engine
    torch.cuda.empty_cache()
    return out


def _latent_attention_times(cfg, device, timer: Timer, layer: int) -> Dict[str, float]:
    """The attention launches of a latent-attention layer alone (folded queries in, summed latents
    out): a 2,048-token prompt, and 8 single tokens at position 2,048."""
    from ..engine import StepEntry

    engine = _engine(cfg, device, DECODE_BATCH, DECODE_CONTEXT)
    _fill(engine)
    mixer = engine.model.blocks[layer].mixer
    memory = engine.memories[layer]
    p = mixer.params
    H, R, r, d = p.n_heads, p.kv_rank, p.rot_dim, p.head_dim
    gen = torch.Generator().manual_seed(SEED)
    out = {}

    def context(entries):
        reqs = engine._validate(entries)
        for e, rq in zip(entries, reqs):
            engine.cache.reserve(rq, rq.length + len(e.tokens))
        engine.cache.flush_tables()
        return engine.build_context(entries, reqs)

    def run(t, ctx):
        qa = torch.randn(H, t, R, generator=gen).to(device, torch.bfloat16)
        q = torch.randn(t, H, d + r, generator=gen).to(device, torch.bfloat16)
        gate = torch.randn(t, H, generator=gen).to(device, torch.bfloat16)
        o = torch.empty_like(qa)
        return timer.us(lambda: engine.ops.latent_attention(qa, q[:, :, d:], o, gate, memory, ctx, H, R, r, p.softmax_scale))

    engine.admit("p")
    us = run(PREFILL_TOKENS, context([StepEntry("p", [1] * PREFILL_TOKENS, [])]))
    keys = PREFILL_TOKENS * (PREFILL_TOKENS + 1) // 2
    out["prefill_us"] = round(us, 1)
    out["prefill_tflops"] = round(2 * H * keys * (2 * R + r) / (us * 1e-6) / 1e12, 1)
    engine.release("p")
    ids = [f"d{i}" for i in range(DECODE_BATCH)]
    for rid in ids:
        rq = engine.admit(rid)
        engine.cache.reserve(rq, DECODE_CONTEXT - 1)
        engine.cache.advance(rq, DECODE_CONTEXT - 1)
    us = run(DECODE_BATCH, context([StepEntry(rid, [1], []) for rid in ids]))
    out["decode_us"] = round(us, 1)
    out["decode_gbs"] = round(DECODE_BATCH * DECODE_CONTEXT * mixer.entry * 2 / (us * 1e-6) / 1e9, 1)
    engine.ops.check_status()
    del engine
    torch.cuda.empty_cache()
    return out


def zeladra_kernel_table(size, device, peaks) -> Dict[str, dict]:
    """The kernels of the Zeladra design alone at one size, each beside the like kernel of the
    Llama shape where there is one: microseconds and the fraction of the roofline."""
    from ..cache import LayerMemory
    from ..csrc.ops import Ops
    from ..engine.step import StepContext
    from ..parts.base import StreamUpdate

    width, _layers, heads, kv, head_dim, ffn, vocab, window = size
    ops = Ops(torch.bfloat16, device)
    timer = Timer(device)
    gen = torch.Generator().manual_seed(SEED)
    hbm, tensor = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12
    table: Dict[str, dict] = {}

    def bw(name, us, nbytes):
        table[name] = dict(us=round(us, 1), gbs=round(nbytes / (us * 1e-6) / 1e9, 1), hbm_frac=round(nbytes / (us * 1e-6) / hbm, 3))

    def rand(*shape, dtype=torch.bfloat16):
        return torch.randn(*shape, generator=gen).to(device, dtype)

    streams = 2
    for t in (PREFILL_TOKENS, DECODE_BATCH):
        h, delta = rand(t, streams, width, dtype=torch.float32), rand(t, width)
        out = torch.empty(t, width, dtype=torch.bfloat16, device=device)
        w, b = rand(width, dtype=torch.float32), rand(width, dtype=torch.float32)
        mix, oc, ic = (rand(*sh, dtype=torch.float32) for sh in ((streams, streams), (streams,), (streams,)))
        up = StreamUpdate(delta, mix, oc)
        bw(f"norm+sum t={t}: layer norm over {streams} streams (update, sum, norm)",
           timer.us(lambda: ops.stream_norm(h, w, b, 1e-5, out, update=up, in_coef=ic)), t * width * (8 * streams + 2 + 2))
        h1, wb = rand(t, width, dtype=torch.float32), rand(width)
        bw(f"norm+sum t={t}: rmsnorm (sum, norm)", timer.us(lambda: ops.rmsnorm(h1, wb, 1e-5, out=out, delta=delta)),
           t * width * (4 + 4 + 2 + 2))

    # the state-space mixer's own kernels at this size
    ssm = zeladra_config(*size)["layers"][1]["mixer"]
    H, P, N, G, taps = ssm["heads"], ssm["vdim"], ssm["state"], ssm["groups"], ssm["conv"]
    inner, channels = H * P, H * P + 2 * G * N
    cols = 2 * inner + 2 * G * N + H
    state = torch.zeros(DECODE_BATCH, H * N * P + (taps - 1) * channels, dtype=torch.float32, device=device)
    conv_w, conv_b = rand(channels, taps, dtype=torch.float32), rand(channels, dtype=torch.float32)
    vec = [rand(H, dtype=torch.float32) for _ in range(3)]
    norm_w = rand(inner, dtype=torch.float32)
    for t, n_seqs in ((PREFILL_TOKENS, 1), (DECODE_BATCH, DECODE_BATCH)):
        proj = rand(t, cols)
        ctx = StepContext(device)
        per = t // n_seqs
        ctx.req = torch.arange(n_seqs, dtype=torch.int32, device=device).repeat_interleave(per)
        ctx.seq_slot = torch.arange(n_seqs, dtype=torch.int32, device=device)
        ctx.seq_start = torch.arange(0, t + 1, per, dtype=torch.int32, device=device)
        ctx.n_tokens, ctx.n_seqs = t, n_seqs
        xbc = ops.mamba2_conv(proj, inner, channels, conv_w, conv_b, state, H * N * P, taps, ctx)
        bw(f"state-space t={t}: convolution + SiLU", timer.us(lambda: ops.mamba2_conv(
            proj, inner, channels, conv_w, conv_b, state, H * N * P, taps, ctx)), t * channels * (2 + 4))
        y = ops.mamba2_scan(xbc, proj, inner + channels, *vec, state, ctx, H, G, N, P)
        state_bytes = n_seqs * H * N * P * 8
        bw(f"state-space t={t}: recurrence ({n_seqs} sequences)", timer.us(lambda: ops.mamba2_scan(
            xbc, proj, inner + channels, *vec, state, ctx, H, G, N, P)), t * (channels + inner) * 4 + state_bytes)
        bw(f"state-space t={t}: gate + norm in parts", timer.us(lambda: ops.gated_part_norm(
            y, proj[:, :inner], norm_w, ssm["norm_groups"], 1e-5, ctx)), t * inner * (4 + 2 + 2))
        state.zero_()

    geometry = (heads, kv, head_dim)
    small = (width, 3, heads, kv, head_dim, ffn, 1024)
    z = zeladra_config(*small, window)
    lat = z["layers"][0]["mixer"]
    table[f"attention softmax (zeladra 'attention', window {window}, keeps 4)"] = _attention_times(z, device, timer, 2, window, *geometry)
    table[f"attention softmax (llama, window {window})"] = _attention_times(llama_config(*small, window=window), device, timer, 0,
                                                                          window, *geometry)
    table["attention over the cached latent (zeladra 'latent_attention', causal)"] = _latent_attention_times(z, device, timer, 0)
    table["attention softmax (llama, causal)"] = _attention_times(llama_config(*small), device, timer, 0, None, *geometry)
    for name, row in table.items():
        if "prefill_tflops" in row:
            row["prefill_tensor_frac"] = round(row["prefill_tflops"] * 1e12 / tensor, 3)
            row["decode_hbm_frac"] = round(row["decode_gbs"] * 1e9 / hbm, 3)
    # whole mixers (projections included)
    row = _mixer_times(z, device, timer, 0)
    keys = PREFILL_TOKENS * (PREFILL_TOKENS + 1) // 2
    entry = lat["kv_rank"] + lat["rot_dim"]
    row["attention_flops_prefill"] = 2 * heads * keys * (entry + lat["kv_rank"])
    row["cache_bytes_decode"] = DECODE_BATCH * DECODE_CONTEXT * entry * 2
    table["mixer latent attention (zeladra, causal; whole mixer)"] = row
    table["mixer state-space (zeladra; whole mixer)"] = _mixer_times(z, device, timer, 1)
    table["mixer attention (zeladra, window; whole mixer)"] = _mixer_times(z, device, timer, 2)
    table["mixer attention (llama, causal; whole mixer)"] = _mixer_times(llama_config(*small), device, timer, 0)
    return table


def tanupel_kernel_table(size, device, peaks) -> Dict[str, dict]:
    """The kernels of the Tanupel design alone at one size, each beside the like kernel of the
    closest model where there is one (the Llama shape for norms, attention and the feed-forward;
    Zeladra's state-space mixer for the recurrence): microseconds and the fraction of the roofline."""
    from ..csrc.ops import Ops
    from ..engine.step import StepContext

    width, _layers, heads, kv, head_dim, ffn, vocab, window = size
    ops = Ops(torch.bfloat16, device)
    timer = Timer(device)
    gen = torch.Generator().manual_seed(SEED)
    hbm, tensor = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12
    table: Dict[str, dict] = {}

    def bw(name, us, nbytes):
        table[name] = dict(us=round(us, 1), gbs=round(nbytes / (us * 1e-6) / 1e9, 1), hbm_frac=round(nbytes / (us * 1e-6) / hbm, 3))

    def rand(*shape, dtype=torch.bfloat16):
        return torch.randn(*shape, generator=gen).to(device, dtype)

    def context(t, n_seqs):
        ctx = StepContext(device)
        per = t // n_seqs
        ctx.req = torch.arange(n_seqs, dtype=torch.int32, device=device).repeat_interleave(per)
        ctx.seq_slot = torch.arange(n_seqs, dtype=torch.int32, device=device)
        ctx.seq_start = torch.arange(0, t + 1, per, dtype=torch.int32, device=device)
        ctx.n_tokens, ctx.n_seqs = t, n_seqs
        return ctx

    few = lambda t: t == DECODE_BATCH  # few tokens: time the captured launches (device time, not the host's)
    cfg = tanupel_config(*size)
    right = cfg["layers"][0]["mixer"]["right"]
    att = cfg["layers"][1]["mixer"]
    for t in (PREFILL_TOKENS, DECODE_BATCH):
        h = rand(t, width, dtype=torch.float32)
        out = torch.empty(t, width, dtype=torch.bfloat16, device=device)
        terms = [(rand(t, width), c) for c in (0.25, 0.5, 0.5)]
        w32, row = rand(width, dtype=torch.float32), rand(width, dtype=torch.float32)
        bw(f"norm+sum t={t}: one-plus rmsnorm of a sum (3 summands with factors, a row vector, sum, norm)",
           timer.us(lambda: ops.rmsnorm_sum(h, terms, w32, 1e-5, out=out, row=row, one_plus=True), graph=few(t)), t * width * (4 + 4 + 3 * 2 + 2))
        delta, wb = rand(t, width), rand(width)
        bw(f"norm+sum t={t}: rmsnorm (sum, norm; llama)", timer.us(lambda: ops.rmsnorm(h, wb, 1e-5, out=out, delta=delta), graph=few(t)),
           t * width * (4 + 4 + 2 + 2))
        q, k = rand(t, att["heads"] * head_dim), rand(t, att["kv_heads"] * head_dim)
        req = torch.zeros(t, dtype=torch.int32, device=device)
        bw(f"query/key norm t={t}: mean squares over the whole projections",
           timer.us(lambda: ops.qk_rstd(q, k, q.shape[1], k.shape[1], 1e-5, req), graph=few(t)), t * (q.shape[1] + k.shape[1]) * 2)

    # the gated delta rule's own kernels, beside the state-space mixer's of Zeladra at this size
    H, G, d, dv, taps = right["heads"], right["kv_heads"], right["dim"], right["vdim"], right["conv"]
    channels = 2 * G * d + H * dv
    state = torch.zeros(DECODE_BATCH, H * dv * d + (taps - 1) * channels, dtype=torch.float32, device=device)
    conv_w = rand(channels, taps, dtype=torch.float32)
    dt_bias, a_log, norm_w = rand(H * d, dtype=torch.float32), rand(H, dtype=torch.float32), rand(dv, dtype=torch.float32)
    for t, n_seqs in ((PREFILL_TOKENS, 1), (DECODE_BATCH, DECODE_BATCH)):
        proj, a, b, z = rand(t, channels), rand(t, H * d), rand(t, H), rand(t, H * dv)
        ctx = context(t, n_seqs)
        bw(f"delta rule t={t}: convolution + SiLU", timer.us(lambda: ops.conv_silu(
            proj, 0, channels, conv_w, state, H * dv * d, taps, ctx), graph=few(t)), t * channels * (2 + 4))
        qkv = ops.conv_silu(proj, 0, channels, conv_w, state, H * dv * d, taps, ctx)
        state_bytes = n_seqs * H * dv * d * 8
        bw(f"delta rule t={t}: recurrence ({n_seqs} sequences, {H} heads, state {d} x {dv})", timer.us(lambda: ops.delta_scan(
            qkv, a, b, dt_bias, a_log, state, ctx, H, G, d, dv), graph=few(t)), t * (channels * 4 + H * d * 2 + H * dv * 4) + state_bytes)
        y = ops.delta_scan(qkv, a, b, dt_bias, a_log, state, ctx, H, G, d, dv)
        bw(f"delta rule t={t}: norm per head + gate", timer.us(lambda: ops.head_norm_gate(y, z, norm_w, H, dv, 1e-5, ctx), graph=few(t)),
           t * H * dv * (4 + 2 + 2))
        state.zero_()
    ssm = zeladra_config(*size)["layers"][1]["mixer"]
    sH, P, N, sG, staps = ssm["heads"] // 2, ssm["vdim"], ssm["state"], ssm["groups"], ssm["conv"]  # half the heads: a state of like size
    inner, sch = sH * P, sH * P + 2 * sG * N
    cols = 2 * inner + 2 * sG * N + sH
    sstate = torch.zeros(DECODE_BATCH, sH * N * P + (staps - 1) * sch, dtype=torch.float32, device=device)
    sconv_w, sconv_b = rand(sch, staps, dtype=torch.float32), rand(sch, dtype=torch.float32)
    vec = [rand(sH, dtype=torch.float32) for _ in range(3)]
    for t, n_seqs in ((PREFILL_TOKENS, 1), (DECODE_BATCH, DECODE_BATCH)):
        proj = rand(t, cols)
        ctx = context(t, n_seqs)
        xbc = ops.mamba2_conv(proj, inner, sch, sconv_w, sconv_b, sstate, sH * N * P, staps, ctx)
        bw(f"state-space (zeladra) t={t}: recurrence ({n_seqs} sequences, {sH} heads, state {N} x {P})", timer.us(lambda: ops.mamba2_scan(
            xbc, proj, inner + sch, *vec, sstate, ctx, sH, sG, N, P), graph=few(t)), t * (sch + inner) * 4 + n_seqs * sH * N * P * 8)
        sstate.zero_()

    # routed experts beside a dense gated feed-forward of as many parameters
    mlp = cfg["layers"][2]["mlp"]
    E, top, f = mlp["router"]["experts"], mlp["router"]["top"], mlp["expert"]["ff"]
    w13, w2 = rand(E, 2 * f, width), rand(E, width, f)
    w1, w3 = w13[:, :f], w13[:, f:]
    router, corr = rand(E, width, dtype=torch.float32), 0.01 * rand(E, dtype=torch.float32)
    wd13, wd = rand(2 * ffn, width), rand(width, ffn)
    for t in (PREFILL_TOKENS, DECODE_BATCH):
        x = rand(t, width)
        ctx = context(t, 1)
        logits = ops.moe_logits(x, router)
        ids, weights = ops.moe_route(logits, corr, top, ctx)
        row = dict(router_logits_us=round(timer.us(lambda: ops.moe_logits(x, router), graph=few(t)), 1),
                   choice_us=round(timer.us(lambda: ops.moe_route(logits, corr, top, ctx), graph=few(t)), 1))
        us = timer.us(lambda: ops.moe_experts(x, ids, weights, w1, w3, w2, w13), graph=few(t))
        row["experts_us"] = round(us, 1)
        row["experts_tflops"] = round(6 * t * top * f * width / (us * 1e-6) / 1e12, 1)
        row["experts_tensor_frac"] = round(6 * t * top * f * width / (us * 1e-6) / tensor, 3)
        touched = min(E, t * top)
        row["experts_weight_gbs"] = round(touched * 3 * f * width * 2 / (us * 1e-6) / 1e9, 1)
        row["experts_hbm_frac"] = round(touched * 3 * f * width * 2 / (us * 1e-6) / hbm, 3)
        table[f"routed experts t={t}: {top} of {E} experts of {f} rows"] = row

        def dense():
            g = ops.linear_swiglu(x, wd13)
            if g is None:
                g = torch.empty(t, ffn, dtype=torch.bfloat16, device=device)
                ops.silu_gate(ops.linear(x, wd13), g)
            return ops.linear(g, wd)
        us = timer.us(dense, graph=few(t))
        table[f"dense gated feed-forward t={t}: {ffn} rows (llama)"] = dict(
            us=round(us, 1), tflops=round(6 * t * ffn * width / (us * 1e-6) / 1e12, 1),
            tensor_frac=round(6 * t * ffn * width / (us * 1e-6) / tensor, 3),
            weight_gbs=round(3 * ffn * width * 2 / (us * 1e-6) / 1e9, 1), hbm_frac=round(3 * ffn * width * 2 / (us * 1e-6) / hbm, 3))

    small = (width, 2, heads, kv, head_dim, ffn, 1024)
    tz = tanupel_config(*small)
    left = tz["layers"][0]["mixer"]["left"]
    table["attention softmax, capped scores (tanupel pair's left half, causal)"] = _attention_times(
        tz, device, timer, 0, None, left["heads"], left["kv_heads"], head_dim, pick=lambda m: m.left)
    table["attention softmax (tanupel 'attention', causal)"] = _attention_times(tz, device, timer, 1, None, heads, kv, head_dim)
    table["attention softmax (llama, causal)"] = _attention_times(llama_config(*small), device, timer, 0, None, heads, kv, head_dim)
    for name, row in table.items():
        if "prefill_tflops" in row:
            row["prefill_tensor_frac"] = round(row["prefill_tflops"] * 1e12 / tensor, 3)
            row["decode_hbm_frac"] = round(row["decode_gbs"] * 1e9 / hbm, 3)
    # whole mixers (projections included) and whole feed-forwards
    table["mixer pair (tanupel: capped attention beside the delta rule; whole mixer)"] = _mixer_times(tz, device, timer, 0)
    table["mixer pair's right half alone (tanupel delta rule; whole mixer)"] = _mixer_times(tz, device, timer, 0, pick=lambda b: b.mixer.right)
    table["mixer attention (tanupel, projection-wide query/key norm; whole mixer)"] = _mixer_times(tz, device, timer, 1)
    table["mixer attention (llama, causal; whole mixer)"] = _mixer_times(llama_config(*small), device, timer, 0)
    return table


def palulorn_kernel_table(size, device, peaks) -> Dict[str, dict]:
    """The kernels of the Palulorn design alone at one size, each beside the like kernel of the closest
    model where there is one (Tanupel's delta rule for the matrix memory, its routed experts, the Llama
    shape's attention and norm): microseconds and the fraction of the roofline."""
    from ..csrc.ops import Ops
    from ..engine.step import StepContext

    width, _layers, heads, kv, head_dim, ffn, vocab, window = size
    ops = Ops(torch.bfloat16, device)
    timer = Timer(device)
    gen = torch.Generator().manual_seed(SEED)
    hbm, tensor = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12
    table: Dict[str, dict] = {}

    def bw(name, us, nbytes):
        table[name] = dict(us=round(us, 1), gbs=round(nbytes / (us * 1e-6) / 1e9, 1), hbm_frac=round(nbytes / (us * 1e-6) / hbm, 3))

    def rand(*shape, dtype=torch.bfloat16):
        return torch.randn(*shape, generator=gen).to(device, dtype)

    def context(t, n_seqs):
        ctx = StepContext(device)
        per = t // n_seqs
        ctx.req = torch.arange(n_seqs, dtype=torch.int32, device=device).repeat_interleave(per)
        ctx.pos = torch.arange(t, dtype=torch.int32, device=device) % per + (DECODE_CONTEXT if n_seqs > 1 else 0)
        ctx.seq_slot = torch.arange(n_seqs, dtype=torch.int32, device=device)
        ctx.seq_start = torch.arange(0, t + 1, per, dtype=torch.int32, device=device)
        ctx.n_tokens, ctx.n_seqs = t, n_seqs
        return ctx

    few = lambda t: t == DECODE_BATCH  # few tokens: time the captured launches (device time, not the host's)
    cfg = palulorn_config(*size)
    left, right = cfg["layers"][0]["mixer"]["left"], cfg["layers"][0]["mixer"]["right"]
    att, lru = cfg["layers"][1]["mixer"], cfg["layers"][2]["mixer"]
    for t in (PREFILL_TOKENS, DECODE_BATCH):
        h = rand(t, width, dtype=torch.float32)
        out = torch.empty(t, width, dtype=torch.bfloat16, device=device)
        out32 = torch.empty(t, width, dtype=torch.float32, device=device)
        y, wb = rand(t, width), rand(width)
        bw(f"norm t={t}: rmsnorm of a half's output over the width (16-bit in, 32-bit out; twice a pair)",
           timer.us(lambda: ops.rmsnorm(y, wb, 1e-5, out=out32), graph=few(t)), t * width * (2 + 4))
        terms = [(rand(t, width, dtype=torch.float32), 0.5), (rand(t, width, dtype=torch.float32), 0.5)]
        bw(f"norm+sum t={t}: rmsnorm of a sum (the pair's two normed outputs with factors, sum, norm)",
           timer.us(lambda: ops.rmsnorm_sum(h, terms, wb, 1e-5, out=out), graph=few(t)), t * width * (4 + 4 + 2 * 4 + 2))
        delta = rand(t, width)
        bw(f"norm+sum t={t}: rmsnorm (sum, norm; llama)", timer.us(lambda: ops.rmsnorm(h, wb, 1e-5, out=out, delta=delta), graph=few(t)),
           t * width * (4 + 4 + 2 + 2))
        bw(f"pass input t={t}: sum and rounding of the stream before the map",
           timer.us(lambda: ops.rmsnorm_sum(h, [(delta, 1.0)], None, 0.0, out=out), graph=few(t)), t * width * (4 + 4 + 2 + 2))
        ctx = context(t, 1 if t > DECODE_BATCH else DECODE_BATCH)
        q, k = rand(t, att["heads"] * head_dim), rand(t, att["kv_heads"] * head_dim)
        bw(f"query/key norm t={t}: a factor per (token, head)",
           timer.us(lambda: ops.qk_head_factors(q, k, ctx.pos, ctx.req, att["heads"], att["kv_heads"], head_dim, head_dim, 1e-5),
                    graph=few(t)), t * (q.shape[1] + k.shape[1]) * 2)
        o, gate = rand(t, left["heads"] * head_dim), rand(t, left["heads"])
        bw(f"head gate t={t}: a head's output times its sigmoid gate, in place",
           timer.us(lambda: ops.head_gate(o, gate, ctx.req, left["heads"], head_dim), graph=few(t)), t * o.shape[1] * 4)

    # the matrix memory's kernels, beside the delta rule's of Tanupel at the same heads and state
    H, d, dv = right["heads"], right["dim"], right["vdim"]
    floats = ops.mlstm_state_floats(H, d, dv)
    bias, norm_w = rand(2 * H, dtype=torch.float32), rand(H * dv, dtype=torch.float32)
    dr = tanupel_config(*size)["layers"][0]["mixer"]["right"]
    G, taps = dr["kv_heads"], dr["conv"]
    dch = 2 * G * d + H * dv
    dstate = torch.zeros(DECODE_BATCH, H * dv * d + (taps - 1) * dch, dtype=torch.float32, device=device)
    dt_bias, a_log = rand(H * d, dtype=torch.float32), rand(H, dtype=torch.float32)
    for t, n_seqs in ((PREFILL_TOKENS, 1), (DECODE_BATCH, DECODE_BATCH)):
        ctx = context(t, n_seqs)
        state = torch.zeros(DECODE_BATCH, floats, dtype=torch.float32, device=device)
        q, k, v, z = rand(t, H * d), rand(t, H * d), rand(t, H * dv), rand(t, H * dv)
        gates = rand(t, 2 * H, dtype=torch.float32)
        run = lambda: ops.mlstm_scan(gates.clone(), bias, 15.0, q, k, v, state, ctx, H, d, dv, d ** -0.5)
        nbytes = t * (2 * H * d + H * dv) * 2 + t * H * (dv + 1) * 4 + n_seqs * floats * 8
        bw(f"matrix memory t={t}: gates, maxima, recurrence ({n_seqs} sequences, {H} heads, state {d} x {dv} + normaliser)",
           timer.us(run, graph=few(t)), nbytes)
        y, coef = run()
        bw(f"matrix memory t={t}: division, norm per head, gate", timer.us(lambda: ops.mlstm_out(y, coef, z, norm_w, H, dv, 1e-5, ctx),
                                                                        graph=few(t)), t * H * dv * (4 + 2 + 2))
        qkv, a, b = rand(t, dch, dtype=torch.float32), rand(t, H * d), rand(t, H)
        bw(f"delta rule (tanupel) t={t}: recurrence ({n_seqs} sequences, {H} heads, state {d} x {dv})", timer.us(lambda: ops.delta_scan(
            qkv, a, b, dt_bias, a_log, dstate, ctx, H, G, d, dv), graph=few(t)), t * (dch * 4 + H * d * 2 + H * dv * 4) + n_seqs * H * dv * d * 8)
        dstate.zero_()

    # the gated linear recurrent unit
    W, blocks, ltaps = lru["width"], lru["blocks"], lru["conv"]
    bwid = W // blocks
    br, bi, rate = rand(W, dtype=torch.float32), rand(W, dtype=torch.float32), -rand(W, dtype=torch.float32).abs()
    conv_w, conv_b = rand(W, ltaps, dtype=torch.float32), rand(W, dtype=torch.float32)
    w_gates_t = rand(blocks, bwid, 2 * bwid)
    for t, n_seqs in ((PREFILL_TOKENS, 1), (DECODE_BATCH, DECODE_BATCH)):
        ctx = context(t, n_seqs)
        state = torch.zeros(DECODE_BATCH, W + (ltaps - 1) * W, dtype=torch.float32, device=device)
        xb, yb = rand(t, W), rand(t, W)
        bw(f"recurrent unit t={t}: convolution with bias", timer.us(lambda: ops.time_conv(
            xb, 0, W, conv_w, conv_b, state, W, ltaps, ctx, out_dtype=torch.bfloat16), graph=few(t)), t * W * (2 + 2))
        u = ops.time_conv(xb, 0, W, conv_w, conv_b, state, W, ltaps, ctx, out_dtype=torch.bfloat16)
        us = timer.us(lambda: ops.block_products(u.view(t, blocks, bwid), w_gates_t, None), graph=few(t))
        table[f"recurrent unit t={t}: block-diagonal gate maps ({blocks} blocks of {bwid}; the library's batched product)"] = dict(
            us=round(us, 1), tflops=round(4 * t * W * bwid / (us * 1e-6) / 1e12, 1))
        gates = ops.block_products(u.view(t, blocks, bwid), w_gates_t, None)
        bw(f"recurrent unit t={t}: coefficients and chain ({n_seqs} sequences, {W} channels)", timer.us(lambda: ops.rglru_scan(
            gates, u, br, bi, rate, yb, state, 0, ctx, blocks), graph=few(t)), t * W * (8 + 2 + 8 + 8 + 2 + 2))

    # routed experts without a gate beside Tanupel's gated ones of as many parameters
    mlp = cfg["layers"][0]["mlp"]
    E, top, f = mlp["router"]["experts"], mlp["router"]["top"], mlp["expert"]["ff"]
    groups = (mlp["router"]["groups"]["count"], mlp["router"]["groups"]["keep"], 2)
    w_up, w_down = rand(E, f, width), rand(E, width, f)
    tf = ffn // E
    w13, w2 = rand(E, 2 * tf, width), rand(E, width, tf)
    router = rand(E, width, dtype=torch.float32)
    for t in (PREFILL_TOKENS, DECODE_BATCH):
        x = rand(t, width)
        ctx = context(t, 1)
        logits = ops.moe_logits(x, router)
        route = lambda: ops.moe_route(logits, None, top, ctx, renormalize=True, score="sigmoid", groups=groups, renorm_eps=1e-20,
                                      weight_scale=2.0)
        ids, weights = route()
        row = dict(router_logits_us=round(timer.us(lambda: ops.moe_logits(x, router), graph=few(t)), 1),
                   choice_us=round(timer.us(route, graph=few(t)), 1))
        us = timer.us(lambda: ops.moe_experts(x, ids, weights, w_up, None, w_down, w_up, act="relu2"), graph=few(t))
        flops = 4 * t * top * f * width
        touched = min(E, t * top)
        row.update(experts_us=round(us, 1), experts_tflops=round(flops / (us * 1e-6) / 1e12, 1),
                   experts_tensor_frac=round(flops / (us * 1e-6) / tensor, 3),
                   experts_hbm_frac=round(touched * 2 * f * width * 2 / (us * 1e-6) / hbm, 3))
        table[f"routed experts t={t}: {top} of {E} ungated experts of {f} rows, squared ReLU"] = row
        ids2, weights2 = ops.moe_route(logits, None, top, ctx)
        us = timer.us(lambda: ops.moe_experts(x, ids2, weights2, w13[:, :tf], w13[:, tf:], w2, w13), graph=few(t))
        flops = 6 * t * top * tf * width
        table[f"routed experts (tanupel) t={t}: {top} of {E} gated experts of {tf} rows"] = dict(
            choice_us=round(timer.us(lambda: ops.moe_route(logits, None, top, ctx), graph=few(t)), 1),
            experts_us=round(us, 1), experts_tflops=round(flops / (us * 1e-6) / 1e12, 1),
            experts_tensor_frac=round(flops / (us * 1e-6) / tensor, 3),
            experts_hbm_frac=round(touched * 3 * tf * width * 2 / (us * 1e-6) / hbm, 3))

    small = (width, 3, heads, kv, head_dim, ffn, 1024)
    pz = palulorn_config(*small, window)
    table["attention softmax with a sink, values = keys (palulorn pair's left half, causal)"] = _attention_times(
        pz, device, timer, 0, None, left["heads"], left["kv_heads"], head_dim, pick=lambda m: m.left)
    table[f"attention softmax (palulorn 'attention', window {window})"] = _attention_times(pz, device, timer, 1, window, heads, kv, head_dim)
    table["attention softmax (llama, causal)"] = _attention_times(llama_config(*small), device, timer, 0, None, heads, kv, head_dim)
    table[f"attention softmax (llama, window {window})"] = _attention_times(llama_config(*small, window=window), device, timer, 0,
                                                                          window, heads, kv, head_dim)
    for name, row in table.items():
        if "prefill_tflops" in row:
            row["prefill_tensor_frac"] = round(row["prefill_tflops"] * 1e12 / tensor, 3)
            row["decode_hbm_frac"] = round(row["decode_gbs"] * 1e9 / hbm, 3)
    # whole mixers (projections included)
    table["mixer pair (palulorn: attention with a sink beside the matrix memory, both normed; whole mixer)"] = _mixer_times(pz, device, timer, 0)
    table["mixer pair's left half alone (palulorn; whole mixer)"] = _mixer_times(pz, device, timer, 0, pick=lambda b: b.mixer.left)
    table["mixer pair's right half alone (palulorn matrix memory; whole mixer)"] = _mixer_times(pz, device, timer, 0, pick=lambda b: b.mixer.right)
    table["mixer attention (palulorn: convolution, norm per head, window; whole mixer)"] = _mixer_times(pz, device, timer, 1)
    table["mixer recurrent unit (palulorn; whole mixer)"] = _mixer_times(pz, device, timer, 2)
    table["feed-forward (palulorn: routed and shared experts; whole)"] = _mixer_times(pz, device, timer, 0, pick=lambda b: b.ffn)
    tz = tanupel_config(width, 2, heads, kv, head_dim, ffn, 1024)
    table["mixer pair (tanupel: capped attention beside the delta rule; whole mixer)"] = _mixer_times(tz, device, timer, 0)
    table["mixer attention (llama, causal; whole mixer)"] = _mixer_times(llama_config(*small), device, timer, 0)
    return table


def run(sizes: List[str], peaks: dict, kernels: bool = True, design: str = "sinorax") -> dict:
    device = torch.device("cuda:0")
    torch.cuda.set_device(device)
    if design == "palulorn":
        out = {"metric": "prefill and decode tokens/s of Palulorn beside Tanupel and a Llama-shaped model of equal size (bf16, random weights)",
               "unit": "tokens/s", "dtype": "bf16", "data": "synthetic (random weights, uniform random token ids)",
               "config": dict(prefill_tokens=PREFILL_TOKENS, decode_batch=DECODE_BATCH, decode_context=DECODE_CONTEXT, page=PAGE,
                              l2="flushed before every timed kernel; model steps stream all weights"),
               "peaks": peaks, "sizes": {}}
        for name in sizes:
            size = SIZES[name]
            entry = dict(width=size[0], layers=size[1], heads=size[2], kv_heads=size[3], head_dim=size[4], swiglu_ffn=size[5],
                         vocab=size[6], window=size[7], experts=8, top=2, expert_ffn=size[5] * 3 // 2 // 8)
            entry["palulorn"] = model_throughput(palulorn_config(*size), device)
            entry["tanupel"] = model_throughput(tanupel_config(*size), device)
            entry["llama"] = model_throughput(llama_config(*size[:7]), device)
            if kernels:
                entry["kernels"] = palulorn_kernel_table(size, device, peaks)
            out["sizes"][name] = entry
        return out
    if design == "tanupel":
        out = {"metric": "prefill and decode tokens/s of Tanupel beside a Llama-shaped model of equal size (bf16, random weights)",
               "unit": "tokens/s", "dtype": "bf16", "data": "synthetic (random weights, uniform random token ids)",
               "config": dict(prefill_tokens=PREFILL_TOKENS, decode_batch=DECODE_BATCH, decode_context=DECODE_CONTEXT, page=PAGE,
                              l2="flushed before every timed kernel; model steps stream all weights"),
               "peaks": peaks, "sizes": {}}
        for name in sizes:
            size = SIZES[name]
            entry = dict(width=size[0], layers=size[1], heads=size[2], kv_heads=size[3], head_dim=size[4], swiglu_ffn=size[5],
                         vocab=size[6], experts=8, top=2, expert_ffn=size[5] // 8)
            entry["tanupel"] = model_throughput(tanupel_config(*size), device)
            entry["llama"] = model_throughput(llama_config(*size[:7]), device)
            if kernels:
                entry["kernels"] = tanupel_kernel_table(size, device, peaks)
            out["sizes"][name] = entry
        return out
    if design == "zeladra":
        out = {"metric": "prefill and decode tokens/s of Zeladra beside a Llama-shaped model of equal size (bf16, random weights)",
               "unit": "tokens/s", "dtype": "bf16", "data": "synthetic (random weights, uniform random token ids)",
               "config": dict(prefill_tokens=PREFILL_TOKENS, decode_batch=DECODE_BATCH, decode_context=DECODE_CONTEXT, page=PAGE,
                              l2="flushed before every timed kernel; model steps stream all weights"),
               "peaks": peaks, "sizes": {}}
        for name in sizes:
            size = SIZES[name]
            entry = dict(width=size[0], layers=size[1], heads=size[2], kv_heads=size[3], head_dim=size[4], swiglu_ffn=size[5],
                         vocab=size[6], window=size[7])
            entry["zeladra"] = model_throughput(zeladra_config(*size), device)
            entry["llama"] = model_throughput(llama_config(*size[:7]), device)
            if kernels:
                entry["kernels"] = zeladra_kernel_table(size, device, peaks)
            out["sizes"][name] = entry
        return out
    out = {"metric": "prefill and decode tokens/s of Sinorax beside a Llama-shaped model of equal size (bf16, random weights)",
           "unit": "tokens/s", "dtype": "bf16", "data": "synthetic (random weights, uniform random token ids)",
           "config": dict(prefill_tokens=PREFILL_TOKENS, decode_batch=DECODE_BATCH, decode_context=DECODE_CONTEXT, page=PAGE,
                          l2="flushed before every timed kernel; model steps stream all weights"),
           "peaks": peaks, "sizes": {}}
    for name in sizes:
        size = SIZES[name]
        entry = dict(width=size[0], layers=size[1], heads=size[2], kv_heads=size[3], head_dim=size[4], swiglu_ffn=size[5],
                     dense_ffn=size[5] * 3 // 2, vocab=size[6], window=size[7])
        entry["sinorax"] = model_throughput(sinorax_config(*size), device)
        entry["llama"] = model_throughput(llama_config(*size[:7]), device)
        if kernels:
            entry["kernels"] = kernel_table(size, device, peaks)
        out["sizes"][name] = entry
    return out


if __name__ == "__main__":
    print(json.dumps(run(list(SIZES), dict(hbm_gbs=6650.0, bf16_tflops=1590.0))))
