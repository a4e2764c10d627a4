"""Palulorn through the engine against the plain implementation of ``plain_palulorn.py``: each
mechanism alone, whole prompts against token-by-token decoding, portions down to two tokens, unequal
batches, pages and slots used again, keys far away, at page borders and at a window's edges, states
that carry what was long ago, the first tokens of a sequence, long decoding, sizes that pad or equal
one, and greedy generation through ``Fastgen.generate``."""

import copy
import queue
from pathlib import Path

import numpy as np
import pytest
import torch

import helpers as H
import plain_palulorn as pp
from fastgen_b200.config import ConfigError, model_args_from_config
from fastgen_b200.weights import write_random_model
from test_tanupel_gpu import _close, _context, _draw_all, _ops, _run_mixer, _tol, _value

DEV = "cuda:0"


def _sink(heads, kv, dim, scale, temp=None):
    m = dict(heads=heads, kv_heads=kv, dim=dim, vdim=dim, scale=scale)
    if temp:
        m["q_temp"] = dict(coef=temp[0], every=temp[1])
    return m


def _memory(heads, dim, vdim, cap):
    return dict(heads=heads, dim=dim, vdim=vdim, gate_cap=cap)


def _pair(left, right):
    return dict(left=left, right=right)


def _lru(width, blocks, conv):
    return dict(width=width, blocks=blocks, conv=conv)


def _attn(heads, kv, dim, vdim, scale, conv=None, rot=None, window=None):
    m = dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, scale=scale)
    if conv:
        m["conv"] = conv
    if rot:
        dims, base, factor = rot
        m["rot"] = dict(dims=dims, base=base)
        if factor:
            m["rot"]["scaling"] = dict(factor=factor)
    if window:
        m["mask"] = dict(size=window)
    return m


def _moe(experts, top, ff, groups=None, scale=1.0, shared=None):
    router = dict(experts=experts, top=top, scale=scale)
    if groups:
        router["groups"] = dict(count=groups[0], keep=groups[1])
    mlp = dict(kind="moe", expert=dict(ff=ff), router=router)
    if shared:
        mlp["shared"] = dict(ff=shared)
    return mlp


def _layer(kind, mixer, mlp):
    return dict(type=kind, mixer=mixer, mlp=mlp)


# a run of two layers passed twice, opened by a pair; value heads larger than key heads and padded; a
# window shorter than two pages; groups of experts; a layer without a feed-forward; a temperature that
# changes every seven positions
PA = dict(
    architecture="Palulorn", vocab=211, width=96, norm=dict(eps=1e-5), embedding=dict(scale=3.0),
    loop=dict(start=1, stop=3, times=2),
    layers=[
        _layer("attention", _attn(6, 3, 16, 32, 0.2, conv=2, rot=(8, 5000.0, 8.0), window=20), _moe(6, 3, 40, (3, 2), 2.0, 24)),
        _layer("parallel", _pair(_sink(4, 2, 32, 0.15, (0.5, 7)), _memory(3, 24, 40, 10.0)), _moe(5, 2, 24)),
        _layer("rglru", _lru(80, 5, 3), None),
        _layer("attention", _attn(2, 1, 48, 48, 0.12, conv=4, rot=(24, 300.0, None), window=9), _moe(8, 1, 16, (4, 1), 0.5, 8)),
    ],
)
# no repeated run, no embedding scale; one head, one block, one expert, one tap; an attention layer
# with no convolution, no rotation and no window; a head of 64 (the size of the tcgen05 kernel)
PB = dict(
    architecture="Palulorn", vocab=97, width=64, norm=dict(eps=1e-6),
    layers=[
        _layer("parallel", _pair(_sink(1, 1, 64, 0.1), _memory(1, 33, 5, 4.0)), _moe(1, 1, 56)),
        _layer("rglru", _lru(64, 1, 1), _moe(4, 4, 16, (2, 2), 1.0, 16)),
        _layer("attention", _attn(4, 1, 16, 8, 0.25), None),
        _layer("attention", _attn(2, 2, 64, 64, 0.12, conv=3, rot=(64, 1e4, 2.0), window=70), _moe(6, 2, 8, (2, 1))),
    ],
)
# the whole model is the repeated run (three passes from the first layer to the last); a state of 160
# rows a head; a window of one key
PC = dict(
    architecture="Palulorn", vocab=130, width=80, norm=dict(eps=1e-5), embedding=dict(scale=0.5),
    loop=dict(start=0, stop=3, times=3),
    layers=[
        _layer("parallel", _pair(_sink(5, 1, 16, 0.2, (0.3, 16)), _memory(2, 160, 12, 15.0)), _moe(3, 3, 32, None, 1.5, 8)),
        _layer("rglru", _lru(120, 3, 4), _moe(4, 2, 16, (2, 1), 1.0)),
        _layer("attention", _attn(2, 2, 80, 16, 0.11, conv=2, rot=(40, 2000.0, 4.0), window=1), None),
    ],
)
# a run of one layer passed once, in the middle
PD = dict(
    architecture="Palulorn", vocab=64, width=48, norm=dict(eps=1e-5),
    loop=dict(start=1, stop=2, times=1),
    layers=[
        _layer("rglru", _lru(48, 2, 2), _moe(4, 2, 16, (2, 2), 1.0, 8)),
        _layer("parallel", _pair(_sink(2, 1, 32, 0.2, (1.0, 1)), _memory(3, 16, 16, 8.0)), _moe(9, 4, 8, (3, 2), 2.5)),
        _layer("attention", _attn(3, 1, 16, 16, 0.25, conv=8, rot=(8, 100.0, None), window=33), _moe(2, 1, 24)),
    ],
)
# sizes that fit no kernel's favourite: a width that is no multiple of eight, heads in groups of three,
# head sizes that are padded, a memory of 200 rows, a window longer than any prompt here, a run of two
# layers in the middle passed four times, sixteen experts in eight groups
PE = dict(
    architecture="Palulorn", vocab=173, width=100, norm=dict(eps=1e-6), embedding=dict(scale=7.5),
    loop=dict(start=1, stop=3, times=4),
    layers=[
        _layer("attention", _attn(6, 2, 40, 24, 0.16, conv=1, rot=(20, 777.0, 2.5), window=500), _moe(16, 4, 12, (8, 3), 1.75, 20)),
        _layer("rglru", _lru(72, 3, 5), _moe(3, 2, 28)),
        _layer("parallel", _pair(_sink(6, 2, 80, 0.1, (0.7, 5)), _memory(1, 200, 36, 20.0)), None),
        _layer("parallel", _pair(_sink(3, 3, 16, 0.3), _memory(5, 8, 24, 3.0)), _moe(2, 2, 36, (1, 1), 0.8, 4)),
    ],
)
CONFIGS = {"pa": (PA, 3), "pb": (PB, 5), "pc": (PC, 8), "pd": (PD, 9), "pe": (PE, 12)}


def make_dir(tmp_path, name, std=0.1):
    cfg, seed = CONFIGS[name]
    return write_random_model(Path(tmp_path) / name, cfg, seed, dtype=torch.bfloat16, norm_jitter=0.3, std=std)


_plain = {}


def plain_logits(model_dir, tokens):
    key = (str(model_dir), tuple(tokens))
    if key not in _plain:
        cfg, w = pp.read_model(model_dir)
        _plain[key] = pp.forward(cfg, w, list(tokens)).numpy()
    return _plain[key]


# The bfloat16 rule of this design's models: a row of logits may differ from the plain one by T_L2 of
# the row's l2 norm and, in its worst entry, by T_MAX of the row's largest logit.  A memory's read-out is
# divided by its own size head by head, so a sequence's first tokens, whose read-out is a sum of one or
# two terms that may nearly cancel, carry their rounding at full size: of the rows of a comparison a
# share of T_SHARE may be up to T_FAR times as far.  float32 rows are held to ``helpers.check_row``'s 1e-4.
T_L2, T_MAX, T_SHARE, T_FAR = 0.05, 0.06, 0.08, 4.0


def row_distance(row, ref):
    """A bfloat16 row's distance from the plain one in units of the rule (1: at the rule's edge)."""
    l2 = float(np.linalg.norm(row - ref) / max(np.linalg.norm(ref), 1e-30))
    mx = float(np.abs(row - ref).max()) / max(float(np.abs(ref).max()), 1e-30)
    return max(l2 / T_L2, mx / T_MAX)


def check_rows(pairs, dtype):
    """``pairs``: (what, row, plain row).  float32: every row by itself; bfloat16: the share rule."""
    if dtype == torch.float32:
        # (1e-4 of a logit; the same share of rows may be farther: a pass amplifies what the passes before
        # left, and the plain implementation in float32 is as far from itself in float64 at such rows)
        dist = [(float(np.abs(row - ref).max()) / 1e-4, what) for what, row, ref in pairs]
    else:
        dist = [(row_distance(row, ref), what) for what, row, ref in pairs]
    worst = max(dist)
    assert worst[0] <= T_FAR, f"{worst[1]}: {worst[0]:.2f} times the rule's distance (at most {T_FAR})"
    over = [x for x in dist if x[0] > 1.0]
    assert len(over) <= max(1, T_SHARE * len(dist)), f"{len(over)} of {len(dist)} rows beyond the rule, e.g. {over[:3]}"


def compare(model_dir, requests, got, dtype):
    pairs = []
    for rid, toks in requests.items():
        ref = plain_logits(model_dir, toks)
        assert set(got[rid]) == set(range(len(toks))), f"{rid}: positions missing"
        pairs += [(f"{rid} pos {p}", row, ref[p]) for p, row in got[rid].items()]
    check_rows(pairs, dtype)


def _requests(vocab, lengths, seed):
    return {f"r{i}": H.random_tokens(vocab, n, seed + i) for i, n in enumerate(lengths)}


# ---------------------------------------------------------------------------------
# the description and the cache bookkeeping (no GPU)
# ---------------------------------------------------------------------------------
def test_description_reads_every_size_from_the_configuration():
    args = model_args_from_config(PA)
    assert (args.dim, args.vocab_size, args.streams, len(args.layers)) == (96, 211, None, 4)
    assert args.embedder.params.scale == 3.0 and model_args_from_config(PB).embedder.params.scale == 1.0
    att = args.layers[0].mixer.params
    assert (att.n_heads, att.n_kv_heads, att.head_dim, att.v_head_dim, att.softmax_scale) == (6, 3, 16, 32, 0.2)
    assert (att.qk_norm, att.qk_norm_eps, att.window, att.conv, att.bias, att.o_bias) == ("head", 1e-5, 20, 2, True, False)
    assert not (att.sink or att.head_gate or att.shared_kv) and att.q_temp is None and att.qk_layout == "half_split"
    rope = att.position.params
    assert (rope.rot_dims, rope.theta, rope.linear_factor, rope.scaling) == (8, 5000.0, 8.0, None)
    assert args.layers[3].mixer.params.position.params.linear_factor is None
    pair = args.layers[1].mixer.params
    left, right = pair.left.params, pair.right.params
    assert (pair.left_scale, pair.right_scale) == (0.5, 0.5)
    assert pair.left_norm.params.dim == pair.right_norm.params.dim == 96
    assert left.sink and left.head_gate and left.shared_kv and left.bias and left.o_bias and left.window is None
    assert left.q_temp == (0.5, 7) and left.position.kind == "none" and left.qk_norm is None
    assert (right.n_heads, right.head_dim, right.v_head_dim, right.gate_cap, right.eps) == (3, 24, 40, 10.0, 1e-5)
    lru = args.layers[2].mixer.params
    assert (lru.width, lru.blocks, lru.conv, lru.decay) == (80, 5, 3, 8.0)
    assert args.layers[2].ffn is None and args.layers[2].ffn_norm is None
    moe = args.layers[0].ffn.params
    assert (moe.n_experts, moe.top, moe.ffn_dim, moe.groups, moe.weight_scale) == (6, 3, 40, (3, 2), 2.0)
    assert (moe.score, moe.renormalize, moe.renorm_eps, moe.correction, moe.act, moe.group_top) == (
        "sigmoid", True, 1e-20, False, "relu2", 2)
    assert moe.shared.params.ffn_dim == 24 and moe.shared.params.act == "relu2"
    assert args.layers[1].ffn.params.groups is None and args.layers[1].ffn.params.shared is None
    assert all(l.block == "prenorm" and not l.mixer_norm.params.one_plus for l in args.layers)
    # the run of layers 1..2 twice: every run has a cache and a state of its own and opens by mixing
    # the embedding output in
    assert [(e.layer, e.step_row, e.mix_input, e.kv_from) for e in args.schedule] == [
        (0, None, False, None), (1, 0, True, None), (2, None, False, None), (1, 1, True, None), (2, None, False, None),
        (3, None, False, None)]
    assert [(e.layer, e.step_row) for e in model_args_from_config(PC).schedule] == [
        (0, 0), (1, None), (2, None), (0, 1), (1, None), (2, None), (0, 2), (1, None), (2, None)]
    assert [(e.layer, e.mix_input) for e in model_args_from_config(PD).schedule] == [(0, False), (1, True), (2, False)]
    assert model_args_from_config(PB).step_table_name is None and model_args_from_config(PB).pass_input_name is None
    assert args.pass_input_name == "loop.in" and args.step_table_name == "loop.step"


def test_description_errors_name_the_place():
    bad = copy.deepcopy(PA)
    bad["layers"][2]["type"] = "rglru_9"
    with pytest.raises(ConfigError, match="rglru_9"):
        model_args_from_config(bad)
    bad = copy.deepcopy(PA)
    del bad["layers"][1]["mixer"]["right"]["gate_cap"]
    with pytest.raises(ConfigError, match=r"layers\[1\]\.mixer\.right.*gate_cap"):
        model_args_from_config(bad)
    bad = copy.deepcopy(PA)
    bad["layers"][0]["mlp"]["router"]["groups"]["count"] = 4
    with pytest.raises(ConfigError, match=r"layers\[0\]"):
        model_args_from_config(bad)
    bad = copy.deepcopy(PA)
    bad["loop"]["stop"] = 5
    with pytest.raises(ConfigError, match="loop"):
        model_args_from_config(bad)
    bad = copy.deepcopy(PA)
    bad["layers"][1]["mixer"]["left"]["vdim"] = 16
    with pytest.raises(ConfigError, match=r"layers\[1\]\.mixer\.left"):
        model_args_from_config(bad)
    bad = copy.deepcopy(PA)
    bad["layers"][2]["mixer"]["blocks"] = 7
    with pytest.raises(ConfigError, match=r"layers\[2\]"):
        model_args_from_config(bad)


def test_random_folder_holds_exactly_the_tensors_of_the_description(tmp_path):
    from safetensors.torch import load_file

    tensors = load_file(str(make_dir(tmp_path, "pa") / "model.safetensors"))
    names = set(tensors)
    assert {"embed", "head", "final.norm", "loop.step", "loop.in", "l0.norm1", "l0.norm2", "l0.mix.q.norm", "l0.mix.v.conv",
            "l0.mix.v.b", "l0.mlp.router", "l0.mlp.e5.down", "l0.mlp.shared.up", "l1.mix.left.sink", "l1.mix.left.g",
            "l1.mix.left.o.b", "l1.mix.left.out", "l1.mix.right.out", "l1.mix.right.norm", "l1.mix.right.i.b",
            "l1.mix.right.f", "l2.mix.ra", "l2.mix.ri.b", "l2.mix.lam", "l2.mix.conv.b", "l2.mix.y.b"} <= names
    assert not {"l2.norm2", "l2.mlp.router", "l0.mix.o.b", "l1.mix.left.v", "l1.mix.left.v.b", "l1.mlp.shared.up",
                "l0.mlp.e0.gate", "l0.mlp.correction", "l1.mix.left.q.norm", "l1.mix.right.q.b"} & names
    assert tensors["loop.step"].shape == (2, 96) and tensors["loop.in"].shape == (96, 192)
    assert tensors["l2.mix.ra"].shape == (5, 16, 16) and tensors["l2.mix.conv"].shape == (80, 3)
    assert tensors["l0.mix.q.norm"].shape == (16,) and tensors["l0.mix.k.conv"].shape == (48, 2)
    assert tensors["l1.mix.right.norm"].shape == (120,) and tensors["l1.mix.left.g"].shape == (4, 96)
    assert "loop.in" not in set(load_file(str(make_dir(tmp_path, "pb") / "model.safetensors")))


def test_every_pass_has_a_cache_and_a_state_of_its_own():
    """Two passes over (pair, recurrent block): six runs; every attention has pages, every recurrence
    a state, and an attention with a convolution has both; pages and slots come back and are taken again."""
    from fastgen_b200.cache import CacheManager
    from fastgen_b200.engine.model import Model

    model = Model(model_args_from_config(PA), ops=None)
    caches, states = model.cache_specs(), model.state_specs()
    assert len(caches) == len(states) == 6
    assert [c is not None for c in caches] == [True, True, False, True, False, True]
    assert all(s is not None for s in states)
    assert caches[0].window == 20 and caches[0].head_dim == 32 and caches[1].window is None
    assert states[0].shape == ((2 - 1) * (6 + 2 * 3) * 32,)
    assert states[1].shape == states[3].shape == (3 * (40 + 1) * 24 + 3,)
    assert states[2].shape == (80 + 2 * 80,)
    cache = CacheManager(caches, states, [None] * 6, page_size=8, n_pages=12, max_requests=2, max_length=64)
    a = cache.admit("a")
    cache.reserve(a, 20)
    cache.advance(a, 20)
    b = cache.admit("b")
    cache.reserve(b, 9)
    cache.advance(b, 9)
    cache.check()
    slot = a.slot
    cache.release("a")
    c = cache.admit("c")
    assert c.slot == slot
    cache.reserve(c, 40)
    cache.advance(c, 40)
    cache.check()
    cache.release("b")
    cache.release("c")
    assert all(f == g.pool.n_pages for f, g in zip(cache.free_pages(), cache.groups))


# ---------------------------------------------------------------------------------
# mechanisms alone
# ---------------------------------------------------------------------------------
def _drawn_mixer(kind, m, dim, g, std=0.3, tweak=None, eps=1e-5):
    """A mixer of the given sizes and its random tensors (bfloat16 values), not bound yet."""
    from fastgen_b200.config import palulorn as cfg
    from fastgen_b200.parts import make_mixer

    build = {"parallel": cfg._pair, "left": cfg._sink_attention, "right": cfg._matrix_memory, "rglru": cfg._recurrent,
             "attention": cfg._window_attention}[kind]
    mixer = make_mixer(build(dim, eps, m, "mix.", "test"))
    return mixer, _draw_all(mixer, g, std, tweak)


def _mixer_and_cache(kind, m, dim, dtype, g, page=8, n_pages=16, std=0.3, tweak=None, eps=1e-5):
    """A mixer of the given sizes with random tensors, bound, with a cache of its own."""
    from fastgen_b200.cache import CacheManager

    ops = _ops(dtype)
    mixer, w = _drawn_mixer(kind, m, dim, g, std, tweak, eps)
    mixer.bind({local: w[name].to(DEV) for local, name in mixer.names.items()}, ops)
    cache = CacheManager([mixer.cache_spec()], [mixer.state_spec()], [None], page, n_pages, 2, page * n_pages,
                         dtype=dtype, device=DEV, tensor_map_factory=ops.make_kv_tensor_maps)
    return mixer, cache, {k: v.double() for k, v in w.items()}, ops


PORTIONS = (33, 1, 1, 7, 1, 2, 3, 1, 26)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sizes", [(4, 2, 32, 0.15, (0.5, 7)), (1, 1, 64, 0.1, None), (5, 1, 16, 0.2, (0.3, 16)),
                                   (2, 1, 32, 0.2, (1.0, 1)), (8, 2, 64, 0.11, (0.2, 40)), (2, 2, 128, 0.04, (0.6, 3)),
                                   (3, 3, 24, 0.3, None), (16, 2, 48, 0.14, (0.1, 50))])
def test_attention_with_a_sink_alone(dtype, sizes):
    """Keys that are the values, biases, the temperature of the query's position, the sink in the
    denominator, the gate per head: a portion, single tokens and short portions across pages of eight;
    then the pages are freed and taken again.  Leaving out the sink, the gate or the temperature would
    each give another output."""
    heads, kv, d, scale, temp = sizes
    g = torch.Generator().manual_seed(heads * 100 + d)
    m = _sink(heads, kv, d, scale, temp)
    mixer, cache, w, ops = _mixer_and_cache("left", m, 40, dtype, g)
    x = torch.randn(75, 40, generator=g).to(dtype)
    ref = pp.sink_attention(x.double(), m, w, "mix.")
    big = float(ref.abs().max())
    no_sink = pp.sink_attention(x.double(), m, dict(w, **{"mix.sink": torch.full((heads,), -1e9, dtype=torch.float64)}), "mix.")
    assert float((no_sink - ref).abs().max()) > 0.05 * big
    if temp:
        assert float((pp.sink_attention(x.double(), dict(m, q_temp=None), w, "mix.") - ref).abs().max()) > 0.01 * big
    out, req = _run_mixer(mixer, cache, x, PORTIONS, dtype)
    ops.check_status()
    _close(out, ref, dtype)
    cache.release("r")
    out2, _ = _run_mixer(mixer, cache, x[:30], (2, 1, 27), dtype, rid="again")
    _close(out2, ref[:30], dtype, big)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("mode", ["prompt", "decoded"])
@pytest.mark.parametrize("d", [16, 64])
def test_far_key_beside_the_sink(dtype, mode, d):
    """One key 400 positions back has a score far above all others; the sink of one head is as large, so
    that head gives the key about half of the weight, and the other head, whose sink is small, nearly all
    of it.  Without the key, or without the sink, the output is another one: in a prompt portion and for
    tokens decoded alone, with the key on the first of many pages."""
    heads, kv, n = 2, 1, 420
    g = torch.Generator().manual_seed(21)
    m = _sink(heads, kv, d, 1.0, (0.25, 128))

    def tweak(w):
        for h in range(heads):
            w["mix.q"][h * d + d - 1, :] = 0
            w["mix.q"][h * d + d - 1, 0] = 1.0
        w["mix.k"][d - 1, :] = 0
        w["mix.k"][d - 1, 1] = 1.0
        w["mix.q.b"][:] = 0
        w["mix.k.b"][:] = 0
        w["mix.sink"][:] = torch.tensor([12.0, -3.0]).bfloat16()
        w["mix.g"][:] = 0  # every gate one half
    mixer, cache, w, ops = _mixer_and_cache("left", m, 24, dtype, g, page=16, n_pages=32, std=0.05, tweak=tweak)
    x = 0.3 * torch.randn(n, 24, generator=g)
    x[:, :2] = 0.0
    far, q1, q2 = 3, n - 1, n - 40
    x[far, 1] = 3.0
    x[q1, 0] = x[q2, 0] = 2.0  # score 6 times the temperature of the position (1.3 and more): about the sink
    x = x.to(dtype)
    ref = pp.sink_attention(x.double(), m, w, "mix.")
    x0 = x.clone()
    x0[far] = 0
    without = pp.sink_attention(x0.double(), m, w, "mix.")
    no_sink = pp.sink_attention(x.double(), m, dict(w, **{"mix.sink": torch.full((heads,), -1e9, dtype=torch.float64)}), "mix.")
    for q in (q1, q2):
        scale = float(ref[q].abs().max())
        assert float((ref[q] - without[q]).abs().max()) > 0.15 * scale
        assert float((ref[q] - no_sink[q]).abs().max()) > 0.15 * scale
    out, _ = _run_mixer(mixer, cache, x, (300, 120) if mode == "prompt" else (300, 70) + (1,) * 50, dtype)
    ops.check_status()
    for q in (q1, q2):
        assert float((out[q] - ref[q]).abs().max()) <= _tol(dtype) * float(ref[q].abs().max()), q
    _close(out, ref, dtype)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sizes", [(3, 24, 40, 10.0), (1, 33, 5, 4.0), (2, 160, 12, 15.0), (3, 16, 16, 8.0), (6, 40, 56, 12.0),
                                   (2, 64, 9, 2.0), (4, 128, 32, 15.0), (1, 256, 64, 5.0), (8, 32, 128, 30.0), (2, 8, 1, 1.0)])
def test_matrix_memory_alone(dtype, sizes):
    """Capped log gates, the running maximum that starts at zero, state and normaliser, the floor of
    the denominator, norm per head, gate: a prompt portion, single tokens and short portions through the
    state of a slot; then the slot is used again and starts from zero."""
    g = torch.Generator().manual_seed(sum(int(s) for s in sizes))
    m = _memory(*sizes)
    mixer, cache, w, ops = _mixer_and_cache("right", m, 72, dtype, g)
    x = torch.randn(60, 72, generator=g).to(dtype)
    ref = pp.matrix_memory(x.double(), m, w, "mix.", 1e-5)
    out, req = _run_mixer(mixer, cache, x, (30, 1, 1, 7, 1, 2, 3, 1, 14), dtype)
    ops.check_status()
    # a head of one value column norms to a sign, which no rounding survives: compared in size only
    cmp = (lambda t: t.abs()) if sizes[2] == 1 else (lambda t: t)
    _close(cmp(out), cmp(ref), dtype)
    slot = req.slot
    cache.release("r")
    out2, req2 = _run_mixer(mixer, cache, x[:20], (1, 2, 17), dtype, rid="again")
    assert req2.slot == slot
    _close(cmp(out2), cmp(ref[:20]), dtype, float(ref.abs().max()))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_the_running_maximum_starts_at_zero_and_the_gates_are_capped(dtype):
    """Input gates far below zero: with a maximum that started at minus infinity the first write would
    be rescaled to one; started at zero it stays tiny and the floor exp(-m) = 1 of the denominator
    decides.  And sums far above the cap are capped."""
    g = torch.Generator().manual_seed(5)
    m = _memory(2, 16, 8, 6.0)

    def tweak(w):
        w["mix.i"][:] = 0
        w["mix.i.b"][:] = torch.tensor([-4.0, 40.0]).bfloat16()  # head 0: far below zero; head 1: capped at 6
        w["mix.f.b"][:] = torch.tensor([3.0, -40.0]).bfloat16()   # head 1: forget gate capped at logsigmoid(-6)
    mixer, cache, w, ops = _mixer_and_cache("right", m, 32, dtype, g, tweak=tweak)
    x = torch.randn(40, 32, generator=g).to(dtype)
    ref = pp.matrix_memory(x.double(), m, w, "mix.", 1e-5)
    out, _ = _run_mixer(mixer, cache, x, (1, 1, 1, 17, 2, 18), dtype)
    ops.check_status()
    _close(out, ref, dtype)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("kind", ["right", "rglru"])
def test_state_carries_what_was_long_ago(dtype, kind):
    """Next to no forgetting: what was written 150 tokens back still makes most of the read-out, through
    portions and single tokens (a state lost or zeroed on the way would show)."""
    g = torch.Generator().manual_seed(5)
    if kind == "right":
        m = _memory(2, 16, 8, 15.0)

        def tweak(w):
            w["mix.f"][:] = 0
            w["mix.f.b"][:] = 14.0  # logsigmoid(14): next to no forgetting
            w["mix.i"][:] = 0
            w["mix.i.b"][:] = -2.0
        ref_fn = lambda xx, w: pp.matrix_memory(xx, m, w, "mix.", 1e-5)
    else:
        m = _lru(32, 2, 3)

        def tweak(w):
            w["mix.lam"][:] = -9.0  # softplus(-9) ~ 1e-4: a ~ 1 - 1e-3 r
            w["mix.x.b"][:] = 0     # (a bias would be written at every token and outweigh the one input)
            w["mix.conv.b"][:] = 0
        ref_fn = lambda xx, w: pp.gated_linear_recurrence(xx, m, w, "mix.")
    mixer, cache, w, ops = _mixer_and_cache(kind, m, 32, dtype, g, std=0.2, n_pages=32, tweak=tweak)
    x = 0.02 * torch.randn(170, 32, generator=g)
    x[5] = 2.0 * torch.randn(32, generator=g)
    x = x.to(dtype)
    ref = ref_fn(x.double(), w)
    x0 = x.clone()
    x0[5] = 0
    other = ref_fn(x0.double(), w)
    assert float((ref[160] - other[160]).abs().max()) > 0.2 * float(ref[160].abs().max())
    out, _ = _run_mixer(mixer, cache, x, (4, 3, 90, 2) + (1,) * 50 + (21,), dtype)
    ops.check_status()
    _close(out, ref, dtype)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sizes", [(80, 5, 3), (64, 1, 1), (120, 3, 4), (48, 2, 2), (288, 4, 3), (36, 36, 8), (256, 2, 5)])
def test_gated_linear_recurrence_alone(dtype, sizes):
    """Both branches, the convolution with its bias and its last inputs, the block-diagonal gate maps,
    the decay and the recurrence from zero: a prompt portion, single tokens and short portions through
    the state of a slot; then the slot is used again."""
    g = torch.Generator().manual_seed(sum(sizes))
    m = _lru(*sizes)
    mixer, cache, w, ops = _mixer_and_cache("rglru", m, 72, dtype, g)
    x = torch.randn(60, 72, generator=g).to(dtype)
    ref = pp.gated_linear_recurrence(x.double(), m, w, "mix.")
    out, req = _run_mixer(mixer, cache, x, (30, 1, 1, 7, 1, 2, 3, 1, 14), dtype)
    ops.check_status()
    _close(out, ref, dtype)
    slot = req.slot
    cache.release("r")
    out2, req2 = _run_mixer(mixer, cache, x[:20], (1, 2, 17), dtype, rid="again")
    assert req2.slot == slot
    _close(out2, ref[:20], dtype, float(ref.abs().max()))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sizes", [
    # heads, key/value heads, key size, value size, scale, taps, (turned dimensions, base, factor), window
    (6, 3, 16, 32, 0.2, 2, (8, 5000.0, 8.0), 20),
    (2, 1, 48, 48, 0.12, 4, (24, 300.0, None), 9),
    (4, 1, 16, 8, 0.25, None, None, None),
    (2, 2, 64, 64, 0.12, 3, (64, 1e4, 2.0), 70),
    (2, 2, 80, 16, 0.11, 2, (40, 2000.0, 4.0), 1),
    (3, 1, 16, 16, 0.25, 8, (8, 100.0, None), 33),
    (4, 2, 96, 48, 0.08, 2, (48, 1e5, 3.0), 24),
    (2, 1, 128, 128, 0.09, 2, (64, 1e4, 2.0), None),
])
def test_window_attention_alone(dtype, sizes):
    """Biases, the convolution on q, k and v with its last inputs, the norm per head, a part of each
    head turned (dimension i with dimension i + half) with divided frequencies, the window: a portion,
    single tokens and short portions across pages of eight; then pages and slot are freed and taken again."""
    heads, kv, d, dv, scale, conv, rot, window = sizes
    g = torch.Generator().manual_seed(heads * 100 + d)
    m = _attn(heads, kv, d, dv, scale, conv, rot, window)
    mixer, cache, w, ops = _mixer_and_cache("attention", m, 40, dtype, g)
    x = torch.randn(75, 40, generator=g).to(dtype)
    ref = pp.window_attention(x.double(), m, w, "mix.", 1e-5)
    if window and window < 60:
        wider = pp.window_attention(x.double(), dict(m, mask=dict(size=window + 1)), w, "mix.", 1e-5)
        assert float((wider - ref).abs().max()) > 0.005 * float(ref.abs().max())
    out, req = _run_mixer(mixer, cache, x, PORTIONS, dtype)
    ops.check_status()
    _close(out, ref, dtype)
    cache.release("r")
    out2, _ = _run_mixer(mixer, cache, x[:30], (2, 1, 27), dtype, rid="again")
    _close(out2, ref[:30], dtype, float(ref.abs().max()))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("mode", ["prompt", "decoded"])
def test_keys_at_the_window_edge_and_at_page_borders(dtype, mode):
    """Few keys have a score far above the others: for some queries such a key is the last one inside
    the window, for others the first one outside; some sit on the last place of a page or the first of
    the next.  A window one key wider or narrower gives another output at those queries."""
    g = torch.Generator().manual_seed(23)
    d, window = 16, 21
    m = _attn(2, 2, d, d, 2.5, None, (4, 100.0, None), window)

    def tweak(w):
        # a head's last dimension (which does not turn): every query is large there (input channel 0),
        # a key only where input channel 1 is
        for h in range(2):
            for t, col in (("mix.q", 0), ("mix.k", 1)):
                w[t][h * d + d - 1, :] = 0
                w[t][h * d + d - 1, col] = 4.0
                w[t + ".b"][:] = 0
        w["mix.q.norm"][:] = 1.0
        w["mix.k.norm"][:] = 1.0
    mixer, cache, w, ops = _mixer_and_cache("attention", m, 24, dtype, g, page=8, n_pages=16, std=0.05, tweak=tweak)
    x = _edge_inputs(g)
    loud = LOUD
    x = x.to(dtype)
    ref = pp.window_attention(x.double(), m, w, "mix.", 1e-5)
    wider = pp.window_attention(x.double(), dict(m, mask=dict(size=window + 1)), w, "mix.", 1e-5)
    narrower = pp.window_attention(x.double(), dict(m, mask=dict(size=window - 1)), w, "mix.", 1e-5)
    for i in loud:
        inside, outside = i + window - 1, i + window  # the last query that sees key i, the first that does not
        assert float((ref[inside] - narrower[inside]).abs().max()) > 0.05 * float(ref[inside].abs().max())
        assert float((ref[outside] - wider[outside]).abs().max()) > 0.05 * float(ref[outside].abs().max())
    plans = ((8, 24, 8, 7, 1, 16, 32), (96,), (27, 2, 3, 64)) if mode == "prompt" else ((7, 1, 1, 23) + (1,) * 64,)
    for portions in plans:
        out, _ = _run_mixer(mixer, cache, x, portions, dtype)
        ops.check_status()
        _close(out, ref, dtype)
        cache.release("r")


LOUD = (7, 8, 31, 32, 47, 48, 63)


def _edge_inputs(g):
    x = 0.3 * torch.randn(96, 24, generator=g)
    x[:, 0] = 1.0
    x[:, 1] = 0.01
    for i in LOUD:
        x[i, 1] = 3.0
    return x


def _feed_forward_alone(mlp, dim, dtype, g, std=0.3, tweak=None):
    from fastgen_b200.config.palulorn import _feed_forward
    from fastgen_b200.parts import make_feed_forward

    ops = _ops(dtype)
    ff = make_feed_forward(_feed_forward(dim, mlp, "mlp.", "test"))
    w = _draw_all(ff, g, std, tweak)
    ff.bind({local: w[name].to(DEV) for local, name in ff.names.items()}, ops)
    return ff, {k: v.double() for k, v in w.items()}, ops


def _clear_choices(x, mlp, w, margin):
    """Tokens whose choice of groups and of experts rests on no close call."""
    r = mlp["router"]
    s = torch.sigmoid(x @ w["mlp.router"].T)
    ok = torch.ones(x.shape[0], dtype=torch.bool)
    allowed = torch.ones_like(s, dtype=torch.bool)
    if r.get("groups"):
        count, keep = r["groups"]["count"], r["groups"]["keep"]
        per = r["experts"] // count
        gs = s.view(-1, count, per).topk(min(2, per), dim=-1).values.sum(-1)
        c = torch.sort(gs, dim=-1, descending=True)
        if keep < count:
            ok &= (c.values[:, keep - 1] - c.values[:, keep]) > margin
        keep_mask = torch.zeros_like(gs, dtype=torch.bool).scatter_(1, c.indices[:, :keep], True)
        allowed = keep_mask[:, :, None].expand(-1, -1, per).reshape(s.shape)
    c = torch.sort(torch.where(allowed, s, torch.full_like(s, -1.0)), dim=-1, descending=True).values
    if r["top"] < c.shape[1]:
        ok &= (c[:, r["top"] - 1] - c[:, r["top"]]) > margin
    return ok


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sizes", [(6, 3, 40, (3, 2), 2.0, 24), (5, 2, 24, None, 1.0, None), (8, 1, 16, (4, 1), 0.5, 8),
                                   (1, 1, 56, None, 1.0, None), (4, 4, 16, (2, 2), 1.0, 16), (9, 4, 8, (3, 2), 2.5, None),
                                   (8, 3, 80, (4, 3), 1.25, 48), (64, 6, 24, (8, 3), 1.0, 8), (33, 5, 16, (33, 7), 3.0, None),
                                   (12, 2, 32, (2, 1), 1.0, 16)])
@pytest.mark.parametrize("tokens", [1, 3, 70, 600])
def test_routed_experts_alone(dtype, sizes, tokens):
    """Sigmoid scores in float32, the groups' scores (the two largest added), the choice among the best
    groups, the chosen scores divided by their sum and multiplied by the router's scale, experts with a
    squared ReLU and no gate, the shared expert; one expert, all experts, groups of one, more experts
    than a warp has lanes; one token, a few, more tokens than experts, and a prompt's worth."""
    experts, top, ff, groups, scale, shared = sizes
    g = torch.Generator().manual_seed(experts * 10 + top)
    mlp = _moe(experts, top, ff, groups, scale, shared)
    part, w, ops = _feed_forward_alone(mlp, 48, dtype, g)
    x = torch.randn(tokens, 48, generator=g).to(dtype)
    ref = pp.routed_experts(x.double(), mlp, w, "mlp.")
    out = _value(part.forward(x.to(DEV), _context(0, 0, tokens))).cpu()
    ops.check_status()
    ok = _clear_choices(x.double(), mlp, w, 1e-5)  # both see the same rounded input: float32 sums are that close
    assert int(ok.sum()) >= (tokens * 2 + 2) // 3
    _close(out[ok], ref[ok], dtype, float(ref.abs().max()))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_the_groups_limit_the_choice(dtype):
    """The two experts with the largest scores sit in two groups that each hold nothing else of note; a
    third group holds two middling experts whose scores add up to more.  With one group kept, both
    choices come from that third group: choosing by score alone, or scoring a group by its best expert,
    would each give another output."""
    g = torch.Generator().manual_seed(31)
    experts, top = 6, 2
    mlp = _moe(experts, top, 32, (3, 1), 1.5, None)

    def tweak(w):
        rows = torch.zeros(experts, 48)
        rows[:, 0] = torch.tensor([4.0, -6.0, 3.5, -6.0, 1.5, 1.4])  # logits for x[0] = 1
        w["mlp.router"] = rows.bfloat16()
    part, w, ops = _feed_forward_alone(mlp, 48, dtype, g, tweak=tweak)
    x = 0.5 * torch.randn(40, 48, generator=g)
    x[:, 0] = 1.0
    x = x.to(dtype)
    xd = x.double()
    ref = pp.routed_experts(xd, mlp, w, "mlp.")
    s = torch.sigmoid(xd @ w["mlp.router"].T)

    def expert(e, rows):
        return (torch.relu(rows @ w[f"mlp.e{e}.up"].T) ** 2) @ w[f"mlp.e{e}.down"].T
    want = torch.stack([sum(1.5 * s[t, e] / (s[t, 4] + s[t, 5]) * expert(e, xd[t:t + 1])[0] for e in (4, 5)) for t in range(40)])
    assert float((want - ref).abs().max()) < 1e-9
    by_score = torch.stack([sum(1.5 * s[t, e] / (s[t, 0] + s[t, 2]) * expert(e, xd[t:t + 1])[0] for e in (0, 2)) for t in range(40)])
    assert float((by_score - ref).abs().max()) > 0.2 * float(ref.abs().max())
    out = _value(part.forward(x.to(DEV), _context(0, 0, 40))).cpu()
    ops.check_status()
    _close(out, ref, dtype)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_two_mixers_side_by_side(dtype):
    """Both halves read the same input; each output is normed over the model width with its own weight
    and the result is half their sum; the attention of the pair has the pages, the memory the slot's state."""
    g = torch.Generator().manual_seed(41)
    m = _pair(_sink(4, 2, 32, 0.15, (0.5, 7)), _memory(3, 24, 40, 10.0))
    mixer, cache, w, ops = _mixer_and_cache("parallel", m, 56, dtype, g, std=0.25)
    x = torch.randn(50, 56, generator=g).to(dtype)
    ref = pp.two_mixers(x.double(), m, w, "mix.", 1e-5)
    left = pp.sink_attention(x.double(), m["left"], w, "mix.left.")
    right = pp.matrix_memory(x.double(), m["right"], w, "mix.right.", 1e-5)
    assert float((ref - 0.5 * (left + right)).abs().max()) > 0.05 * float(ref.abs().max())
    out, _ = _run_mixer(mixer, cache, x, (20, 1, 1, 2, 5, 1, 20), dtype)
    ops.check_status()
    _close(out, ref, dtype)


# ---------------------------------------------------------------------------------
# whole models through the engine
# ---------------------------------------------------------------------------------
def model_dir(tmp_path, name, dtype):
    """The model folder of a configuration.  In bfloat16 the engine's activations differ from the plain
    implementation's by a percent, which turns a token's choice of experts wherever two scores are that
    close, so in the folder of the bfloat16 runs all experts of a layer are the same expert: whichever
    are chosen, their weights add up to the router's scale and the output is the same.  Choices that
    depend on the token are held in float32, and in bfloat16 by ``test_routed_experts_alone``."""
    from safetensors.torch import load_file, save_file

    if dtype == torch.float32:
        return make_dir(tmp_path, name)
    d = make_dir(Path(tmp_path) / "alike", name)
    f = Path(d) / "model.safetensors"
    tensors = load_file(str(f))
    for key in list(tensors):
        parts = key.split(".")
        if len(parts) == 4 and parts[1] == "mlp" and parts[2].startswith("e") and parts[2][1:].isdigit():
            tensors[key] = tensors[f"{parts[0]}.mlp.e0.{parts[3]}"].clone()
    save_file(tensors, str(f))
    return d


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("name", ["pa", "pb", "pc", "pd", "pe"])
@pytest.mark.parametrize("plan", ["whole", "decode", "portions", "mixed"])
def test_replay(tmp_path, name, dtype, plan):
    """Whole prompts (of one and two tokens too), prompts with a decoded tail that passes the windows,
    portions of 2 to 17 tokens, and mixed batches of up to four requests whose pages and slots are used
    again, all against the plain implementation run on whole sequences."""
    d = model_dir(tmp_path, name, dtype)
    vocab = CONFIGS[name][0]["vocab"]
    page = 16
    if plan == "mixed":
        requests = _requests(vocab, [70, 33, 1, 90, 18, 64, 47, 2], 40)
        steps = H.plan_mixed(requests, seed=5)
    else:
        requests = _requests(vocab, [1, 2, 37, 150] if plan != "portions" else [2, 95], 20)
        steps = {"whole": H.plan_whole, "decode": lambda r: H.plan_decode_tail(r, 45), "portions": H.plan_portions}[plan](requests)
    outputs, engine = H.run_engine(d, dtype, steps, page, H.max_live_tokens(steps, page) + 2 * page)
    compare(d, requests, H.collect(steps, outputs), dtype)
    assert engine.cache.n_live == 0 and all(f == g.pool.n_pages for f, g in zip(engine.cache.free_pages(), engine.cache.groups))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("name", ["pa", "pc"])
def test_batching_changes_nothing(tmp_path, dtype, name):
    """A request's logits in a batch of unequal requests equal those it gets alone (bitwise in float32,
    where every sum has a fixed order; within rounding in bfloat16)."""
    d = model_dir(tmp_path, name, dtype)
    requests = _requests(CONFIGS[name][0]["vocab"], [41, 5, 77, 20], 60)
    alone = H.plan_portions(requests, sizes=(9, 1, 1, 30))
    out_a, _ = H.run_engine(d, dtype, alone, 8, H.max_live_tokens(alone, 8) + 32)
    got_a = H.collect(alone, out_a)
    mixed = H.plan_mixed(requests, seed=2)
    out_m, _ = H.run_engine(d, dtype, mixed, 8, H.max_live_tokens(mixed, 8) + 32)
    got_m = H.collect(mixed, out_m)
    pairs = []
    for rid, toks in requests.items():
        for p in range(len(toks)):
            if dtype == torch.float32:
                assert np.array_equal(got_a[rid][p], got_m[rid][p]), (rid, p)
            pairs.append((f"{rid} {p}", got_m[rid][p], got_a[rid][p]))
    check_rows(pairs, dtype)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("name", ["pa", "pb", "pc"])
def test_steps_replayed_from_graphs_change_nothing(tmp_path, dtype, name):
    """Steps captured as CUDA graphs (single tokens, and prompt portions padded to a few shapes) give
    what the same steps give launched kernel by kernel: states and convolution inputs are advanced by the
    replays only, never by a capture, and padding lanes choose no expert."""
    d = model_dir(tmp_path, name, dtype)
    requests = _requests(CONFIGS[name][0]["vocab"], [41, 5, 77, 20], 61)
    mixed = H.plan_mixed(requests, seed=3)
    room = H.max_live_tokens(mixed, 8) + 32
    out_g, eng = H.run_engine(d, dtype, mixed, 8, room, max_step_tokens=64)
    assert eng.graphs is not None and eng.step_graphs is not None and eng.step_graphs.replays > 0
    out_p, _ = H.run_engine(d, dtype, mixed, 8, room, num_cuda_graphs=0)
    got_g, got_p = H.collect(mixed, out_g), H.collect(mixed, out_p)
    pairs = []
    for rid, toks in requests.items():
        for p in range(len(toks)):
            if dtype == torch.float32:
                assert np.array_equal(got_g[rid][p], got_p[rid][p]), (rid, p)
            pairs.append((f"{rid} {p}", got_g[rid][p], got_p[rid][p]))
    check_rows(pairs, dtype)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_long_decoding(tmp_path, dtype):
    """200 tokens decoded one by one after a two-token prompt, over many pages of eight: every pass's
    cache grows by itself, the windows pass over decoded tokens and every pass's state is carried."""
    d = model_dir(tmp_path, "pa", dtype)
    requests = _requests(211, [202], 77)
    steps = H.plan_decode_tail(requests, 200)
    outputs, engine = H.run_engine(d, dtype, steps, 8, 232)
    compare(d, requests, H.collect(steps, outputs), dtype)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("name", ["pa", "pd"])
def test_slots_used_again_start_from_zero(tmp_path, dtype, name):
    """Two slots only: six requests pass through them one after the other, some ending in the middle of
    a step of the others; a state or a convolution input left by a slot's earlier request would show in
    the first tokens of the next."""
    d = model_dir(tmp_path, name, dtype)
    requests = _requests(CONFIGS[name][0]["vocab"], [30, 9, 41, 3, 26, 12], 81)
    steps = H.plan_mixed(requests, seed=7, max_live=2)
    outputs, engine = H.run_engine(d, dtype, steps, 8, H.max_live_tokens(steps, 8) + 16, max_requests=2)
    compare(d, requests, H.collect(steps, outputs), dtype)
    assert engine.cache.n_live == 0


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("name", ["pa", "pc"])
def test_greedy_generation_through_the_entry_point(tmp_path, dtype, name):
    """``Fastgen.generate`` with its scheduler (portions of 16 tokens, batches of 3, graphs) against
    greedy decoding with the plain implementation."""
    from fastgen_b200.engine import Fastgen, GenArgs, HfLoader, Packet

    d = model_dir(tmp_path, name, dtype)
    cfg, w = pp.read_model(d)
    vocab = cfg["vocab"]
    prompts = [H.random_tokens(vocab, n, 90 + n) for n in (7, 1, 40, 23)]
    fg = Fastgen.build(HfLoader(d), GenArgs(use_sampling=False, max_gen=12, cache_block=16, max_seq=128, max_batch=3,
                                            max_prefill=16),
                       tp_mesh=None, device=torch.device(DEV), dtype=dtype)
    q = queue.Queue()
    for i, p in enumerate(prompts):
        q.put(Packet(thread_id=i, tokens=p))
    q.put(None)
    got = {pkt.thread_id: pkt.tokens for pkt in fg.generate(q)}
    fg.destroy()
    for i, p in enumerate(prompts):
        assert len(got[i]) == 12
        if dtype == torch.float32:
            assert got[i] == pp.greedy(cfg, w, p, 12), i
        else:
            seq = list(p)
            for tok in got[i]:
                logits = pp.forward(cfg, w, seq)[-1]
                assert float(logits[tok]) >= float(logits.max()) - 0.03 * float(logits.abs().max())
                seq.append(tok)
