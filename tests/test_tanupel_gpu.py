"""Tanupel through the engine against the plain implementation of ``plain_tanupel.py``: each
mechanism alone, whole prompts against token-by-token decoding, portions down to two tokens,
unequal batches, pages and slots used again, keys far away and at page borders, a state that
carries what was long ago, the first tokens of a sequence, long decoding, sizes that pad or equal
one, and greedy generation through ``Fastgen.generate``."""

import copy
import queue
from pathlib import Path

import numpy as np
import pytest
import torch

import helpers as H
import plain_tanupel as pt
from fastgen_b200.config import ConfigError, PartSpec, model_args_from_config
from fastgen_b200.weights import write_random_model

DEV = "cuda:0"


def _rot(dims, base=10000.0, scaling=None):
    rot = dict(dims=dims, base=base)
    if scaling:
        rot["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return rot


def _attn(heads, kv, dim, vdim, scale, dims=None, base=10000.0, scaling=None, softcap=None):
    m = dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, scale=scale)
    if dims:
        m["rot"] = _rot(dims, base, scaling)
    if softcap is not None:
        m["softcap"] = softcap
    return m


def _delta(heads, kv, dim, vdim, conv, decay_rank=8, gate_rank=8):
    return dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, conv=conv, decay_rank=decay_rank, gate_rank=gate_rank)


def _pair(left, right, left_scale, right_scale):
    return dict(left=left, right=right, left_scale=left_scale, right_scale=right_scale)


def _dense(ff):
    return dict(kind="dense", ff=ff)


def _moe(experts, top, ff):
    return dict(kind="moe", expert=dict(ff=ff), router=dict(experts=experts, top=top))


def _layer(kind, mixer, mlp):
    return dict(type=kind, mixer=mixer, mlp=mlp)


# a run of two layers passed twice, opened by a pair; routed experts with three of five; value heads
# larger and smaller than query heads; frequencies bent by wavelength, divided, and as they are; a
# layer without a feed-forward; fewer query/key heads than heads in the delta rule
TA = dict(
    architecture="Tanupel", vocab=211, width=96, norm=dict(eps=1e-5), embedding=dict(scale=3.0), residual_mult=0.4,
    loop=dict(start=1, stop=3, times=2),
    layers=[
        _layer("attention", _attn(6, 3, 16, 32, 0.2, dims=8, base=5000.0, scaling=(8.0, 1.0, 4.0, 64)), _moe(5, 3, 40)),
        _layer("parallel", _pair(_attn(4, 2, 32, 16, 0.15, dims=32, base=1e4, scaling=(2.0,), softcap=5.0),
                                 _delta(4, 2, 24, 40, 3, 8, 12), 0.7, 1.3), _dense(72)),
        _layer("attention", _attn(2, 1, 48, 48, 0.12, dims=24, base=300.0), None),
        _layer("parallel", _pair(_attn(3, 3, 16, 16, 0.3, dims=4, base=1e6, scaling=(4.0,), softcap=2.0),
                                 _delta(2, 2, 40, 8, 2, 5, 16), 1.0, 0.5), _moe(7, 1, 24)),
    ],
)
# no repeated run, no embedding scale, a multiplier of one; one expert of one; a convolution of one
# tap (no inputs to keep); a delta rule of one head with a state of one column; heads that rotate whole
TB = dict(
    architecture="Tanupel", vocab=97, width=64, norm=dict(eps=1e-6),
    layers=[
        _layer("parallel", _pair(_attn(2, 2, 16, 16, 0.25, dims=16, base=777.0, scaling=(1.5,), softcap=50.0),
                                 _delta(1, 1, 33, 1, 1, 3, 1), 1.0, 1.0), _moe(1, 1, 56)),
        _layer("attention", _attn(4, 1, 16, 8, 0.25, dims=16, base=1e4, scaling=(4.0, 1.0, 2.0, 16)), _dense(100)),
        _layer("parallel", _pair(_attn(1, 1, 64, 64, 0.1, dims=2, base=50.0, scaling=(3.0,), softcap=1.0),
                                 _delta(6, 3, 8, 24, 8, 2, 2), 0.3, 2.0), None),
    ],
)
# the whole model is the repeated run (three passes from the first layer to the last); a state of
# 200 rows; experts that all serve every token
TC = dict(
    architecture="Tanupel", vocab=130, width=80, norm=dict(eps=1e-5), embedding=dict(scale=0.5), residual_mult=0.25,
    loop=dict(start=0, stop=2, times=3),
    layers=[
        _layer("parallel", _pair(_attn(5, 1, 16, 32, 0.2, dims=16, base=1e4, scaling=(2.0,), softcap=8.0),
                                 _delta(2, 1, 200, 12, 4, 16, 8), 0.9, 0.8), _moe(3, 3, 32)),
        _layer("attention", _attn(2, 2, 80, 16, 0.11, dims=40, base=2000.0, scaling=(2.0, 1.0, 8.0, 32)), _dense(48)),
    ],
)
# a run of one layer passed once, in the middle
TD = dict(
    architecture="Tanupel", vocab=64, width=48, norm=dict(eps=1e-5), residual_mult=0.5,
    loop=dict(start=1, stop=2, times=1),
    layers=[
        _layer("attention", _attn(3, 1, 16, 16, 0.25, dims=8, base=100.0), _dense(64)),
        _layer("parallel", _pair(_attn(2, 1, 32, 32, 0.2, dims=16, base=1e4, scaling=(8.0,), softcap=3.0),
                                 _delta(3, 3, 16, 16, 4, 4, 4), 1.0, 1.0), _moe(4, 2, 16)),
        _layer("attention", _attn(3, 1, 16, 16, 0.25, dims=8, base=100.0), _moe(9, 4, 8)),
    ],
)
CONFIGS = {"ta": (TA, 3), "tb": (TB, 5), "tc": (TC, 8), "td": (TD, 9)}


def make_dir(tmp_path, name, std=0.1):
    cfg, seed = CONFIGS[name]
    return write_random_model(Path(tmp_path) / name, cfg, seed, dtype=torch.bfloat16, norm_jitter=0.3, std=std)


_plain = {}


def plain_logits(model_dir, tokens):
    key = (str(model_dir), tuple(tokens))
    if key not in _plain:
        cfg, w = pt.read_model(model_dir)
        _plain[key] = pt.forward(cfg, w, list(tokens)).numpy()
    return _plain[key]


# The bfloat16 rule of this design's models: a row of logits may differ from the plain one by T_L2
# of the row's l2 norm and, in its worst entry, by T_MAX of the row's largest logit.  A pair of
# mixers rounds to bfloat16 about twice as often as one attention, and a repeated run passes every
# rounding through the same weights again.  float32 rows are held to ``helpers.check_row``'s 1e-4.
T_L2, T_MAX = 0.045, 0.055


def check_row(row, ref, dtype, what):
    if dtype == torch.float32:
        return H.check_row(row, ref, dtype, what)
    l2 = float(np.linalg.norm(row - ref) / max(np.linalg.norm(ref), 1e-30))
    mx = float(np.abs(row - ref).max()) / max(float(np.abs(ref).max()), 1e-30)
    assert l2 <= T_L2, f"{what}: l2 error {l2:.4f} of the row's norm (allowed {T_L2})"
    assert mx <= T_MAX, f"{what}: worst entry off by {mx:.4f} of the largest logit (allowed {T_MAX})"


def compare(model_dir, requests, got, dtype):
    for rid, toks in requests.items():
        ref = plain_logits(model_dir, toks)
        assert set(got[rid]) == set(range(len(toks))), f"{rid}: positions missing"
        for p, row in got[rid].items():
            check_row(row, ref[p], dtype, f"{rid} pos {p}")


def _requests(vocab, lengths, seed):
    return {f"r{i}": H.random_tokens(vocab, n, seed + i) for i, n in enumerate(lengths)}


# ---------------------------------------------------------------------------------
# the description and the cache bookkeeping (no GPU)
# ---------------------------------------------------------------------------------
def test_description_reads_every_size_from_the_configuration():
    args = model_args_from_config(TA)
    assert (args.dim, args.vocab_size, args.streams, len(args.layers)) == (96, 211, None, 4)
    assert args.embedder.params.scale == 3.0 and model_args_from_config(TB).embedder.params.scale == 1.0
    att = args.layers[0].mixer.params
    assert (att.n_heads, att.n_kv_heads, att.head_dim, att.v_head_dim, att.softmax_scale) == (6, 3, 16, 32, 0.2)
    assert att.qk_norm == "projection" and att.qk_norm_eps == 1e-5 and att.softcap is None and att.window is None
    rope = att.position.params
    assert (rope.rot_dims, rope.theta, rope.linear_factor) == (8, 5000.0, None) and rope.scaling.factor == 8.0
    pair = args.layers[1].mixer.params
    left, right = pair.left.params, pair.right.params
    assert (pair.left_scale, pair.right_scale, left.softcap) == (0.7, 1.3, 5.0)
    assert left.position.params.linear_factor == 2.0 and left.position.params.scaling is None
    assert (right.n_heads, right.n_kv_heads, right.head_dim, right.v_head_dim, right.conv) == (4, 2, 24, 40, 3)
    assert args.layers[2].mixer.params.position.params.scaling is None
    assert args.layers[2].mixer.params.position.params.linear_factor is None
    assert args.layers[2].ffn is None and args.layers[1].ffn.params.ffn_dim == 72
    moe = args.layers[3].ffn.params
    assert (moe.n_experts, moe.top, moe.ffn_dim, moe.correction, moe.renormalize) == (7, 1, 24, True, False)
    assert all(l.block == "parallel" and l.ffn_norm is None and l.block_params.residual_mult == 0.4 for l in args.layers)
    assert all(l.mixer_norm.params.one_plus for l in args.layers) and args.final_norm.params.one_plus
    # the run of layers 1..2 twice: every run has a cache and a state of its own
    assert [(e.layer, e.step_row, e.kv_from) for e in args.schedule] == [
        (0, None, None), (1, 0, None), (2, None, None), (1, 1, None), (2, None, None), (3, None, None)]
    assert [(e.layer, e.step_row) for e in model_args_from_config(TC).schedule] == [
        (0, 0), (1, None), (0, 1), (1, None), (0, 2), (1, None)]
    assert [(e.layer, e.step_row) for e in model_args_from_config(TD).schedule] == [(0, None), (1, 0), (2, None)]
    assert model_args_from_config(TB).step_table_name is None
    assert model_args_from_config(TB).layers[0].block_params.residual_mult == 1.0


def test_a_pair_divides_its_frequencies_whatever_the_scaling_names():
    cfg = copy.deepcopy(TA)
    cfg["layers"][1]["mixer"]["left"]["rot"]["scaling"] = dict(factor=2.0, low=1.0, high=4.0, original=64)
    rope = model_args_from_config(cfg).layers[1].mixer.params.left.params.position.params
    assert rope.linear_factor == 2.0 and rope.scaling is None


def test_description_errors_name_the_place():
    bad = copy.deepcopy(TA)
    bad["layers"][2]["type"] = "attention_9"
    with pytest.raises(ConfigError, match="attention_9"):
        model_args_from_config(bad)
    bad = copy.deepcopy(TA)
    del bad["layers"][1]["mixer"]["right"]["conv"]
    with pytest.raises(ConfigError, match=r"layers\[1\]\.mixer\.right.*conv"):
        model_args_from_config(bad)
    bad = copy.deepcopy(TA)
    bad["layers"][3]["mlp"]["router"]["top"] = 8
    with pytest.raises(ConfigError, match=r"layers\[3\]"):
        model_args_from_config(bad)
    bad = copy.deepcopy(TA)
    bad["loop"]["stop"] = 5
    with pytest.raises(ConfigError, match="loop"):
        model_args_from_config(bad)
    bad = copy.deepcopy(TA)
    bad["layers"][0]["mlp"]["kind"] = "dense_9"
    with pytest.raises(ConfigError, match="dense_9"):
        model_args_from_config(bad)
    bad = copy.deepcopy(TA)
    bad["layers"][0]["mixer"]["heads"] = 5
    with pytest.raises(ConfigError, match=r"layers\[0\]"):
        model_args_from_config(bad)


def test_random_folder_holds_exactly_the_tensors_of_the_description(tmp_path):
    from safetensors.torch import load_file

    tensors = load_file(str(make_dir(tmp_path, "ta") / "model.safetensors"))
    names = set(tensors)
    assert {"embed", "head", "final.norm", "loop.step", "l0.norm1", "l0.mix.q.norm", "l0.mlp.router", "l0.mlp.correction",
            "l0.mlp.e4.down", "l1.mix.left.k.norm", "l1.mix.right.q.conv", "l1.mix.right.A_log", "l1.mix.right.a2",
            "l1.mix.right.dt_bias", "l1.mix.right.g1", "l1.mix.right.b", "l1.mix.right.norm", "l1.mlp.gate",
            "l3.mlp.e6.up"} <= names
    assert not {"l2.mlp.gate", "l2.mlp.router", "l0.norm2", "l0.mlp.e5.up", "l1.mix.q", "l2.mix.left.q"} & names
    assert tensors["loop.step"].shape == (2, 96) and tensors["l1.mix.right.a1"].shape == (8, 96)
    assert tensors["l1.mix.right.g2"].shape == (160, 12) and tensors["l1.mix.right.a2"].shape == (96, 8)
    assert tensors["l0.mix.q.norm"].shape == (96,) and tensors["l0.mix.k.norm"].shape == (48,)
    assert "loop.step" not in set(load_file(str(make_dir(tmp_path, "tb") / "model.safetensors")))


def test_frequencies():
    from fastgen_b200.config.tanupel import _rope
    from fastgen_b200.parts import make_position

    for dims, base, sc in ((8, 5000.0, (8.0, 1.0, 4.0, 64)), (16, 1e4, (4.0, 1.0, 2.0, 16)), (40, 2000.0, (2.0, 1.0, 8.0, 32)),
                           (32, 1e4, (2.0,)), (4, 1e6, (4.0,)), (24, 300.0, None), (12, 1e4, (4.0, 2.0, 16.0, 4096))):
        rot = _rot(dims, base, sc)
        part = make_position(_rope(rot, 64, "test"))
        want = pt.rotary_frequencies(base, dims, rot.get("scaling"))
        table = part.table("cpu").double()  # a head of 64: 32 pairs, those that do not turn have frequency zero
        assert torch.allclose(table[: dims // 2], want, rtol=2e-6) and not table[dims // 2 :].any(), (dims, base, sc)


def test_every_pass_has_a_cache_and_a_state_of_its_own():
    """Two passes over (pair, attention): six runs, six caches, and a state for each run of a pair;
    pages and slots come back when a request ends and are taken again."""
    from fastgen_b200.cache import CacheManager
    from fastgen_b200.engine.model import Model

    model = Model(model_args_from_config(TA), ops=None)
    caches, states = model.cache_specs(), model.state_specs()
    assert len(caches) == len(states) == 6 and all(c is not None for c in caches)
    assert [s is not None for s in states] == [False, True, False, True, False, True]
    assert states[1].shape == states[3].shape == (4 * 24 * 40 + 2 * (2 * 2 * 24 + 4 * 40),)
    cache = CacheManager(caches, states, [None] * 6, page_size=8, n_pages=12, max_requests=2, max_length=64)
    a = cache.admit("a")
    cache.reserve(a, 20)
    cache.advance(a, 20)
    assert all(len(p) == 3 for p in a.pages) and len({id(g) for g in cache.groups}) >= 1
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
def _ops(dtype):
    from fastgen_b200.csrc.ops import Ops

    return Ops(dtype, DEV)


def _context(slot, start, n):
    from fastgen_b200.engine.step import StepContext

    ctx = StepContext(DEV)
    ctx.host_seq_slot, ctx.host_seq_cached, ctx.host_seq_start = [slot], [start], [0, n]
    ctx.pos = torch.arange(start, start + n, dtype=torch.int32, device=DEV)
    ctx.req = torch.full((n,), slot, dtype=torch.int32, device=DEV)
    ctx.seq_slot = torch.tensor([slot], dtype=torch.int32, device=DEV)
    ctx.seq_start = torch.tensor([0, n], dtype=torch.int32, device=DEV)
    ctx.seq_cached = torch.tensor([start], dtype=torch.int32, device=DEV)
    ctx.n_tokens, ctx.n_seqs = n, 1
    return ctx


def _value(out):
    """A part's output as one float64 tensor (a sum that has not been formed is formed)."""
    from fastgen_b200.parts.base import ScaledSum

    if isinstance(out, ScaledSum):
        assert out.row is None
        return sum(c * t.double() for t, c in out.terms)
    return out.double()


def _run_mixer(mixer, cache, x, portions, dtype, rid="r", entry=0):
    """One request through a mixer in portions; returns the outputs and the request."""
    req = cache.admit(rid)
    outs, start = [], 0
    for n in portions:
        cache.reserve(req, start + n)
        cache.flush_tables()
        ctx = _context(req.slot, start, n)
        outs.append(_value(mixer.forward(x[start:start + n].to(DEV, dtype), ctx, cache.memory(entry))))
        cache.advance(req, start + n)
        start += n
    assert start == x.shape[0]
    return torch.cat(outs).cpu(), req


def _draw_all(part, g, std, tweak):
    from fastgen_b200.weights.random_init import draw

    w = {}
    for s in part.weight_specs():
        t = draw(s, g, 0.4)
        if s.init[0] == "normal" and s.init[1] == 0.02:
            t = t * (std / 0.02)
        w[s.name] = t.bfloat16()
    if tweak:
        tweak(w)
    return w


def _mixer_and_cache(kind, m, dim, dtype, g, page=8, n_pages=16, std=0.3, tweak=None, eps=1e-5):
    """A mixer of the given sizes with random tensors, bound, with a cache of its own."""
    from fastgen_b200.cache import CacheManager
    from fastgen_b200.config.tanupel import _MIXERS
    from fastgen_b200.parts import make_mixer

    ops = _ops(dtype)
    mixer = make_mixer(_MIXERS[kind](dim, eps, m, "mix.", "test"))
    w = _draw_all(mixer, g, std, tweak)
    mixer.bind({local: w[name].to(DEV) for local, name in mixer.names.items()}, ops)
    cache = CacheManager([mixer.cache_spec()], [mixer.state_spec()], [None], page, n_pages, 2, page * n_pages,
                         dtype=dtype, device=DEV, tensor_map_factory=ops.make_kv_tensor_maps)
    return mixer, cache, {k: v.double() for k, v in w.items()}, ops


def _tol(dtype):
    return 2e-5 if dtype == torch.float32 else 2.5e-2


def _close(out, ref, dtype, scale=None):
    scale = float(ref.abs().max()) if scale is None else scale
    err = float((out - ref).abs().max())
    assert err <= _tol(dtype) * scale, f"off by {err / scale:.2e} of the largest value (allowed {_tol(dtype):.1e})"


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("streams", [0, 1, 3, 4])
def test_one_plus_norm_of_a_sum(dtype, streams):
    """``h += row + sum_i c_i y_i`` in float32 and the norm with the factor ``1 + w``, in one kernel: with no
    summand, one, three and four, with and without a row vector; with rows gathered ``h`` stays."""
    from fastgen_b200.parts import RMSNormParams, make_norm
    from fastgen_b200.parts.base import ScaledSum

    ops = _ops(dtype)
    g = torch.Generator().manual_seed(streams)
    t, dim = 11, 200
    norm = make_norm(PartSpec("rmsnorm", RMSNormParams(dim, 1e-5, one_plus=True), {"weight": "w"}))
    w = 0.3 * torch.randn(dim, generator=g)
    norm.bind({"weight": w.to(DEV)}, ops)
    x = 3 * torch.randn(t, dim, generator=g) + 0.5
    ys = [torch.randn(t, dim, generator=g).to(dtype) for _ in range(streams)]
    coefs = [0.3, 1.1, 0.6, 2.0][:streams]
    row = torch.randn(dim, generator=g)
    for with_row in (False, True):
        total = ScaledSum([(y.to(DEV), c) for y, c in zip(ys, coefs)], row.to(DEV) if with_row else None)
        new = x.double() + sum(c * y.double() for y, c in zip(ys, coefs)) + (row.double() if with_row else 0.0)
        want = pt.unit_rms(new, 1e-5) * (1.0 + w.double())
        h = x.clone().to(DEV)
        got = norm.add_forward(h, total if (streams or with_row) else None)
        _close(got.double().cpu(), want, dtype)
        assert float((h.double().cpu() - new).abs().max()) <= 1e-6 * float(new.abs().max())
        rows = torch.tensor([7, 0, 7, 10], dtype=torch.int32, device=DEV)
        h2 = x.clone().to(DEV)
        got = norm.add_forward(h2, total if (streams or with_row) else None, rows=rows)
        _close(got.double().cpu(), want[[7, 0, 7, 10]], dtype)
        assert torch.equal(h2.cpu(), x)
    _close(norm.forward(x.to(DEV)).double().cpu(), pt.unit_rms(x.double(), 1e-5) * (1.0 + w.double()), dtype)
    ops.check_status()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sizes", [(4, 2, 24, 40, 3), (1, 1, 33, 1, 1), (6, 3, 8, 24, 8), (2, 1, 200, 12, 4), (3, 3, 16, 16, 4),
                                   (2, 2, 64, 9, 2), (4, 1, 128, 32, 4), (1, 1, 256, 64, 2), (8, 8, 32, 128, 4)])
def test_gated_delta_rule_alone(dtype, sizes):
    """Convolutions, unit norms, decays per key channel, the corrected write, read-out, norm and
    gate: a prompt portion, single tokens and short portions through the state of a slot; then the
    slot is used again and starts from zero."""
    g = torch.Generator().manual_seed(sum(sizes))
    m = _delta(*sizes, decay_rank=6, gate_rank=10)
    mixer, cache, w, ops = _delta_alone(m, 72, dtype, g)
    x = torch.randn(60, 72, generator=g).to(dtype)
    ref = pt.gated_delta_rule(x.double(), m, w, "mix.", 1e-5)
    out, req = _run_mixer(mixer, cache, x, (30, 1, 1, 7, 1, 2, 3, 1, 14), dtype)
    ops.check_status()
    _close(out, ref, dtype)
    slot = req.slot
    cache.release("r")
    out2, req2 = _run_mixer(mixer, cache, x[:20], (1, 2, 17), dtype, rid="again")
    assert req2.slot == slot
    _close(out2, ref[:20], dtype, float(ref.abs().max()))


def _delta_alone(m, dim, dtype, g, tweak=None, std=0.3, n_pages=16):
    """The delta rule as a mixer of its own (in the design it is the right half of a pair)."""
    from fastgen_b200.cache import CacheManager
    from fastgen_b200.config.tanupel import _gated_delta
    from fastgen_b200.parts import make_mixer

    ops = _ops(dtype)
    mixer = make_mixer(_gated_delta(dim, 1e-5, m, "mix.", "test"))
    w = _draw_all(mixer, g, std, tweak)
    mixer.bind({local: w[name].to(DEV) for local, name in mixer.names.items()}, ops)
    cache = CacheManager([mixer.cache_spec()], [mixer.state_spec()], [None], 8, n_pages, 2, 8 * n_pages,
                         dtype=dtype, device=DEV, tensor_map_factory=ops.make_kv_tensor_maps)
    return mixer, cache, {k: v.double() for k, v in w.items()}, ops


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_state_carries_what_was_long_ago(dtype):
    """A decay close to one: a value written 150 tokens back still makes most of the read-out,
    through portions and single tokens (a state lost or zeroed on the way would show)."""
    g = torch.Generator().manual_seed(4)
    m = _delta(2, 1, 16, 8, 2, 4, 4)

    def tweak(w):
        w["mix.A_log"] = torch.full((2,), -12.0).bfloat16()  # exp(-exp(-12) softplus(.)): next to no decay
    mixer, cache, w, ops = _delta_alone(m, 32, dtype, g, tweak=tweak, std=0.2, n_pages=32)
    x = 0.02 * torch.randn(170, 32, generator=g)
    x[5] = 2.0 * torch.randn(32, generator=g)
    x = x.to(dtype)
    ref = pt.gated_delta_rule(x.double(), m, w, "mix.", 1e-5)
    x0 = x.clone()
    x0[5] = 0
    other = pt.gated_delta_rule(x0.double(), m, w, "mix.", 1e-5)
    assert float((ref[160] - other[160]).abs().max()) > 0.2 * float(ref[160].abs().max())
    out, _ = _run_mixer(mixer, cache, x, (4, 3, 90, 2) + (1,) * 50 + (21,), dtype)
    ops.check_status()
    _close(out, ref, dtype)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_decay_acts_per_head_and_key_channel(dtype):
    """One key channel of one head forgets at once (a large bias of its decay) while all others keep
    nearly everything: swapping the bias to the same channel of the other head, or to the next
    channel, gives another result, and the kernel gives the one of the layout heads x channels."""
    g = torch.Generator().manual_seed(6)
    m = _delta(2, 2, 8, 8, 1, 4, 4)
    at = 1 * 8 + 3  # head 1, channel 3

    def tweak(w, at=at):
        w["mix.A_log"] = torch.zeros(2).bfloat16()
        w["mix.a1"] = torch.zeros_like(w["mix.a1"])
        bias = torch.full((16,), -8.0)
        bias[at] = 6.0
        w["mix.dt_bias"] = bias.bfloat16()
    mixer, cache, w, ops = _delta_alone(m, 32, dtype, g, tweak=tweak)
    x = torch.randn(40, 32, generator=g).to(dtype)
    ref = pt.gated_delta_rule(x.double(), m, w, "mix.", 1e-5)
    for other in (0 * 8 + 3, 1 * 8 + 4):
        w2 = dict(w)
        bias = torch.full((16,), -8.0, dtype=torch.float64)
        bias[other] = 6.0
        w2["mix.dt_bias"] = bias
        alt = pt.gated_delta_rule(x.double(), m, w2, "mix.", 1e-5)
        assert float((alt - ref).abs().max()) > 0.1 * float(ref.abs().max())
    out, _ = _run_mixer(mixer, cache, x, (17, 1, 1, 21), dtype)
    ops.check_status()
    _close(out, ref, dtype)
