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
# tap (no inputs to keep); a delta rule of one head (a state of one column is in the rule's own test:
# its norm is a sign, which no rounding survives); heads that rotate whole
TB = dict(
    architecture="Tanupel", vocab=97, width=64, norm=dict(eps=1e-6),
    layers=[
        _layer("parallel", _pair(_attn(2, 2, 16, 16, 0.25, dims=16, base=777.0, scaling=(1.5,), softcap=50.0),
                                 _delta(1, 1, 33, 5, 1, 3, 1), 1.0, 1.0), _moe(1, 1, 56)),
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


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sizes", [
    # heads, key/value heads, key size, value size, scale, turned dimensions, base, scaling, cap, divide
    (6, 3, 16, 32, 0.2, 8, 5000.0, (8.0, 1.0, 4.0, 64), None, False),
    (4, 2, 32, 16, 0.15, 32, 1e4, (2.0,), 5.0, True),
    (4, 2, 32, 16, 0.15, 16, 1e4, (2.0, 1.0, 4.0, 64), 5.0, True),   # a pair's attention divides all the same
    (2, 1, 48, 48, 0.12, 24, 300.0, None, None, False),
    (1, 1, 64, 64, 0.1, 2, 50.0, (3.0,), 1.0, True),
    (5, 1, 16, 32, 0.2, 16, 1e4, (2.0,), 8.0, True),
    (2, 2, 80, 16, 0.11, 40, 2000.0, (2.0, 1.0, 8.0, 32), None, False),
    (3, 3, 24, 24, 0.3, None, 1.0, None, 2.0, False),                # no positions at all
    (4, 2, 64, 64, 0.12, 32, 1e4, (2.0,), 3.0, True),                # capped, at the head sizes of the tcgen05 kernel
    (2, 1, 128, 128, 0.09, 64, 1e4, (2.0,), 4.0, True),
    (2, 2, 128, 64, 0.09, 128, 5e5, (4.0, 1.0, 4.0, 32), None, False),
])
def test_attention_alone(dtype, sizes):
    """Queries and keys normed over the whole projection, a part of each head turned (dimension i
    with dimension i + half), frequencies bent by wavelength, divided or left, scores capped or
    not, value heads larger and smaller than key heads: a portion, single tokens and short
    portions across pages of eight; then the pages are freed and taken again."""
    from fastgen_b200.config.tanupel import _attention
    from fastgen_b200.cache import CacheManager
    from fastgen_b200.parts import make_mixer

    heads, kv, d, dv, scale, dims, base, scaling, cap, divide = sizes
    g = torch.Generator().manual_seed(heads * 100 + d)
    m = _attn(heads, kv, d, dv, scale, dims=dims, base=base, scaling=scaling, softcap=cap)
    ops = _ops(dtype)
    mixer = make_mixer(_attention(40, 1e-5, m, "mix.", "test", by_wavelength=not divide))
    w = _draw_all(mixer, g, 0.3, None)
    mixer.bind({local: w[name].to(DEV) for local, name in mixer.names.items()}, ops)
    cache = CacheManager([mixer.cache_spec()], [mixer.state_spec()], [None], 8, 16, 2, 128, dtype=dtype, device=DEV,
                         tensor_map_factory=ops.make_kv_tensor_maps)
    w = {k: v.double() for k, v in w.items()}
    x = torch.randn(75, 40, generator=g).to(dtype)
    ref = pt.softmax_attention(x.double(), m, w, "mix.", 1e-5, linear_scaling=divide)
    if scaling and len(scaling) == 4:
        alt = pt.softmax_attention(x.double(), m, w, "mix.", 1e-5, linear_scaling=not divide)
        assert float((alt - ref).abs().max()) > 0.02 * float(ref.abs().max())
    out, req = _run_mixer(mixer, cache, x, (33, 1, 1, 7, 1, 2, 3, 1, 26), dtype)
    ops.check_status()
    _close(out, ref, dtype)
    cache.release("r")
    out2, _ = _run_mixer(mixer, cache, x[:30], (2, 1, 27), dtype, rid="again")
    _close(out2, ref[:30], dtype, float(ref.abs().max()))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("mode", ["prompt", "decoded"])
@pytest.mark.parametrize("d", [16, 64])
def test_far_key_shows_through_the_cap(dtype, mode, d):
    """One key 400 positions back has a score far above all others, through a dimension that is not
    turned.  Capped, it takes about half of the weight; uncapped it would take all of it, and
    without the key the output is another one: in a prompt portion and for tokens decoded alone,
    with the key on the first of many pages."""
    from fastgen_b200.config.tanupel import _attention

    heads, kv, n, cap = 2, 1, 420, 6.0
    g = torch.Generator().manual_seed(21)
    m = _attn(heads, kv, d, d, 3.0, dims=8, base=1e4, scaling=(2.0,), softcap=cap)

    def tweak(w):
        for h in range(heads):
            w["mix.q"][h * d + d - 1, :] = 0
            w["mix.q"][h * d + d - 1, 0] = 4.0
        w["mix.k"][d - 1, :] = 0
        w["mix.k"][d - 1, 1] = 4.0
        w["mix.q.norm"][:] = 1.0
        w["mix.k.norm"][:] = 1.0
    mixer, cache, w, ops = _mixer_and_cache("attention", m, 24, dtype, g, page=16, n_pages=32, std=0.05, tweak=tweak)
    x = 0.3 * torch.randn(n, 24, generator=g)
    x[:, :2] = 0.0
    far, q1, q2 = 3, n - 1, n - 40
    x[far, 1] = 3.0
    x[q1, 0] = x[q2, 0] = 3.0
    x = x.to(dtype)
    ref = pt.softmax_attention(x.double(), m, w, "mix.", 1e-5, False)
    x0 = x.clone()
    x0[far] = 0
    without = pt.softmax_attention(x0.double(), m, w, "mix.", 1e-5, False)
    uncapped = pt.softmax_attention(x.double(), dict(m, softcap=None), w, "mix.", 1e-5, False)
    for q in (q1, q2):
        scale = float(ref[q].abs().max())
        assert float((ref[q] - without[q]).abs().max()) > 0.15 * scale
        assert float((ref[q] - uncapped[q]).abs().max()) > 0.15 * scale
    out, _ = _run_mixer(mixer, cache, x, (300, 120) if mode == "prompt" else (300, 70) + (1,) * 50, dtype)
    ops.check_status()
    for q in (q1, q2):
        assert float((out[q] - ref[q]).abs().max()) <= _tol(dtype) * float(ref[q].abs().max()), q
    _close(out, ref, dtype)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_keys_at_page_borders(dtype):
    """The only keys that matter sit on the last place of a page and the first of the next; the
    queries come as portions that end and start there, and as single tokens."""
    g = torch.Generator().manual_seed(23)
    d = 16
    m = _attn(2, 2, d, d, 2.5, dims=4, base=100.0)

    def tweak(w):
        for h in range(2):
            for t in ("mix.q", "mix.k"):
                w[t][h * d + d - 1, :] = 0
                w[t][h * d + d - 1, 0] = 4.0
        w["mix.q.norm"][:] = 1.0
        w["mix.k.norm"][:] = 1.0
    mixer, cache, w, ops = _mixer_and_cache("attention", m, 24, dtype, g, page=8, n_pages=16, std=0.05, tweak=tweak)
    x = 0.3 * torch.randn(64, 24, generator=g)
    x[:, 0] = 0.0
    for i in (7, 8, 31, 32, 40, 47, 48, 63):
        x[i, 0] = 3.0
    x = x.to(dtype)
    ref = pt.softmax_attention(x.double(), m, w, "mix.", 1e-5, False)
    for portions in ((8, 24, 8, 7, 1, 16), (7, 1, 1, 23) + (1,) * 32, (64,)):
        out, _ = _run_mixer(mixer, cache, x, portions, dtype)
        ops.check_status()
        _close(out, ref, dtype)
        cache.release("r")


def _feed_forward_alone(mlp, dim, dtype, g, std=0.3, tweak=None):
    from fastgen_b200.config.tanupel import _feed_forward
    from fastgen_b200.parts import make_feed_forward

    ops = _ops(dtype)
    ff = make_feed_forward(_feed_forward(dim, mlp, "mlp.", "test"))
    w = _draw_all(ff, g, std, tweak)
    ff.bind({local: w[name].to(DEV) for local, name in ff.names.items()}, ops)
    return ff, {k: v.double() for k, v in w.items()}, ops


def _clear_choices(x, mlp, w, margin):
    """Tokens whose last chosen expert leads the best one left out by more than ``margin``."""
    s = torch.softmax(x @ w["mlp.router"].T, dim=-1)
    c = torch.sort(s + w["mlp.correction"], dim=-1, descending=True).values
    top = mlp["router"]["top"]
    if top == c.shape[1]:
        return torch.ones(x.shape[0], dtype=torch.bool)
    return (c[:, top - 1] - c[:, top]) > margin


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sizes", [(5, 3, 40), (7, 1, 24), (1, 1, 56), (3, 3, 32), (12, 2, 96), (9, 4, 8), (33, 5, 16),
                                   (64, 8, 24)])
@pytest.mark.parametrize("tokens", [1, 3, 70, 600])
def test_routed_experts_alone(dtype, sizes, tokens):
    """Softmax over all experts in float32, the choice by score plus correction, the weights by
    the score alone and not renormalized; one expert, all experts, more experts than a warp has
    lanes; one token, a few, more tokens than experts, and a prompt's worth (whose products in
    bfloat16 are the grouped ones over the experts' gathered rows, some experts without a row)."""
    experts, top, ff = sizes
    g = torch.Generator().manual_seed(experts * 10 + top)
    mlp = _moe(experts, top, ff)
    part, w, ops = _feed_forward_alone(mlp, 48, dtype, g)
    x = torch.randn(tokens, 48, generator=g).to(dtype)
    ref = pt.routed_experts(x.double(), mlp, w, "mlp.")
    out = _value(part.forward(x.to(DEV), _context(0, 0, tokens))).cpu()
    ops.check_status()
    ok = _clear_choices(x.double(), mlp, w, 1e-5)  # both see the same rounded input: float32 sums are that close
    assert int(ok.sum()) >= (tokens * 2 + 2) // 3
    _close(out[ok], ref[ok], dtype, float(ref.abs().max()))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_the_correction_chooses_and_does_not_weigh(dtype):
    """A correction that lifts the expert with the smallest score into the choice: the output is
    that expert's, weighted by its small score; adding the correction to the weight, dividing by
    the chosen scores' sum, or choosing by the score alone would each give another output."""
    g = torch.Generator().manual_seed(31)
    experts, top = 6, 2
    mlp = _moe(experts, top, 32)

    def tweak(w):
        w["mlp.router"] = (0.2 * torch.randn(experts, 48, generator=g)).bfloat16()
        w["mlp.router"][4] = -w["mlp.router"][0]      # expert 4 scores low where expert 0 scores high
        corr = torch.zeros(experts)
        corr[4] = 5.0
        w["mlp.correction"] = corr.bfloat16()
    part, w, ops = _feed_forward_alone(mlp, 48, dtype, g, tweak=tweak)
    x = torch.randn(40, 48, generator=g).to(dtype)
    xd = x.double()
    ref = pt.routed_experts(xd, mlp, w, "mlp.")
    s = torch.softmax(xd @ w["mlp.router"].T, dim=-1)
    choice = torch.topk(s + w["mlp.correction"], top, dim=-1).indices
    assert bool((choice == 4).any(dim=-1).all())

    def expert(e, rows):
        a = rows @ w[f"mlp.e{e}.gate"].T
        return (pt.silu(a) * (rows @ w[f"mlp.e{e}.up"].T)) @ w[f"mlp.e{e}.down"].T
    others = []
    for how in ("corrected weight", "renormalized", "score alone"):
        alt = torch.zeros_like(ref)
        for t in range(40):
            ids = torch.topk(s[t], top).indices if how == "score alone" else choice[t]
            wts = s[t, ids]
            if how == "corrected weight":
                wts = wts + w["mlp.correction"][ids]
            if how == "renormalized":
                wts = wts / wts.sum()
            alt[t] = sum(wt * expert(int(e), xd[t:t + 1])[0] for e, wt in zip(ids, wts))
        others.append(alt)
        assert float((alt - ref).abs().max()) > 0.2 * float(ref.abs().max()), how
    out = _value(part.forward(x.to(DEV), _context(0, 0, 40))).cpu()
    ops.check_status()
    ok = _clear_choices(xd, mlp, w, 1e-5)
    _close(out[ok], ref[ok], dtype, float(ref.abs().max()))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_two_mixers_side_by_side(dtype):
    """Both halves read the same input; the sum takes each half with its own scale; the attention
    of the pair has the pages, the delta rule the slot's state."""
    g = torch.Generator().manual_seed(41)
    m = _pair(_attn(4, 2, 32, 16, 0.15, dims=16, base=1e4, scaling=(2.0, 1.0, 4.0, 64), softcap=5.0),
              _delta(4, 2, 24, 40, 3, 8, 12), 0.7, 1.3)
    mixer, cache, w, ops = _mixer_and_cache("parallel", m, 56, dtype, g, std=0.25)
    x = torch.randn(50, 56, generator=g).to(dtype)
    ref = pt.two_mixers(x.double(), m, w, "mix.", 1e-5)
    left = pt.softmax_attention(x.double(), m["left"], w, "mix.left.", 1e-5, True)
    right = pt.gated_delta_rule(x.double(), m["right"], w, "mix.right.", 1e-5)
    assert float((ref - (0.7 * left + 1.3 * right)).abs().max()) < 1e-9
    assert float((ref - (left + right)).abs().max()) > 0.05 * float(ref.abs().max())
    out, _ = _run_mixer(mixer, cache, x, (20, 1, 1, 2, 5, 1, 20), dtype)
    ops.check_status()
    _close(out, ref, dtype)


# ---------------------------------------------------------------------------------
# whole models through the engine
# ---------------------------------------------------------------------------------
def model_dir(tmp_path, name, dtype):
    """The model folder of a configuration.  In bfloat16 the engine's activations differ from the
    plain implementation's by a percent, which turns a token's choice of experts wherever two
    choice scores are that close, so the folder of the bfloat16 runs gets corrections two apart
    (scores lie between 0 and 1): there every token takes the same experts, with weights of its
    own.  Choices that depend on the token are held in float32, and in bfloat16 by
    ``test_routed_experts_alone``."""
    from safetensors.torch import load_file, save_file

    if dtype == torch.float32:
        return make_dir(tmp_path, name)
    d = make_dir(Path(tmp_path) / "apart", name)
    f = Path(d) / "model.safetensors"
    tensors = load_file(str(f))
    g = torch.Generator().manual_seed(CONFIGS[name][1])
    for key in [k for k in tensors if k.endswith(".correction")]:
        n = tensors[key].numel()
        tensors[key] = (2.0 * torch.randperm(n, generator=g)).to(tensors[key].dtype)
    save_file(tensors, str(f))
    return d


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("name", ["ta", "tb", "tc", "td"])
@pytest.mark.parametrize("plan", ["whole", "decode", "portions", "mixed"])
def test_replay(tmp_path, name, dtype, plan):
    """Whole prompts (of one and two tokens too), prompts with a decoded tail, portions of 2 to 17
    tokens, and mixed batches of up to four requests whose pages and slots are used again, all
    against the plain implementation run on whole sequences."""
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
@pytest.mark.parametrize("name", ["ta", "tc"])
def test_batching_changes_nothing(tmp_path, dtype, name):
    """A request's logits in a batch of unequal requests equal those it gets alone (bitwise in
    float32, where every sum has a fixed order; within rounding in bfloat16)."""
    d = model_dir(tmp_path, name, dtype)
    requests = _requests(CONFIGS[name][0]["vocab"], [41, 5, 77, 20], 60)
    alone = H.plan_portions(requests, sizes=(9, 1, 1, 30))
    out_a, _ = H.run_engine(d, dtype, alone, 8, H.max_live_tokens(alone, 8) + 32)
    got_a = H.collect(alone, out_a)
    mixed = H.plan_mixed(requests, seed=2)
    out_m, _ = H.run_engine(d, dtype, mixed, 8, H.max_live_tokens(mixed, 8) + 32)
    got_m = H.collect(mixed, out_m)
    for rid, toks in requests.items():
        for p in range(len(toks)):
            if dtype == torch.float32:
                assert np.array_equal(got_a[rid][p], got_m[rid][p]), (rid, p)
            else:
                check_row(got_m[rid][p], got_a[rid][p], dtype, f"{rid} {p}")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("name", ["ta", "tc"])
def test_steps_replayed_from_graphs_change_nothing(tmp_path, dtype, name):
    """Steps captured as CUDA graphs (single tokens, and prompt portions padded to a few shapes)
    give what the same steps give launched kernel by kernel: states and convolution inputs are
    advanced by the replays only, never by a capture, and padding lanes choose no expert."""
    d = model_dir(tmp_path, name, dtype)
    requests = _requests(CONFIGS[name][0]["vocab"], [41, 5, 77, 20], 61)
    mixed = H.plan_mixed(requests, seed=3)
    room = H.max_live_tokens(mixed, 8) + 32
    out_g, eng = H.run_engine(d, dtype, mixed, 8, room, max_step_tokens=64)
    assert eng.graphs is not None and eng.step_graphs is not None and eng.step_graphs.replays > 0
    out_p, _ = H.run_engine(d, dtype, mixed, 8, room, num_cuda_graphs=0)
    got_g, got_p = H.collect(mixed, out_g), H.collect(mixed, out_p)
    for rid, toks in requests.items():
        for p in range(len(toks)):
            if dtype == torch.float32:
                assert np.array_equal(got_g[rid][p], got_p[rid][p]), (rid, p)
            else:
                check_row(got_g[rid][p], got_p[rid][p], dtype, f"{rid} {p}")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_long_decoding(tmp_path, dtype):
    """200 tokens decoded one by one after a two-token prompt, over many pages of eight: every
    pass's cache grows by itself and every pass's state is carried."""
    d = model_dir(tmp_path, "ta", dtype)
    requests = _requests(211, [202], 77)
    steps = H.plan_decode_tail(requests, 200)
    outputs, engine = H.run_engine(d, dtype, steps, 8, 232)
    compare(d, requests, H.collect(steps, outputs), dtype)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("name", ["ta", "td"])
def test_slots_used_again_start_from_zero(tmp_path, dtype, name):
    """Two slots only: six requests pass through them one after the other, some ending in the
    middle of a step of the others; a state or a convolution input left by a slot's earlier
    request would show in the first tokens of the next."""
    d = model_dir(tmp_path, name, dtype)
    requests = _requests(CONFIGS[name][0]["vocab"], [30, 9, 41, 3, 26, 12], 81)
    steps = H.plan_mixed(requests, seed=7, max_live=2)
    outputs, engine = H.run_engine(d, dtype, steps, 8, H.max_live_tokens(steps, 8) + 16, max_requests=2)
    compare(d, requests, H.collect(steps, outputs), dtype)
    assert engine.cache.n_live == 0


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("name", ["ta", "tc"])
def test_greedy_generation_through_the_entry_point(tmp_path, dtype, name):
    """``Fastgen.generate`` with its scheduler (portions of 16 tokens, batches of 3, graphs)
    against greedy decoding with the plain implementation."""
    from fastgen_b200.engine import Fastgen, GenArgs, HfLoader, Packet

    d = model_dir(tmp_path, name, dtype)
    cfg, w = pt.read_model(d)
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
            assert got[i] == pt.greedy(cfg, w, p, 12), i
        else:
            seq = list(p)
            for tok in got[i]:
                logits = pt.forward(cfg, w, seq)[-1]
                assert float(logits[tok]) >= float(logits.max()) - 0.03 * float(logits.abs().max())
                seq.append(tok)
