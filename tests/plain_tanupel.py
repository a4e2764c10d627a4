"""A plain, slow implementation of the Tanupel design: whole sequences, no cache, float64 by default.

One function per mechanism, written from the design's equations in this file's own notation
and sharing no code with the package.  ``forward(config, tensors, tokens)`` runs one sequence
and returns the logits of every position (and, on request, the residual stream after every
run of a layer).  ``tensors`` maps checkpoint names to torch tensors.

Notation: ``T`` tokens, positions ``0 .. T-1``; linear weights are stored ``[out, in]``.
"""

from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

DT = torch.float64


def _w(tensors, name):
    return tensors[name].to(DT)


# -- small pieces ---------------------------------------------------------------------------


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def rotary_frequencies(base: float, dims: int, scaling: Optional[dict]) -> torch.Tensor:
    """Frequencies of the ``dims/2`` pairs.  A scaling with ``low``/``high``/``original`` bends the
    long wavelengths (kept below ``original/high``, divided by ``factor`` above ``original/low``,
    blended in between); one with ``factor`` alone divides every frequency."""
    i = torch.arange(dims // 2, dtype=DT)
    f = base ** (-2.0 * i / dims)
    if not scaling:
        return f
    factor = float(scaling["factor"])
    if "original" not in scaling:
        return f / factor
    orig, low, high = float(scaling["original"]), float(scaling["low"]), float(scaling["high"])
    out = f.clone()
    for n in range(f.numel()):
        wavelength = 2 * math.pi / float(f[n])
        if wavelength < orig / high:
            continue
        if wavelength > orig / low:
            out[n] = f[n] / factor
        else:
            s = (orig / wavelength - low) / (high - low)
            out[n] = (1 - s) * f[n] / factor + s * f[n]
    return out


def rotate_halves(x, positions, freqs):
    """``x`` [T, heads, size]: among a head's first ``2P`` dimensions, dimension ``i`` and dimension
    ``i + P`` of position ``p`` turn together by ``p * freqs[i]``; the others stay."""
    half = freqs.numel()
    ang = positions.to(DT)[:, None, None] * freqs
    c, s = torch.cos(ang), torch.sin(ang)
    a, b = x[..., :half], x[..., half : 2 * half]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., 2 * half :]], dim=-1)


def causal_conv(x, taps):
    """``x`` [T, C], ``taps`` [C, K]: ``y[t] = sum_j taps[:, K-1-j] x[t-j]`` with zeros before the start."""
    t, k = x.shape[0], taps.shape[1]
    padded = torch.cat([torch.zeros(k - 1, x.shape[1], dtype=x.dtype), x], dim=0)
    y = torch.zeros_like(x)
    for j in range(k):
        y = y + padded[j : j + t] * taps[:, j]
    return y


# -- mixers -----------------------------------------------------------------------------------


def softmax_attention(h, m, tensors, prefix, eps, linear_scaling: bool):
    """Grouped-query causal softmax attention; queries and keys are RMS-normed over the whole
    projection (all heads at once) before they are rotated; with ``softcap`` a score ``s`` becomes
    ``cap * tanh(s / cap)``."""
    t = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = h @ _w(tensors, prefix + "q").T
    k = h @ _w(tensors, prefix + "k").T
    v = h @ _w(tensors, prefix + "v").T
    q = unit_rms(q, eps) * _w(tensors, prefix + "q.norm")
    k = unit_rms(k, eps) * _w(tensors, prefix + "k.norm")
    rot = m.get("rot")
    q, k, v = q.reshape(t, H, d), k.reshape(t, G, d), v.reshape(t, G, dv)
    if rot:
        scaling = rot.get("scaling")
        if linear_scaling and scaling:
            scaling = {"factor": scaling["factor"]}
        f = rotary_frequencies(float(rot["base"]), int(rot["dims"]), scaling)
        pos = torch.arange(t)
        q, k = rotate_halves(q, pos, f), rotate_halves(k, pos, f)
    group = H // G
    cap = m.get("softcap")
    i = torch.arange(t)
    seen = i[None, :] <= i[:, None]
    outs = []
    for head in range(H):
        g = head // group
        s = (q[:, head] @ k[:, g].T) * float(m["scale"])
        if cap:
            s = float(cap) * torch.tanh(s / float(cap))
        s = s.masked_fill(~seen, float("-inf"))
        outs.append(torch.softmax(s, dim=-1) @ v[:, g])
    o = torch.cat(outs, dim=-1)
    return o @ _w(tensors, prefix + "o").T


def gated_delta_rule(h, m, tensors, prefix, eps):
    """A matrix state per head that forgets per key channel and is corrected towards the new value:
    ``S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q``."""
    t = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(h @ _w(tensors, prefix + "q").T, _w(tensors, prefix + "q.conv"))).reshape(t, G, d)
    k = silu(causal_conv(h @ _w(tensors, prefix + "k").T, _w(tensors, prefix + "k.conv"))).reshape(t, G, d)
    v = silu(causal_conv(h @ _w(tensors, prefix + "v").T, _w(tensors, prefix + "v.conv"))).reshape(t, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ _w(tensors, prefix + "b").T)  # [T, H]
    a = (h @ _w(tensors, prefix + "a1").T) @ _w(tensors, prefix + "a2").T + _w(tensors, prefix + "dt_bias")
    rate = torch.exp(_w(tensors, prefix + "A_log"))  # [H]
    g = torch.exp(-rate[None, :, None] * softplus(a).reshape(t, H, d))  # [T, H, d]
    gate = torch.sigmoid((h @ _w(tensors, prefix + "g1").T) @ _w(tensors, prefix + "g2").T).reshape(t, H, dv)
    group = H // G
    out = torch.zeros(t, H, dv, dtype=DT)
    for head in range(H):
        j = head // group
        S = torch.zeros(d, dv, dtype=DT)
        for n in range(t):
            S = g[n, head][:, None] * S
            u = beta[n, head] * (v[n, head] - S.T @ k[n, j])
            S = S + torch.outer(k[n, j], u)
            out[n, head] = S.T @ q[n, j]
    out = unit_rms(out, eps) * _w(tensors, prefix + "norm") * gate
    return out.reshape(t, H * dv) @ _w(tensors, prefix + "o").T


def two_mixers(h, m, tensors, prefix, eps):
    left = softmax_attention(h, m["left"], tensors, prefix + "left.", eps, linear_scaling=True)
    right = gated_delta_rule(h, m["right"], tensors, prefix + "right.", eps)
    return float(m["left_scale"]) * left + float(m["right_scale"]) * right


# -- feed-forwards ----------------------------------------------------------------------------


def gated_mlp(h, tensors, prefix):
    return (silu(h @ _w(tensors, prefix + "gate").T) * (h @ _w(tensors, prefix + "up").T)) @ _w(tensors, prefix + "down").T


def routed_experts(h, mlp, tensors, prefix):
    """Every token goes through its ``top`` experts: those with the largest ``softmax(router) +
    correction``; an expert's weight is its softmax score itself, not renormalised."""
    n, top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
    s = torch.softmax(h @ _w(tensors, prefix + "router").T, dim=-1)
    choice = s + _w(tensors, prefix + "correction")
    picked = torch.topk(choice, top, dim=-1).indices  # [T, top]
    out = torch.zeros_like(h)
    for e in range(n):
        y = gated_mlp(h, tensors, f"{prefix}e{e}.")
        weight = (s[:, e : e + 1] * (picked == e).any(-1, keepdim=True))
        out = out + weight * y
    return out


# -- the model --------------------------------------------------------------------------------


def run_order(config) -> List[tuple]:
    """(layer, number of the pass it opens or None) in the order the layers run."""
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    start, stop, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    order = [(i, None) for i in range(start)]
    for p in range(times):
        order += [(i, p if i == start else None) for i in range(start, stop)]
    return order + [(i, None) for i in range(stop, n)]


def forward(config, tensors: Dict[str, torch.Tensor], tokens, return_layers: bool = False):
    eps = float(config["norm"]["eps"])
    mult = float(config.get("residual_mult", 1.0))
    x = _w(tensors, "embed")[torch.as_tensor(tokens, dtype=torch.long)] * float((config.get("embedding") or {}).get("scale", 1.0))
    after = []
    for i, opens in run_order(config):
        layer = config["layers"][i]
        p = f"l{i}."
        if opens is not None:
            x = x + _w(tensors, "loop.step")[opens]
        h = unit_rms(x, eps) * (1.0 + _w(tensors, p + "norm1"))
        if layer["type"] == "attention":
            mixed = softmax_attention(h, layer["mixer"], tensors, p + "mix.", eps, linear_scaling=False)
        elif layer["type"] == "parallel":
            mixed = two_mixers(h, layer["mixer"], tensors, p + "mix.", eps)
        else:
            raise ValueError(layer["type"])
        mlp = layer.get("mlp")
        ff = 0.0
        if mlp is not None:
            ff = gated_mlp(h, tensors, p + "mlp.") if mlp["kind"] == "dense" else routed_experts(h, mlp, tensors, p + "mlp.")
        x = x + mult * (mixed + ff)
        after.append(x.clone())
    h = unit_rms(x, eps) * (1.0 + _w(tensors, "final.norm"))
    logits = h @ _w(tensors, "head").T
    if return_layers:
        return logits, torch.stack(after)
    return logits


def read_model(model_dir, dtype=DT):
    """``(config, tensors)`` of a model folder."""
    import json
    from pathlib import Path

    from safetensors.torch import load_file

    with open(Path(model_dir) / "config.json") as f:
        config = json.load(f)
    tensors = {k: v.to(dtype) for k, v in load_file(str(Path(model_dir) / "model.safetensors")).items()}
    return config, tensors


def greedy(config, tensors, prompt, n_new: int):
    seq, out = list(prompt), []
    for _ in range(n_new):
        tok = int(forward(config, tensors, seq)[-1].argmax())
        out.append(tok)
        seq.append(tok)
    return out
