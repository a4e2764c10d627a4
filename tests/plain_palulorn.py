"""A plain, slow implementation of the Palulorn design: whole sequences, no cache, float64 by default.

One function per mechanism, written from the design's equations in this file's own notation and
sharing no code with the package.  ``forward(config, tensors, tokens)`` runs one sequence and
returns the logits of every position (and, on request, the residual stream after every run of a
layer).  ``tensors`` maps checkpoint names to torch tensors.

Notation: ``T`` tokens at positions ``0 .. T-1``; linear weights are stored ``[out, in]``.
"""

from __future__ import annotations

import math
from typing import Dict, List

import torch

DT = torch.float64


def _w(tensors, name):
    return tensors[name].to(DT)


# -- small pieces ---------------------------------------------------------------------------


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def log_sigmoid(z):
    return -softplus(-z)


def time_conv(x, taps, bias=None):
    """``x`` [T, C], ``taps`` [C, K]: ``y[t] = sum_j taps[:, j] x[t - (K-1) + j]``, zeros before the start."""
    k = taps.shape[1]
    padded = torch.cat([torch.zeros(k - 1, x.shape[1], dtype=x.dtype), x], dim=0)
    y = torch.zeros_like(x)
    for j in range(k):
        y = y + padded[j : j + x.shape[0]] * taps[:, j]
    return y if bias is None else y + bias


def turn_halves(x, freqs):
    """``x`` [T, heads, size]; among a head's first ``2P`` dimensions, ``i`` and ``i + P`` of position
    ``p`` turn together by ``p * freqs[i]``."""
    half = freqs.numel()
    ang = torch.arange(x.shape[0], dtype=DT)[:, None, None] * freqs
    c, s = torch.cos(ang), torch.sin(ang)
    a, b = x[..., :half], x[..., half : 2 * half]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., 2 * half :]], dim=-1)


# -- mixers -----------------------------------------------------------------------------------


def sink_attention(h, m, tensors, prefix):
    """Causal attention whose values are its keys, with a per-head sink in the softmax's
    denominator, a query temperature that grows with the position and a per-head output gate."""
    T = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    q = (h @ _w(tensors, prefix + "q").T + _w(tensors, prefix + "q.b")).view(T, H, d)
    k = (h @ _w(tensors, prefix + "k").T + _w(tensors, prefix + "k.b")).view(T, G, d)
    v = k
    qt = m.get("q_temp")
    if qt:
        pos = torch.arange(T, dtype=DT)
        q = q * (1.0 + float(qt["coef"]) * torch.log(torch.floor((pos + 1) / float(qt["every"])) + 1.0))[:, None, None]
    gate = torch.sigmoid(h @ _w(tensors, prefix + "g").T)  # [T, H]
    sink = _w(tensors, prefix + "sink")
    out = torch.zeros(T, H, v.shape[-1], dtype=DT)
    group = H // G
    for head in range(H):
        kh, vh = k[:, head // group], v[:, head // group]
        for i in range(T):
            s = (kh[: i + 1] @ q[i, head]) * float(m["scale"])
            top = torch.maximum(s.max(), sink[head])
            e = torch.exp(s - top)
            out[i, head] = (e @ vh[: i + 1]) / (e.sum() + torch.exp(sink[head] - top))
    out = out * gate[:, :, None]
    return out.reshape(T, -1) @ _w(tensors, prefix + "o").T + _w(tensors, prefix + "o.b")


def matrix_memory(h, m, tensors, prefix, eps):
    """The matrix memory with exponential gates and a running maximum that starts at zero."""
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    cap = float(m["gate_cap"])
    q = (h @ _w(tensors, prefix + "q").T).view(T, H, d) * d ** -0.5
    k = (h @ _w(tensors, prefix + "k").T).view(T, H, d)
    v = (h @ _w(tensors, prefix + "v").T).view(T, H, dv)
    gi = cap * torch.tanh((h @ _w(tensors, prefix + "i").T + _w(tensors, prefix + "i.b")) / cap)
    gf = log_sigmoid(cap * torch.tanh((h @ _w(tensors, prefix + "f").T + _w(tensors, prefix + "f.b")) / cap))
    out = torch.zeros(T, H, dv, dtype=DT)
    for head in range(H):
        S = torch.zeros(d, dv, dtype=DT)
        n = torch.zeros(d, dtype=DT)
        mx = torch.zeros((), dtype=DT)
        for t in range(T):
            new = torch.maximum(gf[t, head] + mx, gi[t, head])
            keep, write = torch.exp(gf[t, head] + mx - new), torch.exp(gi[t, head] - new)
            S = keep * S + write * torch.outer(k[t, head], v[t, head])
            n = keep * n + write * k[t, head]
            mx = new
            den = torch.maximum((n @ q[t, head]).abs(), torch.exp(-mx)) + 1e-6
            out[t, head] = (S.T @ q[t, head]) / den
    out = unit_rms(out, eps).reshape(T, -1) * _w(tensors, prefix + "norm")
    out = out * torch.sigmoid(h @ _w(tensors, prefix + "g").T)
    return out @ _w(tensors, prefix + "o").T


def two_mixers(h, m, tensors, prefix, eps):
    left = sink_attention(h, m["left"], tensors, prefix + "left.")
    right = matrix_memory(h, m["right"], tensors, prefix + "right.", eps)
    left = unit_rms(left, eps) * _w(tensors, prefix + "left.out")
    right = unit_rms(right, eps) * _w(tensors, prefix + "right.out")
    return 0.5 * (left + right)


def gated_linear_recurrence(h, m, tensors, prefix):
    """Two branches; one passes a causal convolution and a per-channel recurrence whose decay and
    input gate come from block-diagonal maps of the convolution's output."""
    T = h.shape[0]
    W, B = m["width"], m["blocks"]
    y = gelu_tanh(h @ _w(tensors, prefix + "y").T + _w(tensors, prefix + "y.b"))
    u = time_conv(h @ _w(tensors, prefix + "x").T + _w(tensors, prefix + "x.b"), _w(tensors, prefix + "conv"),
                  _w(tensors, prefix + "conv.b"))
    ub = u.view(T, B, W // B)
    r = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, _w(tensors, prefix + "ra")) + _w(tensors, prefix + "ra.b"))
    i = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, _w(tensors, prefix + "ri")) + _w(tensors, prefix + "ri.b"))
    r, i = r.reshape(T, W), i.reshape(T, W)
    log_a = -8.0 * r * softplus(_w(tensors, prefix + "lam"))
    a = torch.exp(log_a)
    S = torch.zeros(W, dtype=DT)
    out = torch.zeros(T, W, dtype=DT)
    for t in range(T):
        S = a[t] * S + torch.sqrt(1.0 - a[t] ** 2) * i[t] * u[t]
        out[t] = S
    return (out * y) @ _w(tensors, prefix + "o").T


def window_attention(h, m, tensors, prefix, eps):
    """Grouped-query softmax attention over a sliding window; q, k, v pass a short causal
    convolution, q and k a per-head RMS norm and a partial rotation."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = h @ _w(tensors, prefix + "q").T + _w(tensors, prefix + "q.b")
    k = h @ _w(tensors, prefix + "k").T + _w(tensors, prefix + "k.b")
    v = h @ _w(tensors, prefix + "v").T + _w(tensors, prefix + "v.b")
    if m.get("conv"):
        q = time_conv(q, _w(tensors, prefix + "q.conv"))
        k = time_conv(k, _w(tensors, prefix + "k.conv"))
        v = time_conv(v, _w(tensors, prefix + "v.conv"))
    q = unit_rms(q.view(T, H, d), eps) * _w(tensors, prefix + "q.norm")
    k = unit_rms(k.view(T, G, d), eps) * _w(tensors, prefix + "k.norm")
    v = v.view(T, G, dv)
    rot = m.get("rot")
    if rot:
        dims = int(rot["dims"])
        f = float(rot["base"]) ** (-2.0 * torch.arange(dims // 2, dtype=DT) / dims)
        if rot.get("scaling"):
            f = f / float(rot["scaling"]["factor"])
        q, k = turn_halves(q, f), turn_halves(k, f)
    window = int(m["mask"]["size"]) if m.get("mask") else None
    out = torch.zeros(T, H, dv, dtype=DT)
    group = H // G
    for head in range(H):
        kh, vh = k[:, head // group], v[:, head // group]
        for i in range(T):
            lo = 0 if window is None else max(0, i - window + 1)
            s = (kh[lo : i + 1] @ q[i, head]) * float(m["scale"])
            out[i, head] = torch.softmax(s, dim=0) @ vh[lo : i + 1]
    return out.reshape(T, -1) @ _w(tensors, prefix + "o").T


# -- feed-forward -------------------------------------------------------------------------------


def squared_relu_mlp(h, tensors, prefix):
    return (torch.relu(h @ _w(tensors, prefix + "up").T) ** 2) @ _w(tensors, prefix + "down").T


def routed_experts(h, mlp, tensors, prefix):
    """Sigmoid scores; the experts of the best groups only (a group's score: its two largest scores
    added); the chosen scores divided by their sum and multiplied by the router's scale; a shared
    expert beside them."""
    r = mlp["router"]
    E, top = int(r["experts"]), int(r["top"])
    s = torch.sigmoid(h @ _w(tensors, prefix + "router").T)  # [T, E]
    allowed = torch.ones_like(s, dtype=torch.bool)
    groups = r.get("groups")
    if groups:
        count, keep = int(groups["count"]), int(groups["keep"])
        per = E // count
        g = s.view(-1, count, per)
        gs = g.topk(min(2, per), dim=-1).values.sum(-1)  # [T, count]
        best = gs.topk(keep, dim=-1).indices
        allowed_g = torch.zeros_like(gs, dtype=torch.bool)
        allowed_g.scatter_(1, best, True)
        allowed = allowed_g[:, :, None].expand(-1, -1, per).reshape(-1, E)
    choice = torch.where(allowed, s, torch.full_like(s, -1.0)).topk(top, dim=-1).indices  # [T, top]
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        chosen = s[t, choice[t]]
        weights = chosen / (chosen.sum() + 1e-20) * float(r.get("scale", 1.0))
        for wgt, e in zip(weights, choice[t].tolist()):
            out[t] = out[t] + wgt * squared_relu_mlp(h[t : t + 1], tensors, f"{prefix}e{e}.")[0]
    if mlp.get("shared"):
        out = out + squared_relu_mlp(h, tensors, prefix + "shared.")
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
    x0 = _w(tensors, "embed")[torch.as_tensor(tokens, dtype=torch.long)] * float((config.get("embedding") or {}).get("scale", 1.0))
    x = x0
    after = []
    for i, opens in run_order(config):
        layer = config["layers"][i]
        p = f"l{i}."
        if opens is not None:
            # a pass opens by mixing the stream with the embedding output, then its step vector
            x = torch.cat([x, x0], dim=-1) @ _w(tensors, "loop.in").T + _w(tensors, "loop.step")[opens]
        h = unit_rms(x, eps) * _w(tensors, p + "norm1")
        kind, m = layer["type"], layer["mixer"]
        if kind == "parallel":
            mixed = two_mixers(h, m, tensors, p + "mix.", eps)
        elif kind == "rglru":
            mixed = gated_linear_recurrence(h, m, tensors, p + "mix.")
        elif kind == "attention":
            mixed = window_attention(h, m, tensors, p + "mix.", eps)
        else:
            raise ValueError(kind)
        x = x + mixed
        mlp = layer.get("mlp")
        if mlp is not None:
            x = x + routed_experts(unit_rms(x, eps) * _w(tensors, p + "norm2"), mlp, tensors, p + "mlp.")
        after.append(x.clone())
    h = unit_rms(x, eps) * _w(tensors, "final.norm")
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
