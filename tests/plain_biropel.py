"""Biropel, plainly: whole sequences, no cache, one function per mechanism, float64 (or float32) torch on the CPU.

This file shares no code with the package. It takes the config.json dictionary and a dictionary of tensors under
the checkpoint's names, and returns logits [tokens, vocab] (and, if asked, the sum of the streams after every layer).

Notation: T tokens, D width, H query heads, G key/value heads, d the width of a query or key head, e the width of
a value head, N the width of a state-space state, s the number of residual streams. A linear weight W is stored
[out, in]; `lin(W, x)` is x W^T.
"""
from __future__ import annotations

import math
from typing import List, Mapping, Optional, Tuple

import torch
import torch.nn.functional as F


def lin(weight: torch.Tensor, x: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    y = x @ weight.to(x.dtype).t()
    return y + bias.to(x.dtype) if bias is not None else y


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x divided by the root mean square of its last axis, eps under the root."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    return unit_rms(x, eps) * weight.to(x.dtype)


# ------------------------------------------------------------------------------------------------- positions
def frequencies(rot: Mapping) -> Tuple[torch.Tensor, float]:
    """(frequency per pair [dims/2] in float64, factor on cosine and sine). Plain: base^(-2i/n), 1. Stretched:
    pairs that turn often keep their frequency, pairs that turn seldom have it divided by `factor`, a linear
    ramp over the pair index in between; factor 0.1 ln(factor) + 1."""
    n, base = int(rot["dims"]), float(rot["base"])
    index = torch.arange(n // 2, dtype=torch.float64)
    freq = base ** (-2.0 * index / n)
    scaling = rot.get("scaling")
    if not scaling:
        return freq, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def pair_of(turns: float) -> float:
        return n * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(pair_of(float(scaling["slow"]))), n - 1)
    ramp = torch.clamp((index - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return freq / factor * ramp + freq * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x: torch.Tensor, rot: Mapping) -> torch.Tensor:
    """x [T, heads, w]: entry i of the first rot.dims entries is paired with entry i + dims/2 and the pair turned by
    position * frequency; the other entries pass."""
    n = int(rot["dims"])
    half = n // 2
    freq, factor = frequencies(rot)
    angle = torch.arange(x.shape[0], dtype=torch.float64)[:, None] * freq[None, :]
    cos = (torch.cos(angle) * factor).to(x.dtype)[:, None, :]
    sin = (torch.sin(angle) * factor).to(x.dtype)[:, None, :]
    u, v, rest = x[..., :half], x[..., half:n], x[..., n:]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, rest], -1)


def query_temperature(T: int, coef: float, every: int, dtype) -> torch.Tensor:
    """[T]: 1 + coef ln(floor((p + 1) / every) + 1)."""
    p = torch.arange(T, dtype=torch.float64)
    return (1.0 + coef * torch.log(torch.floor((p + 1.0) / every) + 1.0)).to(dtype)


# ------------------------------------------------------------------------------------------------- attention
def visible(T: int, window: Optional[int]) -> torch.Tensor:
    """[T, T] boolean: query i sees key j when 0 <= i - j (and i - j < window where there is one)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    seen = j <= i
    if window is not None:
        seen = seen & (i - j < int(window))
    return seen


def attend(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, mask: torch.Tensor,
           softcap: Optional[float]) -> torch.Tensor:
    """q [T, H, d], k [T, G, d], v [T, G, e] -> [T, H * e]; query head h reads key/value head h // (H / G)."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = []
    for h in range(H):
        g = h // (H // G)
        scores = (q[:, h] @ k[:, g].t()) * scale
        if softcap:
            scores = softcap * torch.tanh(scores / softcap)
        scores = scores.masked_fill(~mask, float("-inf"))
        out.append(torch.softmax(scores, -1) @ v[:, g])
    return torch.cat(out, -1)


def softmax_attention(h: torch.Tensor, tensors: Mapping, prefix: str, mixer: Mapping, eps: float,
                      borrowed=None, biased: bool = False, gated: bool = False, unit_qk: bool = False):
    """The softmax attention of every mixer that has one. Returns (y [T, D], (keys, values)) with the keys as a
    later layer would borrow them: after every change made to them here."""
    T = h.shape[0]
    H, G, d, e = int(mixer["heads"]), int(mixer["kv_heads"]), int(mixer["dim"]), int(mixer["vdim"])
    bias = (lambda name: tensors[prefix + name + ".b"]) if biased else (lambda name: None)
    q = lin(tensors[prefix + "q"], h, bias("q")).reshape(T, H, d)
    rot = mixer.get("rot")
    if borrowed is None:
        k = lin(tensors[prefix + "k"], h, bias("k")).reshape(T, G, d)
        v = lin(tensors[prefix + "v"], h, bias("v")).reshape(T, G, e)
        if unit_qk:
            k = unit_rms(k, eps)
        if rot:
            k = rotate(k, rot)
    else:
        k, v = borrowed
    if unit_qk:
        q = unit_rms(q, eps)
    if rot:
        q = rotate(q, rot)
    temp = mixer.get("q_temp")
    if temp:
        q = q * query_temperature(T, float(temp["coef"]), int(temp["every"]), q.dtype)[:, None, None]
    mask = mixer.get("mask")
    seen = visible(T, int(mask["size"]) if mask else None)
    mixed = attend(q, k, v, float(mixer["scale"]), seen, mixer.get("softcap"))
    if gated:
        mixed = mixed * torch.sigmoid(lin(tensors[prefix + "g"], h))
    return lin(tensors[prefix + "o"], mixed), (k, v)


# ------------------------------------------------------------------------------------------------- recurrences
def causal_conv(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """x [T, C], weight [C, taps] whose last column multiplies the current token; zeros before the start."""
    T, C = x.shape
    taps = weight.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=x.dtype), x], 0)
    y = bias.to(x.dtype)[None, :].expand(T, C).clone()
    for j in range(taps):
        y = y + padded[j:j + T] * weight[:, j].to(x.dtype)[None, :]
    return y


def state_space(h: torch.Tensor, tensors: Mapping, prefix: str, mixer: Mapping, eps: float) -> torch.Tensor:
    """The selective state-space mixer with a scalar decay per head."""
    T = h.shape[0]
    heads, e, N, groups = int(mixer["heads"]), int(mixer["vdim"]), int(mixer["state"]), int(mixer["groups"])
    inner = heads * e
    proj = lin(tensors[prefix + "in"], h)
    z, rest, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * groups * N], proj[:, 2 * inner + 2 * groups * N:]
    rest = F.silu(causal_conv(rest, tensors[prefix + "conv"], tensors[prefix + "conv.b"]))
    x = rest[:, :inner].reshape(T, heads, e)
    B = rest[:, inner:inner + groups * N].reshape(T, groups, N)
    C = rest[:, inner + groups * N:].reshape(T, groups, N)
    dt = F.softplus(dt + tensors[prefix + "dt_bias"].to(h.dtype))
    rate = torch.exp(tensors[prefix + "A_log"].to(h.dtype))
    skip = tensors[prefix + "D"].to(h.dtype)
    y = torch.zeros(T, heads, e, dtype=h.dtype)
    for head in range(heads):
        g = head // (heads // groups)
        S = torch.zeros(N, e, dtype=h.dtype)
        for t in range(T):
            S = torch.exp(-rate[head] * dt[t, head]) * S + dt[t, head] * torch.outer(B[t, g], x[t, head])
            y[t, head] = S.t() @ C[t, g] + skip[head] * x[t, head]
    y = y.reshape(T, inner) * F.silu(z)
    parts = int(mixer["norm_groups"])
    y = unit_rms(y.reshape(T, parts, inner // parts), eps).reshape(T, inner) * tensors[prefix + "norm"].to(h.dtype)
    return lin(tensors[prefix + "o"], y)


def matrix_memory(h: torch.Tensor, tensors: Mapping, prefix: str, mixer: Mapping, eps: float) -> torch.Tensor:
    """The matrix memory with exponential input gates, kept finite by a running maximum of the log gates."""
    T = h.shape[0]
    heads, d, e, cap = int(mixer["heads"]), int(mixer["dim"]), int(mixer["vdim"]), float(mixer["gate_cap"])
    q = (lin(tensors[prefix + "q"], h) * d ** -0.5).reshape(T, heads, d)
    k = lin(tensors[prefix + "k"], h).reshape(T, heads, d)
    v = lin(tensors[prefix + "v"], h).reshape(T, heads, e)
    log_in = cap * torch.tanh(lin(tensors[prefix + "i"], h, tensors[prefix + "i.b"]) / cap)
    log_keep = F.logsigmoid(cap * torch.tanh(lin(tensors[prefix + "f"], h, tensors[prefix + "f.b"]) / cap))
    out = torch.zeros(T, heads, e, dtype=h.dtype)
    for head in range(heads):
        S = torch.zeros(d, e, dtype=h.dtype)
        n = torch.zeros(d, dtype=h.dtype)
        m = torch.zeros((), dtype=h.dtype)
        for t in range(T):
            m_new = torch.maximum(log_keep[t, head] + m, log_in[t, head])
            keep, write = torch.exp(log_keep[t, head] + m - m_new), torch.exp(log_in[t, head] - m_new)
            S = keep * S + write * torch.outer(k[t, head], v[t, head])
            n = keep * n + write * k[t, head]
            m = m_new
            out[t, head] = S.t() @ q[t, head] / (torch.maximum(torch.abs(n @ q[t, head]), torch.exp(-m)) + 1e-6)
    out = unit_rms(out, eps).reshape(T, heads * e) * tensors[prefix + "norm"].to(h.dtype)
    out = out * torch.sigmoid(lin(tensors[prefix + "g"], h))
    return lin(tensors[prefix + "o"], out)


# ------------------------------------------------------------------------------------------------- sublayers
def squared_relu_mlp(h: torch.Tensor, tensors: Mapping, prefix: str) -> torch.Tensor:
    return lin(tensors[prefix + "down"], torch.relu(lin(tensors[prefix + "up"], h)) ** 2)


def mixer_of(layer: Mapping, index: int, h: torch.Tensor, tensors: Mapping, eps: float, kept: List):
    """The layer's mixer on its normalised input; `kept[j]` = (keys, values) that layer j left."""
    prefix = f"l{index}.mix."
    mixer = layer["mixer"]
    kind = layer["type"]
    if kind == "attention":
        source = mixer.get("kv_from")
        y, kv = softmax_attention(h, tensors, prefix, mixer, eps, borrowed=kept[source] if source is not None else None,
                                  biased=True, gated=True)
        kept[index] = kv if source is None else None
        return y
    if kind == "parallel":
        left, _ = softmax_attention(h, tensors, prefix + "left.", mixer["left"], eps)
        right = state_space(h, tensors, prefix + "right.", mixer["right"], eps)
    elif kind == "parallel_2":
        left, _ = softmax_attention(h, tensors, prefix + "left.", mixer["left"], eps, unit_qk=True)
        right = matrix_memory(h, tensors, prefix + "right.", mixer["right"], eps)
    else:
        raise ValueError(f"unknown layer type {kind}")
    return 0.5 * (rms_norm(left, tensors[prefix + "left.out"], eps) + rms_norm(right, tensors[prefix + "right.out"], eps))


def forward(config: Mapping, tensors: Mapping, tokens, dtype=torch.float64, layers_out: Optional[list] = None):
    """Logits [T, vocab]. `layers_out`, a list, receives the sum of the streams after every layer."""
    eps = float(config["norm"]["eps"])
    ids = torch.as_tensor(list(tokens), dtype=torch.long)
    x = rms_norm(tensors["embed"].to(dtype)[ids], tensors["embed.norm"], eps)
    count = config.get("streams")
    streams = [x.clone() for _ in range(int(count))] if count else None
    kept: List = [None] * len(config["layers"])
    for index, layer in enumerate(config["layers"]):
        prefix = f"l{index}."
        sublayers = [("1", lambda h: mixer_of(layer, index, h, tensors, eps, kept))]
        if layer.get("mlp") is not None:
            if layer["mlp"]["kind"] != "dense":
                raise ValueError("unknown feed-forward kind")
            sublayers.append(("2", lambda h: squared_relu_mlp(h, tensors, prefix + "mlp.")))
        for number, sublayer in sublayers:
            norm = tensors[prefix + "norm" + number]
            if streams is None:
                x = x + sublayer(rms_norm(x, norm, eps))
                continue
            read = tensors[f"{prefix}hc{number}.in"].to(dtype)
            write = tensors[f"{prefix}hc{number}.out"].to(dtype)
            mix = tensors[f"{prefix}hc{number}.mix"].to(dtype)       # [from, to]
            y = sublayer(rms_norm(sum(read[s] * streams[s] for s in range(len(streams))), norm, eps))
            streams = [sum(mix[s, t] * streams[s] for s in range(len(streams))) + write[t] * y
                       for t in range(len(streams))]
        if layers_out is not None:
            layers_out.append(sum(streams) if streams is not None else x.clone())
    if streams is not None:
        x = sum(streams)
    return lin(tensors["head"], rms_norm(x, tensors["final.norm"], eps))
