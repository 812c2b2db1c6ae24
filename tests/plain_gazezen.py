"""Gazezen, plainly: whole sequences, no cache, one function per mechanism, float64 or float32 torch on the CPU.

This file shares no code with the package. It takes the config.json dictionary and a dictionary of tensors under
the checkpoint's names, and returns logits [tokens, vocab] (and, if asked, the stream after every layer run).

Notation: T tokens, D width, H query heads, G key/value heads, d the width of a query or key head, e the width
of a value head, r the width of the cached latent, p the width of the rotated part. A linear weight W is stored
[out, in]; `lin(W, x)` is x W^T.
"""
from __future__ import annotations

import math
from typing import List, Mapping, Optional

import torch


def lin(weight: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    return x @ weight.to(x.dtype).t()


def centred_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """(x - mean) / sqrt(mean of squared deviations + eps) * weight; no bias."""
    centred = x - x.mean(-1, keepdim=True)
    return centred / torch.sqrt((centred * centred).mean(-1, keepdim=True) + eps) * weight.to(x.dtype)


def rms_weighted(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * weight.to(x.dtype)


def frequencies(rot: Mapping, dtype) -> (torch.Tensor, float):
    """The rotation's frequency per pair and the factor on cosine and sine. Without `scaling`: base^(-2i/n) and 1.
    With it, frequencies of slow pairs are divided by `factor`, fast pairs keep theirs, and a ramp blends between."""
    n, base = int(rot["dims"]), float(rot["base"])
    index = torch.arange(n // 2, dtype=torch.float64)
    freq = base ** (-2.0 * index / n)
    scaling = rot.get("scaling")
    if not scaling:
        return freq.to(dtype), 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def turn_dim(turns: float) -> float:
        return n * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(turn_dim(float(scaling["fast"]))), 0)
    hi = min(math.ceil(turn_dim(float(scaling["slow"]))), n - 1)
    ramp = torch.clamp((index - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    freq = freq / factor * ramp + freq * (1.0 - ramp)
    return freq.to(dtype), 0.1 * math.log(factor) + 1.0


def rotate(x: torch.Tensor, rot: Mapping) -> torch.Tensor:
    """x [T, ..., w]: the first rot.dims entries of the last axis are turned by the token's position (entry i is
    paired with entry i + dims/2); the rest pass."""
    n = int(rot["dims"])
    half = n // 2
    freq, factor = frequencies(rot, x.dtype)
    T = x.shape[0]
    angle = torch.arange(T, dtype=x.dtype)[:, None] * freq[None, :]
    shape = [T] + [1] * (x.dim() - 2) + [half]
    cos, sin = (torch.cos(angle) * factor).reshape(shape), (torch.sin(angle) * factor).reshape(shape)
    u, v, rest = x[..., :half], x[..., half:n], x[..., n:]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, rest], -1)


def window_mask(T: int, size: Optional[int]) -> torch.Tensor:
    """[T, T] boolean: query i sees key j when 0 <= i - j (< size, if there is one)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    seen = j <= i
    if size is not None:
        seen = seen & (i - j < int(size))
    return seen


def softmax_rows(scores: torch.Tensor, mask: torch.Tensor, sink: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Softmax over the visible keys; with `sink` (a number) the denominator also holds exp(sink)."""
    scores = scores.masked_fill(~mask, float("-inf"))
    if sink is None:
        return torch.softmax(scores, -1)
    top = torch.maximum(scores.max(-1, keepdim=True).values, sink)
    weights = torch.exp(scores - top)
    return weights / (weights.sum(-1, keepdim=True) + torch.exp(sink - top))


def attention(h: torch.Tensor, w: Mapping[str, torch.Tensor], prefix: str, mixer: Mapping) -> torch.Tensor:
    T = h.shape[0]
    H, G, d, e = mixer["heads"], mixer["kv_heads"], mixer["dim"], mixer["vdim"]
    q = lin(w[prefix + "q"], h).reshape(T, H, d)
    k = lin(w[prefix + "k"], h).reshape(T, G, d)
    v = lin(w[prefix + "v"], h).reshape(T, G, e)
    if mixer.get("rot"):
        q, k = rotate(q, mixer["rot"]), rotate(k, mixer["rot"])
    mask = window_mask(T, (mixer.get("mask") or {}).get("size"))
    gate = torch.sigmoid(lin(w[prefix + "g"], h))                    # [T, H]
    heads = []
    for head in range(H):
        g = head // (H // G)
        sink = w[prefix + "sink"][head].to(h.dtype) if prefix + "sink" in w else None
        weights = softmax_rows((q[:, head] @ k[:, g].t()) * float(mixer["scale"]), mask, sink)
        heads.append((weights @ v[:, g]) * gate[:, head:head + 1])
    return lin(w[prefix + "o"], torch.cat(heads, -1))


def latent_attention(h: torch.Tensor, w: Mapping[str, torch.Tensor], prefix: str, mixer: Mapping, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, d, p, e, r = mixer["heads"], mixer["dim"], mixer["rot_dim"], mixer["vdim"], mixer["kv_rank"]
    q = lin(w[prefix + "q"], h).reshape(T, H, d + p)
    down = lin(w[prefix + "dkv"], h)
    latent = rms_weighted(down[:, :r], w[prefix + "dkv.norm"], eps)
    shared_key = rotate(down[:, r:], mixer["rot"])                   # [T, p], one for all heads
    q_plain, q_rot = q[..., :d], rotate(q[..., d:], mixer["rot"])
    k_plain = lin(w[prefix + "uk"], latent).reshape(T, H, d)
    v = lin(w[prefix + "uv"], latent).reshape(T, H, e)
    mask = window_mask(T, (mixer.get("mask") or {}).get("size"))
    gate = torch.sigmoid(lin(w[prefix + "g"], h))
    heads = []
    for head in range(H):
        scores = (q_plain[:, head] @ k_plain[:, head].t() + q_rot[:, head] @ shared_key.t()) * float(mixer["scale"])
        heads.append((softmax_rows(scores, mask) @ v[:, head]) * gate[:, head:head + 1])
    return lin(w[prefix + "o"], torch.cat(heads, -1))


def gelu_erf(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def expert(h: torch.Tensor, w: Mapping[str, torch.Tensor], prefix: str) -> torch.Tensor:
    return lin(w[prefix + "down"], gelu_erf(lin(w[prefix + "up"], h)))


def choose(scores: torch.Tensor, top: int, groups: Optional[Mapping]) -> torch.Tensor:
    """The indices of the `top` largest scores of one token; with groups, only among the experts of the `keep`
    groups (runs of neighbours of equal length) whose best score is largest."""
    allowed = scores.clone()
    if groups:
        count, keep = int(groups["count"]), int(groups["keep"])
        per = scores.shape[0] // count
        best = scores.reshape(count, per).max(-1).values
        kept = torch.topk(best, keep).indices.tolist()
        for g in range(count):
            if g not in kept:
                allowed[g * per:(g + 1) * per] = float("-inf")
    return torch.topk(allowed, top).indices


def routed_feed_forward(h: torch.Tensor, w: Mapping[str, torch.Tensor], prefix: str, mlp: Mapping,
                        given: Optional[torch.Tensor] = None, margin: float = 0.0) -> torch.Tensor:
    """`given` [T, top]: another implementation's choices. A token takes them instead of its own only if they are
    its own choice once the given experts' scores are raised and the others' lowered by the factor `margin` (a
    close call that fell the other way); the weights are always this function's own scores."""
    router = mlp["router"]
    top, groups = int(router["top"]), router.get("groups")
    scores = torch.softmax(lin(w[prefix + "router"], h), -1)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        chosen = choose(scores[t], top, groups)
        if given is not None and sorted(given[t].tolist()) != sorted(chosen.tolist()):
            tilted = scores[t] * (1.0 - margin)
            tilted[given[t].long()] = scores[t, given[t].long()] * (1.0 + margin)
            if sorted(choose(tilted, top, groups).tolist()) == sorted(given[t].tolist()):
                chosen = given[t].long()
        total = scores[t, chosen].sum() + 1e-20
        for index in chosen.tolist():
            out[t] += scores[t, index] / total * expert(h[t:t + 1], w, f"{prefix}e{index}.")[0]
    if mlp.get("shared"):
        out = out + expert(h, w, prefix + "shared.")
    return out


def run_order(config: Mapping) -> List[tuple]:
    """(layer, pass number or None) in the order the layers run; the pass number is given at the first layer
    of each pass of the looped range."""
    count = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return [(index, None) for index in range(count)]
    start, stop, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    order = [(index, None) for index in range(start)]
    for t in range(times):
        order += [(index, t if index == start else None) for index in range(start, stop)]
    return order + [(index, None) for index in range(stop, count)]


def forward(config: Mapping, w: Mapping[str, torch.Tensor], tokens, dtype=torch.float64,
            streams: Optional[List[torch.Tensor]] = None, choices: Optional[List[torch.Tensor]] = None,
            margin: float = 0.0) -> torch.Tensor:
    """`choices`: for every run of a layer with a feed-forward, in the order they run, the experts [T, top] that
    another implementation chose (see `routed_feed_forward`)."""
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    w = {name: (tensor.to(dtype) if tensor.is_floating_point() else tensor) for name, tensor in w.items()}
    eps = float(config["norm"]["eps"])
    x = w["embed"][tokens]
    routed_runs = 0
    for index, step in run_order(config):
        layer, prefix = config["layers"][index], f"l{index}."
        if step is not None:
            x = x + w["loop.step"][step]
        h = centred_norm(x, w[prefix + "norm1"], eps)
        if layer["type"] == "attention":
            mixed = attention(h, w, prefix + "mix.", layer["mixer"])
        else:
            mixed = latent_attention(h, w, prefix + "mix.", layer["mixer"], eps)
        x = x + centred_norm(mixed, w[prefix + "norm1b"], eps)
        if layer.get("mlp") is not None:
            h = centred_norm(x, w[prefix + "norm2"], eps)
            given = choices[routed_runs] if choices is not None else None
            routed_runs += 1
            x = x + centred_norm(routed_feed_forward(h, w, prefix + "mlp.", layer["mlp"], given, margin),
                                 w[prefix + "norm2b"], eps)
        if streams is not None:
            streams.append(x.clone())
    return lin(w["head"], centred_norm(x, w["final.norm"], eps)) * float(config.get("logit_scale", 1.0))
