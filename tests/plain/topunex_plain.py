"""Plain, slow implementation of the Topunex decoder: one function per mechanism, whole sequences only.

Written from the design's equations with dense tensors on the CPU: no cache, no pages, no
portions, no batch.  Nothing here is imported by the product package and nothing of the product is
imported here.  Notation: ``h`` [L, width] is a sublayer's input for the L tokens of one sequence,
positions are 0 .. L-1, weights are stored [out, in] and applied as ``h @ W.T``.

A layer is  x = x + N1(mixer(x));  x = x + N2(ff(x))  with N an RMS norm: the sublayers read the
stream itself and only their outputs are normed.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def rms_norm(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def rotary_frequencies(base: float, dims: int, scaling: Optional[dict], dtype=torch.float64) -> torch.Tensor:
    """f_i = base^(-2i/dims), i < dims/2, then the wavelength-dependent rescaling: a frequency whose wavelength
    2 pi / f is shorter than original/high stays, one longer than original/low is divided by factor, and between
    the two the divided and the plain frequency are blended linearly in original/wavelength."""
    freqs = []
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        if scaling is not None:
            factor, low, high, original = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
            wavelength = 2.0 * math.pi / f
            if wavelength < original / high:
                pass
            elif wavelength > original / low:
                f = f / factor
            else:
                s = (original / wavelength - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        freqs.append(f)
    return torch.tensor(freqs, dtype=dtype)


def rotate_halves(x: torch.Tensor, positions: torch.Tensor, freqs: torch.Tensor) -> torch.Tensor:
    """x [L, heads, D]: element i and element i + n (n = len(freqs)) form a pair that turns by position * freqs[i];
    elements from 2n on pass unchanged."""
    n = freqs.numel()
    angle = positions.to(x.dtype)[:, None] * freqs.to(x.dtype)[None, :]          # [L, n]
    cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    u, v = x[..., :n], x[..., n:2 * n]
    out = x.clone()
    out[..., :n] = u * cos - v * sin
    out[..., n:2 * n] = v * cos + u * sin
    return out


def visible_keys(L: int, size: Optional[int], keep_first: int) -> torch.Tensor:
    """[L, L] bool: query i sees key j when j <= i and (i - j < size or j < keep_first)."""
    i = torch.arange(L)[:, None]
    j = torch.arange(L)[None, :]
    near = torch.ones(L, L, dtype=torch.bool) if size is None else (i - j < size)
    return (j <= i) & (near | (j < keep_first))


def capped(scores: torch.Tensor, cap: Optional[float]) -> torch.Tensor:
    return scores if not cap else cap * torch.tanh(scores / cap)


def softmax_with_sink(scores: torch.Tensor, visible: torch.Tensor, sink: Optional[torch.Tensor]) -> torch.Tensor:
    """scores [H, L, L]; the denominator holds one more term per head, exp(sink[h]), that has no value."""
    scores = scores.masked_fill(~visible, float("-inf"))
    if sink is None:
        return torch.softmax(scores, dim=-1)
    H, L, _ = scores.shape
    extra = sink.to(scores.dtype).view(H, 1, 1).expand(H, L, 1)
    return torch.softmax(torch.cat([scores, extra], dim=-1), dim=-1)[..., :-1]


def attention(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    """Grouped attention whose values are the projected keys.  ``w``: the mixer's tensors by their short names
    (q, q.b, k, k.b, sink, g, o, o.b)."""
    L = h.shape[0]
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    pos = torch.arange(L)
    q = (h @ w["q"].T + w["q.b"]).view(L, H, D)
    k = (h @ w["k"].T + w["k.b"]).view(L, G, D)
    value = k.clone()                                       # as projected: before rotation and norm
    rot = m.get("rot")
    if rot is not None:
        freqs = rotary_frequencies(float(rot["base"]), int(rot["dims"]), rot.get("scaling"))
        q, k = rotate_halves(q, pos, freqs), rotate_halves(k, pos, freqs)
    q, k = rms_norm(q, None, eps), rms_norm(k, None, eps)
    group = H // G
    k_of_head = k.repeat_interleave(group, dim=1)            # head h uses key head h // group
    v_of_head = value.repeat_interleave(group, dim=1)
    scores = capped(torch.einsum("ihd,jhd->hij", q, k_of_head) * m["scale"], m.get("softcap"))
    mask = m.get("mask")
    vis = visible_keys(L, None if mask is None else mask.get("size"), 0 if mask is None else int(mask.get("keep_first", 0)))
    p = softmax_with_sink(scores, vis[None], w.get("sink"))
    heads = torch.einsum("hij,jhd->ihd", p, v_of_head).reshape(L, H * D)
    heads = heads * torch.sigmoid(h @ w["g"].T)
    return heads @ w["o"].T + w["o.b"]


def dense_ff(h: torch.Tensor, w: Dict[str, torch.Tensor]) -> torch.Tensor:
    g = h @ w["gate"].T + w["gate.b"]
    u = h @ w["up"].T + w["up.b"]
    return (g * torch.sigmoid(g) * u) @ w["down"].T + w["down.b"]


def expert(h: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor, limit: float) -> torch.Tensor:
    g = torch.clamp(h @ gate.T, max=limit)
    u = torch.clamp(h @ up.T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ down.T


def routed(h: torch.Tensor, router: torch.Tensor, top: int, scale: float):
    """(chosen experts [L, top], their weights [L, top]): sigmoid scores, the ``top`` largest, times ``scale``."""
    s = torch.sigmoid(h @ router.T)
    val, idx = torch.topk(s, top, dim=-1)
    return idx, val * scale


def route_margins(h: torch.Tensor, router: torch.Tensor, top: int) -> torch.Tensor:
    """[L]: how far the router's logits of the last chosen and the first rejected expert lie apart, relative to the
    largest logit's magnitude (infinite where every expert is chosen).  A small margin is a close call: rounding may
    choose otherwise."""
    z = h @ router.T
    if top >= z.shape[1]:
        return torch.full((h.shape[0],), float("inf"), dtype=h.dtype)
    ordered = torch.sort(z, dim=-1, descending=True).values
    return (ordered[:, top - 1] - ordered[:, top]) / z.abs().max(dim=-1).values.clamp_min(1e-30)


def moe_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], mlp: dict, margins: Optional[list] = None) -> torch.Tensor:
    r, e = mlp["router"], mlp["expert"]
    idx, weight = routed(h, w["router"], int(r["top"]), float(r["scale"]))
    if margins is not None:
        margins.append(route_margins(h, w["router"], int(r["top"])))
    out = torch.zeros(h.shape[0], w["e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for c in range(idx.shape[1]):
            x = int(idx[t, c])
            out[t] += weight[t, c] * expert(h[t:t + 1], w[f"e{x}.gate"], w[f"e{x}.up"], w[f"e{x}.down"], float(e["limit"]))[0]
    shared = mlp.get("shared")
    if shared is not None:
        out = out + expert(h, w["shared.gate"], w["shared.up"], w["shared.down"], float(shared["limit"]))
    return out


def sub(weights: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {n[len(prefix):]: t for n, t in weights.items() if n.startswith(prefix)}


def forward(cfg: dict, weights: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float64,
            streams: Optional[list] = None, margins: Optional[list] = None) -> torch.Tensor:
    """Logits [L, vocab] of one whole sequence.  ``streams``: a list that receives the stream after every layer;
    ``margins``: a list that receives every routed layer's ``route_margins``."""
    w = {n: t.to(dtype) for n, t in weights.items()}
    eps = float(cfg["norm"]["eps"])
    x = w["embed"][torch.tensor(list(tokens))]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        if layer["type"] != "attention":
            raise ValueError(f"layer type {layer['type']}")
        x = x + rms_norm(attention(x, sub(w, p + "mix."), layer["mixer"], eps), w[p + "norm1"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            ff = dense_ff(x, sub(w, p + "mlp.")) if mlp["kind"] == "dense" else moe_ff(x, sub(w, p + "mlp."), mlp, margins)
            x = x + rms_norm(ff, w[p + "norm2"], eps)
        if streams is not None:
            streams.append(x.clone())
    return rms_norm(x, w["final.norm"], eps) @ w["head"].T
