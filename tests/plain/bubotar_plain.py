"""Plain, slow implementation of the Bubotar decoder: one function per mechanism, whole sequences only.

Written from the design's equations with dense tensors on the CPU: no cache, no pages, no
portions, no batch.  Nothing here is imported by the product package and nothing of the product is
imported here.  Notation: ``h`` [L, width] is a sublayer's input for the L tokens of one sequence,
positions are 0 .. L-1, weights are stored [out, in] and applied as ``h @ W.T``.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def rms_norm(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def rotate_pairs(x: torch.Tensor, positions: torch.Tensor, base: float, dims: int) -> torch.Tensor:
    """x [L, ..., D]: neighbours (2i, 2i+1), i < dims/2, turn by the angle position * base^(-2i/dims)."""
    out = x.clone()
    i = torch.arange(dims // 2, dtype=x.dtype)
    freq = base ** (-2.0 * i / dims)
    angle = positions.to(x.dtype)[:, None] * freq[None, :]              # [L, dims/2]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [dims // 2]
    cos, sin = torch.cos(angle).view(shape), torch.sin(angle).view(shape)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


def softmax_rows(scores: torch.Tensor, visible: torch.Tensor) -> torch.Tensor:
    scores = scores.masked_fill(~visible, float("-inf"))
    return torch.softmax(scores, dim=-1)


def latent_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float,
                     shared: Optional[Dict[str, torch.Tensor]] = None) -> (torch.Tensor, Dict[str, torch.Tensor]):
    """Attention over a compressed latent.  ``w`` holds the mixer's tensors by their short names.  ``shared``: the
    latent and the rotated key part of the layer this one borrows them from (then ``w`` has no 'dkv').  Returns the
    mixer's output and what this layer would lend."""
    L = h.shape[0]
    H, dim, rot_dim, vdim, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(L)
    q = (h @ w["q"].T).view(L, H, dim + rot_dim)
    q_plain, q_rot = q[..., :dim], rotate_pairs(q[..., dim:], pos, m["rot"]["base"], m["rot"]["dims"])
    if shared is None:
        down = h @ w["dkv"].T
        latent = rms_norm(down[:, :rank], w["dkv.norm"], eps)
        key_rot = rotate_pairs(down[:, rank:], pos, m["rot"]["base"], m["rot"]["dims"])
        shared = {"latent": latent, "key_rot": key_rot}
    latent, key_rot = shared["latent"], shared["key_rot"]
    k_plain = (latent @ w["uk"].T).view(L, H, dim)
    value = (latent @ w["uv"].T).view(L, H, vdim)
    scores = (torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihd,jd->hij", q_rot, key_rot)) * m["scale"]
    visible = pos[None, :] <= pos[:, None]
    p = softmax_rows(scores, visible[None])
    heads = torch.einsum("hij,jhd->ihd", p, value).reshape(L, H * vdim)
    heads = heads * torch.sigmoid(h @ w["g"].T)
    return heads @ w["o"].T, shared


def distance_slopes(n_heads: int, dtype) -> torch.Tensor:
    return torch.tensor([2.0 ** (-8.0 * (k + 1) / n_heads) for k in range(n_heads)], dtype=dtype)


def dense_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, slopes: Optional[torch.Tensor] = None,
                    chunk: Optional[int] = None, window: Optional[int] = None, first: int = 0) -> torch.Tensor:
    """q [Lq, H, D], k [L, H, D], v [L, H, Dv] with one key/value head per query head; the queries sit at positions
    first .. first + Lq - 1, the keys at 0 .. L - 1.  Causal; optional distance bias, chunk mask and window."""
    qpos, kpos = first + torch.arange(q.shape[0]), torch.arange(k.shape[0])
    scores = torch.einsum("ihd,jhd->hij", q, k) * scale
    if slopes is not None:
        scores = scores - slopes.to(q.dtype)[:, None, None] * (qpos[:, None] - kpos[None, :]).to(q.dtype)[None]
    visible = kpos[None, :] <= qpos[:, None]
    if chunk:
        visible = visible & ((kpos[None, :] // chunk) == (qpos[:, None] // chunk))
    if window:
        visible = visible & (kpos[None, :] > qpos[:, None] - window)
    return torch.einsum("hij,jhd->ihd", softmax_rows(scores, visible[None]), v)


def chunked_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict) -> torch.Tensor:
    """Grouped heads, no rotation; the score loses slope_h * (i - j); a query sees earlier keys of its own chunk."""
    L = h.shape[0]
    H, G, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w["q"].T).view(L, H, dim)
    k = (h @ w["k"].T).view(L, G, dim).repeat_interleave(H // G, dim=1)
    v = (h @ w["v"].T).view(L, G, vdim).repeat_interleave(H // G, dim=1)
    out = dense_attention(q, k, v, m["scale"], distance_slopes(H, h.dtype), (m.get("mask") or {}).get("size"))
    return out.reshape(L, H * vdim) @ w["o"].T


def silu(x: torch.Tensor) -> torch.Tensor:
    return x * torch.sigmoid(x)


def softplus(x: torch.Tensor) -> torch.Tensor:
    return torch.where(x > 30.0, x, torch.log1p(torch.exp(torch.clamp(x, max=30.0))))


def causal_conv(x: torch.Tensor, taps: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """x [L, C]; taps [C, T], the last column weighs the current token; zeros before the start."""
    L, C = x.shape
    T = taps.shape[1]
    padded = torch.cat([torch.zeros(T - 1, C, dtype=x.dtype), x], dim=0)
    out = bias[None, :].expand(L, C).clone()
    for t in range(T):
        out = out + padded[t:t + L] * taps[:, t][None, :]
    return out


def selective_scan(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict) -> torch.Tensor:
    L = h.shape[0]
    inner, n_state, dt_rank = m["inner"], m["state"], m["dt_rank"]
    xz = h @ w["in"].T
    x, z = xz[:, :inner], xz[:, inner:]
    x = silu(causal_conv(x, w["conv"], w["conv.b"]))
    proj = x @ w["x"].T
    dt, B, C = proj[:, :dt_rank], proj[:, dt_rank:dt_rank + n_state], proj[:, dt_rank + n_state:]
    dt = softplus(dt @ w["dt"].T + w["dt.b"])                          # [L, inner]
    A = -torch.exp(w["A_log"])                                         # [inner, state]
    state = torch.zeros(inner, n_state, dtype=h.dtype)
    ys = []
    for t in range(L):
        state = torch.exp(dt[t][:, None] * A) * state + (dt[t] * x[t])[:, None] * B[t][None, :]
        ys.append(state @ C[t] + w["D"] * x[t])
    y = torch.stack(ys) * silu(z)
    return y @ w["o"].T


def clamped_glu(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict) -> torch.Tensor:
    limit = m["limit"]
    g = torch.clamp(h @ w["gate"].T, max=limit)
    u = torch.clamp(h @ w["up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w["down"].T


def sub(weights: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {n[len(prefix):]: t for n, t in weights.items() if n.startswith(prefix)}


def forward(cfg: dict, weights: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float64,
            residuals: Optional[list] = None) -> torch.Tensor:
    """Logits [L, vocab] of one sequence.  ``residuals``: a list that receives the stream after every layer."""
    w = {n: t.to(dtype) for n, t in weights.items()}
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(tokens, dtype=torch.long)]
    lent: Dict[int, Dict[str, torch.Tensor]] = {}
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        m = layer["mixer"]
        h = rms_norm(x, w[p + "norm1"], eps)
        mix = sub(w, p + "mix.")
        if layer["type"] == "latent_attention":
            src = m.get("kv_from")
            y, lent[i] = latent_attention(h, mix, m, eps, None if src is None else lent[src])
        elif layer["type"] == "mamba1":
            y = selective_scan(h, mix, m)
        elif layer["type"] == "attention":
            y = chunked_attention(h, mix, m)
        else:
            raise ValueError(f"layer {i}: unknown type {layer['type']}")
        x = x + rms_norm(y, w[p + "norm1b"], eps)
        if layer.get("mlp") is not None:
            h = rms_norm(x, w[p + "norm2"], eps)
            x = x + rms_norm(clamped_glu(h, sub(w, p + "mlp."), layer["mlp"]), w[p + "norm2b"], eps)
        if residuals is not None:
            residuals.append(x.clone())
    return (rms_norm(x, w["final.norm"], eps) @ w["head"].T) * cfg.get("logit_scale", 1.0)


def greedy_generate(cfg: dict, weights: Dict[str, torch.Tensor], prompt: List[int], n_new: int) -> List[int]:
    seq, out = list(prompt), []
    for _ in range(n_new):
        out.append(int(torch.argmax(forward(cfg, weights, seq)[-1])))
        seq.append(out[-1])
    return out
