"""Attention over a compressed latent: one cached row per token, expanded per head on the fly."""
from __future__ import annotations

from typing import Dict, List

import torch

from .. import ops
from ..cache.manager import CachedTensor, CacheNeed
from ..config.registry import MIXERS, POSITIONS
from ..config.specs import MixerSpec
from .base import CacheView, Mixer, StepContext, WeightSpec


@MIXERS.register("latent_attention")
class LatentAttention(Mixer):
    """Every head's query has ``head_dim`` plain dimensions and ``rot_dim`` rotated ones.  A down projection of the
    input gives ``kv_rank`` numbers, RMS-normed into the latent c, and ``rot_dim`` numbers that are rotated at the
    token's position and serve all heads as the rotated key part.  Per head the plain key is W_uk[h] c and the value
    W_uv[h] c; only c and the rotated key part are cached, as one row [c | key_rot] per token.

    The keys and values are never expanded: with q_abs[h] = W_uk[h]^T q_plain[h] the score is
    (q_abs[h] . c + q_rot[h] . key_rot) * scale, and the head's output is W_uv[h] (sum_j p_j c_j).  So the attention
    itself runs with one shared key/value head over the cached rows (key = the whole row, value = its first
    ``kv_rank`` elements) and the two expansions become per-head products on the query and on the output side
    (``ops.heads_linear``).  Queries stay float32 from their rotation to the scores.

    Options (``spec.extra``): ``kv_rank``, ``rot_dim``, ``latent_norm_eps``, ``gated`` (the concatenated heads are
    multiplied by sigmoid(W_g h), h the mixer's input).  ``spec.position`` gives the rotation (its table's
    ``rotary_dim`` leading dimensions of the rotated part turn, in neighbouring pairs).  With ``own_kv`` False the
    mixer has no down projection and attends over the rows another layer cached this step, with its own expansions.
    """

    def __init__(self, spec: MixerSpec, prefix: str, dtype: torch.dtype):
        self.rank = int(spec.option("kv_rank", 0))
        self.rot_dim = int(spec.option("rot_dim", 0))
        self.norm_eps = float(spec.option("latent_norm_eps", 1e-6))
        self.gated = bool(spec.option("gated", False))
        if spec.n_heads <= 0 or spec.head_dim <= 0 or spec.value_dim <= 0 or self.rank <= 0 or self.rot_dim < 0:
            raise ValueError("latent attention: heads, head sizes and the latent's rank must be positive")
        if self.rot_dim and spec.position is None:
            raise ValueError("latent attention: a rotated part needs a position encoding")
        if spec.position is not None and spec.position.rotary_dim > self.rot_dim:
            raise ValueError(f"latent attention: {spec.position.rotary_dim} rotating dimensions exceed rot_dim {self.rot_dim}")
        self.spec, self.prefix, self.dtype = spec, prefix, dtype
        self.position = POSITIONS.get(spec.position.kind)(spec.position) if spec.position is not None else None
        name = spec.tensor_name
        self.names = {r: name(r, d) for r, d in (("q", "q_proj.weight"), ("down", "kv_down_proj.weight"),
                                                 ("latent_norm", "kv_norm.weight"), ("up_k", "k_up_proj.weight"),
                                                 ("up_v", "v_up_proj.weight"), ("gate", "gate_proj.weight"),
                                                 ("o", "o_proj.weight"))}
        self.w_in = self.w_uk_t = self.w_uv = self.w_o = self.latent_norm = None

    @property
    def row(self) -> int:
        return self.rank + self.rot_dim

    # ---------------------------------------------------------------- weights
    def weight_specs(self) -> List[WeightSpec]:
        s, p, nm = self.spec, self.prefix, self.names
        specs = [WeightSpec(p + nm["q"], (s.n_heads * (s.head_dim + self.rot_dim), s.hidden))]
        if s.own_kv:
            specs += [WeightSpec(p + nm["down"], (self.row, s.hidden)),
                      WeightSpec(p + nm["latent_norm"], (self.rank,), role="vector", init="ones_normal")]
        specs += [WeightSpec(p + nm["up_k"], (s.n_heads * s.head_dim, self.rank)),
                  WeightSpec(p + nm["up_v"], (s.n_heads * s.value_dim, self.rank))]
        if self.gated:
            specs.append(WeightSpec(p + nm["gate"], (s.n_heads * s.value_dim, s.hidden)))
        specs.append(WeightSpec(p + nm["o"], (s.hidden, s.n_heads * s.value_dim)))
        return specs

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        s, p, nm = self.spec, self.prefix, self.names
        rows = [tensors[p + nm["q"]]]
        if s.own_kv:
            rows.append(tensors[p + nm["down"]])
            self.latent_norm = tensors[p + nm["latent_norm"]]
        if self.gated:
            rows.append(tensors[p + nm["gate"]])
        self.w_in = torch.cat(rows, dim=0).contiguous() if len(rows) > 1 else rows[0]      # rows: q | down | gate
        # per head [inputs, outputs]: the key expansion as stored serves the query side (head_dim -> rank), the value
        # expansion is transposed once (rank -> value_dim)
        self.w_uk_t = tensors[p + nm["up_k"]].view(s.n_heads, s.head_dim, self.rank).contiguous()
        self.w_uv = tensors[p + nm["up_v"]].view(s.n_heads, s.value_dim, self.rank).transpose(1, 2).contiguous()
        self.w_o = tensors[p + nm["o"]]

    def weight_bytes(self) -> int:
        ts = [self.w_in, self.w_uk_t, self.w_uv, self.w_o, self.latent_norm]
        return sum(t.numel() * t.element_size() for t in ts if t is not None)

    def cache_need(self) -> CacheNeed:
        return CacheNeed.paged((CachedTensor("latent", 1, self.row),), self.spec.window)

    # ---------------------------------------------------------------- one step
    def forward(self, ctx: StepContext, h: torch.Tensor, cache: CacheView) -> torch.Tensor:
        s, n, H = self.spec, ctx.n_tokens, self.spec.n_heads
        q_width = H * (s.head_dim + self.rot_dim)
        proj = ctx.scratch("latent.in", (n, self.w_in.shape[0]))
        ops.linear(h, self.w_in, proj)
        q = proj[:, :q_width]
        down = proj[:, q_width:q_width + self.row] if s.own_kv else None
        gate = proj[:, self.w_in.shape[0] - H * s.value_dim:] if self.gated else None
        pool = cache.pools["latent"]
        q_full = ctx.scratch("latent.q", (n, H, self.row), torch.float32)
        ops.heads_linear(q.view(n, H, s.head_dim + self.rot_dim)[:, :, :s.head_dim], self.w_uk_t, q_full[:, :, :self.rank])
        if self.position is not None:
            cos, sin = self.position.tables(ctx)
        else:
            cos = sin = ctx.scratch("latent.norope", (n, 0), torch.float32)
        ops.latent_prepare(q, down, self.latent_norm, self.norm_eps, cos, sin, cache.slots if s.own_kv else None,
                           pool if s.own_kv else None, q_full, H, s.head_dim, self.rot_dim, self.rank, cache.page_size)
        mixed = ctx.scratch("latent.mixed", (n, H, self.rank))
        ops.paged_attention_general(ctx, q_full, pool, pool, mixed, cache.block_table, s.scale, s.window, s.chunk, None,
                                    key_width=self.row, value_width=self.rank)
        heads = ctx.scratch("latent.heads", (n, H, s.value_dim))
        ops.heads_linear(mixed, self.w_uv, heads, gate)
        out = ctx.scratch("latent.out", (n, s.hidden))
        ops.linear(heads.view(n, H * s.value_dim), self.w_o, out)
        return out
