"""The selective state-space mixer: input projection, short causal convolution, selective scan, gate, output projection."""
from __future__ import annotations

import os
from typing import Dict, List

import torch

from .. import ops
from ..cache.manager import CacheNeed
from ..config.registry import MIXERS
from ..config.specs import MixerSpec
from .base import CacheView, Mixer, StepContext, WeightSpec

PROMPT_MIN_TOKENS = 16      # steps of more tokens take a scan kernel for portions ...
CHUNKED_MIN_TOKENS = 32     # ... the one that is parallel over tokens where a portion has this many
CHUNKED = os.environ.get("PULSAR_SCAN_CHUNKED", "1") != "0"


@MIXERS.register("selective_scan")
class SelectiveScan(Mixer):
    """W_in h = [x | z] (``inner`` channels each); x passes a causal convolution of ``conv`` taps per channel and silu;
    W_x x = [r: dt_rank | B: state | C: state]; dt = softplus(W_dt r + dt_bias) per channel, A = -exp(A_log);
    S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n;  y_c = sum_n S[c, n] C_n + D_c x_c;  out = W_o (y * silu(z)).

    The state of a sequence, S [inner, state] and the convolution's last ``conv - 1`` inputs per channel, is float32 and
    lives in the sequence's slot of the cache manager's state arena; it starts at zero and is carried from step to step.
    A step's portions and single tokens run together: every kernel takes what it needs to know about the step (where
    each sequence's tokens begin, which slot is its own) from the step's device arrays, so a step of single tokens can be
    replayed from a CUDA graph.  dt, the decay and the recurrence are float32 (``ops.selective_scan`` does the dt
    product itself); the three projections are the engine's ordinary products.

    Options (``spec.extra``): ``inner``, ``state``, ``dt_rank``, ``conv``.
    """

    def __init__(self, spec: MixerSpec, prefix: str, dtype: torch.dtype):
        self.inner = int(spec.option("inner", 0))
        self.n_state = int(spec.option("state", 0))
        self.dt_rank = int(spec.option("dt_rank", 0))
        self.taps = int(spec.option("conv", 0))
        if min(self.inner, self.n_state, self.dt_rank, self.taps) <= 0:
            raise ValueError("selective scan: inner, state, dt_rank and conv must be positive")
        self.spec, self.prefix, self.dtype = spec, prefix, dtype
        name = spec.tensor_name
        self.names = {r: name(r, d) for r, d in (("in", "in_proj.weight"), ("conv", "conv1d.weight"), ("conv_bias", "conv1d.bias"),
                                                 ("x", "x_proj.weight"), ("dt", "dt_proj.weight"), ("dt_bias", "dt_proj.bias"),
                                                 ("a_log", "A_log"), ("d", "D"), ("o", "out_proj.weight"))}
        self.w = {}

    @property
    def tail_offset(self) -> int:
        return self.inner * self.n_state

    def weight_specs(self) -> List[WeightSpec]:
        s, p, nm = self.spec, self.prefix, self.names
        return [WeightSpec(p + nm["in"], (2 * self.inner, s.hidden)),
                WeightSpec(p + nm["conv"], (self.inner, self.taps), role="vector", init="taps"),
                WeightSpec(p + nm["conv_bias"], (self.inner,), role="vector", init="small"),
                WeightSpec(p + nm["x"], (self.dt_rank + 2 * self.n_state, self.inner)),
                WeightSpec(p + nm["dt"], (self.inner, self.dt_rank), init="wide"),
                WeightSpec(p + nm["dt_bias"], (self.inner,), role="vector", init="step_bias"),
                WeightSpec(p + nm["a_log"], (self.inner, self.n_state), role="vector", init="decay_log"),
                WeightSpec(p + nm["d"], (self.inner,), role="vector", init="ones_normal"),
                WeightSpec(p + nm["o"], (s.hidden, self.inner))]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.w = {role: tensors[self.prefix + n] for role, n in self.names.items()}
        # the two parts of the input-dependent projection as products of their own (steps with prompt portions)
        self.w_x_r = self.w["x"][:self.dt_rank].contiguous()
        self.w_x_bc = self.w["x"][self.dt_rank:].contiguous()

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.w.values())

    def cache_need(self) -> CacheNeed:
        return CacheNeed.state((self.inner * (self.n_state + self.taps - 1),), torch.float32)

    def forward(self, ctx: StepContext, h: torch.Tensor, cache: CacheView) -> torch.Tensor:
        n, w = ctx.n_tokens, self.w
        xz = ctx.scratch("scan.xz", (n, 2 * self.inner))
        ops.linear(h, w["in"], xz)
        x = ctx.scratch("scan.x", (n, self.inner))
        ops.causal_conv_silu(ctx, xz, self.inner, w["conv"], w["conv_bias"], cache.state, self.tail_offset, x)
        y = ctx.scratch("scan.y", (n, self.inner))
        chunked = CHUNKED and ctx.max_q_len >= CHUNKED_MIN_TOKENS and ops.selective_scan_chunked_supported(self.n_state)
        if n > PROMPT_MIN_TOKENS and (chunked or ops.selective_scan_prompt_supported(self.n_state)):
            # many tokens: the step sizes' product runs as a product (float32 out), and a scan kernel for portions follows:
            # parallel over tokens where a portion is long, else eight tokens side by side (a captured step of single
            # tokens never comes here)
            r = ctx.scratch("scan.r", (n, self.dt_rank))
            ops.linear(x, self.w_x_r, r)
            bc = ctx.scratch("scan.bc", (n, 2 * self.n_state))
            ops.linear(x, self.w_x_bc, bc)
            dt_pre = ctx.scratch("scan.dt", (n, self.inner), torch.float32)
            ops.linear(r, w["dt"], dt_pre)
            ops.selective_scan_prompt(ctx, x, xz, bc, dt_pre, w["dt_bias"], w["a_log"], w["d"], cache.state, self.tail_offset,
                                      self.taps, y, chunked=chunked)
        else:
            proj = ctx.scratch("scan.proj", (n, self.dt_rank + 2 * self.n_state))
            ops.linear(x, w["x"], proj)
            ops.selective_scan(ctx, x, xz, proj, w["dt"], w["dt_bias"], w["a_log"], w["d"], cache.state, self.tail_offset,
                               self.taps, y)
        out = ctx.scratch("scan.out", (n, self.spec.hidden))
        ops.linear(y, w["o"], out)
        return out
