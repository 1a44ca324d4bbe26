"""Bubotar through the engine against the plain implementation (tests/plain/bubotar_plain.py): configuration on the
CPU; on a GPU each mechanism alone, prompts against token-by-token decoding, portions, mixed batches with pages and
state slots used again, crafted keys at the edges of chunks and pages, long decoding, and greedy generation through
the public entry point."""
import copy
import json
import math
import os
import random
import subprocess
import sys
import types

import pytest
import torch

import helpers
from helpers import TOL
from plain import bubotar_plain as plain


def latent(heads, dim, rot_dim, vdim, rank, base=5000.0, dims=None, scale=None, kv_from=None):
    m = dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=rank, scale=scale or 1.0 / math.sqrt(dim + rot_dim),
             rot=dict(base=base, dims=dims or rot_dim))
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def scan(inner, state, dt_rank, conv):
    return dict(inner=inner, state=state, dt_rank=dt_rank, conv=conv)


def attn(heads, kv_heads, dim, vdim, size, scale=None):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale or 1.0 / math.sqrt(dim))
    if size:
        m["mask"] = dict(size=size)
    return m


def layer(kind, mixer, ff=None, limit=1.5):
    return dict(type=kind, mixer=mixer, mlp=None if ff is None else dict(kind="dense", ff=ff, limit=limit))


def config(layers, vocab, width, eps=1e-5, logit_scale=1.0):
    return dict(architecture="Bubotar", vocab=vocab, width=width, norm=dict(eps=eps), logit_scale=logit_scale, layers=layers)


# Every size differs between the configurations; odd head counts, rotation of only a part of the rotated dimensions,
# a chunk that no page size divides, a state larger than 64 (the wide thread layout of the scan), one tap only,
# one key/value head, as many key/value heads as query heads, a borrowed latent, layers without feed-forward.
BUBO_A = config([
    layer("attention", attn(4, 2, 16, 24, 10), ff=96),
    layer("latent_attention", latent(3, 16, 8, 12, 24), ff=80, limit=1.0),
    layer("mamba1", scan(48, 6, 5, 4)),
    layer("latent_attention", latent(2, 8, 8, 20, 24, kv_from=1), ff=72),
    layer("mamba1", scan(40, 12, 3, 2), ff=64),
], vocab=200, width=64, eps=1e-5, logit_scale=0.7)
BUBO_B = config([
    layer("mamba1", scan(72, 70, 9, 1), ff=56),
    layer("latent_attention", latent(1, 24, 16, 16, 40, base=300.0, dims=12)),
    layer("attention", attn(3, 3, 8, 8, 7), ff=48, limit=3.0),
    layer("attention", attn(6, 1, 12, 4, 33)),
    layer("latent_attention", latent(5, 4, 16, 8, 40, base=300.0, dims=12, kv_from=1), ff=40),
    layer("latent_attention", latent(2, 12, 4, 12, 16, base=77.0), ff=40),
], vocab=131, width=48, eps=3e-6, logit_scale=1.0)
ONLY_SCAN = config([layer("mamba1", scan(32, 4, 2, 3), ff=32), layer("mamba1", scan(24, 9, 4, 5))], vocab=90, width=32)
ALONE = {
    "latent": config([layer("latent_attention", latent(3, 8, 8, 12, 16))], vocab=64, width=40),
    "latent_ff": config([layer("latent_attention", latent(2, 16, 4, 8, 12), ff=56)], vocab=64, width=40),
    "scan": config([layer("mamba1", scan(56, 10, 6, 3))], vocab=64, width=40),
    "attention": config([layer("attention", attn(4, 2, 12, 20, 9))], vocab=64, width=40),
    "attention_unmasked": config([layer("attention", attn(2, 1, 8, 8, None), ff=24)], vocab=64, width=40),
}
CONFIGS = {"A": (BUBO_A, 11, 8), "B": (BUBO_B, 12, 4), "S": (ONLY_SCAN, 13, 16)}      # config, seed, page size


# ------------------------------------------------------------------ configuration (CPU)
def test_config_becomes_parts_with_shared_cache_entries():
    from pulsar_b200.config import config_from_dict
    from pulsar_b200.models import build_model
    cfg = config_from_dict(copy.deepcopy(BUBO_A))
    spec = cfg.model_spec()
    assert [(c.block, c.cache) for c in spec.run_order] == [(0, 0), (1, 1), (2, 2), (3, 1), (4, 3)]
    assert [b.mixer.kind for b in spec.blocks] == ["attention", "latent_attention", "selective_scan", "latent_attention",
                                                   "selective_scan"]
    assert spec.blocks[2].feed_forward is None and spec.blocks[3].mixer.own_kv is False
    assert spec.logit_scale == 0.7 and cfg.to_dict() == BUBO_A
    model = build_model(cfg, torch.float32)
    names = {w.name for w in model.weight_specs()}
    assert {"embed", "head", "final.norm", "l0.norm1", "l0.norm2b", "l0.mix.k", "l1.mix.dkv", "l1.mix.dkv.norm", "l1.mix.g",
            "l2.mix.conv.b", "l2.mix.A_log", "l2.mix.dt.b", "l3.mix.uk", "l4.mlp.down"} <= names
    assert "l3.mix.dkv" not in names and "l2.norm2" not in names and "l2.mlp.gate" not in names
    needs = model.cache_needs()
    assert [n.kind for n in needs] == ["paged_kv", "paged_kv", "state", "state"]
    assert needs[2].state_shape == (48 * (6 + 3),) and needs[1].tensors[0].width == 24 + 8


@pytest.mark.parametrize("edit,match", [
    (lambda c: c["layers"][3]["mixer"].update(kv_from=4), "earlier"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=0), "latent of its own"),
    (lambda c: c["layers"][3]["mixer"].update(kv_rank=8), "equal"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][2].update(type="mamba7"), "not one of"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=10), "rot"),
    (lambda c: c["layers"][0]["mlp"].update(kind="sparse"), "dense"),
    (lambda c: c["layers"][2]["mixer"].pop("state"), "state"),
])
def test_config_errors(edit, match):
    from pulsar_b200.config import ConfigError, config_from_dict
    raw = copy.deepcopy(BUBO_A)
    edit(raw)
    with pytest.raises(ConfigError, match=match):
        config_from_dict(raw)


def test_plain_mechanisms_agree_with_token_by_token_loops():
    """The oracle's vectorised forms against the equations written out one token and one pair at a time."""
    g = torch.Generator().manual_seed(3)
    x = torch.randn(9, 6, generator=g, dtype=torch.float64)
    taps, bias = torch.randn(6, 3, generator=g, dtype=torch.float64), torch.randn(6, generator=g, dtype=torch.float64)
    got = plain.causal_conv(x, taps, bias)
    for t in range(9):
        for c in range(6):
            want = bias[c] + sum(taps[c, k] * x[t - 2 + k, c] for k in range(3) if t - 2 + k >= 0)
            assert abs(float(got[t, c] - want)) < 1e-12
    v = torch.randn(5, 2, 6, generator=g, dtype=torch.float64)
    turned = plain.rotate_pairs(v, torch.arange(5), 100.0, 4)
    for p in range(5):
        for i in range(2):
            a = p * 100.0 ** (-2.0 * i / 4)
            u, w = v[p, 1, 2 * i], v[p, 1, 2 * i + 1]
            assert abs(float(turned[p, 1, 2 * i] - (u * math.cos(a) - w * math.sin(a)))) < 1e-12
            assert abs(float(turned[p, 1, 2 * i + 1] - (w * math.cos(a) + u * math.sin(a)))) < 1e-12
    assert torch.equal(turned[..., 4:], v[..., 4:])
    q, k, val = (torch.randn(7, 2, 4, generator=g, dtype=torch.float64) for _ in range(3))
    slopes = plain.distance_slopes(2, torch.float64)
    out = plain.dense_attention(q, k, val, 0.5, slopes, chunk=3)
    for i in range(7):
        js = [j for j in range(i + 1) if j // 3 == i // 3]
        s = torch.tensor([float(q[i, 1] @ k[j, 1]) * 0.5 - float(slopes[1]) * (i - j) for j in js], dtype=torch.float64)
        want = (torch.softmax(s, 0)[:, None] * val[js, 1]).sum(0)
        assert float((out[i, 1] - want).abs().max()) < 1e-12


# ------------------------------------------------------------------ GPU
gpu = pytest.mark.gpu


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for name, raw in list(ALONE.items()) + [(n, c[0]) for n, c in CONFIGS.items()]:
        d = tmp_path_factory.mktemp(f"bubo{name}")
        helpers.make_folder(d, copy.deepcopy(raw), 100 + len(out), store_dtype=torch.bfloat16)   # bfloat16 values: both precisions hold them exactly
        out[name] = str(d)
    return out


def _reference(folder, requests):
    cfg, w = helpers.read_folder(folder)
    return {rid: plain.forward(cfg, w, list(toks), torch.float64) for rid, toks in requests.items()}


def _replay(folder, dtype, trace, max_tokens, page_size, max_running=4):
    from pulsar_b200.replay import Replay
    rp = Replay(folder, dtype, max_tokens, page_size=page_size, max_running=max_running)
    got = {}
    for rec, rows in zip(trace.records, trace.rows):
        logits = rp.run_step(rec)
        for i, key in enumerate(rows):
            got[key] = logits[i]
    rp.cache.check_consistency()
    assert rp.cache.live_requests() == []
    assert all(f == g.allocator.n for f, g in zip(rp.cache.n_free_pages(), rp.cache.groups))
    return got, rp


def _compare(got, ref, dtype, what):
    assert got
    worst = 0.0
    for (rid, pos), row in sorted(got.items()):
        err = helpers.rel_err(row, ref[rid][pos])
        worst = max(worst, err)
        assert err < TOL[dtype], f"{what}: request {rid} position {pos}: error {err:.3e} (first wrong place)"
    helpers.report(what, worst, dtype)


def _round64(n):
    return -(-n // 64) * 64


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(ALONE))
def test_each_mechanism_alone(folders, name, dtype):
    rng = random.Random(5)
    toks = helpers.random_tokens(rng, 45, 64)
    ref = _reference(folders[name], {"a": toks})
    got, _ = _replay(folders[name], dtype, helpers.trace_whole(toks), 64, 8)
    _compare(got, ref, dtype, f"alone[{name}] whole")
    got, _ = _replay(folders[name], dtype, helpers.trace_portions(toks, [5, 2, 11, 3, 2]), 64, 4)
    _compare(got, ref, dtype, f"alone[{name}] portions")


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_prompt_tail_and_portions_agree_with_the_plain_logits(folders, name, dtype):
    raw, seed, page = CONFIGS[name]
    rng = random.Random(seed)
    toks = helpers.random_tokens(rng, 93, raw["vocab"])
    ref = _reference(folders[name], {"a": toks})
    for what, trace in (("whole", helpers.trace_whole(toks)), ("tail", helpers.trace_tail(toks, 40)),
                        ("portions", helpers.trace_portions(toks, [7, 2, 13, 2, 5, 17, 3])),
                        ("pairs", helpers.trace_portions(toks[:31], [2]))):
        got, _ = _replay(folders[name], dtype, trace, _round64(len(toks)), page)
        _compare(got, ref, dtype, f"{name} {what}")


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_mixed_batches_with_pages_and_slots_used_again(folders, name, dtype):
    raw, seed, page = CONFIGS[name]
    rng = random.Random(seed + 30)
    lengths = [40, 23, 64, 9, 31, 50, 17, 28, 45, 1, 2]
    requests = {f"r{i}": helpers.random_tokens(rng, n, raw["vocab"]) for i, n in enumerate(lengths)}
    ref = _reference(folders[name], requests)
    trace = helpers.trace_mixed(requests, rng, max_live=3)
    budget = sum(sorted(_round64(n) for n in lengths)[-3:])
    got, rp = _replay(folders[name], dtype, trace, budget, page, max_running=3)      # 11 requests through 3 state slots
    assert len(got) == sum(lengths)
    _compare(got, ref, dtype, f"{name} mixed")


@gpu
def test_a_batch_of_unequal_requests_equals_each_alone(folders):
    raw, seed, page = CONFIGS["A"]
    rng = random.Random(77)
    requests = {f"q{i}": helpers.random_tokens(rng, n, raw["vocab"]) for i, n in enumerate([37, 5, 22])}
    together = helpers.Trace()
    together.step([(rid, toks[:-4], range(len(toks) - 4)) for rid, toks in requests.items()])
    for k in range(4, 0, -1):
        together.step([(rid, toks[len(toks) - k:len(toks) - k + 1], [0]) for rid, toks in requests.items()],
                      end=list(requests) if k == 1 else [])
    both, _ = _replay(folders["A"], "float32", together, 3 * 64, page)
    for rid, toks in requests.items():
        alone, _ = _replay(folders["A"], "float32", helpers.trace_tail(toks, 4, rid), 64, page)
        for key, row in alone.items():
            assert helpers.rel_err(both[key], row) < 2e-6, f"{key}: a batch changed the logits"


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_keeps_the_state(folders, dtype):
    raw, seed, page = CONFIGS["B"]
    rng = random.Random(9)
    toks = helpers.random_tokens(rng, 230, raw["vocab"])
    ref = _reference(folders["B"], {"a": toks})
    got, rp = _replay(folders["B"], dtype, helpers.trace_tail(toks, 220), _round64(len(toks)), page)
    _compare(got, ref, dtype, "long decoding")
    assert rp.runner.graph_replays > 150          # the steps of single tokens ran from a captured graph


def _paged(rows, page_size, order):
    """rows [L, heads, width] -> pool [pages, heads, page, width] with logical page i at page order[i], and the table."""
    L, heads, width = rows.shape
    n_pages = -(-L // page_size)
    pool = torch.zeros(max(order) + 1, heads, page_size, width, dtype=rows.dtype)
    for lp in range(n_pages):
        part = rows[lp * page_size:(lp + 1) * page_size]
        pool[order[lp], :, :part.shape[0]] = part.transpose(0, 1)
    return pool, torch.tensor([order[:n_pages]], dtype=torch.int32)


def _step_context(q_lens, kv_lens):
    """What the attention wrappers read of a step: its device arrays, the lengths on the host, scratch memory."""
    cu = [0]
    for n in q_lens:
        cu.append(cu[-1] + n)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32).cuda()
    return types.SimpleNamespace(cu_q=i32(cu), kv_len=i32(kv_lens), n_seqs=len(q_lens), host=types.SimpleNamespace(q_lens=list(q_lens)),
                                 seq_of_token=i32([s for s, n in enumerate(q_lens) for _ in range(n)]),
                                 scratch=lambda tag, shape, dtype=None: torch.empty(shape, dtype=dtype, device="cuda"))


@gpu
@pytest.mark.parametrize("tiled", [True, False])
@pytest.mark.parametrize("decode", [False, True])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_one_key_that_stands_out_at_every_edge(dtype, decode, tiled):
    """General attention kernel: one key is made to dominate wherever it is visible.  It is put far back among hundreds, on
    both sides of a page border, and just inside and just outside the query's chunk and window; a mask that is one token
    off moves the whole output."""
    from pulsar_b200 import ops
    g = torch.Generator().manual_seed(21)
    L, H, G, D, Dv, page, chunk, window = 389, 4, 2, 24, 16, 16, 50, 70
    order = list(range(40))
    random.Random(4).shuffle(order)
    slopes = plain.distance_slopes(H, torch.float64)
    cases = []
    for mask in ("none", "chunk", "window"):
        last = L - 1
        first_seen = {"none": 0, "chunk": last // chunk * chunk, "window": last - window + 1}[mask]
        spots = {3, 15, 16, 17, 127, 128, last - 1, last, first_seen, first_seen + 1}
        if first_seen > 0:
            spots |= {first_seen - 1, first_seen - 2}
        cases += [(mask, s) for s in sorted(spots)]
    for mask, spot in cases:
        q = torch.randn(L, H, D, generator=g, dtype=torch.float64)
        k = torch.randn(L, G, D, generator=g, dtype=torch.float64)
        v = torch.randn(L, G, Dv, generator=g, dtype=torch.float64)
        q[..., 0] = 3.0                                       # every query looks along dimension 0 ...
        k[spot, :, 0] = 60.0                                  # ... where one key is far larger than the rest
        q, k, v = (t.to(dtype).to(torch.float64) for t in (q, k, v))
        kw = dict(chunk=chunk if mask == "chunk" else None, window=window if mask == "window" else None)
        want = plain.dense_attention(q, k.repeat_interleave(H // G, 1), v.repeat_interleave(H // G, 1), 0.3, slopes, **kw)
        k_pool, table = _paged(k.to(dtype), page, order)
        v_pool, _ = _paged(v.to(dtype), page, order)
        n_q = 1 if decode else L
        ctx = _step_context([n_q], [L])
        out = torch.empty(n_q, H, Dv, dtype=dtype, device="cuda")
        ops.paged_attention_general(ctx, q[L - n_q:].float().cuda().contiguous(), k_pool.cuda(), v_pool.cuda(), out, table.cuda(),
                                    0.3, kw["window"], kw["chunk"], slopes.float().cuda(), tiled=tiled)
        err = float((out.double().cpu() - want[L - n_q:]).abs().max() / want.abs().max())
        assert err < (2e-5 if dtype == torch.float32 else 1e-2), f"mask {mask}, key at {spot}: error {err:.3e}"


@gpu
@pytest.mark.parametrize("dims", [(64, 64), (128, 128), (192, 128)])
def test_tensor_core_kernel_keeps_scores_and_weights_at_float32(dims):
    """The tensor-core form of the general attention (bfloat16 pages, float32 queries split into two halves) against the
    plain one in float64: two sequences of unequal length with cached parts, grouped heads, one dominant key per mask at
    the edges of chunk, window and page.  The bar is far below one bfloat16 rounding of a query or of a softmax weight."""
    from pulsar_b200 import ops
    g = torch.Generator().manual_seed(33)
    D, Dv = dims
    H, G, page, chunk, window = 4, 2, 8, 70, 45
    lens, starts = [233, 97], [40, 0]                     # the first sequence has 40 tokens in the cache already
    order = list(range(64))
    random.Random(6).shuffle(order)
    slopes = plain.distance_slopes(H, torch.float64)
    for mask, spot in (("none", 5), ("chunk", 139), ("chunk", 140), ("window", 187), ("window", 188), ("none", 231), ("chunk", 64)):
        qs, ks, vs, wants = [], [], [], []
        for L, start in zip(lens, starts):
            q = torch.randn(L, H, D, generator=g, dtype=torch.float64)
            k = torch.randn(L, G, D, generator=g, dtype=torch.float64)
            v = torch.randn(L, G, Dv, generator=g, dtype=torch.float64)
            q[..., 0] = 3.0
            if spot < L:
                k[spot, :, 0] = 40.0
            k, v = k.to(torch.bfloat16).double(), v.to(torch.bfloat16).double()
            q = q.float().double()
            kw = dict(chunk=chunk if mask == "chunk" else None, window=window if mask == "window" else None)
            want = plain.dense_attention(q[start:], k.repeat_interleave(H // G, 1), v.repeat_interleave(H // G, 1), 0.11, slopes,
                                         first=start, **kw)
            qs.append(q[start:]); ks.append(k); vs.append(v); wants.append(want)
        # both sequences in one pool: the second one's pages follow the first one's in a shuffled order
        n_pages = [-(-L // page) for L in lens]
        k_pool = torch.zeros(64, G, page, D, dtype=torch.bfloat16)
        v_pool = torch.zeros(64, G, page, Dv, dtype=torch.bfloat16)
        table = torch.zeros(2, max(n_pages), dtype=torch.int32)
        at = 0
        for s, L in enumerate(lens):
            for lp in range(n_pages[s]):
                pid = order[at]; at += 1
                table[s, lp] = pid
                part_k, part_v = ks[s][lp * page:(lp + 1) * page], vs[s][lp * page:(lp + 1) * page]
                k_pool[pid, :, :part_k.shape[0]] = part_k.transpose(0, 1).to(torch.bfloat16)
                v_pool[pid, :, :part_v.shape[0]] = part_v.transpose(0, 1).to(torch.bfloat16)
        ctx = _step_context([L - st for L, st in zip(lens, starts)], lens)
        q_all = torch.cat(qs).float().cuda().contiguous()
        out = torch.empty(q_all.shape[0], H, Dv, dtype=torch.bfloat16, device="cuda")
        ops.paged_attention_general(ctx, q_all, k_pool.cuda(), v_pool.cuda(), out, table.cuda(), 0.11, kw["window"], kw["chunk"],
                                    slopes.float().cuda(), tensor_cores=True)
        want = torch.cat(wants)
        err = float((out.double().cpu() - want).abs().max() / want.abs().max())
        assert err < 6e-3, f"mask {mask}, key at {spot}: error {err:.3e}"          # the output's own bfloat16 rounding: 4e-3
        # against the CUDA-core kernel, which is float32 throughout, the two agree to the output's rounding
        ref = torch.empty_like(out)
        ops.paged_attention_general(ctx, q_all, k_pool.cuda(), v_pool.cuda(), ref, table.cuda(), 0.11, kw["window"], kw["chunk"],
                                    slopes.float().cuda(), tensor_cores=False)
        assert float((out.float() - ref.float()).abs().max() / want.abs().max()) < 8e-3


@gpu
@pytest.mark.parametrize("tiled", [True, False])
def test_value_as_the_leading_part_of_the_key_row(tiled):
    """The layout of latent attention: one pool, the value is the first elements of the key row, one shared head."""
    from pulsar_b200 import ops
    g = torch.Generator().manual_seed(8)
    L, H, rank, rot, page = 75, 5, 24, 8, 4
    rows = torch.randn(L, 1, rank + rot, generator=g, dtype=torch.float64)
    q = torch.randn(L, H, rank + rot, generator=g, dtype=torch.float64)
    rows[40, 0, 1] = 25.0
    q[..., 1] = 2.0
    want = plain.dense_attention(q, rows.expand(L, H, rank + rot), rows[..., :rank].expand(L, H, rank), 0.2)
    pool, table = _paged(rows.float(), page, list(reversed(range(19))))
    ctx = _step_context([L], [L])
    out = torch.empty(L, H, rank, dtype=torch.float32, device="cuda")
    pool = pool.cuda()
    ops.paged_attention_general(ctx, q.float().cuda(), pool, pool, out, table.cuda(), 0.2, key_width=rank + rot, value_width=rank,
                                tiled=tiled)
    assert float((out.double().cpu() - want).abs().max()) < 2e-5


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_small_kernels_against_their_formulas(dtype):
    from pulsar_b200 import ops
    g = torch.Generator().manual_seed(17)
    tol = 1e-5 if dtype == torch.float32 else 1.5e-2
    rnd = lambda *s: torch.randn(*s, generator=g).to(dtype)

    def close(got, want, what):
        err = float((got.double().cpu() - want.double()).abs().max() / want.double().abs().max())
        assert err < tol, f"{what}: {err:.3e}"
    # per-head products on views, with and without the gate
    n, H, K, M = 11, 3, 10, 7
    wide, w, gate = rnd(n, H * (K + 6)), rnd(H, M, K), rnd(n, 5 + H * M)
    a = wide.view(n, H, K + 6)[:, :, :K]
    out = torch.zeros(n, H, M + 3, dtype=torch.float32, device="cuda")
    w_km = w.transpose(1, 2).contiguous().cuda()          # the kernel takes each head's weights [inputs, outputs]
    ops.heads_linear(a.cuda(), w_km, out[:, :, :M])
    close(out[:, :, :M], torch.einsum("nhk,hmk->nhm", a.double(), w.double()), "heads_linear")
    assert float(out[:, :, M:].abs().max()) == 0.0
    gated = torch.empty(n, H, M, dtype=dtype, device="cuda")
    ops.heads_linear(a.cuda(), w_km, gated, gate.cuda()[:, 5:])
    close(gated, torch.einsum("nhk,hmk->nhm", a.double(), w.double()) * torch.sigmoid(gate[:, 5:].double()).view(n, H, M), "gated heads")
    # the norm behind a sublayer, the addition and the next norm in one kernel
    for width in (52, 50, 4100):                # rows in registers (one and two vectors a thread), and the plain kernel
        residual, delta = torch.randn(n, width, generator=g), rnd(n, width)
        w_post, w_next = 1 + 0.1 * torch.randn(width, generator=g), 1 + 0.1 * torch.randn(width, generator=g)
        res_dev, normed = residual.cuda(), torch.empty(n, width, dtype=dtype, device="cuda")
        ops.post_norm_add(res_dev, delta.cuda(), w_post.cuda(), 1e-5, w_next.cuda(), 2e-5, normed)
        want = residual.double() + plain.rms_norm(delta.double(), w_post.double(), 1e-5)
        close(res_dev, want, f"post_norm_add ({width}): the stream")
        close(normed, plain.rms_norm(want, w_next.double(), 2e-5), f"post_norm_add ({width}): the next norm")
        res_dev = residual.cuda()
        ops.post_norm_add(res_dev, delta.cuda(), w_post.cuda(), 1e-5)
        close(res_dev, want, f"post_norm_add ({width}) without a next norm")
    # clamped gating
    gu = (3 * torch.randn(n, 2 * 18, generator=g)).to(dtype)
    act = torch.empty(n, 18, dtype=dtype, device="cuda")
    ops.clamped_glu(gu.cuda(), act, 1.25, 1.702)
    gg, uu = gu[:, :18].double().clamp(max=1.25), gu[:, 18:].double().clamp(-1.25, 1.25)
    close(act, gg * torch.sigmoid(1.702 * gg) * (uu + 1), "clamped_glu")


@gpu
@pytest.mark.parametrize("rows", [1, 8, 16, 40, 200])
def test_clamped_gating_inside_the_gate_up_product(rows):
    """The gate/up product with the clamped gating in its epilogue (the weight-streaming kernel up to 16 rows, the tcgen05
    kernel above 128) and the unfused path between them, against the formula; SwiGLU through the same kernels is unchanged."""
    from pulsar_b200 import ops
    g = torch.Generator().manual_seed(rows)
    width, inter = 128, 192
    a = torch.randn(rows, width, generator=g).to(torch.bfloat16)
    w = (torch.randn(2 * inter, width, generator=g) * 0.3).to(torch.bfloat16)
    ctx = types.SimpleNamespace(scratch=lambda tag, shape, dtype=None: torch.empty(shape, dtype=dtype, device="cuda"))
    gu = a.double() @ w.double().T
    gate, up = gu[:, :inter], gu[:, inter:]
    out = torch.empty(rows, inter, dtype=torch.bfloat16, device="cuda")
    ops.gated_linear(ctx, a.cuda(), w.cuda(), out, gating=(1.5, 1.702, 1.0))
    gg, uu = gate.clamp(max=1.5), up.clamp(-1.5, 1.5)
    want = gg * torch.sigmoid(1.702 * gg) * (uu + 1)
    assert float((out.double().cpu() - want).abs().max() / want.abs().max()) < 1e-2
    ops.gated_linear(ctx, a.cuda(), w.cuda(), out)
    want = gate * torch.sigmoid(gate) * up
    assert float((out.double().cpu() - want).abs().max() / want.abs().max()) < 1e-2


@gpu
def test_scan_kernels_carry_their_state_across_portions():
    """Convolution and scan over two sequences whose tokens arrive in portions of 1 to 7, against the whole sequences
    in one go; the second sequence's slot was used before and zeroed."""
    from pulsar_b200 import ops
    g = torch.Generator().manual_seed(31)
    inner, S, R, taps = 20, 70, 4, 4
    lens = [23, 9]
    arena = torch.randn(3, inner * (S + taps - 1), generator=g).cuda()
    slots = [2, 0]
    arena[slots] = 0.0
    w_dt, dt_b = torch.randn(inner, R, generator=g) * 0.5, torch.randn(inner, generator=g) - 1
    a_log, d_skip = torch.log(0.5 + 4 * torch.rand(inner, S, generator=g)), torch.randn(inner, generator=g)
    conv_w, conv_b = torch.randn(inner, taps, generator=g) * 0.5, torch.randn(inner, generator=g) * 0.1
    xz = [torch.randn(n, 2 * inner, generator=g) for n in lens]
    bc = [torch.randn(n, R + 2 * S, generator=g) for n in lens]      # stands for the projection of the convolution's output
    want = []
    for s in range(2):
        x = plain.silu(plain.causal_conv(xz[s][:, :inner].double(), conv_w.double(), conv_b.double()))
        dt = plain.softplus(bc[s][:, :R].double() @ w_dt.double().T + dt_b.double())
        state = torch.zeros(inner, S, dtype=torch.float64)
        ys = []
        for t in range(lens[s]):
            state = torch.exp(dt[t][:, None] * -torch.exp(a_log.double())) * state + (dt[t] * x[t])[:, None] * bc[s][t, R:R + S].double()[None]
            ys.append((state @ bc[s][t, R + S:].double() + d_skip.double() * x[t]) * plain.silu(xz[s][t, inner:].double()))
        want.append(torch.stack(ys))
    at = [0, 0]
    got = [[], []]
    cuts = [[3, 1, 7, 2, 1, 1, 8], [1, 2, 6]]
    dev = lambda t: t.cuda().contiguous()
    for step in range(7):
        live = [s for s in range(2) if step < len(cuts[s])]
        ns = [cuts[s][step] for s in live]
        rows_xz = torch.cat([xz[s][at[s]:at[s] + n] for s, n in zip(live, ns)])
        rows_bc = torch.cat([bc[s][at[s]:at[s] + n] for s, n in zip(live, ns)])
        cu = [0]
        for n in ns:
            cu.append(cu[-1] + n)
        ctx = types.SimpleNamespace(cu_q=dev(torch.tensor(cu, dtype=torch.int32)), n_seqs=len(live),
                                    seq_of_token=dev(torch.tensor([i for i, n in enumerate(ns) for _ in range(n)], dtype=torch.int32)),
                                    state_slots=dev(torch.tensor([slots[s] for s in live], dtype=torch.int32)))
        x = torch.empty(sum(ns), inner, device="cuda")
        ops.causal_conv_silu(ctx, dev(rows_xz), inner, dev(conv_w), dev(conv_b), arena, inner * S, x)
        y = torch.empty(sum(ns), inner, device="cuda")
        ops.selective_scan(ctx, x, dev(rows_xz), dev(rows_bc), dev(w_dt), dev(dt_b), dev(a_log), dev(d_skip), arena, inner * S, taps, y)
        for i, (s, n) in enumerate(zip(live, ns)):
            got[s].append(y[cu[i]:cu[i + 1]].cpu())
            at[s] += n
    for s in range(2):
        err = float((torch.cat(got[s]).double() - want[s]).abs().max() / want[s].abs().max())
        assert err < 2e-5, f"sequence {s}: {err:.3e}"
    assert float(arena[1].abs().min()) > 0.0        # the slot nobody used was left alone


@gpu
@pytest.mark.parametrize("chunked", [False, True])
def test_scan_kernels_for_portions(chunked):
    """The two scan kernels for portions (step sizes from a product of their own) over three sequences of 1, 300 and 517
    tokens with states carried in: against the recurrence written out token by token in float64."""
    from pulsar_b200 import ops
    g = torch.Generator().manual_seed(51)
    inner, S, taps = 21, 12, 3
    lens, slots = [1, 300, 517], [3, 0, 1]
    arena = (0.3 * torch.randn(4, inner * (S + taps - 1), generator=g)).cuda()
    start = arena.clone().cpu()
    dt_b, d_skip = torch.randn(inner, generator=g) - 1, torch.randn(inner, generator=g)
    a_log = torch.log(0.02 + 2 * torch.rand(inner, S, generator=g))            # slow decays too: far tokens stay in the state
    n = sum(lens)
    x, xz = torch.randn(n, inner, generator=g), torch.randn(n, 2 * inner, generator=g)
    bc, dt_pre = torch.randn(n, 2 * S, generator=g), torch.randn(n, inner, generator=g)
    want, at = [], 0
    for L, slot in zip(lens, slots):
        state = start[slot, :inner * S].view(inner, S).double()
        for t in range(at, at + L):
            dt = plain.softplus(dt_pre[t].double() + dt_b.double())
            state = torch.exp(dt[:, None] * -torch.exp(a_log.double())) * state + (dt * x[t].double())[:, None] * bc[t, :S].double()[None]
            want.append((state @ bc[t, S:].double() + d_skip.double() * x[t].double()) * plain.silu(xz[t, inner:].double()))
        at += L
    want = torch.stack(want)
    ctx = _step_context(lens, lens)
    ctx.state_slots = torch.tensor(slots, dtype=torch.int32).cuda()
    y = torch.empty(n, inner, device="cuda")
    dev = lambda t: t.cuda().contiguous()
    ops.selective_scan_prompt(ctx, dev(x), dev(xz), dev(bc), dev(dt_pre), dev(dt_b), dev(a_log), dev(d_skip), arena, inner * S, taps, y,
                              chunked=chunked)
    err = float((y.double().cpu() - want).abs().max() / want.abs().max())
    assert err < 2e-5, f"{err:.3e}"
    assert torch.equal(arena[2].cpu(), start[2])             # the slot nobody used
    tail = arena[1, inner * S:].view(inner, taps - 1).cpu()      # the last inputs of the 517-token sequence
    assert torch.equal(tail, xz[n - (taps - 1):, :inner].T.contiguous())


@gpu
def test_greedy_generation_through_the_engine(folders):
    from pulsar_b200.api import generate
    raw, seed, page = CONFIGS["A"]
    cfg, w = helpers.read_folder(folders["A"])
    rng = random.Random(41)
    prompts = [helpers.random_tokens(rng, n, raw["vocab"]) for n in (19, 4, 33)]
    got = generate(folders["A"], prompts, 12, dtype="float32", page_size=page, num_pages=40, max_sessions=4, max_running=2,
                   max_chunk_size=7, device="cuda:0")
    assert got == [plain.greedy_generate(cfg, w, p, 12) for p in prompts]
    got16 = generate(folders["A"], prompts, 5, dtype="bfloat16", page_size=page, num_pages=40, max_sessions=4, max_running=3,
                     max_chunk_size=16, device="cuda:0")
    for p, new in zip(prompts, got16):
        seq = list(p)
        for tok in new:
            row = plain.forward(cfg, w, seq, torch.float64)[-1]
            assert float(row.max() - row[tok]) <= TOL["bfloat16"] * float(row.abs().max())
            seq.append(tok)


@gpu
def test_command_line_and_trace_program(folders, tmp_path):
    """The framework's two programs on a Bubotar folder: greedy tokens from bin/pulsar-generate, and logits from
    bin/trace_run fed with steps on its standard input (a prompt in two portions, then single tokens)."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    raw, seed, page = CONFIGS["B"]
    cfg, w = helpers.read_folder(folders["B"])
    out = subprocess.run([sys.executable, os.path.join(root, "bin", "pulsar-generate"), "--model", folders["B"], "--dtype", "float32",
                          "--prompt_ids", "5,4,3,2,1,0,7", "--prompt_ids", "9 8", "--gen_tokens", "6", "--max_pages", "64", "--eos_id",
                          "-1", "--json"], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr
    got = json.loads(out.stdout.strip().splitlines()[-1])["outputs"]
    assert got == [plain.greedy_generate(cfg, w, p, 6) for p in ([5, 4, 3, 2, 1, 0, 7], [9, 8])]
    rng = random.Random(3)
    toks = helpers.random_tokens(rng, 40, raw["vocab"])
    trace = helpers.Trace()
    trace.step([("x", toks[:21], [20])])
    trace.step([("x", toks[21:37], [0, 15])])
    for i in range(37, 40):
        trace.step([("x", toks[i:i + 1], [0])], end=["x"] if i == 39 else [])
    run = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", folders["B"], "--dtype", "float32", "--out", str(tmp_path),
                          "--max-tokens", "64"], input=trace.lines(), capture_output=True, text=True, timeout=600)
    assert run.returncode == 0, run.stderr
    assert [ln for ln in run.stdout.splitlines() if ln.startswith("done ")] == [f"done {i}" for i in range(len(trace.records))]
    ref = plain.forward(cfg, w, toks, torch.float64)
    for i, rows in enumerate(trace.rows):
        got = torch.from_file(str(tmp_path / f"{i}.f32"), size=len(rows) * raw["vocab"], dtype=torch.float32).view(len(rows), -1)
        for j, (_, pos) in enumerate(rows):
            assert helpers.rel_err(got[j], ref[pos]) < TOL["float32"]
