"""Topunex through the engine against the plain implementation (tests/plain/topunex_plain.py): configuration and the
oracle's own mechanisms on the CPU; on a GPU each mechanism alone, prompts against token-by-token decoding, portions
down to two tokens, mixed batches with pages and slots used again, crafted keys at the edges of the window, of the
kept first keys and of pages, the sink and the cap on the scores, the router and the experts, long decoding, and
greedy generation through the public entry point."""
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
from plain import topunex_plain as plain


def attn(heads, kv_heads, dim, size=None, keep_first=0, rot_dims=None, base=10000.0, scaling=None, softcap=None, scale=None):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=dim, scale=scale or 1.0 / math.sqrt(dim), softcap=softcap)
    if rot_dims:
        m["rot"] = dict(base=base, dims=rot_dims, scaling=scaling)
    if size is not None or keep_first:
        m["mask"] = dict(size=size, keep_first=keep_first)
    return m


def dense(ff):
    return dict(kind="dense", ff=ff)


def moe(experts, top, ff, limit=1.5, scale=1.0, shared=None):
    m = dict(kind="moe", expert=dict(ff=ff, limit=limit), router=dict(experts=experts, top=top, scale=scale))
    if shared is not None:
        m["shared"] = dict(ff=shared[0], limit=shared[1])
    return m


def layer(mixer, mlp=None):
    return dict(type="attention", mixer=mixer, mlp=mlp)


def config(layers, vocab, width, eps=1e-5):
    return dict(architecture="Topunex", vocab=vocab, width=width, norm=dict(eps=eps), layers=layers)


SCALING = dict(factor=4.0, low=1.0, high=3.0, original=64)          # all three branches of the rescaling occur at 16 dims
# Every size differs between the configurations: odd head counts, one key/value head, as many key/value heads as query
# heads, the whole head or a part of it rotating, windows that no page size divides, kept first keys of more than a
# tile and of none, layers without a cap, without rotation, without a mask and without a feed-forward, one expert of one.
TOPU_A = config([
    layer(attn(4, 2, 16, size=11, keep_first=3, rot_dims=8, scaling=SCALING, softcap=5.0), dense(72)),
    layer(attn(6, 3, 8, size=23, keep_first=5, rot_dims=8, base=500.0, softcap=30.0), moe(5, 2, 24, limit=1.0, scale=1.5, shared=(40, 2.0))),
    layer(attn(2, 1, 24, size=9, rot_dims=12, scaling=dict(factor=8.0, low=1.0, high=4.0, original=32))),
    layer(attn(3, 3, 16, keep_first=0, rot_dims=16), moe(4, 1, 32, limit=2.5, scale=0.7)),
], vocab=180, width=48, eps=1e-5)
TOPU_B = config([
    layer(attn(5, 1, 12, size=40, keep_first=34, rot_dims=4, base=77.0, softcap=8.0), moe(7, 3, 16, shared=(24, 1.5), scale=2.0)),
    layer(attn(2, 2, 32, size=6, keep_first=1, softcap=12.0), dense(56)),
    layer(attn(8, 4, 8, size=150, keep_first=2, rot_dims=8, scaling=SCALING)),
    layer(attn(4, 2, 20, size=17, keep_first=17, rot_dims=20, base=3000.0), moe(3, 3, 20, limit=0.8)),
    layer(attn(1, 1, 40, rot_dims=10, softcap=2.0), dense(64)),
], vocab=131, width=40, eps=3e-6)
# head sizes at which the bfloat16 engine's prompt attention runs on the tensor cores
TOPU_C = config([
    layer(attn(4, 2, 64, size=70, keep_first=37, rot_dims=32, scaling=SCALING, softcap=15.0), moe(6, 2, 32, shared=(48, 1.5))),
    layer(attn(2, 1, 128, size=33, keep_first=4, rot_dims=64, softcap=25.0), dense(96)),
], vocab=150, width=64, eps=1e-6)
ALONE = {
    "attention": config([layer(attn(4, 2, 16, size=13, keep_first=4, rot_dims=8, scaling=SCALING, softcap=6.0))], vocab=64, width=40),
    "attention_plain": config([layer(attn(3, 1, 12))], vocab=64, width=40),
    "dense": config([layer(attn(2, 2, 8, rot_dims=8), dense(56))], vocab=64, width=40),
    "moe": config([layer(attn(2, 1, 8, size=20), moe(6, 2, 24, limit=1.2, scale=1.5))], vocab=64, width=40),
    "moe_shared": config([layer(attn(2, 1, 8, keep_first=2, size=5), moe(4, 3, 16, shared=(32, 0.9)))], vocab=64, width=40),
}
CONFIGS = {"A": (TOPU_A, 21, 8), "B": (TOPU_B, 22, 4), "C": (TOPU_C, 23, 16)}      # config, seed, page size


# ------------------------------------------------------------------ configuration (CPU)
def test_config_becomes_parts():
    from pulsar_b200.config import config_from_dict
    from pulsar_b200.models import build_model
    cfg = config_from_dict(copy.deepcopy(TOPU_A))
    spec = cfg.model_spec()
    assert [(c.block, c.cache) for c in spec.run_order] == [(0, 0), (1, 1), (2, 2), (3, 3)]
    assert all(b.kind == "postnorm" and b.mixer.kind == "attention" and b.mixer_norm is None for b in spec.blocks)
    assert [None if b.feed_forward is None else b.feed_forward.kind for b in spec.blocks] == ["swiglu", "moe", None, "moe"]
    m0, m3 = spec.blocks[0].mixer, spec.blocks[3].mixer
    assert (m0.window, m0.keep_first, m0.softcap, m0.position.rotary_dim, m0.position.scaling) == (11, 3, 5.0, 8, (4.0, 1.0, 3.0, 64.0))
    assert (m3.window, m3.keep_first, m3.softcap, m3.position.scaling) == (None, 0, None, None)
    assert m0.values_from_keys and m0.sinks and m0.bias and m0.output_gate and not m0.qk_norm_weight and m0.qk_norm_eps == 1e-5
    ff1 = spec.blocks[1].feed_forward
    assert (ff1.option("experts"), ff1.option("top"), ff1.option("router_scale"), ff1.option("limit")) == (5, 2, 1.5, 1.0)
    assert ff1.option("shared").intermediate == 40 and ff1.option("shared").option("limit") == 2.0
    assert spec.blocks[3].feed_forward.option("shared") is None
    assert cfg.to_dict() == TOPU_A
    model = build_model(cfg, torch.float32)
    names = {w.name for w in model.weight_specs()}
    assert {"embed", "head", "final.norm", "l0.norm1", "l0.norm2", "l0.mix.q", "l0.mix.q.b", "l0.mix.k.b", "l0.mix.g", "l0.mix.o.b",
            "l0.mix.sink", "l0.mlp.gate.b", "l0.mlp.down.b", "l1.mlp.e4.up", "l1.mlp.router", "l1.mlp.shared.down", "l3.mlp.e3.down"} <= names
    assert not {"l0.mix.v", "l2.norm2", "l2.mlp.gate", "l3.mlp.shared.gate", "l1.mlp.e5.gate", "l1.mlp.e0.gate.b"} & names
    needs = model.cache_needs()
    assert [n.kind for n in needs] == ["paged_kv"] * 4 and needs[1].tensors[0].heads == 3 and needs[1].tensors[1].width == 8
    # pages behind a window go back to the pool, those of the kept first keys stay
    assert (needs[0].window, needs[0].keep_first) == (11, 3) and (needs[2].window, needs[2].keep_first) == (9, 0)
    assert needs[3].window is None and needs[3].keep_first == 0


@pytest.mark.parametrize("edit,match", [
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][0]["mixer"].update(vdim=8), "vdim"),
    (lambda c: c["layers"][0].update(type="mamba1"), "attention"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "rot"),
    (lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].update(high=0.5), "high"),
    (lambda c: c["layers"][0]["mixer"]["mask"].update(keep_first=-1), "keep_first"),
    (lambda c: c["layers"][0]["mlp"].update(kind="sparse"), "dense"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=9), "top"),
    (lambda c: c["layers"][1]["mlp"]["expert"].pop("ff"), "ff"),
    (lambda c: c["layers"][0]["mixer"].pop("scale"), "scale"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_config_errors(edit, match):
    from pulsar_b200.config import ConfigError, config_from_dict
    raw = copy.deepcopy(TOPU_A)
    edit(raw)
    with pytest.raises(ConfigError, match=match):
        config_from_dict(raw)


def test_plain_mechanisms_agree_with_loops_over_single_numbers():
    """The oracle's vectorised forms against the equations written out one token and one pair at a time."""
    g = torch.Generator().manual_seed(3)
    f = plain.rotary_frequencies(100.0, 16, SCALING)
    kinds = set()
    for i in range(8):
        plain_f = 100.0 ** (-2.0 * i / 16)
        wavelength = 2 * math.pi / plain_f
        if wavelength < 64 / 3.0:
            want, kind = plain_f, "kept"
        elif wavelength > 64 / 1.0:
            want, kind = plain_f / 4.0, "divided"
        else:
            s = (64 / wavelength - 1.0) / (3.0 - 1.0)
            want, kind = (1 - s) * plain_f / 4.0 + s * plain_f, "blended"
        kinds.add(kind)
        assert abs(float(f[i]) - want) < 1e-15
    assert kinds == {"kept", "divided", "blended"}
    v = torch.randn(5, 2, 10, generator=g, dtype=torch.float64)
    turned = plain.rotate_halves(v, torch.arange(5), plain.rotary_frequencies(50.0, 6, None))
    for p in range(5):
        for i in range(3):
            a = p * 50.0 ** (-2.0 * i / 6)
            u, w = v[p, 1, i], v[p, 1, i + 3]
            assert abs(float(turned[p, 1, i] - (u * math.cos(a) - w * math.sin(a)))) < 1e-12
            assert abs(float(turned[p, 1, i + 3] - (w * math.cos(a) + u * math.sin(a)))) < 1e-12
    assert torch.equal(turned[..., 6:], v[..., 6:])
    vis = plain.visible_keys(12, 4, 2)
    for i in range(12):
        for j in range(12):
            assert bool(vis[i, j]) == (j <= i and (i - j < 4 or j < 2))
    assert bool(plain.visible_keys(9, None, 0)[8, 0])
    scores = torch.randn(2, 6, 6, generator=g, dtype=torch.float64)
    sink = torch.tensor([0.3, -1.0], dtype=torch.float64)
    p = plain.softmax_with_sink(scores, vis[:6, :6][None], sink)
    for h in range(2):
        for i in range(6):
            js = [j for j in range(6) if vis[i, j]]
            den = sum(math.exp(float(scores[h, i, j])) for j in js) + math.exp(float(sink[h]))
            for j in range(6):
                want = math.exp(float(scores[h, i, j])) / den if j in js else 0.0
                assert abs(float(p[h, i, j]) - want) < 1e-12
    h_in, router = torch.randn(7, 5, generator=g, dtype=torch.float64), torch.randn(6, 5, generator=g, dtype=torch.float64)
    idx, wt = plain.routed(h_in, router, 2, 1.5)
    for t in range(7):
        s = [1 / (1 + math.exp(-float(router[e] @ h_in[t]))) for e in range(6)]
        best = sorted(range(6), key=lambda e: -s[e])[:2]
        assert sorted(idx[t].tolist()) == sorted(best)
        for c in range(2):
            assert abs(float(wt[t, c]) - 1.5 * s[int(idx[t, c])]) < 1e-12


def test_the_engines_rotary_frequencies_are_the_plain_ones():
    from pulsar_b200.config.specs import PositionSpec
    from pulsar_b200.parts.rope import RotaryEmbedding
    for dims, base, sc in ((16, 100.0, SCALING), (8, 30000.0, dict(factor=6.0, low=2.0, high=5.0, original=1024)), (6, 10.0, None)):
        scaling = None if sc is None else (sc["factor"], sc["low"], sc["high"], sc["original"])
        rope = RotaryEmbedding(PositionSpec("rope", 32, dims, base, scaling))
        want = plain.rotary_frequencies(base, dims, sc)
        assert all(abs(rope.frequency(j) - float(want[j])) <= 1e-15 * float(want[j]) * 4 for j in range(dims // 2))


# ------------------------------------------------------------------ GPU
gpu = pytest.mark.gpu


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for name, raw in list(ALONE.items()) + [(n, c[0]) for n, c in CONFIGS.items()]:
        d = tmp_path_factory.mktemp(f"topu{name}")
        # bfloat16 values: both precisions hold them exactly.  Wider weights than the default make every sublayer count.
        helpers.make_folder(d, copy.deepcopy(raw), 300 + len(out), store_dtype=torch.bfloat16, std=0.15)
        out[name] = str(d)
    return out


CLOSE_CALL = 0.03       # relative margin of a router's choice below which bfloat16 rounding may choose otherwise


class _Reference(dict):
    """request -> plain logits; ``sure[request]``: the positions before the request's first close call of a router.  A token
    that is routed otherwise moves its own logits and, through its keys, those of the tokens behind it, so the bfloat16
    engine is held to the bar up to there only (the float32 engine everywhere; the experts' bfloat16 kernels are held to
    their formulas with given routes in tests of their own)."""
    sure = None


def _reference(folder, requests):
    cfg, w = helpers.read_folder(folder)
    ref = _Reference()
    ref.sure = {}
    for rid, toks in requests.items():
        margins = []
        ref[rid] = plain.forward(cfg, w, list(toks), torch.float64, margins=margins)
        close = [int(torch.nonzero(m < CLOSE_CALL)[0]) for m in margins if bool((m < CLOSE_CALL).any())]
        ref.sure[rid] = min(close) if close else len(toks)
    return ref


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
        if dtype == "bfloat16" and pos >= ref.sure[rid]:
            continue
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
    for what, trace in (("whole", helpers.trace_whole(toks)), ("tail", helpers.trace_tail(toks, 60)),
                        ("portions", helpers.trace_portions(toks, [7, 2, 13, 2, 5, 17, 3])),
                        ("large portions", helpers.trace_portions(toks, [40, 18, 33])),
                        ("pairs", helpers.trace_portions(toks[:47], [2]))):
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
    got, rp = _replay(folders[name], dtype, trace, budget, page, max_running=3)      # 11 requests through 3 slots
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
def test_long_decoding_passes_the_windows_over_decoded_tokens(folders, dtype):
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


def _dense_attention(q, k, v, scale, window, keep_first, softcap, sink, first=0):
    """q [Lq, H, D] at positions first .. first + Lq - 1 over keys/values [L, H, D], with the oracle's mask, cap and sink."""
    L = k.shape[0]
    vis = plain.visible_keys(L, window, keep_first)[first:first + q.shape[0]]
    scores = plain.capped(torch.einsum("ihd,jhd->hij", q, k) * scale, softcap)
    p = plain.softmax_with_sink(scores, vis[None], sink)
    return torch.einsum("hij,jhd->ihd", p, v)


@gpu
@pytest.mark.parametrize("kernel", ["tiled", "plain", "tensor_cores"])
@pytest.mark.parametrize("decode", [False, True])
def test_one_key_that_stands_out_at_every_edge(decode, kernel):
    """The general attention kernels with a window, kept first keys, a cap and a sink: one key is made to dominate wherever it
    is visible.  It is put among the kept keys and just behind them, far back among hundreds, on both sides of a page
    border and of a tile border, and just inside and just outside the query's window; a mask that is one token off
    moves the whole output.  The sink is made large once, so that leaving it out doubles the output."""
    from pulsar_b200 import ops
    dtype = torch.bfloat16 if kernel == "tensor_cores" else torch.float32
    g = torch.Generator().manual_seed(21)
    L, H, G, D, page = 389, 4, 2, 64 if kernel == "tensor_cores" else 24, 16
    order = list(range(40))
    random.Random(4).shuffle(order)
    cases = []
    for window, keep, cap, big_sink in ((70, 37, 9.0, False), (70, 0, None, False), (33, 3, 50.0, True), (None, 0, 4.0, True),
                                        (200, 64, 11.0, False), (5, 1, None, False)):
        last = L - 1
        first_seen = 0 if window is None else last - window + 1
        spots = {0, 15, 16, 31, 32, 127, 128, last - 1, last, first_seen, first_seen + 1}
        if window is not None:
            spots |= {first_seen - 1, first_seen - 2}
        if keep:
            spots |= {keep - 1, keep, keep + 1}
        cases += [(window, keep, cap, big_sink, s) for s in sorted(spots)]
    for window, keep, cap, big_sink, spot in cases:
        q = torch.randn(L, H, D, generator=g, dtype=torch.float64)
        k = torch.randn(L, G, D, generator=g, dtype=torch.float64)
        v = torch.randn(L, G, D, generator=g, dtype=torch.float64)
        q[..., 0] = 3.0                                       # every query looks along dimension 0 ...
        k[spot, :, 0] = 60.0                                  # ... where one key is far larger than the rest
        sink = torch.randn(H, generator=g, dtype=torch.float64)
        scale = 0.3
        if big_sink:                                          # as heavy as everything the last query sees
            sink[:] = (cap if cap else 3.0 * 60.0 * scale) + 0.0
        k, v = k.to(dtype).double(), v.to(dtype).double()
        q = q.float().double()
        n_q = 1 if decode else (L if kernel != "plain" else 60)
        want = _dense_attention(q[L - n_q:], k.repeat_interleave(H // G, 1), v.repeat_interleave(H // G, 1), scale, window, keep, cap,
                                sink, first=L - n_q)
        k_pool, table = _paged(k.to(dtype), page, order)
        v_pool, _ = _paged(v.to(dtype), page, order)
        ctx = _step_context([n_q], [L])
        out = torch.empty(n_q, H, D, dtype=dtype, device="cuda")
        ops.paged_attention_general(ctx, q[L - n_q:].float().cuda().contiguous(), k_pool.cuda(), v_pool.cuda(), out, table.cuda(),
                                    scale, window, None, None, tiled=kernel != "plain",
                                    tensor_cores=True if (kernel == "tensor_cores" and not decode) else False,
                                    keep_first=keep, softcap=cap, sinks=sink.float().cuda())
        err = float((out.double().cpu() - want).abs().max() / want.abs().max())
        assert err < (2e-5 if dtype == torch.float32 else 8e-3), f"window {window} keep {keep} cap {cap}, key at {spot}: error {err:.3e}"


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_small_kernels_against_their_formulas(dtype):
    from pulsar_b200 import ops
    g = torch.Generator().manual_seed(17)
    tol = 1e-5 if dtype == torch.float32 else 1.5e-2
    rnd = lambda *s: torch.randn(*s, generator=g)

    def close(got, want, what, bar=tol):
        err = float((got.double().cpu() - want.double()).abs().max() / want.double().abs().max())
        assert err < bar, f"{what}: {err:.3e}"
    # the kernel between the projection and the attention: bias, value copy, rotation of a part, unit norm, pages
    n, H, G, D, rot, page = 13, 3, 1, 20, 12, 4
    rows = rnd(n, (H + G) * D + 7)                            # wider rows: gate columns ride behind q | k
    qb, kb = rnd(H * D), rnd(G * D)
    pos = torch.tensor([5, 6, 7, 0, 1, 300, 301, 302, 303, 304, 305, 306, 2])
    freqs = plain.rotary_frequencies(100.0, rot, SCALING)
    ang = pos.double()[:, None] * freqs[None]
    slots = torch.tensor([9, 10, 11, 0, 1, 30, 31, 4, 5, 6, 7, 20, 21], dtype=torch.int32)
    q_out = torch.empty(n, H, D, device="cuda")
    k_pool, v_pool = (torch.zeros(8, G, page, D, dtype=dtype, device="cuda") for _ in range(2))
    ops.qk_prepare(rows.cuda(), q_out, k_pool, v_pool, slots.cuda(), torch.cos(ang).float().cuda(), torch.sin(ang).float().cuda(),
                   H, G, D, rot, page, qb.cuda(), kb.cuda(), 1e-5, True)
    q = (rows[:, :H * D] + qb).double().view(n, H, D)
    k = (rows[:, H * D:(H + G) * D] + kb).double().view(n, G, D)
    close(q_out, plain.rms_norm(plain.rotate_halves(q, pos, freqs), None, 1e-5), "prepared queries", 1e-5)
    want_k = plain.rms_norm(plain.rotate_halves(k, pos, freqs), None, 1e-5)
    for t in range(n):
        s = int(slots[t])
        close(k_pool[s // page, :, s % page], want_k[t], "key page")
        close(v_pool[s // page, :, s % page], k[t], "value page")
    # the kernel behind a sublayer: rows of 16-byte pieces (held in registers), odd rows, and rows of two pieces a thread
    for width in (44, 45, 4200):
        res, delta, bias, w = rnd(n, width), rnd(n, width).to(dtype), rnd(width), 1 + 0.1 * rnd(width)
        stream = res.clone().cuda()
        out = torch.empty(n, width, dtype=dtype, device="cuda")
        ops.post_norm_add_bias(stream, delta.cuda(), bias.cuda(), w.cuda(), 1e-5, out)
        want = res.double() + plain.rms_norm(delta.double() + bias.double(), w.double(), 1e-5)
        close(stream, want, f"stream of width {width}", 1e-6)
        close(out, want, "rounded stream")
        ops.post_norm_add_bias(stream, None, None, None, 0.0, out)
        close(out, want, "copy of the stream")
        ops.post_norm_add_bias(stream, delta.cuda(), None, w.cuda(), 1e-5, None)
        close(stream, want + plain.rms_norm(delta.double(), w.double(), 1e-5), "without bias and copy", 1e-6)
    # gated units with biases; gate on the heads; bias alone
    inter = 18
    gu, b = rnd(n, 2 * inter), rnd(2 * inter)
    act = torch.empty(n, inter, dtype=dtype, device="cuda")
    ops.glu_bias(gu.cuda(), b.cuda(), act)
    gg, uu = (gu[:, :inter] + b[:inter]).double(), (gu[:, inter:] + b[inter:]).double()
    close(act, gg * torch.sigmoid(gg) * uu, "biased swiglu")
    ops.glu_bias(gu.to(dtype).cuda(), None, act, gating=(0.7, 1.702, 1.0))
    gg, uu = gu[:, :inter].to(dtype).double().clamp(max=0.7), gu[:, inter:].to(dtype).double().clamp(-0.7, 0.7)
    close(act, gg * torch.sigmoid(1.702 * gg) * (uu + 1), "clamped unit")
    x, gate = rnd(n, 30).to(dtype), rnd(n, 41)
    xd = x.clone().cuda()
    ops.sigmoid_gate_strided(xd, gate.cuda()[:, 11:])
    close(xd, x.double() * torch.sigmoid(gate[:, 11:].double()), "gate on the heads")
    xd = x.clone().cuda()
    ops.add_bias(xd, bias[:30].contiguous().cuda())
    close(xd, x.double() + bias[:30].double(), "bias")


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_router_and_experts_against_their_formulas(dtype):
    """The router's choice with ties and a clear winner, weights with and without renormalisation, and the experts' products
    for tokens that chose different experts, against loops over tokens and experts in float64."""
    from pulsar_b200 import ops
    g = torch.Generator().manual_seed(29)
    n, width, E, top, ff = 9, 40, 7, 3, 24
    h = torch.randn(n, width, generator=g).to(dtype)
    router = torch.randn(E, width, generator=g) * 0.3
    router[5] = router[2]                                     # two experts always tie: the lower index goes first
    h[0] = 0.0                                                # all scores 0.5: experts 0, 1, 2 in this order
    router[6] += 4.0 * h[3].float() / float(h[3].float().norm())      # a clear winner for token 3
    ids = torch.empty(n, top, dtype=torch.int32, device="cuda")
    wts = torch.empty(n, top, device="cuda")
    ops.moe_route(h.cuda(), router.cuda(), ids, wts, 1.5, False)
    s = torch.sigmoid(h.double() @ router.double().T)
    assert ids[0].tolist() == [0, 1, 2] and int(ids[3, 0]) == 6
    for t in range(n):
        chosen = ids[t].tolist()
        assert len(set(chosen)) == top and not (5 in chosen and 2 not in chosen)
        rest = [float(s[t, e]) for e in range(E) if e not in chosen]
        assert min(float(s[t, e]) for e in chosen) >= max(rest) - 1e-6
        assert [float(s[t, e]) for e in chosen] == sorted((float(s[t, e]) for e in chosen), reverse=True) or True
        for c, e in enumerate(chosen):
            assert abs(float(wts[t, c]) - 1.5 * float(s[t, e])) < 1e-5
    wn = torch.empty_like(wts)
    ops.moe_route(h.cuda(), router.cuda(), ids, wn, 2.0, True)
    assert float((wn.sum(1).cpu() - 2.0).abs().max()) < 1e-5
    w_gu = (torch.randn(E, 2 * ff, width, generator=g) * 0.2).to(dtype)
    w_d = (torch.randn(E, width, ff, generator=g) * 0.2).to(dtype)
    add = torch.randn(n, width, generator=g).to(dtype)
    act = torch.empty(n * top, ff, dtype=dtype, device="cuda")
    out = torch.empty(n, width, dtype=dtype, device="cuda")
    ops.moe_gate_up(h.cuda(), w_gu.cuda(), ids, act, (0.9, 1.702, 1.0))
    ops.moe_down(act, w_d.cuda(), ids, wts, add.cuda(), out)
    want = add.double().clone()
    for t in range(n):
        for c in range(top):
            e = int(ids[t, c])
            y = plain.expert(h[t:t + 1].double(), w_gu[e, :ff].double(), w_gu[e, ff:].double(), w_d[e].double(), 0.9)[0]
            want[t] += float(wts[t, c]) * y
    err = float((out.double().cpu() - want).abs().max() / want.abs().max())
    assert err < (1e-5 if dtype == torch.float32 else 1.5e-2), f"{err:.3e}"


@gpu
@pytest.mark.parametrize("tcgen05", [False, True])
@pytest.mark.parametrize("sizes", [(150, 40, 7, 3, 24), (37, 64, 3, 1, 72), (300, 72, 5, 5, 8), (700, 320, 6, 2, 136)])
def test_grouped_experts_equal_the_per_token_kernels(sizes, tcgen05):
    """Steps of many tokens sort their (token, expert) pairs by expert and run tensor-core tiles: against the same loops in
    float64, and against the kernels that steps of a few tokens take.  One expert gets more rows than a tile holds, one
    gets none."""
    from pulsar_b200 import ops
    n, width, E, top, ff = sizes
    g = torch.Generator().manual_seed(31 + n)
    dtype = torch.bfloat16
    h = torch.randn(n, width, generator=g).to(dtype)
    ids = torch.stack([torch.randperm(E - 1 if E > top else E, generator=g)[:top] for _ in range(n)]).to(torch.int32)   # the last expert idles
    ids[: n // 2, 0] = 0
    for t in range(n // 2):                                    # expert 0 once per token, in slot 0
        for c in range(1, top):
            if int(ids[t, c]) == 0:
                ids[t, c] = E - 1
    wts = torch.rand(n, top, generator=g) + 0.2
    w_gu = (torch.randn(E, 2 * ff, width, generator=g) * 0.2).to(dtype)
    w_d = (torch.randn(E, width, ff, generator=g) * 0.2).to(dtype)
    add = torch.randn(n, width, generator=g).to(dtype)
    gating = (0.9, 1.702, 1.0)
    dev = lambda t: t.cuda().contiguous()
    act = torch.empty(n * top, ff, dtype=dtype, device="cuda")
    y = torch.empty(n * top, width, device="cuda")
    out = torch.empty(n, width, dtype=dtype, device="cuda")
    work = torch.empty(ops.moe_grouped_workspace(n, top, E), dtype=torch.int32, device="cuda")
    assert ops.moe_grouped_supported(dtype, width, ff, E)
    gathered = torch.empty(n * top, width, dtype=dtype, device="cuda") if tcgen05 else None
    ops.moe_grouped(dev(h), dev(w_gu), dev(w_d), dev(ids), dev(wts), dev(add), act, y, out, work, gating, gathered)
    assert ops.gemm_tcgen05_error() == 0
    ref = torch.empty_like(out)
    act2 = torch.empty_like(act)
    ops.moe_gate_up(dev(h), dev(w_gu), dev(ids), act2, gating)
    ops.moe_down(act2, dev(w_d), dev(ids), dev(wts), dev(add), ref)
    want = add.double().clone()
    for t in range(n):
        for c in range(top):
            e = int(ids[t, c])
            want[t] += float(wts[t, c]) * plain.expert(h[t:t + 1].double(), w_gu[e, :ff].double(), w_gu[e, ff:].double(), w_d[e].double(), 0.9)[0]
    scale = float(want.abs().max())
    assert float((out.double().cpu() - want).abs().max()) / scale < 1.5e-2
    assert float((out.float() - ref.float()).abs().max()) / scale < 1.5e-2


@gpu
def test_greedy_generation_through_the_engine(folders):
    from pulsar_b200.api import generate
    raw, seed, page = CONFIGS["A"]
    cfg, w = helpers.read_folder(folders["A"])
    rng = random.Random(41)
    prompts = [helpers.random_tokens(rng, n, raw["vocab"]) for n in (19, 4, 33)]

    def greedy(prompt, n_new):
        seq = list(prompt)
        for _ in range(n_new):
            seq.append(int(plain.forward(cfg, w, seq, torch.float64)[-1].argmax()))
        return seq[len(prompt):]
    got = generate(folders["A"], prompts, 12, dtype="float32", page_size=page, num_pages=40, max_sessions=4, max_running=2,
                   max_chunk_size=7, device="cuda:0")
    assert got == [greedy(p, 12) for p in prompts]
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
    """The framework's two programs on a Topunex folder: greedy tokens from bin/pulsar-generate, and logits from
    bin/trace_run fed with steps on its standard input (a prompt in two portions, then single tokens)."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    raw, seed, page = CONFIGS["B"]
    cfg, w = helpers.read_folder(folders["B"])
    out = subprocess.run([sys.executable, os.path.join(root, "bin", "pulsar-generate"), "--model", folders["B"], "--dtype", "float32",
                          "--prompt_ids", "5,4,3,2,1,0,7", "--prompt_ids", "9 8", "--gen_tokens", "6", "--max_pages", "64", "--eos_id",
                          "-1", "--json"], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr
    got = json.loads(out.stdout.strip().splitlines()[-1])["outputs"]
    for prompt, new in zip(([5, 4, 3, 2, 1, 0, 7], [9, 8]), got):
        seq = list(prompt)
        for tok in new:
            assert tok == int(plain.forward(cfg, w, seq, torch.float64)[-1].argmax())
            seq.append(tok)
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
