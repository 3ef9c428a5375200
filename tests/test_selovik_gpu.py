"""Selovik on the GPU against the plain implementation: the new kernels against float64 torch,
every mechanism alone, whole prompts against token-by-token decoding, portions down to two
tokens, unequal batches against each request alone, slots and pages used again, keys far away,
at page borders and on both sides of every window's edge with attention made sharp, the first
tokens, long decoding with windows passing over decoded tokens, other sizes, greedy generation
through the Python entry point, and the replay program."""
import json
import math
import os
import random
import subprocess

import numpy as np
import pytest
import torch

import plain_selovik as P
from helpers import TraceBuilder, check_logits, random_tokens, read_step, three_cuts
from selovik_models import (CONFIGS, attention, config, dense, layer, load_weights, make_model, moe, read_config,
                            yarn)

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DTYPES = ["float32", "bfloat16"]
F = torch.float64
# a router's choice between two experts whose corrected scores lie closer than this may go either way
# in bfloat16 (the scores are probabilities; the rows that the routers of deeper layers read carry the
# rounding of everything before them); such positions are left out, and they must be a minority
CLOSE_CALL = 0.005


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    return {name: make_model(str(tmp_path_factory.mktemp(f"selovik_{name}")), cfg, seed=900 + i)
            for i, (name, cfg) in enumerate(CONFIGS.items())}


_engines, _plain = {}, {}


def engine_for(models, name, dtype):
    from nnis_b200.engine import Engine
    if (name, dtype) not in _engines:
        _engines[(name, dtype)] = Engine.from_dir(models[name], dtype=dtype, max_tokens=64 * 96)
    return _engines[(name, dtype)]


def plain_of(model_dir, dtype, tokens):
    """(logits, smallest gap of any router's choice at each position)"""
    key = (model_dir, dtype, tuple(tokens))
    if key not in _plain:
        bf = dtype == "bfloat16"
        probe = {}
        logits = P.forward(list(tokens), load_weights(model_dir, bf), read_config(model_dir), emulate_bf16=bf, probe=probe)
        gaps = torch.stack(probe["gaps"]).min(0).values if probe.get("gaps") else torch.full((len(tokens),), math.inf)
        _plain[key] = (logits, gaps)
    return _plain[key]


def plain_logits(models, name, dtype, tokens):
    return plain_of(models[name], dtype, tokens)[0]


def check_rows(model_dir, dtype, rows, what):
    """rows: (tokens of the request, position, logits row).  bfloat16 rows at a router's close call are
    left out (at most a third of them)."""
    keep, skipped = [], 0
    for toks, pos, row in rows:
        logits, gaps = plain_of(model_dir, dtype, toks)
        if dtype == "bfloat16" and float(gaps[pos]) < CLOSE_CALL:
            skipped += 1
            continue
        keep.append((row, logits[pos]))
    assert skipped <= max(2, len(rows) // 3), f"{what}: {skipped} of {len(rows)} rows at a close call"
    if keep:
        check_logits(np.stack([r for r, _ in keep]), torch.stack([w for _, w in keep]), dtype, what)


def replay_and_check(models, name, dtype, trace, sequences, tmp_path, what):
    from nnis_b200.engine.replay import replay
    engine = engine_for(models, name, dtype)
    out = str(tmp_path / f"out_{name}_{dtype}")
    replay(engine, trace.lines, out)
    usage = engine.cache.usage()
    assert usage["slots_held"] == 0 and not any(usage["pages_held"]), usage
    engine.cache.check()
    vocab = read_config(models[name])["vocab"]
    rows = []
    for step, places in trace.rows.items():
        got = read_step(out, step, vocab)
        assert got.shape[0] == len(places)
        rows += [(sequences[rid], pos, got[i]) for i, (rid, pos) in enumerate(places)]
    check_rows(models[name], dtype, rows, f"{what} {name} {dtype}")


def run_whole(engine, tokens, want=None):
    from nnis_b200.engine import SequenceStep
    slot = engine.acquire_slot()
    try:
        return engine.step([SequenceStep(slot, tokens, list(range(len(tokens))) if want is None else want)]).cpu().numpy()
    finally:
        engine.release_slot(slot)


# ---- the new kernels against plain torch -------------------------------------------------------
def test_pair_embedding_hashes_the_token_before_across_steps():
    """Rows of two sequences in one step, a later portion, single tokens: the token before the first
    row of a portion comes from the slot's state, which then holds the portion's last token."""
    from nnis_b200.csrc import ops
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(1)
    for dtype in (torch.float32, torch.bfloat16):
        for vocab, width, buckets, mp, mc in ((50, 24, 7, 3, 5), (300, 100, 101, 31, 17), (9, 256, 1, 1, 1)):
            table = torch.randn(vocab, width, generator=g).to(dtype).to(dev)
            pair = torch.randn(buckets + 1, width, generator=g).to(dtype).to(dev)
            seqs = {3: [int(t) for t in torch.randint(0, vocab, (11,), generator=g)],
                    0: [int(t) for t in torch.randint(0, vocab, (6,), generator=g)]}
            last = torch.full((5,), -7, dtype=torch.int32, device=dev)
            status = torch.zeros(1, dtype=torch.int32, device=dev)

            def run(portions, decode):
                toks = [t for slot, a, b in portions for t in seqs[slot][a:b]]
                pos = [p for slot, a, b in portions for p in range(a, b)]
                seq = [i for i, (slot, a, b) in enumerate(portions) for _ in range(a, b)]
                i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
                hidden = torch.empty(len(toks), width, device=dev)
                ops.embed_pair(table, pair, i32(toks), i32(pos), i32(seq), i32([s for s, _, _ in portions]),
                               None if decode else i32([b - a for _, a, b in portions]), last, hidden, status, 1.5,
                               buckets, mp, mc)
                want = []
                for slot, a, b in portions:
                    for p in range(a, b):
                        row = buckets if p == 0 else (seqs[slot][p - 1] * mp + seqs[slot][p] * mc) % buckets
                        want.append(table[seqs[slot][p]].double() * 1.5 + pair[row].double())
                assert torch.allclose(hidden.double(), torch.stack(want), atol=1e-6, rtol=1e-6), (portions, decode)
                for slot, a, b in portions:
                    assert int(last[slot]) == seqs[slot][b - 1]

            run([(3, 0, 4), (0, 0, 1)], False)   # two prompts, one of a single token
            run([(0, 1, 3), (3, 4, 9)], False)   # later portions, the other way round
            run([(3, 9, 10), (0, 3, 4)], True)   # single tokens
            run([(3, 10, 11)], True)
            run([(0, 4, 6)], False)              # a portion of two tokens
            assert int(status[0]) == 0
    # without a second table: the scaled row, no state
    hidden = torch.empty(2, 24, device=dev)
    table = torch.randn(50, 24, generator=g).to(dev)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
    ops.embed_pair(table, None, i32([4, 9]), i32([0, 1]), i32([0, 0]), i32([0]), i32([2]), None, hidden,
                   torch.zeros(1, dtype=torch.int32, device=dev), 0.25, 0, 0, 0)
    assert torch.equal(hidden, table[[4, 9]] * 0.25)


def test_two_norms_of_the_same_rows_in_one_pass():
    from nnis_b200.csrc import ops
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(2)
    for n, width in ((1, 7), (5, 76), (70, 96), (200, 1024), (3, 2050)):
        x = torch.randn(n, width, generator=g) * 3
        w1, w2 = torch.randn(width, generator=g), torch.randn(width, generator=g)
        unit = x.double() / torch.sqrt((x.double() ** 2).mean(-1, keepdim=True) + 1e-5)
        for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 1e-2)):
            a, b = torch.empty(n, width, dtype=dtype, device=dev), torch.empty(n, width, dtype=dtype, device=dev)
            ops.rmsnorm_pair(x.to(dev), w1.to(dev), w2.to(dev), 1e-5, a, b)
            assert torch.allclose(a.cpu().double(), unit * w1.double(), atol=tol, rtol=tol)
            assert torch.allclose(b.cpu().double(), unit * w2.double(), atol=tol, rtol=tol)
            one = torch.empty(n, width, dtype=dtype, device=dev)
            ops.rmsnorm(x.to(dev), w2.to(dev), 1e-5, one)
            assert torch.allclose(b.float(), one.float(), atol=tol, rtol=tol)


def test_stream_steps_relu_squared_and_scaled_logits():
    from nnis_b200.csrc import ops
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(3)
    x, kept, row = torch.randn(9, 76, generator=g), torch.randn(9, 76, generator=g), torch.randn(76, generator=g)
    for k, r in ((kept, row), (None, row), (kept, None)):
        h = x.to(dev).clone()
        ops.stream_enter(h, None if k is None else k.to(dev), None if r is None else r.to(dev))
        want = x + (0 if k is None else k) + (0 if r is None else r)
        assert torch.allclose(h.cpu(), want, atol=1e-6)
    h = x.to(dev).clone()
    ops.scale_rows(h, 0.7)
    assert torch.allclose(h.cpu(), x * 0.7, atol=1e-7)
    z = torch.linspace(-5, 5, 1001)
    for dtype in (torch.float32, torch.bfloat16):
        out = torch.empty(1001, dtype=dtype, device=dev)
        ops.act_rows(z.to(dev), out, ops.RELU2)
        assert torch.equal(out.cpu(), (torch.clamp(z, min=0) ** 2).to(dtype))


@pytest.mark.parametrize("outputs, experts, top, groups, keep", [(8, 5, 3, 4, 2), (12, 7, 4, 3, 1), (16, 12, 4, 4, 3),
                                                                 (6, 6, 2, 1, 1), (4, 3, 1, 1, 1), (70, 64, 6, 10, 4)])
def test_the_router_chooses_by_corrected_scores_within_the_best_groups(outputs, experts, top, groups, keep):
    from nnis_b200.csrc import ops
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(outputs)
    n, width = 150, 76
    h = torch.randn(n, width, generator=g)
    w = {"r.router": torch.randn(outputs, width, generator=g) * 0.2, "r.correction": torch.randn(outputs, generator=g) * 0.1}
    r = {"experts": experts, "identity": outputs - experts, "top": top, "groups": {"count": groups, "keep": keep}}
    probe = {}
    ids, weights = P.route(h.double(), {k: v.double() for k, v in w.items()}, "r", r, probe)
    pos = torch.arange(n, dtype=torch.int32)
    pos[7] = -1  # a padding row
    got_ids = torch.full((n, top), 99, dtype=torch.int32, device=dev)
    got_w = torch.empty(n, top, device=dev)
    passed = torch.empty(n, device=dev)
    ops.moe_route_choice(h.to(dev), w["r.router"].to(dev), w["r.correction"].to(dev), pos.to(dev), got_ids, got_w,
                         passed, experts, top, groups, keep)
    got_ids, got_w, passed = got_ids.cpu(), got_w.cpu(), passed.cpu()
    assert (got_ids[7] == -1).all() and float(passed[7]) == 0
    clear = [t for t in range(n) if t != 7 and float(probe["gaps"][0][t]) > 1e-5]
    assert len(clear) > n - 10
    for t in clear:
        want = [e if e < experts else -1 for e in ids[t].tolist()]
        assert got_ids[t].tolist() == want, t
        assert torch.allclose(got_w[t].double(), weights[t], atol=1e-6)
        assert abs(float(passed[t]) - float(weights[t][ids[t] >= experts].sum())) < 1e-6


def _plain_two_maps(q, k, v, window, scale, lam, post, eps, gate, start=0):
    """q [T, H, 2, d] (rows at positions start ..), k [S, G, 2, d], v [S, G, dv], float64."""
    T, H = q.shape[:2]
    S, G = k.shape[:2]
    i = torch.arange(start, start + T)[:, None]
    j = torch.arange(S)[None, :]
    visible = (j <= i) & (i - j < window if window else j >= 0)
    out = torch.zeros(T, H, v.shape[-1], dtype=F)
    for a in range(H):
        kv = a // (H // G)
        parts = []
        for c in range(2):
            s = (q[:, a, c] @ k[:, kv, c].T) * scale
            parts.append(torch.softmax(s.masked_fill(~visible, -math.inf), -1) @ v[:, kv])
        o = parts[0] - lam * parts[1]
        out[:, a] = o / torch.sqrt((o * o).mean(-1, keepdim=True) + eps) * post
    out = out.reshape(T, -1)
    return out * gate if gate is not None else out


@pytest.mark.parametrize("H, G, dk, dv, window", [(4, 2, 16, 24, 9), (6, 3, 24, 40, 50), (3, 3, 10, 34, 64), (5, 1, 18, 6, 1),
                                                  (8, 1, 12, 40, 70), (2, 1, 64, 128, 0), (8, 2, 32, 200, 65), (2, 2, 130, 8, 300),
                                                  (3, 1, 5, 7, 10), (16, 2, 32, 64, 33)])
def test_attention_with_two_maps_in_every_cut(H, G, dk, dv, window):
    """The attention kernel alone, over a cache whose pages are scattered: a prompt, a later portion
    and single tokens, with the key range whole and in slices, against plain float64."""
    from nnis_b200.csrc import ops
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(H * 100 + dk)
    S, page = 200, 64
    lam, post, eps, scale = 0.37, 0.6, 1e-5, 1.3 / math.sqrt(dk)
    for dtype, tol in ((torch.float32, 2e-5), (torch.bfloat16, 2e-2)):
        q = torch.randn(S, H, 2, dk, generator=g).to(dtype)
        k = torch.randn(S, G, 2, dk, generator=g).to(dtype)
        v = torch.randn(S, G, dv, generator=g).to(dtype)
        gate = torch.rand(S, H * dv, generator=g)
        pages = [5, 2, 9, 0]  # where the sequence's pages lie in the cache
        k_cache = torch.full((10, G, page, 2 * dk), 50.0, dtype=dtype)  # (what other pages hold must not matter)
        v_cache = torch.full((10, G, page, dv), -50.0, dtype=dtype)
        for t in range(S):
            k_cache[pages[t // page], :, t % page] = k[t].reshape(G, 2 * dk)
            v_cache[pages[t // page], :, t % page] = v[t]
        table = torch.tensor([[7, 7, 7, 7], pages], dtype=torch.int32, device=dev)  # the sequence is row 1 of the batch
        want = _plain_two_maps(q.double(), k.double(), v.double(), window, scale, lam, post, eps, gate.double())
        for a, b, splits in ((0, 130, 1), (130, 190, 1), (190, 191, 1), (191, 192, 3), (192, 200, 2), (0, 200, 4)):
            n = b - a
            pos = torch.arange(a, b, dtype=torch.int32, device=dev)
            seq = torch.ones(n, dtype=torch.int32, device=dev)
            out = torch.full((n, H * dv), 9.0, dtype=dtype, device=dev)
            partial = torch.empty(n * H * splits * (2 * dv + 4), device=dev) if splits > 1 else None
            ops.attention_diff(q[a:b].reshape(n, -1).to(dev), k_cache.to(dev), v_cache.to(dev), pos, seq, table,
                               gate[a:b].to(dev), out, H, G, window, scale, lam, post, eps, splits, partial)
            assert torch.allclose(out.cpu().double(), want[a:b], atol=tol, rtol=tol), (dtype, a, b, splits)
        # a padding row is left alone
        pos = torch.tensor([150, -1, 151], dtype=torch.int32, device=dev)
        out = torch.full((3, H * dv), 9.0, dtype=dtype, device=dev)
        ops.attention_diff(q[[150, 0, 151]].reshape(3, -1).to(dev), k_cache.to(dev), v_cache.to(dev), pos,
                           torch.ones(3, dtype=torch.int32, device=dev), table, None, out, H, G, window, scale, lam,
                           post, eps)
        assert (out[1] == 9.0).all()
        assert torch.allclose(out[[0, 2]].cpu().double(), (want / gate.double())[[150, 151]], atol=tol, rtol=tol)


@pytest.mark.parametrize("H, G, dk, dv, window", [(4, 2, 32, 64, 100), (2, 1, 32, 128, 70), (6, 2, 64, 64, 0), (3, 3, 64, 128, 64),
                                                  (2, 2, 128, 128, 129), (4, 1, 128, 64, 65)])
def test_prompt_attention_on_the_tensor_cores(H, G, dk, dv, window):
    """The tensor-core prompt form against plain float64 and against the any-size kernel: two sequences in one
    step, one of them a later portion that starts inside a page, tiles that end inside a page."""
    from nnis_b200.csrc import ops
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(H * 1000 + dk + dv)
    lam, post, eps, scale = 0.8, 0.5, 1e-5, 1.2 / math.sqrt(dk)
    lens, starts = [230, 150], [0, 75]       # the second sequence already holds 75 positions
    counts = [lens[0], lens[1] - starts[1]]
    pages = [[3, 0, 6, 1], [2, 7, 5]]
    k_cache = torch.full((8, G, 64, 2 * dk), 50.0, dtype=torch.bfloat16)
    v_cache = torch.full((8, G, 64, dv), -50.0, dtype=torch.bfloat16)
    qs, want = [], []
    for i, n in enumerate(lens):
        q = torch.randn(n, H, 2, dk, generator=g).bfloat16()
        k = torch.randn(n, G, 2, dk, generator=g).bfloat16()
        v = torch.randn(n, G, dv, generator=g).bfloat16()
        gate = torch.rand(n, H * dv, generator=g)
        for t in range(n):
            k_cache[pages[i][t // 64], :, t % 64] = k[t].reshape(G, 2 * dk)
            v_cache[pages[i][t // 64], :, t % 64] = v[t]
        full = _plain_two_maps(q.double(), k.double(), v.double(), window, scale, lam, post, eps, gate.double())
        qs.append((q[starts[i]:].reshape(counts[i], -1), gate[starts[i]:]))
        want.append(full[starts[i]:])
    q = torch.cat([a for a, _ in qs]).to(dev)
    gate = torch.cat([b for _, b in qs]).to(dev)
    want = torch.cat(want)
    table = torch.tensor([pages[0], pages[1] + [-1]], dtype=torch.int32, device=dev)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
    tiles = i32([(i, q0) for i, c in enumerate(counts) for q0 in range(0, c, 64)])
    out = torch.full((sum(counts), H * dv), 9.0, dtype=torch.bfloat16, device=dev)
    assert ops.attention_diff_mma_takes(dk, dv, 64)
    ops.attention_diff_mma(q, k_cache.to(dev), v_cache.to(dev), tiles, i32([0, counts[0]]), i32(starts), i32(counts), table,
                           gate, out, H, G, window, scale, lam, post, eps)
    assert torch.allclose(out.cpu().double(), want, atol=3e-2, rtol=3e-2)
    pos = i32(list(range(lens[0])) + list(range(starts[1], lens[1])))
    seq = i32([0] * counts[0] + [1] * counts[1])
    other = torch.empty_like(out)
    ops.attention_diff(q, k_cache.to(dev), v_cache.to(dev), pos, seq, table, gate, other, H, G, window, scale, lam, post, eps)
    assert torch.allclose(out.float(), other.float(), atol=3e-2, rtol=3e-2)


def test_rotation_of_every_map_before_the_cache():
    """qkv_prep with two maps a head: each map's first values turned by itself, the magnitude on
    cosine and sine, keys into the cache row, the gates' sigmoid."""
    from nnis_b200.csrc import ops
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(8)
    for H, G, dk, dv, dims, mag in ((4, 2, 16, 24, 8, 1.2), (3, 1, 10, 6, 10, 1.0), (2, 2, 32, 40, 0, 1.3), (5, 5, 6, 34, 2, 0.9),
                                    (2, 1, 5, 3, 4, 1.1)):
        n = 70
        rot = {"dims": dims, "base": 100.0}
        f, _ = P.rotation_frequencies(rot) if dims else (torch.zeros(0, dtype=F), 1.0)
        a = torch.randn(n, H * 2 * dk + G * 2 * dk + G * dv + H * dv, generator=g)
        pos = torch.arange(3, 3 + n, dtype=torch.int32)
        table = torch.tensor([[1, 0]], dtype=torch.int32, device=dev)
        q = torch.empty(n, H * 2 * dk, device=dev)
        kc, vc = torch.zeros(2, G, 64, 2 * dk, device=dev), torch.zeros(2, G, 64, dv, device=dev)
        gate = torch.empty(n, H * dv, device=dev)
        freq = torch.cat([f.float(), torch.zeros(1)]).to(dev)
        ops.qkv_prep(a.to(dev), None, None, freq, pos.to(dev), torch.zeros(n, dtype=torch.int32, device=dev), table, q,
                     kc, vc, gate, H, G, 2 * dk, dv, dims, 1e-5, pairing="half", maps=2, magnitude=mag)

        def turned(x, heads):  # [n, heads * 2, dk]
            x = x.double().view(n, heads * 2, dk)
            if not dims:
                return x
            ang = pos.double()[:, None] * f.float().double()[None, :]
            c, s = (torch.cos(ang) * mag)[:, None], (torch.sin(ang) * mag)[:, None]
            u, w_ = x[..., :dims // 2], x[..., dims // 2:dims]
            return torch.cat([u * c - w_ * s, w_ * c + u * s, x[..., dims:]], -1)
        nq, nk = H * 2 * dk, G * 2 * dk
        assert torch.allclose(q.cpu().double(), turned(a[:, :nq], H).reshape(n, -1), atol=2e-4, rtol=1e-5)
        want_k = turned(a[:, nq:nq + nk], G).reshape(n, G, 2 * dk)
        for t in range(n):
            p = int(pos[t])
            assert torch.allclose(kc[[1, 0][p // 64], :, p % 64].cpu().double(), want_k[t], atol=2e-4, rtol=1e-5)
            assert torch.equal(vc[[1, 0][p // 64], :, p % 64].cpu().reshape(-1), a[t, nq + nk:nq + nk + G * dv])
        assert torch.allclose(gate.cpu(), torch.sigmoid(a[:, nq + nk + G * dv:]), atol=1e-6)


# ---- whole models against the plain implementation -----------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["mixed", "odd", "loop_all", "loop_once", "heads64"])
def test_each_configuration_alone(models, name, dtype, tmp_path):
    rng = random.Random(11)
    vocab = read_config(models[name])["vocab"]
    sequences, trace = {}, TraceBuilder()
    # the first tokens, a page's border, windows' edges
    for i, n in enumerate((1, 2, 3, 50, 63, 64, 65, 131, 300)):
        sequences[f"w{i}"] = random_tokens(rng, n, vocab)
        trace.step([(f"w{i}", sequences[f"w{i}"], range(n))], end=[f"w{i}"])
    toks = sequences["d"] = random_tokens(rng, 75, vocab)  # decoding from the second token on
    trace.step([("d", toks[:1], [0])])
    for t in range(1, 75):
        trace.step([("d", toks[t:t + 1], [0])], end=["d"] if t == 74 else [])
    replay_and_check(models, name, dtype, trace, sequences, tmp_path, "alone")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["mixed", "odd", "heads64"])
def test_whole_last_tokens_and_unequal_batches(models, name, dtype, tmp_path):
    vocab = read_config(models[name])["vocab"]
    trace, sequences = three_cuts(random.Random(3), vocab)
    replay_and_check(models, name, dtype, trace, sequences, tmp_path, "three cuts")


@pytest.mark.parametrize("name", ["mixed", "odd", "loop_all"])
def test_portions_batches_and_reuse_agree_with_each_request_alone(models, name):
    """float32: the same position's logits whatever the cut, the batch, the slot or the pages."""
    from nnis_b200.engine import SequenceStep
    engine = engine_for(models, name, "float32")
    vocab = read_config(models[name])["vocab"]
    rng = random.Random(9)
    prompts = [random_tokens(rng, n, vocab) for n in (200, 3, 67, 130)]
    alone = [run_whole(engine, p) for p in prompts]
    scale = max(float(np.abs(a).max()) for a in alone)
    for p, a in zip(prompts, alone):
        check_logits(a, plain_logits(models, name, "float32", p), "float32", "alone")
    # portions of several sizes, down to two tokens and one
    for cuts in ([2, 2, 60, 1, 64, 71], [64, 64, 64, 8], [199, 1], [1, 199], [39, 2, 7, 152], [3, 17, 16, 164],
                 [1, 1, 1, 2, 130, 65]):
        slot = engine.acquire_slot()
        rows, at = [], 0
        for c in cuts:
            rows.append(engine.step([SequenceStep(slot, prompts[0][at:at + c], list(range(c)))]).cpu().numpy())
            at += c
        engine.release_slot(slot)
        assert at == 200 and np.abs(np.concatenate(rows) - alone[0]).max() < 3e-5 * scale, cuts
    # one batch of all four, then the same again in slots and pages that were used before
    for _ in range(2):
        slots = [engine.acquire_slot() for _ in prompts]
        heads = [max(1, len(p) - 20) for p in prompts]
        got = engine.step([SequenceStep(s, p[:h], list(range(h))) for s, p, h in zip(slots, prompts, heads)]).cpu().numpy()
        at = 0
        for i, h in enumerate(heads):
            assert np.abs(got[at:at + h] - alone[i][:h]).max() < 3e-5 * scale
            at += h
        live = list(range(len(prompts)))
        step = 0
        while live:  # decoded together; the shorter ones end earlier
            batch = [SequenceStep(slots[i], prompts[i][heads[i] + step:heads[i] + step + 1], [0]) for i in live]
            got = engine.step(batch).cpu().numpy()
            for r, i in enumerate(live):
                assert np.abs(got[r] - alone[i][heads[i] + step]).max() < 3e-5 * scale, (i, step)
            step += 1
            for i in list(live):
                if heads[i] + step == len(prompts[i]):
                    engine.release_slot(slots[i])
                    live.remove(i)
    assert engine.cache.usage()["slots_held"] == 0
    engine.cache.check()


def test_a_slot_used_again_forgets_its_last_token(models):
    """The token before a sequence's first token is nothing, whatever the slot's last owner left;
    a snapshot brings a sequence back with the token it ended on."""
    from nnis_b200.engine import SequenceStep
    engine = engine_for(models, "mixed", "float32")
    vocab = read_config(models["mixed"])["vocab"]
    rng = random.Random(2)
    a, b = random_tokens(rng, 90, vocab), random_tokens(rng, 33, vocab)
    want = run_whole(engine, b)
    slot = engine.acquire_slot()
    engine.step([SequenceStep(slot, a, [])])
    engine.release_slot(slot)
    again = engine.acquire_slot()
    assert again == slot
    got = engine.step([SequenceStep(again, b[:20], list(range(20)))]).cpu().numpy()
    kept = engine.snapshot(again)
    rest = engine.step([SequenceStep(again, b[20:], list(range(13)))]).cpu().numpy()
    assert np.abs(np.concatenate([got, rest]) - want).max() < 3e-5 * np.abs(want).max()
    engine.restore(kept)
    engine.step([SequenceStep(again, a[:5], [])])  # other tokens after the snapshot
    engine.restore(kept)
    rest = engine.step([SequenceStep(again, b[20:], list(range(13)))]).cpu().numpy()
    assert np.abs(rest - want[20:]).max() < 3e-5 * np.abs(want).max()
    engine.release_slot(again)


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_prompt_shape_that_recurs_is_captured_and_replayed(models, dtype):
    """A large prompt step whose shape comes a second time is recorded as a CUDA graph and replayed from
    the third time on: the kept embedding output, the loop's rows and the last tokens must all live
    where the graph expects them.  Other tokens every time, the same shape."""
    from nnis_b200.engine import Engine, SequenceStep
    engine = Engine.from_dir(models["mixed"], dtype=dtype, max_tokens=64 * 64)
    vocab = read_config(models["mixed"])["vocab"]
    rng = random.Random(77)
    graphs = []
    for round_ in range(4):
        a, b = random_tokens(rng, 300, vocab), random_tokens(rng, 40, vocab)
        slots = [engine.acquire_slot(), engine.acquire_slot()]
        got = engine.step([SequenceStep(slots[0], a[:290], [0, 150, 289]), SequenceStep(slots[1], b[:30], [29])]).cpu().numpy()
        more = engine.step([SequenceStep(slots[0], a[290:291], [0]), SequenceStep(slots[1], b[30:31], [0])]).cpu().numpy()
        for s_ in slots:
            engine.release_slot(s_)
        graphs.append(len(engine._step_graphs))
        rows = [(a, 0, got[0]), (a, 150, got[1]), (a, 289, got[2]), (b, 29, got[3]), (a, 290, more[0]), (b, 30, more[1])]
        check_rows(models["mixed"], dtype, rows, f"captured step, round {round_}")
    assert graphs == [0, 1, 1, 1], graphs


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["mixed", "sharp"])
def test_long_decoding_lets_every_window_pass_over_decoded_tokens(models, name, dtype, tmp_path):
    vocab = read_config(models[name])["vocab"]
    toks = random_tokens(random.Random(21), 5 + 330, vocab)
    trace = TraceBuilder()
    trace.step([("a", toks[:5], [4])])
    for t in range(5, len(toks)):
        trace.step([("a", toks[t:t + 1], [0])], end=["a"] if t == len(toks) - 1 else [])
    replay_and_check(models, name, dtype, trace, {"a": toks}, tmp_path, "long decoding")


def _sharpen(model_dir, out_dir, layer_index, query_pos, key_pos, tokens, cfg):
    """A copy of the model whose layer ``layer_index`` has, in map 1 of every head, one score that stands
    out: the query at ``query_pos`` against the key at ``key_pos``.  Done through the first layer's
    input rows: the rows of W_q and W_k that are not rotated get a large component along the
    normed embedding of those two tokens (which must differ from all others)."""
    from safetensors.torch import load_file, save_file
    os.makedirs(out_dir, exist_ok=True)
    w = load_file(os.path.join(model_dir, "model.safetensors"))
    plain = {k: v.double() for k, v in w.items()}
    x = P.embedding(tokens, plain, cfg)
    h = P.centred_norm(x, plain[f"l{layer_index}.norm1"], cfg["norm"]["eps"])
    m = cfg["layers"][layer_index]["mixer"]
    d, dims = m["dim"], m["rot"]["dims"]
    assert dims < d, "the test needs an unrotated value in every map"
    hq, hk = h[query_pos] / h[query_pos].norm(), h[key_pos] / h[key_pos].norm()
    q, k = plain[f"l{layer_index}.mix.q"].clone(), plain[f"l{layer_index}.mix.k"].clone()
    for a in range(m["heads"]):
        q[a * 2 * d + d - 1] = hq * 6.0   # the last value of map 1: never rotated
    for a in range(m["kv_heads"]):
        k[a * 2 * d + d - 1] = hk * 6.0
    w[f"l{layer_index}.mix.q"], w[f"l{layer_index}.mix.k"] = q.to(torch.bfloat16), k.to(torch.bfloat16)
    save_file(w, os.path.join(out_dir, "model.safetensors"))
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(cfg, f)
    return out_dir


@pytest.mark.parametrize("window, distance", [(40, 39), (40, 40), (64, 63), (64, 64), (65, 64), (65, 65), (129, 128),
                                              (129, 129), (300, 299), (7, 6), (7, 7)])
def test_a_key_just_inside_and_just_outside_the_window(window, distance, tmp_path):
    """One key is made to dominate map 1 of the first layer for one query, ``distance`` tokens back.
    Inside the window (distance < window) the output at the query depends on that key's token;
    outside it does not.  Checked against the plain implementation, in a prompt, with the query in a
    later portion, and decoded alone, and directly: changing the key's token changes the query's logits
    if and only if the key is visible."""
    from nnis_b200.engine import Engine, SequenceStep
    cfg = config(97, 64, 1e-5, [layer(attention(4, 2, 16, 24, window, 8, 1.0, diff=0.4, base=100.0), dense(48)),
                                layer(attention(2, 1, 12, 16, 1, 0, 0.5), None)], scale=2.0)
    base = make_model(str(tmp_path / "base"), cfg, 31)
    rng = random.Random(window * 1000 + distance)
    n = 320
    qp = n - 3
    kp = qp - distance
    toks = [rng.randrange(2, 97) for _ in range(n)]
    toks[kp], toks[qp] = 0, 1   # tokens that appear nowhere else (no pair table here: a token's row is its own)
    d = _sharpen(base, str(tmp_path / "sharp"), 0, qp, kp, toks, cfg)
    w = load_weights(d, False)
    probe = {}
    want = P.forward(toks, w, cfg, probe=probe)
    a1 = probe["weights"][0][0]  # layer 0, head 0, map 1
    if distance < window:
        assert float(a1[qp, kp]) > 0.5, float(a1[qp, kp])   # the key stands out
    else:
        assert float(a1[qp, kp]) == 0.0
    other = list(toks)
    other[kp] = 50
    moved = float((P.forward(other, w, cfg)[qp] - want[qp]).abs().max())
    # (the second layer sees one token only, so the key reaches the query through the first layer's window alone)
    assert (moved > 1e-3) == (distance < window), (moved, window, distance)
    for dtype in DTYPES:
        engine = Engine.from_dir(d, dtype=dtype, max_tokens=1024)
        bf = dtype == "bfloat16"
        ref = P.forward(toks, load_weights(d, bf), cfg, emulate_bf16=bf) if bf else want
        for cut in (n, qp, qp - 1, kp + 1, kp):   # whole; the query decoded alone; a portion's start at the query, after the key, at the key
            slot = engine.acquire_slot()
            got = []
            if cut == n:
                got.append(engine.step([SequenceStep(slot, toks, [qp, n - 1])]).cpu().numpy())
            else:
                engine.step([SequenceStep(slot, toks[:cut], [])])
                if cut == qp:
                    got.append(engine.step([SequenceStep(slot, toks[qp:qp + 1], [0])]).cpu().numpy())
                    got.append(engine.step([SequenceStep(slot, toks[qp + 1:], [n - qp - 2])]).cpu().numpy())
                else:
                    got.append(engine.step([SequenceStep(slot, toks[cut:], [qp - cut, n - 1 - cut])]).cpu().numpy())
            engine.release_slot(slot)
            check_logits(np.concatenate(got), ref[[qp, n - 1]], dtype, f"window {window} distance {distance} cut {cut} {dtype}")
        if not bf:
            slot = engine.acquire_slot()
            changed = engine.step([SequenceStep(slot, other, [qp])]).cpu().numpy()
            engine.release_slot(slot)
            seen = float(np.abs(changed[0] - want[qp].numpy()).max()) > 1e-3
            assert seen == (distance < window)


def test_far_keys_and_page_borders_with_sharp_attention(models, tmp_path):
    """Random sharp heads put most of a query's weight on single keys anywhere in their windows (300,
    129 and 64 tokens): prompts that end on both sides of page borders, portions that start there,
    and tokens decoded across them."""
    from nnis_b200.engine import SequenceStep
    vocab = read_config(models["sharp"])["vocab"]
    rng = random.Random(5)
    probe = {}
    toks = random_tokens(rng, 450, vocab)
    P.forward(toks, load_weights(models["sharp"], False), read_config(models["sharp"]), probe=probe)
    peak = torch.stack([m[0].max(-1).values for m in probe["weights"]])[:, 100:]
    assert float(peak.mean()) > 0.5  # sharp: half a query's weight on one key, on average
    far = torch.stack([(m[0].argmax(-1) - torch.arange(450)).abs() for m in probe["weights"]])
    assert int(far.max()) > 120      # and some of those keys lie far back
    for dtype in DTYPES:
        engine = engine_for(models, "sharp", dtype)
        for cuts in ([450], [63, 1, 64, 1, 127, 194], [64, 64, 64, 64, 64, 64, 66], [128, 1, 1, 1, 62, 257], [300, 150]):
            slot = engine.acquire_slot()
            rows, at = [], 0
            for c in cuts:
                got = engine.step([SequenceStep(slot, toks[at:at + c], list(range(c)))]).cpu().numpy()
                rows += [(toks, at + i, got[i]) for i in range(c)]
                at += c
            engine.release_slot(slot)
            check_rows(models["sharp"], dtype, rows, f"sharp {dtype} {cuts}")


def _random_config(rng):
    width = rng.choice([40, 64, 76, 96, 128])
    layers = []
    n_layers = rng.randint(1, 4)
    for _ in range(n_layers):
        kv = rng.randint(1, 3)
        dim = rng.choice([2, 5, 6, 8, 10, 16, 24, 32, 40, 64])
        dims = rng.choice([0, 2, dim // 2 * 2, (dim // 4) * 2])
        scaling = rng.choice([None, yarn(rng.choice([2.0, 8.0, 32.0]), rng.choice([16, 64, 1024]), rng.choice([4.0, 32.0]),
                                         rng.choice([0.5, 1.0]))])
        mixer = attention(kv * rng.randint(1, 4), kv, dim, rng.choice([4, 6, 16, 24, 34, 64, 72, 130]),
                          rng.choice([1, 2, 17, 63, 64, 65, 100, 1000]), dims, rng.choice([0.2, 0.5, 1.0]) * 4 / math.sqrt(dim) / 4,
                          diff=rng.choice([0.1, 0.5, 0.8, 1.0, 0.0]), base=rng.choice([10.0, 10000.0, 500000.0]), scaling=scaling)
        kind = rng.random()
        if kind < 0.25:
            mlp = None
        elif kind < 0.5:
            mlp = dense(rng.choice([8, 20, 72, 130]))
        else:
            count = rng.choice([1, 1, 2, 3, 4])
            size = rng.randint(1, 4)
            outputs = count * size
            identity = rng.randint(0, outputs - 1)
            keep = rng.randint(1, count)
            mlp = moe(outputs - identity, rng.randint(1, keep * size), rng.choice([8, 12, 24, 40]), identity=identity,
                      groups=(count, keep) if count > 1 or rng.random() < 0.5 else None,
                      shared=rng.choice([None, 16, 28]))
        layers.append(layer(mixer, mlp))
    loop = None
    if rng.random() < 0.7:
        start = rng.randint(0, n_layers - 1)
        loop = (start, rng.randint(start + 1, n_layers), rng.randint(1, 3))
    bigram = rng.choice([None, (rng.choice([1, 13, 101, 1009]), rng.randint(0, 40), rng.randint(1, 40))])
    return config(rng.choice([50, 131, 256, 577]), width, rng.choice([1e-5, 1e-6]), layers, loop=loop,
                  scale=rng.choice([1.0, 0.5, 12.0]), bigram=bigram, logit_scale=rng.choice([1.0, 2.0, 0.3]))


@pytest.mark.parametrize("trial", range(12))
def test_configurations_drawn_at_random(trial, tmp_path):
    """A prompt in one step, a second portion and six tokens one by one, both dtypes, on a model
    whose sizes, layer order, loop and constants are drawn at random: whatever kernels the sizes select."""
    from nnis_b200.engine import Engine, SequenceStep
    rng = random.Random(8000 + trial)
    cfg = _random_config(rng)
    d = make_model(str(tmp_path / "m"), cfg, seed=trial)
    toks = random_tokens(rng, 150, cfg["vocab"])
    for dtype in DTYPES:
        engine = Engine.from_dir(d, dtype=dtype, max_tokens=4096)
        slot = engine.acquire_slot()
        got = [engine.step([SequenceStep(slot, toks[:101], list(range(101)))]).cpu().numpy(),
               engine.step([SequenceStep(slot, toks[101:144], list(range(43)))]).cpu().numpy()]
        for t in range(144, 150):
            got.append(engine.step([SequenceStep(slot, toks[t:t + 1], [0])]).cpu().numpy())
        engine.release_slot(slot)
        engine.check_status()
        got = np.concatenate(got)
        check_rows(d, dtype, [(toks, i, got[i]) for i in range(150)], f"random configuration {trial} {dtype}: {json.dumps(cfg)}")


def _middle_config(rng):
    """Sizes of a small real model (widths of a few hundred, maps of 32 to 128, a few thousand vocabulary
    entries): the shapes at which the tensor-core products, the decode projections over tiles of rows and
    the tensor-core attention take over from the any-size kernels."""
    width = rng.choice([192, 256, 320, 384, 512])
    layers = []
    n_layers = rng.randint(2, 4)
    for _ in range(n_layers):
        dim = rng.choice([32, 64, 128])
        kv = rng.choice([1, 2, 4])
        mixer = attention(kv * rng.choice([1, 2, 3, 4]), kv, dim, rng.choice([64, 128, 128, 32, 96]), rng.choice([64, 100, 128, 200, 4096]),
                          rng.choice([dim, dim // 2, 16]), 4 / dim, diff=rng.choice([0.3, 0.5, 0.8]),
                          base=rng.choice([10000.0, 500000.0]), scaling=rng.choice([None, yarn(8.0, 256, 32.0, 1.0)]))
        mlp = rng.choice([None, dense(rng.choice([384, 512, 768])),
                          moe(6, 2, rng.choice([64, 128]), identity=2, groups=(4, 3), shared=rng.choice([None, 128])),
                          moe(8, 3, 64, shared=256)])
        layers.append(layer(mixer, mlp))
    loop = rng.choice([None, (0, n_layers, 2), (1, n_layers, 2), (0, 1, 3)])
    return config(rng.choice([640, 1000, 2048, 4099]), width, 1e-6, layers, loop=loop, scale=rng.choice([1.0, 8.0]),
                  bigram=rng.choice([None, (251, 31, 17)]), logit_scale=rng.choice([1.0, 2.0]))


@pytest.mark.parametrize("trial", range(6))
def test_middle_sizes_drawn_at_random(trial, tmp_path):
    """A batch of two prompts (one of them in two portions) and eight tokens decoded together, both
    dtypes, at sizes of a small real model."""
    from nnis_b200.engine import Engine, SequenceStep
    rng = random.Random(9300 + trial)
    cfg = _middle_config(rng)
    d = make_model(str(tmp_path / "m"), cfg, seed=40 + trial)
    a, b = random_tokens(rng, 208, cfg["vocab"]), random_tokens(rng, 77, cfg["vocab"])
    for dtype in DTYPES:
        engine = Engine.from_dir(d, dtype=dtype, max_tokens=2048)
        sa, sb = engine.acquire_slot(), engine.acquire_slot()
        rows = []  # (request's tokens, position, logits row)
        got = engine.step([SequenceStep(sa, a[:130], [0, 63, 64, 129]), SequenceStep(sb, b[:69], [0, 68])]).cpu().numpy()
        rows += [(a, p, got[i]) for i, p in enumerate([0, 63, 64, 129])] + [(b, 0, got[4]), (b, 68, got[5])]
        got = engine.step([SequenceStep(sa, a[130:200], [0, 69])]).cpu().numpy()
        rows += [(a, 130, got[0]), (a, 199, got[1])]
        for t in range(8):
            got = engine.step([SequenceStep(sa, a[200 + t:201 + t], [0]), SequenceStep(sb, b[69 + t:70 + t], [0])]).cpu().numpy()
            rows += [(a, 200 + t, got[0]), (b, 69 + t, got[1])]
        engine.release_slot(sa)
        engine.release_slot(sb)
        engine.check_status()
        check_rows(d, dtype, rows, f"middle size {trial} {dtype}: {json.dumps(cfg)}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_through_the_entry_point(models, dtype):
    from nnis_b200 import LLM
    d = models["mixed"]
    cfg = read_config(d)
    bf = dtype == "bfloat16"
    w = load_weights(d, bf)
    llm = LLM(d, dtype=dtype, max_tokens=64 * 32, max_batch=3)
    prompts = [[5, 9, 1, 200, 33], [7], [100, 101, 102, 103, 104, 105, 106, 107, 108], [250, 3], [9] * 70]
    results = llm.generate(prompts, max_new_tokens=10, stop_token_ids=())
    for p, r in zip(prompts, results):
        assert r.ok and r.finish_reason == "length"
        if not bf:
            assert r.token_ids == P.greedy_generate(cfg, w, p, 10), (dtype, p)
        else:  # a bfloat16 near-tie may go either way: every pick must be (nearly) the plain best
            seq = list(p)
            for t in r.token_ids:
                logits = P.forward(seq, w, cfg, emulate_bf16=True)[-1]
                assert float(logits.max() - logits[t]) <= 0.05 * max(1.0, float(logits.abs().max())), (p, t)
                seq.append(t)
    # a session goes on from where generation left it, the last token and all
    session = llm.new_session()
    from nnis_b200 import GenerationConfig
    ids = session.generate(prompts[0], GenerationConfig(6))
    more = session.decode_one(17)
    if not bf:
        want = P.forward(prompts[0] + ids + [17], w, cfg)[-1]
        check_logits(np.asarray(more).reshape(1, -1), want[None, :], dtype, "session")
    assert llm.engine.cache.usage()["slots_held"] <= 1


def test_sampled_generation_and_the_command_line(models, tmp_path):
    """Sampling with a seed repeats itself, and the command line's generate runs the design."""
    import sys
    from nnis_b200 import LLM
    from nnis_b200.sampling import SamplingConfig
    llm = LLM(models["odd"], dtype="bfloat16", max_tokens=2048, max_batch=2)
    policy = SamplingConfig.seeded(5).with_temperature(0.9).with_top_k(40)
    a = llm.generate([[1, 2, 3], [9, 8]], max_new_tokens=12, sampling=policy, stop_token_ids=())
    b = llm.generate([[1, 2, 3], [9, 8]], max_new_tokens=12, sampling=policy, stop_token_ids=())
    assert [r.token_ids for r in a] == [r.token_ids for r in b] and all(len(r.token_ids) == 12 for r in a)
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "nnis"), "generate", "--model", models["loop_all"],
                        "--prompt-ids", "4,5,6", "--max-new-tokens", "5", "--dtype", "float32"],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    want = P.greedy_generate(read_config(models["loop_all"]), load_weights(models["loop_all"], False), [4, 5, 6], 5)
    assert r.stdout.split() == [str(t) for t in want]


def test_replay_program_runs_a_model_folder(models, tmp_path):
    cfg = read_config(models["loop_all"])
    toks = random_tokens(random.Random(4), 40, cfg["vocab"])
    trace = TraceBuilder()
    trace.step([("a", toks[:30], [0, 29]), ("b", toks[:7], [6])])
    trace.step([("a", toks[30:31], [0]), ("b", toks[7:8], [0])], end=["b"])
    trace.step([("a", toks[31:32], [])], end=["a"])
    out = str(tmp_path / "out")
    r = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", models["loop_all"], "--dtype", "float32",
                        "--out", out, "--max-tokens", "256"], input="\n".join(trace.lines) + "\n",
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    assert not os.path.exists(os.path.join(out, "2.f32"))
    want = plain_logits(models, "loop_all", "float32", toks)
    check_logits(read_step(out, 0, cfg["vocab"]), torch.stack([want[0], want[29], want[6]]), "float32", "program")
    check_logits(read_step(out, 1, cfg["vocab"]), torch.stack([want[30], want[7]]), "float32", "program")
