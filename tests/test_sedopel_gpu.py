"""Sedopel on the GPU against the plain implementation: the new kernels against float32
torch, every mechanism alone, whole prompts against token-by-token decoding, portions down
to two tokens, unequal batches against each request alone, slots and pages used again, keys
far away and at page borders with attention made sharp, far writes of the recurrent mixers,
the first tokens, long decoding, other sizes, greedy generation through the Python entry
point, and the replay program."""
import json
import math
import os
import random
import subprocess

import numpy as np
import pytest
import torch

import plain_sedopel as P
from helpers import TraceBuilder, check_logits, random_tokens, read_step, three_cuts
from sedopel_models import CONFIGS, load_weights, make_model, read_config

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DTYPES = ["float32", "bfloat16"]


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    return {name: make_model(str(tmp_path_factory.mktemp(f"sedopel_{name}")), cfg, seed=700 + i)
            for i, (name, cfg) in enumerate(CONFIGS.items())}


_engines, _plain = {}, {}


def engine_for(models, name, dtype):
    from nnis_b200.engine import Engine
    if (name, dtype) not in _engines:
        _engines[(name, dtype)] = Engine.from_dir(models[name], dtype=dtype, max_tokens=64 * 64)
    return _engines[(name, dtype)]


def plain_logits(models, name, dtype, tokens):
    key = (name, dtype, tuple(tokens))
    if key not in _plain:
        bf = dtype == "bfloat16"
        _plain[key] = P.forward(read_config(models[name]), load_weights(models[name], bf), tokens, emulate_bf16=bf)
    return _plain[key]


def replay_and_check(models, name, dtype, trace, sequences, tmp_path, what):
    from nnis_b200.engine.replay import replay
    engine = engine_for(models, name, dtype)
    out = str(tmp_path / f"out_{name}_{dtype}")
    replay(engine, trace.lines, out)
    usage = engine.cache.usage()
    assert usage["slots_held"] == 0 and not any(usage["pages_held"]), usage
    engine.cache.check()
    vocab = read_config(models[name])["vocab"]
    for step, rows in trace.rows.items():
        got = read_step(out, step, vocab)
        assert got.shape[0] == len(rows)
        want = torch.stack([plain_logits(models, name, dtype, sequences[rid])[pos] for rid, pos in rows])
        check_logits(got, want, dtype, f"{what} {name} {dtype} step {step}")


def run_whole(engine, tokens, want=None):
    from nnis_b200.engine import SequenceStep
    slot = engine.acquire_slot()
    try:
        return engine.step([SequenceStep(slot, tokens, list(range(len(tokens))) if want is None else want)]).cpu().numpy()
    finally:
        engine.release_slot(slot)


# ---- the new kernels against plain float32 torch ----------------------------------------------
def test_depth_mix_keeps_every_result_and_weights_them():
    from nnis_b200.csrc import ops
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(1)
    for n, width, most in ((5, 76, 4), (1, 7, 2), (33, 1000, 6)):
        history = torch.zeros(most, n, width, device=dev)
        kept = [torch.randn(n, width, generator=g)]
        history[0] = kept[0].to(dev)
        for terms in range(2, most + 1):
            result, w = torch.randn(n, width, generator=g), torch.randn(terms, generator=g)
            hidden = result.to(dev).clone()
            ops.depth_mix(hidden, history, w.to(dev), terms)
            kept.append(result)
            want = sum(w[j].double() * kept[j].double() for j in range(terms))
            assert torch.equal(history[terms - 1].cpu(), result)
            assert torch.allclose(hidden.cpu().double(), want, atol=1e-5, rtol=1e-5)


def test_closing_a_sub_layer_norms_adds_mixes_and_norms_again():
    """The kernel that ends a sub-layer, in each of its forms: the norm of the branch added to the
    stream (and the branch zero again), with and without the depth mix, with and without the norm
    that reads the rows next, in both operand dtypes and for widths that are no multiples of four."""
    from nnis_b200.csrc import ops
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(5)

    def rms(x, w, eps):
        return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w

    for n, width, most in ((5, 76, 4), (2, 7, 3), (9, 1000, 5), (3, 2048, 2)):
        for terms in (0, 2, most):
            for follower in (None, torch.float32, torch.bfloat16):
                branch, stream = torch.randn(n, width, generator=g) * 3, torch.randn(n, width, generator=g)
                w, w_next = torch.rand(width, generator=g) + 0.5, torch.rand(width, generator=g) + 0.5
                kept, mix = torch.randn(most, n, width, generator=g), torch.randn(max(terms, 1), generator=g)
                b, h, hist = branch.to(dev), stream.to(dev), kept.to(dev).clone()
                normed = torch.full((n, width), 7.0, dtype=follower, device=dev) if follower else None
                ops.sandwich_close(b, w.to(dev), 1e-5, h, hist if terms else None, mix.to(dev) if terms else None, terms,
                                   w_next.to(dev) if follower else None, 1e-6 if follower else 0.0, normed)
                result = stream.double() + rms(branch.double(), w.double(), 1e-5)
                want = result
                if terms:
                    want = mix[terms - 1].double() * result + sum(mix[j].double() * kept[j].double() for j in range(terms - 1))
                    assert torch.allclose(hist[terms - 1].cpu().double(), result, atol=1e-5, rtol=1e-5)
                    assert torch.equal(hist[:terms - 1].cpu(), kept[:terms - 1]) and torch.equal(hist[terms:].cpu(), kept[terms:])
                assert not b.any()
                assert torch.allclose(h.cpu().double(), want, atol=2e-5, rtol=1e-5)
                if follower:
                    again = rms(h.cpu().double(), w_next.double(), 1e-6)
                    tol = 1e-5 if follower == torch.float32 else 1e-2
                    assert torch.allclose(normed.cpu().double(), again, atol=tol, rtol=tol)


def test_gelu_rows_in_both_forms():
    from nnis_b200.csrc import ops
    dev = torch.device("cuda:0")
    x = torch.linspace(-9, 9, 4001)
    for kind, approx in ((ops.GELU_ERF, "none"), (ops.GELU_TANH, "tanh")):
        want = torch.nn.functional.gelu(x.double(), approximate=approx)
        out = torch.empty(4001, dtype=torch.float32, device=dev)
        ops.act_rows(x.to(dev), out, kind)
        assert torch.allclose(out.cpu().double(), want, atol=2e-6)
        out16 = torch.empty(4001, dtype=torch.bfloat16, device=dev)
        ops.act_rows(x.to(dev), out16, kind)
        assert torch.equal(out16.cpu(), out.cpu().to(torch.bfloat16))
    # the two forms differ by more than the bound above somewhere: neither can stand in for the other
    assert float((torch.nn.functional.gelu(x.double()) - torch.nn.functional.gelu(x.double(), approximate="tanh")).abs().max()) > 1e-4


@pytest.mark.parametrize("H, G, dim, vdim, taps", [(2, 1, 16, 16, 3), (4, 2, 24, 40, 4), (3, 3, 10, 7, 1), (6, 2, 72, 33, 2),
                                                   (1, 1, 256, 64, 5), (2, 2, 136, 130, 3)])
def test_delta_rule_kernels_in_portions_against_the_recurrence(H, G, dim, vdim, taps):
    """Two sequences of unequal length, each in three steps (several tokens, one token as a step of
    single tokens, several again) in two of four slots; prep, scan and finish against the recurrence
    in float64, and the other slots stay as they were."""
    from nnis_b200.csrc import ops
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(H * 100 + dim)
    channels = 2 * G * dim + H * vdim
    row_len = channels + H * vdim + 2 * H
    lengths = (45, 23)
    rows_all = [torch.randn(T, row_len, generator=g) for T in lengths]
    conv_w = torch.empty(channels, taps).uniform_(-1, 1, generator=g)
    a_log, dt_bias = torch.empty(H).uniform_(-6, 0, generator=g), torch.empty(H).uniform_(-1, 1, generator=g)
    norm_w = torch.rand(vdim, generator=g) + 0.5

    def plain(rows):
        T = rows.shape[0]
        x = rows.double()
        conv = P.short_convolution(x[:, :channels], conv_w.double())
        q = P.unit(conv[:, :G * dim].reshape(T, G, dim)) * dim ** -0.5
        k = P.unit(conv[:, G * dim:2 * G * dim].reshape(T, G, dim))
        v = conv[:, 2 * G * dim:].reshape(T, H, vdim)
        beta = torch.sigmoid(x[:, channels + H * vdim:channels + H * vdim + H])
        dec = torch.exp(-torch.exp(a_log.double()) * P.softplus(x[:, channels + H * vdim + H:] + dt_bias.double()))
        out = torch.zeros(T, H, vdim, dtype=torch.float64)
        for i in range(H):
            j = i // (H // G)
            S = torch.zeros(dim, vdim, dtype=torch.float64)
            for t in range(T):
                S = dec[t, i] * S
                u = beta[t, i] * (v[t, i] - S.T @ k[t, j])
                S = S + torch.outer(k[t, j], u)
                out[t, i] = S.T @ q[t, j]
        gate = P.silu(x[:, channels:channels + H * vdim]).reshape(T, H, vdim)
        return (P.rms_norm(out, None, 1e-5) * norm_w.double() * gate).reshape(T, H * vdim)

    want = [plain(r) for r in rows_all]
    slots = 4
    state = torch.zeros(slots, H, dim, vdim, device=dev)
    tail = torch.zeros(slots, max(taps - 1, 1), channels, device=dev)
    seq_slots = torch.tensor([2, 0], dtype=torch.int32, device=dev)
    got = [[], []]
    for cut in ((0, 20, 0, 9), (20, 21, 9, 10), (21, 45, 10, 23)):
        counts = (cut[1] - cut[0], cut[3] - cut[2])
        rows = torch.cat([rows_all[0][cut[0]:cut[1]], rows_all[1][cut[2]:cut[3]]]).to(dev)
        n = rows.shape[0]
        pos = torch.tensor(list(range(cut[0], cut[1])) + list(range(cut[2], cut[3])), dtype=torch.int32, device=dev)
        seq = torch.tensor([0] * counts[0] + [1] * counts[1], dtype=torch.int32, device=dev)
        single = counts == (1, 1)  # a step of single tokens has no table of sequences
        first = None if single else torch.tensor([0, counts[0]], dtype=torch.int32, device=dev)
        count = None if single else torch.tensor(counts, dtype=torch.int32, device=dev)
        qkv = torch.empty(n, channels, device=dev)
        beta_g = torch.empty(n, 2 * H, device=dev)
        ops.delta_prep(rows, conv_w.to(dev), tail, a_log.to(dev), dt_bias.to(dev), pos, seq, seq_slots, first, count, qkv,
                       beta_g, H, G, dim, vdim, 1e-6, dim ** -0.5)
        o_raw = torch.empty(n, H * vdim, device=dev)
        ops.delta_scan(qkv, beta_g, state, pos, seq, seq_slots, first, count, o_raw, H, G, dim, vdim)
        out = torch.empty(n, H * vdim, device=dev)
        ops.delta_finish(o_raw, rows, channels, norm_w.to(dev), pos, out, H, vdim, 1e-5)
        got[0].append(out[:counts[0]].cpu())
        got[1].append(out[counts[0]:].cpu())
    assert float(state[1].abs().max()) == 0.0 and float(state[3].abs().max()) == 0.0  # no other slot is touched
    for i in range(2):
        have = torch.cat(got[i]).double()
        assert torch.allclose(have, want[i], atol=2e-4 * float(want[i].abs().max()), rtol=0), (i, float((have - want[i]).abs().max()))
    if taps > 1:  # the convolutions' state: the last taps - 1 inputs, oldest first
        assert torch.equal(tail[2, :, :].cpu(), rows_all[0][45 - (taps - 1):, :channels])


@pytest.mark.parametrize("H, G, dim, vdim", [(2, 1, 64, 64), (4, 2, 24, 40), (3, 3, 10, 7), (2, 2, 136, 33), (1, 1, 256, 70),
                                            (2, 1, 128, 128)])
def test_delta_rule_runs_side_by_side_agree_with_the_walk_in_order(H, G, dim, vdim):
    """A step of three sequences (300, 131 and 64 tokens) that go on from states which an earlier
    step left: cut into runs of 64 tokens and put together, against the same kernel walking every
    sequence in order, and that against the recurrence in float64.  The decays reach from fast to
    almost none, so the first run's tokens still count in the last."""
    from nnis_b200.csrc import ops
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(dim + vdim)
    channels = 2 * G * dim + H * vdim
    counts = (300, 131, 64)
    n = sum(counts)
    unit = lambda x: x / torch.sqrt((x * x).sum(-1, keepdim=True) + 1e-6)
    q = unit(torch.randn(n, G, dim, generator=g)) * dim ** -0.5
    k = unit(torch.randn(n, G, dim, generator=g))
    v = torch.randn(n, H, vdim, generator=g)
    qkv = torch.cat([q.reshape(n, -1), k.reshape(n, -1), v.reshape(n, -1)], 1).to(dev)
    beta = torch.rand(n, H, generator=g)
    decay = torch.exp(-torch.exp(torch.empty(H).uniform_(-7, -1, generator=g))[None, :] * torch.rand(n, H, generator=g) * 2)
    beta_g = torch.cat([beta, decay], 1).to(dev)
    begin = torch.randn(4, H, dim, vdim, generator=g) * 0.3
    pos = torch.cat([torch.arange(5, 5 + c) for c in counts]).to(torch.int32).to(dev)
    seq = torch.cat([torch.full((c,), i) for i, c in enumerate(counts)]).to(torch.int32).to(dev)
    slots = torch.tensor([3, 0, 1], dtype=torch.int32, device=dev)
    first = torch.tensor([0, 300, 431], dtype=torch.int32, device=dev)
    count = torch.tensor(counts, dtype=torch.int32, device=dev)
    outs, states = [], []
    for runs in (False, True):
        state = begin.to(dev).clone()
        o_raw = torch.zeros(n, H * vdim, device=dev)
        extra = {}
        if runs:
            segments, first_segment = ops.scan_segments(counts, 64)
            assert segments.shape[0] == 5 + 3 + 1
            extra = dict(segments=torch.from_numpy(segments).to(dev), seq_first_segment=torch.from_numpy(first_segment).to(dev),
                         seg_len=64, seg_state=torch.full((9, H, dim, vdim), 7.0, device=dev),
                         seg_trans=torch.full((9, H, dim, dim), 7.0, device=dev), q_run=torch.full((n, H, dim), 7.0, device=dev))
        ops.delta_scan(qkv, beta_g, state, pos, seq, slots, first, count, o_raw, H, G, dim, vdim, **extra)
        outs.append(o_raw.cpu().double().reshape(n, H, vdim))
        states.append(state.cpu().double())
    want_o = torch.zeros(n, H, vdim, dtype=torch.float64)
    want_s = begin.double().clone()
    at = 0
    for i, c in enumerate(counts):
        for hh in range(H):
            j = hh // (H // G)
            S = begin[int(slots[i]), hh].double().clone()
            for t in range(at, at + c):
                S = decay[t, hh].double() * S
                u = beta[t, hh].double() * (v[t, hh].double() - S.T @ k[t, j].double())
                S = S + torch.outer(k[t, j].double(), u)
                want_o[t, hh] = S.T @ q[t, j].double()
            want_s[int(slots[i]), hh] = S
        at += c
    scale_o, scale_s = float(want_o.abs().max()), float(want_s.abs().max())
    for got_o, got_s in zip(outs, states):
        assert float((got_o - want_o).abs().max()) < 2e-5 * scale_o, float((got_o - want_o).abs().max()) / scale_o
        assert float((got_s - want_s).abs().max()) < 2e-5 * scale_s
        assert torch.equal(got_s[2], begin[2].double())  # the slot that no sequence holds
    # the first run's tokens count at the end: without them the last outputs of the long sequence differ clearly
    assert float(decay[:300].max()) > 0.999


# ---- whole models ------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["softmax", "heads64", "lightning", "delta", "dense"])
def test_each_mechanism_alone(models, name, dtype, tmp_path):
    rng = random.Random(11)
    vocab = read_config(models[name])["vocab"]
    sequences, trace = {}, TraceBuilder()
    # the first tokens, a page's border, more tokens than a tile of the scans and than a run of them
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


@pytest.mark.parametrize("name", ["mixed", "odd"])
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


def test_a_slot_used_again_starts_from_nothing(models):
    """Both recurrent states and the convolutions' last inputs are zero when a slot is taken again,
    whatever its last owner left; a snapshot brings a sequence back."""
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
    engine.step([SequenceStep(again, a[:5], [])])
    engine.restore(kept)
    rest = engine.step([SequenceStep(again, b[20:], list(range(13)))]).cpu().numpy()
    assert np.abs(rest - want[20:]).max() < 3e-5 * np.abs(want).max()
    engine.release_slot(again)


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_prompt_shape_that_recurs_is_captured_and_replayed(models, dtype):
    """A large prompt step whose shape comes a second time is recorded as a CUDA graph and replayed from
    the third time on: the states, the runs' tables, the branch buffers and the kept results of the
    layers must all live where the graph expects them.  Other tokens every time, the same shape."""
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
        for toks, pos, row in rows:
            want = plain_logits(models, "mixed", dtype, toks)[pos][None, :]
            check_logits(row[None, :], want, dtype, f"captured step, round {round_}, position {pos}")
    assert graphs == [0, 1, 1, 1], graphs


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_over_page_borders(models, dtype, tmp_path):
    vocab = read_config(models["mixed"])["vocab"]
    toks = random_tokens(random.Random(21), 5 + 200, vocab)
    trace = TraceBuilder()
    trace.step([("a", toks[:5], [4])])
    for t in range(5, len(toks)):
        trace.step([("a", toks[t:t + 1], [0])], end=["a"] if t == len(toks) - 1 else [])
    replay_and_check(models, "mixed", dtype, trace, {"a": toks}, tmp_path, "long decoding")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["lightning", "delta", "mixed"])
def test_long_prompts_of_the_recurrent_mixers_in_runs_and_portions(models, name, dtype, tmp_path):
    """Prompts longer than several runs of the recurrent kernels, alone, in a batch with short ones,
    continued after a first portion, and decoded on: a state lost or joined wrongly at a run's edge
    shows, since the slowest heads forget next to nothing over hundreds of tokens."""
    vocab = read_config(models[name])["vocab"]
    rng = random.Random(31)
    a, b, c = (random_tokens(rng, n, vocab) for n in (700, 257, 40))
    trace = TraceBuilder()
    trace.step([("a", a[:690], [0, 63, 64, 65, 127, 128, 129, 255, 256, 257, 511, 512, 689])])
    for t in range(690, 700):
        trace.step([("a", a[t:t + 1], [0])], end=["a"] if t == 699 else [])
    trace.step([("b", b[:100], [99]), ("c", c[:39], [38])])          # a first portion, then runs after it
    trace.step([("b", b[100:], list(range(150, 157))), ("c", c[39:], [0])], end=["b", "c"])
    trace.step([("a2", a, [256, 600, 699]), ("c2", c, [39]), ("b2", b, [255, 256])], end=["a2", "c2", "b2"])
    replay_and_check(models, name, dtype, trace, {"a": a, "b": b, "c": c, "a2": a, "c2": c, "b2": b}, tmp_path,
                     "runs")


def test_a_far_token_reaches_the_end_through_each_recurrent_mixer(models):
    """Changing the third token of 450 moves the last position's logits by far more than the bound
    the engine is held to, in the plain implementation, through the lightning attention alone and
    through the delta rule alone: a state that forgot it, or decayed it once too often, would show.
    The engine, fed the prompt in portions with single tokens at the end, agrees with both."""
    from nnis_b200.engine import SequenceStep
    for name in ("lightning", "delta"):
        cfg = read_config(models[name])
        toks = random_tokens(random.Random(5), 450, cfg["vocab"])
        other = list(toks)
        other[2] = (toks[2] + 1) % cfg["vocab"]
        w = load_weights(models[name], False)
        base, moved = P.forward(cfg, w, toks)[-1], P.forward(cfg, w, other)[-1]
        assert float((base - moved).abs().max()) > 20 * 1e-4 * float(base.abs().max()), name
        engine = engine_for(models, name, "float32")
        for seq, want in ((toks, base), (other, moved)):
            slot = engine.acquire_slot()
            engine.step([SequenceStep(slot, seq[:3], [])])
            engine.step([SequenceStep(slot, seq[3:300], [])])
            engine.step([SequenceStep(slot, seq[300:447], [])])
            for t in range(447, 450):
                got = engine.step([SequenceStep(slot, seq[t:t + 1], [0])]).cpu().numpy()
            engine.release_slot(slot)
            check_logits(got, want[None, :], "float32", f"far token, {name}")


def test_far_keys_and_page_borders_with_sharp_attention(models, tmp_path):
    """Scores times a large scale: most of a query's weight lies on one key, and the plain
    implementation says which.  Among those keys are far ones, ones on both sides of page borders
    and the very first; the temperatures of the heads differ, so a head that took another's would
    look elsewhere."""
    cfg = read_config(models["sharp"])
    toks = random_tokens(random.Random(8), 420, cfg["vocab"])
    probes = {}
    P.forward(cfg, load_weights(models["sharp"], False), toks, probes=probes)
    for layer in (0, 1):
        weights = torch.stack(probes[layer]["weights"])  # [heads, T, T]
        top, arg = weights.max(dim=-1)
        queries = torch.arange(420)[None, :].expand_as(arg)
        strong = top > 0.5
        assert int(strong.sum()) > 150, int(strong.sum())
        distance = (queries - arg)[strong]
        assert int((distance > 200).sum()) >= 5 and int((distance > 64).sum()) >= 30
        in_page = (arg % 64)[strong & (queries // 64 != arg // 64)]
        assert int((in_page == 63).sum()) >= 1 and int((in_page == 0).sum()) >= 1
        assert int((arg[strong & (queries > 100)] < 3).sum()) >= 1  # one of the first keys, from far on
    trace = TraceBuilder()
    trace.step([("w", toks, range(420))], end=["w"])
    trace.step([("d", toks[:150], range(150))])
    for t in range(150, 300):
        trace.step([("d", toks[t:t + 1], [0])])
    trace.step([("d", toks[300:], range(120))], end=["d"])  # and a later portion that starts inside a page
    for dtype in DTYPES:
        replay_and_check(models, "sharp", dtype, trace, {"w": toks, "d": toks}, tmp_path, "sharp")


def _random_config(rng):
    """Sizes, layer order, heads, taps, decays and constants drawn at random (small ones)."""
    from sedopel_models import config, delta, lightning, parallel, softmax
    width = rng.choice([8, 24, 36, 40, 64, 72, 100, 128])
    layers = []
    for _ in range(rng.randint(1, 6)):
        ff = rng.choice([None, None, 8, 16, 40, 64, 96, 136])
        if rng.random() < 0.55:
            kv = rng.randint(1, 3)
            dim = 2 * rng.randint(1, 40)
            left = softmax(kv * rng.randint(1, 4), kv, dim, rng.randint(1, 70), 2 * rng.randint(0, dim // 2),
                           rng.choice([0.1, 0.25, 1.0]), base=rng.choice([10.0, 10000.0, 1e6]))
            right = lightning(rng.choice([1, 3, 8, 16, 24, 32, 48, 64, 100, 128]), rng.randint(1, 70),
                              [rng.choice([1.0, 0.999, 0.97, 0.8, 0.3]) for _ in range(rng.randint(1, 4))])
            layers.append(parallel(left, right, ff))
        else:
            kv = rng.randint(1, 3)
            layers.append(delta(kv * rng.randint(1, 3), kv, rng.choice([1, 3, 8, 16, 24, 32, 48, 64, 100, 128]),
                                rng.randint(1, 70), rng.randint(1, 5), ff))
    return config(rng.choice([50, 131, 256, 577]), width, rng.choice([1e-5, 1e-6]), layers)


@pytest.mark.parametrize("trial", range(10))
def test_configurations_drawn_at_random(trial, tmp_path):
    """A prompt in one step, a second portion and six tokens one by one, both dtypes, on a model
    whose sizes, layer order and constants are drawn at random: whatever kernels the sizes select."""
    from nnis_b200.engine import Engine, SequenceStep
    rng = random.Random(8000 + trial)
    cfg = _random_config(rng)
    d = make_model(str(tmp_path / "m"), cfg, seed=trial)
    toks = random_tokens(rng, 150, cfg["vocab"])
    for dtype in DTYPES:
        bf = dtype == "bfloat16"
        want = P.forward(cfg, load_weights(d, bf), toks, emulate_bf16=bf)
        engine = Engine.from_dir(d, dtype=dtype, max_tokens=1024)
        slot = engine.acquire_slot()
        got = [engine.step([SequenceStep(slot, toks[:101], list(range(101)))]).cpu().numpy(),
               engine.step([SequenceStep(slot, toks[101:144], list(range(43)))]).cpu().numpy()]
        for t in range(144, 150):
            got.append(engine.step([SequenceStep(slot, toks[t:t + 1], [0])]).cpu().numpy())
        engine.release_slot(slot)
        engine.check_status()
        check_logits(np.concatenate(got), want, dtype, f"random configuration {trial} {dtype}: {json.dumps(cfg)}")


def _middle_config(rng):
    """Sizes of a small real model (widths of a few hundred, heads of 32 to 128, a few thousand
    vocabulary entries): the shapes at which the tensor-core products, the decode projections
    over tiles of rows and the tensor-core attention take over from the any-size kernels."""
    from sedopel_models import config, delta, lightning, parallel, softmax
    width = rng.choice([192, 256, 320, 384, 512])
    layers = []
    for _ in range(rng.randint(3, 5)):
        ff = rng.choice([None, 384, 512, 768])
        if rng.random() < 0.5:
            dim = rng.choice([32, 64, 128])
            kv = rng.choice([1, 2, 4])
            left = softmax(kv * rng.choice([1, 2, 3, 4]), kv, dim, rng.choice([dim, dim, 32, 96]), rng.choice([dim, dim // 2, 16]),
                           dim ** -0.5 * 4 / math.sqrt(dim), base=rng.choice([10000.0, 500000.0]))
            right = lightning(rng.choice([32, 64, 128]), rng.choice([32, 64, 96]),
                              [rng.choice([0.999, 0.99, 0.9, 0.6]) for _ in range(rng.choice([2, 4, 8]))])
            layers.append(parallel(left, right, ff))
        else:
            kv = rng.choice([1, 2, 4])
            layers.append(delta(kv * rng.choice([1, 2]), kv, rng.choice([32, 64, 128]), rng.choice([32, 64, 128]),
                                rng.choice([2, 3, 4]), ff))
    return config(rng.choice([640, 1000, 2048, 4099]), width, 1e-6, layers)


@pytest.mark.parametrize("trial", range(5))
def test_middle_sizes_drawn_at_random(trial, tmp_path):
    """A batch of two prompts (one of them in two portions) and eight tokens decoded together, both
    dtypes, at sizes of a small real model."""
    from nnis_b200.engine import Engine, SequenceStep
    rng = random.Random(9300 + trial)
    cfg = _middle_config(rng)
    d = make_model(str(tmp_path / "m"), cfg, seed=40 + trial)
    a, b = random_tokens(rng, 208, cfg["vocab"]), random_tokens(rng, 77, cfg["vocab"])
    for dtype in DTYPES:
        bf = dtype == "bfloat16"
        want = {name: P.forward(cfg, load_weights(d, bf), toks, emulate_bf16=bf) for name, toks in (("a", a), ("b", b))}
        engine = Engine.from_dir(d, dtype=dtype, max_tokens=2048)
        sa, sb = engine.acquire_slot(), engine.acquire_slot()
        rows = []  # (request, position, logits row)
        got = engine.step([SequenceStep(sa, a[:130], [0, 63, 64, 129]), SequenceStep(sb, b[:69], [0, 68])]).cpu().numpy()
        rows += [("a", p, got[i]) for i, p in enumerate([0, 63, 64, 129])] + [("b", 0, got[4]), ("b", 68, got[5])]
        got = engine.step([SequenceStep(sa, a[130:200], [0, 69])]).cpu().numpy()
        rows += [("a", 130, got[0]), ("a", 199, got[1])]
        for t in range(8):
            got = engine.step([SequenceStep(sa, a[200 + t:201 + t], [0]), SequenceStep(sb, b[69 + t:70 + t], [0])]).cpu().numpy()
            rows += [("a", 200 + t, got[0]), ("b", 69 + t, got[1])]
        engine.release_slot(sa)
        engine.release_slot(sb)
        engine.check_status()
        what = f"middle size {trial} {dtype}: {json.dumps(cfg)}"
        check_logits(np.stack([row for _, _, row in rows]), torch.stack([want[r][p] for r, p, _ in rows]), dtype, what)


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
                logits = P.forward(cfg, w, seq, emulate_bf16=True)[-1]
                assert float(logits.max() - logits[t]) <= 0.05 * max(1.0, float(logits.abs().max())), (p, t)
                seq.append(t)
    # a session goes on from where generation left it, state and all
    session = llm.new_session()
    from nnis_b200 import GenerationConfig
    ids = session.generate(prompts[0], GenerationConfig(6))
    more = session.decode_one(17)
    if not bf:
        want = P.forward(cfg, w, prompts[0] + ids + [17])[-1]
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
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "nnis"), "generate", "--model", models["odd"],
                        "--prompt-ids", "4,5,6", "--max-new-tokens", "5", "--dtype", "float32"],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    want = P.greedy_generate(read_config(models["odd"]), load_weights(models["odd"], False), [4, 5, 6], 5)
    assert r.stdout.split() == [str(t) for t in want]


def test_replay_program_runs_a_model_folder(models, tmp_path):
    cfg = read_config(models["odd"])
    toks = random_tokens(random.Random(4), 40, cfg["vocab"])
    trace = TraceBuilder()
    trace.step([("a", toks[:30], [0, 29]), ("b", toks[:7], [6])])
    trace.step([("a", toks[30:31], [0]), ("b", toks[7:8], [0])], end=["b"])
    trace.step([("a", toks[31:32], [])], end=["a"])
    out = str(tmp_path / "out")
    r = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", models["odd"], "--dtype", "float32",
                        "--out", out, "--max-tokens", "256"], input="\n".join(trace.lines) + "\n",
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    assert not os.path.exists(os.path.join(out, "2.f32"))
    want = plain_logits(models, "odd", "float32", toks)
    check_logits(read_step(out, 0, cfg["vocab"]), torch.stack([want[0], want[29], want[6]]), "float32", "program")
    check_logits(read_step(out, 1, cfg["vocab"]), torch.stack([want[30], want[7]]), "float32", "program")
