"""Selovik without a GPU: configuration round trip and errors by key, tensor names, the run order
of a looped model, what the design asks of the cache (a key row of both maps, the embedding's last
token), and the plain mechanisms against closed forms."""
import copy
import math

import pytest
import torch

import plain_selovik as P
from selovik_models import CONFIGS, LOOP_ALL, LOOP_ONCE, MIXED, ODD, load_weights, make_model, read_config

F = torch.float64


def test_configuration_round_trip_and_spec():
    from nnis_b200.config import config_from_dict
    for cfg in CONFIGS.values():
        typed = config_from_dict(cfg)
        assert config_from_dict(typed.to_dict()).to_dict() == typed.to_dict()
        spec = typed.to_spec()
        assert [l.block for l in spec.layers] == ["parallel"] * len(cfg["layers"])
        for i, layer in enumerate(cfg["layers"]):
            parts = spec.layers[i].parts
            assert ("ffn" in parts) == ("ffn_norm" in parts) == (layer["mlp"] is not None)
            assert parts["mixer"].kind == "differential_attention"
            assert parts["norm"]["offset"] == 1.0
    spec = config_from_dict(MIXED).to_spec()
    a = spec.layers[0].part("mixer")
    assert (a["heads"], a["kv_heads"], a["dim"], a["vdim"], a["window"], a["diff"]) == (6, 3, 24, 40, 50, 0.3)
    assert a["position"]["pairing"] == "half" and a["position"]["dims"] == 8 and a["position"]["base"] == 1000.0
    assert a["position"]["scaling"] == {"ramp": "index", "factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}
    assert spec.layers[1].part("mixer")["position"]["scaling"] is None
    assert spec.layers[0].part("ffn").kind == "mlp" and spec.layers[0].part("ffn")["activation"] == "relu2"
    m = spec.layers[1].part("ffn")
    assert m.kind == "moe" and (m["experts"], m["identity"], m["top"], m["groups"], m["keep"]) == (5, 3, 3, 4, 2)
    assert m["scores"] == "softmax_all" and m["weight_on"] == "output" and m["shared"]["intermediate_size"] == 40
    assert spec.layers[3].part("ffn")["shared"] is None and spec.layers[3].part("ffn")["groups"] == 1
    assert spec.embedding.kind == "pair_hash_embedding" and spec.embedding["scale"] == 3.0
    assert spec.embedding["pair"] == {"name": "bigram", "buckets": 101, "mul_prev": 7, "mul_cur": 13}
    assert "pair" not in config_from_dict(ODD).to_spec().embedding.params
    assert spec.head["tied_to"] == "embed" and spec.head["scale"] == 0.7


def test_a_loop_is_a_schedule_that_names_its_layers_once_per_pass():
    from nnis_b200.config import config_from_dict
    from nnis_b200.config.spec import StreamEnter
    sched = config_from_dict(MIXED).to_spec().schedule
    assert [e.layer for e in sched] == [0, 1, 2, 1, 2, 1, 2, 3]
    enters = {i: e.enter for i, e in enumerate(sched) if e.enter is not None}
    assert enters == {1: StreamEnter(False, "loop.step", 3, 0), 3: StreamEnter(True, "loop.step", 3, 1),
                      5: StreamEnter(True, "loop.step", 3, 2)}
    assert all(e.cache_of is None for e in sched)  # a cache per pass
    sched = config_from_dict(LOOP_ALL).to_spec().schedule
    assert [e.layer for e in sched] == [0, 1, 0, 1] and sched[0].enter == StreamEnter(False, "loop.step", 2, 0)
    sched = config_from_dict(LOOP_ONCE).to_spec().schedule
    assert [e.layer for e in sched] == [0, 1] and sched[1].enter == StreamEnter(False, "loop.step", 1, 0)
    assert all(e.enter is None for e in config_from_dict(ODD).to_spec().schedule)
    assert [(i, t) for i, t, first in P.run_order(MIXED) if first] == [(1, 0), (1, 1), (1, 2)]


@pytest.mark.parametrize("change, word", [
    (lambda c: c.update(architecture="Other"), "architecture"),
    (lambda c: c["layers"][0].update(type="conv"), "not a mixer"),
    (lambda c: c["layers"][0]["mixer"].update(heads=5), "multiple"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=26), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][0]["mixer"].pop("diff"), "diff"),
    (lambda c: c["layers"][0]["mixer"]["mask"].update(size=0), "size"),
    (lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].pop("fast"), "fast"),
    (lambda c: c["layers"][0]["mlp"].update(kind="experts"), "dense, moe"),
    (lambda c: c["layers"][0]["mlp"].pop("ff"), "ff"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=5), "top"),
    (lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(count=3), "groups"),
    (lambda c: c["layers"][1]["mlp"]["expert"].pop("ff"), "ff"),
    (lambda c: c["loop"].update(stop=9), "loop"),
    (lambda c: c["loop"].update(times=0), "times"),
    (lambda c: c["embedding"]["bigram"].update(buckets=0), "buckets"),
    (lambda c: c["norm"].pop("eps"), "eps"),
    (lambda c: c.update(layers=[]), "at least one layer"),
])
def test_configuration_errors_name_the_key(change, word):
    from nnis_b200.config import ConfigError, config_from_dict
    cfg = copy.deepcopy(MIXED)
    change(cfg)
    with pytest.raises(ConfigError) as e:
        config_from_dict(cfg)
    assert word in str(e.value)


def test_tensor_names_and_shapes(tmp_path):
    from nnis_b200.config import config_from_dict
    from nnis_b200.engine.model import DecoderModel
    specs = DecoderModel.weight_specs_of(config_from_dict(MIXED).to_spec())
    shapes = {n: tuple(s.shape) for n, s in specs.items() if s.role != "unused"}
    assert shapes["embed"] == (307, 96) and shapes["bigram"] == (102, 96) and shapes["embed.norm"] == (96,)
    assert shapes["loop.step"] == (3, 96) and shapes["final.norm"] == (96,)
    assert shapes["l0.mix.q"] == (6 * 2 * 24, 96) and shapes["l0.mix.k"] == (3 * 2 * 24, 96)
    assert shapes["l0.mix.v"] == (3 * 40, 96) and shapes["l0.mix.g"] == (6 * 40, 96) and shapes["l0.mix.o"] == (96, 6 * 40)
    assert all(shapes[f"l0.mix.{n}"] == (24,) for n in ("lq1", "lk1", "lq2", "lk2"))
    assert shapes["l0.mlp.up"] == (72, 96) and shapes["l0.mlp.down"] == (96, 72)
    assert shapes["l1.mlp.router"] == (8, 96) and shapes["l1.mlp.correction"] == (8,)
    assert shapes["l1.mlp.e4.gate"] == (24, 96) and shapes["l1.mlp.e4.down"] == (96, 24) and "l1.mlp.e5.gate" not in shapes
    assert shapes["l1.mlp.shared.up"] == (40, 96) and "l3.mlp.shared.up" not in shapes
    assert "l2.norm2" not in shapes and specs["l2.norm2"].role == "unused" and "l2.mlp.up" not in shapes
    assert "head" not in shapes
    d = make_model(str(tmp_path / "m"), MIXED, 3)
    assert set(load_weights(d, False)) == set(shapes)
    assert "loop.step" not in DecoderModel.weight_specs_of(config_from_dict(ODD).to_spec())


def test_the_cache_serves_both_maps_keys_and_the_embeddings_last_token():
    from nnis_b200.cache import CacheManager, KVRequest, StateRequest
    from nnis_b200.config import config_from_dict
    from nnis_b200.engine.model import DecoderModel
    model = DecoderModel(config_from_dict(MIXED).to_spec(), torch.float32, torch.device("cpu"))
    requests = model.cache_requests()
    assert len(requests) == 8 + 1
    assert requests[0] == KVRequest(3, 48, 50, True, 40) and requests[1] == requests[3] == requests[5]
    assert requests[1] == KVRequest(1, 32, 9, True, 16) and requests[-1] == StateRequest((1,), torch.int32)
    cache = CacheManager(requests, torch.float32, torch.device("cpu"), 64 * 8, 4, 1 << 20)
    # the three passes of a looped layer have storage of their own within one group
    views = [cache.view(i) for i in (1, 3, 5)]
    assert len({v.k.data_ptr() for v in views}) == 3 and len({v.group for v in views}) == 1
    last = cache.view(8).state
    assert last.dtype == torch.int32 and tuple(last.shape) == (4, 1)
    slot = cache.acquire()
    last[slot] = 77
    kept = cache.snapshot(slot)
    last[slot] = 5
    cache.restore(kept)
    assert int(last[slot]) == 77
    cache.release(slot)
    assert cache.acquire() == slot and int(last[slot]) == 0
    odd = DecoderModel(config_from_dict(ODD).to_spec(), torch.float32, torch.device("cpu"))
    assert odd.cache_requests()[-1] is None  # no pair table, no state


def test_the_position_encoding_blends_frequencies_by_index():
    from nnis_b200.parts.position import RotaryFrequencies
    for rot in (MIXED["layers"][0]["mixer"]["rot"], ODD["layers"][1]["mixer"]["rot"],
                {"dims": 64, "base": 500000.0, "scaling": {"factor": 8.0, "original": 4096, "fast": 32.0, "slow": 1.0}}):
        part = RotaryFrequencies({"dims": rot["dims"], "base": rot["base"], "pairing": "half",
                                  "scaling": {"ramp": "index", **rot["scaling"]}}, "", torch.float32, torch.device("cpu"))
        want, mag = P.rotation_frequencies(rot)
        assert torch.equal(part.frequencies()[:-1], want.to(torch.float32))
        assert part.magnitude == mag == 0.1 * math.log(rot["scaling"]["factor"]) + 1.0
    # the fast end keeps its frequencies, the slow end has them divided by the factor
    f, _ = P.rotation_frequencies({"dims": 64, "base": 10000.0,
                                   "scaling": {"factor": 8.0, "original": 2048, "fast": 32.0, "slow": 1.0}})
    plain = torch.tensor([10000.0 ** (-2.0 * i / 64) for i in range(32)], dtype=F)
    assert torch.equal(f[:5], plain[:5]) and torch.allclose(f[-3:], plain[-3:] / 8.0, rtol=1e-15)
    assert all(plain[i] / 8 < f[i] < plain[i] for i in range(15, 20))


def test_plain_rotation_turns_every_map_by_itself_and_scales_it():
    rot = {"dims": 4, "base": 100.0, "scaling": {"factor": 2.0, "original": 8, "fast": 4.0, "slow": 0.5}}
    f, mag = P.rotation_frequencies(rot)
    x = torch.arange(1, 13, dtype=F).view(1, 2, 6).repeat(3, 1, 1)  # two maps of six values, three positions
    y = P.rotate(x, torch.arange(3), rot)
    assert torch.equal(y[..., 4:], x[..., 4:])  # beyond dims: unchanged
    for p in range(3):
        for m in range(2):
            for i in range(2):  # value i turns with value i + 2
                a, b = x[p, m, i], x[p, m, i + 2]
                c, s = math.cos(p * f[i]) * mag, math.sin(p * f[i]) * mag
                assert abs(y[p, m, i] - (a * c - b * s)) < 1e-12 and abs(y[p, m, i + 2] - (b * c + a * s)) < 1e-12
    # the magnitude makes a turned pair longer by its factor
    assert abs(torch.linalg.norm(y[2, 0, :4]) / torch.linalg.norm(x[2, 0, :4]) - mag) < 1e-12


def _attention_weights(tmp_path, window, T=12):
    cfg = copy.deepcopy(LOOP_ONCE)
    cfg["layers"] = [cfg["layers"][1]]
    cfg.pop("loop")
    cfg["layers"][0]["mixer"]["mask"]["size"] = window
    d = make_model(str(tmp_path / f"w{window}"), cfg, 5)
    w = load_weights(d, False)
    h = torch.randn(T, cfg["width"], dtype=F, generator=torch.Generator().manual_seed(1))
    probe = {}
    out = P.attention(h, w, "l0.mix", cfg["layers"][0]["mixer"], 1e-5, False, probe)
    return cfg, w, h, out, probe


def test_plain_attention_sees_a_window_and_nothing_ahead(tmp_path):
    for window in (1, 3, 5, 100):
        _, _, _, _, probe = _attention_weights(tmp_path, window)
        for maps in probe["weights"]:
            for a in maps:
                for i in range(a.shape[0]):
                    seen = [j for j in range(a.shape[1]) if a[i, j] > 0]
                    assert seen == list(range(max(0, i - window + 1), i + 1))
                    assert abs(a[i].sum() - 1) < 1e-12


def test_plain_attention_is_the_normed_difference_of_two_maps(tmp_path):
    cfg, w, h, out, probe = _attention_weights(tmp_path, 100)
    m = cfg["layers"][0]["mixer"]
    lam = math.exp(float((w["l0.mix.lq1"] * w["l0.mix.lk1"]).sum())) \
        - math.exp(float((w["l0.mix.lq2"] * w["l0.mix.lk2"]).sum())) + m["diff"]
    assert abs(P.difference_weight(w, "l0.mix", m) - lam) < 1e-15 and abs(lam - m["diff"]) > 1e-3
    v = (h @ w["l0.mix.v"].T).view(-1, m["kv_heads"], m["vdim"])
    heads = []
    for a, (a1, a2) in enumerate(probe["weights"]):
        o = a1 @ v[:, 0] - lam * (a2 @ v[:, 0])
        heads.append(o / torch.sqrt((o * o).mean(-1, keepdim=True) + 1e-5) * (1 - m["diff"]))
        assert not torch.allclose(a1, a2)  # two maps, not one
    gated = torch.cat(heads, -1) * torch.sigmoid(h @ w["l0.mix.g"].T)
    assert torch.allclose(out, gated @ w["l0.mix.o"].T, atol=1e-12)


def test_plain_router_chooses_within_the_best_groups_and_weighs_by_plain_scores():
    g = torch.Generator().manual_seed(3)
    h = torch.randn(40, 16, dtype=F, generator=g)
    w = {"r.router": torch.randn(12, 16, dtype=F, generator=g), "r.correction": torch.randn(12, dtype=F, generator=g) * 0.2}
    r = {"experts": 9, "identity": 3, "top": 3, "groups": {"count": 4, "keep": 2}}
    ids, weights = P.route(h, w, "r", r)
    s = torch.softmax(h @ w["r.router"].T, -1)
    c = s + w["r.correction"]
    for t in range(40):
        best = sorted(range(4), key=lambda k: -float(c[t, 3 * k:3 * k + 3].max()))[:2]
        allowed = [e for k in best for e in range(3 * k, 3 * k + 3)]
        want = sorted(allowed, key=lambda e: -float(c[t, e]))[:3]
        assert ids[t].tolist() == want
        assert torch.equal(weights[t], s[t, want])  # the scores without the correction, not renormalised
    assert float(weights.sum(-1).max()) < 1.0
    # a masked group is out even where every allowed choice score is negative
    w["r.correction"] = w["r.correction"] - 5.0
    ids2, _ = P.route(h, w, "r", r)
    assert torch.equal(ids2, ids)


def test_plain_identity_experts_hand_the_input_on(tmp_path):
    cfg = copy.deepcopy(ODD)
    mlp = cfg["layers"][2]["mlp"]  # seven experts and five identity outputs, top four of one group
    d = make_model(str(tmp_path / "m"), cfg, 9)
    w = load_weights(d, False)
    h = torch.randn(30, cfg["width"], dtype=F, generator=torch.Generator().manual_seed(2))
    out = P.experts_ff(h, w, "l2.mlp", mlp, False)
    ids, weights = P.route(h, w, "l2.mlp", mlp["router"])
    assert (ids >= 7).any() and (ids < 7).any()
    for t in range(30):
        want = torch.zeros(cfg["width"], dtype=F)
        for e, s in zip(ids[t].tolist(), weights[t]):
            want += s * (h[t] if e >= 7 else P.gated_expert(h[t:t + 1], w, f"l2.mlp.e{e}", False)[0])
        assert torch.allclose(out[t], want, atol=1e-12)


def test_plain_embedding_hashes_the_token_before(tmp_path):
    d = make_model(str(tmp_path / "m"), MIXED, 4)
    w = load_weights(d, False)
    toks = [5, 300, 5, 5, 17]
    rows = P.bigram_rows(toks, MIXED["embedding"])
    assert rows == [101, (5 * 7 + 300 * 13) % 101, (300 * 7 + 5 * 13) % 101, (5 * 7 + 5 * 13) % 101, (5 * 7 + 17 * 13) % 101]
    x = P.embedding(toks, w, MIXED)
    raw = w["embed"][toks] * 3.0 + w["bigram"][rows]
    want = raw / torch.sqrt((raw * raw).mean(-1, keepdim=True) + 1e-5) * (1 + w["embed.norm"])
    assert torch.allclose(x, want, atol=1e-12)
    assert not torch.allclose(x[2], x[3])  # the same token after another one


def test_plain_feed_forward_is_relu_squared():
    g = torch.Generator().manual_seed(1)
    w = {"f.up": torch.randn(8, 5, dtype=F, generator=g), "f.down": torch.randn(5, 8, dtype=F, generator=g)}
    h = torch.randn(3, 5, dtype=F, generator=g)
    assert torch.allclose(P.dense_ff(h, w, "f", False), torch.clamp(h @ w["f.up"].T, min=0) ** 2 @ w["f.down"].T)


def test_plain_forward_runs_every_configuration_and_prefixes_agree(tmp_path):
    for i, (name, cfg) in enumerate(CONFIGS.items()):
        if name == "heads64":
            continue
        d = make_model(str(tmp_path / name), cfg, 20 + i)
        w = load_weights(d, False)
        toks = [(7 * t + 3) % cfg["vocab"] for t in range(40)]
        layers = []
        full = P.forward(toks, w, read_config(d), layers_out=layers)
        assert full.shape == (40, cfg["vocab"]) and torch.isfinite(full).all()
        assert len(layers) == len(P.run_order(cfg))
        part = P.forward(toks[:17], w, cfg)
        assert torch.allclose(full[:17], part, atol=1e-9)  # causal throughout
        both = P.forward(toks, w, cfg, emulate_bf16=True)
        assert 1e-6 < float((both - full).abs().max()) < 0.2 * float(full.abs().max())
