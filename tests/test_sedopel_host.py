"""Sedopel without a GPU: configuration round trip and errors by key, tensor names, what the
design asks of the cache (two requests for one layer, a state with the convolutions' last
inputs), and the plain mechanisms against closed forms."""
import copy
import math

import pytest
import torch

import plain_sedopel as P
from sedopel_models import CONFIGS, MIXED, ODD, load_weights, make_model, read_config

F = torch.float64


def test_configuration_round_trip_and_spec():
    from nnis_b200.config import config_from_dict
    for cfg in CONFIGS.values():
        typed = config_from_dict(cfg)
        assert config_from_dict(typed.to_dict()).to_dict() == typed.to_dict()
        spec = typed.to_spec()
        assert [l.block for l in spec.layers] == ["sandwich"] * len(cfg["layers"])
        for i, layer in enumerate(cfg["layers"]):
            parts = spec.layers[i].parts
            assert ("ffn" in parts) == ("ffn_norm" in parts) == ("ffn_post_norm" in parts) == (layer["mlp"] is not None)
            assert spec.layers[i].params["depth_mix"]["terms"] == i + 2
            assert spec.layers[i].params["depth_mix"]["most"] == len(cfg["layers"]) + 1
            assert parts["mixer"].kind == ("mixer_pair" if layer["type"] == "parallel" else "gated_delta_rule")
    spec = config_from_dict(MIXED).to_spec()
    pair = spec.layers[1].part("mixer")
    left, right = pair["left"], pair["right"]
    assert left.kind == "sink_attention" and left["qk_norm"] == "head" and left["gate"] == "value" and not left["sink"]
    assert left["position"]["pairing"] == "half" and left["position"]["dims"] == 8 and left["position"]["base"] == 1000.0
    assert left["scale"] == 0.3 and left["vdim"] == 40 and left["head_scale"]
    assert right.kind == "retention" and right["decay"] == (0.9, 0.999, 0.5) and right["activation"] == "silu"
    assert right["norm"] == "joined" and right["gate"] == "sigmoid" and right["key_scale"] == 1.0
    assert pair["weight"] == 0.5
    one = copy.deepcopy(MIXED)
    one["layers"][1]["mixer"]["right"]["decay"] = 0.75  # one number stands for every head
    assert config_from_dict(one).to_spec().layers[1].part("mixer")["right"]["decay"] == (0.75, 0.75, 0.75)
    delta = spec.layers[0].part("mixer")
    assert delta["taps"] == 4 and delta["kv_heads"] == 2 and delta["unit_eps"] == 1e-6 and delta["eps"] == 1e-5
    assert spec.layers[0].part("ffn")["activation"] == "gelu" and spec.layers[0].part("ffn")["intermediate_size"] == 72


@pytest.mark.parametrize("change, word", [
    (lambda c: c.update(architecture="Other"), "architecture"),
    (lambda c: c["layers"][0].update(type="conv"), "not a mixer"),
    (lambda c: c["layers"][0]["mixer"].update(heads=5), "multiple"),
    (lambda c: c["layers"][0]["mixer"].update(conv=0), "conv"),
    (lambda c: c["layers"][1]["mixer"]["left"].update(heads=7), "multiple"),
    (lambda c: c["layers"][1]["mixer"]["left"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][1]["mixer"]["left"]["rot"].update(dims=26), "rot.dims"),
    (lambda c: c["layers"][1]["mixer"]["left"].pop("scale"), "scale"),
    (lambda c: c["layers"][1]["mixer"]["right"].update(decay=[0.5]), "decay"),
    (lambda c: c["layers"][1]["mixer"]["right"].update(decay=[0.5, 1.5, 0.2]), "decay"),
    (lambda c: c["layers"][1]["mixer"].pop("right"), "right"),
    (lambda c: c["layers"][0]["mlp"].update(kind="experts"), "dense"),
    (lambda c: c["layers"][0]["mlp"].pop("ff"), "ff"),
    (lambda c: c["norm"].pop("eps"), "eps"),
    (lambda c: c.update(layers=[]), "layers"),
    (lambda c: c.update(width=0), "width"),
])
def test_configuration_errors_name_the_key(change, word):
    from nnis_b200.config import ConfigError, config_from_dict
    cfg = copy.deepcopy(MIXED)
    change(cfg)
    with pytest.raises(ConfigError, match=word):
        config_from_dict(cfg)


def test_tensor_names_and_shapes(tmp_path):
    from nnis_b200.config import config_from_dict
    from nnis_b200.engine.model import DecoderModel
    want = DecoderModel.weight_specs_of(config_from_dict(MIXED).to_spec())
    for name in ("embed", "head", "final.norm", "l0.norm1", "l0.norm1b", "l0.norm2", "l0.norm2b", "l0.mix.q", "l0.mix.q.conv",
                 "l0.mix.k.conv", "l0.mix.v.conv", "l0.mix.b", "l0.mix.a", "l0.mix.A_log", "l0.mix.dt_bias", "l0.mix.norm",
                 "l0.mix.g", "l0.mix.o", "l0.mlp.up", "l0.mlp.down", "l0.dwa", "l1.mix.left.q", "l1.mix.left.temp",
                 "l1.mix.left.g", "l1.mix.left.out", "l1.mix.right.norm", "l1.mix.right.out", "l1.mix.right.g", "l4.dwa"):
        assert name in want, name
    for name in ("l2.norm2", "l2.mlp.up", "l3.norm2b", "l0.mix.q.weight", "l1.mix.left.q.norm", "l1.mix.left.sink"):
        assert name not in want, name
    assert want["l0.dwa"].shape == (2,) and want["l4.dwa"].shape == (6,)
    assert want["l0.mix.q"].shape == (2 * 24, 96) and want["l0.mix.v"].shape == (4 * 16, 96)
    assert want["l0.mix.v.conv"].shape == (64, 4) and want["l0.mix.b"].shape == (4, 96) and want["l0.mix.norm"].shape == (16,)
    assert want["l1.mix.left.g"].shape == (6 * 40, 96) and want["l1.mix.left.o"].shape == (96, 6 * 40)
    assert want["l1.mix.left.temp"].shape == (6,) and want["l1.mix.right.norm"].shape == (3 * 24,)
    assert want["l1.mix.right.q"].shape == (3 * 16, 96) and want["l1.mix.left.out"].shape == (96,)
    # every configuration's random folder holds exactly the wanted names
    for i, (name, cfg) in enumerate(CONFIGS.items()):
        d = make_model(str(tmp_path / name), cfg, seed=i)
        assert set(load_weights(d, False)) == set(DecoderModel.weight_specs_of(config_from_dict(cfg).to_spec())), name


def test_the_cache_serves_a_pair_of_requests_and_the_convolutions_inputs():
    from nnis_b200.cache import CacheManager, KVRequest, StateRequest
    requests = [(KVRequest(3, 24, 0, True, 40), StateRequest((3, 16, 24))),
                StateRequest((4, 24, 16), extra=(((3, 112), torch.float32),)),
                (KVRequest(3, 24, 0, True, 40), StateRequest((1, 40, 8)))]
    cache = CacheManager(requests, torch.bfloat16, torch.device("cpu"), 640, 4, 1 << 20)
    pair, delta, other = cache.view(0), cache.view(1), cache.view(2)
    assert isinstance(pair, tuple) and len(pair) == 2 and len(cache.groups) == 1
    assert pair[0].group == other[0].group and tuple(pair[0].v.shape[1:]) == (3, 64, 40)
    assert pair[1].state.dtype == torch.float32 and tuple(pair[1].state.shape) == (4, 3, 16, 24)
    assert tuple(delta.extra[0].shape) == (4, 3, 112) and tuple(other[1].state.shape) == (4, 1, 40, 8)
    slot = cache.acquire()
    for x in (pair[1].state, delta.state, delta.extra[0], other[1].state):
        x[slot].fill_(2.0)
    kept = cache.snapshot(slot)
    delta.extra[0][slot].fill_(9.0)
    pair[1].state[slot].fill_(9.0)
    cache.restore(kept)
    assert float(delta.extra[0][slot].max()) == 2.0 and float(pair[1].state[slot].max()) == 2.0
    cache.release(slot)
    assert cache.acquire() == slot  # a slot taken again starts from nothing
    assert all(float(x[slot].abs().max()) == 0.0 for x in (pair[1].state, delta.state, delta.extra[0], other[1].state))
    cache.check()


# ---- the plain mechanisms against closed forms ----------------------------------------------
def test_plain_rotation_pairs_a_value_with_the_one_half_the_range_on():
    x = (torch.arange(2 * 1 * 7, dtype=F).reshape(2, 1, 7) + 1)
    y = P.rotate_halves(x, torch.tensor([0, 3]), 4, 100.0)
    assert torch.equal(y[0], x[0]) and torch.equal(y[1, 0, 4:], x[1, 0, 4:])
    # values 0 and 2 turn by 3 * 100^0, values 1 and 3 by 3 * 100^(-2/4)
    for i, f in ((0, 1.0), (1, 0.1)):
        c, s = math.cos(3 * f), math.sin(3 * f)
        a, b = float(x[1, 0, i]), float(x[1, 0, i + 2])
        assert abs(float(y[1, 0, i]) - (a * c - b * s)) < 1e-12 and abs(float(y[1, 0, i + 2]) - (b * c + a * s)) < 1e-12
    assert torch.equal(P.rotate_halves(x, torch.tensor([5, 9]), 0, 100.0), x)
    # a rotation: the product of a rotated query and key depends on the distance alone
    torch.manual_seed(0)
    q, k = torch.randn(1, 1, 6, dtype=F), torch.randn(1, 1, 6, dtype=F)
    dots = [float((P.rotate_halves(q, torch.tensor([p + 4]), 6, 50.0) * P.rotate_halves(k, torch.tensor([p]), 6, 50.0)).sum())
            for p in (0, 11, 250)]
    assert abs(dots[0] - dots[1]) < 1e-9 and abs(dots[0] - dots[2]) < 1e-9


def _softmax_weights(T, temp, scale, q_rows, k_rows):
    m = {"heads": 2, "kv_heads": 1, "dim": 2, "vdim": 1, "scale": scale, "rot": {"dims": 0, "base": 10.0}}
    w = {"a.q": q_rows, "a.k": k_rows, "a.v": torch.tensor([[1.0, 0.0]], dtype=F), "a.temp": torch.tensor(temp, dtype=F),
         "a.g": torch.zeros(2, 2, dtype=F), "a.o": torch.eye(2, dtype=F)}
    probe = {}
    h = torch.stack([torch.tensor([1.0, float(t)], dtype=F) for t in range(T)])
    out = P.softmax_attention(h, w, "a", m, 1e-12, False, probe)
    return probe["weights"], out


def test_plain_softmax_attention_is_causal_normed_per_head_and_has_a_temperature():
    # q = (1, 0) whatever the token; k = (1, t) normed to root mean square 1: k_t = sqrt(2) (1, t) / |(1, t)|
    q_rows = torch.tensor([[1.0, 0.0], [0.0, 0.0], [3.0, 0.0], [0.0, 0.0]], dtype=F)  # head 1's q is thrice head 0's: the norm undoes it
    k_rows = torch.eye(2, dtype=F)
    weights, out = _softmax_weights(5, [1.0, 2.0], 0.7, q_rows, k_rows)
    for head, temp in ((0, 1.0), (1, 2.0)):
        a = weights[head]
        assert torch.equal(a, torch.tril(a)) and torch.allclose(a.sum(-1), torch.ones(5, dtype=F))
        score = torch.tensor([math.sqrt(2.0) * math.sqrt(2.0) / math.hypot(1.0, t) * 0.7 * temp for t in range(5)], dtype=F)
        for i in range(5):
            assert torch.allclose(a[i, :i + 1], torch.softmax(score[:i + 1], 0), atol=1e-9)
    # all values are one, the gate's logits zero: every output value is a half
    assert torch.allclose(out, torch.full((5, 2), 0.5, dtype=F))


def test_plain_lightning_attention_is_the_decayed_sum():
    torch.manual_seed(2)
    T, W, H, d, dv = 6, 5, 2, 3, 2
    m = {"heads": H, "dim": d, "vdim": dv, "decay": [0.5, 1.0]}
    w = {"a.q": torch.randn(H * d, W, dtype=F), "a.k": torch.randn(H * d, W, dtype=F), "a.v": torch.randn(H * dv, W, dtype=F),
         "a.g": torch.randn(H * dv, W, dtype=F), "a.norm": torch.rand(H * dv, dtype=F) + 0.5, "a.o": torch.eye(H * dv, dtype=F)}
    h = torch.randn(T, W, dtype=F)
    got = P.lightning_attention(h, w, "a", m, 1e-9, False)
    q, k, v = (P.silu(h @ w[f"a.{p}"].T) for p in "qkv")
    for t in range(T):
        o = torch.cat([sum(m["decay"][i] ** (t - j) * (q[t, i * d:(i + 1) * d] @ k[j, i * d:(i + 1) * d]) * v[j, i * dv:(i + 1) * dv]
                           for j in range(t + 1)) for i in range(H)])
        want = o / torch.sqrt((o * o).mean() + 1e-9) * w["a.norm"] * torch.sigmoid(h[t] @ w["a.g"].T)
        assert torch.allclose(got[t], want, atol=1e-9)


def test_plain_short_convolution_reads_the_last_inputs_and_zeros_before_the_start():
    torch.manual_seed(3)
    x, taps = torch.randn(7, 4, dtype=F), torch.randn(4, 3, dtype=F)
    got = P.short_convolution(x, taps)
    want = torch.nn.functional.conv1d(torch.nn.functional.pad(x.T[None], (2, 0)), taps[:, None, :], groups=4)[0].T
    assert torch.allclose(got, P.silu(want), atol=1e-12)
    assert torch.allclose(got[0], P.silu(x[0] * taps[:, 2]))  # the last column is the current token's
    one = P.short_convolution(x, taps[:, 2:])                 # one tap: no memory
    assert torch.allclose(one, P.silu(x * taps[:, 2]))


def _delta_weights(W, H, G, d, dv, taps=1):
    """Projections that pass the input through: h = [q (G d) | k (G d) | v (H dv) | b (H) | a (H)]."""
    assert W == 2 * G * d + H * dv + 2 * H
    eye = torch.eye(W, dtype=F)
    conv = lambda n: torch.cat([torch.zeros(n, taps - 1, dtype=F), torch.ones(n, 1, dtype=F)], 1)
    at = [0, G * d, 2 * G * d, 2 * G * d + H * dv, 2 * G * d + H * dv + H, W]
    return {"a.q": eye[at[0]:at[1]], "a.k": eye[at[1]:at[2]], "a.v": eye[at[2]:at[3]], "a.b": eye[at[3]:at[4]],
            "a.a": eye[at[4]:at[5]], "a.q.conv": conv(G * d), "a.k.conv": conv(G * d), "a.v.conv": conv(H * dv),
            "a.A_log": torch.zeros(H, dtype=F), "a.dt_bias": torch.zeros(H, dtype=F), "a.norm": torch.ones(dv, dtype=F),
            "a.g": torch.zeros(H * dv, W, dtype=F), "a.o": torch.eye(H * dv, dtype=F)}, at


def test_plain_delta_rule_replaces_what_a_key_holds_and_decays_the_rest():
    """With beta = 1 and no decay a write makes the state answer its key with its value exactly,
    whatever was there; keys at right angles do not disturb one another; the decay shrinks what is
    kept by its factor a token."""
    H, G, d, dv = 1, 1, 2, 2
    w, at = _delta_weights(8, H, G, d, dv)
    big = 40.0  # sigmoid(40) = 1; softplus(-40) = 0, so the decay is exp(0) = 1

    def row(q, k, v, b=big, a=-big):
        return torch.tensor(list(q) + list(k) + list(v) + [b, a], dtype=F)
    def pre(y):  # silu acts on q, k and v: the x with silu(x) = y, y >= 0
        lo, hi = 0.0, 50.0
        for _ in range(200):
            mid = (lo + hi) / 2
            lo, hi = (mid, hi) if mid / (1 + math.exp(-mid)) < y else (lo, mid)
        return lo
    e0, e1 = (pre(1.0), 0.0), (0.0, pre(1.0))
    v1, v2, v3 = (pre(0.5), pre(2.0)), (pre(3.0), pre(1.0)), (pre(0.25), pre(4.0))
    h = torch.stack([row(e0, e0, v1), row(e1, e1, v2), row(e0, e0, v3), row(e1, e0, (0.0, 0.0), b=-big)])
    m = {"heads": H, "kv_heads": G, "dim": d, "vdim": dv, "conv": 1}
    probe = {}
    got = P.delta_mixer(h, w, "a", m, 1e-12, False, probe)
    assert torch.allclose(probe["decay"], torch.ones(4, 1, dtype=F), atol=1e-12)
    rms = lambda o: o / torch.sqrt((o * o).mean() + 1e-12)
    # the gate's logits are zero and silu(0) = 0: nothing comes out; then the gate reads b's input
    assert float(got.abs().max()) == 0.0
    w["a.g"][:, 6] = 1.0  # gate logits = b's input: silu(40) = 40 on the first three rows
    got = P.delta_mixer(h, w, "a", m, 1e-12, False)
    unit_q = d ** -0.5  # the unit query times dim^-1/2 (unit_eps shifts it by 5e-7)
    for t, v in ((0, (0.5, 2.0)), (1, (3.0, 1.0)), (2, (0.25, 4.0))):
        want = rms(torch.tensor(v, dtype=F) * unit_q) * P.silu(torch.tensor(big, dtype=F))
        assert torch.allclose(got[t], want, rtol=1e-5), (t, got[t], want)
    # token 3 writes nothing (beta = 0) and reads key e1: still v2, after key e0 was written twice
    want = rms(torch.tensor((3.0, 1.0), dtype=F) * unit_q) * P.silu(torch.tensor(-big, dtype=F))
    assert torch.allclose(got[3], want, rtol=1e-5)
    # with a decay: a = 0, A_log = 0, dt_bias = 0 gives g = exp(-softplus(0)) = 1/2 a token
    h2 = torch.stack([row(e0, e0, v1, a=0.0), row(e0, e1, (0.0, 0.0), b=-big, a=0.0), row(e0, e1, (0.0, 0.0), b=-big, a=0.0)])
    probe = {}
    w["a.g"] = torch.zeros(H * dv, 8, dtype=F)
    w["a.g"][:, 7] = 1.0
    w["a.norm"] = torch.ones(dv, dtype=F)
    P.delta_mixer(h2, w, "a", m, 1e-12, False, probe)
    assert torch.allclose(probe["decay"], torch.full((3, 1), 0.5, dtype=F), atol=1e-12)


def test_plain_delta_rule_is_its_matrix_form():
    """S_t = g_t (I - beta_t k_t k_t^T) S_(t-1) + beta_t k_t v_t^T, o_t = S_t^T q_t, with several heads on one
    key head, a convolution of three taps and decays from A_log and dt_bias."""
    torch.manual_seed(5)
    T, W, H, G, d, dv, taps = 9, 7, 4, 2, 3, 2, 3
    m = {"heads": H, "kv_heads": G, "dim": d, "vdim": dv, "conv": taps}
    w = {"a.q": torch.randn(G * d, W, dtype=F), "a.k": torch.randn(G * d, W, dtype=F), "a.v": torch.randn(H * dv, W, dtype=F),
         "a.b": torch.randn(H, W, dtype=F), "a.a": torch.randn(H, W, dtype=F), "a.g": torch.randn(H * dv, W, dtype=F),
         "a.q.conv": torch.randn(G * d, taps, dtype=F), "a.k.conv": torch.randn(G * d, taps, dtype=F),
         "a.v.conv": torch.randn(H * dv, taps, dtype=F), "a.A_log": torch.randn(H, dtype=F), "a.dt_bias": torch.randn(H, dtype=F),
         "a.norm": torch.rand(dv, dtype=F) + 0.5, "a.o": torch.eye(H * dv, dtype=F)}
    h = torch.randn(T, W, dtype=F)
    got = P.delta_mixer(h, w, "a", m, 1e-7, False).view(T, H, dv)
    conv = lambda p: P.short_convolution(h @ w[f"a.{p}"].T, w[f"a.{p}.conv"])
    q, k, v = conv("q").view(T, G, d), conv("k").view(T, G, d), conv("v").view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) / math.sqrt(d)
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w["a.b"].T)
    g = torch.exp(-torch.exp(w["a.A_log"]) * torch.log1p(torch.exp(h @ w["a.a"].T + w["a.dt_bias"])))
    gate = P.silu(h @ w["a.g"].T).view(T, H, dv)
    for i in range(H):
        j = i // 2
        S = torch.zeros(d, dv, dtype=F)
        for t in range(T):
            S = g[t, i] * (torch.eye(d, dtype=F) - beta[t, i] * torch.outer(k[t, j], k[t, j])) @ S \
                + beta[t, i] * torch.outer(k[t, j], v[t, i])
            o = S.T @ q[t, j]
            want = o / torch.sqrt((o * o).mean() + 1e-7) * w["a.norm"] * gate[t, i]
            assert torch.allclose(got[t, i], want, atol=1e-9), (i, t)


def test_plain_feed_forward_is_the_erf_gelu():
    w = {"a.up": torch.tensor([[1.0], [-2.0], [0.25]], dtype=F), "a.down": torch.eye(3, dtype=F)}
    got = P.feed_forward(torch.tensor([[1.5]], dtype=F), w, "a", False)[0]
    want = torch.nn.functional.gelu(torch.tensor([1.5, -3.0, 0.375], dtype=F))  # (the exact form, not the tanh one)
    assert torch.allclose(got, want, atol=1e-12)
    assert abs(float(got[0]) - 1.5 * 0.5 * (1 + math.erf(1.5 / math.sqrt(2)))) < 1e-12


def test_plain_depth_average_weights_every_result_so_far(tmp_path):
    """The stream after layer i is sum_j dwa_i[j] X_j, X_0 the embedding output and X_(j+1) layer j's
    result before its own averaging; checked by rebuilding it from the streams the forward reports."""
    cfg = copy.deepcopy(CONFIGS["dense"])
    cfg["layers"] = cfg["layers"] * 3
    d = make_model(str(tmp_path / "m"), cfg, seed=3)
    w = {k: v.to(F) for k, v in load_weights(d, False).items()}
    toks = [3, 1, 4, 1, 5, 9, 2, 6]
    streams = []
    P.forward(cfg, w, toks, streams=streams)
    x = w["embed"][torch.tensor(toks)]
    results = [x]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}"
        x = x + P.rms_norm(P.delta_mixer(P.rms_norm(x, w[p + ".norm1"], 1e-5), w, p + ".mix", layer["mixer"], 1e-5, False),
                           w[p + ".norm1b"], 1e-5)
        x = x + P.rms_norm(P.feed_forward(P.rms_norm(x, w[p + ".norm2"], 1e-5), w, p + ".mlp", False), w[p + ".norm2b"], 1e-5)
        results.append(x)
        x = torch.stack([w[p + ".dwa"][j] * results[j] for j in range(i + 2)]).sum(0)
        assert torch.allclose(streams[i], x, atol=1e-12)
    assert all(float((w[f"l{i}.dwa"] - 1).abs().min()) > 0.05 for i in range(3))  # no weight that a one would hide


def test_plain_forward_runs_every_configuration_and_prefixes_agree(tmp_path):
    """Causality: the logits of a prefix are the logits of the whole at those positions."""
    for i, (name, cfg) in enumerate(CONFIGS.items()):
        d = make_model(str(tmp_path / name), cfg, seed=i)
        w = load_weights(d, False)
        toks = [(7 * j + i) % cfg["vocab"] for j in range(30)]
        whole = P.forward(read_config(d), w, toks)
        part = P.forward(read_config(d), w, toks[:17])
        assert torch.isfinite(whole).all() and torch.allclose(whole[:17], part, atol=1e-9), name
    assert ODD["width"] % 8 and MIXED["layers"][0]["type"] == "delta"
