"""Selovik, plainly: whole sequences, no cache, no batches, float64, one function per
mechanism, written from the design's equations.  It reads config.json's keys and the
tensor names by itself and shares no code with the package.

``emulate_bf16`` rounds where the bfloat16 engine rounds (the normed rows that feed the
projections, q and the cached k and v after the rotation, the gated heads before the output
projection, the feed-forwards' activations); embedding sum, norms, angles, scores, softmax,
the two maps' difference and its norm, routers and the residual sum stay exact.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F = torch.float64


def bf(x: torch.Tensor, on: bool) -> torch.Tensor:
    return x.to(torch.bfloat16).to(F) if on else x


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def centred_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """The stored weight lies around zero: the multiplier is 1 + w."""
    return rms(x, eps) * (1.0 + w.to(F))


# ---- embedding ----------------------------------------------------------------------------
def bigram_rows(tokens: List[int], e: dict) -> List[int]:
    """Row of the pair table for every token: a hash of (token before, token); the first
    token of a sequence takes the table's last row."""
    b = e["bigram"]
    rows = []
    for i, t in enumerate(tokens):
        rows.append(b["buckets"] if i == 0 else (tokens[i - 1] * b["mul_prev"] + t * b["mul_cur"]) % b["buckets"])
    return rows


def embedding(tokens: List[int], w: Dict[str, torch.Tensor], cfg: dict) -> torch.Tensor:
    e = cfg["embedding"]
    x = w["embed"].to(F)[tokens] * float(e["scale"])
    if e.get("bigram"):
        x = x + w["bigram"].to(F)[bigram_rows(tokens, e)]
    return centred_norm(x, w["embed.norm"], cfg["norm"]["eps"])


# ---- rotation -----------------------------------------------------------------------------
def rotation_frequencies(rot: dict) -> (torch.Tensor, float):
    """f_i = base^(-2i/dims), slowed down at long wavelengths; returns them with the number
    that multiplies every cosine and sine."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, original = float(sc["factor"]), float(sc["original"])

    def turn_to_dim(turns):  # the (fractional) index whose wavelength makes `turns` turns over `original`
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(turn_to_dim(float(sc["fast"]))), 0)
    hi = min(math.ceil(turn_to_dim(float(sc["slow"]))), dims - 1)
    ramp = torch.clamp((torch.arange(dims // 2, dtype=F) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x: torch.Tensor, positions: torch.Tensor, rot: dict) -> torch.Tensor:
    """x [T, heads, d]: of the first ``dims`` values, value i turns with value i + dims/2."""
    dims = int(rot["dims"])
    half = dims // 2
    if half == 0:
        return x
    f, mag = rotation_frequencies(rot)
    angle = positions.to(F)[:, None] * f[None, :]
    c, s = (torch.cos(angle) * mag)[:, None, :], (torch.sin(angle) * mag)[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., dims:]], dim=-1)


# ---- differential attention ---------------------------------------------------------------
def difference_weight(w, p, m) -> float:
    lam = math.exp(float((w[p + ".lq1"].to(F) * w[p + ".lk1"].to(F)).sum())) \
        - math.exp(float((w[p + ".lq2"].to(F) * w[p + ".lk2"].to(F)).sum())) + float(m["diff"])
    return lam


def attention(h, w, p, m, eps, e16, probe=None):
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    positions = torch.arange(T)
    # [T, head, map, d]: every map of every head is turned by itself
    q = rotate((h @ w[p + ".q"].to(F).T).view(T, H * 2, d), positions, m["rot"]).view(T, H, 2, d)
    k = rotate((h @ w[p + ".k"].to(F).T).view(T, G * 2, d), positions, m["rot"]).view(T, G, 2, d)
    q, k = bf(q, e16), bf(k, e16)
    v = bf((h @ w[p + ".v"].to(F).T).view(T, G, dv), e16)
    size = int(m["mask"]["size"])
    i = torch.arange(T)
    visible = (i[:, None] >= i[None, :]) & (i[:, None] - i[None, :] < size)
    lam = difference_weight(w, p, m)
    out = torch.zeros(T, H, dv, dtype=F)
    for a in range(H):
        g = a // (H // G)
        maps = []
        for c in range(2):
            s = (q[:, a, c] @ k[:, g, c].T) * float(m["scale"])
            maps.append(torch.softmax(s.masked_fill(~visible, -math.inf), dim=-1))
        if probe is not None:
            probe.setdefault("weights", []).append(maps)
        o = maps[0] @ v[:, g] - lam * (maps[1] @ v[:, g])
        out[:, a] = rms(o, eps) * (1.0 - float(m["diff"]))
    gated = bf(out.reshape(T, H * dv) * torch.sigmoid(h @ w[p + ".g"].to(F).T), e16)
    return gated @ w[p + ".o"].to(F).T


# ---- feed-forwards ------------------------------------------------------------------------
def silu(x):
    return x * torch.sigmoid(x)


def dense_ff(h, w, p, e16):
    return bf(torch.relu(h @ w[p + ".up"].to(F).T) ** 2, e16) @ w[p + ".down"].to(F).T


def gated_expert(h, w, p, e16):
    return bf(silu(h @ w[p + ".gate"].to(F).T) * (h @ w[p + ".up"].to(F).T), e16) @ w[p + ".down"].to(F).T


def route(h, w, p, r, probe=None):
    """ids [T, top] over experts and identity experts together, and the scores of the chosen."""
    total = int(r["experts"]) + int(r.get("identity", 0))
    s = torch.softmax(h @ w[p + ".router"].to(F).T, dim=-1)
    choice = s + w[p + ".correction"].to(F) if (p + ".correction") in w else s.clone()
    groups = r.get("groups")
    group_gap = torch.full((h.shape[0],), math.inf, dtype=F)
    if groups and int(groups["count"]) > 1:
        count, keep = int(groups["count"]), int(groups["keep"])
        best = choice.view(-1, count, total // count).max(dim=-1).values
        kept = torch.zeros_like(best, dtype=torch.bool)
        kept.scatter_(1, best.topk(keep, dim=-1).indices, True)
        choice = choice.masked_fill(~kept.repeat_interleave(total // count, dim=1), -math.inf)
        if keep < count:  # how clearly the last group kept beats the first one left out
            ranked = best.sort(dim=-1, descending=True).values
            group_gap = ranked[:, keep - 1] - ranked[:, keep]
    ids = choice.topk(int(r["top"]), dim=-1).indices
    if probe is not None:
        # how clearly the choice was made: the last expert chosen against the first one left out, and the groups
        ordered = choice.sort(dim=-1, descending=True).values
        gap = ordered[:, int(r["top"]) - 1] - ordered[:, int(r["top"])] if total > int(r["top"]) \
            else torch.full((h.shape[0],), math.inf, dtype=F)
        probe.setdefault("gaps", []).append(torch.minimum(gap, group_gap))
    return ids, s.gather(1, ids)


def experts_ff(h, w, p, mlp, e16, probe=None):
    r = mlp["router"]
    E = int(r["experts"])
    ids, weights = route(h, w, p, r, probe)
    out = torch.zeros(h.shape[0], w[p + ".e0.down"].shape[0] if E else h.shape[1], dtype=F)
    for t in range(h.shape[0]):
        for e, s in zip(ids[t].tolist(), weights[t]):
            # the last `identity` outputs of the router stand for experts that hand their input on
            out[t] += s * (gated_expert(h[t:t + 1], w, f"{p}.e{e}", e16)[0] if e < E else h[t])
    if mlp.get("shared"):
        out = out + gated_expert(h, w, p + ".shared", e16)
    return out


# ---- the model ----------------------------------------------------------------------------
def run_order(cfg: dict) -> List[tuple]:
    """(layer, pass number or None, first of its pass) in the order the layers run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop or int(loop["times"]) <= 0:
        return [(i, None, False) for i in range(n)]
    start, stop, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    order = [(i, None, False) for i in range(start)]
    for t in range(times):
        order += [(i, t, i == start) for i in range(start, stop)]
    return order + [(i, None, False) for i in range(stop, n)]


def forward(tokens: List[int], w: Dict[str, torch.Tensor], cfg: dict, emulate_bf16: bool = False,
            probe: Optional[dict] = None, layers_out: Optional[list] = None) -> torch.Tensor:
    eps = float(cfg["norm"]["eps"])
    e16 = emulate_bf16
    x0 = embedding(tokens, w, cfg)
    x = x0.clone()
    for i, t, first in run_order(cfg):
        layer = cfg["layers"][i]
        p = f"l{i}"
        if first:
            if t > 0:
                x = x + x0
            x = x + w["loop.step"].to(F)[t]
        h1 = bf(centred_norm(x, w[p + ".norm1"], eps), e16)
        y = attention(h1, w, p + ".mix", layer["mixer"], eps, e16, probe)
        mlp = layer.get("mlp")
        if mlp is not None:
            h2 = bf(centred_norm(x, w[p + ".norm2"], eps), e16)  # (of the same x as the mixer's)
            y = y + (dense_ff(h2, w, p + ".mlp", e16) if mlp["kind"] == "dense"
                     else experts_ff(h2, w, p + ".mlp", mlp, e16, probe))
        x = x + y
        if layers_out is not None:
            layers_out.append(x.clone())
    h = bf(centred_norm(x, w["final.norm"], eps), e16)
    return (h @ w["embed"].to(F).T) * float(cfg.get("logit_scale", 1.0))


def greedy_generate(cfg: dict, w: Dict[str, torch.Tensor], prompt: List[int], n: int) -> List[int]:
    """n tokens, each the largest logit after everything so far (ties to the lower id)."""
    seq, out = list(prompt), []
    for _ in range(n):
        logits = forward(seq, w, cfg)[-1]
        t = int(torch.nonzero(logits == logits.max())[0])
        out.append(t)
        seq.append(t)
    return out
