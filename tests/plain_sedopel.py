"""Sedopel, plainly: whole sequences, no cache, no batches, float64, one function per
mechanism, written from the design's equations.  It reads config.json's keys and the
tensor names by itself and shares no code with the package.

``emulate_bf16`` rounds where the bfloat16 engine rounds (the normed rows that feed the
projections, q, k and v of the softmax attention as they are cached, the lightning
attention's projections, every sub-layer's last activation before its output projection);
norms, scores, softmax, recurrences and what enters them, the depth-weighted sum and the
residual sum stay exact.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F = torch.float64
UNIT_EPS = 1e-6


def bf(x: torch.Tensor, on: bool) -> torch.Tensor:
    return x.to(torch.bfloat16).to(F) if on else x


def rms_norm(x: torch.Tensor, w: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return y if w is None else y * w


def silu(x):
    return x * torch.sigmoid(x)


def softplus(x):
    return torch.where(x > 30, x, torch.log1p(torch.exp(torch.clamp(x, max=30))))


def gelu_erf(x):
    return 0.5 * x * (1.0 + torch.erf(x / math.sqrt(2.0)))


# ---- rotation --------------------------------------------------------------------------
def rotate_halves(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x [T, heads, d]: of the first ``dims`` values of every head, value i and value
    i + dims / 2 are turned together by position * base^(-2i / dims); the rest pass."""
    half = dims // 2
    if half == 0:
        return x
    f = torch.tensor([float(base) ** (-2.0 * i / dims) for i in range(half)], dtype=F)
    angle = positions.to(F)[:, None] * f[None, :]
    c, s = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., dims:]], dim=-1)


# ---- softmax attention with a temperature per head and a gate per value -------------------
def softmax_attention(h, w, p, m, eps, e16, probe=None):
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    positions = torch.arange(T)
    q = rotate_halves((h @ w[p + ".q"].T).view(T, H, d), positions, m["rot"]["dims"], m["rot"]["base"])
    k = rotate_halves((h @ w[p + ".k"].T).view(T, G, d), positions, m["rot"]["dims"], m["rot"]["base"])
    q = bf(rms_norm(q, None, eps) * w[p + ".temp"].to(F)[None, :, None], e16)  # the temperature rides on q
    k = bf(rms_norm(k, None, eps), e16)
    v = bf((h @ w[p + ".v"].T).view(T, G, dv), e16)
    visible = torch.tril(torch.ones(T, T, dtype=torch.bool))
    out = torch.zeros(T, H, dv, dtype=F)
    for i in range(H):
        j = i // (H // G)
        s = (q[:, i] @ k[:, j].T) * float(m["scale"])
        a = torch.softmax(s.masked_fill(~visible, -math.inf), dim=-1)
        if probe is not None:
            probe.setdefault("weights", []).append(a)
        out[:, i] = a @ v[:, j]
    gated = bf(out.reshape(T, H * dv) * torch.sigmoid(h @ w[p + ".g"].T), e16)
    return gated @ w[p + ".o"].T


# ---- lightning attention -------------------------------------------------------------------
def lightning_attention(h, w, p, m, eps, e16):
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = silu(bf(h @ w[p + ".q"].T, e16)).view(T, H, d)
    k = silu(bf(h @ w[p + ".k"].T, e16)).view(T, H, d)
    v = silu(bf(h @ w[p + ".v"].T, e16)).view(T, H, dv)
    out = torch.zeros(T, H, dv, dtype=F)
    for i in range(H):
        S = torch.zeros(d, dv, dtype=F)
        for t in range(T):
            S = float(m["decay"][i]) * S + torch.outer(k[t, i], v[t, i])
            out[t, i] = S.T @ q[t, i]
    joined = rms_norm(out.reshape(T, H * dv), w[p + ".norm"].to(F), eps)
    gated = bf(joined * torch.sigmoid(bf(h @ w[p + ".g"].T, e16)), e16)
    return gated @ w[p + ".o"].T


def parallel_mixer(h, w, p, m, eps, e16, probe=None):
    left = rms_norm(softmax_attention(h, w, p + ".left", m["left"], eps, e16, probe), w[p + ".left.out"].to(F), eps)
    right = rms_norm(lightning_attention(h, w, p + ".right", m["right"], eps, e16), w[p + ".right.out"].to(F), eps)
    return 0.5 * (left + right)


# ---- gated delta rule ----------------------------------------------------------------------
def short_convolution(x: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """x [T, channels], taps [channels, n]: y_t = sum_j taps[:, j] * x_(t - (n - 1 - j)), zeros before
    the start; then silu."""
    T, n = x.shape[0], taps.shape[1]
    padded = torch.cat([torch.zeros(n - 1, x.shape[1], dtype=F), x], dim=0)
    y = torch.zeros_like(x)
    for j in range(n):
        y = y + padded[j:j + T] * taps[:, j].to(F)[None, :]
    return silu(y)


def unit(x):
    return x / torch.sqrt((x * x).sum(dim=-1, keepdim=True) + UNIT_EPS)


def delta_decay(h, w, p):
    """The decay per token and head: exp(-exp(A_log) * softplus(W_a h + dt_bias))."""
    return torch.exp(-torch.exp(w[p + ".A_log"].to(F)) * softplus(h @ w[p + ".a"].T + w[p + ".dt_bias"].to(F)))


def delta_mixer(h, w, p, m, eps, e16, probe=None):
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = unit(short_convolution(h @ w[p + ".q"].T, w[p + ".q.conv"]).view(T, G, d)) * d ** -0.5
    k = unit(short_convolution(h @ w[p + ".k"].T, w[p + ".k.conv"]).view(T, G, d))
    v = short_convolution(h @ w[p + ".v"].T, w[p + ".v.conv"]).view(T, H, dv)
    beta = torch.sigmoid(h @ w[p + ".b"].T)
    g = delta_decay(h, w, p)
    if probe is not None:
        probe["decay"] = g
    out = torch.zeros(T, H, dv, dtype=F)
    for i in range(H):
        j = i // (H // G)
        S = torch.zeros(d, dv, dtype=F)
        for t in range(T):
            S = g[t, i] * S
            u = beta[t, i] * (v[t, i] - S.T @ k[t, j])
            S = S + torch.outer(k[t, j], u)
            out[t, i] = S.T @ q[t, j]
    normed = rms_norm(out, None, eps) * w[p + ".norm"].to(F)[None, None, :]
    gated = bf(normed * silu(h @ w[p + ".g"].T).view(T, H, dv), e16)
    return gated.reshape(T, H * dv) @ w[p + ".o"].T


# ---- feed-forward ---------------------------------------------------------------------------
def feed_forward(h, w, p, e16):
    return bf(gelu_erf(h @ w[p + ".up"].T), e16) @ w[p + ".down"].T


# ---- the model ---------------------------------------------------------------------------------
def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int], emulate_bf16: bool = False,
            probes: Optional[dict] = None, streams: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence.  ``probes[layer]`` receives what a test may want to look
    at (attention weights, decays); ``streams`` the stream after every layer."""
    w = {k: v.to(F) for k, v in w.items()}
    e16, eps = emulate_bf16, float(cfg["norm"]["eps"])
    x = w["embed"][torch.tensor(tokens, dtype=torch.long)]
    results = [x]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}"
        probe = probes.setdefault(i, {}) if probes is not None else None
        h = bf(rms_norm(x, w[p + ".norm1"], eps), e16)
        if layer["type"] == "parallel":
            mixed = parallel_mixer(h, w, p + ".mix", layer["mixer"], eps, e16, probe)
        else:
            mixed = delta_mixer(h, w, p + ".mix", layer["mixer"], eps, e16, probe)
        x = x + rms_norm(mixed, w[p + ".norm1b"], eps)
        if layer["mlp"] is not None:
            h = bf(rms_norm(x, w[p + ".norm2"], eps), e16)
            x = x + rms_norm(feed_forward(h, w, p + ".mlp", e16), w[p + ".norm2b"], eps)
        results.append(x)
        x = sum(w[p + ".dwa"][j] * results[j] for j in range(i + 2))
        if streams is not None:
            streams.append(x)
    return bf(rms_norm(x, w["final.norm"], eps), e16) @ w["head"].T


def greedy_generate(cfg, w, prompt: List[int], n: int) -> List[int]:
    seq, out = list(prompt), []
    for _ in range(n):
        t = int(torch.argmax(forward(cfg, w, seq)[-1]))
        out.append(t)
        seq.append(t)
    return out
