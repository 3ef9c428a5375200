"""Gated delta rule: a recurrent mixer whose state is corrected toward each new value.

With h the part's input, ``kv_heads`` heads of q and k (``dim`` values each) and ``heads``
heads of v (``vdim`` values; head i reads q/k head i // (heads / kv_heads)):

* q = W_q h, k = W_k h, v = W_v h; each passes a short causal convolution per channel over its
  last ``taps`` inputs (weights [channels, taps], the last column is the current token's, no bias,
  zeros before the sequence's start) and silu.
* Every q and k head is made a unit vector, x / sqrt(sum(x^2) + unit_eps); q is also
  multiplied by dim^-1/2.
* beta = sigmoid(W_b h), one per head; the decay g = exp(-exp(A_log) * softplus(W_a h + dt_bias)),
  one per head.
* Per head, in this order:  S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
  (the read-out sees the token's own write).
* Each head's o is divided by its root mean square (``eps``), multiplied by a weight per value
  that all heads share and by silu(W_g h), and W_o adds the result into the residual rows.

The recurrence is linear in the state: S_after = P S_before + S_run over a stretch of tokens, with P the
product of the tokens' g (I - beta k k^T).  A long prompt is cut into runs of 128 tokens that are walked side
by side from nothing (which also yields P, as the fate of an identity matrix under the same walk), put
together in order, and finished by one product a run.

S [heads, dim, vdim] and the convolutions' last taps - 1 inputs are float32 in the cache's state
area, one of each per slot, zero when a slot is taken, so a later portion of a prompt or a single
token goes on from what the tokens before left.  One product makes all six projections in
float32; everything after it (convolution, unit vectors, beta, the decay, the state, the norm and
the gate) is float32 in every dtype.

params: hidden_size, heads, kv_heads, dim, vdim, taps, eps, unit_eps, names {q, k, v, q_conv,
k_conv, v_conv, b, a, a_log, dt_bias, g, norm, o}.
"""
from __future__ import annotations

from typing import Dict, Mapping

import torch

from ..cache import StateRequest, StateView
from ..csrc import ops
from ..weights.loader import WeightSpec
from .base import MIXERS, Part
from .linear import ADD_F32, STORE_F32, linear


class GatedDeltaRule(Part):
    def __init__(self, params, prefix, dtype, device):
        super().__init__(params, prefix, dtype, device)
        self.hidden = int(params["hidden_size"])
        self.heads = int(params["heads"])
        self.kv_heads = int(params["kv_heads"])
        self.dim = int(params["dim"])
        self.vdim = int(params["vdim"])
        self.taps = int(params["taps"])
        self.eps = float(params["eps"])
        self.unit_eps = float(params.get("unit_eps", 1e-6))
        self.names = params["names"]
        if self.heads % self.kv_heads:
            raise ValueError(f"delta rule: heads={self.heads} is no multiple of kv_heads={self.kv_heads}")
        if not 0 < self.dim <= 256:
            raise ValueError("delta rule kernels take key sizes up to 256")
        if self.taps < 1:
            raise ValueError("delta rule: the convolution has at least one tap")
        self.channels = 2 * self.kv_heads * self.dim + self.heads * self.vdim
        self.w_in = self.w_o = self.conv = self.a_log = self.dt_bias = self.norm = None

    def _name(self, key: str) -> str:
        return self.tensor_name(self.names[key])

    def _projections(self):
        G, H = self.kv_heads, self.heads
        return (("q", G * self.dim), ("k", G * self.dim), ("v", H * self.vdim), ("g", H * self.vdim),
                ("b", H), ("a", H))

    def weight_specs(self) -> Dict[str, WeightSpec]:
        W, H, G = self.hidden, self.heads, self.kv_heads
        specs = {self._name(p): WeightSpec((rows, W), "matrix", fan_in=W) for p, rows in self._projections()}
        for p, rows in (("q_conv", G * self.dim), ("k_conv", G * self.dim), ("v_conv", H * self.vdim)):
            specs[self._name(p)] = WeightSpec((rows, self.taps), "vector", fan_in=self.taps)
        specs[self._name("a_log")] = WeightSpec((H,), "vector")
        specs[self._name("dt_bias")] = WeightSpec((H,), "vector")
        specs[self._name("norm")] = WeightSpec((self.vdim,), "vector", init="ones")
        specs[self._name("o")] = WeightSpec((W, H * self.vdim), "matrix", fan_in=H * self.vdim)
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.w_in = torch.cat([tensors[self._name(p)] for p, _ in self._projections()], 0).contiguous()
        self.conv = torch.cat([tensors[self._name(p)] for p in ("q_conv", "k_conv", "v_conv")], 0).contiguous()
        self.a_log = tensors[self._name("a_log")]
        self.dt_bias = tensors[self._name("dt_bias")]
        self.norm = tensors[self._name("norm")]
        self.w_o = tensors[self._name("o")]

    def parameter_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w_in, self.w_o))

    def cache_request(self) -> StateRequest:
        return StateRequest((self.heads, self.dim, self.vdim), torch.float32,
                            extra=(((max(self.taps - 1, 1), self.channels), torch.float32),))

    def check_shared_cache(self, view) -> None:
        raise ValueError("a delta rule mixer keeps a state of its own")

    def step_flops(self, counts, starts) -> float:
        W, H = self.hidden, self.heads
        return 2.0 * sum(counts) * (W * self.w_in.shape[0] + H * self.vdim * W + self.channels * self.taps
                                    + 3 * H * self.dim * self.vdim)

    SEGMENTS, FIRST_SEGMENT = "delta/segments", "delta/first_segment"

    def step_tables(self, counts, starts, have=()):
        """Prompt steps with a sequence longer than two runs: the runs of every sequence, worked side
        by side (the same list for every delta rule layer of the model)."""
        seg = ops.DELTA_SEGMENT
        if seg <= 0 or max(counts) <= 2 * seg or self.SEGMENTS in have:
            return {}
        segments, first = ops.scan_segments(counts, seg)
        return {self.SEGMENTS: segments, self.FIRST_SEGMENT: first}

    def forward(self, x: torch.Tensor, ctx, residual: torch.Tensor, cache: StateView) -> None:
        n = residual.shape[0]
        H, G, ws = self.heads, self.kv_heads, ctx.workspace
        rows = ws.get("delta_in", (n, self.w_in.shape[0]), torch.float32)
        linear(x, self.w_in, None, rows, STORE_F32, decode=ctx.decode)
        qkv = ws.get("delta_qkv", (n, self.channels), torch.float32)
        beta_g = ws.get("delta_beta_g", (n, 2 * H), torch.float32)
        ops.delta_prep(rows, self.conv, cache.extra[0], self.a_log, self.dt_bias, ctx.token_pos, ctx.token_seq,
                       ctx.seq_slots, ctx.seq_first_row, ctx.seq_count, qkv, beta_g, H, G, self.dim, self.vdim,
                       self.unit_eps, self.dim ** -0.5)
        o_raw = ws.get("delta_o", (n, H * self.vdim), torch.float32)
        segments = ctx.tables.get(self.SEGMENTS) if not ctx.decode else None
        runs = segments.shape[0] if segments is not None else 0
        ops.delta_scan(qkv, beta_g, cache.state, ctx.token_pos, ctx.token_seq, ctx.seq_slots, ctx.seq_first_row,
                       ctx.seq_count, o_raw, H, G, self.dim, self.vdim, segments=segments,
                       seq_first_segment=ctx.tables.get(self.FIRST_SEGMENT), seg_len=ops.DELTA_SEGMENT,
                       seg_state=ws.get("delta_run_state", (runs, H, self.dim, self.vdim), torch.float32) if runs else None,
                       seg_trans=ws.get("delta_run_trans", (runs, H, self.dim, self.dim), torch.float32) if runs else None,
                       q_run=ws.get("delta_run_q", (n, H, self.dim), torch.float32) if runs else None)
        gated = ws.get("delta_gated", (n, H * self.vdim), self.dtype)
        ops.delta_finish(o_raw, rows, self.channels, self.norm, ctx.token_pos, gated, H, self.vdim, self.eps)
        linear(gated, self.w_o, None, residual, ADD_F32, ws, decode=ctx.decode)


MIXERS.register("gated_delta_rule", GatedDeltaRule)
