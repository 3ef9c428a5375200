"""Retention: linear attention with a fixed decay per head and a state of fixed size.

Per head, with q = W_q h and k = W_k h rotated by position (rotate-half over the
first ``rot dims``) and k scaled by dim^-1/2, v = W_v h:

    S_t = decay_h * S_{t-1} + k_t v_t^T        o_t = S_t^T q_t

No softmax, no denominator.  Each head's o is divided by its root mean square (no
weight), the heads are joined, multiplied by silu(W_g h) and projected by W_o into
the residual stream.  S [heads, dim, vdim] is float32, starts at zero and is the
layer's whole memory of a sequence: it lives in the cache's state area, one per
slot, so a later chunk or a single token goes on from what the tokens before left.

Single tokens update the state in registers.  Prompts go 32 tokens at a time (the
recurrence written as three small products per chunk, all float32); a long prompt is
cut into runs of 256 tokens that start from zero side by side, after which the states
between the runs are put together in order and every token receives what the tokens
before its run contribute.

Variants, each a parameter: ``activation`` "silu" passes q, k and v through silu before the
recurrence (lightning attention's form); ``key_scale`` replaces dim^-1/2 (1.0: no scale);
``norm`` "joined" divides a token's joined heads by ONE root mean square and multiplies by a
weight per value (names["norm"]) instead of a norm per head; ``gate`` "sigmoid" multiplies by
sigmoid(W_g h) instead of silu(W_g h).  A position encoding of zero ``dims`` rotates nothing.

params: hidden_size, heads, dim, vdim, decay (one per head), eps, position (a
``rope_frequencies`` PartSpec), activation, key_scale, norm, gate, names {q, k, v, g, o, norm}.
"""
from __future__ import annotations

from typing import Dict, Mapping

import torch

from ..cache import StateRequest, StateView
from ..csrc import ops
from ..weights.loader import WeightSpec
from .base import MIXERS, POSITIONS, Part
from .linear import ADD_F32, STORE, linear


class Retention(Part):
    def __init__(self, params, prefix, dtype, device):
        super().__init__(params, prefix, dtype, device)
        self.hidden = int(params["hidden_size"])
        self.heads = int(params["heads"])
        self.dim = int(params["dim"])
        self.vdim = int(params["vdim"])
        self.eps = float(params["eps"])
        self.decay_values = [float(d) for d in params["decay"]]
        self.names = params["names"]
        if len(self.decay_values) != self.heads:
            raise ValueError(f"retention: {len(self.decay_values)} decays for {self.heads} heads")
        if not 0 < self.dim <= 256:
            raise ValueError("retention kernels take key sizes up to 256")
        pos = params["position"]
        self.position = POSITIONS.build(pos.kind, pos.params, prefix, dtype, device)
        if not hasattr(self.position, "frequencies"):
            raise ValueError("retention rotates by a table of frequencies (rope_frequencies)")
        if self.position.dims > self.dim:
            raise ValueError(f"rotation over {self.position.dims} dimensions of heads of {self.dim}")
        self.activation = params.get("activation") or "none"
        self.key_scale = params.get("key_scale")
        self.norm = params.get("norm", "head")
        self.gate = params.get("gate", "silu")
        if self.activation not in ("none", "silu") or self.norm not in ("head", "joined") \
                or self.gate not in ("silu", "sigmoid"):
            raise ValueError(f"retention: activation {self.activation!r}, norm {self.norm!r} or gate "
                             f"{self.gate!r} is not known")
        self.w_in = self.w_o = self.norm_weight = None
        self._decay = None

    def _name(self, key: str) -> str:
        return self.tensor_name(self.names[key])

    def weight_specs(self) -> Dict[str, WeightSpec]:
        W, H = self.hidden, self.heads
        specs = {self._name("q"): WeightSpec((H * self.dim, W), "matrix", fan_in=W),
                 self._name("k"): WeightSpec((H * self.dim, W), "matrix", fan_in=W),
                 self._name("v"): WeightSpec((H * self.vdim, W), "matrix", fan_in=W),
                 self._name("g"): WeightSpec((H * self.vdim, W), "matrix", fan_in=W),
                 self._name("o"): WeightSpec((W, H * self.vdim), "matrix", fan_in=H * self.vdim)}
        if self.norm == "joined":
            specs[self._name("norm")] = WeightSpec((H * self.vdim,), "vector", init="ones")
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.w_in = torch.cat([tensors[self._name(p)] for p in ("q", "k", "v", "g")], 0).contiguous()
        self.w_o = tensors[self._name("o")]
        self._decay = torch.tensor(self.decay_values, dtype=torch.float32, device=self.w_o.device)
        if self.norm == "joined":
            self.norm_weight = tensors[self._name("norm")]

    def parameter_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w_in, self.w_o))

    def cache_request(self) -> StateRequest:
        return StateRequest((self.heads, self.dim, self.vdim), torch.float32)

    def check_shared_cache(self, view) -> None:
        raise ValueError("retention keeps a state of its own")

    def step_flops(self, counts, starts) -> float:
        H, W = self.heads, self.hidden
        return 2.0 * sum(counts) * (W * 2 * H * (self.dim + self.vdim) + H * self.vdim * W
                                    + 2 * H * self.dim * self.vdim)

    SEGMENTS, FIRST_SEGMENT = "retention/segments", "retention/first_segment"

    def step_tables(self, counts, starts, have=()):
        """Prompt steps with a sequence longer than a run: the runs of every sequence, worked
        side by side (the same list for every retention layer of the model)."""
        seg = ops.RETENTION_SEGMENT
        if not ops.retention_takes_segments(self.dim) or max(counts) <= seg or self.SEGMENTS in have:
            return {}
        segments, first = ops.retention_segments(counts, seg)
        return {self.SEGMENTS: segments, self.FIRST_SEGMENT: first}

    def forward(self, x: torch.Tensor, ctx, residual: torch.Tensor, cache: StateView) -> None:
        n = residual.shape[0]
        H, ws = self.heads, ctx.workspace
        qkvg = ws.get("retention_in", (n, 2 * H * (self.dim + self.vdim)), self.dtype)
        linear(x, self.w_in, None, qkvg, STORE, decode=ctx.decode)
        o_raw = ws.get("retention_o", (n, H * self.vdim), torch.float32)
        gated = ws.get("retention_gated", (n, H * self.vdim), self.dtype)
        segments = ctx.tables.get(self.SEGMENTS) if ops.retention_takes_segments(self.dim) else None
        seg_state = ws.get("retention_runs", (segments.shape[0], H, self.dim, self.vdim), torch.float32) \
            if segments is not None else None
        ops.retention(qkvg, self.position.frequencies(), self._decay, cache.state, ctx.token_pos,
                      ctx.token_seq, ctx.seq_slots, ctx.seq_first_row, ctx.seq_start, ctx.seq_count,
                      o_raw, gated, H, self.dim, self.vdim, self.position.dims, self.eps,
                      segments=segments, seq_first_segment=ctx.tables.get(self.FIRST_SEGMENT),
                      seg_state=seg_state, seg_len=ops.RETENTION_SEGMENT,
                      activation=self.activation == "silu",
                      key_scale=None if self.key_scale is None else float(self.key_scale),
                      norm_weight=self.norm_weight, gate=self.gate)
        linear(gated, self.w_o, None, residual, ADD_F32, ws, decode=ctx.decode)


MIXERS.register("retention", Retention)
