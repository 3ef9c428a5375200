"""Differential attention: grouped-query attention over the paged cache in which every head
has TWO attention maps over the same values, and the head's output is their difference, normed.

With h the part's input, H query heads, G key/value heads (query head i reads key/value head
i // (H / G)), maps of ``dim`` values and values of ``vdim``:

* q = W_q h has H * 2 * dim rows and k = W_k h has G * 2 * dim rows, head by head [map 1 | map 2];
  v = W_v h has G * vdim rows; no biases.
* Every map of every q and k head is rotated by position over its own first ``dims`` values (the
  position encoding's frequencies and pairing; its ``magnitude`` multiplies every cosine and sine).
* Map c of head i: softmax over the visible keys of scale * q_c . k_c; a query at position p sees
  keys j <= p and, with ``window`` > 0, j > p - window.
* With a1, a2 the two maps' weighted sums of the same values and lambda = exp(lq1 . lk1) -
  exp(lq2 . lk2) + ``diff`` (four learned vectors of ``dim`` values: one number for the layer, worked
  out once at load): o = a1 - lambda * a2, then o / sqrt(mean(o^2) + eps) over the head's vdim values
  (no weight), times (1 - ``diff``).
* With ``gate`` the joined heads are multiplied value by value by sigmoid(W_g h) before W_o.

Keys after the rotation (both maps side by side: a cache row of 2 * dim values per key/value head)
and values live in the cache.  One projection makes q, k, v and the gate's logits in float32 (their
matrices are stacked at load); ``qkv_prep`` rotates, stores and takes the sigmoid; one attention
kernel serves prompts, later portions and single tokens alike (a warp holds the query heads that
share a key/value head, both maps of each); prompt steps in bfloat16 whose sizes the tensor-core
form takes run that (``attention_diff_mma``).  Scores, softmax, the difference, its norm and the
gate's sigmoid are float32 in every dtype.

params: hidden_size, heads, kv_heads, dim, vdim, scale, window, diff, gate, eps, position (a
``rope_frequencies`` PartSpec), names {q, k, v, o, gate, lq1, lk1, lq2, lk2}.
"""
from __future__ import annotations

import math
from typing import Dict, Mapping, Optional

import numpy as np
import torch

from ..cache import PAGE_SIZE, KVRequest, KVView
from ..csrc import ops
from ..weights.loader import WeightSpec
from .base import MIXERS, POSITIONS, Part
from .linear import ADD_F32, STORE_F32, linear


class DifferentialAttention(Part):
    MAPS = 2

    def __init__(self, params, prefix, dtype, device):
        super().__init__(params, prefix, dtype, device)
        self.hidden = int(params["hidden_size"])
        self.heads = int(params["heads"])
        self.kv_heads = int(params["kv_heads"])
        self.dim = int(params["dim"])
        self.vdim = int(params["vdim"])
        self.scale = float(params["scale"])
        self.window = int(params.get("window") or 0)
        self.diff = float(params["diff"])
        self.has_gate = bool(params.get("gate", True))
        self.eps = float(params.get("eps", 1e-6))
        self.names = params["names"]
        if self.heads % self.kv_heads:
            raise ValueError(f"heads={self.heads} is not a multiple of kv_heads={self.kv_heads}")
        if not 0 < self.dim <= 512 or not 0 < self.vdim <= 256:
            raise ValueError(f"differential attention takes maps of up to 512 values and values of up to 256; "
                             f"got {self.dim}, {self.vdim}")
        pos = params["position"]
        self.position = POSITIONS.build(pos.kind, pos.params, prefix, dtype, device)
        if not hasattr(self.position, "frequencies"):
            raise ValueError("differential attention rotates by a table of frequencies")
        self.pairing = getattr(self.position, "pairing", "half")
        if self.position.dims > self.dim:
            raise ValueError(f"rotation over {self.position.dims} values of maps of {self.dim}")
        self.gate_cols = self.heads * self.vdim if self.has_gate else 0
        self.w_in = self.w_o = None
        self.lam = 0.0

    def _name(self, key: str) -> str:
        return self.tensor_name(self.names[key])

    def _projections(self):
        rows = [("q", self.heads * self.MAPS * self.dim), ("k", self.kv_heads * self.MAPS * self.dim),
                ("v", self.kv_heads * self.vdim)]
        if self.has_gate:
            rows.append(("gate", self.gate_cols))
        return rows

    def weight_specs(self) -> Dict[str, WeightSpec]:
        W = self.hidden
        specs = {self._name(p): WeightSpec((rows, W), "matrix", fan_in=W) for p, rows in self._projections()}
        specs[self._name("o")] = WeightSpec((W, self.heads * self.vdim), "matrix", fan_in=self.heads * self.vdim)
        for key in ("lq1", "lk1", "lq2", "lk2"):
            specs[self._name(key)] = WeightSpec((self.dim,), "vector")
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.w_in = torch.cat([tensors[self._name(p)] for p, _ in self._projections()], 0).contiguous()
        self.w_o = tensors[self._name("o")]
        lq1, lk1, lq2, lk2 = (tensors[self._name(k)].detach().to("cpu", torch.float64) for k in ("lq1", "lk1", "lq2", "lk2"))
        self.lam = math.exp(float((lq1 * lk1).sum())) - math.exp(float((lq2 * lk2).sum())) + self.diff

    def parameter_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w_in, self.w_o))

    # -- cache ------------------------------------------------------------
    def cache_request(self) -> Optional[KVRequest]:
        # a key row holds both maps' keys
        return KVRequest(self.kv_heads, self.MAPS * self.dim, self.window, True, self.vdim)

    def check_shared_cache(self, view: KVView) -> None:
        raise ValueError("differential attention keeps a cache of its own")

    def step_flops(self, counts, starts) -> float:
        H, W = self.heads, self.hidden
        flops = 2.0 * sum(counts) * W * (self.w_in.shape[0] + H * self.vdim)
        for c, st in zip(counts, starts):
            keys = 0
            for q in range(c):
                p = st + q
                keys += min(p + 1, self.window) if self.window else p + 1
            flops += 2.0 * H * self.MAPS * (self.dim + self.vdim) * keys
        return flops

    # -- work lists ---------------------------------------------------------
    TILES_64 = "prefill_mma/tiles64"  # (sequence, first query) per 64 queries of the step

    def _mma_prompt(self) -> bool:
        return self.dtype == torch.bfloat16 and ops.attention_diff_mma_takes(self.dim, self.vdim, PAGE_SIZE)

    def step_tables(self, counts, starts, have=()):
        """The 64-query tiles of the tensor-core prompt kernel (the same list for every layer)."""
        if not self._mma_prompt() or self.TILES_64 in have:
            return {}
        tiles = [(i, q0) for i, c in enumerate(counts) for q0 in range(0, int(c), 64)]
        return {self.TILES_64: np.asarray(tiles, dtype=np.int32).reshape(-1, 2)}

    # -- run --------------------------------------------------------------
    def forward(self, x: torch.Tensor, ctx, residual: torch.Tensor, cache: KVView) -> None:
        n = residual.shape[0]
        H, G, ws = self.heads, self.kv_heads, ctx.workspace
        dk2 = self.MAPS * self.dim
        table = ctx.page_tables[cache.group]
        rows = ws.get("diff_attention_in", (n, self.w_in.shape[0]), torch.float32)
        linear(x, self.w_in, None, rows, STORE_F32, decode=ctx.decode)
        q = ws.get("diff_attention_q", (n, H * dk2), self.dtype)
        gate = ws.get("diff_attention_gate", (n, self.gate_cols), torch.float32) if self.has_gate else None
        ops.qkv_prep(rows, None, None, self.position.frequencies(), ctx.token_pos, ctx.token_seq, table, q,
                     cache.k, cache.v, gate, H, G, dk2, self.vdim, self.position.dims, self.eps,
                     pairing=self.pairing, maps=self.MAPS, magnitude=float(getattr(self.position, "magnitude", 1.0)))
        out = ws.get("diff_attention_out", (n, H * self.vdim), self.dtype)
        post = 1.0 - self.diff
        if not ctx.decode and self._mma_prompt() and self.TILES_64 in ctx.tables:
            ops.attention_diff_mma(q, cache.k, cache.v, ctx.tables[self.TILES_64], ctx.seq_first_row, ctx.seq_start,
                                   ctx.seq_count, table, gate, out, H, G, self.window, self.scale, self.lam, post,
                                   self.eps)
        else:
            splits = ctx.attention_splits(n * H)
            if self.window:  # a slice has at least 64 keys of the window
                splits = max(1, min(splits, -(-self.window // 64)))
            partial = ws.get("diff_attention_partial", (n * H * splits * (2 * self.vdim + 4),), torch.float32) \
                if splits > 1 else None
            ops.attention_diff(q, cache.k, cache.v, ctx.token_pos, ctx.token_seq, table, gate, out, H, G,
                               self.window, self.scale, self.lam, post, self.eps, splits, partial)
        linear(out, self.w_o, None, residual, ADD_F32, ws, decode=ctx.decode)


MIXERS.register("differential_attention", DifferentialAttention)
