"""Attention with a sink: grouped-query attention over the paged cache whose softmax
carries one more term, whose scores are capped, and whose heads are gated.

With h the part's input, H query heads of ``dim`` values, G key/value heads (query head
i reads key/value head i // (H / G)) with values of ``vdim``:

* q = W_q h, k = W_k h, v = W_v h, no biases.  With ``qk_norm`` (True) q and k are divided by
  their root mean square taken over the WHOLE projection (all heads at once) and
  multiplied by a weight per column, before the rotation.  With ``qk_norm == "head"`` every
  head of q and of k is divided by its own root mean square AFTER the rotation, without a weight.
* q and k are rotated by position over the first ``dims`` values of every head (the
  position encoding's frequencies; neighbouring pairs, or, for an encoding whose ``pairing`` is
  "half", value i with value i + dims / 2).
* With ``head_scale`` the scores of head i are also multiplied by a learned number per head
  (names["head_scale"]: a temperature); it is folded into q.
* score = cap * tanh(scale * q.k / cap) (``softcap`` 0: no cap); a query at position p sees
  keys j <= p of its own chunk (``chunk`` > 0: floor(j / chunk) == floor(p / chunk), chunks
  counted from position 0 of the sequence) and window (``window`` > 0: j > p - window).
* With ``sink`` the softmax's denominator also holds exp(sink_i), a learned number per
  head with no key and no value.
* With ``gate`` (True or "head") head i's output is multiplied by sigmoid(W_g h)_i before W_o; with
  ``gate == "value"`` W_g has a row per output value and the joined heads are multiplied value by
  value by sigmoid(W_g h).

Keys (after norm and rotation) and values live in the cache; with ``kv == "shared"`` the
part has no k/v projection, norm or cache of its own and reads another schedule entry's.
One projection makes q, k, v and the gate's logits in float32 (their matrices are
stacked at load); ``qkv_prep`` norms, rotates, stores and takes the sigmoid; the attention
kernel serves prompts, later portions and single tokens alike; prompt steps in bfloat16 with
key and value heads of 64 or 128 run a tensor-core form of it (``attention_sink_mma``).

params: hidden_size, heads, kv_heads, dim, vdim, scale, softcap, chunk, window, sink,
gate, qk_norm, head_scale, eps, position (a ``rope_frequencies`` PartSpec),
kv ("own" | "shared"), names {q, k, v, o, q_norm, k_norm, sink, gate, head_scale}.
"""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import numpy as np
import torch

from ..cache import PAGE_SIZE, KVRequest, KVView
from ..csrc import ops
from ..weights.loader import WeightSpec
from .base import MIXERS, POSITIONS, Part
from .linear import ADD_F32, STORE_F32, linear


class SinkAttention(Part):
    def __init__(self, params, prefix, dtype, device):
        super().__init__(params, prefix, dtype, device)
        self.hidden = int(params["hidden_size"])
        self.heads = int(params["heads"])
        self.kv_heads = int(params["kv_heads"])
        self.dim = int(params["dim"])
        self.vdim = int(params["vdim"])
        self.scale = float(params["scale"])
        self.softcap = float(params.get("softcap") or 0.0)
        self.chunk = int(params.get("chunk") or 0)
        self.window = int(params.get("window") or 0)
        self.has_sink = bool(params.get("sink", False))
        gate = params.get("gate", False)
        if gate not in (False, True, None, "head", "value"):
            raise ValueError(f"sink attention: gate {gate!r} is not known (head, value)")
        self.has_gate = bool(gate)
        self.gate_by_value = gate == "value"
        norm = params.get("qk_norm", False)
        if norm not in (False, True, None, "whole", "head"):
            raise ValueError(f"sink attention: qk_norm {norm!r} is not known (whole, head)")
        self.head_norm = norm == "head"
        self.qk_norm = bool(norm) and not self.head_norm
        self.has_head_scale = bool(params.get("head_scale", False))
        self.eps = float(params.get("eps", 1e-6))
        self.own_kv = params.get("kv", "own") == "own"
        self.names = params["names"]
        if self.heads % self.kv_heads:
            raise ValueError(f"heads={self.heads} is not a multiple of kv_heads={self.kv_heads}")
        if self.dim % 2 or not 0 < self.dim <= 1024 or not 0 < self.vdim <= 256:
            raise ValueError(f"sink attention takes even key sizes up to 1024 and value sizes up to 256; "
                             f"got {self.dim}, {self.vdim}")
        pos = params["position"]
        self.position = POSITIONS.build(pos.kind, pos.params, prefix, dtype, device)
        if not hasattr(self.position, "frequencies"):
            raise ValueError("sink attention rotates by a table of frequencies")
        self.pairing = getattr(self.position, "pairing", "neighbours")
        if self.qk_norm and self.pairing != "neighbours":
            raise ValueError("sink attention: the norm over whole projections goes with neighbouring pairs")
        if self.position.dims > self.dim:
            raise ValueError(f"rotation over {self.position.dims} values of heads of {self.dim}")
        self.stored_kv = self.kv_heads if self.own_kv else 0
        self.gate_cols = (self.heads * self.vdim if self.gate_by_value else self.heads) if self.has_gate else 0
        self.w_in = self.w_o = self.q_norm = self.k_norm = self.sink = self.head_scale = None

    def _name(self, key: str) -> str:
        return self.tensor_name(self.names[key])

    def _projections(self):
        rows = [("q", self.heads * self.dim)]
        if self.own_kv:
            rows += [("k", self.kv_heads * self.dim), ("v", self.kv_heads * self.vdim)]
        if self.has_gate:
            rows.append(("gate", self.gate_cols))
        return rows

    def weight_specs(self) -> Dict[str, WeightSpec]:
        W = self.hidden
        specs = {self._name(p): WeightSpec((rows, W), "matrix", fan_in=W) for p, rows in self._projections()}
        specs[self._name("o")] = WeightSpec((W, self.heads * self.vdim), "matrix", fan_in=self.heads * self.vdim)
        if self.qk_norm:
            specs[self._name("q_norm")] = WeightSpec((self.heads * self.dim,), "vector", init="ones")
            if self.own_kv:
                specs[self._name("k_norm")] = WeightSpec((self.kv_heads * self.dim,), "vector", init="ones")
        if self.has_sink:
            specs[self._name("sink")] = WeightSpec((self.heads,), "vector")
        if self.has_head_scale:
            specs[self._name("head_scale")] = WeightSpec((self.heads,), "vector", init="ones")
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.w_in = torch.cat([tensors[self._name(p)] for p, _ in self._projections()], 0).contiguous()
        self.w_o = tensors[self._name("o")]
        if self.qk_norm:
            self.q_norm = tensors[self._name("q_norm")]
            self.k_norm = tensors[self._name("k_norm")] if self.own_kv else None
        if self.has_sink:
            self.sink = tensors[self._name("sink")]
        if self.has_head_scale:
            self.head_scale = tensors[self._name("head_scale")]

    def parameter_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w_in, self.w_o))

    # -- cache ------------------------------------------------------------
    def cache_request(self) -> Optional[KVRequest]:
        # (a chunked mask frees no pages: a layer that shares this cache may have another mask)
        return KVRequest(self.kv_heads, self.dim, self.window, True, self.vdim) if self.own_kv else None

    def check_shared_cache(self, view: KVView) -> None:
        if not isinstance(view, KVView) or view.v is None \
                or tuple(view.k.shape[1:]) != (self.kv_heads, view.page_size, self.dim) \
                or view.v.shape[3] != self.vdim or (view.window and view.window != self.window):
            raise ValueError("the shared cache does not fit this attention's heads, sizes or window")

    def step_flops(self, counts, starts) -> float:
        H, W = self.heads, self.hidden
        flops = 2.0 * sum(counts) * W * (self.w_in.shape[0] + H * self.vdim)
        for c, st in zip(counts, starts):
            keys = 0
            for q in range(c):
                p = st + q
                lo = max(0, p - self.window + 1) if self.window else 0
                if self.chunk:
                    lo = max(lo, p // self.chunk * self.chunk)
                keys += p + 1 - lo
            flops += 2.0 * H * (self.dim + self.vdim) * keys
        return flops

    # -- work lists ---------------------------------------------------------
    TILES_64 = "prefill_mma/tiles64"  # (sequence, first query) per 64 queries of the step

    def _mma_prompt(self) -> bool:
        return self.dtype == torch.bfloat16 and ops.attention_sink_mma_takes(self.dim, self.vdim, PAGE_SIZE)

    def step_tables(self, counts, starts, have=()):
        """The 64-query tiles of the tensor-core prompt kernel (the same list for every layer)."""
        if not self._mma_prompt() or self.TILES_64 in have:
            return {}
        tiles = [(i, q0) for i, c in enumerate(counts) for q0 in range(0, int(c), 64)]
        return {self.TILES_64: np.asarray(tiles, dtype=np.int32).reshape(-1, 2)}

    # -- run --------------------------------------------------------------
    def forward(self, x: torch.Tensor, ctx, residual: torch.Tensor, cache: KVView) -> None:
        n = residual.shape[0]
        H, G, ws = self.heads, self.stored_kv, ctx.workspace
        table = ctx.page_tables[cache.group]
        rows = ws.get("sink_attention_in", (n, self.w_in.shape[0]), torch.float32)
        linear(x, self.w_in, None, rows, STORE_F32, decode=ctx.decode)
        q = ws.get("sink_attention_q", (n, H * self.dim), self.dtype)
        gate = ws.get("sink_attention_gate", (n, self.gate_cols), torch.float32) if self.has_gate else None
        ops.qkv_prep(rows, self.q_norm, self.k_norm, self.position.frequencies(), ctx.token_pos, ctx.token_seq,
                     table if G else None, q, cache.k if G else None, cache.v if G else None, gate, H, G,
                     self.dim, self.vdim, self.position.dims, self.eps, pairing=self.pairing,
                     head_norm=self.head_norm, q_scale=self.head_scale)
        out = ws.get("sink_attention_out", (n, H * self.vdim), self.dtype)
        if not ctx.decode and self._mma_prompt() and self.TILES_64 in ctx.tables:
            ops.attention_sink_mma(q, cache.k, cache.v, ctx.tables[self.TILES_64], ctx.seq_first_row, ctx.seq_start,
                                   ctx.seq_count, table, self.sink, gate, out, H, self.kv_heads, self.window,
                                   self.chunk, self.scale, self.softcap)
            linear(out, self.w_o, None, residual, ADD_F32, ws, decode=ctx.decode)
            return
        splits = ctx.attention_splits(n * H)
        partial = ws.get("attn_partial", (n * H * splits * (self.vdim + 2),), torch.float32) if splits > 1 else None
        ops.attention_sink(q, cache.k, cache.v, ctx.token_pos, ctx.token_seq, table, self.sink, gate, out, H,
                           self.kv_heads, self.window, self.chunk, self.scale, self.softcap, splits, partial)
        linear(out, self.w_o, None, residual, ADD_F32, ws, decode=ctx.decode)


MIXERS.register("sink_attention", SinkAttention)
