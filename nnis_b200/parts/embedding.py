"""Token embedding and the linear head that ends the model.

The head reads the embedding's table when the two are tied; there is no second
copy (NNIS keeps a transposed copy: crates/nnis-model/src/safetensors_loader.rs:755-786).
Logits are float32 in every dtype (crates/nnis-model/src/runtime.rs:1109-1116).
"""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..csrc import ops
from ..weights.loader import WeightSpec
from .base import EMBEDDINGS, HEADS, NORMS, Part
from .linear import STORE_F32, linear


class TokenEmbedding(Part):
    """params: vocab_size, hidden_size, name."""

    def __init__(self, params, prefix, dtype, device):
        super().__init__(params, prefix, dtype, device)
        self.vocab = int(params["vocab_size"])
        self.width = int(params["hidden_size"])
        self.name = self.tensor_name(params["name"])
        self.table: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {self.name: WeightSpec((self.vocab, self.width), "matrix")}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.table = tensors[self.name]

    def forward(self, tokens: torch.Tensor, hidden: torch.Tensor, status: torch.Tensor) -> None:
        ops.embed(self.table, tokens, hidden, status)


class NormedTokenEmbedding(TokenEmbedding):
    """The same followed by a norm of the embedded rows (in place, float32).
    params: vocab_size, hidden_size, name, norm (a PartSpec of ``NORMS``)."""

    def __init__(self, params, prefix, dtype, device):
        super().__init__(params, prefix, dtype, device)
        norm = params["norm"]
        self.norm = NORMS.build(norm.kind, norm.params, prefix, dtype, device)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {**super().weight_specs(), **self.norm.weight_specs()}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        super().load(tensors)
        self.norm.load(tensors)

    def forward(self, tokens: torch.Tensor, hidden: torch.Tensor, status: torch.Tensor) -> None:
        ops.embed(self.table, tokens, hidden, status)
        self.norm.forward(hidden, hidden)


class PairHashEmbedding(NormedTokenEmbedding):
    """x = table[token] * scale + pair[row], then the norm: ``pair`` is a second table of
    ``buckets`` + 1 rows, and a token's row is (token before * mul_prev + token * mul_cur) mod
    buckets, the last row for a sequence's first token.  The token before is part of a sequence's
    state: the embedding asks the cache for one int32 per slot, which holds the last token that
    a step brought, so that a later portion or a single token finds it there.
    params: vocab_size, hidden_size, name, norm, scale (1.0), and optionally pair {name, buckets,
    mul_prev, mul_cur} (without it: the scaled embedding and the norm, no state)."""

    def __init__(self, params, prefix, dtype, device):
        super().__init__(params, prefix, dtype, device)
        self.scale = float(params.get("scale", 1.0))
        pair = params.get("pair")
        self.pair_name = self.tensor_name(pair["name"]) if pair else None
        self.buckets = int(pair["buckets"]) if pair else 0
        self.mul_prev = int(pair["mul_prev"]) if pair else 0
        self.mul_cur = int(pair["mul_cur"]) if pair else 0
        if pair and self.buckets <= 0:
            raise ValueError("pair embedding: buckets must be positive")
        self.pair_table: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        specs = super().weight_specs()
        if self.pair_name:
            specs[self.pair_name] = WeightSpec((self.buckets + 1, self.width), "matrix")
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        super().load(tensors)
        if self.pair_name:
            self.pair_table = tensors[self.pair_name]

    def cache_request(self):
        from ..cache import StateRequest
        return StateRequest((1,), torch.int32) if self.pair_name else None

    def forward(self, tokens: torch.Tensor, hidden: torch.Tensor, status: torch.Tensor) -> None:
        raise RuntimeError("this embedding needs the step's context and its state: forward_step")

    def forward_step(self, ctx, hidden: torch.Tensor, status: torch.Tensor, cache) -> None:
        """The step's rows from ``ctx.tokens``; ``cache``: the view of the state asked for (None
        without a pair table)."""
        ops.embed_pair(self.table, self.pair_table, ctx.tokens, ctx.token_pos, ctx.token_seq, ctx.seq_slots,
                       None if ctx.decode else ctx.seq_count, cache.state if cache is not None else None, hidden,
                       status, self.scale, self.buckets, self.mul_prev, self.mul_cur)
        self.norm.forward(hidden, hidden)


class LinearHead(Part):
    """params: vocab_size, hidden_size, name, tied_to (tensor stem or None), softcap
    (0: none; else logits <- softcap * tanh(logits / softcap), which changes no greedy pick),
    scale (1: none; the logits are multiplied by it, before a cap; a greedy pick is fused only
    with a positive one)."""

    def __init__(self, params, prefix, dtype, device):
        super().__init__(params, prefix, dtype, device)
        self.scale = float(params.get("scale", 1.0))
        self.softcap = float(params.get("softcap") or 0.0)
        self.vocab = int(params["vocab_size"])
        self.width = int(params["hidden_size"])
        tied = params.get("tied_to")
        self.tied = tied is not None
        self.name = self.tensor_name(tied if self.tied else params["name"])
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {self.name: WeightSpec((self.vocab, self.width), "matrix",
                                      fan_in=0 if self.tied else self.width)}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.weight = tensors[self.name]

    def parameter_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def step_flops(self, counts, starts, wanted: int = 0) -> float:
        return 2.0 * self.vocab * self.width * wanted

    def forward(self, x: torch.Tensor, logits: torch.Tensor) -> None:
        # (few rows: the decode projection kernel where it takes the shape)
        linear(x, self.weight, None, logits, STORE_F32, decode=True)
        if self.scale != 1.0:
            ops.scale_rows(logits, self.scale)
        if self.softcap:
            ops.softcap_rows(logits, self.softcap)

    def fuses_norm(self, norm, rows: int) -> bool:
        return (getattr(norm, "kind", None) == "rmsnorm" and self.dtype == torch.bfloat16 and self.scale > 0
                and rows <= ops.GEMV_HEAD_ROWS
                and ops.gemv_takes(rows, self.vocab, self.width, ops.EPI_STORE_F32, self.device, True))

    def forward_pick(self, hidden: torch.Tensor, norm, rows: torch.Tensor, picks: torch.Tensor,
                     scratch: torch.Tensor, logits: Optional[torch.Tensor] = None,
                     next_tokens: Optional[torch.Tensor] = None,
                     next_pos: Optional[torch.Tensor] = None) -> None:
        """Final norm, head and greedy pick in one kernel; optionally the logits
        too, and the decode state moved on (tokens = picks, positions + 1)."""
        ops.gemv_bf16(self.weight, None, picks, ops.EPI_ARGMAX, hidden=hidden,
                      norm_weight=norm.weight, eps=norm.eps, rows=rows, m=picks.numel(),
                      logits=logits, scratch=scratch, next_tokens=next_tokens, next_pos=next_pos)
        if self.scale != 1.0 and logits is not None:
            ops.scale_rows(logits, self.scale)
        if self.softcap and logits is not None:
            ops.softcap_rows(logits, self.softcap)

    def pick_scratch_ints(self, rows: int) -> int:
        return ops.argmax_scratch_ints(rows, self.vocab, self.width, self.device)

    def forward_normed(self, hidden: torch.Tensor, norm, rows: torch.Tensor,
                       logits: torch.Tensor) -> None:
        """Final norm of the wanted rows folded into the head (few rows)."""
        ops.gemv_bf16(self.weight, None, logits, ops.EPI_STORE_F32, hidden=hidden,
                      norm_weight=norm.weight, eps=norm.eps, rows=rows, m=logits.shape[0])
        if self.scale != 1.0:
            ops.scale_rows(logits, self.scale)
        if self.softcap:
            ops.softcap_rows(logits, self.softcap)


EMBEDDINGS.register("token_embedding", TokenEmbedding)
EMBEDDINGS.register("normed_token_embedding", NormedTokenEmbedding)
EMBEDDINGS.register("pair_hash_embedding", PairHashEmbedding)
HEADS.register("linear_head", LinearHead)
