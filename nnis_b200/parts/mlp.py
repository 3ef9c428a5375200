"""Gated feed-forward: down( act(gate(x)) * up(x) ), added to the residual.

Gate and up are one projection (their matrices stacked along the output rows
at load) with float32 output; the activation kernel rounds once to the operand
dtype.  Steps 14-18 of NNIS's token pass
(crates/nnis-model/src/runtime.rs:1054-1093).

params: hidden_size, intermediate_size, activation, bias, names {gate, up, down}.
Activations: "silu" (silu(gate) * up, fused into the products' epilogues where those
exist) and "glu_clamp" with ``limit`` and ``alpha``: g' sigmoid(alpha g') (u' + 1) with
g' = min(gate, limit), u' = up clamped to [-limit, limit] (in the tcgen05 product's epilogue where
that product runs; a kernel of its own after a float32 product elsewhere).
"""
from __future__ import annotations

from typing import Dict, Mapping

import torch

from ..csrc import ops
from ..weights.loader import WeightSpec
from .base import FEED_FORWARDS, Part, begin_norm
from .linear import ADD_F32, STORE_F32, linear


class GatedMLP(Part):
    def __init__(self, params, prefix, dtype, device):
        super().__init__(params, prefix, dtype, device)
        self.hidden = int(params["hidden_size"])
        self.inter = int(params["intermediate_size"])
        self.bias = bool(params.get("bias", False))
        self.names = params["names"]
        self.activation = params.get("activation", "silu")
        if self.activation not in ("silu", "glu_clamp"):
            raise ValueError(f"gated_mlp: activation {params['activation']!r} has no kernel")
        self.limit = float(params.get("limit", 0.0))
        self.alpha = float(params.get("alpha", 1.0))
        if self.activation == "glu_clamp" and not self.limit > 0:
            raise ValueError("gated_mlp: glu_clamp needs a positive limit")
        self.w_gu = self.b_gu = self.w_down = self.b_down = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        H, I = self.hidden, self.inter
        specs = {self.tensor_name(self.names["gate"]): WeightSpec((I, H), "matrix", fan_in=H),
                 self.tensor_name(self.names["up"]): WeightSpec((I, H), "matrix", fan_in=H),
                 self.tensor_name(self.names["down"]): WeightSpec((H, I), "matrix", fan_in=I)}
        if self.bias:
            specs[self.tensor_name(self.names["gate"], "bias")] = WeightSpec((I,), "vector")
            specs[self.tensor_name(self.names["up"], "bias")] = WeightSpec((I,), "vector")
            specs[self.tensor_name(self.names["down"], "bias")] = WeightSpec((H,), "vector")
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        n = self.names
        self.w_gu = torch.cat([tensors[self.tensor_name(n["gate"])],
                               tensors[self.tensor_name(n["up"])]], 0).contiguous()
        self.w_down = tensors[self.tensor_name(n["down"])]
        if self.bias:
            self.b_gu = torch.cat([tensors[self.tensor_name(n["gate"], "bias")],
                                   tensors[self.tensor_name(n["up"], "bias")]], 0).contiguous()
            self.b_down = tensors[self.tensor_name(n["down"], "bias")]

    def parameter_bytes(self) -> int:
        return sum(t.numel() * t.element_size()
                   for t in (self.w_gu, self.w_down, self.b_gu, self.b_down) if t is not None)

    def step_flops(self, counts, starts) -> float:
        return 2.0 * 3 * self.hidden * self.inter * sum(counts)

    def _fused_gate_up(self, ctx, n: int, normed: bool = False) -> bool:
        """The fused bfloat16 decode kernel for gate/up (few rows, one token each)."""
        return (self.dtype == torch.bfloat16 and ctx.decode and self.activation == "silu"
                and ops.gemv_pays(n, 2 * self.inter, self.hidden, ops.EPI_GATED, self.device, normed))

    def _fused_down(self, ctx, n: int) -> bool:
        return (self.dtype == torch.bfloat16 and ctx.decode
                and ops.gemv_pays(n, self.hidden, self.inter, ops.EPI_ADD_F32, self.device))

    def fuses_norm(self, norm, ctx, n: int) -> bool:
        return getattr(norm, "kind", None) == "rmsnorm" and self._fused_gate_up(ctx, n, normed=True)

    def shares_norm(self, norm, ctx, n: int) -> bool:
        """Whether gate/up can end a norm that the projection before it began."""
        return (getattr(norm, "kind", None) == "rmsnorm" and self.dtype == torch.bfloat16 and ctx.decode
                and self.activation == "silu"
                and ops.gemv_shares_norm(n, 2 * self.inter, self.hidden, ops.EPI_GATED, self.device))

    def forward(self, x: torch.Tensor, ctx, residual: torch.Tensor) -> None:
        self._run(ctx, residual, x=x)

    def forward_shared(self, begun, residual: torch.Tensor, ctx) -> None:
        """The same on rows that the part before left weighted, with their sums of squares."""
        self._run(ctx, residual, begun=begun)

    def forward_normed(self, hidden: torch.Tensor, norm, ctx) -> None:
        """The same with the block's norm folded into the gate/up projection."""
        self._run(ctx, hidden, hidden=hidden, norm=norm)

    def _run(self, ctx, residual, x=None, hidden=None, norm=None, begun=None) -> None:
        n = residual.shape[0]
        ws = ctx.workspace
        act = ws.get("act", (n, self.inter), self.dtype)
        if begun is not None:
            ops.gemv_bf16(self.w_gu, self.b_gu, act, ops.EPI_GATED, x=begun.x, shares=begun.shares,
                          eps=begun.norm.eps, m=n)
        elif self._fused_gate_up(ctx, n, normed=hidden is not None):
            ops.gemv_bf16(self.w_gu, self.b_gu, act, ops.EPI_GATED, x=x, hidden=hidden,
                          norm_weight=norm.weight if norm is not None else None,
                          eps=norm.eps if norm is not None else 0.0, m=n)
        elif self.activation == "silu" and self.dtype == torch.bfloat16 \
                and ops.gemm_tc_takes(n, 2 * self.inter, self.hidden):
            # tensor-core product with the activation in its epilogue
            ops.gemm_tc(x, self.w_gu, self.b_gu, act, ops.GEMM_GATED)
        elif self.activation == "glu_clamp" and self.dtype == torch.bfloat16 \
                and ops.gemm_tc_takes(n, 2 * self.inter, self.hidden):
            # the same product with the clamped activation in its epilogue
            ops.gemm_tc_glu_clamp(x, self.w_gu, self.b_gu, act, self.limit, self.alpha)
        else:
            gate_up = ws.get("gate_up", (n, 2 * self.inter), torch.float32)
            linear(x, self.w_gu, self.b_gu, gate_up, STORE_F32, decode=ctx.decode)
            if self.activation == "silu":
                ops.silu_mul(gate_up, act)
            else:
                ops.glu_clamp(gate_up, act, self.limit, self.alpha)
        if self._fused_down(ctx, n):
            ops.gemv_bf16(self.w_down, self.b_down, residual, ops.EPI_ADD_F32, x=act,
                          emit=begin_norm(ctx, n, self.hidden))
        else:
            linear(act, self.w_down, self.b_down, residual, ADD_F32, ws)


class DenseMLP(Part):
    """Feed-forward without a gate: down(act(up(x))), added to the residual.  The activation is
    applied to the first product's float32 sums and rounded once to the operand dtype: in the
    product's own epilogue in bfloat16 (tensor-core and decode kernels), by a kernel of its own
    otherwise.

    params: hidden_size, intermediate_size, activation ("gelu": 0.5 z (1 + erf(z / sqrt 2));
    "gelu_tanh": 0.5 z (1 + tanh(sqrt(2 / pi) (z + 0.044715 z^3))); "relu2": max(z, 0)^2), names {up, down}."""
    ACTIVATIONS = {"gelu": ops.GELU_ERF, "gelu_tanh": ops.GELU_TANH, "relu2": ops.RELU2}
    FUSED = {ops.GELU_ERF: ops.GEMM_ACT_GELU_ERF, ops.GELU_TANH: ops.GEMM_ACT_GELU_TANH,
             ops.RELU2: ops.GEMM_ACT_RELU2}  # the products' codes

    def __init__(self, params, prefix, dtype, device):
        super().__init__(params, prefix, dtype, device)
        self.hidden = int(params["hidden_size"])
        self.inter = int(params["intermediate_size"])
        self.names = params["names"]
        self.activation = params.get("activation", "gelu")
        if self.activation not in self.ACTIVATIONS:
            raise ValueError(f"mlp: activation {self.activation!r} has no kernel ({sorted(self.ACTIVATIONS)})")
        self.w_up = self.w_down = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        H, I = self.hidden, self.inter
        return {self.tensor_name(self.names["up"]): WeightSpec((I, H), "matrix", fan_in=H),
                self.tensor_name(self.names["down"]): WeightSpec((H, I), "matrix", fan_in=I)}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.w_up = tensors[self.tensor_name(self.names["up"])]
        self.w_down = tensors[self.tensor_name(self.names["down"])]

    def parameter_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w_up, self.w_down))

    def step_flops(self, counts, starts) -> float:
        return 2.0 * 2 * self.hidden * self.inter * sum(counts)

    def forward(self, x: torch.Tensor, ctx, residual: torch.Tensor) -> None:
        n = residual.shape[0]
        ws = ctx.workspace
        kind = self.ACTIVATIONS[self.activation]
        act = ws.get("act", (n, self.inter), self.dtype)
        # bfloat16: the activation rides in the first product's epilogue (the float32 sums, rounded once)
        if self.dtype == torch.bfloat16 and ctx.decode and ops.gemv_pays(n, self.inter, self.hidden, ops.EPI_STORE,
                                                                         x.device):
            ops.gemv_bf16(self.w_up, None, act, ops.EPI_STORE, x=x, act=self.FUSED[kind])
        elif self.dtype == torch.bfloat16 and ops.gemm_tc_takes(n, self.inter, self.hidden):
            ops.gemm_tc_act(x, self.w_up, None, act, self.FUSED[kind])
        else:
            up = ws.get("mlp_up", (n, self.inter), torch.float32)
            linear(x, self.w_up, None, up, STORE_F32, decode=ctx.decode)
            ops.act_rows(up, act, kind)
        linear(act, self.w_down, None, residual, ADD_F32, ws, decode=ctx.decode)


FEED_FORWARDS.register("gated_mlp", GatedMLP)
FEED_FORWARDS.register("mlp", DenseMLP)
