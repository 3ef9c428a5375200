"""Mixture of experts: every token runs ``top`` of ``experts`` small feed-forward
layers and, optionally, a shared one.

An expert is ``W_down act(W_up h)`` with act = relu squared, no biases.  The router's
logits ``z = W_r h + b`` are float32 (its matrix is kept in float32); the ``top``
largest choose the experts and a softmax over the chosen logits alone weighs them.
The shared expert has the same form, runs for every token and is multiplied by
``sigmoid(w_sg . h)``, one number per token; that number is an extra output row of
the shared expert's up-projection, and since it scales the whole output it is
applied to the activation, before the down-projection adds into the residual.

The experts' matrices are stacked ([experts, ff, width] and [experts, width, ff]) so
that one kernel serves all of them from the router's ids.  Steps of few tokens run a
product per (token, chosen expert); prompt steps in bfloat16 sort the pairs by expert and
run two grouped products on the tensor cores: the tcgen05 kernel of the dense projections
with one weight matrix per tile of 128 rows where an expert gets many rows, 64 x 64
mma.sync tiles where it gets few.

A second form (``activation`` "silu_gated"): the expert is W_down (silu(W_gate x) * (W_up x))
with x = score * h: the router's scores are sigmoid(z) (``scores`` "sigmoid"), used as they
are, and they multiply the expert's INPUT (``weight_on`` "input"); the output is the plain sum
of the chosen experts'.  Gate and up are stacked per expert with their rows interleaved ([experts,
2 ff, width]); the score multiplies their float32 sums, which is the product with score * h.
Prompt steps in bfloat16 sort the pairs by expert and run grouped products: on mma.sync tiles
(score and activation in the first product's epilogue) where an expert gets few rows, on the
tcgen05 kernel (float32 sums, then a row-wise kernel for score and activation) where it gets many.

A third form (``scores`` "softmax_all" with gated experts and ``weight_on`` "output"): the scores
are ONE softmax over all the router's outputs; the choice goes by score + a stored correction per
output (``names["correction"]``), group by group (``groups`` equal runs of neighbouring outputs, a
run's score its largest corrected score, only the ``keep`` best runs can be chosen), and the chosen
scores weigh the experts' OUTPUTS as they are, not renormalised.  The router's last ``identity``
outputs have no matrices: such an expert hands its input on, so the token's output takes weight *
h from it.  The shared expert of this form is a gated feed-forward of its own (``shared``: a
``gated_mlp`` PartSpec) that runs for every token.

params: hidden_size, experts, top, ff, shared_ff (0: no shared expert), activation
("relu2" | "silu_gated"), scores ("softmax" over the chosen logits | "sigmoid" | "softmax_all"),
weight_on ("output" | "input"), identity, groups, keep, shared (a PartSpec), names {router,
router_bias (optional), correction (optional), expert (a format with {e}), up, down, gate (gated
experts), shared_up, shared_down, shared_gate}.
"""
from __future__ import annotations

from typing import Dict, Mapping

import torch

from ..csrc import ops
from ..weights.loader import WeightSpec
from .base import FEED_FORWARDS, Part
from .mlp import GatedMLP
from .linear import ADD_F32, STORE_F32, linear


class MoEFeedForward(Part):
    GROUPED_FROM = 32  # tokens of a prompt step from which the pairs are sorted by expert
    TCGEN05_ROWS = 96  # (token, expert) pairs an expert on average from which runs are padded to 128 rows

    def __init__(self, params, prefix, dtype, device):
        super().__init__(params, prefix, dtype, device)
        self.hidden = int(params["hidden_size"])
        self.experts = int(params["experts"])
        self.top = int(params["top"])
        self.ff = int(params["ff"])
        self.shared_ff = int(params.get("shared_ff") or 0)
        self.names = params["names"]
        self.activation = params.get("activation", "relu2")
        self.scores = params.get("scores", "softmax")
        self.weight_on = params.get("weight_on", "output")
        self.identity = int(params.get("identity") or 0)
        self.groups = int(params.get("groups") or 1)
        self.keep = int(params.get("keep") or self.groups)
        self.by_choice = self.scores == "softmax_all"
        if (self.activation, self.scores, self.weight_on) not in (("relu2", "softmax", "output"),
                                                                  ("silu_gated", "sigmoid", "input"),
                                                                  ("silu_gated", "softmax_all", "output")):
            raise ValueError(f"moe: no kernel for activation {self.activation!r} with {self.scores!r} scores "
                             f"on the expert's {self.weight_on}")
        self.gated = self.activation == "silu_gated"
        if self.gated and self.shared_ff:
            raise ValueError("moe: the gated form's shared expert is a part of its own (shared)")
        self.outputs = self.experts + self.identity  # of the router
        if not self.by_choice and (self.identity or self.groups != 1 or params.get("shared") is not None):
            raise ValueError("moe: identity experts, groups and a shared part go with softmax_all scores")
        if not 0 < self.top <= self.outputs:
            raise ValueError(f"moe: top={self.top} of {self.outputs} experts")
        if self.groups <= 0 or self.outputs % self.groups or not 0 < self.keep <= self.groups \
                or self.top > self.keep * (self.outputs // self.groups):
            raise ValueError(f"moe: {self.groups} groups (keep {self.keep}) over {self.outputs} router outputs "
                             f"with top={self.top}")
        shared = params.get("shared")
        self.shared = GatedMLP(shared.params, prefix, dtype, device) if shared is not None else None
        self.correction = None
        self.w_router = self.b_router = self.w_up = self.w_down = None
        self.w_shared_up = self.w_shared_down = None

    def _expert(self, e: int, which: str) -> str:
        return self.tensor_name(self.names["expert"].format(e=e) + "." + self.names[which])

    def weight_specs(self) -> Dict[str, WeightSpec]:
        W = self.hidden
        # the router is held in float32 whatever the operand dtype ("vector": kept as float32)
        specs = {self.tensor_name(self.names["router"]): WeightSpec((self.outputs, W), "vector", fan_in=W)}
        if self.names.get("correction"):
            specs[self.tensor_name(self.names["correction"])] = WeightSpec((self.outputs,), "vector")
        if self.shared is not None:
            specs.update(self.shared.weight_specs())
        if self.names.get("router_bias"):
            specs[self.tensor_name(self.names["router_bias"])] = WeightSpec((self.experts,), "vector")
        for e in range(self.experts):
            if self.gated:
                specs[self._expert(e, "gate")] = WeightSpec((self.ff, W), "matrix", fan_in=W)
            specs[self._expert(e, "up")] = WeightSpec((self.ff, W), "matrix", fan_in=W)
            specs[self._expert(e, "down")] = WeightSpec((W, self.ff), "matrix", fan_in=self.ff)
        if self.shared_ff:
            specs[self.tensor_name(self.names["shared_up"])] = WeightSpec((self.shared_ff, W), "matrix", fan_in=W)
            specs[self.tensor_name(self.names["shared_down"])] = WeightSpec((W, self.shared_ff), "matrix",
                                                                           fan_in=self.shared_ff)
            specs[self.tensor_name(self.names["shared_gate"])] = WeightSpec((1, W), "matrix", fan_in=W)
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.w_router = tensors[self.tensor_name(self.names["router"])]
        self.b_router = tensors[self.tensor_name(self.names["router_bias"])] \
            if self.names.get("router_bias") else None
        self.correction = tensors[self.tensor_name(self.names["correction"])] \
            if self.names.get("correction") else None
        if self.shared is not None:
            self.shared.load(tensors)
        if self.gated:  # per expert, row 2f the gate's and row 2f + 1 the up-projection's of feature f
            self.w_up = torch.stack([torch.stack([tensors[self._expert(e, "gate")], tensors[self._expert(e, "up")]], 1)
                                     .reshape(2 * self.ff, self.hidden) for e in range(self.experts)]).contiguous()
        else:
            self.w_up = torch.stack([tensors[self._expert(e, "up")] for e in range(self.experts)]).contiguous()
        self.w_down = torch.stack([tensors[self._expert(e, "down")] for e in range(self.experts)]).contiguous()
        if self.shared_ff:
            up = tensors[self.tensor_name(self.names["shared_up"])]
            gate = tensors[self.tensor_name(self.names["shared_gate"])]
            # the gate's row after the up-projection's, then zero rows up to a multiple of eight
            # (the decode projection kernels take output rows in eights)
            pad = up.new_zeros((-(self.shared_ff + 1) % 8, self.hidden))
            self.w_shared_up = torch.cat([up, gate, pad], 0).contiguous()
            self.w_shared_down = tensors[self.tensor_name(self.names["shared_down"])]

    def parameter_bytes(self) -> int:
        """What a step of one token reads: the router, ``top`` experts, the shared one."""
        per_expert = (3 if self.gated else 2) * self.ff * self.hidden * self.w_up.element_size()
        shared = sum(t.numel() * t.element_size() for t in (self.w_shared_up, self.w_shared_down)
                     if t is not None)
        if self.shared is not None:
            shared += self.shared.parameter_bytes()
        return self.w_router.numel() * 4 + self.top * per_expert + shared

    def step_bytes(self, rows: int) -> int:
        """Bytes of weights that a step of ``rows`` tokens reads when the router spreads them
        evenly: the experts that at least one token chooses (experts * (1 - (1 - top / experts)
        ^ rows) of them in expectation), the router and the shared expert."""
        per_expert = (3 if self.gated else 2) * self.ff * self.hidden * self.w_up.element_size()
        chosen = self.experts * (1.0 - (1.0 - self.top / self.experts) ** max(1, rows))
        return int(self.parameter_bytes() + (chosen - self.top) * per_expert)

    def step_flops(self, counts, starts) -> float:
        W = self.hidden
        per_token = W * self.outputs + (3 if self.gated else 2) * self.top * self.ff * W \
            + self.shared_ff * (2 * W + 1) + W
        shared = self.shared.step_flops(counts, starts) if self.shared is not None else 0.0
        return 2.0 * sum(counts) * per_token + shared

    def forward(self, x: torch.Tensor, ctx, residual: torch.Tensor) -> None:
        n = residual.shape[0]
        ws = ctx.workspace
        ids = ws.get("moe_ids", (n, self.top), torch.int32)
        weights = ws.get("moe_weights", (n, self.top), torch.float32)
        if self.by_choice:
            self._forward_by_choice(x, ctx, residual, ids, weights)
            return
        ops.moe_route(x, self.w_router, self.b_router, ctx.token_pos, ids, weights, self.top,
                      sigmoid_scores=self.scores == "sigmoid")
        grouped_gated = self.gated and self.dtype == torch.bfloat16 and not ctx.decode and n >= self.GROUPED_FROM \
            and ops.MOE_GROUPED and ops.moe_grouped_takes(self.hidden, self.ff, self.experts)
        if grouped_gated and ops.TC_GEMM and n * self.top >= self.TCGEN05_ROWS * self.experts:
            # many tokens an expert: runs padded to 128 rows, both products on the tcgen05 kernel
            tiles = ops.moe_grouped_tc_tiles(n * self.top, self.experts)
            ops.moe_grouped_gated_tc(x, self.w_up, self.w_down, ids, weights,
                                     ws.get("moe_perm", (tiles * 128,), torch.int32),
                                     ws.get("moe_place", (n * self.top,), torch.int32),
                                     ws.get("moe_tile_expert", (tiles,), torch.int32),
                                     ws.get("moe_x_sorted", (tiles * 128, self.hidden), self.dtype),
                                     ws.get("moe_up_sorted", (tiles * 128, 2 * self.ff), torch.float32),
                                     ws.get("moe_act_sorted", (tiles * 128, self.ff), self.dtype),
                                     ws.get("moe_y_sorted", (tiles * 128, self.hidden), torch.float32), residual,
                                     self.top)
            return
        if grouped_gated:
            tiles = ops.moe_grouped_tiles(n * self.top, self.experts)
            ops.moe_grouped_gated(x, self.w_up, self.w_down, ids, weights,
                                  ws.get("moe_perm", (tiles * 64,), torch.int32),
                                  ws.get("moe_place", (n * self.top,), torch.int32),
                                  ws.get("moe_tile_expert", (tiles,), torch.int32),
                                  ws.get("moe_act_sorted", (tiles * 64, self.ff), self.dtype),
                                  ws.get("moe_y_sorted", (tiles * 64, self.hidden), torch.float32), residual, self.top)
            return
        if self.gated:
            act = ws.get("moe_act", (n, self.top, self.ff), self.dtype)
            ops.moe_experts_gated(x, self.w_up, self.w_down, ids, weights, ctx.token_pos, act, residual, self.top)
            return
        grouped = self.dtype == torch.bfloat16 and not ctx.decode and n >= self.GROUPED_FROM \
            and ops.moe_grouped_takes(self.hidden, self.ff, self.experts)
        if grouped and ops.TC_GEMM and n * self.top >= self.TCGEN05_ROWS * self.experts:
            # many tokens an expert: runs padded to 128 rows, both products on the tcgen05 kernel
            tiles = ops.moe_grouped_tc_tiles(n * self.top, self.experts)
            ops.moe_grouped_tc(x, self.w_up, self.w_down, ids, weights,
                               ws.get("moe_perm", (tiles * 128,), torch.int32),
                               ws.get("moe_place", (n * self.top,), torch.int32),
                               ws.get("moe_tile_expert", (tiles,), torch.int32),
                               ws.get("moe_x_sorted", (tiles * 128, self.hidden), self.dtype),
                               ws.get("moe_act_sorted", (tiles * 128, self.ff), self.dtype),
                               ws.get("moe_y_sorted", (tiles * 128, self.hidden), torch.float32), residual,
                               self.top)
        elif grouped:
            # pairs sorted by expert in runs padded to 64 rows, grouped products on mma.sync tiles
            tiles = ops.moe_grouped_tiles(n * self.top, self.experts)
            ops.moe_grouped(x, self.w_up, self.w_down, ids, weights,
                            ws.get("moe_perm", (tiles * 64,), torch.int32),
                            ws.get("moe_place", (n * self.top,), torch.int32),
                            ws.get("moe_tile_expert", (tiles,), torch.int32),
                            ws.get("moe_act_sorted", (tiles * 64, self.ff), self.dtype),
                            ws.get("moe_y_sorted", (tiles * 64, self.hidden), torch.float32), residual, self.top)
        else:
            act = ws.get("moe_act", (n, self.top, self.ff), self.dtype)
            ops.moe_experts(x, self.w_up, self.w_down, ids, weights, ctx.token_pos, act, residual, self.top)
        if self.shared_ff:
            up = ws.get("moe_shared_up", (n, self.w_shared_up.shape[0]), torch.float32)
            linear(x, self.w_shared_up, None, up, STORE_F32, decode=ctx.decode)
            shared_act = ws.get("moe_shared_act", (n, self.shared_ff), self.dtype)
            ops.relu2_gate(up, shared_act)
            linear(shared_act, self.w_shared_down, None, residual, ADD_F32, ws, decode=ctx.decode)


    def _forward_by_choice(self, x, ctx, residual, ids, weights) -> None:
        """The form whose scores are one softmax over all outputs (see the module's text)."""
        n = residual.shape[0]
        ws = ctx.workspace
        passed = ws.get("moe_pass_weight", (n,), torch.float32)
        ops.moe_route_choice(x, self.w_router, self.correction, ctx.token_pos, ids, weights, passed, self.experts,
                             self.top, self.groups, self.keep)
        pass_weight = passed if self.identity else None
        grouped = self.dtype == torch.bfloat16 and not ctx.decode and n >= self.GROUPED_FROM and ops.MOE_GROUPED \
            and ops.moe_grouped_takes(self.hidden, self.ff, self.experts)
        if grouped and ops.TC_GEMM and n * self.top >= self.TCGEN05_ROWS * self.experts:
            # many tokens an expert: runs padded to 128 rows, both products on the tcgen05 kernel
            tiles = ops.moe_grouped_tc_tiles(n * self.top, self.experts)
            ops.moe_grouped_gated_tc(x, self.w_up, self.w_down, ids, weights,
                                     ws.get("moe_perm", (tiles * 128,), torch.int32),
                                     ws.get("moe_place", (n * self.top,), torch.int32),
                                     ws.get("moe_tile_expert", (tiles,), torch.int32),
                                     ws.get("moe_x_sorted", (tiles * 128, self.hidden), self.dtype),
                                     ws.get("moe_up_sorted", (tiles * 128, 2 * self.ff), torch.float32),
                                     ws.get("moe_act_sorted", (tiles * 128, self.ff), self.dtype),
                                     ws.get("moe_y_sorted", (tiles * 128, self.hidden), torch.float32), residual,
                                     self.top, on_output=True, pass_weight=pass_weight)
        elif grouped:
            tiles = ops.moe_grouped_tiles(n * self.top, self.experts)
            ops.moe_grouped_gated(x, self.w_up, self.w_down, ids, weights,
                                  ws.get("moe_perm", (tiles * 64,), torch.int32),
                                  ws.get("moe_place", (n * self.top,), torch.int32),
                                  ws.get("moe_tile_expert", (tiles,), torch.int32),
                                  ws.get("moe_act_sorted", (tiles * 64, self.ff), self.dtype),
                                  ws.get("moe_y_sorted", (tiles * 64, self.hidden), torch.float32), residual,
                                  self.top, on_output=True, pass_weight=pass_weight)
        else:
            act = ws.get("moe_act", (n, self.top, self.ff), self.dtype)
            ops.moe_experts_gated_out(x, self.w_up, self.w_down, ids, weights, pass_weight, ctx.token_pos, act,
                                      residual, self.top)
        if self.shared is not None:
            self.shared.forward(x, ctx, residual)


FEED_FORWARDS.register("moe", MoEFeedForward)
