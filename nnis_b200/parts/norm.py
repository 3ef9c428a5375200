"""RMSNorm with a per-channel weight (NNIS: crates/nnis-model/src/kernels.rs:15-48)."""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..csrc import ops
from ..weights.loader import WeightSpec
from .base import NORMS, Part


class RMSNorm(Part):
    """params: size, eps, name (tensor stem), and optionally ``offset``: the stored tensor w lies
    around zero and the multiplier is offset + w (added once at load, in float32, so every kernel
    that takes this norm's weight, alone or folded into a projection, serves it unchanged)."""
    kind = "rmsnorm"  # parts that can fold this norm into their first projection look for it

    def __init__(self, params, prefix, dtype, device):
        super().__init__(params, prefix, dtype, device)
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.offset = float(params.get("offset") or 0.0)
        self.name = self.tensor_name(params["name"])
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {self.name: WeightSpec((self.size,), "vector", init="normal" if self.offset else "ones")}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.weight = tensors[self.name]
        if self.offset:
            self.weight = (self.weight.to(torch.float32) + self.offset).contiguous()

    def parameter_bytes(self) -> int:
        return self.size * 4

    def forward(self, x: torch.Tensor, out: torch.Tensor,
                rows: Optional[torch.Tensor] = None) -> None:
        ops.rmsnorm(x, self.weight, self.eps, out, rows)


class GroupRMSNorm(RMSNorm):
    """RMS norm in groups: the row is cut into ``groups`` equal consecutive runs, each
    divided by its own sqrt(mean(run^2) + eps), and the whole multiplied by the weight.
    params: size, eps, groups, name.  No projection folds this norm into itself (its
    ``kind`` is not "rmsnorm"), so it always runs as a kernel of its own."""
    kind = "group_rmsnorm"

    def __init__(self, params, prefix, dtype, device):
        super().__init__(params, prefix, dtype, device)
        self.groups = int(params.get("groups", 1))
        if self.groups <= 0 or self.size % self.groups:
            raise ValueError(f"norm: {self.groups} groups do not divide {self.size}")

    def forward(self, x: torch.Tensor, out: torch.Tensor,
                rows: Optional[torch.Tensor] = None) -> None:
        ops.group_rmsnorm(x, self.weight, self.eps, self.groups, out, rows)


NORMS.register("rmsnorm", RMSNorm)
NORMS.register("group_rmsnorm", GroupRMSNorm)
