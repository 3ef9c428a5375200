"""Two mixers side by side: both read the same input, each output gets a norm of its own over
the model width, and the part's result is a weighted sum of the two normed outputs.

    out = weight * (rms(left(h)) * w_left + rms(right(h)) * w_right)

Each member is any registered mixer, built from its own ``PartSpec``; it adds its output up in a
zeroed float32 buffer exactly as it would into the residual stream, and one kernel norms that
buffer, scales it and adds it to the rows this part was given (the same kernel that closes a
sub-layer of the ``branch_norm`` arrangement).  The members keep caches of their own: the part
asks the cache for both requests at once and hands each member its view.

params: hidden_size, eps, weight (0.5: half the sum), left, right (``PartSpec``s of mixers),
names {left_norm, right_norm}.
"""
from __future__ import annotations

from typing import Dict, Mapping

import torch

from ..csrc import ops
from ..weights.loader import WeightSpec
from .base import MIXERS, Part


class MixerPair(Part):
    def __init__(self, params, prefix, dtype, device):
        super().__init__(params, prefix, dtype, device)
        self.hidden = int(params["hidden_size"])
        self.eps = float(params["eps"])
        self.weight = float(params.get("weight", 0.5))
        self.names = params["names"]
        self.members = tuple(MIXERS.build(params[side].kind, params[side].params, prefix, dtype, device)
                             for side in ("left", "right"))
        self.device_only = all(getattr(m, "device_only", True) for m in self.members)
        self.norm_weights = [None, None]

    def _norm_names(self):
        return (self.tensor_name(self.names["left_norm"]), self.tensor_name(self.names["right_norm"]))

    def weight_specs(self) -> Dict[str, WeightSpec]:
        specs: Dict[str, WeightSpec] = {}
        for m in self.members:
            specs.update(m.weight_specs())
        for name in self._norm_names():
            specs[name] = WeightSpec((self.hidden,), "vector", init="ones")
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        for m in self.members:
            m.load(tensors)
        self.norm_weights = [tensors[name] for name in self._norm_names()]

    def parameter_bytes(self) -> int:
        return sum(m.parameter_bytes() for m in self.members) + 2 * self.hidden * 4

    def step_flops(self, counts, starts) -> float:
        return sum(m.step_flops(counts, starts) for m in self.members)

    def step_tables(self, counts, starts, have=()):
        tables: Dict[str, object] = {}
        for m in self.members:
            for name, arr in m.step_tables(counts, starts, tuple(have) + tuple(tables)).items():
                tables.setdefault(name, arr)
        return tables

    def cache_request(self):
        return tuple(m.cache_request() for m in self.members)

    def check_shared_cache(self, view) -> None:
        raise ValueError("a pair of mixers keeps caches of its own")

    def forward(self, x: torch.Tensor, ctx, residual: torch.Tensor, cache) -> None:
        n, width = residual.shape
        # (the kernel that closes a member leaves its buffer zero again; prompt steps fill it anyway:
        # a step that was abandoned half-way may have left anything)
        branch = ctx.workspace.kept_zero("pair_member_out", (n, width), torch.float32)
        emit, ctx.emit_for = ctx.emit_for, None  # a norm of this part's own follows each member
        for member, view, w in zip(self.members, cache, self.norm_weights):
            if not ctx.decode:
                branch.zero_()
            member.forward(x, ctx, branch, view)
            ops.norm_scale_add(branch, w, self.eps, self.weight, residual, clear=True)
        ctx.emit_for = emit


MIXERS.register("mixer_pair", MixerPair)
