"""Arrangements of the parts of a layer.

``Block`` is what the model needs of an arrangement: its parts (for weights and
work lists), what it wants of the cache, and ``forward``.  An arrangement reads
its parts from ``LayerSpec.parts`` by the roles it knows, so one with other or more
sub-layers (a post-norm, one norm for parallel branches, a third sub-layer) is a
class registered in ``BLOCKS``, not a change here.

``parallel``: with n = norm(h), h += mixer(n) + ffn(n); roles norm, mixer, ffn; with the role
ffn_norm the feed-forward reads a norm of its own of the same h: h += mixer(norm(h)) + ffn(ffn_norm(h)).

``branch_norm``: h += m * norm1(mixer(h)); h += m * norm2(ffn(h)): the sub-layers read the
stream itself and the norm stands on their OUTPUT; roles mixer, mixer_norm, and optionally
ffn, ffn_norm; ``LayerSpec.params["residual_mult"]`` is m.

``sandwich``: h += norm1b(mixer(norm1(h))); h += norm2b(ffn(norm2(h))): a norm before and a norm
after every sub-layer; roles mixer_norm, mixer, mixer_post_norm and, optionally, ffn_norm, ffn,
ffn_post_norm.  With ``LayerSpec.params["depth_mix"]`` the block's result is kept beside the
results of the blocks before it, and what goes on is a learned weighted sum of them all.

``prenorm``: h += mixer(norm1(h)); h += ffn(norm2(h)) - the order of NNIS's
decoder (crates/nnis-model/src/runtime.rs:946-1097); roles mixer_norm, mixer,
ffn_norm, ffn.  In decode steps a norm may be shared out between the projections on
either side of it (``parts.base.SharedNorm``): the block tells the part before a norm
which norm follows, and hands what that part left to the part after it.
"""
from __future__ import annotations

import dataclasses
import os
from typing import Dict, Mapping, Sequence

import torch

from ..csrc import ops

from ..weights.loader import WeightSpec
from .base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, Part


class Block:
    """Base of the arrangements: subclasses build their parts in ``__init__`` (with
    ``build``), list them in ``parts()`` and run them in ``forward``.  ``mixer`` is
    the part that owns the layer's cache, if any."""
    mixer = None

    def __init__(self, layer_spec, dtype: torch.dtype, device: torch.device):
        self.spec = layer_spec
        self.dtype = dtype
        self.device = device

    def build(self, registry, role: str) -> Part:
        part = self.spec.part(role)
        return registry.build(part.kind, part.params, self.spec.prefix, self.dtype, self.device)

    def parts(self) -> Sequence[Part]:
        raise NotImplementedError

    def forward(self, hidden: torch.Tensor, ctx, cache) -> None:
        raise NotImplementedError

    # -- what the model asks of every arrangement --------------------------------
    def cache_request(self):
        return self.mixer.cache_request() if self.mixer is not None else None

    def check_shared_cache(self, view) -> None:
        self.mixer.check_shared_cache(view)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        specs: Dict[str, WeightSpec] = {}
        for part in self.parts():
            specs.update(part.weight_specs())
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        for part in self.parts():
            part.load(tensors)

    def parameter_bytes(self) -> int:
        return sum(part.parameter_bytes() for part in self.parts())

    def step_flops(self, counts, starts) -> float:
        return sum(part.step_flops(counts, starts) for part in self.parts())

    def step_tables(self, counts, starts, have=()) -> Dict[str, object]:
        tables: Dict[str, object] = {}
        for part in self.parts():
            wants = getattr(part, "step_tables", None)
            if wants is not None:
                for name, arr in wants(counts, starts, tuple(have) + tuple(tables)).items():
                    tables.setdefault(name, arr)
        return tables


class PreNormBlock(Block):
    def __init__(self, layer_spec, dtype: torch.dtype, device: torch.device):
        super().__init__(layer_spec, dtype, device)
        self.mixer_norm = self.build(NORMS, "mixer_norm")
        self.mixer = self.build(MIXERS, "mixer")
        self.ffn_norm = self.build(NORMS, "ffn_norm")
        self.ffn = self.build(FEED_FORWARDS, "ffn")

    def parts(self):
        return (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn)

    @staticmethod
    def _shares(part, norm, ctx, n: int) -> bool:
        return bool(getattr(part, "shares_norm", None)) and part.shares_norm(norm, ctx, n)

    def first_shared_norm(self, ctx, n: int):
        """The norm this block applies first, if its mixer will take it begun by the part
        that runs before this block (asked by the model before that part runs)."""
        return self.mixer_norm if self._shares(self.mixer, self.mixer_norm, ctx, n) else None

    def forward(self, hidden: torch.Tensor, ctx, cache) -> None:
        n, width = hidden.shape
        normed = ctx.workspace.get("normed", (n, width), self.dtype)
        begun = ctx.take_shared_norm(self.mixer_norm)
        # the mixer's last projection may begin the norm before the feed-forward
        ctx.emit_for = self.ffn_norm if self._shares(self.ffn, self.ffn_norm, ctx, n) else None
        if begun is not None:
            self.mixer.forward_shared(begun, hidden, ctx, cache)
        # a part may fold the norm before it into its first kernel (decode steps)
        elif getattr(self.mixer, "fuses_norm", None) and self.mixer.fuses_norm(self.mixer_norm, ctx, n):
            self.mixer.forward_normed(hidden, self.mixer_norm, ctx, cache)
        else:
            self.mixer_norm.forward(hidden, normed)
            self.mixer.forward(normed, ctx, hidden, cache)
        begun = ctx.take_shared_norm(self.ffn_norm)
        # ... and the feed-forward's the first norm of the block that runs next
        ctx.emit_for = ctx.next_norm
        if begun is not None:
            self.ffn.forward_shared(begun, hidden, ctx)
        elif getattr(self.ffn, "fuses_norm", None) and self.ffn.fuses_norm(self.ffn_norm, ctx, n):
            self.ffn.forward_normed(hidden, self.ffn_norm, ctx)
        else:
            self.ffn_norm.forward(hidden, normed)
            self.ffn.forward(normed, ctx, hidden)
        ctx.emit_for = None


class ParallelBlock(Block):
    """One norm, two branches that both read it: with h = norm(x),
    x += mixer(h) + ffn(h).  Roles: norm, mixer and, optionally, ffn (a layer
    without a feed-forward has none).  Both branches add into the float32 residual;
    the feed-forward reads the normed rows, which the mixer leaves as they are.  With the optional
    role ffn_norm each branch has a norm of its own, x += mixer(norm(x)) + ffn(ffn_norm(x)), both of the
    SAME x: both are taken before either branch adds into the stream (two RMS norms in one pass).

    In steps of single tokens the branches run side by side: such a step is a chain of
    short kernels that wait for one another, and the two branches meet only in the residual
    sum.  The feed-forward then runs on a stream of its own, with buffers of its own, into a
    zeroed float32 branch buffer that one kernel adds to the residual when both are done
    (inside a captured step the fork and the join are edges of the graph).
    ``NNIS_PARALLEL_BRANCHES=0`` runs them one after the other."""
    SIDE_BY_SIDE = os.environ.get("NNIS_PARALLEL_BRANCHES", "1") != "0"

    def __init__(self, layer_spec, dtype: torch.dtype, device: torch.device):
        super().__init__(layer_spec, dtype, device)
        self.norm = self.build(NORMS, "norm")
        self.mixer = self.build(MIXERS, "mixer")
        self.ffn = self.build(FEED_FORWARDS, "ffn") if "ffn" in layer_spec.parts else None
        self.ffn_norm = self.build(NORMS, "ffn_norm") if self.ffn is not None and "ffn_norm" in layer_spec.parts \
            else None

    def parts(self):
        return tuple(p for p in (self.norm, self.mixer, self.ffn_norm, self.ffn) if p is not None)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        specs = super().weight_specs()
        # (a layer without a feed-forward has no use for its norm; a folder may still hold it)
        for stem in self.spec.params.get("tolerated", ()):
            specs.setdefault(f"{self.spec.prefix}.{stem}", WeightSpec((-1,), "unused"))
        return specs

    def forward(self, hidden: torch.Tensor, ctx, cache) -> None:
        n, width = hidden.shape
        ws = ctx.workspace
        # (a buffer of its own: parts may use "normed" for their own rows)
        normed = ws.get("normed_parallel", (n, width), self.dtype)
        ctx.emit_for = None  # the next norm reads both branches' sum: no part may begin it
        if self.ffn_norm is not None:
            # the feed-forward's rows are made before the mixer adds into the stream they are taken from
            normed_ffn = ws.get("normed_parallel_ffn", (n, width), self.dtype)
            a, b = self.norm, self.ffn_norm
            if getattr(a, "kind", None) == getattr(b, "kind", None) == "rmsnorm" and a.eps == b.eps:
                ops.rmsnorm_pair(hidden, a.weight, b.weight, a.eps, normed, normed_ffn)
            else:
                a.forward(hidden, normed)
                b.forward(hidden, normed_ffn)
            mixer_in, normed = normed, normed_ffn
        else:
            self.norm.forward(hidden, normed)
            mixer_in = normed
        if self.ffn is None:
            self.mixer.forward(mixer_in, ctx, hidden, cache)
        elif self.SIDE_BY_SIDE and ctx.decode and width % 4 == 0:
            main = torch.cuda.current_stream()
            side = ws.stream("feed_forward")
            fork, join = torch.cuda.Event(), torch.cuda.Event()
            fork.record(main)
            side.wait_event(fork)
            branch_ctx = dataclasses.replace(ctx, workspace=ws.child("feed_forward"))
            branch = branch_ctx.workspace.get("branch_sum", (n, width), torch.float32)
            with torch.cuda.stream(side):
                branch.zero_()
                self.ffn.forward(normed, branch_ctx, branch)
                join.record(side)
            self.mixer.forward(mixer_in, ctx, hidden, cache)
            main.wait_event(join)
            ops.add_rows(hidden, branch)
        else:
            self.mixer.forward(mixer_in, ctx, hidden, cache)
            self.ffn.forward(normed, ctx, hidden)


class BranchNormBlock(Block):
    """A norm on each sub-layer's output and a multiplier: with m = ``residual_mult``,
    x += m * norm1(mixer(x)), then x += m * norm2(ffn(x)).  The sub-layers read x itself (in
    the operand dtype); each adds its output up in a zeroed float32 branch buffer, as it would
    into the residual stream, and one kernel norms that buffer, scales it, adds it to the
    stream and leaves the buffer zero again.  In bfloat16 the same kernel leaves the new rows of the stream in bfloat16 for the
    sub-layer that reads them next (``ctx.hidden_copy`` across blocks).  Roles: mixer,
    mixer_norm and, optionally, ffn with ffn_norm.  The norms are RMS norms (``rmsnorm``)."""

    def __init__(self, layer_spec, dtype: torch.dtype, device: torch.device):
        super().__init__(layer_spec, dtype, device)
        self.mult = float(layer_spec.params.get("residual_mult", 1.0))
        self.mixer = self.build(MIXERS, "mixer")
        self.mixer_norm = self.build(NORMS, "mixer_norm")
        self.ffn = self.build(FEED_FORWARDS, "ffn") if "ffn" in layer_spec.parts else None
        self.ffn_norm = self.build(NORMS, "ffn_norm") if self.ffn is not None else None
        for norm in (self.mixer_norm, self.ffn_norm):
            if norm is not None and getattr(norm, "kind", None) != "rmsnorm":
                raise ValueError("branch_norm: the norm on a sub-layer's output is an rmsnorm")

    def parts(self):
        return tuple(p for p in (self.mixer, self.mixer_norm, self.ffn, self.ffn_norm) if p is not None)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        specs = super().weight_specs()
        # a layer without a feed-forward has no use for the second norm; a folder may still hold it
        for stem in self.spec.params.get("tolerated", ()):
            specs.setdefault(f"{self.spec.prefix}.{stem}", WeightSpec((-1,), "unused"))
        return specs

    def _close(self, branch, norm, hidden, ctx, n, width):
        """hidden += m * norm(branch); returns what the next sub-layer reads."""
        if self.dtype == torch.float32:
            ops.norm_scale_add(branch, norm.weight, norm.eps, self.mult, hidden, clear=True)
            return hidden
        # (two buffers in turn: the sub-layer that just ran may still be the reader of one)
        ctx.copy_turn = 1 - getattr(ctx, "copy_turn", 0)
        x = ctx.workspace.get(f"stream_copy{ctx.copy_turn}", (n, width), self.dtype)
        ops.norm_scale_add(branch, norm.weight, norm.eps, self.mult, hidden, x, clear=True)
        return x

    def forward(self, hidden: torch.Tensor, ctx, cache) -> None:
        n, width = hidden.shape
        ws = ctx.workspace
        ctx.emit_for = None  # no part may begin a norm here: none reads the stream
        x, ctx.hidden_copy = ctx.hidden_copy, None
        if self.dtype == torch.float32:
            x = hidden
        elif x is None:
            x = ws.get("stream_copy_first", (n, width), self.dtype)
            ops.cast_rows(hidden, x)
        # the kernel that norms the branch buffer leaves it zero for the next sub-layer; steps of
        # single tokens (a chain of short launches, mostly inside a captured graph) rely on that,
        # prompt steps fill it anyway (a step that was abandoned half-way may have left anything)
        branch = ws.kept_zero("branch_out", (n, width), torch.float32)
        if not ctx.decode:
            branch.zero_()
        self.mixer.forward(x, ctx, branch, cache)
        x = self._close(branch, self.mixer_norm, hidden, ctx, n, width)
        if self.ffn is not None:
            self.ffn.forward(x, ctx, branch)
            x = self._close(branch, self.ffn_norm, hidden, ctx, n, width)
        ctx.hidden_copy = x if self.dtype != torch.float32 else None


class SandwichBlock(Block):
    """A norm before and a norm after each sub-layer: x += norm1b(mixer(norm1(x))), then
    x += norm2b(ffn(norm2(x))).  The sub-layer adds its output up in a zeroed float32 branch buffer,
    as it would into the residual stream, and one kernel norms that buffer and adds it to the stream
    (leaving the buffer zero again).  Roles: mixer_norm, mixer, mixer_post_norm and, optionally, ffn_norm,
    ffn, ffn_post_norm; the norms after the sub-layers are RMS norms (``rmsnorm``).

    ``LayerSpec.params["depth_mix"]`` = {"name": tensor stem, "terms": t, "most": m} turns on the depth-weighted
    average: with X_0 what the first such block of a run was given and X_t-1 this block's result, the
    stream that goes on is sum_j w[j] X_j over the t results so far (w: the block's tensor of t
    weights).  The results live in the step's workspace, one float32 copy of the stream each (room for m,
    the most terms of any block of the model, so that the buffer never moves inside a run); the first
    block of a run (``terms == 2``) keeps its own input as X_0."""

    def __init__(self, layer_spec, dtype: torch.dtype, device: torch.device):
        super().__init__(layer_spec, dtype, device)
        self.mixer_norm = self.build(NORMS, "mixer_norm")
        self.mixer = self.build(MIXERS, "mixer")
        self.mixer_post = self.build(NORMS, "mixer_post_norm")
        self.ffn = self.build(FEED_FORWARDS, "ffn") if "ffn" in layer_spec.parts else None
        self.ffn_norm = self.build(NORMS, "ffn_norm") if self.ffn is not None else None
        self.ffn_post = self.build(NORMS, "ffn_post_norm") if self.ffn is not None else None
        for norm in (self.mixer_post, self.ffn_post):
            if norm is not None and getattr(norm, "kind", None) != "rmsnorm":
                raise ValueError("sandwich: the norm on a sub-layer's output is an rmsnorm")
        mix = layer_spec.params.get("depth_mix")
        self.mix_terms = int(mix["terms"]) if mix else 0
        self.mix_most = max(int(mix.get("most", 0)), self.mix_terms) if mix else 0
        self.mix_name = f"{layer_spec.prefix}.{mix['name']}" if mix else None
        if mix and self.mix_terms < 2:
            raise ValueError("sandwich: a depth mix has at least two terms (the input and this block's result)")
        self.mix_weights = None

    def parts(self):
        return tuple(p for p in (self.mixer_norm, self.mixer, self.mixer_post, self.ffn_norm, self.ffn,
                                 self.ffn_post) if p is not None)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        specs = super().weight_specs()
        if self.mix_name:
            specs[self.mix_name] = WeightSpec((self.mix_terms,), "vector", init="ones")
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        super().load(tensors)
        if self.mix_name:
            self.mix_weights = tensors[self.mix_name]

    def _close(self, branch, post, hidden, history, follower, normed) -> bool:
        """The kernel that ends a sub-layer: the norm of its output into the stream, the depth mix
        if ``history`` is given, and the norm ``follower`` of the rows the stream then holds, if it is
        an RMS norm.  True if ``normed`` was written."""
        fused = follower is not None and getattr(follower, "kind", None) == "rmsnorm"
        ops.sandwich_close(branch, post.weight, post.eps, hidden, history, self.mix_weights if history is not None else None,
                           self.mix_terms if history is not None else 0,
                           follower.weight if fused else None, follower.eps if fused else 0.0, normed if fused else None)
        return fused

    def forward(self, hidden: torch.Tensor, ctx, cache) -> None:
        n, width = hidden.shape
        ws = ctx.workspace
        ctx.emit_for = None  # a norm of the branch follows every sub-layer: none may begin the next one
        history = None
        if self.mix_terms:
            history = ws.get("depth_history", (self.mix_most, n, width), torch.float32)
            if self.mix_terms == 2:
                ops.copy_async(history[0], hidden)
        normed = ws.get("normed_sandwich", (n, width), self.dtype)
        branch = ws.kept_zero("branch_out", (n, width), torch.float32)
        if not ctx.decode:
            branch.zero_()
        begun, ctx.normed_rows = ctx.normed_rows, None
        if begun is None or begun[0] is not self.mixer_norm or begun[1].data_ptr() != normed.data_ptr():
            self.mixer_norm.forward(hidden, normed)
        self.mixer.forward(normed, ctx, branch, cache)
        # the block after this one, if it is of this arrangement, finds its first norm done
        after = ctx.next_block.mixer_norm if isinstance(ctx.next_block, SandwichBlock) else None
        if self.ffn is None:
            if self._close(branch, self.mixer_post, hidden, history, after, normed):
                ctx.normed_rows = (after, normed)
            return
        if not self._close(branch, self.mixer_post, hidden, None, self.ffn_norm, normed):
            self.ffn_norm.forward(hidden, normed)
        self.ffn.forward(normed, ctx, branch)
        if self._close(branch, self.ffn_post, hidden, history, after, normed):
            ctx.normed_rows = (after, normed)


BLOCKS.register("prenorm", PreNormBlock)
BLOCKS.register("sandwich", SandwichBlock)
BLOCKS.register("branch_norm", BranchNormBlock)
BLOCKS.register("parallel", ParallelBlock)
