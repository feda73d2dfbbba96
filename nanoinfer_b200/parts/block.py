"""Arrangements: the order in which the parts of one layer run.

``parallel``: ``x += mixer(norm_a(x)) + feed_forward(norm_b(x))``, both of the same x, optionally followed by a mix
with the step's earlier streams.

``output_norm``: ``x += mult * norm(mixer(x)); x += mult * norm(feed_forward(x))``: the norms stand on the branches'
outputs, the branches read the stream as it is.

``sandwich_norm``: ``x += norm_b(mixer(norm_a(x))); x += norm_d(feed_forward(norm_c(x)))``: a norm before and after each
sublayer.

``pre_norm``: ``x += mixer(norm(x)); x += feed_forward(norm(x))`` with a norm of its own before each
(cpp/src/model.cpp:364-400, nanoinfer/layers.py:328-339). The residual stream ``x`` is 32-bit and
both sums are made in 32-bit inside the projections that produce the addends.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..registry import register_arrangement
from .base import PENDING_STREAM_OP, LayerCache, StepContext, normed_input


class PreNormBlock:
    """parts: ``mixer_norm``, ``mixer``, ``ffn_norm``, ``ffn``."""

    part_names = ("mixer_norm", "mixer", "ffn_norm", "ffn")

    def __init__(self, parts: Dict[str, object]):
        self.mixer_norm, self.mixer = parts["mixer_norm"], parts["mixer"]
        self.ffn_norm, self.ffn = parts["ffn_norm"], parts["ffn"]

    def forward(self, x32: torch.Tensor, ctx: StepContext, cache: LayerCache) -> None:
        # A part that says so takes its norm unresolved and lets its first projection apply it.
        self.mixer.forward(normed_input(self.mixer_norm, self.mixer, x32), x32, ctx, cache)
        self.ffn.forward(normed_input(self.ffn_norm, self.ffn, x32), x32, ctx)


class ParallelBlock:
    """``x <- x + mixer(norm_a(x)) + feed_forward(norm_b(x))``: both branches read the same x. parts: ``mixer_norm``,
    ``mixer``; optionally ``ffn`` (a layer without a feed-forward) with ``ffn_norm`` (without it the feed-forward reads
    the mixer's norm: one norm for both branches), and ``depth`` (a part with
    ``begin(x32, ctx)`` before and ``forward(x32, ctx)`` after the layer: what goes on is a mix of this and earlier
    results). Both norms are computed before either branch adds to the stream."""

    resolves_pending = True     # it looks for work left pending on the stream itself (and may fold it into its norms)

    def __init__(self, parts: Dict[str, object]):
        self.mixer_norm, self.mixer = parts["mixer_norm"], parts["mixer"]
        self.ffn_norm, self.ffn = parts.get("ffn_norm"), parts.get("ffn")
        self.depth = parts.get("depth")
        if self.ffn is None and self.ffn_norm is not None:
            raise ValueError("a parallel block without a feed-forward has no norm for one")
        self.part_names = tuple(n for n in ("mixer_norm", "mixer", "ffn_norm", "ffn", "depth") if parts.get(n) is not None)

    def forward(self, x32: torch.Tensor, ctx: StepContext, cache: LayerCache) -> None:
        shared = self.ffn is not None and self.ffn_norm is None      # both branches read the mixer's norm
        together = getattr(self.mixer_norm, "forward_with", None) if type(self.mixer_norm) is type(self.ffn_norm) else None
        pending = ctx.scratch.pop(PENDING_STREAM_OP, None)      # what the layer before left to do on the stream
        fused = pending is not None and together is not None and hasattr(pending, "run_with_norms") \
            and self.mixer_norm.size == self.ffn_norm.size and self.mixer_norm.eps == self.ffn_norm.eps
        if pending is not None and not fused:
            pending.run(x32, ctx)
        if fused:                       # the pending sum and both norms in one pass over the rows
            h_mixer, h_ffn = pending.run_with_norms(x32, ctx, self.mixer_norm, self.ffn_norm)
        elif together is not None:      # two norms of one kind: the stream is read once
            h_mixer, h_ffn = together(self.ffn_norm, x32)
        else:
            h_mixer = self.mixer_norm.forward(x32)
            h_ffn = h_mixer if shared else (self.ffn_norm.forward(x32) if self.ffn is not None else None)
        if self.depth is not None:
            self.depth.begin(x32, ctx)
        self.mixer.forward(h_mixer, x32, ctx, cache)
        if self.ffn is not None:
            self.ffn.forward(h_ffn, x32, ctx)
        if self.depth is not None:
            self.depth.forward(x32, ctx)


class OutputNormBlock:
    """``x <- x + mult * norm_a(mixer(x))``, then ``x <- x + mult * norm_b(feed_forward(x))``: the branches read the stream
    itself (in the compute dtype), and each norm stands on its branch's output. parts: ``mixer``, ``mixer_norm`` and
    optionally ``ffn`` with ``ffn_norm``; ``mult``: the factor on what a branch adds. The norms offer
    ``add_normed(y32, x32, mult, h_out, clear)``.

    A branch adds its result into a zeroed 32-bit buffer as it would into the stream (sums over K splits and over experts
    included); the norm's kernel reads that buffer, adds to the stream, writes the stream's rounding for the next branch
    and leaves the buffer zeroed: one pass per branch. The buffer and the rounded stream live in the step's scratch, so
    that consecutive layers of this arrangement share them (the layer before has left both ready)."""

    part_names = ("mixer", "mixer_norm", "ffn", "ffn_norm")
    _SCRATCH = "output_norm.buffers"

    def __init__(self, parts: Dict[str, object], mult: float = 1.0):
        self.mixer, self.mixer_norm = parts["mixer"], parts["mixer_norm"]
        self.ffn, self.ffn_norm = parts.get("ffn"), parts.get("ffn_norm")
        if (self.ffn is None) != (self.ffn_norm is None):
            raise ValueError("a feed-forward and the norm on its output come together")
        self.mult = float(mult)
        self.part_names = tuple(n for n in OutputNormBlock.part_names if parts.get(n) is not None)

    def forward(self, x32: torch.Tensor, ctx: StepContext, cache: LayerCache) -> None:
        rt = self.mixer.rt
        same = rt.dtype == torch.float32        # the branches then read the stream itself
        held = ctx.scratch.get(self._SCRATCH)
        if held is None or held[0] is not x32:
            y32 = torch.zeros_like(x32)
            h = x32 if same else torch.empty(x32.shape, dtype=rt.dtype, device=x32.device)
            if not same:
                rt.ops.unary(x32, h, "copy")
            held = (x32, y32, h)
            ctx.scratch[self._SCRATCH] = held
        _, y32, h = held
        self.mixer.forward(h, y32, ctx, cache)
        self.mixer_norm.add_normed(y32, x32, self.mult, None if same else h, clear=True)
        if self.ffn is not None:
            self.ffn.forward(h, y32, ctx)
            self.ffn_norm.add_normed(y32, x32, self.mult, None if same else h, clear=True)


class SandwichNormBlock:
    """``x <- x + mixer_out_norm(mixer(mixer_norm(x)))``, then ``x <- x + ffn_out_norm(feed_forward(ffn_norm(x)))``: every
    sublayer reads a norm of the stream and its output is normed again before it is added. parts: ``mixer_norm``,
    ``mixer``, ``mixer_out_norm`` and optionally ``ffn_norm``, ``ffn``, ``ffn_out_norm`` (all three or none).

    A sublayer adds its result into a zeroed 32-bit buffer as it would into the stream (sums over K splits and over experts
    included). ONE kernel per sublayer then reads that buffer, norms it, adds it to the 32-bit stream, leaves the buffer
    zeroed and writes the NEXT sublayer's input norm of the new stream (``add_normed(..., then=)``): the stream is read
    once per sublayer. Consecutive layers of this arrangement hand the buffer and the next layer's normed input on through
    the step's scratch, so only the model's first layer runs a norm kernel of its own."""

    part_names = ("mixer_norm", "mixer", "mixer_out_norm", "ffn_norm", "ffn", "ffn_out_norm")
    _SCRATCH = "sandwich_norm.buffers"

    def __init__(self, parts: Dict[str, object]):
        self.mixer_norm, self.mixer, self.mixer_out_norm = parts["mixer_norm"], parts["mixer"], parts["mixer_out_norm"]
        self.ffn_norm, self.ffn, self.ffn_out_norm = parts.get("ffn_norm"), parts.get("ffn"), parts.get("ffn_out_norm")
        if len({self.ffn_norm is None, self.ffn is None, self.ffn_out_norm is None}) != 1:
            raise ValueError("a feed-forward comes with the norm before it and the norm on its output")
        self.part_names = tuple(n for n in SandwichNormBlock.part_names if parts.get(n) is not None)
        self.next_block = None      # the block that runs next in the schedule, when it is of this kind (set by link())

    def link(self, following) -> None:
        """Told once after construction which block follows in the schedule (None at the end): when it is of this kind, the
        last norm kernel of this block also writes that block's first input."""
        self.next_block = following if isinstance(following, SandwichNormBlock) else None

    def forward(self, x32: torch.Tensor, ctx: StepContext, cache: LayerCache) -> None:
        rt = self.mixer.rt
        held = ctx.scratch.pop(self._SCRATCH, None)
        if held is not None and held[0] is x32 and held[3] is self:
            _, y32, h = held[:3]
        else:
            y32 = torch.zeros_like(x32)
            h = self.mixer_norm.forward(x32)
        self.mixer.forward(h, y32, ctx, cache)
        nxt = self.next_block
        if self.ffn is not None:
            self.mixer_out_norm.add_normed(y32, x32, 1.0, h, clear=True, then=self.ffn_norm)
            self.ffn.forward(h, y32, ctx)
            last = self.ffn_out_norm
        else:
            last = self.mixer_out_norm
        if nxt is not None:
            last.add_normed(y32, x32, 1.0, h, clear=True, then=nxt.mixer_norm)
            ctx.scratch[self._SCRATCH] = (x32, y32, h, nxt)
        else:
            last.add_normed(y32, x32, 1.0, None, clear=False)


register_arrangement("pre_norm", PreNormBlock)
register_arrangement("sandwich_norm", SandwichNormBlock)
register_arrangement("output_norm", OutputNormBlock)
register_arrangement("parallel", ParallelBlock)
