"""RMSNorm: ``x * 1/sqrt(mean(x^2) + eps) * gain``, computed in 32-bit.

Reference: cpp/src/ops.cpp:272-292 (eps inside the root, added to the mean; gain last) and
nanoinfer/layers.py:21-38.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..registry import register_part
from .base import FoldedNorm, Norm, Runtime
from .spec import PartSpec, TensorSpec


class RMSNorm(Norm):
    """params: ``size`` (width of a row), ``eps``, optionally ``gain_offset`` (a gain stored around zero: the row is
    multiplied by ``gain_offset + gain``, summed once in 32-bit when the weights are loaded) and ``gain_scale`` (a constant
    factor on the normed row, e.g. a factor on the logits when this is the norm before the head: it is multiplied into the
    gain vector in 32-bit at load). tensors: ``gain [size]``."""

    graph_safe = True   # launches do not depend on which requests are in the batch

    @staticmethod
    def spec(size: int, eps: float, gain_name: str, gain_offset: float = 0.0, gain_scale: float = 1.0) -> PartSpec:
        params = {"size": size, "eps": eps}
        if gain_offset:
            params["gain_offset"] = float(gain_offset)
        if gain_scale != 1.0:
            params["gain_scale"] = float(gain_scale)
        return PartSpec("rmsnorm", params, {"gain": TensorSpec(gain_name, (size,), "bias" if gain_offset else "gain")})

    def __init__(self, spec: PartSpec, tensors: Dict[str, torch.Tensor], rt: Runtime):
        super().__init__(spec, tensors, rt)
        self.size = int(spec.params["size"])
        self.eps = float(spec.params["eps"])
        offset, factor = float(spec.params.get("gain_offset", 0.0)), float(spec.params.get("gain_scale", 1.0))
        gain = tensors["gain"].to(torch.float32) + offset if offset else tensors["gain"]
        self.gain = rt.vector32(gain.to(torch.float32) * factor if factor != 1.0 else gain)

    def forward(self, x32: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        n = x32.shape[0] if rows is None else rows.shape[0]
        out = torch.empty((n, self.size), dtype=self.rt.dtype, device=x32.device)
        self.ops.rmsnorm(x32, self.gain, self.eps, out, rows)
        return out

    def fold_into_projection(self, x32: torch.Tensor) -> Optional[FoldedNorm]:
        return FoldedNorm(x32, self.gain, self.eps, "rms")

    def add_normed(self, y32: torch.Tensor, x32: torch.Tensor, mult: float = 1.0, h_out: Optional[torch.Tensor] = None,
                   clear: bool = False, then: Optional["RMSNorm"] = None) -> None:
        """``x32 += mult * norm(y32)``: the norm stands on a branch's OUTPUT and its result goes into the stream. With
        ``h_out`` the new stream is also written there in that tensor's type (what the next branch reads); with ``clear``
        ``y32`` is left zeroed for the next branch to add into. With ``then`` (the norm BEFORE the next branch) ``h_out``
        gets that norm of the new stream instead. One pass over the rows."""
        if then is None:
            self.ops.rmsnorm_add(y32, self.gain, self.eps, float(mult), x32, h_out, clear)
        else:
            self.ops.rmsnorm_add(y32, self.gain, self.eps, float(mult), x32, h_out, clear, next_gain32=then.gain, next_eps=then.eps)

    def forward_with(self, other: "RMSNorm", x32: torch.Tensor):
        """``(self.forward(x32), other.forward(x32))`` with the rows read once: for blocks whose branches read the same
        stream through norms of their own. ``other`` must be an RMSNorm of the same size and eps."""
        if other.size != self.size or other.eps != self.eps:
            return self.forward(x32), other.forward(x32)
        a = torch.empty((x32.shape[0], self.size), dtype=self.rt.dtype, device=x32.device)
        b = torch.empty_like(a)
        self.ops.rmsnorm_pair(x32, self.gain, other.gain, self.eps, a, b)
        return a, b


register_part("rmsnorm", RMSNorm)

