"""SwiGLU feed-forward: ``down( silu(gate(h)) * up(h) )``, no biases, added to the residual stream.

``silu(g) = g / (1 + exp(-g))`` in 32-bit. Reference: cpp/src/model.cpp:217-223,
cpp/src/ops.cpp:86-100, nanoinfer/layers.py:243-258.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..registry import register_part
from .base import FeedForward, Runtime, StepContext, as_tensor
from .spec import PartSpec, TensorSpec


class SwiGLU(FeedForward):
    """params: ``hidden``, ``intermediate``. tensors: ``gate_w up_w [intermediate, hidden]``,
    ``down_w [hidden, intermediate]``."""

    graph_safe = True   # launches do not depend on which requests are in the batch
    accepts_lazy_norm = True   # its first projection can apply the norm while reading its input

    @staticmethod
    def spec(prefix: str, hidden: int, intermediate: int,
             names=("gate_proj.weight", "up_proj.weight", "down_proj.weight")) -> PartSpec:
        """``names``: what the gate, up and down matrices are called behind ``prefix``."""
        return PartSpec("swiglu", {"hidden": hidden, "intermediate": intermediate}, {
            "gate_w": TensorSpec(f"{prefix}.{names[0]}", (intermediate, hidden)),
            "up_w": TensorSpec(f"{prefix}.{names[1]}", (intermediate, hidden)),
            "down_w": TensorSpec(f"{prefix}.{names[2]}", (hidden, intermediate)),
        })

    def __init__(self, spec: PartSpec, tensors: Dict[str, torch.Tensor], rt: Runtime):
        super().__init__(spec, tensors, rt)
        self.hidden = int(spec.params["hidden"])
        self.intermediate = int(spec.params["intermediate"])
        # One fused operand: rows [gate | up].
        self.w_gate_up = rt.matrix(torch.cat([tensors["gate_w"], tensors["up_w"]], dim=0))
        self.w_down = rt.matrix(tensors["down_w"])

    def forward(self, h: torch.Tensor, residual32: torch.Tensor, ctx: StepContext) -> None:
        act = torch.empty((h.shape[0], self.intermediate), dtype=self.rt.dtype, device=h.device)
        self.ops.linear_swiglu(h, self.w_gate_up, act)
        self.ops.linear(act, self.w_down, None, residual32, "add")


class PolyNormFeedForward(FeedForward):
    """``down(act(up(h)))`` with biases and ``act(z) = c0 N(z) + c1 N(z^2) + c2 N(z^3) + c3``: powers element by
    element, ``N`` divides a token's vector by its root mean square (``eps`` inside the root), in 32-bit.
    params: ``hidden``, ``intermediate``, ``eps``. tensors: ``up_w [intermediate, hidden]``, ``up_b``,
    ``down_w [hidden, intermediate]``, ``down_b``, ``coef [4]``."""

    graph_safe = True   # launches do not depend on which requests are in the batch

    @staticmethod
    def spec(prefix: str, hidden: int, intermediate: int, eps: float) -> PartSpec:
        return PartSpec("polynorm_ffn", {"hidden": hidden, "intermediate": intermediate, "eps": eps}, {
            "up_w": TensorSpec(f"{prefix}.up", (intermediate, hidden)),
            "up_b": TensorSpec(f"{prefix}.up.b", (intermediate,), "bias"),
            "down_w": TensorSpec(f"{prefix}.down", (hidden, intermediate)),
            "down_b": TensorSpec(f"{prefix}.down.b", (hidden,), "bias"),
            "coef": TensorSpec(f"{prefix}.act", (4,), "unit"),
        })

    def __init__(self, spec: PartSpec, tensors: Dict[str, torch.Tensor], rt: Runtime):
        super().__init__(spec, tensors, rt)
        self.hidden, self.intermediate = int(spec.params["hidden"]), int(spec.params["intermediate"])
        self.eps = float(spec.params["eps"])
        self.w_up, self.b_up = rt.matrix(tensors["up_w"]), rt.vector32(tensors["up_b"])
        self.w_down, self.b_down = rt.matrix(tensors["down_w"]), rt.vector32(tensors["down_b"])
        self.coef = rt.vector32(tensors["coef"])

    def forward(self, h: torch.Tensor, residual32: torch.Tensor, ctx: StepContext) -> None:
        z32 = torch.empty((h.shape[0], self.intermediate), dtype=torch.float32, device=h.device)
        self.ops.linear(h, self.w_up, self.b_up, z32, "f32")
        act = torch.empty((h.shape[0], self.intermediate), dtype=self.rt.dtype, device=h.device)
        self.ops.poly_norm(z32, self.coef, self.eps, act)
        self.ops.linear(act, self.w_down, self.b_down, residual32, "add")


class RoutedExperts(FeedForward):
    """A mixture of experts: ``experts`` gated feed-forwards ``W_down (silu(W_gate x) * (W_up x))`` without biases, of
    which every token uses ``top``. Router: logits ``z = W_router h`` in 32-bit, scores ``sigmoid(z)``; the ``top`` largest
    are chosen (the first of equal ones); a chosen expert's score is its weight, as it is (``renormalize`` is not among
    the options), and it multiplies the expert's INPUT: the output is ``sum_e expert_e(score_e * h)``, added to the
    residual stream.

    params: ``hidden``, ``ff`` (an expert's inner width), ``experts``, ``top``. tensors: ``router [experts, hidden]`` and per
    expert i ``e<i>_gate, e<i>_up [ff, hidden]``, ``e<i>_down [hidden, ff]``; they are stacked once at load into
    ``[experts, 2 ff, hidden]`` (gate rows, then up rows) and ``[experts, hidden, ff]``."""

    graph_safe = True   # the launches depend on the token count alone: the tile table of the routing lives on the device

    @staticmethod
    def spec(prefix: str, hidden: int, ff: int, experts: int, top: int) -> PartSpec:
        t = {"router": TensorSpec(f"{prefix}.router", (experts, hidden))}
        for i in range(experts):
            t[f"e{i}_gate"] = TensorSpec(f"{prefix}.e{i}.gate", (ff, hidden))
            t[f"e{i}_up"] = TensorSpec(f"{prefix}.e{i}.up", (ff, hidden))
            t[f"e{i}_down"] = TensorSpec(f"{prefix}.e{i}.down", (hidden, ff))
        return PartSpec("routed_experts", {"hidden": hidden, "ff": ff, "experts": experts, "top": top}, t)

    def __init__(self, spec: PartSpec, tensors: Dict[str, torch.Tensor], rt: Runtime):
        super().__init__(spec, tensors, rt)
        p = spec.params
        self.hidden, self.ff = int(p["hidden"]), int(p["ff"])
        self.experts, self.top = int(p["experts"]), int(p["top"])
        if not (1 <= self.top <= self.experts):
            raise ValueError(f"a token uses {self.top} of {self.experts} experts")
        self.w_router = rt.matrix(tensors["router"])
        self.w_gate_up = rt.matrix(torch.stack([torch.cat([tensors[f"e{i}_gate"], tensors[f"e{i}_up"]], dim=0)
                                                for i in range(self.experts)]))
        self.w_down = rt.matrix(torch.stack([tensors[f"e{i}_down"] for i in range(self.experts)]))

    def forward(self, h, residual32: torch.Tensor, ctx: StepContext) -> None:
        h = as_tensor(h)
        m, dev = h.shape[0], h.device
        chosen = torch.empty((m, self.top), dtype=torch.int32, device=dev)
        weight = torch.empty((m, self.top), dtype=torch.float32, device=dev)
        # a short step (decoding): router, choice and grouping are one launch where the backend has one
        step = getattr(self.ops, "moe_step", None)
        plan = step(h, self.w_router, self.top, self.w_gate_up, self.w_down, chosen, weight) if step is not None else None
        if plan is not None:
            self.ops.moe_experts(h, chosen, weight, self.w_gate_up, self.w_down, residual32, plan=plan)
            return
        z32 = torch.empty((m, self.experts), dtype=torch.float32, device=dev)
        self.ops.linear(h, self.w_router, None, z32, "f32")
        self.ops.moe_route(z32, self.top, chosen, weight)
        self.ops.moe_experts(h, chosen, weight, self.w_gate_up, self.w_down, residual32)


register_part("routed_experts", RoutedExperts)
register_part("swiglu", SwiGLU)
register_part("polynorm_ffn", PolyNormFeedForward)
