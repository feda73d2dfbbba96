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
    """A mixture of experts: ``experts`` small feed-forwards without biases, of which every token uses ``top``. Router: logits
    ``z = W_router h`` in 32-bit; the ``top`` outputs with the largest scores are chosen (the first of equal ones); the
    result, the weighted sum of the chosen experts, is added to the residual stream.

    The form without options: experts ``W_down (silu(W_gate x) * (W_up x))``, scores ``sigmoid(z)``, a chosen expert's score is
    its weight as it is, and it multiplies the expert's INPUT: ``sum_e expert_e(score_e * h)``.

    Options (params):

    * ``score`` "softmax": the scores are the softmax of a token's logits over ALL router outputs;
    * ``correction``: a stored number per router output is added to the scores for the CHOICE only; the weights are the
      scores without it;
    * ``renormalize``: the chosen scores are divided by their sum (+ 1e-20);
    * ``weight_on`` "output": the weight multiplies the expert's result, ``sum_e score_e * expert_e(h)``;
    * ``gated`` False: an expert is ``W_down relu(W_up x)^2`` (tensors ``e<i>_up``, ``e<i>_down``);
    * ``identity`` n: the router has n more outputs behind the experts' that stand for no weights: such a choice adds
      ``weight * h``;
    * ``shared`` ff: one more expert of the experts' form, ``ff`` wide, that every token uses; its result is multiplied by
      ``sigmoid(W_sg h)``, one number per token (tensors ``shared_up``, ``shared_down``, ``shared_sg [1, hidden]``; for
      experts without a gate, whose inner channels do not meet before the down product: the shared expert is cut into
      pieces of the experts' width (the last one filled up with zero rows, which add nothing) that stand FIRST in the
      stacked matrices and that every token uses with the weight ``sigmoid(W_sg h)``, so it runs inside the same grouped
      products as the chosen experts). Its gate logit is one more row of the router's product.

    params: ``hidden``, ``ff`` (an expert's inner width), ``experts``, ``top`` and the options. tensors: ``router [experts +
    identity, hidden]`` and per expert i ``e<i>_gate, e<i>_up [ff, hidden]``, ``e<i>_down [hidden, ff]``; they are stacked once at
    load into ``[experts, 2 ff, hidden]`` (gate rows, then up rows; ``[experts, ff, hidden]`` without gates) and
    ``[experts, hidden, ff]``."""

    graph_safe = True   # the launches depend on the token count alone: the tile table of the routing lives on the device

    @staticmethod
    def spec(prefix: str, hidden: int, ff: int, experts: int, top: int, *, score: str = "sigmoid", correction: bool = False,
             renormalize: bool = False, weight_on: str = "input", gated: bool = True, identity: int = 0, shared: int = 0) -> PartSpec:
        t = {"router": TensorSpec(f"{prefix}.router", (experts + identity, hidden))}
        if correction:
            t["correction"] = TensorSpec(f"{prefix}.correction", (experts + identity,), "bias")
        for i in range(experts):
            if gated:
                t[f"e{i}_gate"] = TensorSpec(f"{prefix}.e{i}.gate", (ff, hidden))
            t[f"e{i}_up"] = TensorSpec(f"{prefix}.e{i}.up", (ff, hidden))
            t[f"e{i}_down"] = TensorSpec(f"{prefix}.e{i}.down", (hidden, ff))
        if shared:
            t["shared_up"] = TensorSpec(f"{prefix}.shared.up", (shared, hidden))
            t["shared_down"] = TensorSpec(f"{prefix}.shared.down", (hidden, shared))
            t["shared_sg"] = TensorSpec(f"{prefix}.shared.sg", (1, hidden))
        params = {"hidden": hidden, "ff": ff, "experts": experts, "top": top}
        options = {"score": score, "correction": bool(correction), "renormalize": bool(renormalize), "weight_on": weight_on,
                   "gated": bool(gated), "identity": int(identity), "shared": int(shared)}
        defaults = {"score": "sigmoid", "correction": False, "renormalize": False, "weight_on": "input", "gated": True, "identity": 0, "shared": 0}
        params.update({k: v for k, v in options.items() if v != defaults[k]})
        return PartSpec("routed_experts", params, t)

    def __init__(self, spec: PartSpec, tensors: Dict[str, torch.Tensor], rt: Runtime):
        super().__init__(spec, tensors, rt)
        p = spec.params
        self.hidden, self.ff = int(p["hidden"]), int(p["ff"])
        self.experts, self.top = int(p["experts"]), int(p["top"])
        self.score, self.renormalize = str(p.get("score", "sigmoid")), bool(p.get("renormalize", False))
        self.weight_on, self.gated = str(p.get("weight_on", "input")), bool(p.get("gated", True))
        self.identity, self.shared = int(p.get("identity", 0)), int(p.get("shared", 0))
        self.outputs = self.experts + self.identity         # what the router chooses among
        if not (1 <= self.top <= self.outputs):
            raise ValueError(f"a token uses {self.top} of {self.outputs} router outputs")
        if self.score not in ("sigmoid", "softmax") or self.weight_on not in ("input", "output"):
            raise ValueError(f"unknown router score '{self.score}' or place of the weight '{self.weight_on}'")
        if self.shared and self.gated:
            raise ValueError("an expert that every token uses is built for experts without a gate")
        # the shared expert's gate logit is one more row of the router's product
        rows = [tensors["router"]] + ([tensors["shared_sg"]] if self.shared else [])
        self.w_router = rt.matrix(torch.cat(rows, dim=0))
        self.correction = rt.vector32(tensors["correction"]) if p.get("correction") else None
        first = (lambda i: torch.cat([tensors[f"e{i}_gate"], tensors[f"e{i}_up"]], dim=0)) if self.gated else (lambda i: tensors[f"e{i}_up"])
        ups = [first(i) for i in range(self.experts)]
        downs = [tensors[f"e{i}_down"] for i in range(self.experts)]
        self.pieces = -(-self.shared // self.ff) if self.shared else 0     # the shared expert as experts of the common width
        if self.shared:
            if self.weight_on != "output":
                raise ValueError("a shared expert's gate multiplies its result: the weights of this mixture stand on the output")
            up, down = tensors["shared_up"], tensors["shared_down"]
            fill = self.pieces * self.ff - self.shared
            if fill:
                up = torch.cat([up, torch.zeros((fill, self.hidden), dtype=up.dtype)], dim=0)
                down = torch.cat([down, torch.zeros((self.hidden, fill), dtype=down.dtype)], dim=1)
            ups = [up[j * self.ff:(j + 1) * self.ff] for j in range(self.pieces)] + ups
            downs = [down[:, j * self.ff:(j + 1) * self.ff] for j in range(self.pieces)] + downs
        self.w_gate_up = rt.matrix(torch.stack(ups))
        self.w_down = rt.matrix(torch.stack(downs))
        self.plain = self.score == "sigmoid" and not self.renormalize and self.correction is None and self.weight_on == "input" \
            and self.gated and not self.identity and not self.shared

    def forward(self, h, residual32: torch.Tensor, ctx: StepContext) -> None:
        h = as_tensor(h)
        m, dev = h.shape[0], h.device
        if self.plain:
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
            return
        extra, always = (1, self.pieces) if self.shared else (0, 0)
        chosen = torch.empty((m, self.top + always), dtype=torch.int32, device=dev)
        weight = torch.empty((m, self.top + always), dtype=torch.float32, device=dev)
        options = dict(score=self.score, renormalize=self.renormalize, correction32=self.correction, always=always)
        step = getattr(self.ops, "moe_step", None)
        plan = step(h, self.w_router, self.top, self.w_gate_up, self.w_down, chosen, weight, n_real=self.experts + always, extra=extra,
                    **options) if step is not None else None
        if plan is None:
            z32 = torch.empty((m, self.outputs + extra), dtype=torch.float32, device=dev)
            self.ops.linear(h, self.w_router, None, z32, "f32")
            self.ops.moe_route(z32[:, :self.outputs], self.top, chosen, weight, **options)
        self.ops.moe_experts(h, chosen, weight, self.w_gate_up, self.w_down, residual32, plan=plan, gated=self.gated,
                             weight_on=self.weight_on, outputs=self.outputs + always)
        if self.identity:
            self.ops.moe_identity(h, residual32, chosen, weight, self.experts + always)


register_part("routed_experts", RoutedExperts)
register_part("swiglu", SwiGLU)
register_part("polynorm_ffn", PolyNormFeedForward)
