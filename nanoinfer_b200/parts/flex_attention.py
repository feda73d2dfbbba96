"""Softmax attention over the paged cache with the options that decoder designs combine: keys and values of
different widths, a short causal convolution on q, k and v, a per-head RMS norm of q and k, rotation of part of a head,
a bias by distance, a soft cap on the scores, a window or a chunked mask, a sigmoid gate on the output.

With ``q = W_q h + b_q`` (likewise k, v), in this order:

* convolution (``conv`` taps > 0): ``y_t = sum_j w[:, j] u_(t - taps + 1 + j)`` per channel, zeros before the request's
  start; the request's last ``taps - 1`` projected rows are kept in its state;
* ``qk_norm``: every head of q and k is divided by its root mean square (``eps`` inside the root) and multiplied by a
  gain of the head's size that all heads share; with ``qk_norm`` = "whole" the root mean square is taken over ALL heads
  of a token's q (and of its k) at once, before they are split into heads, and the gains have the projections' sizes;
* ``v_mix``: the layers of a model that set it share the values of the first of them: that one ("first") leaves its
  projected values of the step's tokens for the later ones ("blend"), whose values become
  ``(1 - lambda) v + lambda v_first`` with a learned number ``lambda`` each; the blend is what is cached;
* ``rot`` = (dims, base): the first ``dims`` elements of every q and k head are turned by ``position * base^(-2i/dims)``,
  element i paired with i + dims/2 (``rot_layout`` "half") or 2i with 2i + 1 ("interleaved"); with ``rot_factor`` f
  every frequency is divided by f (linear position scaling); the angle is formed in 32-bit;
* ``unit_norm_after_rot``: every head of q and k is divided by its root mean square AFTER the rotation, no gain;
* ``values_from_keys``: there is no value projection; a value head is the key head as projected, before norm and
  rotation (``vdim`` = ``dim``);
* ``score = (q . k) * scale``; with ``softcap`` c: ``c tanh(score / c)``; with ``slope_span`` s: head h of H loses
  ``2^(-s (h + 1) / H) * (i - j)`` at distance i - j;
* position i sees j <= i; with ``window`` w only j > i - w; with ``chunk`` c only ``floor(j / c) == floor(i / c)``,
  counted from the request's position 0;
* softmax in 32-bit; with ``sink`` the denominator holds ``exp(sink_h)`` once more, a learned number per head without
  key or value, neither scaled nor capped; weighted sum of v (``vdim`` wide), times ``sigmoid(W_g h)`` with ``out_gate``, then
  ``out_scale * (W_o . + b_o)`` is added to the residual stream.

What is cached per position is the key after convolution, norm and rotation, and the value after convolution.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..registry import register_part
from .base import CacheNeed, LayerCache, Mixer, PagedTensor, Runtime, StateNeed, StepContext, as_tensor
from .spec import PartSpec, TensorSpec


def rotary_frequencies(dims: int, base: float, factor: float = 1.0) -> torch.Tensor:
    """``base^(-2i/dims) / factor`` for the ``dims/2`` pairs, computed in 64-bit and rounded to 32-bit once."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    return (torch.pow(torch.tensor(float(base), dtype=torch.float64), -2.0 * i / float(dims)) / float(factor)).to(torch.float32)


class FlexAttention(Mixer):
    """params: ``hidden heads kv_heads dim vdim scale eps`` and the options ``bias`` (q, k, v), ``out_bias``, ``conv``
    (taps), ``qk_norm``, ``rot`` ((dims, base) or None), ``softcap``, ``slope_span``, ``window``, ``chunk``,
    ``out_gate``, ``out_scale``, ``rot_layout``, ``rot_factor``, ``unit_norm_after_rot``, ``values_from_keys``, ``sink``,
    ``v_mix`` (None, "first" or "blend"). tensors: ``q k o``, ``v`` unless the values are the keys, and, by option,
    ``q_b k_b v_b o_b q_conv k_conv v_conv q_norm k_norm g sink vmix``."""

    graph_safe = True   # launches do not depend on which requests are in the batch
    V_FIRST = "flex_attention.v_first"      # key of the step's scratch under which the first v_mix layer leaves its values

    @staticmethod
    def spec(prefix: str, hidden: int, heads: int, kv_heads: int, dim: int, vdim: int, scale: float, eps: float, *,
             bias: bool = False, out_bias: bool = False, conv: int = 0, qk_norm: bool = False, rot=None,
             softcap: float = 0.0, slope_span: float = 0.0, window: int = 0, chunk: int = 0, out_gate: bool = False,
             out_scale: float = 1.0, rot_layout: str = "half", rot_factor: float = 1.0, unit_norm_after_rot: bool = False,
             values_from_keys: bool = False, sink: bool = False, v_mix=None) -> PartSpec:
        """``qk_norm``: False, True (per head, a gain of the head's size) or "whole"."""
        nq, nk, nv = heads * dim, kv_heads * dim, kv_heads * vdim
        t = {"q": TensorSpec(f"{prefix}.q", (nq, hidden)), "k": TensorSpec(f"{prefix}.k", (nk, hidden)),
             "v": TensorSpec(f"{prefix}.v", (nv, hidden)), "o": TensorSpec(f"{prefix}.o", (hidden, heads * vdim))}
        projected = ("q", nq), ("k", nk), ("v", nv)
        if values_from_keys:
            del t["v"]
            projected = projected[:2]
        if bias:
            for name, n in projected:
                t[name + "_b"] = TensorSpec(f"{prefix}.{name}.b", (n,), "bias")
        if out_bias:
            t["o_b"] = TensorSpec(f"{prefix}.o.b", (hidden,), "bias")
        if conv:
            for name, n in projected:
                t[name + "_conv"] = TensorSpec(f"{prefix}.{name}.conv", (n, conv), "unit")
        if qk_norm:
            t["q_norm"] = TensorSpec(f"{prefix}.q.norm", (nq if qk_norm == "whole" else dim,), "gain")
            t["k_norm"] = TensorSpec(f"{prefix}.k.norm", (nk if qk_norm == "whole" else dim,), "gain")
        if sink:
            t["sink"] = TensorSpec(f"{prefix}.sink", (heads,), "unit")
        if v_mix == "blend":
            t["vmix"] = TensorSpec(f"{prefix}.vmix", (), "mix01")
        if out_gate:
            t["g"] = TensorSpec(f"{prefix}.g", (heads * vdim, hidden))
        params = {"hidden": hidden, "heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": float(scale),
                  "eps": float(eps), "bias": bias, "out_bias": out_bias, "conv": int(conv), "qk_norm": qk_norm,
                  "rot": None if rot is None else (int(rot[0]), float(rot[1])), "softcap": float(softcap),
                  "slope_span": float(slope_span), "window": int(window), "chunk": int(chunk), "out_gate": out_gate,
                  "out_scale": float(out_scale), "rot_layout": str(rot_layout), "rot_factor": float(rot_factor),
                  "unit_norm_after_rot": bool(unit_norm_after_rot), "values_from_keys": bool(values_from_keys),
                  "sink": bool(sink), "v_mix": v_mix}
        return PartSpec("flex_attention", params, t)

    def __init__(self, spec: PartSpec, tensors: Dict[str, torch.Tensor], rt: Runtime):
        super().__init__(spec, tensors, rt)
        p = spec.params
        self.hidden, self.heads, self.kv_heads = int(p["hidden"]), int(p["heads"]), int(p["kv_heads"])
        self.dim, self.vdim = int(p["dim"]), int(p["vdim"])
        if self.heads % self.kv_heads:
            raise ValueError(f"heads ({self.heads}) must be a multiple of kv_heads ({self.kv_heads})")
        self.scale, self.eps, self.out_scale = float(p["scale"]), float(p["eps"]), float(p.get("out_scale", 1.0))
        self.taps, self.softcap = int(p.get("conv", 0)), float(p.get("softcap", 0.0))
        self.window, self.chunk = int(p.get("window", 0)), int(p.get("chunk", 0))
        self.nq, self.nk, self.nv = self.heads * self.dim, self.kv_heads * self.dim, self.kv_heads * self.vdim
        self.values_from_keys = bool(p.get("values_from_keys"))
        if self.values_from_keys and (self.vdim != self.dim or self.taps):
            raise ValueError("values that are the projected keys have the keys' width, and no convolution stands between")
        if self.values_from_keys:
            self.nv = 0
        self.unit_norm_after = bool(p.get("unit_norm_after_rot"))
        self.rot_layout = str(p.get("rot_layout", "half"))
        if self.rot_layout not in ("half", "interleaved"):
            raise ValueError(f"unknown layout of rotated pairs '{self.rot_layout}'")
        self.n_qkv = self.nq + self.nk + self.nv
        self.out_gate = bool(p.get("out_gate"))
        self.n_gate = self.heads * self.vdim if self.out_gate else 0
        # One product for everything that reads h: rows [q | k | v | gate]; the gate has no bias.
        named = ("q", "k") if self.values_from_keys else ("q", "k", "v")
        rows = [tensors[n] for n in named] + ([tensors["g"]] if self.out_gate else [])
        self.w_in = rt.matrix(torch.cat(rows, dim=0))
        self.b_in = None
        if p.get("bias"):
            b = torch.zeros(self.n_qkv + self.n_gate, dtype=torch.float32)
            b[:self.n_qkv] = torch.cat([tensors[n + "_b"] for n in named]).to(torch.float32)
            self.b_in = rt.vector32(b)
        self.conv_w = rt.vector32(torch.cat([tensors[n + "_conv"] for n in named], dim=0)) if self.taps else None
        self.q_gain = rt.vector32(tensors["q_norm"]) if p.get("qk_norm") else None
        self.k_gain = rt.vector32(tensors["k_norm"]) if p.get("qk_norm") else None
        self.norm_whole = p.get("qk_norm") == "whole"
        self.sinks = rt.vector32(tensors["sink"]) if p.get("sink") else None
        self.v_mix = p.get("v_mix")
        if self.v_mix not in (None, "first", "blend") or (self.v_mix and self.values_from_keys):
            raise ValueError(f"v_mix is None, 'first' or 'blend' (and needs values of its own), not {self.v_mix!r}")
        self.vmix = rt.vector32(tensors["vmix"].reshape(1)) if self.v_mix == "blend" else None
        rot = p.get("rot")
        self.rot_dims = 0 if rot is None else int(rot[0])
        if self.rot_dims % 2 or self.rot_dims > self.dim:
            raise ValueError(f"rotated width {self.rot_dims} must be even and at most the head size {self.dim}")
        self.freq = rotary_frequencies(self.rot_dims, float(rot[1]), float(p.get("rot_factor", 1.0))).to(rt.device) if self.rot_dims else None
        span = float(p.get("slope_span", 0.0))
        self.slopes = None
        if span:
            h = torch.arange(1, self.heads + 1, dtype=torch.float64)
            self.slopes = torch.pow(torch.tensor(2.0, dtype=torch.float64), -span * h / self.heads).to(torch.float32).to(rt.device)
        self.w_o = rt.matrix(tensors["o"])
        # the sum that reaches the stream is out_scale * (W_o a + b_o): the factor goes on a (in 32-bit) and on b_o
        self.b_o = rt.vector32(tensors["o_b"].to(torch.float32) * self.out_scale) if p.get("out_bias") else None

    def cache_need(self) -> CacheNeed:
        # a chunk never looks further back than its own size, so pages behind it can go like a window's
        keep = self.window if self.window else self.chunk
        # (values that are the projected keys are still cached beside the keys: the cached key is normed and rotated)
        return CacheNeed((PagedTensor("k", self.kv_heads, self.dim), PagedTensor("v", self.kv_heads, self.vdim)), keep)

    def state_need(self) -> Optional[StateNeed]:
        return StateNeed(((self.taps - 1) * self.n_qkv,), torch.float32) if self.taps > 1 else None

    def forward(self, h: torch.Tensor, residual32: torch.Tensor, ctx: StepContext, cache: LayerCache) -> None:
        h = as_tensor(h)
        m, dev, ops = h.shape[0], h.device, self.ops
        p32 = torch.empty((m, self.n_qkv + self.n_gate), dtype=torch.float32, device=dev)
        ops.linear(h, self.w_in, self.b_in, p32, "f32")
        qkv32 = p32[:, :self.n_qkv]
        if self.taps:
            conv32 = torch.empty((m, self.n_qkv), dtype=torch.float32, device=dev)
            ops.conv_step(qkv32, self.conv_w, None, "none", cache.state, 0, ctx, conv32, self.taps)
            qkv32 = conv32
        q = torch.empty((m, self.nq), dtype=self.rt.dtype, device=dev)
        v_first = None
        if self.v_mix == "first":       # kept alive by the step's scratch until the last layer that blends has read it
            ctx.scratch[self.V_FIRST] = qkv32[:, self.nq + self.nk:]
        elif self.v_mix == "blend":
            v_first = ctx.scratch.get(self.V_FIRST)
            if v_first is None or tuple(v_first.shape) != (m, self.nv):
                raise ValueError("a layer that blends its values found no values of the same shape left by an earlier layer of this step")
        # norm, rotation, queries in the storage type, keys and values into their pages
        ops.attention_prepare(qkv32, q, self.heads, self.kv_heads, self.dim, self.vdim, self.q_gain, self.k_gain, self.eps,
                              self.freq, self.rot_dims, ctx, cache.block_table, cache.page_size, cache.pages["k"], cache.pages["v"],
                              cache.writes, layout=self.rot_layout, unit_norm_after=self.unit_norm_after,
                              values_are_keys=self.values_from_keys, norm_whole=self.norm_whole, v_first32=v_first, vmix32=self.vmix)
        gated = self.out_gate
        attn = torch.empty((m, self.heads * self.vdim), dtype=torch.float32 if gated else self.rt.dtype, device=dev)
        ops.attention_flex(q, attn, self.heads, self.kv_heads, self.dim, self.vdim, self.scale, self.softcap, self.slopes,
                           self.window, self.chunk, 1.0 if gated else self.out_scale, ctx, cache.block_table, cache.page_size,
                           cache.pages["k"], cache.pages["v"], sinks32=self.sinks)
        if gated:
            a = torch.empty((m, self.heads * self.vdim), dtype=self.rt.dtype, device=dev)
            ops.gated_norm(attn, a, gate32=p32[:, self.n_qkv:], gate_kind="sigmoid", out_scale=self.out_scale)
            attn = a
        ops.linear(attn, self.w_o, self.b_o, residual32, "add")


register_part("flex_attention", FlexAttention)
