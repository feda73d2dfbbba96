"""Attention whose keys and values come out of a cached low-rank latent.

Per token the cache holds ONE row for all heads: the latent ``c = rmsnorm(W_dkv h)[:rank]`` and a rotated key part
``kr`` of ``rot`` elements (the last rows of ``W_dkv h``, not normed, rotated by the token's position) that every
head shares. Queries go through a latent too: ``q = W_uq rmsnorm(W_dq h)``, laid out head by head as
``[plain | rotated]``. Head ``n``: key ``[W_uk,n c | kr]``, value ``W_uv,n c``, score
``(q_plain . W_uk,n c + q_rot . kr) * scale`` over the positions the window lets it see, softmax in 32-bit, then
``W_o`` over the concatenated heads, added to the residual stream. Options: a **sink** per head (a learned number whose
exponential joins the softmax's denominator once: no key, no value, not scaled) and a **gate** on the output (the
concatenated heads times ``sigmoid(W_g h)`` before ``W_o``). The rotated pairs are interleaved or half-split, as the
position encoding says.

The kernels never expand keys or values per cached position: the query is carried into the latent space
(``W_uk,n^T q_plain``), scored against the cached rows as they are, and ``W_uv,n`` is applied to the weighted sum of
latents. A layer may read the rows that an earlier layer cached (its schedule entry names that entry) and has then no
down projection for keys and values of its own.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..registry import register_part
from .base import CacheNeed, LayerCache, Mixer, PagedTensor, PositionEncoding, Runtime, StepContext
from .spec import PartSpec, TensorSpec


class LatentAttention(Mixer):
    """params: ``hidden``, ``heads``, ``dim`` (plain query/key width of a head), ``rot_dim`` (rotated width),
    ``vdim`` (value width), ``q_rank``, ``kv_rank``, ``scale``, ``window`` (0 = all keys), ``keep`` (how many of the
    last positions the cache has to keep: the largest window of the layers that read it; 0 = all), ``eps``,
    ``position`` (name of a shared ``frequency_rotary`` encoding), ``owns_kv`` (False: the rows of another entry), ``sink``,
    ``out_gate``. tensors: ``dq dq_norm uq uk uv o`` and, with ``owns_kv``, ``dkv dkv_norm``; by option ``sink [heads]``,
    ``g [heads * vdim, hidden]``."""

    graph_safe = True   # launches do not depend on which requests are in the batch

    @staticmethod
    def spec(prefix: str, hidden: int, heads: int, dim: int, rot_dim: int, vdim: int, q_rank: int, kv_rank: int,
             scale: float, window: int, keep: int, eps: float, position: str, owns_kv: bool = True, sink: bool = False,
             out_gate: bool = False) -> PartSpec:
        t = {
            "dq": TensorSpec(f"{prefix}.dq", (q_rank, hidden)),
            "dq_norm": TensorSpec(f"{prefix}.dq.norm", (q_rank,), "gain"),
            "uq": TensorSpec(f"{prefix}.uq", (heads * (dim + rot_dim), q_rank)),
            "uk": TensorSpec(f"{prefix}.uk", (heads * dim, kv_rank)),
            "uv": TensorSpec(f"{prefix}.uv", (heads * vdim, kv_rank)),
            "o": TensorSpec(f"{prefix}.o", (hidden, heads * vdim)),
        }
        if owns_kv:
            t["dkv"] = TensorSpec(f"{prefix}.dkv", (kv_rank + rot_dim, hidden))
            t["dkv_norm"] = TensorSpec(f"{prefix}.dkv.norm", (kv_rank,), "gain")
        if sink:
            t["sink"] = TensorSpec(f"{prefix}.sink", (heads,), "unit")
        if out_gate:
            t["g"] = TensorSpec(f"{prefix}.g", (heads * vdim, hidden))
        return PartSpec("latent_attention", {
            "hidden": hidden, "heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank,
            "kv_rank": kv_rank, "scale": scale, "window": window, "keep": keep, "eps": eps, "position": position,
            "owns_kv": owns_kv, "sink": bool(sink), "out_gate": bool(out_gate)}, t)

    def __init__(self, spec: PartSpec, tensors: Dict[str, torch.Tensor], rt: Runtime):
        super().__init__(spec, tensors, rt)
        p = spec.params
        self.hidden, self.heads = int(p["hidden"]), int(p["heads"])
        self.dim, self.rot_dim, self.vdim = int(p["dim"]), int(p["rot_dim"]), int(p["vdim"])
        self.q_rank, self.kv_rank = int(p["q_rank"]), int(p["kv_rank"])
        self.scale, self.eps = float(p["scale"]), float(p["eps"])
        self.window, self.keep = int(p.get("window", 0)), int(p.get("keep", 0))
        if self.keep and (not self.window or self.window > self.keep):
            raise ValueError("the cache keeps fewer positions than the window reads")
        self.owns_kv = bool(p.get("owns_kv", True))
        self.position_name = str(p["position"])
        self.g_dq = rt.vector32(tensors["dq_norm"])
        self.w_uq, self.w_uk, self.w_uv = rt.matrix(tensors["uq"]), rt.matrix(tensors["uk"]), rt.matrix(tensors["uv"])
        self.w_o = rt.matrix(tensors["o"])
        self.w_dkv = self.g_dkv = None
        self.sink = rt.vector32(tensors["sink"]) if p.get("sink") else None
        self.out_gate = bool(p.get("out_gate"))
        # One product for everything that reads h: rows [dq | g | dkv], each part starting on a multiple of 8 columns
        rows, self._cols, at = [], {}, 0
        for name, on in (("dq", True), ("g", self.out_gate), ("dkv", self.owns_kv)):
            if not on:
                continue
            w = tensors[name]
            self._cols[name] = (at, at + w.shape[0])
            pad = (-w.shape[0]) % 8
            rows += [w] + ([torch.zeros((pad, w.shape[1]), dtype=w.dtype)] if pad else [])
            at += w.shape[0] + pad
        self.w_in = rt.matrix(torch.cat(rows, dim=0))
        if self.owns_kv:
            self.g_dkv = rt.vector32(tensors["dkv_norm"])
        self._freq = None
        self._layout = "interleaved"

    def cache_need(self) -> CacheNeed:
        return CacheNeed((PagedTensor("latent", 1, self.kv_rank + self.rot_dim),), self.keep)

    def bind_positions(self, positions: Dict[str, PositionEncoding]) -> None:
        freq = getattr(positions[self.position_name], "frequencies", None)
        if freq is None:
            raise ValueError("latent attention binds to a position encoding that gives frequencies")
        self._freq = freq()
        self._layout = getattr(positions[self.position_name], "layout", "interleaved")
        if self._freq[2] != self.rot_dim:
            raise ValueError(f"the position encoding rotates {self._freq[2]} elements, the mixer {self.rot_dim}")

    def forward(self, h: torch.Tensor, residual32: torch.Tensor, ctx: StepContext, cache: LayerCache) -> None:
        m, dev, ops = h.shape[0], h.device, self.ops
        freq, mag, _ = self._freq
        pages = cache.pages["latent"]
        p32 = torch.empty((m, self.w_in.shape[0]), dtype=torch.float32, device=dev)
        ops.linear(h, self.w_in, None, p32, "f32")
        if cache.writes:
            if not self.owns_kv:
                raise ValueError("a layer that reads another layer's latents has none of its own to cache")
            lo, hi = self._cols["dkv"]
            ops.latent_store(p32[:, lo:hi], self.g_dkv, self.eps, freq, mag, ctx, cache.block_table, cache.page_size, pages,
                             self.kv_rank, self.rot_dim, layout=self._layout)
        cq32 = p32[:, :self.q_rank]
        cq = torch.empty((m, self.q_rank), dtype=self.rt.dtype, device=dev)
        ops.gated_norm(cq32, cq, groups=1, eps=self.eps, gain32=self.g_dq)      # an RMS norm of rows that lie apart
        q32 = torch.empty((m, self.heads * (self.dim + self.rot_dim)), dtype=torch.float32, device=dev)
        ops.linear(cq, self.w_uq, None, q32, "f32")
        q_width, q_dtype = ops.latent_query_layout(pages.dtype, self.kv_rank, self.rot_dim)     # what the attention kernel reads
        qa = torch.empty((m, self.heads * q_width), dtype=q_dtype, device=dev)
        ops.latent_query(q32, self.w_uk, freq, mag, ctx.positions, qa, self.heads, self.dim, self.kv_rank, self.rot_dim,
                         layout=self._layout)
        lat32 = torch.empty((m, self.heads * self.kv_rank), dtype=torch.float32, device=dev)
        ops.latent_attention(qa, lat32, ctx, cache.block_table, cache.page_size, pages, self.heads, self.kv_rank,
                             self.rot_dim, self.scale, self.window, sink32=self.sink)
        attn = torch.empty((m, self.heads * self.vdim), dtype=self.rt.dtype, device=dev)
        gate32 = p32[:, self._cols["g"][0]:self._cols["g"][1]] if self.out_gate else None
        ops.latent_value(lat32, self.w_uv, attn, self.heads, self.vdim, self.kv_rank, gate32=gate32)
        ops.linear(attn, self.w_o, None, residual32, "add")


register_part("latent_attention", LatentAttention)
