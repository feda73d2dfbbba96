"""The kernel library as Python sees it: loads ``libnanoinfer_b200.so`` (building it first if needed)
and wraps each exported function. There is no other implementation behind these calls: if the
library cannot be built or loaded, or the device is not a CUDA device, they raise.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p
from types import SimpleNamespace
from typing import Optional

import torch

from . import build as _build
from ..config.kernel_options import KernelOptions
from ..parts.base import LazyNorm


class KernelError(RuntimeError):
    pass


_DT = {torch.float32: 0, torch.bfloat16: 1}
_EPI = {"store": 0, "add": 1, "f32": 2, "swiglu": 3}
_LAYOUT = {"interleaved": 0, "half": 1}     # which elements of a rotated vector make a pair


def _ptr(t: Optional[torch.Tensor]) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


def _need(t: torch.Tensor, dtype, what: str, contiguous: bool = True):
    if not t.is_cuda:
        raise KernelError(f"{what}: tensor is on {t.device}, the kernels run on CUDA only")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{what}: expected {dtype}, got {t.dtype}")
    if contiguous and not t.is_contiguous():
        raise KernelError(f"{what}: tensor must be contiguous")


class _StreamScope:
    def __init__(self, ops):
        self.ops = ops

    def __enter__(self):
        self.prev = self.ops._bound_stream
        self.ops._bound_stream = c_void_p(torch.cuda.current_stream().cuda_stream)
        return self

    def __exit__(self, *exc):
        self.ops._bound_stream = self.prev
        return False


class Kernels:
    """The kernel library as one engine sees it: the loaded library (shared by all instances of the process), this
    instance's options, which never change, and its scratch memory."""

    name = "cuda-sm100a"

    def __init__(self, lib_path: str, options: Optional[KernelOptions] = None):
        self.lib_path = lib_path
        self.options = options if options is not None else KernelOptions()
        self.launches = 0           # kernel launches issued through this object (graph replays add theirs)
        self._bound_stream = None   # the stream of the enclosing stream_scope(), if any
        self._op_events = None      # time_ops(): (what, event) behind every launch
        self._timeline = None       # timeline_start(): the device buffer the kernels note their times in
        self._norm_before_small_m = False   # set while a product resolves its LazyNorm: what kernel the norm is followed by
        self.sm_count = 0           # SMs of the device, asked when the instance is made ready (load_kernels)
        self._ws_scratch = None                # scratch and counters of the small-M GEMM's cross-CTA split
        self._ws_counters = None
        self._ws_attn_counters = None
        try:
            self._lib = ctypes.CDLL(lib_path)
        except OSError as e:
            raise KernelError(f"cannot load the kernel library {lib_path}: {e}") from e
        self._lib.nib_last_error.restype = ctypes.c_char_p
        for name in ("nib_embed", "nib_rmsnorm", "nib_rope_store", "nib_gemm_simt", "nib_attention_generic",
                     "nib_gemm_smallm", "nib_gemm_smallm_supported", "nib_gemm_tc", "nib_gemm_tc_splitk",
                     "nib_gemm_tc_pair", "nib_gemm_tc_supported", "nib_gemm_tc_error", "nib_attention_mma_supported",
                     "nib_attention_prefill_mma", "nib_attention_decode_mma", "nib_attention_decode_tma",
                     "nib_attention_decode_tma_supported",
                     "nib_attention_decode_tma_error", "nib_argmax", "nib_argmax_chunked", "nib_sample", "nib_repetition_penalty", "nib_device_arch",
                     "nib_sm_count", "nib_gemm_smallm_qkv", "nib_gemm_smallm_qkv_supported", "nib_gemm_tc_qkv",
                     "nib_gemm_tc_qkv_supported", "nib_poly_norm", "nib_depth_mix", "nib_unary", "nib_head_norm_gate",
                     "nib_delta_rule_scan", "nib_causal_conv", "nib_rglru_scan", "nib_latent_store", "nib_latent_query",
                     "nib_latent_attention", "nib_latent_value", "nib_latent_attention_mma", "nib_latent_attention_mma_supported",
                     "nib_latent_attention_mma_qwidth", "nib_block_diag_smallm", "nib_rmsnorm_pair", "nib_rmsnorm_pair_supported", "nib_head_product_supported",
                     "nib_head_product_nk", "nib_head_product_kn", "nib_depth_mix_norm_pair", "nib_embed_scaled", "nib_gated_norm",
                     "nib_linear_state_scan", "nib_conv_tokens", "nib_conv_tail", "nib_conv_step", "nib_token_shift", "nib_decay_map", "nib_step_sizes",
                     "nib_attention_prepare", "nib_attention_flex", "nib_attention_flex_mma", "nib_attention_flex_mma_supported",
                     "nib_rmsnorm_add", "nib_moe_route", "nib_moe_max_tiles", "nib_moe_group", "nib_moe_gemm_simt", "nib_moe_combine",
                     "nib_moe_tc_supported", "nib_moe_tc_error", "nib_moe_gather_rows", "nib_moe_gemm_tc", "nib_moe_step", "nib_moe_step_supported"):
            getattr(self._lib, name).restype = c_int

    # ---- plumbing ---------------------------------------------------------------------------
    def _check(self, rc: int, what: str) -> None:
        self.launches += 1
        if rc != 0:
            raise KernelError(f"{what}: {self._lib.nib_last_error().decode()}")
        if self._op_events is not None:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record(torch.cuda.current_stream())
            self._op_events.append((what, ev))

    # ---- where the time goes ----------------------------------------------------------------
    def time_ops(self, on: bool = True):
        """Eager launches only. While on, an event is recorded behind every launch; ``op_times()`` then gives
        (what, microseconds) per launch, the time from the launch before it to its own end. Events between
        kernels end the overlap of programmatic dependent launch, so this suits steps whose kernels run for
        tens of microseconds (prompt portions); a decode step is read with ``timeline_start`` instead."""
        if on:
            start = torch.cuda.Event(enable_timing=True)
            start.record(torch.cuda.current_stream())
            self._op_events = [("start", start)]
        else:
            self._op_events = None

    def op_times(self):
        torch.cuda.synchronize()
        ev = self._op_events or []
        out = [(what, 1000.0 * ev[i - 1][1].elapsed_time(e)) for i, (what, e) in enumerate(ev) if i > 0]
        self._op_events = ev[-1:] if ev else None
        return out

    def timeline_start(self, capacity: int = 8192) -> None:
        """From now on the kernels launched (and the graphs captured) note the GPU's nanosecond timer at their
        entry, after their wait for the earlier kernels and at their end (first CTA, first thread):
        ``timeline()`` returns the notes. Works inside captured graphs and leaves the overlap of dependent
        launches as it is; the notes cost a few hundred nanoseconds each."""
        self._timeline = torch.zeros(1 + 2 * capacity, dtype=torch.int64, device="cuda")
        self._lib.nib_trace_set(c_void_p(self._timeline.data_ptr()), c_int(capacity))

    def timeline_clear(self) -> None:
        if self._timeline is not None:
            torch.cuda.synchronize()
            self._timeline.zero_()
            torch.cuda.synchronize()

    def timeline(self):
        """[(t_ns, kernel, tag, phase)] in time order; phase 0 entry, 1 after the wait, 2 done."""
        if self._timeline is None:
            return []
        torch.cuda.synchronize()
        h = self._timeline.cpu().tolist()
        n = min(int(h[0]), (len(h) - 1) // 2)
        notes = []
        for i in range(n):
            code, t = h[1 + 2 * i], h[2 + 2 * i]
            notes.append((t, TIMELINE_KERNELS.get(code >> 16, str(code >> 16)), (code >> 8) & 0xff, code & 0xff))
        return sorted(notes)

    def timeline_stop(self) -> None:
        """Kernels launched from now on note nothing. Graphs captured while the timeline was on still write into its
        buffer, which therefore stays allocated."""
        self._lib.nib_trace_set(c_void_p(0), c_int(0))

    def _stream(self) -> c_void_p:
        if self._bound_stream is not None:
            return self._bound_stream
        return c_void_p(torch.cuda.current_stream().cuda_stream)

    def stream_scope(self):
        """Within the scope the kernels launch on the stream that is current at its start, looked up once: a
        forward pass issues some two hundred launches, and asking torch for the current stream costs about
        as much as a launch. The caller must not switch streams inside the scope."""
        return _StreamScope(self)

    def device_arch(self) -> int:
        return self._lib.nib_device_arch()

    # ---- kernels ----------------------------------------------------------------------------
    def embed(self, ids, table, out32, scale=1.0):
        """out32[t] = table[ids[t]] * scale."""
        _need(ids, torch.int32, "embed ids"); _need(table, None, "embed table"); _need(out32, torch.float32, "embed out")
        m, hidden = out32.shape
        self._check(self._lib.nib_embed_scaled(_ptr(ids), _ptr(table), _ptr(out32), c_int(m), c_int(hidden),
                                               c_int(table.shape[0]), c_int(_DT[table.dtype]), c_float(scale), self._stream()), "embed")

    def rmsnorm(self, x32, gain32, eps, out, rows=None):
        _need(x32, torch.float32, "rmsnorm x"); _need(gain32, torch.float32, "rmsnorm gain"); _need(out, None, "rmsnorm out")
        if rows is not None:
            _need(rows, torch.int32, "rmsnorm rows")
        n, hidden = out.shape
        if x32.shape[1] != hidden or gain32.numel() != hidden:
            raise KernelError("rmsnorm: widths differ")
        self._check(self._lib.nib_rmsnorm(_ptr(x32), _ptr(gain32), _ptr(rows), _ptr(out), c_int(n), c_int(hidden),
                                          c_float(eps), c_int(_DT[out.dtype]), c_int(1 if self._norm_before_small_m else 0),
                                          self._stream()), "rmsnorm")

    def with_options(self, options: Optional[KernelOptions] = None, **changes) -> "Kernels":
        """Another instance on the same library and the same scratch memory (so: for use on the same stream) whose
        options are ``options``, or this instance's with ``changes``. Its launch counter starts at this one's value."""
        import copy
        import dataclasses
        k = copy.copy(self)
        k.options = options if options is not None else dataclasses.replace(self.options, **changes)
        return k

    def ensure_workspace(self, device) -> None:
        """Scratch memory that kernels share between launches (allocated once, outside any graph capture)."""
        if self._ws_scratch is None:
            self._ws_scratch = torch.empty(8 * 1024 * 1024, dtype=torch.float32, device=device)
            self._ws_counters = torch.zeros(16 * 1024, dtype=torch.int32, device=device)
            self._ws_attn_counters = torch.zeros(64 * 1024, dtype=torch.int32, device=device)
            self._ws_argmax = torch.zeros(4096 * 64, dtype=torch.int64, device=device)
            self._ws_argmax_counters = torch.zeros(4096, dtype=torch.int32, device=device)

    def linear(self, a, w, bias32, out, mode):
        """out[M,N] (=, +=) a[M,K] . w[N,K]^T (+ bias). mode: 'store' | 'add' (float out) | 'f32' (float out).
        ``a`` may be a LazyNorm: the small-M kernel then applies the norm while it reads the residual stream."""
        lazy = a if isinstance(a, LazyNorm) else None
        dtype = a.dtype
        if lazy is None:
            _need(a, None, "linear a")
        _need(w, dtype, "linear w"); _need(out, None, "linear out")
        if bias32 is not None:
            _need(bias32, torch.float32, "linear bias")
        m, k = a.shape
        n = w.shape[0]
        if w.shape[1] != k or tuple(out.shape) != (m, n):
            raise KernelError(f"linear: shapes a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)} do not fit")
        want_out = dtype if mode == "store" else torch.float32
        if out.dtype != want_out:
            raise KernelError(f"linear[{mode}]: out must be {want_out}, got {out.dtype}")
        self._gemm(a, w, bias32, out, m, n, k, _EPI[mode])

    def _route(self, m: int, rows: int, k: int, epi: int, has_norm: bool):
        """Which kernel multiplies ``m`` tokens with ``rows x k`` bfloat16 weights, and whether a lazy
        norm is applied inside it. Measured on B200 with cold weights at the projection sizes of the 0.5B,
        1.5B and 7B models: the small-M kernel (weights streamed straight into mma.sync fragments) wins
        while the weights are few or the tcgen05 kernel would have few tiles and cannot split K cheaply;
        the tcgen05 kernel wins for wide outputs, for more tokens, and, with K split over CTAs and summed
        by reductions in memory, for every sum into the residual stream with a long K. The fused norm
        re-reads the 32-bit activations in every CTA, which pays only for few tokens and narrow outputs."""
        if self.options.gemm_route is not None:
            return ("tc", False) if self.options.gemm_route in ("tc", "tc_pair") else ("smallm", has_norm and self.options.gemm_route == "smallm_fused")
        if self.options.smallm_ksplit or self.options.smallm_cross:
            return "smallm", has_norm
        weight_bytes = 2 * rows * k
        if epi == _EPI["add"]:
            small = m <= 16 and k <= 2048
        elif epi == _EPI["store"]:
            small = m <= 64 and rows <= 6144
        elif epi == _EPI["swiglu"]:
            small = (m <= 8 and weight_bytes <= 64e6) or (m <= 16 and weight_bytes <= 12e6)
        else:
            small = m <= 16 and weight_bytes <= 32e6
        # (inside the gate/up product the norm measured slower, +2 us a layer at the 0.5B widths: 300 CTAs re-read
        # the 32-bit activations; the norm kernel before it costs less)
        fuse = has_norm and small and epi != _EPI["swiglu"] and (m <= 8 or (m <= 16 and k <= 1024))
        return ("smallm" if small else "tc"), fuse

    def _use_pair(self, m: int, rows: int, k: int, epi: int) -> bool:
        """Whether pairs of SMs (cta_group::2, tiles of 256 features) take this product."""
        if self.options.gemm_route is not None:
            return self.options.gemm_route == "tc_pair"
        if self.options.tc_token_tile or self.options.tc_splits or m < 256:
            return False
        if epi == _EPI["add"]:      # with K split over pairs of SMs (at least 8 blocks of 64 per item)
            tiles = -(-rows // 256) * -(-m // 256)
            pairs = self.sm_count // 2
            splits = max(1, min(pairs // tiles, (k // 64) // 8)) if tiles < pairs else 1
            return tiles * splits >= 48
        # measured on B200 at the projection sizes of the 0.5B, 1.5B and 7B models, 512..4096 tokens: tiles
        # of 256 tokens x 256 features on two SMs win once there are enough of them to fill the GPU; the
        # fused gate/up form (gate rows in one CTA, up rows in the other) wins from 256 tokens on
        if epi == _EPI["swiglu"]:
            return True
        tiles = -(-rows // 256) * -(-m // 256)
        return tiles >= 48

    def _resolve(self, lazy, before_small_m: bool):
        """The norm's values for a product that cannot apply the norm itself. The norm kernel is told what follows it: a
        small-M product of up to 16 tokens has next to no set-up of its own and is let in late (see nib_rmsnorm); measured at batch 8:
        0.730 -> 0.715 ms a step at the 0.5B widths, 1.72 -> 1.60 ms at the 1.5B widths, and the opposite before a
        tcgen05 product."""
        self._norm_before_small_m = before_small_m
        try:
            return lazy.resolve()
        finally:
            self._norm_before_small_m = False

    @staticmethod
    def _foldable(lazy) -> bool:
        """Whether the kernels can apply this norm themselves: the kinds they know, and only while nobody has
        computed it (a computed norm is just a tensor)."""
        return lazy is not None and lazy.resolved is None and lazy.fold.kind == "rms"

    def _gemm(self, a, w, bias32, out, m, n, k, epi):
        """bfloat16 goes to the small-M kernel or to the tcgen05 kernel (see ``_route``); shapes neither
        takes, and 32-bit, run the CUDA-core kernel."""
        lazy = a if isinstance(a, LazyNorm) else None
        if lazy is not None and not self._foldable(lazy):
            a, lazy = lazy.resolve(), None
        bf16 = a.dtype == torch.bfloat16 and not self.options.force_simt_gemm
        if bf16 and self.options.tc_token_tile == 0:
            kernel, fuse = self._route(m, w.shape[0], k, epi, lazy is not None)
            if lazy is not None and not fuse:
                a, lazy = self._resolve(lazy, kernel == "smallm" and m <= 16), None
            src = lazy.fold.x32 if lazy is not None else a
            if kernel == "smallm" and self._lib.nib_gemm_smallm_supported(
                    _ptr(src), _ptr(w), c_int(m), c_int(k), c_int(src.stride(0)), c_int(4 if lazy is not None else 2)) == 1:
                self.ensure_workspace(src.device)
                gain = lazy.fold.gain32 if lazy is not None else None
                self._check(self._lib.nib_gemm_smallm(
                    _ptr(src), _ptr(w), _ptr(bias32), _ptr(out), c_int(m), c_int(n), c_int(k), c_int(src.stride(0)),
                    c_int(out.stride(0)), c_int(epi), _ptr(gain), c_float(lazy.fold.eps if lazy is not None else 0.0),
                    c_int(self.options.smallm_ksplit), c_int(self.options.smallm_cross), _ptr(self._ws_scratch), _ptr(self._ws_counters),
                    c_longlong(self._ws_scratch.numel()), c_int(self._ws_counters.numel()), self._stream()),
                    "linear (small M)")
                return
        if lazy is not None:
            a = lazy.resolve()
        if bf16 and self._lib.nib_gemm_tc_supported(_ptr(a), _ptr(w), c_int(k), c_int(a.stride(0))) == 1:
            if self._use_pair(m, w.shape[0], k, epi):
                self._check(self._lib.nib_gemm_tc_pair(
                    _ptr(a), _ptr(w), _ptr(bias32), _ptr(out), c_int(m), c_int(n), c_int(k), c_int(a.stride(0)),
                    c_int(out.stride(0)), c_int(epi), c_int(self.options.pair_n_tile), c_int(self.options.tc_splits), self._stream()),
                    "linear (tensor cores, two SMs per tile)")
                return
            self.ensure_workspace(a.device)
            self._check(self._lib.nib_gemm_tc_splitk(
                _ptr(a), _ptr(w), _ptr(bias32), _ptr(out), c_int(m), c_int(n), c_int(k), c_int(a.stride(0)),
                c_int(out.stride(0)), c_int(epi), c_int(self.options.tc_token_tile), c_int(self.options.tc_splits),
                _ptr(self._ws_scratch), _ptr(self._ws_counters), c_longlong(self._ws_scratch.numel()),
                c_longlong(self._ws_counters.numel()), self._stream()), "linear (tensor cores)")
            return
        self._check(self._lib.nib_gemm_simt(_ptr(a), _ptr(w), _ptr(bias32), _ptr(out), c_int(m), c_int(n), c_int(k),
                                            c_int(a.stride(0)), c_int(out.stride(0)), c_int(epi), c_int(_DT[a.dtype]),
                                            self._stream()), "linear")

    def gemm_tc_error(self) -> int:
        """The error word of the tensor-core GEMM's bounded waits (0 = none); synchronises and clears it."""
        return self._lib.nib_gemm_tc_error()

    def linear_swiglu(self, a, w_gate_up, out):
        """out[M,I] = silu(a . w[:I]^T) * (a . w[I:]^T)."""
        if not isinstance(a, LazyNorm):
            _need(a, None, "swiglu a")
        _need(w_gate_up, a.dtype, "swiglu w"); _need(out, a.dtype, "swiglu out")
        m, k = a.shape
        inter = w_gate_up.shape[0] // 2
        if w_gate_up.shape[0] != 2 * inter or w_gate_up.shape[1] != k or tuple(out.shape) != (m, inter):
            raise KernelError("linear_swiglu: shapes do not fit")
        self._gemm(a, w_gate_up, None, out, m, inter, k, _EPI["swiglu"])

    def qkv_project(self, a, w_qkv, bias32, qkv, heads, kv_heads, head_dim, positions, req_index, rotary,
                    block_table, page_size, k_pages, v_pages, writes):
        """qkv = a . w_qkv^T + bias with query and key heads rotated by their positions; with ``writes`` the
        rotated keys and the values also go into the cache pages. ``a`` may be a LazyNorm.

        Up to 16 tokens of bfloat16 take one kernel for all of it (bias, rotation and the page write are the
        small-M product's epilogue, the norm its prologue); so do the tiles of 128 tokens of the one-CTA tcgen05
        product (heads of 64 or 128 that are rotated whole); everything else is the product followed by
        ``rope_store``."""
        lazy = a if isinstance(a, LazyNorm) else None
        if lazy is not None and not self._foldable(lazy):
            a, lazy = lazy.resolve(), None
        m, k = a.shape
        n = w_qkv.shape[0]
        rot = 0 if rotary is None else rotary[2]
        fused = fused_tc = False
        o = self.options
        if a.dtype == torch.bfloat16 and o.fuse_qkv and not o.force_simt_gemm and o.tc_token_tile in (0, 128) \
                and o.gemm_route in (None, "smallm", "smallm_fused", "tc") and not o.smallm_ksplit and not o.smallm_cross:
            kernel, with_norm = self._route(m, n, k, _EPI["store"], lazy is not None)
            if lazy is not None and not with_norm:
                a, lazy = self._resolve(lazy, kernel == "smallm" and m <= 16), None
            src = lazy.fold.x32 if lazy is not None else a
            fused = kernel == "smallm" and o.tc_token_tile == 0 and qkv.stride(0) % 2 == 0 and self._lib.nib_gemm_smallm_qkv_supported(
                _ptr(src), _ptr(w_qkv), c_int(m), c_int(k), c_int(src.stride(0)), c_int(4 if lazy is not None else 2),
                c_int(head_dim), c_int(rot)) == 1
            # the one-CTA tcgen05 product takes tiles of 128 tokens from 65 tokens on (nib_gemm_tc_splitk's choice)
            fused_tc = not fused and kernel == "tc" and (m > 64 or o.tc_token_tile == 128) and o.tc_splits in (0, 1) \
                and not self._use_pair(m, n, k, _EPI["store"]) and self._lib.nib_gemm_tc_qkv_supported(
                    _ptr(a), _ptr(w_qkv), _ptr(bias32), _ptr(qkv), c_int(k), c_int(a.stride(0)), c_int(qkv.stride(0)),
                    c_int(head_dim), c_int(rot)) == 1
        if not fused and not fused_tc:
            self.linear(a, w_qkv, bias32, qkv, "store")
            self.rope_store(qkv, heads, kv_heads, head_dim, positions, req_index, rotary, block_table, page_size,
                            k_pages, v_pages, writes)
            return
        _need(w_qkv, torch.bfloat16, "qkv w"); _need(qkv, torch.bfloat16, "qkv out")
        _need(positions, torch.int32, "positions"); _need(req_index, torch.int32, "req_index")
        if n != (heads + 2 * kv_heads) * head_dim or tuple(qkv.shape) != (m, n) or w_qkv.shape[1] != k:
            raise KernelError("qkv_project: shapes do not fit the head counts")
        if bias32 is not None:
            _need(bias32, torch.float32, "qkv bias")
        cos = sin = None
        if rotary is not None:
            cos, sin, _ = rotary
            _need(cos, torch.float32, "cos"); _need(sin, torch.float32, "sin")
            if cos.shape[1] != rot // 2:
                raise KernelError("qkv_project: table width must be rot/2")
        num_pages = bt_stride = 0
        if writes:
            _need(block_table, torch.int32, "block_table", contiguous=False)
            _need(k_pages, torch.bfloat16, "k_pages"); _need(v_pages, torch.bfloat16, "v_pages")
            if tuple(k_pages.shape[1:]) != (kv_heads, page_size, head_dim) or block_table.stride(1) != 1:
                raise KernelError("qkv_project: pages or block table do not fit")
            num_pages, bt_stride = k_pages.shape[0], block_table.stride(0)
        if fused_tc:
            self._check(self._lib.nib_gemm_tc_qkv(
                _ptr(a), _ptr(w_qkv), _ptr(bias32), _ptr(qkv), c_int(m), c_int(heads), c_int(kv_heads), c_int(head_dim),
                c_int(k), c_int(a.stride(0)), c_int(qkv.stride(0)), _ptr(positions), _ptr(req_index), _ptr(cos), _ptr(sin),
                c_int(rot), _ptr(block_table if writes else None), c_int(bt_stride), c_int(page_size),
                _ptr(k_pages if writes else None), _ptr(v_pages if writes else None), c_int(num_pages),
                c_int(1 if writes else 0), self._stream()), "q/k/v projection (tensor cores) with rotation and page write")
            return
        gain = lazy.fold.gain32 if lazy is not None else None
        self._check(self._lib.nib_gemm_smallm_qkv(
            _ptr(src), _ptr(w_qkv), _ptr(bias32), _ptr(qkv), c_int(m), c_int(heads), c_int(kv_heads), c_int(head_dim),
            c_int(k), c_int(src.stride(0)), c_int(qkv.stride(0)), _ptr(gain), c_float(lazy.fold.eps if lazy is not None else 0.0),
            _ptr(positions), _ptr(req_index), _ptr(cos), _ptr(sin), c_int(rot), _ptr(block_table if writes else None),
            c_int(bt_stride), c_int(page_size), _ptr(k_pages if writes else None), _ptr(v_pages if writes else None),
            c_int(num_pages), c_int(1 if writes else 0), self._stream()), "q/k/v projection with rotation and page write")

    def rope_store(self, qkv, heads, kv_heads, head_dim, positions, req_index, rotary, block_table,
                   page_size, k_pages, v_pages, writes):
        _need(qkv, None, "rope qkv"); _need(positions, torch.int32, "positions"); _need(req_index, torch.int32, "req_index")
        m = qkv.shape[0]
        if qkv.shape[1] != (heads + 2 * kv_heads) * head_dim:
            raise KernelError("rope_store: qkv width does not fit the head counts")
        cos = sin = None
        rot = 0
        if rotary is not None:
            cos, sin, rot = rotary
            _need(cos, torch.float32, "cos"); _need(sin, torch.float32, "sin")
            if cos.shape[1] != rot // 2:
                raise KernelError("rope_store: table width must be rot/2")
        num_pages = 0
        bt_stride = 0
        if writes:
            _need(block_table, torch.int32, "block_table", contiguous=False)
            _need(k_pages, qkv.dtype, "k_pages"); _need(v_pages, qkv.dtype, "v_pages")
            if tuple(k_pages.shape[1:]) != (kv_heads, page_size, head_dim):
                raise KernelError(f"rope_store: pages {tuple(k_pages.shape)} do not fit kv_heads/page_size/head_dim")
            if block_table.stride(1) != 1:
                raise KernelError("rope_store: block_table rows must be dense")
            num_pages, bt_stride = k_pages.shape[0], block_table.stride(0)
        self._check(self._lib.nib_rope_store(
            _ptr(qkv), _ptr(positions), _ptr(req_index), _ptr(cos), _ptr(sin), c_int(rot),
            _ptr(block_table if writes else None), c_int(bt_stride), c_int(page_size),
            _ptr(k_pages if writes else None), _ptr(v_pages if writes else None), c_int(m), c_int(heads),
            c_int(kv_heads), c_int(head_dim), c_int(num_pages), c_int(1 if writes else 0),
            c_int(_DT[qkv.dtype]), self._stream()), "rope_store")

    def attention(self, qkv, out, heads, kv_heads, head_dim, scale, window, ctx, block_table,
                  page_size, k_pages, v_pages, own_kv=False):
        """Attention of every token of the step over its request's cached keys (positions lo..own).

        bfloat16 with a supported head size runs on the tensor cores: the leading requests that bring one
        token each go to the decode kernel (keys split over CTAs), the others to the prefill kernel.
        Everything else (32-bit, other head sizes) runs the general kernel. ``own_kv``: the rows of ``qkv`` also
        hold each token's own rotated key and its value, the same that its page holds (a decode kernel may then
        take them from the row instead of waiting for the page write)."""
        _need(qkv, None, "attention qkv"); _need(out, qkv.dtype, "attention out")
        _need(k_pages, qkv.dtype, "k_pages"); _need(v_pages, qkv.dtype, "v_pages")
        _need(block_table, torch.int32, "block_table", contiguous=False)
        if tuple(k_pages.shape[1:]) != (kv_heads, page_size, head_dim):
            raise KernelError(f"attention: pages {tuple(k_pages.shape)} do not fit kv_heads/page_size/head_dim")
        if block_table.stride(1) != 1:
            raise KernelError("attention: block_table rows must be dense")
        m = qkv.shape[0]
        num_pages, bt_stride = k_pages.shape[0], block_table.stride(0)
        fast = qkv.dtype == torch.bfloat16 and not self.options.force_general_attention and \
            self._lib.nib_attention_mma_supported(c_int(heads), c_int(kv_heads), c_int(head_dim)) == 1
        if not fast:
            self._check(self._lib.nib_attention_generic(
                _ptr(qkv), c_int(qkv.stride(0)), _ptr(out), _ptr(ctx.positions), _ptr(ctx.req_index), _ptr(block_table),
                c_int(bt_stride), c_int(page_size), _ptr(k_pages), _ptr(v_pages), c_int(num_pages),
                c_int(m), c_int(heads), c_int(kv_heads), c_int(head_dim), c_float(scale), c_int(window),
                c_int(_DT[qkv.dtype]), self._stream()), "attention")
            return
        q_lens, ctx_lens = ctx.host.q_lens, ctx.host.ctx_lens
        n_req = len(q_lens)
        n_dec = 0
        if heads // kv_heads <= 16:
            while n_dec < n_req and q_lens[n_dec] == 1:
                n_dec += 1
        if n_dec:
            tma = self._decode_tma_ok(heads, kv_heads, head_dim, page_size)
            splits = self.decode_splits(n_dec, kv_heads, max(ctx_lens[:n_dec]), window, tma, head_dim)
            part_o = part_ml = counters = None
            if splits > 1 and not tma and not self.options.separate_combine and n_dec * kv_heads <= 64 * 1024:
                self.ensure_workspace(qkv.device)
                counters = self._ws_attn_counters
            parts = splits // 8 if tma else splits      # the TMA kernel merges up to eight splits inside a cluster
            if parts > 1:
                part_o = torch.empty(n_dec * heads * parts * head_dim, dtype=torch.float32, device=qkv.device)
                part_ml = torch.empty(n_dec * heads * parts * 2, dtype=torch.float32, device=qkv.device)
            common = (_ptr(qkv), c_int(qkv.stride(0)), _ptr(out), _ptr(ctx.ctx_lens), _ptr(block_table), c_int(bt_stride),
                      c_int(page_size), _ptr(k_pages), _ptr(v_pages), c_int(num_pages), c_int(n_dec), c_int(heads),
                      c_int(kv_heads), c_int(head_dim), c_float(scale), c_int(window), c_int(splits))
            if tma:
                self._check(self._lib.nib_attention_decode_tma(*common, c_int(1 if own_kv else 0), _ptr(part_o), _ptr(part_ml), self._stream()),
                            "attention decode (TMA)")
                counters = None
            else:
                self._check(self._lib.nib_attention_decode_mma(*common, _ptr(part_o), _ptr(part_ml), _ptr(counters),
                                                               self._stream()), "attention decode")
            if parts > 1 and counters is None:
                self.launches += 1
        if n_dec < n_req:
            q_start = c_void_p(ctx.q_start.data_ptr() + 4 * n_dec)
            lens = c_void_p(ctx.ctx_lens.data_ptr() + 4 * n_dec)
            table = c_void_p(block_table.data_ptr() + 4 * n_dec * bt_stride)
            if not self.options.force_mma_prefill and self._lib.nib_attention_prefill_tc_supported(
                    c_int(heads), c_int(kv_heads), c_int(head_dim), c_int(page_size), c_int(qkv.stride(0))) == 1:
                self._check(self._lib.nib_attention_prefill_tc(
                    _ptr(qkv), c_int(qkv.stride(0)), _ptr(out), q_start, lens, table, c_int(bt_stride), c_int(page_size),
                    _ptr(k_pages), _ptr(v_pages), c_int(num_pages), c_int(n_req - n_dec), c_int(max(q_lens[n_dec:])),
                    c_int(m), c_int(heads), c_int(kv_heads), c_int(head_dim), c_float(scale), c_int(window), c_float(0.0), c_int(0), None,
                    self._stream()), "attention prefill (tcgen05)")
            else:
                self._check(self._lib.nib_attention_prefill_mma(
                    _ptr(qkv), c_int(qkv.stride(0)), _ptr(out), q_start, lens, table, c_int(bt_stride), c_int(page_size),
                    _ptr(k_pages), _ptr(v_pages), c_int(num_pages), c_int(n_req - n_dec), c_int(max(q_lens[n_dec:])),
                    c_int(heads), c_int(kv_heads), c_int(head_dim), c_float(scale), c_int(window), self._stream()),
                    "attention prefill")

    def attention_tc_error(self) -> int:
        """The error word of the tcgen05 attention's bounded waits (0 = none); synchronises and clears it."""
        return self._lib.nib_attention_tc_error()

    def _decode_tma_ok(self, heads, kv_heads, head_dim, page_size) -> bool:
        return self.options.decode_tma and page_size > 0 and self._lib.nib_attention_decode_tma_supported(
            c_int(heads), c_int(kv_heads), c_int(head_dim), c_int(page_size)) == 1

    def attention_decode_tma_error(self) -> int:
        """The error word of the TMA decode kernel's bounded waits (0 = none); synchronises and clears it."""
        return self._lib.nib_attention_decode_tma_error()

    def check_device_errors(self) -> None:
        """Raises ``KernelError`` if a bounded wait of a tcgen05 or TMA kernel has run out since the last check.

        Such a kernel returns instead of hanging, and what it wrote is not to be trusted. The words are read
        with a 4-byte copy each, which waits for the device: call it where the host waits anyway (a request
        finishes, a run ends, results are about to be written out)."""
        raise_device_errors([
            ("tensor-core GEMM (gemm_tcgen05.cu)", self.gemm_tc_error(), _GEMM_TC_ROLES),
            ("tcgen05 prefill attention (attention_tcgen05.cu)", self.attention_tc_error(), _ATTN_TC_ROLES),
            ("TMA decode attention (attention_decode_tma.cu)", self.attention_decode_tma_error(), _DECODE_TMA_ROLES),
            ("routed experts on the tensor cores (moe_tcgen05.cu)", self._lib.nib_moe_tc_error(), _GEMM_TC_ROLES),
        ])

    def decode_splits(self, n_tokens: int, kv_heads: int, max_ctx: int, window: int, tma: bool = False,
                      head_dim: int = 128) -> int:
        """Into how many CTAs the keys of a decoding token are split. The kernel with TMA page loads keeps
        several tiles in flight per CTA: about 256 CTAs in all (measured best from 1 to 64 requests), at
        least four of its tiles (128 keys for heads of 64, else 64) each. The cp.async kernel: two key tiles per CTA (both are in flight at once, so a
        CTA waits for memory once), as long as that does not make more CTAs than fill the GPU about eight
        times."""
        if self.options.fixed_decode_splits:
            return _cluster_splits(self.options.fixed_decode_splits) if tma else self.options.fixed_decode_splits
        keys = min(max_ctx, window) if window > 0 else max_ctx
        tiles = -(-keys // 64) + 1
        if tma:
            want = max(1, round(256 / max(1, n_tokens * kv_heads)))
            tile_keys = 128 if head_dim == 64 else 64           # the kernel's tile
            n = max(1, min(want, -(-keys // tile_keys) // 4, 64))
            return _cluster_splits(n)
        most = max(1, (8 * self.sm_count) // max(1, n_tokens * kv_heads))
        return max(1, min(-(-tiles // 2), most, 64))

    # ---- row-wise and element-wise kernels that several designs share (pointwise.cu) -------------
    @staticmethod
    def _rows(t, dtype, what):
        """A matrix whose rows are dense but may lie apart (a slice of the columns of a wider one)."""
        _need(t, dtype, what, contiguous=False)
        if t.dim() != 2 or t.stride(1) != 1:
            raise KernelError(f"{what}: rows must be dense")

    def rmsnorm_pair(self, x32, gain_a32, gain_b32, eps, out_a, out_b):
        """Two RMS norms of the same rows with different gains (the two branches of a parallel block): the rows are read
        and their statistic computed once where the width allows, else one after the other."""
        if self._lib.nib_rmsnorm_pair_supported(c_int(x32.shape[1])) != 1:
            self.rmsnorm(x32, gain_a32, eps, out_a)
            self.rmsnorm(x32, gain_b32, eps, out_b)
            return
        _need(x32, torch.float32, "rmsnorm_pair x"); _need(gain_a32, torch.float32, "rmsnorm_pair gain"); _need(gain_b32, torch.float32, "rmsnorm_pair gain")
        _need(out_a, None, "rmsnorm_pair out"); _need(out_b, out_a.dtype, "rmsnorm_pair out")
        n, hidden = x32.shape
        if tuple(out_a.shape) != (n, hidden) or tuple(out_b.shape) != (n, hidden) or gain_a32.numel() != hidden or gain_b32.numel() != hidden:
            raise KernelError("rmsnorm_pair: shapes do not fit")
        self._check(self._lib.nib_rmsnorm_pair(_ptr(x32), _ptr(gain_a32), _ptr(gain_b32), _ptr(out_a), _ptr(out_b), c_int(n), c_int(hidden),
                                               c_float(eps), c_int(_DT[out_a.dtype]), self._stream()), "rmsnorm (two gains)")

    def poly_norm(self, z32, coef32, eps, out):
        """out = c0 N(z) + c1 N(z^2) + c2 N(z^3) + c3 per row, N(y) = y / sqrt(mean(y^2) + eps); coef32 = (c0..c3)."""
        self._rows(z32, torch.float32, "poly_norm z"); self._rows(out, None, "poly_norm out")
        _need(coef32, torch.float32, "poly_norm coefficients")
        if z32.shape != out.shape or coef32.numel() != 4:
            raise KernelError("poly_norm: shapes do not fit")
        self._check(self._lib.nib_poly_norm(_ptr(z32), c_int(z32.stride(0)), _ptr(coef32), _ptr(out), c_int(out.stride(0)),
                                            c_int(z32.shape[0]), c_int(z32.shape[1]), c_float(eps), c_int(_DT[out.dtype]),
                                            self._stream()), "poly_norm")

    def depth_mix(self, hist32, x32, coef32, n):
        """hist32[n-1] = x32, then x32 = sum_{j<n} coef32[j] * hist32[j] (ascending j)."""
        _need(hist32, torch.float32, "depth_mix history"); _need(x32, torch.float32, "depth_mix x"); _need(coef32, torch.float32, "depth_mix coefficients")
        if hist32.shape[0] < n or tuple(hist32.shape[1:]) != tuple(x32.shape) or coef32.numel() < n:
            raise KernelError("depth_mix: shapes do not fit")
        self._check(self._lib.nib_depth_mix(_ptr(hist32), _ptr(x32), _ptr(coef32), c_int(n), c_longlong(x32.numel()),
                                            self._stream()), "depth_mix")

    def depth_mix_norm_pair(self, hist32, x32, coef32, n, gain_a32, gain_b32, eps, out_a, out_b):
        """``depth_mix`` followed by ``rmsnorm_pair`` of the new x32, in one pass over the rows where the width allows."""
        if self._lib.nib_rmsnorm_pair_supported(c_int(x32.shape[1])) != 1:
            self.depth_mix(hist32, x32, coef32, n)
            self.rmsnorm_pair(x32, gain_a32, gain_b32, eps, out_a, out_b)
            return
        _need(hist32, torch.float32, "depth_mix history"); _need(x32, torch.float32, "depth_mix x"); _need(coef32, torch.float32, "depth_mix coefficients")
        _need(gain_a32, torch.float32, "gain"); _need(gain_b32, torch.float32, "gain"); _need(out_a, None, "norm out"); _need(out_b, out_a.dtype, "norm out")
        rows, hidden = x32.shape
        if hist32.shape[0] < n or tuple(hist32.shape[1:]) != (rows, hidden) or coef32.numel() < n or tuple(out_a.shape) != (rows, hidden) \
                or tuple(out_b.shape) != (rows, hidden) or gain_a32.numel() != hidden or gain_b32.numel() != hidden:
            raise KernelError("depth_mix_norm_pair: shapes do not fit")
        self._check(self._lib.nib_depth_mix_norm_pair(_ptr(hist32), _ptr(x32), _ptr(coef32), c_int(n), _ptr(gain_a32), _ptr(gain_b32),
                                                      _ptr(out_a), _ptr(out_b), c_int(rows), c_int(hidden), c_float(eps), c_int(_DT[out_a.dtype]),
                                                      self._stream()), "depth_mix + rmsnorm (two gains)")

    def unary(self, in32, out, kind):
        """out = f(in32) element by element with a change of storage type; kind: 'tanh' | 'copy' | 'sigmoid'."""
        self._rows(in32, torch.float32, "unary in"); self._rows(out, None, "unary out")
        if in32.shape != out.shape:
            raise KernelError("unary: shapes differ")
        self._check(self._lib.nib_unary(_ptr(in32), c_int(in32.stride(0)), _ptr(out), c_int(out.stride(0)), c_int(in32.shape[0]),
                                        c_int(in32.shape[1]), c_int({"tanh": 0, "copy": 1, "sigmoid": 2}[kind]),
                                        c_int(_DT[out.dtype]), self._stream()), "unary")

    def head_norm_gate(self, o32, gate32, gain32, eps, heads, d, out):
        """out[t, h, :] = o32[t, h, :] / rms(o32[t, h, :]) * gain32[h, :] * sigmoid(gate32[t, h, :])."""
        self._rows(o32, torch.float32, "head_norm_gate o"); self._rows(gate32, torch.float32, "head_norm_gate gate")
        self._rows(out, None, "head_norm_gate out"); _need(gain32, torch.float32, "head_norm_gate gain")
        m = o32.shape[0]
        if o32.shape[1] != heads * d or tuple(gate32.shape) != (m, heads * d) or tuple(out.shape) != (m, heads * d) or gain32.numel() != heads * d:
            raise KernelError("head_norm_gate: shapes do not fit")
        self._check(self._lib.nib_head_norm_gate(_ptr(o32), c_int(o32.stride(0)), _ptr(gate32), c_int(gate32.stride(0)), _ptr(gain32),
                                                 _ptr(out), c_int(out.stride(0)), c_int(m), c_int(heads), c_int(d), c_float(eps),
                                                 c_int(_DT[out.dtype]), self._stream()), "head_norm_gate")

    def block_diag_linear(self, a_blocks, w_blocks, bias32, out32, a32=None):
        """out32[b] = a_blocks[b] . w_blocks[b]^T + bias32[b] for every block b: a_blocks [blocks, tokens, k],
        w_blocks [blocks, n, k], bias32 [blocks, n] or None, out32 [blocks, tokens, n] floats. ``a32``: the same
        activations as floats, token-major [tokens, blocks * k]. Up to 16 tokens take one launch for all blocks on the
        CUDA cores (a decode step); more tokens take one launch on the tensor cores where the block size allows (from
        ``a32``, rounded to bfloat16 on the way), else a product per block on the matrix kernels."""
        _need(a_blocks, None, "block_diag_linear a"); _need(w_blocks, a_blocks.dtype, "block_diag_linear w"); _need(out32, torch.float32, "block_diag_linear out")
        nb, m, k = a_blocks.shape
        n = w_blocks.shape[1]
        if tuple(w_blocks.shape) != (nb, n, k) or tuple(out32.shape) != (nb, m, n) or (bias32 is not None and tuple(bias32.shape) != (nb, n)):
            raise KernelError("block_diag_linear: shapes do not fit")
        if m <= 16:
            if bias32 is not None:
                _need(bias32, torch.float32, "block_diag_linear bias")
            self._check(self._lib.nib_block_diag_smallm(_ptr(a_blocks), _ptr(w_blocks), _ptr(bias32), _ptr(out32), c_int(nb), c_int(m),
                                                        c_int(n), c_int(k), c_int(_DT[a_blocks.dtype]), self._stream()), "block-diagonal product (few tokens)")
            return
        if a32 is not None and w_blocks.dtype == torch.bfloat16 and not self.options.force_simt_gemm \
                and self._lib.nib_head_product_supported(c_int(0), c_int(k), c_int(n)) == 1:
            _need(a32, torch.float32, "block_diag_linear a32")
            if tuple(a32.shape) != (m, nb * k):
                raise KernelError("block_diag_linear: a32 does not fit")
            self._check(self._lib.nib_head_product_nk(_ptr(a32), c_int(nb * k), _ptr(w_blocks), _ptr(bias32), _ptr(out32), c_int(n),
                                                      c_longlong(m * n), c_int(1), c_int(m), c_int(nb), c_int(n), c_int(k), _ptr(None), c_int(0),
                                                      self._stream()), "block-diagonal product (tensor cores)")
            return
        for b in range(nb):
            self.linear(a_blocks[b], w_blocks[b], None if bias32 is None else bias32[b], out32[b], "f32")

    def rmsnorm_add(self, y32, gain32, eps, mult, x32, h_out=None, clear=False, next_gain32=None, next_eps=0.0):
        """x32 += mult * y32 / rms(y32) * gain32, row by row (``eps`` inside the root): the residual sum of a block whose norm
        stands on a sublayer's output. ``h_out``: the new x32 also in that tensor's type. ``clear``: y32 is left zeroed.
        With ``next_gain32`` what goes to ``h_out`` is the next sublayer's norm of the new row instead:
        x32 / rms(x32) * next_gain32 with ``next_eps``."""
        self._rows(y32, torch.float32, "rmsnorm_add y"); self._rows(x32, torch.float32, "rmsnorm_add x"); _need(gain32, torch.float32, "rmsnorm_add gain")
        m, n = x32.shape
        if tuple(y32.shape) != (m, n) or gain32.numel() != n or not y32.is_contiguous() or not x32.is_contiguous():
            raise KernelError("rmsnorm_add: shapes do not fit")
        if h_out is not None:
            _need(h_out, None, "rmsnorm_add h")
            if tuple(h_out.shape) != (m, n):
                raise KernelError("rmsnorm_add: h_out has the stream's shape")
        if next_gain32 is not None:
            _need(next_gain32, torch.float32, "rmsnorm_add next gain")
            if next_gain32.numel() != n or h_out is None:
                raise KernelError("rmsnorm_add: the next norm has a gain of the row's size and a tensor to go to")
        self._check(self._lib.nib_rmsnorm_add(_ptr(y32), _ptr(gain32), _ptr(x32), _ptr(h_out), c_int(m), c_int(n), c_float(eps), c_float(mult),
                                              c_int(1 if clear else 0), c_int(_DT[h_out.dtype] if h_out is not None else 0), _ptr(next_gain32),
                                              c_float(next_eps), self._stream()), "rmsnorm_add")

    # ---- routed experts (moe.cu) ---------------------------------------------------------------------------
    def moe_route(self, z32, top, sel_e, sel_w, score="sigmoid", renormalize=False, correction32=None, always=0):
        """From the router logits z32 [tokens, experts]: sel_e [tokens, top] int32 = the experts with the largest logits (the
        first of equal ones), sel_w [tokens, top] = sigmoid of their logits. Options: ``score`` 'softmax' (over all the logits
        of a token); ``correction32`` [experts] is added to the scores for the choice alone; ``renormalize`` divides the chosen
        scores by their sum + 1e-20. With an option z32 is overwritten by the scores. ``always`` n: every token also uses the
        first n of the stacked experts (the pieces of a shared expert), so a chosen router output o is written as expert
        o + n; sel_e and sel_w are [tokens, top + n], the last n entries of a row being the experts 0..n-1, each weighted by
        sigmoid of the logit that stands behind the router's in the token's row (z32 is then a view of a wider matrix)."""
        self._rows(z32, torch.float32, "moe_route z"); _need(sel_e, torch.int32, "moe_route experts"); _need(sel_w, torch.float32, "moe_route weights")
        m, experts = z32.shape
        if tuple(sel_e.shape) != (m, top + always) or tuple(sel_w.shape) != (m, top + always) or (always and z32.stride(0) <= experts):
            raise KernelError("moe_route: shapes do not fit")
        if correction32 is not None:
            _need(correction32, torch.float32, "moe_route correction")
            if correction32.numel() != experts:
                raise KernelError("moe_route: one correction per router output")
        self._check(self._lib.nib_moe_route(_ptr(z32), c_int(z32.stride(0)), _ptr(sel_e), _ptr(sel_w), c_int(m), c_int(experts), c_int(top),
                                            c_int(_moe_mode(score, renormalize)), _ptr(correction32), c_int(always), self._stream()), "moe_route")

    def _moe_tc(self, h, w_gate_up, w_down) -> bool:
        """bfloat16 in widths of 8 takes the tensor-core products; everything else (32-bit, odd widths) the CUDA cores."""
        experts, _, hidden = w_gate_up.shape
        return h.dtype == torch.bfloat16 and not self.options.force_simt_gemm and self._lib.nib_moe_tc_supported(
            _ptr(h), c_int(h.stride(0)), _ptr(w_gate_up), _ptr(w_down), c_int(experts), c_int(hidden), c_int(w_down.shape[2])) == 1

    def _moe_tables(self, n, experts, tc, dev):
        """Row tiles of 128 for the tensor cores (of 32 while an expert gets few rows: a decode step), of 64 for the CUDA
        cores; the index arrays of ``n`` entries: row_of, src_of, the tile table and its length."""
        tile_rows = (32 if n <= 32 * experts else 128) if tc else 64
        max_tiles = self._lib.nib_moe_max_tiles(c_int(n), c_int(experts), c_int(tile_rows))
        idx = torch.empty(2 * n + 3 * max_tiles + 1, dtype=torch.int32, device=dev)
        return SimpleNamespace(tile_rows=tile_rows, max_tiles=max_tiles, row_of=idx[:n], src_of=idx[n:2 * n],
                               tiles=idx[2 * n:2 * n + 3 * max_tiles], n_tiles=idx[2 * n + 3 * max_tiles:], rows=None)

    def moe_step(self, h, w_router, top, w_gate_up, w_down, sel_e, sel_w, score="sigmoid", renormalize=False, correction32=None,
                 n_real=None, extra=0, z_extra=None, always=0):
        """A step of few tokens: router logits (32-bit sums over the stored ``h``), the choice, the grouping and the rows
        in the experts' order in ONE launch. Fills sel_e and sel_w like ``moe_route`` (same options) and returns what
        ``moe_experts`` takes as ``plan``; None when the step is too large for one block (the caller then takes the separate
        steps). ``n_real``: the first so many router outputs are experts (the others get no rows to multiply). ``extra``: the
        last so many rows of ``w_router`` are no router outputs; their logits go to ``z_extra`` [tokens, extra] (if given).
        ``always``: as for ``moe_route`` (then ``extra`` is 1: that row's logit is the gate; ``n_real`` counts those experts too)."""
        _need(h, None, "moe_step h"); _need(w_router, h.dtype, "moe_step router")
        m, hidden = h.shape
        experts = w_router.shape[0] - extra
        n_real = experts + always if n_real is None else n_real
        if m == 0 or self.options.no_moe_step or top > experts or m * (top + always) * hidden > (1 << 20) or \
                self._lib.nib_moe_step_supported(c_int(m), c_int(hidden), c_int(experts + extra), c_int(top)) != 1:
            return None
        if always and (extra != 1 or tuple(sel_e.shape) != (m, top + always)):
            raise KernelError("moe_step: always-used experts need the gate's row behind the router's and entries of top + always a token")
        if extra and z_extra is not None:
            _need(z_extra, torch.float32, "moe_step extra logits")
            if tuple(z_extra.shape) != (m, extra):
                raise KernelError("moe_step: the extra logits are [tokens, extra]")
        if correction32 is not None:
            _need(correction32, torch.float32, "moe_step correction")
            if correction32.numel() != experts:
                raise KernelError("moe_step: one correction per router output")
        tc = self._moe_tc(h, w_gate_up, w_down)
        plan = self._moe_tables(m * (top + always), experts + always, tc, h.device)
        if tc:
            plan.rows = torch.empty((m * (top + always), hidden), dtype=h.dtype, device=h.device)
        self._check(self._lib.nib_moe_step(_ptr(h), c_int(h.stride(0)), _ptr(w_router), c_int(m), c_int(hidden), c_int(experts), c_int(top),
                                           _ptr(sel_e), _ptr(sel_w), c_int(plan.tile_rows), _ptr(plan.row_of), _ptr(plan.src_of), _ptr(plan.tiles),
                                           _ptr(plan.n_tiles), c_int(plan.max_tiles), _ptr(plan.rows), c_int(_DT[h.dtype]),
                                           c_int(_moe_mode(score, renormalize)), _ptr(correction32), c_int(n_real), c_int(extra), _ptr(z_extra),
                                           c_int(always), self._stream()), "experts: router, choice and grouping of a short step")
        return plan

    def moe_experts(self, h, sel_e, sel_w, w_gate_up, w_down, out32, plan=None, gated=True, weight_on="input", outputs=None):
        """out32[t] += sum over the token's choices c of W_down,e (silu(W_gate,e x) * (W_up,e x)) with e = sel_e[t, c] and
        x = sel_w[t, c] * h[t]: the weight stands on the expert's input. w_gate_up [experts, 2 ff, hidden] (gate rows, then up
        rows), w_down [experts, hidden, ff]. ``plan``: what ``moe_step`` returned for these choices. Options: ``gated`` False:
        experts W_down relu(W_up x)^2 with w_gate_up [experts, ff, hidden]; ``weight_on`` 'output': x = h[t] and the weight
        multiplies the expert's result; ``outputs``: how many outputs the router has when some of them (from ``experts`` on)
        are no experts: choices of those add nothing here.

        On the CUDA cores a token's choices are summed in ascending order; on the tensor cores they are added into the
        token's row by reductions in memory, in no fixed order."""
        _need(h, None, "moe_experts h"); _need(w_gate_up, h.dtype, "moe_experts w_gate_up"); _need(w_down, h.dtype, "moe_experts w_down")
        _need(sel_e, torch.int32, "moe_experts experts"); _need(sel_w, torch.float32, "moe_experts weights"); _need(out32, torch.float32, "moe_experts out")
        m, hidden = h.shape
        experts, top, ff = w_gate_up.shape[0], sel_e.shape[1], w_down.shape[2]
        if tuple(w_gate_up.shape) != (experts, (2 if gated else 1) * ff, hidden) or tuple(w_down.shape) != (experts, hidden, ff) \
                or tuple(out32.shape) != (m, hidden) or tuple(sel_e.shape) != (m, top) or tuple(sel_w.shape) != (m, top):
            raise KernelError("moe_experts: shapes do not fit")
        if weight_on not in ("input", "output"):
            raise KernelError(f"moe_experts: the weight stands on the input or the output, not '{weight_on}'")
        if m == 0:
            return
        n, dev, dt = m * top, h.device, c_int(_DT[h.dtype])
        first, w_out = c_int(1 if gated else 2), c_int(1 if weight_on == "output" else 0)
        outputs = experts if outputs is None else outputs
        tc = self._moe_tc(h, w_gate_up, w_down)
        p = plan
        if p is None:
            p = self._moe_tables(n, outputs, tc, dev)
            self._check(self._lib.nib_moe_group(_ptr(sel_e), c_int(n), c_int(outputs), c_int(p.tile_rows), _ptr(p.row_of), _ptr(p.src_of), _ptr(p.tiles),
                                                _ptr(p.n_tiles), c_int(p.max_tiles), c_int(experts), self._stream()), "moe_group")
        act = torch.empty((n, ff), dtype=h.dtype, device=dev)
        if tc:
            if p.rows is None:
                p.rows = torch.empty((n, hidden), dtype=h.dtype, device=dev)
                self._check(self._lib.nib_moe_gather_rows(_ptr(h), c_int(h.stride(0)), _ptr(p.rows), c_int(hidden), _ptr(p.src_of), c_int(n), c_int(hidden),
                                                          c_int(top), self._stream()), "experts: rows in the experts' order")
            self._check(self._lib.nib_moe_gemm_tc(first, _ptr(p.rows), c_int(hidden), c_int(n), _ptr(w_gate_up), c_int(experts), _ptr(act), c_int(ff),
                                                  _ptr(p.tiles), _ptr(p.n_tiles), c_int(p.max_tiles), _ptr(p.src_of), _ptr(sel_w), c_int(top), c_int(ff),
                                                  c_int(hidden), c_int(0), c_int(p.tile_rows), w_out, self._stream()), "experts: gate, up, activation (tensor cores)")
            self._check(self._lib.nib_moe_gemm_tc(c_int(0), _ptr(act), c_int(ff), c_int(n), _ptr(w_down), c_int(experts), _ptr(out32), c_int(out32.stride(0)),
                                                  _ptr(p.tiles), _ptr(p.n_tiles), c_int(p.max_tiles), _ptr(p.src_of), _ptr(sel_w), c_int(top), c_int(hidden),
                                                  c_int(ff), c_int(1 if top == 1 else 2), c_int(p.tile_rows), w_out, self._stream()), "experts: down (tensor cores)")
            return
        scatter = top == 1      # one choice per token: its result goes straight into the token's row
        # (rows of choices that are no experts belong to no tile: they must read as zeros in the sum of a token's choices)
        y = out32 if scatter else (torch.empty if outputs == experts else torch.zeros)((n, hidden), dtype=torch.float32, device=dev)
        self._check(self._lib.nib_moe_gemm_simt(first, _ptr(h), c_int(h.stride(0)), _ptr(w_gate_up), _ptr(act), c_int(ff), _ptr(p.tiles), _ptr(p.n_tiles),
                                                c_int(p.max_tiles), _ptr(p.src_of), _ptr(sel_w), c_int(top), c_int(ff), c_int(hidden), c_int(0), dt,
                                                w_out, self._stream()), "experts: gate, up, activation")
        self._check(self._lib.nib_moe_gemm_simt(c_int(0), _ptr(act), c_int(ff), _ptr(w_down), _ptr(y), c_int(y.stride(0)), _ptr(p.tiles), _ptr(p.n_tiles),
                                                c_int(p.max_tiles), _ptr(p.src_of), _ptr(sel_w), c_int(top), c_int(hidden), c_int(ff), c_int(1 if scatter else 0),
                                                dt, w_out, self._stream()), "experts: down")
        if not scatter:
            self._check(self._lib.nib_moe_combine(_ptr(y), _ptr(p.row_of), _ptr(out32), c_int(m), c_int(hidden), c_int(top), self._stream()),
                        "experts: sum of a token's choices")

    def moe_identity(self, h, out32, sel_e, sel_w, n_real):
        """Identity outputs of a router: out32[t] += (the sum of sel_w[t, c] over the choices with sel_e[t, c] >= n_real) * h[t]."""
        _need(h, None, "moe_identity h"); _need(sel_e, torch.int32, "moe_identity experts"); _need(sel_w, torch.float32, "moe_identity weights")
        self._rows(out32, torch.float32, "moe_identity out")
        m, hidden = h.shape
        top = sel_e.shape[1]
        if tuple(sel_e.shape) != (m, top) or tuple(sel_w.shape) != (m, top) or tuple(out32.shape) != (m, hidden):
            raise KernelError("moe_identity: shapes do not fit")
        self._check(self._lib.nib_moe_identity(_ptr(h), c_int(h.stride(0)), _ptr(sel_e), _ptr(sel_w), c_int(top), c_int(n_real), _ptr(out32),
                                               c_int(out32.stride(0)), c_int(hidden), c_int(m), c_int(_DT[h.dtype]), self._stream()), "moe_identity")

    # ---- gate, norm in groups, skip (pointwise.cu) ---------------------------------------------------------
    def gated_norm(self, o32, out, groups=0, eps=0.0, gain32=None, gate32=None, gate_kind="none", gate_first=False,
                   skip32=None, skip_coef32=None, out_scale=1.0):
        """Row by row: y = o32 (+ skip_coef32[head of c] * skip32); times act(gate32) if ``gate_first``; with ``groups`` > 0
        divided by the root mean square of each of ``groups`` equal parts (``eps`` inside the root); times ``gain32`` (a gain
        per channel, or one of a part's size shared by the parts); times act(gate32) if not ``gate_first``; times
        ``out_scale``. gate_kind: 'none' | 'sigmoid' | 'silu'. ``skip_coef32`` holds one coefficient per head."""
        self._rows(o32, torch.float32, "gated_norm o"); self._rows(out, None, "gated_norm out")
        m, n = o32.shape
        if tuple(out.shape) != (m, n):
            raise KernelError("gated_norm: shapes do not fit")
        kind = {"none": 0, "sigmoid": 1, "silu": 2}[gate_kind]
        if (kind != 0) != (gate32 is not None) or (skip32 is None) != (skip_coef32 is None):
            raise KernelError("gated_norm: a gate needs its kind, a skip its coefficients")
        for t, what in ((gate32, "gate"), (skip32, "skip")):
            if t is not None:
                self._rows(t, torch.float32, f"gated_norm {what}")
                if tuple(t.shape) != (m, n):
                    raise KernelError(f"gated_norm: {what} does not fit")
        for t, what in ((gain32, "gain"), (skip_coef32, "skip coefficients")):
            if t is not None:
                _need(t, torch.float32, f"gated_norm {what}")
        norm = 1 if groups else 0
        if not groups:      # no norm: any split of the row will do; parts of about 128 channels keep the warps short
            groups = next((g for g in range(max(1, n // 128), n + 1) if n % g == 0), 1)
        if gain32 is not None and gain32.numel() not in (n, n // groups):
            raise KernelError("gated_norm: the gain has neither a row's size nor a part's")
        self._check(self._lib.nib_gated_norm(
            _ptr(o32), c_int(o32.stride(0)), _ptr(gate32), c_int(0 if gate32 is None else gate32.stride(0)), c_int(kind),
            c_int(1 if gate_first else 0), _ptr(gain32), c_int(0 if gain32 is None else gain32.numel()), _ptr(skip32),
            c_int(0 if skip32 is None else skip32.stride(0)), _ptr(skip_coef32), c_int(0 if skip_coef32 is None else skip_coef32.numel()),
            c_int(groups), c_int(norm), c_float(eps), c_float(out_scale), _ptr(out), c_int(out.stride(0)), c_int(m), c_int(n),
            c_int(_DT[out.dtype]), self._stream()), "gated_norm")

    # ---- matrix states that decay (linear_state.cu) -------------------------------------------------------
    @staticmethod
    def _state_row(state, off, size, what):
        """A state tensor [slots, n] of floats whose rows are dense (a slice of a wider state's columns will do)."""
        _need(state, torch.float32, what, contiguous=False)
        if state.dim() != 2 or state.stride(1) != 1 or off < 0 or off + size > state.shape[1]:
            raise KernelError(f"{what}: the state does not hold {size} floats from column {off}")

    def linear_state_scan(self, q32, k32, v32, w32, state, state_off, ctx, o32, heads, kq_heads, dk, dv, q_scale=1.0,
                          bonus32=None, v_scale32=None, seg_len=None):
        """Per request and head, over the step's tokens in order, from and into ``state[slot, state_off:]`` (laid out
        [head, value channel, key channel]): S <- diag(w) S + k (v_scale v)^T, o = S^T (q_scale q); with ``bonus32``
        [heads, dk] instead o = (S_old + diag(bonus) k v^T)^T q before the update. q32, k32: [tokens, kq_heads * dk]
        (head h reads key head h // (heads / kq_heads)); v32, o32: [tokens, heads * dv]; w32: [tokens, heads * dk] (a
        decay per key channel) or [tokens, heads] (one per head); v_scale32: [tokens, heads].

        A step in which a request brings 256 tokens or more, and whose walk in order would not fill the GPU, is walked in
        segments of 128 tokens or more side by side (every
        segment from a zero state, the end states chained with the products of the segments' decays, then every segment
        again from its true entry state): the result then depends on the cut by rounding. ``seg_len``: None = that rule,
        0 = never, another multiple of 8 = segments of that length whenever a request brings more."""
        for t, what, width in ((q32, "q", kq_heads * dk), (k32, "k", kq_heads * dk), (v32, "v", heads * dv), (o32, "o", heads * dv)):
            self._rows(t, torch.float32, f"linear_state_scan {what}")
            if tuple(t.shape) != (q32.shape[0], width):
                raise KernelError(f"linear_state_scan: {what} does not fit")
        self._rows(w32, torch.float32, "linear_state_scan w")
        if w32.shape[0] != q32.shape[0] or w32.shape[1] not in (heads * dk, heads):
            raise KernelError("linear_state_scan: the decay is neither per key channel nor per head")
        per_channel = w32.shape[1] == heads * dk and not (dk == 1 and w32.shape[1] == heads)
        if bonus32 is not None:
            _need(bonus32, torch.float32, "linear_state_scan bonus")
            if bonus32.numel() != heads * dk:
                raise KernelError("linear_state_scan: the bonus does not fit")
        if v_scale32 is not None:
            _need(v_scale32, torch.float32, "linear_state_scan v_scale")
            if tuple(v_scale32.shape) != (q32.shape[0], heads):
                raise KernelError("linear_state_scan: v_scale does not fit")
        self._state_row(state, state_off, heads * dv * dk, "linear_state_scan state")
        n_req, longest = ctx.host.num_requests, max(ctx.host.q_lens)
        if seg_len is None:
            # segments pay (the work doubles) while the walk in order leaves SMs idle or with one warp per scheduler:
            # as many segments as bring the blocks to about eight per SM, none shorter than 128 tokens
            want = (8 * max(1, self.sm_count)) // max(1, -(-dv // 16) * heads * n_req)
            seg_len = max(128, -(-(-(-longest // want)) // 8) * 8) if longest >= 256 and want >= 2 else 0
        n_seg = -(-longest // seg_len) if seg_len and longest > seg_len else 1
        scratch = None
        if n_seg > 1:
            floats = n_req * n_seg * heads * (dv * dk + dk)
            if floats * 4 > (1 << 29):      # half a gigabyte of entry states: walk in order instead
                n_seg = 1
            else:
                scratch = torch.empty(floats, dtype=torch.float32, device=q32.device)
                self.launches += 2
        self._check(self._lib.nib_linear_state_scan(
            _ptr(q32), c_int(q32.stride(0)), _ptr(k32), c_int(k32.stride(0)), _ptr(v32), c_int(v32.stride(0)), _ptr(w32),
            c_int(w32.stride(0)), c_int(1 if per_channel else 0), _ptr(bonus32), _ptr(v_scale32), _ptr(state), c_longlong(state.stride(0)),
            c_int(state_off), _ptr(ctx.q_start), _ptr(ctx.state_slots), _ptr(o32), c_int(o32.stride(0)), c_int(ctx.host.num_requests),
            c_int(heads), c_int(kq_heads), c_int(dk), c_int(dv), c_float(q_scale), c_int(n_seg), c_int(seg_len if n_seg > 1 else 0), _ptr(scratch),
            self._stream()), "linear_state_scan")

    def conv_tokens(self, x32, w32, bias32, act, state, state_off, ctx, out32, taps):
        """out32[t, c] = act(bias32[c] + sum_j w32[c, j] * x32[t - (taps-1-j), c]) within each request; inputs before the
        step's first token come from ``state[slot, state_off + i * width + c]`` (i = 0 oldest). act: 'none' | 'silu'."""
        self._rows(x32, torch.float32, "conv_tokens x"); self._rows(out32, torch.float32, "conv_tokens out"); _need(w32, torch.float32, "conv_tokens w")
        m, width = x32.shape
        if tuple(w32.shape) != (width, taps) or tuple(out32.shape) != (m, width) or (bias32 is not None and bias32.numel() != width):
            raise KernelError("conv_tokens: shapes do not fit")
        if bias32 is not None:
            _need(bias32, torch.float32, "conv_tokens bias")
        if taps > 1:
            self._state_row(state, state_off, (taps - 1) * width, "conv_tokens state")
        self._check(self._lib.nib_conv_tokens(
            _ptr(x32), c_int(x32.stride(0)), _ptr(w32), _ptr(bias32), c_int({"none": 0, "silu": 1}[act]), _ptr(state if taps > 1 else None),
            c_longlong(state.stride(0) if taps > 1 else 0), c_int(state_off), _ptr(ctx.q_start), _ptr(ctx.req_index), _ptr(ctx.state_slots),
            _ptr(out32), c_int(out32.stride(0)), c_int(m), c_int(width), c_int(taps), self._stream()), "conv_tokens")

    def conv_tail(self, x32, state, state_off, ctx, taps):
        """The state's history rows become each request's last taps-1 rows of x32 (older rows move up when the step brought
        fewer). Runs after ``conv_tokens`` of the same step has read them."""
        self._rows(x32, torch.float32, "conv_tail x")
        self._state_row(state, state_off, (taps - 1) * x32.shape[1], "conv_tail state")
        self._check(self._lib.nib_conv_tail(_ptr(x32), c_int(x32.stride(0)), _ptr(state), c_longlong(state.stride(0)), c_int(state_off),
                                            _ptr(ctx.q_start), _ptr(ctx.state_slots), c_int(ctx.host.num_requests), c_int(x32.shape[1]),
                                            c_int(taps), self._stream()), "conv_tail")

    def conv_step(self, x32, w32, bias32, act, state, state_off, ctx, out32, taps):
        """``conv_tokens`` followed by ``conv_tail``: the convolution of the step's tokens, then the history moves on. Steps
        in which no request brings more than 16 tokens (a decode step) take one launch for both."""
        if max(ctx.host.q_lens) > 16 or taps > 16:
            self.conv_tokens(x32, w32, bias32, act, state, state_off, ctx, out32, taps)
            if taps > 1:
                self.conv_tail(x32, state, state_off, ctx, taps)
            return
        self._rows(x32, torch.float32, "conv_step x"); self._rows(out32, torch.float32, "conv_step out"); _need(w32, torch.float32, "conv_step w")
        m, width = x32.shape
        if tuple(w32.shape) != (width, taps) or tuple(out32.shape) != (m, width) or (bias32 is not None and bias32.numel() != width):
            raise KernelError("conv_step: shapes do not fit")
        if bias32 is not None:
            _need(bias32, torch.float32, "conv_step bias")
        if taps > 1:
            self._state_row(state, state_off, (taps - 1) * width, "conv_step state")
        self._check(self._lib.nib_conv_step(
            _ptr(x32), c_int(x32.stride(0)), _ptr(w32), _ptr(bias32), c_int({"none": 0, "silu": 1}[act]), _ptr(state if taps > 1 else None),
            c_longlong(state.stride(0) if taps > 1 else 0), c_int(state_off), _ptr(ctx.q_start), _ptr(ctx.state_slots), _ptr(out32),
            c_int(out32.stride(0)), c_int(ctx.host.num_requests), c_int(width), c_int(taps), self._stream()), "conv_step")

    def token_shift(self, h, mu32, state, state_off, ctx, mixes):
        """mixes[s, t] = h[t] + (h[t-1] - h[t]) * mu32[s]; the token before a request's first one in the step is
        ``state[slot, state_off:]``, which then becomes the request's last h."""
        _need(h, None, "token_shift h"); _need(mu32, torch.float32, "token_shift mu"); _need(mixes, h.dtype, "token_shift out")
        m, width = h.shape
        if mu32.dim() != 2 or mu32.shape[1] != width or tuple(mixes.shape) != (mu32.shape[0], m, width):
            raise KernelError("token_shift: shapes do not fit")
        self._state_row(state, state_off, width, "token_shift state")
        self._check(self._lib.nib_token_shift(_ptr(h), _ptr(mu32), c_int(mu32.shape[0]), _ptr(state), c_longlong(state.stride(0)), c_int(state_off),
                                              _ptr(ctx.q_start), _ptr(ctx.req_index), _ptr(ctx.state_slots), _ptr(mixes), c_int(m), c_int(width),
                                              c_int(_DT[h.dtype]), self._stream()), "token_shift")

    def decay_map(self, z32, out32, kind, param):
        """kind 'sigmoid_root': sigmoid(z)^(1/param); 'exp_neg_exp': exp(-exp(z)). Rounded to 32 bits once."""
        self._rows(z32, torch.float32, "decay_map z"); self._rows(out32, torch.float32, "decay_map out")
        if z32.shape != out32.shape:
            raise KernelError("decay_map: shapes differ")
        self._check(self._lib.nib_decay_map(_ptr(z32), c_int(z32.stride(0)), _ptr(out32), c_int(out32.stride(0)), c_int(z32.shape[0]),
                                            c_int(z32.shape[1]), c_int({"sigmoid_root": 0, "exp_neg_exp": 1}[kind]), c_float(param),
                                            self._stream()), "decay_map")

    def step_sizes(self, dt_raw32, dt_bias32, a_log32, dt_out, decay_out):
        """dt_out = softplus(dt_raw32 + dt_bias32), decay_out = exp(-exp(a_log32) * dt_out), per (token, head)."""
        self._rows(dt_raw32, torch.float32, "step_sizes dt"); _need(dt_bias32, torch.float32, "step_sizes bias"); _need(a_log32, torch.float32, "step_sizes A")
        _need(dt_out, torch.float32, "step_sizes out"); _need(decay_out, torch.float32, "step_sizes out")
        m, heads = dt_raw32.shape
        if dt_bias32.numel() != heads or a_log32.numel() != heads or tuple(dt_out.shape) != (m, heads) or tuple(decay_out.shape) != (m, heads):
            raise KernelError("step_sizes: shapes do not fit")
        self._check(self._lib.nib_step_sizes(_ptr(dt_raw32), c_int(dt_raw32.stride(0)), _ptr(dt_bias32), _ptr(a_log32), _ptr(dt_out), _ptr(decay_out),
                                             c_int(m), c_int(heads), self._stream()), "step_sizes")

    # ---- attention with options (attention_flex.cu) --------------------------------------------------------
    def attention_prepare(self, qkv32, q_out, heads, kv_heads, dim, vdim, q_gain32, k_gain32, eps, freq32, rot_dims, ctx,
                          block_table, page_size, k_pages, v_pages, writes, layout="half", unit_norm_after=False,
                          values_are_keys=False, norm_whole=False, v_first32=None, vmix32=None):
        """From the 32-bit rows [q | k | v]: optional per-head RMS norm of q and k (gains of ``dim``), rotation of the first
        ``rot_dims`` elements of every q and k head by position * freq32 (``layout`` 'half': element i with i + rot_dims/2;
        'interleaved': 2i with 2i + 1), with ``unit_norm_after`` every q and k head divided by its root mean square after
        the rotation (no gain), queries into ``q_out`` in the storage type, and with ``writes`` keys and values into their
        pages. With ``values_are_keys`` the rows are [q | k] and a value head is the key head as projected. With
        ``norm_whole`` the gains have the size of the whole projection (heads * dim, kv_heads * dim) and the root mean square
        is taken over all of a token's q (and k) at once. With ``v_first32`` [tokens, kv_heads * vdim] (32-bit rows of any
        stride) a value is written as (1 - vmix32[0]) v + vmix32[0] v_first32."""
        self._rows(qkv32, torch.float32, "attention_prepare qkv"); _need(q_out, None, "attention_prepare q")
        m = qkv32.shape[0]
        if qkv32.shape[1] != (heads + kv_heads) * dim + (0 if values_are_keys else kv_heads * vdim) or tuple(q_out.shape) != (m, heads * dim) \
                or (values_are_keys and vdim != dim):
            raise KernelError("attention_prepare: widths do not fit the head counts")
        flags = {"half": 0, "interleaved": 1}[layout] | (2 if unit_norm_after else 0) | (4 if values_are_keys else 0) | (8 if norm_whole else 0)
        for t, n_heads in ((q_gain32, heads), (k_gain32, kv_heads)):
            if t is not None:
                _need(t, torch.float32, "attention_prepare gain")
                if t.numel() != (n_heads * dim if norm_whole else dim):
                    raise KernelError("attention_prepare: a gain has the size of a head (of the whole projection with norm_whole)")
        ld_first = 0
        if v_first32 is not None:
            self._rows(v_first32, torch.float32, "attention_prepare v_first"); _need(vmix32, torch.float32, "attention_prepare vmix")
            if tuple(v_first32.shape) != (m, kv_heads * vdim) or vmix32.numel() != 1 or values_are_keys:
                raise KernelError("attention_prepare: the values to blend with are [tokens, kv_heads * vdim], the factor one number")
            ld_first = v_first32.stride(0)
        if rot_dims:
            _need(freq32, torch.float32, "attention_prepare freq")
            if freq32.numel() != rot_dims // 2:
                raise KernelError("attention_prepare: one frequency per rotated pair")
        num_pages = bt_stride = 0
        if writes:
            _need(block_table, torch.int32, "block_table", contiguous=False)
            _need(k_pages, q_out.dtype, "k_pages"); _need(v_pages, q_out.dtype, "v_pages")
            if tuple(k_pages.shape[1:]) != (kv_heads, page_size, dim) or tuple(v_pages.shape[1:]) != (kv_heads, page_size, vdim) \
                    or block_table.stride(1) != 1 or v_pages.shape[0] != k_pages.shape[0]:
                raise KernelError("attention_prepare: pages or block table do not fit")
            num_pages, bt_stride = k_pages.shape[0], block_table.stride(0)
        self._check(self._lib.nib_attention_prepare(
            _ptr(qkv32), c_int(qkv32.stride(0)), _ptr(q_out), _ptr(q_gain32), _ptr(k_gain32), c_float(eps), _ptr(freq32 if rot_dims else None),
            c_int(rot_dims), _ptr(ctx.positions), _ptr(ctx.req_index), _ptr(block_table if writes else None), c_int(bt_stride), c_int(page_size),
            _ptr(k_pages if writes else None), _ptr(v_pages if writes else None), c_int(num_pages), c_int(m), c_int(heads), c_int(kv_heads),
            c_int(dim), c_int(vdim), c_int(1 if writes else 0), c_int(_DT[q_out.dtype]), c_int(flags), _ptr(v_first32), c_int(ld_first),
            _ptr(vmix32 if v_first32 is not None else None), self._stream()), "attention_prepare")

    def attention_flex(self, q, out, heads, kv_heads, dim, vdim, scale, softcap, slopes32, window, chunk, out_scale, ctx,
                       block_table, page_size, k_pages, v_pages, sinks32=None):
        """Softmax attention of every token of the step over its request's cached keys: j <= own position, within
        ``window`` (0 = none) and within the own block of ``chunk`` positions (0 = none); score = (q . k) * scale, capped
        by ``softcap`` * tanh(. / softcap) (0 = none), minus slopes32[head] * distance (None = none). ``out``
        [tokens, heads * vdim] in float or the storage type, times ``out_scale``. With ``sinks32`` [heads] the softmax's
        denominator holds exp(sinks32[head]) once more (no key, no value, neither scaled nor capped)."""
        _need(q, None, "attention q"); _need(out, None, "attention out")
        _need(k_pages, q.dtype, "k_pages"); _need(v_pages, q.dtype, "v_pages"); _need(block_table, torch.int32, "block_table", contiguous=False)
        m = q.shape[0]
        if tuple(k_pages.shape[1:]) != (kv_heads, page_size, dim) or tuple(v_pages.shape[1:]) != (kv_heads, page_size, vdim) \
                or q.shape[1] != heads * dim or tuple(out.shape) != (m, heads * vdim) or block_table.stride(1) != 1:
            raise KernelError("attention_flex: shapes do not fit")
        if out.dtype not in (torch.float32, q.dtype):
            raise KernelError("attention_flex: out is float or of the storage type")
        if slopes32 is not None:
            _need(slopes32, torch.float32, "attention slopes")
            if slopes32.numel() != heads:
                raise KernelError("attention_flex: one slope per head")
        if sinks32 is not None:
            _need(sinks32, torch.float32, "attention sinks")
            if sinks32.numel() != heads:
                raise KernelError("attention_flex: one sink per head")
        n_rep = heads // max(1, kv_heads)
        if q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and dim == vdim and slopes32 is None and out_scale == 1.0 \
                and max(ctx.host.q_lens) * n_rep > 64 and not self.options.force_general_attention and not self.options.force_mma_prefill \
                and self._lib.nib_attention_prefill_tc_supported(c_int(heads), c_int(kv_heads), c_int(dim), c_int(page_size), c_int(q.stride(0))) == 1:
            # prompt portions with heads of 64 or 128 (keys and values alike): the tcgen05 kernel's instance with options
            self._check(self._lib.nib_attention_prefill_tc(
                _ptr(q), c_int(q.stride(0)), _ptr(out), _ptr(ctx.q_start), _ptr(ctx.ctx_lens), _ptr(block_table), c_int(block_table.stride(0)),
                c_int(page_size), _ptr(k_pages), _ptr(v_pages), c_int(k_pages.shape[0]), c_int(ctx.host.num_requests), c_int(max(ctx.host.q_lens)),
                c_int(m), c_int(heads), c_int(kv_heads), c_int(dim), c_float(scale), c_int(window), c_float(softcap), c_int(chunk), _ptr(sinks32),
                self._stream()), "attention (options, tcgen05)")
            return
        if q.dtype == torch.bfloat16 and not self.options.force_general_attention and page_size > 0 \
                and self._lib.nib_attention_flex_mma_supported(c_int(heads), c_int(kv_heads), c_int(dim), c_int(vdim), c_int(q.stride(0))) == 1:
            # bfloat16 heads of up to 128 (multiples of 8): tensor cores, prompt portions and decoded tokens alike
            longest, splits, part_o, part_ml = max(ctx.host.q_lens), 1, None, None
            if longest * (heads // kv_heads) <= 64:
                # a step of few tokens per request (decoding): a CTA that walks a long context alone waits for memory
                # tile after tile; two tiles per CTA are both in flight at once
                keys = max(ctx.host.ctx_lens)
                for bound in (window, chunk):
                    keys = min(keys, bound) if bound > 0 else keys
                most = max(1, (4 * max(1, self.sm_count)) // max(1, ctx.host.num_requests * kv_heads))
                splits = self.options.fixed_decode_splits or max(1, min(-(-(keys // 64 + 1) // 2), most, 32))
                if splits > 1:
                    part_o = torch.empty(m * heads * splits * vdim, dtype=torch.float32, device=q.device)
                    part_ml = torch.empty(m * heads * splits * 2, dtype=torch.float32, device=q.device)
                    self.launches += 1
            self._check(self._lib.nib_attention_flex_mma(
                _ptr(q), c_int(q.stride(0)), _ptr(out), c_int(1 if out.dtype == torch.float32 else 0), _ptr(ctx.q_start), _ptr(ctx.ctx_lens),
                _ptr(block_table), c_int(block_table.stride(0)), c_int(page_size), _ptr(k_pages), _ptr(v_pages), c_int(k_pages.shape[0]),
                c_int(ctx.host.num_requests), c_int(max(ctx.host.q_lens)), c_int(heads), c_int(kv_heads), c_int(dim), c_int(vdim), c_float(scale),
                c_float(softcap), _ptr(slopes32), c_int(window), c_int(chunk), c_float(out_scale), c_int(splits), _ptr(part_o), _ptr(part_ml),
                c_int(m), _ptr(sinks32), self._stream()), "attention (options, tensor cores)")
            return
        self._check(self._lib.nib_attention_flex(
            _ptr(q), c_int(q.stride(0)), _ptr(out), c_int(1 if out.dtype == torch.float32 else 0), _ptr(ctx.positions), _ptr(ctx.req_index),
            _ptr(block_table), c_int(block_table.stride(0)), c_int(page_size), _ptr(k_pages), _ptr(v_pages), c_int(k_pages.shape[0]), c_int(m),
            c_int(heads), c_int(kv_heads), c_int(dim), c_int(vdim), c_float(scale), c_float(softcap), _ptr(slopes32), c_int(window), c_int(chunk),
            c_float(out_scale), _ptr(sinks32), c_int(_DT[q.dtype]), self._stream()), "attention (options)")

    # ---- recurrent mixers (recurrent.cu) -------------------------------------------------------------
    def delta_rule_scan(self, r32, k32, v32, a_logit32, w_logit32, state, ctx, o32, heads, d):
        """The generalized delta rule over every request's tokens in order, from and into ``state[slot]``
        ([slots, heads, d (value channel), d (key channel)] floats). r32, k32, v32, a_logit32 are column slices of one
        matrix (equal row strides); o32[t, h, :] = S_t^T r_t."""
        for t, what in ((r32, "r"), (k32, "k"), (v32, "v"), (a_logit32, "a"), (w_logit32, "w"), (o32, "o")):
            self._rows(t, torch.float32, f"delta_rule_scan {what}")
        _need(state, torch.float32, "delta_rule_scan state")
        m = r32.shape[0]
        if any(tuple(t.shape) != (m, heads * d) for t in (r32, k32, v32, a_logit32, w_logit32, o32)) \
                or len({t.stride(0) for t in (r32, k32, v32, a_logit32)}) != 1 or tuple(state.shape[1:]) != (heads, d, d):
            raise KernelError("delta_rule_scan: shapes do not fit")
        work = torch.empty((3, m, heads * d), dtype=torch.float32, device=r32.device)      # decay, unit key, removal per (token, channel)
        self._check(self._lib.nib_delta_rule_scan(
            _ptr(r32), _ptr(k32), _ptr(v32), _ptr(a_logit32), c_int(r32.stride(0)), _ptr(w_logit32), c_int(w_logit32.stride(0)),
            _ptr(state), _ptr(ctx.q_start), _ptr(ctx.state_slots), _ptr(o32), c_int(o32.stride(0)), _ptr(work), c_int(m),
            c_int(ctx.host.num_requests), c_int(heads), c_int(d), self._stream()), "delta_rule_scan")

    def causal_conv(self, x32, w32, bias32, state, hist_row0, ctx, u32, u_blocks, taps, blocks):
        """u = bias + sum_j w[:, j] * x[t - (taps-1-j)] per channel within each request; inputs before the step's first
        token come from ``state[slot, hist_row0 : hist_row0 + taps - 1]``. u32: [tokens, width] floats; u_blocks:
        the same values as [blocks, tokens, width / blocks] in the storage type."""
        self._rows(x32, torch.float32, "causal_conv x"); _need(w32, torch.float32, "causal_conv w"); _need(bias32, torch.float32, "causal_conv bias")
        _need(state, torch.float32, "causal_conv state"); _need(u32, torch.float32, "causal_conv u32"); _need(u_blocks, None, "causal_conv u_blocks")
        m, width = x32.shape
        if tuple(w32.shape) != (width, taps) or state.shape[2] != width or hist_row0 + taps - 1 > state.shape[1] \
                or tuple(u32.shape) != (m, width) or tuple(u_blocks.shape) != (blocks, m, width // blocks):
            raise KernelError("causal_conv: shapes do not fit")
        self._check(self._lib.nib_causal_conv(
            _ptr(x32), c_int(x32.stride(0)), _ptr(w32), _ptr(bias32), _ptr(state), c_int(state.shape[1]), c_int(hist_row0),
            _ptr(ctx.q_start), _ptr(ctx.req_index), _ptr(ctx.state_slots), _ptr(u32), _ptr(u_blocks), c_int(m), c_int(width),
            c_int(taps), c_int(blocks), c_int(_DT[u_blocks.dtype]), self._stream()), "causal_conv")

    def rglru_scan(self, u32, gates32, y_logit32, x32, softplus_lam32, state, ctx, out, taps, blocks):
        """S <- a S + sqrt(1 - a^2) (i * u), a = exp(-8 r softplus(lam)), r | i = sigmoid of a block's gate logits
        (gates32: [blocks, tokens, 2 * width / blocks]); out = S * gelu_tanh(y_logit32). ``state[slot, 0]`` is S;
        rows 1.. become the request's last taps-1 rows of x32."""
        _need(u32, torch.float32, "rglru_scan u"); _need(gates32, torch.float32, "rglru_scan gates"); self._rows(y_logit32, torch.float32, "rglru_scan y")
        self._rows(x32, torch.float32, "rglru_scan x"); _need(softplus_lam32, torch.float32, "rglru_scan lam"); _need(state, torch.float32, "rglru_scan state")
        _need(out, None, "rglru_scan out")
        m, width = u32.shape
        work = torch.empty((3, m, width), dtype=torch.float32, device=u32.device)      # decay, input and gelu per (token, channel)
        if tuple(gates32.shape) != (blocks, m, 2 * (width // blocks)) or tuple(state.shape[1:]) != (taps, width) \
                or tuple(out.shape) != (m, width) or tuple(y_logit32.shape) != (m, width) or tuple(x32.shape) != (m, width):
            raise KernelError("rglru_scan: shapes do not fit")
        self._check(self._lib.nib_rglru_scan(
            _ptr(u32), _ptr(gates32), _ptr(y_logit32), c_int(y_logit32.stride(0)), _ptr(x32), c_int(x32.stride(0)),
            _ptr(softplus_lam32), _ptr(state), _ptr(ctx.q_start), _ptr(ctx.state_slots), _ptr(out), _ptr(work), c_int(m),
            c_int(ctx.host.num_requests), c_int(width), c_int(taps), c_int(blocks), c_int(_DT[out.dtype]), self._stream()), "rglru_scan")

    # ---- attention through a latent (latent_attention.cu) -------------------------------------------
    def latent_store(self, z32, gain32, eps, freq32, mag, ctx, block_table, page_size, pages, rank, rot, layout="interleaved"):
        """Cache rows [rms-normed z[:, :rank] * gain | z[:, rank:] rotated by position * freq32]; ``layout`` 'interleaved':
        pairs (2i, 2i + 1), 'half': pairs (i, i + rot/2)."""
        self._rows(z32, torch.float32, "latent_store z"); _need(gain32, torch.float32, "latent_store gain"); _need(freq32, torch.float32, "latent_store freq")
        _need(pages, None, "latent_store pages"); _need(block_table, torch.int32, "block_table", contiguous=False)
        if z32.shape[1] != rank + rot or tuple(pages.shape[1:]) != (1, page_size, rank + rot) or freq32.numel() != rot // 2 \
                or block_table.stride(1) != 1:
            raise KernelError("latent_store: shapes do not fit")
        self._check(self._lib.nib_latent_store(
            _ptr(z32), c_int(z32.stride(0)), _ptr(gain32), c_float(eps), _ptr(freq32), c_float(mag), _ptr(ctx.positions),
            _ptr(ctx.req_index), _ptr(block_table), c_int(block_table.stride(0)), c_int(page_size), _ptr(pages),
            c_int(pages.shape[0]), c_int(z32.shape[0]), c_int(rank), c_int(rot), c_int(_DT[pages.dtype]), c_int(_LAYOUT[layout]),
            self._stream()), "latent_store")

    def _latent_mma(self, dtype, rank, rot) -> bool:
        """Whether the tensor-core kernels run the attention over rows of ``rank + rot`` elements of ``dtype``."""
        return dtype == torch.bfloat16 and not self.options.force_general_attention \
            and self._lib.nib_latent_attention_mma_supported(c_int(rank), c_int(rot)) == 1

    def latent_query_layout(self, dtype, rank, rot):
        """(elements per (token, head), element type) of the query rows that ``latent_attention`` reads for a cache of
        ``dtype``: floats of rank + rot for the general kernel, bfloat16 rows padded to a multiple of 16 for the
        tensor-core kernels."""
        if self._latent_mma(dtype, rank, rot):
            return self._lib.nib_latent_attention_mma_qwidth(c_int(rank), c_int(rot)), torch.bfloat16
        return rank + rot, torch.float32

    def latent_query(self, q32, w_uk, freq32, mag, positions, qa, heads, dn, rank, rot, layout="interleaved"):
        """qa[t, h] = [W_uk,h^T q32[t, h, :dn] | q32[t, h, dn:] rotated | zeros]; w_uk: [heads * dn, rank] as stored;
        qa: [tokens, heads * width] in the layout ``latent_query_layout`` gives; ``layout``: the rotated pairs, as in
        ``latent_store``."""
        self._rows(q32, torch.float32, "latent_query q"); _need(w_uk, None, "latent_query w_uk"); _need(qa, None, "latent_query qa")
        _need(freq32, torch.float32, "latent_query freq")
        m = q32.shape[0]
        ldq = qa.shape[1] // heads
        if q32.shape[1] != heads * (dn + rot) or tuple(w_uk.shape) != (heads * dn, rank) or qa.shape[0] != m \
                or qa.shape[1] != heads * ldq or ldq < rank + rot:
            raise KernelError("latent_query: shapes do not fit")
        if qa.dtype == torch.bfloat16 and w_uk.dtype == torch.bfloat16 and not self.options.force_simt_gemm \
                and self._lib.nib_head_product_supported(c_int(1), c_int(dn), c_int(rank)) == 1:
            # one small product per head on the tensor cores (the warp-per-row form walks a head's matrix row by row, one
            # round trip to memory each: 40-80 us for the 8 tokens of a decode step at heads of 128)
            self._check(self._lib.nib_head_product_kn(_ptr(q32), c_int(q32.stride(0)), _ptr(w_uk), _ptr(freq32), c_float(mag), _ptr(positions),
                                                      _ptr(qa), c_int(ldq), c_int(m), c_int(heads), c_int(rank), c_int(dn), c_int(rot),
                                                      c_int(_LAYOUT[layout]), self._stream()), "latent_query (tensor cores)")
            return
        self._check(self._lib.nib_latent_query(_ptr(q32), c_int(q32.stride(0)), _ptr(w_uk), _ptr(freq32), c_float(mag), _ptr(positions),
                                               _ptr(qa), c_int(ldq), c_int(_DT[qa.dtype]), c_int(m), c_int(heads), c_int(dn), c_int(rank),
                                               c_int(rot), c_int(_DT[w_uk.dtype]), c_int(_LAYOUT[layout]), self._stream()), "latent_query")

    def latent_attention(self, qa, lat32, ctx, block_table, page_size, pages, heads, rank, rot, scale, window, sink32=None):
        """lat32[t, h] = sum_j softmax_j((qa[t, h] . row_j) * scale) * row_j[:rank] over the cached rows of the token's
        request at positions lo..own (lo = own - window + 1 with a window). bfloat16 rows of a supported width run on
        the tensor cores: the leading requests that bring one token each go to the decode kernel (keys split over
        CTAs), the others to the kernel for prompt portions; everything else runs the general kernel. ``sink32`` (one
        number per head): exp(sink32[h]) is added to the softmax's denominator once, with no value behind it."""
        if sink32 is not None:
            _need(sink32, torch.float32, "latent_attention sink")
            if sink32.numel() != heads:
                raise KernelError("latent_attention: one sink per head")
        _need(qa, None, "latent_attention qa"); _need(lat32, torch.float32, "latent_attention out"); _need(pages, None, "latent_attention pages")
        _need(block_table, torch.int32, "block_table", contiguous=False)
        m = qa.shape[0]
        qw, qdt = self.latent_query_layout(pages.dtype, rank, rot)
        if tuple(qa.shape) != (m, heads * qw) or qa.dtype != qdt or tuple(lat32.shape) != (m, heads * rank) \
                or tuple(pages.shape[1:]) != (1, page_size, rank + rot) or block_table.stride(1) != 1:
            raise KernelError("latent_attention: shapes do not fit")
        bt_stride = block_table.stride(0)
        if qdt == torch.float32:
            self._check(self._lib.nib_latent_attention(
                _ptr(qa), _ptr(lat32), _ptr(ctx.positions), _ptr(ctx.req_index), _ptr(block_table), c_int(bt_stride),
                c_int(page_size), _ptr(pages), c_int(pages.shape[0]), c_int(m), c_int(heads), c_int(rank), c_int(rot), c_float(scale),
                c_int(window), c_int(_DT[pages.dtype]), _ptr(sink32), self._stream()), "latent_attention")
            return
        q_lens, ctx_lens = ctx.host.q_lens, ctx.host.ctx_lens
        n_req = len(q_lens)
        n_dec = 0
        while n_dec < n_req and q_lens[n_dec] == 1:
            n_dec += 1
        tail = (c_int(heads), c_int(rank), c_int(rot), c_float(scale), c_int(window))
        if n_dec:
            keys = max(ctx_lens[:n_dec])
            keys = min(keys, window) if window > 0 else keys
            tiles = -(-keys // 64) + 1
            most = max(1, (4 * self.sm_count) // max(1, n_dec * -(-heads // 16)))
            splits = self.options.fixed_decode_splits or max(1, min(-(-tiles // 2), most, 32))
            part_o = part_ml = None
            if splits > 1:
                part_o = torch.empty(n_dec * heads * splits * 192, dtype=torch.float32, device=qa.device)
                part_ml = torch.empty(n_dec * heads * splits * 2, dtype=torch.float32, device=qa.device)
            self._check(self._lib.nib_latent_attention_mma(
                c_int(1), _ptr(qa), _ptr(lat32), _ptr(ctx.q_start), _ptr(ctx.ctx_lens), _ptr(block_table), c_int(bt_stride),
                c_int(page_size), _ptr(pages), c_int(pages.shape[0]), c_int(n_dec), c_int(1), *tail, c_int(splits),
                _ptr(part_o), _ptr(part_ml), _ptr(sink32), self._stream()), "latent attention decode (mma)")
            if splits > 1:
                self.launches += 1
        if n_dec < n_req:
            # rows of qa and lat32 are addressed through q_start, whose entries count from the step's first row
            self._check(self._lib.nib_latent_attention_mma(
                c_int(0), _ptr(qa), _ptr(lat32), c_void_p(ctx.q_start.data_ptr() + 4 * n_dec), c_void_p(ctx.ctx_lens.data_ptr() + 4 * n_dec),
                c_void_p(block_table.data_ptr() + 4 * n_dec * bt_stride), c_int(bt_stride), c_int(page_size), _ptr(pages),
                c_int(pages.shape[0]), c_int(n_req - n_dec), c_int(max(q_lens[n_dec:])), *tail, c_int(1), _ptr(None), _ptr(None),
                _ptr(sink32), self._stream()), "latent attention prefill (mma)")

    def latent_value(self, lat32, w_uv, out, heads, dv, rank, gate32=None):
        """out[t, h*dv + j] = w_uv[h*dv + j, :] . lat32[t, h, :], times sigmoid(gate32[t, h*dv + j]) with a gate."""
        ldg = 0
        if gate32 is not None:
            self._rows(gate32, torch.float32, "latent_value gate")
            if tuple(gate32.shape) != (lat32.shape[0], heads * dv):
                raise KernelError("latent_value: the gate has the output's shape")
            ldg = gate32.stride(0)
        _need(lat32, torch.float32, "latent_value lat"); _need(w_uv, None, "latent_value w_uv"); self._rows(out, w_uv.dtype, "latent_value out")
        m = lat32.shape[0]
        if tuple(lat32.shape) != (m, heads * rank) or tuple(w_uv.shape) != (heads * dv, rank) or tuple(out.shape) != (m, heads * dv):
            raise KernelError("latent_value: shapes do not fit")
        if w_uv.dtype == torch.bfloat16 and not self.options.force_simt_gemm \
                and self._lib.nib_head_product_supported(c_int(0), c_int(rank), c_int(dv)) == 1:
            self._check(self._lib.nib_head_product_nk(_ptr(lat32), c_int(lat32.stride(0)), _ptr(w_uv), _ptr(None), _ptr(out), c_int(out.stride(0)),
                                                      c_longlong(dv), c_int(0), c_int(m), c_int(heads), c_int(dv), c_int(rank), _ptr(gate32), c_int(ldg),
                                                      self._stream()), "latent_value (tensor cores)")
            return
        self._check(self._lib.nib_latent_value(_ptr(lat32), _ptr(w_uv), _ptr(out), c_int(out.stride(0)), c_int(m), c_int(heads),
                                               c_int(dv), c_int(rank), c_int(_DT[w_uv.dtype]), _ptr(gate32), c_int(ldg), self._stream()), "latent_value")

    def argmax(self, logits, out):
        """First index of each row's maximum. Few rows of a large vocabulary are cut into pieces for many CTAs."""
        _need(logits, torch.float32, "argmax logits"); _need(out, torch.int32, "argmax out")
        rows, vocab = logits.shape
        chunks = min(64, max(1, (2 * self.sm_count) // max(1, rows)), vocab // 2048)
        if chunks > 1 and rows <= 4096:
            self.ensure_workspace(logits.device)
            self._check(self._lib.nib_argmax_chunked(_ptr(logits), c_int(rows), c_int(vocab), _ptr(out), c_int(chunks),
                                                     _ptr(self._ws_argmax), _ptr(self._ws_argmax_counters), self._stream()),
                        "argmax")
            return
        self._check(self._lib.nib_argmax(_ptr(logits), c_int(rows), c_int(vocab), _ptr(out), self._stream()), "argmax")

    def repetition_penalty(self, logits, seen, seen_start, penalty, pending=None):
        """``pending`` [rows] int32 on the device: one more id per row, penalised unless the row's list holds it."""
        _need(logits, torch.float32, "penalty logits"); _need(seen, torch.int32, "seen")
        _need(seen_start, torch.int32, "seen_start"); _need(penalty, torch.float32, "penalty")
        rows, vocab = logits.shape
        if pending is not None:
            _need(pending, torch.int32, "pending tokens")
            if pending.numel() < rows:
                raise KernelError("repetition_penalty: fewer pending tokens than rows")
        self._check(self._lib.nib_repetition_penalty(_ptr(logits), c_int(rows), c_int(vocab), _ptr(seen), _ptr(seen_start),
                                                     _ptr(penalty), _ptr(pending), self._stream()), "repetition_penalty")

    def sample(self, logits, temperature, top_k, top_p, uniform, out):
        _need(logits, torch.float32, "sample logits"); _need(temperature, torch.float32, "temperature")
        _need(top_k, torch.int32, "top_k"); _need(top_p, torch.float32, "top_p")
        _need(uniform, torch.float32, "uniform"); _need(out, torch.int32, "sample out")
        rows, vocab = logits.shape
        self._check(self._lib.nib_sample(_ptr(logits), c_int(rows), c_int(vocab), _ptr(temperature), _ptr(top_k),
                                         _ptr(top_p), _ptr(uniform), _ptr(out), self._stream()), "sample")


# kernel ids of the timeline (common.cuh: NibTraceKernel)
TIMELINE_KERNELS = {1: "embed", 2: "rmsnorm", 3: "rope_store", 4: "gemm_smallm", 5: "gemm_stream", 6: "gemm_tc",
                    7: "attention_decode", 8: "attention_combine", 9: "argmax", 10: "attention_decode_mma",
                    11: "gemm_pair", 12: "attention_prefill"}


def _moe_mode(score: str, renormalize: bool) -> int:
    """The router's options as the kernels' flag word."""
    if score not in ("sigmoid", "softmax"):
        raise KernelError(f"experts: scores are 'sigmoid' or 'softmax', not '{score}'")
    return (1 if score == "softmax" else 0) | (2 if renormalize else 0)


def _cluster_splits(n: int) -> int:
    """The split count the TMA decode kernel takes, at most ``n``: one cluster of 1, 2, 4 or 8 CTAs merges its
    splits in shared memory; beyond that whole clusters of 8, whose results a second kernel merges."""
    return (n // 8) * 8 if n >= 8 else 1 << (max(1, n).bit_length() - 1)


# what the code in the upper half of an error word says about the wait that ran out
_GEMM_TC_ROLES = {1: "copy warp: a stage was never freed", 2: "MMA warp: a stage was never filled",
                  3: "epilogue: the accumulator never arrived", 4: "MMA warp: the accumulator buffer was never drained",
                  5: "pair kernel, copy warp: a stage was never freed", 6: "pair kernel, MMA warp: the accumulator buffer was never drained",
                  7: "pair kernel, MMA warp: a stage was never filled", 8: "pair kernel, epilogue: the accumulator never arrived"}
_ATTN_TC_ROLES = {1: "copy warp: a key/value stage was never freed", 2: "MMA warp: the queries never arrived",
                  3: "MMA warp: keys, values or probabilities never arrived", 4: "softmax warps: scores or outputs never arrived"}
_DECODE_TMA_ROLES = {1: "consumer warps: a page tile never arrived", 2: "copy warp: a stage was never freed"}


def raise_device_errors(words) -> None:
    """``words``: (kernel name, error word, {code: role}) triples; raises one ``KernelError`` naming every
    kernel whose word is not zero, with the role of the wait that ran out and the block it ran in."""
    bad = []
    for name, word, roles in words:
        if word == 0:
            continue
        if word < 0:
            bad.append(f"{name}: the error word could not be read")
            continue
        code, block = word >> 16, word & 0xFFFF
        bad.append(f"{name}: a bounded wait ran out in block {block} ({roles.get(code, f'code {code}')})")
    if bad:
        raise KernelError("a kernel gave up waiting; the results of this run are not to be trusted: " + "; ".join(bad))


_LIBRARY: Optional[Kernels] = None      # the instance that loaded the library; the others share its handle


def load_kernels(options: Optional[KernelOptions] = None, verbose: bool = True) -> Kernels:
    """The kernel library with ``options`` (default: every choice left to the library). The library is built and loaded
    once per process; every call returns an instance of its own, with its own options and scratch memory. Raises if
    there is no CUDA device."""
    global _LIBRARY
    if _LIBRARY is None:
        lib_path = _build.build(verbose=verbose)
        k = Kernels(lib_path)
        if not torch.cuda.is_available():
            raise KernelError("no CUDA device: this engine runs on an NVIDIA B200 (sm_100a) only")
        arch = k.device_arch()
        if arch != 100:
            raise KernelError(f"the kernels are built for sm_100a; this device is sm_{arch}")
        k.sm_count = max(1, k._lib.nib_sm_count())
        _LIBRARY = k
    k = _LIBRARY.with_options(options if options is not None else KernelOptions())
    k._ws_scratch = None
    k.ensure_workspace(torch.device("cuda", torch.cuda.current_device()))
    return k
