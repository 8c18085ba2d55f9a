"""The kernel library as Python sees it: loads ``libnanoinfer_b200.so`` (building it first if needed)
and wraps each exported function. There is no other implementation behind these calls: if the
library cannot be built or loaded, or the device is not a CUDA device, they raise.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from . import build as _build
from ..config.kernel_options import KernelOptions
from ..parts.base import LazyNorm


class KernelError(RuntimeError):
    pass


_DT = {torch.float32: 0, torch.bfloat16: 1}
_EPI = {"store": 0, "add": 1, "f32": 2, "swiglu": 3}


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
                     "nib_gemm_tc_qkv_supported"):
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
    def embed(self, ids, table, out32):
        _need(ids, torch.int32, "embed ids"); _need(table, None, "embed table"); _need(out32, torch.float32, "embed out")
        m, hidden = out32.shape
        self._check(self._lib.nib_embed(_ptr(ids), _ptr(table), _ptr(out32), c_int(m), c_int(hidden),
                                        c_int(table.shape[0]), c_int(_DT[table.dtype]), self._stream()), "embed")

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
                    c_int(m), c_int(heads), c_int(kv_heads), c_int(head_dim), c_float(scale), c_int(window),
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
