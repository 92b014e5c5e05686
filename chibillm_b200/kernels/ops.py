"""The operations the parts are made of, each a launch of a CUDA kernel of this
package.  There is no other implementation behind these calls: a tensor that
is not on a CUDA device, or a library that cannot be built or loaded, raises.

All functions write into tensors the caller provides (so a step allocates
nothing once its workspace exists) and launch on torch's current stream.
"""
from __future__ import annotations

import ctypes
from typing import Dict, Optional

import torch

from . import library
from ..csrc import build

F32, BF16 = 0, 1
_CODES = {torch.float32: F32, torch.bfloat16: BF16}


class KernelError(RuntimeError):
    pass


def _code(t: torch.Tensor) -> int:
    try:
        return _CODES[t.dtype]
    except KeyError:
        raise KernelError(f"element type {t.dtype} is not supported (float32 or bfloat16)") from None


def _need_cuda(*tensors: Optional[torch.Tensor]) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("chibillm_b200 runs on a CUDA device only; got a tensor on "
                              f"'{t.device}' (there is no CPU path)")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _check(status: int, what: str) -> None:
    if status == 0:
        return
    if status == -1:
        raise KernelError(f"{what}: invalid argument")
    if status == -2:
        raise KernelError(f"{what}: sizes outside what the kernel supports")
    raise KernelError(f"{what}: CUDA error {status}")


def _rows_contiguous(t: torch.Tensor, what: str) -> None:
    if t.dim() != 2 or t.stride(1) != 1:
        raise KernelError(f"{what} must be 2-d with contiguous rows, got shape {tuple(t.shape)} "
                          f"strides {t.stride()}")


class PendingSum:
    """The partial sums [splits, M, N] (32-bit) of a matrix product whose K range
    was split over CTAs, waiting for a kernel that adds them up together with what
    follows the product (residual and norm, SwiGLU, per-head norm and rotation).
    The sums live in one of two scratch arrays that split products take in turn,
    so a pending sum is good until two more split products have been started; one
    that is read later than that raises instead of handing out another product's
    numbers."""

    def __init__(self, kernels, partial: torch.Tensor, splits: int, M: int, N: int,
                 turn: int = 0, stamp: Optional[int] = None):
        self.kernels, self._partial, self.splits, self.M, self.N = kernels, partial, splits, M, N
        self._turn, self._stamp = turn, stamp

    @property
    def partial(self) -> torch.Tensor:
        if self._stamp is not None and self.kernels._partial_stamps[self._turn] != self._stamp:
            raise KernelError("the partial sums of this product have been overwritten: a pending product "
                              "must be consumed before two more split products are started")
        return self._partial

    def add_into(self, residual: torch.Tensor) -> None:
        """residual += the product."""
        self.kernels.reduce_residual_rmsnorm(self, residual, None, 0.0, 0.0, None)


class ScaledRows:
    """A norm's output without the factor of each row: ``tensor`` holds
    x * (w + offset) in bfloat16 and ``ssq`` [rows, parts] sums of squares of x, so
    that RMSNorm(x)[m] = tensor[m] * rsqrt(sum(ssq[m]) / n + eps).  The factor
    commutes with a matrix product, and ``linear`` / ``linear_swiglu`` apply it to
    their sums; ``materialise`` applies it in place for any other reader."""

    def __init__(self, kernels, tensor: torch.Tensor, ssq: torch.Tensor, parts: int, eps: float, n: int):
        self.kernels, self.tensor, self.ssq, self.parts, self.eps, self.n = kernels, tensor, ssq, parts, eps, n

    @property
    def shape(self):
        return self.tensor.shape

    @property
    def dtype(self):
        return self.tensor.dtype

    def materialise(self) -> torch.Tensor:
        self.kernels.scale_rows(self)
        return self.tensor


class DeferredProduct:
    """residual += x @ w^T of many rows, not launched yet: the norm that follows
    may have the product write the norm's output as well (``finish_with_norm``);
    anybody else adds it (``add_into``)."""

    def __init__(self, kernels, x: torch.Tensor, w: torch.Tensor):
        self.kernels, self.x, self.w = kernels, x, w

    def add_into(self, residual: torch.Tensor) -> None:
        self.kernels.linear(self.x, self.w, residual, residual=residual)

    def finish_with_norm(self, residual: torch.Tensor, weight: torch.Tensor, eps: float, offset: float,
                         out: torch.Tensor, scaled_ok: bool):
        """Adds the product into ``residual`` and normalises: returns ``out`` (the
        norm's output) or, if the reader takes them, ScaledRows over ``out``."""
        k = self.kernels
        if scaled_ok:
            scaled = k.linear_residual_norm(self.x, self.w, residual, weight, eps, offset, out)
            if scaled is not None:
                return scaled
        self.add_into(residual)
        k.rmsnorm(residual, weight, eps, offset, out)
        return out


_STREAM_SCRATCH: Dict[torch.device, torch.Tensor] = {}

# torch's own fast path to the current stream's handle (a plain integer): the public
# torch.cuda.current_stream() builds a Stream object through several Python layers, a quarter
# of the host time of a step that launches a few hundred kernels
_raw_current_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


class CudaKernels:
    """The one set of operations of the product path."""

    name = "cuda"

    def __init__(self, device: torch.device, timeline: bool = False):
        if not torch.cuda.is_available():
            raise KernelError("no CUDA device is available; chibillm_b200 has no CPU path")
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise KernelError(f"device '{device}' is not a CUDA device; chibillm_b200 has no CPU path")
        # timeline: libraries built with -DCHIBI_TIMELINE, whose CTAs note their times (kernels/timeline.py)
        self.timeline = None
        self._defines = ()
        if timeline:
            from .timeline import DEFINE, Timeline
            self.timeline = Timeline(self.device)
            self._defines = (DEFINE,)
        self.lib = self._load("chibi_kernels")
        self.profiler = None        # a LaunchProfiler while the profiling mode is on
        self._device_index = self.device.index if self.device.index is not None else torch.cuda.current_device()
        self.error = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._error_host: Optional[torch.Tensor] = None
        self.launches = 0           # kernels of this package launched so far
        self.use_tensor_cores = True
        self.tensor_core_calls = 0  # matrix products that ran on the tcgen05 kernel
        self.tcgen05_attention_variant = 0   # 0: chosen by size; 1 / 2: query tiles per CTA (for tests)
        self._scratch_buf: Optional[torch.Tensor] = None
        self.scratch_generation = 0
        self.supports_graphs = True     # every op is a plain launch on the current stream
        self._attention_libs = {}
        self._attention_tc_libs = {}
        self.use_tcgen05_attention = True
        self._partial_bufs = [None, None]
        self._partial_turn = 0
        self._partial_stamps = [0, 0]     # how often each of the two arrays has been handed out
        self._ssq_bufs = [None, None]
        self._ssq_turn = 0
        # Many rows: the product that completes the residual also writes the following RMSNorm's
        # output, up to the factor of each row, which the next product applies to its sums.
        # up to so many rows a product streams the weights once with the rows as the instruction's
        # columns (and its K range split over CTAs); beyond, the kernel for many rows runs
        self.few_rows_max = int(self.lib.chibi_gemm_few_rows_max())
        self.fold_norms = True
        self.fold_heads = True           # many rows: the q | k | v product finishes its heads itself
        # many rows: an activation in the product's epilogue (True), or a kernel of its own after it
        self.fold_activation = False
        # The K range of a product with few rows is split over CTAs.  Their partial sums go through
        # global scratch to a second kernel that also does what follows the product.
        self.fuse_split_products = True
        self.sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count
        # rows of a tile of the experts' products: the plain kernel's and the tensor-core kernel's
        self._expert_tile_rows = (int(self.lib.chibi_expert_tile_rows()),
                                  int(self.lib.chibi_expert_tile_rows_tensor_cores()))
        # the many-row product shares its last, partly filled round of tiles out by K blocks and
        # needs room for one tile of partial sums per SM
        # (one per process, never freed: the library keeps the pointer)
        if self.device not in _STREAM_SCRATCH:
            _STREAM_SCRATCH.clear()
            _STREAM_SCRATCH[self.device] = torch.empty(2 * self.sm_count * 128 * 256, dtype=torch.float32,
                                                       device=self.device)
            scratch = _STREAM_SCRATCH[self.device]
            _check(self.lib.chibi_gemm_set_stream_scratch(_ptr(scratch), scratch.numel()), "stream scratch")

    def enable_profiling(self):
        """Time every launch from now on (kernels/profile.py); returns the profiler.
        Steps are no longer captured into CUDA graphs while this is on."""
        from .profile import LaunchProfiler, ProfiledLibrary
        if self.profiler is None:
            self.profiler = LaunchProfiler()
            self.lib = ProfiledLibrary(self.lib, self.profiler)
            for libs in (self._attention_libs, self._attention_tc_libs):
                for d in list(libs):
                    libs[d] = ProfiledLibrary(libs[d], self.profiler)
            self.supports_graphs = False
        return self.profiler

    def _load(self, name: str, defines=()):
        lib = library.load(name, tuple(defines) + self._defines)
        if self.timeline is not None:
            self.timeline.attach(lib, name)
        return lib

    def _profiled(self, lib):
        if self.profiler is None:
            return lib
        from .profile import ProfiledLibrary
        return ProfiledLibrary(lib, self.profiler)

    def share_out_last_round(self, enabled: bool) -> None:
        """Whether the many-row product deals the K blocks of a thinly filled last round
        of tiles out to all SMs (the default) or computes every tile whole."""
        scratch = _STREAM_SCRATCH[self.device] if enabled else None
        _check(self.lib.chibi_gemm_set_stream_scratch(_ptr(scratch), scratch.numel() if enabled else 0),
               "stream scratch")

    def pairs_of_ctas(self, mode: str = "policy", min_rows: int = 256) -> None:
        """How the many-row product uses pairs of CTAs on tiles of 256 x 256 (tcgen05.mma of 256
        rows issued by one CTA for both): "policy" where that is the fastest cut of the output
        (the default, from ``min_rows`` rows on), "never", or "always" (from 256 rows on, whenever
        the columns come in whole tiles of 256)."""
        _check(self.lib.chibi_gemm_set_pair_tiles({"never": 0, "policy": 1, "always": 2, "always narrow": 3}[mode], int(min_rows)),
               "pairs of CTAs")

    def scale_rows(self, rows: ScaledRows) -> None:
        """rows.tensor *= the factor of each row, in place."""
        t = rows.tensor
        _rows_contiguous(t, "scale_rows")
        self.launches += 1
        _check(self.lib.chibi_scale_rows(_ptr(t), t.shape[0], t.shape[1], t.stride(0), _ptr(rows.ssq), rows.parts,
                                         float(rows.eps), rows.n, self._stream()), "scale_rows")

    def linear_residual_norm(self, x: torch.Tensor, w: torch.Tensor, residual: torch.Tensor,
                             weight: torch.Tensor, eps: float, offset: float,
                             out: torch.Tensor) -> Optional[ScaledRows]:
        """residual += x @ w^T and, from the same kernel, the RMSNorm of the new
        residual without the rows' factor (see ScaledRows).  None if the kernel for
        many rows does not take these shapes; nothing has run then."""
        M, K = x.shape
        N = w.shape[0]
        parts = self.lib.chibi_gemm_bf16_norm_parts(M, N, K)
        if not (self.use_tensor_cores and self.fold_norms and M > self.few_rows_max and parts > 0 and x.dtype == torch.bfloat16
                and w.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and residual.dtype == torch.float32
                and residual.shape == (M, N) and out.shape == (M, N) and weight.shape == (N,)
                and weight.is_contiguous() and weight.dtype in (torch.bfloat16, torch.float32)):
            return None
        _need_cuda(x, w, residual, weight, out)
        for t, what in ((x, "x"), (w, "w"), (residual, "residual"), (out, "out")):
            _rows_contiguous(t, f"linear_residual_norm: {what}")
        ssq = self._ssq_buffer(M * parts)
        norm = library.NormOut(_ptr(weight), _code(weight), float(offset), _ptr(out), out.stride(0), _ptr(ssq),
                               ssq.numel())
        status = self.lib.chibi_gemm_bf16_rows(
            _ptr(x), _ptr(w), _ptr(residual), F32, _ptr(residual), M, N, K, x.stride(0), w.stride(0),
            residual.stride(0), residual.stride(0), 0, None, ctypes.byref(norm), None, _ptr(self.error),
            self._stream())
        if status == -2:
            return None
        _check(status, "linear (+ residual, + norm output)")
        self.launches += 1
        self.tensor_core_calls += 1
        return ScaledRows(self, out, ssq, parts, eps, N)

    def _ssq_buffer(self, floats: int) -> torch.Tensor:
        """Two buffers in turn: the sums of squares of one norm are read while the
        product that follows the next norm already writes its own."""
        self._ssq_turn ^= 1
        buf = self._ssq_bufs[self._ssq_turn]
        if buf is None or buf.numel() < floats:
            buf = torch.empty(max(floats, 1 << 16), dtype=torch.float32, device=self.device)
            self._ssq_bufs[self._ssq_turn] = buf
            self.scratch_generation += 1
        return buf

    def _linear_of_scaled(self, x: ScaledRows, w: torch.Tensor, out: torch.Tensor, swiglu: bool,
                          activation: Optional[str] = None) -> bool:
        """out = (the factor of each row) * (x.tensor @ w^T), with SwiGLU or an
        activation if asked, from the kernel for many rows; False if it does not take
        the shapes."""
        t = x.tensor
        M, K = t.shape
        N = w.shape[0]
        if not (self.use_tensor_cores and M > self.few_rows_max and N % 128 == 0 and w.dtype == torch.bfloat16
                and out.dtype == torch.bfloat16 and w.shape[1] == K
                and out.shape == (M, N // 2 if swiglu else N)):
            return False
        _need_cuda(t, w, out)
        for u, what in ((t, "x"), (w, "w"), (out, "out")):
            _rows_contiguous(u, f"linear: {what}")
        scale = library.RowScale(_ptr(x.ssq), x.parts, float(x.eps), x.n)
        status = self.lib.chibi_gemm_bf16_rows(
            _ptr(t), _ptr(w), _ptr(out), BF16, None, M, N, K, t.stride(0), w.stride(0), out.stride(0), 0,
            1 if swiglu else (2 + self._EPILOGUE_ACTIVATIONS[activation] if activation is not None else 0),
            ctypes.byref(scale), None, None, _ptr(self.error), self._stream())
        if status == -2:
            return False
        _check(status, "linear (rows with a factor)")
        self.launches += 1
        self.tensor_core_calls += 1
        return True

    # ---- the q | k | v product of many rows that finishes its heads itself
    def finishes_heads(self, rows: int, d: int, rotary_dim: int, dtype: torch.dtype) -> bool:
        """Whether ``linear_heads`` takes a step of so many rows with this head size."""
        return bool(self.use_tensor_cores and self.fold_heads and rows > self.few_rows_max and d == 128 and rotary_dim == d
                    and dtype == torch.bfloat16)

    def rope_table(self, positions: torch.Tensor, inv_freq: torch.Tensor, rotary_dim: int,
                   out: torch.Tensor) -> None:
        """out[t] = the cosines, then the sines, of float(positions[t]) * inv_freq[j]."""
        _need_cuda(positions, inv_freq, out)
        T, half = positions.numel(), rotary_dim // 2
        if positions.dtype != torch.int32 or inv_freq.dtype != torch.float32 or inv_freq.numel() < half \
                or out.dtype != torch.float32 or out.shape != (T, 2 * half) or not out.is_contiguous():
            raise KernelError("rope_table: int32 positions, float32 inv_freq and out [T, rotary_dim]")
        self.launches += 1
        _check(self.lib.chibi_rope_table(_ptr(positions), _ptr(inv_freq), T, half, _ptr(out), self._stream()),
               "rope_table")

    def cache_slots(self, positions: torch.Tensor, seq_of_token: torch.Tensor, seq_rows: Optional[torch.Tensor],
                    block_table: torch.Tensor, nkv: int, page_size: int, num_pages: int, d: int,
                    out: torch.Tensor) -> None:
        """out[t] = where token t's key (and value) of kv head 0 lies in a cache
        [pages, nkv, page_size, d], in elements; -1 and a recorded error if its
        block table has no page there."""
        _need_cuda(positions, seq_of_token, seq_rows, block_table, out)
        _rows_contiguous(block_table, "cache_slots: block_table")
        T = positions.numel()
        if out.dtype != torch.int64 or out.numel() != T or not out.is_contiguous():
            raise KernelError("cache_slots: out must be contiguous int64 [T]")
        self.launches += 1
        _check(self.lib.chibi_cache_slots(_ptr(positions), _ptr(seq_of_token), _ptr(seq_rows), _ptr(block_table),
                                          block_table.stride(0), T, nkv, page_size, num_pages, d, _ptr(out),
                                          _ptr(self.error), self._stream()), "cache_slots")

    def linear_heads(self, x, w: torch.Tensor, q_out: torch.Tensor, k_cache: Optional[torch.Tensor],
                     v_cache: Optional[torch.Tensor], q_norm_w: Optional[torch.Tensor],
                     k_norm_w: Optional[torch.Tensor], cos_sin: torch.Tensor, slots: Optional[torch.Tensor],
                     nq: int, nkv: int, d: int, page_size: int, eps: float, norm_offset: float) -> bool:
        """q | k | v = x @ w^T of many rows with every head finished by the product's
        own epilogue: per-head RMSNorm (if weights are given), rotation of the whole
        head with ``cos_sin`` (``rope_table``), query heads to ``q_out``, key and
        value heads to the cache slots ``slots`` (``cache_slots``).  x may be
        ScaledRows.  False if the kernel does not take the shapes; nothing has run then."""
        scale = None
        if isinstance(x, ScaledRows):
            scale = library.RowScale(_ptr(x.ssq), x.parts, float(x.eps), x.n)
            x = x.tensor
        append = k_cache is not None
        T, K = x.shape
        N = w.shape[0]
        if not self.finishes_heads(T, d, d, x.dtype) or w.dtype != torch.bfloat16 or w.shape[1] != K \
                or N != (nq + (2 * nkv if append else 0)) * d or q_out.dtype != torch.bfloat16:
            return False
        for t in (q_norm_w, k_norm_w):
            if t is not None and (t.dtype not in (torch.bfloat16, torch.float32) or t.numel() != d
                                  or not t.is_contiguous()):
                return False
        if (q_norm_w is None) != (k_norm_w is None) or (q_norm_w is not None and q_norm_w.dtype != k_norm_w.dtype):
            return False
        _need_cuda(x, w, q_out, k_cache, v_cache, q_norm_w, k_norm_w, cos_sin, slots)
        _rows_contiguous(x, "linear_heads: x")
        _rows_contiguous(w, "linear_heads: w")
        if q_out.shape != (T, nq * d) or not q_out.is_contiguous() or cos_sin.dtype != torch.float32 \
                or cos_sin.shape != (T, d) or not cos_sin.is_contiguous():
            raise KernelError("linear_heads: q_out [T, nq * d] bfloat16 and cos_sin [T, d] float32")
        if append and (k_cache.dtype != torch.bfloat16 or tuple(k_cache.shape[1:]) != (nkv, page_size, d)
                       or not k_cache.is_contiguous() or v_cache is None or v_cache.shape != k_cache.shape
                       or not v_cache.is_contiguous() or slots is None or slots.dtype != torch.int64
                       or slots.numel() != T):
            raise KernelError("linear_heads: caches [pages, nkv, page_size, d] bfloat16 and int64 slots [T]")
        heads = library.HeadsOut(_ptr(cos_sin), _ptr(slots) if append else None, _ptr(q_out), _ptr(k_cache),
                                 _ptr(v_cache), _ptr(q_norm_w), _ptr(k_norm_w),
                                 _code(q_norm_w) if q_norm_w is not None else F32, nq, nkv if append else 0,
                                 page_size, float(eps), float(norm_offset))
        status = self.lib.chibi_gemm_bf16_rows(
            _ptr(x), _ptr(w), None, BF16, None, T, N, K, x.stride(0), w.stride(0), N, 0, 0,
            ctypes.byref(scale) if scale is not None else None, None, ctypes.byref(heads), _ptr(self.error),
            self._stream())
        if status == -2:
            return False
        _check(status, "linear (q | k | v heads)")
        self.launches += 1
        self.tensor_core_calls += 1
        return True

    def _scratch(self, floats: int) -> torch.Tensor:
        """32-bit scratch for kernels that split a reduction over several CTAs."""
        if self._scratch_buf is None or self._scratch_buf.numel() < floats:
            self._scratch_buf = torch.empty(max(floats, 1 << 22), dtype=torch.float32, device=self.device)
            self.scratch_generation += 1
        return self._scratch_buf

    # ------------------------------------------------------------------ helpers
    def _stream(self) -> int:
        """The handle of this device's current stream (asked for at every launch:
        the caller may be inside a stream capture or a stream context)."""
        if _raw_current_stream is not None:
            return _raw_current_stream(self._device_index)
        return torch.cuda.current_stream(self.device).cuda_stream

    def error_word_async(self) -> None:
        """Starts the copy of the error word to the host; ``check_error_copy`` reads it
        once the caller has waited for an event recorded after this call."""
        if self._error_host is None:
            self._error_host = torch.zeros(1, dtype=torch.int32, pin_memory=True)
        self._error_host.copy_(self.error, non_blocking=True)

    def check_error_copy(self) -> None:
        if self._error_host is not None:
            self._raise_for(int(self._error_host[0]))

    def check_error_word(self) -> None:
        """Synchronises and raises if a kernel met an index outside its tables."""
        self._raise_for(int(self.error.item()))

    def _raise_for(self, code: int) -> None:
        if code:
            self.error.zero_()
            # a shared-out round of tiles that gave up may have left its counters non-zero
            self.lib.chibi_gemm_reset_stream_counters(self._stream())
            what = {1: "a token id outside the vocabulary", 2: "a page id outside the pool (append)",
                    3: "a page id outside the pool (attention)",
                    4: "a block-table update outside the table",
                    5: "a table entry outside its range (an expert, or a token id of a per-layer token input)",
                    11: "a wait that ran out (matrix product: loader)",
                    12: "a wait that ran out (matrix product: tensor-core issuer)",
                    13: "a wait that ran out (matrix product: epilogue)",
                    14: "a wait that ran out (matrix product: accumulator hand-over)",
                    15: "a wait that ran out (matrix product: partial sums of a shared tile)",
                    16: "a wait that ran out (matrix product: slot of a shared tile)",
                    17: "a wait that ran out (matrix product by pairs of CTAs: loader)",
                    18: "a wait that ran out (matrix product by pairs of CTAs: tensor-core issuer)",
                    19: "a wait that ran out (matrix product by pairs of CTAs: epilogue)",
                    20: "a wait that ran out (matrix product by pairs of CTAs: accumulator hand-over)",
                    31: "a wait that ran out (experts' product: loader)",
                    32: "a wait that ran out (experts' product: tensor-core issuer)",
                    33: "a wait that ran out (experts' product: epilogue)",
                    **{c: f"a wait that ran out (tcgen05 attention, point {c})" for c in range(21, 30)}}.get(code, f"code {code}")
            raise KernelError(f"a kernel refused {what}")

    # ------------------------------------------------------------------ ops
    def embed(self, tokens: torch.Tensor, table: torch.Tensor, out: torch.Tensor) -> None:
        _need_cuda(tokens, table, out)
        if tokens.dtype != torch.int32 or not tokens.is_contiguous():
            raise KernelError("embed: tokens must be contiguous int32")
        _rows_contiguous(table, "embed: table")
        if not out.is_contiguous() or out.shape != (tokens.numel(), table.shape[1]):
            raise KernelError("embed: out must be contiguous [tokens, hidden]")
        if not table.is_contiguous():
            raise KernelError("embed: table must be contiguous")
        self.launches += 1
        _check(self.lib.chibi_embed(_ptr(tokens), _ptr(table), _code(table), _ptr(out), _code(out),
                                    tokens.numel(), table.shape[1], table.shape[0],
                                    _ptr(self.error), self._stream()), "embed")

    def rmsnorm(self, x: torch.Tensor, weight: torch.Tensor, eps: float, offset: float,
                out: torch.Tensor) -> None:
        """x, out: [groups, n] (rows may be strided); weight [n]."""
        _need_cuda(x, weight, out)
        _rows_contiguous(x, "rmsnorm: x")
        _rows_contiguous(out, "rmsnorm: out")
        n = x.shape[1]
        if weight.shape != (n,) or not weight.is_contiguous() or out.shape != x.shape:
            raise KernelError(f"rmsnorm: weight {tuple(weight.shape)} / out {tuple(out.shape)} do not "
                              f"match x {tuple(x.shape)}")
        self.launches += 1
        _check(self.lib.chibi_rmsnorm(_ptr(x), _code(x), _ptr(weight), _code(weight), _ptr(out),
                                      _code(out), x.shape[0], n, x.stride(0), out.stride(0),
                                      float(eps), float(offset), self._stream()), "rmsnorm")

    def _partial_buffer(self, floats: int) -> torch.Tensor:
        self._partial_turn ^= 1
        self._partial_stamps[self._partial_turn] += 1
        buf = self._partial_bufs[self._partial_turn]
        if buf is None or buf.numel() < floats:
            buf = torch.empty(max(floats, 1 << 21), dtype=torch.float32, device=self.device)
            self._partial_bufs[self._partial_turn] = buf
            self.scratch_generation += 1
        return buf

    def linear_partial(self, x: torch.Tensor, w: torch.Tensor, max_splits: int = 0) -> Optional[PendingSum]:
        """Start x @ w^T with the K range split over CTAs and leave the partial
        sums for a fused consumer; None if this product is not one that is split
        (then use ``linear``).  ``max_splits``: at most so many splits (a consumer
        that fetches only so many partial sums in one go says so)."""
        if isinstance(x, ScaledRows):
            return None                  # many rows: such a product is not split
        if not (self.use_tensor_cores and self.fuse_split_products and x.is_cuda
                and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16):
            return None
        _rows_contiguous(x, "linear: x")
        _rows_contiguous(w, "linear: w")
        M, K = x.shape
        N = w.shape[0]
        if w.shape[1] != K:
            raise KernelError(f"linear: shapes x {tuple(x.shape)} w {tuple(w.shape)}")
        splits = self.lib.chibi_gemm_bf16_splits_capped(M, N, K, int(max_splits))
        if splits <= 1 or N % 4 != 0:
            return None
        buf = self._partial_buffer(splits * M * N)
        status = self.lib.chibi_gemm_bf16_partial(_ptr(x), _ptr(w), M, N, K, x.stride(0), w.stride(0),
                                                  _ptr(buf), buf.numel(), int(max_splits), _ptr(self.error),
                                                  self._stream())
        if status == -2:
            return None
        _check(status, "linear (split product)")
        self.launches += 1
        self.tensor_core_calls += 1
        return PendingSum(self, buf[:splits * M * N].view(splits, M, N), splits, M, N,
                          self._partial_turn, self._partial_stamps[self._partial_turn])

    @staticmethod
    def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> Optional[torch.Tensor]:
        """[gate; up] rearranged for ``linear_swiglu``: blocks of 64 gate rows, each
        followed by the 64 up rows of the same features.  None if the sizes do not
        allow it (the number of features must be a multiple of 64)."""
        inter, k = gate.shape
        if gate.shape != up.shape or inter % 64 != 0 or k % 8 != 0 or gate.dtype != torch.bfloat16 \
                or up.dtype != torch.bfloat16:
            return None
        return torch.stack([gate.view(inter // 64, 64, k), up.view(inter // 64, 64, k)], dim=1).reshape(2 * inter, k).contiguous()

    def linear_swiglu(self, x: torch.Tensor, w_interleaved: torch.Tensor, out: torch.Tensor) -> bool:
        """out[M, I] = silu(x @ gate^T) * (x @ up^T) in one kernel, with the weights
        as ``interleave_gate_up`` arranges them.  False if the kernel refuses the
        shapes (the caller then takes the two-kernel way)."""
        if isinstance(x, ScaledRows):
            if self._linear_of_scaled(x, w_interleaved, out, swiglu=True):
                return True
            x = x.materialise()
        _need_cuda(x, w_interleaved, out)
        _rows_contiguous(x, "linear_swiglu: x")
        _rows_contiguous(w_interleaved, "linear_swiglu: w")
        _rows_contiguous(out, "linear_swiglu: out")
        M, K = x.shape
        N = w_interleaved.shape[0]
        if w_interleaved.shape[1] != K or out.shape != (M, N // 2) or out.dtype != torch.bfloat16 \
                or x.dtype != torch.bfloat16 or w_interleaved.dtype != torch.bfloat16:
            raise KernelError("linear_swiglu: shapes or element types")
        if not self.use_tensor_cores:
            return False
        pending = self.linear_partial(x, w_interleaved) if M <= self.few_rows_max else None
        if pending is not None or M <= 64:
            if pending is None:
                # a shape whose K range is not split: the whole product, then the same kernel
                # that otherwise adds up the splits (here: one) applies SwiGLU
                buf = self._partial_buffer(M * N)
                self.linear(x, w_interleaved, buf[:M * N].view(M, N))
                pending = PendingSum(self, buf[:M * N].view(1, M, N), 1, M, N, self._partial_turn,
                                     self._partial_stamps[self._partial_turn])
            self.reduce_swiglu(pending, out, interleaved=True)
            return True
        status = self.lib.chibi_gemm_bf16_fused(
            _ptr(x), _ptr(w_interleaved), _ptr(out), BF16, None, M, N, K, x.stride(0),
            w_interleaved.stride(0), out.stride(0), 0, 1, _ptr(self.error), self._stream())
        if status == -2:
            return False
        _check(status, "linear_swiglu")
        self.launches += 1
        self.tensor_core_calls += 1
        return True

    def reduce_residual_rmsnorm(self, pending: PendingSum, residual: torch.Tensor,
                                weight: Optional[torch.Tensor], eps: float, offset: float,
                                out: Optional[torch.Tensor]) -> None:
        """residual += pending; out = RMSNorm(residual) if a weight is given."""
        _need_cuda(residual, weight, out)
        _rows_contiguous(residual, "reduce_residual_rmsnorm: residual")
        if residual.dtype != torch.float32 or residual.shape != (pending.M, pending.N):
            raise KernelError("reduce_residual_rmsnorm: residual must be float32 [M, N]")
        if weight is not None:
            _rows_contiguous(out, "reduce_residual_rmsnorm: out")
            if weight.shape != (pending.N,) or out.shape != residual.shape:
                raise KernelError("reduce_residual_rmsnorm: weight / out shapes")
        status = self.lib.chibi_reduce_residual_rmsnorm(
            _ptr(pending.partial), pending.splits, pending.M, pending.N, _ptr(residual), residual.stride(0),
            _ptr(weight), _code(weight) if weight is not None else F32, _ptr(out),
            _code(out) if out is not None else F32, out.stride(0) if out is not None else 0,
            float(eps), float(offset), self._stream())
        if status == -2:
            # a width the fused kernel does not take: add up, then normalise
            self.launches += 1
            _check(self.lib.chibi_add_into(_ptr(residual), _ptr(pending.partial[0]), F32,
                                           residual.numel(), self._stream()), "add_into")
            for s in range(1, pending.splits):
                self.launches += 1
                _check(self.lib.chibi_add_into(_ptr(residual), _ptr(pending.partial[s]), F32,
                                               residual.numel(), self._stream()), "add_into")
            if weight is not None:
                self.rmsnorm(residual, weight, eps, offset, out)
            return
        self.launches += 1
        _check(status, "reduce_residual_rmsnorm")

    def reduce_swiglu(self, pending: PendingSum, out: torch.Tensor, interleaved: bool = False) -> None:
        """out = silu(gate) * up from the pending [gate | up] product (or, with
        ``interleaved``, from a product with ``interleave_gate_up`` weights)."""
        _need_cuda(out)
        inter = pending.N // 2
        if not out.is_contiguous() or out.shape != (pending.M, inter):
            raise KernelError("reduce_swiglu: out must be contiguous [M, N / 2]")
        self.launches += 1
        _check(self.lib.chibi_reduce_swiglu(_ptr(pending.partial), pending.splits, pending.M, inter,
                                            _ptr(out), _code(out), 1 if interleaved else 0,
                                            self._stream()), "reduce_swiglu")

    def qk_norm_rope_append_partial(self, pending: PendingSum, q_out, k_cache, v_cache, q_norm_w, k_norm_w,
                                    inv_freq, rotary_dim, eps, norm_offset, positions, seq_of_token,
                                    block_table, nq, nkv, d, page_size, seq_rows=None) -> None:
        """qk_norm_rope_append on a pending q | k | v product (bfloat16 outputs)."""
        _need_cuda(q_out, k_cache, v_cache, q_norm_w, k_norm_w, inv_freq, positions, seq_of_token,
                   block_table, seq_rows)
        T = pending.M
        append = k_cache is not None
        tied = append and v_cache is None       # the values are the keys: q | k, keys only
        width = (nq + (1 if tied else 2) * nkv) * d if append else nq * d
        if pending.N != width or q_out.shape != (T, nq * d) or q_out.dtype != torch.bfloat16 \
                or not q_out.is_contiguous():
            raise KernelError("qk_norm_rope_append_partial: shapes")
        if append and (k_cache.dtype != torch.bfloat16 or tuple(k_cache.shape[1:]) != (nkv, page_size, d)
                       or not k_cache.is_contiguous() or not (tied or v_cache.is_contiguous())):
            raise KernelError("qk_norm_rope_append_partial: cache")
        w_type = _code(q_norm_w) if q_norm_w is not None else F32
        self.launches += 1
        _check(self.lib.chibi_qk_norm_rope_append_partial(
            _ptr(pending.partial), pending.splits, T, width, _ptr(q_out), _ptr(k_cache), _ptr(v_cache),
            _ptr(q_norm_w), _ptr(k_norm_w), w_type, _ptr(inv_freq), _ptr(positions), _ptr(seq_of_token),
            _ptr(seq_rows), _ptr(block_table), block_table.stride(0) if append else 0, nq, nkv, d,
            int(rotary_dim), page_size, k_cache.shape[0] if append else 0, float(eps), float(norm_offset),
            (2 if tied else 1) if append else 0, _ptr(self.error), self._stream()), "qk_norm_rope_append_partial")

    def linear(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor,
               residual: Optional[torch.Tensor] = None, defer: bool = False) -> Optional[PendingSum]:
        """out[M, N] = x[M, K] @ w[N, K]^T (+ residual, 32-bit, may alias out).
        With ``defer`` (only together with a residual that aliases out) a split
        product is left pending -- the caller adds it later -- and is returned."""
        if isinstance(x, ScaledRows):
            if residual is None and self._linear_of_scaled(x, w, out, swiglu=False):
                return None
            x = x.materialise()
        if defer and residual is not None and residual is out:
            pending = self.linear_partial(x, w)
            if pending is not None:
                return pending
            if self.use_tensor_cores and self.fold_norms and x.shape[0] > self.few_rows_max and x.dtype == torch.bfloat16 \
                    and w.dtype == torch.bfloat16 and residual.dtype == torch.float32:
                return DeferredProduct(self, x, w)
        _need_cuda(x, w, out, residual)
        _rows_contiguous(x, "linear: x")
        _rows_contiguous(w, "linear: w")
        _rows_contiguous(out, "linear: out")
        M, K = x.shape
        N = w.shape[0]
        if w.shape[1] != K or out.shape != (M, N):
            raise KernelError(f"linear: shapes x {tuple(x.shape)} w {tuple(w.shape)} out {tuple(out.shape)}")
        if residual is not None:
            _rows_contiguous(residual, "linear: residual")
            if residual.dtype != torch.float32 or residual.shape != (M, N):
                raise KernelError("linear: residual must be float32 [M, N]")
        if x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and self.use_tensor_cores:
            splits = self.lib.chibi_gemm_bf16_splits(M, N, K)
            if splits > 0:
                scratch = self._scratch(splits * M * N) if splits > 1 else None
                status = self.lib.chibi_gemm_bf16(
                    _ptr(x), _ptr(w), _ptr(out), _code(out), _ptr(residual), M, N, K, x.stride(0),
                    w.stride(0), out.stride(0), residual.stride(0) if residual is not None else 0,
                    _ptr(scratch), scratch.numel() if scratch is not None else 0, _ptr(self.error),
                    self._stream())
                if status == 0:
                    self.launches += 2 if splits > 1 else 1
                    self.tensor_core_calls += 1
                    return
                if status != -2:
                    _check(status, "linear (tensor cores)")
        self.launches += 1
        _check(self.lib.chibi_gemm_simt(
            _ptr(x), _code(x), _ptr(w), _code(w), _ptr(out), _code(out), _ptr(residual), M, N, K,
            x.stride(0), w.stride(0), out.stride(0),
            residual.stride(0) if residual is not None else 0, self._stream()), "linear")

    def qk_norm_rope_append(self, qkv: torch.Tensor, q_out: torch.Tensor,
                            k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
                            q_norm_w: Optional[torch.Tensor], k_norm_w: Optional[torch.Tensor],
                            inv_freq: Optional[torch.Tensor], rotary_dim: int, eps: float,
                            norm_offset: float, positions: torch.Tensor,
                            seq_of_token: torch.Tensor, block_table: Optional[torch.Tensor],
                            nq: int, nkv: int, d: int, page_size: int,
                            seq_rows: Optional[torch.Tensor] = None) -> None:
        """Per head: RMSNorm (when a weight is given), split-half rotation of the
        first ``rotary_dim`` features, then q -> q_out, k and v -> cache pages.
        qkv: [T, (nq + 2 nkv) d], or [T, nq d] when no cache is given (the layer
        then reads another layer's cache).  Cache: [pages, nkv, page_size, d].
        Sequence s uses row ``seq_rows[s]`` of the block table (row s when None).
        A key cache without a value cache: the values are the keys, qkv is q | k."""
        _need_cuda(qkv, q_out, k_cache, v_cache, q_norm_w, k_norm_w, inv_freq, positions,
                   seq_of_token, block_table, seq_rows)
        _rows_contiguous(qkv, "qk_norm_rope_append: qkv")
        T = qkv.shape[0]
        append = k_cache is not None
        tied = append and v_cache is None
        width = (nq + (1 if tied else 2) * nkv) * d if append else nq * d
        if qkv.shape[1] < width or not q_out.is_contiguous() or q_out.shape != (T, nq * d):
            raise KernelError("qk_norm_rope_append: qkv / q_out shapes")
        if q_out.dtype != qkv.dtype:
            raise KernelError("qk_norm_rope_append: q_out must have qkv's element type")
        if (q_norm_w is None) != (k_norm_w is None):
            raise KernelError("qk_norm_rope_append: give both norm weights or none")
        if rotary_dim and (inv_freq is None or inv_freq.dtype != torch.float32
                           or inv_freq.numel() < rotary_dim // 2):
            raise KernelError("qk_norm_rope_append: inv_freq must hold rotary_dim/2 float32 values")
        num_pages = 0
        table_stride = 0
        if append:
            if (k_cache.dim() != 4 or not k_cache.is_contiguous() or tuple(k_cache.shape[1:]) != (nkv, page_size, d)
                    or not (tied or (k_cache.shape == v_cache.shape and v_cache.is_contiguous()))):
                raise KernelError(f"qk_norm_rope_append: cache shape {tuple(k_cache.shape)}")
            num_pages = k_cache.shape[0]
            _rows_contiguous(block_table, "qk_norm_rope_append: block_table")
            table_stride = block_table.stride(0)
        w_type = _code(q_norm_w) if q_norm_w is not None else F32
        self.launches += 1
        _check(self.lib.chibi_qk_norm_rope_append(
            _ptr(qkv), _code(qkv), qkv.stride(0), _ptr(q_out), _ptr(k_cache), _ptr(v_cache),
            _code(k_cache) if append else F32, _ptr(q_norm_w), _ptr(k_norm_w), w_type,
            _ptr(inv_freq), _ptr(positions), _ptr(seq_of_token), _ptr(seq_rows), _ptr(block_table),
            table_stride, T,
            nq, nkv, d, int(rotary_dim), page_size, num_pages, float(eps), float(norm_offset),
            (2 if tied else 1) if append else 0, _ptr(self.error), self._stream()), "qk_norm_rope_append")

    def attention(self, q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                  out: torch.Tensor, block_table: torch.Tensor, q_start: torch.Tensor,
                  ctx_len: torch.Tensor, seq_of_token: torch.Tensor, positions: torch.Tensor,
                  nq: int, nkv: int, d: int, page_size: int, scale: float,
                  window: Optional[int], max_q_len: int, max_ctx_len: int, min_q_len: int = 0,
                  seq_rows: Optional[torch.Tensor] = None, softcap: Optional[float] = None,
                  distance_bias=None, chunk: Optional[int] = None, value_dim: Optional[int] = None,
                  sink: Optional[torch.Tensor] = None, kv_share: int = 1) -> None:
        """Causal attention of every token over its sequence's pages.  bfloat16
        with a head size that is a multiple of 16 runs on the tensor cores (one
        library per head size, compiled when first needed); everything else, the
        32-bit path included, runs the plain kernel.  ``softcap`` c: a scaled score
        s becomes c * tanh(s / c).  ``distance_bias`` (r1, r2), float32 [nq] each:
        r1[h] * ln(1 + r2[h] * (i - j)) is taken off the score of query i and key j.
        ``v_cache`` may be ``k_cache`` itself (values tied to the keys).  ``chunk`` C: a
        query sees only the keys of its own block of C positions, counted from the
        sequence's start.  ``value_dim``: the size of a value head where it is not d
        (the value cache is [pages, nkv, page, value_dim], out [T, nq * value_dim]);
        such a layer runs its prompt portions on the tensor cores too where both sizes are multiples of
        16, and the plain kernel otherwise.  ``sink``, float32 [nq]: exp(sink[h]) joins the
        softmax's denominator of head h (unscaled, once, with no value).  ``distance_bias``
        (slopes, None): slopes[h] * (i - j) is taken off instead.  ``kv_share`` n: n consecutive
        key heads share one value head (the value cache has nkv / n heads).  ``out`` may be
        float32 whatever q's type; these two run prompt portions on the ``mma.sync`` prompt kernel and
        steps of single tokens on the plain kernel."""
        _need_cuda(q, k_cache, v_cache, out, block_table, q_start, ctx_len, seq_of_token, positions,
                   seq_rows, sink)
        if sink is not None and (sink.dtype != torch.float32 or sink.numel() != nq or not sink.is_contiguous()):
            raise KernelError("attention: the sink is a contiguous float32 [nq] tensor")
        r1 = r2 = None
        if distance_bias is not None:
            r1, r2 = distance_bias
            _need_cuda(r1, r2)
            for r in (r1, r2):
                if r is not None and (r.dtype != torch.float32 or r.numel() != nq or not r.is_contiguous()):
                    raise KernelError("attention: the distance bias is contiguous float32 [nq] tensors")
            if r1 is None:
                raise KernelError("attention: a distance bias needs its first tensor")
        cap = float(softcap) if softcap is not None else 0.0
        if cap < 0.0:
            raise KernelError("attention: the soft cap must be positive")
        T = q.shape[0]
        dv = d if value_dim is None else int(value_dim)
        chunk = int(chunk or 0)
        if chunk < 0:
            raise KernelError("attention: the chunk size must be positive")
        if not q.is_contiguous() or not out.is_contiguous() or q.shape != (T, nq * d) or out.shape != (T, nq * dv):
            raise KernelError("attention: q must be contiguous [T, nq*d] and out [T, nq*value_dim]")
        if out.dtype != q.dtype and out.dtype != torch.float32:
            raise KernelError("attention: out must have q's element type or be float32")
        kv_share = int(kv_share)
        if kv_share < 1 or nkv % kv_share != 0:
            raise KernelError("attention: kv_share must divide the number of key heads")
        if (k_cache.dim() != 4 or v_cache.dim() != 4 or not k_cache.is_contiguous()
                or not v_cache.is_contiguous() or tuple(k_cache.shape[1:]) != (nkv, page_size, d)
                or tuple(v_cache.shape) != (k_cache.shape[0], nkv // kv_share, page_size, dv)):
            raise KernelError(f"attention: cache shapes {tuple(k_cache.shape)} / {tuple(v_cache.shape)}")
        _rows_contiguous(block_table, "attention: block_table")
        tensor_cores = self.use_tensor_cores and q.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16 \
            and d % 16 == 0 and d <= 256
        special = kv_share != 1 or out.dtype != q.dtype or dv != d
        if tensor_cores and special and max_q_len > 1 and dv % 16 == 0 and dv <= 256:
            # value heads of a size of their own, shared by several key heads, or a 32-bit output: the
            # prompt kernel of a library built for (d, dv) takes all sequences of a step that brings a
            # prompt portion; steps of single tokens stay with the plain kernel
            self._attention_mma_prompt(q, k_cache, v_cache, out, block_table, q_start, ctx_len, nq, nkv, d, dv,
                                       page_size, scale, window, max_q_len, seq_rows, cap, r1, r2, chunk, sink,
                                       kv_share)
            return
        if tensor_cores and not special:
            self._attention_mma(q, k_cache, v_cache, out, block_table, q_start, ctx_len, nq, nkv, d,
                                page_size, scale, window, max_q_len, max_ctx_len, min_q_len, seq_rows, cap, r1, r2,
                                chunk, sink)
            return
        self.launches += 1
        _check(self.lib.chibi_attention_generic_shared(
            _ptr(q), _code(q), _ptr(k_cache), _ptr(v_cache), _code(k_cache), _ptr(out), _code(out),
            _ptr(block_table), block_table.stride(0), _ptr(q_start), _ptr(ctx_len),
            _ptr(seq_of_token), _ptr(seq_rows), _ptr(positions), T, nq, nkv, d, dv, page_size,
            k_cache.shape[0], float(scale), int(window or 0), chunk, cap, _ptr(r1), _ptr(r2), _ptr(sink),
            kv_share, _ptr(self.error), self._stream()), "attention")

    def _attention_mma_prompt(self, q, k_cache, v_cache, out, block_table, q_start, ctx_len, nq, nkv, d, dv,
                              page_size, scale, window, max_q_len, seq_rows, softcap, bias_r1, bias_r2, chunk, sink,
                              kv_share) -> None:
        key = d if dv == d else (d, dv)
        lib = self._attention_libs.get(key)
        if lib is None:
            defines = (f"CHIBI_HEAD_DIM={d}",) + ((f"CHIBI_VALUE_DIM={dv}",) if dv != d else ())
            lib = self._load("chibi_attention_mma", defines)
            if lib.chibi_attention_mma_head_dim() != d or lib.chibi_attention_mma_value_dim() != dv:
                raise KernelError(f"the attention library for head sizes {d} / {dv} was built for other sizes")
            lib = self._attention_libs[key] = self._profiled(lib)
        self.launches += 1
        _check(lib.chibi_attention_mma_prompt(
            _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), 1 if out.dtype == torch.float32 else 0,
            _ptr(block_table), block_table.stride(0), _ptr(seq_rows), _ptr(q_start), _ptr(ctx_len), ctx_len.numel(),
            nq, nkv, int(kv_share), page_size, k_cache.shape[0], float(scale), int(window or 0), int(chunk),
            int(max_q_len), float(softcap), _ptr(bias_r1), _ptr(bias_r2), _ptr(sink), _ptr(self.error),
            self._stream()), "attention (tensor cores, prompt)")

    def decode_attention_splits(self, seqs: int, nq: int, nkv: int, max_ctx_len: int) -> int:
        """Key ranges per sequence of the decode attention kernel: as many CTAs as
        are resident at once (two per SM) and no more, so that no CTA waits for a
        second round; at least 128 keys per range (two tiles for each of a CTA's
        four warps) and at most 32 ranges: every range costs its CTA a prologue and
        the merge a partial result to fetch (one sequence of 2,048 keys: 33 ranges
        1.250 ms a step of 12 layers, 16 ranges 1.207; of 8,192 keys: 37 ranges
        1.296, 32 ranges 1.279, 64 ranges 1.374)."""
        ctas = seqs * nkv * ((nq // nkv + 15) // 16)
        slots = 2 * self.sm_count
        if ctas <= slots:
            return max(1, min(slots // ctas, -(-max_ctx_len // 128), 32))
        # More CTAs than slots even with one range each: a last round with a few CTAs in it
        # costs as much as a full one (38 sequences x 8 kv heads = 304 CTAs on 296 slots: 21 %
        # of a step more than 36 sequences).  With s ranges there are ceil(ctas * s / slots)
        # rounds of 1 / s of the keys each, and every CTA pays for its start and for its share
        # of the merge what 0.03 of the keys + 200 keys take (fitted to steps of 12 layers at 38
        # to 128 sequences of 2,048 keys and of 6 layers at 40 to 96 sequences of 8,192, the query
        # rows ready in memory): the s that makes rounds * (1 / s + that) least, more ranges only
        # where they gain a twentieth, at most four, of 512 keys or more.
        start = 0.03 + 200.0 / max(max_ctx_len, 1)
        best, least = 1, -(-ctas // slots) * (1.0 + start)
        for s in range(2, 5):
            if max_ctx_len // s < 512:
                break
            cost = -(-ctas * s // slots) * (1.0 / s + start)
            if cost < 0.95 * least:
                best, least = s, cost
        return best

    def prompt_attention_key_ranges(self, seqs: int, nq: int, nkv: int, max_q_len: int, max_ctx_len: int) -> int:
        """Key ranges per row tile of the tcgen05 prompt attention: 1 unless the step
        has so few query rows that the CTAs (a tile of 128 rows for each kv head and
        sequence) fill half the SMs or less while the context is long; then as many
        ranges as fill the SMs, of at least 512 keys each, at most eight."""
        ctas = -(-max_q_len * (nq // nkv) // 128) * nkv * seqs
        if ctas * 2 > self.sm_count or max_ctx_len < 1024:
            return 1
        return max(1, min(8, self.sm_count // ctas, max_ctx_len // 512))

    def _attention_mma(self, q, k_cache, v_cache, out, block_table, q_start, ctx_len, nq, nkv, d,
                       page_size, scale, window, max_q_len, max_ctx_len, min_q_len, seq_rows,
                       softcap: float = 0.0, bias_r1=None, bias_r2=None, chunk: int = 0, sink=None) -> None:
        lib = self._attention_libs.get(d)
        if lib is None:
            lib = self._load("chibi_attention_mma", (f"CHIBI_HEAD_DIM={d}",))
            if lib.chibi_attention_mma_head_dim() != d:
                raise KernelError(f"the attention library for head size {d} was built for another size")
            lib = self._attention_libs[d] = self._profiled(lib)
        seqs = ctx_len.numel()
        mode = 1 if max_q_len == 1 else (2 if min_q_len > 1 else 3)
        if mode & 2 and self.use_tcgen05_attention and d in build.TCGEN05_ATTENTION_HEAD_DIMS \
                and page_size >= 8 and 128 % page_size == 0:
            # prompt portions on tcgen05; one-token sequences stay with the split-key kernel
            tc = self._attention_tc_libs.get(d)
            if tc is None:
                tc = self._load("chibi_attention_tc", (f"CHIBI_HEAD_DIM={d}",))
                if tc.chibi_attention_tc_head_dim() != d:
                    raise KernelError(f"the tcgen05 attention library for head size {d} was built for another size")
                tc = self._attention_tc_libs[d] = self._profiled(tc)
            kv_splits = self.prompt_attention_key_ranges(seqs, nq, nkv, max_q_len, max_ctx_len)
            part = self._scratch(q.shape[0] * nq * kv_splits * (d + 2)) if kv_splits > 1 else None
            status = tc.chibi_attention_prefill_tc(
                _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(block_table), block_table.stride(0),
                _ptr(seq_rows), _ptr(q_start), _ptr(ctx_len), seqs, nq, nkv, page_size, k_cache.shape[0],
                float(scale), int(window or 0), int(chunk), 1 if mode & 1 else 0, int(max_q_len),
                int(self.tcgen05_attention_variant), kv_splits, _ptr(part),
                part.numel() if part is not None else 0, q.shape[0], float(softcap), _ptr(bias_r1), _ptr(bias_r2),
                _ptr(sink), _ptr(self.error), self._stream())
            if status == 0:
                # (key ranges belong to the kernel with one query tile per CTA, and bring a merge kernel)
                self.launches += 2 if kv_splits > 1 and self.tcgen05_attention_variant != 2 else 1
                mode &= 1
                if mode == 0:
                    return
            elif status != -2:
                _check(status, "attention (tcgen05)")
        splits, scratch = 1, None
        if mode & 1:
            splits = self.decode_attention_splits(seqs, nq, nkv, max_ctx_len)
            if splits > 1:
                scratch = self._scratch(seqs * nq * splits * (d + 2))
        status = lib.chibi_attention_mma(
            _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(block_table), block_table.stride(0),
            _ptr(seq_rows), _ptr(q_start), _ptr(ctx_len), seqs, nq, nkv, page_size, k_cache.shape[0], float(scale),
            int(window or 0), int(chunk), mode, int(max_q_len), splits, _ptr(scratch),
            scratch.numel() if scratch is not None else 0, float(softcap), _ptr(bias_r1), _ptr(bias_r2),
            _ptr(sink), _ptr(self.error), self._stream())
        self.launches += (1 if mode & 1 else 0) + (1 if mode & 1 and splits > 1 else 0) + (1 if mode & 2 else 0)
        _check(status, "attention (tensor cores)")

    def attention_decode_from_partial(self, pending: PendingSum, k_cache: torch.Tensor, v_cache: torch.Tensor,
                                      out: torch.Tensor, block_table: torch.Tensor, q_start: torch.Tensor,
                                      ctx_len: torch.Tensor, nq: int, nkv: int, d: int, page_size: int,
                                      scale: float, window: Optional[int], max_ctx_len: int,
                                      q_norm_w: Optional[torch.Tensor], k_norm_w: Optional[torch.Tensor],
                                      inv_freq: torch.Tensor, rotary_dim: int, eps: float, norm_offset: float,
                                      append: bool, seq_rows: Optional[torch.Tensor] = None) -> bool:
        """Decode attention straight from the pending q | k | v product of a step in
        which every sequence brings one token: the attention kernel adds the partial
        sums, applies the per-head norm and the rotation and appends the new key and
        value itself.  False if the kernel does not take these sizes (the caller then
        runs ``qk_norm_rope_append_partial`` and ``attention``)."""
        if not (self.use_tensor_cores and d == 128 and rotary_dim == d and nq // nkv <= 6
                and k_cache.dtype == torch.bfloat16 and out.dtype == torch.bfloat16):
            return False
        # More CTAs than are resident at once (from 38 sequences of 8 kv heads on): the sequences are
        # then cut into key ranges so that the rounds come out even, and every range's CTA would add
        # up, normalise and rotate the same query rows again; one kernel that leaves them in memory
        # and the attention kernel after it are 1 to 6 % of a step faster (12 layers, 2,048 keys,
        # 38 / 48 / 64 / 96 / 128 sequences: 2.39 / 2.50 / 2.68 / 3.47 / 4.17 -> 2.29 / 2.39 /
        # 2.65 / 3.40 / 4.09 ms).
        if ctx_len.numel() * nkv * ((nq // nkv + 15) // 16) > 2 * self.sm_count:
            return False
        for w in (q_norm_w, k_norm_w):
            if w is not None and w.dtype != torch.bfloat16:
                return False
        _need_cuda(k_cache, v_cache, out, block_table, q_start, ctx_len, seq_rows, q_norm_w, k_norm_w, inv_freq)
        seqs = ctx_len.numel()
        width = (nq + 2 * nkv) * d if append else nq * d
        if pending.M != seqs or pending.N != width or out.shape != (seqs, nq * d) or not out.is_contiguous() \
                or tuple(k_cache.shape[1:]) != (nkv, page_size, d) or not k_cache.is_contiguous() \
                or not v_cache.is_contiguous():
            raise KernelError("attention_decode_from_partial: shapes")
        lib = self._attention_libs.get(d)
        if lib is None:
            lib = self._load("chibi_attention_mma", (f"CHIBI_HEAD_DIM={d}",))
            lib = self._attention_libs[d] = self._profiled(lib)
        splits = self.decode_attention_splits(seqs, nq, nkv, max_ctx_len)
        scratch = self._scratch(seqs * nq * splits * (d + 2)) if splits > 1 else None
        status = lib.chibi_attention_decode_fused(
            _ptr(pending.partial), pending.splits, width, seqs, _ptr(k_cache), _ptr(v_cache), _ptr(out),
            _ptr(block_table), block_table.stride(0), _ptr(seq_rows), _ptr(q_start), _ptr(ctx_len), seqs, nq, nkv,
            page_size, k_cache.shape[0], float(scale), int(window or 0), 0, splits, _ptr(scratch),
            scratch.numel() if scratch is not None else 0, _ptr(q_norm_w), _ptr(k_norm_w), _ptr(inv_freq),
            float(eps), float(norm_offset), 1 if append else 0, _ptr(self.error), self._stream())
        if status == -2:
            return False
        _check(status, "attention (decode, from the partial sums)")
        self.launches += 2 if splits > 1 else 1
        return True

    def apply_table_updates(self, table: torch.Tensor, updates: torch.Tensor, capacity: int) -> None:
        """table[row][index] = page for the (row, index, page) triples that follow
        the count in ``updates`` (int32: [count, row, index, page, ...])."""
        _need_cuda(table, updates)
        if table.dtype != torch.int32 or updates.dtype != torch.int32 or table.dim() != 2 \
                or not table.is_contiguous() or updates.numel() < 1 + 3 * capacity:
            raise KernelError("apply_table_updates: int32 table [rows, blocks] and 1 + 3 * capacity updates")
        self.launches += 1
        _check(self.lib.chibi_apply_table_updates(_ptr(table), table.shape[1], table.shape[0],
                                                  _ptr(updates), int(capacity), _ptr(self.error),
                                                  self._stream()), "apply_table_updates")

    def swiglu(self, gate_up: torch.Tensor, out: torch.Tensor) -> None:
        _need_cuda(gate_up, out)
        if not gate_up.is_contiguous() or not out.is_contiguous() or gate_up.shape[1] != 2 * out.shape[1] \
                or gate_up.shape[0] != out.shape[0]:
            raise KernelError("swiglu: gate_up must be contiguous [T, 2I] and out [T, I]")
        self.launches += 1
        _check(self.lib.chibi_swiglu(_ptr(gate_up), _code(gate_up), _ptr(out), _code(out),
                                     out.shape[0], out.shape[1], self._stream()), "swiglu")

    # ---- parts with a fixed-size state, and the row-wise helpers around them
    def short_conv(self, x: torch.Tensor, weight: torch.Tensor, history: torch.Tensor, out: torch.Tensor,
                   q_start: torch.Tensor, positions: torch.Tensor, state_slots: torch.Tensor, max_q_len: int,
                   weight_t: Optional[torch.Tensor] = None) -> None:
        """out_t = x_t + sum_j weight[:, j] * x_(t - taps + 1 + j) along each sequence of
        the step.  ``history`` [slots, max(taps - 1, 1), D] (x's type, oldest first)
        gives what lies before a sequence's first token of the step and takes the
        sequence's last taps - 1 inputs.  ``weight_t`` (the weight transposed,
        [taps, D]) lets the kernel with 16 bytes of channels per thread run."""
        _need_cuda(x, weight, history, out, q_start, state_slots)
        _rows_contiguous(x, "short_conv: x")
        _rows_contiguous(out, "short_conv: out")
        T, D = x.shape
        taps = weight.shape[1]
        if weight.shape != (D, taps) or weight.dtype != torch.float32 or not weight.is_contiguous() \
                or out.shape != x.shape or out.dtype != x.dtype or history.dtype != x.dtype \
                or not history.is_contiguous() or tuple(history.shape[1:]) != (max(taps - 1, 1), D) \
                or out.data_ptr() == x.data_ptr():
            raise KernelError("short_conv: weight float32 [D, taps], history [slots, taps - 1, D] and out of x's type")
        if weight_t is not None and (weight_t.dtype != torch.float32 or weight_t.shape != (taps, D)
                                     or not weight_t.is_contiguous() or not weight_t.is_cuda):
            raise KernelError("short_conv: weight_t must be the weight transposed, contiguous float32 [taps, D]")
        self.launches += 1
        _check(self.lib.chibi_short_conv(_ptr(x), _code(x), x.stride(0), _ptr(weight), _ptr(weight_t), _ptr(history),
                                         _ptr(out),
                                         out.stride(0), _ptr(q_start), _ptr(state_slots), state_slots.numel(),
                                         int(max_q_len), D, taps, self._stream()), "short_conv")

    def decay_logits(self, low: torch.Tensor, w2t: torch.Tensor, out: torch.Tensor) -> None:
        """out[t] = tanh(low[t]) @ w2t for steps of few tokens: low [T, rank] (rows may be
        strided), w2t float32 [rank, W], out float32 [T, W]."""
        _need_cuda(low, w2t, out)
        _rows_contiguous(low, "decay_logits: low")
        T, rank = low.shape
        if w2t.dtype != torch.float32 or w2t.dim() != 2 or w2t.shape[0] != rank or not w2t.is_contiguous() \
                or out.dtype != torch.float32 or out.shape != (T, w2t.shape[1]) or not out.is_contiguous():
            raise KernelError("decay_logits: w2t float32 [rank, W] and out float32 [T, W]")
        self.launches += 1
        _check(self.lib.chibi_decay_logits(_ptr(low), _code(low), low.stride(0), _ptr(w2t), _ptr(out), T,
                                           w2t.shape[1], rank, self._stream()), "decay_logits")

    def delta_rule(self, proj: torch.Tensor, decay_logits: torch.Tensor, decay_bias: torch.Tensor,
                   removal_bias: torch.Tensor, state: torch.Tensor, o: torch.Tensor, q_start: torch.Tensor,
                   state_slots: torch.Tensor, heads: int, d: int, rank: int, decay_scale: float, key_eps: float,
                   max_q_len: int) -> None:
        """The generalised delta rule over the step's tokens of every sequence.
        ``proj`` [T, 5 * heads * d + rank] holds r | k | v | gate | removal | low;
        ``decay_logits`` float32 [T, heads * d] holds tanh(low) W2^T.  Per head:
        w = exp(-decay_scale * sigmoid(decay_logits + decay_bias)),
        a = sigmoid(removal + removal_bias), u = k / sqrt(sum(k^2) + key_eps);
        S <- diag(w) S - (a u)(u^T S) + k v^T; o = S^T r.  ``state`` [slots, heads, d, d]
        float32 holds S with the value index before the key index."""
        _need_cuda(proj, decay_logits, decay_bias, removal_bias, state, o, q_start, state_slots)
        _rows_contiguous(proj, "delta_rule: proj")
        T = proj.shape[0]
        W = heads * d
        for t, shape, what in ((decay_logits, (T, W), "decay_logits"), (decay_bias, (W,), "decay_bias"),
                               (removal_bias, (W,), "removal_bias"), (o, (T, W), "o")):
            if t.dtype != torch.float32 or tuple(t.shape) != shape or not t.is_contiguous():
                raise KernelError(f"delta_rule: {what} must be contiguous float32 {shape}")
        if proj.shape[1] != 5 * W + rank or state.dtype != torch.float32 or not state.is_contiguous() \
                or tuple(state.shape[1:]) != (heads, d, d):
            raise KernelError("delta_rule: proj [T, 5 * heads * d + rank] and state float32 [slots, heads, d, d]")
        self.launches += 1
        _check(self.lib.chibi_delta_rule(_ptr(proj), _code(proj), proj.stride(0), _ptr(decay_logits),
                                         _ptr(decay_bias), _ptr(removal_bias), _ptr(state), _ptr(o), _ptr(q_start),
                                         _ptr(state_slots), state_slots.numel(), int(max_q_len), heads, d, rank,
                                         float(decay_scale), float(key_eps), self._stream()), "delta_rule")

    def gated_group_norm(self, x: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, eps: float, group: int,
                         out: torch.Tensor) -> None:
        """out = x / sqrt(mean(x^2 over each run of ``group`` features) + eps) * weight * sigmoid(gate)."""
        _need_cuda(x, gate, weight, out)
        _rows_contiguous(gate, "gated_group_norm: gate")
        T, W = x.shape
        if x.dtype != torch.float32 or not x.is_contiguous() or W % group != 0 or gate.shape != x.shape \
                or weight.dtype != torch.float32 or weight.shape != (W,) or not weight.is_contiguous() \
                or out.shape != x.shape or not out.is_contiguous():
            raise KernelError("gated_group_norm: x float32 [T, W], gate [T, W], weight float32 [W], out [T, W]")
        self.launches += 1
        _check(self.lib.chibi_gated_group_norm(_ptr(x), _ptr(gate), _code(gate), gate.stride(0), _ptr(weight),
                                               _ptr(out), _code(out), T, W // group, group, float(eps),
                                               self._stream()), "gated_group_norm")

    def scale(self, x: torch.Tensor, factor: float) -> None:
        """x *= factor, in place (float32)."""
        _need_cuda(x)
        if x.dtype != torch.float32 or not x.is_contiguous():
            raise KernelError("scale: x must be contiguous float32")
        self.launches += 1
        _check(self.lib.chibi_scale(_ptr(x), float(factor), x.numel(), self._stream()), "scale")

    def cast_rows(self, x: torch.Tensor, out: torch.Tensor, activation: Optional[str] = None) -> None:
        """out = x (or act(x)) in out's type; both [rows, n], rows may be strided."""
        _need_cuda(x, out)
        _rows_contiguous(x, "cast_rows: x")
        _rows_contiguous(out, "cast_rows: out")
        if x.shape != out.shape:
            raise KernelError("cast_rows: shapes")
        self.launches += 1
        if activation is not None and activation not in self.ACTIVATIONS:
            raise KernelError(f"cast_rows: activation must be one of {sorted(self.ACTIVATIONS)}")
        _check(self.lib.chibi_cast_rows(_ptr(x), _code(x), x.stride(0), _ptr(out), _code(out), out.stride(0),
                                        x.shape[0], x.shape[1],
                                        self.ACTIVATIONS[activation] if activation is not None else -1,
                                        self._stream()), "cast_rows")

    def add_row_vector(self, acc: torch.Tensor, vec: torch.Tensor) -> None:
        """acc[r, :] += vec for every row (both float32)."""
        _need_cuda(acc, vec)
        _rows_contiguous(acc, "add_row_vector: acc")
        if acc.dtype != torch.float32 or vec.dtype != torch.float32 or vec.shape != (acc.shape[1],) \
                or not vec.is_contiguous():
            raise KernelError("add_row_vector: acc float32 [rows, n] and vec float32 [n]")
        self.launches += 1
        _check(self.lib.chibi_add_row_vector(_ptr(acc), acc.stride(0), _ptr(vec), acc.shape[0], acc.shape[1],
                                             self._stream()), "add_row_vector")

    ACTIVATIONS = {"gelu": 0, "gelu_tanh": 1, "silu": 2, "relu": 3, "tanh": 4, "relu2": 5}

    _EPILOGUE_ACTIVATIONS = {"gelu": 0, "gelu_tanh": 1, "silu": 2, "relu": 3}    # what a product's epilogue takes

    def activation(self, x: torch.Tensor, kind: str) -> None:
        """x = act(x) in place, computed in 32-bit."""
        _need_cuda(x)
        if not x.is_contiguous() or kind not in self.ACTIVATIONS:
            raise KernelError(f"activation: contiguous x and one of {sorted(self.ACTIVATIONS)}")
        self.launches += 1
        _check(self.lib.chibi_activation(_ptr(x), _code(x), x.numel(), self.ACTIVATIONS[kind], self._stream()),
               "activation")

    def linear_activation(self, x, w: torch.Tensor, out: torch.Tensor, kind: str) -> bool:
        """out = act(x @ w^T) with the activation applied to the 32-bit sums: by the
        kernel that adds up a split product (few rows) or in the product's epilogue
        (many rows; x may be ScaledRows).  False if neither takes the shapes;
        nothing has run then."""
        if kind not in self.ACTIVATIONS:
            raise KernelError(f"linear_activation: one of {sorted(self.ACTIVATIONS)}")
        if isinstance(x, ScaledRows):
            return self.fold_activation and kind in self._EPILOGUE_ACTIVATIONS \
                and self._linear_of_scaled(x, w, out, swiglu=False, activation=kind)
        pending = self.linear_partial(x, w)
        if pending is None and not self.fold_activation:
            return False
        if pending is None:
            # many rows: the activation is the product's epilogue
            M, K = x.shape
            N = w.shape[0]
            if not (self.use_tensor_cores and M > 64 and kind in self._EPILOGUE_ACTIVATIONS
                    and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
                    and out.dtype == torch.bfloat16 and w.shape[1] == K and out.shape == (M, N)
                    and x.is_cuda and x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1):
                return False
            status = self.lib.chibi_gemm_bf16_fused(
                _ptr(x), _ptr(w), _ptr(out), BF16, None, M, N, K, x.stride(0), w.stride(0), out.stride(0), 0,
                2 + self._EPILOGUE_ACTIVATIONS[kind], _ptr(self.error), self._stream())
            if status == -2:
                return False
            _check(status, "linear_activation")
            self.launches += 1
            self.tensor_core_calls += 1
            return True
        if not out.is_contiguous() or out.shape != (pending.M, pending.N):
            raise KernelError("linear_activation: out must be contiguous [M, N]")
        self.launches += 1
        _check(self.lib.chibi_reduce_activation(_ptr(pending.partial), pending.splits, pending.M * pending.N,
                                                _ptr(out), _code(out), self.ACTIVATIONS[kind], self._stream()),
               "reduce_activation")
        return True

    # ---- parts of layer_ops.cu
    def heads_rotate_append(self, qkv: torch.Tensor, q_out: torch.Tensor, k_cache: Optional[torch.Tensor],
                            v_cache: Optional[torch.Tensor], inv_freq: Optional[torch.Tensor], rotary_dim: int,
                            amplitude: float, unit_norm: bool, eps: float, positions: torch.Tensor,
                            seq_of_token: torch.Tensor, block_table: Optional[torch.Tensor], nq: int, nkv: int,
                            d: int, dv: int, page_size: int, seq_rows: Optional[torch.Tensor] = None) -> None:
        """Per head of a row q | k | v ([T, nq d + nkv d + nkv dv]; [T, nq d] without a
        cache): rotation of the first ``rotary_dim`` features (cosines and sines times
        ``amplitude``), then, with ``unit_norm``, the head divided by its root mean
        square; q -> q_out, k and v -> cache pages ([pages, nkv, page, d] and [.., dv])."""
        _need_cuda(qkv, q_out, k_cache, v_cache, inv_freq, positions, seq_of_token, block_table, seq_rows)
        _rows_contiguous(qkv, "heads_rotate_append: qkv")
        T = qkv.shape[0]
        append = k_cache is not None
        width = nq * d + (nkv * (d + dv) if append else 0)
        if qkv.shape[1] < width or not q_out.is_contiguous() or q_out.shape != (T, nq * d) or q_out.dtype != qkv.dtype:
            raise KernelError("heads_rotate_append: qkv / q_out shapes or types")
        if rotary_dim and (inv_freq is None or inv_freq.dtype != torch.float32 or inv_freq.numel() < rotary_dim // 2):
            raise KernelError("heads_rotate_append: inv_freq must hold rotary_dim/2 float32 values")
        num_pages = table_stride = 0
        if append:
            if (v_cache is None or not k_cache.is_contiguous() or not v_cache.is_contiguous()
                    or tuple(k_cache.shape[1:]) != (nkv, page_size, d)
                    or tuple(v_cache.shape) != (k_cache.shape[0], nkv, page_size, dv) or v_cache.dtype != k_cache.dtype):
                raise KernelError(f"heads_rotate_append: cache shapes {tuple(k_cache.shape)}")
            num_pages = k_cache.shape[0]
            _rows_contiguous(block_table, "heads_rotate_append: block_table")
            table_stride = block_table.stride(0)
        self.launches += 1
        _check(self.lib.chibi_heads_rotate_append(
            _ptr(qkv), _code(qkv), qkv.stride(0), _ptr(q_out), _ptr(k_cache), _ptr(v_cache),
            _code(k_cache) if append else F32, _ptr(inv_freq), float(amplitude), _ptr(positions), _ptr(seq_of_token),
            _ptr(seq_rows), _ptr(block_table), table_stride, T, nq, nkv, d, dv, int(rotary_dim), page_size, num_pages,
            float(eps), 1 if unit_norm else 0, 1 if append else 0, _ptr(self.error), self._stream()),
            "heads_rotate_append")

    def gated_activation(self, gate_up: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
                         kind: str, interleaved: bool = False) -> None:
        """out = act(gate + b_gate) * (up + b_up); gate_up [T, 2 n] (gate columns first, or,
        ``interleaved``, blocks of 16 gate columns each followed by its 16 up columns),
        bias [2 n] or None."""
        _need_cuda(gate_up, bias, out)
        _rows_contiguous(gate_up, "gated_activation: gate_up")
        T, n = out.shape
        if gate_up.shape != (T, 2 * n) or not out.is_contiguous() or out.dtype != gate_up.dtype \
                or kind not in self.ACTIVATIONS or (bias is not None and (bias.shape != (2 * n,)
                                                                          or not bias.is_contiguous())):
            raise KernelError("gated_activation: shapes, types or activation")
        self.launches += 1
        _check(self.lib.chibi_gated_activation(_ptr(gate_up), _code(gate_up), gate_up.stride(0), _ptr(bias),
                                               _code(bias) if bias is not None else F32, _ptr(out), T, n,
                                               self.ACTIVATIONS[kind], 1 if interleaved else 0, self._stream()),
               "gated_activation")

    def route_words(self, pairs: int, experts: int) -> int:
        """int32 values of the routing scratch for ``pairs`` (token, choice) pairs."""
        tile = self._expert_tile_rows[0]
        return (experts + 1) + 3 * pairs + 2 * ((pairs + tile - 1) // tile + experts)

    # from so many (token, choice) pairs on the experts' products run on tcgen05.  Its tiles of 128 rows
    # are computed whole, also for a decode step's one or two rows, while the mma.sync kernel skips empty
    # row blocks; streaming the weights by TMA wins all the same (8 and 64 tokens, 8 experts of
    # 2,048 x 3,072: 125 / 135 -> 103 / 89 us; of 4,096 x 6,144: 305 / 350 -> 209 / 227 us)
    EXPERTS_TCGEN05_MIN_PAIRS = 1
    use_tcgen05_experts = True

    def expert_tensor_cores(self, dtype: torch.dtype, hidden: int, inner: int) -> bool:
        """Whether ``routed_experts`` runs experts of these sizes on the tensor cores; their
        gate | up matrices are then to be stacked with ``interleave_expert_gate_up``."""
        return self.use_tensor_cores and dtype == torch.bfloat16 and hidden % 32 == 0 and inner % 32 == 0

    def experts_on_tcgen05(self, dtype: torch.dtype, hidden: int, inner: int) -> bool:
        """Whether ``routed_experts`` runs the products of many rows of such experts on tcgen05."""
        return self.expert_tensor_cores(dtype, hidden, inner) and hidden % 64 == 0 and inner % 64 == 0 \
            and self.use_tcgen05_experts

    @staticmethod
    def interleave_expert_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
        """[2 F, D]: blocks of 16 gate rows, each followed by its 16 up rows (F a multiple of 16)."""
        F, D = gate.shape
        return torch.stack([gate.view(F // 16, 16, D), up.view(F // 16, 16, D)], dim=1).reshape(2 * F, D)

    def routed_experts(self, x: torch.Tensor, tokens: torch.Tensor, table: torch.Tensor, gate_up: torch.Tensor,
                       down: torch.Tensor, acc: torch.Tensor, route: torch.Tensor, act: torch.Tensor,
                       y: torch.Tensor, kind: str, weight: float, interleaved: bool = False,
                       sorted_x: Optional[torch.Tensor] = None) -> None:
        """acc[t] += weight * sum over the experts that ``table[tokens[t]]`` names (in the
        table's order) of down_e (act(gate_e x[t]) * (up_e x[t])).  gate_up [E, 2 F, D]
        (gate rows first), down [E, D, F], table int32 [vocab, top]; scratch: route int32
        (``route_words``), act [T top, F] in x's type, y float32 [T top, D].  Four
        launches; nothing is read on the host.  ``interleaved``: gate_up's experts hold
        blocks of 16 gate rows and their 16 up rows (``interleave_expert_gate_up``); with
        bfloat16 and sizes that are multiples of 32 the products then run on the tensor
        cores: with ``sorted_x`` (scratch [T top, D] in x's type), sizes that are multiples
        of 64 on tcgen05 (the rows are first copied into sorted order, which TMA needs), else
        with ``mma.sync``."""
        _need_cuda(x, tokens, table, gate_up, down, acc, route, act, y)
        _rows_contiguous(x, "routed_experts: x")
        _rows_contiguous(acc, "routed_experts: acc")
        T, D = x.shape
        E, F2, _ = gate_up.shape
        F = F2 // 2
        vocab, top = table.shape
        pairs = T * top
        if (gate_up.shape != (E, 2 * F, D) or down.shape != (E, D, F) or not gate_up.is_contiguous()
                or not down.is_contiguous() or down.dtype != gate_up.dtype or table.dtype != torch.int32
                or not table.is_contiguous() or tokens.dtype != torch.int32 or acc.dtype != torch.float32
                or acc.shape != (T, D) or route.dtype != torch.int32 or route.numel() < self.route_words(pairs, E)
                or act.shape != (pairs, F) or act.dtype != x.dtype or not act.is_contiguous()
                or y.shape != (pairs, D) or y.dtype != torch.float32 or not y.is_contiguous()
                or kind not in self.ACTIVATIONS):
            raise KernelError("routed_experts: shapes or types")
        stream = self._stream()
        self.launches += 4
        fast = interleaved and gate_up.dtype == torch.bfloat16 and self.expert_tensor_cores(x.dtype, D, F) \
            and x.stride(0) % 8 == 0
        tile = self._expert_tile_rows[1 if fast else 0]
        flag = 1 if interleaved else 0
        _check(self.lib.chibi_route_by_table(_ptr(tokens), _ptr(table), vocab, top, E, T, tile, _ptr(route),
                                             _ptr(self.error), stream), "routed_experts (route)")
        if fast and sorted_x is not None and pairs >= self.EXPERTS_TCGEN05_MIN_PAIRS \
                and self.experts_on_tcgen05(x.dtype, D, F):
            _need_cuda(sorted_x)
            if sorted_x.shape != (pairs, D) or sorted_x.dtype != x.dtype or not sorted_x.is_contiguous() \
                    or not x.is_contiguous():
                raise KernelError("routed_experts: sorted_x is contiguous [T top, D] of x's type")
            max_tiles = (pairs + tile - 1) // tile + E
            rows = route[E + 1 + 2 * pairs + 2 * max_tiles:E + 1 + 3 * pairs + 2 * max_tiles]
            self.gather_rows(x, rows, sorted_x)
            s1 = self.lib.chibi_expert_rows_tc(_ptr(sorted_x), _ptr(gate_up), _ptr(act), F, _ptr(route), pairs, E,
                                               2 * F, D, 1, self.ACTIVATIONS[kind], _ptr(self.error), stream)
            if s1 == 0:
                _check(self.lib.chibi_expert_rows_tc(_ptr(act), _ptr(down), _ptr(y), D, _ptr(route), pairs, E, D, F, 0,
                                                     0, _ptr(self.error), stream), "routed_experts (down, tcgen05)")
                _check(self.lib.chibi_combine_experts(_ptr(y), _ptr(route), _ptr(acc), acc.stride(0), T, D, top, E,
                                                      float(weight), None, stream), "routed_experts (combine)")
                self.tensor_core_calls += 2
                return
            if s1 != -2:
                _check(s1, "routed_experts (gate | up, tcgen05)")
        _check(self.lib.chibi_expert_rows_gemm(_ptr(x), _code(x), x.stride(0), 1, top, _ptr(gate_up), _code(gate_up),
                                               _ptr(act), F, _ptr(route), pairs, E, F, D, 1, self.ACTIVATIONS[kind],
                                               tile, flag, stream), "routed_experts (gate | up)")
        _check(self.lib.chibi_expert_rows_gemm(_ptr(act), _code(act), F, 0, top, _ptr(down), _code(down), _ptr(y), D,
                                               _ptr(route), pairs, E, D, F, 0, 0, tile, 0, stream),
               "routed_experts (down)")
        if fast:
            self.tensor_core_calls += 2
        _check(self.lib.chibi_combine_experts(_ptr(y), _ptr(route), _ptr(acc), acc.stride(0), T, D, top, E,
                                              float(weight), None, stream), "routed_experts (combine)")

    def combine_experts(self, y: torch.Tensor, route: torch.Tensor, acc: torch.Tensor, top: int, experts: int,
                        weight: float) -> None:
        """acc[t] += weight * sum over the token's choices s (in their order) of
        y[row_of_pair[t top + s]]; ``route`` is laid out as ``routed_experts`` lays it out
        (offsets [experts + 1] | pair_of_row [pairs] | row_of_pair [pairs] | ...)."""
        _need_cuda(y, route, acc)
        T, D = acc.shape
        if y.shape != (T * top, D) or y.dtype != torch.float32 or not y.is_contiguous() or acc.dtype != torch.float32 \
                or route.dtype != torch.int32 or route.numel() < experts + 1 + 2 * T * top:
            raise KernelError("combine_experts: shapes or types")
        _rows_contiguous(acc, "combine_experts: acc")
        self.launches += 1
        _check(self.lib.chibi_combine_experts(_ptr(y), _ptr(route), _ptr(acc), acc.stride(0), T, D, top, experts,
                                              float(weight), None, self._stream()), "combine_experts")

    # ---- parts of mixer_ops.cu
    def norm_rows(self, y: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], eps: float, offset: float,
                  centered: bool, residual: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> None:
        """v = norm(y) * (weight + offset) + bias over the rows of the float32 y [T, n]:
        ``centered`` takes the mean off first and divides by the root of the mean squared
        deviation + eps (layer norm), else by the root of the mean square + eps.  With
        ``residual`` (float32 [T, n]) residual += v and ``out``, if given, takes the new
        residual in its own type; without it ``out`` takes v."""
        _need_cuda(y, weight, bias, residual, out)
        if y.dim() != 2 or y.dtype != torch.float32 or not y.is_contiguous():
            raise KernelError("norm_rows: y is contiguous float32 [T, n]")
        T, n = y.shape
        if weight.shape != (n,) or not weight.is_contiguous() or (bias is not None and (
                bias.shape != (n,) or bias.dtype != weight.dtype or not bias.is_contiguous())):
            raise KernelError("norm_rows: weight and bias are contiguous [n] of one type")
        for t, what in ((residual, "residual"), (out, "out")):
            if t is not None and (t.shape != (T, n) or not t.is_contiguous()):
                raise KernelError(f"norm_rows: {what} is contiguous [T, n]")
        if residual is None and out is None:
            raise KernelError("norm_rows: nowhere to write")
        if residual is not None and residual.dtype != torch.float32:
            raise KernelError("norm_rows: the residual is float32")
        self.launches += 1
        _check(self.lib.chibi_norm_rows(_ptr(y), _ptr(weight), _ptr(bias), _code(weight), float(eps), float(offset),
                                        1 if centered else 0, _ptr(residual), _ptr(out),
                                        _code(out) if out is not None else F32, T, n, self._stream()), "norm_rows")

    def token_shift(self, x: torch.Tensor, mix: torch.Tensor, state: torch.Tensor, q_start: torch.Tensor,
                    seq_of_token: torch.Tensor, state_slots: torch.Tensor, out: torch.Tensor) -> None:
        """out[t] = x[t] + (x[t - 1] - x[t]) * mix for the float32 x [T, n]; the token before a
        sequence's first of this step is ``state[slot]`` (float32 [slots, n]), which then
        takes the sequence's last x of this step."""
        _need_cuda(x, mix, state, q_start, seq_of_token, state_slots, out)
        T, n = x.shape
        if (x.dtype != torch.float32 or not x.is_contiguous() or mix.dtype != torch.float32 or mix.shape != (n,)
                or state.dtype != torch.float32 or state.dim() != 2 or state.shape[1] != n or not state.is_contiguous()
                or out.shape != (T, n) or not out.is_contiguous()):
            raise KernelError("token_shift: shapes or types")
        self.launches += 1
        _check(self.lib.chibi_token_shift(_ptr(x), _ptr(mix), _ptr(state), _ptr(q_start), _ptr(seq_of_token),
                                          _ptr(state_slots), _ptr(out), _code(out), T, n, self._stream()),
               "token_shift")

    def latent_prepare(self, proj: torch.Tensor, cq: torch.Tensor, k_cache: Optional[torch.Tensor],
                       q_norm: torch.Tensor, kv_norm: Optional[torch.Tensor], eps: float,
                       inv_freq: Optional[torch.Tensor], q_rank: int, kv_rank: int, rot: int, positions: torch.Tensor,
                       seq_of_token: torch.Tensor, block_table: Optional[torch.Tensor], page_size: int,
                       seq_rows: Optional[torch.Tensor] = None) -> None:
        """From rows c_q | c | k_rot ([T, q_rank + kv_rank + rot]; [T, q_rank] without a
        cache): cq = RMSNorm(c_q) * q_norm; the cache row of the token's position
        ([pages, 1, page, rot + kv_rank]) takes the rotated k_rot, then RMSNorm(c) * kv_norm."""
        _need_cuda(proj, cq, k_cache, q_norm, kv_norm, inv_freq, positions, seq_of_token, block_table, seq_rows)
        _rows_contiguous(proj, "latent_prepare: proj")
        T = proj.shape[0]
        append = k_cache is not None
        if proj.shape[1] < q_rank + (kv_rank + rot if append else 0) or cq.shape != (T, q_rank) \
                or not cq.is_contiguous() or cq.dtype != proj.dtype or q_norm.dtype != torch.float32 \
                or q_norm.numel() != q_rank:
            raise KernelError("latent_prepare: shapes or types")
        num_pages = table_stride = 0
        if append:
            if (tuple(k_cache.shape[1:]) != (1, page_size, rot + kv_rank) or not k_cache.is_contiguous()
                    or kv_norm is None or kv_norm.dtype != torch.float32 or kv_norm.numel() != kv_rank
                    or inv_freq is None or inv_freq.dtype != torch.float32 or inv_freq.numel() < rot // 2):
                raise KernelError("latent_prepare: cache, norm weight or frequencies")
            num_pages = k_cache.shape[0]
            _rows_contiguous(block_table, "latent_prepare: block_table")
            table_stride = block_table.stride(0)
        self.launches += 1
        _check(self.lib.chibi_latent_prepare(
            _ptr(proj), _code(proj), proj.stride(0), _ptr(cq), _ptr(k_cache), _code(k_cache) if append else F32,
            _ptr(q_norm), _ptr(kv_norm), float(eps), _ptr(inv_freq), q_rank, kv_rank, rot, _ptr(positions),
            _ptr(seq_of_token), _ptr(seq_rows), _ptr(block_table), table_stride, page_size, num_pages, T,
            _ptr(self.error), self._stream()), "latent_prepare")

    def qkv_bias_norm_append(self, proj: torch.Tensor, q_out: torch.Tensor, k_cache: Optional[torch.Tensor],
                             v_cache: Optional[torch.Tensor], bias: Optional[torch.Tensor],
                             q_norm: Optional[torch.Tensor], k_norm: Optional[torch.Tensor], eps: Optional[float],
                             inv_freq: Optional[torch.Tensor], rot: int, positions: torch.Tensor,
                             seq_of_token: torch.Tensor, block_table: Optional[torch.Tensor], nq: int, nkv: int, d: int,
                             dv: int, page_size: int, seq_rows: Optional[torch.Tensor] = None) -> None:
        """From rows q | k | v | ... ([T, >= nq d + nkv d + nkv dv]; q only without a
        cache): + bias (float32, as wide as what is read), q and k each divided by the root
        mean square of their WHOLE width and multiplied by q_norm / k_norm (float32; None:
        no norm), the first ``rot`` features of every head rotated; q -> q_out, k and v ->
        cache pages ([pages, nkv, page, d] and [.., dv])."""
        _need_cuda(proj, q_out, k_cache, v_cache, bias, q_norm, k_norm, inv_freq, positions, seq_of_token,
                   block_table, seq_rows)
        _rows_contiguous(proj, "qkv_bias_norm_append: proj")
        T = proj.shape[0]
        append = k_cache is not None
        width = nq * d + (nkv * (d + dv) if append else 0)
        if proj.shape[1] < width or q_out.shape != (T, nq * d) or not q_out.is_contiguous() or q_out.dtype != proj.dtype:
            raise KernelError("qkv_bias_norm_append: proj / q_out shapes or types")
        for t, n in ((bias, width), (q_norm, nq * d), (k_norm, nkv * d)):
            if t is not None and (t.dtype != torch.float32 or t.numel() < n or not t.is_contiguous()):
                raise KernelError("qkv_bias_norm_append: bias and norm weights are contiguous float32")
        if rot and (inv_freq is None or inv_freq.dtype != torch.float32 or inv_freq.numel() < rot // 2):
            raise KernelError("qkv_bias_norm_append: inv_freq must hold rot/2 float32 values")
        num_pages = table_stride = 0
        if append:
            if (v_cache is None or not k_cache.is_contiguous() or not v_cache.is_contiguous()
                    or tuple(k_cache.shape[1:]) != (nkv, page_size, d)
                    or tuple(v_cache.shape) != (k_cache.shape[0], nkv, page_size, dv) or v_cache.dtype != k_cache.dtype
                    or (q_norm is not None and k_norm is None)):
                raise KernelError(f"qkv_bias_norm_append: cache shapes {tuple(k_cache.shape)}")
            num_pages = k_cache.shape[0]
            _rows_contiguous(block_table, "qkv_bias_norm_append: block_table")
            table_stride = block_table.stride(0)
        self.launches += 1
        _check(self.lib.chibi_qkv_bias_norm_append(
            _ptr(proj), _code(proj), proj.stride(0), _ptr(q_out), _ptr(k_cache), _ptr(v_cache),
            _code(k_cache) if append else F32, _ptr(bias), _ptr(q_norm), _ptr(k_norm), float(eps or 0.0),
            _ptr(inv_freq), int(rot), _ptr(positions), _ptr(seq_of_token), _ptr(seq_rows), _ptr(block_table),
            table_stride, nq, nkv, d, dv, page_size, num_pages, T, _ptr(self.error), self._stream()),
            "qkv_bias_norm_append")

    def sigmoid_gate(self, x: torch.Tensor, gate: torch.Tensor) -> None:
        """x *= sigmoid(gate), in place; x contiguous [T, n], gate [T, n] with contiguous rows."""
        _need_cuda(x, gate)
        _rows_contiguous(gate, "sigmoid_gate: gate")
        if not x.is_contiguous() or gate.shape != x.shape or gate.dtype != x.dtype:
            raise KernelError("sigmoid_gate: shapes or types")
        self.launches += 1
        _check(self.lib.chibi_sigmoid_gate(_ptr(x), _ptr(gate), _code(x), gate.stride(0), x.shape[0], x.shape[1],
                                           self._stream()), "sigmoid_gate")

    def recurrence_gates(self, proj: torch.Tensor, bias: torch.Tensor, floor: torch.Tensor, out: torch.Tensor,
                         kw: int) -> None:
        """From rows q | f | v ([T, 2 kw + vw]): out (float32, same shape) = silu(q) |
        floor + (1 - floor) * sigmoid(f + bias) | v."""
        _need_cuda(proj, bias, floor, out)
        _rows_contiguous(proj, "recurrence_gates: proj")
        T, w = proj.shape
        vw = w - 2 * kw
        if vw <= 0 or out.shape != (T, w) or out.dtype != torch.float32 or not out.is_contiguous() \
                or bias.dtype != torch.float32 or floor.dtype != torch.float32 or bias.numel() != kw \
                or floor.numel() != kw:
            raise KernelError("recurrence_gates: shapes or types")
        self.launches += 1
        _check(self.lib.chibi_recurrence_gates(_ptr(proj), _code(proj), proj.stride(0), _ptr(bias), _ptr(floor),
                                               _ptr(out), T, kw, vw, self._stream()), "recurrence_gates")

    def gated_recurrence(self, qfv: torch.Tensor, state: torch.Tensor, o: torch.Tensor, q_start: torch.Tensor,
                         state_slots: torch.Tensor, heads: int, d: int, e: int, max_q_len: int = 0) -> None:
        """Per sequence and head, over the step's tokens in order: S <- diag(f) S + (1 - f) v^T,
        o = S^T q, with q | f | v the float32 rows of ``qfv`` [T, 2 heads d + heads e] as
        ``recurrence_gates`` makes them and S = state[slot, head] (float32 [slots, heads, d, e]),
        read at the start and written back at the end.  o: float32 [T, heads e]."""
        _need_cuda(qfv, state, o, q_start, state_slots)
        T = qfv.shape[0]
        if (qfv.dtype != torch.float32 or not qfv.is_contiguous() or qfv.shape[1] != heads * (2 * d + e)
                or state.dtype != torch.float32 or tuple(state.shape[1:]) != (heads, d, e) or not state.is_contiguous()
                or o.shape != (T, heads * e) or o.dtype != torch.float32 or not o.is_contiguous()):
            raise KernelError("gated_recurrence: shapes or types")
        self.launches += 1
        _check(self.lib.chibi_gated_recurrence(_ptr(qfv), _ptr(state), _ptr(o), _ptr(q_start), _ptr(state_slots),
                                               q_start.numel() - 1, heads, d, e, self._stream()), "gated_recurrence")

    def router_top(self, logits: torch.Tensor, chosen: torch.Tensor, share: torch.Tensor) -> None:
        """chosen[t] (int32 [T, top]) = the experts with the largest logits[t] (float32 [T, E]),
        largest first, ties to the lower number; share[t] = softmax over those logits."""
        _need_cuda(logits, chosen, share)
        _rows_contiguous(logits, "router_top: logits")
        T, E = logits.shape
        top = chosen.shape[1]
        if logits.dtype != torch.float32 or chosen.dtype != torch.int32 or share.dtype != torch.float32 \
                or chosen.shape != (T, top) or share.shape != (T, top) or not chosen.is_contiguous() \
                or not share.is_contiguous() or not (0 < top <= E):
            raise KernelError("router_top: shapes or types")
        self.launches += 1
        _check(self.lib.chibi_router_top(_ptr(logits), logits.stride(0), _ptr(chosen), _ptr(share), T, E, top,
                                         self._stream()), "router_top")

    def chosen_experts(self, x: torch.Tensor, chosen: torch.Tensor, share: torch.Tensor, up: torch.Tensor,
                       down: torch.Tensor, acc: torch.Tensor, route: torch.Tensor, act: torch.Tensor, y: torch.Tensor,
                       kind: str, sorted_x: Optional[torch.Tensor] = None, gated: bool = False,
                       interleaved: bool = False, identity: int = 0) -> None:
        """acc[t] += sum over s of share[t, s] * down_e (act(up_e x[t])), e = chosen[t, s]; up
        [E, F, D], down [E, D, F]; scratch as for ``routed_experts``.  The (token, choice)
        pairs are sorted by expert on the device and the two products run over tiles of one
        expert's rows; nothing is read on the host.  ``gated``: ``up`` is [E, 2 F, D], an
        expert's gate rows followed by its up rows (``interleaved``: in blocks of 16, as
        ``interleave_expert_gate_up`` lays them), and an expert is down(act(gate x) * (up x)).
        ``identity`` n > 0: choice E - 1 names the experts that return their input (times the
        share); the last of the E stacked matrices is a stand-in that is never read, and the
        bucket of these choices gets no tiles: its rows take the tokens' inputs instead."""
        _need_cuda(x, chosen, share, up, down, acc, route, act, y)
        _rows_contiguous(x, "chosen_experts: x")
        _rows_contiguous(acc, "chosen_experts: acc")
        T, D = x.shape
        E, F, _ = up.shape
        if gated:
            F //= 2
        top = chosen.shape[1]
        pairs = T * top
        if (up.shape != (E, (2 if gated else 1) * F, D) or down.shape != (E, D, F) or not up.is_contiguous() or not down.is_contiguous()
                or down.dtype != up.dtype or chosen.dtype != torch.int32 or chosen.shape != (T, top)
                or not chosen.is_contiguous() or share.shape != (T, top) or share.dtype != torch.float32
                or not share.is_contiguous() or acc.dtype != torch.float32 or acc.shape != (T, D)
                or route.dtype != torch.int32 or route.numel() < self.route_words(pairs, E)
                or act.shape != (pairs, F) or act.dtype != x.dtype or not act.is_contiguous()
                or y.shape != (pairs, D) or y.dtype != torch.float32 or not y.is_contiguous()
                or kind not in self.ACTIVATIONS):
            raise KernelError("chosen_experts: shapes or types")
        stream = self._stream()
        self.launches += 4
        # as ``routed_experts``: bfloat16 experts of sizes that are multiples of 32 run on the tensor cores
        # (tiles of 128 rows; multiples of 64: tcgen05), everything else the plain kernel
        fast = up.dtype == torch.bfloat16 and self.expert_tensor_cores(x.dtype, D, F) and x.stride(0) % 8 == 0 \
            and (interleaved or not gated)
        if gated and interleaved and not fast:
            raise KernelError("chosen_experts: interleaved gate and up rows are for the tensor-core kernels")
        tile = self._expert_tile_rows[1 if fast else 0]
        code = self.ACTIVATIONS[kind]
        first, rows_up, flag = (1, 2 * F, 1 if interleaved else 0) if gated else (2, F, 0)
        if identity:
            self.launches += 1          # (the choices come clamped to E - 1: ``router_choose``'s ``last_choice``)
        _check(self.lib.chibi_route_by_table_open(None, _ptr(chosen), T, top, E, T, tile, E - 1 if identity else E,
                                                  _ptr(route), _ptr(self.error), stream), "chosen_experts (route)")
        if identity:
            max_tiles = (pairs + tile - 1) // tile + E
            _check(self.lib.chibi_identity_rows(_ptr(x), _code(x), x.stride(0), _ptr(route), _ptr(y), pairs, E, E - 1,
                                                max_tiles, D, stream), "chosen_experts (identity rows)")
        if fast and sorted_x is not None and pairs >= self.EXPERTS_TCGEN05_MIN_PAIRS \
                and self.experts_on_tcgen05(x.dtype, D, F):
            _need_cuda(sorted_x)
            if sorted_x.shape != (pairs, D) or sorted_x.dtype != x.dtype or not sorted_x.is_contiguous() \
                    or not x.is_contiguous():
                raise KernelError("chosen_experts: sorted_x is contiguous [T top, D] of x's type")
            max_tiles = (pairs + tile - 1) // tile + E
            rows = route[E + 1 + 2 * pairs + 2 * max_tiles:E + 1 + 3 * pairs + 2 * max_tiles]
            self.gather_rows(x, rows, sorted_x)
            s1 = self.lib.chibi_expert_rows_tc(_ptr(sorted_x), _ptr(up), _ptr(act), F, _ptr(route), pairs, E, rows_up, D,
                                               first, code, _ptr(self.error), stream)
            if s1 == 0:
                _check(self.lib.chibi_expert_rows_tc(_ptr(act), _ptr(down), _ptr(y), D, _ptr(route), pairs, E, D, F, 0,
                                                     0, _ptr(self.error), stream), "chosen_experts (down, tcgen05)")
                _check(self.lib.chibi_combine_experts(_ptr(y), _ptr(route), _ptr(acc), acc.stride(0), T, D, top, E,
                                                      1.0, _ptr(share), stream), "chosen_experts (combine)")
                self.tensor_core_calls += 2
                return
            if s1 != -2:
                _check(s1, "chosen_experts (up, tcgen05)")
        _check(self.lib.chibi_expert_rows_gemm(_ptr(x), _code(x), x.stride(0), 1, top, _ptr(up), _code(up), _ptr(act),
                                               F, _ptr(route), pairs, E, F, D, first, code, tile, flag, stream),
               "chosen_experts (up)")
        _check(self.lib.chibi_expert_rows_gemm(_ptr(act), _code(act), F, 0, top, _ptr(down), _code(down), _ptr(y), D,
                                               _ptr(route), pairs, E, D, F, 0, 0, tile, 0, stream),
               "chosen_experts (down)")
        if fast:
            self.tensor_core_calls += 2
        _check(self.lib.chibi_combine_experts(_ptr(y), _ptr(route), _ptr(acc), acc.stride(0), T, D, top, E, 1.0,
                                              _ptr(share), stream), "chosen_experts (combine)")

    def layer_end(self, residual: torch.Tensor, delta: Optional[torch.Tensor], mult: float, side=None,
                  y_in: Optional[torch.Tensor] = None, norm=None, copy_out: Optional[torch.Tensor] = None) -> None:
        """residual += mult * delta; then the per-layer token input, if ``side`` is
        given: (tokens, table [vocab, all], offset, gate [s, n], proj [n, s], norm weight
        [n], activation, eps): y = proj (act(gate x) * table[token, offset:offset + s]),
        x += mult * y / rms(y) * weight -- the two products are done by the kernel unless
        ``y_in`` [T, n] float32 brings y; then, if ``norm`` = (weight, eps, offset, out)
        is given, out = x / rms(x) * (weight + offset); ``copy_out`` [T, n] takes the new
        residual in its own type.  One launch, a block per token."""
        _need_cuda(residual, delta, y_in)
        T, n = residual.shape
        if residual.dtype != torch.float32 or not residual.is_contiguous() or (
                delta is not None and (delta.shape != residual.shape or delta.dtype != torch.float32
                                       or not delta.is_contiguous())):
            raise KernelError("layer_end: residual and delta are contiguous float32 [T, n]")
        tokens = table = gate = proj = side_w = None
        offset = s = vocab = stride = 0
        kind, eps = 1, 0.0
        w_type = F32
        if side is not None:
            tokens, table, offset, gate, proj, side_w, act, eps = side
            _need_cuda(tokens, table, gate, proj, side_w)
            s, vocab, stride = gate.shape[0], table.shape[0], table.stride(0)
            kind = self.ACTIVATIONS[act]
            if (gate.shape != (s, n) or proj.shape != (n, s) or side_w.shape != (n,) or offset + s > table.shape[1]
                    or not (gate.is_contiguous() and proj.is_contiguous() and side_w.is_contiguous())
                    or table.stride(1) != 1 or len({table.dtype, gate.dtype, proj.dtype, side_w.dtype}) != 1
                    or tokens.dtype != torch.int32):
                raise KernelError("layer_end: shapes or types of the token input")
            w_type = _code(gate)
            if y_in is not None and (y_in.shape != (T, n) or y_in.dtype != torch.float32 or not y_in.is_contiguous()):
                raise KernelError("layer_end: y_in is contiguous float32 [T, n]")
        norm_w = out = None
        norm_eps = norm_offset = 0.0
        if norm is not None:
            norm_w, norm_eps, norm_offset, out = norm
            _need_cuda(norm_w, out)
            if norm_w.shape != (n,) or out.shape != (T, n) or not out.is_contiguous() or not norm_w.is_contiguous():
                raise KernelError("layer_end: shapes of the norm")
            if side is not None and (norm_w.dtype != gate.dtype or float(norm_eps) != float(eps)):
                raise KernelError("layer_end: the norm's weight type and eps must be the token input's")
            w_type, eps = _code(norm_w), norm_eps
        if copy_out is not None:
            _need_cuda(copy_out)
            if copy_out.shape != (T, n) or not copy_out.is_contiguous() or (out is not None and out.dtype != copy_out.dtype):
                raise KernelError("layer_end: copy_out is contiguous [T, n], of the norm output's type")
        self.launches += 1
        _check(self.lib.chibi_layer_end(
            _ptr(residual), _ptr(delta), float(mult), _ptr(tokens), _ptr(table), stride, int(offset), vocab, _ptr(gate),
            _ptr(proj), _ptr(side_w), _ptr(y_in), s, kind, float(eps), _ptr(norm_w), float(norm_offset), _ptr(out),
            _ptr(copy_out), _code(out) if out is not None else (_code(copy_out) if copy_out is not None else F32),
            w_type, T, n, _ptr(self.error), self._stream()), "layer_end")

    def side_gate(self, gate: torch.Tensor, tokens: torch.Tensor, table: torch.Tensor, offset: int, kind: str) -> None:
        """gate[t, j] = act(gate[t, j]) * table[tokens[t], offset + j], in place."""
        _need_cuda(gate, tokens, table)
        _rows_contiguous(gate, "side_gate: gate")
        if table.stride(1) != 1 or offset + gate.shape[1] > table.shape[1] or tokens.dtype != torch.int32:
            raise KernelError("side_gate: shapes")
        self.launches += 1
        _check(self.lib.chibi_side_gate(_ptr(gate), _code(gate), gate.stride(0), _ptr(tokens), _ptr(table),
                                        _code(table), table.stride(0), int(offset), table.shape[0], gate.shape[0],
                                        gate.shape[1], self.ACTIVATIONS[kind], _ptr(self.error), self._stream()),
               "side_gate")

    # ---- parts of hybrid_ops.cu
    def bigram_embed(self, residual: torch.Tensor, table: torch.Tensor, kept: torch.Tensor, tokens: torch.Tensor,
                     positions: torch.Tensor, seq_of_token: torch.Tensor, q_start: torch.Tensor,
                     state_slots: torch.Tensor, mul_prev: int, mul_cur: int) -> None:
        """residual[t] += table[(previous token * mul_prev + token * mul_cur) mod buckets], the last row of
        the table ([buckets + 1, n]) for a sequence's first token.  The token before a step's first comes
        from ``kept`` (int32 [slots, 1]), which then takes the sequence's last token of the step."""
        _need_cuda(residual, table, kept, tokens, positions, seq_of_token, q_start, state_slots)
        T, n = residual.shape
        if residual.dtype != torch.float32 or not residual.is_contiguous() or table.dim() != 2 or table.shape[1] != n \
                or table.shape[0] < 2 or not table.is_contiguous() or kept.dtype != torch.int32 \
                or not kept.is_contiguous() or tokens.dtype != torch.int32:
            raise KernelError("bigram_embed: residual float32 [T, n], table [buckets + 1, n], kept int32 [slots, 1]")
        self.launches += 1
        _check(self.lib.chibi_bigram_embed(_ptr(residual), _ptr(table), _code(table), _ptr(tokens), _ptr(positions),
                                           _ptr(seq_of_token), _ptr(q_start), _ptr(state_slots), _ptr(kept), T, n,
                                           table.shape[0] - 1, int(mul_prev), int(mul_cur), self._stream()),
               "bigram_embed")

    def stream_enter(self, x: torch.Tensor, x0: Optional[torch.Tensor], vec: Optional[torch.Tensor]) -> None:
        """x += x0 + vec (float32; x0 [T, n] and the row vector vec [n] may each be None)."""
        _need_cuda(x, x0, vec)
        T, n = x.shape
        if x.dtype != torch.float32 or not x.is_contiguous() \
                or (x0 is not None and (x0.dtype != torch.float32 or x0.shape != x.shape or not x0.is_contiguous())) \
                or (vec is not None and (vec.dtype != torch.float32 or vec.shape != (n,) or not vec.is_contiguous())):
            raise KernelError("stream_enter: contiguous float32 x [T, n], x0 [T, n], vec [n]")
        self.launches += 1
        _check(self.lib.chibi_stream_enter(_ptr(x), _ptr(x0), _ptr(vec), T, n, self._stream()), "stream_enter")

    def add_weighted(self, acc: torch.Tensor, a: torch.Tensor, wa: float, b: Optional[torch.Tensor] = None,
                     wb: float = 0.0) -> None:
        """acc += wa * a + wb * b (all contiguous float32 of one size)."""
        _need_cuda(acc, a, b)
        for t in (acc, a, b):
            if t is not None and (t.dtype != torch.float32 or not t.is_contiguous() or t.numel() != acc.numel()):
                raise KernelError("add_weighted: contiguous float32 arrays of one size")
        self.launches += 1
        _check(self.lib.chibi_add_weighted(_ptr(acc), _ptr(a), float(wa), _ptr(b), float(wb), acc.numel(),
                                           self._stream()), "add_weighted")

    def heads_prepare_append(self, proj: torch.Tensor, q_out: torch.Tensor, k_cache: Optional[torch.Tensor],
                             v_cache: Optional[torch.Tensor], bias: Optional[torch.Tensor],
                             q_norm: Optional[torch.Tensor], k_norm: Optional[torch.Tensor], eps: float,
                             inv_freq: Optional[torch.Tensor], rotary_dim: int, positions: torch.Tensor,
                             seq_of_token: torch.Tensor, block_table: Optional[torch.Tensor], nq: int, nk: int,
                             nv: int, d: int, dv: int, page_size: int,
                             seq_rows: Optional[torch.Tensor] = None) -> None:
        """Per head of a row q | k | v ([T, >= nq d + nk d + nv dv]; [T, >= nq d] without a cache):
        + bias (float32 over the row, or None); q and k heads divided by their root mean square and
        multiplied by ``q_norm`` / ``k_norm`` (float32 [d], both or none); the first ``rotary_dim``
        features rotated; q -> q_out, k -> [pages, nk, page, d], v -> [pages, nv, page, dv]."""
        _need_cuda(proj, q_out, k_cache, v_cache, bias, q_norm, k_norm, inv_freq, positions, seq_of_token,
                   block_table, seq_rows)
        _rows_contiguous(proj, "heads_prepare_append: proj")
        T = proj.shape[0]
        append = k_cache is not None
        width = nq * d + ((nk * d + nv * dv) if append else 0)
        if proj.shape[1] < width or not q_out.is_contiguous() or q_out.shape != (T, nq * d) or q_out.dtype != proj.dtype:
            raise KernelError("heads_prepare_append: proj / q_out shapes or types")
        if (q_norm is None) != (k_norm is None):
            raise KernelError("heads_prepare_append: give both norm weights or none")
        for t, size, what in ((bias, width, "bias"), (q_norm, d, "q_norm"), (k_norm, d, "k_norm")):
            if t is not None and (t.dtype != torch.float32 or t.numel() < size or not t.is_contiguous()):
                raise KernelError(f"heads_prepare_append: {what} must be contiguous float32 of {size} values")
        if rotary_dim and (inv_freq is None or inv_freq.dtype != torch.float32 or inv_freq.numel() < rotary_dim // 2):
            raise KernelError("heads_prepare_append: inv_freq must hold rotary_dim/2 float32 values")
        num_pages = table_stride = 0
        if append:
            if (v_cache is None or not k_cache.is_contiguous() or not v_cache.is_contiguous()
                    or tuple(k_cache.shape[1:]) != (nk, page_size, d)
                    or tuple(v_cache.shape) != (k_cache.shape[0], nv, page_size, dv) or v_cache.dtype != k_cache.dtype):
                raise KernelError(f"heads_prepare_append: cache shapes {tuple(k_cache.shape)}")
            num_pages = k_cache.shape[0]
            _rows_contiguous(block_table, "heads_prepare_append: block_table")
            table_stride = block_table.stride(0)
        self.launches += 1
        _check(self.lib.chibi_heads_prepare_append(
            _ptr(proj), _code(proj), proj.stride(0), _ptr(bias), _ptr(q_norm), _ptr(k_norm), float(eps),
            _ptr(inv_freq) if rotary_dim else None, int(rotary_dim), _ptr(positions), _ptr(seq_of_token),
            _ptr(seq_rows), _ptr(block_table), table_stride, _ptr(q_out), _ptr(k_cache), _ptr(v_cache),
            _code(k_cache) if append else F32, T, nq, nk, nv, d, dv, page_size, num_pages, _ptr(self.error),
            self._stream()), "heads_prepare_append")

    def differential_combine(self, att: torch.Tensor, gate: Optional[torch.Tensor], lam: float, eps: float,
                             out_scale: float, out: torch.Tensor, heads: int, dv: int, group: int) -> None:
        """Per head h of att (float32 [T, 2 * heads * dv]; the ``group`` heads of a key/value head side
        by side, first their first maps, then their second ones):
        o = a1 - lam * a2; out[t, h] = o / sqrt(mean(o^2) + eps) * out_scale * sigmoid(gate[t, h])."""
        _need_cuda(att, gate, out)
        T = att.shape[0]
        if att.dtype != torch.float32 or not att.is_contiguous() or att.shape != (T, heads * 2 * dv) \
                or out.shape != (T, heads * dv) or not out.is_contiguous():
            raise KernelError("differential_combine: att float32 [T, 2 heads dv] and out [T, heads dv]")
        if gate is not None:
            _rows_contiguous(gate, "differential_combine: gate")
            if gate.shape != (T, heads) or gate.dtype != out.dtype:
                raise KernelError("differential_combine: gate [T, heads] of out's type")
        self.launches += 1
        _check(self.lib.chibi_differential_combine(_ptr(att), _ptr(gate), _code(out),
                                                   gate.stride(0) if gate is not None else 0, float(lam), float(eps),
                                                   float(out_scale), _ptr(out), T, heads, dv, int(group),
                                                   self._stream()), "differential_combine")

    def causal_conv(self, x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor],
                    history: torch.Tensor, out: torch.Tensor, q_start: torch.Tensor, state_slots: torch.Tensor,
                    max_q_len: int, activation: Optional[str] = None, weight_t: Optional[torch.Tensor] = None) -> None:
        """out_t = act(bias + sum_j weight[:, j] * x_(t - taps + 1 + j)) per channel along each sequence
        of the step (zeros before a sequence's start); ``history`` as for ``short_conv``."""
        _need_cuda(x, weight, bias, history, out, q_start, state_slots, weight_t)
        _rows_contiguous(x, "causal_conv: x")
        _rows_contiguous(out, "causal_conv: out")
        T, D = x.shape
        taps = weight.shape[1]
        if weight.shape != (D, taps) or weight.dtype != torch.float32 or not weight.is_contiguous() \
                or out.shape != x.shape or out.dtype != x.dtype or history.dtype != x.dtype \
                or not history.is_contiguous() or tuple(history.shape[1:]) != (max(taps - 1, 1), D) \
                or (bias is not None and (bias.dtype != torch.float32 or bias.shape != (D,) or not bias.is_contiguous())) \
                or (activation is not None and activation not in self.ACTIVATIONS):
            raise KernelError("causal_conv: weight float32 [D, taps], bias float32 [D], history [slots, taps - 1, D]")
        if weight_t is not None and (weight_t.dtype != torch.float32 or weight_t.shape != (taps, D)
                                     or not weight_t.is_contiguous()):
            raise KernelError("causal_conv: weight_t must be the weight transposed, contiguous float32 [taps, D]")
        self.launches += 1
        _check(self.lib.chibi_causal_conv(_ptr(x), _code(x), x.stride(0), _ptr(weight), _ptr(weight_t), _ptr(history),
                                          _ptr(out), out.stride(0), _ptr(q_start), _ptr(state_slots),
                                          state_slots.numel(), int(max_q_len), D, taps, _ptr(bias),
                                          self.ACTIVATIONS[activation] if activation is not None else -1, 0,
                                          self._stream()), "causal_conv")

    def state_space_scan(self, xbc: torch.Tensor, dt: torch.Tensor, dt_bias: torch.Tensor, a_log: torch.Tensor,
                         skip: torch.Tensor, state: torch.Tensor, y: torch.Tensor, q_start: torch.Tensor,
                         state_slots: torch.Tensor, heads: int, groups: int, e: int, n: int) -> None:
        """Per head h (group g = h // (heads / groups)) over the step's tokens of every sequence:
        step = softplus(dt[t, h] + dt_bias[h]); S <- exp(-exp(a_log[h]) * step) S + step * B_t x_t^T;
        y_t = S^T C_t + skip[h] * x_t.  xbc [T, heads e + 2 groups n] holds x | B | C; ``state`` float32
        [slots, heads, e, n] (value column first) is read and left per request; y float32 [T, heads e]."""
        _need_cuda(xbc, dt, dt_bias, a_log, skip, state, y, q_start, state_slots)
        _rows_contiguous(xbc, "state_space_scan: xbc")
        _rows_contiguous(dt, "state_space_scan: dt")
        T = xbc.shape[0]
        if xbc.shape[1] != heads * e + 2 * groups * n or dt.shape != (T, heads) or dt.dtype != xbc.dtype \
                or state.dtype != torch.float32 or not state.is_contiguous() or tuple(state.shape[1:]) != (heads, e, n) \
                or y.dtype != torch.float32 or y.shape != (T, heads * e) or not y.is_contiguous():
            raise KernelError("state_space_scan: shapes or types")
        for t in (dt_bias, a_log, skip):
            if t.dtype != torch.float32 or t.shape != (heads,) or not t.is_contiguous():
                raise KernelError("state_space_scan: dt_bias, a_log and skip are contiguous float32 [heads]")
        self.launches += 1
        _check(self.lib.chibi_state_space_scan(_ptr(xbc), _code(xbc), xbc.stride(0), _ptr(dt), dt.stride(0),
                                               _ptr(dt_bias), _ptr(a_log), _ptr(skip), _ptr(state), _ptr(y),
                                               _ptr(q_start), _ptr(state_slots), state_slots.numel(), heads, groups,
                                               e, n, self._stream()), "state_space_scan")

    def gated_group_rms(self, y: torch.Tensor, z: torch.Tensor, weight: torch.Tensor, eps: float, parts: int,
                        out: torch.Tensor) -> None:
        """v = y * silu(z); out = v / sqrt(mean(v^2 over each of ``parts`` equal parts) + eps) * weight."""
        _need_cuda(y, z, weight, out)
        _rows_contiguous(z, "gated_group_rms: z")
        T, W = y.shape
        if y.dtype != torch.float32 or not y.is_contiguous() or z.shape != y.shape or W % parts != 0 \
                or weight.dtype != torch.float32 or weight.shape != (W,) or not weight.is_contiguous() \
                or out.shape != y.shape or not out.is_contiguous() or out.dtype != z.dtype:
            raise KernelError("gated_group_rms: y float32 [T, W], z [T, W], weight float32 [W], out [T, W] of z's type")
        self.launches += 1
        _check(self.lib.chibi_gated_group_rms(_ptr(y), _ptr(z), _code(z), z.stride(0), _ptr(weight), float(eps),
                                              _ptr(out), T, W, int(parts), self._stream()), "gated_group_rms")

    def clamped_swish_gate(self, gate_up: torch.Tensor, out: torch.Tensor, limit: float, slope: float) -> None:
        """g = min(gate, limit), u = clamp(up, -limit, limit); out = g * sigmoid(slope * g) * (u + 1);
        gate_up [T, 2 n] holds the gate columns, then the up columns."""
        _need_cuda(gate_up, out)
        _rows_contiguous(gate_up, "clamped_swish_gate: gate_up")
        T, n = out.shape
        if gate_up.shape != (T, 2 * n) or not out.is_contiguous() or out.dtype != gate_up.dtype:
            raise KernelError("clamped_swish_gate: gate_up [T, 2 n] and out [T, n] of one type")
        self.launches += 1
        _check(self.lib.chibi_clamped_swish_gate(_ptr(gate_up), _code(gate_up), gate_up.stride(0), _ptr(out), T, n,
                                                 float(limit), float(slope), self._stream()), "clamped_swish_gate")

    def router_choose(self, logits: torch.Tensor, correction: Optional[torch.Tensor], chosen: torch.Tensor,
                      share: torch.Tensor, group_count: int, group_keep: int, scale: float,
                      last_choice: Optional[int] = None) -> None:
        """s = softmax(logits[t]) (float32 [T, n]); choice = s + correction; of ``group_count`` equal
        groups of neighbours only the ``group_keep`` with the largest best choice stay open;
        chosen[t] (int32 [T, top]) = the open outputs with the largest choice, largest first, ties to
        the lower number; share[t] = s[chosen] * scale.  ``last_choice``: numbers above it are written
        as it (outputs that all name the same thing, such as experts that return their input)."""
        _need_cuda(logits, correction, chosen, share)
        _rows_contiguous(logits, "router_choose: logits")
        T, n = logits.shape
        top = chosen.shape[1]
        if logits.dtype != torch.float32 or chosen.dtype != torch.int32 or share.dtype != torch.float32 \
                or chosen.shape != (T, top) or share.shape != (T, top) or not chosen.is_contiguous() \
                or not share.is_contiguous() or not (0 < top <= n) \
                or (correction is not None and (correction.dtype != torch.float32 or correction.shape != (n,)
                                                or not correction.is_contiguous())):
            raise KernelError("router_choose: shapes or types")
        self.launches += 1
        _check(self.lib.chibi_router_choose(_ptr(logits), logits.stride(0), _ptr(correction), _ptr(chosen),
                                            _ptr(share), T, n, top, int(group_count), int(group_keep), float(scale),
                                            n - 1 if last_choice is None else int(last_choice), self._stream()),
               "router_choose")

    def scaled_add_norm(self, residual: torch.Tensor, delta: torch.Tensor, vec: Optional[torch.Tensor],
                        norm=None) -> None:
        """residual += vec * delta (vec float32 [n] or None for ones); then, with ``norm`` = (weight,
        eps, offset, out): out = residual / rms(residual) * (weight + offset).  One launch."""
        _need_cuda(residual, delta, vec)
        T, n = residual.shape
        if residual.dtype != torch.float32 or not residual.is_contiguous() or delta.dtype != torch.float32 \
                or delta.shape != residual.shape or not delta.is_contiguous() \
                or (vec is not None and (vec.dtype != torch.float32 or vec.shape != (n,) or not vec.is_contiguous())):
            raise KernelError("scaled_add_norm: contiguous float32 residual and delta [T, n], vec [n]")
        w = out = None
        eps = offset = 0.0
        if norm is not None:
            w, eps, offset, out = norm
            _need_cuda(w, out)
            if w.shape != (n,) or not w.is_contiguous() or out.shape != (T, n) or not out.is_contiguous():
                raise KernelError("scaled_add_norm: shapes of the norm")
        self.launches += 1
        _check(self.lib.chibi_scaled_add_norm(_ptr(residual), _ptr(delta), _ptr(vec), _ptr(w),
                                              _code(w) if w is not None else F32, float(eps), float(offset),
                                              _ptr(out), _code(out) if out is not None else F32, T, n,
                                              self._stream()), "scaled_add_norm")

    def softcap(self, x: torch.Tensor, cap: float) -> None:
        """x = cap * tanh(x / cap), in place (float32)."""
        _need_cuda(x)
        if x.dtype != torch.float32 or not x.is_contiguous() or not cap > 0:
            raise KernelError("softcap: x must be contiguous float32 and the cap positive")
        self.launches += 1
        _check(self.lib.chibi_softcap(_ptr(x), float(cap), x.numel(), self._stream()), "softcap")

    def zero(self, x: torch.Tensor) -> None:
        _need_cuda(x)
        if x.dtype != torch.float32 or not x.is_contiguous():
            raise KernelError("zero: x must be contiguous float32")
        self.launches += 1
        _check(self.lib.chibi_zero(_ptr(x), x.numel(), self._stream()), "zero")

    def gather_rows(self, x: torch.Tensor, rows: torch.Tensor, out: torch.Tensor) -> None:
        _need_cuda(x, rows, out)
        if not x.is_contiguous() or not out.is_contiguous() or rows.dtype != torch.int32 \
                or out.shape != (rows.numel(), x.shape[1]):
            raise KernelError("gather_rows: shapes")
        self.launches += 1
        _check(self.lib.chibi_gather_rows(_ptr(x), _code(x), _ptr(rows), _ptr(out), _code(out),
                                          rows.numel(), x.shape[1], x.shape[0], self._stream()),
               "gather_rows")

    def cast(self, x: torch.Tensor, out: torch.Tensor) -> None:
        _need_cuda(x, out)
        if not x.is_contiguous() or not out.is_contiguous() or x.numel() != out.numel():
            raise KernelError("cast: shapes")
        self.launches += 1
        _check(self.lib.chibi_cast(_ptr(x), _code(x), _ptr(out), _code(out), x.numel(),
                                   self._stream()), "cast")

    def add_into(self, acc: torch.Tensor, x: torch.Tensor) -> None:
        _need_cuda(acc, x)
        if acc.dtype != torch.float32 or not acc.is_contiguous() or not x.is_contiguous() \
                or acc.numel() != x.numel():
            raise KernelError("add_into: acc must be contiguous float32 of x's size")
        self.launches += 1
        _check(self.lib.chibi_add_into(_ptr(acc), _ptr(x), _code(x), x.numel(), self._stream()),
               "add_into")

    def sample(self, logits: torch.Tensor, temperature: Optional[torch.Tensor],
               uniform: Optional[torch.Tensor], out: torch.Tensor) -> None:
        """Greedy rows (temperature <= 0 or None) take the arg max, ties to the
        lowest id; other rows sample by inverse CDF with the given uniform."""
        _need_cuda(logits, temperature, uniform, out)
        _rows_contiguous(logits, "sample: logits")
        if logits.dtype != torch.float32 or out.dtype != torch.int32 or out.numel() != logits.shape[0]:
            raise KernelError("sample: logits float32 [R, V], out int32 [R]")
        for t in (temperature, uniform):
            if t is not None and (t.dtype != torch.float32 or t.numel() != logits.shape[0]):
                raise KernelError("sample: temperature / uniform must be float32 [R]")
        scratch = self._scratch(logits.shape[0] * 128) if temperature is None else None
        self.launches += 2 if temperature is None else 1
        _check(self.lib.chibi_sample(_ptr(logits), logits.stride(0), logits.shape[0], logits.shape[1],
                                     _ptr(temperature), _ptr(uniform), _ptr(out), _ptr(scratch),
                                     scratch.numel() if scratch is not None else 0, self._stream()),
               "sample")
