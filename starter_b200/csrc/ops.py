"""The call table of the CUDA extension: torch tensors in, kernels launched on torch's current stream.

Every function here launches hand-written sm_100a kernels from this folder's
``.cu`` files through their ``extern "C"`` entry points.  Matrix products in
bfloat16 with many rows go to cuBLAS through ``torch.matmul``, where the
reference's engine calls the same library (engine/model.py:291,295,297,299).
There is no CPU path and no other backend: without a CUDA device or without
the compiled library, ``get_ops`` raises.
"""

from __future__ import annotations

import contextlib
import ctypes
import weakref
import os
from ctypes import POINTER, Structure, c_float, c_int, c_longlong, c_ulonglong, c_void_p

import torch

from .build import BuildError, load

F32, BF16 = 0, 1
_RAW_STREAM = getattr(torch._C, "_cuda_getCurrentRawStream", None)   # (device index) -> cudaStream_t as an int


class KernelError(RuntimeError):
    """A kernel launch was refused (sizes it does not take) or failed."""


class SbBatch(Structure):
    _fields_ = [("seq_slot", c_void_p), ("cu_q", c_void_p), ("row_seq", c_void_p), ("lengths", c_void_p),
                ("n_seqs", c_int), ("n_rows", c_int), ("null_slot", c_int), ("reserved", c_int)]


class SbKV(Structure):
    _fields_ = [("k", c_void_p), ("v", c_void_p), ("table", c_void_p), ("table_width", c_int),
                ("ring_pages", c_int), ("n_kv_heads", c_int), ("head_dim", c_int)]


class SbFusedQK(Structure):
    _fields_ = [("qkv", c_void_p), ("q_norm", c_void_p), ("k_norm", c_void_p), ("cos_t", c_void_p), ("sin_t", c_void_p),
                ("status", c_void_p), ("eps", c_float), ("norm_f32", c_int), ("store_kv", c_int), ("reserved", c_int),
                ("next_w", c_void_p), ("next_bytes", c_longlong)]


def _code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16 tensors, not {dtype}")


def _ptr(t):
    return None if t is None else c_void_p(t.data_ptr())


class Ops:
    name = "cuda"

    # bfloat16 products with at most this many rows stay on this library's own kernels
    GENERAL_GEMM_MAX_WORK = 1 << 22

    def __init__(self, lib: ctypes.CDLL):
        self.lib = lib
        self.launches = 0  # kernels of this library launched so far (cuBLAS calls are not counted)
        lib.sb_error_string.restype = ctypes.c_char_p
        lib.sb_tile_matrix_elements.restype = c_longlong
        lib.sb_tile_matrix_elements.argtypes = [c_int, c_int, c_int]
        lib.sb_error_string.argtypes = [c_int]
        sig = {
            "sb_embed": [c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p],
            "sb_gather_rows": [c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
            "sb_rmsnorm": [c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p],
            "sb_swiglu": [c_int, c_void_p, c_void_p, c_int, c_int, c_void_p],
            "sb_advance_lengths": [SbBatch, c_void_p, c_void_p],
            "sb_gemm_general": [c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
            "sb_qk_rope_store": [c_int, c_int, c_void_p, c_void_p, SbBatch, SbKV, c_int, c_int, c_void_p, c_void_p,
                                 c_float, c_void_p, c_void_p, c_int, c_void_p, c_void_p],
            "sb_attention_general": [c_int, c_void_p, c_void_p, SbBatch, SbKV, c_int, c_float, c_int, c_void_p],
            "sb_gemm_skinny": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                               c_int, c_void_p, c_void_p, c_void_p, c_void_p],
            "sb_gemm_skinny_normed": [c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                      c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p],
            "sb_tile_matrix": [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
            "sb_gemm_stream": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                               c_void_p, c_void_p],
            "sb_gemm_stream_plan": [c_int, c_int, c_int, POINTER(c_int), POINTER(c_int), POINTER(c_int)],
            "sb_attn_prefill_tc": [c_void_p, c_void_p, SbBatch, SbKV, c_int, c_float, c_int, c_int, c_int, c_void_p, c_void_p],
            "sb_attn_prefill": [c_void_p, c_void_p, SbBatch, SbKV, c_int, c_float, c_int, c_int, c_void_p],
            "sb_attn_decode_balanced": [c_void_p, c_void_p, SbBatch, SbKV, c_int, c_float, c_int, c_int, c_void_p, c_void_p,
                                        c_void_p],
            "sb_attn_decode": [c_void_p, c_void_p, SbBatch, SbKV, c_int, c_float, c_int, c_int, c_void_p, c_void_p, c_void_p],
            "sb_attn_decode_balanced_fused": [SbFusedQK, c_void_p, SbBatch, SbKV, c_int, c_float, c_int, c_int, c_void_p,
                                              c_void_p, c_void_p],
            "sb_attn_decode_fused": [SbFusedQK, c_void_p, SbBatch, SbKV, c_int, c_float, c_int, c_int, c_void_p, c_void_p,
                                     c_void_p],
            "sb_argmax": [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p],
            "sb_sample": [c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_ulonglong, c_void_p, c_void_p, c_int,
                          c_void_p, c_void_p],
        }
        for name, argtypes in sig.items():
            fn = getattr(lib, name)
            fn.argtypes = argtypes
            fn.restype = c_int
        lib.sb_set_pdl.argtypes = [c_int]
        lib.sb_set_pdl.restype = None
        self._scratch = {}
        self._sm_count = None
        self.force_skinny = None  # (K slices, tiled, warps) for tests and tuning runs; None = the rules below
        self._tiled_bytes = 0     # bytes of tile-major copies alive (a copy hangs on its matrix as ._sb_tiled = (copy, halves))
        self.decode_copy = os.environ.get("STARTER_B200_DECODE_COPY", "auto")   # "1", "0" or "auto"
        self.use_stream = os.environ.get("STARTER_B200_STREAM", "1") != "0"  # the TMA + tcgen05 product for decode
        self._kernel_status = None
        self._status_override = None
        self.decode_balanced = os.environ.get("STARTER_B200_ATTN", "balanced") != "split"
        self.force_decode_route = os.environ.get("STARTER_B200_ATTN_ROUTE") or None   # "split" or "balanced", for tests and tuning runs; None = the rule in _decode_route
        self.fuse_qk = os.environ.get("STARTER_B200_FUSE_QK", "1") != "0"
        # With the balanced kernel (more pairs than blocks fit at once) the preparation stays a kernel of its own: a block
        # walks several (sequence, kv head) pairs one after another and pays each pair's preparation on its own path.
        # Measured in the step (4B sizes, context 4,096): batch 64 8.74 ms with the preparation inside, 8.54 ms apart;
        # the split-key kernel is the other way round (batch 32: 5.41 inside, 5.53 apart).
        self.fuse_qk_balanced = os.environ.get("STARTER_B200_FUSE_QK_BALANCED", "0") != "0"
        self.prefetch_next_bytes = int(os.environ.get("STARTER_B200_PREFETCH_MAX", 24 << 20))
        self.prefill_tensor_memory = os.environ.get("STARTER_B200_PREFILL", "tc") != "mma"

    # ---- plumbing -----------------------------------------------------------------------

    @staticmethod
    def _stream():
        """torch's current stream as a raw handle.  Asked for at every launch: torch.cuda.current_stream() builds a
        Stream object and costs the host ~14 us a call (measured: a quarter of the host's time in an eager step);
        the raw query is a fraction of a microsecond."""
        if _RAW_STREAM is not None:
            return c_void_p(_RAW_STREAM(torch.cuda.current_device()))
        return c_void_p(torch.cuda.current_stream().cuda_stream)

    def _check(self, code: int, what: str) -> None:
        self.launches += 1
        if code:
            raise KernelError(f"{what}: {self.lib.sb_error_string(code).decode()} (code {code})")

    @staticmethod
    def _batch(ctx) -> SbBatch:
        b = ctx.scratch.get("sb_batch")
        if b is None:
            b = SbBatch(ctx.seq_slot.data_ptr(), ctx.cu_q.data_ptr(), ctx.row_seq.data_ptr(), ctx.lengths.data_ptr(),
                        ctx.n_seqs, ctx.n_rows, ctx.cache.null_slot, 0)
            ctx.scratch["sb_batch"] = b
        return b

    @staticmethod
    def _kv(layer_cache) -> SbKV:
        kv = getattr(layer_cache, "_sb_kv", None)
        if kv is None:
            g = layer_cache.group
            kv = SbKV(layer_cache.k.data_ptr(), layer_cache.v.data_ptr(), g.table.data_ptr(), g.table_width,
                      g.ring_pages, g.request.num_kv_heads, g.request.head_dim)
            layer_cache._sb_kv = kv
        return kv

    def set_dependent_launch(self, on: bool) -> None:
        """Launch kernels so that each may start its preamble (weight fetches, barrier set-up) while the
        one before it in the stream is finishing; see common.cuh."""
        self.lib.sb_set_pdl(int(bool(on)))

    DECODE_COPY_SHARE = 0.2   # "auto": tile-major copies are made while they stay below this share of the device's memory

    def _forget_copy(self, nbytes: int) -> None:
        self._tiled_bytes -= nbytes

    def prepare_matrix(self, w: torch.Tensor, halves: int = 1) -> torch.Tensor:
        """A weight matrix [out, in] as the products want it: contiguous, in the run's dtype.  ``halves``: 2 for
        a fused [gate; up] matrix (linear_swiglu pairs row r of the first half with row r of the second).

        For bfloat16 matrices a second, tile-major copy is kept for the decode product (gemm_skinny.cu: one
        contiguous piece per warp and turn instead of sixteen short ones; 4-7% of a decode step on the 4B
        shapes), as long as all such copies together stay below DECODE_COPY_SHARE of the device's memory
        (STARTER_B200_DECODE_COPY=1 always, =0 never).  Products with many rows read the row-major matrix."""
        if w.dim() != 2:
            raise KernelError(f"a weight matrix has two axes, got shape {tuple(w.shape)}")
        _code(w.dtype)
        w = w.contiguous()
        if (w.is_cuda and w.dtype == torch.bfloat16 and w.shape[1] % 8 == 0 and w.shape[0] % halves == 0
                and self.decode_copy != "0" and getattr(w, "_sb_tiled", None) is None):
            rows = w.shape[0] // halves
            n = self.lib.sb_tile_matrix_elements(rows, w.shape[1], halves)
            total = torch.cuda.get_device_properties(w.device).total_memory
            if self.decode_copy == "1" or self._tiled_bytes + 2 * n <= self.DECODE_COPY_SHARE * total:
                tiled = torch.empty(n, dtype=torch.bfloat16, device=w.device)
                self._check(self.lib.sb_tile_matrix(_ptr(w), _ptr(tiled), rows, w.shape[1], halves, self._stream()), "tile_matrix")
                w._sb_tiled = (tiled, halves)   # lives and dies with the matrix object that the parts hold
                self._tiled_bytes += 2 * n
                weakref.finalize(w, self._forget_copy, 2 * n)
        return w

    # ---- rows ---------------------------------------------------------------------------

    def embed(self, tokens, table, status):
        out = torch.empty((tokens.shape[0], table.shape[1]), dtype=table.dtype, device=table.device)
        self._check(self.lib.sb_embed(_code(table.dtype), _ptr(tokens), _ptr(table), _ptr(out), tokens.shape[0],
                                      table.shape[1], table.shape[0], _ptr(status), self._stream()), "embed")
        return out

    def gather_rows(self, x, rows):
        out = torch.empty((rows.shape[0], x.shape[1]), dtype=x.dtype, device=x.device)
        self._check(self.lib.sb_gather_rows(_code(x.dtype), _ptr(x), _ptr(rows), _ptr(out), rows.shape[0], x.shape[1],
                                            self._stream()), "gather_rows")
        return out

    def _norm_dtypes(self, x, w):
        if x.dtype == torch.float32 and w.dtype != torch.float32:
            raise KernelError("a float32 run needs float32 norm weights")
        return _code(x.dtype), _code(w.dtype)

    def rmsnorm(self, x, w, eps):
        dt, wdt = self._norm_dtypes(x, w)
        out = torch.empty_like(x)
        self._check(self.lib.sb_rmsnorm(dt, wdt, _ptr(x), None, _ptr(w), _ptr(out), x.shape[0], x.shape[1], eps,
                                        self._stream()), "rmsnorm")
        return out

    def add_rmsnorm(self, x, delta, w, eps):
        dt, wdt = self._norm_dtypes(x, w)
        out = torch.empty_like(x)
        self._check(self.lib.sb_rmsnorm(dt, wdt, _ptr(x), _ptr(delta), _ptr(w), _ptr(out), x.shape[0], x.shape[1], eps,
                                        self._stream()), "add_rmsnorm")
        return out

    def swiglu(self, gu):
        inter = gu.shape[1] // 2
        out = torch.empty((gu.shape[0], inter), dtype=gu.dtype, device=gu.device)
        self._check(self.lib.sb_swiglu(_code(gu.dtype), _ptr(gu), _ptr(out), gu.shape[0], inter, self._stream()), "swiglu")
        return out

    def advance_lengths(self, ctx):
        self._check(self.lib.sb_advance_lengths(self._batch(ctx), _ptr(ctx.lengths), self._stream()), "advance_lengths")

    # ---- products -----------------------------------------------------------------------

    # The mma.sync product takes up to 32 rows.  Measured in the step (B200): to 16 rows it beats cuBLAS + the SwiGLU
    # kernel (1.7B sizes at batch 16: 1.84 -> 1.76 ms a step, 4B sizes: 3.89 -> 3.82 ms), from 17 rows on it needs 128
    # registers and loses (4B sizes at batch 32: 6.64 against 5.35 ms).
    SKINNY_MAX_ROWS = int(os.environ.get("STARTER_B200_SKINNY_MAX_ROWS", 16))
    STREAM_MIN_ROWS = 9   # the TMA + tcgen05 product serves the output head from here on
    STREAM_MAX_ROWS = 32   # 778 MB head, us by rows (this kernel / cuBLAS): 16: 126 / 132, 32: 130 / 134, 48: 137 / 131, 64: 138 / 133
    STREAM_MIN_WORK = int(os.environ.get("STARTER_B200_STREAM_MIN", 300_000_000))  # elements of W below which the simpler kernels do as well

    def kernel_status(self, device) -> torch.Tensor:
        """A status word of the kernels that are not tied to a step (bit 4: a wait inside a kernel timed out)."""
        if self._status_override is not None:
            return self._status_override
        if self._kernel_status is None:
            self._kernel_status = torch.zeros(1, dtype=torch.int32, device=device)
        return self._kernel_status

    @contextlib.contextmanager
    def status_into(self, word: torch.Tensor):
        """While this is open, kernels that are not tied to a step raise their bits in ``word`` (int32 [1] on
        the device): a captured step then carries all its status in the word that travels with its tokens."""
        before, self._status_override = self._status_override, word
        try:
            yield
        finally:
            self._status_override = before

    def read_kernel_status(self) -> int:
        if self._kernel_status is None:
            return 0
        bits = int(self._kernel_status.item())
        if bits:
            self._kernel_status.zero_()
        return bits

    def _stream_product(self, a, w, n_out, gate_up, out_float32):
        """The TMA + tcgen05 weight-streaming product (see gemm_stream.cu)."""
        M, K = a.shape
        key = ("gemm_stream", a.device, n_out, K, gate_up, M <= 16, M <= 32)
        plan = self._scratch.get(key)
        if plan is None:
            grid, tiles, parts = c_int(), c_int(), c_int()
            self.lib.sb_gemm_stream_plan(n_out, K, self.sm_count(), ctypes.byref(grid), ctypes.byref(tiles), ctypes.byref(parts))
            bn = 16 if M <= 16 else (32 if M <= 32 else 64)
            floats = tiles.value * parts.value * bn * (2 if gate_up else 1) * 128
            plan = (grid.value, parts.value, torch.empty(floats, dtype=torch.float32, device=a.device),
                    torch.zeros(tiles.value, dtype=torch.int32, device=a.device))
            self._scratch[key] = plan
        grid, parts, partial, counters = plan
        out = torch.empty((M, n_out), dtype=torch.float32 if out_float32 else torch.bfloat16, device=a.device)
        self._check(self.lib.sb_gemm_stream(_ptr(a), _ptr(w), _ptr(out), M, n_out, K, int(gate_up), int(out_float32), grid,
                                            parts, _ptr(partial), _ptr(counters), _ptr(self.kernel_status(a.device)),
                                            self._stream()), "gemm_stream")
        return out

    def _takes_stream(self, M, n_out, K, gate_up) -> bool:
        """Measured on a B200 (microbench.py): per launch the TMA-fed kernel pays about 9 us before and
        after it streams (set-up, first data, the pass through scratch for shared tiles) and then streams
        at 6.3-6.9 TB/s; the warp-level kernel pays about 3 us and streams at 4.7 TB/s, more on very large
        matrices.  So: the output head for 9 to 32 rows, nothing smaller; from 33 rows on cuBLAS is ahead there too."""
        return (self.use_stream and self.STREAM_MIN_ROWS <= M <= (32 if gate_up else self.STREAM_MAX_ROWS)
                and K % 8 == 0 and K >= 64 and n_out * K * (2 if gate_up else 1) >= self.STREAM_MIN_WORK)

    def skinny_splits(self, blocks: int, K: int) -> int:
        """K slices per block of 16 weight rows: enough blocks for three per SM, but no slice
        shorter than 3072 columns (measured on the 4B shapes, in the decode step, with the slices
        meeting through cluster shared memory: short slices cost more in the meeting than they
        gain in parallelism; 1 slice for q/k/v, output and gate/up, 3 for down)."""
        return max(1, min(round(3 * self.sm_count() / blocks), K // 3072))

    def skinny_warps(self, n_blocks: int, nt: int = 1) -> int:
        """Warps per block.  Eight-warp blocks fit four to an SM (two from 17 rows on, where the kernel takes 128
        registers); when the blocks number a little more than that (608 for 592 places), the few left over run as a
        second wave on an empty GPU.  Four-warp blocks fit twice as many to an SM, so the same blocks run at once."""
        resident8 = (4 if nt <= 2 else 2) * self.sm_count()
        return 4 if resident8 < n_blocks <= (2 if nt <= 2 else 2.2) * resident8 else 8

    # Rows up to which a layer's norms and residual sums run inside its products (gemm_skinny.cuh) instead of in the
    # norm kernel.  Off: measured in the decode step on a B200 (4B layer sizes, context 4,096), the fold removes 72
    # of 259 launches and still loses: batch 1: 2.155 -> 2.194 ms a step, batch 8: 2.810 -> 2.889, batch 16: 3.765 ->
    # 4.301.  Every block of 16 weight rows norms all the activation rows again (608 blocks do the work of 8), and
    # that costs more than the launch it saves (about 2 us: a step without any norm is 0.12 to 0.15 ms shorter).
    FOLD_MAX_ROWS = int(os.environ.get("STARTER_B200_FOLD_MAX_ROWS", 0))

    def folds(self, rows: int, dtype) -> bool:
        """Whether a step of this many rows should hand its norms and residual sums to ``linear`` and
        ``linear_swiglu`` (``norm=``, ``add_to=``).  The decode product can take them for bfloat16, up to 16 rows
        and inner sizes that are multiples of 8."""
        return dtype == torch.bfloat16 and rows <= min(self.FOLD_MAX_ROWS, self.SKINNY_MAX_ROWS, 16)

    def _can_fold(self, rows: int, dtype, K: int) -> bool:
        return dtype == torch.bfloat16 and rows <= min(self.SKINNY_MAX_ROWS, 16) and K % 8 == 0

    def _skinny(self, a, w, n_out, gate_up, out_float32, norm=None, add_to=None):
        """The weight-streaming product for a handful of rows (see gemm_skinny.cuh).

        norm: (weight, eps) or (weight, eps, stats) of an RMSNorm to take of a's rows first; stats is what the product
        that wrote a left behind (below), without it every block reads the rows once more.
        add_to: a bfloat16 [M, n_out] tensor that the product is added to, or an object with such a tensor as ``x``
        and a field ``stats`` (a residual stream), which then receives the statistics of the new rows: the sums of
        squares of each 16 columns, [M, ceil(n_out / 16)] floats."""
        M, K = a.shape
        blocks = -(-n_out // 16)
        want = self.skinny_splits(blocks, K) if self.force_skinny is None else self.force_skinny[0]
        k_per_split = -(-K // want // 128) * 128 if want > 1 else -(-K // 128) * 128
        n_splits = -(-K // k_per_split)
        nt = -(-M // 8)   # activation tiles of 8 rows
        key = ("gemm_skinny", a.device, nt, n_out, n_splits, gate_up)
        buf = self._scratch.get(key)
        if buf is None:
            floats = blocks * n_splits * (2 if gate_up else 1) * 16 * 8 * nt if n_splits > 1 else 1
            buf = (torch.empty(floats, dtype=torch.float32, device=a.device),
                   torch.zeros(blocks, dtype=torch.int32, device=a.device))
            self._scratch[key] = buf
        stats_out = None
        if add_to is not None:
            out = add_to.x if hasattr(add_to, "stats") else add_to
            if out_float32 or out.dtype != torch.bfloat16 or tuple(out.shape) != (M, n_out) or not out.is_contiguous():
                raise KernelError(f"the product adds to a contiguous bfloat16 [{M}, {n_out}] tensor")
            if out is not add_to:
                stats_out = torch.empty((M, blocks), dtype=torch.float32, device=a.device)
        else:
            out = torch.empty((M, n_out), dtype=torch.float32 if out_float32 else torch.bfloat16, device=a.device)
        warps = self.skinny_warps(blocks * n_splits, -(-M // 8)) if self.force_skinny is None or len(self.force_skinny) < 3 else self.force_skinny[2]
        copy = getattr(w, "_sb_tiled", None)
        if copy is not None and (copy[1] != (2 if gate_up else 1) or (self.force_skinny is not None and not self.force_skinny[1])):
            copy = None   # tiled for the other pairing of rows, or a test asks for the row-major path
        src = copy[0] if copy is not None else w
        tail = (M, n_out, K, n_splits, k_per_split, int(gate_up), int(out_float32), int(copy is not None), warps,
                int(add_to is not None), _ptr(stats_out), _ptr(buf[0]), _ptr(buf[1]), self._stream())
        if norm is None:
            self._check(self.lib.sb_gemm_skinny(_ptr(a), _ptr(src), _ptr(out), *tail), "gemm_skinny")
        else:
            gamma, eps, stats = norm if len(norm) == 3 else (*norm, None)
            if M > 16 or gamma.dtype != torch.bfloat16 or gamma.numel() != K:
                raise KernelError(f"the norm folded into a product takes up to 16 rows and a bfloat16 weight of {K} values")
            if stats is not None and (stats.dtype != torch.float32 or tuple(stats.shape) != (M, -(-K // 16))):
                raise KernelError(f"the rows' statistics are [{M}, {-(-K // 16)}] floats, not {tuple(stats.shape)} {stats.dtype}")
            self._check(self.lib.sb_gemm_skinny_normed(_ptr(a), _ptr(gamma), float(eps), _ptr(stats), _ptr(src), _ptr(out),
                                                       *tail), "gemm_skinny_normed")
        if stats_out is not None:
            add_to.stats = stats_out
        return out

    def linear(self, a, w, out_float32=False, norm=None, add_to=None):
        """a [M, K] times w [N, K] transposed -> [M, N] in a's dtype, or 32-bit when asked.

        float32: this library's CUDA-core product, always.  bfloat16: the weight-streaming kernels for up
        to 16 rows (and for the output head up to 64), cuBLAS for larger products, the CUDA-core product for what is left.

        norm=(weight, eps[, statistics]): the product of the RMSNorm of a's rows; add_to=x: x += product, in place, x
        returned (see ``_skinny``).  Both for bfloat16 and up to 16 rows: the decode product takes them in its prologue
        and epilogue; ``folds`` says whether that pays."""
        M, K = a.shape
        N = w.shape[0]
        if w.shape[1] != K or a.dtype != w.dtype:
            raise KernelError(f"linear: a is {tuple(a.shape)} {a.dtype}, w is {tuple(w.shape)} {w.dtype}")
        if norm is not None or add_to is not None:
            if not self._can_fold(M, a.dtype, K):
                raise KernelError(f"linear: no folded norm or sum for {M} rows of {K} {a.dtype} values")
            return self._skinny(a, w, N, False, out_float32, norm, add_to)
        if a.dtype == torch.bfloat16 and K % 8 == 0:
            if self._takes_stream(M, N, K, False):
                return self._stream_product(a, w, N, False, out_float32)
            if M <= self.SKINNY_MAX_ROWS:
                return self._skinny(a, w, N, False, out_float32)
            if M * N * K > self.GENERAL_GEMM_MAX_WORK:
                if out_float32:
                    return torch.mm(a, w.t(), out_dtype=torch.float32)
                return torch.mm(a, w.t())
        out = torch.empty((M, N), dtype=torch.float32 if out_float32 else a.dtype, device=a.device)
        self._check(self.lib.sb_gemm_general(_code(a.dtype), int(out_float32 or a.dtype == torch.float32), _ptr(a), _ptr(w),
                                             _ptr(out), M, N, K, self._stream()), "gemm_general")
        return out

    def linear_swiglu(self, h, w_gate_up, norm=None):
        """swiglu(h @ w_gate_up^T) for a fused [gate; up] matrix: [M, K] -> [M, rows / 2].  norm: as in ``linear``."""
        M, K = h.shape
        if norm is not None:
            if not self._can_fold(M, h.dtype, K) or h.dtype != w_gate_up.dtype:
                raise KernelError(f"linear_swiglu: no folded norm for {M} rows of {K} {h.dtype} values")
            return self._skinny(h, w_gate_up, w_gate_up.shape[0] // 2, True, False, norm)
        if h.dtype == torch.bfloat16 and w_gate_up.dtype == torch.bfloat16 and K % 8 == 0:
            if self._takes_stream(M, w_gate_up.shape[0] // 2, K, True):
                return self._stream_product(h, w_gate_up, w_gate_up.shape[0] // 2, True, False)
            if M <= self.SKINNY_MAX_ROWS:
                return self._skinny(h, w_gate_up, w_gate_up.shape[0] // 2, True, False)
        return self.swiglu(self.linear(h, w_gate_up))

    # ---- attention ----------------------------------------------------------------------

    def qk_norm_rope_store(self, ctx, qkv, layer_cache, n_heads, n_kv_heads, head_dim, q_norm, k_norm, eps, rotary):
        dt = _code(qkv.dtype)
        wdt = _code(q_norm.dtype) if q_norm is not None else dt
        if qkv.shape[1] != (n_heads + 2 * n_kv_heads) * head_dim:
            raise KernelError("qk_norm_rope_store: qkv has the wrong width")
        if head_dim > 512:
            raise KernelError(f"qk_norm_rope_store takes head sizes up to 512, not {head_dim}")
        q = torch.empty((qkv.shape[0], n_heads * head_dim), dtype=qkv.dtype, device=qkv.device)
        cos = sin = None
        rotary_dim = 0
        if rotary is not None:
            cos, sin, rotary_dim = rotary
            if cos.dtype != qkv.dtype or cos.shape[1] * 2 != rotary_dim:
                raise KernelError("qk_norm_rope_store: rotary tables do not fit the run")
            if cos.shape[0] < ctx.kv_bound:
                raise KernelError(f"the rotary table covers {cos.shape[0]} positions, the step reaches {ctx.kv_bound}")
        kv = self._kv(layer_cache)
        if kv.head_dim != head_dim or (n_kv_heads and kv.n_kv_heads != n_kv_heads):
            raise KernelError("qk_norm_rope_store: the layer's cache has other head sizes than the mixer")
        self._check(self.lib.sb_qk_rope_store(dt, wdt, _ptr(qkv), _ptr(q), self._batch(ctx), kv, n_heads, n_kv_heads,
                                              _ptr(q_norm), _ptr(k_norm), eps, _ptr(cos), _ptr(sin), rotary_dim,
                                              _ptr(ctx.status), self._stream()), "qk_rope_store")
        return q

    def sm_count(self) -> int:
        if self._sm_count is None:
            self._sm_count = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
        return self._sm_count

    def decode_resident(self, head_dim: int) -> int:
        """Blocks of the split-key decode attention that the GPU holds at once (two per SM at head size 128:
        100 KB of shared memory each)."""
        return (2 if head_dim > 64 else 4) * self.sm_count()

    def decode_splits(self, n_seqs: int, n_kv_heads: int, max_pages: int, head_dim: int = 128) -> int:
        """How many blocks share one (sequence, kv head).  Measured on a B200 at a context of 4,096 with 8 kv heads,
        in the whole decode step (ms a step for splits 2 / 4 / 6 / 8 / 16):
          batch 1 (8 pairs):   - / 2.32 / 2.18 / 2.13 / 2.16        batch 2 (16 pairs): 2.68 / 2.30 / 2.19 / 2.60 / 2.28
          batch 4 (32 pairs): - / 2.38 / 2.41 (5) / 2.79 / 2.71     batch 8 (64 pairs): 2.80 / 2.81 / 3.14 / 3.39 / 3.51
          batch 16 (128 pairs): 2 splits 3.80, 3 splits 4.16        batch 32 (256 pairs): 1 split 5.33, 2 splits 5.50
        About 64 to 128 blocks in all is best while the pairs are few (every block then has an SM and the deeper
        pipeline to itself, and a share pays its fixed costs once: loading the queries, merging the warps, meeting
        the other shares); clusters of 7 or 8 blocks are slow as soon as there are 16 or more of them (7 splits at
        batch 2: 2.65 ms), so beyond 8 pairs a pair has 6 splits at most.  A function of shapes only, so that a
        captured graph stays valid as sequences grow."""
        if os.environ.get("STARTER_B200_ATTN_SPLITS"):   # a tuning override; the kernel refuses what its merge cannot hold
            return max(1, min(int(os.environ["STARTER_B200_ATTN_SPLITS"]), 256))
        pairs = max(n_seqs * n_kv_heads, 1)
        if pairs <= 8:
            want = 8 if max_pages <= 96 else 16     # a cache of 16,384 tokens a sequence: 2.44 ms with 16, 2.65 with 8
        elif pairs <= 16:
            want = 6
        elif pairs <= 32:
            want = 4
        elif pairs <= 64:
            want = 4 if max_pages <= 96 else 2      # batch 8 at 16,384 tokens: 4.83 ms with 2, 4.99 with 4, 5.78 with 8
        else:
            want = 256 // pairs
        return max(1, min(want, max_pages, self.decode_resident(head_dim) // pairs))

    def _decode_scratch(self, device, n_seqs, n_heads, n_kv_heads, head_dim, n_splits):
        key = ("attn_decode", device, n_seqs, n_heads, n_kv_heads, head_dim, n_splits)
        buf = self._scratch.get(key)
        if buf is None:
            floats = max(n_seqs * n_heads * n_splits * (head_dim + 2), 1)
            buf = (torch.empty(floats, dtype=torch.float32, device=device),
                   torch.zeros(n_seqs * n_kv_heads, dtype=torch.int32, device=device))
            self._scratch[key] = buf
        return buf

    def _decode_route(self, ctx, kv, n_heads):
        """Which decode kernel serves a step of one token per sequence (bfloat16 cache with head size 64 or 128, at most
        16 query heads per kv head): "split" (a grid of (sequence, kv head, split), the blocks handed out by the
        hardware as others end) or "balanced" (one block per SM, equal shares of all pages, worked out on the device
        from the lengths); None when the step is of another kind.

        Measured alone at 4B sizes with sequences of equal length (us, balanced / split with one block per pair):
        batch 64 at context 2,048: 95.8 / 87.9, at 4,096: 168.3 / 163.8; batch 128 at 2,048: 175 / 169; batch 256 at 1,024:
        191 / 173; in the step at batch 64: 8.50 / 8.36 ms.  The balanced kernel pays ~6 us before its first page and its
        blocks end up to 10 us apart; blocks handed out one by one even that out by themselves.  With very unequal
        lengths (``ctx.uneven``: the longest sequence more than three times the mean) the split kernel, whose blocks per
        pair are a matter of shapes, leaves the longest sequence to a few blocks, and the balanced kernel takes over at
        every batch size.  One sequence of 16,384 tokens among others of 256 (us, split / balanced): batch 8: 81 / 27,
        batch 16: 83 / 34, batch 32: 153 / 41, batch 64: 162 / 43; one of 4,096: 18 / 20, 27 / 21, 45 / 28, 53 / 34."""
        if kv.head_dim not in (64, 128) or n_heads % kv.n_kv_heads or n_heads // kv.n_kv_heads > 16:
            return None
        if not (ctx.max_q_len == 1 and ctx.n_rows == ctx.n_seqs):
            return None
        if self.force_decode_route is not None:
            return self.force_decode_route
        if self.decode_balanced and getattr(ctx, "uneven", False) and ctx.n_seqs <= 1024:
            return "balanced"
        return "split"

    def uneven_matters(self, n_seqs: int) -> bool:
        """Whether a decode step of this many sequences would run other kernels when its context says ``uneven``
        (so that a caller who keeps captured graphs need not keep two alike)."""
        return self.force_decode_route is None and self.decode_balanced and 2 <= n_seqs <= 1024

    def _split_decode(self, ctx, kv, n_heads) -> bool:
        return self._decode_route(ctx, kv, n_heads) == "split"

    def _balanced_scratch(self, device, ctx, kv, n_heads):
        grid = min(self.sm_count(), 512)
        key = ("attn_decode_balanced", device, ctx.n_seqs, n_heads, kv.n_kv_heads, kv.head_dim, grid)
        buf = self._scratch.get(key)
        if buf is None:
            pairs = ctx.n_seqs * kv.n_kv_heads
            floats = (pairs + grid) * (n_heads // kv.n_kv_heads) * (kv.head_dim + 2)
            buf = self._scratch[key] = (torch.empty(floats, dtype=torch.float32, device=device),
                                        torch.zeros(pairs, dtype=torch.int32, device=device))
        return grid, buf

    def qk_attention(self, ctx, qkv, layer_cache, n_heads, n_kv_heads, head_dim, q_norm, k_norm, eps, rotary, scale, window,
                     then=None):
        """qk_norm_rope_store and attention in one kernel, for the steps that the split-key decode kernel serves and a
        rotary encoding over the whole head (or none).  Returns None when the step is not of that kind: the caller then
        makes the two calls."""
        if not self.fuse_qk or qkv.dtype != torch.bfloat16 or layer_cache.group.k.dtype != torch.bfloat16:
            return None
        kv = self._kv(layer_cache)
        route = self._decode_route(ctx, kv, n_heads)
        if kv.head_dim != head_dim or (n_kv_heads and kv.n_kv_heads != n_kv_heads) or route is None:
            return None
        if route == "balanced" and not self.fuse_qk_balanced:
            return None
        if qkv.shape[1] != (n_heads + 2 * n_kv_heads) * head_dim:
            raise KernelError("qk_attention: qkv has the wrong width")
        cos = sin = None
        if rotary is not None:
            cos, sin, rotary_dim = rotary
            if rotary_dim != head_dim or cos.dtype != torch.bfloat16:
                return None
            if cos.shape[1] * 2 != rotary_dim:
                raise KernelError("qk_attention: rotary tables do not fit the run")
            if cos.shape[0] < ctx.kv_bound:
                raise KernelError(f"the rotary table covers {cos.shape[0]} positions, the step reaches {ctx.kv_bound}")
        norm_f32 = 0
        for w in (q_norm, k_norm):
            if w is not None:
                if w.dtype not in (torch.float32, torch.bfloat16):
                    return None
                norm_f32 = int(w.dtype == torch.float32)
        if q_norm is not None and k_norm is not None and q_norm.dtype != k_norm.dtype:
            return None
        # `then`: the matrix that the next product streams; the kernel asks for it into L2 as it finishes its keys
        next_w, next_bytes = None, 0
        if then is not None and self.prefetch_next_bytes > 0 and then.dtype == torch.bfloat16:
            copy = getattr(then, "_sb_tiled", None)
            src = copy[0] if copy is not None and ctx.n_rows <= self.SKINNY_MAX_ROWS else then
            next_w, next_bytes = c_void_p(src.data_ptr()), min(src.numel() * 2, self.prefetch_next_bytes) & ~15
        fused = SbFusedQK(_ptr(qkv), _ptr(q_norm), _ptr(k_norm), _ptr(cos), _ptr(sin), _ptr(ctx.status), float(eps), norm_f32,
                          int(n_kv_heads > 0), 0, next_w, next_bytes)
        out = torch.empty((qkv.shape[0], n_heads * head_dim), dtype=qkv.dtype, device=qkv.device)
        if route == "balanced":
            grid, buf = self._balanced_scratch(qkv.device, ctx, kv, n_heads)
            self._check(self.lib.sb_attn_decode_balanced_fused(fused, _ptr(out), self._batch(ctx), kv, n_heads, scale,
                                                               int(window or 0), grid, _ptr(buf[0]), _ptr(buf[1]),
                                                               self._stream()), "attn_decode_balanced_fused")
            return out
        n_splits = self.decode_splits(ctx.n_seqs, kv.n_kv_heads, layer_cache.group.table_width, kv.head_dim)
        partial, counters = self._decode_scratch(qkv.device, ctx.n_seqs, n_heads, kv.n_kv_heads, kv.head_dim, n_splits)
        self._check(self.lib.sb_attn_decode_fused(fused, _ptr(out), self._batch(ctx), kv, n_heads, scale, int(window or 0),
                                                  n_splits, _ptr(partial), _ptr(counters), self._stream()), "attn_decode_fused")
        return out

    def attention(self, ctx, q, layer_cache, n_heads, scale, window):
        """Causal attention of the step's rows over the layer's cache.  bfloat16 with head size 64 or
        128: the split-key decode kernel for steps of one token per sequence, the flash kernel for
        everything else.  Other head sizes and float32 take the general kernel."""
        out = torch.empty_like(q)
        kv = self._kv(layer_cache)
        if kv.head_dim > 256:
            raise KernelError(f"attention takes head sizes up to 256, not {kv.head_dim}")
        if n_heads % kv.n_kv_heads:
            raise KernelError(f"{n_heads} query heads cannot share {kv.n_kv_heads} key/value heads evenly")
        if q.dtype == torch.bfloat16 and kv.head_dim in (64, 128):
            decode = ctx.max_q_len == 1 and ctx.n_rows == ctx.n_seqs and n_heads // kv.n_kv_heads <= 16
            split = decode and self._split_decode(ctx, kv, n_heads)
            if decode and not split:
                # More pairs than blocks fit at once: one block per SM, each with an equal share of all pages.
                grid, buf = self._balanced_scratch(q.device, ctx, kv, n_heads)
                self._check(self.lib.sb_attn_decode_balanced(_ptr(q), _ptr(out), self._batch(ctx), kv, n_heads, scale,
                                                             int(window or 0), grid, _ptr(buf[0]), _ptr(buf[1]),
                                                             self._stream()), "attn_decode_balanced")
            elif split:
                g = layer_cache.group
                n_splits = self.decode_splits(ctx.n_seqs, kv.n_kv_heads, g.table_width, kv.head_dim)
                partial, counters = self._decode_scratch(q.device, ctx.n_seqs, n_heads, kv.n_kv_heads, kv.head_dim, n_splits)
                self._check(self.lib.sb_attn_decode(_ptr(q), _ptr(out), self._batch(ctx), kv, n_heads, scale,
                                                    int(window or 0), n_splits, _ptr(partial), _ptr(counters),
                                                    self._stream()), "attn_decode")
            elif (self.prefill_tensor_memory and kv.head_dim == 128
                  and ctx.max_q_len * (n_heads // kv.n_kv_heads) >= 128):
                # long pieces at head size 128: the tcgen05 kernel (S and O in tensor memory, TMA for keys and values)
                self._check(self.lib.sb_attn_prefill_tc(_ptr(q), _ptr(out), self._batch(ctx), kv, n_heads, scale,
                                                        int(window or 0), ctx.max_q_len, layer_cache.group.pool_pages + 1,
                                                        _ptr(self.kernel_status(q.device)), self._stream()), "attn_prefill_tc")
            else:
                self._check(self.lib.sb_attn_prefill(_ptr(q), _ptr(out), self._batch(ctx), kv, n_heads, scale,
                                                     int(window or 0), ctx.max_q_len, self._stream()), "attn_prefill")
            return out
        self._check(self.lib.sb_attention_general(_code(q.dtype), _ptr(q), _ptr(out), self._batch(ctx), kv,
                                                  n_heads, scale, int(window or 0), self._stream()), "attention_general")
        return out

    # ---- sampling -----------------------------------------------------------------------

    def argmax(self, logits):
        rows = logits.shape[0]
        out = torch.empty(rows, dtype=torch.int32, device=logits.device)
        key = ("argmax", logits.device, rows)
        buf = self._scratch.get(key)
        if buf is None:
            buf = self._scratch[key] = (torch.empty(rows * 32, dtype=torch.float32, device=logits.device),
                                        torch.empty(rows * 32, dtype=torch.int32, device=logits.device))
        self._check(self.lib.sb_argmax(_ptr(logits), _ptr(out), rows, logits.shape[1], _ptr(buf[0]), _ptr(buf[1]),
                                       self._stream()), "argmax")
        return out

    def sample(self, logits, temperature, top_k, seed, request_ids, steps, advance=False, device_params=None):
        """``device_params``: int32 [4] on the device {temperature's float bits, top_k, seed low, seed high};
        when given, the kernel reads them there as it runs (a captured step then serves every setting)."""
        out = torch.empty(logits.shape[0], dtype=torch.int32, device=logits.device)
        self._check(self.lib.sb_sample(_ptr(logits), _ptr(out), logits.shape[0], logits.shape[1], float(temperature),
                                       int(top_k), int(seed) & ((1 << 64) - 1), _ptr(request_ids), _ptr(steps),
                                       int(bool(advance)), _ptr(device_params), self._stream()), "sample")
        return out


_OPS = None


def get_ops(verbose: bool = True) -> Ops:
    """The extension's call table.  Raises if there is no CUDA device or the library cannot be built."""
    global _OPS
    if _OPS is None:
        if not torch.cuda.is_available():
            raise BuildError("no CUDA device: this library runs on a B200 only and has no other path")
        _OPS = Ops(load(verbose=verbose))
    return _OPS
