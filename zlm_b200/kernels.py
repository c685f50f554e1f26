"""Python face of the CUDA kernel library (``csrc/*.cu`` -> ``libzlm_b200.so``).

Every method takes torch tensors that already live on the GPU, checks what the
kernel cannot check itself (dtype, contiguity, shapes), and launches on torch's
current stream.  There is no CPU path: constructing ``CudaKernels`` without the
library or without a GPU raises.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_void_p
from typing import Optional

import torch

F32, BF16 = 0, 1
PAGE_TOKENS = 64

_DT = {torch.float32: F32, torch.bfloat16: BF16}

STORE, ACCUM, STORE_F32, SWIGLU = 0, 1, 2, 3
GATED_LIMIT = 8          # g sigmoid(alpha g) (u + 1) on clamped halves; its two constants are set before the product
GATED_GELU = 7      # as SWIGLU with gelu_tanh(gate) instead of silu(gate)


class KernelError(RuntimeError):
    pass


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """[2I, K] with rows 8 gate, 8 up, 8 gate, ...: the layout ``linear_swiglu`` wants."""
    I, K = gate.shape
    assert up.shape == (I, K) and I % 8 == 0
    return torch.stack([gate.view(I // 8, 8, K), up.view(I // 8, 8, K)], dim=1).reshape(2 * I, K).contiguous()


def attention_len_bucket(max_len: int) -> int:
    """The longest sequence of a step in pages, rounded up: powers of two up to 8, then
    multiples of 8.  The decode attention sizes its grid by it, so a captured decode step
    holds for every step with the same bucket."""
    pages = (max_len + PAGE_TOKENS - 1) // PAGE_TOKENS
    bucket = 1
    while bucket < pages and bucket < 8:
        bucket *= 2
    if bucket < pages:
        bucket = (pages + 7) // 8 * 8
    return bucket


DECODE_BLOCKS_PER_SM = 3      # blocks of the decode attention that an SM holds at a time


def decode_splits(rows: int, nkv: int, len_bucket: int, blocks: int = 148 * DECODE_BLOCKS_PER_SM):
    """How the decode attention cuts a sequence's pages: (splits, pages per split).
    ``len_bucket`` is the longest sequence of the step in pages, rounded up, so that the
    choice (and a captured graph) holds for many steps; ``blocks`` is what the device holds
    at a time (its SMs x 3).

    A block's start (the query, its first pages) and end (merging its warps, writing its
    partial result) cost about as much as several pages, and one block streams a page in
    about 0.8 us however idle the memory is (two pages in flight).  Timed inside whole decode
    steps (Qwen3-8B and 0.6B sizes, contexts 2,048 and 4,095; timed alone, kernel after
    kernel, fewer and longer parts look better than they are in a step, where every block's
    first two pages are loaded while the kernels before still run):
    - more (token, kv head) pairs than the device holds blocks (batch 64 at 8 kv heads): parts
      for two waves of blocks (at 2,100 tokens 5.7 TB/s with two waves against 5.5 with four and
      4.6 with sixteen; one part a pair 113 us against 95), one wave for short sequences;
    - otherwise one part for every block the device holds, parts of at least two pages, and no
      second wave of blocks (a few blocks over, 448 on 444 places at batch 8, cost nothing in a
      step while the parts are of up to 12 pages; 224 pairs cut in two parts of 25 pages cost
      a step 5 %): so from 223 pairs on there is one part and no combine (batch 32: a step 5 to 7 %
      shorter than with two waves; batch 16 at 4,095 tokens 2 to 3 % shorter with three parts
      than with seven);
    - up to 32 pairs (batch 1 to 4 at 8 kv heads) the parts' own chains of pages bound the kernel
      and the combine reads every part: as many parts as give half of what the device holds, of
      at least 4 pages (2 for sequences of up to 16 pages, 8 at 32 pairs): batch 1 at 4,095
      tokens 16 parts of 4 pages instead of 32 of 2, a step 3 % (8B sizes) to 7 % (0.6B) shorter."""
    pairs = max(1, rows * nkv)
    if pairs > blocks:
        work = len_bucket * pairs
        waves = 2 if work >= 16 * blocks else 1
        per = max(2, -(-work // (blocks * waves)))
    elif pairs <= 32:
        wanted = -(-(blocks // 2) // pairs)
        least = 8 if pairs == 32 else (2 if len_bucket <= 16 else 4)
        per = max(least, -(-len_bucket // wanted))
    else:
        per = max(2, -(-len_bucket * pairs // blocks))
        # (a few blocks over, 64 pairs x 7 on 444 places, are let be where the parts are short; four
        # blocks of 25 pages that start when the first places come free cost a step 5 %)
        while per < len_bucket and -(-len_bucket // per) * pairs * 10 > blocks * (11 if per <= 12 else 10):
            per += 1
    per = min(per, max(1, len_bucket))
    splits = -(-len_bucket // per)
    while splits > 1024:
        per *= 2
        splits = -(-len_bucket // per)
    return splits, per


def latent_decode_splits(rows: int, tiles: int, len_bucket: int, wave: int):
    """How the latent attention's decode step cuts a sequence's pages: (splits, pages per split).  A page of
    records is several times a page of one kv head's keys, a block holds two of them in flight and an SM holds
    few such blocks (``wave``: what the device holds at a time), so a block's own chain of pages is what a
    step waits for: as many splits as fill one wave, of two pages at least (one more kernel, the combine, reads
    every split's partial result)."""
    pairs = max(1, rows * tiles)
    per = max(2, -(-len_bucket * pairs // max(1, wave)))
    per = min(per, max(1, len_bucket))
    splits = -(-len_bucket // per)
    while splits > 1024:
        per *= 2
        splits = -(-len_bucket // per)
    return splits, per


def _dt(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise KernelError(f"unsupported dtype {t.dtype}") from None


def _span_bytes(t: torch.Tensor) -> int:
    """Bytes from the tensor's first element to the end of its last one."""
    if t.numel() == 0:
        return 0
    last = sum((n - 1) * st for n, st in zip(t.shape, t.stride()))
    return (last + 1) * t.element_size()


# what a status code's family byte stands for (tc_common.cuh: TC_FAMILY)
_STATUS_FAMILY = {1: "tcgen05 product", 2: "tcgen05 prefill attention"}


class CudaKernels:
    """Loads (building first if needed) the kernel library and exposes its entry
    points.  One instance per process is enough; see ``get_kernels``."""

    name = "cuda"

    def __init__(self, verbose_build: bool = True, variant: str = ""):
        from .csrc.build import library_path
        self.variant = variant
        self.lib_path = library_path(verbose=verbose_build, variant=variant)
        self.lib = ctypes.CDLL(self.lib_path)
        self.lib.zlm_last_error.restype = ctypes.c_char_p
        self.lib.zlm_launch_count.restype = ctypes.c_longlong
        if self.lib.zlm_page_tokens() != PAGE_TOKENS:
            raise KernelError("kernel library and Python disagree on the cache page size")
        if not torch.cuda.is_available():
            raise KernelError("zlm_b200 needs a CUDA GPU (sm_100a); none is visible and there is no CPU path")
        # binds the status block (pinned host memory the kernels report to) for every part of
        # the library; it copies to device symbols, so it happens here, outside any capture
        if self.lib.zlm_runtime_init() != 0:
            raise KernelError(self.lib.zlm_last_error().decode())
        self.lib.zlm_bounds_first_address.restype = ctypes.c_ulonglong
        self.bounds_check = bool(self.lib.zlm_bounds_check_build())
        self._ranges = []
        # blocks the decode attention cuts its work for; None: what the device holds at a time
        self.decode_blocks: Optional[int] = None
        self.sm_count = int(torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count)
        self._fn = {}
        self._shares = None            # (output, scratch, shares, accumulate) of a product left in shares of K (see linear)
        self.defer_shares = True       # whether linear(defer=True) may leave a product so
        self._candidates = None        # (address of the last logits a few-token product wrote, rows, width, blocks, values, indices)
        # An RMSNorm between two streaming products without a kernel of its own (see ``expect_norm``):
        self.lazy_norms = True         # whether that may happen at all
        self._norm_hint = None         # the weight of the norm that is to follow the next product into the stream
        self._norm_halves = None       # (stream, rows times weight, sums of squares, blocks, weight): a product left them
        self._lazy_ok = False          # the next norm's output is read by products only (the arrangement's word)
        self._lazy = None              # (out, stream, weight, eps, rows times weight, sums of squares, blocks): a norm not run
        self._blank = None             # a tensor that is to be taken as zeros (see expect_blank)
        self.gated_activations = ("silu", "gelu_tanh", "swish_limit")      # what linear_swiglu's ``act`` takes
        self._scratch = {}
        self.scratch_generation = 0
        self._launches = 0

    def scratch(self, name: str, n: int, dtype: torch.dtype, device) -> torch.Tensor:
        """Scratch memory that a kernel needs beyond its operands.  It grows when asked for
        more and keeps its address otherwise; ``scratch_generation`` counts the moves, so
        that a captured graph that holds an old address is not replayed."""
        buf = self._scratch.get(name)
        if buf is None or buf.numel() < n or buf.dtype != dtype or buf.device != device:
            self._scratch[name] = buf = torch.empty(max(n, 1 << 16), dtype=dtype, device=device)
            self.scratch_generation += 1
        return buf

    def launches(self) -> int:
        """Kernels that the library has launched so far (those captured into a graph are counted
        once, when they are captured)."""
        return int(self.lib.zlm_launch_count())

    # -- plumbing ---------------------------------------------------------
    def _call(self, name: str, *args):
        fn = self._fn.get(name)
        if fn is None:
            fn = getattr(self.lib, name)
            fn.restype = c_int
            self._fn[name] = fn
        if self.bounds_check:
            self._register_ranges()
        rc = fn(*args)
        self._launches += 1
        if rc != 0:
            raise KernelError(self.lib.zlm_last_error().decode())
        if self.bounds_check:
            self.check_bounds(name)

    def _p(self, t: Optional[torch.Tensor]) -> c_void_p:
        """The tensor's address as a kernel argument.  In the bounds-check build the bytes it
        spans are also noted as memory the next call may touch."""
        if t is None:
            return c_void_p(0)
        if self._shares is not None:
            # a product whose shares of K are not added up yet: whoever touches its output gets it finished first
            lo, n = self._shares[0].data_ptr(), _span_bytes(self._shares[0])
            if t.data_ptr() < lo + n and lo < t.data_ptr() + _span_bytes(t):
                noted, self._ranges = self._ranges, []      # (this happens while a call's arguments are gathered)
                self.flush_shares()
                self._ranges = noted
        if self._lazy is not None or self._norm_halves is not None:
            self._touch_norms(t)
        if self._blank is not None and self._overlap(t, self._blank):
            blank, self._blank = self._blank, None
            blank.zero_()           # somebody other than the expected product comes first: the zeros are made real
        if self.bounds_check:
            self._ranges.append((t.data_ptr(), _span_bytes(t)))
        return c_void_p(t.data_ptr())

    @staticmethod
    def _overlap(a: torch.Tensor, b: torch.Tensor) -> bool:
        return a.data_ptr() < b.data_ptr() + _span_bytes(b) and b.data_ptr() < a.data_ptr() + _span_bytes(a)

    def _touch_norms(self, t: torch.Tensor) -> None:
        """A kernel is about to be given ``t``.  Halves of a norm that a product left are void once anything
        else touches the stream they belong to.  A norm that was not run is run now if ``t`` is its output;
        if ``t`` is its stream, the part that was to read the output has gone on to write (the arrangement
        said that it reads before it writes and nobody reads afterwards), and the norm is forgotten."""
        if self._norm_halves is not None and self._overlap(t, self._norm_halves[0]):
            self._norm_halves = None
        if self._lazy is not None:
            if self._overlap(t, self._lazy[0]):
                noted, self._ranges = self._ranges, []      # (this happens while a call's arguments are gathered)
                self.finish_norm()
                self._ranges = noted
            elif self._overlap(t, self._lazy[1]):
                self._lazy = None

    def expect_norm(self, weight: Optional[torch.Tensor]) -> None:
        """An arrangement's word that ``rmsnorm`` with this weight is the next reader of the stream after
        the next product into it (``linear(..., accumulate=True, defer=True)``); None takes it back.  A
        streaming product (up to 16 tokens) then also leaves the normed rows but for their scale, and
        the rows' sums of squares block by block; ``rmsnorm`` launches nothing, and the streaming
        products that read its output take the scale from those sums and apply it to their own sums.
        Two launches fewer a layer in a decode step.  Whatever else is given the norm's output through this
        class has the norm run first (``finish_norm``), so the word is never wrong, only sometimes
        useless; code that reads it by other means says so beforehand (``norm_output_read_by_products``)."""
        self._norm_hint = weight if self.lazy_norms else None

    def norm_output_read_by_products(self, yes: bool) -> None:
        """An arrangement's word on the next ``rmsnorm``: its output is read only through this class,
        before the reading part writes into the stream, and by nobody after that.  Holds for one call."""
        self._lazy_ok = bool(yes) and self.lazy_norms

    def forget_pending(self) -> None:
        """Drops what one call left for a later one (shares of K, a norm's halves, a norm not run, the
        arrangement's words) without finishing any of it: for the start of a step, where anything still
        pending belongs to a step that was given up."""
        self._shares = self._norm_hint = self._norm_halves = self._lazy = self._blank = None
        self._lazy_ok = False

    def finish_norm(self) -> None:
        """Runs a norm that ``rmsnorm`` left to the products after it."""
        if self._lazy is None:
            return
        out, x, w, eps = self._lazy[:4]
        self._lazy = None
        R, H = out.shape
        self._call("zlm_rmsnorm", self._p(out), c_int(_dt(out)), self._p(x), self._p(w), c_int(_dt(w)),
                   self._p(None), c_int(R), c_int(H), c_float(eps), self._stream())

    def _register_ranges(self) -> None:
        lib = self.lib
        if lib.zlm_bounds_clear_ranges() != 0:
            raise KernelError(lib.zlm_last_error().decode())
        for base, n in self._ranges:
            if n and lib.zlm_bounds_add_range(c_void_p(base), ctypes.c_ulonglong(n)) != 0:
                raise KernelError(lib.zlm_last_error().decode())
        self._ranges = []

    def check_bounds(self, what: str = "") -> None:
        """Bounds-check build: waits for the device and raises if a kernel asked for memory
        outside the tensors it was given (the access itself was skipped)."""
        torch.cuda.synchronize()
        n = int(self.lib.zlm_bounds_violations())
        if n:
            site = int(self.lib.zlm_bounds_first_site())
            addr = int(self.lib.zlm_bounds_first_address())
            self.lib.zlm_bounds_reset()
            raise KernelError(f"{what}: {n} accesses outside the tensors passed; the first at address "
                              f"{addr:#x}, source file id {site >> 16} line {site & 0xffff}")

    # -- the status word ----------------------------------------------------
    def status(self, sync: bool = False) -> int:
        """0, or the mark of the first bounded wait inside a kernel that gave up:
        (kernel family << 8) | place of the wait.  The word lives in pinned host memory
        that the GPU writes directly, so reading it costs nothing and waits for nothing;
        it tells of the kernels that have finished (``sync`` waits for all of them first)."""
        if sync:
            torch.cuda.synchronize()
        return int(self.lib.zlm_status())

    def clear_status(self) -> None:
        self.lib.zlm_status_clear()

    def check_status(self, sync: bool = False) -> None:
        """Raises if a kernel's bounded wait gave up: what that kernel computed, and
        everything after it, is not to be trusted.  The word is cleared, so that the
        caller may go on (the GPU and the library remain usable)."""
        code = self.status(sync)
        if code:
            self.clear_status()
            family = _STATUS_FAMILY.get(code >> 8, f"kernel family {code >> 8}")
            raise KernelError(f"a bounded wait inside a {family} kernel gave up (place {code & 0xff}, "
                              f"status {code:#x}): results since the last check are not valid")

    @staticmethod
    def _stream() -> c_void_p:
        return c_void_p(torch.cuda.current_stream().cuda_stream)

    def check_linear(self, what: str, w: torch.Tensor) -> None:
        """Raises at once, with the weight's name, if no kernel takes a product with this
        weight [N, K]: the bf16 kernels read 16 bytes (8 elements) of a row at a time."""
        if w.dtype == torch.bfloat16 and w.shape[1] % 8 != 0:
            raise KernelError(f"{what} [{w.shape[0]}, {w.shape[1]}]: the bfloat16 kernels need an inner size "
                              f"that is a multiple of 8 (run this model with dtype float32)")

    # -- kernels ----------------------------------------------------------
    def embed(self, out: torch.Tensor, table: torch.Tensor, ids: torch.Tensor) -> None:
        """out[t, :] = table[ids[t], :] widened to fp32."""
        T, H = out.shape
        assert out.dtype == torch.float32 and ids.dtype == torch.int32 and table.shape[1] == H
        assert out.is_contiguous() and table.is_contiguous()
        self._call("zlm_embed", self._p(out), self._p(table), c_int(_dt(table)),
                   self._p(ids), c_int(T), c_int(H), c_int(table.shape[0]), self._stream())

    def rmsnorm(self, out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, eps: float,
                rows: Optional[torch.Tensor] = None) -> None:
        """out[r] = x[rows[r] or r] * rsqrt(mean(x^2) + eps) * w; x is the fp32 stream."""
        R, H = out.shape
        assert x.dtype == torch.float32 and x.shape[1] == H and w.shape == (H,)
        assert out.is_contiguous() and x.is_contiguous() and w.is_contiguous()
        assert rows is None or (rows.dtype == torch.int32 and rows.numel() >= R)
        halves, self._norm_halves = self._norm_halves, None
        ok, self._lazy_ok = self._lazy_ok, False
        if (halves is not None and ok and rows is None and out.dtype == torch.bfloat16
                and halves[0].data_ptr() == x.data_ptr() and tuple(halves[0].shape) == (R, H)
                and halves[4].data_ptr() == w.data_ptr()):
            # the product before left this norm's halves and only streaming products read ``out``: nothing to launch
            self._lazy = (out, x, w, float(eps)) + tuple(halves[1:4])
            return
        self._lazy = None
        taken = self._takes_shares(x, ACCUM) if (rows is None and x.shape[0] == R) else None
        if taken is not None:
            self._call("zlm_rmsnorm_shares", self._p(out), c_int(_dt(out)), self._p(x), self._p(w), c_int(_dt(w)),
                       c_int(R), c_int(H), c_float(eps), self._p(taken[0]), c_int(taken[1]), self._stream())
            return
        self._call("zlm_rmsnorm", self._p(out), c_int(_dt(out)), self._p(x),
                   self._p(w), c_int(_dt(w)), self._p(rows), c_int(R), c_int(H),
                   c_float(eps), self._stream())

    def swiglu(self, out: torch.Tensor, gu: torch.Tensor) -> None:
        """out[t, i] = silu(gu[t, i]) * gu[t, I + i]."""
        T, I = out.shape
        assert gu.shape == (T, 2 * I) and gu.dtype == out.dtype
        assert out.is_contiguous() and gu.is_contiguous()
        self._call("zlm_swiglu", self._p(out), self._p(gu), c_int(_dt(out)),
                   c_int(T), c_int(I), self._stream())

    def linear(self, out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, accumulate: bool = False,
               impl: Optional[str] = None, defer: bool = False) -> None:
        """out = x @ w.T (out in x's dtype, or fp32), or out += x @ w.T into the fp32
        residual stream when ``accumulate``.  w is [N, K] row-major and is not written by any kernel
        of the same step (in a decode step the products' first loads of w do not wait for the kernels
        before them).  bf16 products pick
        their kernel by the number of tokens: "gemv" (register-fragment streaming, up to
        8), "tc" (TMA + tcgen05, from 9 on), "mma" (mma.sync, what the others do not take);
        ``impl`` forces one (tests).

        ``defer``: the caller expects ``rmsnorm`` (for a product into the stream) or
        ``qk_norm_rope_write`` (for a q/k/v projection) to read ``out`` next.  A few-token product
        that cuts K into shares may then leave them to that kernel, which adds them up on its way
        (two launches fewer per layer at 17 to 64 tokens); any other use of ``out`` through this
        class finishes the product first, so the hint is never wrong, only sometimes useless."""
        T, K = x.shape
        N = w.shape[0]
        if self._candidates is not None and self._candidates[0] == out.data_ptr():
            self._candidates = None         # whatever writes this tensor now, the old candidates are not its
        assert w.shape[1] == K and out.shape == (T, N) and w.dtype == x.dtype
        assert x.stride(1) == 1 and out.stride(1) == 1 and w.is_contiguous()
        ldx, ldy = x.stride(0), out.stride(0)
        if accumulate:
            assert out.dtype == torch.float32
            blank = self._blank
            if (blank is not None and blank.data_ptr() == out.data_ptr() and tuple(blank.shape) == tuple(out.shape)
                    and out.is_contiguous()):
                self._blank = None
                accumulate = defer = False       # adding to zeros: a plain store of the fp32 sums
        if x.dtype == torch.float32:
            assert out.dtype == torch.float32 and ldx == K
            self._call("zlm_gemm_f32", self._p(out), self._p(x),
                       self._p(w), c_int(T), c_int(N), c_int(K), c_int(ldy),
                       c_int(1 if accumulate else 0), self._stream())
            return
        if x.dtype != torch.bfloat16:
            raise KernelError(f"linear: unsupported dtype {x.dtype}")
        mode = ACCUM if accumulate else (STORE_F32 if out.dtype == torch.float32 else STORE)
        if mode == STORE:
            assert out.dtype == torch.bfloat16
        if accumulate and defer:
            hint, self._norm_hint = self._norm_hint, None
            if (hint is not None and impl is None and self.streams_weights(T, N) and out.is_contiguous()
                    and hint.is_contiguous() and tuple(hint.shape) == (N,)):
                self._gemv(out, x, w, T, N, K, ldx, ldy, ACCUM, norm_weight=hint)
                return
        if (defer and self.defer_shares and impl is None and mode in (ACCUM, STORE) and T > 16 and out.is_contiguous()
                and not self.streams_weights(T, N)):
            ks = int(self.lib.zlm_gemm_tc_shares_plan(c_int(T), c_int(N), c_int(K), c_int(ldx)))
            if ks > 1:
                self.flush_shares()
                scratch = self.scratch("gemm_tc.partials", ks * T * N, torch.float32, out.device)
                self._call("zlm_gemm_tc_shares", self._p(x), self._p(w), c_int(T), c_int(N), c_int(K), c_int(ldx),
                           self._p(scratch), self._stream())
                self._shares = (out, scratch, ks, mode)
                return
        self._bf16_product(out, x, w, T, N, K, ldx, ldy, mode, impl)

    def flush_shares(self) -> None:
        """Finishes a product that ``linear(defer=True)`` left in shares of K (its second kernel), and a
        norm that was left to the products after it."""
        self.finish_norm()
        self._norm_halves = None
        if self._shares is None:
            return
        out, scratch, ks, mode = self._shares
        self._shares = None
        T, N = out.shape
        self._call("zlm_gemm_tc_add_shares", self._p(out), self._p(scratch), c_int(T), c_int(N), c_int(out.stride(0)),
                   c_int(mode), c_int(ks), self._stream())

    def _takes_shares(self, t: torch.Tensor, mode: int):
        """The pending shares if they are those of ``t`` (whole, in this mode), else None after finishing them."""
        if self._shares is None:
            return None
        out, scratch, ks, m = self._shares
        if out.data_ptr() == t.data_ptr() and tuple(out.shape) == tuple(t.shape) and out.stride() == t.stride() and m == mode:
            self._shares = None
            return scratch, ks
        return None

    # outputs from which a product counts as "as wide as a vocabulary" (see streams_weights)
    WIDE_PRODUCT = 65536

    def streams_weights(self, tokens: int, N: int) -> bool:
        """Whether a bf16 product of this many tokens and N outputs runs as the register-fragment
        streaming product (else a tcgen05 form).  Measured at Qwen3-8B sizes: it wins up to 16
        tokens (a layer's four products at 9 / 16 tokens: 78 / 84 us against 88 / 90 us), except
        for products as wide as a vocabulary, whose thousand tiles the persistent tcgen05 form
        streams faster from 9 tokens on (191 against 197 to 216 us)."""
        return tokens <= 8 or (tokens <= 16 and N < self.WIDE_PRODUCT)

    def _bf16_product(self, out, x, w, T, N, K, ldx, ldy, mode, impl) -> None:
        if impl is None:
            # few tokens: the streaming product; from 17 tokens on the tcgen05 forms
            tc_ok = self.lib.zlm_gemm_tc_supported(T, N, K, ldx)
            small = self.streams_weights(T, N)
            impl = "gemv" if (small or (T <= 16 and not tc_ok)) else ("tc" if tc_ok else "mma")
        if impl == "tc":
            self.flush_shares()             # the shares' scratch is about to be written again
            ks = self.lib.zlm_gemm_tc_ksplit(T, N, K)
            scratch = self.scratch("gemm_tc.partials", ks * T * N, torch.float32, out.device) if ks > 1 else None
            self._call("zlm_gemm_tc", self._p(out), self._p(x), self._p(w),
                       c_int(T), c_int(N), c_int(K), c_int(ldx), c_int(ldy), c_int(mode), self._p(scratch),
                       self._stream())
            return
        if impl == "gemv":
            self._gemv(out, x, w, T, N, K, ldx, ldy, mode)
            return
        self._call("zlm_gemm_bf16_mma", self._p(out), self._p(x), self._p(w),
                   c_int(T), c_int(N), c_int(K), c_int(ldx), c_int(ldy), c_int(mode), self._stream())

    def _gemv(self, out, x, w, T, N, K, ldx, ldy, mode, norm_weight: Optional[torch.Tensor] = None) -> None:
        """The streaming product, with what it may carry beside its sums: candidates for the argmax of
        logits, the scale of a norm that was not run (``x`` is that norm's output), the halves of the
        norm that follows (``norm_weight``)."""
        lazy = self._lazy
        if not (lazy is not None and lazy[0].data_ptr() == x.data_ptr() and tuple(lazy[0].shape) == (T, K) and ldx == K):
            lazy = None
        nb = int(self.lib.zlm_gemv_blocks(c_int(N)))
        cv = ci = nxt = sq = None
        if mode == STORE_F32 and out.is_contiguous():
            # fp32 outputs of a few-token product are logits: the product also leaves, for every
            # token, the best of each block's 16 outputs, and ``argmax`` of the same tensor picks
            # among those candidates instead of reading the logits again
            cv = self.scratch("gemv.best_values", T * nb, torch.float32, out.device)
            ci = self.scratch("gemv.best_indices", T * nb, torch.int32, out.device)
        if norm_weight is not None:
            nxt = self.scratch("gemv.norm_rows", T * N, torch.bfloat16, out.device)
            sq = self.scratch("gemv.norm_squares", T * nb, torch.float32, out.device)
        # a norm not run: its rows times weight stand in for x, the scale comes from the sums of squares
        px = self._p(lazy[4]) if lazy is not None else self._p(x)
        self._call("zlm_gemv_bf16_norms", self._p(out), px, self._p(w), c_int(T), c_int(N), c_int(K),
                   c_int(ldx), c_int(ldy), c_int(mode), self._p(cv), self._p(ci),
                   self._p(lazy[5]) if lazy is not None else c_void_p(0), c_int(lazy[6] if lazy is not None else 0),
                   c_float(lazy[3] if lazy is not None else 0.0), self._p(norm_weight),
                   c_int(_dt(norm_weight) if norm_weight is not None else 0), self._p(nxt), self._p(sq), self._stream())
        if cv is not None:
            self._candidates = (out.data_ptr(), T, N, nb, cv, ci)
        if norm_weight is not None:
            self._norm_halves = (out, nxt, sq, nb, norm_weight)

    def set_gemm_form(self, form: Optional[str] = None, width: int = 0) -> None:
        """Forces the many-token tcgen05 product's form ("single": one block per tile,
        "pair": two blocks per tile with cta_group::2) and tile width (256, 240, 224; pairs also 128);
        None / 0 give the choice back to the dispatcher.  For tests and measurements."""
        code = {None: 0, "single": 1, "pair": 2}[form]
        if self.lib.zlm_gemm_tc_set_form(c_int(code), c_int(width)) != 0:
            raise KernelError(self.lib.zlm_last_error().decode())

    def set_prefill_attention_heads(self, heads: int = 0) -> None:
        """Forces how many heads of a kv group share a block of the tcgen05 prefill attention
        (1 or 2; 0 gives the choice back to the dispatcher).  For tests and measurements."""
        if self.lib.zlm_attention_prefill_tc_set_heads(c_int(heads)) != 0:
            raise KernelError(self.lib.zlm_last_error().decode())

    def linear_swiglu(self, out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, impl: Optional[str] = None,
                      act: str = "silu", limit: float = 0.0, alpha: float = 1.702) -> None:
        """out[t, c] = act(x[t] . gate_c) * (x[t] . up_c) in one pass over w (bf16).  w is
        [2I, K] with the rows in groups of 16: 8 gate channels, then the 8 matching up
        channels (``interleave_gate_up``); out is [T, I].  ``act``: "silu", "gelu_tanh", or "swish_limit":
        g sigmoid(alpha g) (u + 1) with g = min(gate, limit), u = clamp(up, -limit, limit), whose two constants a
        one-thread kernel hands to the product's translation unit right before it."""
        T, K = x.shape
        N = w.shape[0]
        assert x.dtype == w.dtype == out.dtype == torch.bfloat16 and w.shape[1] == K and N % 16 == 0
        assert out.shape == (T, N // 2) and x.stride(1) == 1 and out.stride(1) == 1 and w.is_contiguous()
        if act == "swish_limit":
            assert limit > 0
            if impl is None:
                tc_ok = self.lib.zlm_gemm_tc_supported(T, N, K, x.stride(0))
                impl = "gemv" if (self.streams_weights(T, N) or (T <= 16 and not tc_ok)) else ("tc" if tc_ok else "mma")
            unit = {"gemv": "gemv_bf16", "tc": "gemm_tcgen05", "mma": "gemm_bf16_mma"}[impl]
            self.flush_shares()
            self._call("zlm_set_gate_" + unit, c_float(limit), c_float(alpha), self._stream())
            self._bf16_product(out, x, w, T, N, K, x.stride(0), out.stride(0), GATED_LIMIT, impl)
            return
        self._bf16_product(out, x, w, T, N, K, x.stride(0), out.stride(0),
                           {"silu": SWIGLU, "gelu_tanh": GATED_GELU}[act], impl)

    def rope_table(self, out: torch.Tensor, inv_freq: torch.Tensor, n_rot: int, token_pos: torch.Tensor) -> None:
        """out [2, n_rot/2, T] fp32: cos and sin of token_pos[t] * inv_freq[i], the step's rotation
        table (the same for every layer with the same frequencies); tokens innermost, so that the
        32 token rows of a warp in the projection's epilogue read neighbouring floats."""
        T = token_pos.shape[0]
        assert out.dtype == torch.float32 and out.is_contiguous() and out.numel() == T * n_rot
        assert inv_freq.dtype == torch.float32 and inv_freq.numel() * 2 == n_rot and token_pos.dtype == torch.int32
        self._call("zlm_rope_table", self._p(out), self._p(inv_freq), c_int(n_rot), self._p(token_pos), c_int(T),
                   self._stream())

    def qkv_rope_supported(self, x: torch.Tensor, w: torch.Tensor, nq: int, nkv: int, hd: int, n_rot: int) -> bool:
        """Whether ``linear_qkv_rope`` takes this step: bf16, many tokens, heads that divide a tile."""
        if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
            return False
        return bool(self.lib.zlm_gemm_tc_qkv_supported(c_int(x.shape[0]), c_int(w.shape[0]), c_int(w.shape[1]),
                                                       c_int(x.stride(0)), c_int(nq), c_int(nkv), c_int(hd), c_int(n_rot)))

    def linear_qkv_rope(self, q_out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, q_w: Optional[torch.Tensor],
                        k_w: Optional[torch.Tensor], eps: float, cos_sin: Optional[torch.Tensor],
                        token_pos: torch.Tensor, token_slot: torch.Tensor, block_table: Optional[torch.Tensor],
                        pool: Optional[torch.Tensor], nq: int, nkv: int, hd: int) -> None:
        """The fused q/k/v projection x @ w.T (w rows [q | k | v]) with its epilogue doing what
        ``qk_norm_rope_write`` does: per-head RMSNorm of q and k, rotation by ``cos_sin`` (from
        ``rope_table``), k and v into the paged pool; q_out [T, nq*hd] receives q.  With nkv == 0
        w holds q rows only."""
        T, K = x.shape
        N = w.shape[0]
        assert q_out.shape == (T, nq * hd) and q_out.dtype == torch.bfloat16 and q_out.stride(1) == 1
        assert w.shape == ((nq + 2 * nkv) * hd, K) and w.is_contiguous() and x.stride(1) == 1
        if nkv:
            assert pool is not None and pool.dtype == torch.bfloat16 and pool.is_contiguous()
            assert tuple(pool.shape[1:]) == (2, nkv, PAGE_TOKENS, hd) and block_table.dtype == torch.int32
        if q_w is not None:
            assert q_w.shape == (hd,) and (nkv == 0 or (k_w is not None and k_w.dtype == q_w.dtype))
        if cos_sin is not None:
            assert cos_sin.dtype == torch.float32 and cos_sin.numel() == T * hd and cos_sin.is_contiguous()
        self._call("zlm_gemm_tc_qkv", self._p(q_out), self._p(x), self._p(w), c_int(T), c_int(N), c_int(K),
                   c_int(x.stride(0)), c_int(q_out.stride(0)), self._p(q_w), self._p(k_w),
                   c_int(_dt(q_w) if q_w is not None else F32), c_float(eps), self._p(cos_sin),
                   self._p(token_pos), self._p(token_slot), self._p(block_table),
                   c_int(block_table.stride(0) if block_table is not None else 0), self._p(pool), c_int(nq), c_int(nkv),
                   c_int(hd), self._stream())

    def qk_norm_rope_write(self, qkv: torch.Tensor, q_w: Optional[torch.Tensor],
                           k_w: Optional[torch.Tensor], eps: float,
                           inv_freq: Optional[torch.Tensor], n_rot: int, token_pos: torch.Tensor,
                           token_slot: torch.Tensor, block_table: Optional[torch.Tensor],
                           pool: Optional[torch.Tensor], nq: int, nkv: int, hd: int,
                           write: bool = True) -> None:
        """On qkv [T, (nq + 2 nkv) hd]: per-head RMSNorm of q and k (if weights are
        given), rotation of q and k by the token's position (if inv_freq is given); q is
        updated in place; with ``write`` k and v go to the token's place in the paged
        pool, without it k is updated in place and v is left alone.  With nkv == 0 only
        q is touched (a layer that reads another layer's cache)."""
        T = qkv.shape[0]
        assert qkv.shape[1] == (nq + 2 * nkv) * hd and qkv.stride(1) == 1
        has_norm = q_w is not None
        if has_norm:
            assert q_w.shape == (hd,) and (nkv == 0 or (k_w is not None and k_w.shape == (hd,) and k_w.dtype == q_w.dtype))
        if inv_freq is not None:
            assert inv_freq.dtype == torch.float32 and inv_freq.numel() * 2 == n_rot
        else:
            n_rot = 0
        write = bool(write and nkv)
        if write:
            assert pool is not None and pool.dtype == qkv.dtype and pool.is_contiguous()
            assert tuple(pool.shape[1:]) == (2, nkv, PAGE_TOKENS, hd)
            assert block_table is not None and block_table.dtype == torch.int32
        taken = self._takes_shares(qkv, STORE) if T < 512 else None
        args = (self._p(qkv), c_int(_dt(qkv)), c_int(qkv.stride(0)),
                self._p(q_w), self._p(k_w), c_int(_dt(q_w) if has_norm else F32),
                c_int(1 if has_norm else 0), c_float(eps), self._p(inv_freq), c_int(n_rot),
                self._p(token_pos), self._p(token_slot),
                self._p(block_table), c_int(block_table.stride(0) if block_table is not None else 0),
                self._p(pool), c_int(nq), c_int(nkv), c_int(hd), c_int(1 if write else 0), c_int(T))
        if taken is not None:
            self._call("zlm_qk_norm_rope_write_shares", *args, self._p(taken[0]), c_int(taken[1]), self._stream())
        else:
            self._call("zlm_qk_norm_rope_write", *args, self._stream())

    def attention(self, out: torch.Tensor, q: torch.Tensor, pool: torch.Tensor, block_table: torch.Tensor,
                  token_pos: torch.Tensor, token_slot: torch.Tensor, nq: int, nkv: int, hd: int,
                  scale: float, window: int, plan=None, len_bucket: Optional[int] = None,
                  v_dim: Optional[int] = None, sink: bool = False, chunk: int = 0, softcap: float = 0.0,
                  sinks: Optional[torch.Tensor] = None, v_share: int = 1) -> None:
        """out[t, h] = softmax(q[t, h] . K * scale) V over the keys [start, pos[t]] of the
        token's slot; q may be a column view of the fused qkv buffer.  ``plan`` is the
        step's context (one token per sequence: the split-KV kernel; whole prompts or
        chunks: the flash kernels; none: the generic kernel); ``len_bucket`` is the longest
        sequence in pages as ``attention_len_bucket`` rounds it (computed if absent).  ``sink``: the
        softmax's denominator is 1 + sum exp(s), as if one more key of score 0 without a value stood
        in every row; ``sinks`` [nq] fp32: that key's score is sinks[h] instead of 0.  ``chunk``: a query sees
        only the keys of its own chunk of that many positions (counted from position 0 of the sequence).
        ``softcap``: scores become softcap * tanh(score / softcap) after the scale.  ``v_share``: that many
        neighbouring key heads read one value head; a page of the pool is then [nkv key heads | nkv / v_share
        value heads] of [PAGE_TOKENS, hd] each (with 1, the ordinary [2, nkv, PAGE_TOKENS, hd])."""
        T = q.shape[0]
        if sinks is not None:
            assert sinks.dtype == torch.float32 and sinks.shape == (nq,) and sinks.is_contiguous()
            sink = True
        sk = c_int(1 if sink else 0)
        assert out.shape == (T, nq * hd) and q.shape[1] == nq * hd and q.dtype == out.dtype == pool.dtype
        assert q.stride(1) == 1 and out.stride(1) == 1 and pool.is_contiguous()
        assert v_share >= 1 and nkv % v_share == 0 and chunk >= 0 and softcap >= 0
        assert pool[0].numel() == (nkv + nkv // v_share) * PAGE_TOKENS * hd and pool.shape[-1] == hd
        extra = (c_int(chunk), c_float(softcap), self._p(sinks), c_int(v_share))
        if (plan is not None and plan.is_decode and q.dtype == torch.bfloat16
                and self.lib.zlm_attention_decode_supported(nq, nkv, hd)):
            if len_bucket is None:
                len_bucket = attention_len_bucket(plan.max_len)
            splits, per = decode_splits(T, nkv, len_bucket, self.decode_blocks or self.sm_count * DECODE_BLOCKS_PER_SM)
            part_o = part_ml = None
            if splits > 1:
                part_o = plan.scratch("attn.part_o", (T * nq * splits * hd,), torch.float32)
                part_ml = plan.scratch("attn.part_ml", (T * nq * splits * 2,), torch.float32)
            # (a decode step writes one position per sequence: every page below that one is from earlier
            # steps, and its load need not wait for the kernel that wrote this step's keys and values)
            self._call("zlm_attention_decode_fresh", self._p(out), c_int(out.stride(0)),
                       self._p(q), c_int(q.stride(0)), self._p(pool),
                       self._p(block_table), c_int(block_table.stride(0)),
                       self._p(token_pos), self._p(token_slot), c_int(T), c_int(nq),
                       c_int(nkv), c_int(hd), c_float(scale), c_int(window), c_int(splits), c_int(per),
                       self._p(part_o), self._p(part_ml), c_int(max(1, int(getattr(plan, "max_new", 1) or 1))),
                       sk, *extra, self._stream())
            return
        if (plan is not None and not plan.is_decode and q.dtype == torch.bfloat16
                and getattr(plan, "cu_seqlens", None) is not None
                and self.lib.zlm_attention_prefill_supported(nq, nkv, hd)):
            impl = getattr(plan, "attention_impl", None)
            if impl != "mma" and self.lib.zlm_attention_prefill_tc_supported(nq, nkv, hd, q.stride(0), out.stride(0)):
                self._call("zlm_attention_prefill_tc", self._p(out), c_int(out.stride(0)),
                           self._p(q), c_int(q.stride(0)), c_int(T), self._p(pool),
                           ctypes.c_longlong(pool.shape[0]), self._p(block_table),
                           c_int(block_table.stride(0)), self._p(plan.cu_seqlens),
                           self._p(plan.seq_slot), self._p(plan.seq_start), c_int(plan.R),
                           c_int(plan.max_new), c_int(nq), c_int(nkv), c_int(hd), c_float(scale), c_int(window),
                           sk, *extra, self._stream())
                return
            if (impl != "mma" and v_dim is not None and v_dim < hd
                    and self.lib.zlm_attention_prefill_tc_vd_supported(nq, nkv, hd, v_dim, q.stride(0), out.stride(0))):
                # keys of 192 over values of 128 on the tcgen05 kernel (out's columns from v_dim on become zeros)
                self._call("zlm_attention_prefill_tc_vd", self._p(out), c_int(out.stride(0)),
                           self._p(q), c_int(q.stride(0)), c_int(T), self._p(pool),
                           ctypes.c_longlong(pool.shape[0]), self._p(block_table),
                           c_int(block_table.stride(0)), self._p(plan.cu_seqlens),
                           self._p(plan.seq_slot), self._p(plan.seq_start), c_int(plan.R),
                           c_int(plan.max_new), c_int(nq), c_int(nkv), c_int(hd), c_int(v_dim), c_float(scale),
                           c_int(window), sk, *extra, self._stream())
                return
            if v_dim is not None and v_dim < hd and self.lib.zlm_attention_prefill_vd_supported(nq, nkv, hd, v_dim):
                # values narrower than keys (their rows in the pool are padded to the keys' width): the padding is
                # neither loaded nor multiplied, and out's columns from v_dim on become zeros
                self._call("zlm_attention_prefill_vd", self._p(out), c_int(out.stride(0)), self._p(q), c_int(q.stride(0)),
                           self._p(pool), self._p(block_table), c_int(block_table.stride(0)), self._p(plan.cu_seqlens),
                           self._p(plan.seq_slot), self._p(plan.seq_start), c_int(plan.R), c_int(plan.max_new), c_int(nq),
                           c_int(nkv), c_int(hd), c_int(v_dim), c_float(scale), c_int(window), sk, *extra, self._stream())
                return
            self._call("zlm_attention_prefill", self._p(out), c_int(out.stride(0)),
                       self._p(q), c_int(q.stride(0)), self._p(pool),
                       self._p(block_table), c_int(block_table.stride(0)),
                       self._p(plan.cu_seqlens), self._p(plan.seq_slot),
                       self._p(plan.seq_start), c_int(plan.R), c_int(plan.max_new), c_int(nq),
                       c_int(nkv), c_int(hd), c_float(scale), c_int(window), sk, *extra, self._stream())
            return
        self._call("zlm_attention_generic", self._p(out), c_int(out.stride(0)),
                   self._p(q), c_int(q.stride(0)), c_int(_dt(q)), self._p(pool),
                   self._p(block_table), c_int(block_table.stride(0)),
                   self._p(token_pos), self._p(token_slot), c_int(T), c_int(nq),
                   c_int(nkv), c_int(hd), c_float(scale), c_int(window), sk, *extra, self._stream())

    # -- short convolution, retention, gated heads (see csrc/short_conv.cu, csrc/retention.cu) --------------
    def conv_norm_write(self, q_out: torch.Tensor, proj: torch.Tensor, conv_w: torch.Tensor, state: Optional[torch.Tensor],
                        plan, block_table: torch.Tensor, pool: torch.Tensor, nq: int, nkv: int, dim: int, vdim: int,
                        taps: int, norm: bool, eps: float) -> None:
        """On the fused projection ``proj`` [T, >= channels] (columns [q: nq*dim | k: nkv*dim | v: nkv*vdim | ...]): a
        causal convolution of ``taps`` taps over time on every channel (``conv_w`` [channels, taps]; the values before a
        step's first token come from ``state`` [slots, taps-1, channels], which is brought up to date afterwards), then
        q and k heads divided by their root mean square over ``dim`` (``norm``); q goes to ``q_out`` [T, nq*hdp], k and v
        to the token's place in the paged ``pool`` [pages, 2, nkv, PAGE_TOKENS, hdp], heads padded with zeros to hdp."""
        T = proj.shape[0]
        hdp = pool.shape[-1]
        C = (nq + nkv) * dim + nkv * vdim
        assert proj.shape[1] >= C and proj.stride(1) == 1 and conv_w.shape == (C, taps) and conv_w.is_contiguous()
        assert q_out.shape == (T, nq * hdp) and q_out.stride(1) == 1 and pool.is_contiguous()
        assert tuple(pool.shape[1:]) == (2, nkv, PAGE_TOKENS, hdp) and block_table.dtype == torch.int32
        assert proj.dtype == conv_w.dtype == q_out.dtype == pool.dtype
        if taps > 1:
            assert state is not None and tuple(state.shape[1:]) == (taps - 1, C) and state.is_contiguous() and state.dtype == proj.dtype
        self._call("zlm_conv_norm_write", self._p(q_out), c_int(q_out.stride(0)), self._p(proj), c_int(proj.stride(0)),
                   self._p(conv_w), self._p(state if taps > 1 else None), c_int(_dt(proj)), self._p(plan.token_pos),
                   self._p(plan.token_slot), self._p(plan.token_seq), self._p(plan.seq_start), self._p(plan.cu_seqlens),
                   self._p(plan.seq_slot), self._p(block_table), c_int(block_table.stride(0)), self._p(pool), c_int(T),
                   c_int(plan.R), c_int(nq), c_int(nkv), c_int(dim), c_int(vdim), c_int(hdp), c_int(taps),
                   c_int(1 if norm else 0), c_float(eps), self._stream())

    def head_gate(self, out: torch.Tensor, o: torch.Tensor, g: torch.Tensor, heads: int, v_dim: int, norm: bool,
                  eps: float, act: str) -> None:
        """out[t, h*v_dim + e] = o[t, h, e] * act(g[t, h*v_dim + e]) for e < v_dim; with ``norm`` every head of o is first
        divided by its root mean square (fp32).  o [T, heads, >= v_dim] may be fp32 whatever the compute dtype and may be
        a view with padded heads; act is "sigmoid" or "silu"; out [T, heads*v_dim] has no padding."""
        T = o.shape[0]
        assert o.dim() == 3 and o.shape[1] == heads and o.shape[2] >= v_dim and o.stride(2) == 1
        assert out.shape == (T, heads * v_dim) and out.stride(1) == 1 and g.shape == (T, heads * v_dim) and g.stride(1) == 1
        assert out.dtype == g.dtype and o.dtype in (out.dtype, torch.float32)
        self._call("zlm_head_gate", self._p(out), c_int(out.stride(0)), self._p(o), c_int(1 if o.dtype == torch.float32 else 0),
                   c_int(o.stride(0)), c_int(o.stride(1)), self._p(g), c_int(g.stride(0)), c_int(_dt(out)), c_int(T),
                   c_int(heads), c_int(v_dim), c_int(1 if norm else 0), c_float(eps), c_int({"sigmoid": 0, "silu": 1}[act]),
                   self._stream())

    # tokens of a sequence from which a step's retention runs in pieces side by side, and the pieces' length
    RETENTION_PIECES_FROM = 256
    RETENTION_PIECE = 64

    def retention(self, o: torch.Tensor, proj: torch.Tensor, q_off: int, k_off: int, v_off: int,
                  inv_freq: Optional[torch.Tensor], n_rot: int, decay: torch.Tensor, state: torch.Tensor, plan,
                  heads: int, dim: int, v_dim: int, k_scale: float, pieces: Optional[bool] = None,
                  cos_sin: Optional[torch.Tensor] = None) -> None:
        """o [T, heads*v_dim] fp32 = S_t^T q_t with S_t = decay_h S_(t-1) + k_t v_t^T per head, q and k rotated (first
        ``n_rot`` coordinates of a head, halves against each other, by pos * inv_freq) and k scaled by ``k_scale``; q, k,
        v are columns of ``proj`` from q_off, k_off, v_off on; ``state`` [slots, heads, dim, v_dim] fp32 holds S between
        steps.  Long prompts run in pieces side by side (``pieces`` forces or forbids that).  ``cos_sin``: the step's
        rotation table [2, n_rot/2, T] (``rope_table``) where a step computes it once for all layers; without it the
        kernel forms cosines and sines itself."""
        T = proj.shape[0]
        assert o.shape == (T, heads * v_dim) and o.dtype == torch.float32 and o.is_contiguous() and proj.stride(1) == 1
        assert state.dtype == torch.float32 and tuple(state.shape[1:]) == (heads, dim, v_dim) and state.is_contiguous()
        assert decay.dtype == torch.float32 and decay.numel() == heads
        if inv_freq is not None and n_rot:
            assert inv_freq.dtype == torch.float32 and inv_freq.numel() * 2 == n_rot
        else:
            n_rot = 0
        if cos_sin is not None:
            assert n_rot and cos_sin.dtype == torch.float32 and cos_sin.is_contiguous() and cos_sin.numel() == T * n_rot
        tail = (c_int(heads), c_int(dim), c_int(v_dim), c_float(k_scale), self._p(cos_sin), c_int(T), self._stream())
        head = (self._p(o), self._p(proj), c_int(proj.stride(0)), c_int(q_off), c_int(k_off), c_int(v_off), c_int(_dt(proj)),
                self._p(inv_freq if n_rot else None), c_int(n_rot), self._p(decay), self._p(state), self._p(plan.cu_seqlens),
                self._p(plan.seq_slot), self._p(plan.seq_start), c_int(plan.R))
        if pieces is None:
            pieces = plan.max_new >= self.RETENTION_PIECES_FROM
        if pieces:
            # as many pieces a sequence as the longest one has (a shorter sequence's last pieces are empty): nothing
            # about the step's sequences has to be carried to the device beyond what the step has there already
            L = self.RETENTION_PIECE
            maxp = (int(plan.max_new) + L - 1) // L
            part = plan.scratch("retention.part_state", (plan.R * maxp * heads * dim * v_dim,), torch.float32)
            self._call("zlm_retention_parts", *head, c_int(maxp), c_int(L), self._p(part), *tail)
            return
        self._call("zlm_retention", *head, *tail[:-1], c_int(int(getattr(plan, "max_new", 0) or 0)), tail[-1])

    def attn_prep(self, q_out: torch.Tensor, proj: torch.Tensor, conv_w: Optional[torch.Tensor], state: Optional[torch.Tensor],
                  plan, block_table: torch.Tensor, pool: torch.Tensor, nq: int, nkv: int, dim: int, vdim: int, taps: int,
                  norm: str, q_w: Optional[torch.Tensor], k_w: Optional[torch.Tensor], eps: float,
                  inv_freq: Optional[torch.Tensor], n_rot: int, rot_scale: float = 1.0) -> None:
        """``conv_norm_write`` in its general form: the convolution is optional (``conv_w`` None), the norm of q and k is
        "none", "unit" (per head, no weight), "head" (per head, weights ``q_w`` / ``k_w`` [dim] shared by the heads) or
        "row" (over all heads of q, and of k, at once, weights [nq*dim] / [nkv*dim]), and the first ``n_rot`` coordinates
        of every q and k head are rotated (i against i + n_rot/2) by pos * inv_freq[i], cosines and sines times
        ``rot_scale``."""
        T = proj.shape[0]
        hdp = pool.shape[-1]
        C = (nq + nkv) * dim + nkv * vdim
        mode = {"none": 0, "unit": 1, "head": 2, "row": 3}[norm]
        assert proj.shape[1] >= C and proj.stride(1) == 1 and q_out.shape == (T, nq * hdp) and q_out.stride(1) == 1
        assert tuple(pool.shape[1:]) == (2, nkv, PAGE_TOKENS, hdp) and pool.is_contiguous() and block_table.dtype == torch.int32
        assert proj.dtype == q_out.dtype == pool.dtype
        if conv_w is not None:
            assert conv_w.shape == (C, taps) and conv_w.is_contiguous() and conv_w.dtype == proj.dtype
            if taps > 1:
                assert state is not None and tuple(state.shape[1:]) == (taps - 1, C) and state.is_contiguous() and state.dtype == proj.dtype
        else:
            taps = 1
        if mode >= 2:
            want_q, want_k = ((dim,), (dim,)) if mode == 2 else ((nq * dim,), (nkv * dim,))
            assert q_w is not None and k_w is not None and tuple(q_w.shape) == want_q and tuple(k_w.shape) == want_k
            assert q_w.dtype == k_w.dtype and q_w.is_contiguous() and k_w.is_contiguous()
        if inv_freq is not None and n_rot:
            assert inv_freq.dtype == torch.float32 and inv_freq.numel() * 2 == n_rot and n_rot <= dim
        else:
            n_rot = 0
        self._call("zlm_attn_prep", self._p(q_out), c_int(q_out.stride(0)), self._p(proj), c_int(proj.stride(0)),
                   self._p(conv_w), self._p(state if (conv_w is not None and taps > 1) else None), c_int(_dt(proj)),
                   self._p(plan.token_pos), self._p(plan.token_slot), self._p(plan.token_seq), self._p(plan.seq_start),
                   self._p(plan.cu_seqlens), self._p(plan.seq_slot), self._p(block_table), c_int(block_table.stride(0)),
                   self._p(pool), c_int(T), c_int(plan.R), c_int(nq), c_int(nkv), c_int(dim), c_int(vdim), c_int(hdp),
                   c_int(taps), c_int(mode), self._p(q_w if mode >= 2 else None), self._p(k_w if mode >= 2 else None),
                   c_int(_dt(q_w) if mode >= 2 else F32), c_float(eps), self._p(inv_freq if n_rot else None), c_int(n_rot),
                   c_float(rot_scale), self._stream())

    def norm_gate(self, out: torch.Tensor, o: torch.Tensor, g: Optional[torch.Tensor], heads: int, v_dim: int, group: str,
                  weight: Optional[torch.Tensor], eps: float, act: str, out_scale: float = 1.0) -> None:
        """out[t, c] = o[t, c] / rms(group of c) * weight * act(g[t, c]) * out_scale for o fp32 [T, heads*v_dim]: ``group``
        "none", "head" (every head of v_dim columns by itself) or "row" (all heads together); ``weight`` None, [v_dim]
        (shared by the heads) or [heads*v_dim]; ``act`` "sigmoid", "silu" or "none" (no gate)."""
        T, N = o.shape
        assert N == heads * v_dim and o.dtype == torch.float32 and o.is_contiguous()
        assert out.shape == (T, N) and out.stride(1) == 1
        a = {"sigmoid": 0, "silu": 1, "none": 2}[act]
        if a != 2:
            assert g is not None and g.shape == (T, N) and g.stride(1) == 1 and g.dtype == out.dtype
        w_rows = 0
        if weight is not None:
            assert weight.is_contiguous() and weight.numel() in (v_dim, N)
            w_rows = 1 if (weight.numel() == N and heads > 1) else 0
        self._call("zlm_norm_gate", self._p(out), c_int(out.stride(0)), self._p(o), self._p(g if a != 2 else None),
                   c_int(g.stride(0) if a != 2 else 0), c_int(_dt(out)), c_int(T), c_int(heads), c_int(v_dim),
                   c_int({"none": 0, "head": 1, "row": 2}[group]), self._p(weight),
                   c_int(_dt(weight) if weight is not None else F32), c_int(w_rows), c_float(eps), c_int(a),
                   c_float(out_scale), self._stream())

    # -- recurrent mixers (see csrc/recurrent.cu) ---------------------------------------------------------------
    # tokens of a sequence from which a step's recurrences run in pieces side by side, and the pieces' length
    RECURRENT_PIECES_FROM = 128
    RECURRENT_PIECE = 32

    def rglru(self, out: torch.Tensor, proj: torch.Tensor, x_off: int, y_off: int, bx: Optional[torch.Tensor],
              by: Optional[torch.Tensor], conv_w: torch.Tensor, conv_b: Optional[torch.Tensor], a_r: torch.Tensor,
              a_i: torch.Tensor, c_r: Optional[torch.Tensor], c_i: Optional[torch.Tensor], lam: torch.Tensor, c_decay: float,
              state: torch.Tensor, plan, width: int, blocks: int, taps: int, out_scale: float = 1.0,
              gates: Optional[torch.Tensor] = None, pieces: Optional[bool] = None) -> None:
        """The real-gated linear recurrent unit behind its convolution.  ``proj`` [T, >= 2*width] holds the x branch from
        column x_off and the y branch from y_off, without their biases ``bx`` / ``by``; u = conv(x + bx) + conv_b (``conv_w``
        [width, taps]); r, i = sigmoid(A u_b + c) with ``a_r`` / ``a_i`` [blocks, width/blocks, width/blocks] (out, in) on the
        blocks of u; a = exp(-c_decay * r * softplus(lam)); S = a S + sqrt(1 - a^2) i u; out [T, width] = S * gelu_tanh(y + by)
        * out_scale in the compute dtype.  ``state`` [slots, taps, width] fp32: row 0 is S, the others the newest x + bx.
        ``gates`` [blocks, 2*width/blocks, width/blocks] (the rows of a_r[b], then of a_i[b]): bfloat16 steps of more than 16
        tokens compute the gates' logits block by block as products of the library with fp32 sums and fp32 output.  Long
        prompts run in pieces side by side (``pieces`` forces or forbids that)."""
        T = proj.shape[0]
        W = width
        dt = proj.dtype
        assert out.shape == (T, W) and out.stride(1) == 1 and out.dtype == dt and proj.stride(1) == 1
        assert state.dtype == torch.float32 and tuple(state.shape[1:]) == (taps, W) and state.is_contiguous()
        bs = W // blocks
        assert conv_w.shape == (W, taps) and conv_w.is_contiguous() and conv_w.dtype == dt
        for m in (a_r, a_i):
            assert m.shape == (blocks, bs, bs) and m.is_contiguous() and m.dtype == dt
        for v in (bx, by, conv_b, c_r, c_i, lam):
            assert v is None or (v.numel() == W and v.is_contiguous() and v.dtype == dt)
        u = plan.scratch("rglru.u", (T, W), torch.float32)
        z = plan.scratch("rglru.z", (T, blocks, 2 * bs), torch.float32)
        max_new = int(getattr(plan, "max_new", 0) or 0)
        if pieces is None:
            pieces = max_new >= self.RECURRENT_PIECES_FROM
        part = None
        if pieces:
            maxp = (max_new + self.RECURRENT_PIECE - 1) // self.RECURRENT_PIECE
            part = plan.scratch("rglru.pieces", (2 * plan.R * maxp * W,), torch.float32)
        by_products = (gates is not None and dt == torch.bfloat16 and T > 16 and bs % 8 == 0 and W % 8 == 0)
        u16 = plan.scratch("rglru.u16", (T, W), dt) if by_products else None

        def call(phase: int) -> None:
            self._call("zlm_rglru", self._p(out), c_int(out.stride(0)), self._p(u), self._p(u16), self._p(z), self._p(proj),
                       c_int(proj.stride(0)), c_int(x_off), c_int(y_off), self._p(bx), self._p(by), self._p(conv_w),
                       self._p(conv_b), self._p(a_r), self._p(a_i), self._p(c_r), self._p(c_i), self._p(lam), c_float(c_decay),
                       self._p(state), c_int(_dt(proj)), self._p(plan.token_pos), self._p(plan.token_slot),
                       self._p(plan.token_seq), self._p(plan.seq_start), self._p(plan.cu_seqlens), self._p(plan.seq_slot),
                       c_int(T), c_int(plan.R), c_int(W), c_int(blocks), c_int(taps), c_float(out_scale), c_int(max_new),
                       self._p(part), c_int(phase), self._stream())
        if not by_products:
            call(0)
            return
        assert gates.shape == (blocks, 2 * bs, bs) and gates.is_contiguous() and gates.dtype == dt
        call(1)
        N, K, ldx, ldy = 2 * bs, bs, W, 2 * W
        if self.bounds_check or not self.lib.zlm_gemm_tc_supported(T, N, K, ldx):
            for b in range(blocks):
                self.linear(z[:, b], u16[:, b * bs:(b + 1) * bs], gates[b])
        else:
            # the same product a block, without the host's work of ``linear`` for each (operands of one tensor each,
            # a block's share found by address)
            self.flush_shares()
            ks = int(self.lib.zlm_gemm_tc_ksplit(T, N, K))
            scratch = self.scratch("gemm_tc.partials", ks * T * N, torch.float32, z.device) if ks > 1 else None
            pz, pu, pg, ps, st = self._p(z).value, self._p(u16).value, self._p(gates).value, self._p(scratch), self._stream()
            for b in range(blocks):
                self._call("zlm_gemm_tc", c_void_p(pz + b * N * 4), c_void_p(pu + b * K * 2), c_void_p(pg + b * N * K * 2),
                           c_int(T), c_int(N), c_int(K), c_int(ldx), c_int(ldy), c_int(STORE_F32), ps, st)
        call(2)

    def lowrank_decay(self, alpha: torch.Tensor, proj: torch.Tensor, lo_off: int, w2: torch.Tensor, b: Optional[torch.Tensor],
                      tau: float) -> None:
        """alpha [T, C] fp32 = sigmoid(w2 lo + b)^(1/tau), lo = ``rank`` columns of proj from lo_off on, w2 [C, rank]."""
        T = proj.shape[0]
        C, rank = w2.shape
        assert alpha.shape == (T, C) and alpha.dtype == torch.float32 and alpha.is_contiguous() and proj.stride(1) == 1
        assert w2.is_contiguous() and w2.dtype == proj.dtype and (b is None or (b.numel() == C and b.dtype == proj.dtype and b.is_contiguous()))
        self._call("zlm_lowrank_decay", self._p(alpha), self._p(proj), c_int(proj.stride(0)), c_int(lo_off), self._p(w2),
                   self._p(b), c_int(_dt(proj)), c_int(T), c_int(C), c_int(rank), c_float(tau), self._stream())

    def linear_attention(self, o: torch.Tensor, proj: torch.Tensor, q_off: int, k_off: int, v_off: int,
                         alpha: Optional[torch.Tensor], head_decay: Optional[torch.Tensor], state: torch.Tensor, plan,
                         heads: int, dim: int, v_dim: int, q_scale: float = 1.0, pieces: Optional[bool] = None) -> None:
        """o [T, heads*v_dim] fp32 = S_t^T q_t with S_t = diag(alpha_t) S_(t-1) + k_t v_t^T per head; q (times ``q_scale``),
        k, v are columns of ``proj`` from q_off, k_off, v_off on; ``alpha`` [T, heads*dim] fp32 gives a decay per token and
        key channel, or ``head_decay`` [heads] fp32 one per head; ``state`` [slots, heads, dim, v_dim] fp32.  Long prompts
        run in pieces of 32 tokens side by side: every piece from a zero state, the pieces' states chained, and a second
        pass that adds what the state before a piece gives its tokens (``pieces`` forces or forbids that)."""
        T = proj.shape[0]
        assert o.shape == (T, heads * v_dim) and o.dtype == torch.float32 and o.is_contiguous() and proj.stride(1) == 1
        assert state.dtype == torch.float32 and tuple(state.shape[1:]) == (heads, dim, v_dim) and state.is_contiguous()
        if alpha is not None:
            assert alpha.shape == (T, heads * dim) and alpha.dtype == torch.float32 and alpha.is_contiguous()
        else:
            assert head_decay is not None and head_decay.dtype == torch.float32 and head_decay.numel() == heads
        max_new = int(getattr(plan, "max_new", 0) or 0)
        if pieces is None:
            pieces = max_new >= self.RECURRENT_PIECES_FROM
        part = None
        if pieces:
            maxp = (max_new + self.RECURRENT_PIECE - 1) // self.RECURRENT_PIECE
            part = plan.scratch("linear_attention.pieces", (plan.R * maxp * heads * dim * (v_dim + 1),), torch.float32)
        self._call("zlm_linear_attention", self._p(o), self._p(proj), c_int(proj.stride(0)), c_int(q_off), c_int(k_off),
                   c_int(v_off), self._p(alpha), self._p(head_decay if alpha is None else None), self._p(state), c_int(_dt(proj)),
                   self._p(plan.seq_slot), self._p(plan.cu_seqlens), c_int(T), c_int(plan.R), c_int(heads), c_int(dim),
                   c_int(v_dim), c_float(q_scale), c_int(max_new), self._p(part), self._stream())

    def scaled_sum(self, out: torch.Tensor, a: torch.Tensor, alpha: float, b: torch.Tensor, beta: float,
                   accumulate: bool = True) -> None:
        """out += alpha a + beta b (or out = ..., also when ``out`` is the tensor that ``expect_blank`` named); fp32
        tensors of one shape."""
        assert out.dtype == a.dtype == b.dtype == torch.float32 and out.shape == a.shape == b.shape
        assert out.is_contiguous() and a.is_contiguous() and b.is_contiguous()
        blank = self._blank
        if blank is not None and blank.data_ptr() == out.data_ptr() and tuple(blank.shape) == tuple(out.shape):
            self._blank = None
            accumulate = False
        self._call("zlm_scaled_sum", self._p(out), self._p(a), c_float(alpha), self._p(b), c_float(beta),
                   ctypes.c_longlong(out.numel()), c_int(1 if accumulate else 0), self._stream())

    def softcap_(self, x: torch.Tensor, cap: float) -> None:
        """x = cap * tanh(x / cap) for a contiguous fp32 tensor (logits)."""
        assert x.dtype == torch.float32 and x.is_contiguous()
        if self._candidates is not None and self._candidates[0] == x.data_ptr():
            self._candidates = None
        self._call("zlm_softcap_f32", self._p(x), ctypes.c_longlong(x.numel()), c_float(cap), self._stream())

    def silu_rows(self, x: torch.Tensor, cols: int) -> None:
        """x[:, :cols] = silu(x[:, :cols]) in place."""
        T = x.shape[0]
        assert x.stride(1) == 1 and 0 <= cols <= x.shape[1]
        self._call("zlm_silu_rows", self._p(x), c_int(x.stride(0)), c_int(_dt(x)), c_int(T), c_int(cols), self._stream())

    def gated_limit(self, out: torch.Tensor, gu: torch.Tensor, limit: float, alpha: float) -> None:
        """out[t, i] = g sigmoid(alpha g) (u + 1) with g = min(gu[t, i], limit), u = clamp(gu[t, I + i], -limit, limit)."""
        T, I = out.shape
        assert gu.shape == (T, 2 * I) and gu.dtype == out.dtype and out.is_contiguous() and gu.is_contiguous()
        self._call("zlm_gated_limit", self._p(out), self._p(gu), c_int(_dt(out)), c_int(T), c_int(I), c_float(limit),
                   c_float(alpha), self._stream())

    # -- latent attention (see csrc/latent_attention.cu) --------------------
    def latent_prep(self, q: torch.Tensor, q_rot: torch.Tensor, dkv: Optional[torch.Tensor],
                    c_weight: Optional[torch.Tensor], eps: float,
                    inv_freq: Optional[torch.Tensor], n_rot: int, token_pos: torch.Tensor, token_slot: torch.Tensor,
                    block_table: Optional[torch.Tensor], pool: Optional[torch.Tensor], heads: int, dim: int,
                    rot_dim: int, kv_rank: int, rec_out: Optional[torch.Tensor] = None) -> None:
        """Per token: the rotated parts of the heads' queries (q [T, heads * (dim + rot_dim)], each head
        [dim | rot_dim]) are turned by the token's position, neighbouring pairs (2i, 2i+1) by
        pos * inv_freq[i], and written to q_rot [T, heads, rot_dim] (any token and head strides; it may
        be the view q[:, :, dim:] itself); and, where ``dkv`` [T, kv_rank + rot_dim] is given, the token's record
        [RMSNorm(dkv[:kv_rank]) * c_weight | rotated dkv[kv_rank:]] goes to its place in the paged
        ``pool`` [pages, PAGE_TOKENS, kv_rank + rot_dim], and also to row t of ``rec_out`` [T, kv_rank + rot_dim] if given."""
        T = q.shape[0]
        assert q.shape[1] == heads * (dim + rot_dim) and q.stride(1) == 1
        assert rec_out is None or (dkv is not None and rec_out.shape == (T, kv_rank + rot_dim) and rec_out.stride(1) == 1
                                   and rec_out.dtype == q.dtype)
        assert q_rot.shape == (T, heads, rot_dim) and q_rot.dtype == q.dtype and (rot_dim == 0 or q_rot.stride(2) == 1)
        if inv_freq is not None:
            assert inv_freq.dtype == torch.float32 and inv_freq.numel() * 2 == n_rot
        else:
            n_rot = 0
        if dkv is not None:
            assert dkv.shape == (T, kv_rank + rot_dim) and dkv.stride(1) == 1 and dkv.dtype == q.dtype
            assert pool is not None and pool.dtype == q.dtype and pool.is_contiguous()
            assert tuple(pool.shape[1:]) == (PAGE_TOKENS, kv_rank + rot_dim) and block_table.dtype == torch.int32
            assert c_weight is not None and c_weight.shape == (kv_rank,) and c_weight.is_contiguous()
        self._call("zlm_latent_prep", self._p(q), c_int(q.stride(0)), self._p(q_rot), c_int(q_rot.stride(0)),
                   c_int(q_rot.stride(1)), self._p(dkv),
                   c_int(dkv.stride(0) if dkv is not None else 0), c_int(_dt(q)), self._p(c_weight if dkv is not None else None),
                   c_int(_dt(c_weight) if dkv is not None else F32), c_float(eps), self._p(inv_freq), c_int(n_rot),
                   self._p(token_pos), self._p(token_slot), self._p(block_table if dkv is not None else None),
                   c_int(block_table.stride(0) if dkv is not None else 0), self._p(pool if dkv is not None else None),
                   c_int(T), c_int(heads), c_int(dim), c_int(rot_dim), c_int(kv_rank), self._p(rec_out),
                   c_int(rec_out.stride(0) if rec_out is not None else 0), self._stream())

    def latent_gather(self, rec: torch.Tensor, pool: torch.Tensor, block_table: torch.Tensor, token_pos: torch.Tensor,
                      token_slot: torch.Tensor) -> None:
        """rec[t] = the record of token t (position token_pos[t] of slot token_slot[t]) from the paged ``pool``."""
        T, R = rec.shape
        assert rec.is_contiguous() and pool.is_contiguous() and rec.dtype == pool.dtype
        assert tuple(pool.shape[1:]) == (PAGE_TOKENS, R) and block_table.dtype == torch.int32
        self._call("zlm_latent_gather", self._p(rec), self._p(pool), self._p(block_table), c_int(block_table.stride(0)),
                   self._p(token_pos), self._p(token_slot), c_int(_dt(rec)), c_int(T), c_int(R), self._stream())

    def latent_unfold(self, spool: torch.Tensor, stable: torch.Tensor, kv: torch.Tensor, rec: torch.Tensor,
                      token_pos: torch.Tensor, token_seq: torch.Tensor, heads: int, dim: int, rot_dim: int, v_dim: int,
                      kv_rank: int) -> None:
        """Per-head keys and values of the step's tokens into a pool of the attention kernels' layout
        [pages, 2, heads, PAGE_TOKENS, dim + rot_dim]: K = [kv[t, h*dim : (h+1)*dim] | rec[t, kv_rank:]],
        V = [kv[t, heads*dim + h*v_dim : ...] | 0]; ``stable`` [sequences of the step, pages] names the pages."""
        T = kv.shape[0]
        hd = dim + rot_dim
        assert kv.shape == (T, heads * (dim + v_dim)) and kv.stride(1) == 1 and rec.shape[0] == T and rec.stride(1) == 1
        assert spool.is_contiguous() and tuple(spool.shape[1:]) == (2, heads, PAGE_TOKENS, hd) and spool.dtype == kv.dtype
        assert stable.dtype == torch.int32 and stable.dim() == 2
        self._call("zlm_latent_unfold", self._p(spool), self._p(stable), c_int(stable.stride(0)), self._p(kv),
                   c_int(kv.stride(0)), self._p(rec), c_int(rec.stride(0)), self._p(token_pos), self._p(token_seq),
                   c_int(_dt(kv)), c_int(T), c_int(heads), c_int(dim), c_int(rot_dim), c_int(v_dim), c_int(kv_rank),
                   self._stream())

    def head_linear(self, out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, impl: Optional[str] = None) -> None:
        """out[t, h, :] = w[h] @ x[t, h, :] for per-head matrices w [heads, N, K]; x [T, heads, K] and out
        [T, heads, N] may be views with any token and head strides (innermost contiguous)."""
        T, H, K = x.shape
        N = w.shape[1]
        assert w.shape == (H, N, K) and w.is_contiguous() and out.shape == (T, H, N)
        assert x.dtype == w.dtype == out.dtype and x.stride(2) == 1 and out.stride(2) == 1
        if (x.dtype == torch.bfloat16 and T > 16 and impl != "plain" and x.data_ptr() % 16 == 0
                and self.lib.zlm_head_linear_mma_supported(c_int(K), c_int(x.stride(0)), c_int(x.stride(1)))):
            # many tokens: tiles of tokens per head on the tensor cores
            self._call("zlm_head_linear_mma", self._p(out), c_int(out.stride(0)), c_int(out.stride(1)), self._p(x),
                       c_int(x.stride(0)), c_int(x.stride(1)), self._p(w), c_int(T), c_int(H), c_int(N), c_int(K),
                       self._stream())
            return
        self._call("zlm_head_linear", self._p(out), c_int(out.stride(0)), c_int(out.stride(1)), self._p(x),
                   c_int(x.stride(0)), c_int(x.stride(1)), self._p(w), c_int(_dt(x)), c_int(T), c_int(H), c_int(N),
                   c_int(K), self._stream())

    def latent_attention(self, out: torch.Tensor, q: torch.Tensor, pool: torch.Tensor, block_table: torch.Tensor,
                         token_pos: torch.Tensor, token_slot: torch.Tensor, heads: int, kv_rank: int, rot_dim: int,
                         scale: float, window: int = 0, plan=None, len_bucket: Optional[int] = None,
                         impl: Optional[str] = None, chunk: int = 0, sinks: Optional[torch.Tensor] = None) -> None:
        """out[t, h, :kv_rank] = sum_j softmax_j(q[t, h] . rec_j * scale) rec_j[:kv_rank] over the records
        [start, pos[t]] of the token's slot in ``pool`` [pages, PAGE_TOKENS, kv_rank + rot_dim]: one
        key/value record per token that every head reads (q [T, heads * (kv_rank + rot_dim)]).  ``plan`` is
        the step's context: with it bf16 steps run on the tensor-core kernel where it takes the sizes (kv_rank
        and rot_dim multiples of 16); without it, in 32-bit, or with ``impl="plain"``, the plain kernel runs.
        Both kernels have both options.
        ``sinks`` [heads] fp32: exp(sinks[h]) joins the softmax's denominator of head h, without a value.  ``chunk``:
        a query sees only the records of its own chunk of that many positions."""
        T = q.shape[0]
        D = kv_rank + rot_dim
        if sinks is not None:
            assert sinks.dtype == torch.float32 and sinks.shape == (heads,) and sinks.is_contiguous()
        assert q.shape[1] == heads * D and out.shape == (T, heads * kv_rank) and q.dtype == out.dtype == pool.dtype
        assert q.stride(1) == 1 and out.stride(1) == 1 and pool.is_contiguous()
        assert tuple(pool.shape[1:]) == (PAGE_TOKENS, D)
        if (q.dtype == torch.bfloat16 and plan is not None and impl != "plain"
                and self.lib.zlm_latent_attention_mma_supported(c_int(heads), c_int(kv_rank), c_int(rot_dim))
                and q.data_ptr() % 16 == 0 and (q.stride(0) * 2) % 16 == 0 and out.stride(0) % 2 == 0):
            # the tensor-core kernel: a decode step cuts the sequences' pages into splits (all heads of a tile
            # share one pass over the records: the head tiles stand where the other attention has kv heads);
            # prompts and portions give a block several neighbouring tokens that share the staged pages
            tiles = (heads + 15) // 16
            if plan.is_decode:
                if len_bucket is None:
                    len_bucket = attention_len_bucket(plan.max_len)
                wave = self.decode_blocks or self.sm_count * int(
                    self.lib.zlm_latent_attention_mma_blocks_per_sm(c_int(kv_rank), c_int(rot_dim)))
                splits, per = latent_decode_splits(T, tiles, len_bucket, wave)
                qt, fresh = 1, max(1, int(getattr(plan, "max_new", 1) or 1))
            else:
                splits, per = 1, max(1, (int(plan.max_len) + PAGE_TOKENS - 1) // PAGE_TOKENS)
                qt, fresh = int(self.lib.zlm_latent_attention_mma_tokens(c_int(kv_rank), c_int(rot_dim))), 0
            part_o = part_ml = None
            if splits > 1:
                part_o = plan.scratch("lat.part_o", (T * heads * splits * kv_rank,), torch.float32)
                part_ml = plan.scratch("lat.part_ml", (T * heads * splits * 2,), torch.float32)
            self._call("zlm_latent_attention_mma", self._p(out), c_int(out.stride(0)), self._p(q), c_int(q.stride(0)),
                       self._p(pool), self._p(block_table), c_int(block_table.stride(0)), self._p(token_pos),
                       self._p(token_slot), c_int(T), c_int(heads), c_int(kv_rank), c_int(rot_dim), c_float(scale),
                       c_int(window), c_int(qt), c_int(splits), c_int(per), self._p(part_o), self._p(part_ml),
                       c_int(fresh), c_int(chunk), self._p(sinks), self._stream())
            return
        self._call("zlm_latent_attention", self._p(out), c_int(out.stride(0)), self._p(q), c_int(q.stride(0)),
                   c_int(_dt(q)), self._p(pool), self._p(block_table), c_int(block_table.stride(0)),
                   self._p(token_pos), self._p(token_slot), c_int(T), c_int(heads), c_int(kv_rank), c_int(rot_dim),
                   c_float(scale), c_int(window), c_int(chunk), self._p(sinks), self._stream())

    # -- the stream of designs that norm a sublayer's output (see csrc/stream_ops.cu) -------------------------
    def embed_scaled(self, out: torch.Tensor, table: torch.Tensor, ids: torch.Tensor, scale: float,
                     pair: Optional[torch.Tensor] = None, buckets: int = 0, mul_prev: int = 0, mul_cur: int = 0,
                     plan=None, prev_state: Optional[torch.Tensor] = None) -> None:
        """out[t] = table[ids[t]] * scale, plus, with a ``pair`` table [buckets + 1, H], the row
        (ids[t-1] * mul_prev + ids[t] * mul_cur) mod buckets (the row ``buckets`` for a sequence's first token).  The
        token before a step's first one comes from ``prev_state`` [slots] int32, which then receives the step's last
        token of every sequence."""
        T, H = out.shape
        assert out.dtype == torch.float32 and ids.dtype == torch.int32 and table.shape[1] == H
        assert out.is_contiguous() and table.is_contiguous()
        if pair is not None:
            assert pair.shape == (buckets + 1, H) and pair.dtype == table.dtype and pair.is_contiguous()
            assert prev_state is not None and prev_state.dtype == torch.int32 and plan is not None
        ll = ctypes.c_longlong
        self._call("zlm_embed_scaled", self._p(out), self._p(table), c_int(_dt(table)), c_float(scale), self._p(pair),
                   c_int(buckets), ll(mul_prev), ll(mul_cur), self._p(ids),
                   self._p(plan.token_pos if pair is not None else None), self._p(plan.token_seq if pair is not None else None),
                   self._p(plan.cu_seqlens if pair is not None else None), self._p(plan.seq_slot if pair is not None else None),
                   self._p(prev_state if pair is not None else None), c_int(T), c_int(H), c_int(table.shape[0]), self._stream())

    def norm_scale_add(self, stream: torch.Tensor, y: torch.Tensor, w: torch.Tensor, eps: float,
                       layer_scale: Optional[torch.Tensor] = None, cast_out: Optional[torch.Tensor] = None) -> None:
        """stream[t] += y[t] / sqrt(mean(y[t]^2) + eps) * w (* layer_scale), in fp32; y fp32 or the compute dtype.
        ``cast_out`` (bfloat16, the stream's shape) receives the stream's new rows rounded once."""
        R, H = stream.shape
        assert stream.dtype == torch.float32 and y.shape == (R, H) and w.shape == (H,)
        assert stream.is_contiguous() and y.is_contiguous() and w.is_contiguous()
        assert layer_scale is None or (layer_scale.shape == (H,) and layer_scale.is_contiguous())
        assert cast_out is None or (cast_out.dtype == torch.bfloat16 and cast_out.shape == (R, H) and cast_out.is_contiguous())
        self._call("zlm_norm_scale_add", self._p(stream), self._p(y), c_int(_dt(y)), self._p(w), c_int(_dt(w)),
                   self._p(layer_scale), c_int(_dt(layer_scale) if layer_scale is not None else F32), c_int(R), c_int(H),
                   c_float(eps), self._p(cast_out), self._stream())

    NORM_ADD_NORM_MAX = 11264        # the widest row the fused pair of norms holds in shared memory

    def norm_add_norm(self, stream: torch.Tensor, y: torch.Tensor, w1: torch.Tensor, eps1: float, out2: torch.Tensor,
                      w2: torch.Tensor, eps2: float) -> None:
        """stream[t] += y[t] / sqrt(mean(y[t]^2) + eps1) * w1, then out2[t] = stream[t] / sqrt(mean(stream[t]^2) + eps2)
        * w2 (the compute dtype): a sublayer's closing norm with its residual add, and the next sublayer's opening norm,
        in one kernel.  y fp32."""
        R, H = stream.shape
        assert stream.dtype == y.dtype == torch.float32 and y.shape == (R, H) and out2.shape == (R, H)
        assert stream.is_contiguous() and y.is_contiguous() and out2.is_contiguous() and H <= self.NORM_ADD_NORM_MAX
        assert w1.shape == (H,) and w2.shape == (H,) and w1.is_contiguous() and w2.is_contiguous()
        self._call("zlm_norm_add_norm", self._p(stream), self._p(y), self._p(w1), c_int(_dt(w1)), c_float(eps1),
                   self._p(out2), c_int(_dt(out2)), self._p(w2), c_int(_dt(w2)), c_float(eps2), c_int(R), c_int(H),
                   self._stream())

    def cast_rows(self, out: torch.Tensor, x: torch.Tensor) -> None:
        """out = x rounded to bfloat16 (x fp32, both contiguous and of one shape)."""
        assert x.dtype == torch.float32 and out.dtype == torch.bfloat16 and out.shape == x.shape
        assert x.is_contiguous() and out.is_contiguous()
        self._call("zlm_cast_rows", self._p(out), self._p(x), ctypes.c_longlong(x.numel()), self._stream())

    def gated_act(self, out: torch.Tensor, gu: torch.Tensor, act: str = "silu") -> None:
        """out[t, i] = act(gu[t, i]) * gu[t, I + i]; act "silu" or "gelu_tanh"."""
        T, I = out.shape
        assert gu.shape == (T, 2 * I) and gu.dtype == out.dtype and out.is_contiguous() and gu.is_contiguous()
        self._call("zlm_gated_act", self._p(out), self._p(gu), c_int(_dt(out)), c_int(T), c_int(I),
                   c_int({"silu": 0, "gelu_tanh": 1}[act]), self._stream())

    def scale_(self, x: torch.Tensor, s: float) -> None:
        """x *= s for a contiguous fp32 tensor (logits times a constant)."""
        assert x.dtype == torch.float32 and x.is_contiguous()
        if self._candidates is not None and self._candidates[0] == x.data_ptr():
            self._candidates = None         # the candidates a few-token product left hold the unscaled values
        self._call("zlm_scale_f32", self._p(x), ctypes.c_longlong(x.numel()), c_float(s), self._stream())

    def head_scalar_gate(self, x: torch.Tensor, g: torch.Tensor) -> None:
        """x[t, h, :] *= sigmoid(g[t, h]) in place; x [T, heads, V] and g [T, heads] may be views (innermost contiguous)."""
        T, H, V = x.shape
        assert g.shape == (T, H) and g.dtype == x.dtype and x.stride(2) == 1 and g.stride(1) == 1
        self._call("zlm_head_scalar_gate", self._p(x), c_int(x.stride(0)), c_int(x.stride(1)), self._p(g), c_int(g.stride(0)),
                   c_int(_dt(x)), c_int(T), c_int(H), c_int(V), self._stream())

    def expect_blank(self, t: Optional[torch.Tensor]) -> None:
        """An arrangement's word that ``t`` (fp32) is to be taken as zeros although it holds anything: the next product
        added into it, ``linear(t, ..., accumulate=True)``, stores instead of adding.  Whatever else is given ``t``
        first through this class has it cleared then, so the word is never wrong."""
        self._blank = t

    def swap_blank(self, t: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """``expect_blank(t)`` that hands back the tensor named before and not yet used up (None if none): for a part that
        runs other parts on blank rows of its own while a word on its own output is still pending, and puts that word
        back afterwards."""
        was, self._blank = self._blank, t
        return was

    # -- differential attention (see csrc/diff_attention.cu) --------------------------------------------------
    def diff_prep(self, q_out: torch.Tensor, proj: torch.Tensor, q_w: torch.Tensor, k_w: torch.Tensor, eps: float,
                  inv_freq: Optional[torch.Tensor], n_rot: int, token_pos: torch.Tensor, token_slot: torch.Tensor,
                  block_table: torch.Tensor, pool: torch.Tensor, heads: int, kv_heads: int, dim: int, vdim: int) -> None:
        """On the fused projection ``proj`` [T, >= (2 heads + 2 kv_heads) dim + kv_heads vdim] (columns [q: heads x 2 maps x
        dim | k: kv_heads x 2 x dim | v: kv_heads x vdim]): every map of q and k is RMS-normed over dim (weights ``q_w``,
        ``k_w``), its neighbouring pairs (2i, 2i+1), i < n_rot/2, are turned by pos * inv_freq[i]; q goes to ``q_out``
        [T, 2 heads, hdp] as query heads (g*2 + m)*rep + j, k and v to the token's place of the paged ``pool``
        [pages, 2 kv_heads key heads + kv_heads value heads, PAGE_TOKENS, hdp], padded with zeros to hdp."""
        T = proj.shape[0]
        hdp = pool.shape[-1]
        assert proj.shape[1] >= (2 * heads + 2 * kv_heads) * dim + kv_heads * vdim and proj.stride(1) == 1
        assert q_out.shape == (T, 2 * heads * hdp) and q_out.stride(1) == 1 and q_out.dtype == proj.dtype == pool.dtype
        assert pool.is_contiguous() and pool[0].numel() == 3 * kv_heads * PAGE_TOKENS * hdp and block_table.dtype == torch.int32
        assert q_w.shape == (dim,) and k_w.shape == (dim,) and q_w.dtype == k_w.dtype and q_w.is_contiguous() and k_w.is_contiguous()
        if inv_freq is not None and n_rot:
            assert inv_freq.dtype == torch.float32 and inv_freq.numel() * 2 == n_rot
        else:
            n_rot = 0
        self._call("zlm_diff_prep", self._p(q_out), c_int(q_out.stride(0)), self._p(proj), c_int(proj.stride(0)),
                   c_int(_dt(proj)), self._p(q_w), self._p(k_w), c_int(_dt(q_w)), c_float(eps),
                   self._p(inv_freq if n_rot else None), c_int(n_rot), self._p(token_pos), self._p(token_slot),
                   self._p(block_table), c_int(block_table.stride(0)), self._p(pool), c_int(T), c_int(heads), c_int(kv_heads),
                   c_int(dim), c_int(vdim), c_int(hdp), self._stream())

    def diff_combine(self, out: torch.Tensor, a: torch.Tensor, heads: int, kv_heads: int, vdim: int, hdp: int, lam: float,
                     post: float, eps: float) -> None:
        """out[t, h, :] = unit_rms(a1 - lam * a2) * post over vdim, where a1, a2 are the attention's outputs of head h's
        two maps in ``a`` [T, 2 heads, hdp] (the order ``diff_prep`` gives the query heads)."""
        T = a.shape[0]
        assert a.shape == (T, 2 * heads * hdp) and out.shape == (T, heads * vdim) and a.dtype == out.dtype
        assert a.stride(1) == 1 and out.stride(1) == 1
        self._call("zlm_diff_combine", self._p(out), c_int(out.stride(0)), self._p(a), c_int(a.stride(0)), c_int(_dt(a)),
                   c_int(T), c_int(heads), c_int(kv_heads), c_int(vdim), c_int(hdp), c_float(lam), c_float(post), c_float(eps),
                   self._stream())

    # -- routed experts (see csrc/moe.cu) -------------------------------------
    def moe_route(self, idx: torch.Tensor, wgt: torch.Tensor, x: torch.Tensor, w_router: torch.Tensor, top: int,
                  gate: Optional[torch.Tensor] = None, w_gate: Optional[torch.Tensor] = None,
                  score: str = "sigmoid", renormalize: bool = False, correction: Optional[torch.Tensor] = None,
                  groups: int = 1, keep: int = 1, weight_scale: float = 1.0, group_top: int = 1) -> None:
        """idx / wgt [T, top]: the experts with the largest scores of W_router x (fp32 logits; ``score``
        "sigmoid" or "softmax") and those scores (divided by their sum if ``renormalize``); gate [T] =
        sigmoid(w_gate . x) where a shared expert has a gate.  ``correction`` (fp32 [E]) is added to the scores for the
        choice only; the experts form ``groups`` equal groups of neighbours of which the ``keep`` with the largest best
        choice score (``group_top`` 2: the largest sum of its two best choice scores) can be chosen; the weights are the
        scores times ``weight_scale``."""
        T, K = x.shape
        E = w_router.shape[0]
        assert w_router.shape == (E, K) and w_router.is_contiguous() and w_router.dtype == x.dtype and x.stride(1) == 1
        assert idx.dtype == torch.int32 and wgt.dtype == torch.float32 and idx.is_contiguous() and wgt.is_contiguous()
        assert idx.shape == (T, top) and wgt.shape == (T, top)
        if w_gate is not None:
            assert w_gate.numel() == K and w_gate.is_contiguous() and w_gate.dtype == x.dtype
            assert gate is not None and gate.dtype == torch.float32 and gate.numel() >= T
        self._call("zlm_moe_route", self._p(idx), self._p(wgt), self._p(gate if w_gate is not None else None), self._p(x),
                   c_int(x.stride(0)), self._p(w_router), self._p(w_gate), c_int(_dt(x)), c_int(T), c_int(E), c_int(K),
                   c_int(top), c_int({"sigmoid": 0, "softmax": 1}[score]), c_int(1 if renormalize else 0),
                   *self._route_extras(correction, E, groups, keep, weight_scale, group_top), self._stream())

    def _route_extras(self, correction, E, groups, keep, weight_scale, group_top=1):
        if correction is not None:
            assert correction.dtype == torch.float32 and correction.shape == (E,) and correction.is_contiguous()
        assert group_top in (1, 2)
        return self._p(correction), c_int(groups), c_int(keep), c_int(group_top), c_float(weight_scale)

    def moe_choose(self, idx: torch.Tensor, wgt: torch.Tensor, logits: torch.Tensor, experts: int, top: int,
                   gate: Optional[torch.Tensor] = None, score: str = "sigmoid", renormalize: bool = False,
                   correction: Optional[torch.Tensor] = None, groups: int = 1, keep: int = 1,
                   weight_scale: float = 1.0, group_top: int = 1) -> None:
        """``moe_route``'s choice from fp32 logits [T, experts (+ 1)] that a product left (column ``experts`` is the
        shared expert's gate logit if ``gate`` is given)."""
        T = logits.shape[0]
        assert logits.dtype == torch.float32 and logits.stride(1) == 1 and logits.shape[1] >= experts + (1 if gate is not None else 0)
        assert idx.dtype == torch.int32 and wgt.dtype == torch.float32 and idx.shape == (T, top) and wgt.shape == (T, top)
        assert idx.is_contiguous() and wgt.is_contiguous()
        self._call("zlm_moe_choose", self._p(idx), self._p(wgt), self._p(gate), self._p(logits), c_int(logits.stride(0)),
                   c_int(T), c_int(experts), c_int(top), c_int(1 if gate is not None else 0),
                   c_int({"sigmoid": 0, "softmax": 1}[score]), c_int(1 if renormalize else 0),
                   *self._route_extras(correction, experts, groups, keep, weight_scale, group_top), self._stream())

    _ACT_KINDS = {"relu2": 0, "swiglu": 1, "swiglu_interleaved": 2}

    def moe_up(self, act: torch.Tensor, x: torch.Tensor, w_up: torch.Tensor, idx: torch.Tensor, wgt: torch.Tensor,
               scale_input: bool = True, activation: str = "relu2") -> None:
        """act[t, j, :] = relu(W_up[idx[t, j]] (wgt[t, j] x[t]))^2 (``scale_input``), or wgt[t, j] * relu(W_up[..] x[t])^2;
        w_up [experts, F, K], act [T, top, F].  ``activation`` "swiglu": w_up is [experts, 2F, K], an expert's gate rows then
        its up rows, and the activation is silu(gate) * up ("swiglu_interleaved": the rows in groups of 8 gate, 8 up).
        A choice of an index from ``experts`` on (an identity expert) writes nothing."""
        T, K = x.shape
        top = idx.shape[1]
        F = act.shape[2]
        kind = self._ACT_KINDS[activation]
        E = w_up.shape[0]
        assert w_up.shape == (E, F * (2 if kind else 1), K) and w_up.is_contiguous() and act.shape == (T, top, F) and act.is_contiguous()
        assert x.dtype == w_up.dtype == act.dtype and x.stride(1) == 1
        self._call("zlm_moe_up", self._p(act), self._p(x), c_int(x.stride(0)), self._p(w_up), self._p(idx), self._p(wgt),
                   c_int(_dt(x)), c_int(T), c_int(top), c_int(F), c_int(K), c_int(1 if scale_input else 0), c_int(kind),
                   c_int(E), self._stream())

    def moe_down(self, stream: torch.Tensor, act: torch.Tensor, w_down: torch.Tensor, idx: torch.Tensor,
                 identity_input: Optional[torch.Tensor] = None, wgt: Optional[torch.Tensor] = None) -> None:
        """stream[t] += sum_j W_down[idx[t, j]] act[t, j]; w_down [experts, N, F], stream fp32 [T, N].  With
        ``identity_input`` x [T, N] and ``wgt``, a choice of an index from ``experts`` on adds wgt[t, j] * x[t]."""
        T, top, F = act.shape
        E, N, _ = w_down.shape
        assert w_down.shape == (E, N, F) and w_down.is_contiguous() and act.is_contiguous() and act.dtype == w_down.dtype
        assert stream.dtype == torch.float32 and stream.shape == (T, N) and stream.is_contiguous()
        x = identity_input
        if x is not None:
            assert x.shape == (T, N) and x.stride(1) == 1 and x.dtype == act.dtype and wgt is not None and wgt.is_contiguous()
        self._call("zlm_moe_down", self._p(stream), self._p(act), self._p(w_down), self._p(idx), c_int(_dt(act)), c_int(T),
                   c_int(top), c_int(F), c_int(N), c_int(E), self._p(x), c_int(x.stride(0) if x is not None else 0),
                   self._p(wgt if x is not None else None), self._stream())

    def moe_grouped(self, stream: torch.Tensor, x: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor,
                    idx: torch.Tensor, wgt: torch.Tensor, scale_input: bool = True, impl: Optional[str] = None,
                    activation: str = "relu2", identity: bool = False) -> None:
        """What ``moe_up`` and ``moe_down`` compute, for steps of many tokens (bf16): the (token, choice) pairs
        are sorted by expert on the device and every expert's rows go through its matrices as tiles of one
        grouped tensor-core product, so an expert's weights are read once per tile, not once per token.  Two
        forms (``impl`` forces one): "tc", TMA + tcgen05 on tiles of 128 rows, where an expert gets about half
        a tile or more; "mma", mma.sync on tiles of 16 to 128 rows, for fewer rows an expert.  ``activation``
        "swiglu_interleaved": w_up is [E, 2F, K], an expert's rows in sixteens of 8 gate and 8 up rows, and the first
        product's epilogue writes silu(gate) * up ("tc" only).  ``identity``: a choice of an index from E on adds
        wgt * x[t] and takes no row of any product."""
        T, K = x.shape
        E, _, F = w_down.shape
        top = idx.shape[1]
        gated = activation == "swiglu_interleaved"
        assert activation in ("relu2", "swiglu_interleaved")
        assert x.dtype == w_up.dtype == w_down.dtype == torch.bfloat16 and x.stride(1) == 1
        assert w_up.shape == (E, F * (2 if gated else 1), K) and w_down.shape == (E, K, F) and w_up.is_contiguous() and w_down.is_contiguous()
        assert stream.dtype == torch.float32 and stream.shape == (T, K) and stream.is_contiguous()
        assert idx.shape == (T, top) and wgt.shape == (T, top) and idx.is_contiguous() and wgt.is_contiguous()
        P = T * top
        if impl is None:
            # rows an expert gets on average: from about half a tile of 128 on, the tcgen05 grouped product
            impl = "tc" if ((P >= 64 * E or gated or identity) and K % 8 == 0 and F % 8 == 0 and x.stride(0) % 8 == 0) else "mma"
        if impl != "tc" and (gated or identity):
            raise KernelError("moe_grouped: gated or identity experts run on the tcgen05 form only (sizes multiples of 8)")
        if impl == "tc":
            # pairs sorted into tiles of 128 rows that start at an expert's first row; the inputs gathered (with the
            # pair's weight, which scales the expert's input) into that order; both products as grouped tcgen05
            # products that look up each token tile's expert; the choices' rows added into the stream in order
            tiles = (P + 127) // 128 + min(E, P)
            rows = tiles * 128
            ints = self.scratch("moe.padded", rows + P + 3 * tiles, torch.int32, x.device)
            xs = self.scratch("moe.padded_x", rows * K, torch.bfloat16, x.device)
            act = self.scratch("moe.padded_act", rows * F, torch.bfloat16, x.device)
            y = self.scratch("moe.padded_out", rows * K, torch.float32, x.device)
            perm, inv, table = ints[:rows], ints[rows:rows + P], ints[rows + P:]
            self._call("zlm_moe_sort_padded", self._p(idx), c_int(P), c_int(E), c_int(tiles), self._p(ints), self._stream())
            self._call("zlm_moe_gather", self._p(xs), self._p(x), c_int(x.stride(0)), self._p(perm), self._p(wgt), c_int(rows),
                       c_int(top), c_int(K), c_int(1 if scale_input else 0), self._stream())
            self._call("zlm_gemm_tc_grouped", self._p(act), self._p(xs), self._p(w_up), self._p(table), c_int(tiles), c_int(E),
                       c_int(2 * F if gated else F), c_int(K), c_int(F), c_int(3 if gated else 6), self._stream())
            self._call("zlm_gemm_tc_grouped", self._p(y), self._p(act), self._p(w_down), self._p(table), c_int(tiles), c_int(E),
                       c_int(K), c_int(F), c_int(K), c_int(2), self._stream())
            self._call("zlm_moe_combine", self._p(stream), self._p(y), self._p(inv), self._p(None if scale_input else wgt),
                       c_int(T), c_int(top), c_int(K), self._p(x if identity else None), c_int(x.stride(0)),
                       self._p(wgt if identity else None), self._stream())
            return
        bm = int(self.lib.zlm_moe_grouped_tile_rows(c_int(P), c_int(E)))
        tiles = int(self.lib.zlm_moe_grouped_max_tiles(c_int(P), c_int(E), c_int(bm)))
        ints = self.scratch("moe.sorted", 2 * P + 3 * tiles, torch.int32, x.device)
        act = self.scratch("moe.sorted_act", P * F, torch.bfloat16, x.device)
        y = self.scratch("moe.sorted_out", P * K, torch.float32, x.device)
        self._call("zlm_moe_grouped", self._p(stream), self._p(x), c_int(x.stride(0)), self._p(w_up), self._p(w_down),
                   self._p(idx), self._p(wgt), c_int(T), c_int(top), c_int(E), c_int(F), c_int(K),
                   c_int(1 if scale_input else 0), self._p(ints), self._p(act), self._p(y), self._stream())

    def relu2_scale(self, out: torch.Tensor, u: torch.Tensor, row_scale: Optional[torch.Tensor] = None) -> None:
        """out[t, i] = relu(u[t, i])^2 * row_scale[t]."""
        T, F = u.shape
        assert out.shape == (T, F) and out.dtype == u.dtype and out.is_contiguous() and u.is_contiguous()
        assert row_scale is None or (row_scale.dtype == torch.float32 and row_scale.numel() >= T)
        self._call("zlm_relu2_scale", self._p(out), self._p(u), self._p(row_scale), c_int(_dt(u)), c_int(T), c_int(F),
                   self._stream())

    def argmax(self, out: torch.Tensor, logits: torch.Tensor, fresh: bool = False) -> None:
        """out[r] = index of the highest logit of row r, ties to the lowest index.  ``fresh``: the
        caller vouches that ``logits`` is what ``linear`` wrote last into this tensor and nothing
        has written it since (the engine's logits on their way to the sampler); the few-token
        product then has left every block's best candidates, and the logits are not read again."""
        R, V = logits.shape
        assert logits.dtype == torch.float32 and logits.stride(1) == 1 and out.dtype == torch.int32
        cand = self._candidates if fresh else None
        if cand is not None and cand[0] == logits.data_ptr() and cand[1] >= R and cand[2] == V and logits.is_contiguous():
            # these logits came from the few-token product just before: it left the candidates
            _, _, _, nb, cv, ci = cand
            self._call("zlm_argmax_candidates", self._p(out), self._p(cv), self._p(ci), c_int(R), c_int(nb), self._stream())
            return
        sv = self.scratch("argmax.values", R * 64, torch.float32, logits.device)
        si = self.scratch("argmax.indices", R * 64, torch.int32, logits.device)
        self._call("zlm_argmax", self._p(out), self._p(logits), c_int(R), c_int(V),
                   c_int(logits.stride(0)), self._p(sv), self._p(si), self._stream())

    def set_pdl(self, on: bool) -> None:
        """Launch the decode-path kernels with programmatic dependent launch (a kernel's
        blocks are scheduled, and its weights start streaming, while the kernel before it
        drains) or in plain stream order."""
        self.lib.zlm_set_pdl(c_int(1 if on else 0))

    def gemm_tc_status(self) -> int:
        """0 unless a bounded wait inside a tcgen05 kernel (product or attention) gave up
        since the status was last cleared (synchronises)."""
        return self.status(sync=True)

    def test_bounded_wait(self, limit_ns: int):
        """Runs the tcgen05 kernels' give-up path on purpose, once, in a one-block kernel
        made of the same helpers (a wait with the limit ``limit_ns`` on a barrier at which
        nobody arrives), and returns (code it reported, other waits released by the abort
        flag, nanoseconds the kernel took, its TMA copy had landed)."""
        src = torch.zeros((128, 64), dtype=torch.bfloat16, device="cuda")
        out = torch.zeros(4, dtype=torch.int32, device="cuda")
        self._call("zlm_test_bounded_wait", self._p(src), self._p(out), ctypes.c_ulonglong(int(limit_ns)),
                   self._stream())
        torch.cuda.synchronize()
        code, released, ns, landed = out.tolist()
        return code, bool(released), ns, bool(landed)

    def sample(self, out: torch.Tensor, logits: torch.Tensor, temperature: float, top_k: int, top_p: float,
               seed: int, request: torch.Tensor, position: torch.Tensor, form: Optional[str] = None) -> None:
        """out[r] = a draw from softmax(logits[r] / temperature) restricted to the top_k
        best and to the nucleus of mass top_p; the uniform of row r is a hash of
        (seed, request[r], position[r]).  ``form`` forces one of the kernel's two forms
        (tests): "cluster" (8 blocks per row, the row in distributed shared memory) or
        "block" (one block per row; rows too long for the cluster form)."""
        R, V = logits.shape
        assert logits.dtype == torch.float32 and logits.stride(1) == 1 and out.dtype == torch.int32
        assert request.dtype == torch.int32 and position.dtype == torch.int32
        self._call("zlm_sample", self._p(out), self._p(logits), c_int(R), c_int(V),
                   c_int(logits.stride(0)), c_float(temperature), c_int(top_k), c_float(top_p),
                   ctypes.c_ulonglong(seed & 0xFFFFFFFFFFFFFFFF), self._p(request),
                   self._p(position), c_int({None: 0, "block": 1, "cluster": 2}[form]), self._stream())


_KERNELS: Optional[CudaKernels] = None
_VARIANT = ""


def set_build_variant(variant: str) -> None:
    """Which build of the library ``get_kernels`` loads: "" (the ordinary one) or "check"
    (the bounds-check build).  To be called before the first ``get_kernels``."""
    global _VARIANT, _KERNELS
    if _KERNELS is not None and _KERNELS.variant != variant:
        raise KernelError("the kernel library is loaded already; choose the build variant before first use")
    _VARIANT = variant


def get_kernels() -> CudaKernels:
    global _KERNELS
    if _KERNELS is None:
        _KERNELS = CudaKernels(variant=_VARIANT)
    return _KERNELS
