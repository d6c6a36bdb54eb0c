"""`CudaKernels`: the product kernel set.  Hand-written CUDA for sm_100a under
`spite_b200/csrc`, compiled in-tree and called through ctypes on the current
torch stream.  There is no other implementation in the package: without a CUDA
device or without the compiled libraries every call raises.
"""
from __future__ import annotations

import collections
import ctypes as C
import math
import os

import torch

from . import build
from .api import KernelError, KernelSet, KernelTimeout, Routing

_DT = {torch.float32: 0, torch.bfloat16: 1}
_STATUS = {-1: "malformed argument", -2: "size not supported by this kernel", -3: "launch failed"}

EPI_STORE, EPI_STORE_F32, EPI_ADD_F32, EPI_SWIGLU = 0, 1, 2, 3
_WINDOW = {"full": 0, "chunk": 1, "sliding": 2}


class GemmParams(C.Structure):
    _fields_ = [("A", C.c_void_p), ("W", C.c_void_p), ("C", C.c_void_p),
                ("a_rows", C.c_void_p), ("c_rows", C.c_void_p), ("group_offsets", C.c_void_p),
                ("row_scale", C.c_void_p),
                ("lda", C.c_longlong), ("ldc", C.c_longlong), ("w_group_stride", C.c_longlong),
                ("n_groups", C.c_int), ("M", C.c_int), ("N", C.c_int), ("K", C.c_int),
                ("epilogue", C.c_int), ("scale_by_a_row", C.c_int)]


class StepTokens(C.Structure):
    _fields_ = [("positions", C.c_void_p), ("seg_of_token", C.c_void_p), ("block_table", C.c_void_p),
                ("table_width", C.c_int), ("n_tokens", C.c_int)]


class PagedCache(C.Structure):
    _fields_ = [("kv", C.c_void_p), ("v_offset", C.c_longlong), ("n_pages", C.c_int),
                ("page_size", C.c_int), ("num_kv_heads", C.c_int), ("head_dim", C.c_int)]


class QkPrepareParams(C.Structure):
    _fields_ = [("qkv", C.c_void_p), ("q_out", C.c_void_p), ("inv_freq", C.c_void_p),
                ("q_gain", C.c_void_p), ("k_gain", C.c_void_p),
                ("qk_norm_eps", C.c_float), ("norm_before_rotation", C.c_int), ("pairing", C.c_int),
                ("rotary_dim", C.c_int), ("temperature_floor", C.c_int),
                ("temperature_scale", C.c_float), ("num_heads", C.c_int), ("write_cache", C.c_int)]


class AttentionParams(C.Structure):
    _fields_ = [("q", C.c_void_p), ("out", C.c_void_p), ("num_heads", C.c_int),
                ("window_kind", C.c_int), ("window_size", C.c_int), ("softmax_scale", C.c_float)]


class AttnMmaExtra(C.Structure):
    _fields_ = [("cu_seqlens", C.c_void_p), ("o_part", C.c_void_p), ("ml_part", C.c_void_p),
                ("n_segments", C.c_int), ("tokens_per_block", C.c_int), ("n_splits", C.c_int),
                ("seg_min_tokens", C.c_int), ("seg_max_tokens", C.c_int)]


class AttnDecodeExtra(C.Structure):
    _fields_ = [("cu_seqlens", C.c_void_p), ("partial", C.c_void_p), ("tickets", C.c_void_p),
                ("n_segments", C.c_int), ("tokens_per_block", C.c_int), ("n_splits", C.c_int),
                ("seg_min_tokens", C.c_int), ("seg_max_tokens", C.c_int), ("cache_settled", C.c_int)]


class SampleParams(C.Structure):
    _fields_ = [("logits", C.c_void_p), ("work", C.c_void_p), ("temperature", C.c_void_p),
                ("top_k", C.c_void_p), ("top_p", C.c_void_p), ("min_p", C.c_void_p),
                ("repetition_penalty", C.c_void_p), ("context", C.c_void_p),
                ("context_offsets", C.c_void_p), ("rng_state", C.c_void_p),
                ("out_tokens", C.c_void_p), ("vocab", C.c_int)]


# Libraries whose kernels wait on mbarriers with a limit.  A kernel that gives up records a code in its
# library's word of one small buffer in pinned host memory, which the device writes directly: the host
# reads it after any point at which it has waited for a step's results, without another copy or wait.
_WAITING_LIBRARIES = ("gemm_tc", "gemm_tc_pair", "gemm_stream", "attention_tc", "attention_decode", "gemm_tc_experts")
_error_words = None          # pinned int32 [len(_WAITING_LIBRARIES)], one per process
_configured: set = set()


def _error_buffer():
    global _error_words
    if _error_words is None:
        _error_words = torch.zeros(len(_WAITING_LIBRARIES), dtype=torch.int32).pin_memory()
    return _error_words


def _ptr(t):
    return None if t is None else t.data_ptr()


def _check(status, what):
    if status != 0:
        raise KernelError(f"{what}: {_STATUS.get(status, f'status {status}')}")


def stream_cut(M: int, N: int, K: int, groups: int, swiglu: bool, slots: int, smem: int, nt: int, *,
               item_cost: float = 2.0, split_item_cost: float = 6.0, split_cost: float = 1.5, slice_cost: float = 1.0,
               max_slices: int = 8, slices_min_rows: int = 4, cluster_max_splits: int = 0, cluster_cost: float = 0.0):
    """(k slices inside a block, k splits across blocks) of the weight-streaming kernel for a product of M rows,
    N output columns (per group) and depth K on `slots` resident blocks of `smem` bytes, `nt` token columns.

    A product of few tiles of 128 rows (a dense projection at a few tokens: 40 to 128 tiles for 296 to 444
    resident blocks) would leave most multiprocessors without work, and the ones that have some are then
    bound by what a single one can pull; so the items are made smaller until they fill the resident blocks
    about once: lower tiles with the k blocks of a stage side by side (the sums meet in shared memory), or k
    splits across blocks (partial sums through global memory, a ticket, a second pass over as many partial
    tiles as there are splits).  The cost of a choice is its rounds of items times (stages an item + what an
    item costs besides, in stages of 16 KiB: `item_cost` for any item, `split_item_cost` + `split_cost` a split
    if its sums cross blocks through global memory, `cluster_cost` if the splits, no more than
    `cluster_max_splits`, can be one thread-block cluster with all clusters resident at once, `slice_cost` if
    its slices meet in shared memory); at least four stages stay together.

    Measured on B200, us, (slices, splits) forced, each product alone.  Eight tokens (444 blocks): qkv 7168 x
    5120: (1, 5) 19.6, (2, 1) 20.9, (4, 1) 17.3, (8, 1) 21.3, (2, 2) 18.9; output projection 5120 x 5120: (1, 7)
    16.5, (4, 1) 14.2, (8, 1) 13.0, (4, 2) 13.1; shared down 5120 x 8192: (1, 7) 21.6, (4, 1) 20.8, (8, 1) 18.6;
    seven experts' gate/up: (1, 1) 220, (1, 2) 199.5, (2, 1) 197.4, (4, 1) 195.5; their down product: (1, 1)
    117.6, (2, 1) 113.5, (4, 1) 107.3, (8, 1) 113.4.  One token (296 blocks with rings twice as deep): slices
    bring nothing, qkv (1, 5) 17.5, (2, 2) 17.0, (4, 1) 19.5; output projection (1, 7) 13.9, (2, 2) 14.1, (4, 1)
    17.1.  In the decode step (ms at 4 / 6 / 8 / 12 / 16 tokens): no slices 4.64 / 5.64 / 6.63 / 8.38 / 9.67;
    slices everywhere 4.89 / 5.85 / 6.51 / 8.68 / 9.45; for one-group products only 4.73 / 5.62 / 6.52 / 8.41 /
    9.53; for the experts' products only 4.76 / 5.83 / 6.63 / 8.68 / 9.60.  The experts' products are faster
    alone with slices and slower in the step: with tiles of 128 rows some blocks end early and the next
    kernel's blocks start under the rest.  So the caller allows slices for one-group products from
    `slices_min_rows` rows on (the kernel set's defaults: six), and tiles of 128 rows otherwise."""
    best, best_cost = (1, 1), None
    for slices in (1, 2, 4, 8):
        if K % (64 * slices) or (swiglu and slices == 8):
            continue
        if slices > 1 and (M < slices_min_rows or slices > max_slices):
            continue
        stage_bytes = 16384 + max(1024, slices * nt * 128)
        if slices > 1 and (smem - 5504 - (8 - 8 // slices) * 64 * nt) // stage_bytes < 2:
            continue                                          # a ring of one stage
        rows = 128 // slices
        tiles = -(-N // (rows // 2 if swiglu else rows)) * groups
        stages = K // (64 * slices)
        for s in range(1, max(1, min(32, stages // 4)) + 1):
            rounds = -(-tiles * s // slots)
            fixed = item_cost + (slice_cost if slices > 1 else 0.0)
            if s > 1 and slices == 1 and s <= cluster_max_splits and tiles * s <= slots:
                fixed += cluster_cost                         # the splits as one cluster: their sums meet in shared memory
            elif s > 1:
                fixed += split_item_cost + split_cost * s
            cost = rounds * (-(-stages // s) + fixed)
            if best_cost is None or cost < best_cost:
                best, best_cost = (slices, s), cost
            if tiles * s >= 4 * slots:
                break
    return best


class CudaKernels(KernelSet):
    def __init__(self, dtype: torch.dtype, device="cuda:0"):
        if dtype not in _DT:
            raise KernelError(f"no kernel set for {dtype}; use torch.bfloat16 or torch.float32")
        if not torch.cuda.is_available():
            raise KernelError("spite_b200 needs a CUDA device (sm_100a); there is no CPU path")
        self.dtype = dtype
        self.device = torch.device(device)
        self._dt = _DT[dtype]
        self._libs = {}
        self.launches = 0          # kernels launched so far (for measurement reports)
        self.attention_scratch_bytes = 0   # partial results of the last split-key attention call
        self.launches_by_library = collections.Counter()   # the same, by kernel library
        self.sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count
        # Which kernel takes which shape.  The numbers are measured choices (what was measured stands beside
        # each); they are plain attributes, so a measurement script can set another value on the object.
        # One switch is read from the environment, for finding a fault: SPITE_NO_TCGEN05=1 keeps every
        # tcgen05 kernel (products and attention) out, and shapes fall to the mma.sync and CUDA-core kernels.
        no_tc = os.environ.get("SPITE_NO_TCGEN05", "") not in ("", "0")
        self.use_tcgen05 = not no_tc
        self.use_tcgen05_attention = not no_tc
        self.attention_tc_min_tokens = 0       # fewest tokens of a request in a step that go to the tcgen05 attention (0: one full tile of rows)
        # most key splits of decode attention: beyond about twenty the merge by the last block costs more than the
        # extra blocks bring (one request at 8,192 keys: 22 us with 37 splits, 17.6 us with 18)
        self.attention_max_splits = 24
        self.use_decode_attention = True       # the TMA-fed decode kernel (head sizes 64 and 128, pages of a multiple of 64 keys)
        # row counts up to which the weight-streaming kernel is preferred over the tcgen05 one
        self.skinny_max_rows = 16
        self.skinny_blocks = 2 * self.sm_count
        # one-group products of at least this many rows run on pairs of multiprocessors
        self.tc_pair_min_rows = 256
        # grouped products with at least this many rows per group on average do too.  Measured at Scout's expert
        # shapes with 512 rows a group: 1324 against 1340 us (gate/up) and 676 against 682 us (down): what the pair
        # saves in shared-memory traffic, the part-filled last tile of 256 rows gives back.
        self.tc_pair_min_group_rows = 512
        self.skinny_tall_rows = 0
        # grouped products with at most this many rows per group on average run with the operands swapped
        self.use_tc_experts = True
        self.tc_experts_max_group_rows = 64
        self.tc_experts_down_min_groups = 64
        # the TMA weight-streaming kernel for decode products
        self.use_stream = True
        # what a work item costs besides its stages, in stages of 16 KiB: any item; one whose sums cross blocks (a
        # fence, a ticket, a second pass: about 2.7 us) and every k split of it; one whose k slices meet in shared memory
        self.stream_item_cost = 2.0
        self.stream_split_item_cost = 6.0
        self.stream_split_cost = 1.5
        self.stream_slice_cost = 1.0
        self.stream_max_slices = 8             # 1: tiles of 128 rows only
        self.stream_slices_min_rows = 6        # products of fewer rows keep tiles of 128 rows (see stream_cut)
        self.stream_slices_grouped = False     # ... and so do grouped products
        self.stream_cluster_max_rows = 3       # up to this many rows the k splits of a tile are a thread-block cluster (0: never)
        # ... if they are no more than this (the hardware takes up to 8).  Measured in the decode step at one / two /
        # three tokens: no clusters 2.780 / 3.348 / 4.114 ms, clusters of two (the gate/up products) 2.748 / 3.335 /
        # 4.079, up to four 2.749 / 3.313 / 4.082, up to eight 2.753 / 3.316 / 4.083; clusters of seven (the 40 tiles of
        # an output projection) are not all resident at once and are refused by the kernel's launcher
        self.stream_cluster_max_splits = 4
        # what such an item costs besides its stages (see stream_cut).  9 (qkv in four splits as clusters, the output
        # and down projections in seven through global memory) against 4, 2, 1 (all three in four): 2.714 against
        # 2.738, 2.727, 2.726 ms at one token
        self.stream_cluster_cost = 9.0
        # one-group products of up to this many rows stream their weights too (16: never; the kernel takes up to 32).
        # Decode step at 20 / 24 / 32 requests: 11.98 / 12.63 / 14.07 ms against 12.17 / 13.07 / 14.30 on tcgen05
        self.stream_max_rows = 32
        self.stream_force = None               # (k slices, k splits) for every call, for measurements
        # (shared memory per block, resident blocks) for up to 3 tokens and for more: measured in the decode step at
        # Scout shapes, one token 2.90 ms with (110 KiB, 2 per multiprocessor) against 3.01 with (74 KiB, 3), eight
        # tokens 7.10 against 7.02, sixty-four alike; one block per multiprocessor with 110 or 200 KiB: 3.2 and 3.1 ms
        self.stream_shape = [(110 * 1024, 2 * self.sm_count), (74 * 1024, 3 * self.sm_count)]
        self._tickets, self._tickets_n = {}, 65536       # arrival counters of the k splits (zero between calls), per stream

    # ------------------------------------------------------------------ helpers
    def _count(self, library, n=1):
        self.launches += n
        self.launches_by_library[library] += n

    def _lib(self, name):
        lib = self._libs.get(name)
        if lib is None:
            lib = self._libs[name] = build.load(name)
            if name in _WAITING_LIBRARIES and name not in _configured:
                word = _error_buffer().data_ptr() + 4 * _WAITING_LIBRARIES.index(name)
                _check(self._configure_waits(lib, name, 0, word, 0), f"{name}: configure_waits")
                _configured.add(name)
        return lib

    @staticmethod
    def _configure_waits(lib, name, limit_cycles, error_word, extra_tx):
        return getattr(lib, f"spite_{name}_configure_waits")(C.c_longlong(limit_cycles), C.c_void_p(error_word),
                                                             C.c_int(extra_tx))

    def configure_waits(self, library: str, *, limit_cycles: int = 0, extra_tx: int = 0):
        """Set the limit (clock cycles; 0: the default of about two seconds) of the bounded waits in
        `library`'s kernels for later launches.  `extra_tx` exists for one test: it makes the first
        barrier of every block of `gemm_tc` incomplete, so that the waits on it run out."""
        lib = self._lib(library)
        word = _error_buffer().data_ptr() + 4 * _WAITING_LIBRARIES.index(library)
        _check(self._configure_waits(lib, library, limit_cycles, word, extra_tx), f"{library}: configure_waits")

    def errors(self) -> dict:
        words = _error_buffer()
        out = {}
        for i, name in enumerate(_WAITING_LIBRARIES):
            code = int(words[i])
            if code:
                out[name] = code
                words[i] = 0
        return out

    @staticmethod
    def _stream():
        return C.c_void_p(torch.cuda.current_stream().cuda_stream)

    def _t(self, t, dtype=None, name="tensor"):
        if t.device.type != "cuda" or not t.is_contiguous():
            raise KernelError(f"{name} must be a contiguous CUDA tensor")
        if dtype is not None and t.dtype != dtype:
            raise KernelError(f"{name} must be {dtype}, is {t.dtype}")
        return t

    # ------------------------------------------------------------------ elementwise
    def embed(self, table, token_ids, out_h, *, scale=1.0):
        self._t(table, self.dtype, "table"); self._t(token_ids, torch.int32, "token_ids")
        self._t(out_h, torch.float32, "out_h")
        V, d = table.shape
        st = self._lib("elementwise").spite_embed(
            self._dt, C.c_void_p(table.data_ptr()), C.c_void_p(token_ids.data_ptr()),
            C.c_void_p(out_h.data_ptr()), token_ids.numel(), d, V, C.c_float(scale), self._stream())
        self._count("elementwise", 1)
        _check(st, "embed")

    def transform_logits(self, logits, *, scale=1.0, softcap=None):
        self._t(logits, torch.float32, "logits")
        st = self._lib("elementwise").spite_transform_logits(
            C.c_void_p(logits.data_ptr()), C.c_longlong(logits.numel()), C.c_float(scale),
            C.c_float(softcap or 0.0), self._stream())
        self._count("elementwise", 1)
        _check(st, "transform_logits")

    def rms_norm(self, h, gain, eps, out, rows=None):
        self._t(h, torch.float32, "h"); self._t(gain, torch.float32, "gain"); self._t(out, None, "out")
        if rows is not None:
            self._t(rows, torch.int32, "rows")
        n, d = out.shape
        st = self._lib("elementwise").spite_rms_norm(
            _DT[out.dtype], C.c_void_p(h.data_ptr()), C.c_void_p(gain.data_ptr()),
            C.c_void_p(_ptr(rows)), C.c_void_p(out.data_ptr()), n, d, C.c_float(eps), self._stream())
        self._count("elementwise", 1)
        _check(st, "rms_norm")

    def clear_pages(self, kv, page_ids):
        self._t(kv, None, "cache")
        if not page_ids:
            return
        caches, two, pages = kv.shape[0], kv.shape[1], kv.shape[2]
        page_bytes = kv.stride(2) * kv.element_size()
        ids = (C.c_int * len(page_ids))(*page_ids)
        st = self._lib("elementwise").spite_clear_pages(
            C.c_void_p(kv.data_ptr()), C.c_longlong(caches * two), C.c_longlong(kv.stride(1) * kv.element_size()),
            C.c_longlong(page_bytes), pages, ids, len(page_ids), self._stream())
        self._count("elementwise", -(-len(page_ids) // 60))
        _check(st, "clear_pages")

    # ------------------------------------------------------------------ matrix products
    def _gemm(self, p: GemmParams, what, max_rows_per_group, gather_src=None):
        """Pick the kernel.  bfloat16: up to 16 rows (a decode step) go to the TMA weight-streaming
        kernel when K is a multiple of 64, else to the register-ring streaming kernel; more rows to
        the tcgen05 kernels (TMA-fed, accumulators in TMEM): one group of 256 rows and more, or groups
        of 512 rows on average, on pairs of multiprocessors, the rest on one block a tile; a very
        tall matrix (output head) goes there even with few rows.  float32, and shapes those refuse, go to the CUDA-core kernel.
        `gather_src` is the tensor whose rows `p.a_rows` gathers: the tcgen05 kernel wants contiguous
        rows, so they are gathered first."""
        if self.dtype == torch.bfloat16:
            grouped = bool(p.group_offsets)
            # measured on B200 at Scout shapes: the streaming kernel wins up to 16 rows except on very
            # tall matrices (output head), where the TMA pipeline of the tcgen05 kernel streams better
            few = p.M <= self.skinny_max_rows and not (not grouped and p.N >= 65536 and p.M > self.skinny_tall_rows)
            tc_ok = self.use_tcgen05 and p.K % 8 == 0 and p.lda % 8 == 0
            # ... and a one-group product of up to 32 rows in place (the dense projections of a larger decode batch)
            more = (not grouped and not p.a_rows and 16 < p.M <= self.stream_max_rows and p.N < 65536)
            if (few or more) and self.use_stream and p.K % 64 == 0 and max_rows_per_group <= (32 if more else 16):
                st = self._gemm_stream(p, int(max_rows_per_group), grouped)
                if st != -2:
                    self._count("gemm_stream", 1)
                    _check(st, what + " (streaming)")
                    return
            if few or (not tc_ok and max_rows_per_group <= 64):
                st = self._lib("gemm_skinny").spite_gemm_skinny(C.byref(p), int(max_rows_per_group), self.skinny_blocks,
                                                                self._stream())
                if st != -2:                       # -2: shape outside the kernel's domain, fall through
                    self._count("gemm_skinny", 1)
                    _check(st, what)
                    return
            if tc_ok:
                orig = p
                if gather_src is not None:
                    keep = torch.empty_like(gather_src)
                    st = self._lib("elementwise").spite_gather_rows(
                        C.c_void_p(gather_src.data_ptr()), C.c_void_p(p.a_rows), C.c_void_p(keep.data_ptr()),
                        gather_src.shape[0], C.c_longlong(gather_src.shape[1] * gather_src.element_size()),
                        self._stream())
                    self._count("elementwise", 1)
                    _check(st, "gather_rows")
                    p = GemmParams.from_buffer_copy(p)
                    p.A = keep.data_ptr()          # rows are in place now; a_rows only indexes the row scale
                if grouped and self.use_tc_experts and self._few_rows_per_group(p):
                    # groups of few rows each (experts of a prompt portion): the weights as the 128-row operand, a
                    # group's tokens as the instruction's columns
                    st = self._lib("gemm_tc_experts").spite_gemm_tc_experts(C.byref(p), self.sm_count, self._stream())
                    if st != -2:
                        self._count("gemm_tc_experts", 1)
                        _check(st, what + " (tcgen05, experts)")
                        return
                if p.M >= (self.tc_pair_min_group_rows * p.n_groups if grouped else self.tc_pair_min_rows):
                    # a product of many rows (per group) on pairs of multiprocessors (tcgen05 cta_group::2)
                    st = self._lib("gemm_tc_pair").spite_gemm_tc_pair(C.byref(p), self.sm_count // 2, self._stream())
                    if st != -2:
                        self._count("gemm_tc_pair", 1)
                        _check(st, what + " (tcgen05, pairs)")
                        return
                st = self._lib("gemm_tc").spite_gemm_tc(C.byref(p), self.sm_count, self._stream())
                if st != -2:
                    self._count("gemm_tc", 1)
                    _check(st, what + " (tcgen05)")
                    return
                p = orig
                if max_rows_per_group <= 64:       # refused (alignment): the streaming kernel may still take it
                    st = self._lib("gemm_skinny").spite_gemm_skinny(C.byref(p), int(max_rows_per_group),
                                                                    self.skinny_blocks, self._stream())
                    if st != -2:
                        self._count("gemm_skinny", 1)
                        _check(st, what)
                        return
        st = self._lib("gemm_simt").spite_gemm_simt(self._dt, C.byref(p), self._stream())
        self._count("gemm_simt", 1)
        _check(st, what)

    def _few_rows_per_group(self, p) -> bool:
        """Does a grouped product go to the kernel with swapped operands?  Measured on B200 at Scout's expert
        shapes (us, swapped against 128-row tiles).  Gate/up with SwiGLU, 16 experts: 427/437 at 256 tokens,
        437/464 at 1,024, 630/503 at 2,048 (half the groups then exceed a token tile and run twice); 128
        experts: 3,159/3,300 at 1,024, 3,284/3,849 at 8,192.  Down product into the residual stream, 16
        experts: 264/244 at 256, 276/254 at 1,024, 344/293 at 2,048; 128 experts: 1,749/1,705 at 2,048,
        1,905/2,006 at 8,192.  So: gate/up up to 64 rows a group on average, the down product only with
        many groups of 32 to 64 rows."""
        avg = p.M / p.n_groups
        if p.epilogue == EPI_SWIGLU:
            return avg <= self.tc_experts_max_group_rows
        if p.epilogue == EPI_ADD_F32:
            return p.n_groups >= self.tc_experts_down_min_groups and 32 <= avg <= self.tc_experts_max_group_rows
        return False

    def _gemm_stream(self, p, max_rows_per_group, grouped):
        """The TMA weight-streaming kernel for decode steps: picks the tile height (k slices inside the block)
        and the k splits across blocks so that the work items are many enough to spread evenly, and lends the
        scratch for the partial sums of the splits."""
        swiglu = p.epilogue == EPI_SWIGLU
        groups = min(p.n_groups, p.M) if grouped else 1
        smem, blocks = self.stream_shape[0 if p.M <= 3 or p.M > 16 else 1]      # (the tokens of many rows need the larger ring)
        nt = 8 if max_rows_per_group <= 8 else 16 if max_rows_per_group <= 16 else 32
        slices, splits = self.stream_force or self._stream_cut(p.M, p.N, p.K, groups, swiglu, blocks, smem, nt, grouped)
        rows = 128 // slices
        tiles = -(-p.N // (rows // 2 if swiglu else rows)) * groups
        lib = self._lib("gemm_stream")
        stream = torch.cuda.current_stream().cuda_stream
        if slices == 1 and 2 <= splits <= self.stream_cluster_max_splits and p.M <= self.stream_cluster_max_rows:
            # the k splits of a tile as one thread-block cluster: their sums meet in shared memory
            st = lib.spite_gemm_stream(C.byref(p), max_rows_per_group, 1, 1, blocks, smem, splits, None, C.c_longlong(0),
                                       None, 0, C.c_void_p(stream))
            if st != -2:
                return st
        scratch, n_floats = None, 0
        if splits > 1:
            if tiles > self._tickets_n:
                return -2
            n_floats = tiles * splits * nt * rows
            scratch = torch.empty(n_floats, dtype=torch.float32, device=self.device)
        # the k splits' arrival counters: one set per stream, since calls that share a set must not overlap
        tickets = self._tickets.get(stream)
        if tickets is None and splits > 1:
            tickets = self._tickets[stream] = torch.zeros(self._tickets_n, dtype=torch.int32, device=self.device)
        return lib.spite_gemm_stream(
            C.byref(p), max_rows_per_group, slices, 0, blocks, smem, splits, C.c_void_p(_ptr(scratch)),
            C.c_longlong(n_floats), C.c_void_p(_ptr(tickets)), self._tickets_n, C.c_void_p(stream))

    def _stream_cut(self, M: int, N: int, K: int, groups: int, swiglu: bool, slots: int, smem: int, nt: int,
                    grouped: bool):
        return stream_cut(M, N, K, groups, swiglu, slots, smem, nt, item_cost=self.stream_item_cost,
                          split_item_cost=self.stream_split_item_cost, split_cost=self.stream_split_cost,
                          slice_cost=self.stream_slice_cost,
                          max_slices=(min(2, self.stream_max_slices) if nt > 16 else self.stream_max_slices)
                          if self.stream_slices_grouped or not grouped else 1,
                          slices_min_rows=self.stream_slices_min_rows,
                          cluster_max_splits=self.stream_cluster_max_splits if M <= self.stream_cluster_max_rows else 0,
                          cluster_cost=self.stream_cluster_cost)

    def attention_tc_error(self) -> int:
        """Error code left by a tcgen05 attention block that gave up waiting (0: none); clears it. Synchronises."""
        torch.cuda.synchronize(self.device)
        words = _error_buffer()
        code, words[3] = int(words[3]), 0
        return code

    def gemm_tc_error(self) -> int:
        """Error code left by a product kernel's block that gave up waiting (0: none); clears it. Synchronises."""
        torch.cuda.synchronize(self.device)
        words = _error_buffer()
        code = int(words[0]) or int(words[1]) or int(words[2]) or int(words[5])
        words[:3] = 0
        words[5] = 0
        return code

    def linear(self, x, w, out, *, accumulate=False, row_scale=None):
        self._t(x, self.dtype, "x"); self._t(w, self.dtype, "w"); self._t(out, None, "out")
        M, K = x.shape
        N = w.shape[0]
        if w.shape[1] != K or tuple(out.shape) != (M, N):
            raise KernelError(f"linear: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} do not fit")
        if accumulate:
            if out.dtype != torch.float32:
                raise KernelError("linear(accumulate=True) needs a float32 output")
            epi = EPI_ADD_F32
        elif out.dtype == torch.float32 and self.dtype != torch.float32:
            epi = EPI_STORE_F32
        elif out.dtype == self.dtype:
            epi = EPI_STORE
        else:
            raise KernelError(f"linear: output type {out.dtype} not supported")
        p = GemmParams(A=x.data_ptr(), W=w.data_ptr(), C=out.data_ptr(), a_rows=None, c_rows=None,
                       group_offsets=None, row_scale=_ptr(row_scale), lda=K, ldc=N, w_group_stride=0,
                       n_groups=1, M=M, N=N, K=K, epilogue=epi, scale_by_a_row=0)
        self._gemm(p, "linear", M)

    def linear_swiglu(self, x, w_gate_up, out, *, row_scale=None):
        self._t(x, self.dtype, "x"); self._t(w_gate_up, self.dtype, "w"); self._t(out, self.dtype, "out")
        M, K = x.shape
        F = w_gate_up.shape[0] // 2
        if w_gate_up.shape != (2 * F, K) or tuple(out.shape) != (M, F):
            raise KernelError("linear_swiglu: shapes do not fit")
        p = GemmParams(A=x.data_ptr(), W=w_gate_up.data_ptr(), C=out.data_ptr(), a_rows=None, c_rows=None,
                       group_offsets=None, row_scale=_ptr(row_scale), lda=K, ldc=F, w_group_stride=0,
                       n_groups=1, M=M, N=F, K=K, epilogue=EPI_SWIGLU, scale_by_a_row=0)
        self._gemm(p, "linear_swiglu", M)

    def grouped_linear_swiglu(self, x, w_gate_up, sorted_rows, offsets, row_scale, out):
        self._t(x, self.dtype, "x"); self._t(w_gate_up, self.dtype, "w"); self._t(out, self.dtype, "out")
        self._t(sorted_rows, torch.int32, "sorted_rows"); self._t(offsets, torch.int32, "offsets")
        M, K = x.shape
        E, F2, K2 = w_gate_up.shape
        F = F2 // 2
        if K2 != K or tuple(out.shape) != (M, F) or offsets.numel() != E + 1 or sorted_rows.numel() != M:
            raise KernelError("grouped_linear_swiglu: shapes do not fit")
        p = GemmParams(A=x.data_ptr(), W=w_gate_up.data_ptr(), C=out.data_ptr(),
                       a_rows=sorted_rows.data_ptr(), c_rows=None, group_offsets=offsets.data_ptr(),
                       row_scale=_ptr(row_scale), lda=K, ldc=F, w_group_stride=F2 * K,
                       n_groups=E, M=M, N=F, K=K, epilogue=EPI_SWIGLU, scale_by_a_row=1)
        self._gemm(p, "grouped_linear_swiglu", M, gather_src=x)

    def grouped_linear_accumulate(self, a, w_down, sorted_rows, offsets, h):
        self._t(a, self.dtype, "a"); self._t(w_down, self.dtype, "w"); self._t(h, torch.float32, "h")
        M, F = a.shape
        E, d, F2 = w_down.shape
        if F2 != F or h.shape[1] != d or offsets.numel() != E + 1 or sorted_rows.numel() != M:
            raise KernelError("grouped_linear_accumulate: shapes do not fit")
        p = GemmParams(A=a.data_ptr(), W=w_down.data_ptr(), C=h.data_ptr(), a_rows=None,
                       c_rows=sorted_rows.data_ptr(), group_offsets=offsets.data_ptr(), row_scale=None,
                       lda=F, ldc=d, w_group_stride=d * F, n_groups=E, M=M, N=d, K=F,
                       epilogue=EPI_ADD_F32, scale_by_a_row=0)
        self._gemm(p, "grouped_linear_accumulate", M)

    # ------------------------------------------------------------------ attention
    def _step_tokens(self, batch, group):
        bt = batch.block_tables[group]
        return StepTokens(positions=batch.positions.data_ptr(), seg_of_token=batch.seg_of_token.data_ptr(),
                          block_table=bt.data_ptr(), table_width=bt.shape[1], n_tokens=batch.n_tokens)

    def _paged(self, cache):
        kv = cache.kv                       # [2, pages, nkv, page_size, hd]
        self._t(kv, self.dtype, "cache")
        return PagedCache(kv=kv.data_ptr(), v_offset=kv.stride(0), n_pages=kv.shape[1],
                          page_size=kv.shape[3], num_kv_heads=kv.shape[2], head_dim=kv.shape[4])

    def qk_prepare(self, qkv, q_out, batch, cache, *, num_heads, rotation, qk_norm, temperature):
        self._t(qkv, self.dtype, "qkv"); self._t(q_out, self.dtype, "q_out")
        head_dim = cache.kv.shape[4]
        inv_freq, pairing, rotary_dim = None, 0, head_dim
        if rotation is not None:
            inv_freq = self._t(rotation.inv_freq, torch.float32, "inv_freq")
            pairing = {"neighbours": 0, "halves": 1}[rotation.pairing]
            rotary_dim = int(rotation.rotary_dim or head_dim)
            if inv_freq.numel() != rotary_dim // 2:
                raise KernelError(f"qk_prepare: {inv_freq.numel()} frequencies for {rotary_dim} rotating elements")
        eps, before, q_gain, k_gain = 0.0, 0, None, None
        if qk_norm is not None:
            eps, before = float(qk_norm.eps), int(qk_norm.before_rotation)
            for g in (qk_norm.q_gain, qk_norm.k_gain):
                if g is not None and (self._t(g, torch.float32, "gain").numel() != head_dim):
                    raise KernelError("qk_prepare: a gain vector must have head_dim elements")
            q_gain, k_gain = qk_norm.q_gain, qk_norm.k_gain
        floor, scale = (int(temperature[0]), float(temperature[1])) if temperature else (0, 0.0)
        p = QkPrepareParams(qkv=qkv.data_ptr(), q_out=q_out.data_ptr(), inv_freq=_ptr(inv_freq),
                            q_gain=_ptr(q_gain), k_gain=_ptr(k_gain), qk_norm_eps=eps,
                            norm_before_rotation=before, pairing=pairing, rotary_dim=rotary_dim,
                            temperature_floor=floor, temperature_scale=scale, num_heads=num_heads,
                            write_cache=int(cache.write))
        b, c = self._step_tokens(batch, cache.group), self._paged(cache)
        st = self._lib("attention").spite_qk_prepare(self._dt, C.byref(p), C.byref(b), C.byref(c), self._stream())
        self._count("attention", 1)
        _check(st, "qk_prepare")

    def paged_attention(self, q, out, batch, cache, *, num_heads, window, softmax_scale, cache_settled=False):
        self._t(q, self.dtype, "q"); self._t(out, self.dtype, "out")
        p = AttentionParams(q=q.data_ptr(), out=out.data_ptr(), num_heads=num_heads,
                            window_kind=_WINDOW[window.kind], window_size=int(window.size),
                            softmax_scale=float(softmax_scale))
        b, c = self._step_tokens(batch, cache.group), self._paged(cache)
        group = num_heads // c.num_kv_heads
        if (self.dtype == torch.bfloat16 and c.head_dim % 16 == 0 and c.head_dim <= 128 and group <= 16
                and c.page_size % 16 == 0 and batch.segments):
            # Tensor-core kernels; rows are (token, head of a kv group) pairs.  Segments of many
            # tokens (prompt portions) go to the kernel with 64 rows a block and warps that own
            # rows; segments of few tokens (decode) to the kernel with 16 rows a block whose
            # warps and blocks split the keys.
            big_from = -(-32 // group) if c.page_size % 32 == 0 else 1 << 30
            tpb, tpb_rows, tpb_tc = max(1, 16 // group), max(1, 64 // group), max(1, 128 // group)
            # tcgen05 kernel (two tiles of 128 rows a block): head sizes 64 and 128, pages of a multiple of 64 keys
            tc_from = 1 << 30
            if c.head_dim in (64, 128) and c.page_size % 64 == 0 and self.use_tcgen05_attention:
                tc_from = max(big_from, self.attention_tc_min_tokens or tpb_tc)
            n_small = n_big = n_tc = 0
            longest = 1
            for s in batch.segments:
                if s.n_tokens >= tc_from:
                    n_tc += -(-s.n_tokens // (2 * tpb_tc))        # a block serves two tiles of 128 rows
                    continue
                if s.n_tokens >= big_from:
                    n_big += -(-s.n_tokens // tpb_rows)
                    continue
                n_small += -(-s.n_tokens // tpb)
                last = s.start_pos + s.n_tokens - 1
                longest = max(longest, last - window.lowest_visible(max(s.start_pos, last - tpb + 1)) + 1)
            if n_tc:
                x = AttnMmaExtra(cu_seqlens=batch.cu_seqlens.data_ptr(), o_part=None, ml_part=None,
                                 n_segments=len(batch.segments), tokens_per_block=tpb_tc, n_splits=1,
                                 seg_min_tokens=tc_from, seg_max_tokens=0x7fffffff)
                st = self._lib("attention_tc").spite_paged_attention_tc(
                    C.byref(p), C.byref(b), C.byref(c), C.byref(x), n_tc, self.sm_count, self._stream())
                self._count("attention_tc", 1)
                _check(st, "paged_attention (tcgen05, prompt portions)")
            if n_big:
                x = AttnMmaExtra(cu_seqlens=batch.cu_seqlens.data_ptr(), o_part=None, ml_part=None,
                                 n_segments=len(batch.segments), tokens_per_block=tpb_rows, n_splits=1,
                                 seg_min_tokens=big_from, seg_max_tokens=tc_from - 1)
                st = self._lib("attention_rows").spite_paged_attention_rows(
                    C.byref(p), C.byref(b), C.byref(c), C.byref(x), n_big, self._stream())
                self._count("attention_rows", 1)
                _check(st, "paged_attention (tensor cores, prompt portions)")
            if not n_small:
                return
            if batch.context_bucket:            # fixed launch shape for a captured step
                longest = batch.context_bucket if window.kind == "full" else min(batch.context_bucket, window.size)
            if c.head_dim in (64, 128) and c.page_size % 64 == 0 and self.use_decode_attention:
                self._attention_decode(p, b, c, batch, n_small, tpb, big_from - 1, longest, num_heads, cache_settled)
                return
            tiles = -(-longest // 16) + 1
            base = n_small * c.num_kv_heads
            # key splits: fill the resident blocks (three per multiprocessor) once if the step is
            # small, else pick the split count whose last wave is fullest
            slots = 3 * self.sm_count
            if base <= slots:
                splits = slots // base
            elif base >= 4 * slots:
                splits = 1
            else:
                splits = max(range(1, 5), key=lambda s: (base * s / slots) / -(-base * s // slots))
            splits = max(1, min(splits, tiles // 8, self.attention_max_splits, 32))
            o_part = ml_part = None
            if splits > 1:
                # one row per token place of this kernel's blocks: tokens of longer segments take none
                o_part = torch.empty((n_small * tpb, num_heads, splits, c.head_dim), dtype=torch.float32,
                                     device=q.device)
                ml_part = torch.empty((n_small * tpb, num_heads, splits, 2), dtype=torch.float32, device=q.device)
                self.attention_scratch_bytes = (o_part.numel() + ml_part.numel()) * 4
            x = AttnMmaExtra(cu_seqlens=batch.cu_seqlens.data_ptr(), o_part=_ptr(o_part), ml_part=_ptr(ml_part),
                             n_segments=len(batch.segments), tokens_per_block=tpb, n_splits=splits,
                             seg_min_tokens=0, seg_max_tokens=big_from - 1)
            st = self._lib("attention_mma").spite_paged_attention_mma(
                C.byref(p), C.byref(b), C.byref(c), C.byref(x), n_small, self._stream())
            self._count("attention_mma", 1 + (splits > 1))
            _check(st, "paged_attention (tensor cores)")
            return
        st = self._lib("attention").spite_paged_attention(self._dt, C.byref(p), C.byref(b), C.byref(c),
                                                          self._stream())
        self._count("attention", 1)
        _check(st, "paged_attention")

    def _attention_decode(self, p, b, c, batch, n_small, tpb, seg_max, longest, num_heads, cache_settled):
        """Decoded tokens (and portions too short for the row kernels) on the TMA-fed decode kernel: as many
        key splits as fill the resident blocks once, partial results merged by the last block of a split set."""
        stage = 2 * c.head_dim * 64 * 2                         # 64 keys and 64 values of one kv head
        tiles = -(-longest // 64) + 1
        base = n_small * c.num_kv_heads
        per_sm = max(1, min(4, (225 * 1024) // (3 * stage + 2048)))
        slots = per_sm * self.sm_count
        if base <= slots:
            splits = slots // base
        elif base >= 4 * slots:
            splits = 1
        else:
            splits = max(range(1, 5), key=lambda s: (base * s / slots) / -(-base * s // slots))
        splits = max(1, min(splits, tiles // 2, self.attention_max_splits))
        n_stages = max(2, min(3 if per_sm > 1 else 6, -(-tiles // splits)))
        partial = tickets = None
        if splits > 1:
            if base > self._tickets_n:
                raise KernelError(f"paged_attention: {base} (request block, kv head) pairs exceed the {self._tickets_n} tickets")
            partial = torch.empty((base * splits * 16 * (c.head_dim + 4),), dtype=torch.float32, device=self.device)
            self.attention_scratch_bytes = partial.numel() * 4
            stream = torch.cuda.current_stream().cuda_stream
            tickets = self._tickets.get(stream)
            if tickets is None:
                tickets = self._tickets[stream] = torch.zeros(self._tickets_n, dtype=torch.int32, device=self.device)
        x = AttnDecodeExtra(cu_seqlens=batch.cu_seqlens.data_ptr(), partial=_ptr(partial), tickets=_ptr(tickets),
                            n_segments=len(batch.segments), tokens_per_block=tpb, n_splits=splits,
                            seg_min_tokens=0, seg_max_tokens=seg_max, cache_settled=int(bool(cache_settled)))
        st = self._lib("attention_decode").spite_paged_attention_decode(
            C.byref(p), C.byref(b), C.byref(c), C.byref(x), n_small, n_stages, self._stream())
        self._count("attention_decode", 1)
        _check(st, "paged_attention (decode)")

    # ------------------------------------------------------------------ mixture of experts
    def moe_route(self, x, w_router, top_k, want_logits=False) -> Routing:
        self._t(x, self.dtype, "x"); self._t(w_router, torch.float32, "w_router")
        M, d = x.shape
        E = w_router.shape[0]
        dev = x.device
        ids = torch.empty((top_k, M), dtype=torch.int32, device=dev)
        wts = torch.empty((top_k, M), dtype=torch.float32, device=dev)
        offsets = torch.empty((top_k, E + 1), dtype=torch.int32, device=dev)
        rows = torch.empty((top_k, M), dtype=torch.int32, device=dev)
        logits = torch.empty((M, E), dtype=torch.float32, device=dev)
        st = self._lib("moe").spite_moe_route(
            self._dt, C.c_void_p(x.data_ptr()), C.c_void_p(w_router.data_ptr()), M, d, E, top_k,
            C.c_void_p(ids.data_ptr()), C.c_void_p(wts.data_ptr()), C.c_void_p(_ptr(logits)),
            C.c_void_p(offsets.data_ptr()), C.c_void_p(rows.data_ptr()), self._stream())
        self._count("moe", 2)
        _check(st, "moe_route")
        return Routing(ids, wts, offsets, rows, logits if want_logits else None)

    # ------------------------------------------------------------------ sampling
    def argmax(self, logits):
        self._t(logits, torch.float32, "logits")
        R, V = logits.shape
        out = torch.empty(R, dtype=torch.int32, device=logits.device)
        st = self._lib("sampling").spite_argmax(C.c_void_p(logits.data_ptr()), R, V,
                                                C.c_void_p(out.data_ptr()), self._stream())
        self._count("sampling", 1)
        _check(st, "argmax")
        return out

    def sample(self, logits, *, temperature, top_k=None, top_p=None, min_p=None, repetition_penalty=None,
               context=None, context_offsets=None, rng_state):
        self._t(logits, torch.float32, "logits"); self._t(temperature, torch.float32, "temperature")
        self._t(rng_state, torch.int64, "rng_state")
        R, V = logits.shape
        work = torch.empty_like(logits)
        out = torch.empty(R, dtype=torch.int32, device=logits.device)
        p = SampleParams(logits=logits.data_ptr(), work=work.data_ptr(), temperature=temperature.data_ptr(),
                         top_k=_ptr(top_k), top_p=_ptr(top_p), min_p=_ptr(min_p),
                         repetition_penalty=_ptr(repetition_penalty), context=_ptr(context),
                         context_offsets=_ptr(context_offsets), rng_state=rng_state.data_ptr(),
                         out_tokens=out.data_ptr(), vocab=V)
        st = self._lib("sampling").spite_sample(C.byref(p), R, self._stream())
        self._count("sampling", 1)
        _check(st, "sample")
        return out
