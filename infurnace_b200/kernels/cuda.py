"""The CUDA kernel set: thin, checked calls into the compiled libraries.

Every method takes device tensors, checks what the kernel assumes (dtype, contiguity,
matching sizes) and launches on torch's current stream.  There is no CPU path: without
a CUDA device or without the compiled library the constructor raises
:class:`~infurnace_b200.errors.KernelError`.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from ..errors import KernelError
from .build import load_library

F32, BF16 = 0, 1
# the `epilogue` argument of the products: 0 plain, 1 silu_gate (w holds gate rows, then up rows), 16 * u: plain with the
# unary function u applied to every element (csrc/common.cuh: ifb_unary)
EPILOGUES = {"none": 0, "silu_gate": 1, "relu2": 16, "silu": 32, "sigmoid": 48, "gelu_tanh": 64, "tanh": 80}
_CODES = {torch.float32: F32, torch.bfloat16: BF16}
_ERRORS = {1: "a dtype (or combination of dtypes) has no kernel", 2: "a size is outside what the kernel takes",
           3: "an address or row length breaks the kernel's alignment rule", 4: "arguments contradict each other"}


def _code(t):
    try:
        return _CODES[t.dtype]
    except KeyError:
        raise KernelError(f"dtype {t.dtype} has no kernel; float32 and bfloat16 do") from None


def _ptr(t):
    return 0 if t is None else t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
if _raw_stream is None:                       # an older torch: the public, slower way
    def _raw_stream(device_index):
        return torch.cuda.current_stream(device_index).cuda_stream


def _check(status, what):
    if status == 0:
        return
    if status > 0:
        raise KernelError(f"{what}: refused: {_ERRORS.get(status, status)}")
    raise KernelError(f"{what}: CUDA launch failed with error {-status}")


def _dense(t, name, dtype=None):
    if not t.is_cuda:
        raise KernelError(f"{name} is not on a CUDA device")
    if not t.is_contiguous():
        raise KernelError(f"{name} is not contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} has dtype {t.dtype}, expected {dtype}")
    return t


class CudaKernels:
    name = "cuda"

    def __init__(self, progress=None):
        if not torch.cuda.is_available():
            raise KernelError("no CUDA device is available; this engine has no CPU path")
        self._progress = progress
        self.launches = 0          # kernels launched through this object
        self.scratch_generation = 0  # bumped when a scratch buffer moves: captured graphs go stale
        self.core = load_library("core", progress=progress)
        c = self.core
        c.ifb_embed.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]
        c.ifb_random_normal.argtypes = [c_void_p, c_int, c_longlong, ctypes.c_ulonglong, c_float, c_float, c_void_p]
        c.ifb_rmsnorm.argtypes = [c_void_p, c_void_p, c_int, c_longlong, c_void_p, c_int, c_float, c_void_p, c_int,
                                  c_void_p, c_int, c_int, c_void_p]
        c.ifb_qk_norm_rope_store.argtypes = [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int,
                                             c_float, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                             c_void_p]
        c.ifb_rope_table.argtypes = [c_void_p, c_void_p, c_int, c_void_p, c_int, c_float, c_void_p]
        c.ifb_sample.argtypes = [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p]
        c.ifb_argmax_rows.argtypes = [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]
        self._argmax_scratch = None    # (values, indices, counters) of the several-blocks-per-row argmax
        c.ifb_linear_simt.argtypes = [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                      c_void_p]
        c.ifb_linear_skinny.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int,
                                        c_int, c_int, c_void_p]
        c.ifb_linear_gemv.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int,
                                      c_float, c_int, c_void_p]
        c.ifb_linear_gemv_residual_norm.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                                    c_int, c_int, c_int, c_void_p]
        c.ifb_linear_gemv_qkv.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int,
                                          c_float, c_int, c_void_p, c_void_p, c_int, c_float, c_void_p, c_void_p, c_void_p,
                                          c_int, c_void_p]
        self.fused_qkv = os.environ.get("INFURNACE_FUSED_QKV", "1") != "0"
        self.fused_qkv_calls = 0
        c.ifb_linear_gemv_set_plan.argtypes = [c_int]
        c.ifb_linear_gemv_set_plan.restype = None
        c.ifb_linear_skinny_scratch.argtypes = [c_int, c_int, c_int, c_int, c_void_p, c_void_p]
        c.ifb_linear_skinny_scratch.restype = None
        self._lin_partials = None
        self._lin_counters = None
        self.gemv_max_rows = 64        # up to here: the kernel without global partial sums
        # up to here norms are folded into products (the kernels take 64 rows; beyond 32 the separate norm measured faster)
        self.fold_max_rows = int(os.environ.get("INFURNACE_FOLD_MAX_ROWS", "32"))
        self.split_min_keys = int(os.environ.get("INFURNACE_SPLIT_MIN_KEYS", "256"))   # fewest keys a split of a context gets
        self.talk_mma = os.environ.get("INFURNACE_TALK_MMA", "1") != "0"    # talking attention on tensor cores where it fits
        self.talk_mma_calls = 0
        self.talk_split_calls = 0      # of these, with the keys of a tile split over several CTAs
        self.scan_block_min = int(os.environ.get("INFURNACE_SCAN_BLOCK_MIN", "97"))     # tokens of the longest request from
        self.scan_blocked_calls = 0                                                    # which the recurrence runs in blocks
        self._scan_scratch = None
        self._hyb = None               # the library of sandwich-norm blocks, state recurrences, stream attention, routed experts
        self._lat = None               # the library of decoders with latent attention
        self._ls_scratch = None
        self._gu_scratch = None
        self.gated_unit_chunked_calls = 0
        self._rg_scratch = None
        self.rglru_chunked_calls = 0
        self.moe_tensor_cores = os.environ.get("INFURNACE_MOE_MMA", "1") != "0"
        self.moe_tcgen05 = os.environ.get("INFURNACE_MOE_TCGEN05", "1") != "0"     # prompts' expert products on tcgen05
        self.moe_tcgen05_calls = 0
        self.linear_scan_blocked_calls = 0
        self.stream_attention_calls = 0
        self._mix = None               # the library of post-norm sublayers, the gated recurrence and talking attention
        self._tc = None                # the tcgen05 library, loaded when a product first has more than tc_min_rows rows
        # device int: non-zero after a kernel recorded a fault it contained (a bounded barrier wait that gave up, a
        # token id outside the vocabulary); read by check_device_errors
        self._dev_err = torch.zeros(1, dtype=torch.int32, device="cuda")
        self.attention_tma = True      # keys and values by TMA where the sizes allow (else 16-byte async copies)
        self.attention_tc = True       # prompts on tcgen05 where the sizes allow (head size 128, pages of 16/32/64)
        self._attn_tc = None
        self.tc_attention_calls = 0    # launches of the tcgen05 attention kernel, of the small-q kernel, and of the latter
        self.small_q_calls = 0         # with keys and values by TMA (what ran is what tests of the product path ask)
        self.small_q_tma_calls = 0
        self.tc_shared_k_calls = 0     # tcgen05 products with the k range shared by a cluster; with a folded norm
        self.tc_folded_calls = 0
        self._err_armed = False
        self.tc_min_rows = 65
        if os.environ.get("INFURNACE_GATE_PLAN"):
            self.core.ifb_linear_gemv_set_gate_plan(int(os.environ["INFURNACE_GATE_PLAN"]))
        self.tc_split_min_k = int(os.environ.get("INFURNACE_TC_SPLIT_MIN_K", "256"))
        self.fused_qkv_tc = os.environ.get("INFURNACE_FUSED_QKV_TC", "1") != "0"
        self.tc_split_min_rows = int(os.environ.get("INFURNACE_TC_SPLIT_MIN_ROWS", "0"))     # 0: by the matrix
        self.tc_fold_max_rows = int(os.environ.get("INFURNACE_TC_FOLD_MAX_ROWS", "128"))
        self._tc_clusters = {}         # CTAs per cluster -> clusters of the split product that run at a time
        self._route_memo = {}          # what _on_tcgen05 and tcgen05_splits answered (asked several times per launch)
        self._splits_memo = {}
        self._attn_mma = {}        # head size -> library
        self._attn_scratch = None
        self._attn_counters = None
        self.latent_mma_calls = 0      # steps of the latent attention that ran on tensor cores
        self.sm_count = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
        self.attention_scratch_cap = 64 << 20     # bytes of split scratch beyond which a step runs unsplit
        c.ifb_paged_attention_simt.argtypes = [c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                               c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int,
                                               c_void_p]

    @staticmethod
    def _stream():
        # the raw handle of torch's current stream on the current device (torch.cuda.current_stream() builds a Stream
        # object around it on every call, which was a fifth of an eager step's host time)
        return _raw_stream(torch._C._cuda_getDevice())

    # ------------------------------------------------------------------ embedding
    def embed(self, table, ids, out):
        _dense(table, "table"), _dense(ids, "ids", torch.int32), _dense(out, "out", torch.float32)
        n, hidden = out.shape
        if table.shape[1] != hidden or ids.numel() != n:
            raise KernelError("embed: sizes of table, ids and out do not match")
        self.launches += 1
        self._err_armed = True
        _check(self.core.ifb_embed(table.data_ptr(), _code(table), ids.data_ptr(), out.data_ptr(), n, hidden,
                                   table.shape[0], self._dev_err.data_ptr(), self._stream()), "embed")

    def random_normal(self, out, seed64, mean, std):
        """out[i] = mean + std * z_i with z_i approximately N(0, 1), a pure function of (seed64, i): the
        same bits as ``weights.random_init.normal_values``."""
        _dense(out, "out")
        self.launches += 1
        _check(self.core.ifb_random_normal(out.data_ptr(), _code(out), out.numel(), int(seed64) & ((1 << 64) - 1),
                                           float(mean), float(std), self._stream()), "random_normal")

    # ------------------------------------------------------------------ norm
    def rmsnorm(self, x, weight, eps, out, delta=None, rows=None):
        _dense(x, "x", torch.float32), _dense(weight, "weight"), _dense(out, "out")
        hidden = x.shape[1]
        n_out = out.shape[0]
        if weight.numel() != hidden or out.shape[1] != hidden:
            raise KernelError("rmsnorm: widths of x, weight and out do not match")
        splits, stride = 0, 0
        if delta is not None:
            _dense(delta, "delta", torch.float32)
            if delta.dim() == 3:
                splits, stride = delta.shape[0], delta.stride(0)
                drows = delta.shape[1]
            else:
                splits, stride, drows = 1, 0, delta.shape[0]
            if delta.shape[-1] != hidden or drows != x.shape[0]:
                raise KernelError("rmsnorm: delta does not match x")
        if rows is not None:
            _dense(rows, "rows", torch.int32)
            if rows.numel() != n_out:
                raise KernelError("rmsnorm: out has a row for each entry of rows")
        elif n_out != x.shape[0]:
            raise KernelError("rmsnorm: out has a row for each row of x")
        self.launches += 1
        _check(self.core.ifb_rmsnorm(x.data_ptr(), _ptr(delta), splits, stride, weight.data_ptr(), _code(weight),
                                     float(eps), out.data_ptr(), _code(out), _ptr(rows), n_out, hidden,
                                     self._stream()), "rmsnorm")

    # ------------------------------------------------------------------ matrix products
    def linear(self, x, w, out, epilogue="none", row_scale=None):
        """out = x w^T with the epilogue (a key of ``EPILOGUES``).  ``row_scale`` (partials, parts, eps, width), from
        :meth:`linear_residual_norm`, multiplies row n by rsqrt(sum_p partials[p, n] / width + eps)
        before the epilogue; only where :meth:`can_fold_norm` says so."""
        _dense(x, "x"), _dense(w, "w"), _dense(out, "out")
        n, k = x.shape
        o = out.shape[1]
        try:
            epi = EPILOGUES[epilogue]
        except KeyError:
            raise KernelError(f"linear: unknown epilogue {epilogue!r}; known: {', '.join(EPILOGUES)}") from None
        gated = epi == 1
        route = "silu_gate" if gated else "none"          # a unary function changes nothing in the choice of kernel
        if w.shape[1] != k or out.shape[0] != n or w.shape[0] != (2 * o if gated else o):
            raise KernelError(f"linear: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} do not match")
        if row_scale is not None:
            if not self.can_fold_norm(n, x.dtype, w, route) or out.dtype not in (torch.bfloat16, torch.float32):
                raise KernelError("linear: a row scale is taken only by the bfloat16 kernels (see can_fold_norm)")
            partials, parts = row_scale[0], row_scale[1]
            _dense(partials, "row_scale partials", torch.float32)
            if partials.dim() != 2 or partials.shape[0] < parts or partials.shape[1] != n:
                raise KernelError("linear: row_scale partials must be [parts, rows]")
        if x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and k % 8 == 0 \
                and out.dtype in (torch.bfloat16, torch.float32):
            if self._on_tcgen05(n, w, route):
                return self._linear_tcgen05(x, w, out, n, o, k, epi, splits=self.tcgen05_splits(n, o, k, gated),
                                            row_scale=row_scale)
            return self._linear_gemv(x, w, out, n, o, k, epi, row_scale)
        self.launches += 1
        _check(self.core.ifb_linear_simt(x.data_ptr(), _code(x), w.data_ptr(), _code(w), out.data_ptr(), _code(out),
                                         n, o, k, epi, self._stream()), "linear")

    def _on_tcgen05(self, n, w, epilogue="none", shared_k=True):
        key = (n, w.shape[0], w.shape[1], w.dtype, epilogue, shared_k)
        hit = self._route_memo.get(key)
        if hit is None:
            hit = self._route_memo[key] = self._on_tcgen05_rule(n, w, epilogue, shared_k)
        return hit

    def _on_tcgen05_rule(self, n, w, epilogue, shared_k):
        """Which kernel a bfloat16 product of n rows against w runs on.  More than 64 rows: the tcgen05 kernel.
        From ``tc_split_min_rows`` rows, a product with the plain epilogue whose few tiles can share their k
        range in clusters (:meth:`tcgen05_splits`): the tcgen05 kernel in that form, which streams a long k
        faster than the few-rows kernel.  Else up to 8 rows: the few-rows kernel.  Between, by measurement:
        the few-rows kernel re-reads the rows from L2 in every CTA, so for a large weight matrix (from 2^24
        elements, or from 33 rows and 4,096 features) the tcgen05 kernel, which streams the weights once
        through its tiles, is the faster one although most of its 128-row tile is empty."""
        if n >= self.tc_min_rows:
            return True
        if shared_k and epilogue == "none" and n >= self._shared_k_min_rows(w) and w.dtype == torch.bfloat16 \
                and w.shape[1] % 8 == 0 and self.tcgen05_splits(n, w.shape[0], w.shape[1]) > 1:
            return True
        if n <= 8:
            return False
        return w.numel() >= (1 << 24) or (n >= 33 and w.shape[0] >= 4096)

    def _shared_k_min_rows(self, w):
        """From how many rows the tcgen05 kernel with a shared k range beats the few-rows kernel, by
        measurement in a step's graph (o and down products of the 0.6B, 8B and 32B sizes): 17 for a small
        matrix (the few-rows kernel is bound by its round trips, not by its bytes); 9 for a large one (a
        second block of 8 rows costs the few-rows kernel a third more); 1 where the few-rows kernel with
        its one CTA of 16 features per SM (long k) leaves most of its last wave empty (5,120 features:
        320 CTAs on 148 SMs; a decode step of one row of the 32B sizes 14.13 against 13.74 ms)."""
        if self.tc_split_min_rows:
            return self.tc_split_min_rows
        o, k = w.shape
        waves = -(-o // 16) / self.sm_count
        if k > 3072 and -(-waves // 1) / waves > 1.25:
            return 1
        return 9 if w.numel() >= (1 << 23) else 17

    def _linear_tcgen05(self, x, w, out, n, o, k, epi, shape=0, splits=1, row_scale=None, residual=None):
        """shape: 0 lets the library choose its tile shape; 1 narrow, 2 deep, 3 wide, 4 and 5 persistent.
        splits > 1: the k range of a tile is shared by a cluster of that many CTAs.  row_scale: as in
        :meth:`linear`.  residual (x, norm_weight, partials): as in :meth:`linear_residual_norm`."""
        partials, parts, eps, width = row_scale if row_scale is not None else (None, 0, 0.0, 0)
        res_x, res_g, res_partials = residual if residual is not None else (None, None, None)
        self.launches += 1
        self.tc_shared_k_calls += splits > 1
        self.tc_folded_calls += partials is not None or res_x is not None
        self._err_armed = True
        _check(self._tc_lib().ifb_linear_tcgen05_ex(
            x.data_ptr(), w.data_ptr(), out.data_ptr(), _code(out), n, o, k, epi, int(shape), int(splits),
            _ptr(partials), int(parts), float(eps), int(width), _ptr(res_x), _ptr(res_g),
            _code(res_g) if res_g is not None else 0, _ptr(res_partials), self._dev_err.data_ptr(), self._stream()), "linear")

    def _tc_lib(self):
        if self._tc is None:
            self._tc = load_library("linear_tcgen05", progress=self._progress)
            self._tc.ifb_linear_tcgen05_ex.argtypes = [
                c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_float,
                c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p]
            self._tc.ifb_linear_tcgen05_split_clusters.argtypes = [c_int]
            self._tc.ifb_linear_tcgen05_fold_parts.argtypes = [c_int, c_int, c_int]
            self._tc.ifb_linear_tcgen05_qkv.argtypes = [
                c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_float, c_int,
                c_void_p, c_void_p, c_int, c_float, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p]
        return self._tc

    def tcgen05_splits(self, n, o, k, epi=0):
        """How many CTAs (a cluster) share the k range of a tile in the tcgen05 product of up to 512 rows
        (128 with the silu_gate epilogue): the most, up to 8, whose clusters for all tiles of 128 x 128
        run at the same time, each CTA with at least ``tc_split_min_k`` of k; 1 if that is none."""
        key = (n, o, k, bool(epi))
        hit = self._splits_memo.get(key)
        if hit is None:
            hit = self._splits_memo[key] = self._tcgen05_splits_rule(n, o, k, epi)
        return hit

    def _tcgen05_splits_rule(self, n, o, k, epi):
        if n > (128 if epi else 512):
            return 1
        tiles = -(-o // 128) * -(-n // 128)
        for splits in range(min(8, k // self.tc_split_min_k), 1, -1):
            if splits not in self._tc_clusters:
                self._tc_clusters[splits] = int(self._tc_lib().ifb_linear_tcgen05_split_clusters(splits))
            if tiles <= self._tc_clusters[splits]:
                return splits
        return 1

    def _linear_tcgen05_split(self, x, w, out, n, o, k, splits):
        """The one-tile kernel with the k range of a tile shared by a cluster of ``splits`` CTAs."""
        self._linear_tcgen05(x, w, out, n, o, k, 0, splits=splits)

    def check_device_errors(self):
        """Raise if a kernel recorded a fault that it contained: a bounded wait on a barrier that gave
        up, or a token id outside the vocabulary at the embedding (synchronises)."""
        if self._err_armed:
            self._err_armed = False
            code = int(self._dev_err.item())
            if code:
                self._dev_err.zero_()
                if code == 900:
                    raise KernelError("a token id outside the vocabulary reached the embedding (code 900): the step "
                                      "that sampled it had no valid logits; its output is not valid")
                raise KernelError(f"a kernel gave up waiting on a barrier (code {code}); its output is not valid")

    def _linear_gemv(self, x, w, out, n, o, k, epi, row_scale=None):
        self.launches += 1
        partials, parts, eps, width = row_scale if row_scale is not None else (None, 0, 0.0, 0)
        if partials is not None:
            _dense(partials, "row_scale partials", torch.float32)
            if partials.dim() != 2 or partials.shape[0] < parts or partials.shape[1] != n:
                raise KernelError("linear: row_scale partials must be [parts, rows]")
        _check(self.core.ifb_linear_gemv(x.data_ptr(), w.data_ptr(), out.data_ptr(), _code(out), n, o, k, epi,
                                         _ptr(partials), int(parts), float(eps), int(width), self._stream()), "linear")

    # A norm folded into the products around it: RMSNorm(v) = v * g * r with one r per row, so the product that
    # makes v writes v * g and partial sums of v^2, and the product that reads it multiplies by r at its end.
    def can_fold_norm(self, n, dtype, w, epilogue="none"):
        """Whether a product of ``n`` rows of ``dtype`` against ``w`` (with that epilogue) takes or makes a
        folded norm: on the tcgen05 kernel up to ``tc_fold_max_rows`` rows (one tile of rows: with many
        rows the longer epilogue costs what the norm's own launch did), on the few-rows kernel up to
        ``fold_max_rows``."""
        if not (dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.shape[1] % 8 == 0 and n > 0
                and self.fold_max_rows > 0):
            return False
        if self._on_tcgen05(n, w, epilogue):
            return n <= self.tc_fold_max_rows
        return n <= min(self.gemv_max_rows, self.fold_max_rows)

    def fold_parts(self, out_features, n=None, w=None):
        """Partial sums per row that :meth:`linear_residual_norm` writes for a product of ``n`` rows against
        ``w`` (without them: on the few-rows kernel)."""
        if n is not None and w is not None and self._on_tcgen05(n, w):
            splits = self.tcgen05_splits(n, w.shape[0], w.shape[1])
            return int(self._tc_lib().ifb_linear_tcgen05_fold_parts(int(n), int(out_features), int(splits)))
        return int(self.core.ifb_linear_gemv_parts(int(out_features), int(n) if n is not None else 1 << 20))

    def linear_residual_norm(self, a, w, x, norm_weight, out, partials):
        """x += a w^T (x float32, in place); out = x * norm_weight (bfloat16); partials[p, n] = the sum
        of squares of row n of x over part p's features.  With ``linear(..., row_scale=(partials,
        fold_parts(o, n, w), eps, o))`` after it this is x += a w^T followed by an RMSNorm of x."""
        _dense(a, "a", torch.bfloat16), _dense(w, "w", torch.bfloat16), _dense(x, "x", torch.float32)
        _dense(out, "out", torch.bfloat16), _dense(partials, "partials", torch.float32), _dense(norm_weight, "norm_weight")
        n, k = a.shape
        o = w.shape[0]
        parts = self.fold_parts(o, n, w)
        if w.shape[1] != k or x.shape != (n, o) or out.shape != (n, o) or norm_weight.numel() != o \
                or partials.dim() != 2 or partials.shape[0] < parts or partials.shape[1] != n:
            raise KernelError("linear_residual_norm: sizes of a, w, x, norm_weight, out and partials do not match")
        if not self.can_fold_norm(n, a.dtype, w):
            raise KernelError("linear_residual_norm: only for bfloat16 (see can_fold_norm)")
        if self._on_tcgen05(n, w):
            return self._linear_tcgen05(a, w, out, n, o, k, 0, splits=self.tcgen05_splits(n, o, k),
                                        residual=(x, norm_weight, partials))
        self.launches += 1
        _check(self.core.ifb_linear_gemv_residual_norm(
            a.data_ptr(), w.data_ptr(), x.data_ptr(), norm_weight.data_ptr(), _code(norm_weight), out.data_ptr(),
            partials.data_ptr(), n, o, k, self._stream()), "linear_residual_norm")

    # The split-k product with scratch from the caller: not on linear()'s path (tcgen05 takes 65 rows and more, the
    # kernel above 64 and fewer); it is the kernel whose static-scratch variant the library linear_skinny_static exports.
    def linear_splits(self, n, o, k):
        """CTAs that share the k range of one 64-feature tile: enough to cover the SMs twice, and
        at least 256 of k each."""
        blocks = 1 if n <= 8 else 2 if n <= 16 else 4 if n <= 32 else 8
        tiles = -(-o // 64) * -(-n // (blocks * 8))
        return max(1, min(-(-2 * self.sm_count // tiles), k // 256))

    def _linear_skinny(self, x, w, out, n, o, k, epi, splits=None):
        if splits is None:
            splits = self.linear_splits(n, o, k)
        partials = counters = None
        if splits > 1:
            nf, nc = ctypes.c_longlong(), ctypes.c_longlong()
            self.core.ifb_linear_skinny_scratch(n, o, epi, splits, ctypes.byref(nf), ctypes.byref(nc))
            if self._lin_partials is None or self._lin_partials.numel() < nf.value:
                self._lin_partials = torch.empty(max(nf.value, 1 << 20), dtype=torch.float32, device="cuda")
                self.scratch_generation += 1
            if self._lin_counters is None or self._lin_counters.numel() < nc.value:
                self._lin_counters = torch.zeros(max(nc.value, 1 << 14), dtype=torch.int32, device="cuda")
                self.scratch_generation += 1
            partials, counters = self._lin_partials, self._lin_counters
        self.launches += 1
        _check(self.core.ifb_linear_skinny(x.data_ptr(), w.data_ptr(), out.data_ptr(), _code(out), _ptr(partials),
                                           _ptr(counters), n, o, k, epi, splits, self._stream()), "linear")

    # The q | k | v projection of a decode step with the head norm, the rotation and the page store in its epilogue.
    def can_fuse_qkv(self, n, dtype, w_qkv, head_dim, rotary_dim, interleaved, kv_pages):
        """Whether :meth:`linear_qkv_rope_store` takes a step of ``n`` rows: bfloat16, heads rotated whole in
        the half-split pairing (or not rotated); up to 16 rows on the few-rows kernel (heads of 64, 128 or
        256), or up to 128 rows on the tcgen05 kernel in its shared-k form (heads of 128)."""
        if not (self.fused_qkv and n > 0 and dtype == torch.bfloat16 and w_qkv.dtype == torch.bfloat16
                and w_qkv.shape[1] % 8 == 0 and (rotary_dim == 0 or (rotary_dim == head_dim and not interleaved))
                and (kv_pages is None or kv_pages.dtype == torch.bfloat16)):
            return False
        return self._fused_qkv_route(n, w_qkv, head_dim) is not None

    def _fused_qkv_route(self, n, w_qkv, head_dim):
        """"gemv", "tcgen05" or None for the fused q | k | v product of ``n`` rows."""
        if n <= 16 and head_dim in (64, 128, 256) and not self._on_tcgen05(n, w_qkv, shared_k=False):
            return "gemv"
        if n <= 128 and head_dim == 128 and self.fused_qkv_tc and self._on_tcgen05(n, w_qkv) \
                and self.tcgen05_splits(n, w_qkv.shape[0], w_qkv.shape[1]) > 1:
            return "tcgen05"
        return None

    def linear_qkv_rope_store(self, x, w_qkv, qkv, num_heads, num_kv_heads, head_dim, q_weight, k_weight, eps, rope_table,
                              slot_mapping, kv_pages, row_scale=None):
        """qkv = x w_qkv^T, then per head what :meth:`qk_norm_rope_store` does (RMSNorm of the q and k heads,
        rotation by the angles of ``rope_table``, k and v into the pages at ``slot_mapping``), in one launch."""
        _dense(x, "x", torch.bfloat16), _dense(w_qkv, "w_qkv", torch.bfloat16), _dense(qkv, "qkv", torch.bfloat16)
        n, k = x.shape
        width = (num_heads + 2 * num_kv_heads) * head_dim
        if w_qkv.shape != (width, k) or qkv.shape != (n, width):
            raise KernelError("linear_qkv_rope_store: sizes of x, w_qkv and qkv do not match the heads")
        wd = F32
        for wt in (q_weight, k_weight):
            if wt is not None:
                _dense(wt, "norm weight")
                if wt.numel() != head_dim:
                    raise KernelError("linear_qkv_rope_store: norm weight length is not head_dim")
                wd = _code(wt)
        if q_weight is not None and k_weight is not None and q_weight.dtype != k_weight.dtype:
            raise KernelError("linear_qkv_rope_store: q and k norm weights differ in dtype")
        if rope_table is not None:
            _dense(rope_table, "rope_table", torch.float32)
            if rope_table.shape != (n, head_dim):
                raise KernelError("linear_qkv_rope_store: rope_table is [tokens, head_dim]")
        page_size = 1
        if slot_mapping is not None:
            _dense(slot_mapping, "slot_mapping", torch.int32), _dense(kv_pages, "kv_pages", torch.bfloat16)
            if kv_pages.dim() != 5 or kv_pages.shape[1] != 2 or kv_pages.shape[2] != num_kv_heads \
                    or kv_pages.shape[4] != head_dim or slot_mapping.numel() != n:
                raise KernelError("linear_qkv_rope_store: kv_pages is not [pages, 2, kv_heads, page_size, head_dim]")
            page_size = kv_pages.shape[3]
        partials, parts, seps, swidth = row_scale if row_scale is not None else (None, 0, 0.0, 0)
        self.launches += 1
        self.fused_qkv_calls += 1
        route = self._fused_qkv_route(n, w_qkv, head_dim)
        if route is None:
            raise KernelError("linear_qkv_rope_store: no kernel takes these sizes (see can_fuse_qkv)")
        if route == "tcgen05":
            self._err_armed = True
            self.tc_shared_k_calls += 1
            self.tc_folded_calls += partials is not None
            _check(self._tc_lib().ifb_linear_tcgen05_qkv(
                x.data_ptr(), w_qkv.data_ptr(), qkv.data_ptr(), n, num_heads, num_kv_heads, head_dim, k,
                self.tcgen05_splits(n, width, k), _ptr(partials), int(parts), float(seps), int(swidth), _ptr(q_weight),
                _ptr(k_weight), wd, float(eps), _ptr(rope_table), _ptr(slot_mapping),
                _ptr(kv_pages) if slot_mapping is not None else 0, page_size, self._dev_err.data_ptr(), self._stream()),
                "linear_qkv_rope_store")
            return
        _check(self.core.ifb_linear_gemv_qkv(
            x.data_ptr(), w_qkv.data_ptr(), qkv.data_ptr(), n, num_heads, num_kv_heads, head_dim, k, _ptr(partials),
            int(parts), float(seps), int(swidth), _ptr(q_weight), _ptr(k_weight), wd, float(eps), _ptr(rope_table),
            _ptr(slot_mapping), _ptr(kv_pages) if slot_mapping is not None else 0, page_size, self._stream()),
            "linear_qkv_rope_store")

    # ------------------------------------------------------------------ q/k norm, rotation, store
    def rope_table(self, positions, inv_freq, out, gain=1.0):
        """out[tok, i] = gain * (cos, sin)(positions[tok] * inv_freq[i]), float32 ``[tokens, 2 * len(inv_freq)]``."""
        _dense(positions, "positions", torch.int32), _dense(inv_freq, "inv_freq", torch.float32)
        _dense(out, "out", torch.float32)
        n, half = positions.numel(), inv_freq.numel()
        if out.shape != (n, 2 * half):
            raise KernelError("rope_table: out is [tokens, 2 * len(inv_freq)]")
        self.launches += 1
        _check(self.core.ifb_rope_table(positions.data_ptr(), inv_freq.data_ptr(), half, out.data_ptr(), n, float(gain), self._stream()),
               "rope_table")

    def qk_norm_rope_store(self, qkv, num_heads, num_kv_heads, head_dim, q_weight, k_weight, eps, inv_freq,
                           rotary_dim, interleaved, positions, slot_mapping, kv_pages, rope_table=None):
        _dense(qkv, "qkv")
        n = qkv.shape[0]
        if qkv.shape[1] != (num_heads + 2 * num_kv_heads) * head_dim:
            raise KernelError("qk_norm_rope_store: qkv width is not (heads + 2 kv_heads) * head_dim")
        wd = F32
        for wt in (q_weight, k_weight):
            if wt is not None:
                _dense(wt, "norm weight")
                if wt.numel() != head_dim:
                    raise KernelError("qk_norm_rope_store: norm weight length is not head_dim")
                wd = _code(wt)
        if q_weight is not None and k_weight is not None and q_weight.dtype != k_weight.dtype:
            raise KernelError("qk_norm_rope_store: q and k norm weights differ in dtype")
        if inv_freq is not None:
            _dense(inv_freq, "inv_freq", torch.float32), _dense(positions, "positions", torch.int32)
            if inv_freq.numel() != rotary_dim // 2 or positions.numel() != n:
                raise KernelError("qk_norm_rope_store: inv_freq or positions has the wrong length")
            if rope_table is not None:
                _dense(rope_table, "rope_table", torch.float32)
                if rope_table.shape != (n, rotary_dim):
                    raise KernelError("qk_norm_rope_store: rope_table is [tokens, rotary_dim]")
        page_size = 1
        if slot_mapping is not None:
            _dense(slot_mapping, "slot_mapping", torch.int32), _dense(kv_pages, "kv_pages", qkv.dtype)
            if kv_pages.dim() != 5 or kv_pages.shape[1] != 2 or kv_pages.shape[2] != num_kv_heads \
                    or kv_pages.shape[4] != head_dim or slot_mapping.numel() != n:
                raise KernelError("qk_norm_rope_store: kv_pages is not [pages, 2, kv_heads, page_size, head_dim]")
            page_size = kv_pages.shape[3]
        self.launches += 1
        _check(self.core.ifb_qk_norm_rope_store(
            qkv.data_ptr(), _code(qkv), n, num_heads, num_kv_heads, head_dim, _ptr(q_weight), _ptr(k_weight), wd,
            float(eps), _ptr(inv_freq), _ptr(rope_table) if inv_freq is not None else 0, int(rotary_dim),
            int(bool(interleaved)), _ptr(positions), _ptr(slot_mapping),
            _ptr(kv_pages) if slot_mapping is not None else 0, page_size, self._stream()), "qk_norm_rope_store")

    # ------------------------------------------------------------------ attention
    def paged_attention(self, qkv, num_heads, num_kv_heads, head_dim, kv_pages, block_tables, cu_q, seq_lens, out,
                        scale, window, max_q_len, max_seq_len, min_q_len=1, weight_terms=1):
        """``weight_terms`` 2 (tensor-core route only): a softmax weight enters the weighted sum as two bfloat16 terms, its
        rounding and what the rounding left out, so that 16 bits of the float32 weight count; the tcgen05 prompt kernel, which
        has one term, is then not taken."""
        _dense(qkv, "qkv"), _dense(kv_pages, "kv_pages", qkv.dtype), _dense(out, "out", qkv.dtype)
        _dense(cu_q, "cu_q", torch.int32), _dense(seq_lens, "seq_lens", torch.int32)
        if block_tables.dtype != torch.int32 or block_tables.stride(1) != 1:
            raise KernelError("paged_attention: block_tables must be int32 with unit stride along pages")
        n = qkv.shape[0]
        r = seq_lens.numel()
        if cu_q.numel() != r + 1 or block_tables.shape[0] < r or out.shape != (n, num_heads * head_dim):
            raise KernelError("paged_attention: sizes of cu_q, seq_lens, block_tables and out do not match")
        if kv_pages.dim() != 5 or kv_pages.shape[1] != 2 or kv_pages.shape[2] != num_kv_heads \
                or kv_pages.shape[4] != head_dim:
            raise KernelError("paged_attention: kv_pages is not [pages, 2, kv_heads, page_size, head_dim]")
        group = num_heads // num_kv_heads
        if qkv.dtype == torch.bfloat16 and head_dim % 16 == 0 and head_dim <= 256 and group <= 16 \
                and num_heads % num_kv_heads == 0:
            return self._paged_attention_mma(qkv, num_heads, num_kv_heads, head_dim, kv_pages, block_tables, cu_q,
                                             seq_lens, out, scale, window, max_q_len, max_seq_len, n, r,
                                             min_q_len=min_q_len, weight_terms=weight_terms)
        self.launches += 1
        _check(self.core.ifb_paged_attention_simt(
            qkv.data_ptr(), _code(qkv), qkv.stride(0), kv_pages.data_ptr(), block_tables.data_ptr(),
            block_tables.stride(0), cu_q.data_ptr(), seq_lens.data_ptr(), out.data_ptr(), n, r, num_heads,
            num_kv_heads, head_dim, kv_pages.shape[3], float(scale), int(window), self._stream()), "paged_attention")

    def _attention_tc(self, qkv, num_heads, num_kv_heads, head_dim, kv_pages, block_tables, cu_q, seq_lens, out, scale,
                      window, max_q_len, n, r):
        if self._attn_tc is None:
            self._attn_tc = load_library("attention_tc", progress=self._progress)
            self._attn_tc.ifb_attention_tc.argtypes = [c_void_p, c_int, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_void_p,
                                                       c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
                                                       c_int, c_int, c_void_p]
        self._err_armed = True
        self.launches += 1
        self.tc_attention_calls += 1
        _check(self._attn_tc.ifb_attention_tc(
            qkv.data_ptr(), qkv.stride(0), kv_pages.data_ptr(), kv_pages.shape[0], block_tables.data_ptr(),
            block_tables.stride(0), cu_q.data_ptr(), seq_lens.data_ptr(), out.data_ptr(), self._dev_err.data_ptr(), n, r,
            num_heads, num_kv_heads, head_dim, kv_pages.shape[3], float(scale), int(window), int(max_q_len), self._stream()),
            "paged_attention")

    def attention_library(self, head_dim, weight_terms=1):
        if weight_terms not in (1, 2):
            raise KernelError("attention: a softmax weight has one or two bfloat16 terms")
        key = head_dim if weight_terms == 1 else (head_dim, weight_terms)
        lib = self._attn_mma.get(key)
        if lib is None:
            defines = {"HEAD_DIM": head_dim} if weight_terms == 1 else {"HEAD_DIM": head_dim, "WEIGHT_TERMS": weight_terms}
            lib = load_library("attention_mma", defines, progress=self._progress)
            lib.ifb_attention_mma.argtypes = [c_void_p, c_int, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_void_p,
                                              c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                              c_int, c_float, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]
            lib.ifb_attention_mma_scratch_floats.restype = c_longlong
            lib.ifb_attention_mma_scratch_floats.argtypes = [c_int, c_int, c_int]
            self._attn_mma[key] = lib
        return lib

    def attention_splits(self, num_requests, num_kv_heads, max_seq_len, window=0):
        """How many CTAs share one (request, key/value head) of the small-q kernel: as many as
        keep the whole grid resident at once (two CTAs fit on an SM), so that no second wave
        runs, and no fewer than ``split_min_keys`` keys per split (256, four tiles: with 128 a lone
        request's 32 partial results cost more to merge than the shorter splits saved)."""
        reach = min(max_seq_len, window + 16) if window else max_seq_len
        fit = (2 * self.sm_count) // max(1, num_requests * num_kv_heads)
        return max(1, min(fit, -(-reach // self.split_min_keys), 32))

    def attention_scratch(self, floats):
        if self._attn_scratch is None or self._attn_scratch.numel() < floats:
            self._attn_scratch = torch.empty(max(floats, 1 << 16), dtype=torch.float32, device="cuda")
            self.scratch_generation += 1
        return self._attn_scratch

    def _paged_attention_mma(self, qkv, num_heads, num_kv_heads, head_dim, kv_pages, block_tables, cu_q, seq_lens, out,
                             scale, window, max_q_len, max_seq_len, n, r, num_splits=None, min_q_len=1, weight_terms=1):
        lib = self.attention_library(head_dim, weight_terms)
        group = num_heads // num_kv_heads
        only_small = max_q_len * group <= 16
        if num_splits is None:
            num_splits = self.attention_splits(r, num_kv_heads, max_seq_len, window)
        need = lib.ifb_attention_mma_scratch_floats(n, num_heads, num_splits)
        if need * 4 > self.attention_scratch_cap:
            num_splits, need = 1, 0
        scratch = self.attention_scratch(need) if need else None
        counters = None
        if need:
            if self._attn_counters is None or self._attn_counters.numel() < r * num_kv_heads:
                self._attn_counters = torch.zeros(max(r * num_kv_heads, 4096), dtype=torch.int32, device="cuda")
                self.scratch_generation += 1
            counters = self._attn_counters
        use_tc = (not only_small and self.attention_tc and weight_terms == 1 and head_dim == 128 and 128 % group == 0
                  and kv_pages.shape[3] in (16, 32, 64) and kv_pages.data_ptr() % 128 == 0)
        if use_tc:
            self._attention_tc(qkv, num_heads, num_kv_heads, head_dim, kv_pages, block_tables, cu_q, seq_lens, out, scale,
                               window, max_q_len, n, r)
            if min_q_len * group > 16:
                return                 # no request of this step is left for the small-q kernel
            only_small = True          # the tile kernel's requests are done; the small-q kernel takes the rest
        self.launches += 1 + (0 if only_small else 1)
        self.small_q_calls += 1
        if self.attention_tma and head_dim % 64 == 0 and kv_pages.shape[3] in (16, 32, 64) \
                and kv_pages.data_ptr() % 128 == 0 and kv_pages.numel() // head_dim < 0x7fffffff:
            self.small_q_tma_calls += 1        # the library's own condition for its TMA path
        self._err_armed = True
        _check(lib.ifb_attention_mma(
            qkv.data_ptr(), qkv.stride(0), kv_pages.data_ptr(), kv_pages.shape[0], block_tables.data_ptr(),
            block_tables.stride(0), cu_q.data_ptr(), seq_lens.data_ptr(), out.data_ptr(), _ptr(scratch), _ptr(counters),
            self._dev_err.data_ptr(), n, r, num_heads, num_kv_heads, head_dim, kv_pages.shape[3], float(scale), int(window),
            int(max_q_len), int(num_splits), 1, 0 if only_small else 1, 1 if self.attention_tma else 0, self._stream()),
            "paged_attention")

    # ------------------------------------------------------------------ post-norm sublayers, recurrence, talking attention
    def _mix_lib(self):
        if self._mix is None:
            m = self._mix = load_library("mixers", progress=self._progress)
            m.ifb_embed_sinusoid.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                             c_int, c_void_p, c_void_p]
            m.ifb_residual_postnorm.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_float, c_void_p, c_int,
                                                c_int, c_void_p]
            m.ifb_cast_rows.argtypes = [c_void_p, c_void_p, c_longlong, c_void_p]
            m.ifb_wide_norm_store.argtypes = [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_float,
                                              c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p]
            m.ifb_gated_scan_slabs.argtypes = [c_int, c_int]
            m.ifb_gated_scan.argtypes = [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_float,
                                         c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int,
                                         c_int, c_int, c_int, c_int, c_void_p]
            m.ifb_gated_scan_scratch_floats.restype = c_longlong
            m.ifb_gated_scan_scratch_floats.argtypes = [c_int, c_int, c_int, c_int, c_int]
            m.ifb_attention_talk.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                             c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                             c_float, c_float, c_void_p]
            m.ifb_attention_talk_mma_fits.argtypes = [c_int, c_int, c_int]
            m.ifb_attention_talk_mma.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                                 c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                                 c_float, c_float, c_int, c_void_p, c_void_p]
        return self._mix

    def embed_sinusoid(self, table, ids, positions, inv_freq, out, half=None):
        """out[n] = table[ids[n]] + e(positions[n]) in float32, e[2i] = sin(p * inv_freq[i]), e[2i+1] = cos of the
        same angle (inv_freq float64).  ``half``: the same rows in bfloat16, for the products that read them."""
        _dense(table, "table"), _dense(ids, "ids", torch.int32), _dense(positions, "positions", torch.int32)
        _dense(inv_freq, "inv_freq", torch.float64), _dense(out, "out", torch.float32)
        n, hidden = out.shape
        if table.shape[1] != hidden or ids.numel() != n or positions.numel() != n or inv_freq.numel() != (hidden + 1) // 2:
            raise KernelError("embed_sinusoid: sizes of table, ids, positions, inv_freq and out do not match")
        if half is not None and (_dense(half, "half", torch.bfloat16).shape != out.shape):
            raise KernelError("embed_sinusoid: half has the shape of out")
        self.launches += 1
        self._err_armed = True
        _check(self._mix_lib().ifb_embed_sinusoid(table.data_ptr(), _code(table), ids.data_ptr(), positions.data_ptr(),
                                                  inv_freq.data_ptr(), out.data_ptr(), _ptr(half), n, hidden, table.shape[0],
                                                  self._dev_err.data_ptr(), self._stream()), "embed_sinusoid")

    def residual_postnorm(self, x, y, g, scale, eps, half=None):
        """x += y / sqrt(mean(y^2) + eps) * g * scale, row by row in float32 (g: one number, scale: per feature).
        ``half``: the updated rows in bfloat16."""
        _dense(x, "x", torch.float32), _dense(y, "y", torch.float32), _dense(g, "g"), _dense(scale, "scale")
        n, hidden = x.shape
        if y.shape != x.shape or g.numel() != 1 or scale.numel() != hidden:
            raise KernelError("residual_postnorm: sizes of x, y, g and scale do not match")
        if half is not None and (_dense(half, "half", torch.bfloat16).shape != x.shape):
            raise KernelError("residual_postnorm: half has the shape of x")
        self.launches += 1
        _check(self._mix_lib().ifb_residual_postnorm(x.data_ptr(), y.data_ptr(), g.data_ptr(), _code(g), scale.data_ptr(),
                                                     _code(scale), float(eps), _ptr(half), n, hidden, self._stream()),
               "residual_postnorm")

    def cast_rows(self, x, out):
        """out = x rounded to bfloat16 (x float32, same shape)."""
        _dense(x, "x", torch.float32), _dense(out, "out", torch.bfloat16)
        if out.shape != x.shape:
            raise KernelError("cast_rows: out has the shape of x")
        self.launches += 1
        _check(self._mix_lib().ifb_cast_rows(x.data_ptr(), out.data_ptr(), x.numel(), self._stream()), "cast_rows")

    def wide_norm_store(self, proj, q_width, k_width, v_col, head_dim, q_weight, k_weight, eps, q_out, slot_mapping, kv_pages):
        """proj [n, >= q_width + k_width] float32 holds q then k of every token.  q_out = RMSNorm of the whole q
        (one statistic per token) times q_weight; the key page gets the same of k; the value page gets k as
        projected (``v_col`` < 0) or proj[:, v_col : v_col + k_width].  A weight of None: no norm."""
        _dense(proj, "proj", torch.float32), _dense(q_out, "q_out")
        n, ld = proj.shape
        wd = F32
        for wt, width in ((q_weight, q_width), (k_weight, k_width)):
            if wt is not None:
                _dense(wt, "norm weight")
                if wt.numel() != width:
                    raise KernelError("wide_norm_store: a norm weight has the length of its whole projection")
                wd = _code(wt)
        if q_weight is not None and k_weight is not None and q_weight.dtype != k_weight.dtype:
            raise KernelError("wide_norm_store: q and k norm weights differ in dtype")
        if q_out.shape != (n, q_width) or ld < q_width + k_width or (v_col >= 0 and ld < v_col + k_width):
            raise KernelError("wide_norm_store: sizes of proj and q_out do not match the widths")
        page_size = 1
        if slot_mapping is not None:
            _dense(slot_mapping, "slot_mapping", torch.int32), _dense(kv_pages, "kv_pages", q_out.dtype)
            if kv_pages.dim() != 5 or kv_pages.shape[1] != 2 or kv_pages.shape[2] * kv_pages.shape[4] != k_width \
                    or kv_pages.shape[4] != head_dim or slot_mapping.numel() != n:
                raise KernelError("wide_norm_store: kv_pages is not [pages, 2, kv_heads, page_size, head_dim]")
            page_size = kv_pages.shape[3]
        self.launches += 1
        _check(self._mix_lib().ifb_wide_norm_store(
            proj.data_ptr(), ld, q_width, k_width, int(v_col), head_dim, _ptr(q_weight), _ptr(k_weight), wd, float(eps),
            q_out.data_ptr(), _code(q_out), _ptr(slot_mapping), _ptr(kv_pages) if slot_mapping is not None else 0, page_size,
            n, self._stream()), "wide_norm_store")

    def gated_scan_slabs(self, dim, vdim):
        """Column slabs a head of the gated recurrence is split into; with more than one, ``gated_scan`` needs ``raw``."""
        return int(self._mix_lib().ifb_gated_scan_slabs(int(dim), int(vdim)))

    def gated_scan(self, proj, q_col, f_col, v_col, bias, lower, norm_weight, eps, state, state_slots, cu_q, seq_lens, out,
                   heads, dim, vdim, raw=None, max_q_len=1):
        """The gated linear recurrence over this step's tokens of every request (csrc/gated_scan.cu): proj [n, ld]
        float32 holds q_raw, f_raw (heads * dim each) and v (heads * vdim) at the given columns; state
        [slots, heads, dim, vdim] float32 is read and written at each request's slot; out [n, heads * vdim] gets the
        normalised outputs.  A request with seq_lens 0 is padding: its state is left alone.  ``max_q_len``: the most
        tokens a request brings; from ``scan_block_min`` on, the requests are cut into blocks of 64 tokens that run
        side by side (three launches), which differs from the one-launch walk by rounding only."""
        _dense(proj, "proj", torch.float32), _dense(state, "state", torch.float32), _dense(out, "out")
        _dense(state_slots, "state_slots", torch.int32), _dense(cu_q, "cu_q", torch.int32), _dense(seq_lens, "seq_lens", torch.int32)
        n, ld = proj.shape
        r = seq_lens.numel()
        hd, hv = heads * dim, heads * vdim
        for t, size, name in ((bias, hd, "bias"), (lower, hd, "lower"), (norm_weight, vdim, "norm_weight")):
            _dense(t, name)
            if t.numel() != size or t.dtype != bias.dtype:
                raise KernelError(f"gated_scan: {name} has the wrong length or a dtype of its own")
        if state.shape[1:] != (heads, dim, vdim) or out.shape != (n, hv) or cu_q.numel() != r + 1 or state_slots.numel() < r \
                or max(q_col, f_col) + hd > ld or v_col + hv > ld:
            raise KernelError("gated_scan: sizes of proj, state, out and the request arrays do not match")
        if raw is not None and (_dense(raw, "raw", torch.float32).shape != (n, hv)):
            raise KernelError("gated_scan: raw is float32 [tokens, heads * vdim]")
        scratch = None
        if max_q_len >= self.scan_block_min:
            need = int(self._mix_lib().ifb_gated_scan_scratch_floats(n, r, heads, dim, vdim))
            if self._scan_scratch is None or self._scan_scratch.numel() < need:
                self._scan_scratch = torch.empty(need, dtype=torch.float32, device="cuda")
                self.scratch_generation += 1
            scratch = self._scan_scratch
            self.scan_blocked_calls += 1
        self.launches += (1 if scratch is None else 3) + (0 if raw is None or self.gated_scan_slabs(dim, vdim) == 1 else 1)
        _check(self._mix_lib().ifb_gated_scan(
            proj.data_ptr(), ld, int(q_col), int(f_col), int(v_col), bias.data_ptr(), lower.data_ptr(), norm_weight.data_ptr(),
            _code(bias), float(eps), state.data_ptr(), state_slots.data_ptr(), cu_q.data_ptr(), seq_lens.data_ptr(),
            out.data_ptr(), _code(out), _ptr(raw), _ptr(scratch), r, n, heads, dim, vdim, self._stream()), "gated_scan")

    def attention_talk(self, q, num_heads, num_kv_heads, head_dim, kv_pages, block_tables, cu_q, seq_lens, out, scale,
                       chunk=0, slope_exponent=0.0, talk=None, gate=None, gate_col=0, max_q_len=0, max_seq_len=0):
        """Attention over the pages with the heads' scores mixed before the softmax (csrc/attention_talk.cu).
        q [n, heads * head_dim]: the queries, already normalised.  ``chunk`` 0: every earlier key is visible.
        ``slope_exponent`` 0: no distance bias.  ``talk`` [heads, heads] or None.  ``gate``: a float32 matrix whose
        columns gate_col .. gate_col + heads * head_dim hold the gate before its sigmoid, or None.  ``max_q_len`` and
        ``max_seq_len`` (the most tokens a request brings, and an upper bound of the longest request after the step; 0:
        unknown) only decide how the work is spread: a step of few tokens over long contexts has its keys split
        over several CTAs."""
        _dense(q, "q"), _dense(kv_pages, "kv_pages", q.dtype), _dense(out, "out", q.dtype)
        _dense(cu_q, "cu_q", torch.int32), _dense(seq_lens, "seq_lens", torch.int32)
        if block_tables.dtype != torch.int32 or block_tables.stride(1) != 1:
            raise KernelError("attention_talk: block_tables must be int32 with unit stride along pages")
        n, r = q.shape[0], seq_lens.numel()
        width = num_heads * head_dim
        if q.shape != (n, width) or out.shape != (n, width) or cu_q.numel() != r + 1 or block_tables.shape[0] < r:
            raise KernelError("attention_talk: sizes of q, out, cu_q, seq_lens and block_tables do not match")
        if kv_pages.dim() != 5 or kv_pages.shape[1] != 2 or kv_pages.shape[2] != num_kv_heads or kv_pages.shape[4] != head_dim:
            raise KernelError("attention_talk: kv_pages is not [pages, 2, kv_heads, page_size, head_dim]")
        if talk is not None and _dense(talk, "talk").shape != (num_heads, num_heads):
            raise KernelError("attention_talk: talk is [heads, heads]")
        gate_ptr = gate_ld = 0
        if gate is not None:
            _dense(gate, "gate", torch.float32)
            if gate.shape[0] != n or gate_col + width > gate.shape[1]:
                raise KernelError("attention_talk: gate has a row per token and heads * head_dim columns from gate_col")
            gate_ptr, gate_ld = gate.data_ptr() + 4 * int(gate_col), gate.shape[1]
        self.launches += 1
        if self.talk_mma and q.dtype == torch.bfloat16 and self._mix_lib().ifb_attention_talk_mma_fits(num_heads, num_kv_heads,
                                                                                                       head_dim):
            # bfloat16 on the tensor cores (csrc/attention_talk_mma.cu); other sizes and float32 run the plain kernel
            self.talk_mma_calls += 1
            splits, parts = self._talk_splits(n, r, num_heads, head_dim, int(chunk or 0), max_q_len, max_seq_len), None
            if splits > 1:
                parts = self.attention_scratch(n * num_heads * splits * (head_dim + 2))
                self.launches += 1
                self.talk_split_calls += 1
            return _check(self._mix_lib().ifb_attention_talk_mma(
                q.data_ptr(), kv_pages.data_ptr(), block_tables.data_ptr(), block_tables.stride(0), cu_q.data_ptr(),
                seq_lens.data_ptr(), _ptr(talk), _code(talk) if talk is not None else 0, gate_ptr, gate_ld, out.data_ptr(), n, r,
                num_heads, num_kv_heads, head_dim, kv_pages.shape[3], int(chunk or 0), float(scale),
                float(slope_exponent or 0.0), splits, _ptr(parts), self._stream()), "attention_talk")
        _check(self._mix_lib().ifb_attention_talk(
            q.data_ptr(), _code(q), kv_pages.data_ptr(), block_tables.data_ptr(), block_tables.stride(0), cu_q.data_ptr(),
            seq_lens.data_ptr(), _ptr(talk), _code(talk) if talk is not None else 0, gate_ptr, gate_ld, out.data_ptr(), n, r,
            num_heads, num_kv_heads, head_dim, kv_pages.shape[3], int(chunk or 0), float(scale), float(slope_exponent or 0.0),
            self._stream()), "attention_talk")

    def _talk_splits(self, n, r, num_heads, head_dim, chunk, max_q_len, max_seq_len):
        """CTAs that share the keys of one query tile of the tensor-core talking attention: 1 unless the step's tiles
        alone leave most SMs idle (few query tokens) and a query may see many keys; then enough to fill the device
        once, with no fewer than four tiles of 32 keys each.  Up to 4 for a prompt of few tiles (see below)."""
        if not max_q_len or not max_seq_len:
            return 1
        reach = min(chunk, max_seq_len) if chunk else max_seq_len
        tiles = (-(-n // 16) + r) * -(-num_heads // 16)
        if max_q_len > 64:
            # a prompt: a tile late in its chunk has many times the keys of an early one, and with less than two CTAs
            # per SM the longest tile is the kernel's time; shares of at most a quarter of the keys even that out
            return max(1, min(4, reach // 128)) if tiles < 2 * self.sm_count else 1
        return max(1, min(self.sm_count // max(1, tiles), reach // 128, 32))

    # ------------------------------------------------------------------ sandwich-norm blocks, state recurrences, routed experts
    def _hyb_lib(self):
        if self._hyb is None:
            m = self._hyb = load_library("hybrid", progress=self._progress)
            m.ifb_residual_norm_update.argtypes = [c_void_p, c_void_p, c_void_p, c_float, c_float, c_void_p, c_int, c_void_p, c_int,
                                                   c_float, c_void_p, c_int, c_int, c_int, c_void_p]
            m.ifb_add_rows.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]
            m.ifb_scaled_sum.argtypes = [c_void_p, c_void_p, c_float, c_int, c_longlong, c_void_p, c_int, c_void_p]
            m.ifb_token_side_gate.argtypes = [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_int,
                                              c_int, c_int, c_void_p]
            m.ifb_softcap.argtypes = [c_void_p, c_float, c_longlong, c_void_p]
            m.ifb_token_shift_mix.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                              c_int, c_int, c_int, c_void_p]
            m.ifb_linear_scan_slabs.argtypes = [c_int, c_int]
            m.ifb_linear_scan_scratch_floats.restype = c_longlong
            m.ifb_linear_scan_scratch_floats.argtypes = [c_int, c_int, c_int, c_int, c_int]
            m.ifb_linear_scan.argtypes = [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int,
                                          c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_float, c_float, c_void_p, c_void_p,
                                          c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                          c_int, c_void_p]
            m.ifb_gated_unit_scan.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                              c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p]
            m.ifb_gated_unit_scratch_floats.restype = c_longlong
            m.ifb_gated_unit_scratch_floats.argtypes = [c_int, c_int, c_int]
            m.ifb_rotary_store.argtypes = [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_int, c_int, c_float,
                                           c_void_p, c_int, c_void_p, c_int, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p,
                                           c_int, c_int, c_int, c_void_p]
            m.ifb_rotate_rows.argtypes = [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]
            m.ifb_paged_attention_streams.argtypes = [c_void_p, c_int, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_int,
                                                      c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                                      c_int, c_float, c_int, c_void_p, c_int, c_void_p]
            m.ifb_moe_route.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p]
            m.ifb_moe_plan.argtypes = [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p]
            m.ifb_moe_linear.argtypes = [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int,
                                         c_int, c_int, c_int, c_int, c_int, c_void_p]
            m.ifb_moe_combine.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p]
            m.ifb_moe_route_plan_small.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                                   c_int, c_int, c_int, c_int, c_float, c_void_p]
            m.ifb_moe_plan_padded.argtypes = [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p]
            m.ifb_moe_gather_rows.argtypes = [c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p]
            m.ifb_rglru_conv.argtypes = [c_void_p, c_longlong, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                         c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_int,
                                         c_int, c_int, c_int, c_int, c_void_p]
            m.ifb_rglru_scratch_floats.restype = c_longlong
            m.ifb_rglru_scratch_floats.argtypes = [c_int, c_int, c_int]
            m.ifb_rglru_scan.argtypes = [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p,
                                         c_longlong, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                         c_void_p, c_int, c_int, c_int, c_void_p]
            m.ifb_moe_gather_scaled.argtypes = [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int,
                                                c_void_p]
        return self._hyb

    def residual_norm_update(self, x, y, post_weight, eps, out=None, next_weight=None, y2=None, scale=1.0, scale2=1.0):
        """x += y / sqrt(mean(y^2) + eps) * post_weight, row by row in float32.  ``out``: the updated rows for the next
        product in out's dtype: x / sqrt(mean(x^2) + eps) * next_weight, or x itself when next_weight is None.
        With ``y2``, y stands for scale * y + scale2 * y2 (two mixers side by side), formed in the same pass."""
        _dense(x, "x", torch.float32), _dense(y, "y", torch.float32), _dense(post_weight, "post_weight")
        n, hidden = x.shape
        if y.shape != x.shape or post_weight.numel() != hidden:
            raise KernelError("residual_norm_update: sizes of x, y and post_weight do not match")
        if next_weight is not None and (out is None or _dense(next_weight, "next_weight").numel() != hidden):
            raise KernelError("residual_norm_update: next_weight needs out and has the row's length")
        if out is not None and _dense(out, "out").shape != x.shape:
            raise KernelError("residual_norm_update: out has the shape of x")
        if y2 is not None and _dense(y2, "y2", torch.float32).shape != x.shape:
            raise KernelError("residual_norm_update: y2 has the shape of x")
        self.launches += 1
        _check(self._hyb_lib().ifb_residual_norm_update(
            x.data_ptr(), y.data_ptr(), _ptr(y2), float(scale), float(scale2), post_weight.data_ptr(), _code(post_weight), _ptr(next_weight),
            _code(next_weight) if next_weight is not None else 0, float(eps), _ptr(out), _code(out) if out is not None else 0,
            n, hidden, self._stream()), "residual_norm_update")

    def add_rows(self, x, rows=None, vec=None, accumulate=True):
        """x (+)= rows + vec: rows float32 of x's shape, vec one row for all; each may be None."""
        _dense(x, "x", torch.float32)
        n, hidden = x.shape
        if rows is not None and _dense(rows, "rows", torch.float32).shape != x.shape:
            raise KernelError("add_rows: rows has the shape of x")
        if vec is not None and _dense(vec, "vec").numel() != hidden:
            raise KernelError("add_rows: vec has the row's length")
        self.launches += 1
        _check(self._hyb_lib().ifb_add_rows(x.data_ptr(), _ptr(rows), _ptr(vec), _code(vec) if vec is not None else 0,
                                            1 if accumulate else 0, n, hidden, self._stream()), "add_rows")

    def scaled_sum(self, total, d, scale, accumulate=True, copy=None):
        """total (+)= scale * d (float32, same shape); ``copy`` (bfloat16 or float32, same shape) also gets the new total."""
        _dense(total, "total", torch.float32), _dense(d, "d", torch.float32)
        if total.shape != d.shape or (copy is not None and _dense(copy, "copy").shape != total.shape):
            raise KernelError("scaled_sum: total, d and copy differ in shape")
        self.launches += 1
        _check(self._hyb_lib().ifb_scaled_sum(total.data_ptr(), d.data_ptr(), float(scale), 1 if accumulate else 0, d.numel(),
                                              _ptr(copy), _code(copy) if copy is not None else 0, self._stream()), "scaled_sum")

    def token_side_gate(self, z, table, ids, offset, activation, out):
        """out[n, j] = act(z[n, j]) * table[ids[n], offset + j]."""
        _dense(z, "z", torch.float32), _dense(table, "table"), _dense(ids, "ids", torch.int32), _dense(out, "out")
        n, dim = z.shape
        unary = EPILOGUES.get(activation, 0) >> 4
        if not unary:
            raise KernelError(f"token_side_gate: activation {activation!r} is no unary function of the kernels")
        if out.shape != z.shape or ids.numel() != n or table.dim() != 2:
            raise KernelError("token_side_gate: sizes of z, ids and out do not match")
        self.launches += 1
        _check(self._hyb_lib().ifb_token_side_gate(z.data_ptr(), table.data_ptr(), _code(table), table.shape[1], table.shape[0],
                                                   ids.data_ptr(), int(offset), unary, out.data_ptr(), _code(out), n, dim,
                                                   self._stream()), "token_side_gate")

    def softcap(self, logits, cap):
        """logits <- cap * tanh(logits / cap), in place."""
        _dense(logits, "logits", torch.float32)
        self.launches += 1
        _check(self._hyb_lib().ifb_softcap(logits.data_ptr(), float(cap), logits.numel(), self._stream()), "softcap")

    def token_shift_mix(self, h, last, state_slots, cu_q, seq_lens, mu, out):
        """out[s, t] = h[t] + (h'[t] - h[t]) * mu[s]; h' is the row before t in its request, or, for a request's first
        row of the step, last[slot], which then takes the request's last row of the step (csrc/sandwich.cu)."""
        _dense(h, "h"), _dense(last, "last", torch.float32), _dense(mu, "mu", torch.float32), _dense(out, "out", h.dtype)
        _dense(state_slots, "state_slots", torch.int32), _dense(cu_q, "cu_q", torch.int32), _dense(seq_lens, "seq_lens", torch.int32)
        n, hidden = h.shape
        r = seq_lens.numel()
        if mu.dim() != 2 or mu.shape[1] != hidden or out.shape != (mu.shape[0], n, hidden) or last.shape[1:] != (hidden,) \
                or cu_q.numel() != r + 1 or state_slots.numel() < r:
            raise KernelError("token_shift_mix: sizes of h, last, mu, out and the request arrays do not match")
        self.launches += 1
        _check(self._hyb_lib().ifb_token_shift_mix(h.data_ptr(), _code(h), last.data_ptr(), state_slots.data_ptr(), cu_q.data_ptr(),
                                                   seq_lens.data_ptr(), mu.data_ptr(), out.data_ptr(), n, r, hidden, mu.shape[0],
                                                   self._stream()), "token_shift_mix")

    @staticmethod
    def _rows_f32(t, name, n, width):
        """(address, leading dimension) of a float32 matrix [n, width] whose rows are contiguous (a slice of columns)."""
        if t.dtype != torch.float32 or not t.is_cuda or t.dim() != 2 or t.shape != (n, width) or (width > 1 and t.stride(1) != 1):
            raise KernelError(f"{name} must be float32 [{n}, {width}] on the device with contiguous rows")
        return t.data_ptr(), t.stride(0)

    def linear_scan(self, q, k, v, w, heads, dim, vdim, state, state_slots, cu_q, seq_lens, out, eps, decay=None, w_bias=None,
                    key_scale=1.0, bonus=None, norm_weight=None, gate=None, max_q_len=1):
        """The recurrence of a matrix state per head over this step's tokens of every request (csrc/linear_scan.cu).
        q, k, w [n, heads * dim], v, gate [n, heads * vdim]: float32, may be column slices.  ``decay`` float32 [heads]:
        a constant decay per head; else the decay is exp(-exp(w + w_bias)).  ``bonus`` [heads * dim]: the output is read
        before the token's update, the token's own k v^T weighted by the bonus.  out = o / rms(o) per head
        (* norm_weight [heads * vdim]) (* silu(gate)).  From ``scan_block_min`` tokens on the requests are cut into blocks
        of 64 tokens that run side by side (three launches)."""
        n = out.shape[0]
        r = seq_lens.numel()
        hd, hv = heads * dim, heads * vdim
        _dense(state, "state", torch.float32), _dense(out, "out")
        _dense(state_slots, "state_slots", torch.int32), _dense(cu_q, "cu_q", torch.int32), _dense(seq_lens, "seq_lens", torch.int32)
        pq, pk, pv = self._rows_f32(q, "q", n, hd), self._rows_f32(k, "k", n, hd), self._rows_f32(v, "v", n, hv)
        pw = self._rows_f32(w, "w", n, hd) if w is not None else (0, 0)
        pg = self._rows_f32(gate, "gate", n, hv) if gate is not None else (0, 0)
        if (decay is None) == (w is None) or (w is None) != (w_bias is None):
            raise KernelError("linear_scan: give either decay, or w with w_bias")
        if decay is not None and _dense(decay, "decay", torch.float32).numel() != heads:
            raise KernelError("linear_scan: decay has one number per head")
        pdt = None
        for t, size, name in ((w_bias, hd, "w_bias"), (bonus, hd, "bonus"), (norm_weight, hv, "norm_weight")):
            if t is None:
                continue
            _dense(t, name)
            if t.numel() != size or (pdt is not None and t.dtype != pdt):
                raise KernelError(f"linear_scan: {name} has the wrong length or a dtype of its own")
            pdt = t.dtype
        if state.shape[1:] != (heads, dim, vdim) or out.shape != (n, hv) or cu_q.numel() != r + 1 or state_slots.numel() < r:
            raise KernelError("linear_scan: sizes of state, out and the request arrays do not match")
        lib = self._hyb_lib()
        raw = None
        slabs = int(lib.ifb_linear_scan_slabs(dim, vdim))
        need = n * hv if slabs > 1 else 0
        scratch = 0
        blocked = max_q_len >= self.scan_block_min and dim <= 128
        if blocked:
            scratch = int(lib.ifb_linear_scan_scratch_floats(n, r, heads, dim, vdim))
            self.linear_scan_blocked_calls += 1
        if need + scratch:
            if self._ls_scratch is None or self._ls_scratch.numel() < need + scratch:
                self._ls_scratch = torch.empty(need + scratch, dtype=torch.float32, device="cuda")
                self.scratch_generation += 1
            raw = self._ls_scratch[:need] if need else None
        self.launches += (3 if blocked else 1) + (1 if slabs > 1 else 0)
        _check(lib.ifb_linear_scan(
            pq[0], pq[1], pk[0], pk[1], pv[0], pv[1], pw[0], pw[1], pg[0], pg[1], _ptr(decay), _ptr(w_bias), _ptr(bonus),
            _ptr(norm_weight), _CODES[pdt] if pdt is not None else 0, float(key_scale), float(eps), state.data_ptr(),
            state_slots.data_ptr(), cu_q.data_ptr(), seq_lens.data_ptr(), out.data_ptr(), _code(out), _ptr(raw),
            self._ls_scratch[need:].data_ptr() if blocked else 0, r, n, heads, dim, vdim, self._stream()), "linear_scan")

    def gated_unit_scan(self, proj, z_bias, x_bias, state, state_slots, cu_q, seq_lens, out, max_q_len=1):
        """minGRU over this step's tokens of every request: proj [n, 3 width] float32 holds z_raw | x_raw | g
        (csrc/linear_scan.cu); state [slots, width] float32.  From ``scan_block_min`` tokens on the requests are cut into
        chunks of 64 tokens that run side by side (two launches), which differs by rounding only."""
        _dense(proj, "proj", torch.float32), _dense(state, "state", torch.float32), _dense(out, "out")
        _dense(z_bias, "z_bias"), _dense(x_bias, "x_bias", z_bias.dtype)
        _dense(state_slots, "state_slots", torch.int32), _dense(cu_q, "cu_q", torch.int32), _dense(seq_lens, "seq_lens", torch.int32)
        n, width = out.shape
        r = seq_lens.numel()
        if proj.shape != (n, 3 * width) or state.shape[1:] != (width,) or z_bias.numel() != width or x_bias.numel() != width \
                or cu_q.numel() != r + 1 or state_slots.numel() < r:
            raise KernelError("gated_unit_scan: sizes of proj, biases, state, out and the request arrays do not match")
        scratch = 0
        if max_q_len >= self.scan_block_min:
            need = int(self._hyb_lib().ifb_gated_unit_scratch_floats(n, r, width))
            if self._gu_scratch is None or self._gu_scratch.numel() < need:
                self._gu_scratch = torch.empty(need, dtype=torch.float32, device="cuda")
                self.scratch_generation += 1
            scratch = self._gu_scratch.data_ptr()
            self.gated_unit_chunked_calls += 1
        self.launches += 2 if scratch else 1
        _check(self._hyb_lib().ifb_gated_unit_scan(proj.data_ptr(), z_bias.data_ptr(), x_bias.data_ptr(), _code(z_bias),
                                                   state.data_ptr(), state_slots.data_ptr(), cu_q.data_ptr(), seq_lens.data_ptr(),
                                                   out.data_ptr(), _code(out), r, n, width, scratch, self._stream()),
               "gated_unit_scan")

    def rglru_conv(self, proj, x_col, x_bias, conv_weight, conv_bias, state, state_slots, cu_q, seq_lens, req_index, u, u_blocks,
                   offsets, tile_block=None, tile=0):
        """The short causal convolution in front of a real-gated recurrence (csrc/rglru.cu): per channel
        u_t = conv_bias + sum_j conv_weight[:, j] * xin_(t - taps + 1 + j), xin = proj[:, x_col : x_col + width] + x_bias, over
        each request's tokens; the taps - 1 inputs before a portion come from state[slot] ([slots, max(taps - 1, 1), width]
        float32), which then takes the portion's last inputs.  u [n, width] float32; u_blocks [blocks, seg, width / blocks]
        in the products' dtype holds the same numbers block-major for the grouped gate products, whose segments go to
        offsets [blocks + 1] (and tile_block [blocks * seg / tile]); u_blocks [blocks, seg, 2 * width / blocks] gets two
        terms per number: the roundings, then what each rounding left out.  The parameters are float32."""
        _dense(proj, "proj", torch.float32), _dense(u, "u", torch.float32), _dense(u_blocks, "u_blocks"), _dense(state, "state", torch.float32)
        for t, name in ((x_bias, "x_bias"), (conv_weight, "conv_weight"), (conv_bias, "conv_bias")):
            _dense(t, name, torch.float32)
        _dense(offsets, "offsets", torch.int32)
        n, width = u.shape
        blocks, seg, rowlen = u_blocks.shape
        terms = 2 if rowlen * blocks == 2 * width else 1
        bs = rowlen // terms
        taps = conv_weight.shape[1]
        if blocks * bs != width or seg < n or proj.shape[0] != n or conv_weight.shape[0] != width or x_bias.numel() != width \
                or conv_bias.numel() != width or state.shape[1:] != (max(taps - 1, 1), width) or offsets.numel() != blocks + 1:
            raise KernelError("rglru_conv: sizes of proj, parameters, state, u and u_blocks do not match")
        if tile_block is not None and _dense(tile_block, "tile_block", torch.int32).numel() * tile != blocks * seg:
            raise KernelError("rglru_conv: tile_block has an entry for every tile of rows")
        self.launches += 1
        _check(self._hyb_lib().ifb_rglru_conv(
            proj.data_ptr(), proj.shape[1], int(x_col), x_bias.data_ptr(), conv_weight.data_ptr(), conv_bias.data_ptr(),
            state.data_ptr(), state_slots.data_ptr(), cu_q.data_ptr(), seq_lens.data_ptr(), req_index.data_ptr(), u.data_ptr(),
            u_blocks.data_ptr(), _code(u_blocks), seg, blocks, offsets.data_ptr(), _ptr(tile_block), int(tile), n, width, taps,
            terms, self._stream()), "rglru_conv")

    def rglru_scan(self, gates, a_bias, i_bias, decay, decay_scale, u, proj, y_col, y_bias, state, state_slots, cu_q, seq_lens, out,
                   max_q_len=1):
        """The real-gated linear recurrence over this step's tokens of every request (csrc/rglru.cu).  gates
        [blocks, seg, 2 bs] float32: the block-diagonal products' raw r | i; r = sigmoid(. + a_bias), i = sigmoid(. + i_bias),
        log a = -decay_scale * r * softplus(decay), S <- a S + sqrt(1 - a^2) * i * u on state [slots, width] float32;
        out = S * gelu_tanh(proj[:, y_col : y_col + width] + y_bias).  From ``scan_block_min`` tokens on the requests are
        run in three launches (the gates' arithmetic side by side for every token, then chunks of 32 tokens side by side
        twice), which differs by rounding only; that form leaves the decays and input terms in ``gates``."""
        _dense(gates, "gates", torch.float32), _dense(u, "u", torch.float32), _dense(proj, "proj", torch.float32)
        _dense(state, "state", torch.float32), _dense(out, "out")
        for t, name in ((a_bias, "a_bias"), (i_bias, "i_bias"), (decay, "decay"), (y_bias, "y_bias")):
            _dense(t, name, torch.float32)
        n, width = out.shape
        blocks, seg, two_bs = gates.shape
        r = seq_lens.numel()
        if blocks * two_bs != 2 * width or seg < n or u.shape != (n, width) or proj.shape[0] != n or state.shape[1:] != (width,) \
                or any(t.numel() != width for t in (a_bias, i_bias, decay, y_bias)) or cu_q.numel() != r + 1 or state_slots.numel() < r:
            raise KernelError("rglru_scan: sizes of gates, parameters, u, proj, state and out do not match")
        lib = self._hyb_lib()
        scratch = 0
        if max_q_len >= self.scan_block_min:
            need = int(lib.ifb_rglru_scratch_floats(n, r, width))
            if self._rg_scratch is None or self._rg_scratch.numel() < need:
                self._rg_scratch = torch.empty(need, dtype=torch.float32, device="cuda")
                self.scratch_generation += 1
            scratch = self._rg_scratch.data_ptr()
            self.rglru_chunked_calls += 1
        self.launches += 3 if scratch else 1
        _check(lib.ifb_rglru_scan(gates.data_ptr(), seg, blocks, a_bias.data_ptr(), i_bias.data_ptr(), decay.data_ptr(),
                                  float(decay_scale), u.data_ptr(), proj.data_ptr(), proj.shape[1], int(y_col), y_bias.data_ptr(),
                                  state.data_ptr(), state_slots.data_ptr(), cu_q.data_ptr(), seq_lens.data_ptr(), out.data_ptr(),
                                  _code(out), scratch, r, n, width, self._stream()), "rglru_scan")

    @staticmethod
    def _stream_pages(t, name, heads, width, dtype):
        """(address, elements between pages, page size) of a page stream [pages, heads, page_size, width]."""
        if t.dtype != dtype or not t.is_cuda or t.dim() != 4 or t.shape[1] != heads or t.shape[3] != width \
                or t.stride(3) != 1 or t.stride(2) != width or t.stride(1) != t.shape[2] * width:
            raise KernelError(f"{name} is not a page stream [pages, {heads}, page_size, {width}] of {dtype}")
        return t.data_ptr(), t.stride(0), t.shape[2]

    def rotary_store(self, qkv, num_heads, num_kv_heads, head_dim, value_head_dim, qk_table, rotary_dim, interleaved, value_eps,
                     v_table, v_interleaved, q_out, k_pages, v_pages, slot_mapping, values_are_keys=False):
        """Rotation of q and k, norm and rotation of v, q row and page stores in one launch (csrc/attention_streams.cu).
        qkv float32 [n, H d + G d + G dv]; tables float32 (cos, sin) pairs per token; value_eps None: no value norm.
        ``values_are_keys``: qkv is [n, H d + G d] and a value head is its key head before the rotation."""
        _dense(qkv, "qkv", torch.float32), _dense(q_out, "q_out")
        n = qkv.shape[0]
        H, G, d, dv = num_heads, num_kv_heads, head_dim, value_head_dim
        if qkv.shape[1] != H * d + G * (d + (0 if values_are_keys else dv)) or q_out.shape != (n, H * d) or (values_are_keys and dv != d):
            raise KernelError("rotary_store: widths of qkv and q_out do not match the heads")
        if qk_table is not None and _dense(qk_table, "qk_table", torch.float32).shape != (n, rotary_dim):
            raise KernelError("rotary_store: qk_table is [tokens, rotary_dim]")
        if v_table is not None and _dense(v_table, "v_table", torch.float32).shape != (n, dv):
            raise KernelError("rotary_store: v_table is [tokens, value_head_dim]")
        pk, pv, ps = (0, 0, 1), (0, 0, 1), 1
        if slot_mapping is not None:
            _dense(slot_mapping, "slot_mapping", torch.int32)
            pk, pv = self._stream_pages(k_pages, "k_pages", G, d, q_out.dtype), self._stream_pages(v_pages, "v_pages", G, dv, q_out.dtype)
            ps = pk[2]
            if pv[2] != ps or slot_mapping.numel() != n:
                raise KernelError("rotary_store: the streams differ in page size, or slot_mapping in length")
        self.launches += 1
        _check(self._hyb_lib().ifb_rotary_store(
            qkv.data_ptr(), qkv.shape[1], H, G, d, dv, _ptr(qk_table), int(rotary_dim), int(bool(interleaved)),
            0 if value_eps is None else 1, float(value_eps or 0.0), _ptr(v_table), int(bool(v_interleaved)), q_out.data_ptr(),
            _code(q_out), pk[0], pk[1], pv[0], pv[1], _ptr(slot_mapping), ps, n, 1 if values_are_keys else 0, self._stream()),
            "rotary_store")

    def rotate_rows(self, rows, table, heads, width, dims, interleaved, back=False):
        """rows [n, heads * width] in place: every head's first ``dims`` entries turned by the token's angles of
        ``table`` ([n, dims] (cos, sin) pairs), forward or back."""
        _dense(rows, "rows"), _dense(table, "table", torch.float32)
        n = rows.shape[0]
        if rows.shape[1] != heads * width or table.shape != (n, dims):
            raise KernelError("rotate_rows: sizes of rows and table do not match")
        self.launches += 1
        _check(self._hyb_lib().ifb_rotate_rows(rows.data_ptr(), _code(rows), table.data_ptr(), n, heads, width, dims,
                                               int(bool(interleaved)), 1 if back else 0, self._stream()), "rotate_rows")

    def paged_attention_streams(self, q, num_heads, num_kv_heads, head_dim, value_head_dim, k_pages, v_pages, block_tables, cu_q,
                                seq_lens, out, scale, window, out_table, out_interleaved, max_q_len=0, max_seq_len=0):
        """Causal softmax attention of q [n, H d] over key and value page streams (csrc/attention_streams.cu), float32
        scores, weights and sums; each head's output is rotated back by the query token's angles of ``out_table``
        ([n, dv] (cos, sin) pairs; None: not)."""
        _dense(q, "q"), _dense(out, "out", q.dtype), _dense(cu_q, "cu_q", torch.int32), _dense(seq_lens, "seq_lens", torch.int32)
        if block_tables.dtype != torch.int32 or block_tables.stride(1) != 1:
            raise KernelError("paged_attention_streams: block_tables must be int32 with unit stride along pages")
        n, r = q.shape[0], seq_lens.numel()
        H, G, d, dv = num_heads, num_kv_heads, head_dim, value_head_dim
        if q.shape != (n, H * d) or out.shape != (n, H * dv) or cu_q.numel() != r + 1 or block_tables.shape[0] < r:
            raise KernelError("paged_attention_streams: sizes of q, out, cu_q, seq_lens and block_tables do not match")
        pk, pv = self._stream_pages(k_pages, "k_pages", G, d, q.dtype), self._stream_pages(v_pages, "v_pages", G, dv, q.dtype)
        if pk[2] != pv[2]:
            raise KernelError("paged_attention_streams: the streams differ in page size")
        if out_table is not None and _dense(out_table, "out_table", torch.float32).shape != (n, dv):
            raise KernelError("paged_attention_streams: out_table is [tokens, value_head_dim]")
        self.launches += 1
        self.stream_attention_calls += 1
        _check(self._hyb_lib().ifb_paged_attention_streams(
            q.data_ptr(), _code(q), pk[0], pk[1], pv[0], pv[1], block_tables.data_ptr(), block_tables.stride(0), cu_q.data_ptr(),
            seq_lens.data_ptr(), out.data_ptr(), n, r, H, G, d, dv, pk[2], float(scale), int(window), _ptr(out_table),
            int(bool(out_interleaved)), self._stream()), "paged_attention_streams")

    @staticmethod
    def _route_mode(logits, experts, scoring, groups, weight_scale):
        """(experts, stride, mode, group count, groups kept, weight scale) of a router call: ``experts`` None means every
        column of ``logits`` is an expert's."""
        if scoring not in ("chosen", "all", "sigmoid"):
            raise KernelError(f"moe_route: scoring {scoring!r}; known: chosen, all, sigmoid")
        count, keep = groups if groups else (1, 1)
        if groups and scoring != "all":
            raise KernelError("moe_route: groups of experts limit the choice only with scoring 'all'")
        return (int(experts) if experts is not None else logits.shape[1], logits.shape[1], {"chosen": 0, "all": 1, "sigmoid": 2}[scoring],
                int(count), int(keep), float(weight_scale))

    def moe_route(self, logits, top, ids, gates, experts=None, scoring="chosen", groups=None, weight_scale=1.0):
        """ids[n] = the indices of row n's ``top`` largest scores, largest first (the lower index among equals).  scoring
        "chosen": the scores are the logits and gates[n] = the softmax over the chosen logits.  scoring "all": the scores are
        the softmax over all experts, gates[n] = score * weight_scale, and with ``groups`` = (count, keep) only experts of the
        ``keep`` groups of neighbours with the largest best score can be chosen.  scoring "sigmoid": the scores are sigmoid(logit)
        per expert and gates[n] = score * weight_scale.  ``experts``: the first that many columns of
        ``logits`` are the router's (the rest belong to someone else).  (csrc/moe.cu)"""
        _dense(logits, "logits", torch.float32), _dense(ids, "ids", torch.int32), _dense(gates, "gates", torch.float32)
        n = logits.shape[0]
        experts, stride, mode, count, keep, ws = self._route_mode(logits, experts, scoring, groups, weight_scale)
        if ids.shape != (n, top) or gates.shape != (n, top):
            raise KernelError("moe_route: ids and gates are [rows, top]")
        self.launches += 1
        _check(self._hyb_lib().ifb_moe_route(logits.data_ptr(), ids.data_ptr(), gates.data_ptr(), n, experts, int(top), stride, mode,
                                             count, keep, ws, self._stream()), "moe_route")

    MOE_SMALL_PAIRS = 512      # up to here the router and the pair list are one launch of one block

    def moe_route_plan(self, logits, top, ids, gates, offsets, perm, pos, experts=None, scoring="chosen", groups=None,
                       weight_scale=1.0):
        """:meth:`moe_route` and :meth:`moe_plan` of a step; one launch where the step has few pairs (decode)."""
        n = logits.shape[0]
        experts, stride, mode, count, keep, ws = self._route_mode(logits, experts, scoring, groups, weight_scale)
        if n * top > self.MOE_SMALL_PAIRS or experts > 256:
            self.moe_route(logits, top, ids, gates, experts=experts, scoring=scoring, groups=groups, weight_scale=weight_scale)
            return self.moe_plan(ids, experts, offsets, perm, pos)
        _dense(logits, "logits", torch.float32), _dense(ids, "ids", torch.int32), _dense(gates, "gates", torch.float32)
        _dense(offsets, "offsets", torch.int32), _dense(perm, "perm", torch.int32), _dense(pos, "pos", torch.int32)
        if ids.shape != (n, top) or gates.shape != (n, top) or offsets.numel() != experts + 1 or perm.numel() != n * top \
                or pos.numel() != n * top:
            raise KernelError("moe_route_plan: sizes of ids, gates, offsets, perm and pos do not match")
        self.launches += 1
        _check(self._hyb_lib().ifb_moe_route_plan_small(logits.data_ptr(), ids.data_ptr(), gates.data_ptr(), n, experts, int(top),
                                                        offsets.data_ptr(), perm.data_ptr(), pos.data_ptr(), stride, mode, count,
                                                        keep, ws, self._stream()),
               "moe_route_plan")

    def moe_plan(self, ids, num_experts, offsets, perm, pos):
        """The (row, choice) pairs listed by expert in ascending pair number: offsets [experts + 1], perm [pairs]
        (place -> pair), pos [pairs] (pair -> place), all int32."""
        _dense(ids, "ids", torch.int32), _dense(offsets, "offsets", torch.int32), _dense(perm, "perm", torch.int32)
        _dense(pos, "pos", torch.int32)
        pairs = ids.numel()
        if offsets.numel() != num_experts + 1 or perm.numel() != pairs or pos.numel() != pairs:
            raise KernelError("moe_plan: sizes of offsets, perm and pos do not match")
        self.launches += 1
        _check(self._hyb_lib().ifb_moe_plan(ids.data_ptr(), pairs, int(num_experts), offsets.data_ptr(), perm.data_ptr(),
                                            pos.data_ptr(), self._stream()), "moe_plan")

    def moe_linear(self, x, w, offsets, perm, top, out, epilogue="none"):
        """Row i of ``out`` belongs to the expert e with offsets[e] <= i < offsets[e + 1] and is x[perm[i] // top] @ w[e]^T
        (perm None: x[i]); w [experts, o, k]; epilogue "silu_gate": w[e] holds gate rows, then up rows.  bfloat16 x and w
        with k a multiple of 8 run on tensor cores (mma.sync), everything else in plain float32 arithmetic."""
        _dense(x, "x"), _dense(w, "w"), _dense(offsets, "offsets", torch.int32), _dense(out, "out")
        gated = epilogue == "silu_gate"
        if epilogue not in ("none", "silu_gate"):
            raise KernelError(f"moe_linear: epilogue {epilogue!r}; known: none, silu_gate")
        rows, o = out.shape
        experts, ow, k = w.shape
        if x.shape[1] != k or ow != (2 * o if gated else o) or offsets.numel() != experts + 1:
            raise KernelError("moe_linear: sizes of x, w, offsets and out do not match")
        if perm is not None:
            if _dense(perm, "perm", torch.int32).numel() != rows or rows != x.shape[0] * top:
                raise KernelError("moe_linear: perm has a place for every (row, choice) pair")
        elif x.shape[0] != rows:
            raise KernelError("moe_linear: without perm, x has a row for each row of out")
        self.launches += 1
        _check(self._hyb_lib().ifb_moe_linear(x.data_ptr(), _code(x), w.data_ptr(), _code(w), offsets.data_ptr(), _ptr(perm),
                                              int(top), out.data_ptr(), _code(out), rows, experts, o, k, 1 if gated else 0,
                                              1 if self.moe_tensor_cores else 0, self._stream()), "moe_linear")

    # The experts' products of a prompt on the tcgen05 kernel: every expert's rows contiguous in segments padded to the
    # kernel's tile of 128 rows (TMA reads whole tiles; a tile has one expert).
    MOE_TILE = 128

    def moe_grouped_tc_ok(self, pairs, dtype, *weights):
        """Whether a step of ``pairs`` (token, choice) pairs runs its experts' products on the tcgen05 kernel: bfloat16,
        more pairs than the few-rows form takes, every k a multiple of 8."""
        return (self.moe_tcgen05 and dtype == torch.bfloat16 and pairs > 256
                and all(w.dtype == torch.bfloat16 and w.shape[2] % 8 == 0 and w.shape[1] % 8 == 0 for w in weights))

    def moe_padded_rows(self, pairs, num_experts):
        """Places of the padded pair list: the most that ``pairs`` pairs over the experts can need, a multiple of the tile."""
        t = self.MOE_TILE
        return -(-(pairs + num_experts * (t - 1)) // t) * t

    def moe_plan_padded(self, ids, num_experts, offsets, perm, pos, tile_expert):
        """As :meth:`moe_plan` with every expert's segment padded to the tile: perm [moe_padded_rows] (-1 in the padding),
        pos [pairs] (pair -> padded place), tile_expert [places / tile] (-1: unused tile)."""
        _dense(ids, "ids", torch.int32), _dense(offsets, "offsets", torch.int32), _dense(perm, "perm", torch.int32)
        _dense(pos, "pos", torch.int32), _dense(tile_expert, "tile_expert", torch.int32)
        pairs = ids.numel()
        if offsets.numel() != num_experts + 1 or pos.numel() != pairs or perm.numel() != tile_expert.numel() * self.MOE_TILE \
                or perm.numel() < pairs + num_experts * (self.MOE_TILE - 1):
            raise KernelError("moe_plan_padded: sizes of offsets, perm, pos and tile_expert do not match")
        self.launches += 1
        _check(self._hyb_lib().ifb_moe_plan_padded(ids.data_ptr(), pairs, int(num_experts), self.MOE_TILE, offsets.data_ptr(),
                                                   perm.data_ptr(), pos.data_ptr(), tile_expert.data_ptr(), tile_expert.numel(),
                                                   self._stream()), "moe_plan_padded")

    def moe_gather(self, x, perm, top, tile_expert, out):
        """out[place] = x[perm[place] // top], zeros in the padding; the rows of unused tiles are left alone."""
        _dense(x, "x", torch.bfloat16), _dense(perm, "perm", torch.int32), _dense(tile_expert, "tile_expert", torch.int32)
        _dense(out, "out", torch.bfloat16)
        if out.shape != (perm.numel(), x.shape[1]) or perm.numel() != tile_expert.numel() * self.MOE_TILE:
            raise KernelError("moe_gather: out has a row for every place of perm")
        self.launches += 1
        _check(self._hyb_lib().ifb_moe_gather_rows(x.data_ptr(), perm.data_ptr(), int(top), tile_expert.data_ptr(), self.MOE_TILE,
                                                   out.data_ptr(), perm.numel(), x.shape[1], self._stream()), "moe_gather")

    def moe_gather_scaled(self, x, perm, top, gates, out, tile_expert=None):
        """out[place] = gates[perm[place]] * x[perm[place] // top] in out's dtype, zeros where perm[place] < 0: what the experts
        read when their weight multiplies their input.  ``gates`` float32 [rows, top] (pair = row * top + choice);
        ``tile_expert``: the padded list's tiles, whose unused ones are left alone."""
        _dense(x, "x"), _dense(perm, "perm", torch.int32), _dense(gates, "gates", torch.float32), _dense(out, "out", x.dtype)
        if out.shape != (perm.numel(), x.shape[1]) or gates.numel() != x.shape[0] * top:
            raise KernelError("moe_gather_scaled: out has a row for every place of perm, gates a number for every pair")
        if tile_expert is not None and _dense(tile_expert, "tile_expert", torch.int32).numel() * self.MOE_TILE != perm.numel():
            raise KernelError("moe_gather_scaled: tile_expert has an entry for every tile of places")
        self.launches += 1
        _check(self._hyb_lib().ifb_moe_gather_scaled(x.data_ptr(), _code(x), perm.data_ptr(), int(top), gates.data_ptr(),
                                                     _ptr(tile_expert), self.MOE_TILE, out.data_ptr(), perm.numel(), x.shape[1],
                                                     self._stream()), "moe_gather_scaled")

    def moe_linear_grouped(self, x, w, tile_expert, out, epilogue="none"):
        """out[place] = x[place] @ w[tile_expert[place // tile]]^T on the tcgen05 kernel (csrc/linear_tcgen05.cu, its grouped
        mode); x [places, k] sorted by expert in padded segments, w [experts, o (2 o with "silu_gate"), k]."""
        _dense(x, "x", torch.bfloat16), _dense(w, "w", torch.bfloat16), _dense(tile_expert, "tile_expert", torch.int32), _dense(out, "out")
        gated = epilogue == "silu_gate"
        if epilogue not in ("none", "silu_gate"):
            raise KernelError(f"moe_linear_grouped: epilogue {epilogue!r}; known: none, silu_gate")
        rows, o = out.shape
        experts, ow, k = w.shape
        if x.shape != (rows, k) or ow != (2 * o if gated else o) or rows != tile_expert.numel() * self.MOE_TILE:
            raise KernelError("moe_linear_grouped: sizes of x, w, tile_expert and out do not match")
        lib = self._tc_lib()
        if not getattr(lib, "_grouped_declared", False):
            lib.ifb_linear_tcgen05_grouped.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                                       c_void_p, c_void_p, c_void_p]
            lib._grouped_declared = True
        self.launches += 1
        self.moe_tcgen05_calls += 1
        self._err_armed = True
        _check(lib.ifb_linear_tcgen05_grouped(x.data_ptr(), w.data_ptr(), out.data_ptr(), _code(out), rows, experts, o, k,
                                              1 if gated else 0, tile_expert.data_ptr(), self._dev_err.data_ptr(), self._stream()),
               "moe_linear_grouped")

    def moe_combine(self, y, pos, gates, out, shared=None, shared_logit=None):
        """out[n] = sum_j gates[n, j] * y[pos[n * top + j]], j ascending, float32 (y may hold more rows than pairs: a
        padded list).  ``shared`` [n, width] float32: + shared[n], times sigmoid(shared_logit[n]) when ``shared_logit`` (a
        column of a float32 matrix) is given."""
        _dense(y, "y", torch.float32), _dense(pos, "pos", torch.int32), _dense(out, "out", torch.float32)
        n = out.shape[0]
        if gates is None:                      # every weight is 1 (the weights went into what the experts read)
            top = pos.numel() // max(n, 1)
        else:
            top = _dense(gates, "gates", torch.float32).shape[1]
            if gates.shape[0] != n:
                raise KernelError("moe_combine: gates has a row for every row of out")
        if pos.numel() != n * top or y.shape[0] < n * top or y.shape[1] != out.shape[1] or out.shape[0] != n:
            raise KernelError("moe_combine: sizes of y, pos, gates and out do not match")
        stride = 0
        if shared is not None:
            if _dense(shared, "shared", torch.float32).shape != out.shape:
                raise KernelError("moe_combine: shared has the shape of out")
            if shared_logit is not None:
                if shared_logit.dtype != torch.float32 or shared_logit.dim() != 1 or shared_logit.shape[0] != n:
                    raise KernelError("moe_combine: shared_logit is one float32 number per row")
                stride = shared_logit.stride(0)
        self.launches += 1
        _check(self._hyb_lib().ifb_moe_combine(y.data_ptr(), pos.data_ptr(), _ptr(gates), out.data_ptr(), n, top,
                                               out.shape[1], _ptr(shared), _ptr(shared_logit) if shared is not None else None,
                                               stride, self._stream()), "moe_combine")

    # ------------------------------------------------------------------ decoders with latent attention (csrc/latent.cu)
    def _lat_lib(self):
        if self._lat is None:
            m = self._lat = load_library("latent", progress=self._progress)
            m.ifb_group_rmsnorm.argtypes = [c_void_p, c_void_p, c_float, c_void_p, c_int, c_int, c_float, c_void_p, c_int, c_void_p,
                                            c_void_p, c_longlong, c_int, c_int, c_void_p]
            m.ifb_depth_average.argtypes = [c_void_p, c_void_p, c_float, c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_int,
                                            c_int, c_float, c_void_p, c_int, c_int, c_int, c_void_p]
            m.ifb_causal_conv.argtypes = [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                          c_void_p, c_int, c_int, c_int, c_void_p]
            m.ifb_latent_prepare.argtypes = [c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_float,
                                             c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                             c_void_p, c_void_p, c_int, c_int, c_void_p, c_longlong, c_int, c_void_p]
            m.ifb_gate_heads.argtypes = [c_void_p, c_int, c_void_p, c_longlong, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p]
            m.ifb_latent_attention.argtypes = [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p,
                                               c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                               c_float, c_int, c_void_p]
            m.ifb_latent_attention_mma.argtypes = [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p,
                                                   c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                                   c_float, c_int, c_int, c_int, c_void_p]
            m.ifb_latent_attention_mma_scratch_floats.restype = c_longlong
            m.ifb_latent_attention_mma_scratch_floats.argtypes = [c_int, c_int, c_int, c_int, c_int]
        return self._lat

    def group_rmsnorm(self, x, weight, groups, eps, out, delta=None, mult=1.0, rows=None, keep=None):
        """The RMS norm in ``groups`` equal parts of the row, each with its own statistic, times ``weight``.  With ``delta``
        the rows of x (float32) first become x + mult * delta (written back unless ``rows`` picks the rows that are normed).
        ``keep`` [n, width] (a float32 view whose rows may be strided) also gets the updated rows."""
        _dense(x, "x", torch.float32), _dense(weight, "weight"), _dense(out, "out")
        n, width = x.shape
        m = n if rows is None else _dense(rows, "rows", torch.int32).numel()
        if out.shape != (m, width) or weight.numel() != width:
            raise KernelError("group_rmsnorm: sizes of x, weight and out do not match")
        if delta is not None and _dense(delta, "delta", torch.float32).shape != x.shape:
            raise KernelError("group_rmsnorm: delta has the shape of x")
        stride = 0
        if keep is not None:
            if keep.dtype != torch.float32 or keep.shape != x.shape or keep.stride(1) != 1 or rows is not None:
                raise KernelError("group_rmsnorm: keep is a float32 view of x's shape with unit stride along the row")
            stride = keep.stride(0)
        self.launches += 1
        _check(self._lat_lib().ifb_group_rmsnorm(x.data_ptr(), _ptr(delta), float(mult), weight.data_ptr(), _code(weight), int(groups),
                                                 float(eps), out.data_ptr(), _code(out), _ptr(rows), _ptr(keep), stride, m, width,
                                                 self._stream()), "group_rmsnorm")

    def depth_average(self, x, delta, mult, hist, depth, coeff, out=None, next_weight=None, groups=1, eps=0.0):
        """hist [n, slots, width] float32 holds X_0 .. X_(depth-1) of every token.  X_depth = x + mult * delta is stored
        there and x becomes sum_j coeff[j] * X_j, j = 0 .. depth; ``out`` gets the norm in groups of the new x with
        ``next_weight``."""
        _dense(x, "x", torch.float32), _dense(hist, "hist", torch.float32), _dense(coeff, "coeff")
        n, width = x.shape
        if hist.dim() != 3 or hist.shape[0] != n or hist.shape[2] != width or not 0 <= depth < hist.shape[1] or coeff.numel() != depth + 1:
            raise KernelError("depth_average: sizes of x, hist and coeff do not match")
        if delta is not None and _dense(delta, "delta", torch.float32).shape != x.shape:
            raise KernelError("depth_average: delta has the shape of x")
        if (out is None) != (next_weight is None) or (out is not None and (_dense(out, "out").shape != x.shape
                                                                            or _dense(next_weight, "next_weight").numel() != width)):
            raise KernelError("depth_average: out and next_weight come together and have x's shape and row length")
        self.launches += 1
        _check(self._lat_lib().ifb_depth_average(x.data_ptr(), _ptr(delta), float(mult), hist.data_ptr(), hist.shape[1], int(depth),
                                                 coeff.data_ptr(), _code(coeff), _ptr(next_weight),
                                                 _code(next_weight) if next_weight is not None else 0, int(groups), float(eps),
                                                 _ptr(out), _code(out) if out is not None else 0, n, width, self._stream()),
               "depth_average")

    def causal_conv(self, h, weight, state, state_slots, cu_q, seq_lens, req_index, out):
        """out_t = h_t + sum_j weight[:, j] * h_(t - taps + 1 + j) over each request's tokens; the taps - 1 inputs before a
        portion come from state[slot] ([slots, taps - 1, width] float32), which then takes the portion's last inputs."""
        _dense(h, "h"), _dense(weight, "weight"), _dense(state, "state", torch.float32), _dense(out, "out", h.dtype)
        n, width = h.shape
        taps = weight.shape[1]
        if weight.shape[0] != width or out.shape != h.shape or state.shape[1:] != (max(taps - 1, 1), width):
            raise KernelError("causal_conv: sizes of h, weight, state and out do not match")
        self.launches += 1
        _check(self._lat_lib().ifb_causal_conv(h.data_ptr(), _code(h), weight.data_ptr(), _code(weight), state.data_ptr(),
                                               state_slots.data_ptr(), cu_q.data_ptr(), seq_lens.data_ptr(), req_index.data_ptr(),
                                               out.data_ptr(), n, width, taps, self._stream()), "causal_conv")

    def latent_prepare(self, proj, heads, dim, rot, rank, down_col, norm_weight, eps, table, dims, q_plain, q_rot, latent_pages,
                       rot_pages, slot_mapping, offsets, tile_head=None, tile=0, q=None, interleaved=False):
        """From a step's product q | latent, rotated key | ... (proj, float32): the normalised latent and the turned rotated
        key part into their page streams ([pages, 1, page_size, width]) at slot_mapping (None: nothing is stored), the
        heads' unrotated query parts head-major into q_plain [heads, seg, dim], their turned rotated parts into q_rot
        [n, heads, rot] (float32).  offsets [heads + 1] gets the segments h * seg of the grouped products that follow,
        tile_head [heads * seg / tile] the head of every tile of rows.  table [n, dims]: (cos, sin) pairs (None: no turn);
        ``interleaved``: a rotation pairs entry 2m with 2m + 1 instead of m with m + dims/2.  ``q`` [n, heads * (dim + rot)]
        float32: the queries come from there (a product of their own) and ``proj`` need not hold them."""
        _dense(proj, "proj", torch.float32), _dense(q_plain, "q_plain"), _dense(latent_pages, "latent_pages", q_plain.dtype)
        _dense(offsets, "offsets", torch.int32), _dense(norm_weight, "norm_weight")
        n, stride = proj.shape
        seg = q_plain.shape[1]
        if q is not None and _dense(q, "q", torch.float32).shape != (n, heads * (dim + rot)):
            raise KernelError("latent_prepare: q is float32 [n, heads * (dim + rot)]")
        if q_plain.shape != (heads, seg, dim) or seg < n or offsets.numel() != heads + 1 or norm_weight.numel() != rank \
                or latent_pages.shape[1] != 1 or latent_pages.shape[3] != rank or (q is None and heads * (dim + rot) > down_col) \
                or down_col + rank + rot > stride:
            raise KernelError("latent_prepare: sizes of proj, q_plain, latent_pages and offsets do not match")
        if rot:
            if _dense(q_rot, "q_rot", torch.float32).shape != (n, heads, rot) or _dense(rot_pages, "rot_pages", q_plain.dtype).shape[3] != rot \
                    or rot_pages.shape[:3] != latent_pages.shape[:3]:
                raise KernelError("latent_prepare: q_rot is [n, heads, rot] and rot_pages has rot entries per slot")
        if table is not None and (_dense(table, "table", torch.float32).shape != (n, dims) or dims > rot or dims % 2):
            raise KernelError("latent_prepare: table is [n, dims] with dims even and at most rot")
        if tile_head is not None and (_dense(tile_head, "tile_head", torch.int32).numel() * tile != heads * seg):
            raise KernelError("latent_prepare: tile_head has an entry for every tile of rows")
        self.launches += 1
        _check(self._lat_lib().ifb_latent_prepare(proj.data_ptr(), stride, heads, dim, rot, rank, down_col, norm_weight.data_ptr(),
                                                  _code(norm_weight), float(eps), _ptr(table), int(dims) if table is not None else 0,
                                                  q_plain.data_ptr(), _code(q_plain), seg, _ptr(q_rot) if rot else None,
                                                  latent_pages.data_ptr(), _ptr(rot_pages) if rot else None, _code(latent_pages),
                                                  _ptr(slot_mapping), offsets.data_ptr(), _ptr(tile_head), int(tile), n,
                                                  _ptr(q), q.shape[1] if q is not None else 0, 1 if interleaved else 0,
                                                  self._stream()), "latent_prepare")

    def latent_attention(self, q_lat, q_rot, latent_pages, rot_pages, block_tables, cu_q, seq_lens, req_index, sink, out, scale,
                         window, tokens, max_q_len=None, max_seq_len=None, exact=False, weight_terms=1):
        """Attention of every head over the request's cached latents (the absorbed form): q_lat [heads, seg, rank] float32,
        q_rot [n, heads, rot] float32 (None without a rotated part), out [heads, seg, rank] = the softmax-weighted sum of
        latents per head.  ``sink`` [heads]: exp of it joins the denominator.  ``window`` 0: every earlier position.

        bfloat16 pages with a latent of at most 256 entries (latent and rotated part multiples of 8), when the caller gives
        the step's longest portion and context: the tensor-core kernel (csrc/attention_latent_mma.cu; float32 scores,
        softmax and sums, the weights rounded to bfloat16 as the left operand of the weighted sum), the context divided
        among several CTAs where a step has few rows; ``weight_terms`` 2: a weight enters the sum as two bfloat16 terms, its
        rounding and what the rounding left out).  float32, other sizes and ``exact``: the plain kernel, a warp per
        (token, head), which keeps float32 weights through the sum."""
        _dense(q_lat, "q_lat", torch.float32), _dense(latent_pages, "latent_pages"), _dense(out, "out", latent_pages.dtype)
        heads, seg, rank = q_lat.shape
        rot = rot_pages.shape[3] if rot_pages is not None else 0
        if out.shape != q_lat.shape or latent_pages.shape[1] != 1 or latent_pages.shape[3] != rank or seg < tokens:
            raise KernelError("latent_attention: sizes of q_lat, latent_pages and out do not match")
        if rot and (_dense(q_rot, "q_rot", torch.float32).shape != (tokens, heads, rot) or _dense(rot_pages, "rot_pages", latent_pages.dtype).shape[:3] != latent_pages.shape[:3]):
            raise KernelError("latent_attention: q_rot is [n, heads, rot] and rot_pages lies beside latent_pages")
        if sink is not None and _dense(sink, "sink").numel() != heads:
            raise KernelError("latent_attention: sink has one number per head")
        if (not exact and max_q_len is not None and max_seq_len is not None and latent_pages.dtype == torch.bfloat16 and rank % 8 == 0
                and rank <= 256 and rot % 8 == 0):
            lib = self._lat_lib()
            requests = cu_q.numel() - 1
            ctas = requests * -(-int(max_q_len) * heads // 64)
            reach = min(int(max_seq_len), int(window) + int(max_q_len)) if window else int(max_seq_len)
            splits = max(1, min((2 * self.sm_count) // ctas, -(-reach // max(64, self.split_min_keys // 2)), 32))
            need = lib.ifb_latent_attention_mma_scratch_floats(requests, int(max_q_len), heads, rank, splits)
            if need * 4 > self.attention_scratch_cap:
                splits, need = 1, 0
            scratch = self.attention_scratch(need) if need else None
            self.launches += 1 + (1 if splits > 1 else 0)
            self.latent_mma_calls += 1
            _check(lib.ifb_latent_attention_mma(q_lat.data_ptr(), _ptr(q_rot) if rot else None, seg, latent_pages.data_ptr(),
                                                _ptr(rot_pages) if rot else None, block_tables.data_ptr(), block_tables.stride(0),
                                                latent_pages.shape[2], cu_q.data_ptr(), seq_lens.data_ptr(), _ptr(sink),
                                                _code(sink) if sink is not None else 0, out.data_ptr(), _ptr(scratch), requests,
                                                int(max_q_len), heads, rank, rot, float(scale), int(window or 0), splits,
                                                int(weight_terms), self._stream()), "latent_attention")
            return
        self.launches += 1
        _check(self._lat_lib().ifb_latent_attention(q_lat.data_ptr(), _ptr(q_rot) if rot else None, seg, latent_pages.data_ptr(),
                                                    _ptr(rot_pages) if rot else None, _code(latent_pages), block_tables.data_ptr(),
                                                    block_tables.stride(0), latent_pages.shape[2], cu_q.data_ptr(), seq_lens.data_ptr(),
                                                    req_index.data_ptr(), _ptr(sink), _code(sink) if sink is not None else 0,
                                                    out.data_ptr(), _code(out), int(tokens), heads, rank, rot, float(scale),
                                                    int(window or 0), self._stream()), "latent_attention")

    def gate_heads(self, y, gate, out, tokens, per_head=False):
        """out[t, h * vdim + v] = y[h, t, v] * sigmoid(gate[t, h * vdim + v]) (gate None: no gate); y [heads, seg, vdim]
        float32, gate a float32 view [n, heads * vdim] whose rows may be strided.  ``per_head``: gate is [n, heads] and a
        head takes one number."""
        _dense(y, "y", torch.float32), _dense(out, "out")
        heads, seg, vdim = y.shape
        if out.shape != (tokens, heads * vdim) or seg < tokens:
            raise KernelError("gate_heads: out is [tokens, heads * vdim]")
        stride = 0
        if gate is not None:
            if gate.dtype != torch.float32 or gate.shape != ((tokens, heads) if per_head else out.shape) or gate.stride(1) != 1:
                raise KernelError("gate_heads: gate is a float32 view of out's shape with unit stride along the row")
            stride = gate.stride(0)
        self.launches += 1
        _check(self._lat_lib().ifb_gate_heads(y.data_ptr(), seg, _ptr(gate), stride, out.data_ptr(), _code(out), int(tokens), heads,
                                              vdim, 1 if per_head else 0, self._stream()), "gate_heads")

    # ------------------------------------------------------------------ sampling
    def sample(self, logits, temperature, uniform, out):
        _dense(logits, "logits", torch.float32), _dense(out, "out", torch.int32)
        m, vocab = logits.shape
        if temperature is not None:
            _dense(temperature, "temperature", torch.float32), _dense(uniform, "uniform", torch.float32)
            if temperature.numel() != m or uniform.numel() != m:
                raise KernelError("sample: one temperature and one uniform number per row")
        if out.numel() != m:
            raise KernelError("sample: out has one entry per row")
        self.launches += 1
        if temperature is None and vocab >= 16384 and m <= 4096:
            # greedy over a large vocabulary: several blocks per row, enough to fill the device about twice
            bpr = max(1, min(64, (2 * self.sm_count) // m, vocab // 2048))
            if bpr > 1:
                if self._argmax_scratch is None:
                    self._argmax_scratch = (torch.empty(4096 * 64, dtype=torch.float32, device="cuda"),
                                            torch.empty(4096 * 64, dtype=torch.int32, device="cuda"),
                                            torch.zeros(4096, dtype=torch.int32, device="cuda"))
                    self.scratch_generation += 1
                vals, idxs, counters = self._argmax_scratch
                return _check(self.core.ifb_argmax_rows(logits.data_ptr(), m, vocab, bpr, vals.data_ptr(), idxs.data_ptr(),
                                                        counters.data_ptr(), out.data_ptr(), self._stream()), "sample")
        _check(self.core.ifb_sample(logits.data_ptr(), m, vocab, _ptr(temperature), _ptr(uniform), out.data_ptr(),
                                    self._stream()), "sample")
