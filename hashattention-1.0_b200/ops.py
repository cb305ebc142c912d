"""Python entry points of the CUDA library: thin, validating wrappers that pass raw device
pointers and the current stream through the C ABI (include/hashattn.h).

Shape / dtype / device problems raise ``ValueError`` before anything is launched, the way the
reference raises on mismatching attention shapes (hashattention/hashattention_llama.py:587-620).
A non-zero library status raises ``RuntimeError``. There is no torch or CPU fallback.
"""
from __future__ import annotations

import ctypes
import math
from dataclasses import dataclass

import torch

from . import _lib
from .cache import GROUP, HEAD_DIM, PAGE, PagedHashKVCache
from .usa import PackedHashWeights


@dataclass(frozen=True)
class Budget:
    """init / heavy / recent budgets with the reference's meaning: ``heavy_budget <= 1.0`` is a
    fraction of the sequence length, ``> 1.0`` an absolute count
    (hashattention/hashattention_llama.py:431-434). ``eval_mode`` / ``retrieve_depth`` are the
    reference's ``usa_eval_mode`` / ``usa_retrieve_depth``: 'simple' keeps the ``hb`` best
    candidates, any other mode every candidate whose score is within ``retrieve_depth`` bits of the
    best one or at least that of the ``hb``-th best (:436-443)."""

    init_budget: int = 128
    heavy_budget: float = 1.0 / 32
    recent_budget: int = 128
    eval_mode: str = "simple"
    retrieve_depth: int = -1

    def heavy_tokens(self, seq_len: int) -> int:
        return int(self.heavy_budget) if self.heavy_budget > 1.0 else int(seq_len * self.heavy_budget)

    def c_struct(self) -> _lib.HaBudget:
        simple = self.eval_mode == "simple"
        return _lib.HaBudget(int(self.init_budget), int(self.recent_budget), float(self.heavy_budget),
                             _lib.HA_EVAL_SIMPLE if simple else _lib.HA_EVAL_DEPTH,
                             0 if simple else int(self.retrieve_depth))

    def max_selected(self, max_seq_len: int) -> int:
        """Upper bound on the heavy tokens of one head: the budget in 'simple' mode, every token otherwise
        (the depth rule keeps all ties, so its sets have no fixed size)."""
        if self.eval_mode == "simple":
            return max(1, min(self.heavy_tokens(max_seq_len), max_seq_len))
        return max(1, max_seq_len)


def _check(t: torch.Tensor, name: str, dtype: torch.dtype, shape, device) -> None:
    if not isinstance(t, torch.Tensor):
        raise ValueError(f"{name} must be a tensor")
    if t.dtype != dtype:
        raise ValueError(f"{name} must be {dtype}, got {t.dtype}")
    if tuple(t.shape) != tuple(shape):
        raise ValueError(f"{name} should be of size {tuple(shape)}, but is {tuple(t.shape)}")
    if t.device != device:
        raise ValueError(f"{name} must live on {device}, got {t.device}")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")


def _raise_on(rc: int, what: str) -> None:
    if rc != _lib.HA_OK:
        raise RuntimeError(f"{what} failed: {_lib.status_str(rc)} (status {rc})")


def _stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


_nvtx_on = False


def set_nvtx(on: bool) -> None:
    """Profiling aid: wrap every library call of this module in an NVTX range named after the entry point
    (``hashattn/ha_decode_step`` ...), so that a timeline shows the step as one block. Off by default."""
    global _nvtx_on
    _nvtx_on = bool(on)


class _call_range:
    """``with _call_range("ha_decode_step"):`` - an NVTX range when switched on, nothing otherwise."""

    def __init__(self, name: str):
        self.name = name
        self.pushed = False

    def __enter__(self):
        if _nvtx_on:
            torch.cuda.nvtx.range_push("hashattn/" + self.name)
            self.pushed = True
        return self

    def __exit__(self, *exc):
        if self.pushed:
            torch.cuda.nvtx.range_pop()
        return False


class SparseDecodeContext:
    """Everything one layer's decode step needs besides q / k_new / v_new: the paged cache, the
    budgets, the packed hash weights, the workspace and the intermediate buffers (query codes,
    selected indices). Creating it allocates; the step functions do not."""

    def __init__(self, cache: PagedHashKVCache, budget: Budget, weights: PackedHashWeights,
                 max_seq_len: int | None = None, sm_scale: float | None = None):
        if cache.device.type != "cuda":
            raise ValueError("the cache must live on a CUDA device")
        self.lib = _lib.load()
        self.cache = cache
        self.budget = budget
        self.weights = weights
        self.device = cache.device
        self.batch = cache.batch
        self.num_kv_heads = cache.num_kv_heads
        self.num_q_heads = cache.num_kv_heads * GROUP
        if weights.wq.shape[0] != self.num_q_heads or weights.wq.device != self.device:
            raise ValueError("packed hash weights do not match the cache's heads / device")
        max_seq_len = cache.max_pages * PAGE if max_seq_len is None else max_seq_len
        self.sel_stride = budget.max_selected(max_seq_len)
        self.sm_scale = 1.0 / math.sqrt(HEAD_DIM) if sm_scale is None else float(sm_scale)
        self.shape = _lib.HaShape(self.batch, self.num_kv_heads, GROUP, HEAD_DIM, PAGE, cache.max_pages,
                                  cache.num_pages, self.sel_stride)
        self.c_budget = budget.c_struct()
        # the LSH baseline keeps, per cache, the largest key norm of every kv-head and a "codes are stale" flag
        self.lsh_state = torch.zeros(2 * self.num_kv_heads, dtype=torch.int32, device=self.device) if weights.lsh else None
        self.c_weights = weights.c_struct(self.lsh_state)
        self.workspace_bytes = int(self.lib.ha_workspace_bytes(self.shape, self.c_budget))
        if self.workspace_bytes == 0:
            raise ValueError("invalid shape or budget for the CUDA library")
        dev = self.device
        self.workspace = torch.empty(self.workspace_bytes, dtype=torch.uint8, device=dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        self.q_codes = torch.zeros(self.batch, self.num_q_heads, dtype=torch.int32, device=dev)
        self.sel_idx = torch.zeros(self.batch, self.num_q_heads, self.sel_stride, dtype=torch.int32, device=dev)
        self.sel_cnt = torch.zeros(self.batch, self.num_q_heads, dtype=torch.int32, device=dev)
        self.reset_workspace()

    def reset_workspace(self) -> None:
        """Clears the workspace (``ha_workspace_init``): once before the first call, and again after a step that
        ended with ``HA_ERR_TIMEOUT`` (its arrival counters and ready words are then in no defined state)."""
        with torch.cuda.device(self.device):
            _raise_on(self.lib.ha_workspace_init(self.shape, self.c_budget, self.workspace.data_ptr(),
                                                 self.workspace_bytes, _stream_ptr(self.device)), "ha_workspace_init")

    # -- argument checks -----------------------------------------------------------------
    def _check_q(self, q):
        _check(q, "q", torch.bfloat16, (self.batch, self.num_q_heads, HEAD_DIM), self.device)

    def _check_kv_new(self, k_new, v_new):
        shape = (self.batch, self.num_kv_heads, HEAD_DIM)
        _check(k_new, "k_new", torch.bfloat16, shape, self.device)
        if v_new is not None:
            _check(v_new, "v_new", torch.bfloat16, shape, self.device)

    def check_status(self) -> None:
        """Reads the device status word (synchronises) and raises if a kernel reported a problem."""
        code = int(self.status.item())
        if code != 0:
            self.status.zero_()
            raise RuntimeError(f"device status: {_lib.status_str(code)} (status {code})")

    # -- stages ------------------------------------------------------------------------------
    def hash_decode(self, q, k_new=None, v_new=None, preact_dbg: torch.Tensor | None = None) -> torch.Tensor:
        """Encodes the new query (and key) and appends the key's code / K / V rows to the cache at
        token ``seq_lens - 1``. Returns the query codes ``[B, Hq]`` (int32 bit patterns)."""
        self._check_q(q)
        if k_new is not None:
            self._check_kv_new(k_new, v_new)
        elif v_new is not None:
            raise ValueError("v_new without k_new")
        if preact_dbg is not None:
            _check(preact_dbg, "preact_dbg", torch.float32, (self.batch, 2, self.num_q_heads, 32), self.device)
        c = self.cache
        with torch.cuda.device(self.device), _call_range("ha_hash_decode"):
            rc = self.lib.ha_hash_decode(
                self.shape, self.c_weights, q.data_ptr(), k_new.data_ptr() if k_new is not None else None,
                v_new.data_ptr() if v_new is not None else None, c.k_pages.data_ptr(), c.v_pages.data_ptr(),
                c.hash_pages.data_ptr(), c.page_table.data_ptr(), c.seq_lens.data_ptr(), self.q_codes.data_ptr(),
                preact_dbg.data_ptr() if preact_dbg is not None else None, self.status.data_ptr(),
                _stream_ptr(self.device))
        _raise_on(rc, "ha_hash_decode")
        return self.q_codes

    def hash_prefill(self, first_token: torch.Tensor | None = None) -> None:
        """Encodes the cached keys ``[first_token[b], seq_lens[b])`` of every sequence into the hash pages."""
        if first_token is not None:
            _check(first_token, "first_token", torch.int32, (self.batch,), self.device)
        c = self.cache
        with torch.cuda.device(self.device), _call_range("ha_hash_prefill"):
            rc = self.lib.ha_hash_prefill(
                self.shape, self.c_weights, c.k_pages.data_ptr(), c.hash_pages.data_ptr(), c.page_table.data_ptr(),
                c.seq_lens.data_ptr(), first_token.data_ptr() if first_token is not None else None,
                self.status.data_ptr(), _stream_ptr(self.device))
        _raise_on(rc, "ha_hash_prefill")

    def score_select(self, q_codes: torch.Tensor | None = None, scores_dbg: torch.Tensor | None = None):
        """Hamming scores + budget selection. Returns ``(sel_idx [B,Hq,sel_stride], sel_cnt [B,Hq])``."""
        q_codes = self.q_codes if q_codes is None else q_codes
        _check(q_codes, "q_codes", torch.int32, (self.batch, self.num_q_heads), self.device)
        if scores_dbg is not None:
            _check(scores_dbg, "scores_dbg", torch.uint8,
                   (self.batch, self.num_q_heads, self.cache.max_pages * PAGE), self.device)
        c = self.cache
        with torch.cuda.device(self.device), _call_range("ha_score_select"):
            rc = self.lib.ha_score_select(
                self.shape, self.c_budget, q_codes.data_ptr(), c.hash_pages.data_ptr(), c.page_table.data_ptr(),
                c.seq_lens.data_ptr(), self.sel_idx.data_ptr(), self.sel_cnt.data_ptr(),
                scores_dbg.data_ptr() if scores_dbg is not None else None, self.workspace.data_ptr(),
                self.workspace_bytes, self.status.data_ptr(), _stream_ptr(self.device))
        _raise_on(rc, "ha_score_select")
        return self.sel_idx, self.sel_cnt

    def score_plan(self, q_codes: torch.Tensor | None = None) -> torch.Tensor:
        """First half of the step after the encoder (``ha_score_plan``): streams the hash pages and leaves the
        score bytes and the selection plan in the workspace. Returns ``sel_cnt [B, Hq]``."""
        q_codes = self.q_codes if q_codes is None else q_codes
        _check(q_codes, "q_codes", torch.int32, (self.batch, self.num_q_heads), self.device)
        c = self.cache
        with torch.cuda.device(self.device), _call_range("ha_score_plan"):
            rc = self.lib.ha_score_plan(
                self.shape, self.c_budget, q_codes.data_ptr(), c.hash_pages.data_ptr(), c.page_table.data_ptr(),
                c.seq_lens.data_ptr(), self.sel_cnt.data_ptr(), self.workspace.data_ptr(), self.workspace_bytes,
                self.status.data_ptr(), _stream_ptr(self.device))
        _raise_on(rc, "ha_score_plan")
        return self.sel_cnt

    def select_attend(self, q, out: torch.Tensor | None = None) -> torch.Tensor:
        """Second half (``ha_select_attend``), on the plan :meth:`score_plan` left in the workspace: selects
        (``sel_idx``) and attends in one kernel. Returns ``out [B, Hq, 128]`` bf16."""
        self._check_q(q)
        out = torch.empty_like(q) if out is None else out
        _check(out, "out", torch.bfloat16, (self.batch, self.num_q_heads, HEAD_DIM), self.device)
        c = self.cache
        with torch.cuda.device(self.device), _call_range("ha_select_attend"):
            rc = self.lib.ha_select_attend(
                self.shape, self.c_budget, q.data_ptr(), c.k_pages.data_ptr(), c.v_pages.data_ptr(),
                c.page_table.data_ptr(), c.seq_lens.data_ptr(), self.sel_idx.data_ptr(), self.sm_scale,
                out.data_ptr(), self.workspace.data_ptr(), self.workspace_bytes, self.status.data_ptr(),
                _stream_ptr(self.device))
        _raise_on(rc, "ha_select_attend")
        return out

    def step_path(self) -> str:
        """The kernels one :meth:`decode_step` launches for this shape, by name."""
        return self.lib.ha_decode_step_path(self.shape, self.c_budget).decode()

    def score_select_static(self, q_codes: torch.Tensor | None = None):
        """:meth:`score_select` through ``ha_score_select_static``: no workspace is handed over, the
        kernels use the scratch buffer built into the library. Meant for hosts that are not allowed to
        allocate device memory for a workspace (a serving plugin's enqueue hook, a process whose pool
        already owns the device). Raises if the shape needs more than the built-in buffer holds.
        Results are identical to :meth:`score_select`; calls that could overlap on the GPU must be
        ordered by the caller, since they all share that one buffer."""
        q_codes = self.q_codes if q_codes is None else q_codes
        _check(q_codes, "q_codes", torch.int32, (self.batch, self.num_q_heads), self.device)
        c = self.cache
        with torch.cuda.device(self.device), _call_range("ha_score_select_static"):
            rc = self.lib.ha_score_select_static(
                self.shape, self.c_budget, q_codes.data_ptr(), c.hash_pages.data_ptr(), c.page_table.data_ptr(),
                c.seq_lens.data_ptr(), self.sel_idx.data_ptr(), self.sel_cnt.data_ptr(), self.status.data_ptr(),
                _stream_ptr(self.device))
        _raise_on(rc, "ha_score_select_static")
        return self.sel_idx, self.sel_cnt

    def sparse_decode(self, q, out: torch.Tensor | None = None, sel_idx=None, sel_cnt=None) -> torch.Tensor:
        """Attention of q over sink + selected + recent rows. Returns ``out [B, Hq, 128]`` bf16."""
        self._check_q(q)
        out = torch.empty_like(q) if out is None else out
        _check(out, "out", torch.bfloat16, (self.batch, self.num_q_heads, HEAD_DIM), self.device)
        sel_idx = self.sel_idx if sel_idx is None else sel_idx
        sel_cnt = self.sel_cnt if sel_cnt is None else sel_cnt
        _check(sel_idx, "sel_idx", torch.int32, (self.batch, self.num_q_heads, self.sel_stride), self.device)
        _check(sel_cnt, "sel_cnt", torch.int32, (self.batch, self.num_q_heads), self.device)
        c = self.cache
        with torch.cuda.device(self.device), _call_range("ha_sparse_decode"):
            rc = self.lib.ha_sparse_decode(
                self.shape, self.c_budget, q.data_ptr(), c.k_pages.data_ptr(), c.v_pages.data_ptr(),
                c.page_table.data_ptr(), c.seq_lens.data_ptr(), sel_idx.data_ptr(), sel_cnt.data_ptr(),
                self.sm_scale, out.data_ptr(), self.workspace.data_ptr(), self.workspace_bytes,
                self.status.data_ptr(), _stream_ptr(self.device))
        _raise_on(rc, "ha_sparse_decode")
        return out

    def decode_step_rows(self, q, k_new, v_new, out: torch.Tensor | None = None) -> torch.Tensor:
        """Multi-token decode on a context built over :class:`ChunkRows` (``ha_decode_step_rows``):
        ``q [rows, Hq, 128]``, ``k_new / v_new [rows, Hkv, 128]`` in the rows' order; the rows' lengths
        must have been set with ``ChunkRows.advance()``."""
        c = self.cache
        if not isinstance(c, ChunkRows):
            raise ValueError("decode_step_rows needs a context built on ChunkRows")
        if self.budget.recent_budget < c.q_len - 1:
            raise NotImplementedError("multi-token decode needs recent_budget >= q_len - 1")
        self._check_q(q)
        self._check_kv_new(k_new, v_new)
        if v_new is None:
            raise ValueError("v_new is required")
        out = torch.empty_like(q) if out is None else out
        _check(out, "out", torch.bfloat16, (self.batch, self.num_q_heads, HEAD_DIM), self.device)
        with torch.cuda.device(self.device), _call_range("ha_decode_step_rows"):
            rc = self.lib.ha_decode_step_rows(
                self.shape, self.c_budget, self.c_weights, q.data_ptr(), k_new.data_ptr(), v_new.data_ptr(),
                c.k_pages.data_ptr(), c.v_pages.data_ptr(), c.hash_pages.data_ptr(), c.page_table.data_ptr(),
                c.seq_lens.data_ptr(), c.budget_lens.data_ptr(), self.q_codes.data_ptr(), self.sel_idx.data_ptr(),
                self.sel_cnt.data_ptr(), self.sm_scale, out.data_ptr(), self.workspace.data_ptr(),
                self.workspace_bytes, self.status.data_ptr(), _stream_ptr(self.device))
        _raise_on(rc, "ha_decode_step_rows")
        return out

    def decode_step(self, q, k_new, v_new, out: torch.Tensor | None = None) -> torch.Tensor:
        """The whole step (encode + append, score + select, sparse attention) in one library call."""
        self._check_q(q)
        self._check_kv_new(k_new, v_new)
        out = torch.empty_like(q) if out is None else out
        _check(out, "out", torch.bfloat16, (self.batch, self.num_q_heads, HEAD_DIM), self.device)
        c = self.cache
        with torch.cuda.device(self.device), _call_range("ha_decode_step"):
            rc = self.lib.ha_decode_step(
                self.shape, self.c_budget, self.c_weights, q.data_ptr(), k_new.data_ptr(),
                v_new.data_ptr() if v_new is not None else None, c.k_pages.data_ptr(), c.v_pages.data_ptr(),
                c.hash_pages.data_ptr(), c.page_table.data_ptr(), c.seq_lens.data_ptr(), self.q_codes.data_ptr(),
                self.sel_idx.data_ptr(), self.sel_cnt.data_ptr(), self.sm_scale, out.data_ptr(),
                self.workspace.data_ptr(), self.workspace_bytes, self.status.data_ptr(), _stream_ptr(self.device))
        _raise_on(rc, "ha_decode_step")
        return out


def rope_split(qkv: torch.Tensor, positions: torch.Tensor, num_q_heads: int, num_kv_heads: int, rope_theta: float):
    """``ha_rope_split``: the fused projection ``qkv [B, (Hq + 2 Hkv) * 128]`` bf16 of one new token per sequence ->
    contiguous ``q [B, Hq, 128]``, ``k_new``, ``v_new [B, Hkv, 128]`` with the rotary embedding applied to q and k
    for ``positions [B]`` (int64, on the device)."""
    B = qkv.shape[0]
    _check(qkv, "qkv", torch.bfloat16, (B, (num_q_heads + 2 * num_kv_heads) * HEAD_DIM), qkv.device)
    _check(positions, "positions", torch.int64, (B,), qkv.device)
    q = torch.empty(B, num_q_heads, HEAD_DIM, dtype=torch.bfloat16, device=qkv.device)
    k = torch.empty(B, num_kv_heads, HEAD_DIM, dtype=torch.bfloat16, device=qkv.device)
    v = torch.empty_like(k)
    with torch.cuda.device(qkv.device):
        rc = _lib.load().ha_rope_split(qkv.data_ptr(), positions.data_ptr(), B, num_q_heads, num_kv_heads, float(rope_theta),
                                       q.data_ptr(), k.data_ptr(), v.data_ptr(), _stream_ptr(qkv.device))
    _raise_on(rc, "ha_rope_split")
    return q, k, v


class ChunkRows:
    """A multi-token decode step laid out as rows for ``ha_decode_step_rows``: ``q_len`` new tokens
    for each of the ``B`` sequences of ``cache`` become ``B * q_len`` rows (sequence-major) that share
    the cache's page pools; row ``b * q_len + i`` sees the first ``old_len[b] + i + 1`` tokens and
    appends token ``old_len[b] + i``. It quacks like a :class:`PagedHashKVCache` with ``B * q_len``
    sequences, so a :class:`SparseDecodeContext` can be built on it (one per chunk length)."""

    def __init__(self, cache: PagedHashKVCache, q_len: int):
        if q_len < 1:
            raise ValueError("q_len must be positive")
        self.base, self.q_len = cache, q_len
        self.device, self.batch, self.num_kv_heads = cache.device, cache.batch * q_len, cache.num_kv_heads
        self.max_pages, self.num_pages = cache.max_pages, cache.num_pages
        self.k_pages, self.v_pages, self.hash_pages = cache.k_pages, cache.v_pages, cache.hash_pages
        self.page_table = cache.page_table.repeat_interleave(q_len, dim=0).contiguous()
        self.seq_lens = torch.zeros(self.batch, dtype=torch.int32, device=self.device)
        self.budget_lens = torch.zeros(self.batch, dtype=torch.int32, device=self.device)
        self._offsets = torch.arange(1, q_len + 1, dtype=torch.int32, device=self.device)

    def advance(self) -> None:
        """Sets the rows' lengths for a chunk that starts at the base cache's current lengths and
        moves the base cache's lengths past the chunk."""
        old = self.base.seq_lens
        self.seq_lens.copy_((old[:, None] + self._offsets[None, :]).reshape(-1))
        self.budget_lens.copy_((old + self.q_len).repeat_interleave(self.q_len))
        old += self.q_len


class HostStepBuffers:
    """Host tensors and device staging buffers for :func:`decode_step_host`. Page-locked host
    tensors (the default) are read and written by the kernels in place; pageable ones
    (``pinned=False``) are copied through the staging buffers."""

    def __init__(self, ctx: SparseDecodeContext, pinned: bool = True):
        B, Hq, Hkv, dev = ctx.batch, ctx.num_q_heads, ctx.num_kv_heads, ctx.device
        pin = dict(dtype=torch.bfloat16, pin_memory=pinned)
        self.q_host = torch.empty(B, Hq, HEAD_DIM, **pin)
        self.k_host = torch.empty(B, Hkv, HEAD_DIM, **pin)
        self.v_host = torch.empty(B, Hkv, HEAD_DIM, **pin)
        self.out_host = torch.empty(B, Hq, HEAD_DIM, **pin)
        self.status_host = torch.zeros(1, dtype=torch.int32, pin_memory=pinned)
        self.status_view = self.status_host.numpy()  # shares the memory
        self.q_dev = torch.empty(B, Hq, HEAD_DIM, dtype=torch.bfloat16, device=dev)
        self.k_dev = torch.empty(B, Hkv, HEAD_DIM, dtype=torch.bfloat16, device=dev)
        self.v_dev = torch.empty(B, Hkv, HEAD_DIM, dtype=torch.bfloat16, device=dev)
        self.out_dev = torch.empty(B, Hq, HEAD_DIM, dtype=torch.bfloat16, device=dev)
        self._bound = None
        self._graph = None

    def bound_call(self, ctx: SparseDecodeContext):
        """``ha_decode_step_host`` with every argument but (stream, synchronize) bound to the buffers
        of ``ctx`` and of this object. The buffers never move, so the argument list is converted to
        C types once instead of at every step."""
        if self._bound is None or self._bound[0] is not ctx:
            c = ctx.cache
            vp, i32, f32, sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_size_t
            fixed = [ctypes.byref(ctx.shape), ctypes.byref(ctx.c_budget), ctypes.byref(ctx.c_weights)] + [vp(t.data_ptr()) for t in (
                self.q_host, self.k_host, self.v_host, self.out_host, self.status_host, self.q_dev, self.k_dev,
                self.v_dev, self.out_dev, c.k_pages, c.v_pages, c.hash_pages, c.page_table, c.seq_lens, ctx.q_codes,
                ctx.sel_idx, ctx.sel_cnt)] + [f32(ctx.sm_scale), vp(ctx.workspace.data_ptr()),
                                              sz(ctx.workspace_bytes), vp(ctx.status.data_ptr())]
            fn = ctx.lib.ha_decode_step_host
            self._bound = (ctx, lambda stream, sync: fn(*fixed, vp(stream), i32(sync)))
        return self._bound[1]

    def graph_for(self, ctx: SparseDecodeContext) -> torch.cuda.CUDAGraph:
        """The CUDA graph of one ``ha_decode_step_host`` call (without the final wait) on these buffers."""
        if self._graph is None or self._graph[0] is not ctx:
            call = self.bound_call(ctx)
            with torch.cuda.device(ctx.device):
                # an eager call first: whatever the library creates at first use must not happen under capture
                # (it writes the same cache slot and outputs the recorded call will write again)
                _raise_on(call(torch.cuda.current_stream(ctx.device).cuda_stream, 1), "ha_decode_step_host")
                torch.cuda.synchronize(ctx.device)
                side, graph = torch.cuda.Stream(ctx.device), torch.cuda.CUDAGraph()
                with torch.cuda.stream(side):
                    with torch.cuda.graph(graph, stream=side):
                        _raise_on(call(side.cuda_stream, 0), "ha_decode_step_host")
            self._graph = (ctx, graph)
        return self._graph[1]

    @property
    def h2d_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.q_host, self.k_host, self.v_host))

    @property
    def d2h_bytes(self) -> int:
        return self.out_host.numel() * self.out_host.element_size() + 4


def decode_step_host(ctx: SparseDecodeContext, buf: HostStepBuffers, synchronize: bool = True,
                     use_graph: bool = False) -> torch.Tensor:
    """Decode step for callers whose q / k_new / v_new / out live in host memory: the step reads
    ``buf.q_host, k_host, v_host`` (in place if page-locked, else through a copy), leaves the result
    in ``buf.out_host`` and (if ``synchronize``) waits and checks the device status.

    ``use_graph``: the first call records the library call (all its kernels, the reads of the host
    buffers and the copies back) into a CUDA graph owned by ``buf``; later calls replay it - one
    launch per step instead of one per kernel. Everything a step reads that changes between steps
    (the host buffers' contents, the sequence lengths) is read at replay time."""
    if use_graph:
        stream = torch.cuda.current_stream(ctx.device)
        buf.graph_for(ctx).replay()
        if synchronize:
            stream.synchronize()
            code = int(buf.status_view[0])  # (a numpy view of the pinned word: no tensor indexing per step)
            if code != 0:
                raise RuntimeError(f"device status: {_lib.status_str(code)} (status {code})")
        return buf.out_host
    call = buf.bound_call(ctx)
    stream = torch.cuda.current_stream(ctx.device).cuda_stream
    if torch.cuda.current_device() == ctx.device.index:
        rc = call(stream, 1 if synchronize else 0)
    else:
        with torch.cuda.device(ctx.device):
            rc = call(stream, 1 if synchronize else 0)
    _raise_on(rc, "ha_decode_step_host")
    return buf.out_host
