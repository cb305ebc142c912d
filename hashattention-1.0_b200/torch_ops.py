"""``torch.ops.hashattn.decode_step``: the decode step as a registered torch operator.

The operator takes only tensors and scalars, so that a traced or exported module (and a CUDA
graph capture) sees one opaque node that mutates the cache pools, the intermediate buffers and
``out``. Its CUDA implementation is the C entry point ``ha_decode_step`` called through ctypes with
``tensor.data_ptr()`` and the current stream; there is no CPU implementation and no other backend
(a CPU tensor ends in torch's "no kernel for this device" error). The fake (meta) implementation
does nothing: every result is written into an argument.

It replaces the decode branch of ``LlamaAttention_heavy_hitter.forward``
(hashattention/hashattention_llama.py:571-623) for ``q_len == 1``.
"""
from __future__ import annotations

import torch

from . import _lib
from .cache import GROUP, HEAD_DIM, PAGE

_MUTATED = ("k_pages", "v_pages", "hash_pages", "q_codes", "sel_idx", "sel_cnt", "workspace", "status", "out")


def _shape_of(q, k_new, k_pages, page_table, sel_idx) -> _lib.HaShape:
    if q.dim() != 3 or k_new.dim() != 3 or q.shape[2] != HEAD_DIM or q.shape[1] != k_new.shape[1] * GROUP:
        raise ValueError(f"q should be of size (B, {GROUP} * Hkv, {HEAD_DIM}) and k_new (B, Hkv, {HEAD_DIM}), "
                         f"but are {tuple(q.shape)} and {tuple(k_new.shape)}")
    if k_pages.dim() != 4 or tuple(k_pages.shape[1:]) != (k_new.shape[1], PAGE, HEAD_DIM):
        raise ValueError(f"k_pages should be of size (num_pages, {k_new.shape[1]}, {PAGE}, {HEAD_DIM}), "
                         f"but is {tuple(k_pages.shape)}")
    return _lib.HaShape(q.shape[0], k_new.shape[1], GROUP, HEAD_DIM, PAGE, page_table.shape[1], k_pages.shape[0],
                        sel_idx.shape[2])


@torch.library.custom_op("hashattn::decode_step", mutates_args=_MUTATED, device_types="cuda")
def decode_step(q: torch.Tensor, k_new: torch.Tensor, v_new: torch.Tensor,
                k_pages: torch.Tensor, v_pages: torch.Tensor, hash_pages: torch.Tensor,
                page_table: torch.Tensor, seq_lens: torch.Tensor,
                wq: torch.Tensor, bq: torch.Tensor, wk: torch.Tensor, bk: torch.Tensor,
                q_codes: torch.Tensor, sel_idx: torch.Tensor, sel_cnt: torch.Tensor,
                workspace: torch.Tensor, status: torch.Tensor, out: torch.Tensor,
                init_budget: int, recent_budget: int, heavy_budget: float, sm_scale: float,
                eval_mode: int = 0, retrieve_depth: int = 0, num_hash_layers: int = 3) -> None:
    lib = _lib.load()
    tensors = dict(q=q, k_new=k_new, v_new=v_new, k_pages=k_pages, v_pages=v_pages, hash_pages=hash_pages,
                   page_table=page_table, seq_lens=seq_lens, wq=wq, bq=bq, wk=wk, bk=bk, q_codes=q_codes,
                   sel_idx=sel_idx, sel_cnt=sel_cnt, workspace=workspace, status=status, out=out)
    for name, t in tensors.items():
        if t.device != q.device:
            raise ValueError(f"{name} must live on {q.device}, got {t.device}")
        if not t.is_contiguous():
            raise ValueError(f"{name} must be contiguous")
    for name in ("q", "k_new", "v_new", "k_pages", "v_pages", "out"):
        if tensors[name].dtype != torch.bfloat16:
            raise ValueError(f"{name} must be torch.bfloat16, got {tensors[name].dtype}")
    if wq.dtype != wk.dtype or wq.dtype not in (torch.bfloat16, torch.float32):
        raise ValueError("hash weights must both be bfloat16 or both float32")
    shape = _shape_of(q, k_new, k_pages, page_table, sel_idx)
    budget = _lib.HaBudget(int(init_budget), int(recent_budget), float(heavy_budget), int(eval_mode),
                           int(retrieve_depth))
    weights = _lib.HaHashWeights(wq.data_ptr(), bq.data_ptr(), wk.data_ptr(), bk.data_ptr(),
                                 _lib.HA_WEIGHTS_BF16 if wq.dtype == torch.bfloat16 else _lib.HA_WEIGHTS_F32,
                                 int(num_hash_layers))
    need = int(lib.ha_workspace_bytes(shape, budget))
    if need == 0 or workspace.numel() * workspace.element_size() < need:
        raise ValueError(f"workspace holds {workspace.numel() * workspace.element_size()} bytes, the step needs {need}")
    with torch.cuda.device(q.device):
        rc = lib.ha_decode_step(shape, budget, weights, q.data_ptr(), k_new.data_ptr(), v_new.data_ptr(),
                                k_pages.data_ptr(), v_pages.data_ptr(), hash_pages.data_ptr(), page_table.data_ptr(),
                                seq_lens.data_ptr(), q_codes.data_ptr(), sel_idx.data_ptr(), sel_cnt.data_ptr(),
                                float(sm_scale), out.data_ptr(), workspace.data_ptr(),
                                workspace.numel() * workspace.element_size(), status.data_ptr(),
                                torch.cuda.current_stream(q.device).cuda_stream)
    if rc != _lib.HA_OK:
        raise RuntimeError(f"ha_decode_step failed: {_lib.status_str(rc)} (status {rc})")


@decode_step.register_fake
def _decode_step_fake(q, k_new, v_new, k_pages, v_pages, hash_pages, page_table, seq_lens, wq, bq, wk, bk,
                      q_codes, sel_idx, sel_cnt, workspace, status, out,
                      init_budget, recent_budget, heavy_budget, sm_scale, eval_mode=0, retrieve_depth=0,
                      num_hash_layers=3) -> None:
    return None


def decode_step_op(ctx, q: torch.Tensor, k_new: torch.Tensor, v_new: torch.Tensor,
                   out: torch.Tensor | None = None) -> torch.Tensor:
    """``torch.ops.hashattn.decode_step`` on the buffers of a :class:`SparseDecodeContext`."""
    out = torch.empty_like(q) if out is None else out
    c, w, b = ctx.cache, ctx.weights, ctx.budget
    torch.ops.hashattn.decode_step(q, k_new, v_new, c.k_pages, c.v_pages, c.hash_pages, c.page_table, c.seq_lens,
                                   w.wq, w.bq, w.wk, w.bk, ctx.q_codes, ctx.sel_idx, ctx.sel_cnt, ctx.workspace,
                                   ctx.status, out, b.init_budget, b.recent_budget, b.heavy_budget, ctx.sm_scale,
                                   ctx.c_budget.eval_mode, ctx.c_budget.retrieve_depth, w.num_layers)
    return out
