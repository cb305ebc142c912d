"""Multi-GPU partitioning of the decode path: every (sequence, kv-head) unit is independent
through hash encoding, scoring, selection and attention (a query head only ever meets the keys
of its own kv-head; hashattention/hashattention_llama.py:159-169, 425-438), so GPUs split the
kv-heads (or the sequences) and exchange nothing until the outputs are concatenated.

One process per GPU; ``torch.distributed`` (NCCL on GPUs, gloo in CPU tests) is used only for
the final gather.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

GROUP = 4  # query heads per kv-head


def kv_head_range(num_kv_heads: int, world_size: int, rank: int) -> tuple[int, int]:
    """kv-heads [j0, j1) owned by ``rank`` when kv-heads are dealt out in contiguous blocks."""
    if world_size < 1 or not 0 <= rank < world_size:
        raise ValueError(f"bad rank {rank} of {world_size}")
    if num_kv_heads % world_size != 0:
        raise ValueError(f"{num_kv_heads} kv-heads cannot be split evenly over {world_size} GPUs")
    per = num_kv_heads // world_size
    return rank * per, (rank + 1) * per


def batch_range(batch: int, world_size: int, rank: int) -> tuple[int, int]:
    """Sequences [b0, b1) owned by ``rank`` (block partition, remainder to the first ranks)."""
    if world_size < 1 or not 0 <= rank < world_size:
        raise ValueError(f"bad rank {rank} of {world_size}")
    base, extra = divmod(batch, world_size)
    b0 = rank * base + min(rank, extra)
    return b0, b0 + base + (1 if rank < extra else 0)


def shard_step_inputs(q: torch.Tensor, k_new: torch.Tensor, v_new: torch.Tensor, world_size: int, rank: int):
    """The slices of one decode step's q [B,Hq,D], k_new / v_new [B,Hkv,D] for ``rank``'s kv-heads."""
    j0, j1 = kv_head_range(k_new.shape[1], world_size, rank)
    return (q[:, j0 * GROUP:j1 * GROUP].contiguous(), k_new[:, j0:j1].contiguous(), v_new[:, j0:j1].contiguous())


def gather_output(out_local: torch.Tensor, group=None) -> torch.Tensor:
    """Concatenates the per-rank outputs [B, Hq/world, D] along the head axis, on every rank.
    The only communication of the path; rank order equals kv-head order. One collective into one buffer
    (``all_gather_into_tensor``) where the backend has it (NCCL), the list form otherwise (gloo)."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return out_local
    world = dist.get_world_size(group)
    local = out_local.contiguous()
    if dist.get_backend(group) == "nccl":
        flat = torch.empty((world,) + tuple(local.shape), dtype=local.dtype, device=local.device)
        dist.all_gather_into_tensor(flat, local, group=group)
        return flat.transpose(0, 1).reshape(local.shape[0], world * local.shape[1], *local.shape[2:])
    parts = [torch.empty_like(local) for _ in range(world)]
    dist.all_gather(parts, local, group=group)
    return torch.cat(parts, dim=1)
