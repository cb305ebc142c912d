"""Retrieval quality of the hash selection: which fraction of the keys with the 32 largest true
attention logits (among the selection candidates) is inside the selected heavy set?

This is the statistic the reference collects in ``usa_local_compute``
(hashattention/hashattention_llama.py:359-395: ``overlap_ratio = |pred & target| / |target|`` with
``target`` = top-32 of QK^T/sqrt(d) over the candidates). There ``pred`` is the top ``S // 16`` of the
hash scores whatever the budget; here it is the heavy set the selection kernels actually emitted
for the context's budget (``ctx.sel_idx`` / ``ctx.sel_cnt``), so the number says what the sparse
attention really got to see. A diagnostic: dense torch ops on the device, not part of the decode path.

    python hashattention-1.0_b200/diagnostics/recall.py [S] [heavy_budget]
"""
from __future__ import annotations

import math
import os
import sys

import torch


def topk_recall(ctx, q: torch.Tensor, topk: int = 32) -> torch.Tensor:
    """``q [B, Hq, 128]`` (the queries of the step that filled ``ctx.sel_idx``) -> recall ``[B, Hq]`` float32;
    NaN where a sequence has no candidate."""
    cache, bud = ctx.cache, ctx.budget
    B, Hq, D = q.shape
    group = Hq // cache.num_kv_heads
    out = torch.full((B, Hq), float("nan"), dtype=torch.float32, device=q.device)
    for b in range(B):
        S = int(cache.seq_lens[b])
        lo = min(bud.init_budget, S)
        hi = max(lo, S - bud.recent_budget)
        if hi <= lo:
            continue
        k, _ = cache.read_kv(b, S)                                              # [Hkv, S, D]
        logits = torch.einsum("hd,hsd->hs", q[b].float(), k.float().repeat_interleave(group, dim=0)) / math.sqrt(D)
        cand = logits[:, lo:hi]
        n = min(topk, hi - lo)
        target = cand.topk(n, dim=-1).indices + lo                              # [Hq, n]
        picked = torch.zeros(Hq, S, dtype=torch.bool, device=q.device)
        for h in range(Hq):
            cnt = int(ctx.sel_cnt[b, h])
            picked[h, ctx.sel_idx[b, h, :cnt].long()] = True
        out[b] = picked.gather(1, target).float().mean(dim=-1)
    return out


def main():
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    sys.path.insert(0, root)
    import __graft_entry__ as entry

    ha = entry.load_package()
    from hashattention_b200 import synthetic

    S = int(sys.argv[1]) if len(sys.argv) > 1 else 8192
    heavy = float(sys.argv[2]) if len(sys.argv) > 2 else 1.0 / 32
    dev = torch.device("cuda:0")
    Hq, Hkv = 32, 8
    cache = ha.PagedHashKVCache(1, Hkv, S, dev)
    synthetic.fill_cache_on_device(cache, [S], seed=0)
    ctx = ha.SparseDecodeContext(cache, ha.Budget(128, heavy, 128), synthetic.make_usa(Hq, 128, seed=0, bf16=True).packed(dev))
    ctx.hash_prefill()
    gen = torch.Generator(device=dev).manual_seed(1)
    q = torch.randn(1, Hq, 128, generator=gen, device=dev).bfloat16()
    k_new = torch.randn(1, Hkv, 128, generator=gen, device=dev).bfloat16()
    ctx.decode_step(q, k_new, k_new)
    ctx.check_status()
    r = topk_recall(ctx, q)
    print(f"S={S} heavy={heavy:.4f}: recall of the true top-32 inside the heavy set, mean over heads "
          f"{float(r.nanmean()):.3f} (random-init hash weights: expect about the budget fraction "
          f"{ctx.budget.heavy_tokens(S) / max(1, S - 256):.3f})")


if __name__ == "__main__":
    main()
