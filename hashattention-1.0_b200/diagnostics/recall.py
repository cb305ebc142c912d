"""Retrieval quality of the hash selection: which fraction of the keys with the 32 largest true
attention logits (among the selection candidates) is inside the selected heavy set?

This is the statistic the reference collects in ``usa_local_compute``
(hashattention/hashattention_llama.py:359-395: ``overlap_ratio = |pred & target| / |target|`` with
``target`` = top-32 of QK^T/sqrt(d) over the candidates). There ``pred`` is the top ``S // 16`` of the
hash scores whatever the budget; here it is the heavy set the selection kernels actually emitted
for the context's budget (``ctx.sel_idx`` / ``ctx.sel_cnt``), so the number says what the sparse
attention really got to see. A diagnostic: dense torch ops on the device, not part of the decode path.

    python hashattention-1.0_b200/diagnostics/recall.py [S] [heavy_budget]
    python hashattention-1.0_b200/diagnostics/recall.py planted [S] [heavy_budget]

The second form plants near-duplicates of the query among the keys (2 % of the positions, cosine 0.9 to the
first query head of each kv-head, as the long-context configuration of the benchmark describes) and reports
how many of them the heavy set of that head contains. With randomly initialised, separately drawn query and key
hash functions there is no reason for the codes of similar vectors to agree, so this number says something
about trained hash weights only; with the synthetic ones it is expected near the budget fraction.
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


def planted_recall(ctx, planted: list[torch.Tensor], group: int = 4) -> torch.Tensor:
    """Fraction of the planted key positions of sequence b that the heavy set of query head ``group * j``
    contains, ``[B, Hkv]``."""
    B, Hkv = len(planted), ctx.num_kv_heads
    out = torch.zeros(B, Hkv, dtype=torch.float32)
    for b, pos in enumerate(planted):
        for j in range(Hkv):
            cnt = int(ctx.sel_cnt[b, j * group])
            picked = set(ctx.sel_idx[b, j * group, :cnt].tolist())
            out[b, j] = sum(1 for t in pos.tolist() if t in picked) / max(1, len(pos))
    return out


def main_planted(argv):
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    sys.path.insert(0, root)
    import __graft_entry__ as entry

    ha = entry.load_package()
    from hashattention_b200 import synthetic

    S = int(argv[0]) if len(argv) > 0 else 8192
    heavy = float(argv[1]) if len(argv) > 1 else 1.0 / 32
    dev = torch.device("cuda:0")
    Hq, Hkv = 32, 8
    inp = synthetic.make_decode_inputs(3, [S], Hq, Hkv, plant_frac=0.02)
    cache = ha.PagedHashKVCache(1, Hkv, S, dev)
    cache.write_kv(0, inp.k[0][:, :S - 1], inp.v[0][:, :S - 1])
    ctx = ha.SparseDecodeContext(cache, ha.Budget(128, heavy, 128), synthetic.make_usa(Hq, 128, seed=0, bf16=True).packed(dev))
    ctx.hash_prefill()
    cache.seq_lens += 1
    q = inp.q.to(dev, torch.bfloat16)
    ctx.decode_step(q, inp.k[0][None, :, -1].to(dev, torch.bfloat16), inp.v[0][None, :, -1].to(dev, torch.bfloat16))
    ctx.check_status()
    r = planted_recall(ctx, inp.planted)
    print(f"S={S} heavy={heavy:.4f}: {len(inp.planted[0])} planted keys; fraction inside the heavy set of their query head, "
          f"mean over kv-heads {float(r.mean()):.3f}; recall of the true top-32: {float(topk_recall(ctx, q).nanmean()):.3f}")


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
    if len(sys.argv) > 1 and sys.argv[1] == "planted":
        main_planted(sys.argv[2:])
    else:
        main()
