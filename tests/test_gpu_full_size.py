"""The decode step at the full sizes of the three benchmark workloads, checked through properties
that do not need a CPU pass over the data: every check is computed on the device with plain torch
fp32 / int64 operations from the cache's own contents.

* the heavy set of every (sequence, head) is exactly the stable top-``hb`` of the Hamming scores of
  the stored codes: right size, no duplicates, inside the candidate range, no unselected candidate
  scores above the weakest selected one, ties at that score taken lowest index first - together
  these determine the set uniquely, which is the reference's rule
  (hashattention/hashattention_llama.py:423-438);
* the output equals fp32 softmax attention over sink + recent + heavy rows (:578-623) within
  max-abs 2e-2 and rel-L2 1e-2 (the output is rounded to bf16);
* every stored key code equals the sign bits of the fp32 hash MLP of the stored key (:204-214)
  wherever the pre-activation is at least 1e-4 from zero;
* a repeated step changes nothing.
"""
import copy

import pytest
import torch

import hashattention_b200 as ha
from hashattention_b200 import synthetic

pytestmark = pytest.mark.gpu

ALL_BITS = 0xFFFFFFFF
INIT, RECENT = 128, 128
HQ, HKV, D = 32, 8, 128
PREFILL_BAND = 1e-4

WORKLOADS = {
    "config1": (lambda: [32768], 1.0 / 32),
    "config3": (lambda: [131072] * 4, 1.0 / 32),
    "config2": (lambda: synthetic.ragged_lengths(2, 32, 16384, 65536), 1.0 / 16),
}


class Stepped:
    def __init__(self, device, name):
        lens_fn, heavy = WORKLOADS[name]
        self.lens = lens_fn()
        self.budget = ha.Budget(INIT, heavy, RECENT)
        self.usa = synthetic.make_usa(HQ, D, seed=3, bf16=True)
        B = len(self.lens)
        self.cache = ha.PagedHashKVCache(B, HKV, max(self.lens), device, shuffle_seed=17)
        synthetic.fill_cache_on_device(self.cache, self.lens, seed=4242)
        self.ctx = ha.SparseDecodeContext(self.cache, self.budget, self.usa.packed(device))
        self.ctx.hash_prefill()
        gen = torch.Generator(device=device).manual_seed(99)
        self.q = torch.randn(B, HQ, D, generator=gen, device=device).bfloat16()
        self.k_new = torch.randn(B, HKV, D, generator=gen, device=device).bfloat16()
        self.v_new = torch.randn(B, HKV, D, generator=gen, device=device).bfloat16()
        self.out = torch.zeros(B, HQ, D, dtype=torch.bfloat16, device=device)
        self.ctx.decode_step(self.q, self.k_new, self.v_new, out=self.out)
        torch.cuda.synchronize()
        self.ctx.check_status()


@pytest.fixture(scope="module", params=list(WORKLOADS))
def stepped(request, device):
    torch.backends.cuda.matmul.allow_tf32 = False
    s = Stepped(device, request.param)
    yield s
    del s
    torch.cuda.empty_cache()


def popcount32(x: torch.Tensor) -> torch.Tensor:
    """Bit count of int64 values in 0..2^32-1."""
    x = x - ((x >> 1) & 0x55555555)
    x = (x & 0x33333333) + ((x >> 2) & 0x33333333)
    x = (x + (x >> 4)) & 0x0F0F0F0F
    return ((x * 0x01010101) >> 24) & 0xFF


def selected_mask(ctx, b: int, S: int) -> torch.Tensor:
    """[Hq, S] bool from the device's index lists; asserts range and uniqueness on the way."""
    idx = ctx.sel_idx[b].to(torch.int64)
    cnt = ctx.sel_cnt[b].to(torch.int64)
    valid = torch.arange(idx.shape[1], device=idx.device)[None, :] < cnt[:, None]
    rows = torch.arange(idx.shape[0], device=idx.device)[:, None].expand_as(idx)
    listed = idx[valid]
    assert int(listed.min()) >= INIT and int(listed.max()) < S - RECENT
    mask = torch.zeros(idx.shape[0], S, dtype=torch.bool, device=idx.device)
    mask[rows[valid], listed] = True
    assert torch.equal(mask.sum(dim=1), cnt), "an index is listed twice"
    return mask


def test_heavy_sets_are_the_stable_top_hb_of_the_stored_codes(stepped):
    ctx, cache = stepped.ctx, stepped.cache
    for b, S in enumerate(stepped.lens):
        hb = min(stepped.budget.heavy_tokens(S), S - INIT - RECENT)
        assert bool((ctx.sel_cnt[b] == hb).all())
        q_codes = ctx.q_codes[b].to(torch.int64) & ALL_BITS
        score = 32 - popcount32(cache.read_codes(b) ^ q_codes[:, None])         # [Hq, S]
        pos = torch.arange(S, device=score.device)[None, :]
        cand = (pos >= INIT) & (pos < S - RECENT)
        sel = selected_mask(ctx, b, S)
        rest = cand & ~sel
        weakest = torch.where(sel, score, 99).min(dim=1).values
        assert bool((torch.where(rest, score, -1).max(dim=1).values <= weakest).all())
        tie = score == weakest[:, None]
        last_taken = torch.where(sel & tie, pos, -1).max(dim=1).values
        first_left = torch.where(rest & tie, pos, S).min(dim=1).values
        assert bool((last_taken < first_left).all()), "ties are not taken lowest index first"


def test_output_is_fp32_attention_over_sink_recent_and_heavy_rows(stepped):
    ctx, cache = stepped.ctx, stepped.cache
    worst_abs = worst_rel = 0.0
    for b, S in enumerate(stepped.lens):
        k, v = cache.read_kv(b)                                                    # [Hkv, S, D]
        assert torch.equal(k[:, -1], stepped.k_new[b]) and torch.equal(v[:, -1], stepped.v_new[b])
        pos = torch.arange(S, device=k.device)[None, :]
        keep = selected_mask(ctx, b, S) | (pos < INIT) | (pos >= S - RECENT)      # [Hq, S]
        q = stepped.q[b].float().view(HKV, HQ // HKV, D)
        logits = torch.einsum("jgd,jsd->jgs", q, k.float()).view(HQ, S) * ctx.sm_scale
        p = torch.softmax(logits.masked_fill(~keep, float("-inf")), dim=-1)
        want = torch.einsum("jgs,jsd->jgd", p.view(HKV, HQ // HKV, S), v.float()).reshape(HQ, D)
        got = stepped.out[b].float()
        worst_abs = max(worst_abs, float((got - want).abs().max()))
        worst_rel = max(worst_rel, float((got - want).norm() / want.norm()))
    assert worst_abs < 2e-2 and worst_rel < 1e-2, (worst_abs, worst_rel)


def test_stored_key_codes_are_the_sign_bits_of_the_fp32_hash_mlp(stepped):
    cache = stepped.cache
    nets = copy.deepcopy(stepped.usa).float().to(cache.device).learning_to_hash_transformation_k
    shifts = torch.arange(32, device=cache.device, dtype=torch.int64)
    in_band = total = 0
    with torch.no_grad():
        for b, S in enumerate(stepped.lens):
            k, _ = cache.read_kv(b)
            got = cache.read_codes(b)
            for h in range(HQ):
                pre = nets[h](k[h // (HQ // HKV)].float())                          # [S, 32]
                want = ((pre > 0).to(torch.int64) << shifts).sum(dim=-1)
                must = ((pre.abs() >= PREFILL_BAND).to(torch.int64) << shifts).sum(dim=-1)
                assert not bool((((got[h] ^ want) & must) != 0).any()), (b, h)
                in_band += int((pre.abs() < PREFILL_BAND).sum())
                total += pre.numel()
    assert in_band < 5e-3 * total, "the exclusion band swallows too many bits to be a check"


def test_a_repeated_step_changes_nothing(stepped):
    ctx = stepped.ctx
    results = []
    for _ in range(3):
        out = torch.zeros_like(stepped.out)
        ctx.sel_cnt.zero_()
        ctx.decode_step(stepped.q, stepped.k_new, stepped.v_new, out=out)
        torch.cuda.synchronize()
        ctx.check_status()
        listed = torch.arange(ctx.sel_idx.shape[-1], device=out.device) < ctx.sel_cnt[..., None]
        results.append((out, ctx.sel_cnt.clone(), torch.where(listed, ctx.sel_idx, -1).sort(dim=-1).values))
    for out, cnt, idx in results:
        assert torch.equal(out, stepped.out)
        assert torch.equal(cnt, results[0][1])
        assert torch.equal(idx, results[0][2])
