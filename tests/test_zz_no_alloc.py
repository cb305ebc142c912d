"""ha_score_select_static: the selection step for hosts that cannot give the library a workspace
(for example a serving plugin whose enqueue hook must not allocate, or a process whose memory pool
has already taken the whole device). It must give exactly what ha_score_select gives, call after
call, while using only the scratch buffer that is compiled into the library.

This file is collected last on purpose: a run that stops at the first failure has then already
exercised every other test."""
import ctypes

import pytest
import torch

import hashattention_b200 as ha
from hashattention_b200 import _lib, synthetic


def test_oversized_shapes_are_refused_before_anything_is_launched():
    lib = _lib.load()
    bud = _lib.HaBudget(128, 128, 1.0 / 32)
    small = _lib.HaShape(1, 8, 4, 128, 256, 128, 128, 1024)
    assert 0 < lib.ha_static_scratch_needed(small) <= (4 << 20)
    huge = _lib.HaShape(64, 8, 4, 128, 256, 512, 64 * 512, 8192)   # needs far more than 4 MiB
    assert lib.ha_static_scratch_needed(huge) > (4 << 20)
    N = None
    dummy = ctypes.c_void_p(256)  # never dereferenced: the size check comes first
    rc = lib.ha_score_select_static(huge, bud, dummy, dummy, dummy, dummy, dummy, dummy, dummy, N)
    assert rc == _lib.HA_ERR_SCRATCH_LIMIT
    assert "built-in buffer" in _lib.status_str(rc)
    assert lib.ha_score_select_static(small, bud, N, N, N, N, N, N, N, N) == _lib.HA_ERR_BAD_ARG


def _compare_static_with_workspace(lib, ctx, cache, q_codes, label):
    """ha_score_select_static against ha_score_select on the same inputs: equal counts, equal sets."""
    ctx.score_select(q_codes)
    want_idx, want_cnt = ctx.sel_idx.clone(), ctx.sel_cnt.clone()
    got_idx = torch.full_like(ctx.sel_idx, -1)
    got_cnt = torch.full_like(ctx.sel_cnt, -1)
    rc = lib.ha_score_select_static(
        ctx.shape, ctx.c_budget, q_codes.data_ptr(), cache.hash_pages.data_ptr(), cache.page_table.data_ptr(),
        cache.seq_lens.data_ptr(), got_idx.data_ptr(), got_cnt.data_ptr(), ctx.status.data_ptr(),
        torch.cuda.current_stream(cache.device).cuda_stream)
    assert rc == _lib.HA_OK, _lib.status_str(rc)
    ctx.check_status()
    assert torch.equal(got_cnt, want_cnt), label
    for b in range(want_cnt.shape[0]):
        for h in range(want_cnt.shape[1]):
            n = int(want_cnt[b, h])
            # the order inside a head's list is not part of the contract (each token once)
            assert torch.equal(got_idx[b, h, :n].sort().values, want_idx[b, h, :n].sort().values), f"{label}: b={b} h={h}"
    return want_idx, want_cnt


def _context(device, lens, Hq, Hkv, budget, seed):
    usa = synthetic.make_usa(Hq, 128, 0, True)
    inp = synthetic.make_decode_inputs(seed, lens, Hq, Hkv)
    cache = ha.PagedHashKVCache(len(lens), Hkv, max(lens), device, shuffle_seed=5)
    for b, S in enumerate(lens):
        cache.write_kv(b, inp.k[b], inp.v[b])
    ctx = ha.SparseDecodeContext(cache, budget, usa.packed(device))
    ctx.hash_prefill()
    return cache, ctx


@pytest.mark.gpu
def test_static_scratch_selection_equals_workspace_selection_on_calls_in_a_row(device):
    """Calls in a row on the one built-in buffer, each finding what the call before left there: the same problem
    twice; then shorter sequences (the tails of the score planes and the histograms of the chunks beyond the new
    lengths are now stale); then another shape and budget, which lays the buffer out differently."""
    Hq, Hkv, lens = 8, 2, [1500, 700, 257]
    cache, ctx = _context(device, lens, Hq, Hkv, ha.Budget(16, 1.0 / 8, 16), 110)
    lib = _lib.load()
    assert lib.ha_static_scratch_needed(ctx.shape) <= (4 << 20)
    gen = torch.Generator(device="cpu").manual_seed(3)

    def codes(batch, heads):
        q = torch.randint(-2 ** 31, 2 ** 31 - 1, (batch, heads), generator=gen, dtype=torch.int64)
        return q.to(torch.int32).to(device)

    for call in range(2):
        q_codes = codes(len(lens), Hq)
        _, cnt = _compare_static_with_workspace(lib, ctx, cache, q_codes, f"call {call}")
        assert int(cnt.min()) > 0
    cache.seq_lens.copy_(torch.tensor([300, 1, 257], dtype=torch.int32))  # shrunk in place
    _, cnt = _compare_static_with_workspace(lib, ctx, cache, codes(len(lens), Hq), "shorter sequences")
    assert cnt[1].tolist() == [0] * Hq and int(cnt[0].min()) > 0
    cache2, ctx2 = _context(device, [5000, 2100], 4, 1, ha.Budget(4, 40.0, 8), 111)   # absolute budget of 40 tokens
    assert lib.ha_static_scratch_needed(ctx2.shape) <= (4 << 20)
    _, cnt2 = _compare_static_with_workspace(lib, ctx2, cache2, codes(2, 4), "another shape")
    assert cnt2.tolist() == [[40] * 4] * 2
    cache.seq_lens.copy_(torch.tensor(lens, dtype=torch.int32))
    q_codes = codes(len(lens), Hq)
    want_idx, want_cnt = _compare_static_with_workspace(lib, ctx, cache, q_codes, "first shape again")
    # the Python wrapper drives the same entry point
    ctx.sel_idx.fill_(-1)
    idx, cnt = ctx.score_select_static(q_codes)
    assert torch.equal(cnt, want_cnt)
    for b in range(len(lens)):
        for h in range(Hq):
            n = int(want_cnt[b, h])
            assert torch.equal(idx[b, h, :n].sort().values, want_idx[b, h, :n].sort().values)
