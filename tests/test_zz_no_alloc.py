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


@pytest.mark.gpu
def test_static_scratch_selection_equals_workspace_selection_on_two_calls_in_a_row(device):
    Hq, Hkv, lens = 8, 2, [1500, 700, 257]
    usa = synthetic.make_usa(Hq, 128, 0, True)
    inp = synthetic.make_decode_inputs(110, lens, Hq, Hkv)
    cache = ha.PagedHashKVCache(len(lens), Hkv, max(lens), device, shuffle_seed=5)
    for b, S in enumerate(lens):
        cache.write_kv(b, inp.k[b], inp.v[b])
    ctx = ha.SparseDecodeContext(cache, ha.Budget(16, 1.0 / 8, 16), usa.packed(device))
    ctx.hash_prefill()
    lib = _lib.load()
    assert lib.ha_static_scratch_needed(ctx.shape) <= (4 << 20)
    gen = torch.Generator(device="cpu").manual_seed(3)
    for call in range(2):  # the second call finds the first call's leftovers in the scratch buffer
        q_codes = torch.randint(-2 ** 31, 2 ** 31 - 1, (len(lens), Hq), generator=gen, dtype=torch.int64)
        q_codes = q_codes.to(torch.int32).to(device)
        ctx.score_select(q_codes)
        want_idx, want_cnt = ctx.sel_idx.clone(), ctx.sel_cnt.clone()
        got_idx = torch.full_like(ctx.sel_idx, -1)
        got_cnt = torch.full_like(ctx.sel_cnt, -1)
        rc = lib.ha_score_select_static(
            ctx.shape, ctx.c_budget, q_codes.data_ptr(), cache.hash_pages.data_ptr(), cache.page_table.data_ptr(),
            cache.seq_lens.data_ptr(), got_idx.data_ptr(), got_cnt.data_ptr(), ctx.status.data_ptr(),
            torch.cuda.current_stream(device).cuda_stream)
        assert rc == _lib.HA_OK, _lib.status_str(rc)
        ctx.check_status()
        assert torch.equal(got_cnt, want_cnt)
        assert int(want_cnt.min()) > 0
        for b in range(len(lens)):
            for h in range(Hq):
                n = int(want_cnt[b, h])
                # the order inside a head's list is not part of the contract (each token once)
                assert torch.equal(got_idx[b, h, :n].sort().values, want_idx[b, h, :n].sort().values), f"call {call}: b={b} h={h}"
    # the Python wrapper drives the same entry point
    ctx.sel_idx.fill_(-1)
    idx, cnt = ctx.score_select_static(q_codes)
    assert torch.equal(cnt, want_cnt)
    for b in range(len(lens)):
        for h in range(Hq):
            n = int(want_cnt[b, h])
            assert torch.equal(idx[b, h, :n].sort().values, want_idx[b, h, :n].sort().values)
