"""Host-side logic that needs no GPU: the USA parameter mirror, weight packing, budgets, the
paged cache bookkeeping (on CPU tensors) and the synthetic input generators."""
import pytest
import torch

import hashattention_b200 as ha
from hashattention_b200 import synthetic
from hashattention_b200.cache import PagedHashKVCache
from oracle import hashattn_oracle as orc


def test_usa_state_dict_layout():
    usa = ha.USA(8, 128, {"lth_int_dim": 128, "lth_final_dim": 32, "lth_thold": 0, "lth_num_layers": 3})
    keys = list(usa.state_dict())
    assert len(keys) == 2 * 8 * 3 * 2
    assert keys[0] == "learning_to_hash_transformation_k.0.0.weight"
    assert "learning_to_hash_transformation_q.7.4.bias" in keys
    assert usa.state_dict()["learning_to_hash_transformation_k.3.4.weight"].shape == (32, 128)
    per_mlp = sum(p.numel() for p in usa.learning_to_hash_transformation_k[0].parameters())
    assert per_mlp == 37152


@pytest.mark.parametrize("params", [
    {"lth_int_dim": 128, "lth_final_dim": 32, "lth_thold": 0, "lth_num_layers": 4},
    {"lth_int_dim": 64, "lth_final_dim": 32, "lth_thold": 0, "lth_num_layers": 3},
    {"lth_int_dim": 128, "lth_final_dim": 64, "lth_thold": 0, "lth_num_layers": 3},
])
def test_usa_rejects_unimplemented_configurations(params):
    with pytest.raises(NotImplementedError):
        ha.USA(8, 128, params)


def test_lsh_baseline_module_and_packing():
    """lth_num_layers = 0: one Linear(129, 32) per head under three names (hashattention_llama.py:130-139); packed as
    columns 0..127 in the W2 slot, column 128 in b0[0..31], the bias in b2, the same buffers for both sides."""
    usa = synthetic.make_usa(4, 128, seed=2, bf16=False, num_layers=0)
    keys = list(usa.state_dict())
    assert keys[0] == "learning_to_hash_transformation.0.1.weight"
    assert "learning_to_hash_transformation_k.3.1.bias" in keys and "learning_to_hash_transformation_q.3.1.bias" in keys
    assert usa.learning_to_hash_transformation_k is usa.learning_to_hash_transformation_q
    lin = usa.learning_to_hash_transformation[1][1]
    assert lin.weight.shape == (32, 129) and abs(float(lin.weight.std()) - 1.0) < 0.1
    p = usa.packed("cpu")
    assert p.lsh and p.wq.shape == (4, 36864) and torch.equal(p.wq, p.wk) and torch.equal(p.bq, p.bk)
    w2 = p.wk[1, 128 * 128 * 2:].reshape(32, 128)
    assert torch.equal(w2, lin.weight[:, :128]) and not bool(p.wk[1, :128 * 128 * 2].any())
    assert torch.equal(p.bk[1, :32], lin.weight[:, 128]) and torch.equal(p.bk[1, 256:], lin.bias)
    with pytest.raises(ValueError):
        p.c_struct()  # the cache's state buffer is required
    state = torch.zeros(2, dtype=torch.int32)
    assert p.c_struct(state).num_layers == ha._lib.HA_HASH_LSH


def test_packing_layout_and_invalidation():
    usa = synthetic.make_usa(4, 128, seed=3, bf16=False)
    p = usa.packed("cpu")
    assert p.dtype_code == ha._lib.HA_WEIGHTS_F32 and p.wq.shape == (4, 36864) and p.bq.shape == (4, 288)
    net = usa.learning_to_hash_transformation_k[2]
    assert torch.equal(p.wk[2, :16384].reshape(128, 128), net[0].weight)
    assert torch.equal(p.wk[2, 16384:32768].reshape(128, 128), net[2].weight)
    assert torch.equal(p.wk[2, 32768:].reshape(32, 128), net[4].weight)
    assert torch.equal(p.bk[2], torch.cat([net[0].bias, net[2].bias, net[4].bias]))
    assert usa.packed("cpu") is p
    usa.load_state_dict(synthetic.make_usa(4, 128, seed=4, bf16=False).state_dict())
    assert usa.packed("cpu") is not p
    b = usa.bfloat16().packed("cpu")
    assert b.dtype_code == ha._lib.HA_WEIGHTS_BF16 and b.wq.dtype == torch.bfloat16 and b.bq.dtype == torch.float32
    s = b.slice_heads(2, 4)
    assert s.wq.shape[0] == 2 and torch.equal(s.wk[0], b.wk[2])


def test_module_list_state_dict_round_trip(tmp_path):
    mods = torch.nn.ModuleList([synthetic.make_usa(4, 128, seed=s, bf16=False) for s in (1, 2)])
    path = tmp_path / "patch.pt"
    torch.save(mods.state_dict(), path)
    assert "1.learning_to_hash_transformation_q.3.2.weight" in mods.state_dict()
    fresh = torch.nn.ModuleList([synthetic.make_usa(4, 128, seed=9, bf16=False) for _ in range(2)])
    fresh[0].packed("cpu")
    fresh.load_state_dict(torch.load(path))
    assert fresh[0]._packed is None
    assert torch.equal(fresh[1].packed("cpu").wq, mods[1].packed("cpu").wq)


def test_budget_matches_reference_arithmetic():
    for S in (1, 100, 4095, 4096, 32768, 131072, 50001):
        for hb in (0.0, 1 / 32, 1 / 16, 0.1, 0.25, 1.0, 1.5, 48.0, 4096.0):
            assert ha.Budget(128, hb, 128).heavy_tokens(S) == orc.heavy_tokens(S, hb)
    assert ha.Budget(128, 0.1, 128).heavy_tokens(50001) == int(50001 * 0.1)


def test_paged_cache_round_trip_on_cpu():
    cache = PagedHashKVCache(3, 2, 700, "cpu", shuffle_seed=5)
    assert cache.max_pages == 3 and cache.num_pages == 9
    assert sorted(cache.page_table.flatten().tolist()) == list(range(9))
    g = torch.Generator().manual_seed(0)
    for b, S in enumerate((700, 256, 1)):
        k = torch.randn(2, S, 128, generator=g).bfloat16()
        v = torch.randn(2, S, 128, generator=g).bfloat16()
        codes = torch.randint(0, 2 ** 32, (8, S), generator=g, dtype=torch.int64)
        cache.write_kv(b, k, v)
        cache.write_codes(b, codes)
        k2, v2 = cache.read_kv(b)
        assert torch.equal(k2, k) and torch.equal(v2, v)
        assert torch.equal(cache.read_codes(b), codes)
    assert cache.seq_lens.tolist() == [700, 256, 1]
    with pytest.raises(ValueError):
        cache.write_kv(0, torch.zeros(2, 800, 128), torch.zeros(2, 800, 128))
    cache.reset()
    assert cache.seq_lens.tolist() == [0, 0, 0]


def test_synthetic_inputs_are_deterministic_and_shaped():
    a = synthetic.make_decode_inputs(1, [300, 300], 8, 2)
    b = synthetic.make_decode_inputs(1, [300, 300], 8, 2)
    assert a.digest() == b.digest() and a.q.shape == (2, 8, 128) and a.k[1].shape == (2, 300, 128)
    assert torch.equal(a.q, a.q.bfloat16().float())
    # outlier channels carry ~8x the energy of the others before RoPE mixes pairs (c, c +- 64)
    energy = a.k[0].pow(2).mean(dim=(0, 1))
    touched = {c for ch in synthetic.OUTLIER_CHANNELS for c in (ch, (ch + 64) % 128)}
    others = [c for c in range(128) if c not in touched]
    assert energy[list(synthetic.OUTLIER_CHANNELS)].min() > 4 * energy[others].max()
    r = synthetic.make_decode_inputs(2, [100, 200, 150], 8, 2)
    assert [k.shape[1] for k in r.k] == [100, 200, 150]
    lens = synthetic.ragged_lengths(2, 32, 16384, 65536)
    assert len(lens) == 32 and min(lens) >= 16384 and max(lens) <= 65536
    assert lens == synthetic.ragged_lengths(2, 32, 16384, 65536)


def test_planted_keys_have_cosine_0p9():
    inp = synthetic.make_decode_inputs(3, [2000], 8, 2, bf16=False, plant_frac=0.02)
    pos = inp.planted[0]
    assert len(pos) == 40 and int(pos.min()) >= 128 and int(pos.max()) < 2000 - 128
    for j in range(2):
        cos = torch.nn.functional.cosine_similarity(inp.k[0][j, pos], inp.q[0, 4 * j][None], dim=-1)
        assert torch.allclose(cos, torch.full_like(cos, 0.9), atol=1e-4)


def test_rope_is_a_rotation():
    x = torch.randn(2, 50, 128)
    cos, sin = synthetic.rope_tables(torch.arange(50))
    y = synthetic.apply_rope(x, cos, sin)
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), rtol=1e-5)
    assert torch.equal(y[:, 0], x[:, 0])


def test_decode_step_is_a_registered_torch_operator_without_a_cpu_kernel():
    """torch.ops.hashattn.decode_step: schema declares what it mutates, the fake implementation runs
    on meta tensors (what a tracer sees), and CPU tensors are refused - there is no CPU fallback."""
    import hashattention_b200  # noqa: F401  (registers the operator)
    op = torch.ops.hashattn.decode_step.default
    schema = str(op._schema)
    for name in ("k_pages", "v_pages", "hash_pages", "q_codes", "sel_idx", "sel_cnt", "workspace", "status", "out"):
        assert f"Tensor(a" in schema and f") {name}" in schema, name
    for name in ("q", "k_new", "page_table", "seq_lens", "wq"):
        assert f"Tensor {name}" in schema, name

    def args(device):
        bf = dict(dtype=torch.bfloat16, device=device)
        i32 = dict(dtype=torch.int32, device=device)
        return (torch.empty(1, 8, 128, **bf), torch.empty(1, 2, 128, **bf), torch.empty(1, 2, 128, **bf),
                torch.empty(4, 2, 256, 128, **bf), torch.empty(4, 2, 256, 128, **bf), torch.empty(4, 2, 256, 4, **i32),
                torch.zeros(1, 4, **i32), torch.ones(1, **i32),
                torch.empty(8, 36864, **bf), torch.empty(8, 288, dtype=torch.float32, device=device),
                torch.empty(8, 36864, **bf), torch.empty(8, 288, dtype=torch.float32, device=device),
                torch.empty(1, 8, **i32), torch.empty(1, 8, 64, **i32), torch.empty(1, 8, **i32),
                torch.empty(1 << 20, dtype=torch.uint8, device=device), torch.zeros(1, **i32),
                torch.empty(1, 8, 128, **bf), 16, 16, 0.125, 0.0884)

    assert op(*args("meta")) is None
    with pytest.raises(NotImplementedError):
        op(*args("cpu"))


def test_nvtx_switch_is_off_by_default_and_costs_nothing_when_off():
    """ops.set_nvtx: the ranges around the library calls are only opened when switched on."""
    from hashattention_b200 import ops
    assert ops._nvtx_on is False
    with ops._call_range("ha_decode_step") as r:
        assert r.pushed is False
    ha.set_nvtx(True)
    try:
        assert ops._nvtx_on is True
    finally:
        ha.set_nvtx(False)
    assert ops._nvtx_on is False
