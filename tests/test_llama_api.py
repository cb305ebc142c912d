"""The reference's Llama-facing API (load_usa / convert_usa / reset_usa / LlamaAttention_heavy_hitter)
on a tiny randomly initialised Llama: structure on CPU, numerics on the GPU against the oracle."""
import pytest
import torch
from transformers import LlamaConfig, LlamaForCausalLM

from hashattention_b200 import hashattention_llama as hal
from hashattention_b200.usa import USA
from oracle import hashattn_oracle as orc


def tiny_config(layers=2):
    cfg = LlamaConfig(hidden_size=512, num_attention_heads=4, num_key_value_heads=1, num_hidden_layers=layers,
                      intermediate_size=1024, vocab_size=1000, max_position_embeddings=2048,
                      rope_parameters={"rope_theta": 500000.0, "rope_type": "default"})
    for k, v in dict(lth_init_dim=128, lth_final_dim=32, lth_thold=0, lth_num_layers=3, init_budget=16,
                     heavy_budget=0.125, recent_budget=16, usa_eval_mode="simple", usa_retrieve_depth=-1).items():
        setattr(cfg, k, v)
    return cfg


def test_load_usa_builds_one_module_per_layer_and_loads_reference_state_dicts(tmp_path):
    cfg = tiny_config(3)
    mods = hal.load_usa(cfg, None, device="cpu")
    assert len(mods) == 3 and all(isinstance(m, USA) for m in mods)
    keys = list(mods.state_dict())
    assert keys[0] == "0.learning_to_hash_transformation_k.0.0.weight" and len(keys) == 3 * 2 * 4 * 6
    path = tmp_path / "patch.pt"
    torch.save(mods.state_dict(), path)
    again = hal.load_usa(cfg, str(path), device="cpu")
    for a, b in zip(mods.state_dict().values(), again.state_dict().values()):
        assert torch.equal(a, b)
    cfg.lth_num_layers = 2     # Linear-SiLU-Linear (hashattention_llama.py:112-120): reference keys 0 and 2
    two = hal.load_usa(cfg, None, device="cpu")
    assert [k for k in two.state_dict() if k.startswith("0.learning_to_hash_transformation_k.0.")] == [
        "0.learning_to_hash_transformation_k.0.0.weight", "0.learning_to_hash_transformation_k.0.0.bias",
        "0.learning_to_hash_transformation_k.0.2.weight", "0.learning_to_hash_transformation_k.0.2.bias"]
    packed = two[0].packed("cpu")
    assert packed.num_layers == 2 and packed.wk.shape == (4, 36864) and float(packed.wk[:, 16384:32768].abs().max()) == 0.0
    cfg.lth_num_layers = 0     # the LSH baseline: one shared Linear(129, 32) per head
    lsh = hal.load_usa(cfg, None, device="cpu")
    assert lsh[0].packed("cpu").lsh and lsh[0].learning_to_hash_transformation[0][1].weight.shape == (32, 129)
    cfg.lth_num_layers = 4     # not a configuration of the reference
    with pytest.raises(NotImplementedError):
        hal.load_usa(cfg, None, device="cpu")


def test_convert_usa_swaps_attention_and_keeps_weights():
    cfg = tiny_config(2)
    torch.manual_seed(0)
    model = LlamaForCausalLM(cfg)
    before = {n: p.clone() for n, p in model.named_parameters() if "self_attn" in n}
    mods = hal.load_usa(cfg, None, device="cpu")
    model = hal.convert_usa(model, cfg, mods, collect_stats=False, train_usa=False)
    for i, layer in enumerate(model.model.layers):
        att = layer.self_attn
        assert isinstance(att, hal.LlamaAttention_heavy_hitter)
        assert att.layer_idx == i and att.usa_module is mods[i] and att.flash_forward is not None
        assert att.q_proj.weight.dtype == torch.bfloat16
        assert (att.init_budget, att.heavy_budget, att.recent_budget) == (16, 0.125, 16)
    for n, p in before.items():
        got = dict(model.named_parameters())[n]
        assert torch.equal(got, p.to(torch.bfloat16))
    assert hal.reset_usa(model) is model
    with pytest.raises(NotImplementedError):
        hal.convert_usa(LlamaForCausalLM(cfg), cfg, mods, collect_stats=True, train_usa=False)


def test_training_and_statistics_entry_points_exist_and_refuse():
    for fn in (hal.set_train_usa_mode, hal.print_stats):
        with pytest.raises(NotImplementedError):
            fn(torch.nn.Linear(2, 2))


def test_unsupported_modes_raise():
    cfg = tiny_config(1)
    cfg.usa_eval_mode, cfg.usa_retrieve_depth = "depth", 3   # the depth rule is supported
    att = hal.LlamaAttention_heavy_hitter(cfg, 0)
    assert (att.usa_eval_mode, att.usa_retrieve_depth) == ("depth", 3)
    cfg = tiny_config(1)
    cfg.num_key_value_heads = 2
    with pytest.raises(NotImplementedError):
        hal.LlamaAttention_heavy_hitter(cfg, 0)


@pytest.mark.gpu
def test_converted_model_prefill_then_decode_matches_oracle(device):
    cfg = tiny_config(2)
    torch.manual_seed(1)
    model = LlamaForCausalLM(cfg).to(torch.bfloat16).to(device).eval()
    mods = hal.load_usa(cfg, None, device=device).bfloat16()
    model = hal.convert_usa(model, cfg, mods, collect_stats=False, train_usa=False)
    att = model.model.layers[0].self_attn
    seen = {}
    att.register_forward_hook(lambda m, args, kwargs, out: seen.update(args=args, kwargs=kwargs, out=out),
                              with_kwargs=True)

    g = torch.Generator().manual_seed(5)
    prompt = torch.randint(0, 1000, (2, 300), generator=g).to(device)
    with torch.no_grad():
        out = model(prompt, use_cache=True)
        cache = out.past_key_values
        nxt = torch.randint(0, 1000, (2, 1), generator=g).to(device)
        out2 = model(nxt, past_key_values=cache, use_cache=True)
    assert bool(torch.isfinite(out2.logits.float()).all())
    att._ctx.check_status()
    assert att._ctx.cache.seq_lens.tolist() == [301, 301]

    # layer 0 of the decode step, recomputed with the oracle from what the module was given
    hs = seen["kwargs"]["hidden_states"] if "hidden_states" in seen["kwargs"] else seen["args"][0]
    cos, sin = seen["kwargs"]["position_embeddings"]
    with torch.no_grad():
        q = att.q_proj(hs).view(2, 1, 4, 128).transpose(1, 2)
        k = att.k_proj(hs).view(2, 1, 1, 128).transpose(1, 2)
        q, k = hal._apply_rotary(q, k, cos, sin)
    kc, vc = hal._layer_kv(cache, 0)  # includes the new token
    assert kc.shape[2] == 301
    assert torch.equal(kc[:, :, -1:].to(torch.bfloat16), k.to(torch.bfloat16))
    ref = orc.decode_step(mods[0].float().cpu(), q[:, :, 0].float().cpu(), kc.float().cpu(), vc.float().cpu(),
                          cfg.init_budget, cfg.recent_budget, cfg.heavy_budget)
    with torch.no_grad():
        want = att.o_proj(ref.reshape(2, 1, 512).to(device, torch.bfloat16)).float().cpu()
    got = seen["out"][0].float().cpu()
    assert float((got - want).abs().max()) < 3e-2 and float((got - want).norm() / want.norm()) < 2e-2

    # a chunk of 4 tokens (2 <= q_len <= 128) goes through the same library path, one row per token
    with torch.no_grad():
        chunk = torch.randint(0, 1000, (2, 4), generator=g).to(device)
        out3 = model(chunk, past_key_values=cache, use_cache=True)
    assert bool(torch.isfinite(out3.logits.float()).all())
    assert att._ctx.cache.seq_lens.tolist() == [305, 305]
    hs = seen["kwargs"]["hidden_states"] if "hidden_states" in seen["kwargs"] else seen["args"][0]
    cos, sin = seen["kwargs"]["position_embeddings"]
    with torch.no_grad():
        q = att.q_proj(hs).view(2, 4, 4, 128).transpose(1, 2)
        k = att.k_proj(hs).view(2, 4, 1, 128).transpose(1, 2)
        q, k = hal._apply_rotary(q, k, cos, sin)
    kc, vc = hal._layer_kv(cache, 0)
    assert kc.shape[2] == 305
    ref = orc.decode_chunk(mods[0].float().cpu(), q.to(torch.bfloat16).float().cpu(), kc.float().cpu(), vc.float().cpu(),
                           cfg.init_budget, cfg.recent_budget, cfg.heavy_budget)
    with torch.no_grad():
        want = att.o_proj(ref.transpose(1, 2).reshape(2, 4, 512).to(device, torch.bfloat16)).float().cpu()
    got = seen["out"][0].float().cpu()
    assert float((got - want).abs().max()) < 3e-2 and float((got - want).norm() / want.norm()) < 2e-2
    for ctx_rows in att._ctx.row_contexts.values():
        ctx_rows.check_status()

    # a second prompt after reset_usa starts from an empty hash cache
    hal.reset_usa(model)
    assert att._ctx.cache.seq_lens.tolist() == [0, 0]
    with torch.no_grad():
        model(prompt[:, :200], use_cache=True)
    assert att._ctx.cache.seq_lens.tolist() == [200, 200]


def test_mistral_host_converts_and_resets_like_the_llama_host():
    """hashattention_mistral mirrors the reference's second host file: same API names, MistralAttention
    modules swapped for MistralAttention_heavy_hitter with the projection weights kept."""
    from transformers import MistralConfig, MistralForCausalLM

    from hashattention_b200 import hashattention_mistral as ham

    cfg = MistralConfig(hidden_size=512, num_attention_heads=4, num_key_value_heads=1, num_hidden_layers=2,
                        intermediate_size=1024, vocab_size=1000, max_position_embeddings=2048, head_dim=128,
                        sliding_window=None)
    for k, v in dict(lth_init_dim=128, lth_final_dim=32, lth_thold=0, lth_num_layers=3, init_budget=16,
                     heavy_budget=0.125, recent_budget=16, usa_eval_mode="simple", usa_retrieve_depth=-1).items():
        setattr(cfg, k, v)
    torch.manual_seed(0)
    model = MistralForCausalLM(cfg)
    before = {n: p.clone() for n, p in model.named_parameters() if "self_attn" in n}
    mods = ham.load_usa(cfg, None, device="cpu")
    model = ham.convert_usa(model, cfg, mods, collect_stats=False, train_usa=False)
    for i, layer in enumerate(model.model.layers):
        att = layer.self_attn
        assert isinstance(att, ham.MistralAttention_heavy_hitter) and att.usa_module is mods[i]
        assert att.flash_forward is not None and att.layer_idx == i
    for n, p in before.items():
        assert torch.equal(dict(model.named_parameters())[n], p.to(torch.bfloat16))
    assert ham.reset_usa(model) is model and ham.set_eval_usa_mode(model) is model


@pytest.mark.gpu
def test_cache_room_is_checked_on_the_host_and_padded_batches_are_refused(device):
    """The module tracks the cached length on the host: a step that would not fit the paged cache raises before
    anything is launched (the kernels would only report it and leave `out` unwritten), and a prefill whose
    attention mask hides keys (a padded batch) is refused instead of attending the pad tokens."""
    cfg = tiny_config(1)
    cfg.usa_decode_headroom = 2
    torch.manual_seed(1)
    model = LlamaForCausalLM(cfg).to(torch.bfloat16).to(device).eval()
    mods = hal.load_usa(cfg, None, device=device).bfloat16()
    model = hal.convert_usa(model, cfg, mods, collect_stats=False, train_usa=False)
    att = model.model.layers[0].self_attn
    g = torch.Generator().manual_seed(6)
    prompt = torch.randint(0, 1000, (2, 254), generator=g).to(device)
    with torch.no_grad():
        cache = model(prompt, use_cache=True).past_key_values
        room = att._ctx.cache.max_pages * 256
        assert room == 256  # 254 + 2 of headroom, one page
        for _ in range(2):
            out = model(torch.randint(0, 1000, (2, 1), generator=g).to(device), past_key_values=cache, use_cache=True)
            assert bool(torch.isfinite(out.logits.float()).all())
        with pytest.raises(ValueError, match="usa_decode_headroom"):
            model(torch.randint(0, 1000, (2, 1), generator=g).to(device), past_key_values=cache, use_cache=True)
    att._ctx.check_status()  # nothing was launched for the refused step
    assert att._ctx.cache.seq_lens.tolist() == [256, 256]

    hal.reset_usa(model)
    mask = torch.ones(2, 200, dtype=torch.long, device=device)
    mask[1, :7] = 0  # left padding of the second prompt
    with torch.no_grad(), pytest.raises(NotImplementedError, match="padded"):
        model(prompt[:, :200], attention_mask=mask, use_cache=True)


@pytest.mark.gpu
def test_mistral_model_prefill_then_decode_on_the_gpu(device):
    from transformers import MistralConfig, MistralForCausalLM

    from hashattention_b200 import hashattention_mistral as ham

    cfg = MistralConfig(hidden_size=512, num_attention_heads=4, num_key_value_heads=1, num_hidden_layers=2,
                        intermediate_size=1024, vocab_size=1000, max_position_embeddings=2048, head_dim=128,
                        sliding_window=None)
    for k, v in dict(lth_init_dim=128, lth_final_dim=32, lth_thold=0, lth_num_layers=3, init_budget=16,
                     heavy_budget=0.125, recent_budget=16, usa_eval_mode="simple", usa_retrieve_depth=-1).items():
        setattr(cfg, k, v)
    torch.manual_seed(1)
    model = MistralForCausalLM(cfg).to(device).bfloat16()
    mods = ham.load_usa(cfg, None, device=device).bfloat16()
    model = ham.convert_usa(model, cfg, mods, collect_stats=False, train_usa=False)
    g = torch.Generator().manual_seed(6)
    prompt = torch.randint(0, 1000, (2, 300), generator=g).to(device)
    with torch.no_grad():
        out = model(prompt, use_cache=True)
        nxt = torch.randint(0, 1000, (2, 1), generator=g).to(device)
        out2 = model(nxt, past_key_values=out.past_key_values, use_cache=True)
    att = model.model.layers[0].self_attn
    att._ctx.check_status()
    assert att._ctx.cache.seq_lens.tolist() == [301, 301]
    assert bool(torch.isfinite(out2.logits.float()).all())
