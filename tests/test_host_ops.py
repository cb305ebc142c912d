"""ha_rope_split (the host-model helper that splits a fused q|k|v projection and applies the rotary embedding)
against the plain torch formula, and the tensor-parallel host's decode step against its own torch path."""
import pytest
import torch

import hashattention_b200 as ha
from hashattention_b200 import llama_tp, ops


@pytest.mark.gpu
def test_rope_split_matches_the_torch_formula(device):
    B, hq, hkv = 3, 8, 2
    g = torch.Generator().manual_seed(4)
    qkv = torch.randn(B, (hq + 2 * hkv) * 128, generator=g).to(torch.bfloat16).to(device)
    pos = torch.tensor([0, 777, 33000], dtype=torch.int64, device=device)
    q, k, v = ops.rope_split(qkv, pos, hq, hkv, 500000.0)
    heads = qkv.view(B, hq + 2 * hkv, 128)
    want_q = llama_tp.rope(heads[:, None, :hq].float(), pos[:, None], 500000.0)[:, 0]
    want_k = llama_tp.rope(heads[:, None, hq:hq + hkv].float(), pos[:, None], 500000.0)[:, 0]
    assert torch.equal(v, heads[:, hq + hkv:])
    # bf16 outputs of fp32 arithmetic; the angle of position 33000 is exact to ~1e-3 rad in fp32 on both sides
    assert float((q.float() - want_q).abs().max()) < 3e-2 and float((k.float() - want_k).abs().max()) < 3e-2
    assert float((q.float() - want_q).norm() / want_q.norm()) < 5e-3


@pytest.mark.gpu
def test_tensor_parallel_host_runs_prefill_and_graph_captured_decode_on_one_gpu(device):
    """One rank (world 1) of the tensor-parallel Llama host with 2 layers: prefill, then decode steps eagerly and
    as a CUDA graph replay; the kernels report no problem and the lengths advance on the device."""
    cfg = llama_tp.LlamaTPConfig(n_layers=2, dim=256, ffn_dim=512, vocab_size=1000, max_seq_len=700)
    model = llama_tp.TPLlama(cfg, 1, 0, device, batch=2, seed=1)
    tokens = llama_tp.tokens_for(cfg, 2, 600, seed=3).to(device)
    cur = model.prefill(tokens)
    nxt = torch.empty_like(cur)
    model.decode_step(cur, nxt)
    cur.copy_(nxt)
    torch.cuda.synchronize()
    graph, side = torch.cuda.CUDAGraph(), torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            model.decode_step(cur, nxt)
            cur.copy_(nxt)
    torch.cuda.current_stream().wait_stream(side)
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    model.check_status()
    assert model.seq_lens.tolist() == [604, 604] and model.pos.tolist() == [604, 604]
    assert bool(((cur >= 0) & (cur < cfg.vocab_size)).all())
