"""The tensor-parallel Llama host of the full-model configuration (llama_tp.py) on CPU: two gloo ranks, each
with its share of every sharded matrix and of the kv-heads, must reproduce the unsharded model - prefill and
greedy decode steps, with the all-reduce after attention and after the MLP as the only communication
(efficiency/tp.py:48-134 of the reference). The attention of a decode step is computed by the oracle here
(no GPU); on GPUs it is the library's decode step (bench.py --workload config4)."""
import os
import socket
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _tiny():
    from hashattention_b200 import llama_tp
    return llama_tp.LlamaTPConfig(n_layers=2, dim=64, n_heads=32, n_kv_heads=8, head_dim=128, ffn_dim=128,
                                  vocab_size=512, init_budget=4, heavy_budget=0.25, recent_budget=4, max_seq_len=64)


def _run(world, rank, tokens, steps):
    """Prefill + `steps` greedy steps of this rank's share; returns the token ids generated."""
    from hashattention_b200 import llama_tp, synthetic
    from oracle import hashattn_oracle as orc
    cfg = _tiny()
    hq = cfg.n_heads // world
    usas = [synthetic.make_usa(cfg.n_heads, cfg.head_dim, seed=i, bf16=False) for i in range(cfg.n_layers)]

    def attention(layer, q, k, v):
        class Shard:  # the hash nets of this rank's query heads
            learning_to_hash_transformation_k = usas[layer].learning_to_hash_transformation_k[rank * hq:(rank + 1) * hq]
            learning_to_hash_transformation_q = usas[layer].learning_to_hash_transformation_q[rank * hq:(rank + 1) * hq]
        return orc.decode_step(Shard, q.float(), k.float(), v.float(), cfg.init_budget, cfg.recent_budget, cfg.heavy_budget)

    model = llama_tp.TPLlama(cfg, world, rank, "cpu", tokens.shape[0], seed=3, attention=attention, dtype=torch.float32)
    out = [model.prefill(tokens)]
    for _ in range(steps):
        nxt = torch.empty_like(out[-1])
        model.decode_step(out[-1], nxt)
        out.append(nxt)
    return torch.stack(out)


def _worker(rank, world, port, tmp):
    sys.path.insert(0, ROOT)
    import __graft_entry__ as entry
    entry.load_package()
    from hashattention_b200 import llama_tp
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        tokens = llama_tp.tokens_for(_tiny(), 2, 24, seed=11)
        got = _run(world, rank, tokens, 3)
        if rank == 0:
            torch.save(got, os.path.join(tmp, "sharded.pt"))
    finally:
        dist.destroy_process_group()


def test_two_rank_tensor_parallel_model_generates_the_unsharded_tokens(tmp_path):
    import __graft_entry__ as entry
    entry.load_package()
    from hashattention_b200 import llama_tp
    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    sharded = torch.load(tmp_path / "sharded.pt")
    want = _run(1, 0, llama_tp.tokens_for(_tiny(), 2, 24, seed=11), 3)
    assert sharded.shape == want.shape == (4, 2)
    assert torch.equal(sharded, want), "two tensor-parallel ranks generate other tokens than one"


def test_every_rank_count_holds_the_same_weights():
    import __graft_entry__ as entry
    entry.load_package()
    from hashattention_b200 import llama_tp
    full = llama_tp.sharded_weight("w1", 1, 128, 64, "col", llama_tp.block_range(1, 0), "cpu", 5, torch.float32)
    halves = [llama_tp.sharded_weight("w1", 1, 128, 64, "col", llama_tp.block_range(2, r), "cpu", 5, torch.float32)
              for r in range(2)]
    assert torch.equal(torch.cat(halves, 0), full)
    full = llama_tp.sharded_weight("w2", 1, 64, 128, "row", llama_tp.block_range(1, 0), "cpu", 5, torch.float32)
    eighths = [llama_tp.sharded_weight("w2", 1, 64, 128, "row", llama_tp.block_range(8, r), "cpu", 5, torch.float32)
               for r in range(8)]
    assert torch.equal(torch.cat(eighths, 1), full)
    assert list(llama_tp.block_range(4, 3)) == [6, 7]
