"""Host-side logic of the multi-GPU path with two gloo ranks on CPU: kv-head sharding of a decode
step, the final gather, and that sharded == unsharded bit for bit. The per-shard compute is done by
the oracle here (no GPU in this test); on GPUs the same partition is exercised by
test_kv_head_partition_is_bit_identical and bench.py --gpus N."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, tmp):
    sys.path.insert(0, ROOT)
    import __graft_entry__ as entry
    entry.load_package()
    from hashattention_b200 import partition, synthetic
    from oracle import hashattn_oracle as orc

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        Hq, Hkv = 16, 4
        usa = synthetic.make_usa(Hq, 128, 0, True)
        inp = synthetic.make_decode_inputs(120, [400, 400], Hq, Hkv)
        q, k, v = inp.q, torch.stack(inp.k), torch.stack(inp.v)
        j0, j1 = partition.kv_head_range(Hkv, world, rank)
        q_l, k_new_l, v_new_l = partition.shard_step_inputs(q, k[:, :, -1], v[:, :, -1], world, rank)
        assert q_l.shape == (2, (j1 - j0) * 4, 128) and torch.equal(k_new_l, k[:, j0:j1, -1])

        class Shard:  # the hash nets of this rank's query heads
            learning_to_hash_transformation_k = usa.learning_to_hash_transformation_k[j0 * 4:j1 * 4]
            learning_to_hash_transformation_q = usa.learning_to_hash_transformation_q[j0 * 4:j1 * 4]

        out_l = orc.decode_step(Shard, q_l, k[:, j0:j1], v[:, j0:j1], 16, 16, 0.125)
        full = partition.gather_output(out_l)
        if rank == 0:
            want = orc.decode_step(usa, q, k, v, 16, 16, 0.125)
            assert full.shape == want.shape and torch.equal(full, want), "sharded result differs from unsharded"
            open(os.path.join(tmp, "ok"), "w").write("ok")
    finally:
        dist.destroy_process_group()


def test_two_rank_kv_head_sharding_equals_unsharded(tmp_path):
    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "ok").exists()


def test_partition_arithmetic():
    import __graft_entry__ as entry
    entry.load_package()
    from hashattention_b200 import partition
    assert [partition.kv_head_range(8, 4, r) for r in range(4)] == [(0, 2), (2, 4), (4, 6), (6, 8)]
    assert partition.kv_head_range(8, 8, 7) == (7, 8) and partition.kv_head_range(8, 1, 0) == (0, 8)
    with pytest.raises(ValueError):
        partition.kv_head_range(8, 3, 0)
    with pytest.raises(ValueError):
        partition.kv_head_range(8, 2, 2)
    ranges = [partition.batch_range(10, 4, r) for r in range(4)]
    assert ranges == [(0, 3), (3, 6), (6, 8), (8, 10)]
    assert partition.batch_range(2, 4, 3) == (2, 2)
    t = torch.arange(6.0).reshape(1, 6, 1)
    assert partition.gather_output(t) is t  # no process group: identity
