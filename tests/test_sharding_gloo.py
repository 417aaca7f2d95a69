"""Request sharding over ranks, world size 2 on CPU (gloo): each rank runs the CPU oracle on the requests it
owns, outputs are all-gathered, and the result must equal the unsharded run. This covers the host logic of the
N > 1 path (partition, per-rank metadata, gather order); the kernels themselves are rank-local."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
from conftest import ROOT

from kvq_b200 import sharding, workloads
from oracle import kvq_oracle as orc


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _oracle(case, cu, sl, bt, q):
    st = case["static"]
    return orc.paged_static_attention(q.float().numpy(), case["kq"].numpy(), case["vq"].numpy(), cu.numpy(), sl.numpy(),
                                      bt.numpy(), case["softmax_scale"], st["k_scale"].numpy(), st["v_scale"].numpy())


def _worker(rank, world, port, interleaved, result_path):
    for p in (ROOT, os.path.join(ROOT, "int8-kvcache_b200")):
        sys.path.insert(0, p)
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    case = workloads.paged_case(70, 12, 2, 128, [1, 3, 1, 8, 2], [100, 300, 33, 257, 64])
    n = len(case["q_lens"])
    owned = sharding.shard_requests(n, rank, world, interleaved)
    cu, sl, bt, rows = sharding.shard_batch(case["cu_seqlens_q"], case["seq_lens"], case["block_table"], owned)
    local = torch.from_numpy(_oracle(case, cu, sl, bt, case["q"][rows]))
    rows_per_rank = [sum(case["q_lens"][r] for r in sharding.shard_requests(n, k, world, interleaved)) for k in range(world)]
    full = sharding.gather_outputs(local, rows_per_rank)
    if rank == 0:
        order = [i for k in range(world) for r in sharding.shard_requests(n, k, world, interleaved)
                 for i in range(int(case["cu_seqlens_q"][r]), int(case["cu_seqlens_q"][r + 1]))]
        want = _oracle(case, case["cu_seqlens_q"], case["seq_lens"], case["block_table"], case["q"])[order]
        np.save(result_path, np.abs(full.numpy() - want).max())
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("interleaved", [False, True])
def test_sharded_attention_equals_unsharded(tmp_path, interleaved):
    path = str(tmp_path / "diff.npy")
    mp.spawn(_worker, args=(2, _free_port(), interleaved, path), nprocs=2, join=True)
    assert float(np.load(path)) == 0.0


def test_shard_requests_partitions():
    for n in (0, 1, 5, 128, 131):
        for world in (1, 2, 4, 8):
            for inter in (False, True):
                parts = [sharding.shard_requests(n, r, world, inter) for r in range(world)]
                assert sorted(i for p in parts for i in p) == list(range(n))
                assert max(map(len, parts)) - min(map(len, parts)) <= 1
    with pytest.raises(ValueError):
        sharding.shard_requests(4, 4, 4)
