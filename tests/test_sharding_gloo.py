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


def _gather_worker(rank, world, port, backend, result_path):
    """Equal shards into a persistent output buffer (the single-collective path) and ragged shards, on `backend`."""
    sys.path.insert(0, os.path.join(ROOT, "int8-kvcache_b200"))
    if backend == "nccl":
        torch.cuda.set_device(rank)
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    dev = torch.device("cuda", rank) if backend == "nccl" else torch.device("cpu")
    dist.init_process_group(backend, init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    ok = True
    for rows in ([3] * world, [2 + k for k in range(world)]):
        gen = torch.Generator().manual_seed(5)
        full = torch.randn(sum(rows), 4, 8, generator=gen).to(torch.bfloat16)
        start = sum(rows[:rank])
        local = full[start:start + rows[rank]].to(dev).contiguous()
        out = torch.full((sum(rows), 4, 8), 7.0, dtype=torch.bfloat16, device=dev)
        got = sharding.gather_outputs(local, rows, out=out)
        ok = ok and got.data_ptr() == out.data_ptr() and torch.equal(out.cpu(), full)
        ok = ok and torch.equal(sharding.gather_outputs(local, rows).cpu(), full)
    try:
        sharding.gather_outputs(local, [1] * world)
        ok = False
    except ValueError:
        pass
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        np.save(result_path, int(flag.item()))
    dist.destroy_process_group()


def test_gather_outputs_gloo(tmp_path):
    path = str(tmp_path / "ok.npy")
    mp.spawn(_gather_worker, args=(2, _free_port(), "gloo", path), nprocs=2, join=True)
    assert int(np.load(path)) == 1


@pytest.mark.gpu
def test_gather_outputs_nccl(tmp_path):
    """The same gather over NCCL between two GPUs of the node (skipped on a single-GPU box)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    path = str(tmp_path / "ok.npy")
    mp.spawn(_gather_worker, args=(2, _free_port(), "nccl", path), nprocs=2, join=True)
    assert int(np.load(path)) == 1


def _peer_gather_worker(rank, world, port, result_path):
    torch.cuda.set_device(rank)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world, device_id=dev)
    ok = True
    rows, shape = 24, (28, 128)   # 24 x 28 x 128 bf16 = 172 KB per rank: several slices per peer
    pg = sharding.PeerGather(rows, shape, torch.bfloat16, dev)
    for step in range(5):         # both buffers, several epochs; every step's rows differ
        gen = torch.Generator().manual_seed(100 + step)
        full = torch.randn(world * rows, *shape, generator=gen).to(torch.bfloat16)
        local = full[rank * rows:(rank + 1) * rows].to(dev).contiguous()
        got = pg.gather(local)
        ok = ok and torch.equal(got.cpu(), full)
        # the NCCL route gives the same rows
        ok = ok and torch.equal(sharding.gather_outputs(local, [rows] * world).cpu(), full)
    pg.check()
    # replay from a CUDA graph: the step counter lives on the device
    src = torch.zeros(rows, *shape, dtype=torch.bfloat16, device=dev)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        pg.gather(src)                       # warm-up on the capture stream (both ranks alike)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        res = pg.gather(src)
    for step in range(3):
        gen = torch.Generator().manual_seed(200 + step)
        full = torch.randn(world * rows, *shape, generator=gen).to(torch.bfloat16)
        src.copy_(full[rank * rows:(rank + 1) * rows])
        graph.replay()
        torch.cuda.synchronize()
        ok = ok and torch.equal(res.cpu(), full)
    pg.check()
    try:
        pg.gather(local[:1])
        ok = False
    except ValueError:
        pass
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        np.save(result_path, int(flag.item()))
    dist.barrier()
    del pg
    dist.destroy_process_group()


@pytest.mark.gpu
def test_peer_gather_two_gpus(tmp_path):
    """kvq_peer_allgather between two GPUs of the node: every rank's rows reach both buffers, step after step
    (skipped on a single-GPU box)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    path = str(tmp_path / "ok.npy")
    mp.spawn(_peer_gather_worker, args=(2, _free_port(), path), nprocs=2, join=True)
    assert int(np.load(path)) == 1


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
