"""Request sharding of the decode path over the GPUs of one node.

Requests are independent, and so are their pages: rank r owns a subset of the requests together with their
block-table rows and physical pages, runs the single-GPU kernels on them, and no collective is needed inside
attention. Only where a consumer needs every rank's rows (e.g. sampling on one rank) are the outputs gathered.
The reference has no counterpart: it relies on vLLM's tensor parallelism and only slices scale rows
(kvq/scales.py:49-56, see kvq_b200.scales.shard).
"""
import ctypes
import os

import torch
import torch.distributed as dist


def shard_requests(num_requests, rank, world_size, interleaved=False):
    """Indices of the requests rank `rank` owns. Contiguous ranges by default (sizes differ by at most one);
    interleaved=True gives r, r + world, r + 2 * world, ... which balances sorted-by-length batches."""
    if not 0 <= rank < world_size:
        raise ValueError(f"rank {rank} outside [0, {world_size})")
    if interleaved:
        return list(range(rank, num_requests, world_size))
    base, extra = divmod(num_requests, world_size)
    start = rank * base + min(rank, extra)
    return list(range(start, start + base + (1 if rank < extra else 0)))


def shard_batch(cu_seqlens_q, seq_lens, block_table, owned):
    """Metadata of the owned requests only: (cu_seqlens_q, seq_lens, block_table, query_rows) where query_rows are
    the rows of the global q/out tensors that belong to this rank, in order."""
    cu = cu_seqlens_q.tolist()
    q_lens = [cu[r + 1] - cu[r] for r in owned]
    rows = [i for r in owned for i in range(cu[r], cu[r + 1])]
    new_cu = torch.zeros(len(owned) + 1, dtype=cu_seqlens_q.dtype)
    if owned:
        new_cu[1:] = torch.cumsum(torch.tensor(q_lens, dtype=cu_seqlens_q.dtype), 0)
    idx = torch.tensor(owned, dtype=torch.long)
    return new_cu, seq_lens[idx], block_table[idx], torch.tensor(rows, dtype=torch.long)


def gather_outputs(local_out, rows_per_rank, group=None, out=None):
    """All-gather of per-rank output rows [T_r, Hq, D] into rank order [sum T_r, Hq, D]. rows_per_rank lists T_r for
    every rank (known to all ranks from the sharding rule). Equal shards go through one all_gather_into_tensor
    straight into `out` (allocated here when not given: pass a persistent buffer to keep the step allocation-free);
    ragged shards are padded to the largest and trimmed after the gather."""
    world = dist.get_world_size(group)
    if len(rows_per_rank) != world or local_out.shape[0] != rows_per_rank[dist.get_rank(group)]:
        raise ValueError(f"rows_per_rank {rows_per_rank} does not describe this group (world {world}, local rows "
                         f"{local_out.shape[0]})")
    total = sum(rows_per_rank)
    if out is None:
        out = local_out.new_empty((total,) + tuple(local_out.shape[1:]))
    elif out.shape[0] != total or out.shape[1:] != local_out.shape[1:] or not out.is_contiguous():
        raise ValueError("out must be a contiguous [sum(rows_per_rank), ...] tensor")
    if len(set(rows_per_rank)) == 1 and local_out.is_contiguous():
        dist.all_gather_into_tensor(out, local_out, group=group)
        return out
    t_max = max(rows_per_rank)
    padded = local_out.new_zeros((t_max,) + tuple(local_out.shape[1:]))
    padded[:local_out.shape[0]] = local_out
    parts = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(parts, padded, group=group)
    torch.cat([p[:n] for p, n in zip(parts, rows_per_rank)], dim=0, out=out)
    return out


class PeerGather:
    """The output all-gather as direct stores into every peer's memory over NVLink (kvq_peer_allgather), for equal
    shards on the GPUs of one node: the rows cross NVLink once, with one flag round trip, in one launch of this
    library's own kernel instead of a library collective.

    Construction is a collective over `group` (NCCL): it allocates two staging buffers and a flag array in symmetric
    memory (torch.distributed._symmetric_memory: every rank gets a mapping of every peer's copy; NVLink multicast is not
    bound, the kernel uses plain peer stores) and raises RuntimeError where that is not available, in which case
    gather_outputs (NCCL) is the route. gather() must be called by every rank, the same number of times; it returns
    `self.out`, the [world * rows, ...] result at a fixed address, complete in stream order. The step counter lives on
    the device, so a CUDA graph that captured gather() can be replayed (by every rank alike)."""

    def __init__(self, rows_per_rank, row_shape, dtype, device, group=None):
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")   # before the first symmetric allocation
        import torch.distributed._symmetric_memory as symm_mem

        from kvq_b200 import _native

        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        if self.world > 8:
            raise RuntimeError("PeerGather serves the GPUs of one node (at most 8 ranks)")
        self.rows, self.row_shape, self.dtype = int(rows_per_rank), tuple(row_shape), dtype
        row_elems = 1
        for d in self.row_shape:
            row_elems *= d
        self.bytes_per_rank = self.rows * row_elems * torch.empty(0, dtype=dtype).element_size()
        if self.bytes_per_rank % 16:
            raise RuntimeError(f"PeerGather: {self.bytes_per_rank} bytes per rank is not a multiple of 16")
        self.lib, self._check = _native.lib(), _native.check
        device = torch.device(device)
        full_shape = (self.world * self.rows,) + self.row_shape
        self.stage = [symm_mem.empty(full_shape, dtype=dtype, device=device) for _ in range(2)]
        self.flags = symm_mem.empty(64, dtype=torch.int32, device=device)
        self.flags.zero_()
        handles = [symm_mem.rendezvous(t, self.group) for t in self.stage]
        flag_handle = symm_mem.rendezvous(self.flags, self.group)
        self._handles = handles + [flag_handle]   # the mappings live as long as this object
        ptrs = ctypes.c_void_p * self.world
        self._stage_ptrs = [ptrs(*[int(p) for p in h.buffer_ptrs]) for h in handles]
        self._flag_ptrs = ptrs(*[int(p) for p in flag_handle.buffer_ptrs])
        self.out = torch.empty(full_shape, dtype=dtype, device=device)
        self.counters = torch.zeros(2, dtype=torch.int32, device=device)   # completed steps, finished blocks
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        torch.cuda.synchronize(device)
        dist.barrier(group=self.group)   # every rank's flags are zero before anyone signals

    def gather(self, local_out):
        """Store this rank's rows [rows, ...] into every rank's staging buffer of this step, wait (on the device,
        bounded) for everyone else's and collect them in `self.out`, which is returned. Asynchronous on the current
        stream; capturable."""
        if tuple(local_out.shape) != (self.rows,) + self.row_shape or local_out.dtype != self.dtype or \
                not local_out.is_contiguous():
            raise ValueError(f"PeerGather.gather: expected a contiguous {(self.rows,) + self.row_shape} {self.dtype} tensor")
        self._check(self.lib.kvq_peer_allgather(local_out.data_ptr(), self.bytes_per_rank, self._stage_ptrs[0],
                                                self._stage_ptrs[1], self._flag_ptrs, self.out.data_ptr(), self.world,
                                                self.rank, self.counters.data_ptr(), self.status.data_ptr(),
                                                torch.cuda.current_stream(local_out.device).cuda_stream))
        return self.out

    def check(self):
        """Synchronizes and raises if a wait for a peer ran out since the last check (a rank that never arrived)."""
        if int(self.status.item()) != 0:
            self.status.zero_()
            raise RuntimeError("PeerGather: a peer's rows did not arrive within the wait limit")
