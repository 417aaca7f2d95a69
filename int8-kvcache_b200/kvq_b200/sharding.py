"""Request sharding of the decode path over the GPUs of one node.

Requests are independent, and so are their pages: rank r owns a subset of the requests together with their
block-table rows and physical pages, runs the single-GPU kernels on them, and no collective is needed inside
attention. Only where a consumer needs every rank's rows (e.g. sampling on one rank) are the outputs gathered.
The reference has no counterpart: it relies on vLLM's tensor parallelism and only slices scale rows
(kvq/scales.py:49-56, see kvq_b200.scales.shard).
"""
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
