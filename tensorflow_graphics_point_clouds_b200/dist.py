"""Multi-GPU plumbing: clouds are the unit of parallelism.

Every op of the path is independent per cloud (keys carry the batch id, the
tube structure is per batch, the neighbor search never crosses batches), so a
batch is split by cloud index across ranks, one process per GPU, and the only
exchange is the sum of the weight gradients.  The reference has no multi-GPU
path at all.
"""
import torch
import torch.distributed as dist


def shard_clouds(num_clouds, world_size, rank):
  """Contiguous cloud range [begin, end) of `rank`; sizes differ by at most one."""
  if not 0 <= rank < world_size:
    raise ValueError("rank %d outside world of size %d" % (rank, world_size))
  base, extra = divmod(num_clouds, world_size)
  begin = rank * base + min(rank, extra)
  end = begin + base + (1 if rank < extra else 0)
  return begin, end


def shard_points(batch_ids, begin, end):
  """Boolean mask of the points whose cloud index lies in [begin, end), and the
  batch ids re-based to the shard (cloud `begin` becomes 0)."""
  mask = (batch_ids >= begin) & (batch_ids < end)
  return mask, batch_ids[mask] - begin


def allreduce_sum_(tensors, group=None):
  """Sums a list of tensors over all ranks with ONE collective (they are
  flattened into one buffer: the weight gradients are small, so the cost is
  launch latency, not bandwidth).  In place; returns the list."""
  if not dist.is_available() or not dist.is_initialized() or dist.get_world_size(group) == 1:
    return tensors
  flat = torch.cat([t.reshape(-1) for t in tensors])
  dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group)
  offset = 0
  for t in tensors:
    n = t.numel()
    t.copy_(flat[offset:offset + n].reshape(t.shape))
    offset += n
  return tensors


def allreduce_max_(tensor, group=None):
  """Element-wise maximum of a tensor over all ranks, in place (the cell counts of
  a sharded batch: pc.PointCloud(num_cells_reduce=allreduce_max_))."""
  if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
    dist.all_reduce(tensor, op=dist.ReduceOp.MAX, group=group)
  return tensor


def max_over_ranks(value, device, group=None):
  """Maximum of a Python float over all ranks (timings are reported as the
  slowest rank's)."""
  t = torch.tensor([float(value)], device=device)
  if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
  return float(t.item())
