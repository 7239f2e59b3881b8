"""Sample-parallel inference across the GPUs of one node.

The sparse samples of a batch are independent (every rulebook, pooling and interpolation
kernel keys on the batch index), so a batch is split into contiguous sample ranges, one per
rank; each rank runs the whole network on its shard and the only exchange is one all-gather
of the pooled per-sample feature rows.  The reference has no multi-GPU code.
"""
import torch
import torch.distributed as dist


def shard_range(n_samples, rank, world_size):
    """[lo, hi) sample range of `rank`: contiguous, sizes differ by at most one."""
    base, extra = divmod(int(n_samples), int(world_size))
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def shard_points(points, feats, batch_ids, n_samples, rank, world_size):
    """Rows of a point batch that belong to this rank, with batch ids re-based to start at 0."""
    lo, hi = shard_range(n_samples, rank, world_size)
    keep = (batch_ids >= lo) & (batch_ids < hi)
    return points[keep], feats[keep], batch_ids[keep] - lo, hi - lo


def shard_sparse(features, indices, n_samples, rank, world_size):
    lo, hi = shard_range(n_samples, rank, world_size)
    keep = (indices[:, 0] >= lo) & (indices[:, 0] < hi)
    idx = indices[keep].clone()
    idx[:, 0] -= lo
    return features[keep], idx, hi - lo


def all_gather_rows(local_rows, n_samples, group=None):
    """[n_local, C] per rank -> [n_samples, C] on every rank, in sample order.  Ragged shards
    are padded to the largest shard for the collective and trimmed afterwards."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return local_rows
    world = dist.get_world_size(group)
    sizes = [shard_range(n_samples, r, world)[1] - shard_range(n_samples, r, world)[0] for r in range(world)]
    if local_rows.shape[0] != sizes[dist.get_rank(group)]:
        raise ValueError("rank %d holds %d rows, expected %d" % (dist.get_rank(group), local_rows.shape[0],
                                                              sizes[dist.get_rank(group)]))
    width = max(sizes)
    padded = local_rows.new_zeros((width, local_rows.shape[1]))
    padded[:local_rows.shape[0]] = local_rows
    gathered = local_rows.new_empty((world * width, local_rows.shape[1]))
    dist.all_gather_into_tensor(gathered, padded, group=group)
    parts = [gathered[r * width:r * width + sizes[r]] for r in range(world)]
    return torch.cat(parts, dim=0)


class RowGatherer(object):
    """all_gather_rows for a loop: the padded send buffer and the gathered receive buffer are
    allocated once, and with equal shards (n_samples divisible by the world size) the local rows
    are sent as they are and the receive buffer IS the result (no padding copy, no concatenation).
    The returned tensor is overwritten by the next call."""

    def __init__(self, n_samples, channels, device, dtype=torch.float32, group=None):
        self.n, self.group = int(n_samples), group
        self.on = dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1
        if not self.on:
            return
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.sizes = [shard_range(self.n, r, self.world)[1] - shard_range(self.n, r, self.world)[0]
                      for r in range(self.world)]
        self.width = max(self.sizes)
        self.even = min(self.sizes) == self.width
        self.gathered = torch.empty((self.world * self.width, int(channels)), dtype=dtype, device=device)
        self.padded = None if self.even else torch.zeros((self.width, int(channels)), dtype=dtype, device=device)

    def __call__(self, local_rows):
        if not self.on:
            return local_rows
        if local_rows.shape[0] != self.sizes[self.rank]:
            raise ValueError("rank %d holds %d rows, expected %d" % (self.rank, local_rows.shape[0], self.sizes[self.rank]))
        if self.even:
            dist.all_gather_into_tensor(self.gathered, local_rows.contiguous(), group=self.group)
            return self.gathered
        self.padded[:local_rows.shape[0]].copy_(local_rows)
        dist.all_gather_into_tensor(self.gathered, self.padded, group=self.group)
        return torch.cat([self.gathered[r * self.width:r * self.width + self.sizes[r]] for r in range(self.world)], dim=0)
