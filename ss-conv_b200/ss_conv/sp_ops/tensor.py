"""Sparse voxel tensor (interface of SS_Conv_lib/ss_conv/sp_ops/tensor.py:22-69)."""
import numpy as np
import torch

from .. import _ext


def scatter_nd(indices, updates, shape):
    """Dense tensor of `shape` with updates written at the integer rows of `indices`."""
    ret = torch.zeros(*shape, dtype=updates.dtype, device=updates.device)
    ndim = indices.shape[-1]
    flat = indices.view(-1, ndim)
    ret[tuple(flat[:, i] for i in range(ndim))] = updates.view(-1, *shape[ndim:])
    return ret


class SparseTensor(object):
    """features [N,C] float32, indices [N,4] int32 rows (batch,x,y,z), the dense spatial shape,
    the batch size, and `indice_dict`, the per-key rulebook cache shared along a network:
    key -> (outids, indices, indice_pairs, indice_pair_num, spatial_shape)."""

    def __init__(self, features, indices, spatial_shape, batch_size, grid=None):
        self.features = features
        self.indices = indices if indices.dtype == torch.int32 else indices.int()
        self.spatial_shape = spatial_shape
        self.batch_size = batch_size
        self.indice_dict = {}
        self.grid = grid

    @property
    def spatial_size(self):
        return np.prod(self.spatial_shape)

    def find_indice_pair(self, key):
        if key is None:
            return None
        return self.indice_dict.get(key, None)

    def dense(self, channels_first=True):
        shape = [self.batch_size] + list(self.spatial_shape) + [self.features.shape[1]]
        res = scatter_nd(self.indices.long(), self.features, shape)
        if not channels_first:
            return res
        nd = len(self.spatial_shape)
        return res.permute(0, nd + 1, *range(1, nd + 1)).contiguous()

    def get_offsets(self):
        """Row offsets [B+1] (int32) of the samples, computed on the device without host syncs
        (the reference loops over the batch with .item(), tensor.py:59-65)."""
        if self.indices.is_cuda:
            return _ext.batch_offsets(self.indices, self.batch_size)
        counts = torch.bincount(self.indices[:, 0].long(), minlength=self.batch_size)
        return torch.cat([counts.new_zeros(1), counts.cumsum(0)]).int()

    @property
    def sparity(self):
        return self.indices.shape[0] / np.prod(self.spatial_shape) / self.batch_size
