"""Sparse average / max pooling modules (interface of SS_Conv_lib/ss_conv/sp_ops/pool.py)."""
import torch.nn as nn

from .. import _ext
from .tensor import SparseTensor
from .ops import get_conv_output_size, get_indice_pairs, _per_dim
from .functional import indice_avgpool, indice_maxpool


class _SparsePool(nn.Module):
    _op = None

    def __init__(self, ndim, kernel_size, stride=1, padding=0, dilation=1, subm=False):
        super().__init__()
        self.ndim = ndim
        self.kernel_size = _per_dim(kernel_size, ndim)
        self.stride = _per_dim(stride, ndim)
        self.padding = _per_dim(padding, ndim)
        self.dilation = _per_dim(dilation, ndim)
        self.subm = subm

    def forward(self, input):
        """A fresh (never cached) regular-convolution rulebook, then one pooling launch."""
        assert isinstance(input, SparseTensor)
        shape = input.spatial_shape
        out_shape = shape if self.subm else get_conv_output_size(shape, self.kernel_size, self.stride, self.padding,
                                                                 self.dilation)
        feats = None
        ahead = None if self.subm else _ext.get_indice_pairs_ahead(input.indices, input.batch_size, out_shape, list(shape),
                                                                   self.kernel_size, self.stride, self.padding,
                                                                   self.dilation, 0)
        if ahead is not None:  # rulebook and pooling queued with a guessed capacity, count read back last
            outids_cap, pairs, pair_num = ahead
            feats_cap = type(self)._op(input.features, pairs, pair_num, pairs.capacity)
            n_out = pairs.resolve()
            if n_out is not None:
                outids, feats = outids_cap[:n_out], feats_cap[:n_out]
        if feats is None:
            outids, pairs, pair_num = get_indice_pairs(input.indices, input.batch_size, shape, self.kernel_size,
                                                       self.stride, self.padding, self.dilation, 0, self.subm, lazy=True)
            feats = type(self)._op(input.features, pairs, pair_num, outids.shape[0])
        out = SparseTensor(feats, outids, out_shape, input.batch_size)
        out.indice_dict = input.indice_dict
        out.grid = input.grid
        return out


class SparseAvgPool(_SparsePool):
    """out = (sum of present inputs) / kernel volume."""
    _op = staticmethod(indice_avgpool)


class SparseMaxPool(_SparsePool):
    """out = max(0, max of present inputs): the output starts from zero."""
    _op = staticmethod(indice_maxpool)
