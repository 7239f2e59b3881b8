"""Sparse average / max pooling modules (interface of SS_Conv_lib/ss_conv/sp_ops/pool.py)."""
import torch
import torch.nn as nn

from .. import _ext
from .tensor import PendingRows, SparseTensor
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
        """A fresh (never cached) regular-convolution rulebook, then one pooling launch.  Like a
        strided convolution it can run ahead of its output count (sp_ops/tensor.py)."""
        assert isinstance(input, SparseTensor)
        shape = input.spatial_shape
        out_shape = shape if self.subm else get_conv_output_size(shape, self.kernel_size, self.stride, self.padding,
                                                                 self.dilation)
        feats_raw, inds_raw, n_in_dev = input.raw()
        if feats_raw.dtype in (torch.float16, torch.bfloat16):
            # features stored in 16 bits by a gated Activation: the pools compute in fp32
            input._features = feats_raw = feats_raw.float()
        if (_ext.AHEAD and not self.subm and feats_raw.is_cuda and feats_raw.dtype == torch.float32
                and not (torch.is_grad_enabled() and feats_raw.requires_grad)):
            ahead, indices_ready = _ext.rulebook_next_to_features(input._rows, lambda: _ext.get_indice_pairs_ahead(
                inds_raw, input.batch_size, out_shape, list(shape), self.kernel_size, self.stride, self.padding,
                self.dilation, 0, n_in_dev=n_in_dev))
            if ahead is not None:
                outids_cap, pairs, pair_num = ahead
                feats_cap = type(self)._op(feats_raw, pairs, pair_num, pairs.capacity)
                out = SparseTensor(feats_cap, outids_cap, out_shape, input.batch_size)
                out.indice_dict = input.indice_dict
                out.grid = input.grid
                key = _ext._geometry_key(shape, self.kernel_size, self.stride, self.padding, self.dilation, 0)

                def redo():
                    t = self._forward_exact(input, out_shape)
                    return t.features, t.indices

                out._rows = PendingRows(pairs._n_out_dev, pairs.capacity, input if input.pending() else None, redo,
                                        lambda n: _ext._note_ratio(key, input.features.shape[0], n))
                out._rows.indices_ready = indices_ready
                return out
        return self._forward_exact(input, out_shape)

    def _forward_exact(self, input, out_shape):
        outids, pairs, pair_num = get_indice_pairs(input.indices, input.batch_size, input.spatial_shape,
                                                   self.kernel_size, self.stride, self.padding, self.dilation, 0,
                                                   self.subm, lazy=True)
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
