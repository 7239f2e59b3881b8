"""Pooling layers (interface of SS_Conv_lib/ss_conv/pool.py:15-92)."""
import torch
import torch.nn as nn

from ss_conv.sp_ops import tensor as tensor_mod
from ss_conv.sp_ops.tensor import SparseTensor
from ss_conv.sp_ops.pool import SparseAvgPool, SparseMaxPool
from ss_conv.sp_ops.functional import global_avgpool, global_maxpool


class AvgPool(SparseAvgPool):
    def __init__(self, kernel_size, stride=1, padding=0, dilation=1, subm=False):
        super().__init__(ndim=3, kernel_size=kernel_size, stride=stride, padding=padding, dilation=dilation, subm=subm)


class MaxPool(SparseMaxPool):
    def __init__(self, kernel_size, stride=1, padding=0, dilation=1, subm=False):
        super().__init__(ndim=3, kernel_size=kernel_size, stride=stride, padding=padding, dilation=dilation, subm=subm)


class _GlobalPool(nn.Module):
    """Per-sample pooling.  Accepts either (features, offsets) or a SparseTensor (whose row
    offsets are then computed on the device); the reference only works with the first form."""
    func = None

    def forward(self, inputs, offsets=None):
        if isinstance(inputs, SparseTensor) and inputs.raw()[0].dtype in (torch.float16, torch.bfloat16):
            inputs._features = inputs.raw()[0].float()     # stored 16-bit features: the pools compute in fp32
        if isinstance(inputs, SparseTensor):
            if inputs.pending() and offsets is None:
                # queue the pooling on the rows as they are, then read the pending counts back;
                # only a tensor that had to be recomputed is pooled again
                out = type(self).func(inputs.raw()[0], inputs.get_offsets().detach())
                if tensor_mod._capture_log is not None or not inputs.resolve():
                    return out          # (while recording a CUDA graph the counts are checked by the replaying side)
            feats = inputs.features
            offsets = inputs.get_offsets() if offsets is None else offsets
        else:
            assert offsets is not None
            feats = inputs
        return type(self).func(feats, offsets.detach())


class GlobalAvgPool(_GlobalPool):
    func = staticmethod(global_avgpool)


class GlobalMaxPool(_GlobalPool):
    func = staticmethod(global_maxpool)
