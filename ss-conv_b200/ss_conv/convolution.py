"""Sparse steerable convolution layer (interface of SS_Conv_lib/ss_conv/convolution.py:19-72)."""
import math

import torch
import torch.nn as nn
from torch.nn.parameter import Parameter

from ss_conv.sp_ops.tensor import SparseTensor
from ss_conv.sp_ops.conv import SparseConvolution
from ss_conv.utils.kernel import SE3Kernel, gaussian_window_wrapper
from ss_conv.utils.utils import Rs2dim


class Convolution(SparseConvolution):
    """Rs_in / Rs_out: lists of (multiplicity, order).  The filters are materialised from the
    steerable basis by one CUDA kernel, straight into the [k,k,k,Cin,Cout] layout: on every
    forward in training mode, once (cached in `self.weight`) in eval mode.  Call
    `reset_cached_weight()` after changing `kernel.weight` of a module in eval mode."""

    def __init__(self, Rs_in, Rs_out, kernel_size, radial_window=gaussian_window_wrapper, dyn_iso=False,
                 verbose=False, stride=1, padding=0, dilation=1, groups=1, bias=False, subm=False, output_padding=0,
                 transposed=False, inverse=False, indice_key=None):
        super().__init__(ndim=3, in_channels=Rs2dim(Rs_in), out_channels=Rs2dim(Rs_out), kernel_size=kernel_size,
                         stride=stride, padding=padding, dilation=dilation, groups=groups, bias=bias, subm=subm,
                         output_padding=output_padding, transposed=transposed, inverse=inverse,
                         indice_key=indice_key)
        self.kernel = SE3Kernel(Rs_in, Rs_out, kernel_size, radial_window=radial_window, dyn_iso=dyn_iso,
                                verbose=verbose)

    def init_parameters(self, bias):
        self.weight = None
        if bias:
            self.bias = Parameter(torch.empty(self.out_channels))
            bound = 1 / math.sqrt(self.calculate_fan_in())
            nn.init.uniform_(self.bias, -bound, bound)
        else:
            self.register_parameter('bias', None)

    def reset_cached_weight(self):
        self.weight = None

    def train(self, mode=True):
        if mode:
            self.weight = None
        return super().train(mode)

    def forward(self, input):
        assert isinstance(input, SparseTensor)
        device = input.raw()[0].device
        if self.kernel.weight.device != device:
            self.kernel.to(device)
        if self.training:
            return self._sparse_conv(input, self.kernel.filters())
        if self.weight is None or self.weight.device != device:
            self.weight = self.kernel.filters()
        return self._sparse_conv(input, self.weight)
