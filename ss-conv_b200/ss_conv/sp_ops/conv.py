"""Sparse convolution module (interface of SS_Conv_lib/ss_conv/sp_ops/conv.py:20-160)."""
import math

import numpy as np
import torch
import torch.nn as nn
from torch.nn.parameter import Parameter

from .tensor import PendingRows, SparseTensor
from .ops import get_conv_output_size, get_deconv_output_size, get_indice_pairs, _per_dim
from .. import _ext
from .functional import indice_conv, indice_inverse_conv, indice_subm_conv


# fp32 features, or features a gated Activation stored as fp16 / bf16 (_ext.set_feature_storage)
_FEATURE_DTYPES = (torch.float32, torch.float16, torch.bfloat16)


class SparseConvolution(nn.Module):
    def __init__(self, ndim, in_channels, out_channels, kernel_size=3, stride=1, padding=0, dilation=1, groups=1,
                 bias=True, subm=False, output_padding=0, transposed=False, inverse=False, indice_key=None):
        super().__init__()
        assert groups == 1
        self.ndim = ndim
        self.in_channels = in_channels
        self.out_channels = out_channels
        self.kernel_size = _per_dim(kernel_size, ndim)
        self.stride = _per_dim(stride, ndim)
        self.padding = _per_dim(padding, ndim)
        self.dilation = _per_dim(dilation, ndim)
        self.output_padding = _per_dim(output_padding, ndim)
        for d, s in zip(self.dilation, self.stride):
            assert s == 1 or d == 1, "don't support this."
        self.conv1x1 = int(np.prod(self.kernel_size)) == 1
        self.transposed = transposed
        self.inverse = inverse
        self.groups = groups
        self.subm = subm
        self.indice_key = indice_key
        self.init_parameters(bias)

    def calculate_fan_in(self):
        return self.in_channels * int(np.prod(self.kernel_size))

    def init_parameters(self, bias):
        self.weight = Parameter(torch.empty(*self.kernel_size, self.in_channels, self.out_channels))
        nn.init.kaiming_uniform_(self.weight, a=math.sqrt(5))
        if bias:
            self.bias = Parameter(torch.empty(self.out_channels))
            bound = 1 / math.sqrt(self.calculate_fan_in())
            nn.init.uniform_(self.bias, -bound, bound)
        else:
            self.register_parameter('bias', None)

    def forward(self, input):
        return self._sparse_conv(input, self.weight)

    def _output_shape(self, spatial_shape):
        if self.subm:
            return spatial_shape
        if self.transposed:
            return get_deconv_output_size(spatial_shape, self.kernel_size, self.stride, self.padding, self.dilation,
                                          self.output_padding)
        return get_conv_output_size(spatial_shape, self.kernel_size, self.stride, self.padding, self.dilation)

    def _sparse_conv(self, input, weight):
        """weight: [kx, ky, kz, Cin, Cout].  Rulebooks are cached in input.indice_dict under
        indice_key; an inverse convolution reuses its partner's rulebook with the pair roles
        exchanged.

        A regular (strided / transposed) convolution without an indice_key can run ahead of its
        output count: rulebook and convolution are queued with a guessed row capacity (also on
        an input whose own count is still pending) and the result is a SparseTensor with pending
        rows; see sp_ops/tensor.py."""
        assert isinstance(input, SparseTensor)
        out_spatial_shape = self._output_shape(input.spatial_shape)
        feats_raw, inds_raw, n_in_dev = input.raw()
        if (_ext.AHEAD and not self.conv1x1 and not self.subm and not self.inverse and self.indice_key is None
                and feats_raw.is_cuda and feats_raw.dtype in _FEATURE_DTYPES
                and not (torch.is_grad_enabled() and (feats_raw.requires_grad or weight.requires_grad))):
            # While a CUDA graph is being recorded, the part of the convolution call that does not
            # need the rulebook (filter packing, staging of the feature rows) goes to a side stream:
            # the graph then runs it next to the rulebook kernels, which leave most of the GPU idle.
            forked = None
            if torch.cuda.is_current_stream_capturing():
                cur, side = torch.cuda.current_stream(feats_raw.device), _ext.side_stream(feats_raw.device)
                side.wait_stream(cur)
                with torch.cuda.stream(side):
                    forked = _ext.conv_prepare(feats_raw, weight)
            ahead, indices_ready = _ext.rulebook_next_to_features(input._rows, lambda: _ext.get_indice_pairs_ahead(
                inds_raw, input.batch_size, out_spatial_shape, list(input.spatial_shape), self.kernel_size, self.stride,
                self.padding, self.dilation, int(self.transposed), n_in_dev=n_in_dev))
            if forked is not None:
                cur.wait_stream(side)
                if ahead is None:
                    _ext._prepared.clear()
            if ahead is not None:
                outids_cap, pairs, pair_num = ahead
                out_cap = indice_conv(feats_raw, weight, pairs, pair_num, pairs.capacity)
                if self.bias is not None:
                    out_cap += self.bias
                out = SparseTensor(out_cap, outids_cap, out_spatial_shape, input.batch_size)
                out.indice_dict = input.indice_dict
                out.grid = input.grid
                key = _ext._geometry_key(input.spatial_shape, self.kernel_size, self.stride, self.padding,
                                         self.dilation, self.transposed)

                def redo():
                    t = self._sparse_conv_exact(input, weight)
                    return t.features, t.indices

                out._rows = PendingRows(pairs._n_out_dev, pairs.capacity, input if input.pending() else None, redo,
                                        lambda n: _ext._note_ratio(key, input.features.shape[0], n))
                out._rows.indices_ready = indices_ready   # the next layer's rulebook may start here
                return out
        if (_ext.AHEAD and input.pending() and not self.conv1x1 and not self.inverse and feats_raw.is_cuda
                and feats_raw.dtype in _FEATURE_DTYPES
                and not (torch.is_grad_enabled() and (feats_raw.requires_grad or weight.requires_grad))):
            # A submanifold convolution, or one that reuses the rulebook cached under its indice_key,
            # keeps the row set of its input: on an input whose count is still on the device it works
            # on the capacity-sized buffers and hands the pending count on (so a whole stack of such
            # layers - a module of the Plain backbones - queues without a host round trip).
            cached = input.find_indice_pair(self.indice_key)
            pairs = None
            if cached is not None and isinstance(cached[2], _ext.LazyPairs) and cached[2].pending() \
                    and cached[2].capacity == inds_raw.shape[0]:
                pairs = cached[2]
            elif cached is None and self.subm:
                pairs = _ext.get_indice_pairs_subm_ahead(inds_raw, input.batch_size, list(input.spatial_shape),
                                                         self.kernel_size, self.dilation, n_in_dev)
                if self.indice_key is not None:
                    input.indice_dict[self.indice_key] = (inds_raw, inds_raw, pairs, None, input.spatial_shape)
            if pairs is not None:
                op = indice_subm_conv if self.subm else indice_conv
                out_cap = op(feats_raw, weight, pairs, None, pairs.capacity)
                if self.bias is not None:
                    out_cap += self.bias
                out = SparseTensor(out_cap, inds_raw, out_spatial_shape if self.subm else input.spatial_shape,
                                   input.batch_size)
                out.indice_dict = input.indice_dict
                out.grid = input.grid
                key = self.indice_key

                def redo():
                    if key is not None:
                        input.indice_dict.pop(key, None)      # the cached table belongs to the pending rows
                    t = self._sparse_conv_exact(input, weight)
                    return t.features, t.indices

                out._rows = PendingRows(n_in_dev, pairs.capacity, input, redo)
                out._rows.indices_ready = getattr(input._rows, "indices_ready", None)
                return out
        return self._sparse_conv_exact(input, weight)

    def _sparse_conv_exact(self, input, weight):
        features, indices = input.features, input.indices
        spatial_shape, batch_size = input.spatial_shape, input.batch_size
        out_spatial_shape = self._output_shape(spatial_shape)

        if self.conv1x1:
            # one kernel offset whose table is the identity: the same gather-GEMM kernels (and their
            # backward) as every other convolution, instead of a library GEMM (the reference calls
            # torch.mm here, sp_ops/conv.py:119-122)
            n = features.shape[0]
            rows = torch.arange(n, dtype=torch.int32, device=features.device)
            pairs = torch.stack([rows, rows]).unsqueeze(0).contiguous()
            num = torch.full((1,), n, dtype=torch.int32, device=features.device)
            input.features = indice_subm_conv(features, weight, pairs, num, n)
            if self.bias is not None:
                input.features += self.bias
            return input

        cached = input.find_indice_pair(self.indice_key)
        if self.inverse:
            assert cached is not None and self.indice_key is not None
            _, outids, indice_pairs, indice_pair_num, out_spatial_shape = cached
            assert indice_pairs.shape[0] == np.prod(self.kernel_size), \
                "inverse conv must have same kernel size as its couple conv"
        elif self.indice_key is not None and cached is not None:
            outids, _, indice_pairs, indice_pair_num, _ = cached
        else:
            outids, indice_pairs, indice_pair_num = get_indice_pairs(
                indices, batch_size, spatial_shape, self.kernel_size, self.stride, self.padding, self.dilation,
                self.output_padding, self.subm, self.transposed, grid=input.grid, lazy=True)
            input.indice_dict[self.indice_key] = (outids, indices, indice_pairs, indice_pair_num, spatial_shape)

        op = indice_subm_conv if self.subm else (indice_inverse_conv if self.inverse else indice_conv)
        out_features = op(features, weight, indice_pairs, indice_pair_num, outids.shape[0])
        if self.bias is not None:
            out_features += self.bias
        out = SparseTensor(out_features, outids, out_spatial_shape, batch_size)
        out.indice_dict = input.indice_dict
        out.grid = input.grid
        return out
