"""Output-size arithmetic and dispatch into the native module
(interface of SS_Conv_lib/ss_conv/sp_ops/ops.py)."""
import torch

from .. import _ext


def _per_dim(v, ndim):
    return list(v) if isinstance(v, (list, tuple)) else [v] * ndim


def get_conv_output_size(input_size, kernel_size, stride, padding, dilation):
    """floor((n + 2p - d(k-1) - 1)/s) + 1 per dimension; kernel_size -1 means 'whole axis'."""
    return [1 if k == -1 else (n + 2 * p - d * (k - 1) - 1) // s + 1
            for n, k, s, p, d in zip(input_size, kernel_size, stride, padding, dilation)]


def get_deconv_output_size(input_size, kernel_size, stride, padding, dilation, output_padding):
    out = []
    for n, k, s, p, op in zip(input_size, kernel_size, stride, padding, output_padding):
        if k == -1:
            raise ValueError("deconv don't support kernel_size < 0")
        out.append((n - 1) * s - 2 * p + k + op)
    return out


def get_indice_pairs(indices, batch_size, spatial_shape, ksize=3, stride=1, padding=0, dilation=1, out_padding=0,
                     subm=False, transpose=False, grid=None, lazy=False):
    """(outids, indice_pairs [K,2,N], indice_pair_num [K]) for a 3-D sparse tensor.
    lazy=True returns the pair lists as a handle that builds the tensor only when it is looked
    at (the layers of this package use that: the CUDA kernels work on the neighbour table)."""
    ndim = indices.shape[1] - 1
    ksize, stride, padding = _per_dim(ksize, ndim), _per_dim(stride, ndim), _per_dim(padding, ndim)
    dilation, out_padding = _per_dim(dilation, ndim), _per_dim(out_padding, ndim)
    for d, s in zip(dilation, stride):
        assert s == 1 or d == 1, "don't support this."
    if subm:
        out_shape = list(spatial_shape)
    elif transpose:
        out_shape = get_deconv_output_size(spatial_shape, ksize, stride, padding, dilation, out_padding)
    else:
        out_shape = get_conv_output_size(spatial_shape, ksize, stride, padding, dilation)
    if ndim != 3:
        raise NotImplementedError
    if lazy:
        return _ext.get_indice_pairs_lazy(indices, batch_size, out_shape, list(spatial_shape), ksize, stride, padding,
                                          dilation, int(subm), int(transpose))
    if grid is None:
        return _ext.get_indice_pairs_3d(indices, batch_size, out_shape, list(spatial_shape), ksize, stride, padding,
                                        dilation, out_padding, int(subm), int(transpose))
    return _ext.get_indice_pairs_grid_3d(indices, grid, batch_size, out_shape, list(spatial_shape), ksize, stride,
                                         padding, dilation, out_padding, int(subm), int(transpose))


def _by_dtype(t, fp32, half):
    if t.dtype == torch.float32:
        return fp32
    if t.dtype == torch.half:
        return half
    raise NotImplementedError


def indice_conv_forward(features, filters, indice_pairs, indice_pair_num, num_activate_out, inverse=False,
                        subm=False):
    fn = _by_dtype(filters, _ext.indice_conv_fp32, _ext.indice_conv_half)
    return fn(features, filters, indice_pairs, indice_pair_num, num_activate_out, int(inverse), int(subm))


def indice_conv_backward(features, filters, out_bp, indice_pairs, indice_pair_num, inverse=False, subm=False):
    fn = _by_dtype(filters, _ext.indice_conv_backward_fp32, _ext.indice_conv_backward_half)
    return fn(features, filters, out_bp, indice_pairs, indice_pair_num, int(inverse), int(subm))


def indice_avgpool_forward(features, indice_pairs, indice_pair_num, num_activate_out, summaryrf):
    fn = _by_dtype(features, _ext.indice_avgpool_fp32, _ext.indice_avgpool_half)
    return fn(features, indice_pairs, indice_pair_num, num_activate_out, summaryrf)


def indice_avgpool_backward(features, out_features, out_bp, indice_pairs, indice_pair_num, summaryrf):
    fn = _by_dtype(features, _ext.indice_avgpool_backward_fp32, _ext.indice_avgpool_backward_half)
    return fn(features, out_features, out_bp, indice_pairs, indice_pair_num, summaryrf)


def indice_maxpool_forward(features, indice_pairs, indice_pair_num, num_activate_out):
    fn = _by_dtype(features, _ext.indice_maxpool_fp32, _ext.indice_maxpool_half)
    return fn(features, indice_pairs, indice_pair_num, num_activate_out)


def indice_maxpool_backward(features, out_features, out_bp, indice_pairs, indice_pair_num):
    fn = _by_dtype(features, _ext.indice_maxpool_backward_fp32, _ext.indice_maxpool_backward_half)
    return fn(features, out_features, out_bp, indice_pairs, indice_pair_num)
