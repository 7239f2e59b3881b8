"""autograd entry points of the sparse ops (interface of
SS_Conv_lib/ss_conv/sp_ops/functional.py:441-453: indice_conv, indice_subm_conv,
indice_inverse_conv, indice_maxpool, indice_avgpool, global_avgpool, global_maxpool,
voxelization, voxel2point_mapping, three_nn, three_interpolate).

Forward and backward passes of the convolution and the pools call the CUDA library; the
backward of the voxelizer / interpolation ops is not built (raises NotImplementedError).
"""
import torch
from torch.autograd import Function

from .. import _ext
from . import ops


def _save(ctx, pairs, *tensors):
    """Pair lists may be a lazy handle (not a tensor): keep them as a plain attribute."""
    ctx.indice_pairs = pairs
    ctx.save_for_backward(*tensors)


def _conv_function(inverse, subm):
    class _Conv(Function):
        @staticmethod
        def forward(ctx, features, filters, indice_pairs, indice_pair_num, num_activate_out):
            _save(ctx, indice_pairs, indice_pair_num, features, filters)
            return ops.indice_conv_forward(features, filters, indice_pairs, indice_pair_num, num_activate_out,
                                           inverse, subm)

        @staticmethod
        def backward(ctx, grad_output):
            indice_pair_num, features, filters = ctx.saved_tensors
            indice_pairs = ctx.indice_pairs
            d_in, d_flt = ops.indice_conv_backward(features, filters, grad_output.contiguous(), indice_pairs,
                                                   indice_pair_num, inverse, subm)
            return d_in, d_flt, None, None, None

    return _Conv


SparseConvFunction = _conv_function(False, False)
SparseInverseConvFunction = _conv_function(True, False)
SubMConvFunction = _conv_function(False, True)


class SparseMaxPoolFunction(Function):
    @staticmethod
    def forward(ctx, features, indice_pairs, indice_pair_num, num_activate_out):
        out = ops.indice_maxpool_forward(features, indice_pairs, indice_pair_num, num_activate_out)
        _save(ctx, indice_pairs, indice_pair_num, features, out)
        return out

    @staticmethod
    def backward(ctx, grad_output):
        indice_pair_num, features, out = ctx.saved_tensors
        indice_pairs = ctx.indice_pairs
        return ops.indice_maxpool_backward(features, out, grad_output.contiguous(), indice_pairs,
                                           indice_pair_num), None, None, None


class SparseAvgPoolFunction(Function):
    @staticmethod
    def forward(ctx, features, indice_pairs, indice_pair_num, num_activate_out, use_gs=True):
        # use_gs: divide by the kernel volume; otherwise by the number of present inputs
        summaryrf = None if use_gs else _ext.indiceSummaryRF(indice_pairs, indice_pair_num, num_activate_out)
        out = ops.indice_avgpool_forward(features, indice_pairs, indice_pair_num, num_activate_out, summaryrf)
        ctx.kernel_volume = int(indice_pairs.shape[0])
        if summaryrf is None:
            _save(ctx, indice_pairs, indice_pair_num, features, out)
        else:
            _save(ctx, indice_pairs, indice_pair_num, features, out, summaryrf)
        return out

    @staticmethod
    def backward(ctx, grad_output):
        saved = ctx.saved_tensors
        indice_pair_num, features, out = saved[:3]
        summaryrf = saved[3] if len(saved) > 3 else torch.full((out.shape[0],), ctx.kernel_volume, dtype=torch.int32,
                                                               device=out.device)
        indice_pairs = ctx.indice_pairs
        return ops.indice_avgpool_backward(features, out, grad_output.contiguous(), indice_pairs, indice_pair_num,
                                           summaryrf), None, None, None, None


def _global_pool_function(native_fp, native_bp):
    class _GlobalPool(Function):
        @staticmethod
        def forward(ctx, feats, proposals_offset):
            n_prop = proposals_offset.size(0) - 1
            n, c = feats.size()
            feats = feats.contiguous()
            proposals_offset = proposals_offset.contiguous().int()
            out = torch.zeros((n_prop, c), dtype=torch.float32, device=feats.device)
            maxidx = torch.zeros((n_prop, c), dtype=torch.int32, device=feats.device)
            native_fp(feats, proposals_offset, out, maxidx, n_prop, c)
            ctx.for_backwards = (maxidx, proposals_offset, n)
            return out

        @staticmethod
        def backward(ctx, d_out):
            maxidx, proposals_offset, n = ctx.for_backwards
            n_prop, c = d_out.size()
            d_feats = torch.zeros((n, c), dtype=torch.float32, device=d_out.device)
            native_bp(d_feats, proposals_offset, maxidx, d_out.contiguous(), n_prop, c)
            return d_feats, None

    return _GlobalPool


GlobalMaxPool = _global_pool_function(_ext.global_maxpool_fp, _ext.global_maxpool_bp)
GlobalAvgPool = _global_pool_function(_ext.global_avgpool_fp, _ext.global_avgpool_bp)


class Voxelization(Function):
    @staticmethod
    def forward(ctx, feats, map_rule, mode=4):
        feats = feats.contiguous()
        map_rule = map_rule.contiguous()
        n, c = feats.size()
        m, width = map_rule.size()
        out = torch.zeros((m, c), dtype=torch.float32, device=feats.device)
        ctx.for_backwards = (map_rule, mode, width - 1, n)
        _ext.voxelize_fp(feats, out, map_rule, mode, m, width - 1, c)
        return out

    @staticmethod
    def backward(ctx, d_out):
        map_rule, mode, max_active, n = ctx.for_backwards
        m, c = d_out.size()
        d_feats = torch.zeros((n, c), dtype=torch.float32, device=d_out.device)
        _ext.voxelize_bp(d_out.contiguous(), d_feats, map_rule, mode, m, max_active, c)
        return d_feats, None, None


class Voxel2Point_Map(Function):
    @staticmethod
    def forward(ctx, inverse, nActive, maxActive, mode=4):
        """Rows [count, point ids...] per voxel; mode 1 first, 2 last, 3/4 all points."""
        inverse = inverse.view(-1).contiguous().int()
        n = inverse.size(0)
        ids = torch.arange(n, dtype=torch.int32, device=inverse.device)
        fill = {1: n, 2: -1, 3: 0, 4: 0}
        assert mode in fill
        maps = torch.full((nActive, maxActive + 1), fill[mode], dtype=torch.int32, device=inverse.device)
        _ext.voxel2point_map(inverse, ids, maps, n, maxActive, mode)
        return maps

    @staticmethod
    def backward(ctx, grad=None):
        return None, None, None, None


class ThreeNN(Function):
    @staticmethod
    def forward(ctx, unknown, known):
        """unknown [N,4], known [M,4] rows (batch,x,y,z) -> (distance [N,3], index [N,3])."""
        unknown, known = unknown.contiguous(), known.contiguous()
        n, m = unknown.size(0), known.size(0)
        dist2 = torch.empty((n, 3), dtype=torch.float32, device=unknown.device)
        idx = torch.empty((n, 3), dtype=torch.int32, device=unknown.device)
        _ext.three_nn(n, m, unknown, known, dist2, idx)
        return torch.sqrt(dist2), idx

    @staticmethod
    def backward(ctx, a=None, b=None):
        return None, None


class ThreeInterpolate(Function):
    @staticmethod
    def forward(ctx, features, idx, weight):
        """features [M,C], idx [N,3], weight [N,3] -> [N,C]."""
        features, idx, weight = features.contiguous(), idx.contiguous(), weight.contiguous()
        m, c = features.size()
        n = idx.size(0)
        ctx.three_interpolate_for_backward = (idx, weight, m)
        out = torch.empty((n, c), dtype=torch.float32, device=features.device)
        _ext.three_interpolate_fp(c, m, n, features, idx, weight, out)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        idx, weight, m = ctx.three_interpolate_for_backward
        n, c = grad_out.size()
        grad_features = torch.zeros((m, c), dtype=torch.float32, device=grad_out.device)
        _ext.three_interpolate_bp(c, n, m, grad_out.contiguous(), idx, weight, grad_features)
        return grad_features, None, None


def _needs_graph(*tensors):
    return torch.is_grad_enabled() and any(t.requires_grad for t in tensors)


def _conv_entry(fn, inverse, subm):
    """Inference calls skip the autograd.Function machinery (tens of microseconds per call)."""
    def call(features, filters, indice_pairs, indice_pair_num, num_activate_out):
        if _needs_graph(features, filters):
            return fn.apply(features, filters, indice_pairs, indice_pair_num, num_activate_out)
        return ops.indice_conv_forward(features, filters, indice_pairs, indice_pair_num, num_activate_out, inverse, subm)
    return call


indice_conv = _conv_entry(SparseConvFunction, False, False)
indice_inverse_conv = _conv_entry(SparseInverseConvFunction, True, False)
indice_subm_conv = _conv_entry(SubMConvFunction, False, True)


def indice_maxpool(features, indice_pairs, indice_pair_num, num_activate_out):
    if _needs_graph(features):
        return SparseMaxPoolFunction.apply(features, indice_pairs, indice_pair_num, num_activate_out)
    return ops.indice_maxpool_forward(features, indice_pairs, indice_pair_num, num_activate_out)


indice_avgpool = SparseAvgPoolFunction.apply
global_maxpool = GlobalMaxPool.apply
global_avgpool = GlobalAvgPool.apply
voxelization = Voxelization.apply
voxel2point_mapping = Voxel2Point_Map.apply
three_nn = ThreeNN.apply
three_interpolate = ThreeInterpolate.apply
