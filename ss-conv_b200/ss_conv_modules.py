"""Composite modules built on the ss_conv layers (interface of Common_utils/ss_conv_modules.py):
SS_Conv = Convolution + BatchNorm + gated Activation + Dropout, and Feature_Steering_Module =
interpolate voxel features at points, move points and irrep features into a per-sample frame,
voxelize again, two steerable convolutions."""
from functools import partial

import numpy as np
import torch
import torch.nn as nn
import torch.nn.functional as F

from ss_conv import _ext
from ss_conv.activation import Activation
from ss_conv.batchnorm import BatchNorm
from ss_conv.convolution import Convolution
from ss_conv.dropout import Dropout
from ss_conv.sp_ops.tensor import SparseTensor
from ss_conv.sp_ops.voxelize import Point2Voxel, Voxel2Point
from ss_conv.utils import SO3
from ss_conv.utils.kernel import gaussian_window_wrapper

radial_window = partial(gaussian_window_wrapper, mode="compromise", border_dist=0, sigma=0.6)


class SS_Conv(nn.Module):
    """irrep_in / irrep_out: multiplicities per order, e.g. (4, 4, 4, 4).  With a gate activation
    the convolution produces one extra scalar per non-scalar output field
    (Common_utils/ss_conv_modules.py:26-117)."""

    def __init__(self, irrep_in, irrep_out, kernel_size, dropout_p=None, radial_window=radial_window, dyn_iso=False,
                 verbose=False, stride=1, padding=0, dilation=1, groups=1, bias=False, subm=False, output_padding=0,
                 transposed=False, inverse=False, use_bn=True, bn_momentum=0.01, bn_affine=True, activation=(None, None),
                 activation_bias=False, activation_checkpoint=True, indice_key=None):
        super().__init__()
        Rs_in = [(m, l) for l, m in enumerate(irrep_in)]
        Rs_out = [(m, l) for l, m in enumerate(irrep_out)]
        Rs_gated = list(Rs_out)
        scalar_act, gate_act = activation if type(activation) is tuple else (activation, activation)
        n_non_scalar = sum(irrep_out[1:])
        if gate_act is not None and n_non_scalar > 0:
            Rs_gated.append((n_non_scalar, 0))
        self.conv = Convolution(Rs_in=Rs_in, Rs_out=Rs_gated, kernel_size=kernel_size, radial_window=radial_window,
                                dyn_iso=dyn_iso, verbose=verbose, stride=stride, padding=padding, dilation=dilation,
                                groups=groups, bias=bias, subm=subm, output_padding=output_padding, transposed=transposed,
                                inverse=inverse, indice_key=indice_key)
        self.bn = BatchNorm(Rs_gated, momentum=bn_momentum, affine=bn_affine) if use_bn else None
        if scalar_act is not None or gate_act is not None:
            self.activation = Activation(Rs_out, activation, bias=activation_bias, checkpoint=activation_checkpoint)
        else:
            self.activation = None
        self.dropout = Dropout(Rs_out, p=dropout_p) if dropout_p is not None and dropout_p > 0 else None

    def forward(self, x):
        x = self.conv(x)
        if self.bn is not None:
            x = self.bn(x)
        if self.activation is not None:
            x = self.activation(x)
        if self.dropout is not None:
            x = self.dropout(x)
        return x


class Feature_Steering_Module(nn.Module):
    """(Common_utils/ss_conv_modules.py:120-224.)  forward(points, feats, ids, r, t, s): r [B,3,3],
    t [B,3], s [B] / [B,1] / [B,3] are the per-sample pose; points and features are moved into
    that frame by one CUDA kernel (ssc_steer_fwd), voxelized and convolved twice."""

    def __init__(self, irrep, kernel_size=3, dropout_p=0.015, use_bn=True, origin_voxel_extent=None,
                 origin_unit_voxel_extent=None, voxel_num_limit=[64, 64, 64], unit_voxel_extent=[0.015, 0.015, 0.015],
                 voxelization_mode=4, frame="reference"):
        super().__init__()
        self.irrep = irrep
        # "reference": the D matrices of rotation_utils.D_from_matrix (what the reference computes);
        # "kernel": the representation in the frame of the filter basis, see SO3.D_from_matrix
        self.frame = frame
        if origin_voxel_extent is not None or origin_unit_voxel_extent is not None:
            self.v2p = Voxel2Point(voxel_extent=origin_voxel_extent, unit_voxel_extent=origin_unit_voxel_extent)
        else:
            self.v2p = None
        self.p2v = Point2Voxel(voxel_num_limit=voxel_num_limit, unit_voxel_extent=unit_voxel_extent,
                               voxelization_mode=voxelization_mode)
        common = dict(activation=(F.relu, torch.sigmoid), dropout_p=dropout_p, use_bn=use_bn)
        self.conv1 = SS_Conv(irrep, irrep, kernel_size, padding=kernel_size // 2, stride=1, subm=False, **common)
        self.conv2 = SS_Conv(irrep, irrep, kernel_size, padding=kernel_size // 2, stride=1, subm=True, **common)
        chan, off, start = [], 0, 0
        for l, m in enumerate(irrep):
            d = 2 * l + 1
            for _ in range(m):
                chan += [[start, d, off]] * d
                start += d
            off += d * d
        self._chan = torch.tensor(chan, dtype=torch.int32)
        self._d_stride = max(off, 1)

    def forward(self, points, feats, ids, r, t, s=None):
        if isinstance(feats, SparseTensor):
            assert self.v2p is not None
            if points is None:
                points, feats, ids = self.v2p(feats)
            else:
                feats = self.v2p(feats, points, ids)
        new_points, new_feats = self.steer(points, feats, ids, r, t, s)
        valid_points, valid_feats, valid_ids, flag = self.p2v(new_points, new_feats, ids)
        if torch.sum(flag) > 0:
            valid_feats = self.conv1(valid_feats)
            valid_feats = self.conv2(valid_feats)
        return valid_points, valid_feats, valid_ids, flag

    def sample_matrices(self, r):
        """[B, sum (2l+1)^2]: the representation matrices D^l(r_b) of every order, back to back."""
        blocks = [SO3.D_from_matrix(r.detach().double().cpu(), l, self.frame).reshape(r.shape[0], -1)
                  for l in range(len(self.irrep))]
        return torch.cat(blocks, dim=1).float()

    def steer(self, points, feats, ids, r, t, s=None):
        """(new_points, new_feats) = per-point change of frame; the pose is treated as constant
        (the reference detaches it too)."""
        dev = feats.device
        scale = None
        if s is not None:
            s = s.detach().float()
            if s.dim() == 2:
                s = s[:, 0] if s.size(1) == 1 else torch.norm(s, dim=1)
            scale = s.contiguous().to(dev)
        dmats = self.sample_matrices(r).to(dev).contiguous()
        chan = self._chan.to(dev)
        return _ext.steer(points.float().contiguous(), feats.float().contiguous(), ids.int().contiguous(),
                          r.detach().float().contiguous().to(dev), t.detach().float().contiguous().to(dev), scale, dmats,
                          chan)
