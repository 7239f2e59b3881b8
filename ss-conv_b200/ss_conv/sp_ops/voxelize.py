"""Point cloud <-> sparse voxel tensor (interface of SS_Conv_lib/ss_conv/sp_ops/voxelize.py)."""
import numpy as np
import torch
import torch.nn as nn

from .. import _ext
from .tensor import PendingRows, SparseTensor
from .functional import three_nn, three_interpolate


class _VoxelFeatures(torch.autograd.Function):
    """Attaches the gradient of the fused voxelizer to its (already computed) voxel features:
    every point receives its voxel's gradient (sum mode 3), divided by the number of points of
    the voxel (mean mode 4), or only the first / last point of the voxel does (modes 1 / 2) —
    voxelize_bp of the reference (SS_Conv_lib/src/voxelize/voxelize_cuda_kernel.h:44-57)."""

    @staticmethod
    def forward(ctx, point_feats, voxel_feats, inverse, mode):
        ctx.save_for_backward(inverse)
        ctx.mode, ctx.n_voxel = int(mode), voxel_feats.shape[0]
        return voxel_feats.view_as(voxel_feats)

    @staticmethod
    def backward(ctx, g):
        (inverse,) = ctx.saved_tensors
        inv = inverse.long()
        d = g[inv]
        if ctx.mode == 4:
            counts = torch.bincount(inv, minlength=ctx.n_voxel).clamp_(min=1)
            d = d / counts[inv].unsqueeze(1).to(d.dtype)
        elif ctx.mode in (1, 2):
            ids = torch.arange(inv.numel(), device=inv.device)
            fill = inv.numel() if ctx.mode == 1 else -1
            chosen = torch.full((ctx.n_voxel,), fill, dtype=torch.long, device=inv.device)
            chosen.scatter_reduce_(0, inv, ids, "amin" if ctx.mode == 1 else "amax")
            d = d * (chosen[inv] == ids).unsqueeze(1).to(d.dtype)
        return d, None, None, None


class Point2Voxel(nn.Module):
    """Bins points of a batch into a voxel grid centred at the origin.

    voxelization_mode: 1 first point, 2 last point, 3 sum, 4 mean of the points of a voxel.
    forward returns (valid_points, SparseTensor, valid_batch_ids, valid_instance_flag) like the
    reference (voxelize.py:29-99).  Differences kept deliberately: a point whose coordinate
    equals +half_extent exactly (cell index == grid size) is dropped instead of producing an
    out-of-range voxel; voxel rows, inverse map and features come from one fused CUDA
    pipeline (cell bitmap + rank) instead of torch.unique + two kernels.
    """

    def __init__(self, voxel_num_limit=[64, 64, 64], unit_voxel_extent=[0.05, 0.05, 0.05], voxelization_mode=4,
                 trusted_batch_size=None):
        """trusted_batch_size (not in the reference): the caller declares that every batch has that
        many samples, batch ids in [0, trusted_batch_size) and every point inside the grid.  The
        module then skips the look at the batch that finds this out (one kernel and one host
        read-back per call) and never waits for the device, so it can be recorded into a CUDA
        graph.  A point that is outside after all is dropped and reported through the kernel status
        word (bit 1), which is checked wherever a row count is read back."""
        super().__init__()
        self.trusted_batch_size = None if trusted_batch_size is None else int(trusted_batch_size)
        self.unit_voxel_extent = torch.tensor(np.array(unit_voxel_extent, dtype=np.float64), dtype=torch.float32)
        self.voxel_num_limit = np.array(voxel_num_limit)
        self.voxelization_mode = voxelization_mode

    def forward(self, point_cloud, feature, batch_ids):
        assert point_cloud.dim() == 2
        device = point_cloud.device
        C = feature.size(1)
        grid_i = [int(v) for v in self.voxel_num_limit]
        unit_f = [float(u) for u in self.unit_voxel_extent]
        if (point_cloud.is_cuda and point_cloud.dtype == torch.float32 and point_cloud.shape[0] > 0
                and batch_ids.dtype in (torch.int32, torch.int64) and point_cloud.is_contiguous()):
            # the common case - every point inside the grid, batch ids already sorted - needs none of
            # the filtering / unique / sort steps below: one kernel and one read-back find that out
            ids32 = batch_ids.contiguous() if batch_ids.dtype == torch.int32 else batch_ids.int()
            if self.trusted_batch_size is not None:
                n_outside, n_down, n_change, last_id = 0, 0, self.trusted_batch_size - 1, self.trusted_batch_size - 1
            else:
                n_outside, n_down, n_change, last_id = _ext.p2v_stats(point_cloud, ids32, grid_i, unit_f)
            if n_outside == 0 and n_down == 0 and last_id >= 0:
                B1 = n_change + 1
                fts = feature.float().contiguous()
                if _ext.AHEAD and not (torch.is_grad_enabled() and feature.requires_grad):
                    # the voxel count stays on the device too: buffers sized by the point count
                    vox, _inverse, vfeat, m_dev = _ext.point2voxel(point_cloud, fts, ids32, max(last_id + 1, B1), grid_i,
                                                                   unit_f, self.voxelization_mode, ahead=True)
                    sparse = SparseTensor(vfeat, vox, self.voxel_num_limit.astype(np.int64), B1)
                    sparse._rows = PendingRows(m_dev, vox.shape[0], None, None)
                    return point_cloud, sparse, batch_ids, torch.ones(B1, dtype=torch.float32, device=device)
                vox, _inverse, vfeat = _ext.point2voxel(point_cloud, fts, ids32, max(last_id + 1, B1), grid_i, unit_f,
                                                        self.voxelization_mode)
                if torch.is_grad_enabled() and feature.requires_grad:
                    vfeat = _VoxelFeatures.apply(fts, vfeat, _inverse, self.voxelization_mode)
                sparse = SparseTensor(vfeat, vox, self.voxel_num_limit.astype(np.int64), B1)
                return point_cloud, sparse, batch_ids, torch.ones(B1, dtype=torch.float32, device=device)
        origin_ids = torch.unique(batch_ids)
        B1 = origin_ids.size(0)
        unit = self.unit_voxel_extent.reshape(1, 3).to(device)
        limit = torch.tensor(self.voxel_num_limit.astype(np.float64), dtype=torch.float32, device=device).reshape(1, 3)
        half = 0.5 * (limit * unit)
        cell = ((point_cloud + half) / unit).int()
        keep = ((torch.abs(point_cloud) > half).sum(1) == 0) & ((cell >= limit.int()).sum(1) == 0)

        if int(keep.sum()) == 0:
            flag = torch.zeros(B1, dtype=torch.float32, device=device)
            pts = torch.zeros(B1, 3, dtype=torch.float32, device=device)
            fts = torch.zeros(B1, C, dtype=torch.float32, device=device)
            ids = origin_ids
        else:
            pts, fts, ids = point_cloud[keep], feature[keep], batch_ids[keep]
            valid_ids = torch.unique(ids)
            B2 = valid_ids.size(0)
            if B1 == B2:
                flag = torch.ones(B1, dtype=torch.float32, device=device)
            else:  # samples that lost every point get one zero point at the origin
                flag = (origin_ids.unsqueeze(1) == valid_ids.unsqueeze(0)).sum(1).float()
                missing = origin_ids[flag == 0]
                pts = torch.cat([pts, torch.zeros(B1 - B2, 3, dtype=torch.float32, device=device)], 0)
                fts = torch.cat([fts, torch.zeros(B1 - B2, C, dtype=torch.float32, device=device)], 0)
                ids = torch.cat([ids, missing], 0)
            order = torch.sort(ids, stable=True)[1]
            pts, fts, ids = pts[order].contiguous(), fts[order].contiguous(), ids[order].contiguous()

        batch_span = int(ids.max().item()) + 1 if ids.numel() else 1
        vox, _inverse, vfeat = _ext.point2voxel(pts.float(), fts.float(), ids, max(batch_span, B1),
                                                [int(v) for v in self.voxel_num_limit],
                                                [float(u) for u in self.unit_voxel_extent], self.voxelization_mode)
        if torch.is_grad_enabled() and fts.requires_grad:
            vfeat = _VoxelFeatures.apply(fts, vfeat, _inverse, self.voxelization_mode)
        sparse = SparseTensor(vfeat, vox, self.voxel_num_limit.astype(np.int64), B1)
        return pts, sparse, ids, flag


class Voxel2Point(nn.Module):
    """Features at arbitrary points by inverse-distance interpolation of the three nearest
    occupied voxel centres of the same sample (voxelize.py:110-162)."""

    def __init__(self, voxel_extent=None, unit_voxel_extent=None):
        super().__init__()
        assert voxel_extent is not None or unit_voxel_extent is not None
        self.voxel_extent = None if voxel_extent is None else np.array(voxel_extent, dtype=np.float64)
        self.unit_voxel_extent = None if unit_voxel_extent is None else np.array(unit_voxel_extent, dtype=np.float64)

    def forward(self, sparse_feat, point_cloud=None, batch_ids=None):
        vx_points, vx_feats = self._get_vertice_feats(sparse_feat)
        if point_cloud is None:
            return vx_points[:, 1:].contiguous(), vx_feats, vx_points[:, 0].contiguous()
        assert batch_ids is not None
        points = torch.cat([batch_ids.float().unsqueeze(1), point_cloud], dim=1)
        return self._get_point_feats(points, vx_points, vx_feats)

    def _get_vertice_feats(self, sparse_tensor):
        feat = sparse_tensor.features
        shape = np.array(sparse_tensor.spatial_shape, dtype=np.float64)
        if self.voxel_extent is not None:
            unit_np, extent_np = self.voxel_extent / shape, self.voxel_extent
        else:
            unit_np, extent_np = self.unit_voxel_extent, self.unit_voxel_extent * shape
        unit = torch.tensor(unit_np, dtype=torch.float32, device=feat.device)
        extent = torch.tensor(extent_np, dtype=torch.float32, device=feat.device)
        centres = sparse_tensor.indices.float()
        centres[:, 1:] = centres[:, 1:] * unit - 0.5 * extent + 0.5 * unit
        return centres.contiguous().detach(), feat

    def _get_point_feats(self, target_points, query_points, query_feats):
        dist, idx = three_nn(target_points, query_points)
        recip = 1.0 / (dist + 1e-8)
        weight = recip / torch.sum(recip, dim=1, keepdim=True)
        return three_interpolate(query_feats, idx, weight)
