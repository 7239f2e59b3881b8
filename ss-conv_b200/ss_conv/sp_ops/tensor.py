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


# While a chain of layers is being recorded into a CUDA graph (ss_conv.graph) nothing may wait for
# the device: resolving a pending count raises, and every PendingRows created is logged so that
# the replaying side can check the counts against the capacities afterwards.
_capture_log = None


class PendingRows(object):
    """Row set of a SparseTensor whose size is still on the device.

    A layer that ran ahead of its output count (see _ext.get_indice_pairs_ahead) hands out tensors
    whose `features` / `indices` buffers have `capacity` rows of which only the first n are
    meaningful, n being the device word `n_dev`.  Layers that understand this keep queueing
    kernels on the buffers (`SparseTensor.raw()`); anything else that looks at `.features` or
    `.indices` triggers `SparseTensor.resolve()`: the chain of counts is read back (parents
    first), and a tensor whose guessed capacity was too small, or whose parent had to be
    recomputed, is recomputed exactly by `redo` (its producer's exact path) followed by the
    row-wise operations applied to it since (`post`)."""

    __slots__ = ("n_dev", "capacity", "parent", "redo", "post", "note", "grad", "indices_ready")

    def __init__(self, n_dev, capacity, parent, redo, note=None):
        self.n_dev, self.capacity, self.parent, self.redo, self.note = n_dev, int(capacity), parent, redo, note
        self.post = []
        self.indices_ready = None   # while a graph is recorded: event after which indices and n_dev are complete
        self.grad = torch.is_grad_enabled()   # a recomputation runs in the mode the layer was called in
        if _capture_log is not None:
            _capture_log.append(self)


class SparseTensor(object):
    """features [N,C] float32, indices [N,4] int32 rows (batch,x,y,z), the dense spatial shape,
    the batch size, and `indice_dict`, the per-key rulebook cache shared along a network:
    key -> (outids, indices, indice_pairs, indice_pair_num, spatial_shape)."""

    def __init__(self, features, indices, spatial_shape, batch_size, grid=None):
        self._features = features
        self._indices = indices if indices.dtype == torch.int32 else indices.int()
        self._rows = None
        self._affine = None       # (scale, shift) of an eval-mode batch norm not applied yet, see _flush_affine
        self.spatial_shape = spatial_shape
        self.batch_size = batch_size
        self.indice_dict = {}
        self.grid = grid

    # -- features / indices resolve a pending row count on first access ---------------------
    def _flush_affine(self):
        """An eval-mode BatchNorm only records its per-channel scale / shift on the tensor so that a
        gated Activation that follows can apply both in one pass; anybody else who looks at the
        features gets them applied here first."""
        if self._affine is not None:
            scale, shift = self._affine
            self._affine = None
            self._features = _ext.bn_gate_forward(self._features, scale, shift, None, self._features.size(1), 0, 0, 0,
                                                  None, None)

    def _take_affine(self):
        aff, self._affine = self._affine, None
        return aff

    @property
    def features(self):
        self._flush_affine()
        if self._rows is not None:
            self.resolve()
        return self._features

    @features.setter
    def features(self, value):
        self._affine = None
        self._features = value

    @property
    def indices(self):
        if self._rows is not None:
            self.resolve()
        return self._indices

    @indices.setter
    def indices(self, value):
        self._indices = value if value.dtype == torch.int32 else value.int()

    def pending(self):
        return self._rows is not None

    def raw(self):
        """(features, indices, n_dev): the buffers as they are; n_dev is None for an exact tensor,
        else the device word with the number of meaningful rows."""
        self._flush_affine()
        return self._features, self._indices, (self._rows.n_dev if self._rows is not None else None)

    def resolve(self):
        """Make the tensor exact.  Returns True when its contents had to be recomputed."""
        self._flush_affine()
        r = self._rows
        if r is None:
            return False
        if _capture_log is not None:
            raise RuntimeError("a row count cannot be read back while a CUDA graph is being recorded: this layer "
                               "needs exact row counts and cannot be part of a captured chain")
        parent_changed = r.parent.resolve() if r.parent is not None else False
        n = _ext.read_count(r.n_dev)        # the kernel status word is checked in the same read-back
        if r.note is not None:
            r.note(n)
        self._rows = None
        if not parent_changed and n <= r.capacity:
            self._features, self._indices = self._features[:n], self._indices[:n]
            return False
        with torch.set_grad_enabled(r.grad):
            feats, inds = r.redo()
            for fn in r.post:
                feats = fn(feats)
        self._features, self._indices = feats, inds
        return True

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
        if self._indices.is_cuda:
            _, inds, n_dev = self.raw()
            return _ext.batch_offsets(inds, self.batch_size, n_dev)
        counts = torch.bincount(self.indices[:, 0].long(), minlength=self.batch_size)
        return torch.cat([counts.new_zeros(1), counts.cumsum(0)]).int()

    @property
    def sparity(self):
        return self.indices.shape[0] / np.prod(self.spatial_shape) / self.batch_size
