"""A chain of sparse layers replayed as one CUDA graph.

Sparse layers have data-dependent output sizes, which normally forces a host round trip per
layer.  With row counts kept on the device and every buffer sized by a capacity
(sp_ops/tensor.py, _ext.get_indice_pairs_ahead) the launch sequence of a whole chain depends only
on the capacities, so it can be recorded once and replayed: the host then pays one graph launch
and one small read-back per batch instead of tens of kernel launches and allocations.

    net = GraphedChain(lambda x: pool(conv(x)), spatial_shape, batch_size, channels, max_rows, device)
    y = net(features, indices)            # SparseTensor (exact) or whatever dense tensor fn returns

Every call copies the batch into the graph's input buffers, replays, then reads all row counts
of the chain back in one copy and checks them against the capacities.  If a capacity was too
small the batch is recomputed eagerly with exact counts (which also raises the capacity hints) and
the graph is recorded again on the next call.  Results live in buffers owned by the graph: use or
copy them before the next call.  The reference has no counterpart.
"""
import torch

from . import _ext
from .sp_ops import tensor as tensor_mod
from .sp_ops.tensor import PendingRows, SparseTensor


class GraphedChain(object):
    def __init__(self, fn, spatial_shape, batch_size, channels, max_rows, device):
        self.fn, self.shape, self.batch, self.dev = fn, spatial_shape, int(batch_size), torch.device(device)
        self.cap = int(max_rows)
        self.feats = torch.zeros((self.cap, int(channels)), dtype=torch.float32, device=self.dev)
        self.inds = torch.zeros((self.cap, 4), dtype=torch.int32, device=self.dev)
        self.n = torch.zeros(1, dtype=torch.int32, device=self.dev)
        self.graph = None
        self.launches = 0           # kernel launches recorded in the graph (= per replay)
        self.replays = 0
        self.fallbacks = 0          # replays whose row counts overflowed a capacity (recomputed eagerly)

    def _eager(self, features, indices, ahead):
        old = _ext.AHEAD
        _ext.AHEAD = ahead
        try:
            out = self.fn(SparseTensor(features, indices, self.shape, self.batch))
            if isinstance(out, SparseTensor):
                out.resolve()
            return out
        finally:
            _ext.AHEAD = old

    def _record(self):
        x = SparseTensor(self.feats, self.inds, self.shape, self.batch)
        x._rows = PendingRows(self.n, self.cap, None, None)
        log = []
        graph = torch.cuda.CUDAGraph()
        l0 = _ext.kernel_launches()
        tensor_mod._capture_log = log
        try:
            with torch.cuda.graph(graph):
                out = self.fn(x)
                counts = torch.cat([self.n] + [r.n_dev.reshape(1) for r in log])   # input count first
        finally:
            tensor_mod._capture_log = None
        self.launches = _ext.kernel_launches() - l0
        self.graph, self.out, self.counts, self.caps = graph, out, counts, [self.cap] + [r.capacity for r in log]
        if len(log) == 0 or (isinstance(out, SparseTensor) and not out.pending()):
            raise RuntimeError("nothing in this chain ran ahead of its row counts (no capacity hints yet?)")

    def __call__(self, features, indices=None):
        """features [n, C] + indices [n, 4], or one SparseTensor.  A SparseTensor whose row count is
        still pending (e.g. straight out of Point2Voxel) is taken as it is: its count joins the
        counts that are checked after the replay, so nothing waits for it before."""
        pending_in = None
        if isinstance(features, SparseTensor):
            if features.pending() and self.graph is not None:
                pending_in = features
            else:
                features, indices = features.features, features.indices
        if pending_in is not None:
            return self._replay_pending(pending_in)
        n = int(features.shape[0])
        if n > self.cap:
            raise ValueError("batch of %d rows exceeds the graph's input capacity %d" % (n, self.cap))
        if self.graph is None:
            # two eager passes: the first records the output/input ratios of every layer, the
            # second runs the capacity-sized path once (allocations, cached filters)
            self._eager(features, indices, False)
            self._eager(features, indices, True)
            torch.cuda.synchronize(self.dev)
            self._record()
        self.feats[:n].copy_(features)
        self.inds[:n].copy_(indices)
        self.n.fill_(n)
        return self._finish(lambda: (features, indices))

    def _replay_pending(self, x):
        f, i, n_dev = x.raw()
        rows = min(self.cap, int(f.shape[0]))
        self.feats[:rows].copy_(f[:rows])
        self.inds[:rows].copy_(i[:rows])
        self.n.copy_(n_dev.reshape(1))               # device to device: the host does not wait for the count

        def exact():
            x.resolve()
            if x.features.shape[0] > self.cap:
                raise ValueError("batch of %d rows exceeds the graph's input capacity %d" % (x.features.shape[0], self.cap))
            return x.features, x.indices
        return self._finish(exact)

    def _finish(self, exact_inputs):
        self.graph.replay()
        self.replays += 1
        counts = self.counts.tolist()                # the one read-back of the batch
        if any(c > cap for c, cap in zip(counts, self.caps)):
            self.graph = None                        # record again (with the raised hints) next time
            self.fallbacks += 1
            return self._eager(*exact_inputs(), False)
        out = self.out
        if isinstance(out, SparseTensor):
            f, i, _ = out.raw()
            res = SparseTensor(f[:counts[-1]], i[:counts[-1]], out.spatial_shape, out.batch_size)
            res.indice_dict, res.grid = out.indice_dict, out.grid
            return res
        return out
