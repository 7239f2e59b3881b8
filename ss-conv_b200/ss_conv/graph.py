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
copy them before the next call.

With depth = 2 (or more) the chain is recorded that many times, each recording with buffers of its
own, and batches can be queued without waiting for the one before:

    a = net.submit(f0, i0)
    b = net.submit(f1, i1)                # queued behind a; the device does not idle in between
    ya = a.result()                       # valid until `depth` more batches have been submitted

submit() returns at once; result() waits for that batch only (an event), checks its row counts
and hands out the exact tensors.  net(f, i) is submit + result.  With streams = 2 the recordings
replay on alternating streams of the chain's own, so that queued batches also overlap on the device;
result() makes the outputs safe to use from the caller's stream.

A producer that can write where it is told needs no copy at all: load(k, f, i) puts a batch into
the input buffers of recording k once, and submit_loaded(k) replays recording k on what its
buffers hold, as often as wanted.

GraphedPoints is the same for a chain that starts from a point cloud: the voxelizer (a
Point2Voxel built with trusted_batch_size, which never waits for the device) is recorded into the
graph together with the layers behind it, so a batch costs the host three small copies, one graph
launch and one read-back.
The reference has no counterpart.
"""
import contextlib
import gc

import torch

from . import _ext
from .sp_ops import tensor as tensor_mod
from .sp_ops.tensor import PendingRows, SparseTensor


@contextlib.contextmanager
def _no_gc():
    """Python's cycle collector must not run while a stream is capturing: a collected object whose
    destructor touches the CUDA runtime (a CUDA graph, a stream) would invalidate the capture."""
    gc.collect()
    was = gc.isenabled()
    gc.disable()
    try:
        yield
    finally:
        if was:
            gc.enable()


class _Recording(object):
    """One capture of the chain: the graph, its input buffers, its outputs and its row counts."""

    def __init__(self, chain):
        dev = chain.dev
        self.feats = torch.zeros((chain.cap, chain.channels), dtype=chain.feature_dtype, device=dev)
        self.inds = torch.zeros((chain.cap, 4), dtype=torch.int32, device=dev)
        self.n = torch.zeros(1, dtype=torch.int32, device=dev)
        self.graph = None
        self.out = self.counts = self.caps = self.host_counts = None
        self.done = torch.cuda.Event()
        self.fence = torch.cuda.Event()     # what the caller's stream had queued when the batch was submitted

    def record(self, chain):
        x = SparseTensor(self.feats, self.inds, chain.shape, chain.batch)
        x._rows = PendingRows(self.n, chain.cap, None, None)
        log = []
        graph = torch.cuda.CUDAGraph()
        l0 = _ext.kernel_launches()
        tensor_mod._capture_log = log
        try:
            pinned = torch.empty(256, dtype=torch.int32).pin_memory()
            with _no_gc(), torch.cuda.graph(graph):
                out = chain.fn(x)
                # input count first, the kernel status word last: it is read back with the counts
                counts = torch.cat([self.n] + [r.n_dev.reshape(1) for r in log] + [_ext.status_word(chain.dev)])
                if counts.shape[0] > pinned.shape[0]:
                    raise RuntimeError("chain with more than %d pending row counts" % (pinned.shape[0] - 1))
                host_counts = pinned[:counts.shape[0]]
                host_counts.copy_(counts, non_blocking=True)    # the one read-back of the batch, part of the graph
        finally:
            tensor_mod._capture_log = None
        chain.launches = _ext.kernel_launches() - l0
        self.graph, self.out, self.counts, self.caps = graph, out, counts, [chain.cap] + [r.capacity for r in log]
        self.host_counts = host_counts
        if len(log) == 0 or (isinstance(out, SparseTensor) and not out.pending()):
            raise RuntimeError("nothing in this chain ran ahead of its row counts (no capacity hints yet?)")


class _Queued(object):
    """A batch that has been queued on one recording; result() finishes it."""

    def __init__(self, chain, rec, exact_inputs):
        self.chain, self.rec, self.exact_inputs = chain, rec, exact_inputs
        self.value = None
        self.finished = False

    def result(self):
        if self.finished:
            return self.value
        rec, chain = self.rec, self.chain
        rec.done.synchronize()                       # this batch only
        counts = rec.host_counts.tolist()
        _ext.raise_on_status(counts.pop(), chain.dev)    # a kernel of the replay gave up: no partial results
        if any(c > cap for c, cap in zip(counts, rec.caps)):
            chain.stale = True                       # record again (with the raised hints) next time
            chain.fallbacks += 1
            self.value = chain._eager(*self.exact_inputs(), False)
        else:
            out = rec.out
            if isinstance(out, SparseTensor):
                f, i, _ = out.raw()
                res = SparseTensor(f[:counts[-1]], i[:counts[-1]], out.spatial_shape, out.batch_size)
                res.indice_dict, res.grid = out.indice_dict, out.grid
                out = res
            self.value = out
        self.finished = True
        self.exact_inputs = None
        return self.value


class GraphedChain(object):
    def __init__(self, fn, spatial_shape, batch_size, channels, max_rows, device, depth=1, streams=1,
                 feature_dtype=torch.float32):
        """feature_dtype: type of the input feature rows the graph is fed with (torch.float16 /
        torch.bfloat16: a caller that holds its features in 16 bits uploads half the bytes; the first
        convolution gathers them as its operands)."""
        self.feature_dtype = feature_dtype
        self.fn, self.shape, self.batch, self.dev = fn, spatial_shape, int(batch_size), torch.device(device)
        self.cap, self.channels, self.depth = int(max_rows), int(channels), max(1, int(depth))
        # streams > 1: recording k replays on stream k % streams, so consecutive batches overlap on the
        # device (the small rulebook kernels of one batch under the convolution of the one before)
        self.exec_streams = [torch.cuda.Stream(self.dev) for _ in range(int(streams))] if int(streams) > 1 else None
        self.recs = None            # `depth` recordings, made on first use
        self.stale = False          # a capacity overflowed: record again before the next replay
        self.turn = 0
        self.loaded = {}            # recording -> (features, indices) put there by load()
        self.queued = []            # per recording: the batch that occupies it (or None)
        self.launches = 0           # kernel launches recorded in the graph (= per replay)
        self.replays = 0
        self.fallbacks = 0          # replays whose row counts overflowed a capacity (recomputed eagerly)

    @property
    def graph(self):
        return None if (self.recs is None or self.stale) else self.recs[0].graph

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

    def _ready(self, features, indices):
        """Recordings exist and are current; (features, indices) is an exact batch to warm up on."""
        if self.recs is not None and not self.stale:
            return
        for q in self.queued:                        # nothing may still be running on the old recordings
            if q is not None:
                q.result()
        # two eager passes: the first records the output/input ratios of every layer, the
        # second runs the capacity-sized path once (allocations, cached filters)
        self._eager(features, indices, False)
        self._eager(features, indices, True)
        torch.cuda.synchronize(self.dev)
        self.recs = [_Recording(self) for _ in range(self.depth)]
        for rec in self.recs:
            rec.record(self)
        self.queued = [None] * self.depth
        self.stale = False
        self.turn = 0
        for k, (f, i) in self.loaded.items():        # batches that lived in the old recordings' buffers
            self._fill(self.recs[k], f, i)

    def _fill(self, rec, features, indices):
        n = int(features.shape[0])
        rec.feats[:n].copy_(features)
        rec.inds[:n].copy_(indices)
        rec.n.fill_(n)

    def _free(self, k):
        old = self.queued[k]
        if old is not None and not old.finished:
            old.result()                             # its buffers are about to be overwritten
        return self.recs[k]

    def load(self, k, features, indices):
        """Copy a batch into the input buffers of recording k (0 <= k < depth) for submit_loaded(k)."""
        n = int(features.shape[0])
        if n > self.cap:
            raise ValueError("batch of %d rows exceeds the graph's input capacity %d" % (n, self.cap))
        self._ready(features, indices)
        self._fill(self._free(k), features, indices)
        self.loaded[k] = (features, indices)

    def submit_loaded(self, k):
        """Replay recording k on the batch that load(k, ...) left in its input buffers: no copy.  The
        previous result of recording k must have been used by now (its buffers are overwritten)."""
        if self.recs is None or self.stale:
            if k not in self.loaded:
                raise RuntimeError("recording %d holds no batch: call load() first" % k)
            self._ready(*self.loaded[k])
        rec = self._free(k)
        return self._launch(rec, lambda: self.loaded[k])

    def _launch(self, rec, exact_inputs):
        k = self.recs.index(rec)
        if self.exec_streams is None:
            rec.graph.replay()
            rec.done.record()
        else:
            stream = self.exec_streams[k % len(self.exec_streams)]
            cur = torch.cuda.current_stream(self.dev)
            rec.fence.record(cur)                    # the batch's inputs (copies queued by the caller's stream) and
            stream.wait_event(rec.fence)             # the caller's reads of this recording's previous output
            torch.cuda.set_stream(stream)
            try:
                rec.graph.replay()
            finally:
                torch.cuda.set_stream(cur)
            rec.done.record(stream)
        self.replays += 1
        q = _Queued(self, rec, exact_inputs)
        self.queued[k] = q
        return q

    def _next(self):
        k = self.turn
        self.turn = (self.turn + 1) % self.depth
        self.loaded.pop(k, None)                     # whatever load() left there is overwritten
        return self._free(k)

    def submit(self, features, indices=None):
        """Queue one batch (features [n, C], indices [n, 4]); returns an object whose result() gives
        what the chain returns.  Does not wait for the device.
        A SparseTensor (indices=None) is accepted too, also one whose row count is still pending."""
        if isinstance(features, SparseTensor):
            if features.pending() and self.graph is not None:
                return self._replay_pending(features)
            features, indices = features.features, features.indices
        n = int(features.shape[0])
        if n > self.cap:
            raise ValueError("batch of %d rows exceeds the graph's input capacity %d" % (n, self.cap))
        self._ready(features, indices)
        rec = self._next()
        self._fill(rec, features, indices)
        return self._launch(rec, lambda: (features, indices))

    def __call__(self, features, indices=None):
        """features [n, C] + indices [n, 4], or one SparseTensor.  A SparseTensor whose row count is
        still pending (e.g. straight out of Point2Voxel) is taken as it is: its count joins the
        counts that are checked after the replay, so nothing waits for it before."""
        return self.submit(features, indices).result()

    def _replay_pending(self, x):
        f, i, n_dev = x.raw()
        rec = self._next()
        rows = min(self.cap, int(f.shape[0]))
        rec.feats[:rows].copy_(f[:rows])
        rec.inds[:rows].copy_(i[:rows])
        rec.n.copy_(n_dev.reshape(1))                # device to device: the host does not wait for the count

        def exact():
            x.resolve()
            if x.features.shape[0] > self.cap:
                raise ValueError("batch of %d rows exceeds the graph's input capacity %d" % (x.features.shape[0], self.cap))
            return x.features, x.indices
        return self._launch(rec, exact)


class _PointRecording(object):
    """One capture of voxelizer + chain over fixed-size point buffers."""

    def __init__(self, owner):
        dev = owner.dev
        self.pts = torch.zeros((owner.n_points, 3), dtype=torch.float32, device=dev)
        self.fts = torch.zeros((owner.n_points, owner.channels), dtype=torch.float32, device=dev)
        self.ids = torch.zeros(owner.n_points, dtype=torch.int32, device=dev)
        self.graph = None
        self.out = self.host_counts = self.caps = None
        self.done = torch.cuda.Event()
        self.fence = torch.cuda.Event()

    def record(self, owner):
        log = []
        graph = torch.cuda.CUDAGraph()
        l0 = _ext.kernel_launches()
        tensor_mod._capture_log = log
        try:
            pinned = torch.empty(256, dtype=torch.int32).pin_memory()
            with _no_gc(), torch.cuda.graph(graph):
                out = owner.fn(owner.p2v(self.pts, self.fts, self.ids)[1])
                counts = torch.cat([r.n_dev.reshape(1) for r in log] + [_ext.status_word(owner.dev)])
                if counts.shape[0] > pinned.shape[0]:
                    raise RuntimeError("chain with more than %d pending row counts" % (pinned.shape[0] - 1))
                host_counts = pinned[:counts.shape[0]]
                host_counts.copy_(counts, non_blocking=True)
        finally:
            tensor_mod._capture_log = None
        owner.launches = _ext.kernel_launches() - l0
        if len(log) == 0:
            raise RuntimeError("nothing in this chain ran ahead of its row counts (no capacity hints yet?)")
        self.graph, self.out, self.host_counts, self.caps = graph, out, host_counts, [r.capacity for r in log]


class _QueuedPoints(object):
    def __init__(self, owner, rec, inputs):
        self.owner, self.rec, self.inputs = owner, rec, inputs
        self.value, self.finished = None, False

    def result(self):
        if self.finished:
            return self.value
        rec, owner = self.rec, self.owner
        rec.done.synchronize()
        counts = rec.host_counts.tolist()
        _ext.raise_on_status(counts.pop(), owner.dev)
        if any(c > cap for c, cap in zip(counts, rec.caps)):
            owner.stale = True
            owner.fallbacks += 1
            self.value = owner._eager(*self.inputs, False)
        else:
            out = rec.out
            if isinstance(out, SparseTensor):
                f, i, _ = out.raw()
                res = SparseTensor(f[:counts[-1]], i[:counts[-1]], out.spatial_shape, out.batch_size)
                res.indice_dict, res.grid = out.indice_dict, out.grid
                out = res
            self.value = out
        self.finished, self.inputs = True, None
        return self.value


class GraphedPoints(object):
    """fn(SparseTensor) -> tensor or SparseTensor, fed by p2v(points, feats, ids).  Every batch has
    exactly n_points points (p2v was built with trusted_batch_size).  submit() / result() / depth /
    streams as in GraphedChain; results live in buffers owned by the graph."""

    def __init__(self, p2v, fn, n_points, channels, device, depth=1, streams=1):
        if p2v.trusted_batch_size is None:
            raise ValueError("GraphedPoints needs a Point2Voxel built with trusted_batch_size")
        self.p2v, self.fn, self.dev = p2v, fn, torch.device(device)
        self.n_points, self.channels, self.depth = int(n_points), int(channels), max(1, int(depth))
        self.exec_streams = [torch.cuda.Stream(self.dev) for _ in range(int(streams))] if int(streams) > 1 else None
        self.recs, self.stale, self.turn, self.queued = None, False, 0, []
        self.launches = self.replays = self.fallbacks = 0

    def _eager(self, points, feats, ids, ahead):
        old = _ext.AHEAD
        _ext.AHEAD = ahead
        try:
            out = self.fn(self.p2v(points, feats, ids)[1])
            if isinstance(out, SparseTensor):
                out.resolve()
            return out
        finally:
            _ext.AHEAD = old

    def _ready(self, points, feats, ids):
        if self.recs is not None and not self.stale:
            return
        for q in self.queued:
            if q is not None:
                q.result()
        self._eager(points, feats, ids, False)       # records the output / input ratio of every layer
        self._eager(points, feats, ids, True)        # the capacity-sized path once (allocations, cached filters)
        torch.cuda.synchronize(self.dev)
        self.recs = [_PointRecording(self) for _ in range(self.depth)]
        for rec in self.recs:
            rec.pts.copy_(points)
            rec.fts.copy_(feats)
            rec.ids.copy_(ids)
            rec.record(self)
        self.queued = [None] * self.depth
        self.stale, self.turn = False, 0

    def submit(self, points, feats, ids):
        if points.shape[0] != self.n_points:
            raise ValueError("batch of %d points, the graph was built for %d" % (points.shape[0], self.n_points))
        self._ready(points, feats, ids)
        k = self.turn
        self.turn = (self.turn + 1) % self.depth
        old = self.queued[k]
        if old is not None and not old.finished:
            old.result()                             # its buffers are about to be overwritten
        rec = self.recs[k]
        rec.pts.copy_(points, non_blocking=True)
        rec.fts.copy_(feats, non_blocking=True)
        rec.ids.copy_(ids, non_blocking=True)
        if self.exec_streams is None:
            rec.graph.replay()
            rec.done.record()
        else:
            stream = self.exec_streams[k % len(self.exec_streams)]
            cur = torch.cuda.current_stream(self.dev)
            rec.fence.record(cur)
            stream.wait_event(rec.fence)
            torch.cuda.set_stream(stream)
            try:
                rec.graph.replay()
            finally:
                torch.cuda.set_stream(cur)
            rec.done.record(stream)
        self.replays += 1
        q = _QueuedPoints(self, rec, (points, feats, ids))
        self.queued[k] = q
        return q

    def __call__(self, points, feats, ids):
        return self.submit(points, feats, ids).result()
