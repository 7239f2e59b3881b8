"""Streaming batches that live in host memory through a device step.

A layer step on B200 takes well under a millisecond while the PCIe copy of its fp32 feature
rows takes longer, so a host-fed loop is copy-bound.  `HostStream` keeps the three legs of a
step on three CUDA streams — upload of batch s+1, compute of batch s, download of batch s-1 —
with two staging buffers per leg, so that the copy engines and the SMs work at the same time.
Every batch is still uploaded from pinned host memory and its result downloaded to pinned host
memory; only the waiting is overlapped.  The reference has no counterpart (it is fed by a
torch DataLoader and `.cuda()` calls on the legacy stream).
"""
import torch


class HostStream:
    """step_fn(*device_tensors) -> tuple of device tensors.

    host_batches: iterable of tuples of pinned CPU tensors; every tensor's leading dimension may
    vary from batch to batch up to `max_rows`.  Iterating yields, per batch and in order, a tuple
    of pinned CPU tensors (views into `depth` rotating result buffers: consume or copy a result
    before asking for the NEXT one - with depth = 2 the download of the following batch is already
    queued into the other buffer, and the one after that reuses this one)."""

    def __init__(self, step_fn, device, max_rows, depth=2, step_reuses_outputs=False):
        """step_reuses_outputs: the step writes its results into the same device buffers on every
        call (a replayed CUDA graph does); the next step then waits until the previous result has
        been downloaded."""
        self.fn, self.dev, self.cap, self.depth = step_fn, torch.device(device), int(max_rows), int(depth)
        self.reuses = bool(step_reuses_outputs)
        self.up = torch.cuda.Stream(self.dev)
        self.down = torch.cuda.Stream(self.dev)
        self.stage_in, self.stage_out = [None] * depth, [None] * depth
        self.in_free = [None] * depth     # event: compute finished reading input slot

    def _upload(self, slot, batch):
        if self.stage_in[slot] is None:
            self.stage_in[slot] = [torch.empty((self.cap,) + tuple(t.shape[1:]), dtype=t.dtype, device=self.dev)
                                   for t in batch]
        views = []
        with torch.cuda.stream(self.up):
            if self.in_free[slot] is not None:
                self.up.wait_event(self.in_free[slot])
            for buf, t in zip(self.stage_in[slot], batch):
                if t.shape[0] > self.cap:
                    raise ValueError("batch of %d rows exceeds the staging capacity %d" % (t.shape[0], self.cap))
                v = buf[:t.shape[0]]
                v.copy_(t, non_blocking=True)
                views.append(v)
            ready = torch.cuda.Event()
            ready.record(self.up)
        return views, ready

    def _download(self, slot, outs, done):
        if self.stage_out[slot] is None:
            self.stage_out[slot] = [torch.empty((self.cap,) + tuple(t.shape[1:]), dtype=t.dtype).pin_memory() for t in outs]
        views = []
        with torch.cuda.stream(self.down):
            self.down.wait_event(done)
            for buf, t in zip(self.stage_out[slot], outs):
                if t.shape[0] > buf.shape[0]:
                    raise ValueError("result of %d rows exceeds the staging capacity %d" % (t.shape[0], buf.shape[0]))
                v = buf[:t.shape[0]]
                v.copy_(t, non_blocking=True)
                t.record_stream(self.down)
                views.append(v)
            landed = torch.cuda.Event()
            landed.record(self.down)
        return views, landed

    def run(self, host_batches):
        compute = torch.cuda.current_stream(self.dev)
        it = iter(host_batches)
        pending = None                   # (views, landed) of the previous batch
        try:
            nxt = self._upload(0, next(it))
        except StopIteration:
            return
        s = 0
        while nxt is not None:
            views, ready = nxt
            try:
                nxt = self._upload((s + 1) % self.depth, next(it))   # overlaps this batch's compute
            except StopIteration:
                nxt = None
            compute.wait_event(ready)
            if self.reuses and pending is not None:
                compute.wait_event(pending[1])       # the previous result has left the step's buffers
            outs = self.fn(*views)
            done = torch.cuda.Event()
            done.record(compute)
            self.in_free[s % self.depth] = done
            prev, pending = pending, self._download(s % self.depth, outs, done)
            s += 1
            if prev is not None:         # the previous result landed while this batch computed
                prev[1].synchronize()
                yield tuple(prev[0])
        if pending is not None:
            pending[1].synchronize()
            yield tuple(pending[0])
