"""Benchmark of the sparse steerable convolution hot path on B200.

Headline workload ("cfg2", the configuration the metric is quoted on): a strided
downsampling SS-Conv layer, irreps (4,4,4,4) = 64 channels in, 64 + 12 gate scalars = 76 out,
kernel 3, stride 2, padding 1, batch 32 on a 64^3 grid with 16384 ellipsoid-surface points per
sample (seeded synthetic stand-in for object-surface data), followed by a sparse MaxPool
(kernel 2, stride 2).  One step = rulebook + filter materialisation + packing +
gather-GEMM (tcgen05, TF32 operands, fp32 accumulate) + pool rulebook + max pool.

metric  : active input voxels per second through the layer (whole job, all ranks)
value   : inputs resident in HBM, CUDA-event timed, max over ranks
e2e     : the same step through the public ss_conv API starting from pinned HOST buffers
          (H2D of indices+features and D2H of the pooled features of every step inside the timed
          region; ss_conv.pipeline.HostStream overlaps the copies of neighbouring steps)
roofline: dominant kernel (conv_fwd_tf32_kernel, with the TF32 staging pass that precedes it)
          algorithmic bytes / its CUDA-event time
cpu_baseline / --impl reference: the reference's own C++ CPU path (oracle/_ref, built from the
          reference sources) on the box's host cores.

python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
For N > 1 launch with torch.distributed.run (one rank per GPU); every rank processes its own
batch of 32 samples (weak scaling, no data-path collective).
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (os.path.join(ROOT, "ss-conv_b200"), os.path.join(ROOT, "oracle")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import numpy as np  # noqa: E402
import torch  # noqa: E402

CFG2 = dict(name="cfg2: SS-Conv (4,4,4,4)->(4,4,4,4)+12 gates, k3 s2 p1, batch 32, 64^3, 16384 pts/sample, + MaxPool k2 s2",
            batch=32, V=64, n_pts=16384, irreps=(4, 4, 4, 4), k=3, stride=2, pad=1, pool_k=2, pool_s=2)
CONV_DRAM_TRAFFIC = 81.0e6  # bytes per launch, from the ncu capture summarised under profiles/
ROTATE = 4  # distinct input batches cycled through so the working set exceeds the 126 MB L2


def rs_of(irreps, gates=False):
    rs = [(m, l) for l, m in enumerate(irreps)]
    if gates:
        rs = rs + [(sum(irreps[1:]), 0)]
    return rs


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return float(p["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (6.65 TB/s)"


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken while the timed region runs: ONE
    nvidia-smi process in loop mode (started before the region, stopped after it), so that the
    sampling costs the benchmarked process nothing."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index, enabled=True):
        self.index, self.samples, self.proc, self.enabled = index, [], None, enabled

    def __enter__(self):
        if self.enabled:
            try:
                self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                              "--format=csv,noheader,nounits", "-lms", "100"],
                                             stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
                time.sleep(0.25)  # let the first samples come in before the timed region starts
            except Exception:
                self.proc = None
        return self

    def __exit__(self, *a):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                out, _ = self.proc.communicate(timeout=5)
            except Exception:
                self.proc.kill()
                out = ""
            for line in out.strip().splitlines():
                f = [x.strip() for x in line.split(",")]
                if len(f) >= 7:
                    self.samples.append(f)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        sm = [float(s[0]) for s in self.samples if s[0].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(s[3 + i].lower().startswith("active") for s in self.samples)]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": float(self.samples[0][1]),
                "reasons": reasons, "samples": len(self.samples)}


# ------------------------------------------------------------------------------ our arm
class Layer:
    """The cfg2 layer built from the public ss_conv modules."""

    def __init__(self, cfg, device):
        from ss_conv.convolution import Convolution
        from ss_conv.pool import MaxPool
        torch.manual_seed(1234)
        self.cfg = cfg
        self.conv = Convolution(rs_of(cfg["irreps"]), rs_of(cfg["irreps"], gates=True), cfg["k"], stride=cfg["stride"],
                                padding=cfg["pad"]).to(device)
        self.conv.train()          # training-mode forward: filters are re-materialised every step
        self.pool = MaxPool(cfg["pool_k"], stride=cfg["pool_s"])

    def step(self, feats, indices):
        from ss_conv.sp_ops.tensor import SparseTensor
        c = self.cfg
        with torch.no_grad():
            x = SparseTensor(feats, indices, [c["V"]] * 3, c["batch"])
            return self.pool(self.conv(x))


BACKBONE = dict(name="backbone: Point2Voxel(32^3, mean) + 4 x [SS-Conv k3 s2 p1 + BatchNorm(eval) + gate(relu, sigmoid)] + "
                     "GlobalAvgPool, irreps (3)->(8,4,2)->(16,8,4)->(32,16,8)->(64,32,16), 1024 points/object, "
                     "global batch 256 sharded by sample",
                irreps=[(3,), (8, 4, 2), (16, 8, 4), (32, 16, 8), (64, 32, 16)], V=32, n_pts=1024, global_batch=256)


class Backbone:
    """The 4-stage backbone of the benchmark configurations, from the public ss_conv modules."""

    def __init__(self, cfg, device):
        from ss_conv.activation import Activation
        from ss_conv.batchnorm import BatchNorm
        from ss_conv.convolution import Convolution
        from ss_conv.pool import GlobalAvgPool
        from ss_conv.sp_ops.voxelize import Point2Voxel
        torch.manual_seed(4321)
        V = cfg["V"]
        self.p2v = Point2Voxel([V] * 3, [1.0 / V] * 3, 4)
        self.stages = []
        for a, b in zip(cfg["irreps"][:-1], cfg["irreps"][1:]):
            conv = Convolution(rs_of(a), rs_of(b, gates=True), 3, stride=2, padding=1).to(device).eval()
            bn = BatchNorm(rs_of(b, gates=True)).to(device).eval()
            with torch.no_grad():
                bn.running_var.uniform_(0.5, 1.5)
                bn.running_mean.normal_(0, 0.1)
            act = Activation(rs_of(b), (torch.relu, torch.sigmoid), bias=False, checkpoint=False)
            self.stages.append((conv, bn, act))
        self.pool = GlobalAvgPool()
        self.graphed = None

    def stages_and_pool(self, x):
        with torch.no_grad():
            for conv, bn, act in self.stages:
                x = act(bn(conv(x)))
            return self.pool(x)

    def submit(self, points, feats, ids):
        """Voxelise eagerly (its voxel count sizes the rest), then the four stages + global pool
        replayed as one recorded CUDA graph (two recordings on two streams: the next batch is queued
        while this one runs).  Returns the queued batch; .result() is the pooled [B, C] tensor."""
        from ss_conv.graph import GraphedChain
        with torch.no_grad():
            x = self.p2v(points, feats, ids)[1]
            if self.graphed is None:
                self.graphed = GraphedChain(self.stages_and_pool, x.spatial_shape, x.batch_size, x.features.shape[1],
                                            int(x.features.shape[0] * 1.05) + 64, x.features.device, depth=2, streams=2)
            return self.graphed.submit(x)   # the voxel count stays on the device (checked after the replay)

    def forward(self, points, feats, ids):
        return self.submit(points, feats, ids).result()


def run_backbone(args, dev, rank, world, dist):
    """Backbone samples/s at a global batch of 256 split by sample over the ranks, including the
    all-gather of the pooled per-sample features (the only collective)."""
    from ss_conv import parallel
    from ss_conv.utils import synthetic as S
    cfg = BACKBONE
    lo, hi = parallel.shard_range(cfg["global_batch"], rank, world)
    pts, fts, ids = S.object_points(range(lo, hi), cfg["n_pts"], base_seed=7000)
    pts, fts, ids = (torch.from_numpy(a).to(dev) for a in (pts, fts, ids))
    net = Backbone(cfg, dev)
    steps = max(3, min(args.steps, 15))

    def step():
        pooled = net.forward(pts, fts, ids)
        return parallel.all_gather_rows(pooled, cfg["global_batch"])

    for _ in range(3):
        out = step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    queued = None
    for _ in range(steps):                     # batch s+1 is voxelised and queued before batch s is waited for
        nxt = net.submit(pts, fts, ids)
        if queued is not None:
            out = parallel.all_gather_rows(queued.result(), cfg["global_batch"])
        queued = nxt
    out = parallel.all_gather_rows(queued.result(), cfg["global_batch"])
    b.record()
    torch.cuda.synchronize()
    ms = torch.tensor([a.elapsed_time(b)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    assert out.shape == (cfg["global_batch"], 240)
    return {"metric": "backbone samples/sec", "value": cfg["global_batch"] * steps / (float(ms) * 1e-3), "unit": "samples/s",
            "global_batch": cfg["global_batch"], "steps": steps, "ms_per_step": float(ms) / steps, "scaling": "strong",
            "workload": cfg["name"] + "; stages + pool replayed as one CUDA graph (two recordings on two streams) after an eager Point2Voxel, batch s+1 voxelised and queued before batch s is waited for", "collective": "all_gather of pooled [B/G,240] fp32 rows" if world > 1 else "none"}


def make_inputs(cfg, sample_base, n_sets):
    from ss_conv.utils import synthetic as S
    sets = []
    for r in range(n_sets):
        ids = range(sample_base + r * cfg["batch"], sample_base + (r + 1) * cfg["batch"])
        ind = S.surface_voxels(ids, cfg["V"], cfg["n_pts"], base_seed=1000)
        feats = S.features(ind.shape[0], sum(m * (2 * l + 1) for l, m in enumerate(cfg["irreps"])), 77 + r)
        sets.append((feats, ind))
    return sets


def run_ours(args):
    from ss_conv import _ext
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback); use --impl reference for the CPU arm")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    cfg = CFG2
    _ext.set_precision("tf32")
    layer = Layer(cfg, dev)
    host_sets = make_inputs(cfg, rank * ROTATE * cfg["batch"], ROTATE)
    dev_sets = [(torch.from_numpy(f).to(dev), torch.from_numpy(i).to(dev)) for f, i in host_sets]
    pinned = [(torch.from_numpy(f).pin_memory(), torch.from_numpy(i).pin_memory()) for f, i in host_sets]
    n_in = [int(i.shape[0]) for _, i in host_sets]

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    # ---- device-resident throughput.  The step (rulebook + materialise + pack + stage + conv +
    # pool rulebook + max pool) is recorded as a CUDA graph over capacity-sized buffers with
    # the row counts kept on the device (ss_conv.graph.GraphedChain).  The chain is recorded once per
    # rotating batch (ROTATE recordings, each with buffers of its own) and every batch is loaded into
    # the input buffers of its recording before the timed region: the inputs are resident in HBM where
    # the kernels read them, a timed step is the replay of the whole layer pass on one batch plus the
    # read-back and check of its row counts.  Step s+1 is queued before the host waits for step s, so
    # the device does not idle during that round trip; the output of a step stays valid while the next
    # ones run.  (The end-to-end loop below feeds new data every step.)
    from ss_conv.graph import GraphedChain
    from ss_conv.sp_ops.tensor import SparseTensor

    def chain(x):
        with torch.no_grad():
            return layer.pool(layer.conv(x))

    def timed_steps(depth, streams, lag):
        """steps/s of the recorded step: `depth` recordings (recording k holds rotating batch k % ROTATE),
        replayed round-robin on `streams` streams, each result taken `lag` steps after its submission."""
        g = GraphedChain(chain, [cfg["V"]] * 3, cfg["batch"], layer.conv.in_channels, max(n_in), dev, depth=depth, streams=streams)
        for k in range(depth):
            g.load(k, *dev_sets[k % ROTATE])
        for w in range(max(args.warmup, depth)):
            g.submit_loaded(w % depth).result()
        barrier()
        r0, f0 = g.replays, g.fallbacks
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        vox, waiting = 0, []
        t_submit = t_result = 0.0
        for s in range(args.steps):
            t0 = time.perf_counter()
            waiting.append(g.submit_loaded(s % depth))
            t1 = time.perf_counter()
            if len(waiting) > lag:
                waiting.pop(0).result()         # an earlier step: wait, check the row counts, exact tensors
            t2 = time.perf_counter()
            t_submit += t1 - t0
            t_result += t2 - t1
            vox += n_in[(s % depth) % ROTATE]
        for q in waiting:
            q.result()
        e1.record()
        barrier()
        host_us[0], host_us[1] = t_submit / args.steps * 1e6, t_result / args.steps * 1e6
        return g, e0.elapsed_time(e1), vox, g.replays - r0, g.fallbacks - f0

    host_us = [0.0, 0.0]    # host time per step of the last timed_steps call: queueing a step / waiting for and checking one

    DEPTH, STREAMS, LAG = 6, 3, 2
    with ClockSampler(local, enabled=(rank == 0)) as clk:
        graphed, ms, voxels, n_replays, graph_fallbacks = timed_steps(DEPTH, STREAMS, LAG)
    launches = n_replays * graphed.launches
    host_submit_us, host_result_us = host_us
    _ext.check_status(dev)
    # the same loop with fp16 operands in the convolution (opt-in precision; reported beside the headline)
    _ext.set_precision("fp16")
    try:
        g16, ms16, vox16, _, fb16 = timed_steps(DEPTH, STREAMS, LAG)
    finally:
        _ext.set_precision("tf32")
    f16_step_ms = ms16 / args.steps
    del g16
    # the same step launched kernel by kernel from Python, for comparison
    eager_steps = min(args.steps, 20)
    for w in range(3):
        layer.step(*dev_sets[w % ROTATE]).resolve()
    barrier()
    eg0, eg1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    eg0.record()
    for s in range(eager_steps):
        layer.step(*dev_sets[s % ROTATE]).resolve()
    eg1.record()
    barrier()
    eager_ms = eg0.elapsed_time(eg1) / eager_steps
    n_out_conv = None

    # ---- end to end from pinned host buffers through the public API: every step uploads its own
    # indices + features from pinned host memory and downloads its pooled result; HostStream
    # overlaps the upload of step s+1 and the download of step s-1 with the compute of step s.
    from ss_conv.pipeline import HostStream

    def dev_step(fd, idd):
        o = graphed(fd, idd)            # the recorded step (its buffers are reused by the next replay)
        return o.features, o.indices

    feed = HostStream(dev_step, dev, max_rows=max(n_in), step_reuses_outputs=True)
    for _ in feed.run(pinned[w % ROTATE] for w in range(3)):
        pass
    barrier()
    t0 = time.perf_counter()
    d2h = 0
    for of, oi in feed.run(pinned[s % ROTATE] for s in range(args.steps)):
        d2h = of.numel() * 4 + oi.numel() * 4
    barrier()
    e2e_s = time.perf_counter() - t0
    vox_e2e = sum(n_in[s % ROTATE] for s in range(args.steps))
    h2d = int(np.mean([f.numel() * 4 + i.numel() * 4 for f, i in pinned]))

    # the same without overlap (upload, compute, download one after the other), for comparison
    def serial_step(s):
        f, i = pinned[s % ROTATE]
        o = graphed(f.to(dev, non_blocking=True), i.to(dev, non_blocking=True))
        return o.features.cpu(), o.indices.cpu()

    serial_step(0)
    barrier()
    t0 = time.perf_counter()
    for s in range(args.steps):
        serial_step(s)
    barrier()
    serial_s = time.perf_counter() - t0

    # ---- dominant kernel alone: conv_fwd_tf32_kernel, CUDA events on the launching stream
    from ss_conv.sp_ops.ops import get_indice_pairs
    kern_ms, alg_bytes, flops = [], [], []
    prepared = []
    with torch.no_grad():
        flt = layer.conv.kernel.filters().reshape(-1, layer.conv.in_channels, layer.conv.out_channels)
        for f, i in dev_sets:
            outids, pairs, num = get_indice_pairs(i, cfg["batch"], [cfg["V"]] * 3, cfg["k"], cfg["stride"], cfg["pad"])
            prepared.append((f, _ext.neighbour_table(pairs, num, outids.shape[0]), outids.shape[0], int(num.sum().item())))
        # the two launches of the convolution call (stage + conv) are recorded as a small CUDA graph per
        # input batch, so that the CUDA events around a replay see device time only (no host gaps)
        conv_graphs = []
        for f, nbr, n_out, P in prepared:
            _ext.conv_forward(f, flt, nbr, n_out, "tf32")
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                _ext.conv_forward(f, flt, nbr, n_out, "tf32")
            conv_graphs.append(g)
        for it in range(3 + 12):
            f, nbr, n_out, P = prepared[it % ROTATE]
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            conv_graphs[it % ROTATE].replay()
            b.record()
            torch.cuda.synchronize()
            if it >= 3:
                kern_ms.append(a.elapsed_time(b))
                K, ci, co = flt.shape
                alg_bytes.append(4 * (f.shape[0] * ci + n_out * co + K * ci * co) + 8 * P)
                flops.append(2.0 * P * ci * co)
    n_out_conv = prepared[0][2]
    # ---- the same call with fp16 operands (opt-in precision 'fp16'; not the headline configuration)
    f16_ms = []
    with torch.no_grad():
        f16_graphs = []
        for f, nbr, n_out, P in prepared:
            _ext.conv_forward(f, flt, nbr, n_out, "fp16")
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                _ext.conv_forward(f, flt, nbr, n_out, "fp16")
            f16_graphs.append(g)
        for it in range(3 + 12):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            f16_graphs[it % ROTATE].replay()
            b.record()
            torch.cuda.synchronize()
            if it >= 3:
                f16_ms.append(a.elapsed_time(b))
        del f16_graphs
    # ---- backward of the same layer (input gradient through the tcgen05 kernel on the input-major
    #      table, tensor-core filter gradient), CUDA events, the rulebook of the forward pass reused
    bwd_ms = []
    with torch.no_grad():
        grads = [torch.randn(n_out, flt.shape[2], device=dev) for _, _, n_out, _ in prepared]
        tables = []
        for (f, i), (_, nbr, n_out, _) in zip(dev_sets, prepared):
            nbr_in = _ext.input_major_table(nbr, f.shape[0])
            tables.append((nbr, nbr_in, _ext.nbr_row_order(nbr_in)))   # tables + row order: per rulebook, reused
        fltT = flt.transpose(1, 2).contiguous()
        bwd_graphs = []
        for k in range(ROTATE):                       # recorded like the forward call: device time only
            f, (nbr, nbr_in, order), g = prepared[k][0], tables[k], grads[k]
            _ext.conv_backward(f, flt, g, nbr, nbr_in, order, "tf32")
            torch.cuda.synchronize()
            cg = torch.cuda.CUDAGraph()
            with torch.cuda.graph(cg):
                keep = _ext.conv_backward(f, flt, g, nbr, nbr_in, order, "tf32")   # the two gradients on parallel branches
            bwd_graphs.append((cg, keep))
        for it in range(2 + 6):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            bwd_graphs[it % ROTATE][0].replay()
            b.record()
            torch.cuda.synchronize()
            if it >= 2:
                bwd_ms.append(a.elapsed_time(b))
    peak, peak_src = peaks()
    achieved = float(np.mean(alg_bytes)) / (float(np.mean(kern_ms)) * 1e-3) / 1e9

    backbone = run_backbone(args, dev, rank, world, dist)
    _ext.set_precision("tf32")

    # ---- reduce over ranks
    stats = torch.tensor([ms, e2e_s, float(voxels), float(vox_e2e), float(launches), serial_s, eager_ms, host_submit_us, host_result_us], dtype=torch.float64, device=dev)
    if world > 1:
        mx = stats.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        sm = stats.clone()
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        ms, e2e_s, serial_s, eager_ms = float(mx[0]), float(mx[1]), float(mx[5]), float(mx[6])
        host_submit_us, host_result_us = float(mx[7]), float(mx[8])
        voxels, vox_e2e, launches = float(sm[2]), float(sm[3]), float(sm[4])
    if rank == 0:
        line = {
            "metric": "active voxels/sec per SS-Conv layer", "value": voxels / (ms * 1e-3), "unit": "voxels/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "tf32 operands, f32 accumulate",
            "data": "synthetic (seeded ellipsoid-surface voxels, N(0,1) features, reference-style N(0,1) kernel weights)",
            "config": {"workload": cfg["name"], "n_in_per_batch": n_in[0], "n_out_conv": n_out_conv,
                       "c_in": layer.conv.in_channels, "c_out": layer.conv.out_channels,
                       "l2": "%d recordings with buffers of their own (inputs, tables, staging, outputs: > 1 GB working set) holding %d "
                             "distinct input batches, replayed in turn: nothing a step reads is still in L2 from its last replay"
                             % (DEPTH, ROTATE),
                       "step": "rulebook + materialise + pack + stage + conv + pool rulebook + maxpool, replayed as one "
                               "CUDA graph (device-side row counts, capacity-sized buffers), one recording per rotating batch "
                               "with the batch resident in its input buffers; a step = replay + read-back and check of the "
                               "row counts, step s+1 queued before the host checks step s; the recordings replay on three "
                               "streams in turn (6 recordings, results taken two steps late), so consecutive steps overlap on the device",
                       "eager_ms_per_step": eager_ms, "graph_fallbacks": graph_fallbacks,
                       "host_us_per_step": {"queue_a_step": host_submit_us, "wait_for_and_check_a_step": host_result_us,
                                            "note": "host time in the timed loop (max over ranks); the second includes waiting for the device"},
                       "parallelism": "sample-sharded x%d, no data-path collective" % world},
            "e2e": {"value": vox_e2e / e2e_s, "unit": "voxels/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": int(d2h),
                    "how": "ss_conv.pipeline.HostStream (upload / compute / download of consecutive steps overlap on 3 streams) "
                           "around the CUDA-graph replay of the step",
                    "serial_value": vox_e2e / serial_s},
            "gpu_launches": int(launches),
            "clocks": clk.summary(),
            "roofline": {"bound": "hbm", "kernel": "stage_features_kernel + conv_fwd_tf32_kernel", "achieved": achieved,
                         "peak": peak, "unit": "GB/s", "frac": achieved / peak, "traffic": CONV_DRAM_TRAFFIC,
                         "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of conv_fwd_tf32_kernel on the "
                                           "cfg2 inputs (profiles/conv_fwd_tf32_cfg2.md)",
                         "peak_source": peak_src,
                         "kernel_ms": float(np.mean(kern_ms)), "algorithmic_bytes": float(np.mean(alg_bytes)),
                         "tensor_tflops": float(np.mean(flops)) / (float(np.mean(kern_ms)) * 1e-3) / 1e12},
        }
        line["backward"] = {"what": "input gradient (forward kernel on the input-major table, rows grouped by parity class) + filter gradient (pair lists compacted inside the call) of the cfg2 convolution, both tcgen05 with TF32 operands; input-major table and row order come with the rulebook",
                            "ms": float(np.mean(bwd_ms)), "voxels_per_s": float(np.mean(n_in)) / (float(np.mean(bwd_ms)) * 1e-3)}
        line["fp16_operands"] = {"what": "the convolution call (stage + conv) of the same layer with precision 'fp16': fp16 "
                                         "operands, f32 accumulate (opt-in; the headline numbers above use TF32 operands)",
                                 "conv_call_ms": float(np.mean(f16_ms)), "tf32_conv_call_ms": float(np.mean(kern_ms)),
                                 "step_ms": f16_step_ms, "step_what": "the timed step loop above with precision 'fp16' (this rank)"}
        line["backbone"] = backbone
        if world == 1:
            line["cpu_baseline"] = cpu_baseline(cfg, budget_s=12.0)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_only(args):
    """A few launches of one kernel group on the cfg2 inputs (small, fixed launch count)."""
    from ss_conv import _ext
    from ss_conv.sp_ops.ops import get_indice_pairs
    dev = torch.device("cuda", 0)
    cfg = CFG2
    _ext.set_precision("tf32")
    layer = Layer(cfg, dev)
    f, i = make_inputs(cfg, 0, 1)[0]
    f, i = torch.from_numpy(f).to(dev), torch.from_numpy(i).to(dev)
    if args.only == "step":
        for _ in range(max(1, args.steps)):
            out = layer.step(f, i)
        torch.cuda.synchronize()
        _ext.check_status(dev)
        print("only=step done, n_in=%d n_pooled=%d" % (i.shape[0], out.indices.shape[0]))
        return
    with torch.no_grad():
        flt = layer.conv.kernel.filters().reshape(-1, layer.conv.in_channels, layer.conv.out_channels)
        for _ in range(max(1, args.steps)):
            outids, pairs, num = get_indice_pairs(i, cfg["batch"], [cfg["V"]] * 3, cfg["k"], cfg["stride"], cfg["pad"])
            if args.only == "conv":
                nbr = _ext.neighbour_table(pairs, num, outids.shape[0])
                for _ in range(4):
                    _ext.conv_forward(f, flt, nbr, outids.shape[0], "tf32")
            elif args.only == "conv_fp16":
                nbr = _ext.neighbour_table(pairs, num, outids.shape[0])
                for _ in range(4):
                    _ext.conv_forward(f, flt, nbr, outids.shape[0], "fp16")
            elif args.only == "backward":     # input gradient (plain and grouped rows) + filter gradient
                nbr = _ext.neighbour_table(pairs, num, outids.shape[0])
                nbr_in = _ext.input_major_table(nbr, i.shape[0])
                order = _ext.nbr_row_order(nbr_in)
                g = torch.randn(outids.shape[0], flt.shape[2], device=dev)
                fltT = flt.transpose(1, 2).contiguous()
                for _ in range(2):
                    _ext.conv_forward(g, fltT, nbr_in, i.shape[0], "tf32")
                    _ext.conv_forward(g, fltT, nbr_in, i.shape[0], "tf32", row_order=order)
                    _ext.conv_wgrad(f, g, nbr)
    torch.cuda.synchronize()
    _ext.check_status(dev)
    print("only=%s done, n_in=%d n_out=%d" % (args.only, i.shape[0], outids.shape[0]))


# ------------------------------------------------------------------------ CPU reference
def ref_step_fn(cfg):
    """One CPU step of the reference's own code path on `n_samples` samples:
    get_indice_pairs_3d + indice_conv_fp32 + pool rulebook + indice_maxpool_fp32 on CPU tensors
    (SS_Conv_lib/src/conv/indice_conv.h:21-131,247-343, SS_Conv_lib/src/pool/indice_maxpool.h:15-50).
    Falls back to the numpy restatement when the compiled reference is absent."""
    from ref_loader import load_ref_ext
    import ssconv_oracle as O
    ext = load_ref_ext()
    V, k, s, p = cfg["V"], cfg["k"], cfg["stride"], cfg["pad"]
    osz = O.conv_output_size([V] * 3, [k] * 3, [s] * 3, [p] * 3, [1] * 3)
    psz = O.conv_output_size(osz, [cfg["pool_k"]] * 3, [cfg["pool_s"]] * 3, [0] * 3, [1] * 3)
    if ext is not None:
        def step(feats, ind, W, batch):
            ti = torch.from_numpy(ind)
            o, pr, n = ext.get_indice_pairs_3d(ti, batch, osz, [V] * 3, [k] * 3, [s] * 3, [p] * 3, [1] * 3, [0] * 3, 0, 0)
            y = ext.indice_conv_fp32(torch.from_numpy(feats), torch.from_numpy(W), pr, n, o.shape[0], 0, 0)
            o2, pr2, n2 = ext.get_indice_pairs_3d(o.contiguous(), batch, psz, osz, [cfg["pool_k"]] * 3, [cfg["pool_s"]] * 3,
                                                  [0] * 3, [1] * 3, [0] * 3, 0, 0)
            return ext.indice_maxpool_fp32(y, pr2, n2, o2.shape[0])
        return step, "reference"

    def step(feats, ind, W, batch):
        o, pr, n = O.get_indice_pairs(ind, batch, [V] * 3, k, s, p, 1, False)
        y = O.indice_conv(feats, W, pr, n, o.shape[0])
        o2, pr2, n2 = O.get_indice_pairs(o, batch, osz, cfg["pool_k"], cfg["pool_s"], 0, 1, False)
        return O.indice_maxpool(y, pr2, n2, o2.shape[0])
    return step, "port"


def cpu_inputs(cfg, n_samples):
    from ss_conv.utils import synthetic as S
    ind = S.surface_voxels(range(n_samples), cfg["V"], cfg["n_pts"], base_seed=1000)
    ci = sum(m * (2 * l + 1) for l, m in enumerate(cfg["irreps"]))
    co = ci + sum(cfg["irreps"][1:])
    feats = S.features(ind.shape[0], ci, 77)
    W = (np.random.RandomState(5).randn(cfg["k"], cfg["k"], cfg["k"], ci, co) / np.sqrt(ci * cfg["k"] ** 3)).astype(np.float32)
    return feats, ind, W


def cpu_baseline(cfg, budget_s=12.0, n_samples=8):
    step, kind = ref_step_fn(cfg)
    feats, ind, W = cpu_inputs(cfg, n_samples)
    step(feats, ind, W, n_samples)  # warm-up
    t0 = time.perf_counter()
    reps = 0
    while reps < 3 or (time.perf_counter() - t0 < budget_s and reps < 200):
        step(feats, ind, W, n_samples)
        reps += 1
    dt = time.perf_counter() - t0
    return {"value": ind.shape[0] * reps / dt, "unit": "voxels/s", "cores": torch.get_num_threads(), "kind": kind,
            "host_cpus": os.cpu_count(),
            "sample": "%d of %d samples of the cfg2 batch (%d active voxels), %d repetitions, same step "
                      "(rulebook + conv + pool rulebook + maxpool; filters pre-materialised); rulebook/gather/scatter "
                      "are single-threaded C++ loops, the GEMM uses torch's CPU threads" % (n_samples, cfg["batch"], ind.shape[0], reps)}


def run_reference(args):
    rank = int(os.environ.get("RANK", 0))
    if rank != 0:
        return
    cfg = CFG2
    n_samples = 8
    step, kind = ref_step_fn(cfg)
    feats, ind, W = cpu_inputs(cfg, n_samples)
    for _ in range(max(1, min(args.warmup, 3))):
        step(feats, ind, W, n_samples)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step(feats, ind, W, n_samples)
    dt = time.perf_counter() - t0
    value = ind.shape[0] * args.steps / dt
    sample = ("each step = %d of the %d samples of the cfg2 batch (%d active voxels) through the reference's C++ CPU "
              "path" % (n_samples, cfg["batch"], ind.shape[0]))
    line = {"impl": "reference", "metric": "active voxels/sec per SS-Conv layer", "value": value, "unit": "voxels/s",
            "n_gpus": int(os.environ.get("WORLD_SIZE", 1)), "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic (same generator as the GPU arm)",
            "config": {"workload": cfg["name"], "sample": sample},
            "cpu_baseline": {"value": value, "unit": "voxels/s", "cores": torch.get_num_threads(), "kind": kind,
                             "host_cpus": os.cpu_count(), "sample": sample},
            "e2e": {"value": value, "unit": "voxels/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--only", default=None, choices=["conv", "conv_fp16", "backward", "rulebook", "step"],
                    help="run just one kernel group of the cfg2 step (or the whole step) a few times (for ncu captures)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    elif args.only:
        run_only(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
