"""Benchmark of the sparse steerable convolution hot path on B200.

Headline workload ("cfg2", the configuration the metric is quoted on): a strided
downsampling SS-Conv layer, irreps (4,4,4,4) = 64 channels in, 64 + 12 gate scalars = 76 out,
kernel 3, stride 2, padding 1, batch 32 on a 64^3 grid with 16384 ellipsoid-surface points per
sample (seeded synthetic stand-in for object-surface data), followed by a sparse MaxPool
(kernel 2, stride 2).  One step = rulebook + filter materialisation + packing +
gather-GEMM (tcgen05, TF32 operands, fp32 accumulate) + pool rulebook + max pool.

metric  : active input voxels per second through the layer (whole job, all ranks)
value   : inputs resident in HBM, CUDA-event timed; the --steps-long region is repeated REGIONS
          times, the median region counts, max over ranks
e2e     : the same step through the public ss_conv API starting from pinned HOST buffers
          (H2D of indices+features and D2H of the pooled features of every step inside the timed
          region; ss_conv.pipeline.HostStream overlaps the copies of neighbouring steps)
roofline: dominant call (stage_features_kernel + conv_fwd_tf32_kernel): algorithmic bytes / its
          CUDA-event time
layers  : the other layer configurations (cfg1, stage 2 of the cfg3 backbone, the wide cfg5 layer):
          rulebook and convolution call, useful TFLOP/s against the tensor-pipe peak
helpers : the bandwidth-bound helper kernels, achieved GB/s against the measured HBM peak
reference_gpu : the reference's own CUDA path (its extension, compiled from its sources) on the same
          device and the same cfg2 batch - the kernel to beat, not part of the timed arm
cpu_baseline / --impl reference: the reference's own C++ CPU path (oracle/_ref, built from the
          reference sources) on the box's host cores, full cfg2 batch.

python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--only ...]
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
# DRAM bytes per launch of the two kernels of the cfg2 convolution call (dram__bytes_read.sum +
# dram__bytes_write.sum), from:  ncu --metrics dram__bytes_read.sum,dram__bytes_write.sum
#   --clock-control none -k regex:"stage_features|conv_fwd_tf32" -c 8 python bench.py --only conv --steps 1
# (staging: 61.4 MB read + 10.9 MB written back, most of the staged image stays in L2;
#  convolution: 76.0 MB read + 1.0 MB written)
NCU_DRAM_BYTES = {"stage_features_kernel": 72.3e6, "conv_fwd_tf32_kernel": 77.0e6}
ROTATE = 4    # distinct input batches cycled through so the working set exceeds the 126 MB L2
REGIONS = 25  # repetitions of the --steps-long timed region; the median region is reported


def rs_of(irreps, gates=False):
    rs = [(m, l) for l, m in enumerate(irreps)]
    if gates:
        rs = rs + [(sum(irreps[1:]), 0)]
    return rs


def channels(irreps, gates=False):
    return sum(m * (2 * l + 1) for l, m in enumerate(irreps)) + (sum(irreps[1:]) if gates else 0)


def peaks():
    """(HBM GB/s, bf16 TFLOP/s burst, source).  TF32 peak is taken as half the bf16 figure."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return float(p["hbm_gbs"]), float(p["bf16_tflops"]), "measured (MEASURED_PEAKS.json: hbm_gbs, bf16_tflops burst; TF32 taken as half of bf16)"
    return 6650.0, 1590.0, "fallback (6.65 TB/s, 1.59 PFLOP/s bf16; TF32 taken as half)"


def pin_rank_to_cores(local, world):
    """Give every rank of the node its own slice of the host cores (by default all ranks share all
    cores and one descheduled Python host halves a max-over-ranks number).  Returns the slice."""
    try:
        cores = sorted(os.sched_getaffinity(0))
        per = max(1, len(cores) // max(1, world))
        mine = cores[local * per:(local + 1) * per] or cores
        os.sched_setaffinity(0, set(mine))
        torch.set_num_threads(max(1, len(mine)))
        return mine
    except Exception:
        return []


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken while the timed region runs: ONE
    nvidia-smi process in loop mode (started before the region, stopped after it)."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index, enabled=True, core=None):
        self.index, self.samples, self.proc, self.enabled, self.core = index, [], None, enabled, core

    def __enter__(self):
        if self.enabled:
            try:
                self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                              "--format=csv,noheader,nounits", "-lms", "100"],
                                             stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
                if self.core is not None:   # keep the sampler off the core that feeds the GPU
                    try:
                        os.sched_setaffinity(self.proc.pid, {self.core})
                    except Exception:
                        pass
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


def graph_ms(fn, reps=20, warm=2):
    """Median device time of fn() in ms: fn is recorded into a CUDA graph (it must not wait for the
    device) and every replay is bracketed by CUDA events, so host gaps between launches do not count."""
    for _ in range(warm):
        keep = fn()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        keep = fn()
    ts = []
    for it in range(reps + 2):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        g.replay()
        b.record()
        torch.cuda.synchronize()
        if it >= 2:
            ts.append(a.elapsed_time(b))
    del keep
    return float(statistics.median(ts))


def eager_ms(fn, reps=10, warm=2):
    """Median time of fn() launched from Python (CUDA events); for calls that wait for the device."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(reps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    return float(statistics.median(ts))


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
                     "GlobalAvgPool, irreps (3)->(8,4,2)->(16,8,4)->(32,16,8)->(64,32,16), 1024 points/object",
                irreps=[(3,), (8, 4, 2), (16, 8, 4), (32, 16, 8), (64, 32, 16)], V=32, n_pts=1024, global_batch=256)


class Backbone:
    """The 4-stage backbone of the benchmark configurations, from the public ss_conv modules.
    Voxelizer, stages and global pool are recorded together into CUDA graphs (ss_conv.graph.GraphedPoints:
    `depth` recordings replayed in turn on `streams` streams), so a batch costs the host three small
    copies, one graph launch and one read-back of the row counts."""

    def __init__(self, cfg, device, objects, depth=4, streams=2):
        from ss_conv.activation import Activation
        from ss_conv.batchnorm import BatchNorm
        from ss_conv.convolution import Convolution
        from ss_conv.pool import GlobalAvgPool
        from ss_conv.sp_ops.voxelize import Point2Voxel
        torch.manual_seed(4321)
        V = cfg["V"]
        self.cfg, self.dev, self.objects = cfg, device, int(objects)
        self.p2v = Point2Voxel([V] * 3, [1.0 / V] * 3, 4, trusted_batch_size=self.objects)
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
        from ss_conv.graph import GraphedPoints
        self.graphed = GraphedPoints(self.p2v, self.stages_and_pool, self.objects * cfg["n_pts"], 3, device,
                                     depth=depth, streams=streams)

    def stages_and_pool(self, x):
        with torch.no_grad():
            for conv, bn, act in self.stages:
                x = act(bn(conv(x)))
            return self.pool(x)

    def submit(self, points, feats, ids):
        return self.graphed.submit(points, feats, ids)


def run_backbone(args, dev, rank, world, dist, objects_per_rank, scaling, overlap=(8, 4, 7)):
    """Backbone samples/s: every rank runs `objects_per_rank` objects per batch, then one all-gather
    of the pooled [objects, 240] rows (the only collective).  `lag` batches are in flight before the
    host waits for the oldest one."""
    from ss_conv import parallel
    from ss_conv.utils import synthetic as S
    cfg = BACKBONE
    total = objects_per_rank * world
    lo = rank * objects_per_rank
    pts, fts, ids = S.object_points(range(lo, lo + objects_per_rank), cfg["n_pts"], base_seed=7000)
    pts, fts, ids = (torch.from_numpy(a).to(dev) for a in (pts, fts, ids))
    ids = ids.int()
    DEPTH, STREAMS, LAG = overlap      # recordings, streams, batches in flight before the host waits
    net = Backbone(cfg, dev, objects_per_rank, depth=DEPTH, streams=STREAMS)
    gather = parallel.RowGatherer(total, 240, dev)
    steps = max(8, min(args.steps, 40))

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    t_host = {"submit": 0.0, "result": 0.0, "gather": 0.0}

    def region(n_steps, clock=False):
        waiting, out = [], None
        for _ in range(n_steps):
            t0 = time.perf_counter()
            waiting.append(net.submit(pts, fts, ids))
            t1 = time.perf_counter()
            if len(waiting) > LAG:
                pooled = waiting.pop(0).result()
                t2 = time.perf_counter()
                out = gather(pooled)
                t3 = time.perf_counter()
                if clock:
                    t_host["result"] += t2 - t1
                    t_host["gather"] += t3 - t2
            if clock:
                t_host["submit"] += t1 - t0
        for q in waiting:
            out = gather(q.result())
        return out

    out = region(max(4, DEPTH + 1))      # records the graphs, warms NCCL up
    barrier()
    regions = []
    for r in range(9):
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        out = region(steps, clock=True)
        b.record()
        torch.cuda.synchronize()
        regions.append(a.elapsed_time(b))
    assert out.shape == (total, 240)
    # device-only time of one replay (no overlap with its neighbours) and of the voxelizer inside it
    rec = net.graphed.recs[0]
    torch.cuda.synchronize()
    solo = []
    for _ in range(5):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        rec.graph.replay()
        b.record()
        torch.cuda.synchronize()
        solo.append(a.elapsed_time(b))
    ms = torch.tensor([statistics.median(regions)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    n_clocked = 9 * steps
    return {"metric": "backbone samples/sec", "value": total * steps / (float(ms) * 1e-3), "unit": "samples/s",
            "global_batch": total, "objects_per_gpu": objects_per_rank, "steps": steps, "regions": len(regions),
            "ms_per_step": float(ms) / steps, "scaling": scaling,
            "ms_per_step_split": {"one_replay_alone_device_ms": float(statistics.median(solo)),
                                  "host_us_queue_a_batch": t_host["submit"] / n_clocked * 1e6,
                                  "host_us_wait_and_check_a_batch": t_host["result"] / n_clocked * 1e6,
                                  "host_us_all_gather_call": t_host["gather"] / n_clocked * 1e6,
                                  "graph_launches_per_batch": net.graphed.launches,
                                  "note": "voxelizer + 4 stages + global pool are ONE graph replay per batch (their kernels "
                                          "are not timed apart); host figures are wall time in the timed loop of this rank, "
                                          "the wait includes waiting for the device"},
            "graph_fallbacks": net.graphed.fallbacks,
            "workload": BACKBONE["name"] + "; %d objects per GPU; %d recordings on %d streams, %d batches in flight" % (objects_per_rank, DEPTH, STREAMS, LAG),
            "collective": "all_gather of pooled [%d,240] fp32 rows" % objects_per_rank if world > 1 else "none"}


def make_inputs(cfg, sample_base, n_sets):
    from ss_conv.utils import synthetic as S
    sets = []
    for r in range(n_sets):
        ids = range(sample_base + r * cfg["batch"], sample_base + (r + 1) * cfg["batch"])
        ind = S.surface_voxels(ids, cfg["V"], cfg["n_pts"], base_seed=1000)
        feats = S.features(ind.shape[0], channels(cfg["irreps"]), 77 + r)
        sets.append((feats, ind))
    return sets


# ---------------------------------------------------------------------- per-layer numbers
def layer_numbers(name, ind, batch, V, k, stride, pad, subm, c_in, c_out, precisions, dev, peak_hbm, peak_bf16):
    """Rulebook and convolution call of one layer configuration (filters given, not materialised):
    device time of the call (staging + kernel, recorded into a graph), useful TFLOP/s = 2 P Cin Cout / t."""
    from ss_conv import _ext
    from ss_conv.sp_ops.ops import get_indice_pairs
    g = torch.Generator(device="cpu").manual_seed(11)
    n_in = int(ind.shape[0])
    ti = torch.from_numpy(ind).to(dev)
    feats = torch.randn(n_in, c_in, generator=g).to(dev)
    K = k ** 3
    W = (torch.randn(K, c_in, c_out, generator=g) / float(np.sqrt(c_in * K))).to(dev)
    build = lambda: get_indice_pairs(ti, batch, [V] * 3, k, stride, pad, 1, 0, subm, False, lazy=True)  # noqa: E731
    outids, pairs, num = build()
    n_out = int(outids.shape[0])
    nbr = _ext.neighbour_table(pairs, num, n_out)
    P = int((nbr >= 0).sum().item())
    rb_ms = eager_ms(build, reps=7)
    res = {"name": name, "n_in": n_in, "n_out": n_out, "pairs": P, "c_in": c_in, "c_out": c_out, "kernel_offsets": K,
           "fill": P / float(K * n_out), "rulebook_ms": rb_ms,
           "rulebook_what": "table [K, n_out] through the public get_indice_pairs (launched from Python, includes its one read-back)"}
    flops = 2.0 * P * c_in * c_out
    alg_bytes = 4.0 * (n_in * c_in + n_out * c_out + K * c_in * c_out) + 8.0 * P
    res["algorithmic_bytes"], res["flops"] = alg_bytes, flops
    ceiling = None
    for prec in precisions:
        prec_id = _ext._PREC_OF[prec]
        uses_pairs = _ext._use_pairs(K, c_in, c_out, n_out, prec_id)
        if uses_pairs:
            _ext.pair_lists(nbr)          # built once per table (kept with it), like the table itself
        ms = graph_ms(lambda: _ext.conv_forward(feats, W, nbr, n_out, prec), reps=15)
        peak_t = peak_bf16 if prec in ("bf16", "fp16") else peak_bf16 / 2
        entry = {"conv_call_ms": ms, "kernel": "pair-list (conv_fwd_pairs_kernel)" if uses_pairs else "output-stationary (conv_fwd_tf32_kernel)",
                 "voxels_per_s": n_in / (ms * 1e-3), "useful_tflops": flops / (ms * 1e-3) / 1e12,
                 "frac_of_tensor_peak": flops / (ms * 1e-3) / 1e12 / peak_t, "tensor_peak_tflops": peak_t,
                 "frac_of_hbm_peak": alg_bytes / (ms * 1e-3) / 1e9 / peak_hbm}
        if uses_pairs:
            other = graph_ms(lambda: _ext.conv_forward(feats, W, nbr, n_out, prec, algo="rows"), reps=7)
            entry["output_stationary_ms"] = other
            entry["pair_lists_build_ms"] = eager_ms(lambda: _ext.pair_lists(nbr.clone()), reps=5)
            if ceiling is None:
                ceiling = scatter_add_ceiling(nbr, n_out, c_out, P)
            red_bytes = 4.0 * P * c_out
            entry["scatter_add"] = {"what": "the pair-list kernel adds every accumulator tile to scattered output rows with fp32 "
                                            "reductions at L2 (4 P Cout bytes per call); ceiling = a kernel that issues nothing but "
                                            "such reductions over the same row order (ssc_scatter_add_rate), timed here",
                                    "bytes_per_call": red_bytes, "ceiling_gbs": ceiling["ceiling_gbs"],
                                    "call_gbs": red_bytes / (ms * 1e-3) / 1e9,
                                    "frac_of_ceiling": red_bytes / (ms * 1e-3) / 1e9 / ceiling["ceiling_gbs"],
                                    "tflops_at_ceiling": ceiling["ceiling_gbs"] * 1e9 / (4.0 * c_out) * 2.0 * c_in * c_out / 1e12,
                                    "rates": {k: v for k, v in ceiling.items() if k != "ceiling_gbs"}}
        res[prec] = entry
    _ext.check_status(dev)
    return res


def scatter_add_ceiling(nbr, n_out, c_out, P):
    """GB/s of fp32 scatter-add reductions the device takes (nothing else running) over the output rows of
    the layer's pair lists: the ceiling (128 bytes per row and instruction, 16 warps per SM) and how the
    rate depends on the shape of a reduction instruction and on the number of issuing warps."""
    from ss_conv import _ext
    # the row order of the kernel's sweep: all offsets walk the output rows together, so at any time
    # the reductions fall into a window of rows that stays in L2; inside the window one offset after
    # the other (neighbouring list positions = distinct rows, as in a tile of the kernel)
    nz = torch.nonzero(nbr >= 0)
    window = 1280
    key = (nz[:, 1] // window) * nbr.shape[0] + nz[:, 0]
    order = nz[:, 1][torch.argsort(key, stable=True)].to(torch.int32).contiguous()
    width = (c_out + 31) // 32 * 32
    scratch = torch.zeros(n_out, width, device=nbr.device)
    sms = torch.cuda.get_device_properties(nbr.device).multi_processor_count

    def rate(lanes, warps):
        steps = max(1, -(-P // (sms * warps * 32)))
        nbytes = _ext.scatter_add_rate(scratch, order, steps, lanes, warps)
        ms = graph_ms(lambda: _ext.scatter_add_rate(scratch, order, steps, lanes, warps), reps=5)
        return nbytes / (ms * 1e-3) / 1e9

    return {"ceiling_gbs": rate(8, 16),
            "gbs_by_bytes_per_row_and_instruction_16_warps": {str(16 * lanes): rate(lanes, 16) for lanes in (1, 2, 4, 8)},
            "gbs_by_warps_per_sm_128_bytes_per_row": {str(w): rate(8, w) for w in (1, 2, 4, 8)}}


def layers_leg(dev, peak_hbm, peak_bf16):
    from ss_conv.utils import synthetic as S
    from ss_conv import _ext
    from ss_conv.sp_ops.ops import get_indice_pairs
    out = {"what": "convolution call = staging of the feature rows + kernel (filters given); tensor peak = measured bf16 "
                   "burst for 16-bit operands, half of it for TF32"}
    ind1 = S.surface_voxels(range(2), 32, 4096, base_seed=1000)
    out["cfg1"] = layer_numbers("cfg1: 32->38 ch, k3 s1 p1 regular, batch 2, 32^3", ind1, 2, 32, 3, 1, 1, False, 32, 38,
                                ("tf32",), dev, peak_hbm, peak_bf16)
    # stage 2 of the cfg3 backbone: its input voxels are the outputs of stage 1 (k3 s2 p1 on the 32^3 voxelization)
    pts, _, ids = S.object_points(range(64), 1024, base_seed=7000)
    cells = np.floor((pts + 0.5) * 32).astype(np.int64)
    vox = np.unique(np.concatenate([ids[:, None], cells], 1), axis=0).astype(np.int32)
    o1, _, _ = get_indice_pairs(torch.from_numpy(vox).to(dev), 64, [32] * 3, 3, 2, 1, 1, 0, False, False, lazy=True)
    out["cfg3_stage2"] = layer_numbers("cfg3 stage 2: 30->72 ch ((8,4,2) -> (16,8,4)+12 gates), k3 s2 p1, batch 64, 16^3",
                                       o1.cpu().numpy(), 64, 16, 3, 2, 1, False, 30, 72, ("tf32",), dev, peak_hbm, peak_bf16)
    ind5 = S.bernoulli_voxels(range(16), 48, 0.10, base_seed=40)
    out["cfg5"] = layer_numbers("cfg5: 256->256 ch, k5 submanifold (125 offsets), batch 16, 48^3, 10 % occupancy",
                                ind5, 16, 48, 5, 1, 2, True, 256, 256, ("tf32", "bf16"), dev, peak_hbm, peak_bf16)
    _ext.check_status(dev)
    return out


# ---------------------------------------------------------------------- helper kernels
def helper_cases(dev):
    """(name, fn, algorithmic bytes) of the bandwidth-bound helper ops on inputs larger than L2;
    fn() launches the op once through the library and does not wait for the device."""
    from ss_conv import _ext
    from ss_conv.sp_ops.ops import get_indice_pairs
    from ss_conv.utils import synthetic as S
    cases = []
    g = torch.Generator(device="cpu").manual_seed(3)
    # sparse pools on a cfg2-like conv output, four batches worth (input 159 MB)
    ind = S.surface_voxels(range(128), 64, 16384, base_seed=2000)
    ti = torch.from_numpy(ind).to(dev)
    o, _, _ = get_indice_pairs(ti, 128, [64] * 3, 3, 2, 1, 1, 0, False, False, lazy=True)
    po, pp, pn = get_indice_pairs(o, 128, [32] * 3, 2, 2, 0, 1, 0, False, False, lazy=True)
    C = 76
    y = torch.randn(o.shape[0], C, generator=g).to(dev)
    n_po = int(po.shape[0])
    nbr = _ext.neighbour_table(pp, pn, n_po)
    P = int((nbr >= 0).sum().item())
    pool_bytes = 4.0 * C * (o.shape[0] + n_po) + 8.0 * P
    cases.append(("maxpool k2 s2 (pool_fwd_kernel<max>)", lambda: _ext.indice_maxpool_fp32(y, pp, pn, n_po), pool_bytes))
    cases.append(("avgpool k2 s2 (pool_fwd_kernel<avg>)", lambda: _ext.indice_avgpool_fp32(y, pp, pn, n_po, None), pool_bytes))
    # global pools: 512 samples x 1200 rows x 240 channels (590 MB)
    B, rows, Cg = 512, 1200, 240
    gf = torch.randn(B * rows, Cg, generator=g).to(dev)
    off = (torch.arange(B + 1, dtype=torch.int32) * rows).to(dev)
    gout = torch.zeros(B, Cg, device=dev)
    gidx = torch.zeros(B, Cg, dtype=torch.int32, device=dev)
    gp_bytes = 4.0 * Cg * (B * rows + B)
    cases.append(("global avg pool (global_pool_kernel)", lambda: _ext.global_avgpool_fp(gf, off, gout, gidx, B, Cg), gp_bytes))
    cases.append(("global max pool (global_pool_kernel)", lambda: _ext.global_maxpool_fp(gf, off, gout, gidx, B, Cg), gp_bytes + 4.0 * B * Cg))
    # fused BatchNorm(eval) + gated activation on [N, 76] -> [N, 64] (2.4 M rows, 1.3 GB)
    from ss_conv.activation import Activation
    from ss_conv.batchnorm import BatchNorm
    from ss_conv.sp_ops.tensor import SparseTensor
    irreps = (4, 4, 4, 4)
    bn = BatchNorm(rs_of(irreps, gates=True)).to(dev).eval()
    act = Activation(rs_of(irreps), (torch.relu, torch.sigmoid), bias=False, checkpoint=False)
    nb = 2400000
    xb = torch.randn(nb, 76, generator=g).to(dev)
    ib = torch.zeros(nb, 4, dtype=torch.int32, device=dev)

    def bn_gate():
        with torch.no_grad():
            return act(bn(SparseTensor(xb, ib, [64] * 3, 1))).features
    cases.append(("BatchNorm(eval) + gate (bn_gate_rows_kernel)", bn_gate, 4.0 * nb * 76 + 4.0 * nb * 64))
    # voxelizer: 4 M points with 3 features into 64^3 x 64 samples
    from ss_conv.sp_ops.voxelize import Point2Voxel
    npt = 4 * 1024 * 1024
    rng = np.random.RandomState(5)
    pts = torch.from_numpy(rng.uniform(-0.499, 0.499, (npt, 3)).astype(np.float32)).to(dev)
    pf = torch.from_numpy(rng.rand(npt, 3).astype(np.float32)).to(dev)
    pid = torch.from_numpy(np.repeat(np.arange(64), npt // 64).astype(np.int32)).to(dev)
    p2v = Point2Voxel([64] * 3, [1.0 / 64] * 3, 4, trusted_batch_size=64)
    with torch.no_grad():
        m_vox = int(p2v(pts, pf, pid)[1].features.shape[0])
    cases.append(("Point2Voxel mean (p2v_* kernels)", lambda: p2v(pts, pf, pid)[1].raw()[0], 4.0 * npt * (3 + 3 + 1) + 4.0 * m_vox * (4 + 3)))
    # interpolation: 2 M points x 64 channels from 400 k voxels
    nq, mk, ci = 2 * 1024 * 1024, 400000, 64
    vfe = torch.randn(mk, ci, generator=g).to(dev)
    idx = torch.from_numpy(rng.randint(0, mk, (nq, 3)).astype(np.int32)).to(dev)
    w = torch.rand(nq, 3, generator=g).to(dev)
    iout = torch.empty(nq, ci, device=dev)
    # compulsory bytes: every voxel row read once, every point row written once, indices + weights
    # (the three gathered rows per point come from L2: the 102 MB of voxel features fit there)
    cases.append(("three_interpolate (three_interpolate_vec4_kernel)", lambda: _ext.three_interpolate_fp(ci, mk, nq, vfe, idx, w, iout),
                  4.0 * nq * ci + 4.0 * mk * ci + 24.0 * nq))
    # 3-NN: compute-bound brute force within a sample; reported as queries/s
    nn_q, nn_m, nn_b = 262144, 65536, 64
    kb = np.repeat(np.arange(nn_b), nn_m // nn_b)
    known = torch.from_numpy(np.concatenate([kb[:, None], rng.uniform(-0.5, 0.5, (nn_m, 3))], 1).astype(np.float32)).to(dev)
    ub = np.repeat(np.arange(nn_b), nn_q // nn_b)
    unk = torch.from_numpy(np.concatenate([ub[:, None], rng.uniform(-0.5, 0.5, (nn_q, 3))], 1).astype(np.float32)).to(dev)
    d2 = torch.empty(nn_q, 3, device=dev)
    i3 = torch.empty(nn_q, 3, dtype=torch.int32, device=dev)
    cases.append(("three_nn (three_nn_kernel), 4096 queries x 1024 voxels per sample", lambda: _ext.three_nn(nn_q, nn_m, unk, known, d2, i3),
                  16.0 * (nn_q + nn_m) + 24.0 * nn_q))
    # filter materialisation of the cfg2 layer (tiny: launch-bound)
    layer = Layer(CFG2, dev)

    def mat():
        with torch.no_grad():
            return layer.conv.kernel.filters()
    cases.append(("materialize_kernel (cfg2 filters)", mat, 4.0 * 27 * 64 * 76 + 4.0 * 22653 + 4.0 * 848))
    return cases


def helpers_leg(dev, peak_hbm):
    out = {"what": "device time of one call recorded into a CUDA graph (median of 10 replays); algorithmic bytes as in "
                   "bytes_pool / bytes_global_pool / bytes_bn_act / bytes_p2v; inputs larger than the 126 MB L2 except where noted"}
    for name, fn, nbytes in helper_cases(dev):
        ms = graph_ms(fn, reps=10)
        out[name] = {"ms": ms, "algorithmic_MB": nbytes / 1e6, "GBps": nbytes / (ms * 1e-3) / 1e9,
                     "frac_of_hbm_peak": nbytes / (ms * 1e-3) / 1e9 / peak_hbm}
    return out


# ------------------------------------------------------------------- reference on the GPU
def reference_gpu_leg(cfg, dev, our_step_ms, our_conv_ms):
    """The reference's own CUDA path (its extension built from its sources: SIMT rulebook kernels,
    gather + cuBLAS GEMM + scatter-add per offset, K pool launches; SS_Conv_lib/src/conv/indice_conv.h:247-343,
    indice_cuda_functor.cu:246-345) on CUDA tensors of the same cfg2 batch, on the same device."""
    try:
        from ref_loader import load_ref_ext
        import ssconv_oracle as O
        ext = load_ref_ext()
        if ext is None:
            return {"unavailable": "oracle/_ref has not been built (python oracle/build_ref.py)"}
        V, k, s, p = cfg["V"], cfg["k"], cfg["stride"], cfg["pad"]
        osz = O.conv_output_size([V] * 3, [k] * 3, [s] * 3, [p] * 3, [1] * 3)
        psz = O.conv_output_size(osz, [cfg["pool_k"]] * 3, [cfg["pool_s"]] * 3, [0] * 3, [1] * 3)
        feats, ind = make_inputs(cfg, 0, 1)[0]
        f, ti = torch.from_numpy(feats).to(dev), torch.from_numpy(ind).to(dev)
        ci, co = channels(cfg["irreps"]), channels(cfg["irreps"], gates=True)
        W = (torch.randn(k, k, k, ci, co) / float(np.sqrt(ci * k ** 3))).to(dev)

        def step():
            o, pr, n = ext.get_indice_pairs_3d(ti, cfg["batch"], osz, [V] * 3, [k] * 3, [s] * 3, [p] * 3, [1] * 3, [0] * 3, 0, 0)
            y = ext.indice_conv_fp32(f, W, pr, n, o.shape[0], 0, 0)
            o2, pr2, n2 = ext.get_indice_pairs_3d(o.contiguous(), cfg["batch"], psz, osz, [cfg["pool_k"]] * 3,
                                                  [cfg["pool_s"]] * 3, [0] * 3, [1] * 3, [0] * 3, 0, 0)
            return ext.indice_maxpool_fp32(y, pr2, n2, o2.shape[0])
        step_ms = eager_ms(step, reps=12, warm=3)
        o, pr, n = ext.get_indice_pairs_3d(ti, cfg["batch"], osz, [V] * 3, [k] * 3, [s] * 3, [p] * 3, [1] * 3, [0] * 3, 0, 0)
        conv_ms = eager_ms(lambda: ext.indice_conv_fp32(f, W, pr, n, o.shape[0], 0, 0), reps=12, warm=3)
        rb_ms = eager_ms(lambda: ext.get_indice_pairs_3d(ti, cfg["batch"], osz, [V] * 3, [k] * 3, [s] * 3, [p] * 3, [1] * 3, [0] * 3, 0, 0), reps=12, warm=3)
        return {"what": "the reference's extension (compiled from SS_Conv_lib/src for sm_100a) on CUDA tensors: "
                        "get_indice_pairs_3d + indice_conv_fp32 (fp32 cuBLAS, TF32 off) + pool rulebook + indice_maxpool_fp32, "
                        "filters given (no materialisation), launched from Python as the reference does; CUDA events, median of 12",
                "step_ms": step_ms, "voxels_per_s": ind.shape[0] / (step_ms * 1e-3), "rulebook_ms": rb_ms, "conv_ms": conv_ms,
                "ours_step_ms": our_step_ms, "ours_conv_call_ms": our_conv_ms,
                "speedup_step": step_ms / our_step_ms, "speedup_conv": conv_ms / our_conv_ms}
    except Exception as e:  # the anchor must never take the bench line down
        return {"unavailable": "reference CUDA path failed: %s" % (str(e)[:200])}


def run_ours(args):
    from ss_conv import _ext
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback); use --impl reference for the CPU arm")
    my_cores = pin_rank_to_cores(local, world)
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        # NCCL writes its version banner to stdout when the communicator comes up; stdout carries
        # ONE line (the JSON), so the banner goes to stderr
        sys.stdout.flush()
        saved = os.dup(1)
        os.dup2(2, 1)
        try:
            dist.init_process_group("nccl", device_id=dev)
            dist.barrier()
            torch.cuda.synchronize()
        finally:
            sys.stdout.flush()
            os.dup2(saved, 1)
            os.close(saved)
    cfg = CFG2
    _ext.set_precision("tf32")
    layer = Layer(cfg, dev)
    host_sets = make_inputs(cfg, rank * ROTATE * cfg["batch"], ROTATE)
    dev_sets = [(torch.from_numpy(f).to(dev), torch.from_numpy(i).to(dev)) for f, i in host_sets]
    pinned = [(torch.from_numpy(f).pin_memory(), torch.from_numpy(i).pin_memory()) for f, i in host_sets]
    n_in = [int(i.shape[0]) for _, i in host_sets]
    peak_hbm, peak_bf16, peak_src = peaks()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    # ---- device-resident throughput.  The step (rulebook + materialise + pack + stage + conv +
    # pool rulebook + max pool) is recorded as a CUDA graph over capacity-sized buffers with
    # the row counts kept on the device (ss_conv.graph.GraphedChain).  The chain is recorded once per
    # rotating batch (each recording with buffers of its own) and every batch is loaded into the input
    # buffers of its recording before the timed region: the inputs are resident in HBM where the kernels
    # read them; a timed step is the replay of the whole layer pass on one batch plus the read-back and
    # check of its row counts.  Step s+1 is queued before the host waits for step s.
    from ss_conv.graph import GraphedChain

    def chain(x):
        with torch.no_grad():
            return layer.pool(layer.conv(x))

    host_us = [0.0, 0.0]

    def timed_steps(depth, streams, lag, regions):
        """(graph, per-region ms list, voxels per region, replays, fallbacks): `depth` recordings
        (recording k holds rotating batch k % ROTATE), replayed round-robin on `streams` streams, each
        result taken `lag` steps after its submission; `regions` repetitions of the --steps-long region."""
        g = GraphedChain(chain, [cfg["V"]] * 3, cfg["batch"], layer.conv.in_channels, max(n_in), dev, depth=depth, streams=streams)
        for k in range(depth):
            g.load(k, *dev_sets[k % ROTATE])
        for w in range(max(args.warmup, 20, depth)):
            g.submit_loaded(w % depth).result()
        r0, f0 = g.replays, g.fallbacks
        times, vox = [], 0
        t_submit = t_result = 0.0
        for _ in range(regions):
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            vox, waiting = 0, []
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
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
        host_us[0], host_us[1] = t_submit / (args.steps * regions) * 1e6, t_result / (args.steps * regions) * 1e6
        return g, times, vox, g.replays - r0, g.fallbacks - f0

    DEPTH, STREAMS, LAG = (int(v) for v in args.overlap.split(","))   # recordings, streams, steps in flight
    with ClockSampler(local, enabled=(rank == 0), core=(my_cores[-1] if len(my_cores) > 1 else None)) as clk:
        graphed, region_ms, voxels, n_replays, graph_fallbacks = timed_steps(DEPTH, STREAMS, LAG, REGIONS)
    ms = float(statistics.median(region_ms))
    launches = graphed.launches * args.steps          # kernels of the library inside ONE timed region
    host_submit_us, host_result_us = host_us
    _ext.check_status(dev)
    # the same loop with 16-bit operands in the convolution (opt-in precisions; reported beside the headline)
    alt_steps = {}
    for prec in ("bf16", "fp16"):
        _ext.set_precision(prec)
        try:
            g16, ms16, _, _, _ = timed_steps(DEPTH, STREAMS, LAG, 7)
            alt_steps[prec] = float(statistics.median(ms16)) / args.steps
            del g16
        finally:
            _ext.set_precision("tf32")
    # the same step launched kernel by kernel from Python, for comparison
    eager_step_ms = eager_ms(lambda: layer.step(*dev_sets[0]).resolve(), reps=10, warm=3)

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
    e2e_regions, d2h = [], 0
    for _ in range(5):
        barrier()
        t0 = time.perf_counter()
        for of, oi in feed.run(pinned[s % ROTATE] for s in range(args.steps)):
            d2h = of.numel() * 4 + oi.numel() * 4
        torch.cuda.synchronize()
        e2e_regions.append(time.perf_counter() - t0)
    e2e_s = float(statistics.median(e2e_regions))
    vox_e2e = sum(n_in[s % ROTATE] for s in range(args.steps))
    h2d = int(np.mean([f.numel() * 4 + i.numel() * 4 for f, i in pinned]))

    # ---- the same loop fed with bf16 feature rows from the host (half the upload; the convolution
    # gathers the uploaded rows as its bf16 operands, there is no staging pass): opt-in, beside the headline
    e2e16, e2e16_s = None, 0.0
    try:
        _ext.set_precision("bf16")
        pinned16 = [(f.to(torch.bfloat16).pin_memory(), i) for f, i in pinned]     # converted once, outside the timed loop
        graphed16 = GraphedChain(chain, [cfg["V"]] * 3, cfg["batch"], layer.conv.in_channels, max(n_in), dev,
                                 feature_dtype=torch.bfloat16)

        def dev_step16(fd, idd):
            o = graphed16(fd, idd)
            return o.features, o.indices

        feed16 = HostStream(dev_step16, dev, max_rows=max(n_in), step_reuses_outputs=True)
        for _ in feed16.run(pinned16[w % ROTATE] for w in range(3)):
            pass
        regs16 = []
        for _ in range(5):
            barrier()
            t0 = time.perf_counter()
            for of, oi in feed16.run(pinned16[s % ROTATE] for s in range(args.steps)):
                pass
            torch.cuda.synchronize()
            regs16.append(time.perf_counter() - t0)
        e2e16_s = float(statistics.median(regs16))
        e2e16 = {"value": None, "unit": "voxels/s",
                 "h2d_bytes_per_step": int(np.mean([f.numel() * 2 + i.numel() * 4 for f, i in pinned16])),
                 "d2h_bytes_per_step": int(d2h),
                 "what": "features uploaded as bf16 rows (converted on the host beforehand), bf16 operands, f32 accumulate and outputs"}
        del graphed16, feed16
    finally:
        _ext.set_precision("tf32")

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
    torch.cuda.synchronize()
    serial_s = time.perf_counter() - t0

    # ---- dominant call alone: stage_features_kernel + conv_fwd_tf32_kernel, recorded as a small CUDA
    # graph per input batch so that the CUDA events around a replay see device time only
    from ss_conv.sp_ops.ops import get_indice_pairs
    prepared = []
    with torch.no_grad():
        flt = layer.conv.kernel.filters().reshape(-1, layer.conv.in_channels, layer.conv.out_channels)
        for f, i in dev_sets:
            outids, pairs, num = get_indice_pairs(i, cfg["batch"], [cfg["V"]] * 3, cfg["k"], cfg["stride"], cfg["pad"])
            prepared.append((f, i, _ext.neighbour_table(pairs, num, outids.shape[0]), outids.shape[0], int(num.sum().item())))

        def conv_call_ms(prec):
            graphs = []
            for f, _, nbr, n_out, P in prepared:
                _ext.conv_forward(f, flt, nbr, n_out, prec)
                torch.cuda.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    keep = _ext.conv_forward(f, flt, nbr, n_out, prec)
                graphs.append((g, keep))
            ts = []
            for it in range(3 + 40):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                graphs[it % ROTATE][0].replay()
                b.record()
                torch.cuda.synchronize()
                if it >= 3:
                    ts.append(a.elapsed_time(b))
            return float(statistics.median(ts))

        kern_ms = conv_call_ms("tf32")
        conv16_ms = {prec: conv_call_ms(prec) for prec in ("bf16", "fp16")}
        K, ci, co = flt.shape
        alg_bytes = float(np.mean([4 * (f.shape[0] * ci + n_out * co + K * ci * co) + 8 * P for f, _, _, n_out, P in prepared]))
        flops = float(np.mean([2.0 * P * ci * co for _, _, _, _, P in prepared]))
        n_out_conv = prepared[0][3]

        # ---- the conv rulebook alone: counting + fill phases with the row count left on the device
        # (the form the recorded step uses), as a graph replay
        f0, i0, nbr0, n_out0, P0 = prepared[0]
        osz = [(cfg["V"] + 2 * cfg["pad"] - cfg["k"]) // cfg["stride"] + 1] * 3
        rb_args = (i0, cfg["batch"], osz, [cfg["V"]] * 3, [cfg["k"]] * 3, [cfg["stride"]] * 3, [cfg["pad"]] * 3, [1] * 3, 0)
        rulebook = None
        if _ext.get_indice_pairs_ahead(*rb_args) is not None:
            rb_ms = graph_ms(lambda: _ext.get_indice_pairs_ahead(*rb_args), reps=20)
            rb_bytes = 16.0 * f0.shape[0] + 16.0 * n_out0 + 8.0 * P0 + 4.0 * K
            rulebook = {"what": "conv rulebook of the cfg2 batch (count + fill, row count left on the device), graph replay",
                        "ms": rb_ms, "algorithmic_bytes": rb_bytes, "GBps": rb_bytes / (rb_ms * 1e-3) / 1e9,
                        "frac_of_hbm_peak": rb_bytes / (rb_ms * 1e-3) / 1e9 / peak_hbm}

        # ---- backward of the same layer (input gradient through the tcgen05 kernel on the input-major
        #      table, tensor-core filter gradient), the rulebook of the forward pass reused
        grads = [torch.randn(n_out, flt.shape[2], device=dev) for _, _, _, n_out, _ in prepared]
        bwd_ts = []
        for kidx in range(2):
            f, _, nbr, n_out, _ = prepared[kidx]
            nbr_in = _ext.input_major_table(nbr, f.shape[0])
            order = _ext.nbr_row_order(nbr_in)
            gr = grads[kidx]
            bwd_ts.append(graph_ms(lambda: _ext.conv_backward(f, flt, gr, nbr, nbr_in, order, "tf32"), reps=6))
        bwd_ms = float(np.mean(bwd_ts))
    achieved = alg_bytes / (kern_ms * 1e-3) / 1e9

    layers = layers_leg(dev, peak_hbm, peak_bf16) if rank == 0 else None
    helpers = helpers_leg(dev, peak_hbm) if (rank == 0 and world == 1) else None
    if world > 1:
        dist.barrier()
    per_gpu_strong = BACKBONE["global_batch"] // world
    backbone = run_backbone(args, dev, rank, world, dist, per_gpu_strong, "strong")
    backbone_weak = run_backbone(args, dev, rank, world, dist, BACKBONE["global_batch"], "weak") if world > 1 else None
    _ext.set_precision("tf32")

    # ---- reduce over ranks
    stats = torch.tensor([ms, e2e_s, float(voxels), float(vox_e2e), float(launches), serial_s, eager_step_ms, host_submit_us,
                          host_result_us, min(region_ms), max(region_ms), e2e16_s], dtype=torch.float64, device=dev)
    if world > 1:
        mx = stats.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        sm = stats.clone()
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        ms, e2e_s, serial_s, eager_step_ms = float(mx[0]), float(mx[1]), float(mx[5]), float(mx[6])
        host_submit_us, host_result_us = float(mx[7]), float(mx[8])
        voxels, vox_e2e, launches = float(sm[2]), float(sm[3]), float(sm[4])
        region_min, region_max, e2e16_s = float(mx[9]), float(mx[10]), float(mx[11])
    else:
        region_min, region_max = min(region_ms), max(region_ms)
    if e2e16 is not None and e2e16_s > 0:
        e2e16["value"] = vox_e2e / e2e16_s
    if rank == 0:
        traffic = NCU_DRAM_BYTES["stage_features_kernel"] + NCU_DRAM_BYTES["conv_fwd_tf32_kernel"]
        line = {
            "metric": "active voxels/sec per SS-Conv layer", "value": voxels / (ms * 1e-3), "unit": "voxels/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "tf32 operands, f32 accumulate",
            "data": "synthetic (seeded ellipsoid-surface voxels, N(0,1) features, reference-style N(0,1) kernel weights)",
            "config": {"workload": cfg["name"], "n_in_per_batch": n_in[0], "n_out_conv": n_out_conv,
                       "c_in": layer.conv.in_channels, "c_out": layer.conv.out_channels,
                       "timing": "the --steps-long region is repeated %d times per rank after >= 20 warm-up steps; the median region is "
                                 "reported (max over ranks of the medians); region min / max below" % REGIONS,
                       "region_ms": {"median": ms, "min": region_min, "max": region_max},
                       "l2": "%d recordings with buffers of their own (inputs, tables, staging, outputs: > 1 GB working set) holding %d "
                             "distinct input batches, replayed in turn: nothing a step reads is still in L2 from its last replay"
                             % (DEPTH, ROTATE),
                       "step": "rulebook + materialise + pack + stage + conv + pool rulebook + maxpool, replayed as one "
                               "CUDA graph (device-side row counts, capacity-sized buffers), one recording per rotating batch "
                               "with the batch resident in its input buffers; a step = replay + read-back and check of the "
                               "row counts and of the kernel status word, step s+1 queued before the host checks step s; the recordings "
                               "replay on %d streams in turn (%d recordings, results taken %d steps late), so consecutive steps overlap on the device"
                               % (STREAMS, DEPTH, LAG),
                       "eager_ms_per_step": eager_step_ms, "graph_fallbacks": graph_fallbacks,
                       "host_us_per_step": {"queue_a_step": host_submit_us, "wait_for_and_check_a_step": host_result_us,
                                            "note": "host time in the timed loop (max over ranks); the second includes waiting for the device"},
                       "host_cores_of_rank0": len(my_cores),
                       "parallelism": "sample-sharded x%d, no data-path collective" % world},
            "e2e": {"value": vox_e2e / e2e_s, "unit": "voxels/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": int(d2h),
                    "how": "ss_conv.pipeline.HostStream (upload / compute / download of consecutive steps overlap on 3 streams) "
                           "around the CUDA-graph replay of the step; fp32 feature rows uploaded; median of 5 regions of --steps steps",
                    "serial_value": vox_e2e / serial_s, "bf16_upload": e2e16},
            "gpu_launches": int(launches),
            "clocks": clk.summary(),
            "roofline": {"bound": "hbm", "kernel": "stage_features_kernel + conv_fwd_tf32_kernel", "achieved": achieved,
                         "peak": peak_hbm, "unit": "GB/s", "frac": achieved / peak_hbm, "traffic": traffic,
                         "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of the two kernels of the timed call on the "
                                           "cfg2 inputs (staging %.1f MB + convolution %.1f MB per launch)"
                                           % (NCU_DRAM_BYTES["stage_features_kernel"] / 1e6, NCU_DRAM_BYTES["conv_fwd_tf32_kernel"] / 1e6),
                         "peak_source": peak_src,
                         "kernel_ms": kern_ms, "algorithmic_bytes": alg_bytes,
                         "tensor_tflops": flops / (kern_ms * 1e-3) / 1e12,
                         "tensor_frac_of_tf32_peak": flops / (kern_ms * 1e-3) / 1e12 / (peak_bf16 / 2)},
        }
        line["rulebook"] = rulebook
        line["backward"] = {"what": "input gradient (forward kernel on the input-major table, rows grouped by parity class) + filter gradient (pair lists compacted inside the call) of the cfg2 convolution, both tcgen05 with TF32 operands; input-major table and row order come with the rulebook",
                            "ms": bwd_ms, "voxels_per_s": float(np.mean(n_in)) / (bwd_ms * 1e-3)}
        line["operands_16bit"] = {"what": "the cfg2 convolution call (stage + conv) and the timed step loop with 16-bit operands, f32 accumulate "
                                          "(opt-in precisions 'bf16' / 'fp16'; the headline numbers above use TF32 operands)",
                                  "tf32_conv_call_ms": kern_ms, "conv_call_ms": conv16_ms, "step_ms": alt_steps,
                                  "roofline_frac_of_hbm": {p: alg_bytes / (t * 1e-3) / 1e9 / peak_hbm for p, t in conv16_ms.items()}}
        line["layers"] = layers
        if helpers is not None:
            line["helpers"] = helpers
        line["backbone"] = backbone
        if backbone_weak is not None:
            line["backbone_weak"] = backbone_weak
        if world == 1:
            line["reference_gpu"] = reference_gpu_leg(cfg, dev, ms / args.steps, kern_ms)
            line["cpu_baseline"] = cpu_baseline(cfg, budget_s=12.0)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_only(args):
    """A few launches of one kernel group (small, fixed launch count), for ncu captures."""
    from ss_conv import _ext
    from ss_conv.sp_ops.ops import get_indice_pairs
    dev = torch.device("cuda", 0)
    cfg = CFG2
    _ext.set_precision("tf32")
    if args.only == "helpers":
        for name, fn, _ in helper_cases(dev):
            for _ in range(2):
                fn()
        torch.cuda.synchronize()
        _ext.check_status(dev)
        print("only=helpers done")
        return
    if args.only == "backbone":
        # three batches of the 4-stage backbone (256 objects), one recording replayed on one stream
        from ss_conv.utils import synthetic as S
        pts, fts, ids = S.object_points(range(256), BACKBONE["n_pts"], base_seed=7000)
        pts, fts, ids = (torch.from_numpy(a).to(dev) for a in (pts, fts, ids))
        net = Backbone(BACKBONE, dev, 256, depth=1, streams=1)
        for _ in range(3):
            pooled = net.submit(pts, fts, ids.int()).result()
        torch.cuda.synchronize()
        _ext.check_status(dev)
        print("only=backbone done, pooled %s, %d launches per replay" % (tuple(pooled.shape), net.graphed.launches))
        return
    if args.only in ("conv5", "conv5_tf32"):
        # the wide layer at half its batch (8 samples, ~88 k voxels: 90 MB of fp32 features, 90 MB of outputs)
        from ss_conv.utils import synthetic as S
        ind = S.bernoulli_voxels(range(8), 48, 0.10, base_seed=40)
        n = ind.shape[0]
        g = torch.Generator(device="cpu").manual_seed(1)
        feats = torch.randn(n, 256, generator=g).to(dev)
        W = (torch.randn(125, 256, 256, generator=g) / 180).to(dev)
        outids, pairs, num = get_indice_pairs(torch.from_numpy(ind).to(dev), 8, [48] * 3, 5, 1, 2, 1, 0, True, False, lazy=True)
        nbr = _ext.neighbour_table(pairs, num, n)
        prec = "tf32" if args.only == "conv5_tf32" else "bf16"
        for _ in range(3):
            _ext.conv_forward(feats, W, nbr, n, prec)
        torch.cuda.synchronize()
        _ext.check_status(dev)
        print("only=%s done, n=%d pairs=%d" % (args.only, n, int((nbr >= 0).sum())))
        return
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
            if args.only in ("conv", "conv_fp16", "conv_bf16"):
                nbr = _ext.neighbour_table(pairs, num, outids.shape[0])
                prec = {"conv": "tf32", "conv_fp16": "fp16", "conv_bf16": "bf16"}[args.only]
                for _ in range(4):
                    _ext.conv_forward(f, flt, nbr, outids.shape[0], prec)
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
    """One CPU step of the reference's own code path:
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
    ci = channels(cfg["irreps"])
    co = channels(cfg["irreps"], gates=True)
    feats = S.features(ind.shape[0], ci, 77)
    W = (np.random.RandomState(5).randn(cfg["k"], cfg["k"], cfg["k"], ci, co) / np.sqrt(ci * cfg["k"] ** 3)).astype(np.float32)
    return feats, ind, W


CPU_SAMPLE = ("the full cfg2 batch (%d samples, %d active voxels) per step through the reference's C++ CPU path: rulebook + conv + "
              "pool rulebook + maxpool; the filter tensor has the layer's shape and scale (its values do not change the "
              "CPU work: the reference's own SE3Kernel Python cannot be imported on the GPU box); rulebook / gather / scatter are "
              "single-threaded C++ loops, the GEMM uses torch's CPU threads")


def cpu_baseline(cfg, budget_s=12.0):
    step, kind = ref_step_fn(cfg)
    n_samples = cfg["batch"]
    feats, ind, W = cpu_inputs(cfg, n_samples)
    step(feats, ind, W, n_samples)  # warm-up
    t0 = time.perf_counter()
    reps = 0
    while reps < 3 or (time.perf_counter() - t0 < budget_s and reps < 200):
        step(feats, ind, W, n_samples)
        reps += 1
    dt = time.perf_counter() - t0
    return {"value": ind.shape[0] * reps / dt, "unit": "voxels/s", "cores": torch.get_num_threads(), "kind": kind,
            "host_cpus": os.cpu_count(), "ms_per_step": dt / reps * 1e3,
            "sample": (CPU_SAMPLE % (n_samples, ind.shape[0])) + "; %d repetitions" % reps}


def run_reference(args):
    rank = int(os.environ.get("RANK", 0))
    if rank != 0:
        return
    cfg = CFG2
    n_samples = cfg["batch"]
    step, kind = ref_step_fn(cfg)
    feats, ind, W = cpu_inputs(cfg, n_samples)
    for _ in range(max(1, min(args.warmup, 3))):
        step(feats, ind, W, n_samples)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step(feats, ind, W, n_samples)
    dt = time.perf_counter() - t0
    value = ind.shape[0] * args.steps / dt
    sample = CPU_SAMPLE % (n_samples, ind.shape[0])
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
    ap.add_argument("--overlap", default="8,4,3",
                    help="layer step loop: recordings of the step, streams they replay on, steps in flight before the host waits")
    ap.add_argument("--only", default=None,
                    choices=["conv", "conv_fp16", "conv_bf16", "conv5", "conv5_tf32", "backward", "rulebook", "step", "helpers", "backbone"],
                    help="run just one kernel group a few times (for ncu captures): the cfg2 convolution call, the wide "
                         "cfg5 layer at half its batch, the backward kernels, the whole cfg2 step, the helper kernels")
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
