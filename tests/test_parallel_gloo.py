"""World-size-2 CPU (gloo) test of the sample-sharding plumbing: shards are disjoint and
complete, and the all-gather reassembles per-sample rows in sample order (ragged shards too)."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, n_samples, out_dir):
    sys.path.insert(0, os.path.join(ROOT, "ss-conv_b200"))
    from ss_conv import parallel
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.RandomState(0)
        n_rows = 40
        indices = torch.from_numpy(np.sort(rng.randint(0, n_samples, n_rows)).astype(np.int32))
        indices = torch.stack([indices, indices * 0, indices * 0, indices * 0], 1)
        feats = torch.arange(n_rows * 3, dtype=torch.float32).view(n_rows, 3)
        f, idx, n_local = parallel.shard_sparse(feats, indices, n_samples, rank, world)
        lo, hi = parallel.shard_range(n_samples, rank, world)
        assert n_local == hi - lo
        assert idx.shape[0] == 0 or (int(idx[:, 0].min()) >= 0 and int(idx[:, 0].max()) < n_local)
        # per-sample "pooled" rows: sum of the sample's features (stand-in for the backbone)
        pooled = torch.zeros(n_local, 3)
        pooled.index_add_(0, idx[:, 0].long(), f)
        full = parallel.all_gather_rows(pooled, n_samples)
        expect = torch.zeros(n_samples, 3)
        expect.index_add_(0, indices[:, 0].long(), feats)
        assert torch.equal(full, expect)
        # the buffered form used in loops (no padding copy / concatenation for equal shards), twice
        gather = parallel.RowGatherer(n_samples, 3, pooled.device)
        for rep in range(2):
            again = gather(pooled * (rep + 1))
            assert torch.equal(again, expect * (rep + 1))
        torch.save(full, os.path.join(out_dir, "r%d.pt" % rank))
    finally:
        dist.destroy_process_group()


def _run(n_samples, tmp_path):
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(2, port, n_samples, str(tmp_path)), nprocs=2, join=True)
    a = torch.load(os.path.join(str(tmp_path), "r0.pt"))
    b = torch.load(os.path.join(str(tmp_path), "r1.pt"))
    assert torch.equal(a, b) and a.shape[0] == n_samples


def test_two_rank_even_shards(tmp_path):
    _run(6, tmp_path)


def test_two_rank_ragged_shards(tmp_path):
    _run(5, tmp_path)
