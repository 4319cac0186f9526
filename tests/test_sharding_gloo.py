"""The N > 1 path on CPU: two gloo ranks shard rows, fold their shards with the CPU oracle's
algorithms and combine the partials the way bench.py / the multi-GPU runs do (all_reduce for
sum / max, gathered (value, global index) pairs for argmax with first-occurrence ties)."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import dali_oracle as oracle
    from dali_b200.sharding import combine_arg_partials, combine_partials, shard_range
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rng = np.random.default_rng(7)
    x = (rng.random((101, 37)) * 2 - 1).astype(np.float32)
    x[10, 5] = x[90, 5] = 0.9999999          # a tie across shards: the lower global row must win
    x[60, 7] = x[61, 7] = -0.9999999
    lo, hi = shard_range(x.shape[0], rank, world)
    mine = x[lo:hi]
    res = {}
    # all-axis and axis-0 sums: local double-accumulated folds, all_reduce of the partials
    s_all = torch.tensor([oracle.sum_f64acc(mine)[0].item()], dtype=torch.float64)
    res["sum_all"] = combine_partials(s_all, "sum").numpy()
    s0 = torch.from_numpy(oracle.sum_f64acc(mine, 0)[0])
    res["sum_0"] = combine_partials(s0, "sum").numpy()
    m0 = torch.from_numpy(oracle.reduce("max", mine, 0))
    res["max_0"] = combine_partials(m0.clone(), "max").numpy()
    # argmax over axis 0 and over everything
    a0 = torch.from_numpy(oracle.argreduce("max", mine, 0))
    res["argmax_0"] = combine_arg_partials(m0, a0, lo, "max").numpy()
    mn0 = torch.from_numpy(oracle.reduce("min", mine, 0))
    an0 = torch.from_numpy(oracle.argreduce("min", mine, 0))
    res["argmin_0"] = combine_arg_partials(mn0, an0, lo, "min").numpy()
    flat_local = int(oracle.argreduce("max", mine))
    v = torch.tensor([mine.reshape(-1)[flat_local]])
    res["argmax_all"] = combine_arg_partials(v, torch.tensor([flat_local]), lo * x.shape[1], "max").numpy()
    # chain: sum(sigmoid(x*w+b)*exp(-x*x)) over sharded elements
    flat = x.reshape(-1)
    a, b = shard_range(flat.size, rank, world)
    part = torch.tensor([oracle.chain_sum(flat[a:b], 0.5, 0.1)[1]], dtype=torch.float64)
    res["chain"] = combine_partials(part, "sum").numpy()
    np.savez(os.path.join(out_dir, "rank%d.npz" % rank), **res)
    dist.destroy_process_group()


def test_two_rank_sharded_reductions(tmp_path):
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import dali_oracle as oracle
    from dali_b200.sharding import shard_range
    assert [shard_range(10, r, 3) for r in range(3)] == [(0, 4), (4, 7), (7, 10)]
    assert shard_range(8, 1, 2) == (4, 8)
    world = 2
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    rng = np.random.default_rng(7)
    x = (rng.random((101, 37)) * 2 - 1).astype(np.float32)
    x[10, 5] = x[90, 5] = 0.9999999
    x[60, 7] = x[61, 7] = -0.9999999
    for rank in range(world):
        r = np.load(os.path.join(str(tmp_path), "rank%d.npz" % rank))
        assert abs(r["sum_all"][0] - x.astype(np.float64).sum()) < 1e-9
        np.testing.assert_allclose(r["sum_0"], x.astype(np.float64).sum(0), atol=1e-9)
        np.testing.assert_array_equal(r["max_0"], oracle.reduce("max", x, 0))
        np.testing.assert_array_equal(r["argmax_0"], oracle.argreduce("max", x, 0))
        np.testing.assert_array_equal(r["argmin_0"], oracle.argreduce("min", x, 0))
        assert r["argmax_0"][5] == 10 and r["argmin_0"][7] == 60          # first occurrence across shards
        assert int(r["argmax_all"][0]) == int(oracle.argreduce("max", x))
        assert abs(r["chain"][0] - oracle.chain_sum(x, 0.5, 0.1)[1]) < 1e-9
