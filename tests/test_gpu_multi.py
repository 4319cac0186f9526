"""Two ranks on two GPUs: every rank holds a shard of the rows (Array.scatter_rows), the same fused kernels run on
every rank and the library combines partial results only where a reduction or a product crosses the sharded
dimension -- once over peer memory (in-kernel for all-axis reductions, one-shot exchange kernels otherwise), once
with everything forced through NCCL.  Skipped on a one-GPU box."""
import os
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _data():
    rng = np.random.default_rng(11)
    x = (rng.random((512, 384)) * 2 - 1).astype(np.float32)
    x[100, 7] = x[400, 7] = 0.99999994          # a tie across the two shards
    w = (rng.standard_normal((384, 64)) * 0.1).astype(np.float32)
    return x, w


def _worker(rank, world, port, out_dir, force_nccl):
    sys.path.insert(0, ROOT)
    if force_nccl:
        os.environ["DALI_B200_ALLREDUCE"] = "nccl"
        os.environ["DALI_B200_XRANK_FUSE"] = "0"
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch.distributed as dist
    import dali_b200
    from dali_b200 import comm
    from dali_b200.array import Array, collectives, last_ir, op, set_default_device
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    lib = dali_b200.load_library()
    lib.init(0)
    set_default_device(rank)
    comm.init_from_torch(lib, rank)
    res = {"transport": np.array(lib.comm_transport())}
    x, w = _data()
    xs = Array.scatter_rows(x)
    lo = xs.shard[1]
    res["lo"] = np.array(lo)
    chain = op.sum(op.sigmoid(xs * np.float32(0.5) + np.float32(0.1)) * op.exp(-xs * xs))
    res["chain"] = chain.numpy()
    res["chain_fused"] = np.array("xrank" in last_ir())
    for k in range(4):                                       # repeated calls: epochs and slot parity
        res["sum_all_%d" % k] = op.sum(xs).numpy()
    res["max_all"] = op.max(xs).numpy()
    res["argmax_all"] = op.argmax(xs).numpy()
    res["mean_all"] = op.mean(xs).numpy()
    res["sum_0"] = op.sum(xs, [0]).numpy()
    res["max_0"] = op.max(xs, [0]).numpy()
    res["min_0"] = op.min(xs, [0]).numpy()
    res["argmax_0"] = op.argmax(xs, 0).numpy()
    res["argmin_0"] = op.argmin(xs, 0).numpy()
    res["mean_0"] = op.mean(xs, [0]).numpy()
    res["softmax_0"] = op.softmax(xs, 0).numpy()             # max and sum over the sharded axis, rows stay local
    res["softmax_1"] = op.softmax(xs, -1).numpy()            # rows are independent: no collective
    before = collectives()[0]
    res["sum_1"] = op.sum(xs, [1]).numpy()
    res["rowwise_collectives"] = np.array(collectives()[0] - before)
    res["proj"] = op.tanh(op.dot(xs, Array(w))).numpy()      # rows x whole weights: local
    res["gram"] = op.dot(xs.transpose(), xs).numpy()         # contracts the sharded dimension: GEMM reduce
    # raw collectives, small (peer exchange) and large (NCCL)
    small = torch.full((1000,), float(rank + 1), device="cuda")
    lib.allreduce(small, 1000, 0, "sum", device=rank)
    big = torch.full((1 << 20,), float(rank + 1), device="cuda")
    lib.allreduce(big, 1 << 20, 0, "sum", device=rank)
    torch.cuda.synchronize()
    res["raw"] = np.array([small[0].item(), small[-1].item(), big[0].item(), big[-1].item()])
    res["error_flag"] = np.array(lib.comm_error_flag())
    np.savez(os.path.join(out_dir, "rank%d.npz" % rank), **res)
    lib.comm_destroy()
    dist.destroy_process_group()


@pytest.mark.parametrize("force_nccl", [False, True])
def test_two_gpu_sharded_expressions(tmp_path, force_nccl):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import dali_oracle as oracle
    import torch.multiprocessing as mp
    world = 2
    port = 29600 + (os.getpid() % 2000) + (7 if force_nccl else 0)
    mp.spawn(_worker, args=(world, port, str(tmp_path), force_nccl), nprocs=world, join=True)
    x, w = _data()
    x64 = x.astype(np.float64)
    s32, s64, sabs = oracle.chain_sum(x, 0.5, 0.1)
    sum0, abs0 = oracle.sum_f64acc(x, 0)
    ranks = [np.load(os.path.join(str(tmp_path), "rank%d.npz" % r)) for r in range(world)]
    for rank, r in enumerate(ranks):
        assert int(r["error_flag"]) == 0
        if force_nccl:
            assert not bool(r["chain_fused"])
        else:
            assert str(r["transport"]) == "nccl+peer" and bool(r["chain_fused"]), str(r["transport"])
        lo, hi = int(r["lo"]), int(r["lo"]) + 256
        assert abs(float(r["chain"]) - s64) <= 1e-5 * sabs
        for k in range(4):
            assert abs(float(r["sum_all_%d" % k]) - x64.sum()) <= 1e-5 * np.abs(x64).sum()
        assert float(r["max_all"]) == x.max()
        assert int(r["argmax_all"]) == int(oracle.argreduce("max", x)) == 100 * 384 + 7
        assert abs(float(r["mean_all"]) - x64.mean()) <= 1e-5 * np.abs(x64).mean()
        assert np.all(np.abs(r["sum_0"] - sum0) <= 1e-5 * abs0)
        np.testing.assert_array_equal(r["max_0"], oracle.reduce("max", x, 0))
        np.testing.assert_array_equal(r["min_0"], oracle.reduce("min", x, 0))
        np.testing.assert_array_equal(r["argmax_0"], oracle.argreduce("max", x, 0))
        np.testing.assert_array_equal(r["argmin_0"], oracle.argreduce("min", x, 0))
        assert r["argmax_0"][7] == 100
        np.testing.assert_allclose(r["mean_0"], x64.mean(0), rtol=0, atol=1e-5 * np.abs(x64).mean(0).max() + 1e-7)
        np.testing.assert_allclose(r["softmax_0"], oracle.softmax(np.ascontiguousarray(x.T)).T[lo:hi], rtol=1e-5, atol=1e-9)
        np.testing.assert_allclose(r["softmax_1"], oracle.softmax(x[lo:hi]), rtol=1e-5, atol=1e-9)
        assert int(r["rowwise_collectives"]) == 0
        np.testing.assert_allclose(r["sum_1"], x64[lo:hi].sum(1), rtol=0, atol=1e-5 * np.abs(x64).sum(1).max())
        np.testing.assert_allclose(r["proj"], np.tanh(x64[lo:hi] @ w.astype(np.float64)), rtol=1e-5, atol=1e-5)
        gram = x64.T @ x64
        assert np.all(np.abs(r["gram"] - gram) <= 1e-5 * (np.abs(x64).T @ np.abs(x64)))
        np.testing.assert_array_equal(r["raw"], [3.0, 3.0, 3.0, 3.0])
    # every rank holds the same bits after a combine
    for key in ("chain", "sum_all_0", "sum_0", "mean_0", "gram"):
        np.testing.assert_array_equal(ranks[0][key], ranks[1][key])
