"""The N > 1 path on CPU: two gloo ranks drive the LIBRARY's communicator through its host transport
(dalib200_comm_init_host): the collectives' dtype / reduction mapping, the (value, index) combine of a sharded
argmax with first-occurrence ties, dalib200_shard_range, and -- in dry-run mode, where the front end lowers and
compiles but launches nothing -- which collective a sharded expression ends in.  Partial results are computed
with the CPU oracle (there is no CPU compute path in the library)."""
import os
import sys

import numpy as np
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _data():
    rng = np.random.default_rng(7)
    x = (rng.random((101, 37)) * 2 - 1).astype(np.float32)
    x[10, 5] = x[90, 5] = 0.9999999          # a tie across shards: the lower global row must win
    x[60, 7] = x[61, 7] = -0.9999999
    return x


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import dali_oracle as oracle
    import dali_b200
    from dali_b200 import comm
    from dali_b200.array import Array, collectives, last_ir, op, set_dry_run
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    lib = dali_b200.load_library()
    comm.init_host_from_torch(lib)
    assert lib.comm_world() == world and lib.comm_rank() == rank and lib.comm_transport() == "host"
    x = _data()
    lo, hi = lib.shard_range(x.shape[0], rank, world)
    mine = x[lo:hi]
    res = {}
    # all-axis and axis-0 sums: local double-accumulated folds (oracle), all-reduce of the partials (library)
    s_all = np.array([oracle.sum_f64acc(mine)[0].item()], np.float64)
    lib.allreduce(s_all, 1, 1, "sum", device=-1)
    res["sum_all"] = s_all
    s0 = np.ascontiguousarray(oracle.sum_f64acc(mine, 0)[0], np.float64)
    lib.allreduce(s0, s0.size, 1, "sum", device=-1)
    res["sum_0"] = s0
    m0 = np.ascontiguousarray(oracle.reduce("max", mine, 0))
    mx = m0.copy()
    lib.allreduce(mx, mx.size, 0, "max", device=-1)
    res["max_0"] = mx
    cnt = np.array([hi - lo], np.int32)
    lib.allreduce(cnt, 1, 2, "sum", device=-1)
    res["rows"] = cnt
    # argmax / argmin over axis 0 and argmax over everything: (value, global index) pairs
    a0 = (oracle.argreduce("max", mine, 0) + lo).astype(np.int32)
    v0 = m0.copy()
    lib.arg_allreduce(v0, a0, v0.size, 0, "max", device=-1)
    res["argmax_0"], res["argmax_0_values"] = a0, v0
    vn = np.ascontiguousarray(oracle.reduce("min", mine, 0))
    an = (oracle.argreduce("min", mine, 0) + lo).astype(np.int32)
    lib.arg_allreduce(vn, an, vn.size, 0, "min", device=-1)
    res["argmin_0"] = an
    flat_local = int(oracle.argreduce("max", mine))
    v = np.array([mine.reshape(-1)[flat_local]], np.float64)
    i = np.array([flat_local + lo * x.shape[1]], np.int32)
    lib.arg_allreduce(v, i, 1, 1, "max", device=-1)
    res["argmax_all"] = i
    # chain: sum(sigmoid(x*w+b)*exp(-x*x)) over sharded elements
    flat = x.reshape(-1)
    a, b = lib.shard_range(flat.size, rank, world)
    part = np.array([oracle.chain_sum(flat[a:b], 0.5, 0.1)[1]], np.float64)
    lib.allreduce(part, 1, 1, "sum", device=-1)
    res["chain"] = part
    # the front end on this rank's shard, lowering only: what the sharded expressions end in
    set_dry_run(True)
    xs = Array.scatter_rows(x)
    assert xs.shape == (hi - lo, x.shape[1]) and xs.shard == (0, lo, x.shape[0])
    plan = []
    for expr in (op.sum(xs), op.max(xs, [0]), op.argmax(xs, 0), op.argmax(xs), op.mean(xs, [0]), op.sum(xs, [1]),
                 op.dot(xs.transpose(), xs), op.softmax(xs, -1)):
        before = collectives()[0]
        expr.eval()
        n, what = collectives()
        plan.append("%d:%s" % (n - before, what if n > before else "-"))
        assert "xrank" not in last_ir()          # the host transport has no peer memory to meet in
    res["plan"] = np.array(plan)
    assert op.sum(xs, [1]).shard == (0, lo, x.shape[0]) and op.sum(xs, [0]).shard[0] == -1
    set_dry_run(False)
    np.savez(os.path.join(out_dir, "rank%d.npz" % rank), **res)
    lib.comm_destroy()
    dist.destroy_process_group()


def test_two_rank_sharded_reductions(tmp_path):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import dali_oracle as oracle
    import dali_b200
    lib = dali_b200.load_library()
    assert [lib.shard_range(10, r, 3) for r in range(3)] == [(0, 4), (4, 7), (7, 10)]
    assert lib.shard_range(8, 1, 2) == (4, 8)
    world = 2
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    x = _data()
    for rank in range(world):
        r = np.load(os.path.join(str(tmp_path), "rank%d.npz" % rank))
        assert abs(r["sum_all"][0] - x.astype(np.float64).sum()) < 1e-9
        np.testing.assert_allclose(r["sum_0"], x.astype(np.float64).sum(0), atol=1e-9)
        np.testing.assert_array_equal(r["max_0"], oracle.reduce("max", x, 0))
        assert int(r["rows"][0]) == x.shape[0]
        np.testing.assert_array_equal(r["argmax_0"], oracle.argreduce("max", x, 0))
        np.testing.assert_array_equal(r["argmax_0_values"], oracle.reduce("max", x, 0))
        np.testing.assert_array_equal(r["argmin_0"], oracle.argreduce("min", x, 0))
        assert r["argmax_0"][5] == 10 and r["argmin_0"][7] == 60          # first occurrence across shards
        assert int(r["argmax_all"][0]) == int(oracle.argreduce("max", x))
        assert abs(r["chain"][0] - oracle.chain_sum(x, 0.5, 0.1)[1]) < 1e-9
        plan = list(r["plan"])
        assert plan[0] == "1:allreduce sum 1 f32"
        assert plan[1] == "1:allreduce max 37 f32"
        assert plan[2] == "1:arg_allreduce max 37 f32"
        assert plan[3] == "1:arg_allreduce max 1 f32"
        assert plan[4] == "1:allreduce sum 37 f32"
        assert plan[5] == "0:-"                                            # rows are independent: no collective
        assert plan[6].startswith("1:allreduce sum %d f32 (product" % (37 * 37))
        assert plan[7] == "0:-"


def test_collectives_need_a_communicator():
    sys.path.insert(0, ROOT)
    import dali_b200
    from dali_b200.capi import DaliB200Error
    lib = dali_b200.load_library()
    assert lib.comm_world() == 0 and lib.comm_rank() == -1 and lib.comm_transport() == "none"
    buf = np.zeros(4, np.float32)
    try:
        lib.allreduce(buf, 4, 0, "sum", device=-1)
        raise AssertionError("expected a failure")
    except DaliB200Error as e:
        assert "no communicator" in str(e)
