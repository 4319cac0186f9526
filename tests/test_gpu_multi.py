"""Two ranks on two GPUs (NCCL): rows / elements sharded, the same fused kernels on every
rank, partials combined as dali_b200/sharding.py says.  Skipped on a one-GPU box."""
import os
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    import dali_b200
    from dali_b200.ir import chain_sum_ir, reduce_ir, softmax_ir
    from dali_b200.sharding import combine_arg_partials, combine_partials, shard_range
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    lib = dali_b200.load_library()
    lib.init(0)
    st = torch.cuda.current_stream().cuda_stream
    rng = np.random.default_rng(11)
    x = (rng.random((512, 384)) * 2 - 1).astype(np.float32)
    x[100, 7] = x[400, 7] = 0.99999994
    lo, hi = shard_range(x.shape[0], rank, world)
    mine = torch.from_numpy(x[lo:hi]).cuda()
    rows = hi - lo
    res = {}
    # chain sum over the rank's elements + all-reduce
    out = torch.zeros(1, device="cuda")
    lib.launch(lib.compile(chain_sum_ir()), (mine.numel(),), [out, mine], scalars=[np.float32(0.5), np.float32(0.1)],
               device=rank, stream=st)
    res["chain"] = combine_partials(out, "sum").cpu().numpy()
    # axis-0 sum / max / argmax over sharded rows
    cols = x.shape[1]
    for kind in ("sum", "max"):
        o = torch.zeros(cols, device="cuda")
        lib.launch(lib.compile(reduce_ir(kind, "f32", 2, 1)), (cols, rows), [o, mine], strides=[None, [1, cols]], device=rank, stream=st)
        res[kind + "_0"] = combine_partials(o, kind).cpu().numpy()
    vmax = torch.zeros(cols, device="cuda")
    lib.launch(lib.compile(reduce_ir("max", "f32", 2, 1)), (cols, rows), [vmax, mine], strides=[None, [1, cols]], device=rank, stream=st)
    amax = torch.zeros(cols, dtype=torch.int32, device="cuda")
    lib.launch(lib.compile(reduce_ir("max", "f32", 2, 1, True)), (cols, rows), [amax, mine], strides=[None, [1, cols]], device=rank, stream=st)
    res["argmax_0"] = combine_arg_partials(vmax, amax, lo, "max").cpu().numpy()
    # softmax rows are independent: no collective, every rank keeps its rows
    sm = torch.empty_like(mine)
    lib.launch(lib.compile(softmax_ir()), (rows, cols), [sm, mine], device=rank, stream=st)
    res["softmax"] = sm.cpu().numpy()
    torch.cuda.synchronize()
    np.savez(os.path.join(out_dir, "rank%d.npz" % rank), **res)
    dist.destroy_process_group()


def test_two_gpu_sharded_expressions(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import dali_oracle as oracle
    from dali_b200.sharding import shard_range
    import torch.multiprocessing as mp
    world = 2
    port = 29600 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    rng = np.random.default_rng(11)
    x = (rng.random((512, 384)) * 2 - 1).astype(np.float32)
    x[100, 7] = x[400, 7] = 0.99999994
    s32, s64, sabs = oracle.chain_sum(x, 0.5, 0.1)
    sum0, abs0 = oracle.sum_f64acc(x, 0)
    for rank in range(world):
        r = np.load(os.path.join(str(tmp_path), "rank%d.npz" % rank))
        assert abs(float(r["chain"][0]) - s64) <= 1e-5 * sabs
        assert np.all(np.abs(r["sum_0"] - sum0) <= 1e-5 * abs0)
        np.testing.assert_array_equal(r["max_0"], oracle.reduce("max", x, 0))
        np.testing.assert_array_equal(r["argmax_0"], oracle.argreduce("max", x, 0))
        assert r["argmax_0"][7] == 100
        lo, hi = shard_range(x.shape[0], rank, world)
        np.testing.assert_allclose(r["softmax"], oracle.softmax(x[lo:hi]), rtol=1e-5, atol=1e-9)
