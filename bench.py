"""Benchmark of the fused-expression hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

One "step" is one pass of a fused expression over one batch of synthetic
input.  Prints ONE JSON line (rank 0).  Workloads (BASELINE.json configs):

  chain    sum(sigmoid(x*w+b) * exp(-x*x)) over 2^31 fp32 elements, one fused
           kernel; sharded over the GPUs with an all-reduce of the partial sums
  softmax  exp(a - max(a,-1)) / sum(...) on fp32 [4096,1024]; rows shard
  reduce   sum / max / argmax over axis -1, axis 0 and all axes of fp32 [8192,8192]
  lstm     LSTM-cell gating on materialised gates (B=256, H=1024)

`value` is whole-job algorithmic GB/s with inputs resident in HBM; `e2e` is the
same metric through dalib200_launch_host with pinned HOST buffers (copies
inside the timed region); `roofline` relates the dominant kernel to the
measured HBM copy bandwidth; `cpu_baseline` is the reference's own CPU path
(oracle/_ref) on a bounded sample, timed on this box's host cores.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SM_COUNT = 148
L2_BYTES = 126 * 1024 * 1024
FALLBACK_HBM_GBS = 6650.0          # earlier measurement on this pool, used if MEASURED_PEAKS.json is absent

# dram__bytes_read.sum + dram__bytes_write.sum per launch from the ncu captures summarised
# under profiles/ (bytes per ALGORITHMIC byte, so it scales with the launch size)
DRAM_TRAFFIC_PER_ALGO_BYTE = {}


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return FALLBACK_HBM_GBS, "fallback"


# ----------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples nvidia-smi clocks / throttle reasons while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.QUERY, "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()     # the exact process started above
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ----------------------------------------------------------------------------- reference CPU arm
def ref_driver_paths():
    d = os.path.join(ROOT, "oracle", "_ref")
    return os.path.join(d, "ref_driver"), os.path.join(d, "cache")


def run_ref_driver(case, args, reps, tmpdir):
    """Runs the reference's own CPU path; returns per-repeat milliseconds."""
    drv, cache = ref_driver_paths()
    if not os.path.exists(drv):
        return None
    env = dict(os.environ)
    env.setdefault("OPENBLAS_NUM_THREADS", str(os.cpu_count() or 1))
    out = subprocess.run([drv, cache, case] + args + [str(reps)], capture_output=True, text=True, env=env, cwd=tmpdir)
    if out.returncode != 0:
        raise RuntimeError("ref_driver failed: " + out.stderr[-2000:])
    for line in out.stdout.splitlines():
        if line.startswith("TIMES_MS"):
            return [float(x) for x in line.split()[1:]]
    return None


# ----------------------------------------------------------------------------- workloads
class Workload:
    name = ""
    dominant_kernel = ""

    def __init__(self, lib, torch, rank, world, device):
        self.lib, self.torch, self.rank, self.world, self.device = lib, torch, rank, world, device
        self.stream = torch.cuda.current_stream().cuda_stream

    def describe(self):
        raise NotImplementedError

    # algorithmic bytes one step moves on THIS rank
    def bytes_per_step(self):
        raise NotImplementedError

    def step(self, i):
        raise NotImplementedError

    def e2e_setup(self):
        raise NotImplementedError

    def e2e_step(self, i):
        raise NotImplementedError


class Chain(Workload):
    """BASELINE config 5: long elementwise chain + all-axis sum, strong-scaled over the ranks."""
    name = "chain"
    TOTAL = 1 << 31

    def __init__(self, *a, total=None):
        super().__init__(*a)
        import numpy as np
        from dali_b200.ir import chain_sum_ir
        self.np = np
        t = self.torch
        self.n = (total or self.TOTAL) // self.world
        t.manual_seed(1234 + 4 + self.rank)
        self.x = t.randn(self.n, dtype=t.float32, device="cuda")
        self.out = t.zeros(1, dtype=t.float32, device="cuda")
        self.h = self.lib.compile(chain_sum_ir())
        self.w, self.b = np.float32(0.5), np.float32(0.1)
        self.scaling = "strong"

    def describe(self):
        return {"workload": "C5 sum(sigmoid(x*w+b)*exp(-x*x)), fp32 x ~ N(0,1), 2^%d elements total, w=0.5 b=0.1"
                            % ((self.n * self.world).bit_length() - 1),
                "elements_per_gpu": self.n, "l2": "input per launch (%d MiB) larger than L2, no flush" % (self.n * 4 >> 20),
                "parallelism": "elements sharded over %d GPU(s), NCCL all-reduce of the partial sums" % self.world}

    def bytes_per_step(self):
        return self.n * 4

    def step(self, i):
        self.lib.launch(self.h, (self.n,), [self.out, self.x], scalars=[self.w, self.b], stream=self.stream)
        if self.world > 1:
            self.torch.distributed.all_reduce(self.out)

    def e2e_setup(self):
        t = self.torch
        self.hx = t.empty(self.n, dtype=t.float32, pin_memory=True)
        self.hx.copy_(self.x)
        self.hout = t.zeros(1, dtype=t.float32, pin_memory=True)
        self.h2d, self.d2h = self.n * 4, 4

    def e2e_step(self, i):
        # host buffers in, host result out: alloc + H2D + kernel + D2H + sync inside the call
        import ctypes
        n = 2
        ptrs = (ctypes.c_void_p * n)(self.hout.data_ptr(), self.hx.data_ptr())
        ext = (ctypes.c_int64 * n)(1, self.n)
        offs = (ctypes.c_int64 * n)(0, 0)
        space = (ctypes.c_int64 * 1)(self.n)
        w = self.np.array([0.5], self.np.float32)
        b = self.np.array([0.1], self.np.float32)
        sc = (ctypes.c_void_p * 2)(w.ctypes.data, b.ctypes.data)
        self.lib.check(self.lib.c.dalib200_launch_host(ctypes.c_uint64(self.h), self.device, space, 1, ptrs, ext, offs, None, n, sc, 2))

    def verify(self):
        """Order-independent check of the resident result against the oracle on a slice."""
        sys.path.insert(0, os.path.join(ROOT, "oracle"))
        import dali_oracle as oracle
        m = min(self.n, 1 << 22)
        xs = self.x[:m].contiguous()
        o = self.torch.zeros(1, dtype=self.torch.float32, device="cuda")
        self.lib.launch(self.h, (m,), [o, xs], scalars=[self.w, self.b], stream=self.stream)
        self.torch.cuda.synchronize()
        s32, s64, sabs = oracle.chain_sum(xs.cpu().numpy(), 0.5, 0.1)
        assert abs(float(o.item()) - s64) <= 1e-5 * sabs, (float(o.item()), s64)

    def cpu_baseline(self, tmpdir, reps):
        np = self.np
        m = 1 << 24
        x = self.x[:m].cpu().numpy()
        np.save(os.path.join(tmpdir, "x.npy"), x)
        times = run_ref_driver("chain", ["x.npy", "0.5", "0.1", "out.npy"], reps, tmpdir)
        if not times:
            return None
        return {"ms": times, "bytes": m * 4, "cores": 1, "kind": "reference",
                "sample": "first 2^24 elements of the same x (reference's generated CPU loop is single-threaded)"}


class Softmax(Workload):
    """BASELINE config 1: naive fused softmax on fp32 [4096,1024]."""
    name = "softmax"
    ROWS, COLS = 4096, 1024

    def __init__(self, *a):
        super().__init__(*a)
        import numpy as np
        from dali_b200.ir import softmax_ir
        self.np = np
        t = self.torch
        t.manual_seed(1234 + 0 + self.rank)
        self.nbuf = 12    # 12 x (16 MiB in + 16 MiB out) = 384 MiB rotates through the 126 MiB L2
        self.a = [t.randn(self.ROWS, self.COLS, dtype=t.float32, device="cuda") for _ in range(self.nbuf)]
        self.o = [t.empty(self.ROWS, self.COLS, dtype=t.float32, device="cuda") for _ in range(self.nbuf)]
        self.h = self.lib.compile(softmax_ir())
        self.scaling = "weak"

    def describe(self):
        return {"workload": "C1 exp(a-max(a,{-1},true))/sum(exped,{-1},true), fp32 [4096,1024] ~ N(0,1) per GPU",
                "l2": "rotating over %d input/output buffer pairs (%d MiB) so every launch misses L2" %
                      (self.nbuf, self.nbuf * 32),
                "parallelism": "rows sharded: each of %d GPU(s) runs its own [4096,1024] batch, no collective" % self.world}

    def bytes_per_step(self):
        return self.ROWS * self.COLS * 8

    def step(self, i):
        k = i % self.nbuf
        self.lib.launch(self.h, (self.ROWS, self.COLS), [self.o[k], self.a[k]], stream=self.stream)

    def e2e_setup(self):
        t = self.torch
        self.ha = t.empty(self.ROWS, self.COLS, dtype=t.float32, pin_memory=True)
        self.ha.copy_(self.a[0])
        self.ho = t.empty(self.ROWS, self.COLS, dtype=t.float32, pin_memory=True)
        self.h2d = self.d2h = self.ROWS * self.COLS * 4

    def e2e_step(self, i):
        import ctypes
        ptrs = (ctypes.c_void_p * 2)(self.ho.data_ptr(), self.ha.data_ptr())
        n = self.ROWS * self.COLS
        ext = (ctypes.c_int64 * 2)(n, n)
        offs = (ctypes.c_int64 * 2)(0, 0)
        space = (ctypes.c_int64 * 2)(self.ROWS, self.COLS)
        self.lib.check(self.lib.c.dalib200_launch_host(ctypes.c_uint64(self.h), self.device, space, 2, ptrs, ext, offs, None, 2, None, 0))

    def verify(self):
        sys.path.insert(0, os.path.join(ROOT, "oracle"))
        import dali_oracle as oracle
        self.step(0)
        self.torch.cuda.synchronize()
        got = self.o[0].cpu().numpy()
        want = oracle.softmax(self.a[0].cpu().numpy())
        assert self.np.allclose(got, want, rtol=1e-5, atol=1e-9)

    def cpu_baseline(self, tmpdir, reps):
        self.np.save(os.path.join(tmpdir, "a.npy"), self.a[0].cpu().numpy())
        times = run_ref_driver("softmax_naive", ["a.npy", "out.npy"], reps, tmpdir)
        if not times:
            return None
        return {"ms": times, "bytes": self.bytes_per_step(), "cores": 1, "kind": "reference",
                "sample": "the full [4096,1024] batch"}


WORKLOADS = {"chain": Chain, "softmax": Softmax}


# ----------------------------------------------------------------------------- main
def reference_arm(args):
    """--impl reference: the reference's own CPU implementation on this box's host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import tempfile
    import numpy as np
    drv, _ = ref_driver_paths()
    if not os.path.exists(drv):
        print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref/ref_driver was not built (no reference checkout at build time)"}))
        return
    peak, _ = measured_peak()
    with tempfile.TemporaryDirectory() as tmp:
        rng = np.random.default_rng(1234 + 4)
        if args.workload == "softmax":
            np.save(os.path.join(tmp, "a.npy"), rng.standard_normal((4096, 1024)).astype(np.float32))
            case, cargs, nbytes = "softmax_naive", ["a.npy", "out.npy"], 4096 * 1024 * 8
            wl = "C1 exp(a-max(a,{-1},true))/sum(exped,{-1},true), fp32 [4096,1024] ~ N(0,1) per GPU"
            sample = "the full [4096,1024] batch per step"
        else:
            m = 1 << 24
            np.save(os.path.join(tmp, "x.npy"), rng.standard_normal(m).astype(np.float32))
            case, cargs, nbytes = "chain", ["x.npy", "0.5", "0.1", "out.npy"], m * 4
            wl = "C5 sum(sigmoid(x*w+b)*exp(-x*x)), fp32 x ~ N(0,1), 2^31 elements total, w=0.5 b=0.1"
            sample = "2^24 elements per step (1/128 of the workload; the reference's int sizes cap a chunk at 2^28)"
        times = run_ref_driver(case, cargs, args.warmup + args.steps, tmp)
    timed = times[args.warmup:]
    ms = sum(timed) / len(timed)
    gbs = nbytes / (ms * 1e-3) / 1e9
    line = {"metric": "fused_expr_hbm_gbs", "value": gbs, "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong" if args.workload == "chain" else "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic", "impl": "reference",
            "config": {"workload": wl},
            "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": 1, "kind": "reference", "sample": sample},
            "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="chain", choices=sorted(WORKLOADS))
    ap.add_argument("--elements", type=int, default=0, help="chain: total elements (profiling on a small case)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        return reference_arm(args)

    import torch
    import dali_b200
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback")
    torch.cuda.set_device(local)
    if world > 1:
        torch.distributed.init_process_group("nccl", device_id=torch.device("cuda", local))
    lib = dali_b200.load_library()
    lib.init(0)
    # the library indexes the devices it bound; with one process per GPU that is `local`
    dev_index = local
    cls = WORKLOADS[args.workload]
    kw = {"total": args.elements} if (args.workload == "chain" and args.elements) else {}
    wl = cls(lib, torch, rank, world, dev_index, **kw)
    if dev_index != 0:
        # route every launch of this process to its own device
        orig_launch = lib.launch
        lib.launch = lambda *a, **k: orig_launch(*a, device=dev_index, **k)
    wl.verify()

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    for i in range(args.warmup):
        wl.step(i)
    barrier()
    sampler = ClockSampler(local)
    sampler.start()
    launches0 = lib.cache_stats()["launches"]
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    # long enough for nvidia-smi to sample clocks under load: repeat the K steps, time each block
    block_ms = []
    t_end = time.time() + 1.5
    while True:
        ev0.record()
        for i in range(args.steps):
            wl.step(args.warmup + i)
        ev1.record()
        barrier()
        block_ms.append(ev0.elapsed_time(ev1))
        if time.time() > t_end or len(block_ms) >= 50:
            break
    launches = (lib.cache_stats()["launches"] - launches0) // len(block_ms)
    clocks = sampler.stop()
    # the reported figure is the FIRST timed block of exactly K steps; the later blocks only
    # keep the GPU busy while clocks are sampled
    ms_total = block_ms[0]
    t = torch.tensor([ms_total], dtype=torch.float64, device="cuda")
    if world > 1:
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    ms_total = float(t.item())
    ms_step = ms_total / args.steps
    job_bytes = wl.bytes_per_step() * world
    value = job_bytes / (ms_step * 1e-3) / 1e9

    peak, peak_kind = measured_peak()
    achieved = wl.bytes_per_step() / (ms_step * 1e-3) / 1e9     # one launch per step on each GPU
    traffic_ratio = DRAM_TRAFFIC_PER_ALGO_BYTE.get(args.workload)
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "traffic": traffic_ratio * wl.bytes_per_step() if traffic_ratio else None,
                "peak_source": peak_kind + " (MEASURED_PEAKS.json hbm_gbs)" if peak_kind == "measured" else "fallback 6.65 TB/s",
                "kernel": lib.last_variant()}

    e2e = None
    if not args.no_e2e:
        wl.e2e_setup()
        for i in range(2):
            wl.e2e_step(i)
        barrier()
        n_e2e = max(1, min(args.steps, 5))
        t0 = time.perf_counter()
        for i in range(n_e2e):
            wl.e2e_step(i)      # synchronous: returns after the result is back in host memory
        barrier()
        dt = (time.perf_counter() - t0) / n_e2e
        te = torch.tensor([dt], dtype=torch.float64, device="cuda")
        if world > 1:
            torch.distributed.all_reduce(te, op=torch.distributed.ReduceOp.MAX)
        e2e = {"value": job_bytes / float(te.item()) / 1e9, "unit": "GB/s", "h2d_bytes_per_step": wl.h2d,
               "d2h_bytes_per_step": wl.d2h, "steps": n_e2e,
               "api": "dalib200_launch_host (pinned host buffers; alloc from pool + H2D + kernel + D2H + sync per step)"}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        import tempfile
        with tempfile.TemporaryDirectory() as tmp:
            r = wl.cpu_baseline(tmp, 8)
        if r:
            best = sorted(r["ms"])[len(r["ms"]) // 2]
            cpu = {"value": r["bytes"] / (best * 1e-3) / 1e9, "unit": "GB/s", "cores": r["cores"], "kind": r["kind"],
                   "sample": r["sample"], "ms": best}

    if rank == 0:
        cfg = wl.describe()
        line = {"metric": "fused_expr_hbm_gbs", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": wl.scaling,
                "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": cfg, "clocks": clocks,
                "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": int(launches),
                "pct_of_measured_hbm_peak": 100.0 * achieved / peak, "pct_of_nominal_8TBs": 100.0 * achieved / 8000.0}
        print(json.dumps(line))
    if world > 1:
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
