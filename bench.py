"""Benchmark of the fused-expression hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

One "step" is one pass of a fused expression over one batch of synthetic
input.  Prints ONE JSON line (rank 0).  Workloads (the benchmark configurations):

  chain    (default, configuration 5: the largest one) sum(sigmoid(x*w+b) * exp(-x*x))
           over 2^31 fp32 elements, sharded over the GPUs (strong scaling); the partial
           sums of the ranks meet inside the kernel through peer memory (NCCL all-reduce
           where the ranks cannot address one another)
  softmax  (config 1) exp(a - max(a,-1)) / sum(...) on fp32 [4096,1024]
  lstm     (config 2) fused LSTM cell step, fp32 B=256 H=1024: one tcgen05 3xTF32 GEMM
           accumulating x.Wx + h.Wh whose epilogue is the whole gating
  reduce   (config 3) --reduce-op sum|max|argmax over --axis -1|0|all of fp32 [8192,8192];
           rows sharded over the GPUs, axis 0 and all end in an all-reduce of the partials
           ((value, index) pairs for argmax)
  gemm     (config 4) tanh(dot(A,B)+bias), bf16 8192^3, fp32 accumulate
  gather   rows of a [65536,256] fp32 table picked by 2^20 int32 indices (op::gather)
The default run also measures the others (all nine reductions) at every N and
reports them under "other_workloads", each with its own roofline, clocks, end-to-end
figure and (N = 1) CPU baseline.

`value` is whole-job algorithmic GB/s with inputs resident in HBM; `e2e` is the
same metric through the public call with pinned HOST buffers (copies inside the
timed region); `roofline` relates the dominant kernel to the measured HBM copy
bandwidth (or the measured bf16 GEMM rate); `cpu_baseline` is the reference's own
CPU path (oracle/_ref) on a bounded sample, timed on this box's host cores.
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
F32, F64, I32 = 0, 1, 2

# dram__bytes_read.sum + dram__bytes_write.sum per launch from ncu captures of the dominant kernels
# (bytes per ALGORITHMIC byte, so it scales with the launch size)
DRAM_TRAFFIC_PER_ALGO_BYTE = {
    "chain": 1.0004,
    "softmax": 0.50,     # the 16 MiB output is still in L2 when the kernel ends
    "reduce": 1.0002,
    "scan": 0.905,       # the tail of the output is written back after the kernel ends
    "transpose": 0.919,  # likewise
}


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
    """One benchmark configuration.  `config(world, **kw)` is the `config` object of the JSON line, a function of the
    command line only (the reference arm prints the same one); `reference_case(np, tmp, **kw)` writes a bounded sample
    of the workload for the reference's CPU path and names the driver case that runs it."""
    name = ""
    scaling = "weak"
    dtype = "f32"
    launches_per_step = 1
    hbm_metric = True          # `value` counts bytes that cross HBM (False: operands that stay in L2, or a tensor-bound step)

    def __init__(self, lib, torch, rank, world, device):
        self.lib, self.torch, self.rank, self.world, self.device = lib, torch, rank, world, device
        self.stream = torch.cuda.current_stream().cuda_stream
        self.peer = world > 1 and lib.comm_transport() == "nccl+peer"

    def bytes_per_step(self):          # algorithmic bytes one step moves on THIS rank
        raise NotImplementedError

    def flops_per_step(self):
        return 0

    def step(self, i):
        self.launch_step(i, self.stream)

    def graph_fn(self):
        """launch(i, stream) of one step's kernels when every launch can be captured (NCCL calls are left eager)."""
        return self.launch_step if (self.world == 1 or self.peer or not self.has_collective()) else None

    def has_collective(self):
        return False

    def dominant(self):
        """(kernel name, bound, algorithmic work per launch, launch(i, stream)) or None = the step itself."""
        return None


def _collective_note(world):
    return ("; partial results meet in peer memory inside / right after the kernel (NCCL where ranks cannot address one another)"
            if world > 1 else "")


class Chain(Workload):
    """Benchmark configuration 5: long elementwise chain + all-axis sum, strong-scaled over the ranks."""
    name = "chain"
    scaling = "strong"
    TOTAL = 1 << 31

    @staticmethod
    def config(world, total=None, **kw):
        total = total or Chain.TOTAL
        n = total // world
        return {"workload": "C5 sum(sigmoid(x*w+b)*exp(-x*x)), fp32 x ~ N(0,1), 2^%d elements total, w=0.5 b=0.1" % (total.bit_length() - 1),
                "elements_per_gpu": n, "l2": "input per launch (%d MiB) larger than L2, no flush" % (n * 4 >> 20),
                "parallelism": "elements sharded over %d GPU(s)%s" % (world, "; the ranks' partial sums are exchanged through peer "
                               "memory inside the kernel that computes them (NCCL all-reduce where ranks cannot address one another)" if world > 1 else "")}

    @staticmethod
    def reference_case(np, tmp, **kw):
        m = 1 << 24
        np.save(os.path.join(tmp, "x.npy"), np.random.default_rng(1234 + 4).standard_normal(m).astype(np.float32))
        return {"case": "chain", "args": ["x.npy", "0.5", "0.1", "out.npy"], "bytes": m * 4, "cores": 1,
                "sample": "2^24 elements per step (1/128 of the workload; the reference's generated loop is single-threaded and its int sizes cap a chunk at 2^28)"}

    def __init__(self, *a, total=None):
        super().__init__(*a)
        import numpy as np
        from dali_b200.ir import chain_sum_ir
        self.np = np
        t = self.torch
        self.total = total or self.TOTAL
        self.n = self.total // self.world
        t.manual_seed(1234 + 4 + self.rank)
        self.x = t.randn(self.n, dtype=t.float32, device="cuda")
        self.out = t.zeros(1, dtype=t.float32, device="cuda")
        self.h = self.lib.compile(chain_sum_ir(xrank=self.peer))
        self.h_local = self.lib.compile(chain_sum_ir())
        self.w, self.b = np.float32(0.5), np.float32(0.1)
        self.launches_per_step = 1 if (self.world == 1 or self.peer) else 2

    def bytes_per_step(self):
        return self.n * 4

    def has_collective(self):
        return self.world > 1

    def launch_step(self, i, stream):
        self.lib.launch(self.h, (self.n,), [self.out, self.x], scalars=[self.w, self.b], device=self.device, stream=stream)
        if self.world > 1 and not self.peer:
            self.lib.allreduce(self.out, 1, F32, "sum", device=self.device, stream=stream)

    def e2e_setup(self):
        t = self.torch
        self.hx = t.empty(self.n, dtype=t.float32, pin_memory=True)
        self.hx.copy_(self.x)
        self.hout = t.zeros(1, dtype=t.float32, pin_memory=True)
        self.dx = t.empty(self.n, dtype=t.float32, device="cuda") if self.world > 1 and not self.peer else None
        self.h2d, self.d2h = self.n * 4, 4
        if self.dx is not None:
            self.e2e_api = "C ABI with caller-managed copies (page-locked host -> device, dalib200_launch, dalib200_allreduce, device -> page-locked host, sync)"

    def e2e_step(self, i):
        if self.dx is not None:
            # (ranks that cannot address one another: the NCCL all-reduce needs the partial sum on the device)
            self.dx.copy_(self.hx, non_blocking=True)
            self.lib.launch(self.h_local, (self.n,), [self.out, self.dx], scalars=[self.w, self.b], device=self.device, stream=self.stream)
            self.lib.allreduce(self.out, 1, F32, "sum", device=self.device, stream=self.stream)
            self.hout.copy_(self.out, non_blocking=True)
            self.torch.cuda.synchronize()
            return
        # host buffers in, host result out: alloc + H2D + kernel (with the ranks' exchange inside) + D2H + sync in one call
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
        """Order-independent check of the resident result against the oracle on a slice; with several ranks also the
        combined sum against the ranks' own partial sums added up by torch.distributed."""
        sys.path.insert(0, os.path.join(ROOT, "oracle"))
        import dali_oracle as oracle
        t = self.torch
        m = min(self.n, 1 << 22)
        xs = self.x[:m].contiguous()
        o = t.zeros(1, dtype=t.float32, device="cuda")
        self.lib.launch(self.h_local, (m,), [o, xs], scalars=[self.w, self.b], device=self.device, stream=self.stream)
        t.cuda.synchronize()
        s32, s64, sabs = oracle.chain_sum(xs.cpu().numpy(), 0.5, 0.1)
        assert abs(float(o.item()) - s64) <= 1e-5 * sabs, (float(o.item()), s64)
        if self.world > 1:
            self.lib.launch(self.h_local, (self.n,), [o, self.x], scalars=[self.w, self.b], device=self.device, stream=self.stream)
            part = o.double()
            t.distributed.all_reduce(part)
            self.step(0)
            t.cuda.synchronize()
            assert self.lib.comm_error_flag() == 0, "a rank did not arrive at the exchange in time"
            assert abs(float(self.out.item()) - float(part.item())) <= 1e-6 * abs(float(part.item())), (float(self.out.item()), float(part.item()))


class Softmax(Workload):
    """Benchmark configuration 1: naive fused softmax on fp32 [4096,1024]."""
    name = "softmax"
    ROWS, COLS = 4096, 1024
    NBUF = 12     # 12 x (16 MiB in + 16 MiB out) = 384 MiB rotates through the 126 MiB L2

    @staticmethod
    def config(world, shape=None, **kw):
        R, C = shape or (Softmax.ROWS, Softmax.COLS)
        nbuf = max(2, min(Softmax.NBUF, (768 << 20) // (R * C * 8)))
        return {"workload": "%sexp(a-max(a,{-1},true))/sum(exped,{-1},true), fp32 [%d,%d] ~ N(0,1) per GPU" % ("C1 " if not shape else "", R, C),
                "l2": "rotating over %d input/output buffer pairs (%d MiB) so every launch misses L2" % (nbuf, nbuf * (R * C * 8 >> 20)),
                "concurrency": "one stream: batch after batch",
                "parallelism": "rows sharded: each of %d GPU(s) runs its own [4096,1024] batch, no collective" % world}

    @staticmethod
    def reference_case(np, tmp, **kw):
        np.save(os.path.join(tmp, "a.npy"), np.random.default_rng(1234).standard_normal((4096, 1024)).astype(np.float32))
        return {"case": "softmax_naive", "args": ["a.npy", "out.npy"], "bytes": 4096 * 1024 * 8, "cores": 1,
                "sample": "the full [4096,1024] batch per step (the reference's generated loops are single-threaded)"}

    def __init__(self, *a, shape=None):
        super().__init__(*a)
        import numpy as np
        from dali_b200.ir import softmax_ir
        self.np = np
        t = self.torch
        t.manual_seed(1234 + 0 + self.rank)
        if shape:
            self.ROWS, self.COLS = shape            # --softmax-shape R,C: few long rows and other shapes (profiling)
        self.nbuf = max(2, min(self.NBUF, (768 << 20) // (self.ROWS * self.COLS * 8)))
        self.a = [t.randn(self.ROWS, self.COLS, dtype=t.float32, device="cuda") for _ in range(self.nbuf)]
        self.o = [t.empty(self.ROWS, self.COLS, dtype=t.float32, device="cuda") for _ in range(self.nbuf)]
        self.h = self.lib.compile(softmax_ir())

    def bytes_per_step(self):
        return self.ROWS * self.COLS * 8

    def launch_step(self, i, stream):
        k = i % self.nbuf
        self.lib.launch(self.h, (self.ROWS, self.COLS), [self.o[k], self.a[k]], device=self.device, stream=stream)

    def extra(self, torch):
        """The same kernel with consecutive (independent) batches on three streams, as a serving loop with several
        requests in flight would issue them: GB/s."""
        g = GraphStepper(torch, self.launch_step, 24, 3)
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(g.stream)
        g.replay()
        e1.record(g.stream)
        torch.cuda.synchronize()
        return {"three_streams_gbs": self.bytes_per_step() * 24 / (e0.elapsed_time(e1) * 1e-3) / 1e9}

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
        rows = list(range(self.ROWS)) if self.ROWS * self.COLS <= (1 << 23) else sorted({0, self.ROWS // 2, self.ROWS - 1})
        got = self.o[0][rows].cpu().numpy()
        a = self.a[0][rows].cpu().numpy()
        if self.COLS <= 65536:
            want = oracle.softmax(a)
        else:
            # (the reference's sequential fp32 sum of a million terms is itself 1e-4 off: long rows are held to the fp64 value)
            e = self.np.exp(a.astype(self.np.float64) - a.max(1, keepdims=True))
            want = e / e.sum(1, keepdims=True)
        assert self.np.allclose(got, want, rtol=1e-5, atol=1e-12)


class GraphStepper:
    """Replays the launches of `fn(i, stream)` for i in range(n) as one CUDA graph (device time without
    Python between the kernels).  With lanes > 1 step i goes to lane i % lanes: independent steps (separate
    batches) form parallel chains in the graph, so one batch's tail overlaps the next one's ramp-up."""

    def __init__(self, torch, fn, n, lanes=1):
        self.torch = torch
        self.stream = torch.cuda.Stream()
        self.side = [torch.cuda.Stream() for _ in range(lanes - 1)]
        self.n = n
        lanes_streams = [self.stream] + self.side
        with torch.cuda.stream(self.stream):
            for i in range(n):
                fn(i, lanes_streams[i % lanes].cuda_stream)      # compile / load / warm pools outside the capture
            torch.cuda.synchronize()
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, stream=self.stream):
                for s_ in self.side:
                    s_.wait_stream(self.stream)                   # fork
                for i in range(n):
                    fn(i, lanes_streams[i % lanes].cuda_stream)
                for s_ in self.side:
                    self.stream.wait_stream(s_)                   # join
        torch.cuda.synchronize()

    def replay(self):
        with self.torch.cuda.stream(self.stream):     # a graph replays on the stream that is current
            self.graph.replay()


class Lstm(Workload):
    """Benchmark configuration 2: fused LSTM cell step, fp32, B=256 H=1024 per GPU."""
    name = "lstm"
    B, H = 256, 1024
    NSET = 6
    hbm_metric = False         # the two weight matrices (32 of the 38.8 MB) are reused every step and stay in L2
    launches_per_step = 2
    dominant_traffic_bytes = 75.8e6      # ncu: 72.4 MB read + 3.4 MB written per launch with a cold L2
    dominant_traffic_note = "ncu capture with a cold L2 (64 MB of split weights read from DRAM); in the timed loop the weights stay in L2"
    e2e_api = ("page-locked host arrays -> lazy Array / op:: expression -> Array::eval_together -> host arrays, in C++ against "
               "the front end's headers (dali_b200/host/programs/lstm_cell_e2e.cpp)")

    @staticmethod
    def config(world, **kw):
        return {"workload": "C2 LSTM cell step: gates = dot(x,Wx)+dot(h,Wh)+b, c' = sig(f)*c + sig(i)*tanh(g), "
                            "h' = sig(o)*tanh(c'); fp32, B=256 H=1024 per GPU, x,h,c ~ N(0,1), W ~ N(0,0.02), b = 0",
                "l2": "activations rotate over %d sets; the two weight matrices are reused every step (as in an RNN) "
                      "and stay in L2: `value` counts their bytes too and is therefore not an HBM bandwidth" % Lstm.NSET,
                "kernels_per_step": "1 tcgen05 3xTF32 GEMM accumulating x.Wx + h.Wh whose epilogue is the whole gating (+ b, sigmoid / tanh, c', h'; the [B,4H] gates are never written) and which leaves h' as the two TF32 parts the next step reads, 1 TF32 split of the step's x",
                "recurrence": "the timed loop is a recurrence: step t+1 reads step t's h' and c'; x_t rotates over the sets, and the split of x_(t+1) is issued on a second stream so that it runs beside step t's GEMM",
                "parallelism": "batch sharded: each of %d GPU(s) runs its own B=256 shard, weights replicated, no collective" % world}

    @staticmethod
    def reference_case(np, tmp, **kw):
        rng = np.random.default_rng(1234 + 1)
        B, H = Lstm.B, Lstm.H
        for k in ("x", "h", "c"):
            np.save(os.path.join(tmp, k + ".npy"), rng.standard_normal((B, H)).astype(np.float32))
        for k in ("Wx", "Wh"):
            np.save(os.path.join(tmp, k + ".npy"), (rng.standard_normal((H, 4 * H)) * 0.02).astype(np.float32))
        np.save(os.path.join(tmp, "b.npy"), np.zeros((1, 4 * H), np.float32))
        return {"case": "lstm", "args": ["x.npy", "h.npy", "c.npy", "Wx.npy", "Wh.npy", "b.npy", "c_out.npy", "h_out.npy"],
                "bytes": 4 * (3 * B * H + 2 * H * 4 * H + 4 * H + 2 * B * H), "flops": 2.0 * 2 * B * H * 4 * H, "cores": os.cpu_count() or 1,
                "sample": "the full B=256 H=1024 cell step (reference: 8 OpenBLAS sgemm on all host cores + 5 single-threaded JIT kernels)"}

    def __init__(self, *a):
        super().__init__(*a)
        import numpy as np
        self.np = np
        t, B, H = self.torch, self.B, self.H
        t.manual_seed(1234 + 1 + self.rank)
        self.nset = self.NSET       # rotating activation sets; weights (2 x 16 MiB, split: 64 MiB) stay hot like in a real RNN
        self.x = [t.randn(B, H, device="cuda") for _ in range(self.nset)]
        self.h = [t.randn(B, H, device="cuda") for _ in range(self.nset)]
        self.c = [t.randn(B, H, device="cuda") for _ in range(self.nset)]
        self.Wx = t.randn(H, 4 * H, device="cuda") * 0.02
        self.Wh = t.randn(H, 4 * H, device="cuda") * 0.02
        self.b = t.zeros(4 * H, device="cuda")
        self.c_new = [t.empty(B, H, device="cuda") for _ in range(self.nset)]
        self.h_new = [t.empty(B, H, device="cuda") for _ in range(self.nset)]
        L = self.lib
        # weights are split once and kept, as the front end keeps them next to the buffer
        self.W = {}
        for name, w in (("Wx", self.Wx), ("Wh", self.Wh)):
            hi, lo = t.empty(4 * H * H, device="cuda"), t.empty(4 * H * H, device="cuda")
            L.gemm_split_tf32(w, H, 4 * H, 4 * H, hi, lo, transpose=True, device=self.device)
            self.W[name] = (hi, lo)
        self.parts = [t.empty(B * H, device="cuda") for _ in range(4)]
        # what the front end emits for eval_together(c', h'): the gating is the epilogue of the gate products
        from dali_b200.ir import lstm_cell_epilogue_ir
        self.h_cell = L.compile(lstm_cell_epilogue_ir())
        # the recurrent loop: state (c, h as its two TF32 parts) and the parts of x, each in two copies by step parity
        self.h_cell_split = L.compile(lstm_cell_epilogue_ir(split_h=True))
        self.xparts = [[t.empty(B * H, device="cuda") for _ in range(2)] for _ in range(2)]
        self.hparts = [[t.empty(B * H, device="cuda") for _ in range(2)] for _ in range(2)]
        self.c_state = [t.empty(B, H, device="cuda") for _ in range(2)]
        self.h_state = [t.empty(B, H, device="cuda") for _ in range(2)]
        self.side = t.cuda.Stream()
        self.reset_state()

    def reset_state(self):
        """Step 0 starts from c[0] and h[0]."""
        self.torch.cuda.synchronize()
        self.c_state[0].copy_(self.c[0])
        self.h_state[0].copy_(self.h[0])
        self.lib.gemm_split_tf32(self.h[0], self.B, self.H, self.H, *self.hparts[0], device=self.device)
        self.torch.cuda.synchronize()

    def bytes_per_step(self):
        B, H = self.B, self.H
        return 4 * (3 * B * H + 2 * H * 4 * H + 4 * H + 2 * B * H)

    def flops_per_step(self):
        return 2 * 2 * self.B * self.H * 4 * self.H

    def split_x(self, i, stream):
        self.lib.gemm_split_tf32(self.x[i % self.nset], self.B, self.H, self.H, *self.xparts[i % 2], device=self.device, stream=stream)

    def launch_cell(self, i, stream):
        """Step i of the recurrence: reads the parts of x_i and the state of parity i % 2, writes the state of the other parity."""
        B, H, W, p = self.B, self.H, self.W, i % 2
        X, Hp, q = self.xparts[p], self.hparts[p], 1 - p
        row = [0, 1]
        self.lib.gemm_fused_sum(0, B, H, [(H, X[0], H, W["Wx"][0], H, X[1], W["Wx"][1]),
                                          (H, Hp[0], H, W["Wh"][0], H, Hp[1], W["Wh"][1])],
                                self.h_cell_split,
                                [self.c_state[q], self.h_state[q], self.b, self.b, self.b, self.b, self.c_state[p],
                                 self.hparts[q][0], self.hparts[q][1]],
                                strides=[None, None, row, row, row, row, None, None, None], offsets=[0, 0, 0, H, 2 * H, 3 * H, 0, 0, 0],
                                device=self.device, stream=stream)

    def launch_step(self, i, stream):
        self.split_x(i, stream)
        self.launch_cell(i, stream)

    def graph_fn(self):
        """One block of `block_steps` steps as the graph captures it: the cells follow one another on the main stream, the
        split of the next step's x goes to a second stream (forked at the block's first step, joined by its last)."""
        n = getattr(self, "block_steps", 0)
        if n < 2:
            return self.launch_step
        t = self.torch
        st = {"calls": 0, "x_ready": None, "prev_cell": None}

        def fn(i, stream):
            main = t.cuda.ExternalStream(stream)
            pos = st["calls"] % n
            st["calls"] += 1
            if pos == 0:
                self.side.wait_stream(main)                    # fork
                self.split_x(i, self.side.cuda_stream)
                st["x_ready"] = t.cuda.Event()
                st["x_ready"].record(self.side)
                st["prev_cell"] = None
            main.wait_event(st["x_ready"])                     # the last step's wait joins the second stream
            self.launch_cell(i, stream)
            if pos + 1 < n:
                done = t.cuda.Event()
                done.record(main)
                if st["prev_cell"] is not None:
                    self.side.wait_event(st["prev_cell"])      # the cell before this one read the parts about to be overwritten
                self.split_x(i + 1, self.side.cuda_stream)
                st["x_ready"] = t.cuda.Event()
                st["x_ready"].record(self.side)
                st["prev_cell"] = done
        return fn

    def launch_gemm(self, stream, k=0):
        B, H, P, W = self.B, self.H, self.parts, self.W
        row = [0, 1]
        self.lib.gemm_fused_sum(0, B, H, [(H, P[0], H, W["Wx"][0], H, P[1], W["Wx"][1]),
                                          (H, P[2], H, W["Wh"][0], H, P[3], W["Wh"][1])],
                                self.h_cell, [self.c_new[k], self.h_new[k], self.b, self.b, self.b, self.b, self.c[k]],
                                strides=[None, None, row, row, row, row, None], offsets=[0, 0, 0, H, 2 * H, 3 * H, 0],
                                device=self.device, stream=stream)

    def dominant(self):
        B, H = self.B, self.H
        return ("tcgen05 3xTF32 GEMM [256,1024]x[1024,4096] + [256,1024]x[1024,4096], one accumulator, LSTM gating as epilogue", "tensor",
                2.0 * 2 * B * H * 4 * H, lambda i, stream: self.launch_gemm(stream))

    def e2e_external(self, warmup, steps):
        """ms per step of dali_b200/host/programs/lstm_cell_e2e.cpp: the cell through the C++ Array / op:: API with
        page-locked host arrays in and out every step."""
        from dali_b200 import build as _build
        exe = os.path.join(ROOT, "dali_b200", "lib", "lstm_cell_e2e")
        if not os.path.exists(exe):
            _build.build_programs()
        cmd = [exe, str(self.device), str(self.B), str(self.H), str(warmup), str(steps)]
        ncpu = os.cpu_count() or 1
        if self.world > 1 and ncpu >= 2 * self.world:
            # every rank's host loop on cores of its own: with all ranks on the same few cores the step time of one
            # rank depends on what the others are doing
            per = ncpu // self.world
            cmd = ["taskset", "-c", "%d-%d" % (self.rank * per, self.rank * per + per - 1)] + cmd
        out = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
        if out.returncode != 0:
            raise RuntimeError("lstm_cell_e2e failed: " + out.stderr[-2000:])
        r = json.loads(out.stdout.strip().splitlines()[-1])
        self.h2d, self.d2h = r["h2d_bytes_per_step"], r["d2h_bytes_per_step"]
        return r["ms_per_step"]

    def verify(self):
        """Two steps of the recurrence from (x_0, h_0, c_0) against the oracle's gating of fp64 gate products, and the
        parts the epilogue leaves of h' against h' itself (hi + lo is exact)."""
        sys.path.insert(0, os.path.join(ROOT, "oracle"))
        import dali_oracle as oracle
        np = self.np
        self.reset_state()
        Wx, Wh = (v.cpu().numpy().astype(np.float64) for v in (self.Wx, self.Wh))
        h, c = self.h[0].cpu().numpy(), self.c[0].cpu().numpy()
        for i in range(2):
            self.step(i)
            self.torch.cuda.synchronize()
            assert self.lib.gemm_error_flag(self.device) == 0
            gates = (self.x[i].cpu().numpy().astype(np.float64) @ Wx + h.astype(np.float64) @ Wh).astype(np.float32)
            c, h = oracle.lstm_gating(gates, c)
            q = (i + 1) % 2
            got_c, got_h = self.c_state[q].cpu().numpy(), self.h_state[q].cpu().numpy()
            assert np.allclose(got_c, c, rtol=1e-5, atol=1e-5 * (i + 1))
            assert np.allclose(got_h, h, rtol=1e-5, atol=1e-5 * (i + 1))
            hi, lo = (v.cpu().numpy().reshape(got_h.shape) for v in self.hparts[q])
            assert np.array_equal(hi + lo, got_h) and np.array_equal(hi.view(np.uint32) & 0x1fff, np.zeros_like(hi, np.uint32))
        self.reset_state()


class Gemm(Workload):
    """Benchmark configuration 4: tanh(dot(A,B)+bias), bf16 8192^3, fp32 accumulate, bf16 out."""
    name = "gemm"
    dtype = "bf16"
    hbm_metric = False
    e2e_api = ("page-locked host arrays of bf16 -> lazy Array / op:: expression op::tanh(op::dot(A, B) + bias).astype(bf16) -> eval -> "
               "host array (the Python face of the C++ front end)")
    N = 8192

    @staticmethod
    def config(world, n=None, **kw):
        n = n or Gemm.N
        return {"workload": "C4 tanh(dot(A,B)+bias), bf16 A,B [%d,%d] ~ N(0,0.02), bias ~ N(0,0.1), fp32 accumulate, bf16 out" % (n, n),
                "l2": "operands + output = %d MiB per launch, larger than L2" % (3 * n * n * 2 >> 20),
                "parallelism": "rows of A sharded: each of %d GPU(s) runs its own [%d,%d] block, B and bias replicated, no collective" % (world, n, n)}

    @staticmethod
    def reference_case(np, tmp, **kw):
        rng = np.random.default_rng(1237)
        m = 2048
        np.save(os.path.join(tmp, "A.npy"), (rng.standard_normal((m, m)) * 0.02).astype(np.float32))
        np.save(os.path.join(tmp, "B.npy"), (rng.standard_normal((m, m)) * 0.02).astype(np.float32))
        np.save(os.path.join(tmp, "bias.npy"), (rng.standard_normal(m) * 0.1).astype(np.float32))
        return {"case": "gemm_tanh", "args": ["A.npy", "B.npy", "bias.npy", "out.npy"], "bytes": 3 * m * m * 2, "flops": 2.0 * m ** 3,
                "cores": os.cpu_count() or 1, "max_reps": 3,
                "sample": "2048^3 in fp32 per step (the reference has no bf16; 1/64 of the flops): OpenBLAS sgemm on all host cores + the reference's single-threaded tanh kernel"}

    def __init__(self, *a, n=None):
        super().__init__(*a)
        import numpy as np
        from dali_b200.ir import gemm_bias_tanh_ir
        self.np = np
        t = self.torch
        n = self.n = n or self.N
        t.manual_seed(1234 + 3 + self.rank)
        self.A = (t.randn(n, n, device="cuda") * 0.02).bfloat16()
        self.Bm = (t.randn(n, n, device="cuda") * 0.02).bfloat16()
        self.bias = t.randn(n, device="cuda") * 0.1
        self.out = t.empty(n, n, device="cuda", dtype=t.bfloat16)
        self.h = self.lib.compile(gemm_bias_tanh_ir("bf16"))

    def bytes_per_step(self):
        return 3 * self.n * self.n * 2

    def flops_per_step(self):
        return 2 * self.n ** 3

    def launch_step(self, i, stream):
        n = self.n
        self.lib.gemm_fused(3, n, n, n, self.A, n, self.Bm, n, self.h, [self.out, self.bias], strides=[None, [0, 1]],
                            device=self.device, stream=stream)

    def dominant(self):
        return ("tcgen05 bf16 GEMM + bias/tanh epilogue", "tensor", float(self.flops_per_step()), self.launch_step)

    def e2e_setup(self):
        t = self.torch
        n = self.n
        # page-locked host buffers holding bf16 bit patterns, seen by numpy as uint16
        self.hA, self.hB, self.hout = (t.empty(n, n, dtype=t.int16, pin_memory=True) for _ in range(3))
        self.hA.copy_(self.A.view(t.int16)); self.hB.copy_(self.Bm.view(t.int16))
        self.hbias = t.empty(n, pin_memory=True); self.hbias.copy_(self.bias)
        self.bits = {k: getattr(self, k).numpy().view(self.np.uint16) for k in ("hA", "hB", "hout")}
        from dali_b200.array import set_default_device
        set_default_device(self.device)
        self.h2d, self.d2h = 2 * n * n * 2 + n * 4, n * n * 2

    def e2e_step(self, i):
        # the call a user makes: page-locked host arrays in, the reference's expression on bf16 Arrays, the result back
        from dali_b200.array import Array, DTYPE_BF16, op
        A, B = Array.borrow(self.bits["hA"], DTYPE_BF16), Array.borrow(self.bits["hB"], DTYPE_BF16)
        bias = Array.borrow(self.hbias.numpy())
        y = op.tanh(op.dot(A, B) + bias[None, :]).astype(DTYPE_BF16)
        y.numpy(out=self.bits["hout"])

    def verify(self):
        """The WHOLE output against tanh(A.float() @ B.float() + bias) computed by torch in fp32 on the device (a checker,
        not part of the path), plus three rows against the fp64 product."""
        np, n, t = self.np, self.n, self.torch
        self.step(0)
        t.cuda.synchronize()
        assert self.lib.gemm_error_flag(self.device) == 0
        prev = t.backends.cuda.matmul.allow_tf32
        t.backends.cuda.matmul.allow_tf32 = False
        bad = 0
        for r0 in range(0, n, 2048):
            want = t.tanh(self.A[r0:r0 + 2048].float() @ self.Bm.float() + self.bias)
            bad += int((~t.isclose(self.out[r0:r0 + 2048].float(), want, rtol=1e-2, atol=4e-3)).sum().item())
        t.backends.cuda.matmul.allow_tf32 = prev
        assert bad == 0, "%d of %d outputs outside rtol 1e-2" % (bad, n * n)
        rows = [0, 129, n - 1]
        a = self.A[rows].float().cpu().numpy().astype(np.float64)
        want = np.tanh(a @ self.Bm.float().cpu().numpy().astype(np.float64) + self.bias.cpu().numpy())
        assert np.allclose(self.out[rows].float().cpu().numpy(), want, rtol=1e-2, atol=4e-3)


class Reduce(Workload):
    """Benchmark configuration 3: sum / max / argmax over axis -1, axis 0 or all axes of fp32 [8192,8192] per GPU.
    The rows of the logical [world * 8192, 8192] array are sharded: axis -1 needs no exchange, axis 0 ends in an
    all-reduce of the [8192] partials and the all-axis forms in an exchange of one value (for argmax: of (value,
    position) pairs, positions being those of the logical array)."""
    name = "reduce"
    N = 8192
    e2e_api = "C ABI with caller-managed copies (page-locked host -> device, dalib200_launch [+ dalib200_allreduce], device -> page-locked host, sync)"

    @staticmethod
    def config(world, op="sum", axis="0", **kw):
        what = {"-1": "axis -1", "0": "axis 0", "all": "all axes"}[str(axis)]
        if world == 1 or str(axis) == "-1":
            par = "rows sharded over %d GPU(s), no collective" % world
        elif op == "argmax":
            par = "rows sharded over %d GPU(s); the ranks' (value, position) pairs are combined, lowest position among equals" % world
        else:
            par = "rows sharded over %d GPU(s); the partial results meet in an all-reduce" % world
        return {"workload": "C3 op::%s over %s of fp32 [8192,8192] ~ U(-1,1) per GPU" % (op, what),
                "l2": "two 256 MiB inputs alternate (512 MiB > L2)", "parallelism": par + _collective_note(world if str(axis) != "-1" else 1)}

    @staticmethod
    def reference_case(np, tmp, op="sum", axis="0", **kw):
        m = 2048
        np.save(os.path.join(tmp, "x.npy"), (np.random.default_rng(1236).random((m, m)) * 2 - 1).astype(np.float32))
        return {"case": "reduce", "args": [op, str(axis), "x.npy", "out.npy"], "bytes": m * m * 4, "cores": 1,
                "sample": "a [2048,2048] array per step (1/16 of the bytes; the reference's generated loop is single-threaded)"}

    def __init__(self, *a, op="sum", axis="0"):
        super().__init__(*a)
        import numpy as np
        from dali_b200.ir import arg_pair_ir, reduce_ir
        self.np = np
        t, N, L = self.torch, self.N, self.lib
        self.op, self.axis = op, str(axis)
        assert op in ("sum", "max", "argmax") and self.axis in ("-1", "0", "all")
        t.manual_seed(1234 + 2 + self.rank)
        self.x = [t.rand(N, N, device="cuda") * 2 - 1 for _ in range(2)]    # 2 x 256 MiB > L2
        self.arg = op == "argmax"
        self.kind = "max" if self.arg else op
        n_out = 1 if self.axis == "all" else N
        self.out = t.zeros(n_out, device="cuda", dtype=t.int32 if self.arg else t.float32)
        self.vals = t.zeros(n_out, device="cuda")
        self.collective = self.world > 1 and self.axis != "-1"
        self.fused = self.collective and self.axis == "all" and self.peer
        self.pair = self.collective and self.arg and not self.fused
        self.rank_ir = 1 if self.axis == "all" else 2
        # position of this rank's shard in the logical array: rows for axis 0, elements for all axes
        offset = self.rank * N if self.axis == "0" else self.rank * N * N
        self.scalars = [np.int32(offset)] if ((self.fused and self.arg) or self.pair) else None
        if self.fused:
            self.h = L.compile(reduce_ir(self.kind, "f32", 1, 1, self.arg, xrank=True))
        elif self.pair:
            self.h = L.compile(arg_pair_ir(self.kind, "f32", self.rank_ir, 1))
        else:
            self.h = L.compile(reduce_ir(self.kind, "f32", self.rank_ir, 1, self.arg))
        self.h_local = L.compile(reduce_ir(self.kind, "f32", self.rank_ir, 1, self.arg))
        self.launches_per_step = 2 if (self.collective and not self.fused) else 1

    def bytes_per_step(self):
        return self.N * self.N * 4

    def has_collective(self):
        return self.collective

    def launch_kernel(self, h, outs, scalars, x, stream):
        N, L = self.N, self.lib
        if self.axis == "all":
            L.launch(h, (N * N,), outs + [x], scalars=scalars, device=self.device, stream=stream)
        elif self.axis == "0":
            # the reduced axis comes last in the program's space: the matrix is handed over with its strides swapped
            L.launch(h, (N, N), outs + [x], strides=[None] * len(outs) + [[1, N]], scalars=scalars, device=self.device, stream=stream)
        else:
            L.launch(h, (N, N), outs + [x], scalars=scalars, device=self.device, stream=stream)

    def launch_step(self, i, stream):
        self.launch_kernel(self.h, [self.vals, self.out] if self.pair else [self.out], self.scalars, self.x[i % 2], stream)
        if self.collective and not self.fused:
            n = self.out.numel()
            if self.pair:
                self.lib.arg_allreduce(self.vals, self.out, n, F32, self.kind, device=self.device, stream=stream)
            else:
                self.lib.allreduce(self.out, n, F32, self.kind, device=self.device, stream=stream)

    def e2e_setup(self):
        t = self.torch
        self.hx = t.empty(self.N, self.N, pin_memory=True); self.hx.copy_(self.x[0])
        self.hout = t.zeros(self.out.numel(), dtype=self.out.dtype, pin_memory=True)
        self.h2d, self.d2h = self.N * self.N * 4, self.out.numel() * 4

    def e2e_step(self, i):
        # page-locked host matrix in, host result out: H2D + kernel (+ the ranks' exchange) + D2H + sync
        self.x[0].copy_(self.hx, non_blocking=True)
        self.launch_step(0, self.stream)
        self.hout.copy_(self.out, non_blocking=True)
        self.torch.cuda.synchronize()

    def verify(self):
        """The rank's own result of the op that is timed (before any exchange) against torch on the device as a checker:
        sums within 1e-5 * sum|x| of the fp64 sum, max and argmax (first occurrence) exactly."""
        t, N = self.torch, self.N
        x = self.x[0]
        self.launch_kernel(self.h_local, [self.out], None, x, self.stream)
        t.cuda.synchronize()
        dim = {"-1": 1, "0": 0}.get(self.axis)
        if self.op == "sum":
            want = x.sum(dtype=t.float64) if dim is None else x.sum(dim, dtype=t.float64)
            bound = 1e-5 * (x.abs().sum(dtype=t.float64) if dim is None else x.abs().sum(dim, dtype=t.float64))
            assert bool(((self.out.double() - want).abs() <= bound).all())
        else:
            m = x.max() if dim is None else x.max(dim).values
            if self.op == "max":
                assert bool((self.out == m).all())
            else:
                big = t.iinfo(t.int64).max
                if dim is None:
                    first = t.where(x.reshape(-1) == m, t.arange(N * N, device="cuda"), big).min()
                else:
                    pos = t.arange(N, device="cuda").reshape((N, 1) if dim == 0 else (1, N))
                    first = t.where(x == m.unsqueeze(dim), pos, big).min(dim).values
                assert bool((self.out.long() == first).all())
        if self.collective:
            self.step(0)
            t.cuda.synchronize()
            assert self.lib.comm_error_flag() == 0, "a rank did not arrive at the exchange in time"


class Cumsum(Workload):
    """Running sum along the rows of fp32 [8192,8192] (op::cumsum; not one of the five benchmark configurations: the first of
    the operators either side of the path, measured to the same bar)."""
    name = "scan"
    N = 8192
    kernel_name = "scan_rows_kernel<float, sum, 256 threads per row, 128-bit> (dalib200_scan)"
    e2e_api = "C ABI with caller-managed copies (page-locked host -> device, dalib200_scan, device -> page-locked host, sync)"

    @staticmethod
    def config(world, shape=None, **kw):
        R, C = shape or (Cumsum.N, Cumsum.N)
        return {"workload": "op::cumsum over the last axis of fp32 [%d,%d] ~ U(-1,1) per GPU (inclusive)" % (R, C),
                "l2": "two 256 MiB inputs alternate, 256 MiB output (768 MiB > L2)",
                "parallelism": "rows sharded: each of %d GPU(s) scans its own rows, no collective" % world}

    @staticmethod
    def reference_case(np, tmp, **kw):
        m = 4
        np.save(os.path.join(tmp, "x.npy"), (np.random.default_rng(1240).random((m, 8192)) * 2 - 1).astype(np.float32))
        return {"case": "scan", "args": ["sum", "1", "x.npy", "out.npy"], "bytes": 2 * m * 8192 * 4, "cores": 1, "max_reps": 3,
                "sample": "4 of the 8192 rows per step (the reference's CPU scan is quadratic in the row length)"}

    def __init__(self, *a, shape=None):
        super().__init__(*a)
        import numpy as np
        self.np = np
        t = self.torch
        t.manual_seed(1234 + 6 + self.rank)
        self.R, self.C = shape or (self.N, self.N)      # --scan-shape R,C: other shapes of the same 256 MiB (profiling)
        self.x = [t.rand(self.R, self.C, device="cuda") * 2 - 1 for _ in range(2)]    # 2 x 256 MiB > L2
        self.out = t.empty(self.R, self.C, device="cuda")

    def bytes_per_step(self):
        return 2 * self.R * self.C * 4

    def launch_step(self, i, stream):
        self.lib.scan(0, 0, 1, self.R, self.C, self.x[i % 2], self.out, device=self.device, stream=stream)

    def e2e_setup(self):
        t = self.torch
        self.hx = t.empty(self.R, self.C, pin_memory=True); self.hx.copy_(self.x[0])
        self.hout = t.empty(self.R, self.C, pin_memory=True)
        self.h2d = self.d2h = self.R * self.C * 4

    def e2e_step(self, i):
        self.x[0].copy_(self.hx, non_blocking=True)
        self.launch_step(0, self.stream)
        self.hout.copy_(self.out, non_blocking=True)
        self.torch.cuda.synchronize()

    def verify(self):
        sys.path.insert(0, os.path.join(ROOT, "oracle"))
        import dali_oracle as oracle
        self.launch_step(0, self.stream)
        self.torch.cuda.synchronize()
        rows = sorted({0, self.R // 2, self.R - 1})
        x = self.x[0][rows].cpu().numpy()
        want = self.np.cumsum(x.astype(self.np.float64), axis=1)
        bound = 1e-5 * self.np.cumsum(self.np.abs(x).astype(self.np.float64), axis=1)
        got = self.out[rows].cpu().numpy()
        assert self.np.all(self.np.abs(got - want) <= bound)
        assert self.np.all(self.np.abs(oracle.scan("sum", x, True) - want) <= bound)


class TransposedMap(Workload):
    """y = tanh(x)^T for fp32 [8192,8192]: an elementwise tree under a transposing view (not one of the five benchmark
    configurations: the strided-view side of every fused kernel, measured to the same bar)."""
    name = "transpose"
    N = 8192
    kernel_name = "map skeleton, 4 x 4 register blocks: 128-bit loads along the operand's rows, 128-bit stores along the destination's"
    e2e_api = "C ABI with caller-managed copies (page-locked host -> device, dalib200_launch, device -> page-locked host, sync)"

    @staticmethod
    def config(world, **kw):
        return {"workload": "y = tanh(x).transpose(), fp32 [8192,8192] ~ N(0,1) per GPU",
                "l2": "two 256 MiB inputs alternate, 256 MiB output (768 MiB > L2)",
                "parallelism": "independent matrices: each of %d GPU(s) transposes its own, no collective" % world}

    @staticmethod
    def reference_case(np, tmp, **kw):
        m = 2048
        np.save(os.path.join(tmp, "x.npy"), np.random.default_rng(1241).standard_normal((m, m)).astype(np.float32))
        return {"case": "unary_t", "args": ["tanh", "x.npy", "out.npy"], "bytes": 2 * m * m * 4, "cores": 1, "max_reps": 5,
                "sample": "a [2048,2048] array per step (1/16 of the bytes)"}

    def __init__(self, *a):
        super().__init__(*a)
        import numpy as np
        from dali_b200.ir import IRBuilder
        self.np = np
        t = self.torch
        t.manual_seed(1234 + 7 + self.rank)
        self.x = [t.randn(self.N, self.N, device="cuda") for _ in range(2)]    # 2 x 256 MiB > L2
        self.out = t.empty(self.N, self.N, device="cuda")
        e = IRBuilder(2, 0)
        O, A = e.arg("f32"), e.arg("f32")
        e.st(O, e.op("tanh", e.ld(A)))
        self.h = self.lib.compile(e.text())

    def bytes_per_step(self):
        return 2 * self.N * self.N * 4

    def launch_step(self, i, stream):
        # out[r, c] = tanh(x[c, r]): the operand is handed over with its strides swapped
        self.lib.launch(self.h, (self.N, self.N), [self.out, self.x[i % 2]], strides=[None, [1, self.N]], device=self.device, stream=stream)

    def e2e_setup(self):
        t = self.torch
        self.hx = t.empty(self.N, self.N, pin_memory=True); self.hx.copy_(self.x[0])
        self.hout = t.empty(self.N, self.N, pin_memory=True)
        self.h2d = self.d2h = self.N * self.N * 4

    def e2e_step(self, i):
        self.x[0].copy_(self.hx, non_blocking=True)
        self.launch_step(0, self.stream)
        self.hout.copy_(self.out, non_blocking=True)
        self.torch.cuda.synchronize()

    def verify(self):
        self.launch_step(0, self.stream)
        self.torch.cuda.synchronize()
        assert ".tile4" in self.lib.last_variant()
        rows = [0, 4097, self.N - 1]
        want = self.np.tanh(self.x[0][:, rows].cpu().numpy().astype(self.np.float64)).T
        self.np.testing.assert_allclose(self.out[rows].cpu().numpy(), want, rtol=1e-5, atol=1e-6)


class GatherRows(Workload):
    """op::gather: 2^20 int32 indices pick rows of a [65536,256] fp32 table (an embedding lookup; the index side of the
    path, measured to the same bar).  Algorithmic bytes: every picked row read once and written once, plus the indices."""
    name = "gather"
    V, D, M = 65536, 256, 1 << 20
    e2e_api = "C ABI with caller-managed copies (page-locked indices -> device, dalib200_launch, gathered rows -> page-locked host, sync)"

    @staticmethod
    def config(world, **kw):
        return {"workload": "op::gather(table, indices): fp32 table [65536,256] ~ N(0,1), 2^20 int32 indices ~ U[0,65536) per GPU",
                "l2": "the 64 MiB table fits L2; the 1 GiB of gathered rows written per step does not",
                "parallelism": "indices sharded: each of %d GPU(s) gathers its own batch from a replicated table, no collective" % world}

    @staticmethod
    def reference_case(np, tmp, **kw):
        rng = np.random.default_rng(1242)
        np.save(os.path.join(tmp, "table.npy"), rng.standard_normal((GatherRows.V, GatherRows.D)).astype(np.float32))
        np.save(os.path.join(tmp, "idx.npy"), rng.integers(0, GatherRows.V, 1 << 16).astype(np.int32))
        return {"case": "gather", "args": ["table.npy", "idx.npy", "out.npy"], "bytes": (1 << 16) * (2 * GatherRows.D * 4 + 4), "cores": 1,
                "timed_by_wall_clock": True,
                "sample": "2^16 of the 2^20 indices per step (the reference's generated loop is single-threaded; wall clock of the whole driver process: loading the 64 MiB table and saving the result included)"}

    def __init__(self, *a):
        super().__init__(*a)
        import numpy as np
        from dali_b200.ir import IRBuilder
        self.np = np
        t = self.torch
        t.manual_seed(1234 + 8 + self.rank)
        self.table = t.randn(self.V, self.D, device="cuda")
        self.idx = [t.randint(0, self.V, (self.M,), device="cuda", dtype=t.int32) for _ in range(2)]
        self.out = t.empty(self.M, self.D, device="cuda")
        e = IRBuilder(2, 0)
        O, S, I = e.arg("f32"), e.arg("f32"), e.arg("i32")
        e.st(O, e.ldx(S, e.ld(I)))
        self.h = self.lib.compile(e.text())

    def bytes_per_step(self):
        return self.M * (2 * self.D * 4 + 4)

    def launch_step(self, i, stream):
        # out[i, j] = table[idx[i], j]: the table is addressed through the index (lead stride D), unit stride along j
        self.lib.launch(self.h, (self.M, self.D), [self.out, self.table, self.idx[i % 2]],
                        strides=[None, [0, 1, self.D], [1, 0]], device=self.device, stream=stream)

    def e2e_setup(self):
        t = self.torch
        self.hidx = t.empty(self.M, dtype=t.int32, pin_memory=True); self.hidx.copy_(self.idx[0])
        self.hout = t.empty(self.M, self.D, pin_memory=True)
        self.h2d, self.d2h = self.M * 4, self.M * self.D * 4

    def e2e_step(self, i):
        self.idx[0].copy_(self.hidx, non_blocking=True)
        self.launch_step(0, self.stream)
        self.hout.copy_(self.out, non_blocking=True)
        self.torch.cuda.synchronize()

    def verify(self):
        self.launch_step(0, self.stream)
        self.torch.cuda.synchronize()
        assert bool((self.out == self.table[self.idx[0].long()]).all())        # bit-exact


WORKLOADS = {"chain": Chain, "softmax": Softmax, "lstm": Lstm, "reduce": Reduce, "gemm": Gemm, "scan": Cumsum,
             "transpose": TransposedMap, "gather": GatherRows}
REDUCE_SWEEP = [(op, axis) for op in ("sum", "max", "argmax") for axis in ("-1", "0", "all")]


def workload_kwargs(args, name):
    kw = {}
    if name == "chain" and args.elements:
        kw["total"] = args.elements
    if name == "gemm" and args.gemm_n:
        kw["n"] = args.gemm_n
    if name == "scan" and args.scan_shape:
        kw["shape"] = tuple(int(v) for v in args.scan_shape.split(","))
    if name == "softmax" and args.softmax_shape:
        kw["shape"] = tuple(int(v) for v in args.softmax_shape.split(","))
    if name == "reduce":
        kw["op"], kw["axis"] = args.reduce_op, args.axis
    return kw


# ----------------------------------------------------------------------------- main
def time_reference(cls, kw, reps, warmup):
    """Per-repeat milliseconds of the reference's own CPU path on the workload's bounded sample, and the sample's description."""
    import tempfile
    import numpy as np
    with tempfile.TemporaryDirectory() as tmp:
        case = cls.reference_case(np, tmp, **kw)
        reps = min(reps, case.get("max_reps", reps))
        if case.get("timed_by_wall_clock"):
            times = []
            for _ in range(min(reps, 3) + 1):
                t0 = time.perf_counter()
                if run_ref_driver(case["case"], case["args"], 1, tmp) is None and not os.path.exists(ref_driver_paths()[0]):
                    return None, case
                times.append((time.perf_counter() - t0) * 1e3)
            times = times[1:]
        else:
            times = run_ref_driver(case["case"], case["args"], reps + warmup, tmp)
            times = times[warmup:] if times else None
    return times, case


def reference_arm(args):
    """--impl reference: the reference's own CPU implementation (oracle/_ref) on this box's host cores,
    same metric and config, a bounded sample per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    drv, _ = ref_driver_paths()
    if not os.path.exists(drv):
        print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref/ref_driver was not built (no reference checkout at build time)"}))
        return
    cls = WORKLOADS[args.workload]
    kw = workload_kwargs(args, args.workload)
    times, case = time_reference(cls, kw, args.steps, args.warmup)
    ms = sum(times) / len(times)
    gbs = case["bytes"] / (ms * 1e-3) / 1e9
    line = {"metric": "fused_expr_hbm_gbs", "value": gbs, "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": cls.scaling,
            "vs_baseline": None, "dtype": "f32", "data": "synthetic", "impl": "reference",
            "config": cls.config(args.gpus, **kw),
            "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": case["cores"], "kind": "reference", "sample": case["sample"]},
            "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    if case.get("flops"):
        line["gemm_tflops"] = case["flops"] / (ms * 1e-3) / 1e12
    print(json.dumps(line))


def measure(wl, torch, world, steps, warmup, lib, local=0, min_blocks=5, clock_seconds=1.5):
    """Times blocks of exactly `steps` steps (device time, max over ranks): the first block is the reported one, at
    least `min_blocks` are run and their median is reported beside it.  Returns a dict."""
    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    for i in range(warmup):
        wl.step(i)
    barrier()
    wl.block_steps = steps
    fn = wl.graph_fn()
    stepper = GraphStepper(torch, lambda i, st: fn(warmup + i, st), steps, getattr(wl, "lanes", 1)) if fn else None
    # the clock sampler starts here, ahead of the spin-up: spawning it takes milliseconds, in which an idle GPU would drop
    # out of the state the warm-up put it in; the timed block below follows the last untimed replay by one barrier only
    sampler = ClockSampler(local)
    sampler.start()
    if stepper:
        barrier()
        t_spin = time.perf_counter()
        for _ in range(2):
            stepper.replay()
        torch.cuda.synchronize()
        # Untimed spin-up on top of the `warmup` steps, ~150 ms of the same replays and the same number on every rank (a
        # step may hold a collective): a GPU that has just come out of idle needs that long to settle at the clocks it
        # then holds, and a strong-scaled step is 1 / N as long at N GPUs, so a fixed number of warm-up steps would
        # time every N in a different power state.  Not for the tensor-bound GEMM, whose roofline is the burst rate of
        # a kernel timed alone: more untimed work would move it to its sustained clocks before the block is timed.
        est = torch.tensor([(time.perf_counter() - t_spin) / 2], dtype=torch.float64, device="cuda")
        if world > 1:
            torch.distributed.all_reduce(est, op=torch.distributed.ReduceOp.MAX)
        est = max(float(est.item()), 1e-5)
        if wl.name != "gemm":
            for _ in range(min(2000, int(0.15 / est) + 1)):
                stepper.replay()
    barrier()
    block_ms = []

    def one_block():
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if stepper:
            ev0.record(stepper.stream)
            stepper.replay()
            ev1.record(stepper.stream)
        else:
            ev0.record()
            for i in range(steps):
                wl.step(warmup + i)
            ev1.record()
        barrier()
        block_ms.append(ev0.elapsed_time(ev1))

    if stepper:
        # the last of the warm-up is one block issued exactly like the timed ones (events, one replay, a barrier): the
        # first block after the long back-to-back spin-up measured a fixed 15-40 us longer than every later one
        one_block()
        block_ms.clear()
    one_block()        # the reported block: exactly `steps` steps
    # more blocks: the median beside the reported figure, and a GPU kept busy while nvidia-smi samples the clocks;
    # every rank must run the same number of them (each ends in a barrier), so the count is agreed on, not timed per rank
    extra = int(min(200, max(min_blocks - 1, clock_seconds * 1e3 / max(block_ms[0], 1e-3))))
    if world > 1:
        cnt = torch.tensor([extra], dtype=torch.int64, device="cuda")
        torch.distributed.all_reduce(cnt, op=torch.distributed.ReduceOp.MAX)
        extra = int(cnt.item())
    for _ in range(extra):
        one_block()
    clocks = sampler.stop()
    if os.environ.get("DALI_BENCH_BLOCKS"):
        sys.stderr.write("blocks(ms/step) %s: %s\n" % (wl.name, " ".join("%.5f" % (b / steps) for b in block_ms[:40])))
    t = torch.tensor([block_ms[0], sorted(block_ms)[len(block_ms) // 2]], dtype=torch.float64, device="cuda")
    if world > 1:
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    res = {"ms_per_step": float(t[0].item()) / steps, "clocks": clocks, "graph": bool(stepper),
           "gpu_launches": steps * wl.launches_per_step,
           "median_block_ms_per_step": float(t[1].item()) / steps, "blocks": len(block_ms)}
    # dominant kernel alone, replayed back to back
    dom = wl.dominant()
    if dom:
        name, bound, work, launch = dom
        reps = 20
        ds = GraphStepper(torch, launch, reps)
        ds.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(ds.stream)
        ds.replay()
        e1.record(ds.stream)
        torch.cuda.synchronize()
        res["dominant"] = {"kernel": name, "bound": bound, "work": work, "ms": e0.elapsed_time(e1) / reps}
    return res


def roofline_of(wl, m, lib):
    peak_hbm, kind = measured_peak()
    dom = m.get("dominant")
    if dom and dom["bound"] == "tensor":
        path = os.path.join(ROOT, "MEASURED_PEAKS.json")
        peak = 1590.0
        sustained = None
        src = "fallback 1.59 PFLOP/s"
        if os.path.exists(path):
            with open(path) as f:
                peaks = json.load(f)
            peak = float(peaks["bf16_tflops"])
            sustained = peaks.get("bf16_tflops_sustained")
            src = "measured (MEASURED_PEAKS.json bf16_tflops, burst: kernel timed alone)"
        achieved = dom["work"] / (dom["ms"] * 1e-3) / 1e12
        out = {}
        if os.path.exists(path) and sustained:
            # the same kernel after seconds of load runs at the power cap's clocks: the fraction of that figure too
            out["frac_of_sustained_peak"] = achieved / float(sustained)
        if "TF32" in dom["kernel"]:
            # three TF32 products per fp32 product, and the dense TF32 rate is half the bf16 rate the peak is measured in
            out["tensor_pipe_equivalent_frac"] = 6.0 * achieved / peak
        return {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                "traffic": getattr(wl, "dominant_traffic_bytes", None), "traffic_note": getattr(wl, "dominant_traffic_note", None),
                **out, "peak_source": src, "kernel": dom["kernel"] + " [" + lib.last_gemm_kernel() + "]",
                "kernel_ms": dom["ms"],
                "note": "algorithmic flops 2*M*N*K per launch; an fp32 product issues three TF32 passes, whose dense rate is half the bf16 rate"
                        if "TF32" in dom["kernel"] else "algorithmic flops 2*M*N*K per launch"}
    ms = dom["ms"] if dom else m["ms_per_step"]
    work = dom["work"] if dom else wl.bytes_per_step()
    achieved = work / (ms * 1e-3) / 1e9
    ratio = DRAM_TRAFFIC_PER_ALGO_BYTE.get(wl.name)
    return {"bound": "hbm", "achieved": achieved, "peak": peak_hbm, "unit": "GB/s", "frac": achieved / peak_hbm,
            "traffic": ratio * work if ratio else None,
            "peak_source": (kind + " (MEASURED_PEAKS.json hbm_gbs)") if kind == "measured" else "fallback 6.65 TB/s",
            "kernel": getattr(wl, "kernel_name", None) or lib.last_variant(), "kernel_ms": ms,
            "note": "per rank: the step's kernel(s), the exchange between the ranks included" if wl.has_collective() else None}


def end_to_end(wl, torch, world, steps):
    """The same metric through the public call with page-locked HOST buffers, copies inside the timed region."""
    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    job_bytes = wl.bytes_per_step() * world
    external = getattr(wl, "e2e_external", None)
    if external:
        # the workload's end-to-end loop is a C++ program written against the front end's own headers
        n_e2e = max(steps, 200)
        barrier()
        dt = external(5, n_e2e) * 1e-3
        barrier()
    else:
        n_e2e = max(1, min(steps, 5))
        wl.e2e_setup()
        for i in range(2):
            wl.e2e_step(i)
        barrier()
        t0 = time.perf_counter()
        for i in range(n_e2e):
            wl.e2e_step(i)      # synchronous: returns after the result is back in host memory
        barrier()
        dt = (time.perf_counter() - t0) / n_e2e
    te = torch.tensor([dt], dtype=torch.float64, device="cuda")
    if world > 1:
        torch.distributed.all_reduce(te, op=torch.distributed.ReduceOp.MAX)
    return {"value": job_bytes / float(te.item()) / 1e9, "unit": "GB/s", "h2d_bytes_per_step": wl.h2d,
            "d2h_bytes_per_step": wl.d2h, "steps": n_e2e, "ms_per_step": float(te.item()) * 1e3,
            "api": getattr(wl, "e2e_api", "dalib200_launch_host / C ABI with pinned host buffers (alloc from pool + H2D + "
                                           "kernel + D2H + sync per step)")}


def cpu_baseline_of(cls, kw):
    times, case = time_reference(cls, kw, 8, 1)
    if not times:
        return None
    best = sorted(times)[len(times) // 2]
    cpu = {"value": case["bytes"] / (best * 1e-3) / 1e9, "unit": "GB/s", "cores": case["cores"], "kind": "reference",
           "sample": case["sample"], "ms": best}
    if case.get("flops"):
        cpu["tflops"] = case["flops"] / (best * 1e-3) / 1e12
    return cpu


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="chain", choices=sorted(WORKLOADS))
    ap.add_argument("--elements", type=int, default=0, help="chain: total elements (profiling on a small case)")
    ap.add_argument("--gemm-n", type=int, default=0, help="gemm: matrix size (profiling on a small case)")
    ap.add_argument("--scan-shape", default="", help="scan: R,C instead of 8192,8192 (the variants for short and for few, very long rows)")
    ap.add_argument("--softmax-shape", default="", help="softmax: R,C instead of 4096,1024 (few long rows: the cluster variant)")
    ap.add_argument("--reduce-op", default="sum", choices=["sum", "max", "argmax"], help="reduce: the reducer")
    ap.add_argument("--axis", default="0", choices=["-1", "0", "all"], help="reduce: the reduced axis")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-others", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    args.warmup = max(args.warmup, 3)

    import torch
    import dali_b200
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback")
    torch.cuda.set_device(local)
    lib = dali_b200.load_library()
    lib.init(0)
    transport = "none"
    if world > 1:
        import datetime
        from dali_b200 import comm
        # a rank that falls out of step ends the run in two minutes, not ten
        torch.distributed.init_process_group("nccl", device_id=torch.device("cuda", local),
                                             timeout=datetime.timedelta(seconds=120))
        comm.init_from_torch(lib, local)       # the library's own communicator: NCCL + the ranks' peer-memory mapping
        transport = lib.comm_transport()
    dev_index = local      # the library indexes the devices it bound; one process per GPU uses its own

    def run(name, kw, steps, warmup, cpu_wanted, e2e_wanted, clock_seconds):
        wl = WORKLOADS[name](lib, torch, rank, world, dev_index, **kw)
        wl.verify()
        m = measure(wl, torch, world, steps, warmup, lib, local, clock_seconds=clock_seconds)
        roofline = roofline_of(wl, m, lib)
        if hasattr(wl, "extra"):
            roofline.update(wl.extra(torch))
        e2e = end_to_end(wl, torch, world, steps) if e2e_wanted else None
        cpu = cpu_baseline_of(WORKLOADS[name], kw) if (cpu_wanted and rank == 0 and world == 1) else None
        return {"wl": wl, "m": m, "roofline": roofline, "e2e": e2e, "cpu": cpu}

    kw = workload_kwargs(args, args.workload)
    main_res = run(args.workload, kw, args.steps, args.warmup, not args.no_cpu, not args.no_e2e, 1.5)
    wl, m = main_res["wl"], main_res["m"]
    ms_step = m["ms_per_step"]
    value = wl.bytes_per_step() * world / (ms_step * 1e-3) / 1e9
    line = {"metric": "fused_expr_hbm_gbs", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "median_block_ms_per_step": m["median_block_ms_per_step"],
            "timed_blocks": m["blocks"], "higher_is_better": True, "scaling": wl.scaling,
            "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic",
            "config": WORKLOADS[args.workload].config(world, **kw), "clocks": m["clocks"], "roofline": main_res["roofline"],
            "cpu_baseline": main_res["cpu"], "e2e": main_res["e2e"],
            "gpu_launches": int(m["gpu_launches"]), "timed_with": "CUDA graph replay of the step's launches" if m["graph"] else "eager launches",
            "rank_exchange": transport}
    if wl.hbm_metric:
        line["pct_of_nominal_8TBs"] = 100.0 * value / world / 8000.0
    if wl.flops_per_step():
        line["gemm_tflops"] = wl.flops_per_step() * world / (ms_step * 1e-3) / 1e12
    del wl, main_res

    if args.workload == "chain" and not args.no_others and not args.elements:
        others = {}
        todo = [("gemm", {}), ("softmax", {}), ("lstm", {})] + [("reduce", {"op": o, "axis": a}) for o, a in REDUCE_SWEEP] + \
               [("scan", {}), ("transpose", {}), ("gather", {})]       # the power-capped GEMM before the GPU is hot
        for name, okw in todo:
            torch.cuda.empty_cache()
            time.sleep(0.5)      # each workload starts from a rested GPU, as its own `--workload` run would (power cap)
            r = run(name, okw, 24, 3, not args.no_cpu, not args.no_e2e, 1.0)
            w, mo = r["wl"], r["m"]
            entry = {"config": WORKLOADS[name].config(world, **okw), "scaling": w.scaling, "ms_per_step": mo["ms_per_step"],
                     "median_block_ms_per_step": mo["median_block_ms_per_step"],
                     "value": w.bytes_per_step() * world / (mo["ms_per_step"] * 1e-3) / 1e9, "unit": "GB/s",
                     "roofline": {k: v for k, v in r["roofline"].items() if v is not None}, "clocks": mo["clocks"],
                     "e2e": r["e2e"], "cpu_baseline": r["cpu"], "gpu_launches": int(mo["gpu_launches"])}
            if w.flops_per_step():
                entry["tflops"] = w.flops_per_step() * world / (mo["ms_per_step"] * 1e-3) / 1e12
            key = name if name != "reduce" else "reduce_%s_axis_%s" % (okw["op"], okw["axis"].replace("-1", "last"))
            others[key] = entry
            del w, r
        line["other_workloads"] = others

    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        lib.comm_destroy()
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
