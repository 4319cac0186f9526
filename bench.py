"""Benchmark of the fused-expression hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

One "step" is one pass of a fused expression over one batch of synthetic
input.  Prints ONE JSON line (rank 0).  Workloads (the benchmark configurations):

  lstm     (default, configuration 2) fused LSTM cell step, fp32 B=256 H=1024:
           gates = dot(x,Wx)+dot(h,Wh)+b on the tensor cores (3xTF32, second GEMM
           with "+ first + b" as epilogue), then the fused sigmoid/tanh gating
  softmax  (config 1) exp(a - max(a,-1)) / sum(...) on fp32 [4096,1024]
  reduce   (config 3) sum over axis 0 of fp32 [8192,8192] (the strided case)
  gemm     (config 4) tanh(dot(A,B)+bias), bf16 8192^3, fp32 accumulate
  chain    (config 5) sum(sigmoid(x*w+b) * exp(-x*x)) over 2^31 fp32 elements,
           sharded over the GPUs with an all-reduce of the partial sums
The default run also measures the other four briefly and reports them under
"other_workloads".

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
DRAM_TRAFFIC_PER_ALGO_BYTE = {
    "chain": 1.0004,     # profiles/chain_sum_all_kernel.md
    "softmax": 0.50,     # profiles/softmax_row_kernel.md: the 16 MiB output is still in L2 when the kernel ends
    "reduce": 1.0002,    # profiles/reduce_8192_row_col_all_kernels.md
    "scan": 0.905,       # profiles/scan_rows_kernel.md: the tail of the output is written back after the kernel ends
    "transpose": 0.919,  # profiles/map_transposing_kernel.md: likewise
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

    def graph_fn(self):
        """launch(i, stream) of one step's kernels when the step has no host-side part, else None."""
        return None

    def dominant(self):
        """(kernel name, bound, algorithmic work per launch, launch(i, stream)) or None = the step itself."""
        return None

    def flops_per_step(self):
        return 0


class Chain(Workload):
    """Benchmark configuration 5: long elementwise chain + all-axis sum, strong-scaled over the ranks."""
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

    launches_per_step = 1

    def launch_step(self, i, stream):
        self.lib.launch(self.h, (self.n,), [self.out, self.x], scalars=[self.w, self.b], device=self.device, stream=stream)

    def step(self, i):
        self.launch_step(i, self.stream)
        if self.world > 1:
            from dali_b200.sharding import combine_partials
            combine_partials(self.out, "sum")           # NCCL all-reduce of one fp32 per rank

    def graph_fn(self):
        return self.launch_step if self.world == 1 else None

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
        self.lib.launch(self.h, (m,), [o, xs], scalars=[self.w, self.b], device=self.device, stream=self.stream)
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
    """Benchmark configuration 1: naive fused softmax on fp32 [4096,1024]."""
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
        self.lanes = int(os.environ.get("DALI_BENCH_SOFTMAX_LANES", "3"))   # independent batches on three streams

    def describe(self):
        return {"workload": "C1 exp(a-max(a,{-1},true))/sum(exped,{-1},true), fp32 [4096,1024] ~ N(0,1) per GPU",
                "l2": "rotating over %d input/output buffer pairs (%d MiB) so every launch misses L2" %
                      (self.nbuf, self.nbuf * 32),
                "concurrency": "%d streams: consecutive batches are independent and may overlap" % self.lanes,
                "parallelism": "rows sharded: each of %d GPU(s) runs its own [4096,1024] batch, no collective" % self.world}

    def bytes_per_step(self):
        return self.ROWS * self.COLS * 8

    launches_per_step = 1

    def launch_step(self, i, stream):
        k = i % self.nbuf
        self.lib.launch(self.h, (self.ROWS, self.COLS), [self.o[k], self.a[k]], device=self.device, stream=stream)

    def step(self, i):
        self.launch_step(i, self.stream)

    def graph_fn(self):
        return self.launch_step

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
    dominant_traffic_bytes = 75.8e6      # profiles/gemm_tcgen05_kernels.md: 72.4 MB read + 3.4 MB written per launch
    dominant_traffic_note = "ncu capture with a cold L2 (64 MB of split weights read from DRAM); in the timed loop the weights stay in L2"
    e2e_api = ("page-locked host arrays -> lazy Array / op:: expression -> Array::eval_together -> host arrays, in C++ against "
               "the front end's headers (dali_b200/host/programs/lstm_cell_e2e.cpp)")

    def __init__(self, *a):
        super().__init__(*a)
        import numpy as np
        from dali_b200.ir import IRBuilder
        self.np = np
        t, B, H = self.torch, self.B, self.H
        t.manual_seed(1234 + 1 + self.rank)
        self.nset = 6       # rotating activation sets; weights (2 x 16 MiB, split: 64 MiB) stay hot like in a real RNN
        self.x = [t.randn(B, H, device="cuda") for _ in range(self.nset)]
        self.h = [t.randn(B, H, device="cuda") for _ in range(self.nset)]
        self.c = [t.randn(B, H, device="cuda") for _ in range(self.nset)]
        self.Wx = t.randn(H, 4 * H, device="cuda") * 0.02
        self.Wh = t.randn(H, 4 * H, device="cuda") * 0.02
        self.b = t.zeros(4 * H, device="cuda")
        self.gates = t.empty(B, 4 * H, device="cuda")
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
        e = IRBuilder(2, 0)
        o, bias = e.arg("f32"), e.arg("f32")
        e.st(o, e.op("add", e.acc(), e.ld(bias)))      # acc = x.Wx + h.Wh (one accumulator), + b
        self.h_epi = L.compile(e.text())
        # what the front end emits for eval_together(c', h'): the gating is the epilogue of the gate products
        from dali_b200.ir import lstm_cell_epilogue_ir
        self.h_cell = L.compile(lstm_cell_epilogue_ir())
        self.scaling = "weak"
        self.launches_per_step = 2

    def describe(self):
        return {"workload": "C2 LSTM cell step: gates = dot(x,Wx)+dot(h,Wh)+b, c' = sig(f)*c + sig(i)*tanh(g), "
                            "h' = sig(o)*tanh(c'); fp32, B=256 H=1024 per GPU, x,h,c ~ N(0,1), W ~ N(0,0.02), b = 0",
                "l2": "activations rotate over %d sets; the two weight matrices are reused every step (as in an RNN) "
                      "and stay in L2" % self.nset,
                "kernels_per_step": "1 TF32 split of x and h, 1 tcgen05 3xTF32 GEMM accumulating x.Wx + h.Wh whose epilogue is the whole gating (+ b, sigmoid / tanh, c', h'): the [B,4H] gates are never written",
                "parallelism": "batch sharded: each of %d GPU(s) runs its own B=256 shard, weights replicated, no collective" % self.world}

    def bytes_per_step(self):
        B, H = self.B, self.H
        return 4 * (3 * B * H + 2 * H * 4 * H + 4 * H + 2 * B * H)

    def flops_per_step(self):
        return 2 * 2 * self.B * self.H * 4 * self.H

    def launch_step(self, i, stream):
        L, B, H, k = self.lib, self.B, self.H, i % self.nset
        d = self.device
        L.gemm_split_tf32_pair(self.x[k], self.h[k], B, H, H, H, *self.parts, device=d, stream=stream)
        self.launch_gemm(stream, k)

    def launch_gemm(self, stream, k=0):
        B, H, P, W = self.B, self.H, self.parts, self.W
        row = [0, 1]
        self.lib.gemm_fused_sum(0, B, H, [(H, P[0], H, W["Wx"][0], H, P[1], W["Wx"][1]),
                                          (H, P[2], H, W["Wh"][0], H, P[3], W["Wh"][1])],
                                self.h_cell, [self.c_new[k], self.h_new[k], self.b, self.b, self.b, self.b, self.c[k]],
                                strides=[None, None, row, row, row, row, None], offsets=[0, 0, 0, H, 2 * H, 3 * H, 0],
                                device=self.device, stream=stream)

    def step(self, i):
        self.launch_step(i, self.stream)

    def graph_fn(self):
        return self.launch_step

    def dominant(self):
        """(name, bound, algorithmic work per launch, launcher) of the dominant kernel."""
        B, H = self.B, self.H
        return ("tcgen05 3xTF32 GEMM [256,1024]x[1024,4096] + [256,1024]x[1024,4096], one accumulator, LSTM gating as epilogue", "tensor",
                2.0 * 2 * B * H * 4 * H, lambda i, stream: self.launch_gemm(stream))

    def e2e_external(self, warmup, steps):
        """ms per step of dali_b200/host/programs/lstm_cell_e2e.cpp: the cell through the C++ Array / op:: API with
        page-locked host arrays in and out every step (the Python face of the same API, e2e_step below, adds
        ~0.1 ms of ctypes calls per step)."""
        from dali_b200 import build as _build
        exe = os.path.join(ROOT, "dali_b200", "lib", "lstm_cell_e2e")
        if not os.path.exists(exe):
            _build.build_programs()
        out = subprocess.run([exe, str(self.device), str(self.B), str(self.H), str(warmup), str(steps)], capture_output=True,
                             text=True, timeout=600)
        if out.returncode != 0:
            raise RuntimeError("lstm_cell_e2e failed: " + out.stderr[-2000:])
        r = json.loads(out.stdout.strip().splitlines()[-1])
        self.h2d, self.d2h = r["h2d_bytes_per_step"], r["d2h_bytes_per_step"]
        return r["ms_per_step"]

    def e2e_setup(self):
        np = self.np
        t = self.torch
        self.pinned = {}
        for k in ("x", "h", "c"):
            self.pinned[k] = t.empty(self.B, self.H, pin_memory=True)
            self.pinned[k].copy_(getattr(self, k)[0])
        for k in ("h_out", "c_out"):
            self.pinned[k] = t.empty(self.B, self.H, pin_memory=True)
        self.host = {k: v.numpy() for k, v in self.pinned.items()}       # numpy views of the page-locked buffers
        from dali_b200.array import Array, set_default_device
        set_default_device(self.device)
        self.fe = {"Wx": Array(self.Wx.cpu().numpy()), "Wh": Array(self.Wh.cpu().numpy()), "b": Array(self.b.cpu().numpy())}
        self.h2d, self.d2h = 3 * self.B * self.H * 4, 2 * self.B * self.H * 4

    def e2e_step(self, i):
        # the call a user makes: (page-locked) host arrays in, lazy expression, eval, results back on the host
        from dali_b200.array import Array, eval_together, op
        H = self.H
        x, h, c = (Array.borrow(self.host[k]) for k in ("x", "h", "c"))
        gates = op.dot(x, self.fe["Wx"]) + op.dot(h, self.fe["Wh"]) + self.fe["b"][None, :]
        i_, f, o = (op.sigmoid(gates[:, k * H:(k + 1) * H]) for k in range(3))
        g = op.tanh(gates[:, 3 * H:4 * H])
        c_new = f * c + i_ * g
        h_new = o * op.tanh(c_new)
        eval_together(c_new, h_new, wait=False)              # one GEMM launch + one gating kernel for both outputs
        self.last = (h_new.numpy(out=self.host["h_out"]), c_new.numpy(out=self.host["c_out"]))

    def verify(self):
        sys.path.insert(0, os.path.join(ROOT, "oracle"))
        import dali_oracle as oracle
        np = self.np
        self.step(0)
        self.torch.cuda.synchronize()
        assert self.lib.gemm_error_flag(self.device) == 0
        x, h, c, Wx, Wh = (v.cpu().numpy().astype(np.float64) for v in (self.x[0], self.h[0], self.c[0], self.Wx, self.Wh))
        gates = (x @ Wx + h @ Wh).astype(np.float32)
        want_c, want_h = oracle.lstm_gating(gates, self.c[0].cpu().numpy())
        assert np.allclose(self.c_new[0].cpu().numpy(), want_c, rtol=1e-5, atol=1e-5)
        assert np.allclose(self.h_new[0].cpu().numpy(), want_h, rtol=1e-5, atol=1e-5)

    def cpu_baseline(self, tmpdir, reps):
        np = self.np
        for k in ("x", "h", "c"):
            np.save(os.path.join(tmpdir, k + ".npy"), getattr(self, k)[0].cpu().numpy())
        np.save(os.path.join(tmpdir, "Wx.npy"), self.Wx.cpu().numpy())
        np.save(os.path.join(tmpdir, "Wh.npy"), self.Wh.cpu().numpy())
        np.save(os.path.join(tmpdir, "b.npy"), self.b.cpu().numpy().reshape(1, -1))
        times = run_ref_driver("lstm", ["x.npy", "h.npy", "c.npy", "Wx.npy", "Wh.npy", "b.npy", "c_out.npy", "h_out.npy"], reps, tmpdir)
        if not times:
            return None
        return {"ms": times, "bytes": self.bytes_per_step(), "cores": os.cpu_count() or 1, "kind": "reference",
                "sample": "the full B=256 H=1024 cell step (reference: 8 OpenBLAS sgemm on all host cores + 5 single-threaded JIT kernels)"}


class Gemm(Workload):
    """Benchmark configuration 4: tanh(dot(A,B)+bias), bf16 8192^3, fp32 accumulate, bf16 out."""
    name = "gemm"
    e2e_api = "C ABI with caller-managed copies (page-locked host -> device, dalib200_gemm_fused, device -> page-locked host, sync)"
    N = 8192

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
        self.scaling = "weak"
        self.launches_per_step = 1

    def describe(self):
        return {"workload": "C4 tanh(dot(A,B)+bias), bf16 A,B [%d,%d] ~ N(0,0.02), bias ~ N(0,0.1), fp32 accumulate, bf16 out" % (self.n, self.n),
                "l2": "operands + output = %d MiB per launch, larger than L2" % (3 * self.n * self.n * 2 >> 20),
                "parallelism": "rows of A sharded: each of %d GPU(s) runs its own [%d,%d] block, B and bias replicated, no collective" % (self.world, self.n, self.n)}

    def bytes_per_step(self):
        return 3 * self.n * self.n * 2

    def flops_per_step(self):
        return 2 * self.n ** 3

    def launch_step(self, i, stream):
        n = self.n
        self.lib.gemm_fused(3, n, n, n, self.A, n, self.Bm, n, self.h, [self.out, self.bias], strides=[None, [0, 1]],
                            device=self.device, stream=stream)

    def step(self, i):
        self.launch_step(i, self.stream)

    def graph_fn(self):
        return self.launch_step

    def dominant(self):
        return ("tcgen05 bf16 GEMM + bias/tanh epilogue", "tensor", float(self.flops_per_step()), self.launch_step)

    def e2e_setup(self):
        t = self.torch
        n = self.n
        self.hA = t.empty(n, n, dtype=t.bfloat16, pin_memory=True); self.hA.copy_(self.A)
        self.hB = t.empty(n, n, dtype=t.bfloat16, pin_memory=True); self.hB.copy_(self.Bm)
        self.hbias = t.empty(n, pin_memory=True); self.hbias.copy_(self.bias)
        self.hout = t.empty(n, n, dtype=t.bfloat16, pin_memory=True)
        self.h2d, self.d2h = 2 * n * n * 2 + n * 4, n * n * 2

    def e2e_step(self, i):
        # bf16 is not a dtype of the reference's Array: the user-facing call for it is the C ABI with
        # caller-managed copies (pinned host -> device, fused GEMM, device -> pinned host)
        t = self.torch
        self.A.copy_(self.hA, non_blocking=True)
        self.Bm.copy_(self.hB, non_blocking=True)
        self.bias.copy_(self.hbias, non_blocking=True)
        self.launch_step(i, self.stream)
        self.hout.copy_(self.out, non_blocking=True)
        t.cuda.synchronize()

    def verify(self):
        np, n = self.np, self.n
        self.step(0)
        self.torch.cuda.synchronize()
        assert self.lib.gemm_error_flag(self.device) == 0
        rows = [0, 129, n - 1]
        a = self.A[rows].float().cpu().numpy().astype(np.float64)
        want = np.tanh(a @ self.Bm.float().cpu().numpy().astype(np.float64) + self.bias.cpu().numpy())
        assert np.allclose(self.out[rows].float().cpu().numpy(), want, rtol=1e-2, atol=4e-3)

    def cpu_baseline(self, tmpdir, reps):
        np = self.np
        m = 2048        # the reference has no bf16: fp32 sgemm + its fused add/tanh kernel on bf16-rounded inputs
        np.save(os.path.join(tmpdir, "A.npy"), self.A[:m, :m].float().cpu().numpy())
        np.save(os.path.join(tmpdir, "B.npy"), self.Bm[:m, :m].float().cpu().numpy())
        np.save(os.path.join(tmpdir, "bias.npy"), self.bias[:m].cpu().numpy())
        times = run_ref_driver("gemm_tanh", ["A.npy", "B.npy", "bias.npy", "out.npy"], min(reps, 3), tmpdir)
        if not times:
            return None
        return {"ms": times, "bytes": 3 * m * m * 2, "flops": 2.0 * m ** 3, "cores": os.cpu_count() or 1, "kind": "reference",
                "sample": "2048^3 fp32 (1/64 of the flops): OpenBLAS sgemm on all host cores + the reference's single-threaded tanh kernel"}


class ReduceAxis0(Workload):
    """Benchmark configuration 3 (the strided case): sum over axis 0 of fp32 [8192,8192]."""
    name = "reduce"
    N = 8192

    def __init__(self, *a):
        super().__init__(*a)
        import numpy as np
        from dali_b200.ir import reduce_ir
        self.np = np
        t = self.torch
        t.manual_seed(1234 + 2 + self.rank)
        self.x = [t.rand(self.N, self.N, device="cuda") * 2 - 1 for _ in range(2)]    # 2 x 256 MiB > L2
        self.out = t.empty(self.N, device="cuda")
        self.h = self.lib.compile(reduce_ir("sum", "f32", 2, 1))
        self.scaling = "weak"
        self.launches_per_step = 1

    def describe(self):
        return {"workload": "C3 op::sum over axis 0 of fp32 [8192,8192] ~ U(-1,1) per GPU",
                "l2": "two 256 MiB inputs alternate (512 MiB > L2)",
                "parallelism": "rows sharded over %d GPU(s); the [8192] partial sums meet in an all-reduce" % self.world}

    def bytes_per_step(self):
        return self.N * self.N * 4

    def launch_step(self, i, stream):
        N = self.N
        self.lib.launch(self.h, (N, N), [self.out, self.x[i % 2]], strides=[None, [1, N]], device=self.device, stream=stream)

    def step(self, i):
        self.launch_step(i, self.stream)
        if self.world > 1:
            from dali_b200.sharding import combine_partials
            combine_partials(self.out, "sum")           # NCCL all-reduce of the [8192] partial sums

    def graph_fn(self):
        return self.launch_step if self.world == 1 else None

    def e2e_setup(self):
        t = self.torch
        self.hx = t.empty(self.N, self.N, pin_memory=True); self.hx.copy_(self.x[0])
        self.hout = self.np.zeros(self.N, self.np.float32)
        self.h2d, self.d2h = self.N * self.N * 4, self.N * 4

    def e2e_step(self, i):
        import ctypes
        N = self.N
        ptrs = (ctypes.c_void_p * 2)(self.hout.ctypes.data, self.hx.data_ptr())
        ext = (ctypes.c_int64 * 2)(N, N * N)
        offs = (ctypes.c_int64 * 2)(0, 0)
        space = (ctypes.c_int64 * 2)(N, N)
        st1 = (ctypes.c_int64 * 2)(1, N)
        st = (ctypes.POINTER(ctypes.c_int64) * 2)(None, ctypes.cast(st1, ctypes.POINTER(ctypes.c_int64)))
        self.lib.check(self.lib.c.dalib200_launch_host(ctypes.c_uint64(self.h), self.device, space, 2, ptrs, ext, offs, st, 2, None, 0))

    def verify(self):
        self.launch_step(0, self.stream)
        self.torch.cuda.synchronize()
        want = self.x[0].sum(0, dtype=self.torch.float64)
        bound = 1e-5 * self.x[0].abs().sum(0, dtype=self.torch.float64)
        assert bool(((self.out.double() - want).abs() <= bound).all())

    def cpu_baseline(self, tmpdir, reps):
        m = 2048
        self.np.save(os.path.join(tmpdir, "x.npy"), self.x[0][:m, :m].contiguous().cpu().numpy())
        times = run_ref_driver("reduce", ["sum", "0", "x.npy", "out.npy"], reps, tmpdir)
        if not times:
            return None
        return {"ms": times, "bytes": m * m * 4, "cores": 1, "kind": "reference", "sample": "a [2048,2048] corner (1/16 of the bytes)"}


class Cumsum(Workload):
    """Running sum along the rows of fp32 [8192,8192] (op::cumsum; not one of the five benchmark configurations: the first of
    the operators either side of the path, measured to the same bar)."""
    name = "scan"
    N = 8192
    kernel_name = "scan_rows_kernel<float, sum, 256 threads per row, 128-bit> (dalib200_scan)"
    e2e_api = "C ABI with caller-managed copies (page-locked host -> device, dalib200_scan, device -> page-locked host, sync)"

    def __init__(self, *a, shape=None):
        super().__init__(*a)
        import numpy as np
        self.np = np
        t = self.torch
        t.manual_seed(1234 + 6 + self.rank)
        self.R, self.C = shape or (self.N, self.N)      # --scan-shape R,C: other shapes of the same 256 MiB (profiling)
        self.x = [t.rand(self.R, self.C, device="cuda") * 2 - 1 for _ in range(2)]    # 2 x 256 MiB > L2
        self.out = t.empty(self.R, self.C, device="cuda")
        self.scaling = "weak"
        self.launches_per_step = 1

    def describe(self):
        return {"workload": "op::cumsum over the last axis of fp32 [%d,%d] ~ U(-1,1) per GPU (inclusive)" % (self.R, self.C),
                "l2": "two 256 MiB inputs alternate, 256 MiB output (768 MiB > L2)",
                "parallelism": "rows sharded: each of %d GPU(s) scans its own rows, no collective" % self.world}

    def bytes_per_step(self):
        return 2 * self.R * self.C * 4

    def launch_step(self, i, stream):
        self.lib.scan(0, 0, 1, self.R, self.C, self.x[i % 2], self.out, device=self.device, stream=stream)

    def step(self, i):
        self.launch_step(i, self.stream)

    def graph_fn(self):
        return self.launch_step

    def e2e_setup(self):
        t = self.torch
        self.hx = t.empty(self.R, self.C, pin_memory=True); self.hx.copy_(self.x[0])
        self.hout = t.empty(self.R, self.C, pin_memory=True)
        self.h2d = self.d2h = self.R * self.C * 4

    def e2e_step(self, i):
        # the C ABI with caller-managed copies (page-locked host -> device, scan, device -> page-locked host)
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

    def cpu_baseline(self, tmpdir, reps):
        # the reference's CPU scan takes time quadratic in the row length (18 s for [2048,2048]): a few full-length rows
        m = 4
        self.np.save(os.path.join(tmpdir, "x.npy"), self.x[0][:m, :8192].contiguous().cpu().numpy())
        times = run_ref_driver("scan", ["sum", "1", "x.npy", "out.npy"], min(reps, 3), tmpdir)
        if not times:
            return None
        return {"ms": times, "bytes": 2 * m * 8192 * 4, "cores": 1, "kind": "reference", "sample": "4 rows of 8192 elements"}


class TransposedMap(Workload):
    """y = tanh(x)^T for fp32 [8192,8192]: an elementwise tree under a transposing view (not one of the five benchmark
    configurations: the strided-view side of every fused kernel, measured to the same bar)."""
    name = "transpose"
    N = 8192
    kernel_name = "map skeleton, 4 x 4 register blocks: 128-bit loads along the operand's rows, 128-bit stores along the destination's"
    e2e_api = "C ABI with caller-managed copies (page-locked host -> device, dalib200_launch, device -> page-locked host, sync)"

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
        self.scaling = "weak"
        self.launches_per_step = 1

    def describe(self):
        return {"workload": "y = tanh(x).transpose(), fp32 [8192,8192] ~ N(0,1) per GPU",
                "l2": "two 256 MiB inputs alternate, 256 MiB output (768 MiB > L2)",
                "parallelism": "independent matrices: each of %d GPU(s) transposes its own, no collective" % self.world}

    def bytes_per_step(self):
        return 2 * self.N * self.N * 4

    def launch_step(self, i, stream):
        # out[r, c] = tanh(x[c, r]): the operand is handed over with its strides swapped
        self.lib.launch(self.h, (self.N, self.N), [self.out, self.x[i % 2]], strides=[None, [1, self.N]], stream=stream)

    def step(self, i):
        self.launch_step(i, self.stream)

    def graph_fn(self):
        return self.launch_step

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

    def cpu_baseline(self, tmpdir, reps):
        m = 2048
        self.np.save(os.path.join(tmpdir, "x.npy"), self.x[0][:m, :m].contiguous().cpu().numpy())
        times = run_ref_driver("unary_t", ["tanh", "x.npy", "out.npy"], min(reps, 5), tmpdir)
        if not times:
            return None
        return {"ms": times, "bytes": 2 * m * m * 4, "cores": 1, "kind": "reference", "sample": "a [2048,2048] corner (1/16 of the bytes)"}


WORKLOADS = {"lstm": Lstm, "softmax": Softmax, "reduce": ReduceAxis0, "gemm": Gemm, "chain": Chain, "scan": Cumsum, "transpose": TransposedMap}


# ----------------------------------------------------------------------------- main
def reference_arm(args):
    """--impl reference: the reference's own CPU implementation (oracle/_ref) on this box's host cores,
    same metric and config, a bounded sample per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import tempfile
    import numpy as np
    drv, _ = ref_driver_paths()
    if not os.path.exists(drv):
        print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref/ref_driver was not built (no reference checkout at build time)"}))
        return
    cores = os.cpu_count() or 1
    with tempfile.TemporaryDirectory() as tmp:
        def save(name, arr):
            np.save(os.path.join(tmp, name), arr)
        w = args.workload
        if w == "lstm":
            rng = np.random.default_rng(1234 + 1)
            B, H = 256, 1024
            for k in ("x", "h", "c"):
                save(k + ".npy", rng.standard_normal((B, H)).astype(np.float32))
            for k in ("Wx", "Wh"):
                save(k + ".npy", (rng.standard_normal((H, 4 * H)) * 0.02).astype(np.float32))
            save("b.npy", np.zeros((1, 4 * H), np.float32))
            case, cargs = "lstm", ["x.npy", "h.npy", "c.npy", "Wx.npy", "Wh.npy", "b.npy", "c_out.npy", "h_out.npy"]
            nbytes = 4 * (3 * B * H + 2 * H * 4 * H + 4 * H + 2 * B * H)
            flops = 2 * 2 * B * H * 4 * H
            wl = ("C2 LSTM cell step: gates = dot(x,Wx)+dot(h,Wh)+b, c' = sig(f)*c + sig(i)*tanh(g), h' = sig(o)*tanh(c'); "
                  "fp32, B=256 H=1024 per GPU, x,h,c ~ N(0,1), W ~ N(0,0.02), b = 0")
            sample, ncores, scaling, dtype = "the full cell step (8 OpenBLAS sgemm on all host cores + 5 single-threaded JIT kernels)", cores, "weak", "f32"
        elif w == "softmax":
            rng = np.random.default_rng(1234)
            save("a.npy", rng.standard_normal((4096, 1024)).astype(np.float32))
            case, cargs, nbytes, flops = "softmax_naive", ["a.npy", "out.npy"], 4096 * 1024 * 8, 0
            wl = "C1 exp(a-max(a,{-1},true))/sum(exped,{-1},true), fp32 [4096,1024] ~ N(0,1) per GPU"
            sample, ncores, scaling, dtype = "the full [4096,1024] batch per step", 1, "weak", "f32"
        elif w == "reduce":
            rng = np.random.default_rng(1236)
            m = 2048
            save("x.npy", (rng.random((m, m)) * 2 - 1).astype(np.float32))
            case, cargs, nbytes, flops = "reduce", ["sum", "0", "x.npy", "out.npy"], m * m * 4, 0
            wl = "C3 op::sum over axis 0 of fp32 [8192,8192] ~ U(-1,1) per GPU"
            sample, ncores, scaling, dtype = "a [2048,2048] array per step (1/16 of the bytes)", 1, "weak", "f32"
        elif w == "gemm":
            rng = np.random.default_rng(1237)
            m = 2048
            save("A.npy", (rng.standard_normal((m, m)) * 0.02).astype(np.float32))
            save("B.npy", (rng.standard_normal((m, m)) * 0.02).astype(np.float32))
            save("bias.npy", (rng.standard_normal(m) * 0.1).astype(np.float32))
            case, cargs, nbytes, flops = "gemm_tanh", ["A.npy", "B.npy", "bias.npy", "out.npy"], 3 * m * m * 2, 2.0 * m ** 3
            wl = "C4 tanh(dot(A,B)+bias), bf16 A,B [8192,8192] ~ N(0,0.02), bias ~ N(0,0.1), fp32 accumulate, bf16 out"
            sample, ncores, scaling, dtype = "2048^3 in fp32 per step (the reference has no bf16; 1/64 of the flops)", cores, "weak", "f32"
        elif w == "transpose":
            rng = np.random.default_rng(1241)
            m = 2048
            save("x.npy", rng.standard_normal((m, m)).astype(np.float32))
            case, cargs, nbytes, flops = "unary_t", ["tanh", "x.npy", "out.npy"], 2 * m * m * 4, 0
            wl = "y = tanh(x).transpose(), fp32 [8192,8192] ~ N(0,1) per GPU"
            sample, ncores, scaling, dtype = "a [2048,2048] array per step (1/16 of the bytes)", 1, "weak", "f32"
        elif w == "scan":
            rng = np.random.default_rng(1240)
            m = 4
            save("x.npy", (rng.random((m, 8192)) * 2 - 1).astype(np.float32))
            case, cargs, nbytes, flops = "scan", ["sum", "1", "x.npy", "out.npy"], 2 * m * 8192 * 4, 0
            wl = "op::cumsum over the last axis of fp32 [8192,8192] ~ U(-1,1) per GPU (inclusive)"
            sample, ncores, scaling, dtype = "4 of the 8192 rows per step (the reference's CPU scan is quadratic in the row length)", 1, "weak", "f32"
        else:
            rng = np.random.default_rng(1234 + 4)
            m = 1 << 24
            save("x.npy", rng.standard_normal(m).astype(np.float32))
            case, cargs, nbytes, flops = "chain", ["x.npy", "0.5", "0.1", "out.npy"], m * 4, 0
            wl = "C5 sum(sigmoid(x*w+b)*exp(-x*x)), fp32 x ~ N(0,1), 2^31 elements total, w=0.5 b=0.1"
            sample, ncores, scaling, dtype = "2^24 elements per step (1/128 of the workload; the reference's int sizes cap a chunk at 2^28)", 1, "strong", "f32"
        times = run_ref_driver(case, cargs, args.warmup + args.steps, tmp)
    timed = times[args.warmup:]
    ms = sum(timed) / len(timed)
    gbs = nbytes / (ms * 1e-3) / 1e9
    line = {"metric": "fused_expr_hbm_gbs", "value": gbs, "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": scaling,
            "vs_baseline": None, "dtype": dtype, "data": "synthetic", "impl": "reference",
            "config": {"workload": wl},
            "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": ncores, "kind": "reference", "sample": sample},
            "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    if flops:
        line["gemm_tflops"] = flops / (ms * 1e-3) / 1e12
    print(json.dumps(line))


def measure(wl, torch, world, steps, warmup, lib, sample_clocks=True, local=0):
    """Times exactly `steps` steps (device time, max over ranks).  Returns a dict."""
    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    for i in range(warmup):
        wl.step(i)
    barrier()
    fn = wl.graph_fn()
    stepper = GraphStepper(torch, lambda i, st: fn(warmup + i, st), steps, getattr(wl, "lanes", 1)) if fn else None
    if stepper:
        barrier()
        t_spin = time.perf_counter()
        for _ in range(2):
            stepper.replay()
        torch.cuda.synchronize()
        # Untimed spin-up on top of the `warmup` steps: a step of tens of microseconds leaves a GPU that has just come
        # out of idle no time to reach its clocks (one default run measured 59 us per LSTM step right after another
        # process had left the GPU idle, 35 us otherwise).  ~150 ms of the same replays, the same number on every
        # rank (a step may hold a collective).  Only for such short steps: a block of milliseconds has warmed the GPU
        # up by itself, and more untimed work would move a power-capped GEMM from its burst clocks to its sustained
        # ones before the block is timed.
        est = torch.tensor([(time.perf_counter() - t_spin) / 2], dtype=torch.float64, device="cuda")
        if world > 1:
            torch.distributed.all_reduce(est, op=torch.distributed.ReduceOp.MAX)
        est = max(float(est.item()), 1e-5)
        if est < 5e-3:
            for _ in range(min(2000, int(0.15 / est) + 1)):
                stepper.replay()
    barrier()
    sampler = ClockSampler(local) if sample_clocks else None
    if sampler:
        sampler.start()
    launches0 = lib.cache_stats()["launches"]
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

    one_block()        # the reported block: exactly `steps` steps
    # more blocks only to keep the GPU busy ~1.5 s while nvidia-smi samples the clocks; every rank must run
    # the same number of them (each ends in a barrier), so the count is agreed on, not timed per rank
    extra = 0
    if sample_clocks:
        extra = int(min(200, max(0, 1500.0 / max(block_ms[0], 1e-3))))
        if world > 1:
            cnt = torch.tensor([extra], dtype=torch.int64, device="cuda")
            torch.distributed.all_reduce(cnt, op=torch.distributed.ReduceOp.MAX)
            extra = int(cnt.item())
    for _ in range(extra):
        one_block()
    clocks = sampler.stop() if sampler else None
    # the reported figure is the FIRST timed block of exactly `steps` steps; later blocks only keep
    # the GPU busy while nvidia-smi samples the clocks
    t = torch.tensor([block_ms[0]], dtype=torch.float64, device="cuda")
    if world > 1:
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    ms_step = float(t.item()) / steps
    res = {"ms_per_step": ms_step, "clocks": clocks, "graph": bool(stepper),
           "gpu_launches": steps * getattr(wl, "launches_per_step", 1),
           "median_block_ms_per_step": sorted(block_ms)[len(block_ms) // 2] / steps}
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
            "kernel": getattr(wl, "kernel_name", None) or lib.last_variant(), "kernel_ms": ms}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="lstm", choices=sorted(WORKLOADS))
    ap.add_argument("--elements", type=int, default=0, help="chain: total elements (profiling on a small case)")
    ap.add_argument("--gemm-n", type=int, default=0, help="gemm: matrix size (profiling on a small case)")
    ap.add_argument("--scan-shape", default="", help="scan: R,C instead of 8192,8192 (the variants for short and for few, very long rows)")
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
    if world > 1:
        import datetime
        # a rank that falls out of step ends the run in two minutes, not ten
        torch.distributed.init_process_group("nccl", device_id=torch.device("cuda", local),
                                             timeout=datetime.timedelta(seconds=120))
    lib = dali_b200.load_library()
    lib.init(0)
    dev_index = local      # the library indexes the devices it bound; one process per GPU uses its own

    def build(name):
        kw = {}
        if name == "chain" and args.elements:
            kw["total"] = args.elements
        if name == "gemm" and args.gemm_n:
            kw["n"] = args.gemm_n
        if name == "scan" and args.scan_shape:
            kw["shape"] = tuple(int(v) for v in args.scan_shape.split(","))
        return WORKLOADS[name](lib, torch, rank, world, dev_index, **kw)

    wl = build(args.workload)
    wl.verify()
    m = measure(wl, torch, world, args.steps, args.warmup, lib, True, local)
    ms_step = m["ms_per_step"]
    job_bytes = wl.bytes_per_step() * world
    value = job_bytes / (ms_step * 1e-3) / 1e9
    roofline = roofline_of(wl, m, lib)

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    e2e = None
    if not args.no_e2e:
        n_e2e = max(1, min(args.steps, 5))
        external = getattr(wl, "e2e_external", None)
        if external:
            # the workload's end-to-end loop is a C++ program written against the front end's own headers
            barrier()
            dt = external(3, max(n_e2e, 20)) * 1e-3
            n_e2e = max(n_e2e, 20)
            barrier()
        else:
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
        e2e = {"value": job_bytes / float(te.item()) / 1e9, "unit": "GB/s", "h2d_bytes_per_step": wl.h2d,
               "d2h_bytes_per_step": wl.d2h, "steps": n_e2e, "ms_per_step": float(te.item()) * 1e3,
               "api": getattr(wl, "e2e_api", "dalib200_launch_host / C ABI with pinned host buffers (alloc from pool + H2D + "
                                              "kernel + D2H + sync per step)")}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        import tempfile
        with tempfile.TemporaryDirectory() as tmp:
            r = wl.cpu_baseline(tmp, 8)
        if r:
            best = sorted(r["ms"])[len(r["ms"]) // 2]
            cpu = {"value": r["bytes"] / (best * 1e-3) / 1e9, "unit": "GB/s", "cores": r["cores"], "kind": r["kind"],
                   "sample": r["sample"], "ms": best}
            if r.get("flops"):
                cpu["tflops"] = r["flops"] / (best * 1e-3) / 1e12

    others = None
    if args.workload == "lstm" and not args.no_others and world == 1:
        others = {}
        for name in ("gemm", "softmax", "reduce", "chain", "scan", "transpose"):   # the power-capped GEMM before the GPU is hot
            del wl
            torch.cuda.empty_cache()
            time.sleep(1.0)      # each workload starts from a rested GPU, as its own `--workload` run would (power cap)
            wl = build(name)
            wl.verify()
            mo = measure(wl, torch, world, 24, 3, lib, False, local)      # 24: whole steps on each of the softmax lanes
            ro = roofline_of(wl, mo, lib)
            entry = {"workload": wl.describe()["workload"], "ms_per_step": mo["ms_per_step"],
                     "gbs": wl.bytes_per_step() / (mo["ms_per_step"] * 1e-3) / 1e9,
                     "roofline": {k: ro[k] for k in ("bound", "achieved", "peak", "unit", "frac", "frac_of_sustained_peak", "kernel") if k in ro}}
            if wl.flops_per_step():
                entry["tflops"] = wl.flops_per_step() / (mo["ms_per_step"] * 1e-3) / 1e12
            others[name] = entry
        wl = build("lstm")

    if rank == 0:
        cfg = wl.describe()
        line = {"metric": "fused_expr_hbm_gbs", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": wl.scaling,
                "vs_baseline": None, "dtype": "bf16" if args.workload == "gemm" else "f32", "data": "synthetic",
                "config": cfg, "clocks": m["clocks"], "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e,
                "gpu_launches": int(m["gpu_launches"]), "timed_with": "CUDA graph replay of the step's launches" if m["graph"] else "eager launches",
                "pct_of_nominal_8TBs": 100.0 * value / world / 8000.0}
        if wl.flops_per_step():
            line["gemm_tflops"] = wl.flops_per_step() * world / (ms_step * 1e-3) / 1e12
        if others:
            line["other_workloads"] = others
        print(json.dumps(line))
    if world > 1:
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
