"""Benchmark of the training-step hot path: fp32 MLP 1024->4096->4096->4096->1024 (tanh hidden,
zero bias, Kaiming-uniform weights), global batch 8192, MSE loss, one Adam step per iteration;
synthetic N(0,1) inputs and targets (seeded). One step = forward + backward + Adam over one batch.

  python bench.py --gpus 1 --steps 10 --warmup 3          # this implementation (B200)
  python bench.py --impl reference --steps 1 --warmup 0   # Endia's CPU algorithm (oracle port)

Under torchrun (--gpus N > 1) the global batch is split over the ranks (strong scaling), the
gradients are all-reduced over NCCL while the backward pass is still running, and the mean over
ranks is folded into Adam's gradient scale. Rank 0 prints one JSON line.
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

DIMS = [1024, 4096, 4096, 4096, 1024]
GLOBAL_BATCH = 8192
METRIC = "train-step samples/s (MLP fwd+bwd+Adam)"
UNIT = "samples/s"


def gemm_flops(batch, dims=DIMS):
    """Sum of 2*M*N*K over the GEMMs of one step: forward, dW for every layer, dX for every layer
    but the first (x needs no gradient)."""
    fwd = sum(2.0 * batch * dims[i] * dims[i + 1] for i in range(len(dims) - 1))
    return fwd + fwd + sum(2.0 * batch * dims[i] * dims[i + 1] for i in range(1, len(dims) - 1))


def make_weights(seed=0, dims=DIMS):
    r = np.random.Generator(np.random.PCG64(seed))
    Ws = []
    for i in range(len(dims) - 1):
        lim = np.sqrt(6.0 / dims[i])
        Ws.append(r.uniform(-lim, lim, (dims[i], dims[i + 1])).astype(np.float32))
    return r, Ws


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            d = json.load(fh)
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d["bf16_tflops_sustained"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons through NVML from a thread while the timed region
    runs (read-only queries)."""

    def __init__(self, gpu_index, period_s=0.01):
        self.gpu, self.period = gpu_index, period_s
        self.samples, self.reasons = [], set()
        self.sm_max = None
        self._stop = None
        self._thread = None

    def start(self):
        import threading
        try:
            import pynvml
            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            idx = self.gpu
            if visible:
                try:
                    idx = int(visible.split(",")[self.gpu])
                except ValueError:
                    idx = self.gpu
            h = pynvml.nvmlDeviceGetHandleByIndex(idx)
            self.sm_max = float(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM))
        except Exception:
            return
        bits = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "sw_thermal_slowdown": 0x20,
                "hw_thermal_slowdown": 0x40}
        self._stop = threading.Event()

        def loop():
            while not self._stop.is_set():
                try:
                    self.samples.append(float(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)))
                    r = pynvml.nvmlDeviceGetCurrentClocksEventReasons(h)
                    for name, bit in bits.items():
                        if r & bit:
                            self.reasons.add(name)
                except Exception:
                    pass
                self._stop.wait(self.period)
        self._thread = threading.Thread(target=loop, daemon=True)
        self._thread.start()

    def stop(self):
        if self._thread is not None:
            self._stop.set()
            self._thread.join(timeout=2)
        sm = self.samples
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": self.sm_max,
                "reasons": sorted(self.reasons), "samples": len(sm)}


class GemmTimer:
    """Brackets every GEMM (or FFT) call with CUDA events on the launching stream."""

    def __init__(self, torch):
        self.torch = torch
        self.records = []
        self._cur = None

    def start(self, flops):
        e0 = self.torch.cuda.Event(enable_timing=True)
        e0.record()
        self._cur = (flops, e0)

    def stop(self):
        e1 = self.torch.cuda.Event(enable_timing=True)
        e1.record()
        self.records.append((self._cur[0], self._cur[1], e1))

    def summary(self):
        ms = sum(a.elapsed_time(b) for _, a, b in self.records)
        fl = sum(f for f, _, _ in self.records)
        return len(self.records), fl, ms


class TrainStep:
    """The step a user of the library writes: nn.mlp + mse + backward + Adam.step + zero_grad."""

    def __init__(self, nd, torch, rank, world, seed=0):
        from endia_b200 import dist as ndist
        self.nd, self.torch, self.rank, self.world = nd, torch, rank, world
        self.local_batch = GLOBAL_BATCH // world
        r, Ws = make_weights(seed)
        x = r.standard_normal((GLOBAL_BATCH, DIMS[0])).astype(np.float32)
        y = r.standard_normal((GLOBAL_BATCH, DIMS[-1])).astype(np.float32)
        lo, hi = rank * self.local_batch, (rank + 1) * self.local_batch
        self.x_host = torch.from_numpy(np.ascontiguousarray(x[lo:hi])).pin_memory()
        self.y_host = torch.from_numpy(np.ascontiguousarray(y[lo:hi])).pin_memory()
        self.loss_host = torch.empty(1, dtype=torch.float32).pin_memory()
        self.W = [nd.Array(w, requires_grad=True) for w in Ws]
        self.B = [nd.Array([DIMS[i + 1]], requires_grad=True) for i in range(len(DIMS) - 1)]
        self.params = [p for wb in zip(self.W, self.B) for p in wb]
        self.X = nd.Array(x[lo:hi])
        self.Y = nd.Array(y[lo:hi])
        self.opt = nd.optim.Adam(self.params, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8)
        self.reducer = None
        if world > 1:
            # an all-reduce per parameter started from the backward walk; ENDIA_B200_DP_MODE=bucket sums
            # all gradients with one all-reduce after the pass instead
            self.reducer = ndist.GradAllReducer(self.params)
            self.opt.grad_scale = 1.0 / world   # global-mean loss = mean of the ranks' local means
        self.flat = ndist.flat_tensor
        self.feeder = None

    def step(self, host_io=False):
        nd = self.nd
        X, Y = self.X, self.Y
        if host_io:
            # every step's batch comes from pinned host memory; its copy runs on a copy stream
            # while the previous step computes (two sets of device input arrays)
            if self.feeder is None:
                from endia_b200.utils.general import HostBatchFeeder
                self.feeder = HostBatchFeeder([self.x_host, self.y_host], [self.X.shape(), self.Y.shape()])
            X, Y = self.feeder.next()
        pred = nd.nn.mlp([X, None] + self.params, activation="tanh")
        loss = nd.mse(pred, Y)
        loss.backward()
        if self.reducer is not None:
            self.reducer.wait()
        self.opt.step()
        loss.zero_grad()
        if host_io:
            self.feeder.prefetch()
            self.loss_host.copy_(self.flat(loss), non_blocking=True)
            self.torch.cuda.current_stream().synchronize()
            return float(self.loss_host[0])
        return loss



FFT_METRIC = "fftn fwd+VJP GB/s"


class FFTStep:
    """c4: 32 signals of 2^20 points, loss = sum(|fft(x)|^2) * 2^-20, forward + VJP w.r.t. x.
    c5: 512^3 grid, loss = sum(real(fftn(x)) * w), forward + VJP; over N ranks the grid is split
    along axis 0 (slab decomposition, one all-to-all per transform)."""

    def __init__(self, nd, torch, workload, rank, world):
        self.nd, self.torch, self.workload, self.rank, self.world = nd, torch, workload, rank, world
        r = np.random.Generator(np.random.PCG64(0))
        if workload == "c4":
            self.shape = (32, 1 << 20)
            x = (r.standard_normal(self.shape, dtype=np.float32) + 1j * r.standard_normal(self.shape, dtype=np.float32)).astype(np.complex64)
            self.x_host = torch.from_numpy(x).pin_memory()
            self.X = nd.Array(x, requires_grad=True)
            self.alg_bytes = 4.0 * x.nbytes
        else:
            n = 512
            self.shape = (n, n, n)
            s0 = n // world
            sub = (s0, n, n)
            r = np.random.Generator(np.random.PCG64(rank))
            x = (r.standard_normal(sub, dtype=np.float32) + 1j * r.standard_normal(sub, dtype=np.float32)).astype(np.complex64)
            self.x_host = torch.from_numpy(x).pin_memory()
            self.alg_bytes = 4.0 * 8.0 * n ** 3
            self.X = nd.Array(x, requires_grad=True)
            # w is split like the result: along axis 1 when the transform is slab-decomposed
            self.W = nd.Array(r.uniform(-1, 1, (n, n // world, n)).astype(np.float32))
        self.loss_host = torch.empty(1, dtype=torch.float32).pin_memory()

    def step(self, host_io=False):
        nd, torch = self.nd, self.torch
        from endia_b200.dist import flat_tensor
        if host_io:
            flat_tensor(self.X).copy_(torch.view_as_real(self.x_host).reshape(-1), non_blocking=True)
        if self.workload == "c4":
            y = nd.fft(self.X)
            loss = nd.sum(nd.square(nd.to_abs(y))) * (1.0 / (1 << 20))
        elif self.world == 1:
            y = nd.fftn(self.X)
            loss = nd.sum(nd.real(y) * self.W)
        else:
            from endia_b200.dist import fftn_slab
            y = fftn_slab(self.X, self.world)
            loss = nd.sum(nd.real(y) * self.W)     # this rank's part of the global sum
        loss.backward()
        dx = self.X.grad()
        loss.zero_grad()
        if host_io:
            self.loss_host.copy_(flat_tensor(loss), non_blocking=True)
            torch.cuda.current_stream().synchronize()
        return dx



class SmallStep:
    """c1: MLP 1-32-32-32-1 (ReLU, bias), batch 128, x ~ U[0,1), y = sin(15x), MSE + Adam: the whole
    step is one kernel launch (nn.fused_train_step)."""
    dims, batch = [1, 32, 32, 32, 1], 128

    def __init__(self, nd, torch):
        self.nd, self.torch = nd, torch
        r = np.random.Generator(np.random.PCG64(0))
        Ws, bs = [], []
        for i in range(4):
            lim = np.sqrt(6.0 / self.dims[i])
            Ws.append(r.uniform(-lim, lim, (self.dims[i], self.dims[i + 1])).astype(np.float32))
            bs.append(r.uniform(-lim, lim, (self.dims[i + 1],)).astype(np.float32))
        x = r.uniform(0, 1, (self.batch, 1)).astype(np.float32)
        y = np.sin(np.float32(15) * x).astype(np.float32)
        self.x_host, self.y_host = torch.from_numpy(x).pin_memory(), torch.from_numpy(y).pin_memory()
        self.W = [nd.Array(w, requires_grad=True) for w in Ws]
        self.B = [nd.Array(b, requires_grad=True) for b in bs]
        self.params = [p for wb in zip(self.W, self.B) for p in wb]
        self.X, self.Y = nd.Array(x), nd.Array(y)
        self.opt = nd.optim.Adam(self.params, lr=1e-3)
        self.loss_host = torch.empty(1, dtype=torch.float32).pin_memory()
        self.samples = self.batch
        self.flops = 1.614e6

    def step(self, host_io=False):
        from endia_b200.dist import flat_tensor
        if host_io:
            flat_tensor(self.X).copy_(self.x_host.reshape(-1), non_blocking=True)
            flat_tensor(self.Y).copy_(self.y_host.reshape(-1), non_blocking=True)
        loss = self.nd.nn.fused_train_step(self.W, self.B, self.X, self.Y, self.opt, activation="relu")
        if host_io:
            self.loss_host.copy_(flat_tensor(loss), non_blocking=True)
            self.torch.cuda.current_stream().synchronize()
        return loss


class PenaltyStep:
    """c3: MLP 256-1024-1024-1 (tanh), batch 4096; loss = mean(f) + 0.1 * mean |df/dx|^2 with
    create_graph=True, then gradients w.r.t. the parameters (double backward)."""
    dims, batch = [256, 1024, 1024, 1], 4096

    def __init__(self, nd, torch):
        self.nd, self.torch = nd, torch
        r = np.random.Generator(np.random.PCG64(0))
        Ws = [r.uniform(-np.sqrt(6.0 / self.dims[i]), np.sqrt(6.0 / self.dims[i]),
                        (self.dims[i], self.dims[i + 1])).astype(np.float32) for i in range(3)]
        x = r.standard_normal((self.batch, self.dims[0])).astype(np.float32)
        self.x_host = torch.from_numpy(x).pin_memory()
        self.W = [nd.Array(w, requires_grad=True) for w in Ws]
        self.B = [nd.Array([self.dims[i + 1]], requires_grad=True) for i in range(3)]
        self.X = nd.Array(x, requires_grad=True)
        self.loss_host = torch.empty(1, dtype=torch.float32).pin_memory()
        self.samples = self.batch
        self.flops = 62.32e9
        # The step is about 110 short launches: replayed as one CUDA graph (the library's
        # CapturedStep) it is bound by the GPU instead of the host. ENDIA_B200_BENCH_GRAPH=0 runs
        # it op by op.
        self.captured = None
        if os.environ.get("ENDIA_B200_BENCH_GRAPH", "1") != "0":
            from endia_b200.utils.general import CapturedStep
            self.captured = CapturedStep(self._eager)

    def step(self, host_io=False):
        from endia_b200.dist import flat_tensor
        if host_io:
            flat_tensor(self.X).copy_(self.x_host.reshape(-1), non_blocking=True)
        loss, grads = self.captured() if self.captured is not None else self._eager()
        if host_io:
            self.loss_host.copy_(flat_tensor(loss), non_blocking=True)
            self.torch.cuda.current_stream().synchronize()
        return grads

    def _eager(self):
        nd = self.nd
        args = [self.X, None]
        for w, b in zip(self.W, self.B):
            args += [w, b]
        f = nd.nn.mlp(args, activation="tanh")
        gx = nd.grad(outs=[nd.sum(f)], inputs=[self.X], create_graph=True)[0]
        loss = nd.mean(f, [0, 1]) + 0.1 * (nd.sum(gx * gx) / float(self.batch))
        grads = nd.grad(outs=[loss], inputs=self.W + self.B)
        return loss, grads


def fft_cpu_baseline(workload):
    """Endia's CPU algorithm for the FFT configs (oracle port: float64 radix-2 with per-axis
    gathers, rows spread over the host threads as the reference's parallelize does), forward + VJP,
    on a bounded sample: c4 on 4 of the 32 signals, c5 on a 256^3 grid (scaled by points*log2)."""
    from oracle import endia_oracle as eo
    eo.build()
    threads = max(1, (os.cpu_count() or 2) // 2)   # the reference uses the physical cores
    eo.config["fft_threads"] = threads
    r = np.random.Generator(np.random.PCG64(0))
    if workload == "c4":
        shape, full = (4, 1 << 20), 32 * (1 << 20) * 20.0
        work = 4 * (1 << 20) * 20.0
    else:
        shape, full = (256, 256, 256), 512.0 ** 3 * 27
        work = 256.0 ** 3 * 24
    x = (r.standard_normal(shape) + 1j * r.standard_normal(shape)).astype(np.complex64)
    t0 = time.perf_counter()
    X = eo.Array(x, requires_grad=True)
    if workload == "c4":
        loss = eo.sum(eo.square(eo.to_abs(eo.fft(X)))) * (1.0 / (1 << 20))
    else:
        loss = eo.sum(eo.real(eo.fftn(X)) * eo.Array(r.uniform(-1, 1, shape).astype(np.float32)))
    loss.backward()
    dt = time.perf_counter() - t0
    eo.config["fft_threads"] = 1
    full_s = dt * full / work
    alg = 4.0 * 8.0 * (32 * (1 << 20) if workload == "c4" else 512 ** 3)
    return {"value": alg / full_s / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
            "sample": "%s forward+VJP on shape %s in %.2f s, scaled by n*log2(n) to the full size" % (
                workload, list(shape), dt), "host_cores_available": os.cpu_count(), "seconds": dt}


def cpu_baseline(sample_rows=48, threads_note=True):
    """Endia's CPU algorithm (the oracle port, faithful mode: single-threaded dot-product matmul,
    one temporary per op, Adam as array expressions) on a bounded sample of the same workload:
    `sample_rows` rows of the batch through the full-size network. Forward+backward scales linearly
    with the batch and the Adam step does not depend on it, so the full-batch time is
    rows-time * (8192 / sample_rows) + Adam-time."""
    from oracle import endia_oracle as eo
    eo.build()
    eo.config["mode"] = "faithful"
    r, Ws = make_weights(0)
    x = r.standard_normal((sample_rows, DIMS[0])).astype(np.float32)
    y = r.standard_normal((sample_rows, DIMS[-1])).astype(np.float32)
    W = [eo.Array(w, requires_grad=True) for w in Ws]
    B = [eo.Array(np.zeros(DIMS[i + 1], np.float32), requires_grad=True) for i in range(len(DIMS) - 1)]
    params = [p for wb in zip(W, B) for p in wb]
    opt = eo.Adam(params)
    t0 = time.perf_counter()
    loss = eo.mse(eo.mlp_forward(eo.Array(x), W, B, "tanh"), eo.Array(y))
    loss.backward()
    t1 = time.perf_counter()
    opt.step()
    t2 = time.perf_counter()
    full = (t1 - t0) * (GLOBAL_BATCH / sample_rows) + (t2 - t1)
    return {"value": GLOBAL_BATCH / full, "unit": UNIT, "cores": 1, "kind": "port",
            "sample": "%d of 8192 batch rows through the full 1024-4096-4096-4096-1024 network "
                      "(fwd+bwd %.2f s, scaled x%.1f) + one full Adam step (%.2f s); the reference's "
                      "matmul is single-threaded (matmul_op.mojo:168-169)" % (
                          sample_rows, t1 - t0, GLOBAL_BATCH / sample_rows, t2 - t1),
            "host_cores_available": os.cpu_count(), "seconds": t2 - t0}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    vals, last = [], None
    for i in range(args.warmup + args.steps):
        last = cpu_baseline(sample_rows=args.cpu_rows)
        if i >= args.warmup:
            vals.append(last["value"])
    value = float(np.mean(vals)) if vals else last["value"]
    last["value"] = value
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1000.0 * GLOBAL_BATCH / value,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": "c2: MLP 1024-4096-4096-4096-1024 tanh, global batch 8192, MSE+Adam",
                       "global_batch": GLOBAL_BATCH},
            "cpu_baseline": last,
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def tc_scheme(gemm_flag):
    """Scheme the two-CTA tcgen05 kernel runs for this --gemm flag (mirrors the library's choice)."""
    if gemm_flag == "3xtf32" or (gemm_flag == "auto" and os.environ.get("ENDIA_B200_TC_SCHEME", "")[:1] in ("3", "0")):
        return "3xtf32"
    return "tf32_bf16x2"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="endia_b200", choices=["endia_b200", "reference"])
    ap.add_argument("--cpu-rows", type=int, default=160)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--gemm", default="auto", choices=["auto", "ffma", "3xtf32", "tf32_bf16x2"],
                    help="auto = tf32_bf16x2 on the two-CTA tcgen05 kernel (one tf32 MMA + two bf16 correction "
                         "MMAs per product), 3xTF32 split-K or FFMA where that kernel does not apply")
    ap.add_argument("--workload", default="c2", choices=["c1", "c2", "c3", "c4", "c5"],
                    help="c2 (default, the headline): MLP train step; c1: small MLP, single-launch step; "
                         "c3: gradient-penalty (second-order) step; c4 / c5: FFT forward + VJP")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
        return
    if args.warmup < 3:
        args.warmup = 3

    import torch
    import endia_b200 as nd
    from endia_b200 import _lib, dist as ndist
    import torch.distributed as tdist

    rank, world = ndist.init_process_group()
    nd._array.device()
    nd.config.gemm_algo = {"auto": _lib.GEMM_AUTO, "ffma": _lib.GEMM_FFMA, "3xtf32": _lib.GEMM_3XTF32,
                           "tf32_bf16x2": _lib.GEMM_TF32_BF16X2}[args.gemm]
    is_fft = args.workload in ("c4", "c5")
    is_small = args.workload in ("c1", "c3")
    if is_fft:
        work = FFTStep(nd, torch, args.workload, rank, world)
    elif args.workload == "c1":
        work = SmallStep(nd, torch)
    elif args.workload == "c3":
        work = PenaltyStep(nd, torch)
    else:
        work = TrainStep(nd, torch, rank, world)

    def barrier():
        if world > 1:
            tdist.barrier()
        torch.cuda.synchronize()

    # More than one rank: the first steps also set up NCCL's channels and buffers for each message
    # size (seen as a slow first ten steps on 8 GPUs), so at least ten untimed steps are run.
    for _ in range(max(args.warmup, 10) if world > 1 else args.warmup):
        work.step()
    barrier()

    # ---- device-resident timing (value) with per-GEMM events
    sampler = ClockSampler(torch.cuda.current_device())
    timer = GemmTimer(torch)
    nd.config.gemm_timer = timer
    nd.config.fft_timer = timer
    launches0 = _lib.lib.endia_b200_launch_count()
    replays0 = getattr(getattr(work, "captured", None), "replays", 0)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        work.step()
    e1.record()
    barrier()
    clocks = sampler.stop()
    nd.config.gemm_timer = None
    nd.config.fft_timer = None
    launches = _lib.lib.endia_b200_launch_count() - launches0
    cap = getattr(work, "captured", None)
    if cap is not None:   # kernels replayed inside a CUDA graph are not seen by the enqueue counter
        launches += cap.launches_per_replay * (cap.replays - replays0)
    ms_total = e0.elapsed_time(e1)
    n_gemm, gemm_fl, gemm_ms = timer.summary()

    # ---- end-to-end timing through the public API with host buffers
    for _ in range(2):
        work.step(host_io=True)
    barrier()
    e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2.record()
    for _ in range(args.steps):
        work.step(host_io=True)
    e3.record()
    barrier()
    ms_e2e = e2.elapsed_time(e3)

    times = torch.tensor([ms_total, ms_e2e, gemm_ms], dtype=torch.float64, device="cuda")
    if world > 1:
        tdist.all_reduce(times, op=tdist.ReduceOp.MAX)
    ms_total, ms_e2e, gemm_ms = [float(t) for t in times.cpu()]
    if rank != 0:
        if world > 1:
            tdist.destroy_process_group()
        return

    pk = peaks()
    if is_small:
        ms_step = ms_total / args.steps
        line = {
            "metric": METRIC if args.workload == "c1" else "gradient-penalty step samples/s (fwd + double backward)",
            "value": work.samples / (ms_step / 1000.0), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "replicas only",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "%s: MLP %s, batch %d" % (args.workload, "-".join(map(str, work.dims)), work.batch),
                       "note": "c1 is bound by launch latency (one launch per step); no roofline is quoted for it"
                               if args.workload == "c1" else "create_graph=True path: every VJP is a composition of ops"},
            "clocks": {"sm_mhz": clocks["sm_mhz"], "sm_max_mhz": clocks["sm_max_mhz"],
                       "reasons": clocks["reasons"], "samples": clocks["samples"]},
            "e2e": {"value": work.samples / (ms_e2e / args.steps / 1000.0), "unit": UNIT,
                    "h2d_bytes_per_step": int(work.x_host.numel() * 4), "d2h_bytes_per_step": 4},
            "gpu_launches": int(launches),
            "roofline": {"bound": "tensor", "achieved": (gemm_fl / (gemm_ms / 1000.0) / 1e12) if gemm_ms > 0 else None,
                         "peak": pk["bf16_tflops_sustained"] / 6.0, "unit": "TFLOP/s", "frac": None, "traffic": None,
                         "kernel": "gemm calls (%d, %.1f%% of the step)" % (n_gemm, 100.0 * gemm_ms / ms_total if ms_total else 0.0),
                         "algorithmic_gflop_per_step": work.flops / 1e9},
        }
        if cap is not None:
            # replayed as one CUDA graph: no per-call events; the whole step against its algorithmic flops
            line["config"]["launch"] = "one CUDA graph per step (%d kernels); ENDIA_B200_BENCH_GRAPH=0 runs op by op" % (
                cap.launches_per_replay)
            line["roofline"]["achieved"] = work.flops / (ms_step / 1000.0) / 1e12
            line["roofline"]["kernel"] = "whole step (algorithmic flops / step time)"
        print(json.dumps(line))
        return
    if is_fft:
        ms_step = ms_total / args.steps
        hbm_peak = pk["hbm_gbs"]
        ach = gemm_fl / (gemm_ms / 1000.0) / 1e9 if gemm_ms > 0 else 0.0
        line = {
            "metric": FFT_METRIC, "value": work.alg_bytes / (ms_step / 1000.0) / 1e9, "unit": "GB/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "c64",
            "data": "synthetic",
            "config": {"workload": "%s: %s complex64, forward + VJP" % (args.workload, list(work.shape)),
                       "parallelism": ("slab%d" % world) if args.workload == "c5" else "single",
                       "algorithmic_bytes_per_step": work.alg_bytes,
                       "l2": "arrays of 256 MiB / 1 GiB exceed the 126 MB L2; no flush"},
            "clocks": {"sm_mhz": clocks["sm_mhz"], "sm_max_mhz": clocks["sm_max_mhz"],
                       "reasons": clocks["reasons"], "samples": clocks["samples"]},
            "e2e": {"value": work.alg_bytes / (ms_e2e / args.steps / 1000.0) / 1e9, "unit": "GB/s",
                    "h2d_bytes_per_step": int(work.x_host.numel() * 8) * world, "d2h_bytes_per_step": 4 * world},
            "gpu_launches": int(launches),
            "roofline": {"bound": "hbm", "achieved": ach, "peak": hbm_peak, "unit": "GB/s",
                         "frac": ach / hbm_peak if hbm_peak else None, "traffic": None,
                         "kernel": "fft_c2c calls (%d, %.1f%% of the step); algorithmic bytes = one read + "
                                   "one write of the array per transform" % (n_gemm, 100.0 * gemm_ms / ms_total),
                         "peak_note": "%s hbm_gbs (copy)" % pk["source"]},
        }
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = fft_cpu_baseline(args.workload)
        print(json.dumps(line))
        if world > 1:
            tdist.destroy_process_group()
        return
    ms_step = ms_total / args.steps
    value = GLOBAL_BATCH / (ms_step / 1000.0)
    tflops = gemm_fl / (gemm_ms / 1000.0) / 1e12 if gemm_ms > 0 else 0.0
    tc = bool(_lib.lib.endia_b200_has_tcgen05()) and args.gemm != "ffma"
    # Tensor-core time per logical product in units of one bf16 MMA: 3xTF32 issues three tf32 MMAs
    # (tf32 runs at half the bf16 rate) = 6; the bf16-compensated scheme one tf32 and two bf16 = 4.
    # The ceiling for logical flops is the measured bf16 throughput divided by that.
    bf16c = tc_scheme(args.gemm) == "tf32_bf16x2"
    peak = pk["bf16_tflops_sustained"] / (4.0 if bf16c else 6.0)
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "c2: MLP 1024-4096-4096-4096-1024 tanh, global batch 8192, MSE+Adam",
                   "global_batch": GLOBAL_BATCH, "per_gpu_batch": GLOBAL_BATCH // world,
                   "parallelism": "dp%d" % world,
                   "gemm": ("tcgen05, one tf32 MMA + two bf16 correction MMAs per product (fp32 accumulate, "
                            "error <= 2.3e-6 of |a||b|)" if bf16c else "tcgen05 3xTF32 (fp32 accumulate)")
                   if tc else "fp32 FFMA",
                   "l2": "activations and weights (>= 32 MiB each, 1.3 GB per step) exceed the 126 MB L2; no flush",
                   "e2e_io": "each step's batch is copied from pinned host memory on a copy stream while the "
                             "previous step computes; the loss is read back every step"},
        "clocks": {"sm_mhz": clocks["sm_mhz"], "sm_max_mhz": clocks["sm_max_mhz"],
                   "reasons": clocks["reasons"], "samples": clocks["samples"]},
        "e2e": {"value": GLOBAL_BATCH / (ms_e2e / args.steps / 1000.0), "unit": UNIT,
                "h2d_bytes_per_step": int(work.x_host.numel() * 4 + work.y_host.numel() * 4) * world,
                "d2h_bytes_per_step": 4 * world},
        "gpu_launches": int(launches),
        "roofline": {"bound": "tensor", "achieved": tflops, "peak": peak, "unit": "TFLOP/s",
                     "frac": tflops / peak if peak else None,
                     # dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant GEMM shape
                     # (8192 x 4096 x 4096, the forward and dX products of the 4096-wide layers), from
                     # the committed ncu capture; the other shapes of the step were not captured
                     "traffic": (1.37e9 if bf16c else 1.49e9) if (tc and world == 1) else None,
                     "traffic_note": "bytes per launch of gemm_tc2p_kernel at 8192x4096x4096 (ncu, profiles/%s); "
                                     "compulsory 0.51e9" % ("gemm_tc2p_tf32_bf16x2_8192x4096x4096_ncu.md" if bf16c
                                                            else "gemm_tc2p_8192x4096x4096_ncu.md"),
                     "kernel": "gemm (%d launches, %.1f%% of the step)" % (
                         n_gemm, 100.0 * gemm_ms / ms_total if ms_total else 0.0),
                     "peak_note": ("%s bf16_tflops_sustained %.1f / 4 (one tf32 MMA = 2 bf16 MMA times, plus two "
                                   "bf16 MMAs per product)" if bf16c else
                                   "%s bf16_tflops_sustained %.1f / 2 (tf32 rate) / 3 (MMAs per 3xTF32 product)") % (
                         pk["source"], pk["bf16_tflops_sustained"]),
                     "frac_of_3xtf32_ceiling": tflops / (pk["bf16_tflops_sustained"] / 6.0),
                     "frac_of_bf16_%s" % pk["source"]: tflops / pk["bf16_tflops_sustained"],
                     "algorithmic_gflop_per_step": gemm_flops(GLOBAL_BATCH) / 1e9 / world},
    }
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(sample_rows=args.cpu_rows)
    print(json.dumps(line))
    if world > 1:
        tdist.destroy_process_group()


if __name__ == "__main__":
    main()
