"""Benchmark of the reverse-mode hot path on B200.

Headline (the JSON line's own metric): c2, the fp32 MLP 1024->4096->4096->4096->1024 (tanh hidden,
zero bias, Kaiming-uniform weights), global batch 8192, MSE loss, one Adam step per iteration;
synthetic N(0,1) inputs and targets (seeded). One step = forward + backward + Adam over one batch.
The same line carries the other configurations as sub-records under "workloads" (c1 small MLP,
c3 gradient-penalty double backward, c4 batched 1-D FFT + VJP, c5 512^3 fftn + VJP) and the c2 step
on the 3xTF32 scheme under "alt".

  python bench.py --gpus 1 --steps 10 --warmup 3          # this implementation (B200), all workloads
  python bench.py --workload c4                            # one workload as the top-level line
  python bench.py --impl reference --steps 2 --warmup 0   # Endia's CPU algorithm (oracle port)

Under torchrun (--gpus N > 1) the c2 batch is split over the ranks (strong scaling) and the
gradients are summed over NCCL; the line then carries the 512^3 fftn as a slab-decomposed
sub-record and, for both, a "parity" record: after the timed loops one step from the seeded weights
is run on all ranks and compared on rank 0 with the same step done by one rank on the whole batch.
Rank 0 prints one JSON line.
"""
import argparse
import json
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

DIMS = [1024, 4096, 4096, 4096, 1024]
GLOBAL_BATCH = 8192
METRIC = "train-step samples/s (MLP fwd+bwd+Adam)"
UNIT = "samples/s"
FFT_METRIC = "fftn fwd+VJP GB/s"


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


def workload_config(workload, world):
    """The `config` object of a workload's line: the same for this implementation and for the
    reference arm (what differs between the arms is reported outside it)."""
    if workload == "c2":
        return {"workload": "c2: MLP 1024-4096-4096-4096-1024 tanh, global batch 8192, MSE+Adam",
                "global_batch": GLOBAL_BATCH, "per_gpu_batch": GLOBAL_BATCH // world, "parallelism": "dp%d" % world,
                "l2": "activations and weights (>= 32 MiB each, 1.3 GB per step) exceed the 126 MB L2; no flush"}
    if workload == "c1":
        return {"workload": "c1: MLP 1-32-32-32-1 relu, bias, batch 128, x ~ U[0,1), y = sin(15x), MSE+Adam",
                "global_batch": 128, "parallelism": "replicas only",
                "l2": "bound by launch latency, no roofline is quoted; an L2 flush between steps would "
                      "time the flush"}
    if workload == "c3":
        return {"workload": "c3: MLP 256-1024-1024-1 tanh, batch 4096, loss = mean(f) + 0.1 mean|df/dx|^2 "
                            "(create_graph=True), gradients to the parameters",
                "global_batch": 4096, "parallelism": "replicas only",
                "l2": "the step's arrays (16 MiB activations, 4 MiB weights) fit the 126 MB L2; a 256 MiB "
                      "buffer is written between timed steps"}
    if workload == "c4":
        return {"workload": "c4: 32 x 2^20 complex64, loss = sum|fft(x)|^2 * 2^-20, forward + VJP",
                "parallelism": "replicas only", "algorithmic_bytes_per_step": 4.0 * 8.0 * 32 * (1 << 20),
                "l2": "the 256 MiB arrays exceed the 126 MB L2; no flush"}
    return {"workload": "c5: 512^3 complex64, loss = sum(real(fftn(x)) * w), forward + VJP",
            "parallelism": ("slab%d" % world) if world > 1 else "single",
            "algorithmic_bytes_per_step": 4.0 * 8.0 * 512 ** 3,
            "l2": "the 1 GiB arrays exceed the 126 MB L2; no flush"}


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


class CallTimer:
    """Brackets every GEMM (or FFT) call with CUDA events on the launching stream."""

    def __init__(self, torch):
        self.torch = torch
        self.records = []
        self._cur = None

    def start(self, work):
        e0 = self.torch.cuda.Event(enable_timing=True)
        e0.record()
        self._cur = (work, e0)

    def stop(self):
        e1 = self.torch.cuda.Event(enable_timing=True)
        e1.record()
        self.records.append((self._cur[0], self._cur[1], e1))

    def summary(self):
        ms = sum(a.elapsed_time(b) for _, a, b in self.records)
        work = sum(f for f, _, _ in self.records)
        return len(self.records), work, ms


# ------------------------------------------------------------------------------------ workloads
class TrainStep:
    """c2, the step a user of the library writes: nn.mlp + mse + backward + Adam.step + zero_grad.
    With more than one rank the batch rows are split contiguously over the ranks and the gradients
    are summed by endia_b200.dist (mode from ENDIA_B200_DP_MODE, default chosen by the library)."""
    samples = GLOBAL_BATCH

    def __init__(self, nd, torch, rank, world, seed=0, data_parallel=True):
        from endia_b200 import dist as ndist
        self.nd, self.torch, self.rank, self.world = nd, torch, rank, world
        self.ndist = ndist
        r, self.Ws_host = make_weights(seed)
        x = r.standard_normal((GLOBAL_BATCH, DIMS[0])).astype(np.float32)
        y = r.standard_normal((GLOBAL_BATCH, DIMS[-1])).astype(np.float32)
        self.local_batch = GLOBAL_BATCH // world
        lo, hi = rank * self.local_batch, (rank + 1) * self.local_batch
        self.x_host = torch.from_numpy(np.ascontiguousarray(x[lo:hi])).pin_memory()
        self.y_host = torch.from_numpy(np.ascontiguousarray(y[lo:hi])).pin_memory()
        self.loss_host = torch.empty(1, dtype=torch.float32).pin_memory()
        self.W = [nd.Array(w, requires_grad=True) for w in self.Ws_host]
        self.B = [nd.Array([DIMS[i + 1]], requires_grad=True) for i in range(len(DIMS) - 1)]
        self.params = [p for wb in zip(self.W, self.B) for p in wb]
        self.X = nd.Array(x[lo:hi])
        self.Y = nd.Array(y[lo:hi])
        self.reducer = None
        self.dp_mode = "single"
        if world > 1 and data_parallel:
            self.opt, self.reducer = ndist.data_parallel_adam(self.params, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8)
            self.dp_mode = self.reducer.mode
        else:
            self.opt = nd.optim.Adam(self.params, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8)
        self.feeder = None
        self.h2d_bytes = int(self.x_host.numel() * 4 + self.y_host.numel() * 4) * world
        self.d2h_bytes = 4 * world
        # More than one rank: a rank's share of the step is short next to the host's cost of
        # enqueuing it (op nodes, graph walk, collectives: about 1.8 ms against 1.3 ms of device
        # work at 8 ranks), so the step is replayed as one CUDA graph, collectives included
        # (the library's CapturedStep). ENDIA_B200_BENCH_GRAPH=0 enqueues it op by op.
        self.captured, self.capture_error = None, None
        if world > 1 and data_parallel and os.environ.get("ENDIA_B200_BENCH_GRAPH", "1") != "0":
            from endia_b200.utils.general import CapturedStep
            try:
                self.captured = CapturedStep(self._device_step, warmup=3, optimizers=[self.opt])
            except Exception as exc:      # e.g. a collective that cannot be captured on this system
                self.capture_error = "%s: %s" % (type(exc).__name__, str(exc)[:200])

    def reset(self):
        """Back to the seeded weights, zero moments and t = 1 (the state the parity step starts from)."""
        from endia_b200._array import drop_operand_parts, stream
        torch = self.torch
        for w, h in zip(self.W, self.Ws_host):
            self.ndist.flat_tensor(w).copy_(torch.from_numpy(h).reshape(-1))
            parts = getattr(w, "_pair16", None)
            if self.captured is not None and parts is not None:
                # the captured step reads the weights' GEMM operand parts from this very buffer
                self.nd._lib.call("endia_b200_bf16_split", w.data_ptr(), parts.data_ptr(), w.size(), stream())
            else:
                drop_operand_parts(w)
        for b in self.B:
            self.ndist.flat_tensor(b).zero_()
        self.opt.reset_state()
        torch.cuda.synchronize()

    def _device_step(self, X=None, Y=None):
        nd = self.nd
        pred = nd.nn.mlp([self.X if X is None else X, None] + self.params, activation="tanh")
        loss = nd.mse(pred, self.Y if Y is None else Y)
        loss.backward()
        if self.reducer is not None:
            self.reducer.wait()
        self.opt.step()
        loss.zero_grad()
        return loss

    def step(self, host_io=False):
        if self.captured is not None:
            # the graph reads the batch from fixed arrays: the step's batch is copied into them first
            flat = self.ndist.flat_tensor
            if host_io:
                # the batch comes from pinned host memory on a copy stream while the previous step
                # computes (two staging sets); a device-to-device copy then fills the graph's inputs
                if self.feeder is None:
                    from endia_b200.utils.general import HostBatchFeeder
                    self.feeder = HostBatchFeeder([self.x_host, self.y_host], [self.X.shape(), self.Y.shape()])
                Xs, Ys = self.feeder.next()
                flat(self.X).copy_(flat(Xs), non_blocking=True)
                flat(self.Y).copy_(flat(Ys), non_blocking=True)
            loss = self.captured()
            if host_io:
                self.feeder.prefetch()
                self.loss_host.copy_(flat(loss), non_blocking=True)
                self.torch.cuda.current_stream().synchronize()
                return float(self.loss_host[0])
            return loss
        X, Y = self.X, self.Y
        if host_io:
            # every step's batch comes from pinned host memory; its copy runs on a copy stream
            # while the previous step computes (two sets of device input arrays)
            if self.feeder is None:
                from endia_b200.utils.general import HostBatchFeeder
                self.feeder = HostBatchFeeder([self.x_host, self.y_host], [self.X.shape(), self.Y.shape()])
            X, Y = self.feeder.next()
        loss = self._device_step(X, Y)
        if host_io:
            self.feeder.prefetch()
            self.loss_host.copy_(self.ndist.flat_tensor(loss), non_blocking=True)
            self.torch.cuda.current_stream().synchronize()
            return float(self.loss_host[0])
        return loss


class FFTStep:
    """c4: 32 signals of 2^20 points, loss = sum(|fft(x)|^2) * 2^-20, forward + VJP w.r.t. x.
    c5: 512^3 grid, loss = sum(real(fftn(x)) * w), forward + VJP; over N ranks the grid is split
    along axis 0 (slab decomposition, one exchange per transform). Rank r's slab is drawn from
    seed r, so that any rank can rebuild the whole grid."""

    def __init__(self, nd, torch, workload, rank, world):
        self.nd, self.torch, self.workload, self.rank, self.world = nd, torch, workload, rank, world
        if workload == "c4":
            r = np.random.Generator(np.random.PCG64(0))
            self.shape = (32, 1 << 20)
            x = self.crandn(r, self.shape)
            self.W = None
        else:
            n = 512
            self.shape = (n, n, n)
            x, w = self.c5_slab(rank, world)
            # w is split like the result: along axis 1 when the transform is slab-decomposed
            self.W = nd.Array(w)
        self.samples = None
        self.alg_bytes = 4.0 * 8.0 * float(np.prod(self.shape))
        self.x_host = torch.from_numpy(x).pin_memory()
        self.X = nd.Array(x, requires_grad=True)
        self.loss_host = torch.empty(1, dtype=torch.float32).pin_memory()
        self.h2d_bytes = int(self.x_host.numel() * 8) * world
        self.d2h_bytes = 4 * world
        self.last_y = None
        # One rank: the step is a handful of launches whose host cost (op nodes, graph walk) is
        # comparable to the transforms themselves at c4's size, so it is replayed as one CUDA graph
        # (the library's CapturedStep), like c3. ENDIA_B200_BENCH_GRAPH=0 enqueues it op by op.
        self.captured = None
        if world == 1 and os.environ.get("ENDIA_B200_BENCH_GRAPH", "1") != "0":
            from endia_b200.utils.general import CapturedStep
            self.captured = CapturedStep(self._eager)

    @staticmethod
    def crandn(r, shape):
        return (r.standard_normal(shape, dtype=np.float32)
                + 1j * r.standard_normal(shape, dtype=np.float32)).astype(np.complex64)

    @classmethod
    def c5_slab(cls, rank, world, n=512):
        """x[rank*n/P : (rank+1)*n/P, :, :] and w[:, rank*n/P : (rank+1)*n/P, :] of the c5 grid."""
        r = np.random.Generator(np.random.PCG64(1000 + rank))
        x = cls.crandn(r, (n // world, n, n))
        w = r.uniform(-1, 1, (n, n // world, n)).astype(np.float32)
        return x, w

    def step(self, host_io=False):
        nd, torch = self.nd, self.torch
        from endia_b200.dist import flat_tensor
        if host_io:
            flat_tensor(self.X).copy_(torch.view_as_real(self.x_host).reshape(-1), non_blocking=True)
        dx = self.captured() if self.captured is not None else self._eager()
        if host_io:
            self.loss_host.copy_(flat_tensor(self.last_loss), non_blocking=True)
            torch.cuda.current_stream().synchronize()
        return dx

    def _eager(self):
        nd = self.nd
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
        self.last_y, self.last_loss = y, loss
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
        self.host = (Ws, bs, x, y)
        self.x_host, self.y_host = torch.from_numpy(x).pin_memory(), torch.from_numpy(y).pin_memory()
        self.W = [nd.Array(w, requires_grad=True) for w in Ws]
        self.B = [nd.Array(b, requires_grad=True) for b in bs]
        self.params = [p for wb in zip(self.W, self.B) for p in wb]
        self.X, self.Y = nd.Array(x), nd.Array(y)
        self.opt = nd.optim.Adam(self.params, lr=1e-3)
        self.loss_host = torch.empty(1, dtype=torch.float32).pin_memory()
        self.samples = self.batch
        self.flops = 1.614e6
        self.h2d_bytes, self.d2h_bytes = int(self.x_host.numel() * 4 + self.y_host.numel() * 4), 4

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
        self.host = (Ws, x)
        self.x_host = torch.from_numpy(x).pin_memory()
        self.W = [nd.Array(w, requires_grad=True) for w in Ws]
        self.B = [nd.Array([self.dims[i + 1]], requires_grad=True) for i in range(3)]
        self.X = nd.Array(x, requires_grad=True)
        self.loss_host = torch.empty(1, dtype=torch.float32).pin_memory()
        self.samples = self.batch
        self.flops = 62.32e9
        self.h2d_bytes, self.d2h_bytes = int(self.x_host.numel() * 4), 4
        # The step is about 85 short launches: replayed as one CUDA graph (the library's
        # CapturedStep) it is bound by the GPU instead of the host. ENDIA_B200_BENCH_GRAPH=0 runs
        # it op by op.
        self.captured = None
        self.feeder = None
        if os.environ.get("ENDIA_B200_BENCH_GRAPH", "1") != "0":
            from endia_b200.utils.general import CapturedStep
            self.captured = CapturedStep(self._eager)

    def step(self, host_io=False):
        from endia_b200.dist import flat_tensor
        if host_io:
            # the batch is staged from pinned host memory on a copy stream while the previous step
            # computes; a device-to-device copy then fills the step's (fixed) input array
            if self.feeder is None:
                from endia_b200.utils.general import HostBatchFeeder
                self.feeder = HostBatchFeeder([self.x_host], [self.X.shape()])
            flat_tensor(self.X).copy_(flat_tensor(self.feeder.next()[0]), non_blocking=True)
        loss, grads = self.captured() if self.captured is not None else self._eager()
        if host_io:
            self.feeder.prefetch()
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


# ------------------------------------------------------------------------------ CPU baselines
def _oracle():
    from oracle import endia_oracle as eo
    eo.build()
    eo.config["mode"] = "faithful"
    return eo


class C2CpuSampler:
    """Endia's CPU algorithm for the c2 step (the oracle port, faithful mode: single-threaded
    dot-product matmul with a materialised transposed rhs, one temporary per op, Adam as array
    expressions) on bounded samples. The forward+backward time is linear in the batch rows with a
    fixed part (the transposing copies of the weights do not depend on the batch), so it is timed
    at two row counts and the full batch is the straight line through them; the Adam step is
    elementwise and is timed on 1/`adam_frac` of the rows of every weight matrix."""

    def __init__(self, rows_small=8, rows_large=40, adam_frac=16):
        self.eo = _oracle()
        self.rows = (int(rows_small), int(rows_large))
        self.adam_frac = adam_frac
        self.r, Ws = make_weights(0)
        eo = self.eo
        self.W = [eo.Array(w, requires_grad=True) for w in Ws]
        self.B = [eo.Array(np.zeros(DIMS[i + 1], np.float32), requires_grad=True) for i in range(len(DIMS) - 1)]
        self.t_rows = {self.rows[0]: [], self.rows[1]: []}
        self.t_adam = []
        self.seconds = 0.0

    def fwd_bwd(self, rows):
        eo = self.eo
        for p in self.W + self.B:
            p.remove_grad()
        x = self.r.standard_normal((rows, DIMS[0])).astype(np.float32)
        y = self.r.standard_normal((rows, DIMS[-1])).astype(np.float32)
        t0 = time.perf_counter()
        loss = eo.mse(eo.mlp_forward(eo.Array(x), self.W, self.B, "tanh"), eo.Array(y))
        loss.backward()
        dt = time.perf_counter() - t0
        self.t_rows[rows].append(dt)
        self.seconds += dt
        return dt

    def adam(self):
        """Adam.step on the leading 1/adam_frac rows of every weight (and the whole biases), with
        the gradients the last backward left; scaled to all parameters."""
        eo = self.eo
        parts, n_part, n_all = [], 0, 0
        for p in self.W + self.B:
            full = p.v
            k = max(1, full.shape[0] // self.adam_frac) if full.ndim == 2 else full.shape[0]
            q = eo.Array(np.ascontiguousarray(full[:k]), requires_grad=True)
            g = p.grad().v.reshape(full.shape if full.ndim == 2 else (1,) + full.shape)
            q.grad_(eo.Array(np.ascontiguousarray(g[:k] if full.ndim == 2 else g)))
            parts.append(q)
            n_part += q.size()
            n_all += p.size()
        opt = eo.Adam(parts)
        t0 = time.perf_counter()
        opt.step()
        dt = time.perf_counter() - t0
        self.seconds += dt
        self.t_adam.append(dt * n_all / n_part)
        for p in self.W + self.B:
            p.remove_grad()

    def sample(self, which):
        """One bounded sample: forward+backward at one of the two row counts (0 = small, 1 = large,
        2 = both) and the Adam fraction."""
        for i in ((0, 1) if which == 2 else (which,)):
            self.fwd_bwd(self.rows[i])
        self.adam()

    def clear(self):
        self.t_rows = {self.rows[0]: [], self.rows[1]: []}
        self.t_adam = []

    def result(self):
        r0, r1 = self.rows
        t0, t1 = float(np.mean(self.t_rows[r0])), float(np.mean(self.t_rows[r1]))
        # (timing noise on a busy host can make the two samples nearly equal: the slope is kept at
        # no less than a tenth of the proportional estimate t1 / r1)
        slope = max((t1 - t0) / (r1 - r0), 0.1 * t1 / r1)
        fixed = max(t0 - slope * r0, 0.0)
        adam = float(np.mean(self.t_adam))
        full = fixed + slope * GLOBAL_BATCH + adam
        return {"value": GLOBAL_BATCH / full, "unit": UNIT, "cores": 1, "kind": "port",
                "extrapolated": True,
                "extrapolation": {"model": "seconds(fwd+bwd) = fixed + per_row * rows, fitted at the two row counts; "
                                           "Adam scaled by the fraction of parameters it ran on",
                                  "rows": [r0, r1], "seconds_at_rows": [t0, t1], "fixed_s": fixed,
                                  "per_row_s": slope, "adam_full_s": adam, "factor_rows": GLOBAL_BATCH / float(r1),
                                  "adam_fraction": 1.0 / self.adam_frac, "full_step_s": full},
                "sample": "%d and %d of 8192 batch rows through the full 1024-4096-4096-4096-1024 network, "
                          "Adam on 1/%d of the parameters; the reference's matmul is single-threaded "
                          "(matmul_op.mojo:168-169)" % (r0, r1, self.adam_frac),
                "host_cores_available": os.cpu_count(), "seconds": self.seconds}


def cpu_baseline_c2():
    s = C2CpuSampler()
    s.sample(2)
    return s.result()


def cpu_baseline_c1():
    """The c1 step in the oracle port at full size (faithful mode), three steps."""
    eo = _oracle()
    r = np.random.Generator(np.random.PCG64(0))
    d = SmallStep.dims
    W, B = [], []
    for i in range(4):
        lim = np.sqrt(6.0 / d[i])
        W.append(eo.Array(r.uniform(-lim, lim, (d[i], d[i + 1])).astype(np.float32), requires_grad=True))
        B.append(eo.Array(r.uniform(-lim, lim, (d[i + 1],)).astype(np.float32), requires_grad=True))
    x = r.uniform(0, 1, (128, 1)).astype(np.float32)
    y = np.sin(np.float32(15) * x).astype(np.float32)
    params = [p for wb in zip(W, B) for p in wb]
    opt = eo.Adam(params)
    n, t0 = 3, time.perf_counter()
    for _ in range(n):
        loss = eo.mse(eo.mlp_forward(eo.Array(x), W, B, "relu"), eo.Array(y))
        loss.backward()
        opt.step()
        for p in params:
            p.remove_grad()
    dt = (time.perf_counter() - t0) / n
    return {"value": 128 / dt, "unit": UNIT, "cores": 1, "kind": "port", "seconds": dt * n,
            "sample": "the full c1 step, %d steps; numpy-driven port, so the interpreter's per-op cost is "
                      "included (the compiled reference has none)" % n,
            "host_cores_available": os.cpu_count()}


def cpu_baseline_c3(rows=96):
    """The c3 step in the oracle port (faithful mode) on `rows` of the 4096 batch rows; every term
    of the loss is a per-sample sum, so the time is scaled by rows."""
    eo = _oracle()
    d = PenaltyStep.dims
    r = np.random.Generator(np.random.PCG64(0))
    W = [eo.Array(r.uniform(-np.sqrt(6.0 / d[i]), np.sqrt(6.0 / d[i]), (d[i], d[i + 1])).astype(np.float32),
                  requires_grad=True) for i in range(3)]
    B = [eo.Array(np.zeros(d[i + 1], np.float32), requires_grad=True) for i in range(3)]
    X = eo.Array(r.standard_normal((rows, d[0])).astype(np.float32), requires_grad=True)
    t0 = time.perf_counter()
    f = eo.mlp_forward(X, W, B, "tanh")
    gx = eo.grad(outs=[eo.sum(f)], inputs=[X], create_graph=True)[0]
    loss = eo.mean(f, [0, 1]) + 0.1 * (eo.sum(gx * gx) / float(rows))
    eo.grad(outs=[loss], inputs=W + B)
    dt = time.perf_counter() - t0
    full = dt * PenaltyStep.batch / rows
    return {"value": PenaltyStep.batch / full, "unit": UNIT, "cores": 1, "kind": "port", "extrapolated": True,
            "sample": "%d of 4096 batch rows in %.2f s, scaled x%.1f" % (rows, dt, PenaltyStep.batch / rows),
            "host_cores_available": os.cpu_count(), "seconds": dt}


def cpu_baseline_fft(workload):
    """Endia's CPU algorithm for the FFT configs (oracle port: float64 radix-2 with per-axis
    gathers, rows spread over the host threads as the reference's parallelize does), forward + VJP,
    on a bounded sample: c4 on 4 of the 32 signals, c5 on a 256^3 grid (scaled by points*log2)."""
    eo = _oracle()
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
    return {"value": alg / full_s / 1e9, "unit": "GB/s", "cores": threads, "kind": "port", "extrapolated": True,
            "sample": "%s forward+VJP on shape %s in %.2f s, scaled by n*log2(n) to the full size" % (
                workload, list(shape), dt), "host_cores_available": os.cpu_count(), "seconds": dt}


CPU_BASELINES = {"c1": cpu_baseline_c1, "c2": cpu_baseline_c2, "c3": cpu_baseline_c3,
                 "c4": lambda: cpu_baseline_fft("c4"), "c5": lambda: cpu_baseline_fft("c5")}


def run_reference(args):
    """The reference arm: Endia's own CPU implementation of the path cannot be built here (Mojo), so
    the oracle port is timed on the host cores. Every step is one bounded sample of the c2 step
    (alternating between the two row counts of the straight-line fit; a single step runs both)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    world = max(1, args.gpus)
    wl = "c2" if args.workload == "all" else args.workload
    if wl != "c2":
        base = CPU_BASELINES[wl]()
        fft = wl in ("c4", "c5")
        line = {"impl": "reference", "metric": FFT_METRIC if fft else METRIC, "value": base["value"],
                "unit": base["unit"], "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": None, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                "dtype": "c64" if fft else "f32", "data": "synthetic", "config": workload_config(wl, world),
                "cpu_baseline": base, "extrapolated": bool(base.get("extrapolated")),
                "e2e": {"value": base["value"], "unit": base["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line))
        return
    s = C2CpuSampler(args.cpu_rows, 5 * args.cpu_rows)
    total = args.warmup + args.steps
    for i in range(total):
        if i == args.warmup:
            s.clear()
        s.sample(2 if args.steps == 1 else (i - args.warmup) % 2)
    base = s.result()
    value = base["value"]
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1000.0 * GLOBAL_BATCH / value,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic", "config": workload_config("c2", world),
            "extrapolated": True, "extrapolation": base["extrapolation"],
            "cpu_baseline": base,
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    if args.workload == "all":
        subs = {}
        for name in ("c1", "c3", "c4", "c5"):
            b = CPU_BASELINES[name]()
            subs[name] = {"metric": FFT_METRIC if name in ("c4", "c5") else METRIC, "value": b["value"],
                          "unit": b["unit"], "config": workload_config(name, 1), "cpu_baseline": b}
        line["workloads"] = subs
    print(json.dumps(line))


# ------------------------------------------------------------------------------ timed regions
class Context:
    def __init__(self, args):
        import torch
        import endia_b200 as nd
        from endia_b200 import _lib, dist as ndist
        import torch.distributed as tdist
        self.torch, self.nd, self._lib, self.ndist, self.tdist = torch, nd, _lib, ndist, tdist
        self.args = args
        # The launcher can state the SM split between NCCL and the persistent GEMM grid (see
        # dist.init_process_group); by default neither is limited.
        self.comm_limits = {"nccl_max_ctas": args.nccl_max_ctas, "gemm_reserve_sms": args.reserve_sms}
        self.rank, self.world = ndist.init_process_group(**self.comm_limits)
        nd._array.device()
        self.pk = peaks()
        self._flush = None

    def barrier(self):
        if self.world > 1:
            self.tdist.barrier()
        self.torch.cuda.synchronize()

    def flush_l2(self):
        """Write a 256 MiB buffer (larger than the 126 MB L2)."""
        if self._flush is None:
            self._flush = self.torch.empty(64 << 20, dtype=self.torch.float32, device="cuda")
        self._flush.zero_()

    def max_over_ranks(self, values):
        t = self.torch.tensor(values, dtype=self.torch.float64, device="cuda")
        if self.world > 1:
            self.tdist.all_reduce(t, op=self.tdist.ReduceOp.MAX)
        return [float(v) for v in t.cpu()]


def timed_region(ctx, work, steps, warmup, flush=False, e2e_steps=None):
    """W untimed steps, then K steps between barriers timed with CUDA events on the launching
    stream (device-resident inputs), then the same K steps end to end through host buffers. With
    `flush` every timed step is bracketed by its own events and a buffer larger than L2 is written
    between steps (outside the events)."""
    torch, nd, lib = ctx.torch, ctx.nd, ctx._lib.lib
    for _ in range(warmup):
        work.step()
    ctx.barrier()
    sampler = ClockSampler(torch.cuda.current_device())
    timer = CallTimer(torch)
    nd.config.gemm_timer = timer
    nd.config.fft_timer = timer
    cap = getattr(work, "captured", None)
    launches0 = lib.endia_b200_launch_count()
    replays0 = getattr(cap, "replays", 0)
    sampler.start()
    ctx.barrier()
    host_s = 0.0
    if flush:
        pairs = []
        for _ in range(steps):
            ctx.flush_l2()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            work.step()
            b.record()
            pairs.append((a, b))
        ctx.barrier()
        ms_total = sum(a.elapsed_time(b) for a, b in pairs)
    else:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        t0 = time.perf_counter()
        for _ in range(steps):
            work.step()
        host_s = time.perf_counter() - t0     # host time to enqueue the steps (no synchronisation inside)
        e1.record()
        ctx.barrier()
        ms_total = e0.elapsed_time(e1)
    clocks = sampler.stop()
    nd.config.gemm_timer = None
    nd.config.fft_timer = None
    launches = lib.endia_b200_launch_count() - launches0
    if cap is not None:   # kernels replayed inside a CUDA graph are not seen by the enqueue counter
        launches += cap.launches_per_replay * (cap.replays - replays0)
    n_calls, call_work, call_ms = timer.summary()
    # ---- end to end through the public API with host buffers
    n_e2e = steps if e2e_steps is None else e2e_steps
    for _ in range(2):
        work.step(host_io=True)
    ctx.barrier()
    e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2.record()
    for _ in range(n_e2e):
        work.step(host_io=True)
    e3.record()
    ctx.barrier()
    ms_e2e = e2.elapsed_time(e3) / n_e2e
    ms_total, ms_e2e, call_ms = ctx.max_over_ranks([ms_total, ms_e2e, call_ms])
    return {"ms_step": ms_total / steps, "ms_e2e_step": ms_e2e, "n_calls": n_calls, "call_work": call_work,
            "call_ms": call_ms, "launches": int(launches), "host_ms_step": 1000.0 * host_s / steps,
            "clocks": {"sm_mhz": clocks["sm_mhz"], "sm_max_mhz": clocks["sm_max_mhz"],
                       "reasons": clocks["reasons"], "samples": clocks["samples"]}}


def tc_scheme(gemm_flag):
    """Scheme the two-CTA tcgen05 kernel runs for this --gemm flag (mirrors the library's choice)."""
    if gemm_flag == "3xtf32" or (gemm_flag == "auto" and os.environ.get("ENDIA_B200_TC_SCHEME", "")[:1] in ("3", "0")):
        return "3xtf32"
    return "tf32_bf16x2"


GEMM_ALGOS = {"auto": "GEMM_AUTO", "ffma": "GEMM_FFMA", "3xtf32": "GEMM_3XTF32", "tf32_bf16x2": "GEMM_TF32_BF16X2"}


def c2_parity(ctx, work):
    """One step from the seeded weights on all ranks against the same step done by rank 0 alone on
    the whole batch: relative differences of the loss, of the weight UPDATE (w_new - w_seed, the
    quantity the step computes) and of the updated weights themselves, max over the tensors."""
    torch, tdist, flat = ctx.torch, ctx.tdist, ctx.ndist.flat_tensor
    work.reset()
    loss = work.step()
    lt = flat(loss).clone()
    tdist.all_reduce(lt)                      # global-mean loss = mean of the ranks' local means
    loss_dp = float(lt.item()) / ctx.world
    got = [flat(p).clone() for p in work.params]
    ctx.barrier()
    out = None
    if ctx.rank == 0:
        one = TrainStep(ctx.nd, torch, 0, 1, data_parallel=False)
        seed = [flat(p).clone() for p in one.params]
        loss_1 = float(flat(one.step()).item())
        torch.cuda.synchronize()
        upd_rel = w_rel = 0.0
        for a, p, s in zip(got, one.params, seed):
            b = flat(p)
            du = (b - s).double().norm().item()
            if du > 0:
                upd_rel = max(upd_rel, (a - b).double().norm().item() / du)
            nb = b.double().norm().item()
            if nb > 0:
                w_rel = max(w_rel, (a - b).double().norm().item() / nb)
        out = {"loss_rel": abs(loss_dp - loss_1) / abs(loss_1), "update_rel_l2": upd_rel, "w_rel_l2": w_rel,
               "against": "the same step on one rank with the whole batch", "ok": bool(
                   abs(loss_dp - loss_1) <= 1e-4 * abs(loss_1) and upd_rel < 1e-3),
               "note": "Adam's first step moves every weight by about lr * sign(g): entries whose gradient is "
                       "within rounding of zero take the other sign in a different summation order, which "
                       "bounds update_rel_l2 from below"}
        del one
    ctx.barrier()
    return out


def c5_parity(ctx, work):
    """The slab-decomposed forward and VJP of this rank against one rank transforming the whole grid
    (rank 0 rebuilds all slabs from their seeds): relative L2 of rank 0's slabs of y and dx."""
    torch, flat = ctx.torch, ctx.ndist.flat_tensor
    dx = work.step()
    y = work.last_y
    ctx.barrier()
    out = None
    if ctx.rank == 0:
        n, P = 512, ctx.world
        xs, ws = zip(*[FFTStep.c5_slab(r, P) for r in range(P)])
        X = ctx.nd.Array(np.concatenate(xs, axis=0), requires_grad=True)
        W = ctx.nd.Array(np.concatenate(ws, axis=1))
        Y = ctx.nd.fftn(X)
        ctx.nd.sum(ctx.nd.real(Y) * W).backward()
        yt = torch.view_as_complex(flat(Y).view(n, n, n, 2))[:, :n // P, :]
        gt = torch.view_as_complex(flat(X.grad()).view(n, n, n, 2))[:n // P]
        ys = torch.view_as_complex(flat(y).view(n, n // P, n, 2))
        gs = torch.view_as_complex(flat(dx).view(n // P, n, n, 2))
        y_rel = ((ys - yt).abs().double().norm() / yt.abs().double().norm()).item()
        g_rel = ((gs - gt).abs().double().norm() / gt.abs().double().norm()).item()
        out = {"y_rel_l2": y_rel, "dx_rel_l2": g_rel, "against": "fftn of the whole grid on one rank",
               "ok": bool(y_rel < 1e-5 and g_rel < 1e-5)}
    ctx.barrier()
    return out


def bench_c2(ctx, steps, warmup, gemm="auto", with_cpu=True, with_parity=True):
    nd, lib = ctx.nd, ctx._lib
    nd.config.gemm_algo = getattr(lib, GEMM_ALGOS[gemm])
    work = TrainStep(nd, ctx.torch, ctx.rank, ctx.world)
    # More than one rank: the first steps also set up NCCL's channels and buffers for each message
    # size (seen as a slow first ten steps on 8 GPUs), so at least ten untimed steps are run.
    t = timed_region(ctx, work, steps, max(warmup, 10) if ctx.world > 1 else warmup)
    if work.captured is not None:
        # a replayed graph has no per-call events: the GEMM calls are timed in three steps enqueued
        # op by op on every rank
        timer = CallTimer(ctx.torch)
        nd.config.gemm_timer = timer
        for _ in range(3):
            work._device_step()
        ctx.barrier()
        nd.config.gemm_timer = None
        t["n_calls"], t["call_work"], call_ms = timer.summary()
        t["call_ms"] = ctx.max_over_ranks([call_ms])[0]
        t["call_steps"] = 3
    parity = c2_parity(ctx, work) if (ctx.world > 1 and with_parity) else None
    nd.config.gemm_algo = lib.GEMM_AUTO
    if ctx.rank != 0:
        return None
    pk = ctx.pk
    world = ctx.world
    value = GLOBAL_BATCH / (t["ms_step"] / 1000.0)
    tflops = t["call_work"] / (t["call_ms"] / 1000.0) / 1e12 if t["call_ms"] > 0 else 0.0
    tc = bool(lib.lib.endia_b200_has_tcgen05()) and gemm != "ffma"
    # Tensor-core time per logical product in units of one bf16 MMA: 3xTF32 issues three tf32 MMAs
    # (tf32 runs at half the bf16 rate) = 6; the bf16-compensated scheme one tf32 and two bf16 = 4.
    # The ceiling for logical flops is the measured bf16 throughput divided by that.
    bf16c = tc_scheme(gemm) == "tf32_bf16x2"
    peak = pk["bf16_tflops_sustained"] / (4.0 if bf16c else 6.0)
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": steps,
        "warmup": warmup, "ms_per_step": t["ms_step"], "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": workload_config("c2", world),
        "implementation": {
            "gemm": ("tcgen05, one tf32 MMA + two bf16 correction MMAs per product (fp32 accumulate, "
                     "error <= 2.3e-6 of |a||b|)" if bf16c else "tcgen05 3xTF32 (fp32 accumulate)") if tc else "fp32 FFMA",
            "data_parallel": work.dp_mode + (
                "" if work.dp_mode != "sharded" else
                (" (per-layer chains beside the backward pass: reduce-scatter, Adam on 1/P, " + (
                    "all-gather by the copy engines into peer memory)" if getattr(work.opt, "_inbox", None) is not None
                    else "NCCL all-gather)") if getattr(work.opt, "pipelined", False)
                 else " (reduce-scatter, one Adam launch on 1/P, NCCL all-gather before use)")),
            "launch": ("one CUDA graph per step, collectives included (%d kernels of this library); "
                       "ENDIA_B200_BENCH_GRAPH=0 enqueues it op by op" % work.captured.launches_per_replay)
            if work.captured is not None else ("op by op" + (
                " (graph capture failed: %s)" % work.capture_error if work.capture_error else "")),
            "comm_limits": {"NCCL_MAX_CTAS": os.environ.get("NCCL_MAX_CTAS"),
                            "ENDIA_B200_TC_RESERVE_SMS": os.environ.get("ENDIA_B200_TC_RESERVE_SMS")} if world > 1 else None,
            "e2e_io": "each step's batch is copied from pinned host memory on a copy stream while the "
                      "previous step computes; the loss is read back every step"},
        "clocks": t["clocks"],
        "e2e": {"value": GLOBAL_BATCH / (t["ms_e2e_step"] / 1000.0), "unit": UNIT,
                "h2d_bytes_per_step": work.h2d_bytes, "d2h_bytes_per_step": work.d2h_bytes},
        "gpu_launches": t["launches"],
        "host_enqueue_ms_per_step": t["host_ms_step"],
        "roofline": {"bound": "tensor", "achieved": tflops, "peak": peak, "unit": "TFLOP/s",
                     "frac": tflops / peak if peak else None,
                     # dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant GEMM shape
                     # (8192 x 4096 x 4096, the forward and dX products of the 4096-wide layers), from
                     # the committed ncu capture; the other shapes of the step were not captured
                     "traffic": (1.37e9 if bf16c else 1.49e9) if (tc and world == 1) else None,
                     "traffic_note": "bytes per launch of gemm_tc2p_kernel at 8192x4096x4096 from one ncu capture "
                                     "(a product without an epilogue; 1.77e9 with bias + tanh + the bf16 operand "
                                     "parts of the output in the epilogue, 0.78e9 compulsory); compulsory 0.51e9",
                     "kernel": "gemm (%d launches per step, %.3f ms of the %.3f ms step)" % (
                         t["n_calls"] // t.get("call_steps", steps), t["call_ms"] / t.get("call_steps", steps),
                         t["ms_step"]),
                     "peak_note": ("%s bf16_tflops_sustained %.1f / 4 (one tf32 MMA = 2 bf16 MMA times, plus two "
                                   "bf16 MMAs per product)" if bf16c else
                                   "%s bf16_tflops_sustained %.1f / 2 (tf32 rate) / 3 (MMAs per 3xTF32 product)") % (
                         pk["source"], pk["bf16_tflops_sustained"]),
                     "frac_of_3xtf32_ceiling": tflops / (pk["bf16_tflops_sustained"] / 6.0),
                     "frac_of_bf16_%s" % pk["source"]: tflops / pk["bf16_tflops_sustained"],
                     "algorithmic_gflop_per_step": gemm_flops(GLOBAL_BATCH) / 1e9 / world},
    }
    if parity is not None:
        line["parity"] = parity
    if world == 1 and with_cpu:
        line["cpu_baseline"] = cpu_baseline_c2()
    return line


def bench_small(ctx, name, steps, warmup, with_cpu=True):
    """c1 / c3 (one GPU; 'replicas only' by the configurations' definition)."""
    nd, torch = ctx.nd, ctx.torch
    work = SmallStep(nd, torch) if name == "c1" else PenaltyStep(nd, torch)
    t = timed_region(ctx, work, steps, warmup, flush=(name == "c3"))
    if ctx.rank != 0:
        return None
    pk = ctx.pk
    ms = t["ms_step"]
    cap = getattr(work, "captured", None)
    line = {"metric": METRIC if name == "c1" else "gradient-penalty step samples/s (fwd + double backward)",
            "value": work.samples / (ms / 1000.0), "unit": UNIT, "n_gpus": 1, "steps": steps, "warmup": warmup,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "replicas only", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic", "config": workload_config(name, 1), "clocks": t["clocks"],
            "e2e": {"value": work.samples / (t["ms_e2e_step"] / 1000.0), "unit": UNIT,
                    "h2d_bytes_per_step": work.h2d_bytes, "d2h_bytes_per_step": work.d2h_bytes},
            "gpu_launches": t["launches"],
            "host_enqueue_ms_per_step": t["host_ms_step"] if name == "c1" else None}
    if name == "c1":
        line["implementation"] = {"launch": "the whole step is one kernel launch (nn.fused_train_step)"}
        line["roofline"] = {"bound": "latency", "achieved": None, "peak": None, "unit": None, "frac": None,
                            "traffic": None, "note": "1.6 MFLOP per step: bound by launch latency, no roofline quoted"}
    else:
        peak = pk["bf16_tflops_sustained"] / 6.0
        ach = work.flops / (ms / 1000.0) / 1e12
        line["implementation"] = {"launch": ("one CUDA graph per step (%d kernels); ENDIA_B200_BENCH_GRAPH=0 runs it "
                                             "op by op" % cap.launches_per_replay) if cap is not None else "op by op",
                                  "note": "create_graph=True path: every VJP is a composition of ops"}
        line["roofline"] = {"bound": "tensor", "achieved": ach, "peak": peak, "unit": "TFLOP/s", "frac": ach / peak,
                            "traffic": None, "kernel": "whole step (algorithmic flops / step time)",
                            "algorithmic_gflop_per_step": work.flops / 1e9,
                            "peak_note": "%s bf16_tflops_sustained %.1f / 6 (3xTF32 ceiling)" % (
                                pk["source"], pk["bf16_tflops_sustained"])}
    if with_cpu:
        line["cpu_baseline"] = CPU_BASELINES[name]()
    return line


def bench_fft(ctx, name, steps, warmup, with_cpu=True, with_parity=True):
    world = ctx.world if name == "c5" else 1
    work = FFTStep(ctx.nd, ctx.torch, name, ctx.rank if name == "c5" else 0, world)
    t = timed_region(ctx, work, steps, warmup, e2e_steps=min(steps, 5))
    parity = c5_parity(ctx, work) if (world > 1 and with_parity) else None
    if work.captured is not None:
        # a replayed graph has no per-call events: the transform calls are timed in three steps
        # enqueued op by op (CUDA events around each endia_b200_fft_c2c_fused call)
        timer = CallTimer(ctx.torch)
        ctx.nd.config.fft_timer = timer
        for _ in range(3):
            work._eager()
        ctx.torch.cuda.synchronize()
        ctx.nd.config.fft_timer = None
        t["n_calls"], t["call_work"], t["call_ms"] = timer.summary()
        t["call_steps"] = 3
    if ctx.rank != 0:
        return None
    pk = ctx.pk
    ms = t["ms_step"]
    hbm = pk["hbm_gbs"]
    ach = t["call_work"] / (t["call_ms"] / 1000.0) / 1e9 if t["call_ms"] > 0 else 0.0
    path = work.alg_bytes / (ms / 1000.0) / 1e9
    line = {"metric": FFT_METRIC, "value": path, "unit": "GB/s", "n_gpus": world, "steps": steps, "warmup": warmup,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "strong" if name == "c5" else "replicas only",
            "vs_baseline": None, "dtype": "c64", "data": "synthetic", "config": workload_config(name, world),
            "clocks": t["clocks"],
            "e2e": {"value": work.alg_bytes / (t["ms_e2e_step"] / 1000.0) / 1e9, "unit": "GB/s",
                    "h2d_bytes_per_step": work.h2d_bytes, "d2h_bytes_per_step": work.d2h_bytes},
            "gpu_launches": t["launches"], "host_enqueue_ms_per_step": t["host_ms_step"],
            "implementation": {
                "launch": ("one CUDA graph per step (%d kernels); ENDIA_B200_BENCH_GRAPH=0 runs it op by op"
                           % work.captured.launches_per_replay) if work.captured is not None else "op by op",
                "fusion": "loss term summed in the last pass of the forward transform, its gradient folded into "
                          "the scale of the VJP transform (ENDIA_B200_FFT_FUSE=0: every op a pass of its own)"},
            "roofline": {"bound": "hbm", "achieved": ach, "peak": hbm * world, "unit": "GB/s",
                         "frac": ach / (hbm * world) if hbm else None, "traffic": None,
                         "kernel": "fft calls (%d per step, %.3f ms per step); algorithmic bytes = one read + one "
                                   "write of the array per transform" % (
                                       t["n_calls"] // t.get("call_steps", steps),
                                       t["call_ms"] / t.get("call_steps", steps)),
                         "path_frac": path / (hbm * world),
                         "path_note": "value / peak: the whole forward+VJP on its 4S algorithmic bytes",
                         "peak_note": "%s hbm_gbs (copy)%s" % (pk["source"], " x %d GPUs" % world if world > 1 else "")}}
    if world > 1:
        n = 512
        line["exchange_bytes_per_gpu_per_transpose"] = 8 * n ** 3 // world * (world - 1) // world
    if parity is not None:
        line["parity"] = parity
    if world == 1 and with_cpu:
        line["cpu_baseline"] = CPU_BASELINES[name]()
    return line


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="endia_b200", choices=["endia_b200", "reference"])
    ap.add_argument("--cpu-rows", type=int, default=8,
                    help="reference arm: the smaller of the two batch-row counts of a c2 sample (the larger is 5x)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--gemm", default="auto", choices=["auto", "ffma", "3xtf32", "tf32_bf16x2"],
                    help="auto = tf32_bf16x2 on the two-CTA tcgen05 kernel (one tf32 MMA + two bf16 correction "
                         "MMAs per product), 3xTF32 split-K or FFMA where that kernel does not apply")
    ap.add_argument("--nccl-max-ctas", type=int, default=-1,
                    help="N > 1: NCCL_MAX_CTAS (0 or default: leave unset)")
    ap.add_argument("--reserve-sms", type=int, default=-1,
                    help="N > 1: SMs left out of the persistent GEMM grid for the collectives (0 or default: none)")
    ap.add_argument("--workload", default="all", choices=["all", "c1", "c2", "c3", "c4", "c5"],
                    help="all (default): the c2 line with the other configurations as sub-records; c2: MLP train "
                         "step alone; c1: small MLP, single-launch step; c3: gradient-penalty (second-order) step; "
                         "c4 / c5: FFT forward + VJP")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
        return
    if args.warmup < 3:
        args.warmup = 3
    # The SM split between NCCL and the persistent GEMM grid can be stated here; measured on the c2
    # step with the copy-engine all-gather, no limits are best: 4 ranks 2.13 ms against 2.19 ms with
    # 16 / 16, and 1.43 against 1.52 ms on the per-rank share of 8 ranks (1024 rows per rank).
    if args.nccl_max_ctas < 0:
        args.nccl_max_ctas = 0
    if args.reserve_sms < 0:
        args.reserve_sms = 0
    args.nccl_max_ctas = args.nccl_max_ctas or None
    args.reserve_sms = args.reserve_sms or None
    ctx = Context(args)
    cpu = not args.no_cpu_baseline
    K, W = args.steps, args.warmup
    wl = args.workload
    if wl in ("c1", "c3"):
        line = bench_small(ctx, wl, K, W, cpu)       # every rank runs its own replica
    elif wl in ("c4", "c5"):
        line = bench_fft(ctx, wl, K, W, cpu)
    else:
        line = bench_c2(ctx, K, W, args.gemm, cpu)
        if wl == "all":
            subs = {}
            if ctx.world == 1:
                if args.gemm == "auto":
                    alt = bench_c2(ctx, min(K, 10), 3, "3xtf32", with_cpu=False)
                    if alt is not None:
                        line["alt"] = {"gemm": "3xtf32", "ms_per_step": alt["ms_per_step"], "value": alt["value"],
                                       "unit": UNIT, "steps": alt["steps"], "roofline": alt["roofline"],
                                       "e2e": alt["e2e"], "clocks": alt["clocks"],
                                       "implementation": alt["implementation"]}
                subs["c1"] = bench_small(ctx, "c1", max(K, 100), W, cpu)
                subs["c3"] = bench_small(ctx, "c3", K, W, cpu)
                subs["c4"] = bench_fft(ctx, "c4", K, W, cpu)
                subs["c5"] = bench_fft(ctx, "c5", min(K, 10), W, cpu)
            else:
                sub = bench_fft(ctx, "c5", min(K, 10), max(W, 5), cpu)
                if sub is not None:
                    subs["c5"] = sub
                    subs["note"] = "c1, c3 and c4 are 'replicas only' at the sizes asked for: they are measured at --gpus 1"
            if line is not None:
                line["workloads"] = subs
    if ctx.rank == 0 and line is not None:
        print(json.dumps(line))
    if ctx.world > 1:
        ctx.tdist.destroy_process_group()


if __name__ == "__main__":
    main()
