"""Single-kernel cases through the C ABI, timed with CUDA events: the unit for micro-benchmarks and
for profiler captures (one kernel, a few launches, a few hundred MB on the device).

  python kernel_bench.py gemm --m 4096 --n 4096 --k 4096 --ta 0 --tb 0 --algo auto
  python kernel_bench.py fft --batch 32 --n 1048576
  python kernel_bench.py fftn --shape 256,256,256
  python kernel_bench.py ew --rows 8192 --cols 4096
  python kernel_bench.py adam --numel 41956352
  python kernel_bench.py actbwd --rows 8192 --cols 4096

Each case prints one JSON line: average milliseconds per call over --reps calls after --warmup,
and the achieved rate on the algorithmic bytes or flops of the call.
"""
import argparse
import ctypes as C
import json
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import endia_b200 as nd  # noqa: E402
from endia_b200 import _lib  # noqa: E402
from endia_b200._array import alloc, stream  # noqa: E402


def _time(fn, warmup, reps, flush=None):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(reps):
        if flush is not None:
            flush.zero_()            # evict L2 between timed calls
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    return total / reps


def _randn(shape, seed=0, complex_=False):
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    n = int(np.prod(shape)) * (2 if complex_ else 1)
    arr = nd.Array(list(shape), is_complex=complex_)
    arr.buf.copy_(torch.randn(n, generator=g, device="cuda", dtype=torch.float32))
    return arr


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=["gemm", "fft", "fftn", "ew", "adam", "actbwd", "reduce"])
    ap.add_argument("--m", type=int, default=4096)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--ta", type=int, default=0)
    ap.add_argument("--tb", type=int, default=0)
    ap.add_argument("--algo", default="auto", choices=["auto", "ffma", "3xtf32", "tf32_bf16x2"])
    ap.add_argument("--epi", default="none", help="gemm: none, or a '+' list of bias, tanh, parts")
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--shape", default="256,256,256")
    ap.add_argument("--rows", type=int, default=8192)
    ap.add_argument("--cols", type=int, default=4096)
    ap.add_argument("--numel", type=int, default=41956352)
    ap.add_argument("--inverse", type=int, default=0)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--flush", type=int, default=1, help="write a 256 MiB buffer between timed calls")
    a = ap.parse_args()
    nd._array.device()
    flush = torch.empty(64 << 20, dtype=torch.float32, device="cuda") if a.flush else None
    out = {"case": a.case}

    if a.case == "gemm":
        algo = {"auto": _lib.GEMM_AUTO, "ffma": _lib.GEMM_FFMA, "3xtf32": _lib.GEMM_3XTF32,
                "tf32_bf16x2": _lib.GEMM_TF32_BF16X2}[a.algo]
        A = _randn((a.k, a.m) if a.ta else (a.m, a.k), 1)
        B = _randn((a.n, a.k) if a.tb else (a.k, a.n), 2)
        Cc = nd.Array([a.m, a.n])
        epi = None
        if a.epi != "none":
            # the epilogue of a fused layer's forward product: bias, tanh and the operand parts of the
            # output; the operands come with their own parts, as they do inside a training step
            epi = _lib.Epilogue()
            epi.alpha, epi.beta = 1.0, 0.0
            keep = [_randn((a.n,), 12), alloc(a.m * a.n), alloc(a.m * a.k), alloc(a.k * a.n)]
            if "bias" in a.epi:
                epi.bias = keep[0].data_ptr()
            if "tanh" in a.epi:
                epi.act = _lib.ACT_TANH
            if "parts" in a.epi:
                epi.c16 = keep[1].data_ptr()
            if algo != _lib.GEMM_3XTF32 and algo != _lib.GEMM_FFMA:
                _lib.call("endia_b200_bf16_split", A.data_ptr(), keep[2].data_ptr(), a.m * a.k, stream())
                _lib.call("endia_b200_bf16_split", B.data_ptr(), keep[3].data_ptr(), a.k * a.n, stream())
                epi.a16, epi.b16 = keep[2].data_ptr(), keep[3].data_ptr()
            epi = C.byref(epi)

        def fn():
            _lib.call("endia_b200_gemm", a.ta, a.tb, a.m, a.n, a.k, A.data_ptr(), A.shape()[1],
                      B.data_ptr(), B.shape()[1], Cc.data_ptr(), a.n, 1, 0, 0, 0, epi, algo, stream())
        ms = _time(fn, a.warmup, a.reps, flush)
        out.update(m=a.m, n=a.n, k=a.k, ta=a.ta, tb=a.tb, algo=a.algo, epi=a.epi, ms=ms,
                   tflops=2.0 * a.m * a.n * a.k / ms / 1e9)
    elif a.case in ("fft", "fftn"):
        shape = (a.batch, a.n) if a.case == "fft" else tuple(int(s) for s in a.shape.split(","))
        dims = [len(shape) - 1] if a.case == "fft" else list(range(len(shape)))
        X = _randn(shape, 3, complex_=True)
        Y = nd.Array(list(shape), is_complex=True)
        cd = (C.c_int32 * len(dims))(*dims)
        nbytes = _lib.lib.endia_b200_fft_scratch_bytes(X.desc(), cd, len(dims))
        scratch = alloc(nbytes // 4 + 1) if nbytes else None

        def fn():
            _lib.call("endia_b200_fft_c2c", X.desc(), Y.desc(), cd, len(dims), a.inverse, 1.0,
                      scratch.data_ptr() if scratch is not None else None, stream())
        ms = _time(fn, a.warmup, a.reps, flush)
        s_bytes = 8.0 * np.prod(shape)
        out.update(shape=list(shape), ms=ms, algorithmic_gbs=2.0 * s_bytes / ms / 1e6,
                   note="algorithmic bytes = one read + one write of the array")
    elif a.case == "ew":
        X, Y = _randn((a.rows, a.cols), 4), _randn((a.cols,), 5)
        Z = nd.Array([a.rows, a.cols])
        Ye = nd.expand(Y, [a.rows, a.cols])

        def fn():
            _lib.call("endia_b200_ew_binary", _lib.BIN_ADD, X.desc(), Ye.desc(), Z.desc(), stream())
        ms = _time(fn, a.warmup, a.reps, flush)
        out.update(rows=a.rows, cols=a.cols, ms=ms, algorithmic_gbs=8.0 * a.rows * a.cols / ms / 1e6,
                   note="bias add: one read + one write of the [rows, cols] array")
    elif a.case == "adam":
        P, G, M, V = (_randn((a.numel,), s) for s in (6, 7, 8, 9))
        V.buf.abs_()
        ptr = lambda t: (C.c_void_p * 1)(t.data_ptr())
        numel = (C.c_int64 * 1)(a.numel)

        def fn():
            _lib.call("endia_b200_adam_step_multi", 1, ptr(P), ptr(G), ptr(M), ptr(V), numel, 1e-3, 0.9,
                      0.999, 1e-8, 1.0, 1.0, stream())
        ms = _time(fn, a.warmup, a.reps, flush)
        out.update(numel=a.numel, ms=ms, algorithmic_gbs=28.0 * a.numel / ms / 1e6,
                   note="7 floats per parameter: read p, g, m, v; write p, m, v")
    elif a.case == "actbwd":
        Aout, G = _randn((a.rows, a.cols), 10), _randn((a.rows, a.cols), 11)
        dS, db = nd.Array([a.rows, a.cols]), nd.Array([1, a.cols])
        sb = _lib.lib.endia_b200_act_bwd_colsum_scratch_bytes(a.rows, a.cols)
        scratch = alloc(sb // 4 + 1)

        def fn():
            _lib.call("endia_b200_act_bwd_colsum", _lib.ACT_TANH, Aout.data_ptr(), G.data_ptr(),
                      dS.data_ptr(), db.data_ptr(), a.rows, a.cols, scratch.data_ptr(), stream())
        ms = _time(fn, a.warmup, a.reps, flush)
        out.update(rows=a.rows, cols=a.cols, ms=ms, algorithmic_gbs=12.0 * a.rows * a.cols / ms / 1e6,
                   note="read activation and gradient, write dS (+ the [cols] bias gradient)")
    elif a.case == "reduce":
        X = _randn((a.rows, a.cols), 12)
        outb = nd.Array([1, a.cols])
        d = X.desc()
        sb = _lib.lib.endia_b200_reduce_scratch_bytes(d, 1)
        scratch = alloc(sb // 4 + 1)

        def fn():
            _lib.call("endia_b200_reduce_add", d, 1, outb.data_ptr(), scratch.data_ptr(), stream())
        ms = _time(fn, a.warmup, a.reps, flush)
        out.update(rows=a.rows, cols=a.cols, ms=ms, algorithmic_gbs=4.0 * a.rows * a.cols / ms / 1e6,
                   note="column sum: one read of the array")
    print(json.dumps(out))


if __name__ == "__main__":
    main()
