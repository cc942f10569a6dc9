"""Generates the golden fixtures under tests/golden/ from the CPU oracle (faithful mode).

Run from the repository root:  python tests/golden/make_golden.py
The reference itself (Mojo) cannot run here, so the fixtures hold the oracle's results for config
c1 (the reference's own CPU-runnable case) and a small FFT case; they pin both the oracle and the
GPU path against regressions.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from oracle import endia_oracle as eo  # noqa: E402
from test_gpu_mlp import make_mlp_inputs, train_step, fwd_unfused  # noqa: E402


def main():
    here = os.path.dirname(os.path.abspath(__file__))
    eo.build()
    Ws, bs, x, y = make_mlp_inputs([1, 32, 32, 32, 1], 128, 0, x_dist="uniform")
    res = train_step(eo, fwd_unfused("relu"), Ws, bs, x, y, steps=1)
    out = {"loss": res["loss"]}
    for i in range(8):
        out["grad_%d" % i] = res["grads"][i]
        out["param_%d" % i] = res["params"][i]
    np.savez_compressed(os.path.join(here, "c1_mlp_step.npz"), **out)
    r = np.random.Generator(np.random.PCG64(0))
    z = (r.standard_normal((4, 256)) + 1j * r.standard_normal((4, 256))).astype(np.complex64)
    Z = eo.Array(z, requires_grad=True)
    Y = eo.fft(Z)
    loss = eo.sum(eo.square(eo.to_abs(Y))) * (1.0 / 256)
    loss.backward()
    np.savez_compressed(os.path.join(here, "fft_256.npz"), x=z, y=Y.to_numpy(), grad=Z.grad().to_numpy(),
                        loss=loss.to_numpy())


if __name__ == "__main__":
    main()
