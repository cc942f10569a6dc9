"""GPU tests of the multi-GPU paths. The slab-decomposed fftn runs with one rank in-process (the
packing, exchange-as-copy and both transform directions), and with two ranks over NCCL when the
machine has two GPUs; the data-parallel training step is compared with the single-GPU step."""
import os
import socket
import subprocess
import sys

import numpy as np
import pytest

from conftest import rng, rel_l2, ROOT

pytestmark = pytest.mark.gpu


def test_fftn_slab_single_rank_matches_fftn(nd):
    from endia_b200.dist import fftn_slab
    r = rng(0)
    z = (r.standard_normal((16, 32, 64)) + 1j * r.standard_normal((16, 32, 64))).astype(np.complex64)
    w = r.uniform(-1, 1, (16, 32, 64)).astype(np.float32)
    X1, X2 = nd.Array(z, requires_grad=True), nd.Array(z, requires_grad=True)
    y1 = fftn_slab(X1, 1)
    y2 = nd.fftn(X2)
    assert rel_l2(y1.to_numpy(), y2.to_numpy()) < 1e-6
    nd.sum(nd.real(y1) * nd.Array(w)).backward()
    nd.sum(nd.real(y2) * nd.Array(w)).backward()
    assert rel_l2(X1.grad().to_numpy(), X2.grad().to_numpy()) < 1e-6
    assert rel_l2(X1.grad().to_numpy(), w.size * np.fft.ifftn(w.astype(np.complex128))) < 1e-5


_WORKER = r'''
import os, sys, numpy as np, torch
sys.path.insert(0, %(root)r)
import endia_b200 as nd
from endia_b200 import dist as ndist
rank, world = ndist.init_process_group()
nd._array.device()
r = np.random.Generator(np.random.PCG64(0))
n0, n1, n2 = 32, 64, 32
z = (r.standard_normal((n0, n1, n2)) + 1j * r.standard_normal((n0, n1, n2))).astype(np.complex64)
w = r.uniform(-1, 1, (n0, n1, n2)).astype(np.float32)
s0, s1 = n0 // world, n1 // world
X = nd.Array(z[rank * s0:(rank + 1) * s0], requires_grad=True)
y = ndist.fftn_slab(X, world)
loss = nd.sum(nd.real(y) * nd.Array(np.ascontiguousarray(w[:, rank * s1:(rank + 1) * s1])))
loss.backward()
yref = np.fft.fftn(z.astype(np.complex128))[:, rank * s1:(rank + 1) * s1]
gref = (w.size * np.fft.ifftn(w.astype(np.complex128)))[rank * s0:(rank + 1) * s0]
e1 = np.linalg.norm(y.to_numpy() - yref) / np.linalg.norm(yref)
e2 = np.linalg.norm(X.grad().to_numpy() - gref) / np.linalg.norm(gref)
print("RESULT", rank, e1, e2, flush=True)
torch.distributed.destroy_process_group()
'''


def test_fftn_slab_two_ranks_nccl(nd, tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "slab_worker.py"
    script.write_text(_WORKER % {"root": ROOT})
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                          "--master-addr", "127.0.0.1", "--master-port", str(port), str(script)],
                         capture_output=True, text=True, timeout=300, env=env)
    lines = [l.split() for l in out.stdout.splitlines() if l.startswith("RESULT")]
    assert len(lines) == 2, out.stdout + out.stderr
    for _, rank, e1, e2 in lines:
        assert float(e1) < 1e-5 and float(e2) < 1e-5


_DP_WORKER = r'''
import os, sys, numpy as np, torch
sys.path.insert(0, %(root)r)
sys.path.insert(0, os.path.join(%(root)r, "tests"))
import endia_b200 as nd
from endia_b200 import dist as ndist
from test_gpu_mlp import make_mlp_inputs
rank, world = ndist.init_process_group()
nd._array.device()
dims, batch = [64, 256, 256, 32], 512
Ws, bs, x, y = make_mlp_inputs(dims, batch, 0)
lo, hi = rank * batch // world, (rank + 1) * batch // world
W = [nd.Array(w.copy(), requires_grad=True) for w in Ws]
B = [nd.Array(b.copy(), requires_grad=True) for b in bs]
params = [p for wb in zip(W, B) for p in wb]
opt = nd.optim.Adam(params, lr=1e-3)
opt.grad_scale = 1.0 / world
red = ndist.GradAllReducer(params, mode=os.environ.get("DP_TEST_MODE", "overlap"))
X, Y = nd.Array(x[lo:hi]), nd.Array(y[lo:hi])
loss = nd.mse(nd.nn.mlp([X, None] + params, activation="tanh"), Y)
loss.backward()
red.wait()
grads = [p.grad().to_numpy() / world for p in params]     # mean over ranks of the local-mean gradients
opt.step()
np.savez(os.path.join(%(out)r, "rank%%d.npz" %% rank), *(grads + [p.to_numpy() for p in params]))
torch.distributed.destroy_process_group()
'''


@pytest.mark.parametrize("mode", ["overlap", "bucket"])
def test_data_parallel_step_matches_single_gpu(nd, oracle, tmp_path, mode):
    """Two ranks, each on half of the batch, gradients all-reduced (per parameter during the
    backward pass, or as one flat bucket after it) and averaged inside Adam: the updated weights
    must equal the single-process result (oracle)."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from test_gpu_mlp import make_mlp_inputs, train_step, fwd_unfused
    from conftest import max_rel
    script = tmp_path / "dp_worker.py"
    script.write_text(_DP_WORKER % {"root": ROOT, "out": str(tmp_path)})
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                          "--master-addr", "127.0.0.1", "--master-port", str(port), str(script)],
                         capture_output=True, text=True, timeout=300,
                         env=dict(os.environ, NCCL_NVLS_ENABLE="0", DP_TEST_MODE=mode))
    assert out.returncode == 0, out.stdout + out.stderr
    Ws, bs, x, y = make_mlp_inputs([64, 256, 256, 32], 512, 0)
    oracle.config["mode"] = "fast"
    try:
        ref = train_step(oracle, fwd_unfused("tanh"), Ws, bs, x, y, steps=1)
    finally:
        oracle.config["mode"] = "faithful"
    n = len(ref["params"])
    for rank in range(2):
        got = np.load(tmp_path / ("rank%d.npz" % rank))
        for i in range(n):
            g_ref, p_ref = ref["grads"][i], ref["params"][i]
            assert max_rel(got["arr_%d" % i].reshape(g_ref.shape), g_ref) < 1e-4
            a = got["arr_%d" % (n + i)]
            tiny = np.abs(g_ref.reshape(p_ref.shape)) < 1e-6     # Adam's step is discontinuous at g = 0
            assert max_rel(np.where(tiny, p_ref, a), p_ref) < 1e-4
            assert np.abs(a - p_ref).max() <= 2.5e-3


_SHARDED_WORKER = r'''
import os, sys, numpy as np, torch
sys.path.insert(0, %(root)r)
sys.path.insert(0, os.path.join(%(root)r, "tests"))
import endia_b200 as nd
from endia_b200 import dist as ndist
from test_gpu_mlp import make_mlp_inputs
rank, world = ndist.init_process_group()
nd._array.device()
dims, batch = [64, 512, 512, 32], 512
Ws, bs, x, y = make_mlp_inputs(dims, batch, 0)
lo, hi = rank * batch // world, (rank + 1) * batch // world
W = [nd.Array(w.copy(), requires_grad=True) for w in Ws]
B = [nd.Array(b.copy(), requires_grad=True) for b in bs]
params = [p for wb in zip(W, B) for p in wb]
opt, red = ndist.data_parallel_adam(params, lr=1e-3, mode="sharded")
assert opt.sharded == [False, False, True, False, False, False], opt.sharded
X, Y = nd.Array(x[lo:hi]), nd.Array(y[lo:hi])
losses = []
for step in range(3):
    loss = nd.mse(nd.nn.mlp([X, None] + params, activation="tanh"), Y)
    loss.backward()
    red.wait()
    opt.step()
    loss.zero_grad()
    losses.append(float(loss.to_numpy()[0]))
assert opt.m[2].shape() == [512 * 512 // world] and opt.m[3].shape() == [1, 512]
np.savez(os.path.join(%(out)r, "rank%%d.npz" %% rank), *([p.to_numpy() for p in params] + [np.array(losses)]))
torch.distributed.destroy_process_group()
'''


@pytest.mark.parametrize("pipeline", ["0", "1", "1-nccl"])
def test_sharded_adam_matches_single_gpu(nd, oracle, tmp_path, pipeline):
    """Two ranks, each on half of the batch, three steps with the sharded optimizer, in each of its
    schedules (gather before use; per-layer chains beside the backward pass with the all-gather
    done by the copy engines into peer memory, or by NCCL) (reduce-scatter
    of the large gradients, 1/P Adam update, all-gather of the updated slices consumed layer by
    layer by the next forward pass): parameters and the mean of the ranks' losses must equal the
    single-process result (oracle)."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from test_gpu_mlp import make_mlp_inputs, train_step, fwd_unfused
    script = tmp_path / "sharded_worker.py"
    script.write_text(_SHARDED_WORKER % {"root": ROOT, "out": str(tmp_path)})
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                          "--master-addr", "127.0.0.1", "--master-port", str(port), str(script)],
                         capture_output=True, text=True, timeout=300,
                         env=dict(os.environ, NCCL_NVLS_ENABLE="0", ENDIA_B200_DP_PIPELINE=pipeline[0],
                                  ENDIA_B200_DP_GATHER="nccl" if pipeline.endswith("nccl") else "peer"))
    assert out.returncode == 0, out.stdout + out.stderr
    Ws, bs, x, y = make_mlp_inputs([64, 512, 512, 32], 512, 0)
    oracle.config["mode"] = "fast"
    try:
        ref = train_step(oracle, fwd_unfused("tanh"), Ws, bs, x, y, steps=3)
    finally:
        oracle.config["mode"] = "faithful"
    n = len(ref["params"])
    got = [np.load(tmp_path / ("rank%d.npz" % rank)) for rank in range(2)]
    mean_loss = 0.5 * (got[0]["arr_%d" % n][-1] + got[1]["arr_%d" % n][-1])
    assert abs(mean_loss - ref["loss"][0]) <= 1e-4 * abs(ref["loss"][0])
    for i in range(n):
        p_ref = ref["params"][i]
        a0, a1 = got[0]["arr_%d" % i], got[1]["arr_%d" % i]
        assert np.array_equal(a0, a1)                  # every rank holds the same gathered weights
        # Adam's first steps move a weight by about lr whatever the gradient's size, so an entry whose
        # gradient changes sign within rounding differs by up to the step length
        assert np.abs(a0 - p_ref).max() <= 3 * 2.5e-3
        close = np.abs(a0 - p_ref) <= 1e-4 * np.maximum(np.abs(p_ref), np.sqrt(np.mean(p_ref ** 2)))
        assert close.mean() > 0.999, (i, close.mean())


_ABI_COMM_WORKER = r'''
import os, sys, ctypes as C, numpy as np
sys.path.insert(0, %(root)r)
rank, world, idfile = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3]
os.environ["LOCAL_RANK"] = str(rank)
import endia_b200 as nd
from endia_b200 import _lib
from endia_b200._array import stream
nd._array.device()
ident = (C.c_ubyte * 128)()
if rank == 0:
    _lib.call("endia_b200_comm_unique_id", ident)
    with open(idfile + ".tmp", "wb") as f:
        f.write(bytes(ident))
    os.replace(idfile + ".tmp", idfile)
else:
    import time
    for _ in range(600):
        if os.path.exists(idfile):
            break
        time.sleep(0.1)
    C.memmove(ident, open(idfile, "rb").read(), 128)
comm = C.c_void_p()
_lib.call("endia_b200_comm_init", rank, world, ident, C.byref(comm))
n = 1 << 20
x = nd.Array(np.full(n, rank + 1, np.float32) + np.arange(n, dtype=np.float32) %% 7)
y = nd.Array([n])
_lib.call("endia_b200_allreduce_sum_f32", comm, x.data_ptr(), y.data_ptr(), n, stream())
want = sum(np.full(n, r + 1, np.float32) + np.arange(n, dtype=np.float32) %% 7 for r in range(world))
ok1 = bool(np.array_equal(y.to_numpy(), want))
blk = 4096
send = nd.Array((np.arange(world * blk, dtype=np.float32) + 1000.0 * rank))
recv = nd.Array([world * blk])
_lib.call("endia_b200_alltoall_bytes", comm, send.data_ptr(), recv.data_ptr(), blk * 4, stream())
got = recv.to_numpy().reshape(world, blk)
ok2 = all(np.array_equal(got[p], np.arange(rank * blk, (rank + 1) * blk, dtype=np.float32) + 1000.0 * p)
          for p in range(world))
st = _lib.lib.endia_b200_alltoall_bytes(comm, send.data_ptr(), send.data_ptr(), blk * 4, stream())
_lib.call("endia_b200_comm_destroy", comm)
print("RESULT", rank, ok1, ok2, st == _lib.EINVAL, flush=True)
'''


def test_c_abi_collectives_two_ranks(nd, tmp_path):
    """endia_b200_comm_init / allreduce_sum_f32 / alltoall_bytes between two processes that share
    nothing but the 128-byte id (written to a file by rank 0)."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "comm_worker.py"
    script.write_text(_ABI_COMM_WORKER % {"root": ROOT})
    idfile = str(tmp_path / "nccl_id.bin")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    env.pop("LOCAL_RANK", None)
    procs = [subprocess.Popen([sys.executable, str(script), str(r), "2", idfile], stdout=subprocess.PIPE,
                              stderr=subprocess.PIPE, text=True, env=env) for r in range(2)]
    outs = [p.communicate(timeout=300) for p in procs]
    lines = [l.split() for o, _ in outs for l in o.splitlines() if l.startswith("RESULT")]
    assert len(lines) == 2, "\n".join(o + e for o, e in outs)
    for l in lines:
        assert l[2:] == ["True", "True", "True"], lines


def test_c_abi_collectives_single_rank(nd):
    """With one rank the sum is the input and the exchange is a copy; bad arguments are refused."""
    import ctypes as C
    from endia_b200 import _lib
    from endia_b200._array import stream
    ident = (C.c_ubyte * 128)()
    _lib.call("endia_b200_comm_unique_id", ident)
    comm = C.c_void_p()
    assert _lib.lib.endia_b200_comm_init(1, 1, ident, C.byref(comm)) == _lib.EINVAL
    _lib.call("endia_b200_comm_init", 0, 1, ident, C.byref(comm))
    x = rng(3).standard_normal(5000).astype(np.float32)
    X, Y, Z = nd.Array(x), nd.Array([5000]), nd.Array([5000])
    _lib.call("endia_b200_allreduce_sum_f32", comm, X.data_ptr(), Y.data_ptr(), 5000, stream())
    _lib.call("endia_b200_alltoall_bytes", comm, X.data_ptr(), Z.data_ptr(), 5000 * 4, stream())
    assert np.array_equal(Y.to_numpy(), x) and np.array_equal(Z.to_numpy(), x)
    assert _lib.lib.endia_b200_allreduce_sum_f32(None, X.data_ptr(), Y.data_ptr(), 5000, stream()) == _lib.EINVAL
    _lib.call("endia_b200_comm_destroy", comm)


def test_sharded_adam_single_rank_equals_adam(nd):
    """Without a process group ShardedAdam has nothing to shard: three steps must give optim.Adam's
    parameters and moments bit for bit (same kernel, same state shapes)."""
    from endia_b200.dist import data_parallel_adam
    from test_gpu_mlp import make_mlp_inputs
    Ws, bs, x, y = make_mlp_inputs([32, 300, 8], 64, 3)

    def run(make_opt):
        W = [nd.Array(w.copy(), requires_grad=True) for w in Ws]
        B = [nd.Array(b.copy(), requires_grad=True) for b in bs]
        params = [p for wb in zip(W, B) for p in wb]
        opt, red = make_opt(params)
        X, Y = nd.Array(x), nd.Array(y)
        for _ in range(3):
            loss = nd.mse(nd.nn.mlp([X, None] + params, activation="relu"), Y)
            loss.backward()
            if red is not None:
                red.wait()
            opt.step()
            loss.zero_grad()
        return [p.to_numpy() for p in params], [m.to_numpy() for m in opt.m], [m.shape() for m in opt.m], opt.t

    a = run(lambda params: data_parallel_adam(params, lr=1e-3, mode="sharded"))
    b = run(lambda params: (nd.optim.Adam(params, lr=1e-3), None))
    assert a[2] == b[2] and a[3] == b[3] == 4.0
    for u, v in zip(a[0] + a[1], b[0] + b[1]):
        assert np.array_equal(u, v)


def test_gather_slices_moves_peer_slices_and_writes_parts(nd):
    """endia_b200_gather_slices: the receiving side of the copy-engine all-gather. The other ranks'
    slices come from the inbox, the own slice stays, and the bf16 operand parts of the whole
    parameter equal endia_b200_bf16_split of the result."""
    from endia_b200 import _lib
    from endia_b200._array import stream, alloc
    r = rng(3)
    n, world, rank = 8 * 4 * 1000, 4, 1
    w = r.standard_normal(n).astype(np.float32)
    inbox = r.standard_normal(n).astype(np.float32)
    W, I = nd.Array(w), nd.Array(inbox)
    parts, want_parts = alloc(n), alloc(n)
    _lib.call("endia_b200_gather_slices", W.data_ptr(), I.data_ptr(), n, rank, world, parts.data_ptr(), stream())
    k = n // world
    want = inbox.copy()
    want[k * rank:k * (rank + 1)] = w[k * rank:k * (rank + 1)]
    assert np.array_equal(W.to_numpy(), want)
    _lib.call("endia_b200_bf16_split", W.data_ptr(), want_parts.data_ptr(), n, stream())
    assert np.array_equal(parts.cpu().numpy().view(np.uint32), want_parts.cpu().numpy().view(np.uint32))
    W2 = nd.Array(w)
    _lib.call("endia_b200_gather_slices", W2.data_ptr(), I.data_ptr(), n, rank, world, None, stream())
    assert np.array_equal(W2.to_numpy(), want)
    st = _lib.lib.endia_b200_gather_slices(W2.data_ptr(), I.data_ptr(), n + 4, rank, world, None, stream())
    assert st == _lib.EINVAL
