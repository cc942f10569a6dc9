"""Data-parallel helpers over torch.distributed (NCCL over NVLink): gradient all-reduce that
overlaps the rest of the backward pass. The reference has no multi-device path; this is the
exchange step the batch-sharded training step needs."""
import os

import torch
import torch.distributed as dist

from ._array import Array, ArrayShape, device


def init_process_group():
    """One process per GPU, launched by torchrun (RANK / LOCAL_RANK / WORLD_SIZE / MASTER_*)."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1:
        # The gradient all-reduce runs beside the backward GEMMs: keep NCCL to 16 CTAs and leave
        # 16 SMs out of the persistent GEMM grid, so that neither waits for the other's SMs.
        os.environ.setdefault("NCCL_MAX_CTAS", "16")
        os.environ.setdefault("ENDIA_B200_TC_RESERVE_SMS", "16")
    if world > 1 and not dist.is_initialized():
        backend = "nccl" if torch.cuda.is_available() else "gloo"
        if backend == "nccl":
            dist.init_process_group(backend, device_id=device())
        else:
            dist.init_process_group(backend)
    return (dist.get_rank(), dist.get_world_size()) if dist.is_initialized() else (0, 1)


def flat_tensor(arr):
    """torch view of an Array's contiguous storage (no copy)."""
    w = 2 if arr.is_complex() else 1
    off = arr.storage_offset() * w
    return arr.buf[off:off + arr.size() * w]


class GradAllReducer:
    """Starts a sum all-reduce of a parameter's gradient the moment the backward walk has produced
    it (last layer first), on the communicator's own stream, so that it overlaps the remaining
    backward GEMMs; wait() joins them before the optimizer step. The mean over ranks is folded into
    the optimizer's gradient scale instead of a separate pass."""

    def __init__(self, params, group=None, overlap=True):
        self.params = list(params)
        self.group = group
        self.overlap = overlap      # False: all-reduce only in wait(), after the backward pass
        self.pending = []
        self.deferred = []
        for p in self.params:
            p.grad_hook = self._hook

    def _hook(self, param, grad):
        g = grad
        if not grad.is_contiguous():
            from .functional._utils import contiguous
            g = contiguous(grad)
            param.grad_(g)
        if not self.overlap:
            self.deferred.append(g)
            return
        self.pending.append(dist.all_reduce(flat_tensor(g), op=dist.ReduceOp.SUM, group=self.group,
                                            async_op=True))

    def wait(self):
        for g in self.deferred:
            self.pending.append(dist.all_reduce(flat_tensor(g), op=dist.ReduceOp.SUM, group=self.group,
                                                async_op=True))
        self.deferred = []
        for w in self.pending:
            w.wait()
        self.pending = []

    def detach(self):
        for p in self.params:
            p.grad_hook = None


# ---------------------------------------------------------------------------------------------
# Slab-decomposed N-D FFT: the array is split along axis 0 over the ranks; the transform over the
# trailing axes is local, one all-to-all re-splits the array along axis 1 so that axis 0 becomes
# local, and the last transform runs there. The result stays split along axis 1 (the VJP runs the
# same steps backwards, so no transpose back is needed).

def slab_pack(local, world):
    """[S0, N1, ...] -> [P, S0, N1/P, ...]: block q holds the part of axis 1 that rank q will own.
    `local` is a torch tensor (any device); returns a contiguous tensor."""
    s0, n1 = local.shape[0], local.shape[1]
    rest = tuple(local.shape[2:])
    return local.reshape((s0, world, n1 // world) + rest).transpose(0, 1).contiguous()


def slab_unpack(blocks, world):
    """Inverse of slab_pack: [P, S0, N1/P, ...] -> [S0, N1, ...]."""
    s0, s1 = blocks.shape[1], blocks.shape[2]
    rest = tuple(blocks.shape[3:])
    return blocks.transpose(0, 1).reshape((s0, world * s1) + rest).contiguous()


def slab_exchange(packed, group=None):
    """All-to-all of the P blocks of `packed` ([P, ...], contiguous): block q goes to rank q; the
    result's block q came from rank q. Received data lands in local memory (NCCL or gloo)."""
    out = torch.empty_like(packed)
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_to_all_single(out, packed, group=group)
    else:
        out.copy_(packed)
    return out


class SlabFFT:
    """fftn of an array whose axis 0 is split over the ranks. `fft_tail(t, inverse)` transforms
    all axes but the first of a local torch tensor, `fft_head(t, inverse)` transforms axis 0; both
    return tensors of the same shape. The product passes GPU kernels, the CPU tests pass torch.fft.

    forward(x_local[S0, N1, ...]) -> y_local[N0, N1/P, ...]   (split along axis 1)
    backward(g_local[N0, N1/P, ...]) -> dx_local[S0, N1, ...] (the VJP: conjugate-direction
    transform without normalisation, endia fftn_op.mojo:43-49)"""

    def __init__(self, fft_tail, fft_head, world, group=None):
        self.fft_tail, self.fft_head, self.world, self.group = fft_tail, fft_head, world, group

    def forward(self, x_local, inverse=False):
        y = self.fft_tail(x_local, inverse)
        blocks = slab_exchange(slab_pack(y, self.world), self.group)
        # block q = rows of axis 0 owned by rank q: stacking the blocks restores axis 0
        full0 = blocks.reshape((blocks.shape[0] * blocks.shape[1],) + tuple(blocks.shape[2:]))
        return self.fft_head(full0, inverse)

    def backward(self, g_local, inverse=True):
        g = self.fft_head(g_local, inverse)
        s0 = g.shape[0] // self.world
        blocks = g.reshape((self.world, s0) + tuple(g.shape[1:]))
        back = slab_exchange(blocks.contiguous(), self.group)
        return self.fft_tail(slab_unpack(back, self.world), inverse)


def _strided_view(arr, shape, stride):
    v = Array(ArrayShape(shape, stride, arr.storage_offset()))
    v.buf = arr.buf
    v.base_ = arr.base()
    v.is_view = True
    v.is_complex_flag = arr.is_complex()
    return v


def _exchange_arrays(src, world, group=None):
    """All-to-all of the `world` equal blocks of a contiguous Array into a new Array."""
    out = Array(ArrayShape(src.shape()))
    out.is_complex_flag = src.is_complex()
    out.buf = torch.empty_like(flat_tensor(src))
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_to_all_single(out.buf, flat_tensor(src), group=group)
    else:
        from . import _lib
        from ._array import stream
        _lib.call("endia_b200_d2d", out.data_ptr(), src.data_ptr(), src.size() * 8, stream())
    return out


def fftn_slab(x_local, world=None, group=None):
    """fftn of a 3-D complex array whose axis 0 is split over the ranks (x_local is this rank's
    slab [N0/P, N1, N2]); returns this rank's slab [N0, N1/P, N2] of the result, split along
    axis 1. Differentiable: the VJP runs the conjugate-direction transforms and the exchange in
    reverse order and returns a gradient laid out like x_local (fftn_op.mojo:43-49). Local
    transforms, the block packing and every other step run in this library's kernels; the
    exchange is one all-to-all into local memory."""
    from .functional._utils import op_array, setup_shape_and_data, copy
    from .functional.fft_ops import run_fft
    if world is None:
        world = dist.get_world_size(group) if dist.is_initialized() else 1
    s0, n1, n2 = x_local.shape()
    n0, s1 = s0 * world, n1 // world
    if n1 % world:
        raise ValueError("fftn_slab: axis 1 (%d) must divide by the number of ranks (%d)" % (n1, world))

    def new_like(shape):
        a = Array(ArrayShape(shape))
        a.is_complex_flag = True
        setup_shape_and_data(a)
        return a

    def forward_impl(x):
        y1 = new_like([s0, n1, n2])
        run_fft(x, y1, [1, 2], False, 1.0)
        # pack: block q = y1[:, q*s1:(q+1)*s1, :]  ->  [P, s0, s1, n2] contiguous
        packed = copy(_strided_view(y1, [world, s0, s1, n2], [s1 * n2, n1 * n2, n2, 1]))
        recv = _exchange_arrays(packed, world, group)          # [P*s0 = n0, s1, n2]
        full0 = _strided_view(recv, [n0, s1, n2], [s1 * n2, n2, 1])
        out = new_like([n0, s1, n2])
        run_fft(full0, out, [0], False, 1.0)
        return out

    def backward_impl(g):
        g0 = new_like([n0, s1, n2])
        run_fft(g, g0, [0], True, 1.0)                           # conj o fft o conj along axis 0
        recv = _exchange_arrays(g0, world, group)              # block q: [s0, s1 (chunk q), n2]
        # unpack: [P, s0, s1, n2] -> [s0, P*s1 = n1, n2]
        unpacked = copy(_strided_view(recv, [s0, world, s1, n2], [s1 * n2, s0 * s1 * n2, n2, 1]))
        flat = _strided_view(unpacked, [s0, n1, n2], [n1 * n2, n2, 1])
        dx = new_like([s0, n1, n2])
        run_fft(flat, dx, [1, 2], True, 1.0)
        return dx

    def call(curr, args):
        res = forward_impl(args[0])
        curr.buf = res.buf

    def vjp(primals, grad, out):
        from .functional._utils import contiguous
        g = contiguous(grad)
        if not g.is_complex():
            raise ValueError("fftn_slab: the incoming gradient must be complex")
        return [backward_impl(g)]
    return op_array(ArrayShape([n0, s1, n2]), [x_local], "fftn_slab", call, vjp=vjp, is_complex_p=True)
