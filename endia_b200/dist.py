"""Data-parallel helpers over torch.distributed (NCCL over NVLink): gradient all-reduce that
overlaps the rest of the backward pass. The reference has no multi-device path; this is the
exchange step the batch-sharded training step needs."""
import os

import torch
import torch.distributed as dist

from ._array import Array, device


def init_process_group():
    """One process per GPU, launched by torchrun (RANK / LOCAL_RANK / WORLD_SIZE / MASTER_*)."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
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

    def __init__(self, params, group=None):
        self.params = list(params)
        self.group = group
        self.pending = []
        for p in self.params:
            p.grad_hook = self._hook

    def _hook(self, param, grad):
        from .functional._utils import contiguous
        g = contiguous(grad)
        if g is not grad:
            param.grad_(g)
        self.pending.append(dist.all_reduce(flat_tensor(g), op=dist.ReduceOp.SUM, group=self.group,
                                            async_op=True))

    def wait(self):
        for w in self.pending:
            w.wait()
        self.pending = []

    def detach(self):
        for p in self.params:
            p.grad_hook = None
