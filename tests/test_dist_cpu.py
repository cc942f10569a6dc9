"""CPU tests (gloo, world size 2) of the host logic of the multi-GPU paths: the slab exchange of
the distributed N-D FFT and the gradient all-reducer of the data-parallel training step. The
local compute is stood in by torch CPU ops; the device kernels are covered by the -m gpu tests."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _slab_worker(rank, world, port, shape, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from endia_b200 import dist as ndist
        g = torch.Generator().manual_seed(0)
        x = torch.complex(torch.randn(shape, generator=g), torch.randn(shape, generator=g))
        w = torch.rand(shape, generator=g) * 2 - 1
        s0, s1 = shape[0] // world, shape[1] // world
        tail_dims = tuple(range(1, len(shape)))

        def f_tail(t, inv):
            return torch.conj(torch.fft.fftn(torch.conj(t), dim=tail_dims)) if inv else torch.fft.fftn(t, dim=tail_dims)

        def f_head(t, inv):
            return torch.conj(torch.fft.fft(torch.conj(t), dim=0)) if inv else torch.fft.fft(t, dim=0)
        slab = ndist.SlabFFT(f_tail, f_head, world)
        y_local = slab.forward(x[rank * s0:(rank + 1) * s0].contiguous())
        y_ref = torch.fft.fftn(x)
        ok_fwd = torch.allclose(y_local, y_ref[:, rank * s1:(rank + 1) * s1], rtol=1e-4, atol=1e-3)
        # VJP of loss = sum(real(y) * w): dx = F^H (w + 0i), with w split like y
        g_local = torch.complex(w[:, rank * s1:(rank + 1) * s1].contiguous(), torch.zeros(shape[0], s1, *shape[2:]))
        dx_local = slab.backward(g_local)
        dx_ref = torch.conj(torch.fft.fftn(torch.complex(w, torch.zeros_like(w))))
        ok_bwd = torch.allclose(dx_local, dx_ref[rank * s0:(rank + 1) * s0], rtol=1e-4, atol=1e-3)
        # pack / unpack are inverse permutations
        t = torch.arange(s0 * shape[1] * 3, dtype=torch.float32).reshape(s0, shape[1], 3)
        ok_perm = torch.equal(ndist.slab_unpack(ndist.slab_pack(t, world), world), t)
        ret[rank] = (bool(ok_fwd), bool(ok_bwd), bool(ok_perm))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("shape", [(8, 8, 8), (4, 16, 8)])
def test_slab_fft_exchange_two_ranks_gloo(shape):
    world = 2
    port = _free_port()
    with mp.Manager() as m:
        ret = m.dict()
        mp.spawn(_slab_worker, args=(world, port, shape, ret), nprocs=world, join=True)
        assert dict(ret) == {0: (True, True, True), 1: (True, True, True)}


class _FakeGrad:
    """Stands in for a device Array: contiguous float32 storage in a torch CPU tensor."""

    def __init__(self, t):
        self.buf = t

    def is_complex(self):
        return False

    def storage_offset(self):
        return 0

    def size(self):
        return self.buf.numel()

    def is_contiguous(self):
        return True


class _FakeParam:
    def __init__(self):
        self.grad_hook = None
        self.g = None

    def grad_(self, g):
        self.g = g


def _reduce_worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from endia_b200 import dist as ndist
        params = [_FakeParam() for _ in range(3)]
        red = ndist.GradAllReducer(params, mode="overlap")
        grads = [_FakeGrad(torch.full((5 + i,), float(rank + 1 + i))) for i in range(3)]
        # the backward walk reports gradients last layer first
        for p, g in reversed(list(zip(params, grads))):
            p.grad_hook(p, g)
        assert len(red.pending) == 3
        red.wait()
        expect = [sum(float(r + 1 + i) for r in range(world)) for i in range(3)]
        ok = all(torch.allclose(g.buf, torch.full_like(g.buf, e)) for g, e in zip(grads, expect))
        red.detach()
        ret[rank] = bool(ok) and all(p.grad_hook is None for p in params) and not red.pending
    finally:
        dist.destroy_process_group()


def test_gradient_allreducer_two_ranks_gloo():
    world = 2
    port = _free_port()
    with mp.Manager() as m:
        ret = m.dict()
        mp.spawn(_reduce_worker, args=(world, port, ret), nprocs=world, join=True)
        assert dict(ret) == {0: True, 1: True}


def _peer_worker(rank, world, port, fail, ret):
    """Host-injected failures of the peer-buffer set-up: the four device primitives are stood in
    by fakes that record their calls; `fail` names the step that fails and on which rank."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from endia_b200 import dist as ndist
        calls = []
        PB = ndist.PeerBuffers
        PB._cache.clear()

        def alloc(nbytes):
            if fail == ("alloc", rank):
                raise MemoryError("injected: the buffer does not fit")
            calls.append("alloc")
            return 1000 + rank, bytes([rank]) * 64

        def open_(handle):
            if fail == ("open", rank):
                raise RuntimeError("injected: no peer access")
            calls.append("open%d" % handle[0])
            return 2000 + handle[0]
        PB._ipc_alloc = staticmethod(alloc)
        PB._ipc_open = staticmethod(open_)
        PB._ipc_close = staticmethod(lambda p: calls.append("close%d" % p))
        PB._ipc_free = staticmethod(lambda p: calls.append("free%d" % p))
        got = PB.get(4096)
        again = PB.get(4096)            # the outcome is remembered: no second collective attempt
        state = "none" if got is None else "ok"
        if got is not None:
            assert again is got and got.ptrs[rank] == 1000 + rank and got.ptrs[1 - rank] == 2000 + (1 - rank)
            bigger = PB.get(8192)       # replaced collectively: the old ones are unmapped and freed
            assert bigger is not got and got.closed and bigger.nbytes == 8192
            PB.release()
            assert bigger.closed and PB._cache == {}
        ret[rank] = (state, again is None if got is None else True, list(calls))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("fail", [None, ("alloc", 1), ("open", 0)])
def test_peer_buffers_all_ranks_agree_on_failure(fail):
    """One rank's allocation or mapping fails (injected on the host): every rank must end up on the
    fallback path, having released what it held, with no rank left inside a collective."""
    world = 2
    port = _free_port()
    with mp.Manager() as m:
        ret = m.dict()
        mp.spawn(_peer_worker, args=(world, port, fail, ret), nprocs=world, join=True)
        out = dict(ret)
    if fail is None:
        for r in range(2):
            state, same, calls = out[r]
            assert state == "ok" and same
            assert calls == ["alloc", "open%d" % (1 - r), "close%d" % (2001 - r), "free%d" % (1000 + r),
                             "alloc", "open%d" % (1 - r), "close%d" % (2001 - r), "free%d" % (1000 + r)]
        return
    assert out[0][0] == out[1][0] == "none" and out[0][1] and out[1][1]
    if fail[0] == "alloc":
        assert out[0][2] == ["alloc", "free1000"] and out[1][2] == []        # the healthy rank frees its buffer
    else:
        assert out[0][2] == ["alloc", "free1000"]                           # rank 0 mapped nothing
        assert out[1][2] == ["alloc", "open0", "close2000", "free1001"]     # rank 1 unmaps, then frees


class _FakeArray(_FakeGrad):
    """A parameter as ShardedAdam's host logic sees it."""

    def __init__(self, t):
        super().__init__(t)
        self.grad_hook = None
        self.g = None

    def shape(self):
        return list(self.buf.shape)

    def grad_(self, g):
        self.g = g


def _sharded_worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from endia_b200 import dist as ndist
        big, small = 1 << 16, 300
        params = [_FakeArray(torch.zeros(big)), _FakeArray(torch.zeros(small)), _FakeArray(torch.zeros(2 * big))]
        opt = ndist.ShardedAdam(params)
        assert opt.sharded == [True, False, True] and opt.grad_scale == 1.0 / world
        assert [None if g is None else g.numel() for g in opt.g_slice] == [big // world, None, 2 * big // world]
        grads = [_FakeGrad(torch.arange(p.size(), dtype=torch.float32) * (rank + 1)) for p in params]
        for p, g in reversed(list(zip(params, grads))):     # the backward walk: last layer first
            p.grad_hook(p, g)
        assert len(opt.pending) == 2 and [i for i, _ in opt.small] == [1]
        for w in opt.pending:
            w.wait()
        scale = sum(r + 1 for r in range(world))
        ok = True
        for i in (0, 2):
            k = params[i].size() // world
            want = torch.arange(params[i].size(), dtype=torch.float32)[k * rank:k * (rank + 1)] * scale
            ok = ok and torch.equal(opt.g_slice[i], want)
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_sharded_adam_reduce_scatter_two_ranks_gloo():
    """Host logic of the sharded optimizer: which tensors are sharded, and that the hook's
    reduce-scatter leaves rank r with the r-th slice of the summed gradient."""
    world = 2
    port = _free_port()
    with mp.Manager() as m:
        ret = m.dict()
        mp.spawn(_sharded_worker, args=(world, port, ret), nprocs=world, join=True)
        assert dict(ret) == {0: True, 1: True}


def _lonely_worker(port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK="0", WORLD_SIZE="2")
    from endia_b200 import dist as ndist
    import time
    t0 = time.time()
    try:
        ndist.init_process_group(timeout_s=3)
        ret["outcome"] = "joined"
    except Exception as exc:      # the rendezvous timed out
        ret["outcome"] = type(exc).__name__
    ret["seconds"] = time.time() - t0


def test_rendezvous_with_a_missing_rank_times_out():
    """Host-side failure injection: rank 1 of 2 never starts. With a timeout the other rank's
    init_process_group ends with an exception after about that long instead of waiting for ever."""
    port = _free_port()
    with mp.Manager() as m:
        ret = m.dict()
        p = mp.get_context("spawn").Process(target=_lonely_worker, args=(port, ret))
        p.start()
        p.join(60)
        assert not p.is_alive()
        assert ret["outcome"] != "joined" and ret["seconds"] < 30, dict(ret)
