"""Data-parallel helpers over torch.distributed (NCCL over NVLink): gradient all-reduce that
overlaps the rest of the backward pass. The reference has no multi-device path; this is the
exchange step the batch-sharded training step needs."""
import os

import torch
import torch.distributed as dist

from ._array import Array, ArrayShape, device, await_pending


def init_process_group(nccl_max_ctas=None, gemm_reserve_sms=None, timeout_s=None):
    """One process per GPU, launched by torchrun (RANK / LOCAL_RANK / WORLD_SIZE / MASTER_*).

    A collective that runs beside the persistent GEMM kernels needs SMs of its own: the GEMM grid
    otherwise holds all of them and NCCL's CTAs (or the GEMM's last CTA pairs) wait. The launcher
    states both limits here, before NCCL and the GEMM read them: `nccl_max_ctas` becomes
    NCCL_MAX_CTAS and `gemm_reserve_sms` the number of SMs left out of the persistent GEMM grid
    (ENDIA_B200_TC_RESERVE_SMS); values already in the environment win, None sets nothing.
    `timeout_s` bounds the rendezvous and every later collective: a rank that never joins (or that
    has left) then ends the others' wait with an exception instead of a hang."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1:
        if nccl_max_ctas is not None:
            os.environ.setdefault("NCCL_MAX_CTAS", str(int(nccl_max_ctas)))
        if gemm_reserve_sms is not None:
            os.environ.setdefault("ENDIA_B200_TC_RESERVE_SMS", str(int(gemm_reserve_sms)))
    if world > 1 and not dist.is_initialized():
        backend = "nccl" if torch.cuda.is_available() else "gloo"
        kw = {}
        if timeout_s is not None:
            import datetime
            kw["timeout"] = datetime.timedelta(seconds=float(timeout_s))
        if backend == "nccl":
            dist.init_process_group(backend, device_id=device(), **kw)
        else:
            dist.init_process_group(backend, **kw)
    return (dist.get_rank(), dist.get_world_size()) if dist.is_initialized() else (0, 1)


def flat_tensor(arr):
    """torch view of an Array's contiguous storage (no copy)."""
    await_pending(arr)
    w = 2 if arr.is_complex() else 1
    off = arr.storage_offset() * w
    return arr.buf[off:off + arr.size() * w]


class GradAllReducer:
    """Sums the parameters' gradients over the ranks before the optimizer step; the mean over ranks
    is folded into the optimizer's gradient scale instead of a separate pass. Modes:

    "overlap"           an all-reduce per parameter is started from a hook the moment the backward
                        walk has produced its gradient (last layer first), on the communicator's
                        stream, beside the remaining backward GEMMs.
    "bucket"            after the backward pass the gradients are gathered into one flat buffer
                        (a device copy of all of them, 0.07 ms for the 168 MB of c2), summed by ONE
                        all-reduce, and the parameters' gradients become views of that buffer.
    "serial"            an all-reduce per parameter after the backward pass.

    Measured on the c2 step: 2 GPUs overlap 4.13-4.21 ms, bucket 4.40-4.60 ms; 8 GPUs overlap
    2.08 ms, bucket 1.94 ms. The persistent GEMM kernels hold every SM, so a collective beside
    them waits for SMs and a GEMM launched beside a collective runs on fewer; with the short
    per-rank steps of 8 ranks one all-reduce after the pass costs less, so groups of 8 or more
    default to "bucket", smaller ones to "overlap" (ENDIA_B200_DP_MODE overrides)."""

    def __init__(self, params, group=None, overlap=None, mode=None):
        self.params = list(params)
        self.group = group
        if mode is None:
            default = "overlap"
            if dist.is_initialized() and dist.get_world_size(group) >= 8:
                default = "bucket"      # short per-rank steps: see the class comment
            mode = os.environ.get("ENDIA_B200_DP_MODE", default) if overlap is None else (
                "overlap" if overlap else "serial")
        if mode not in ("bucket", "overlap", "serial"):
            raise ValueError("GradAllReducer: unknown mode %r" % (mode,))
        self.mode = mode
        self.pending = []
        self.deferred = []
        self.small = []           # (param, grad) of small tensors, summed together in wait()
        self.flat = None
        self.flat_small = None
        for p in self.params:
            p.grad_hook = self._hook

    def _hook(self, param, grad):
        if self.mode == "bucket":
            return
        g = grad
        if not grad.is_contiguous():
            from .functional._utils import contiguous
            g = contiguous(grad)
            param.grad_(g)
        if self.mode == "serial":
            self.deferred.append(g)
            return
        if g.size() < self.SMALL and flat_tensor(g).is_cuda:
            # bias-sized gradients: one collective for all of them instead of one each, whose
            # latency would sit between the large ones on the communicator's stream
            self.small.append((param, g))
            return
        self.pending.append(dist.all_reduce(flat_tensor(g), op=dist.ReduceOp.SUM, group=self.group,
                                            async_op=True))

    SMALL = 1 << 16

    def _reduce_bucket(self, params=None, grads=None, which="flat"):
        from . import _lib
        from ._array import stream
        from .functional._utils import contiguous
        if params is None:
            params = self.params
            grads = [contiguous(p.grad()) for p in params]
        total = sum(g.size() for g in grads)
        flat = getattr(self, which)
        if flat is None or flat.numel() != total:
            flat = torch.empty(total, dtype=torch.float32, device=device())
            setattr(self, which, flat)
        off = 0
        views = []
        for p, g in zip(params, grads):
            n = g.size()
            piece = flat[off:off + n]
            if n:
                _lib.call("endia_b200_d2d", piece.data_ptr(), g.data_ptr(), 4 * n, stream())
            v = Array(ArrayShape(g.shape()))
            v.buf = piece
            views.append(v)
            off += n
        if total:
            dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=self.group)
        for p, v in zip(params, views):
            p.grad_(v)

    def wait(self):
        if self.mode == "bucket":
            self._reduce_bucket()
            return
        for g in self.deferred:
            self.pending.append(dist.all_reduce(flat_tensor(g), op=dist.ReduceOp.SUM, group=self.group,
                                                async_op=True))
        self.deferred = []
        if self.small:
            self._reduce_bucket([p for p, _ in self.small], [g for _, g in self.small], "flat_small")
            self.small = []
        for w in self.pending:
            w.wait()
        self.pending = []

    def detach(self):
        for p in self.params:
            p.grad_hook = None


class ShardedAdam:
    """Adam for the batch-sharded training step with the optimizer sharded over the ranks: the sum of
    the ranks' gradients and the replicated update of optim.Adam become, per large parameter,

      reduce-scatter   the gradient is summed over the ranks the moment the backward walk has
                       produced it (last layer first); rank r receives the r-th 1/P of it,
      update           Adam on this rank's 1/P of the parameter (its slices of m and v are the only
                       optimizer state the rank holds),
      all-gather       the updated slices are gathered in place into every rank's parameter, and the
                       parameter's GEMM operand parts are rewritten (one pass over the weights).

    pipelined=True (default): the steps of a layer run as a chain on a side stream of their own as
    soon as the layer's gradient exists, beside the backward pass of the layers below: reduce-scatter
    (ordered behind the weight-gradient product only, which the layer's VJP enqueues before its dX
    product), Adam on the slice, then the all-gather. Where the ranks can map each other's memory
    the gather is done by the COPY ENGINES: each rank copies its updated slice into an "inbox" on
    every peer (cudaMemcpyAsync over NVLink; no SM is taken from the GEMMs and the communicator
    stays free for the reduce-scatters of the layers below); step() updates the bias-sized tensors
    (one all-reduce, replicated update), joins the chains, passes one barrier and moves the received
    slices into the parameters in the pass that also writes their GEMM operand parts
    (endia_b200_gather_slices). Without peer access the chain ends in an NCCL all-gather
    (ENDIA_B200_DP_GATHER=nccl forces that). The update of a parameter starts DURING backward():
    every backward() must be followed by one step(). Measured per c2 step at 2 / 4 / 8 ranks: 3.99 /
    2.13 / 1.54 ms against 4.12 / 2.23 / 1.73 ms for the schedule below (4.17 / 2.24 ms at 2 / 4 ranks
    with the NCCL gather).
    pipelined=False (ENDIA_B200_DP_PIPELINE=0): backward() only starts the reduce-scatters; step()
    runs ONE multi-tensor update, and NCCL all-gathers start when the parameters are next used (each
    consumer waits for its own parameter: the next forward pass runs beside the later gathers).

    Either way a step is self-contained (every collective it starts is consumed inside it or at the
    next use of the parameters), which lets it be captured as one CUDA graph. The arithmetic per
    element is optim.Adam's (endia/optim/adam.mojo:47-65) with the mean over the ranks folded into
    the gradient scale; the bytes on NVLink are those of the all-reduce it replaces. `m` and `v` hold
    slices for the large parameters (flat, 1/P of the elements) and whole arrays for the small."""
    mode = "sharded"
    SMALL = 1 << 16

    def __init__(self, params, lr=0.001, beta1=0.9, beta2=0.999, eps=1e-8, group=None, pipelined=None):
        self.params = list(params)
        self.lr, self.beta1, self.beta2, self.eps = lr, beta1, beta2, eps
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if pipelined is None:
            pipelined = os.environ.get("ENDIA_B200_DP_PIPELINE", "1") != "0"
        self.pipelined = bool(pipelined) and self.world > 1 and torch.cuda.is_available() \
            and dist.get_backend(group) == "nccl"
        self.t = 1.0
        self.grad_scale = 1.0 / self.world
        self.sharded = [self._shardable(p) for p in self.params]
        self.g_slice = [torch.empty(p.size() // self.world, dtype=torch.float32, device=flat_tensor(p).device)
                        if sh else None for p, sh in zip(self.params, self.sharded)]
        self._m = self._v = None  # moments: allocated (zero) at the first step or first access
        self._early_stream, self._early_used = None, False
        self.pending = []         # reduce-scatters in flight (not pipelined)
        self.small = []           # (index, gradient) of the replicated tensors of this pass
        self.flat_small = None
        self._ready = {}
        self._gathers = None      # all-gathers of the last step, once launched (not pipelined)
        self._chains = {}         # index -> side stream whose chain of this pass is in flight (pipelined)
        self._streams = {}
        self._t_dev = None
        # Pipelined with peer access: the all-gather is done by the copy engines. Every rank has an
        # "inbox" laid out like the sharded parameters (mapped into all ranks through CUDA IPC); a
        # rank copies its updated slice into the peers' inboxes (cudaMemcpyAsync over NVLink: no SM
        # is taken from the GEMMs and the communicator's stream stays free for the reduce-scatters
        # of the layers below), and after one barrier each rank moves the received slices into its
        # parameters in the pass that also writes their GEMM operand parts.
        self._inbox, self._inbox_off = None, {}
        if self.pipelined and os.environ.get("ENDIA_B200_DP_GATHER", "peer") == "peer":
            off, ok = 0, True
            for i, p in enumerate(self.params):
                if self.sharded[i]:
                    self._inbox_off[i] = off
                    off += p.size()
                    ok = ok and p.size() % (8 * self.world) == 0
            made = PeerBuffers._create(4 * off, group) if ok and off else None   # (collective)
            self._inbox = made
            self._bar = torch.zeros(1, device=flat_tensor(self.params[0]).device) if made is not None else None
        if self.pipelined:
            self._state()         # zeroed on the compute stream now: the layers' side streams start from it
        for p in self.params:
            p.grad_hook = self._hook

    def _state(self):
        if self._m is None:
            shapes = [[p.size() // self.world] if sh else p.shape() for p, sh in zip(self.params, self.sharded)]
            self._m = [Array(shape) for shape in shapes]
            self._v = [Array(shape) for shape in shapes]
        return self._m, self._v

    @property
    def m(self):
        return self._state()[0]

    @property
    def v(self):
        return self._state()[1]

    def _reduce_scatter(self, out, inp):
        """Asynchronous sum over the ranks of `inp`, this rank's 1/P of it into `out`."""
        if dist.get_backend(self.group) != "gloo":
            return dist.reduce_scatter_tensor(out, inp, op=dist.ReduceOp.SUM, group=self.group, async_op=True)
        # gloo (CPU runs of the host logic) has no reduce-scatter: all-reduce a copy, keep the slice
        tmp, k, r = inp.clone(), out.numel(), self.rank
        work = dist.all_reduce(tmp, op=dist.ReduceOp.SUM, group=self.group, async_op=True)

        class _Done:
            def wait(self):
                work.wait()
                out.copy_(tmp[k * r:k * (r + 1)])
        return _Done()

    def _early(self, grad, launch):
        """Start a collective on a gradient. A fused layer's VJP enqueues the weight-gradient product
        first and records an event behind it (`_ready_event`); the collective is then ordered behind
        that event on a stream of its own instead of behind everything enqueued so far, so it runs
        beside the layer's dX product. step() joins the stream."""
        ev = getattr(grad, "_ready_event", None)
        if ev is None or not torch.cuda.is_available() or dist.get_backend(self.group) != "nccl":
            return launch()
        if self._early_stream is None:
            self._early_stream = torch.cuda.Stream(device=flat_tensor(grad).device)
        self._early_stream.wait_event(ev)
        with torch.cuda.stream(self._early_stream):
            work = launch()
        self._early_used = True
        return work

    def _shardable(self, p):
        return (self.world > 1 and p.size() >= self.SMALL and p.size() % self.world == 0 and p.is_contiguous()
                and not p.is_complex())

    def _index(self, param):
        for i, p in enumerate(self.params):
            if p is param:
                return i
        raise KeyError("ShardedAdam: unknown parameter")

    def _wants_parts(self, p):
        return p.ndim() == 2 and p.size() % 8 == 0 and p.size() >= 128 * 128

    def _adam(self, indices, grads, stream_ptr, advance):
        """One multi-tensor launch over the listed parameters: this rank's slice of a sharded one
        (gradient = its reduce-scatter result), the whole of a replicated one (gradient from `grads`)."""
        import ctypes as C
        from . import _lib
        from .functional._utils import broadcast_shapes
        P, G, M, V, numel = [], [], [], [], []
        for i in indices:
            p = self.params[i]
            if self.sharded[i]:
                k = p.size() // self.world
                P.append(p.buf.data_ptr() + 4 * k * self.rank)
                G.append(self.g_slice[i].data_ptr())
                numel.append(k)
            else:
                g = grads[i]
                if g.size() != p.size():
                    raise _lib.EndiaError(_lib.ESHAPE, "Adam: gradient %s does not match parameter %s" % (
                        g.shape(), p.shape()))
                P.append(p.data_ptr())
                G.append(g.data_ptr())
                numel.append(p.size())
                shp = broadcast_shapes(self.m[i].shape(), g.shape())     # (1, N) for a bias, as in optim.Adam
                self.m[i].array_shape_ = ArrayShape(shp)
                self.v[i].array_shape_ = ArrayShape(shp)
            M.append(self.m[i].data_ptr())
            V.append(self.v[i].data_ptr())
        n = len(P)
        arr = lambda xs: (C.c_void_p * max(n, 1))(*xs)
        if self._t_dev is not None:
            _lib.call("endia_b200_adam_step_multi_graph", n, arr(P), arr(G), arr(M), arr(V), None,
                      (C.c_int64 * max(n, 1))(*numel), self.lr, self.beta1, self.beta2, self.eps,
                      self._t_dev.data_ptr(), 1 if advance else 0, self.grad_scale, stream_ptr)
        elif n:
            _lib.call("endia_b200_adam_step_multi", n, arr(P), arr(G), arr(M), arr(V), (C.c_int64 * n)(*numel),
                      self.lr, self.beta1, self.beta2, self.eps, self.t, self.grad_scale, stream_ptr)

    def _hook(self, param, grad):
        from .functional._utils import contiguous
        from ._array import flush_readers
        i = self._index(param)
        g = contiguous(grad)
        if g is not grad:
            param.grad_(g)
        if not self.sharded[i]:
            self.small.append((i, g))
            return
        self._ready[i] = True
        rs = self._early(g, lambda: self._reduce_scatter(self.g_slice[i], flat_tensor(g)))
        if not self.pipelined:
            self.pending.append(rs)
            return
        # the layer's chain on its own stream: reduce-scatter -> update of the slice -> all-gather ->
        # operand parts. The layer's own VJP products (the last readers of the old weights in this
        # pass) are on the compute stream ahead of the reduce-scatter, which the chain waits for.
        from . import _lib
        from ._array import alloc
        flush_readers(param)
        side = self._streams.get(i)
        if side is None:
            side = self._streams[i] = torch.cuda.Stream(device=flat_tensor(param).device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            rs.wait()
            self._adam([i], None, side.cuda_stream, advance=False)
            k = param.size() // self.world
            full = param.buf[:param.size()]
            if self._inbox is not None:
                # this rank's slice into every peer's inbox, nearest neighbour first
                src = param.buf.data_ptr() + 4 * k * self.rank
                for d in range(1, self.world):
                    q = (self.rank + d) % self.world
                    _lib.call("endia_b200_d2d", self._inbox.ptrs[q] + 4 * (self._inbox_off[i] + k * self.rank), src,
                              4 * k, side.cuda_stream)
                self._chains[i] = side
                return
            ag = dist.all_gather_into_tensor(full, full[k * self.rank:k * (self.rank + 1)], group=self.group,
                                             async_op=True)
            ag.wait()
            param._tf32_lo = None
            if self._wants_parts(param):
                if getattr(param, "_pair16", None) is None:
                    param._pair16 = alloc(param.size())
                _lib.call("endia_b200_bf16_split", param.buf.data_ptr(), param._pair16.data_ptr(), param.size(),
                          side.cuda_stream)
                param._parts_ptr = param.buf.data_ptr()
            else:
                param._pair16 = None
        self._chains[i] = side

    def wait(self):
        """Nothing to do before step(): kept so that the step reads like the replicated one."""

    def detach(self):
        for p in self.params:
            p.grad_hook = None

    def close(self):
        """Collective: release the peer-mapped inbox of the copy-engine all-gather, if there is one."""
        if self._inbox is not None:
            self._inbox.close()
            self._inbox = None

    def reset_state(self):
        from . import _lib
        from ._array import stream
        self.t = 1.0
        if self._t_dev is not None:
            _lib.call("endia_b200_fill", self._t_dev.data_ptr(), 1, 0, 1.0, 0.0, stream())
        for i, p in enumerate(self.params):
            for st in (self.m[i], self.v[i]):
                if not self.sharded[i]:
                    st.array_shape_ = ArrayShape(p.shape())
                if st.size():
                    _lib.call("endia_b200_memset0", st.data_ptr(), st.size() * 4, stream())

    def step(self):
        from ._array import stream, alloc, flush_readers
        from .functional._utils import contiguous
        for p in self.params:
            flush_readers(p)
        # gradients that no hook has seen (a parameter outside the graph): zeros, like Array.grad()
        seen_small = {i for i, _ in self.small}
        for i, p in enumerate(self.params):
            if self.sharded[i] and not self._ready.get(i):
                self._hook(p, p.grad())
            elif not self.sharded[i] and i not in seen_small:
                self.small.append((i, contiguous(p.grad())))
        small = dict(self.small)
        if self.world > 1 and small:
            # the bias-sized gradients: one collective for all of them
            idx = sorted(small)
            total = sum(small[i].size() for i in idx)
            if self.flat_small is None or self.flat_small.numel() != total:
                self.flat_small = torch.empty(total, dtype=torch.float32, device=flat_tensor(self.params[idx[0]]).device)
            off = 0
            views = {}
            for i in idx:
                k = small[i].size()
                piece = self.flat_small[off:off + k]
                piece.copy_(flat_tensor(small[i]))
                v = Array(ArrayShape(small[i].shape()))
                v.buf = piece
                views[i] = v
                off += k
            dist.all_reduce(self.flat_small, op=dist.ReduceOp.SUM, group=self.group)
            for i in idx:
                self.params[i].grad_(views[i])
            small = views
        capturing = torch.cuda.is_available() and torch.cuda.is_current_stream_capturing()
        if self._early_used:
            torch.cuda.current_stream().wait_stream(self._early_stream)
            self._early_used = False
        if self.pipelined:
            # the replicated tensors here (and the step count), then the layers' chains join
            self._adam(sorted(small), small, stream(), advance=True)
            for i in small:
                self.params[i]._tf32_lo = None
                self.params[i]._pair16 = None
            main = torch.cuda.current_stream()
            for side in self._chains.values():
                main.wait_stream(side)
            if self._inbox is not None and self._chains:
                # every rank's copies are behind it on its stream when it joins this all-reduce, so
                # when it completes here all slices have landed in this rank's inbox
                dist.all_reduce(self._bar, op=dist.ReduceOp.SUM, group=self.group)
                from . import _lib
                for i in sorted(self._chains):
                    p = self.params[i]
                    p._tf32_lo = None
                    wants = self._wants_parts(p)
                    if wants and getattr(p, "_pair16", None) is None:
                        p._pair16 = alloc(p.size())
                    if not wants:
                        p._pair16 = None
                    _lib.call("endia_b200_gather_slices", p.buf.data_ptr(),
                              self._inbox.ptrs[self.rank] + 4 * self._inbox_off[i], p.size(), self.rank, self.world,
                              p._pair16.data_ptr() if wants else None, stream())
                    if wants:
                        p._parts_ptr = p.buf.data_ptr()
            self._chains = {}
        else:
            for w in self.pending:
                w.wait()
            self.pending = []
            for p in self.params:       # a gather of the last step that no consumer has waited for
                await_pending(p)
            self._adam(list(range(len(self.params))), small, stream(), advance=True)
            # The updated slices are gathered when the parameters are next used (first layer first):
            # every sharded parameter carries a completion callback until then.
            for i, p in enumerate(self.params):
                p._tf32_lo = None
                if not self.sharded[i]:
                    p._pair16 = None
                    continue
                wants = self._wants_parts(p)
                if wants and getattr(p, "_pair16", None) is None:
                    p._pair16 = alloc(p.size())
                if not wants:
                    p._pair16 = None
                p._parts_ptr = None      # the parts are stale until the callback has rewritten them
                p._pending = self._completion(i, wants)
            self._gathers = None
        self._ready = {}
        self.small = []
        if not capturing:
            self.t += 1.0     # (a step being captured is not run; after_replay counts its replays)

    def _launch_gathers(self):
        """All-gather of every sharded parameter's updated slices, in parameter order, on the
        communicator's stream (in place: rank r's slice is already where it belongs)."""
        if self._gathers is not None:
            return
        self._gathers = {}
        for i, p in enumerate(self.params):
            if not self.sharded[i]:
                continue
            k = p.size() // self.world
            full = p.buf[:p.size()]
            self._gathers[i] = dist.all_gather_into_tensor(full, full[k * self.rank:k * (self.rank + 1)],
                                                           group=self.group, async_op=True)

    def _completion(self, i, wants_parts):
        p = self.params[i]

        def done():
            from . import _lib
            from ._array import stream
            self._launch_gathers()
            self._gathers[i].wait()          # the compute stream waits for this parameter's gather only
            if wants_parts:
                _lib.call("endia_b200_bf16_split", p.buf.data_ptr(), p._pair16.data_ptr(), p.size(), stream())
                p._parts_ptr = p.buf.data_ptr()
        return done

    def sync(self):
        """Complete every parameter on this rank now (collective: every rank calls it). Without the
        pipeline a sharded parameter is whole on a rank once its gather has run, which the next use
        of the parameter on ALL ranks starts; code that reads parameters on one rank only calls
        this first. (With the pipeline step() leaves the parameters complete.)"""
        for p in self.params:
            await_pending(p)

    # ---- steps replayed from a CUDA graph (utils.CapturedStep(..., optimizers=[self])) -----------
    def begin_capture(self):
        from .functional.init_ops import full
        self._t_dev = full([1], self.t)

    def end_capture(self):
        self._t_dev = None

    def after_replay(self):
        """A replayed step has run the update on the device; the host-side state follows: the step
        count and, without the pipeline, the completion callbacks of the sharded parameters (the
        gathers of the new slices are the first thing the next replay, or the next use on the host,
        does)."""
        self.t += 1.0
        if self.pipelined:
            return
        for i, p in enumerate(self.params):
            if self.sharded[i]:
                p._parts_ptr = None
                p._pending = self._completion(i, getattr(p, "_pair16", None) is not None)
        self._gathers = None


def data_parallel_adam(params, lr=0.001, beta1=0.9, beta2=0.999, eps=1e-8, group=None, mode=None):
    """Optimizer and gradient exchange for a batch-sharded training step: (optimizer, reducer). The
    step calls reducer.wait() after backward() and optimizer.step() after that. Modes
    (ENDIA_B200_DP_MODE overrides): "sharded" (default: ShardedAdam, reduce-scatter + 1/P update +
    all-gather) or one of GradAllReducer's replicated modes "overlap", "bucket", "serial"."""
    from .optim import Adam
    if mode is None:
        mode = os.environ.get("ENDIA_B200_DP_MODE", "sharded")
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if mode == "sharded":
        opt = ShardedAdam(params, lr, beta1, beta2, eps, group)
        return opt, opt
    opt = Adam(params, lr=lr, beta1=beta1, beta2=beta2, eps=eps)
    opt.grad_scale = 1.0 / world     # global-mean loss = mean of the ranks' local means
    return opt, GradAllReducer(params, group, mode=mode)


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


def _strided_view(arr, shape, stride, offset=0):
    v = Array(ArrayShape(shape, stride, arr.storage_offset() + offset))
    v.buf = arr.buf
    v.base_ = arr.base()
    v.is_view = True
    v.is_complex_flag = arr.is_complex()
    return v


class PeerBuffers:
    """One device buffer per rank, mapped into every rank of the machine through CUDA IPC, plus
    the stream-ordered barrier that orders the ranks' accesses (a one-element NCCL all-reduce:
    when it completes on a rank, every rank has reached that point of its stream). A rank writes
    into the others' buffers with endia_b200_copy_strided (plain stores over NVLink).

    Creation is collective and every step of it ends in an agreement (an all-reduce of a success
    flag that every rank reaches whether its own step worked or not), so a failure on one rank -
    an allocation that does not fit, a peer that cannot be mapped - makes ALL ranks release what
    they hold and use the NCCL all-to-all instead; no rank is left inside a collective alone."""

    _cache = {}

    # the four device primitives (class attributes so that a host-side test can stand in for them)
    @staticmethod
    def _ipc_alloc(nbytes):
        import ctypes as C
        from . import _lib
        local, handle = C.c_void_p(), (C.c_ubyte * 64)()
        _lib.call("endia_b200_ipc_alloc", int(nbytes), C.byref(local), handle)
        return local.value, bytes(handle)

    @staticmethod
    def _ipc_open(handle):
        import ctypes as C
        from . import _lib
        p = C.c_void_p()
        _lib.call("endia_b200_ipc_open", (C.c_ubyte * 64).from_buffer_copy(handle), C.byref(p))
        return p.value

    @staticmethod
    def _ipc_close(ptr):
        from . import _lib
        _lib.call("endia_b200_ipc_close", ptr)

    @staticmethod
    def _ipc_free(ptr):
        from . import _lib
        _lib.call("endia_b200_ipc_free", ptr)

    @staticmethod
    def _flag_device(group):
        return device() if dist.get_backend(group) == "nccl" else torch.device("cpu")

    @classmethod
    def _agree(cls, ok, group):
        """True when `ok` holds on every rank (a collective: every rank must call it)."""
        flag = torch.tensor([1.0 if ok else 0.0], device=cls._flag_device(group))
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
        return float(flag.item()) > 0.0

    @classmethod
    def get(cls, nbytes, group=None):
        """Buffers of at least nbytes, created collectively on first use and reused; None when the
        ranks cannot map each other's memory (the exchange then goes through NCCL). Every rank of
        the group must call this with the same nbytes."""
        key = id(group)
        cur = cls._cache.get(key)
        if cur is not None and (cur is False or cur.nbytes >= nbytes):
            return cur or None
        if cur:
            cur.close()          # replaced by larger buffers (all ranks take this branch together)
        made = cls._create(int(nbytes), group)
        cls._cache[key] = made if made is not None else False
        return made

    @classmethod
    def release(cls, group=None):
        """Unmap and free the group's buffers (collective); the next get() creates new ones."""
        cur = cls._cache.pop(id(group), None)
        if cur:
            cur.close()

    @classmethod
    def _create(cls, nbytes, group):
        debug = os.environ.get("ENDIA_B200_DEBUG")
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        local, handle, why = None, b"", None
        try:
            local, handle = cls._ipc_alloc(nbytes)
        except Exception as exc:          # e.g. the buffer does not fit on this rank's device
            why = exc
        if not cls._agree(local is not None, group):
            if local is not None:
                cls._ipc_free(local)
            if debug:
                print("endia_b200: peer buffers unavailable (allocation: %s); using NCCL all-to-all" % (why,))
            return None
        handles = [None] * world
        dist.all_gather_object(handles, handle, group=group)
        ptrs, opened = [None] * world, []
        try:
            for r, h in enumerate(handles):
                if r == rank:
                    ptrs[r] = local
                else:
                    ptrs[r] = cls._ipc_open(h)
                    opened.append(ptrs[r])
        except Exception as exc:          # e.g. no peer access between the devices
            why = exc
        if not cls._agree(why is None, group):
            for p in opened:
                cls._ipc_close(p)
            dist.barrier(group=group)     # every rank has unmapped before any rank frees
            cls._ipc_free(local)
            if debug:
                print("endia_b200: peer buffers unavailable (mapping: %s); using NCCL all-to-all" % (why,))
            return None
        self = cls.__new__(cls)
        self.nbytes, self.group, self.rank, self.world = nbytes, group, rank, world
        self.ptrs = ptrs
        self._flag = torch.zeros(1, device=cls._flag_device(group))
        self.closed = False
        return self

    def close(self):
        """Collective: unmap the peers' buffers, wait until every rank has, free the own buffer."""
        if self.closed:
            return
        self.closed = True
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        for r, p in enumerate(self.ptrs):
            if r != self.rank:
                self._ipc_close(p)
        dist.barrier(group=self.group)
        self._ipc_free(self.ptrs[self.rank])
        self.ptrs = []

    def barrier(self):
        dist.all_reduce(self._flag, group=self.group)

    def tensor(self, rank, shape, stride, offset=0, is_complex=True):
        """C descriptor of a view of rank `rank`'s buffer."""
        from ._lib import Tensor as _CTensor
        t = _CTensor()
        t.data = self.ptrs[rank]
        for i, (e, st) in enumerate(zip(shape, stride)):
            t.shape[i] = e
            t.stride[i] = st
        t.offset = offset
        t.ndim = len(shape)
        t.is_complex = 1 if is_complex else 0
        return t

    def local_array(self, shape):
        """This rank's buffer as a contiguous complex Array (no copy, not owned by the Array)."""
        n = 1
        for e in shape:
            n *= e
        a = Array(ArrayShape(shape))
        a.is_complex_flag = True
        a.buf = _wrap_device_memory(self.ptrs[self.rank], 2 * n)
        a._keepalive = self
        return a


def _wrap_device_memory(ptr, n_floats):
    """float32 torch tensor over device memory this library allocated itself."""
    class _Mem:
        pass
    holder = _Mem()
    holder.__cuda_array_interface__ = {"shape": (int(n_floats),), "typestr": "<f4", "data": (int(ptr), False),
                                       "version": 3, "strides": None}
    return torch.as_tensor(holder, device=device())


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

    peers = None
    if world > 1 and dist.is_initialized() and dist.get_backend(group) == "nccl" \
            and os.environ.get("ENDIA_B200_SLAB_PEER", "1") != "0":
        peers = PeerBuffers.get(8 * s0 * n1 * n2, group)
    rank = dist.get_rank(group) if (dist.is_initialized() and world > 1) else 0

    def push(src_desc_of_block, dst_desc_of_block):
        """Each rank writes block q of its array into its place in rank q's buffer; the barriers
        order the writes against the previous and the next readers of the buffers."""
        from . import _lib
        from ._array import stream
        peers.barrier()
        for i in range(world):
            q = (rank + i) % world          # start with the own block, then round-robin over the peers
            _lib.call("endia_b200_copy_strided", src_desc_of_block(q), dst_desc_of_block(q), stream())
        peers.barrier()

    def forward_impl(x):
        y1 = new_like([s0, n1, n2])
        run_fft(x, y1, [1, 2], False, 1.0)
        if peers is not None:
            # block q = y1[:, q*s1:(q+1)*s1, :] lands as rows [rank*s0, (rank+1)*s0) of rank q's
            # [n0, s1, n2] array: packing, exchange and placement in one pass
            push(lambda q: _strided_view(y1, [s0, s1, n2], [n1 * n2, n2, 1], q * s1 * n2).desc(),
                 lambda q: peers.tensor(q, [s0, s1, n2], [s1 * n2, n2, 1], rank * s0 * s1 * n2))
            out = new_like([n0, s1, n2])
            run_fft(peers.local_array([n0, s1, n2]), out, [0], False, 1.0)
            return out
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
        if peers is not None:
            # block q = g0[q*s0:(q+1)*s0] lands as columns [rank*s1, (rank+1)*s1) of axis 1 of rank
            # q's [s0, n1, n2] array (a strided destination): no unpacking pass
            push(lambda q: _strided_view(g0, [s0, s1, n2], [s1 * n2, n2, 1], q * s0 * s1 * n2).desc(),
                 lambda q: peers.tensor(q, [s0, s1, n2], [n1 * n2, n2, 1], rank * s1 * n2))
            dx = new_like([s0, n1, n2])
            run_fft(peers.local_array([s0, n1, n2]), dx, [1, 2], True, 1.0)
            return dx
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
