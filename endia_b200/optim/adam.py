"""Adam (endia/optim/adam.mojo:17-65) as one fused multi-tensor kernel per step."""
import ctypes as C

from .. import _lib
from .._array import Array, ArrayShape, alloc, stream
from ..functional._utils import contiguous, broadcast_shapes


class Adam:
    def __init__(self, params, lr=0.001, beta1=0.9, beta2=0.999, eps=1e-8):
        self.params = list(params)
        self.lr, self.beta1, self.beta2, self.eps = lr, beta1, beta2, eps
        self.t = 1.0  # the step count starts at 1 (adam.mojo:40)
        self.m = [Array(p.shape()) for p in self.params]
        self.v = [Array(p.shape()) for p in self.params]
        self.grad_scale = 1.0  # folded into the gradient read (1/world_size under data parallelism)

    # ---- steps replayed from a CUDA graph (utils.CapturedStep(..., optimizers=[self])) -----------
    def begin_capture(self):
        """The step count moves to a device float (a host value would be frozen in the graph); called
        by CapturedStep before it captures."""
        from ..functional.init_ops import full
        self._t_dev = full([1], self.t)

    def end_capture(self):
        """Steps enqueued op by op again (the host count is kept current by after_replay)."""
        self._t_dev = None

    def after_replay(self):
        self.t += 1.0

    def reset_state(self):
        """Zero moments with the parameters' shapes and t = 1, as after construction."""
        self.t = 1.0
        if getattr(self, "_t_dev", None) is not None:
            _lib.call("endia_b200_fill", self._t_dev.data_ptr(), 1, 0, 1.0, 0.0, stream())
        for i, p in enumerate(self.params):
            for st in (self.m[i], self.v[i]):
                st.array_shape_ = ArrayShape(p.shape())
                if st.size():
                    _lib.call("endia_b200_memset0", st.data_ptr(), st.size() * 4, stream())

    def step(self):
        from .._array import flush_readers
        n = len(self.params)
        grads = []
        for p in self.params:
            flush_readers(p)
            if not p.is_contiguous():
                raise _lib.EndiaError(_lib.EINVAL, "Adam: parameters must be contiguous arrays")
            grads.append(contiguous(p.grad()))  # zeros when no gradient is stored (_array.mojo:695-698)
        P = (C.c_void_p * n)(*[p.data_ptr() for p in self.params])
        G = (C.c_void_p * n)(*[g.data_ptr() for g in grads])
        M = (C.c_void_p * n)(*[m.data_ptr() for m in self.m])
        V = (C.c_void_p * n)(*[v.data_ptr() for v in self.v])
        numel = (C.c_int64 * n)(*[p.size() for p in self.params])
        for p, g in zip(self.params, grads):
            if g.size() != p.size():
                raise _lib.EndiaError(_lib.ESHAPE, "Adam: gradient %s does not match parameter %s" % (
                    g.shape(), p.shape()))
        # Matrices also get the operand parts of their new value (the bf16 split the two-CTA GEMM
        # reads), so that the products of the next step need not recompute them for the weights
        # (the cache is dropped by any other in-place update).
        parts = []
        for p in self.params:
            if p.ndim() == 2 and p.size() % 8 == 0 and p.size() >= 128 * 128 and not p.is_complex():
                if getattr(p, "_pair16", None) is None:
                    p._pair16 = alloc(p.size())
                p._tf32_lo = None
                p._parts_ptr = p.buf.data_ptr()
                parts.append(p._pair16.data_ptr())
            else:
                p._tf32_lo = None
                p._pair16 = None
                parts.append(None)
        P16 = (C.c_void_p * n)(*parts)
        t_dev = getattr(self, "_t_dev", None)
        if t_dev is not None:
            _lib.call("endia_b200_adam_step_multi_graph", n, P, G, M, V, P16, numel, self.lr, self.beta1,
                      self.beta2, self.eps, t_dev.data_ptr(), 1, self.grad_scale, stream())
        else:
            _lib.call("endia_b200_adam_step_multi_bf16", n, P, G, M, V, P16, numel, self.lr, self.beta1,
                      self.beta2, self.eps, self.t, self.grad_scale, stream())
        # m and v take the broadcast shape of (state, grad): a bias gradient is (1, N), so the
        # moments become (1, N) while the parameter keeps (N) (adam.mojo:49-56, expand_op.mojo:121-126).
        for i, g in enumerate(grads):
            shp = broadcast_shapes(self.m[i].shape(), g.shape())
            self.m[i].array_shape_ = ArrayShape(shp)
            self.v[i].array_shape_ = ArrayShape(shp)
        import torch
        if not torch.cuda.is_current_stream_capturing():
            self.t += 1.0     # (a step being captured is not run; after_replay counts its replays)
