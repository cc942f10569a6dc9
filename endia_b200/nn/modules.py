"""MLP layers (endia/nn/modules/_mlp.mojo:17-82). A layer `act(x @ W + b)` runs as ONE GEMM whose
epilogue adds the bias and applies the activation; its VJP is one fused mask+bias-gradient kernel
and two GEMMs that read transposed operands in place. With create_graph=True the VJP is the
reference's composition of differentiable ops instead, so higher-order gradients work."""
from .. import _lib
from .._array import Array, ArrayShape, alloc, stream, drop_operand_parts, flush_readers
from ..autograd import state as _state
from ..functional import init_ops
from ..functional._utils import op_array, setup_shape_and_data, contiguous
from ..functional.binary_ops import matmul, mul, add, gemm_arrays
from ..functional.comparison_ops import greater
from ..functional.reduce_ops import reduce_add
from ..functional.unary_ops import relu, tanh, sigmoid, square

_ACTS = {None: _lib.ACT_NONE, "none": _lib.ACT_NONE, "relu": _lib.ACT_RELU, "tanh": _lib.ACT_TANH,
         "sigmoid": _lib.ACT_SIGMOID}
_ACT_FNS = {_lib.ACT_RELU: relu, _lib.ACT_TANH: tanh, _lib.ACT_SIGMOID: sigmoid}


def _tanh_out_bwd(y, g):
    """(1 - y^2) * g for a tanh output y (tanh_op.mojo:92) as ONE differentiable op instead of the
    square / sub / mul chain: one pass here, and in the backward pass of a gradient penalty
    dg = (1 - y^2) * G (one pass) and dy = -2 * y * g * G (two passes) instead of the chain's
    ten. With create_graph set again its VJP is written in differentiable ops."""
    from ..functional.binary_ops import fused_binary, binary_op_array

    def vjp(primals, grad, out):
        yy, gg = primals
        zero = Array(0)
        if _state.create_graph:
            dy = mul(mul(yy * -2.0, gg), grad) if yy.requires_grad() else zero
            dg = _tanh_out_bwd(yy, grad) if gg.requires_grad() else zero
        else:
            dy = fused_binary(_lib.BIN_TANH_OUT_BWD2, yy, fused_binary(_lib.BIN_MUL, gg, grad)) \
                if yy.requires_grad() else zero
            dg = fused_binary(_lib.BIN_TANH_OUT_BWD, yy, grad) if gg.requires_grad() else zero
        return [dy, dg]

    def jvp(p, t):
        # d[(1 - y^2) g] = -2 y g dy + (1 - y^2) dg
        return add(mul(mul(p[0] * -2.0, p[1]), t[0]), _tanh_out_bwd(p[0], t[1]))
    return binary_op_array(y, g, "tanh_out_bwd", _lib.BIN_TANH_OUT_BWD, vjp, jvp=jvp)


def _act_bwd_graph(act, out, grad):
    """act'(.) * grad written in differentiable ops of the layer OUTPUT (relu_op.mojo:95,
    tanh_op.mojo:92, sigmoid_op.mojo:98)."""
    if act == _lib.ACT_RELU:
        return mul(greater(out, Array([out.shape()[-1]])), grad)
    if act == _lib.ACT_TANH:
        return _tanh_out_bwd(out, grad)
    if act == _lib.ACT_SIGMOID:
        return mul(mul(out, 1.0 - out), grad)
    return grad


def linear(x, weight, bias=None, activation=None):
    """act(x @ weight + bias) for 2-D x (B, K), weight (K, N), bias (N). Other ranks use the
    unfused op composition of the reference (_mlp.mojo:50-52)."""
    act = _ACTS[activation]
    if x.ndim() != 2 or weight.ndim() != 2 or (bias is not None and bias.ndim() != 1) or x.is_complex() \
            or weight.is_complex():
        pred = matmul(x, weight)
        if bias is not None:
            pred = add(pred, bias)
        return _ACT_FNS[act](pred) if act else pred
    if x.shape()[1] != weight.shape()[0] or (bias is not None and bias.shape()[0] != weight.shape()[1]):
        raise _lib.EndiaError(_lib.ESHAPE, "linear: incompatible shapes %s @ %s + %s" % (
            x.shape(), weight.shape(), bias.shape() if bias is not None else None))
    B, N = x.shape()[0], weight.shape()[1]
    args = [x, weight] + ([bias] if bias is not None else [])

    def call(curr, a):
        setup_shape_and_data(curr)
        if curr.size() == 0:
            return
        epi = _lib.Epilogue()
        epi.alpha, epi.beta, epi.act = 1.0, 0.0, act
        if bias is not None:
            epi.bias = contiguous(a[2]).data_ptr()
        # The layer's output feeds two products (the next layer's forward and its weight gradient):
        # when those run on the bf16-compensated kernel, this product's epilogue writes their
        # operand parts instead of a split kernel later.
        parts = None
        if _state.cache_tf32_lo and curr.requires_grad_flag and (B * N) % 8 == 0 and B * N >= (1 << 20):
            from ..functional.binary_ops import _tc_plan
            if _tc_plan(B, N, N, 1, _state.gemm_algo) == "pair16":
                parts = alloc(B * N)
                epi.c16 = parts.data_ptr()
        gemm_arrays(a[0], a[1], curr, epi=epi)
        if parts is not None:
            curr._pair16 = parts
            curr._parts_ptr = curr.buf.data_ptr()

    def vjp(primals, grad, out):
        xp, wp = primals[0], primals[1]
        zero = Array(0)
        if _state.create_graph:
            ds = _act_bwd_graph(act, out, grad)
            dx = matmul(ds, wp.T()) if _state.wants_grad(xp) else zero
            dw = matmul(xp.T(), ds) if _state.wants_grad(wp) else zero
            res = [dx, dw]
            if bias is not None:
                res.append(reduce_add(ds, [0]) if _state.wants_grad(primals[2]) else zero)
            return res
        need_db = bias is not None and _state.wants_grad(primals[2])
        g = contiguous(grad)
        db = None
        if getattr(grad, "_masked_for", None) is out:
            # the layer above already applied this layer's activation derivative and summed the
            # bias gradient in the epilogue of its dX product
            ds, db = g, grad._db
        elif act or need_db:
            ds = Array(ArrayShape([B, N])) if act else g
            if act:
                ds.name = "linear_vjp"   # a temporary of this pass, never rewritten (see _operand_parts_ptr)
                setup_shape_and_data(ds)
            if need_db:
                db = Array(ArrayShape([1, N]))  # kept dim, like Expand.vjp's reduce_add
                setup_shape_and_data(db)
            nbytes = _lib.lib.endia_b200_act_bwd_colsum_scratch_bytes(B, N) if need_db else 0
            scratch = alloc((nbytes + 3) // 4) if nbytes else None
            # dS feeds two products (dX and dW): when they run on the bf16-compensated kernel its
            # operand parts are written in this pass instead of by a split kernel later
            parts = None
            if act and _state.cache_tf32_lo and (B * N) % 8 == 0 and B * N >= (1 << 20):
                from ..functional.binary_ops import _tc_plan
                if "pair16" in (_tc_plan(B, xp.shape()[1], N, 1, _state.gemm_algo),
                                _tc_plan(xp.shape()[1], N, B, 1, _state.gemm_algo)):
                    parts = alloc(B * N)
            _lib.call("endia_b200_act_bwd_colsum_parts", act, out.data_ptr(), g.data_ptr(),
                      ds.data_ptr() if act else None, db.data_ptr() if need_db else None, B, N,
                      scratch.data_ptr() if scratch is not None else None,
                      parts.data_ptr() if parts is not None else None, stream())
            if parts is not None:
                ds._pair16 = parts
                ds._parts_ptr = ds.buf.data_ptr()
        else:
            ds = g
        # The weight gradient first: nothing in the backward pass waits for it, but a data-parallel
        # hook (reduce-scatter / all-reduce) starts when it exists and then runs beside the dX product.
        dw = zero
        if _state.wants_grad(wp):
            dw = Array(ArrayShape(wp.shape()))
            setup_shape_and_data(dw)
            gemm_arrays(xp.T(), ds, dw)
            if getattr(wp, "grad_hook", None) is not None and xp.requires_grad():
                import torch
                dw._ready_event = torch.cuda.Event()     # "dw exists", ahead of the dX product
                dw._ready_event.record()
        dx = zero
        if _state.wants_grad(xp):
            dx = Array(ArrayShape(xp.shape()))
            dx.name = "linear_vjp"   # a temporary of this pass, never rewritten (see _operand_parts_ptr)
            setup_shape_and_data(dx)
            epi = _mask_epilogue_for(xp, dx)
            parts = None
            if epi is not None and _state.cache_tf32_lo and dx.size() % 8 == 0 and dx.size() >= (1 << 20):
                # dx is then the lower layer's dS, an operand of two more products
                from ..functional.binary_ops import _tc_plan
                rows, cols = xp.shape()
                if _tc_plan(rows, cols, cols, 1, _state.gemm_algo) == "pair16":
                    parts = alloc(dx.size())
                    epi.c16 = parts.data_ptr()
            gemm_arrays(ds, wp.T(), dx, epi=epi)
            if parts is not None:
                dx._pair16 = parts
                dx._parts_ptr = dx.buf.data_ptr()
        res = [dx, dw]
        if bias is not None:
            res.append(db if need_db else zero)
        return res
    def jvp(primals, tangents):
        # act'(out) * (dx @ W + x @ dW + db), from the ops the layer stands for
        z = matmul(primals[0], primals[1])
        dz = add(matmul(tangents[0], primals[1]), matmul(primals[0], tangents[1]))
        if bias is not None:
            z, dz = add(z, primals[2]), add(dz, tangents[2])
        if not act:
            return dz
        return _act_bwd_graph(act, _ACT_FNS[act](z), dz)
    res = op_array(ArrayShape([B, N]), args, "linear", call, vjp=vjp, jvp=jvp)
    res._lin_act = act
    res._lin_bias = bias
    return res


def _mask_epilogue_for(xp, dx):
    """When the input `xp` of a linear layer is itself the output of a fused linear layer with
    this layer as its only consumer, the dX product can finish that layer's backward step in its
    epilogue: dS = dX * act'(xp) and the bias gradient colsum(dS) (the mask of relu/tanh/sigmoid
    VJPs and Expand.vjp's reduction, fused into the GEMM's store). Marks `dx` so that the lower
    layer's VJP takes both as they are. Returns the epilogue, or None when this does not apply.
    Off unless state.fuse_mask_into_dx is set: the accumulators are drained while the tensor pipe
    waits, so work added to the epilogue costs more than the separate fused kernel it replaces
    (c2 step 7.1 ms without, 7.4 ms with)."""
    if not _state.fuse_mask_into_dx:
        return None
    if getattr(xp, "name", "") != "linear" or not hasattr(xp, "_lin_act") or xp.is_view or xp.has_grad() \
            or getattr(xp, "_consumers", 0) != 1 or not xp.is_contiguous() or xp.ndim() != 2:
        return None
    act_prev, bias_prev = xp._lin_act, xp._lin_bias
    need_db = bias_prev is not None and bias_prev.requires_grad()
    if not act_prev and not need_db:
        return None
    rows, cols = xp.shape()
    epi = _lib.Epilogue()
    epi.alpha, epi.beta = 1.0, 0.0
    keep = []
    if act_prev:
        epi.dact, epi.dact_src, epi.ld_dact = act_prev, xp.data_ptr(), cols
    db = None
    if need_db:
        db = Array(ArrayShape([1, cols]))    # kept dim, like Expand.vjp's reduce_add
        setup_shape_and_data(db)
        scratch = alloc(_lib.lib.endia_b200_gemm_colsum_scratch_bytes(rows, cols) // 4 + 1)
        epi.colsum, epi.colsum_scratch = db.data_ptr(), scratch.data_ptr()
        keep.append(scratch)
    dx._masked_for = xp
    dx._db = db
    dx._keep = keep        # the scratch must outlive the enqueued kernels' use of it
    return epi


class MLP:
    """Stack of linear layers (weights stored (in, out)); `activation` on all but the last layer.
    The reference hard-codes ReLU and He-normal initialisation (_mlp.mojo:34-43, 52)."""

    def __init__(self, hidden_dims, compute_backward=False, activation="relu"):
        self.weights, self.biases = [], []
        self.hidden_dims = list(hidden_dims)
        self.num_layers = len(hidden_dims) - 1
        self.compute_backward = compute_backward
        self.activation = activation
        for i in range(self.num_layers):
            self.weights.append(init_ops.rand_he_normal([hidden_dims[i], hidden_dims[i + 1]],
                                                        fan_in=hidden_dims[i],
                                                        requires_grad=compute_backward))
            self.biases.append(init_ops.rand_he_normal([hidden_dims[i + 1]], fan_in=hidden_dims[i],
                                                       requires_grad=compute_backward))

    def forward(self, x):
        pred = x
        for i in range(self.num_layers):
            last = i == self.num_layers - 1
            pred = linear(pred, self.weights[i], self.biases[i], None if last else self.activation)
        return pred

    __call__ = forward

    def params(self):
        out = []
        for w, b in zip(self.weights, self.biases):
            out += [w, b]
        return out

    def __str__(self):
        return "".join("Layer %d\n%s\n%s\n" % (i, w, b)
                       for i, (w, b) in enumerate(zip(self.weights, self.biases)))


def mlp(args, activation="relu"):
    """Functional form: args = [x, target, W0, b0, W1, b1, ...] (_mlp.mojo:71-82)."""
    pred = args[0]
    num_layers = (len(args) - 2) // 2
    for i in range(num_layers):
        last = i == num_layers - 1
        pred = linear(pred, args[2 * i + 2], args[2 * i + 3], None if last else activation)
    return pred


class SmallMLPStep:
    """Prepared single-launch training step for a small MLP (see fused_train_step): gradient
    buffers, the loss scalar and the argument arrays are built once, so that a step costs one
    C-ABI call on the host."""

    def __init__(self, weights, biases, optimizer=None, activation="relu"):
        import ctypes as C
        self.weights, self.biases, self.optimizer = list(weights), list(biases), optimizer
        L = self.L = len(self.weights)
        self.dims = [self.weights[0].shape()[0]] + [w.shape()[1] for w in self.weights]
        for p in self.weights + self.biases:
            if not p.is_contiguous() or p.is_complex():
                raise _lib.EndiaError(_lib.EINVAL, "fused_train_step: parameters must be contiguous and real")
        self.gW = [Array(ArrayShape(w.shape())) for w in self.weights]
        self.gb = [Array(ArrayShape([1, b.shape()[0]])) for b in self.biases]
        self.loss = Array(ArrayShape([1]))
        for g in self.gW + self.gb + [self.loss]:
            setup_shape_and_data(g)

        def ptrs(arrs):
            return (C.c_void_p * L)(*[a.data_ptr() for a in arrs])
        self.c_dims = (C.c_int32 * (L + 1))(*self.dims)
        self.p_W, self.p_b, self.p_gW, self.p_gb = ptrs(self.weights), ptrs(self.biases), ptrs(self.gW), ptrs(self.gb)
        self.act = _ACTS[activation]
        if optimizer is not None:
            if len(optimizer.params) != 2 * L or any(
                    optimizer.params[2 * i] is not self.weights[i] or optimizer.params[2 * i + 1] is not self.biases[i]
                    for i in range(L)):
                raise _lib.EndiaError(_lib.EINVAL, "fused_train_step: optimizer must hold [W0, b0, W1, b1, ...]")
            self.p_mW, self.p_vW = ptrs(optimizer.m[0::2]), ptrs(optimizer.v[0::2])
            self.p_mb, self.p_vb = ptrs(optimizer.m[1::2]), ptrs(optimizer.v[1::2])
        else:
            self.p_mW = self.p_vW = self.p_mb = self.p_vb = None
        self._fn = _lib.lib.endia_b200_mlp_small_step

    def __call__(self, x, target):
        batch = x.shape()[0]
        if x.shape() != [batch, self.dims[0]] or target.shape() != [batch, self.dims[-1]] or \
                not x.is_contiguous() or not target.is_contiguous():
            raise _lib.EndiaError(_lib.ESHAPE, "fused_train_step: x / target do not match the network")
        opt = self.optimizer
        if opt is not None:
            for p in self.weights + self.biases:
                flush_readers(p)
            st = self._fn(self.L, self.c_dims, batch, self.act, x.data_ptr(), target.data_ptr(), self.p_W, self.p_b,
                          self.p_gW, self.p_gb, self.p_mW, self.p_vW, self.p_mb, self.p_vb, self.loss.data_ptr(), 1,
                          opt.lr, opt.beta1, opt.beta2, opt.eps, opt.t, stream())
        else:
            st = self._fn(self.L, self.c_dims, batch, self.act, x.data_ptr(), target.data_ptr(), self.p_W, self.p_b,
                          self.p_gW, self.p_gb, None, None, None, None, self.loss.data_ptr(), 0,
                          0.0, 0.0, 0.0, 0.0, 1.0, stream())
        _lib.check(st)
        for w, b, g1, g2 in zip(self.weights, self.biases, self.gW, self.gb):
            if opt is not None:
                drop_operand_parts(w)
            w.grad_node = g1
            b.grad_node = g2
        if opt is not None:
            if opt.t == 1.0:   # bias moments take the gradient's (1, N) shape, as Adam.step does
                for i in range(self.L):
                    opt.m[2 * i + 1].array_shape_ = ArrayShape([1, self.dims[i + 1]])
                    opt.v[2 * i + 1].array_shape_ = ArrayShape([1, self.dims[i + 1]])
            opt.t += 1.0
        return self.loss


def fused_train_step(weights, biases, x, target, optimizer=None, activation="relu"):
    """One training step of a small MLP in a single kernel launch: forward, mse loss, backward and
    (when `optimizer` is an optim.Adam over exactly these parameters, weights and biases
    interleaved as MLP.params() returns them) the Adam update. Equivalent to

        loss = mse(mlp(x), target); loss.backward(); optimizer.step()

    for networks that fit one CTA's shared memory (EndiaError with status ELIMIT otherwise; use
    the layer-by-layer path then). Returns the loss (shape [1]; the same array is rewritten by the
    next call); every parameter's gradient is stored as by backward() (bias gradients with shape
    (1, N))."""
    key = (tuple(id(w) for w in weights), tuple(id(b) for b in biases), id(optimizer), activation)
    holder = weights[0]
    cached = getattr(holder, "_small_step", None)
    if cached is None or cached[0] != key:
        cached = (key, SmallMLPStep(weights, biases, optimizer, activation))
        holder._small_step = cached
    return cached[1](x, target)
