"""MLP layers (endia/nn/modules/_mlp.mojo:17-82). A layer `act(x @ W + b)` runs as ONE GEMM whose
epilogue adds the bias and applies the activation; its VJP is one fused mask+bias-gradient kernel
and two GEMMs that read transposed operands in place. With create_graph=True the VJP is the
reference's composition of differentiable ops instead, so higher-order gradients work."""
from .. import _lib
from .._array import Array, ArrayShape, alloc, stream
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


def _act_bwd_graph(act, out, grad):
    """act'(.) * grad written in differentiable ops of the layer OUTPUT (relu_op.mojo:95,
    tanh_op.mojo:92, sigmoid_op.mojo:98)."""
    if act == _lib.ACT_RELU:
        return mul(greater(out, Array([out.shape()[-1]])), grad)
    if act == _lib.ACT_TANH:
        return mul(1.0 - square(out), grad)
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
        gemm_arrays(a[0], a[1], curr, epi=epi)

    def vjp(primals, grad, out):
        xp, wp = primals[0], primals[1]
        zero = Array(0)
        if _state.create_graph:
            ds = _act_bwd_graph(act, out, grad)
            dx = matmul(ds, wp.T()) if xp.requires_grad() else zero
            dw = matmul(xp.T(), ds) if wp.requires_grad() else zero
            res = [dx, dw]
            if bias is not None:
                res.append(reduce_add(ds, [0]) if primals[2].requires_grad() else zero)
            return res
        need_db = bias is not None and primals[2].requires_grad()
        g = contiguous(grad)
        db = None
        if act or need_db:
            ds = Array(ArrayShape([B, N])) if act else g
            if act:
                setup_shape_and_data(ds)
            if need_db:
                db = Array(ArrayShape([1, N]))  # kept dim, like Expand.vjp's reduce_add
                setup_shape_and_data(db)
            nbytes = _lib.lib.endia_b200_act_bwd_colsum_scratch_bytes(B, N) if need_db else 0
            scratch = alloc((nbytes + 3) // 4) if nbytes else None
            _lib.call("endia_b200_act_bwd_colsum", act, out.data_ptr(), g.data_ptr(),
                      ds.data_ptr() if act else None, db.data_ptr() if need_db else None, B, N,
                      scratch.data_ptr() if scratch is not None else None, stream())
        else:
            ds = g
        res = []
        if xp.requires_grad():
            dx = Array(ArrayShape(xp.shape()))
            setup_shape_and_data(dx)
            gemm_arrays(ds, wp.T(), dx)
            res.append(dx)
        else:
            res.append(zero)
        if wp.requires_grad():
            dw = Array(ArrayShape(wp.shape()))
            setup_shape_and_data(dw)
            gemm_arrays(xp.T(), ds, dw)
            res.append(dw)
        else:
            res.append(zero)
        if bias is not None:
            res.append(db if need_db else zero)
        return res
    return op_array(ArrayShape([B, N]), args, "linear", call, vjp=vjp)


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
