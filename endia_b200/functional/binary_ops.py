"""Binary elementwise ops with numpy broadcasting and matmul
(endia/functional/binary_ops/). Forward passes enqueue one vectorised kernel that reads
broadcast operands through stride-0 dims; VJPs are compositions of these same ops, so gradients
of gradients work (create_graph=True). When no graph of the gradient is wanted the VJPs switch to
fused single-pass kernels."""
import os

from .. import _lib
from .._array import Array, ArrayShape, alloc, stream
from ..autograd import state as _state
from ._utils import (op_array, setup_shape_and_data, broadcast_shapes, launch_binary, contiguous)
from .view_ops import expand


def _binary_call(opcode):
    def call(curr, args):
        setup_shape_and_data(curr)
        if curr.size():
            launch_binary(opcode, args[0], args[1], curr)
    return call


def binary_op_array(arg0, arg1, name, opcode, vjp, jvp=None):
    """Expand both args to the broadcast shape (views), then register the op on the expanded
    args (binary_ops/_utils.mojo:57-90)."""
    shape = broadcast_shapes(arg0.shape(), arg1.shape())
    a0, a1 = expand(arg0, shape), expand(arg1, shape)
    defer = {}
    if opcode == _lib.BIN_MUL:
        # real(fftn(x)) * w with a plain real w of the same shape: see _deferred.py
        from ._deferred import is_pending, Deferred
        for u, v in ((a0, a1), (a1, a0)):
            if is_pending(u, "re") and not isinstance(v, Deferred) and not v.is_complex() \
                    and not v.requires_grad() and v.is_contiguous() and v.shape() == u.shape():
                defer = {"deferred": "rew", "root": u.root, "w": v}
                break
    return op_array(ArrayShape(shape), [a0, a1], name, _binary_call(opcode), vjp=vjp, jvp=jvp, **defer)


def _zero():
    return Array(0)


def _add_vjp(primals, grad, out):  # add_op.mojo:107-110
    return [grad if primals[0].requires_grad() else _zero(),
            grad if primals[1].requires_grad() else _zero()]


def _sub_vjp(primals, grad, out):  # sub_op.mojo:109-112
    from .unary_ops import neg
    return [grad if primals[0].requires_grad() else _zero(),
            neg(grad) if primals[1].requires_grad() else _zero()]


def _mul_vjp(primals, grad, out):  # mul_op.mojo:125-128 (no conjugation)
    return [mul(grad, primals[1]) if primals[0].requires_grad() else _zero(),
            mul(grad, primals[0]) if primals[1].requires_grad() else _zero()]


def _div_vjp(primals, grad, out):  # div_op.mojo:108-114
    from .unary_ops import neg
    lhs = div(grad, primals[1]) if primals[0].requires_grad() else _zero()
    rhs = div(mul(neg(grad), primals[0]), mul(primals[1], primals[1])) if primals[1].requires_grad() else _zero()
    return [lhs, rhs]


def _pow_vjp(primals, grad, out):  # pow_op.mojo:109-115
    from .unary_ops import log
    lhs = mul(mul(grad, primals[1]), div(out, primals[0])) if primals[0].requires_grad() else _zero()
    rhs = mul(mul(grad, out), log(primals[0])) if primals[1].requires_grad() else _zero()
    return [lhs, rhs]


# Forward-mode rules (the `jvp` slot of each op: add_op.mojo, sub_op.mojo, mul_op.mojo, div_op.mojo,
# pow_op.mojo, matmul_op.mojo): tangents in, tangent out.
def _div_jvp(p, t):
    return sub(div(t[0], p[1]), div(mul(p[0], t[1]), mul(p[1], p[1])))


def _pow_jvp(p, t):
    from .unary_ops import log
    out = pow_to(p[0], p[1])
    return add(mul(mul(t[0], p[1]), div(out, p[0])), mul(mul(t[1], out), log(p[0])))


def add(arg0, arg1):
    return binary_op_array(arg0, arg1, "add", _lib.BIN_ADD, _add_vjp, jvp=lambda p, t: add(t[0], t[1]))


def sub(arg0, arg1):
    return binary_op_array(arg0, arg1, "sub", _lib.BIN_SUB, _sub_vjp, jvp=lambda p, t: sub(t[0], t[1]))


def mul(arg0, arg1):
    return binary_op_array(arg0, arg1, "mul", _lib.BIN_MUL, _mul_vjp,
                           jvp=lambda p, t: add(mul(t[0], p[1]), mul(p[0], t[1])))


def div(arg0, arg1):
    return binary_op_array(arg0, arg1, "div", _lib.BIN_DIV, _div_vjp, jvp=_div_jvp)


def pow_to(arg0, arg1):
    return binary_op_array(arg0, arg1, "pow_to", _lib.BIN_POW, _pow_vjp, jvp=_pow_jvp)


pow = pow_to


def fused_binary(opcode, a, b):
    """Gradient-free single-pass kernel for the fused VJP forms (ENDIA_B200_BIN_*_BWD)."""
    shape = broadcast_shapes(a.shape(), b.shape())
    a0, a1 = expand(a, shape), expand(b, shape)
    out = Array(ArrayShape(shape))
    out.is_complex_flag = a.is_complex() or b.is_complex()
    setup_shape_and_data(out)
    if out.size():
        launch_binary(opcode, a0, a1, out)
    return out


# ------------------------------------------------------------------------------ matmul
def _matmul_shape(s0, s1):
    """Result shape of a batched product (binary_ops/matmul_op.mojo:36-90)."""
    if len(s0) < 2 or len(s1) < 2:
        raise _lib.EndiaError(_lib.ESHAPE, "Error: matmul needs arrays of at least 2 dims")
    if s0[-1] != s1[-2]:
        raise _lib.EndiaError(_lib.ESHAPE, "Error: matmul shapes are incompatible: %s @ %s" % (s0, s1))
    batch = broadcast_shapes(s0[:-2], s1[:-2])
    return batch, batch + [s0[-2], s1[-1]]


def _matrix_layout(a):
    """(transposed, leading dimension) when the last two dims of `a` can feed the GEMM without a
    copy: row-major [r, c] (stride (ld, 1)) or its transposed view (stride (1, ld))."""
    r, c = a.shape()[-2], a.shape()[-1]
    sr, sc = a.stride()[-2], a.stride()[-1]
    if (sc == 1 or c == 1) and (sr >= c or r == 1) and sr != 0:
        return 0, (sr if r > 1 else max(c, 1))
    if (sr == 1 or r == 1) and (sc >= r or c == 1) and sc != 0:
        return 1, (sc if c > 1 else max(r, 1))
    return None


def _batch_stride(a, batch):
    """Single element stride between consecutive batch matrices, or None if not expressible."""
    nb = len(batch)
    if nb == 0:
        return 0
    lead_shape, lead_stride = a.shape()[:-2], a.stride()[:-2]
    total = 1
    for s in batch:
        total *= s
    if total == 1:
        return 0
    if all(st == 0 for st, e in zip(lead_stride, lead_shape) if e != 1):
        return 0
    expect = None
    for e, st in zip(reversed(lead_shape), reversed(lead_stride)):
        if e == 1:
            continue
        if expect is None:
            expect = st * e
            base = st
        else:
            if st != expect:
                return None
            expect = st * e
    return base


_LO_CACHE_MIN = 1 << 20


def _tc_plan(M, N, K, nbatch, algo, linear=True):
    """Which operand parts the tcgen05 kernel that endia_b200_gemm will pick reads: "pair16" (bf16
    split, two-CTA kernel), "lo32" (fp32 low parts, 3xTF32 kernels) or None (FFMA / skinny kernels).
    A wrong guess only costs time: the kernel computes the parts it was not handed."""
    if nbatch != 1 or algo == _lib.GEMM_FFMA or M < 128 or N < 128 or K < 32:
        return None
    if K > 8192:
        # longer reductions run on the two-CTA kernel, which cuts them into short runs, unless the
        # epilogue accumulates into C (beta); otherwise on the FFMA kernel (unless the algorithm is named)
        if N >= 256 and linear:
            return "lo32" if algo == _lib.GEMM_3XTF32 else "pair16"
        return None if algo == _lib.GEMM_AUTO else ("lo32" if algo == _lib.GEMM_3XTF32 or N < 256 else "pair16")
    if algo == _lib.GEMM_3XTF32 or N < 256:
        return "lo32"
    if algo == _lib.GEMM_AUTO and os.environ.get("ENDIA_B200_TC_SCHEME", "")[:1] in ("3", "0"):
        return "lo32"
    return "pair16"


def _operand_parts_ptr(x, kind):
    """Device address of the operand parts (`kind`: "lo32" or "pair16") matching operand view `x`,
    or None. The parts of a whole storage buffer serve every view of it that starts at its first
    element. They are written by the optimizer for weights and computed here once for the result
    of an op (used by two products: the next layer's forward and a weight gradient). Leaves (user
    inputs, parameters) are not cached here, because their storage may be rewritten between steps;
    except while a step is being captured as a CUDA graph (utils.CapturedStep): nothing outside
    the step can write between its ops then, so a leaf is split once per step instead of once per
    product, and the parts are forgotten when the capture ends."""
    base = x.base()
    if base.buf is None or x.buf is not base.buf or base.is_complex():
        return None
    attr = "_tf32_lo" if kind == "lo32" else "_pair16"
    parts = getattr(base, attr, None)
    if parts is None or base._parts_ptr != base.buf.data_ptr():
        n = base.buf.numel()
        leaf = base.name == "arg"
        if (leaf and _state.capture_parts is None) or n < _LO_CACHE_MIN or n % 8 or not _state.cache_tf32_lo:
            return None
        if leaf:
            _state.capture_parts.append(base)
        parts = alloc(n)
        if kind == "lo32":
            _lib.call("endia_b200_tf32_split", base.buf.data_ptr(), parts.data_ptr(), 1, n, n, n, stream())
        else:
            _lib.call("endia_b200_bf16_split", base.buf.data_ptr(), parts.data_ptr(), n, stream())
        setattr(base, attr, parts)
        base._parts_ptr = base.buf.data_ptr()
    off = x.data_ptr() - base.buf.data_ptr()
    if kind == "pair16":
        # [bf16(x) | bf16(lo)] of the whole buffer: only a view that covers all of it can use it
        return parts.data_ptr() if off == 0 and x.size() == base.buf.numel() else None
    return parts.data_ptr() + off


def gemm_arrays(a, b, out, epi=None, algo=None):
    """out = a @ b over the last two dims; a and b are already expanded over the batch dims.
    Transposed views are passed as such (no materialised copy, unlike matmul_op.mojo:107-136)."""
    batch = out.shape()[:-2]
    nbatch = 1
    for s in batch:
        nbatch *= s
    M, N, K = out.shape()[-2], out.shape()[-1], a.shape()[-1]
    la, lb = _matrix_layout(a), _matrix_layout(b)
    sa, sb = _batch_stride(a, batch), _batch_stride(b, batch)
    if la is None or sa is None:
        a = contiguous(a)
        la, sa = _matrix_layout(a), _batch_stride(a, batch)
    if lb is None or sb is None:
        b = contiguous(b)
        lb, sb = _matrix_layout(b), _batch_stride(b, batch)
    if algo is None:
        algo = _state.gemm_algo
    if out.is_complex():
        if not (a.is_complex() and b.is_complex()):
            raise _lib.EndiaError(_lib.EINVAL, "matmul of a complex and a real array is not supported")
        _lib.call("endia_b200_gemm_complex", la[0], lb[0], M, N, K, a.data_ptr(), la[1], b.data_ptr(),
                  lb[1], out.data_ptr(), N, nbatch, sa, sb, M * N, stream())
        return
    # Operand parts kept beside an operand's storage are handed to the tensor-core kernel instead
    # of being recomputed per product.
    linear = epi is None or not epi.beta     # (the kernel's short accumulation runs need beta == 0)
    plan = _tc_plan(M, N, K, nbatch, algo, linear)
    if plan is not None:
        pa, pb = _operand_parts_ptr(a, plan), _operand_parts_ptr(b, plan)
        if pa or pb:
            if epi is None:
                epi = _lib.Epilogue()
                epi.alpha = 1.0
            if plan == "lo32":
                epi.a_lo, epi.b_lo = pa, pb
            else:
                epi.a16, epi.b16 = pa, pb
    timer = _state.gemm_timer
    if timer is not None:
        timer.start(2.0 * M * N * K * nbatch)
    _lib.call("endia_b200_gemm", la[0], lb[0], M, N, K, a.data_ptr(), la[1], b.data_ptr(), lb[1],
              out.data_ptr(), N, nbatch, sa, sb, M * N, epi, algo, stream())
    if timer is not None:
        timer.stop()


def _matmul_call(curr, args):
    setup_shape_and_data(curr)
    if curr.size():
        gemm_arrays(args[0], args[1], curr)


def _matmul_vjp(primals, grad, out):
    # dX = g @ W.T, dW = X.T @ g, each a new differentiable matmul on a transposed view
    # (matmul_op.mojo:278-284). The product with a square W is the mathematically correct one.
    lhs = matmul(grad, primals[1].T()) if _state.wants_grad(primals[0]) else _zero()
    rhs = matmul(primals[0].T(), grad) if _state.wants_grad(primals[1]) else _zero()
    return [lhs, rhs]


def matmul(arg0, arg1):
    batch, shape = _matmul_shape(arg0.shape(), arg1.shape())
    a0 = expand(arg0, batch + arg0.shape()[-2:], ignore_axes=(-2, -1))
    a1 = expand(arg1, batch + arg1.shape()[-2:], ignore_axes=(-2, -1))
    return op_array(ArrayShape(shape), [a0, a1], "matmul", _matmul_call, vjp=_matmul_vjp,
                    jvp=lambda p, t: add(matmul(t[0], p[1]), matmul(p[0], t[1])))
