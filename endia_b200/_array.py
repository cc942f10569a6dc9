"""Device-resident Array (alias Tensor / ndarray): the storage and graph node of Endia
(endia/_array/_array.mojo:56-180 Node, :186-1165 Array) with the float32 buffer living in
B200 HBM. Shape, stride and offset metadata stay on the host and follow ArrayShape semantics
(endia/utils/_array_shape.mojo): element strides, one complex element = one (re, im) pair.

torch is used only as the device allocator / stream provider; every computation goes through the
C ABI of libendia_b200.so.
"""
import ast
import ctypes as C
import os

import numpy as np
import torch

from . import _lib
from ._lib import Tensor as _CTensor

_device = None
_SCALARS = {}   # (length, value) -> shared constant operand, see Array._scalar


def device():
    """The CUDA device of this process (LOCAL_RANK under torchrun), initialised on first use."""
    global _device
    if _device is None:
        if not torch.cuda.is_available():
            raise _lib.EndiaError(_lib.ENODEV, "no CUDA device is available; endia_b200 has no CPU fallback")
        idx = int(os.environ.get("LOCAL_RANK", os.environ.get("ENDIA_B200_DEVICE", "0")))
        torch.cuda.set_device(idx)
        _lib.call("endia_b200_init", idx)
        _device = torch.device("cuda", idx)
    return _device


def stream():
    """Raw cudaStream_t of torch's current stream; every kernel is enqueued on it."""
    return torch._C._cuda_getCurrentRawStream(device().index)


def alloc(n_floats):
    """Uninitialised float32 device storage (every kernel writes its whole output)."""
    return torch.empty(max(int(n_floats), 0), dtype=torch.float32, device=device())


def drop_operand_parts(arr):
    """Forget the cached GEMM operand parts (tf32 low part, bf16 split) of an array whose storage
    has just been rewritten in place."""
    base = arr.base()
    base._tf32_lo = None
    base._pair16 = None


def await_pending(arr):
    """Run and clear the completion callback a storage buffer carries, if any. An asynchronous
    writer (the all-gather of a sharded optimizer step) leaves one on the array it is still
    filling; every accessor of the device pointer calls this first, so a consumer on the compute
    stream waits for exactly the arrays it reads and no others."""
    base = getattr(arr, "base_", None)
    if base is None:
        base = arr
    cb = getattr(base, "_pending", None)
    if cb is not None:
        base._pending = None
        cb()


def watch_input(src, node):
    """Remember that `node`, an array whose kernel is still deferred (it has pending() and runs the
    kernel on access of `buf`), will read `src`'s storage."""
    import weakref
    base = src.base()
    readers = base.__dict__.setdefault("_pending_readers", [])
    readers[:] = [r for r in readers if r() is not None and r().pending()]
    readers.append(weakref.ref(node))


def flush_readers(dst):
    """Enqueue every deferred kernel that still has to read `dst`'s storage; every in-place writer
    of an array's storage calls this first, so that a deferred result is that of the contents it
    was created from."""
    base = dst.base()
    readers = base.__dict__.get("_pending_readers")
    if readers:
        base._pending_readers = []
        for r in readers:
            node = r()
            if node is not None and node.pending():
                node.buf   # noqa: B018  (runs the kernel)


def compute_stride(shape):
    """Row-major element strides (endia/utils/_array_shape.mojo:24-30)."""
    stride = [1] * len(shape)
    for i in range(len(shape) - 2, -1, -1):
        stride[i] = stride[i + 1] * shape[i + 1]
    return stride


class ArrayShape:
    """Shape, element stride and storage offset of an array or view
    (endia/utils/_array_shape.mojo:85-250, evaluated eagerly here)."""
    __slots__ = ("shape", "stride", "storage_offset")

    def __init__(self, shape, stride=None, storage_offset=0):
        self.shape = [int(s) for s in shape]
        self.stride = compute_stride(self.shape) if stride is None else [int(s) for s in stride]
        self.storage_offset = int(storage_offset)

    def ndim(self):
        return len(self.shape)

    def size(self):
        n = 1
        for s in self.shape:
            n *= s
        return n


def _parse_string(text):
    """Array("[1, 2, 3]") literal form (endia/utils/_string_utils.mojo:111)."""
    return np.asarray(ast.literal_eval(text.strip()), dtype=np.float32)


class Array:
    """Handle to a graph node with device storage. Constructor forms (as in the reference):
    Array([2, 3]) zeros of that shape; Array("[1, 2, 3]") literal; Array(numpy_array)."""

    def __init__(self, data=None, requires_grad=False, is_complex=False):
        self.args_ = []
        self.vjp_ = None
        self.jvp_ = None
        self.name = "arg"
        self.meta_data = []
        self.grad_node = None
        self.id = -1
        self.is_view = False
        self.base_ = None
        self.requires_grad_flag = bool(requires_grad)
        self.is_complex_flag = bool(is_complex)
        self.array_shape_ = ArrayShape([0])
        self.buf = None
        if data is None:
            return
        if isinstance(data, ArrayShape):
            self.array_shape_ = data
            return
        if isinstance(data, str):
            data = _parse_string(data)
        if isinstance(data, (int, np.integer)):
            data = [int(data)]
        if isinstance(data, (list, tuple)) and all(isinstance(d, (int, np.integer)) for d in data):
            self.array_shape_ = ArrayShape(data)
            n = self.array_shape_.size() * (2 if is_complex else 1)
            self.buf = alloc(n)
            if n:
                _lib.call("endia_b200_memset0", self.buf.data_ptr(), n * 4, stream())
            return
        arr = np.asarray(data)
        if np.iscomplexobj(arr):
            arr = np.ascontiguousarray(arr.astype(np.complex64))
            self.is_complex_flag = True
            host = arr.view(np.float32).reshape(-1)
        else:
            arr = np.ascontiguousarray(arr.astype(np.float32))
            host = arr.reshape(-1)
            if is_complex:
                raise ValueError("pass a complex numpy array to build a complex Array")
        shape = list(arr.shape) if arr.ndim > 0 else [1]
        self.array_shape_ = ArrayShape(shape)
        self.buf = alloc(host.size)
        if host.size:
            pinned = torch.from_numpy(host.copy()).pin_memory()
            self.buf.copy_(pinned, non_blocking=True)
            torch.cuda.current_stream().synchronize()

    # ---- metadata -------------------------------------------------------------------------
    def array_shape(self):
        return self.array_shape_

    def shape(self):
        return list(self.array_shape_.shape)

    def stride(self):
        return list(self.array_shape_.stride)

    def storage_offset(self):
        return self.array_shape_.storage_offset

    def ndim(self):
        return len(self.array_shape_.shape)

    def size(self):
        return self.array_shape_.size()

    def is_complex(self):
        return self.is_complex_flag

    def requires_grad(self):
        return self.requires_grad_flag

    def requires_grad_(self, flag=True):
        self.requires_grad_flag = bool(flag)
        return self

    def args(self):
        return self.args_

    def base(self):
        return self.base_ if self.base_ is not None else self

    def is_contiguous(self):
        s = self.array_shape_
        return s.storage_offset == 0 and all(
            e == 1 or st == d for e, st, d in zip(s.shape, s.stride, compute_stride(s.shape)))

    def desc(self):
        """ctypes descriptor for the C ABI."""
        await_pending(self)
        t = _CTensor()
        t.data = self.buf.data_ptr() if self.buf is not None and self.buf.numel() else None
        s = self.array_shape_
        if len(s.shape) > _lib.MAX_DIMS:
            raise _lib.EndiaError(_lib.EINVAL, "arrays of more than %d dims are not supported" % _lib.MAX_DIMS)
        for i, (e, st) in enumerate(zip(s.shape, s.stride)):
            t.shape[i] = e
            t.stride[i] = st
        t.offset = s.storage_offset
        t.ndim = len(s.shape)
        t.is_complex = 1 if self.is_complex_flag else 0
        return t

    def data_ptr(self):
        """Device address of the first logical element."""
        await_pending(self)
        w = 2 if self.is_complex_flag else 1
        return self.buf.data_ptr() + 4 * w * self.array_shape_.storage_offset

    # ---- graph ------------------------------------------------------------------------------
    def has_grad(self):
        return self.grad_node is not None

    def grad(self):
        """Stored gradient, or zeros of this shape when none exists (_array.mojo:695-698)."""
        if self.grad_node is None:
            return Array(self.shape(), is_complex=self.is_complex_flag)
        return self.grad_node

    def grad_(self, g):
        self.grad_node = g

    def remove_grad(self):
        self.grad_node = None

    def clear_args(self):
        self.args_ = []
        self.vjp_ = None
        self.jvp_ = None

    def backward(self, create_graph=False):
        from .autograd.functional import backward
        backward(self, create_graph)

    def zero_grad(self):
        from .utils.general import zero_grad_rec
        zero_grad_rec(self)

    def T(self):
        """Swap the last two dims (view); 1-D arrays are returned unchanged (_array.mojo:797-800)."""
        if self.ndim() == 1:
            return self
        from .functional.view_ops import permute
        return permute(self, [-1, -2])

    # ---- host access (explicit synchronisation points) ---------------------------------------
    def to_numpy(self):
        """Copy to the host as float32 (or complex64) in logical order."""
        from .functional._utils import contiguous
        await_pending(self)
        c = contiguous(self)
        n = c.size() * (2 if c.is_complex_flag else 1)
        off = c.array_shape_.storage_offset * (2 if c.is_complex_flag else 1)
        host = c.buf[off:off + n].cpu().numpy()
        if c.is_complex_flag:
            host = host.view(np.complex64)
        return host.reshape(c.shape())

    def load(self, idx):
        flat = self.to_numpy().reshape(-1)
        return float(flat[idx].real) if self.is_complex_flag else float(flat[idx])

    def item(self, idx=0):
        return self.load(idx)

    def __str__(self):
        return np.array2string(self.to_numpy(), separator=", ")

    __repr__ = __str__

    # ---- operator sugar (_array.mojo:957-1099): a scalar becomes full([last_dim], scalar) -------
    def _scalar(self, value):
        """A Python scalar as an operand: an array of the last dim's length filled with it. These
        constants are never written after their fill, so one per (length, value) is kept and
        shared (none is created while a CUDA graph is being captured: its allocations belong to the
        graph; the ones made by the warm-up steps are used)."""
        from .functional.init_ops import full
        key = (self.shape()[-1] if self.ndim() else 1, float(value))
        c = _SCALARS.get(key)
        if c is None:
            if torch.cuda.is_current_stream_capturing():
                return full([key[0]], key[1])
            if len(_SCALARS) >= 256:
                _SCALARS.clear()
            c = _SCALARS[key] = full([key[0]], key[1])
            c.name = "const"
        return c

    def _coerce(self, other):
        return other if isinstance(other, Array) else self._scalar(other)

    def __add__(self, other):
        from .functional.binary_ops import add
        return add(self, self._coerce(other))

    def __radd__(self, other):
        from .functional.binary_ops import add
        return add(self._coerce(other), self)

    def __sub__(self, other):
        from .functional.binary_ops import sub
        return sub(self, self._coerce(other))

    def __rsub__(self, other):
        from .functional.binary_ops import sub
        return sub(self._coerce(other), self)

    def __mul__(self, other):
        from .functional.binary_ops import mul
        return mul(self, self._coerce(other))

    def __rmul__(self, other):
        from .functional.binary_ops import mul
        return mul(self._coerce(other), self)

    def __truediv__(self, other):
        from .functional.binary_ops import div
        return div(self, self._coerce(other))

    def __rtruediv__(self, other):
        from .functional.binary_ops import div
        return div(self._coerce(other), self)

    def __pow__(self, other):
        from .functional.binary_ops import pow_to
        return pow_to(self, self._coerce(other))

    def __matmul__(self, other):
        from .functional.binary_ops import matmul
        return matmul(self, other)

    def __neg__(self):
        from .functional.unary_ops import neg
        return neg(self)

    def _inplace(self, res):
        """In-place update: compute, then copy into this array's storage (_array.mojo:971-1006)."""
        from .functional._utils import copy_into
        copy_into(res, self)
        return self

    def __iadd__(self, other):
        return self._inplace(self.__add__(other))

    def __isub__(self, other):
        return self._inplace(self.__sub__(other))

    def __imul__(self, other):
        return self._inplace(self.__mul__(other))

    def __itruediv__(self, other):
        return self._inplace(self.__truediv__(other))


class LazyComplex(Array):
    """complex(re, 0) whose storage is only written when something asks for it. The gradient of
    real() is such an array (view_ops/real_op.mojo:75-77) and its usual consumer, the
    conjugate-direction FFT of FFTN.vjp, reads the real array itself (the FFT kernels take a real
    input as complex with a zero imaginary part), so the complex copy is never made on that path;
    any other reader gets it on first access of `buf`."""
    re_part = None

    def __init__(self, re):
        super().__init__(ArrayShape(re.shape()))
        self.is_complex_flag = True
        self.name = "complex"
        self.re_part = re
        self._buf = None

    @property
    def buf(self):
        if self._buf is None and self.re_part is not None:
            from .functional.init_ops import complex as make_complex
            from .functional.view_ops import expand
            self._buf = make_complex(self.re_part, expand(Array([1]), self.re_part.shape())).buf
        return self._buf

    @buf.setter
    def buf(self, value):
        self._buf = value

    def materialised(self):
        return self._buf is not None


Tensor = Array
ndarray = Array
