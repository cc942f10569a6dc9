"""Bridges between device Arrays and torch / numpy (endia/utils/array_conversions.mojo:21-59 builds
a torch tensor element by element; here the storage is shared or copied in one transfer)."""
import numpy as np
import torch

from .._array import Array, ArrayShape


def to_torch(arg, copy=True):
    """torch tensor with `arg`'s logical contents on its device: complex64 for complex arrays
    (array_conversions.mojo:25-37), float32 otherwise, requires_grad carried over (:56-57).
    copy=False returns a view of a contiguous array's storage instead."""
    from ..functional._utils import contiguous
    from ..dist import flat_tensor
    c = contiguous(arg)
    flat = flat_tensor(c)
    if arg.is_complex():
        t = torch.view_as_complex(flat.view(*(c.shape() + [2])))
    else:
        t = flat.view(*c.shape())
    if copy or c is not arg:
        t = t.clone()
    if arg.requires_grad() and copy:
        t.requires_grad_(True)
    return t


def from_torch(t, requires_grad=None):
    """Device Array with the contents of a torch tensor (float or complex, any device)."""
    src = t.detach()
    is_c = src.is_complex()
    src = src.to(torch.complex64 if is_c else torch.float32).contiguous()
    out = Array(ArrayShape(list(src.shape) if src.dim() else [1]))
    out.is_complex_flag = is_c
    from .._array import alloc, device
    flat = (torch.view_as_real(src) if is_c else src).reshape(-1)
    out.buf = alloc(flat.numel())
    if flat.numel():
        out.buf.copy_(flat.to(device(), non_blocking=False))
    out.requires_grad_flag = bool(t.requires_grad if requires_grad is None else requires_grad)
    return out


def to_numpy(arg):
    return arg.to_numpy()


def is_close(x, reference, rtol=1e-4):
    """Mean relative error of an Array against a torch tensor or numpy array, the check of the
    reference's tests (array_conversions.mojo:63-135)."""
    ref = reference.detach().cpu().numpy() if isinstance(reference, torch.Tensor) else np.asarray(reference)
    got = x.to_numpy().reshape(ref.shape)
    num = np.abs(got.astype(np.complex128) - ref.astype(np.complex128))
    den = np.abs(ref.astype(np.complex128)) + 1e-6
    return bool(np.mean(num / den) < rtol)
