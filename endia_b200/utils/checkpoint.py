"""Checkpoint and resume of a training run: the parameters and the optimizer's state (Adam's m, v
and step count t; the velocity / cache of the other optimizers) as one raw little-endian float32
file plus a JSON manifest of names, shapes and offsets. The reference has no checkpoint format; what
is stored is exactly the state its step loop carries (benchmarks/mlp_benchmarks/mlp_imp.mojo:47-75,
optim/adam.mojo:17-46), so a resumed run continues bit for bit.

    save(path, params, optimizer)     ->  path + ".bin", path + ".json"
    load(path, params, optimizer)     restores in place (shapes must match the manifest)
"""
import json
import os

import numpy as np

from .. import _lib
from .._array import ArrayShape, drop_operand_parts, flush_readers

FORMAT = "endia_b200.checkpoint.v1"
_STATE_LISTS = ("m", "v", "velocity", "cache")
_SCALARS = ("t", "lr", "beta1", "beta2", "eps", "momentum", "weight_decay", "alpha", "grad_scale")


def _host(arr):
    a = arr.to_numpy()
    if np.iscomplexobj(a):
        a = np.ascontiguousarray(a).view(np.float32)
    return np.ascontiguousarray(a, dtype="<f4").reshape(-1)


def save(path, params, optimizer=None):
    """Write the arrays of `params` (in order) and the optimizer's state arrays and scalars."""
    entries, chunks, offset = [], [], 0

    def put(name, arr):
        nonlocal offset
        data = _host(arr)
        entries.append({"name": name, "shape": arr.shape(), "complex": bool(arr.is_complex()),
                        "offset_floats": offset, "floats": int(data.size)})
        chunks.append(data)
        offset += int(data.size)

    for i, p in enumerate(params):
        put("param.%d" % i, p)
    opt = None
    if optimizer is not None:
        opt = {"type": type(optimizer).__name__, "scalars": {}}
        for key in _SCALARS:
            if hasattr(optimizer, key):
                opt["scalars"][key] = float(getattr(optimizer, key))
        for key in _STATE_LISTS:
            state = getattr(optimizer, key, None)
            if state:
                for i, s in enumerate(state):
                    put("optimizer.%s.%d" % (key, i), s)
    manifest = {"format": FORMAT, "dtype": "<f4", "tensors": entries, "optimizer": opt, "total_floats": offset}
    tmp = path + ".bin.tmp"
    with open(tmp, "wb") as fh:
        for c in chunks:
            fh.write(c.tobytes())
    os.replace(tmp, path + ".bin")
    with open(path + ".json.tmp", "w") as fh:
        json.dump(manifest, fh, indent=1)
    os.replace(path + ".json.tmp", path + ".json")
    return manifest


def load(path, params, optimizer=None):
    """Restore what save() wrote into the given arrays (in place) and optimizer."""
    import torch
    from ..dist import flat_tensor
    with open(path + ".json") as fh:
        manifest = json.load(fh)
    if manifest.get("format") != FORMAT:
        raise _lib.EndiaError(_lib.EINVAL, "checkpoint: unknown format %r" % (manifest.get("format"),))
    blob = np.fromfile(path + ".bin", dtype="<f4")
    if blob.size != manifest["total_floats"]:
        raise _lib.EndiaError(_lib.EINVAL, "checkpoint: %s.bin holds %d floats, the manifest says %d" % (
            path, blob.size, manifest["total_floats"]))
    by_name = {e["name"]: e for e in manifest["tensors"]}

    def get(name, arr, reshape=False):
        e = by_name.get(name)
        if e is None:
            raise _lib.EndiaError(_lib.EINVAL, "checkpoint: no tensor %r" % name)
        if reshape:
            arr.array_shape_ = ArrayShape(e["shape"])      # a bias's moments are (1, N) after the first step
        if e["shape"] != arr.shape() or e["complex"] != bool(arr.is_complex()) or not arr.is_contiguous():
            raise _lib.EndiaError(_lib.ESHAPE, "checkpoint: %s has shape %s, the array %s" % (
                name, e["shape"], arr.shape()))
        flush_readers(arr)
        data = blob[e["offset_floats"]:e["offset_floats"] + e["floats"]]
        flat_tensor(arr).copy_(torch.from_numpy(np.array(data, dtype=np.float32)))
        drop_operand_parts(arr)

    for i, p in enumerate(params):
        get("param.%d" % i, p)
    if optimizer is not None:
        opt = manifest.get("optimizer")
        if not opt or opt["type"] != type(optimizer).__name__:
            raise _lib.EndiaError(_lib.EINVAL, "checkpoint: optimizer state of %r, asked for %r" % (
                opt and opt["type"], type(optimizer).__name__))
        for key, value in opt["scalars"].items():
            setattr(optimizer, key, value)
        for key in _STATE_LISTS:
            state = getattr(optimizer, key, None)
            if state:
                for i, s in enumerate(state):
                    get("optimizer.%s.%d" % (key, i), s, reshape=True)
    return manifest
