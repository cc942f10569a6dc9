"""CPU tests of the host-side metadata rules (shape / stride / offset arithmetic), which must be
bit-exact with the reference's ArrayShape functions."""
import pytest

from endia_b200._array import ArrayShape, compute_stride
from endia_b200.functional._utils import broadcast_shapes
from endia_b200.functional import view_ops, binary_ops, fft_ops
from endia_b200 import _lib


def test_default_strides_row_major():
    assert compute_stride([2, 3, 4]) == [12, 4, 1]
    assert compute_stride([5]) == [1]
    assert ArrayShape([2, 3]).size() == 6


def test_broadcast_shapes_right_aligned():
    assert broadcast_shapes([128, 32], [32]) == [128, 32]
    assert broadcast_shapes([2, 1, 4], [3, 1]) == [2, 3, 4]
    assert broadcast_shapes([1], [7, 5]) == [7, 5]
    with pytest.raises(_lib.EndiaError):
        broadcast_shapes([2, 3], [4])


def test_squeezable_axes_keep_last_when_all_one():
    assert view_ops._squeezable_axes([1, 1]) == [0]          # sum() of a 2-D array has shape [1]
    assert view_ops._squeezable_axes([1, 5, 1]) == [0, 2]
    assert view_ops._squeezable_axes([1]) == []


def test_permute_axes_are_trailing():
    assert view_ops._perm_axes([-1, -2], 3) == [0, 2, 1]
    assert view_ops._perm_axes([1, 0], 2) == [1, 0]
    with pytest.raises(_lib.EndiaError):
        view_ops._perm_axes([0, 1, 2], 2)


def test_matmul_shape_rules():
    assert binary_ops._matmul_shape([8, 3], [3, 5]) == ([], [8, 5])
    assert binary_ops._matmul_shape([2, 1, 8, 3], [4, 3, 5]) == ([2, 4], [2, 4, 8, 5])
    with pytest.raises(_lib.EndiaError):
        binary_ops._matmul_shape([8, 3], [4, 5])
    with pytest.raises(_lib.EndiaError):
        binary_ops._matmul_shape([3], [3, 5])


def test_fft_meta_data_encoding():
    assert fft_ops.encode_fft_params([-1], "backward") == [1, -1, 0]
    assert fft_ops.encode_fft_params([0, 1, 2], "ortho") == [3, 0, 1, 2, 2]
    with pytest.raises(_lib.EndiaError):
        fft_ops.encode_fft_params([0], "bogus")
