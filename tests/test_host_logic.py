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


def test_gemm_operand_parts_plan(monkeypatch):
    """Which operand parts the host hands to endia_b200_gemm for the shapes of the configs: the
    bf16 split where the two-CTA kernel runs, fp32 low parts for the 3xTF32 kernels, none for the
    FFMA and skinny paths."""
    monkeypatch.delenv("ENDIA_B200_TC_SCHEME", raising=False)
    plan = binary_ops._tc_plan
    A = _lib.GEMM_AUTO
    for M, N, K in [(8192, 4096, 1024), (8192, 4096, 4096), (8192, 1024, 4096), (4096, 4096, 8192),
                    (1024, 4096, 8192), (4096, 1024, 256)]:
        assert plan(M, N, K, 1, A) == "pair16", (M, N, K)
    assert plan(256, 1024, 4096, 1, A) == "pair16"      # few tiles, long K: K ranges on the two-CTA kernel
    assert plan(1024, 1024, 4096, 1, A) == "pair16"
    assert plan(4096, 128, 1024, 1, A) == "lo32"        # N < 256: one-CTA kernel
    assert plan(4096, 4096, 16384, 1, A) == "pair16"    # K > 8192: runs of 8192 on the two-CTA kernel
    assert plan(4096, 4096, 16384, 1, A, linear=False) is None   # ... unless an epilogue is fused: FFMA
    assert plan(4096, 1, 1024, 1, A) is None and plan(64, 512, 512, 1, A) is None
    assert plan(8192, 4096, 4096, 2, A) is None         # batched products
    assert plan(8192, 4096, 4096, 1, _lib.GEMM_FFMA) is None
    assert plan(8192, 4096, 4096, 1, _lib.GEMM_3XTF32) == "lo32"
    assert plan(8192, 4096, 4096, 1, _lib.GEMM_TF32_BF16X2) == "pair16"
    monkeypatch.setenv("ENDIA_B200_TC_SCHEME", "3xtf32")
    assert plan(8192, 4096, 4096, 1, A) == "lo32"


def test_bench_reference_arm_prints_contract_line():
    """`bench.py --impl reference` needs no GPU: it times the CPU oracle on a bounded sample and
    prints one JSON line with the keys the reference arm has to carry."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference", "--steps", "1",
                          "--warmup", "0", "--cpu-rows", "4"], capture_output=True, text=True, timeout=900, cwd=root)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["unit"] == "samples/s" and line["value"] > 0
    assert line["higher_is_better"] is True and line["n_gpus"] == 1
    assert line["cpu_baseline"]["kind"] in ("port", "reference") and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"] == {"value": line["value"], "unit": "samples/s", "h2d_bytes_per_step": 0,
                           "d2h_bytes_per_step": 0}
