"""GPU parity of the multiply kernels, through the C ABI's test hook (brisk_cuda_matmul), against the CPU oracle.

The integer block dots, the per-block f32 terms and the order in which a row's terms are added are the reference's,
so the quantised formats must match the oracle BIT FOR BIT (np.array_equal). The unquantised F16/F32 head uses a
different summation order and is held to the reference's own batched-vs-single bound, 1e-4 * (1 + |ref|)
(tests/kernels_test.cpp:160-184).
"""
import numpy as np
import pytest

import helpers as H
from brisk_llm_b200 import engine, formats as F

pytestmark = pytest.mark.gpu
FORMATS = (F.Q4_0, F.Q4_1, F.Q5_0, F.Q8_0, F.Q4_K, F.Q5_K, F.Q6_K, F.TQ2_0)


def check(fmt, rows, cols, n, seed=0, scale=1.0):
    wb, _ = H.random_matrix(fmt, rows, cols, seed=seed + fmt)
    x = (np.random.default_rng(seed + 1).standard_normal((n, cols)) * scale).astype(np.float32)
    want = H.oracle_matmul(fmt, wb, rows, cols, x)
    got = engine.matmul(fmt, wb, rows, cols, x)
    assert got.shape == want.shape
    assert np.array_equal(got, want), (F.NAMES[fmt], rows, cols, n, np.abs(got - want).max())
    return got, want


@pytest.mark.parametrize("fmt", FORMATS, ids=lambda f: F.NAMES[f])
@pytest.mark.parametrize("n", [1, 2, 4, 7, 8, 9, 13, 16, 20, 64])
def test_reference_test_shape(fmt, n):
    # the reference's kernel test shape: 1024 columns, 37 rows (a row count no row group divides)
    check(fmt, 37, 1024, n, seed=n)


@pytest.mark.parametrize("fmt", FORMATS, ids=lambda f: F.NAMES[f])
@pytest.mark.parametrize("rows,cols", [(36, 256), (48, 2048), (130, 3072), (8, 14336)])
def test_ragged_and_wide_rows(fmt, rows, cols):
    check(fmt, rows, cols, 1, seed=rows)
    check(fmt, rows, cols, 5, seed=rows + 1)


@pytest.mark.parametrize("fmt", FORMATS, ids=lambda f: F.NAMES[f])
def test_sweep_shape_small_side(fmt):
    # 1024 x 3072, the smallest matrix of the kernel sweep, at 1, 4 and 512 tokens
    for n in (1, 4, 512):
        check(fmt, 1024, 3072, n, seed=n)


@pytest.mark.parametrize("fmt", FORMATS, ids=lambda f: F.NAMES[f])
def test_zero_and_extreme_activations(fmt):
    rows, cols = 40, 1024
    wb, _ = H.random_matrix(fmt, rows, cols, seed=5)
    rng = np.random.default_rng(9)
    x = rng.standard_normal((4, cols)).astype(np.float32)
    x[0] = 0.0                      # all-zero row: zero scales
    x[1, 256:512] = 0.0             # one all-zero super-block
    x[2, 0], x[2, 1] = 7.0, -7.0    # equal magnitudes: the first sets the Q8_K sign
    x[3] *= 1e4                     # large dynamic range
    want = H.oracle_matmul(fmt, wb, rows, cols, x)
    got = engine.matmul(fmt, wb, rows, cols, x)
    assert np.array_equal(got, want)
    assert np.all(got[0] == 0.0)


@pytest.mark.parametrize("fmt", (F.Q4_0, F.Q8_0), ids=lambda f: F.NAMES[f])
def test_prompt_multiply_on_tcgen05_matches_the_oracle(fmt, monkeypatch):
    """BRISK_CUDA_GEMM=tc: the prompt multiply through tcgen05.mma.kind::i8 and tensor memory (csrc/gemm_tc.cu) instead of
    mma.sync fragments - same integers, same f32 roundings, so the oracle's bits. Ragged rows and token counts (tiles of 128
    rows x 64 tokens), a single K chunk, and the sweep's smallest shape at 512 tokens."""
    monkeypatch.setenv("BRISK_CUDA_GEMM", "tc")
    check(fmt, 37, 1024, 64, seed=1)
    check(fmt, 130, 128, 33, seed=2)
    check(fmt, 300, 3072, 200, seed=3)
    check(fmt, 1024, 3072, 512, seed=4)


@pytest.mark.parametrize("fmt", (F.F16, F.BF16, F.F32), ids=lambda f: F.NAMES[f])
def test_float_head(fmt):
    rng = np.random.default_rng(3)
    w = (rng.standard_normal((77, 2560)) * 0.02).astype(np.float16)
    wb = F.quantize(fmt, w.astype(np.float32))
    x = rng.standard_normal((3, 2560)).astype(np.float32)
    want = H.oracle_matmul(fmt, wb, 77, 2560, x)
    got = engine.matmul(fmt, wb, 77, 2560, x)
    assert np.all(np.abs(got - want) <= 1e-4 * (1 + np.abs(want)))


def test_linearity_at_full_sweep_size():
    # a size-independent property at a full sweep shape (4096 x 14336, Q8_0): doubling the activations doubles every
    # output exactly (power-of-two scaling commutes with the quantiser), and a checksum over rows matches a sampled oracle
    rows, cols = 4096, 14336
    wb, _ = H.random_matrix(F.Q8_0, rows, cols, seed=1)
    x = np.random.default_rng(2).standard_normal((1, cols)).astype(np.float32)
    a = engine.matmul(F.Q8_0, wb, rows, cols, x)
    b = engine.matmul(F.Q8_0, wb, rows, cols, 2 * x)
    assert np.array_equal(2 * a, b)
    sample = np.arange(0, rows, 97)
    rb = F.row_bytes(F.Q8_0, cols)
    wsub = np.concatenate([wb[r * rb:(r + 1) * rb] for r in sample])
    want = H.oracle_matmul(F.Q8_0, wsub, len(sample), cols, x)
    assert np.array_equal(a[:, sample], want)


def test_bad_arguments_fail_with_a_message():
    with pytest.raises(RuntimeError, match="cuda:"):
        engine.matmul(F.Q4_K, np.zeros(144, np.uint8), 1, 128, np.zeros((1, 128), np.float32))
    with pytest.raises(RuntimeError, match="cuda:"):
        engine.matmul(5, np.zeros(144, np.uint8), 1, 256, np.zeros((1, 256), np.float32))
