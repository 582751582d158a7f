"""The word permutation of the padded path for size_n % 256 != 0 (marlin_v100_b200/csrc/gemm_pad.cu), restated in
numpy and checked against the oracle's packing: permuting the packed words of a matrix with N columns must give
exactly the packed tensor of the same codes padded with zero codes to the next multiple of 256 columns.  The
reference layout is the one of csrc/quantization/marlin/gptq_marlin_repack.cu:399-469 (tile interleave chosen by
the divisibility of N)."""
import numpy as np
import pytest
import torch

from oracle import marlin_oracle as mo


def _macro_n_of(n: int) -> int:
    return 256 if n % 256 == 0 else (128 if n % 128 == 0 else 64)


def _packed_col(bits: int, lk: int, n: int, g: int) -> int:
    pf = 32 // bits
    w = 1024 // pf
    macro = g * 64
    return (n // macro) * g * w + (lk * (64 // pf) + (n % 64) // pf) * g + (n % macro) // 64


def _pad_words(src: np.ndarray, n: int, bits: int) -> tuple[np.ndarray, int]:
    pf = 32 // bits
    w = 1024 // pf
    n_pad = (n + 255) // 256 * 256
    g_src = _macro_n_of(n) // 64
    dst = np.zeros((src.shape[0], n_pad * 16 // pf), dtype=np.int64)
    for col in range(dst.shape[1]):
        grp, rem = divmod(col, 4 * w)
        sub, t = rem & 3, rem >> 2
        lk, nv = divmod(t, 64 // pf)
        n0 = grp * 256 + sub * 64 + nv * pf
        if n0 < n:
            dst[:, col] = src[:, _packed_col(bits, lk, n0, g_src)]
    return dst, n_pad


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("n", [64, 128, 192, 320, 384, 640, 832, 1152, 3200])
def test_padded_words_equal_the_packing_of_the_padded_codes(bits, n):
    k = 48
    g = torch.Generator().manual_seed(100 * bits + n)
    q = torch.randint(0, 2 ** bits, (k, n), generator=g, dtype=torch.int32)
    src = mo.marlin_pack(q, bits).numpy().astype(np.int64) & 0xFFFFFFFF
    dst, n_pad = _pad_words(src, n, bits)
    q_pad = torch.cat([q, torch.zeros(k, n_pad - n, dtype=torch.int32)], dim=1)
    ref = mo.marlin_pack(q_pad, bits).numpy().astype(np.int64) & 0xFFFFFFFF
    assert dst.shape == ref.shape
    assert (dst == ref).all()
