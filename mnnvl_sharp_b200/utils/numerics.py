"""Host numerics on numpy arrays: FP8 E4M3 / FP16 / BF16 codecs, input patterns, CPU all-reduce
references and the comparison metrics. All work is done by the native library, so the results
are bit-identical to what the benchmark binary and the device kernels use.

Reference parity: src/e4m3_ref.cc of the reference project (codecs :163-237, patterns :130-161,
CPU reductions :239-281, metrics :283-342) and the summary statistics of src/main.cc:36-49.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import numpy as np

from .. import _native as N

_STORAGE = {"e4m3": np.uint8, "f16": np.uint16, "bf16": np.uint16}


def storage_dtype(dtype: str):
    return _STORAGE[dtype]


def element_size(dtype: str) -> int:
    return np.dtype(_STORAGE[dtype]).itemsize


def encode(dtype: str, values) -> np.ndarray:
    """float32 -> raw codes (round to nearest even; FP8 saturates to +-448, NaN -> 0x7f)."""
    src = np.ascontiguousarray(values, dtype=np.float32)
    out = np.empty(src.shape, dtype=_STORAGE[dtype])
    N.check(N.lib.msharp_encode(N.DTYPES[dtype], src.ctypes.data, out.ctypes.data, src.size))
    return out


def decode(dtype: str, codes) -> np.ndarray:
    src = np.ascontiguousarray(codes, dtype=_STORAGE[dtype])
    out = np.empty(src.shape, dtype=np.float32)
    N.check(N.lib.msharp_decode(N.DTYPES[dtype], src.ctypes.data, out.ctypes.data, src.size))
    return out


def generate(dtype: str, pattern: str, rank: int, count: int, seed: int = 2025, first: int = 0) -> np.ndarray:
    """Raw codes of rank `rank`'s input for elements [first, first + count)."""
    out = np.empty(count, dtype=_STORAGE[dtype])
    N.check(N.lib.msharp_generate(N.DTYPES[dtype], N.PATTERNS[pattern], seed, rank, first, count, out.ctypes.data))
    return out


def reduce_f32(dtype: str, pattern: str, ranks: int, count: int, seed: int = 2025, first: int = 0) -> np.ndarray:
    out = np.empty(count, dtype=np.float32)
    N.check(N.lib.msharp_reduce_f32(N.DTYPES[dtype], N.PATTERNS[pattern], seed, ranks, first, count, out.ctypes.data))
    return out


def reduce_f32_cast(dtype: str, pattern: str, ranks: int, count: int, seed: int = 2025, first: int = 0) -> np.ndarray:
    """cast(float32 sum over ranks): the bitwise expected output for seeded inputs."""
    out = np.empty(count, dtype=_STORAGE[dtype])
    N.check(N.lib.msharp_reduce_f32_cast(N.DTYPES[dtype], N.PATTERNS[pattern], seed, ranks, first, count, out.ctypes.data))
    return out


def reduce_semantic(dtype: str, pattern: str, ranks: int, count: int, seed: int = 2025, first: int = 0) -> np.ndarray:
    """Ranks in order, running sum rounded to fp16 (bf16 for bf16) after every add, final cast."""
    out = np.empty(count, dtype=_STORAGE[dtype])
    N.check(N.lib.msharp_reduce_semantic(N.DTYPES[dtype], N.PATTERNS[pattern], seed, ranks, first, count, out.ctypes.data))
    return out


def reduce_arrays_f32(dtype: str, inputs: list[np.ndarray]) -> np.ndarray:
    """float32 sum, in list order, of explicit per-rank code arrays."""
    arrays = [np.ascontiguousarray(a, dtype=_STORAGE[dtype]) for a in inputs]
    count = arrays[0].size
    ptrs = (ctypes.c_void_p * len(arrays))(*[a.ctypes.data for a in arrays])
    out = np.empty(count, dtype=np.float32)
    N.check(N.lib.msharp_reduce_arrays_f32(N.DTYPES[dtype], ptrs, len(arrays), count, out.ctypes.data))
    return out


@dataclass
class PrecisionMetrics:
    exact_mismatches: int
    requantized_mismatches: int
    max_requantized_ulp_distance: int
    max_abs_error: float
    mean_abs_error: float
    switch_model_mismatches: int


def compare(dtype: str, pattern: str, ranks: int, result, seed: int = 2025) -> PrecisionMetrics:
    res = np.ascontiguousarray(result, dtype=_STORAGE[dtype])
    m = (ctypes.c_double * 6)()
    N.check(N.lib.msharp_compare(N.DTYPES[dtype], N.PATTERNS[pattern], seed, ranks, res.ctypes.data, res.size, m))
    return PrecisionMetrics(int(m[0]), int(m[1]), int(m[2]), float(m[3]), float(m[4]), int(m[5]))


def hash_words(data) -> int:
    """Order-independent 64-bit hash over 32-bit words; equals the device replica hash."""
    words = np.ascontiguousarray(data).view(np.uint32)
    return int(N.lib.msharp_hash_words(words.ctypes.data, words.size))


@dataclass
class TimingStats:
    min: float
    median: float
    p95: float
    max: float


def summarize(values) -> TimingStats:
    """min, upper median v[n//2], p95 = v[min(n-1, ceil(0.95 n) - 1)], max."""
    arr = (ctypes.c_double * len(values))(*[float(v) for v in values])
    out = (ctypes.c_double * 4)()
    N.check(N.lib.msharp_summarize(arr, len(values), out))
    return TimingStats(out[0], out[1], out[2], out[3])
