"""Codecs, input patterns, host reductions, metrics and statistics (CPU only)."""
import math

import numpy as np
import pytest

from mnnvl_sharp_b200.utils import numerics as nm


def py_decode_e4m3(b: int) -> float:
    sign = -1.0 if b & 0x80 else 1.0
    e, m = (b >> 3) & 0xF, b & 7
    if (b & 0x7F) == 0x7F:
        return math.nan
    if e == 0:
        return sign * m * 2.0 ** -9
    return sign * (1 + m / 8) * 2.0 ** (e - 7)


def test_e4m3_decode_all_codes():
    got = nm.decode("e4m3", np.arange(256, dtype=np.uint8))
    for b in range(256):
        want = py_decode_e4m3(b)
        if math.isnan(want):
            assert math.isnan(got[b])
        else:
            assert got[b] == want and math.copysign(1, got[b]) == math.copysign(1, want)


def test_e4m3_roundtrip_all_finite_codes():
    codes = np.array([b for b in range(256) if (b & 0x7F) != 0x7F], dtype=np.uint8)
    assert np.array_equal(nm.encode("e4m3", nm.decode("e4m3", codes)), codes)


def test_e4m3_encode_special_values():
    x = np.array([448.0, 449.0, 464.0, 1e9, np.inf, -np.inf, -500.0, np.nan, 0.0, -0.0, 2.0 ** -10, 2.0 ** -11,
                  3 * 2.0 ** -10, 2.0 ** -6 - 2.0 ** -11], dtype=np.float32)
    got = nm.encode("e4m3", x)
    assert list(got[:8]) == [0x7E, 0x7E, 0x7E, 0x7E, 0x7E, 0xFE, 0xFE, 0x7F]
    assert got[8] == 0x00 and got[9] == 0x80
    assert got[10] == 0x00  # half of the smallest subnormal: tie to even (zero)
    assert got[11] == 0x00
    assert got[12] == 0x02  # 1.5 steps: tie to even (two steps)
    assert got[13] == 0x08  # rounds up into the smallest normal


def test_e4m3_encode_is_nearest_even_on_a_dense_grid():
    finite = np.array(sorted({py_decode_e4m3(b) for b in range(256) if (b & 0x7F) != 0x7F}))
    xs = np.linspace(-460, 460, 200001).astype(np.float32)
    xs = np.concatenate([xs, (np.linspace(-1, 1, 100001) ** 3).astype(np.float32)])
    got = nm.decode("e4m3", nm.encode("e4m3", xs))
    clipped = np.clip(xs.astype(np.float64), -448, 448)
    idx = np.searchsorted(finite, clipped)
    idx = np.clip(idx, 1, len(finite) - 1)
    lo, hi = finite[idx - 1], finite[idx]
    nearest = np.where(clipped - lo < hi - clipped, lo, hi)
    not_tie = (clipped - lo) != (hi - clipped)
    assert np.array_equal(got[not_tie], nearest[not_tie].astype(np.float32))
    err = np.abs(got.astype(np.float64) - clipped)
    assert np.all(err <= np.minimum(clipped - lo, hi - clipped) + 0)


def test_f16_matches_numpy_for_all_codes_and_random_floats():
    codes = np.arange(65536, dtype=np.uint16)
    ours = nm.decode("f16", codes)
    ref = codes.view(np.float16).astype(np.float32)
    both_nan = np.isnan(ours) & np.isnan(ref)
    assert np.array_equal(ours[~both_nan], ref[~both_nan])
    rng = np.random.default_rng(0)
    x = np.concatenate([rng.standard_normal(200000).astype(np.float32) * s for s in (1e-7, 1e-4, 1.0, 300.0, 7e4)])
    x = np.concatenate([x, np.array([65504, 65519.99, 65520, np.inf, -np.inf, 0.0, -0.0, 2.0 ** -24, 2.0 ** -25,
                                     3 * 2.0 ** -25], dtype=np.float32)])
    with np.errstate(over="ignore"):
        want = x.astype(np.float16).view(np.uint16)
    assert np.array_equal(nm.encode("f16", x), want)
    assert nm.encode("f16", np.array([np.nan], dtype=np.float32))[0] == 0x7E00


def test_bf16_matches_torch():
    torch = pytest.importorskip("torch")
    rng = np.random.default_rng(1)
    x = (rng.standard_normal(100000) * 10 ** rng.uniform(-20, 20, 100000)).astype(np.float32)
    want = torch.from_numpy(x).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(nm.encode("bf16", x), want)
    assert np.array_equal(nm.decode("bf16", want), torch.from_numpy(x).to(torch.bfloat16).float().numpy())


def test_reference_patterns_follow_the_published_formulas():
    # E4M3: mix = (i*17) ^ (i>>7) ^ ((rank+1)*29); sign = bit 4; exponent 3 + mix%3; mantissa (mix/3)&7
    for rank in (0, 3, 71):
        idx = np.array([0, 1, 5, 127, 128, 1000, 2 ** 20 + 3, 2 ** 31 + 11], dtype=np.uint64)
        for i in idx:
            i = int(i)
            mix = ((i * 17) ^ (i >> 7) ^ ((rank + 1) * 29)) & 0xFFFFFFFF
            want = (0x80 if (mix >> 4) & 1 else 0) | ((3 + mix % 3) << 3) | ((mix // 3) & 7)
            assert nm.generate("e4m3", "reference", rank, 1, first=i)[0] == want
            table = [0xB800, 0xB400, 0xB000, 0, 0x3000, 0x3400, 0x3800, 0]
            mix16 = ((i * 13) ^ (i >> 5) ^ ((rank + 1) * 7)) & 7
            assert nm.generate("f16", "reference", rank, 1, first=i)[0] == table[mix16]


def test_reference_f16_sum_is_zero_for_eight_ranks_but_tagged_is_not():
    # the weakness of the reference inputs that the tagged pattern exists to avoid
    assert np.all(nm.reduce_f32("f16", "reference", 8, 4096) == 0)
    assert np.count_nonzero(nm.reduce_f32("f16", "tagged", 8, 4096)) > 4000
    assert np.count_nonzero(nm.reduce_f32("e4m3", "tagged", 8, 4096)) > 2000


def test_seeded_patterns_have_the_stated_distributions():
    n = 1 << 18
    u = nm.decode("e4m3", nm.generate("e4m3", "seeded", 2, n, seed=9))
    assert -2.0 <= u.min() and u.max() <= 2.0 and abs(u.mean()) < 0.02 and abs(u.std() - 4 / math.sqrt(12)) < 0.03
    g = nm.decode("f16", nm.generate("f16", "seeded", 2, n, seed=9))
    assert abs(g.mean()) < 0.01 and abs(g.std() - 1.0) < 0.01 and 3.5 < np.abs(g).max() <= 6.0
    assert not np.array_equal(nm.generate("f16", "seeded", 2, 64, seed=9), nm.generate("f16", "seeded", 3, 64, seed=9))
    assert not np.array_equal(nm.generate("f16", "seeded", 2, 64, seed=9), nm.generate("f16", "seeded", 2, 64, seed=10))
    # the generator is a pure function of the element index
    assert np.array_equal(nm.generate("e4m3", "seeded", 1, 100, first=50), nm.generate("e4m3", "seeded", 1, 150)[50:])


@pytest.mark.parametrize("dtype", ["e4m3", "f16", "bf16"])
@pytest.mark.parametrize("pattern", ["reference", "tagged", "seeded"])
def test_host_reductions_agree_with_numpy(dtype, pattern):
    ranks, n = 8, 5000
    inputs = [nm.generate(dtype, pattern, r, n) for r in range(ranks)]
    acc = np.zeros(n, dtype=np.float32)
    for a in inputs:
        acc = acc + nm.decode(dtype, a)
    f32 = nm.reduce_f32(dtype, pattern, ranks, n)
    assert np.array_equal(f32, acc)
    assert np.array_equal(nm.reduce_arrays_f32(dtype, inputs), acc)
    assert np.array_equal(nm.reduce_f32_cast(dtype, pattern, ranks, n), nm.encode(dtype, acc))
    seq = np.zeros(n, dtype=np.float32)
    step = "bf16" if dtype == "bf16" else "f16"
    for a in inputs:
        seq = nm.decode(step, nm.encode(step, seq + nm.decode(dtype, a)))
    assert np.array_equal(nm.reduce_semantic(dtype, pattern, ranks, n), nm.encode(dtype, seq))


def test_exact_patterns_make_both_models_agree():
    for dtype in ("e4m3", "f16", "bf16"):
        for ranks in (2, 4, 8):
            a = nm.reduce_semantic(dtype, "tagged", ranks, 4096)
            b = nm.reduce_f32_cast(dtype, "tagged", ranks, 4096)
            assert np.array_equal(a, b)
    for ranks in (2, 8, 34, 72):  # reference FP8 inputs: every partial sum is exact in fp16
        m = nm.compare("e4m3", "reference", ranks, nm.reduce_semantic("e4m3", "reference", ranks, 1 << 14))
        assert m.exact_mismatches == 0 and m.requantized_mismatches == 0 and m.max_abs_error <= 2 ** -5 * 8


def test_compare_counts_what_it_says():
    ranks, n = 4, 1000
    good = nm.reduce_semantic("e4m3", "reference", ranks, n)
    m = nm.compare("e4m3", "reference", ranks, good)
    assert (m.exact_mismatches, m.requantized_mismatches, m.max_requantized_ulp_distance) == (0, 0, 0)
    bad = good.copy()
    bad[10] = bad[10] + 1 if (bad[10] & 7) < 7 else bad[10] - 1   # one step in magnitude
    bad[20] ^= 0x80  # sign flip
    m = nm.compare("e4m3", "reference", ranks, bad)
    assert m.exact_mismatches == 2 and m.requantized_mismatches == 2 and m.max_requantized_ulp_distance >= 1
    assert m.switch_model_mismatches >= 1
    f16 = nm.reduce_semantic("f16", "tagged", ranks, n)
    f16[5] += 3
    m = nm.compare("f16", "tagged", ranks, f16)
    assert m.exact_mismatches == 1 and m.max_requantized_ulp_distance == 3 and m.switch_model_mismatches == 1


def test_switch_model_accepts_either_neighbour_but_nothing_else():
    # element with an inexact FP8 sum: both bracketing codes pass, two steps away fails
    ranks, n = 2, 4096
    f32 = nm.reduce_f32("e4m3", "reference", ranks, n)
    rne = nm.reduce_f32_cast("e4m3", "reference", ranks, n)
    inexact = np.nonzero(nm.decode("e4m3", rne) != f32)[0]
    assert inexact.size > 100
    i = int(inexact[0])
    below = nm.decode("e4m3", rne)[i] < f32[i]
    mag_up = (rne[i] & 0x80 == 0) == below  # does moving toward the sum mean a larger magnitude?
    other = rne.copy()
    other[i] = rne[i] + 1 if mag_up else rne[i] - 1
    assert nm.compare("e4m3", "reference", ranks, other).switch_model_mismatches == 0
    far = rne.copy()
    far[i] = rne[i] + 2 if mag_up else rne[i] - 2
    assert nm.compare("e4m3", "reference", ranks, far).switch_model_mismatches == 1


def test_hash_is_order_independent_xor_of_mixed_words():
    def mix64(v):
        v &= (1 << 64) - 1
        v ^= v >> 33
        v = (v * 0xFF51AFD7ED558CCD) & ((1 << 64) - 1)
        v ^= v >> 33
        v = (v * 0xC4CEB9FE1A85EC53) & ((1 << 64) - 1)
        v ^= v >> 33
        return v

    words = np.array([0, 1, 0xDEADBEEF, 0xFFFFFFFF, 12345], dtype=np.uint32)
    want = 0
    for i, w in enumerate(words):
        want ^= mix64((int(w) << 32) ^ i)
    assert nm.hash_words(words) == want
    big = np.random.default_rng(2).integers(0, 2 ** 32, 1 << 20, dtype=np.uint32)
    assert nm.hash_words(big) == nm.hash_words(big.copy())
    changed = big.copy()
    changed[777] ^= 1
    assert nm.hash_words(big) != nm.hash_words(changed)


def test_summarize_uses_upper_median_and_ceil_p95():
    s = nm.summarize([4.0, 1.0, 3.0, 2.0])
    assert (s.min, s.median, s.p95, s.max) == (1.0, 3.0, 4.0, 4.0)
    s = nm.summarize(list(range(1, 21)))
    assert (s.median, s.p95) == (11.0, 19.0)
    s = nm.summarize([7.0])
    assert (s.min, s.median, s.p95, s.max) == (7.0, 7.0, 7.0, 7.0)
    s = nm.summarize([])
    assert (s.min, s.median, s.p95, s.max) == (0.0, 0.0, 0.0, 0.0)
