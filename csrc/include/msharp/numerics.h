// Bit-level numerics shared by host code and device kernels.
//
// Everything in this header is integer arithmetic on IEEE bit patterns, so the
// host oracle and the device generators produce identical bits by construction.
// Behavioural parity targets in the reference project (paths within it):
//   src/e4m3_ref.cc:163-225  FP8 E4M3 decode / encode (RNE, saturate-to-finite, NaN 0x7f)
//   src/e4m3_ref.cc:24-92    FP16 <-> FP32 conversion (RNE, subnormals, quiet NaN 0x7e00)
//   src/e4m3_ref.cc:130-161  deterministic input patterns (mirrored on the device at
//                            src/sharp_kernels.cu:20-51)
//   src/sharp_kernels.cu:170-177  64-bit finaliser used by the replica hash
#pragma once

#include <cstddef>
#include <cstdint>
#include <cstring>

#if defined(__CUDACC__)
#define MSHARP_HD __host__ __device__ __forceinline__
#define MSHARP_UNROLL _Pragma("unroll")
#else
#define MSHARP_HD inline
#define MSHARP_UNROLL
#endif

namespace msharp {

// ----------------------------------------------------------------------------- bit casts
MSHARP_HD uint32_t f32_bits(float f) {
#if defined(__CUDA_ARCH__)
  return __float_as_uint(f);
#else
  uint32_t u;
  std::memcpy(&u, &f, sizeof(u));
  return u;
#endif
}

MSHARP_HD float bits_f32(uint32_t u) {
#if defined(__CUDA_ARCH__)
  return __uint_as_float(u);
#else
  float f;
  std::memcpy(&f, &u, sizeof(f));
  return f;
#endif
}

// Round-to-nearest-even right shift of an unsigned integer (shift in 1..31).
MSHARP_HD uint32_t rne_shift_right(uint32_t value, int shift) {
  const uint32_t q = value >> shift;
  const uint32_t rem = value & ((1u << shift) - 1u);
  const uint32_t half = 1u << (shift - 1);
  return q + ((rem > half || (rem == half && (q & 1u))) ? 1u : 0u);
}

// ----------------------------------------------------------------------------- FP8 E4M3 (fn)
// Layout: 1 sign, 4 exponent (bias 7), 3 mantissa. No infinities; 0x7f / 0xff are NaN;
// largest finite magnitude is 448 (0x7e).
MSHARP_HD float decode_e4m3(uint8_t bits) {
  const uint32_t sign = static_cast<uint32_t>(bits & 0x80u) << 24;
  const uint32_t expo = (bits >> 3) & 0x0fu;
  const uint32_t mant = bits & 0x07u;
  if ((bits & 0x7fu) == 0x7fu) {
    return bits_f32(0x7fc00000u);
  }
  if (expo == 0) {
    // Subnormal: mant * 2^-9, exact in binary32. Build it without floating multiplies.
    if (mant == 0) {
      return bits_f32(sign);
    }
    // mant in 1..7 -> normalise into a binary32 pattern.
    int lead = mant >= 4 ? 2 : (mant >= 2 ? 1 : 0);
    const uint32_t frac = (mant << (23 - lead)) & 0x7fffffu;
    const uint32_t e = static_cast<uint32_t>(127 - 9 + lead);
    return bits_f32(sign | (e << 23) | frac);
  }
  return bits_f32(sign | ((expo + 120u) << 23) | (mant << 20));
}

// Round-to-nearest-even, saturate-to-finite: |x| >= 448 (and +-inf) -> +-448, NaN -> 0x7f.
MSHARP_HD uint8_t encode_e4m3(float value) {
  const uint32_t u = f32_bits(value);
  const uint8_t sign = static_cast<uint8_t>((u >> 24) & 0x80u);
  const uint32_t a = u & 0x7fffffffu;
  if (a > 0x7f800000u) {
    return 0x7fu;
  }
  if (a >= 0x43e00000u) {  // 448.0f
    return static_cast<uint8_t>(sign | 0x7eu);
  }
  if (a < 0x3c800000u) {  // below 2^-6: subnormal grid of 2^-9
    const int e = static_cast<int>(a >> 23);
    if (e == 0) {
      return sign;  // binary32 subnormals are far below half of 2^-9
    }
    const int shift = 141 - e;  // value / 2^-9 == mant24 * 2^-shift, shift >= 21
    if (shift > 25) {
      return sign;
    }
    const uint32_t mant24 = (a & 0x7fffffu) | 0x800000u;
    const uint32_t q = rne_shift_right(mant24, shift);  // 0..8; 8 is the smallest normal
    return static_cast<uint8_t>(sign | q);
  }
  // Normal range: drop 20 mantissa bits with RNE; a carry walks into the exponent field.
  const uint32_t code = rne_shift_right(a - (120u << 23), 20);
  return static_cast<uint8_t>(sign | code);
}

// Monotone integer code used for "distance in representable values" metrics.
MSHARP_HD int ordered_code_e4m3(uint8_t bits) {
  const int mag = bits & 0x7f;
  return (bits & 0x80u) ? 0x80 - mag : 0x80 + mag;
}

// ----------------------------------------------------------------------------- FP16
MSHARP_HD float decode_f16(uint16_t h) {
  const uint32_t sign = static_cast<uint32_t>(h & 0x8000u) << 16;
  const uint32_t expo = (h >> 10) & 0x1fu;
  uint32_t mant = h & 0x3ffu;
  if (expo == 0x1fu) {
    return bits_f32(sign | 0x7f800000u | (mant << 13) | (mant ? 0x400000u : 0u));
  }
  if (expo == 0) {
    if (mant == 0) {
      return bits_f32(sign);
    }
    int e = 113;  // 127 - 14
    while ((mant & 0x400u) == 0) {
      mant <<= 1;
      --e;
    }
    return bits_f32(sign | (static_cast<uint32_t>(e) << 23) | ((mant & 0x3ffu) << 13));
  }
  return bits_f32(sign | ((expo + 112u) << 23) | (mant << 13));
}

MSHARP_HD uint16_t encode_f16(float value) {
  const uint32_t u = f32_bits(value);
  const uint16_t sign = static_cast<uint16_t>((u >> 16) & 0x8000u);
  const uint32_t a = u & 0x7fffffffu;
  if (a > 0x7f800000u) {
    return static_cast<uint16_t>(sign | 0x7e00u);
  }
  if (a >= 0x477ff000u) {  // >= 65520 rounds to infinity (also covers inf)
    return static_cast<uint16_t>(sign | 0x7c00u);
  }
  if (a < 0x38800000u) {  // below 2^-14: subnormal grid of 2^-24
    const int e = static_cast<int>(a >> 23);
    const int shift = 126 - e;  // value / 2^-24 == mant24 * 2^-shift
    if (e == 0 || shift > 25) {
      return sign;
    }
    const uint32_t mant24 = (a & 0x7fffffu) | 0x800000u;
    return static_cast<uint16_t>(sign | rne_shift_right(mant24, shift));
  }
  return static_cast<uint16_t>(sign | rne_shift_right(a - (112u << 23), 13));
}

MSHARP_HD float round_to_f16(float value) { return decode_f16(encode_f16(value)); }

MSHARP_HD int ordered_code_f16(uint16_t bits) {
  const int mag = bits & 0x7fff;
  return (bits & 0x8000u) ? 0x8000 - mag : 0x8000 + mag;
}

// ----------------------------------------------------------------------------- BF16
MSHARP_HD float decode_bf16(uint16_t b) { return bits_f32(static_cast<uint32_t>(b) << 16); }

MSHARP_HD uint16_t encode_bf16(float value) {
  const uint32_t u = f32_bits(value);
  if ((u & 0x7fffffffu) > 0x7f800000u) {
    return static_cast<uint16_t>((u >> 16) | 0x0040u);
  }
  const uint32_t rounding = 0x7fffu + ((u >> 16) & 1u);
  return static_cast<uint16_t>((u + rounding) >> 16);
}

MSHARP_HD int ordered_code_bf16(uint16_t bits) { return ordered_code_f16(bits); }

// ----------------------------------------------------------------------------- hashing
// 64-bit avalanche finaliser (the public-domain MurmurHash3 fmix64).
MSHARP_HD uint64_t mix64(uint64_t v) {
  v ^= v >> 33;
  v *= 0xff51afd7ed558ccdull;
  v ^= v >> 33;
  v *= 0xc4ceb9fe1a85ec53ull;
  v ^= v >> 33;
  return v;
}

// Contribution of one 32-bit word at a given word index to the order-independent
// replica hash (all contributions are XORed together).
MSHARP_HD uint64_t hash_term(uint32_t word, uint64_t word_index) {
  return mix64((static_cast<uint64_t>(word) << 32) ^ word_index);
}

// ----------------------------------------------------------------------------- input patterns
enum Pattern : int {
  kPatternReference = 0,  // the reference project's closed-form inputs (exact, order-free sums)
  kPatternSeeded = 1,     // counter-based RNG: uniform[-2,2) -> E4M3, ~N(0,1) -> F16/BF16
  kPatternTagged = 2,     // small exact values whose sum differs per element and per world size
};

// Closed-form E4M3 input of the reference: magnitudes 2^-4 .. 0.46875 on a 2^-7 grid.
MSHARP_HD uint8_t reference_e4m3_byte(int rank, uint64_t element) {
  const uint32_t mix = static_cast<uint32_t>((element * 17u) ^ (element >> 7) ^
                                             (static_cast<uint64_t>(rank + 1) * 29u));
  const uint32_t sign = ((mix >> 4) & 1u) << 7;
  const uint32_t expo = 3u + (mix % 3u);
  const uint32_t mant = (mix / 3u) & 7u;
  return static_cast<uint8_t>(sign | (expo << 3) | mant);
}

// Closed-form F16 input of the reference: an 8-entry table of multiples of 1/8.
MSHARP_HD uint16_t reference_f16_bits(int rank, uint64_t element) {
  const uint32_t mix = static_cast<uint32_t>((element * 13u) ^ (element >> 5) ^
                                             (static_cast<uint64_t>(rank + 1) * 7u)) & 7u;
  // -0.5 -0.25 -0.125 0 0.125 0.25 0.5 0
  const uint64_t table_lo = 0x0000b000b400b800ull;  // entries 0..3, 16 bits each
  const uint64_t table_hi = 0x0000380034003000ull;  // entries 4..7
  const uint64_t table = mix < 4 ? table_lo : table_hi;
  return static_cast<uint16_t>(table >> ((mix & 3u) * 16u));
}

MSHARP_HD uint64_t counter_rng(uint64_t seed, int rank, uint64_t element, uint32_t stream) {
  const uint64_t key = mix64(seed ^ (0x9e3779b97f4a7c15ull * static_cast<uint64_t>(rank + 1)));
  return mix64(key + element * 0xd1342543de82ef95ull + static_cast<uint64_t>(stream) * 0x2545f4914f6cdd1dull);
}

// uniform on [-2, 2) with 24 random bits, exactly representable in binary32.
MSHARP_HD float seeded_uniform_pm2(uint64_t seed, int rank, uint64_t element) {
  const uint32_t u24 = static_cast<uint32_t>(counter_rng(seed, rank, element, 0) >> 40);
  const int32_t centred = static_cast<int32_t>(u24) - (1 << 23);
  // centred * 2^-22: int -> float is exact for |centred| <= 2^23.
  return static_cast<float>(centred) * 2.3841857910156250e-07f;
}

// Approximately N(0,1): sum of twelve 16-bit uniforms (Irwin-Hall, variance exactly 1 up to
// the 2^-16 grid), computed in integers so that host and device agree bit for bit.
MSHARP_HD float seeded_normal(uint64_t seed, int rank, uint64_t element) {
  int32_t sum = 0;
MSHARP_UNROLL
  for (uint32_t s = 0; s < 3; ++s) {
    const uint64_t r = counter_rng(seed, rank, element, 1 + s);
    sum += static_cast<int32_t>(r & 0xffffu) + static_cast<int32_t>((r >> 16) & 0xffffu) +
           static_cast<int32_t>((r >> 32) & 0xffffu) + static_cast<int32_t>((r >> 48) & 0xffffu);
  }
  sum -= 6 * 65535;
  return static_cast<float>(sum) * 1.52587890625e-05f;  // * 2^-16, exact
}

// Tagged pattern: value = ((element mod 61) - 30 + 3*rank) / 8 for 16-bit types (exact sums
// that are never identically zero across ranks); FP8 uses its own small-integer pattern below.
MSHARP_HD float tagged_value(int rank, uint64_t element) {
  const int v = static_cast<int>(element % 61u) - 30 + 3 * (rank % 8);
  return static_cast<float>(v) * 0.125f;
}

MSHARP_HD uint8_t tagged_e4m3_byte(int rank, uint64_t element) {
  // {-1, 0, 1, 2} / 16: the sum over up to 8 ranks is an integer in [-8, 16] sixteenths, which
  // FP8 E4M3 represents exactly (four significant bits), so even the FP8 result is order-free.
  const int v = static_cast<int>(counter_rng(0x7a67u, rank, element, 9) & 3u) - 1;
  return encode_e4m3(static_cast<float>(v) * 0.0625f);
}

MSHARP_HD uint8_t pattern_e4m3_byte(int pattern, uint64_t seed, int rank, uint64_t element) {
  switch (pattern) {
    case kPatternSeeded:
      return encode_e4m3(seeded_uniform_pm2(seed, rank, element));
    case kPatternTagged:
      return tagged_e4m3_byte(rank, element);
    default:
      return reference_e4m3_byte(rank, element);
  }
}

MSHARP_HD uint32_t pattern_e4m3_word(int pattern, uint64_t seed, int rank, uint64_t word) {
  uint32_t packed = 0;
MSHARP_UNROLL
  for (int lane = 0; lane < 4; ++lane) {
    packed |= static_cast<uint32_t>(pattern_e4m3_byte(pattern, seed, rank, word * 4 + lane)) << (8 * lane);
  }
  return packed;
}

MSHARP_HD float pattern_value_16(int pattern, uint64_t seed, int rank, uint64_t element) {
  switch (pattern) {
    case kPatternSeeded:
      return seeded_normal(seed, rank, element);
    case kPatternTagged:
      return tagged_value(rank, element);
    default:
      return decode_f16(reference_f16_bits(rank, element));
  }
}

MSHARP_HD uint16_t pattern_f16_bits(int pattern, uint64_t seed, int rank, uint64_t element) {
  if (pattern == kPatternReference) {
    return reference_f16_bits(rank, element);
  }
  return encode_f16(pattern_value_16(pattern, seed, rank, element));
}

MSHARP_HD uint16_t pattern_bf16_bits(int pattern, uint64_t seed, int rank, uint64_t element) {
  return encode_bf16(pattern_value_16(pattern, seed, rank, element));
}

}  // namespace msharp
