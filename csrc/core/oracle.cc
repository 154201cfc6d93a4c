#include "msharp/oracle.h"

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <functional>
#include <sstream>
#include <thread>

#include "msharp/numerics.h"

namespace msharp {
namespace {

// Run fn(begin, end, worker_index) over [0, n) split into contiguous chunks.
void parallel_for(std::size_t n, int threads,
                  const std::function<void(std::size_t, std::size_t, int)>& fn) {
  if (threads <= 0) {
    threads = default_threads();
  }
  const std::size_t min_chunk = 1u << 14;
  const std::size_t max_workers = std::max<std::size_t>(1, n / min_chunk);
  const int workers = static_cast<int>(std::min<std::size_t>(static_cast<std::size_t>(threads), max_workers));
  if (workers <= 1) {
    fn(0, n, 0);
    return;
  }
  std::vector<std::thread> pool;
  pool.reserve(static_cast<std::size_t>(workers));
  const std::size_t chunk = (n + static_cast<std::size_t>(workers) - 1) / static_cast<std::size_t>(workers);
  for (int w = 0; w < workers; ++w) {
    const std::size_t begin = std::min(n, chunk * static_cast<std::size_t>(w));
    const std::size_t end = std::min(n, begin + chunk);
    pool.emplace_back([=, &fn] { fn(begin, end, w); });
  }
  for (auto& t : pool) {
    t.join();
  }
}

inline float load_input(Dtype dtype, const InputSpec& spec, int rank, std::size_t element) {
  switch (dtype) {
    case Dtype::kE4M3:
      return decode_e4m3(pattern_e4m3_byte(spec.pattern, spec.seed, rank, element));
    case Dtype::kF16:
      return decode_f16(pattern_f16_bits(spec.pattern, spec.seed, rank, element));
    case Dtype::kBF16:
      return decode_bf16(pattern_bf16_bits(spec.pattern, spec.seed, rank, element));
  }
  return 0.0f;
}

// ---- block-wise input generation ----------------------------------------------------------------
// The reductions walk the elements in blocks and the ranks inside a block, so that what depends on
// the rank alone (the key of the counter-based generator) is computed once per block instead of once
// per element, and the inner loops run over contiguous arrays. Values are bit-identical to
// load_input(): same formulas (numerics.h counter_rng / seeded_uniform_pm2 / seeded_normal), same
// float32 additions in rank order.
constexpr std::size_t kBlock = 256;

inline uint64_t rng_key(uint64_t seed, int rank) {
  return mix64(seed ^ (0x9e3779b97f4a7c15ull * static_cast<uint64_t>(rank + 1)));
}

inline uint64_t rng_keyed(uint64_t key, uint64_t element, uint32_t stream) {
  return mix64(key + element * 0xd1342543de82ef95ull + static_cast<uint64_t>(stream) * 0x2545f4914f6cdd1dull);
}

inline float uniform_pm2_keyed(uint64_t key, uint64_t element) {
  const uint32_t u24 = static_cast<uint32_t>(rng_keyed(key, element, 0) >> 40);
  return static_cast<float>(static_cast<int32_t>(u24) - (1 << 23)) * 2.3841857910156250e-07f;
}

inline float normal_keyed(uint64_t key, uint64_t element) {
  int32_t sum = 0;
  for (uint32_t s = 0; s < 3; ++s) {
    const uint64_t r = rng_keyed(key, element, 1 + s);
    sum += static_cast<int32_t>(r & 0xffffu) + static_cast<int32_t>((r >> 16) & 0xffffu) +
           static_cast<int32_t>((r >> 32) & 0xffffu) + static_cast<int32_t>((r >> 48) & 0xffffu);
  }
  sum -= 6 * 65535;
  return static_cast<float>(sum) * 1.52587890625e-05f;
}

// Decoded inputs of `rank` for elements [first, first + count), count <= kBlock.
inline void load_block(Dtype dtype, const InputSpec& spec, int rank, std::size_t first, std::size_t count, float* out) {
  if (spec.pattern == kPatternSeeded) {
    const uint64_t key = rng_key(spec.seed, rank);
    switch (dtype) {
      case Dtype::kE4M3:
        for (std::size_t i = 0; i < count; ++i) {
          out[i] = decode_e4m3(encode_e4m3(uniform_pm2_keyed(key, first + i)));
        }
        return;
      case Dtype::kF16:
        for (std::size_t i = 0; i < count; ++i) {
          out[i] = decode_f16(encode_f16(normal_keyed(key, first + i)));
        }
        return;
      case Dtype::kBF16:
        for (std::size_t i = 0; i < count; ++i) {
          out[i] = decode_bf16(encode_bf16(normal_keyed(key, first + i)));
        }
        return;
    }
  }
  for (std::size_t i = 0; i < count; ++i) {
    out[i] = load_input(dtype, spec, rank, first + i);
  }
}

// Float32 sums (rank order) of one block.
inline void f32_sum_block(Dtype dtype, const InputSpec& spec, std::size_t first, std::size_t count, float* acc) {
  float x[kBlock];
  std::fill(acc, acc + count, 0.0f);
  for (int r = 0; r < spec.ranks; ++r) {
    load_block(dtype, spec, r, first, count, x);
    for (std::size_t i = 0; i < count; ++i) {
      acc[i] += x[i];
    }
  }
}

// Sequential sums with a rounding to the accumulator type after every add (the reference's model).
inline void semantic_sum_block(Dtype dtype, const InputSpec& spec, std::size_t first, std::size_t count, float* acc) {
  float x[kBlock];
  std::fill(acc, acc + count, 0.0f);
  for (int r = 0; r < spec.ranks; ++r) {
    load_block(dtype, spec, r, first, count, x);
    if (dtype == Dtype::kBF16) {
      for (std::size_t i = 0; i < count; ++i) {
        acc[i] = decode_bf16(encode_bf16(acc[i] + x[i]));
      }
    } else {
      for (std::size_t i = 0; i < count; ++i) {
        acc[i] = round_to_f16(acc[i] + x[i]);
      }
    }
  }
}

// Both models of one block with a single pass over the generated inputs.
inline void both_sums_block(Dtype dtype, const InputSpec& spec, std::size_t first, std::size_t count, float* sequential,
                            float* sum32) {
  float x[kBlock];
  std::fill(sequential, sequential + count, 0.0f);
  std::fill(sum32, sum32 + count, 0.0f);
  for (int r = 0; r < spec.ranks; ++r) {
    load_block(dtype, spec, r, first, count, x);
    for (std::size_t i = 0; i < count; ++i) {
      sum32[i] += x[i];
      sequential[i] = dtype == Dtype::kBF16 ? decode_bf16(encode_bf16(sequential[i] + x[i])) : round_to_f16(sequential[i] + x[i]);
    }
  }
}

inline float semantic_sum(Dtype dtype, const InputSpec& spec, std::size_t element) {
  float acc = 0.0f;
  if (dtype == Dtype::kBF16) {
    for (int r = 0; r < spec.ranks; ++r) {
      acc = decode_bf16(encode_bf16(acc + load_input(dtype, spec, r, element)));
    }
  } else {
    for (int r = 0; r < spec.ranks; ++r) {
      acc = round_to_f16(acc + load_input(dtype, spec, r, element));
    }
  }
  return acc;
}

inline void store_cast(Dtype dtype, void* out, std::size_t index, float value) {
  switch (dtype) {
    case Dtype::kE4M3:
      static_cast<uint8_t*>(out)[index] = encode_e4m3(value);
      break;
    case Dtype::kF16:
      static_cast<uint16_t*>(out)[index] = encode_f16(value);
      break;
    case Dtype::kBF16:
      static_cast<uint16_t*>(out)[index] = encode_bf16(value);
      break;
  }
}

inline uint32_t load_code(Dtype dtype, const void* in, std::size_t index) {
  return dtype == Dtype::kE4M3 ? static_cast<const uint8_t*>(in)[index]
                               : static_cast<const uint16_t*>(in)[index];
}

inline float decode_code(Dtype dtype, uint32_t code) {
  switch (dtype) {
    case Dtype::kE4M3:
      return decode_e4m3(static_cast<uint8_t>(code));
    case Dtype::kF16:
      return decode_f16(static_cast<uint16_t>(code));
    case Dtype::kBF16:
      return decode_bf16(static_cast<uint16_t>(code));
  }
  return 0.0f;
}

inline uint32_t encode_code(Dtype dtype, float value) {
  switch (dtype) {
    case Dtype::kE4M3:
      return encode_e4m3(value);
    case Dtype::kF16:
      return encode_f16(value);
    case Dtype::kBF16:
      return encode_bf16(value);
  }
  return 0;
}

inline int ordered_code(Dtype dtype, uint32_t code) {
  return dtype == Dtype::kE4M3 ? ordered_code_e4m3(static_cast<uint8_t>(code))
                               : ordered_code_f16(static_cast<uint16_t>(code));
}

}  // namespace

int default_threads() {
  const unsigned hw = std::thread::hardware_concurrency();
  return static_cast<int>(hw == 0 ? 4 : std::min(hw, 64u));
}

const char* dtype_name(Dtype t) {
  switch (t) {
    case Dtype::kE4M3:
      return "e4m3";
    case Dtype::kF16:
      return "f16";
    case Dtype::kBF16:
      return "bf16";
  }
  return "unknown";
}

std::size_t dtype_size(Dtype t) { return t == Dtype::kE4M3 ? 1 : 2; }

TimingStats summarize(std::vector<double> values) {
  TimingStats s;
  if (values.empty()) {
    return s;
  }
  std::sort(values.begin(), values.end());
  const std::size_t n = values.size();
  s.min = values.front();
  s.max = values.back();
  s.median = values[n / 2];
  const std::size_t rank95 = static_cast<std::size_t>(std::ceil(static_cast<double>(n) * 0.95));
  s.p95 = values[std::min(n - 1, rank95 == 0 ? 0 : rank95 - 1)];
  return s;
}

void generate_input(Dtype dtype, const InputSpec& spec, int rank, std::size_t first_element,
                    std::size_t element_count, void* out, int threads) {
  parallel_for(element_count, threads, [&](std::size_t b, std::size_t e, int) {
    for (std::size_t i = b; i < e; ++i) {
      const std::size_t g = first_element + i;
      switch (dtype) {
        case Dtype::kE4M3:
          static_cast<uint8_t*>(out)[i] = pattern_e4m3_byte(spec.pattern, spec.seed, rank, g);
          break;
        case Dtype::kF16:
          static_cast<uint16_t*>(out)[i] = pattern_f16_bits(spec.pattern, spec.seed, rank, g);
          break;
        case Dtype::kBF16:
          static_cast<uint16_t*>(out)[i] = pattern_bf16_bits(spec.pattern, spec.seed, rank, g);
          break;
      }
    }
  });
}

void reduce_semantic(Dtype dtype, const InputSpec& spec, std::size_t first_element,
                     std::size_t element_count, void* out, int threads) {
  parallel_for(element_count, threads, [&](std::size_t b, std::size_t e, int) {
    float acc[kBlock];
    for (std::size_t at = b; at < e; at += kBlock) {
      const std::size_t count = std::min(kBlock, e - at);
      semantic_sum_block(dtype, spec, first_element + at, count, acc);
      for (std::size_t i = 0; i < count; ++i) {
        store_cast(dtype, out, at + i, acc[i]);
      }
    }
  });
}

void reduce_f32(Dtype dtype, const InputSpec& spec, std::size_t first_element,
                std::size_t element_count, float* out, int threads) {
  parallel_for(element_count, threads, [&](std::size_t b, std::size_t e, int) {
    for (std::size_t at = b; at < e; at += kBlock) {
      f32_sum_block(dtype, spec, first_element + at, std::min(kBlock, e - at), out + at);
    }
  });
}

void reduce_f32_cast(Dtype dtype, const InputSpec& spec, std::size_t first_element,
                     std::size_t element_count, void* out, int threads) {
  parallel_for(element_count, threads, [&](std::size_t b, std::size_t e, int) {
    float acc[kBlock];
    for (std::size_t at = b; at < e; at += kBlock) {
      const std::size_t count = std::min(kBlock, e - at);
      f32_sum_block(dtype, spec, first_element + at, count, acc);
      for (std::size_t i = 0; i < count; ++i) {
        store_cast(dtype, out, at + i, acc[i]);
      }
    }
  });
}

PrecisionMetrics compare(Dtype dtype, const InputSpec& spec, const void* result,
                         std::size_t element_count, int threads) {
  if (threads <= 0) {
    threads = default_threads();
  }
  struct Partial {
    std::size_t exact = 0, requant = 0, switch_model = 0;
    int ulp = 0;
    float max_err = 0.0f;
    double sum_err = 0.0;
    bool nan_err = false;
  };
  std::vector<Partial> partials(static_cast<std::size_t>(threads));
  parallel_for(element_count, threads, [&](std::size_t b, std::size_t e, int w) {
    Partial p;
    float sequential_block[kBlock];
    float sum32_block[kBlock];
    for (std::size_t i = b; i < e; ++i) {
      if ((i - b) % kBlock == 0) {
        both_sums_block(dtype, spec, i, std::min(kBlock, e - i), sequential_block, sum32_block);
      }
      const uint32_t got = load_code(dtype, result, i);
      const float sequential = sequential_block[(i - b) % kBlock];
      const uint32_t want_semantic = encode_code(dtype, sequential);
      // In-switch FP8: the value just below or just above the sum is accepted; a sum that is
      // representable must come back as itself; beyond +-448 the switch may answer NaN.
      bool switch_ok = got == want_semantic;
      if (!switch_ok && dtype == Dtype::kE4M3) {
        const float nearest = decode_code(dtype, want_semantic);
        if ((got & 0x7fu) == 0x7fu) {
          switch_ok = std::fabs(sequential) > 448.0f;
        } else if (nearest == sequential) {
          switch_ok = decode_code(dtype, got) == sequential;  // covers -0 vs +0
        } else {
          const float other = decode_code(dtype, got);
          const int step = std::abs(ordered_code(dtype, got) - ordered_code(dtype, want_semantic));
          switch_ok = step == 1 && (other - sequential) * (nearest - sequential) < 0.0f;
        }
      }
      p.switch_model += !switch_ok;
      const float sum32 = sum32_block[(i - b) % kBlock];
      const uint32_t want_requant = encode_code(dtype, sum32);
      p.exact += got != want_semantic;
      p.requant += got != want_requant;
      p.ulp = std::max(p.ulp, std::abs(ordered_code(dtype, got) - ordered_code(dtype, want_requant)));
      const float err = std::fabs(decode_code(dtype, got) - sum32);
      if (err != err) {
        p.nan_err = true;
      } else {
        p.max_err = std::max(p.max_err, err);
        p.sum_err += err;
      }
    }
    partials[static_cast<std::size_t>(w)] = p;
  });
  PrecisionMetrics m;
  double sum = 0.0;
  bool nan_err = false;
  for (const auto& p : partials) {
    m.exact_mismatches += p.exact;
    m.switch_model_mismatches += p.switch_model;
    m.requantized_mismatches += p.requant;
    m.max_requantized_ulp_distance = std::max(m.max_requantized_ulp_distance, p.ulp);
    m.max_abs_error = std::max(m.max_abs_error, p.max_err);
    sum += p.sum_err;
    nan_err = nan_err || p.nan_err;
  }
  m.mean_abs_error = element_count == 0 ? 0.0 : sum / static_cast<double>(element_count);
  if (nan_err) {
    m.max_abs_error = std::nanf("");
    m.mean_abs_error = std::nan("");
  }
  return m;
}

void reduce_arrays_f32(Dtype dtype, const void* const* inputs, int ranks, std::size_t element_count,
                       float* out, int threads) {
  parallel_for(element_count, threads, [&](std::size_t b, std::size_t e, int) {
    for (std::size_t i = b; i < e; ++i) {
      float acc = 0.0f;
      for (int r = 0; r < ranks; ++r) {
        acc += decode_code(dtype, load_code(dtype, inputs[r], i));
      }
      out[i] = acc;
    }
  });
}

void cast_from_f32(Dtype dtype, const float* in, std::size_t element_count, void* out, int threads) {
  parallel_for(element_count, threads, [&](std::size_t b, std::size_t e, int) {
    for (std::size_t i = b; i < e; ++i) {
      store_cast(dtype, out, i, in[i]);
    }
  });
}

void cast_to_f32(Dtype dtype, const void* in, std::size_t element_count, float* out, int threads) {
  parallel_for(element_count, threads, [&](std::size_t b, std::size_t e, int) {
    for (std::size_t i = b; i < e; ++i) {
      out[i] = decode_code(dtype, load_code(dtype, in, i));
    }
  });
}

uint64_t hash_words(const uint32_t* words, std::size_t word_count, int threads) {
  if (threads <= 0) {
    threads = default_threads();
  }
  std::vector<uint64_t> partial(static_cast<std::size_t>(threads), 0);
  parallel_for(word_count, threads, [&](std::size_t b, std::size_t e, int w) {
    uint64_t h = 0;
    for (std::size_t i = b; i < e; ++i) {
      h ^= hash_term(words[i], i);
    }
    partial[static_cast<std::size_t>(w)] = h;
  });
  uint64_t h = 0;
  for (uint64_t p : partial) {
    h ^= p;
  }
  return h;
}

bool hashes_match(const std::vector<uint64_t>& hashes) {
  for (uint64_t h : hashes) {
    if (h != hashes.front()) {
      return false;
    }
  }
  return true;
}

std::string mismatch_dump(Dtype dtype, const InputSpec& spec, const void* result,
                          std::size_t element_count, std::size_t max_items) {
  std::ostringstream os;
  if (dtype == Dtype::kE4M3) {
    os << "debug_first_words:";
    const auto* bytes = static_cast<const uint8_t*>(result);
    const std::size_t words = std::min(max_items, element_count / 4);
    for (std::size_t w = 0; w < words; ++w) {
      uint32_t got = 0, want = 0;
      for (int lane = 0; lane < 4; ++lane) {
        got |= static_cast<uint32_t>(bytes[w * 4 + lane]) << (8 * lane);
        want |= static_cast<uint32_t>(encode_e4m3(semantic_sum(dtype, spec, w * 4 + lane))) << (8 * lane);
      }
      os << " [" << w << "] got=0x" << std::hex << got << " expected=0x" << want << std::dec;
    }
  } else {
    const std::size_t n = std::min(element_count, max_items);
    os << (dtype == Dtype::kF16 ? "debug_first_f16:" : "debug_first_bf16:");
    for (std::size_t i = 0; i < n; ++i) {
      os << " [" << i << "] got=0x" << std::hex << load_code(dtype, result, i) << " expected=0x"
         << encode_code(dtype, semantic_sum(dtype, spec, i)) << std::dec;
    }
  }
  return os.str();
}

}  // namespace msharp
