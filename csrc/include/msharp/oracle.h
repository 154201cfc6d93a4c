// Host reference for the all-reduce: inputs are regenerated from their closed form, reduced
// on the CPU, and compared against what the GPUs produced.
//
// Parity with the reference project (paths within it):
//   src/e4m3_ref.cc:94-110,239-281  "semantic" model (ranks in order, round to fp16 after every
//                                   add, final encode) and the plain float32 model
//   src/e4m3_ref.cc:283-342         mismatch / distance / error metrics
//   src/main.cc:29-49               min / upper-median / p95 / max summary
// Added here: any input pattern (reference, seeded, tagged), BF16, a thread pool (this code is
// also the timed CPU baseline for 8 ranks x 16 MiB), and a host version of the replica hash.
#pragma once

#include <cstddef>
#include <cstdint>
#include <string>
#include <vector>

namespace msharp {

enum class Dtype : int { kE4M3 = 0, kF16 = 1, kBF16 = 2 };

const char* dtype_name(Dtype t);
std::size_t dtype_size(Dtype t);

struct InputSpec {
  int pattern = 0;        // Pattern enum of numerics.h
  uint64_t seed = 0;      // used by the seeded pattern only
  int ranks = 1;
};

struct PrecisionMetrics {
  std::size_t exact_mismatches = 0;        // vs the sequential-fp16 ("semantic") model
  std::size_t requantized_mismatches = 0;  // vs cast(float32 sum)
  int max_requantized_ulp_distance = 0;    // in representable-value steps
  float max_abs_error = 0.0f;              // vs the float32 sum
  double mean_abs_error = 0.0;
  // FP8 only: results that are neither the representable value just below nor the one just
  // above the sequential-fp16 sum (a representable sum must come back unchanged). Measured on
  // B200: multimem.ld_reduce .acc::f16.e4m3x4 returns either neighbour, not the nearest one,
  // and NaN instead of +-448 on overflow. Equals exact_mismatches for the 16-bit types.
  std::size_t switch_model_mismatches = 0;
};

struct TimingStats {
  double min = 0.0;
  double median = 0.0;  // upper median v[n/2]
  double p95 = 0.0;     // v[min(n-1, ceil(0.95 n) - 1)]
  double max = 0.0;
};

TimingStats summarize(std::vector<double> values);

// Fill `out` (element_count elements of `dtype`, packed) with rank `rank`'s input.
void generate_input(Dtype dtype, const InputSpec& spec, int rank, std::size_t first_element,
                    std::size_t element_count, void* out, int threads = 0);

// Sequential model: acc = round_fp16(acc + x_r) for r = 0..ranks-1, then cast to dtype.
// (For BF16 the running sum is rounded to bf16 instead of fp16.)
void reduce_semantic(Dtype dtype, const InputSpec& spec, std::size_t first_element,
                     std::size_t element_count, void* out, int threads = 0);

// Float32 model: plain binary32 accumulation in rank order, no intermediate rounding.
void reduce_f32(Dtype dtype, const InputSpec& spec, std::size_t first_element,
                std::size_t element_count, float* out, int threads = 0);

// cast(float32 sum) in `dtype`; this is the bitwise expected output for seeded inputs.
void reduce_f32_cast(Dtype dtype, const InputSpec& spec, std::size_t first_element,
                     std::size_t element_count, void* out, int threads = 0);

// Compare `result` (first `element_count` elements of a replica) with both models.
PrecisionMetrics compare(Dtype dtype, const InputSpec& spec, const void* result,
                         std::size_t element_count, int threads = 0);

// Same reduction over explicit per-rank input arrays (used by tests and the Python oracle).
void reduce_arrays_f32(Dtype dtype, const void* const* inputs, int ranks, std::size_t element_count,
                       float* out, int threads = 0);
void cast_from_f32(Dtype dtype, const float* in, std::size_t element_count, void* out, int threads = 0);
void cast_to_f32(Dtype dtype, const void* in, std::size_t element_count, float* out, int threads = 0);

// XOR over hash_term(word, index) for `word_count` 32-bit words: equals the device hash.
uint64_t hash_words(const uint32_t* words, std::size_t word_count, int threads = 0);

bool hashes_match(const std::vector<uint64_t>& hashes);

// Dump of the first mismatching elements, as printed when MNNVL_DEBUG_MISMATCH is set
// (reference: src/main.cc:357-387).
std::string mismatch_dump(Dtype dtype, const InputSpec& spec, const void* result,
                          std::size_t element_count, std::size_t max_items = 16);

int default_threads();

}  // namespace msharp
