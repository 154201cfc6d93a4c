#include "msharp/host_emulation.h"

#include <algorithm>
#include <cstring>
#include <stdexcept>
#include <vector>

#include "msharp/numerics.h"

namespace msharp {

void emulate_allreduce(Bootstrap& comm, const SymmetricMemory& mem, Dtype dtype, std::size_t in_offset,
                       std::size_t out_offset, std::size_t bytes, const float* in_scales, float out_scale_inv) {
  const int world = mem.world();
  const int rank = mem.rank();
  const std::size_t size = dtype_size(dtype);
  if (bytes % size != 0) {
    throw std::runtime_error("emulated all-reduce: size is not a whole number of elements");
  }
  if (in_offset > mem.alloc_bytes || bytes > mem.alloc_bytes - in_offset || out_offset > mem.alloc_bytes ||
      bytes > mem.alloc_bytes - out_offset) {
    throw std::runtime_error("emulated all-reduce: range is outside the allocation");
  }
  const std::size_t elements = bytes / size;
  const std::size_t per_rank = (elements + static_cast<std::size_t>(world) - 1) / static_cast<std::size_t>(world);
  const std::size_t begin = std::min(elements, per_rank * static_cast<std::size_t>(rank));
  const std::size_t end = std::min(elements, begin + per_rank);
  auto slot = [&](int r) { return reinterpret_cast<unsigned char*>(static_cast<uintptr_t>(mem.uc_slots[static_cast<std::size_t>(r)])); };

  comm.barrier();  // opening barrier: every rank's input is in place
  std::vector<unsigned char> slice((end - begin) * size);
  if (end > begin) {
    std::vector<float> sums(end - begin, 0.0f);
    std::vector<float> x(end - begin);
    for (int r = 0; r < world; ++r) {
      cast_to_f32(dtype, slot(r) + in_offset + begin * size, end - begin, x.data(), 1);
      const float scale = in_scales != nullptr ? in_scales[r] : 1.0f;
      for (std::size_t i = 0; i < x.size(); ++i) {
        sums[i] += scale * x[i];
      }
    }
    if (out_scale_inv != 1.0f) {
      for (float& v : sums) {
        v *= out_scale_inv;
      }
    }
    cast_from_f32(dtype, sums.data(), end - begin, slice.data(), 1);
  }
  comm.barrier();  // in place: no slice is overwritten while a peer may still read it
  for (int r = 0; r < world && end > begin; ++r) {
    std::memcpy(slot(r) + out_offset + begin * size, slice.data(), slice.size());
  }
  comm.barrier();  // closing barrier: every slice has landed in every copy
}

void emulate_gemm_partial_bf16(const uint8_t* a, const float* a_scales, const uint8_t* w, const float* w_scales, int m,
                               int n, int k, uint16_t* out_bf16) {
  constexpr int kBlockK = 128;
  if (m <= 0 || n <= 0 || k <= 0 || k % kBlockK != 0 || n % kBlockK != 0) {
    throw std::runtime_error("emulated GEMM: N and K must be positive multiples of 128");
  }
  const int k_blocks = k / kBlockK;
  float table[256];
  for (int c = 0; c < 256; ++c) {
    table[c] = decode_e4m3(static_cast<uint8_t>(c));
  }
  std::vector<float> a_row(static_cast<std::size_t>(k));
  for (int i = 0; i < m; ++i) {
    for (int kk = 0; kk < k; ++kk) {
      a_row[static_cast<std::size_t>(kk)] = table[a[static_cast<std::size_t>(i) * k + kk]];
    }
    for (int j = 0; j < n; ++j) {
      const uint8_t* w_row = w + static_cast<std::size_t>(j) * k;
      float acc = 0.0f;
      for (int kb = 0; kb < k_blocks; ++kb) {
        float partial = 0.0f;
        for (int kk = kb * kBlockK; kk < (kb + 1) * kBlockK; ++kk) {
          partial += a_row[static_cast<std::size_t>(kk)] * table[w_row[kk]];
        }
        acc += partial * (a_scales[static_cast<std::size_t>(i) * k_blocks + kb] *
                          w_scales[static_cast<std::size_t>(j / kBlockK) * k_blocks + kb]);
      }
      out_bf16[static_cast<std::size_t>(i) * n + j] = encode_bf16(acc);
    }
  }
}

}  // namespace msharp
