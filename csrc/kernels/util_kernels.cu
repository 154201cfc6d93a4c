#include <cuda_runtime.h>

#include <mutex>
#include <set>
#include <stdexcept>
#include <string>
#include <utility>

#include "device_comm.cuh"
#include "msharp/kernels.h"
#include "msharp/numerics.h"

namespace msharp {

void check_cuda(cudaError_t code, const char* expression) {
  if (code != cudaSuccess) {
    throw std::runtime_error(std::string(expression) + " failed: " + cudaGetErrorName(code) + ": " +
                             cudaGetErrorString(code));
  }
}

namespace {

constexpr int kThreads = 256;

int blocks_for(std::size_t items, int per_block, int cap) {
  const std::size_t want = (items + static_cast<std::size_t>(per_block) - 1) / static_cast<std::size_t>(per_block);
  return static_cast<int>(want < 1 ? 1 : (want > static_cast<std::size_t>(cap) ? static_cast<std::size_t>(cap) : want));
}

void check_launch(const char* kernel) {
  const cudaError_t err = cudaPeekAtLastError();
  if (err != cudaSuccess) {
    throw std::runtime_error(std::string(kernel) + " launch failed: " + cudaGetErrorString(err));
  }
}

// One thread produces 16 bytes (16 FP8 values or 8 half values) and stores them as one vector.
template <int DT>
__global__ void init_pattern_kernel(uint4* dst, std::size_t vectors, std::size_t tail_words, int pattern,
                                    uint64_t seed, int rank) {
  const std::size_t stride = static_cast<std::size_t>(gridDim.x) * blockDim.x;
  for (std::size_t v = static_cast<std::size_t>(blockIdx.x) * blockDim.x + threadIdx.x; v < vectors; v += stride) {
    uint32_t w[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const uint64_t word = v * 4 + k;
      if constexpr (DT == 0) {
        w[k] = pattern_e4m3_word(pattern, seed, rank, word);
      } else if constexpr (DT == 1) {
        w[k] = static_cast<uint32_t>(pattern_f16_bits(pattern, seed, rank, word * 2)) |
               (static_cast<uint32_t>(pattern_f16_bits(pattern, seed, rank, word * 2 + 1)) << 16);
      } else {
        w[k] = static_cast<uint32_t>(pattern_bf16_bits(pattern, seed, rank, word * 2)) |
               (static_cast<uint32_t>(pattern_bf16_bits(pattern, seed, rank, word * 2 + 1)) << 16);
      }
    }
    dst[v] = make_uint4(w[0], w[1], w[2], w[3]);
  }
  // up to three trailing 32-bit words when the size is not a multiple of 16 bytes
  if (blockIdx.x == 0 && threadIdx.x < tail_words) {
    const uint64_t word = vectors * 4 + threadIdx.x;
    uint32_t value;
    if constexpr (DT == 0) {
      value = pattern_e4m3_word(pattern, seed, rank, word);
    } else if constexpr (DT == 1) {
      value = static_cast<uint32_t>(pattern_f16_bits(pattern, seed, rank, word * 2)) |
              (static_cast<uint32_t>(pattern_f16_bits(pattern, seed, rank, word * 2 + 1)) << 16);
    } else {
      value = static_cast<uint32_t>(pattern_bf16_bits(pattern, seed, rank, word * 2)) |
              (static_cast<uint32_t>(pattern_bf16_bits(pattern, seed, rank, word * 2 + 1)) << 16);
    }
    reinterpret_cast<uint32_t*>(dst)[word] = value;
  }
}

__global__ void poison_kernel(uint4* dst, std::size_t vectors, std::size_t tail_words) {
  const std::size_t stride = static_cast<std::size_t>(gridDim.x) * blockDim.x;
  const uint4 ones = make_uint4(0xffffffffu, 0xffffffffu, 0xffffffffu, 0xffffffffu);
  for (std::size_t v = static_cast<std::size_t>(blockIdx.x) * blockDim.x + threadIdx.x; v < vectors; v += stride) {
    dst[v] = ones;
  }
  if (blockIdx.x == 0 && threadIdx.x < tail_words) {
    reinterpret_cast<uint32_t*>(dst)[vectors * 4 + threadIdx.x] = 0xffffffffu;
  }
}

__global__ void alias_fence_kernel() {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    dev::fence_proxy_alias();
  }
}

__global__ void async_proxy_fence_kernel() {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    dev::fence_proxy_async_global();
  }
}

__device__ __host__ inline uint32_t canary_word(int rank, int i) {
  return 0xC0010000u | ((static_cast<uint32_t>(rank) & 0xffu) << 8) | static_cast<uint32_t>(i);
}

__global__ void canary_write_kernel(uint32_t* self_words, int rank) {
  if (blockIdx.x == 0 && threadIdx.x < kCanaryWords) {
    self_words[threadIdx.x] = canary_word(rank, static_cast<int>(threadIdx.x));
  }
}

__global__ void canary_verify_kernel(DeviceComm comm, PeerPointers slots) {
  if (!dev::grid_peers_barrier(comm, kStatusEntryTimeout)) {
    return;
  }
  dev::fence_proxy_alias();
  for (int item = threadIdx.x; item < comm.world * kCanaryWords; item += blockDim.x) {
    const int slot = item / kCanaryWords;
    const int word = item % kCanaryWords;
    const volatile uint32_t* p = reinterpret_cast<const volatile uint32_t*>(slots.ptr[slot]);
    if (p[word] != canary_word(slot, word)) {
      dev::report(comm, kStatusCanaryMismatch, (static_cast<uint32_t>(slot) << 8) | static_cast<uint32_t>(word));
    }
  }
  // nobody may overwrite its canary before everyone has looked at it
  dev::grid_peers_barrier(comm, kStatusExitTimeout);
}

__global__ void hash_kernel(const uint4* data, std::size_t vectors, std::size_t tail_words, uint64_t* out) {
  uint64_t h = 0;
  const std::size_t stride = static_cast<std::size_t>(gridDim.x) * blockDim.x;
  for (std::size_t v = static_cast<std::size_t>(blockIdx.x) * blockDim.x + threadIdx.x; v < vectors; v += stride) {
    const uint4 q = data[v];
    const uint64_t base = v * 4;
    h ^= hash_term(q.x, base) ^ hash_term(q.y, base + 1) ^ hash_term(q.z, base + 2) ^ hash_term(q.w, base + 3);
  }
  if (blockIdx.x == 0 && threadIdx.x < tail_words) {
    const uint64_t word = vectors * 4 + threadIdx.x;
    h ^= hash_term(reinterpret_cast<const uint32_t*>(data)[word], word);
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    h ^= __shfl_xor_sync(0xffffffffu, h, off);
  }
  __shared__ uint64_t warp_hash[32];
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  if (lane == 0) {
    warp_hash[warp] = h;
  }
  __syncthreads();
  if (warp == 0) {
    h = lane < static_cast<int>((blockDim.x + 31) / 32) ? warp_hash[lane] : 0;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      h ^= __shfl_xor_sync(0xffffffffu, h, off);
    }
    if (lane == 0) {
      atomicXor(reinterpret_cast<unsigned long long*>(out), static_cast<unsigned long long>(h));
    }
  }
}

void require_aligned(const void* p, std::size_t bytes, const char* what) {
  if (reinterpret_cast<uintptr_t>(p) % 16 != 0) {
    throw std::runtime_error(std::string(what) + ": pointer must be 16-byte aligned");
  }
  if (bytes % 4 != 0) {
    throw std::runtime_error(std::string(what) + ": size must be a multiple of 4 bytes");
  }
}

}  // namespace

int device_sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  MSHARP_CUDA(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && cached[dev] != 0) {
    return cached[dev];
  }
  int sms = 0;
  MSHARP_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  if (dev >= 0 && dev < 64) {
    cached[dev] = sms;
  }
  return sms;
}

void ensure_max_dynamic_smem(const void* kernel, int bytes) {
  static std::mutex mu;
  static std::set<std::pair<const void*, int>> done;
  int device = 0;
  MSHARP_CUDA(cudaGetDevice(&device));
  std::lock_guard<std::mutex> lock(mu);
  if (done.count({kernel, device}) != 0) {
    return;
  }
  MSHARP_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
  done.insert({kernel, device});
}

void launch_init_pattern(Dtype dtype, int pattern, uint64_t seed, int rank, void* dst, std::size_t bytes,
                         cudaStream_t stream) {
  require_aligned(dst, bytes, "init");
  const std::size_t vectors = bytes / 16;
  const std::size_t tail_words = (bytes % 16) / 4;
  const int grid = blocks_for(vectors, kThreads, 148 * 16);
  switch (dtype) {
    case Dtype::kE4M3:
      init_pattern_kernel<0><<<grid, kThreads, 0, stream>>>(static_cast<uint4*>(dst), vectors, tail_words, pattern, seed, rank);
      break;
    case Dtype::kF16:
      init_pattern_kernel<1><<<grid, kThreads, 0, stream>>>(static_cast<uint4*>(dst), vectors, tail_words, pattern, seed, rank);
      break;
    case Dtype::kBF16:
      init_pattern_kernel<2><<<grid, kThreads, 0, stream>>>(static_cast<uint4*>(dst), vectors, tail_words, pattern, seed, rank);
      break;
  }
  check_launch("init_pattern_kernel");
}

void launch_poison_fill(void* dst, std::size_t bytes, cudaStream_t stream) {
  require_aligned(dst, bytes, "poison fill");
  const std::size_t vectors = bytes / 16;
  poison_kernel<<<blocks_for(vectors, kThreads, 148 * 16), kThreads, 0, stream>>>(static_cast<uint4*>(dst), vectors,
                                                                                (bytes % 16) / 4);
  check_launch("poison_kernel");
}

void launch_alias_fence(cudaStream_t stream) {
  alias_fence_kernel<<<1, 32, 0, stream>>>();
  check_launch("alias_fence_kernel");
}

void launch_async_proxy_fence(cudaStream_t stream) {
  async_proxy_fence_kernel<<<1, 32, 0, stream>>>();
  check_launch("async_proxy_fence_kernel");
}

void launch_canary_write(uint32_t* self_slot_words, int rank, cudaStream_t stream) {
  canary_write_kernel<<<1, 32, 0, stream>>>(self_slot_words, rank);
  check_launch("canary_write_kernel");
}

void launch_canary_verify(const DeviceComm& comm, const PeerPointers& slots, cudaStream_t stream) {
  canary_verify_kernel<<<1, 128, 0, stream>>>(comm, slots);
  check_launch("canary_verify_kernel");
}

void launch_hash(const void* data, std::size_t bytes, uint64_t* out_hash, cudaStream_t stream) {
  require_aligned(data, bytes, "hash");
  MSHARP_CUDA(cudaMemsetAsync(out_hash, 0, sizeof(uint64_t), stream));
  const std::size_t vectors = bytes / 16;
  hash_kernel<<<blocks_for(vectors, kThreads * 4, 148 * 8), kThreads, 0, stream>>>(static_cast<const uint4*>(data), vectors,
                                                                                 (bytes % 16) / 4, out_hash);
  check_launch("hash_kernel");
}

}  // namespace msharp
