// msharp_hash_no_alloc: the replica hash with its working memory built into the library image.
// See msharp/no_alloc.h for who needs this and for the rules of use.
#include "msharp/no_alloc.h"

#include <cuda_runtime.h>

#include <mutex>
#include <string>

#include "msharp/numerics.h"

namespace {

constexpr int kSlots = 1024;                       // one partial hash per 4 MiB of input
constexpr size_t kBytesPerSlot = 4ull << 20;
constexpr int kThreads = 256;
constexpr int kMaxDevices = 64;

// [0, kSlots): partial hashes, one per block; [kSlots]: how many blocks have delivered theirs.
// Lives in every GPU's copy of the library image. In host code this name is only a stand-in: it
// is not a device address, so host code never hands it to a kernel; it asks the runtime for the
// real address once per device (scratch_for_current_device) and passes that.
static __device__ __align__(256) unsigned long long g_hash_scratch[kSlots + 32];

__global__ void hash_no_alloc_kernel(const uint4* data, size_t vectors, size_t tail_words, unsigned long long* scratch,
                                     unsigned long long* out) {
  unsigned long long h = 0;
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t v = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; v < vectors; v += stride) {
    const uint4 q = data[v];
    const uint64_t base = v * 4;
    h ^= msharp::hash_term(q.x, base) ^ msharp::hash_term(q.y, base + 1) ^ msharp::hash_term(q.z, base + 2) ^
         msharp::hash_term(q.w, base + 3);
  }
  if (blockIdx.x == 0 && threadIdx.x < tail_words) {
    const uint64_t word = vectors * 4 + threadIdx.x;
    h ^= msharp::hash_term(reinterpret_cast<const uint32_t*>(data)[word], word);
  }
  __shared__ unsigned long long warp_hash[kThreads / 32];
  __shared__ bool is_last;
  for (int off = 16; off > 0; off >>= 1) {
    h ^= __shfl_xor_sync(0xffffffffu, h, off);
  }
  if ((threadIdx.x & 31) == 0) {
    warp_hash[threadIdx.x >> 5] = h;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned long long block_hash = 0;
    for (int w = 0; w < kThreads / 32; ++w) {
      block_hash ^= warp_hash[w];
    }
    scratch[blockIdx.x] = block_hash;
    __threadfence();  // the partial is visible before the arrival is counted
    const unsigned long long arrived = atomicAdd(&scratch[kSlots], 1ull);
    is_last = arrived + 1 == gridDim.x;
  }
  __syncthreads();
  if (!is_last) {
    return;
  }
  // the last block to arrive folds all partials
  __threadfence();
  unsigned long long total = 0;
  for (unsigned i = threadIdx.x; i < gridDim.x; i += blockDim.x) {
    total ^= *reinterpret_cast<volatile unsigned long long*>(&scratch[i]);
  }
  for (int off = 16; off > 0; off >>= 1) {
    total ^= __shfl_xor_sync(0xffffffffu, total, off);
  }
  __syncthreads();
  if ((threadIdx.x & 31) == 0) {
    warp_hash[threadIdx.x >> 5] = total;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned long long result = 0;
    for (int w = 0; w < kThreads / 32; ++w) {
      result ^= warp_hash[w];
    }
    *out = result;
    scratch[kSlots] = 0;  // the next call starts from zero arrivals
  }
}

thread_local std::string g_no_alloc_error;

// Device address of g_hash_scratch on the current device, looked up once per device.
cudaError_t scratch_for_current_device(unsigned long long** out) {
  static std::mutex mu;
  static unsigned long long* known[kMaxDevices] = {nullptr};
  int device = 0;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess) {
    return err;
  }
  std::lock_guard<std::mutex> lock(mu);
  if (device >= 0 && device < kMaxDevices && known[device] != nullptr) {
    *out = known[device];
    return cudaSuccess;
  }
  void* address = nullptr;
  err = cudaGetSymbolAddress(&address, g_hash_scratch);
  if (err != cudaSuccess) {
    return err;
  }
  *out = static_cast<unsigned long long*>(address);
  if (device >= 0 && device < kMaxDevices) {
    known[device] = *out;
  }
  return cudaSuccess;
}

int fail(const std::string& message) {
  g_no_alloc_error = message;
  return 1;
}

}  // namespace

extern "C" const char* msharp_no_alloc_last_error(void) { return g_no_alloc_error.c_str(); }

extern "C" int msharp_hash_no_alloc(uint64_t data, size_t bytes, uint64_t out_hash_device, uint64_t stream) {
  if (data == 0 || out_hash_device == 0) {
    return fail("hash_no_alloc: null pointer");
  }
  if (data % 16 != 0 || out_hash_device % 8 != 0) {
    return fail("hash_no_alloc: data must be 16-byte aligned and the result 8-byte aligned");
  }
  if (bytes == 0 || bytes % 4 != 0) {
    return fail("hash_no_alloc: size must be a nonzero multiple of 4 bytes");
  }
  if (bytes > MSHARP_NO_ALLOC_HASH_MAX_BYTES) {
    return fail("hash_no_alloc: " + std::to_string(bytes) + " bytes exceed the " +
                std::to_string(MSHARP_NO_ALLOC_HASH_MAX_BYTES) + " bytes that the built-in scratch array covers");
  }
  unsigned long long* scratch = nullptr;
  cudaError_t err = scratch_for_current_device(&scratch);
  if (err != cudaSuccess) {
    return fail(std::string("hash_no_alloc: cudaGetSymbolAddress failed: ") + cudaGetErrorString(err));
  }
  cudaStream_t s = reinterpret_cast<cudaStream_t>(static_cast<uintptr_t>(stream));
  // The arrival counter must be zero when the kernel starts. The kernel leaves it at zero, but an
  // earlier call that was cut short would not have, so it is cleared here as well (a memset on
  // memory that already exists; nothing is allocated).
  err = cudaMemsetAsync(scratch + kSlots, 0, sizeof(unsigned long long), s);
  if (err != cudaSuccess) {
    return fail(std::string("hash_no_alloc: clearing the arrival counter failed: ") + cudaGetErrorString(err));
  }
  const size_t vectors = bytes / 16;
  const size_t tail_words = (bytes % 16) / 4;
  const size_t want = (bytes + kBytesPerSlot - 1) / kBytesPerSlot;
  const int grid = static_cast<int>(want < 1 ? 1 : (want > kSlots ? kSlots : want));
  hash_no_alloc_kernel<<<grid, kThreads, 0, s>>>(reinterpret_cast<const uint4*>(static_cast<uintptr_t>(data)), vectors,
                                                 tail_words, scratch,
                                                 reinterpret_cast<unsigned long long*>(static_cast<uintptr_t>(out_hash_device)));
  err = cudaPeekAtLastError();
  if (err != cudaSuccess) {
    return fail(std::string("hash_no_alloc: launch failed: ") + cudaGetErrorString(err));
  }
  g_no_alloc_error.clear();
  return 0;
}
