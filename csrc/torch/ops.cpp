// PyTorch operator library: thin TORCH_LIBRARY wrappers over the C interface of libmsharp.so.
// Communicator and buffer handles travel as int64 (they are the pointers returned by the C
// interface); kernels are enqueued on PyTorch's current CUDA stream, so the operators compose
// with torch streams, events and CUDA-graph capture. No Triton, no dispatch layers, no
// cuBLAS / NCCL on these paths. The reference project has no Python or PyTorch surface.
#include <ATen/cuda/CUDAContext.h>
#include <torch/library.h>
#include <torch/torch.h>

#include <stdexcept>
#include <string>

#include "msharp/c_api.h"

namespace {

void check(int rc, const char* what) {
  if (rc != 0) {
    throw std::runtime_error(std::string(what) + ": " + msharp_last_error());
  }
}

// A machine without a CUDA device can only hold communicators on the host-memory driver stand-in,
// whose collectives the native library plays through on the CPU: no stream, CPU tensors.
bool have_device() { return at::hasCUDA() && at::cuda::device_count() > 0; }

uint64_t current_stream() {
  return have_device() ? reinterpret_cast<uint64_t>(at::cuda::getCurrentCUDAStream().stream()) : 0;
}

void* handle(int64_t h) { return reinterpret_cast<void*>(static_cast<intptr_t>(h)); }

int dtype_code(const std::string& name) {
  if (name == "e4m3") return 0;
  if (name == "f16") return 1;
  if (name == "bf16") return 2;
  throw std::invalid_argument("dtype must be e4m3, f16 or bf16");
}

// In-place all-reduce (sum) over the output region of a symmetric buffer.
void all_reduce_pull(int64_t comm, int64_t symm, std::string dtype, bool acc_f32, int64_t offset, int64_t nbytes,
                     int64_t grid, int64_t block, int64_t unroll) {
  check(msharp_allreduce_pull(handle(comm), handle(symm), dtype_code(dtype), acc_f32 ? 1 : 0,
                              static_cast<size_t>(offset), static_cast<size_t>(nbytes), static_cast<int>(grid),
                              static_cast<int>(block), static_cast<int>(unroll), current_stream()),
        "msharp::all_reduce_pull");
}

void all_reduce_sw_f32(int64_t comm, int64_t symm, int64_t offset, int64_t nbytes, const c10::optional<at::Tensor>& in_scales,
                       double out_scale, int64_t grid, int64_t block) {
  uint64_t scales = 0;
  if (in_scales.has_value()) {
    TORCH_CHECK(in_scales->is_cuda() == have_device() && in_scales->scalar_type() == at::kFloat && in_scales->is_contiguous(),
                "in_scales must be a contiguous float32 CUDA tensor");
    scales = reinterpret_cast<uint64_t>(in_scales->data_ptr());
  }
  check(msharp_allreduce_sw_f32(handle(comm), handle(symm), static_cast<size_t>(offset), static_cast<size_t>(nbytes), scales,
                                static_cast<float>(1.0 / out_scale), static_cast<int>(grid), static_cast<int>(block),
                                current_stream()),
        "msharp::all_reduce_sw_f32");
}

void all_reduce_bulk_push(int64_t comm, int64_t symm, std::string dtype, int64_t offset, int64_t nbytes, int64_t grid) {
  check(msharp_allreduce_bulk_push(handle(comm), handle(symm), dtype_code(dtype), static_cast<size_t>(offset),
                                   static_cast<size_t>(nbytes), static_cast<int>(grid), current_stream()),
        "msharp::all_reduce_bulk_push");
}

// Fused block-scaled FP8 GEMM + all-reduce into the symmetric BF16 buffer `out_symm`.
void gemm_allreduce(int64_t comm, int64_t out_symm, const at::Tensor& a, const at::Tensor& a_scales, const at::Tensor& w,
                    const at::Tensor& w_scales, int64_t reducer_ctas) {
  const bool on_device = have_device();
  TORCH_CHECK(a.is_cuda() == on_device && w.is_cuda() == on_device && a_scales.is_cuda() == on_device &&
                  w_scales.is_cuda() == on_device,
              "operands must be CUDA tensors");
  TORCH_CHECK(a.dim() == 2 && w.dim() == 2 && a.size(1) == w.size(1), "A is [M, K], W is [N, K]");
  TORCH_CHECK(a.is_contiguous() && w.is_contiguous() && a_scales.is_contiguous() && w_scales.is_contiguous(),
              "operands must be contiguous");
  TORCH_CHECK(a.element_size() == 1 && w.element_size() == 1, "A and W must be FP8 E4M3 (one byte per element)");
  TORCH_CHECK(a_scales.scalar_type() == at::kFloat && w_scales.scalar_type() == at::kFloat, "scales must be float32");
  const int64_t m = a.size(0), k = a.size(1), n = w.size(0);
  TORCH_CHECK(a_scales.numel() == m * (k / 128) && w_scales.numel() == (n / 128) * (k / 128), "scale tensors have the wrong size");
  check(msharp_gemm_allreduce(handle(comm), handle(out_symm), reinterpret_cast<uint64_t>(a.data_ptr()),
                              reinterpret_cast<uint64_t>(a_scales.data_ptr()), reinterpret_cast<uint64_t>(w.data_ptr()),
                              reinterpret_cast<uint64_t>(w_scales.data_ptr()), static_cast<int>(m), static_cast<int>(n),
                              static_cast<int>(k), static_cast<int>(reducer_ctas), current_stream()),
        "msharp::gemm_allreduce");
}

// A tensor that views `nbytes` of device memory at `ptr` (symmetric memory is not owned by
// PyTorch's allocator). The caller keeps the allocation alive.
at::Tensor tensor_from_ptr(int64_t ptr, int64_t nbytes, int64_t device) {
  auto options = have_device() ? at::TensorOptions().dtype(at::kByte).device(at::kCUDA, static_cast<c10::DeviceIndex>(device))
                               : at::TensorOptions().dtype(at::kByte).device(at::kCPU);
  return at::from_blob(reinterpret_cast<void*>(static_cast<intptr_t>(ptr)), {nbytes}, [](void*) {}, options);
}

}  // namespace

TORCH_LIBRARY(msharp, m) {
  m.def("all_reduce_pull(int comm, int symm, str dtype, bool acc_f32, int offset, int nbytes, int grid, int block, int unroll) -> ()",
        &all_reduce_pull);
  m.def("all_reduce_sw_f32(int comm, int symm, int offset, int nbytes, Tensor? in_scales, float out_scale, int grid, int block) -> ()",
        &all_reduce_sw_f32);
  m.def("all_reduce_bulk_push(int comm, int symm, str dtype, int offset, int nbytes, int grid) -> ()", &all_reduce_bulk_push);
  m.def("gemm_allreduce(int comm, int out_symm, Tensor a, Tensor a_scales, Tensor w, Tensor w_scales, int reducer_ctas) -> ()",
        &gemm_allreduce);
  m.def("tensor_from_ptr(int ptr, int nbytes, int device) -> Tensor", &tensor_from_ptr);
}
