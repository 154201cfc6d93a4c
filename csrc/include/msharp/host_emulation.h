// The collectives played through on the CPU, for communicators that run on the host-memory
// driver stand-in (msharp/fake_driver.h). There the "device" pointers of the symmetric buffers are
// ordinary host pointers into memory that all rank processes share, so a rank can read its peers'
// copies and write into them exactly as the kernels do through NVLink. The emulation keeps the
// kernels' structure (opening barrier, rank r reduces the r-th part and writes it into every copy,
// closing barrier) and the arithmetic of the float32 paths (sum in rank order, one final cast), so
// the code around the kernels (launch wrappers, range checks, Python operators, layers, the
// benchmark's iteration loop and reports) runs and is tested among CPU processes. It measures
// nothing and is never chosen on a real device. The reference project has no such mode: its
// collective runs only on an NVL72 rack.
#pragma once

#include <cstddef>
#include <cstdint>

#include "msharp/bootstrap.h"
#include "msharp/oracle.h"
#include "msharp/symm_mem.h"

namespace msharp {

// All-reduce (sum) of `bytes` bytes of `dtype` elements: inputs at `in_offset` of every rank's
// allocation, results at `out_offset` of every rank's allocation (equal offsets = in place).
// Offsets are relative to the start of each rank's slot. `in_scales` (host pointer, one per rank)
// and `out_scale_inv` apply to FP8 as in the sw_f32 kernel; pass nullptr / 1 otherwise. Collective.
void emulate_allreduce(Bootstrap& comm, const SymmetricMemory& mem, Dtype dtype, std::size_t in_offset,
                       std::size_t out_offset, std::size_t bytes, const float* in_scales, float out_scale_inv);

// One rank's block-scaled FP8 product in float32, rounded to BF16 into out_bf16 [m, n] (row-major):
// a [m, k] and w [n, k] E4M3 codes, a_scales [m, k/128], w_scales [n/128, k/128]. Per K block the
// partial product is scaled and added in float32, as the kernel's promotion warps do.
void emulate_gemm_partial_bf16(const uint8_t* a, const float* a_scales, const uint8_t* w, const float* w_scales, int m,
                               int n, int k, uint16_t* out_bf16);

}  // namespace msharp
