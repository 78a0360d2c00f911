// Host-side helpers shared by all translation units of the library: error reporting,
// launch counting, tensor-map construction, device properties, and the status block that
// kernels report into (see status.cuh).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include "status.cuh"

enum : int {
  NSA_OK = 0,
  NSA_ERR_CUDA = 1,        // a CUDA runtime / driver call failed; see nsa_last_error()
  NSA_ERR_ALIGNMENT = 2,   // pointer or leading dimension not aligned as the kernel needs
  NSA_ERR_SHAPE = 3,       // shape outside what the kernel supports
  NSA_ERR_DRIVER_API = 4,  // cuTensorMapEncodeTiled entry point not available
  NSA_ERR_LIMIT = 5,       // a fixed-capacity resource (static scratch) is too small
};

namespace nsa {
int fail(int code, const char* msg);
int fail_cuda(cudaError_t e, const char* where);
void count_launch(int n = 1);
KernelStatus* status_ptr();
int sm_count();
// 2-D bf16 tensor map with 128-byte swizzle.  `inner` is the contiguous dimension;
// `ld` is the row pitch in elements; box_inner * 2 bytes must be 128.
int make_tmap_2d_bf16(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t ld,
                      uint32_t box_inner, uint32_t box_outer);
// 2-D fp32 tensor map with 128-byte swizzle; box_inner * 4 bytes must be 128.
int make_tmap_2d_f32(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t ld,
                     uint32_t box_inner, uint32_t box_outer);
// General tiled bf16 map (rank <= 5) with explicit byte strides for dims 1..rank-1.
int make_tmap_bf16(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                   const uint64_t* strides_bytes, const uint32_t* box, int swizzle128);
}  // namespace nsa
