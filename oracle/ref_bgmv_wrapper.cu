// Test infrastructure: C entry points around the REFERENCE's own BGMV kernels, compiled from the reference tree where
// it lies (the include path is given by oracle/Makefile; no reference source is copied).  Used only by the GPU
// cross-check test and the golden-vector generator, to pin the CPU oracle against what the reference computes.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdint>

#include "bgmv/bgmv_impl.cuh"  // slora/csrc/bgmv/bgmv_impl.cuh:211-241 (bgmv_kernel launcher)

#define REF_CASE(FI, FO)                                                                                   \
  if (h_in == FI && h_out == FO) {                                                                         \
    bgmv_kernel<FI, FO>(static_cast<nv_half*>(y), static_cast<const nv_half*>(x),                          \
                        static_cast<const nv_half*>(w), start, ranks4, loc, ids, qkvo, batch,              \
                        static_cast<const nv_half*>(scales));                                              \
    return static_cast<int>(cudaGetLastError());                                                           \
  }

// fp16 only; launches on the legacy default stream exactly as the reference does.  Returns -1 for a shape that was
// not instantiated here, else the cudaGetLastError() code.
extern "C" int ref_dispatch_bgmv(void* y, const void* x, const void* w, const int64_t* start, const int64_t* ranks4,
                                 const int64_t* loc, const int64_t* ids, int64_t qkvo, int64_t batch, int h_in,
                                 int h_out, const void* scales) {
  REF_CASE(4096, 8)
  REF_CASE(8, 4096)
  REF_CASE(4096, 16)
  REF_CASE(16, 4096)
  REF_CASE(4096, 64)
  REF_CASE(64, 4096)
  REF_CASE(1024, 16)
  REF_CASE(16, 1024)
  REF_CASE(5120, 64)
  REF_CASE(64, 5120)
  return -1;
}
