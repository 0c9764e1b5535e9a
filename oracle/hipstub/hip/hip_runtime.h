/*
 * TEST INFRASTRUCTURE ONLY.  A stand-in for <hip/hip_runtime.h> that lets the
 * CPU compiler read the reference's getp-csrc/memory/mxfp4.hpp in place, so
 * that its own quantiser source (encode helpers and the body of
 * quantize_pack_mxfp4_block32_kernel) runs on host threads as the pin of the
 * restatement in moe_oracle.c.  Nothing here comes from HIP: the qualifiers
 * become empty, the built-in index variables become thread-local structs that
 * the driver (ref_mxfp4_driver.inc.cpp) sets, and __syncthreads() is a pthread
 * barrier over the threads that play one block.
 */
#pragma once
#include <cmath>
#include <cstddef>
#include <cstdint>
#include <cstring>

#define __device__
#define __global__
#define __host__
#define __constant__
#define __shared__
#define __forceinline__ inline
#define __align__(n)
#define HIP_SYMBOL(x) (x)
#define HIP_CHECK(expr) ((void)(expr))

struct ref_dim3 {
  unsigned x = 0, y = 0, z = 0;
};
extern thread_local ref_dim3 threadIdx, blockIdx;
extern ref_dim3 blockDim, gridDim;
void __syncthreads();

inline int hipMemcpyToSymbol(void *dst, const void *src, size_t n) {
  memcpy(dst, src, n);
  return 0;
}
inline float __uint_as_float(uint32_t u) {
  float f;
  memcpy(&f, &u, 4);
  return f;
}
