/*
 * TEST INFRASTRUCTURE ONLY.
 *
 * Not a translation unit of its own: oracle/Makefile pipes the first part of
 * the reference's getp-csrc/memory/mxfp4.hpp (up to, not including, its bf16
 * dequantisation kernels; read in place from the reference checkout) into the
 * compiler with hipstub/ on the include path and appends this file.  The code
 * below then runs the reference's unmodified
 * quantize_pack_mxfp4_block32_kernel<32> (mxfp4.hpp:139-217) on 32 host
 * threads that play the lanes of one block: threadIdx/blockIdx are set per
 * thread and __syncthreads() is a barrier.  One block of 32 threads is one
 * "logical warp" of the kernel, i.e. one 32-element MXFP4 block; the
 * reference launches 256 threads, which changes nothing per logical warp.
 */
#include <pthread.h>

#include <vector>

thread_local ref_dim3 threadIdx, blockIdx;
ref_dim3 blockDim, gridDim;
/* the kernel's dynamic shared memory: 32 floats + 32 bytes + 1 int */
unsigned char mxfp4_smem[32 * sizeof(float) + 32 + sizeof(int) + 64];

namespace {
pthread_barrier_t g_block_barrier;

struct LaneArgs {
  int lane;
  const float *src;
  size_t n_elems, n_blocks;
  uint8_t *packed, *scales;
};

void *lane_main(void *p) {
  const LaneArgs *a = static_cast<const LaneArgs *>(p);
  threadIdx.x = static_cast<unsigned>(a->lane);
  for (size_t b = 0; b < a->n_blocks; ++b) {
    blockIdx.x = static_cast<unsigned>(b);
    quantize_pack_mxfp4_block32_kernel<32>(a->src, a->n_blocks, 0, a->packed, a->scales, a->n_elems);
    pthread_barrier_wait(&g_block_barrier); /* next block reuses the shared arrays */
  }
  return nullptr;
}
} // namespace

void __syncthreads() { pthread_barrier_wait(&g_block_barrier); }

extern "C" {

/* packed: ceil(n/32)*16 bytes, scales: ceil(n/32) bytes. */
int ref_mxfp4_quantize(const float *src, size_t n_elems, uint8_t *packed, uint8_t *scales) {
  init_mxfp4_lut_on_device();
  blockDim.x = 32;
  const size_t n_blocks = (n_elems + 31) / 32;
  gridDim.x = static_cast<unsigned>(n_blocks);
  if (pthread_barrier_init(&g_block_barrier, nullptr, 32)) return -1;
  std::vector<LaneArgs> args(32);
  std::vector<pthread_t> th(32);
  for (int l = 0; l < 32; ++l) {
    args[l] = LaneArgs{l, src, n_elems, n_blocks, packed, scales};
    if (pthread_create(&th[l], nullptr, lane_main, &args[l])) return -2;
  }
  for (int l = 0; l < 32; ++l) pthread_join(th[l], nullptr);
  pthread_barrier_destroy(&g_block_barrier);
  return 0;
}

/* The reference's per-element decode (mxfp4.hpp:41-57), for the round trip. */
void ref_mxfp4_dequantize(const uint8_t *packed, const uint8_t *scales, size_t n_elems, float *out) {
  for (size_t i = 0; i < n_elems; ++i) out[i] = dequantize_mxfp4_block32(packed, scales, i);
}

} // extern "C"
