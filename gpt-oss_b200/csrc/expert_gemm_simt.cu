// Validation path of the two expert GEMMs on plain CUDA cores (one warp per
// output element, fp32 accumulation, fp16 operands decoded with cvt.e2m1x2).
// It shares nothing with the tensor-core kernel but the packed weights, and
// exists to tell a weight-layout error from a tcgen05 pipeline error on the
// device; moe_forward runs it only when MOE_FWD_SIMT_GEMM is passed.
#include "moe_internal.cuh"
#include "sm100_ptx.cuh"
#include "swiglu.cuh"

namespace moe {

__device__ __forceinline__ int expert_of_row(const int *offsets, int E, int r) {
  int lo = 0, hi = E;  // offsets[lo] <= r < offsets[hi]
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (offsets[mid] <= r) lo = mid; else hi = mid;
  }
  return lo;
}

// dot of one weight row (packed codes inside the 16 KB weight tiles: `codes` points at the row's 64 bytes in the
// first tile of its row block, the next 128 k follow one tile further; raw row-major scales) with an fp16 row
__device__ __forceinline__ float warp_dot_mxfp4(const uint8_t *codes, const uint8_t *scales, const __half *x,
                                                int K, int lane) {
  float acc = 0.f;
  for (int b = lane; b < K / 32; b += 32) {
    const uint4 c = *reinterpret_cast<const uint4 *>(codes + static_cast<size_t>(b >> 2) * kWTileStride + (b & 3) * 16);
    uint32_t w[16];
    sm100::dequant_block32(c, sm100::e8m0_to_f16x2(scales[b]), w);
    const uint4 *xp = reinterpret_cast<const uint4 *>(x + b * 32);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const uint4 xv = xp[q];
      const uint32_t xs[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 wf = __half22float2(*reinterpret_cast<const __half2 *>(&w[q * 4 + j]));
        const float2 xf = __half22float2(*reinterpret_cast<const __half2 *>(&xs[j]));
        acc = fmaf(wf.x, xf.x, acc);
        acc = fmaf(wf.y, xf.y, acc);
      }
    }
  }
#pragma unroll
  for (int off = 16; off; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  return acc;
}

// the 64 code bytes of row `row` of expert e's [R x K] matrix in the first tile of the row's block
__device__ __forceinline__ const uint8_t *tile_row(const uint8_t *w_tiles, int e, int row, int R, int K) {
  const int n_nt = (R + kTileN - 1) / kTileN, n_kc = (K + kChunkK - 1) / kChunkK;
  return w_tiles + (static_cast<size_t>(e) * n_nt + row / kTileN) * n_kc * kWTileStride + (row % kTileN) * (kChunkK / 2);
}

__global__ void __launch_bounds__(256)
simt_mlp1_kernel(const uint8_t *__restrict__ w_tiles, const uint8_t *__restrict__ scales,
                 const __nv_bfloat16 *__restrict__ bias, const __half *__restrict__ x,
                 const int *__restrict__ offsets, int E, int H, int R1, __half *__restrict__ h_out, int ld_h,
                 float limit, float alpha) {
  const int r = blockIdx.x;
  if (r >= offsets[E]) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int j = blockIdx.y * 8 + warp;
  const int Dl = R1 / 2;
  if (j >= Dl) return;
  const int e = expert_of_row(offsets, E, r);
  const size_t row_g = static_cast<size_t>(e) * R1 + 2 * j;
  const __half *xr = x + static_cast<size_t>(r) * H;
  float g = warp_dot_mxfp4(tile_row(w_tiles, e, 2 * j, R1, H), scales + row_g * (H / 32), xr, H, lane);
  float u = warp_dot_mxfp4(tile_row(w_tiles, e, 2 * j + 1, R1, H), scales + (row_g + 1) * (H / 32), xr, H, lane);
  if (lane == 0) {
    g += __bfloat162float(bias[row_g]);
    u += __bfloat162float(bias[row_g + 1]);
    h_out[static_cast<size_t>(r) * ld_h + j] = __float2half_rn(swiglu_clamped(g, u, limit, alpha));
  }
}

__global__ void __launch_bounds__(256)
simt_mlp2_kernel(const uint8_t *__restrict__ w_tiles, const uint8_t *__restrict__ scales,
                 const __nv_bfloat16 *__restrict__ bias, int add_bias, const __half *__restrict__ h,
                 const int *__restrict__ offsets, int E, int Dl, int H, __half *__restrict__ y_out) {
  const int r = blockIdx.x;
  if (r >= offsets[E]) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int i = blockIdx.y * 8 + warp;
  if (i >= H) return;
  const int e = expert_of_row(offsets, E, r);
  const size_t row = static_cast<size_t>(e) * H + i;
  float v = warp_dot_mxfp4(tile_row(w_tiles, e, i, H, Dl), scales + row * (Dl / 32), h + static_cast<size_t>(r) * Dl, Dl, lane);
  if (lane == 0) {
    if (add_bias) v += __bfloat162float(bias[row]);
    y_out[static_cast<size_t>(r) * H + i] = __float2half_rn(v);
  }
}

void launch_simt_mlp1(const uint8_t *w_tiles, const uint8_t *scales_raw, const __nv_bfloat16 *bias,
                      const __half *x, const int *offsets, int E, int H, int R1, __half *h_out, int ld_h,
                      float limit, float alpha, int n_rows, cudaStream_t s) {
  dim3 grid(n_rows, (R1 / 2 + 7) / 8);
  simt_mlp1_kernel<<<grid, 256, 0, s>>>(w_tiles, scales_raw, bias, x, offsets, E, H, R1, h_out, ld_h, limit, alpha);
}

void launch_simt_mlp2(const uint8_t *w_tiles, const uint8_t *scales_raw, const __nv_bfloat16 *bias,
                      int add_bias, const __half *h, const int *offsets, int E, int Dl, int H, __half *y_out,
                      int n_rows, cudaStream_t s) {
  dim3 grid(n_rows, (H + 7) / 8);
  simt_mlp2_kernel<<<grid, 256, 0, s>>>(w_tiles, scales_raw, bias, add_bias, h, offsets, E, Dl, H, y_out);
}

}  // namespace moe
