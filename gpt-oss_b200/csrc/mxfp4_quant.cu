// fp32 -> MXFP4 on the GPU, and loading a layer from an fp32 checkpoint.
//
// Reference: quantize_pack_mxfp4_block32_kernel with its encode helpers
// (getp-csrc/memory/mxfp4.hpp:113-217) and the host loop that feeds it,
// streaming_quantize_copy_mxfp4_cpu_to_gpu (getp_run.cpp:1104-1245), called for
// w_mlp1 / w_mlp2 of the fp32 checkpoint (layout: run.cpp:206-247) by
// copy_weights_to_gpu_120b (getp_run.cpp:1480-1718).  Results are bit-identical
// to the reference's: same block maximum, same exponent rule, same first-best
// scan of the 16 table entries.
//
// Four lanes per 32-element block (the reference gives it a "logical warp" of
// 32), shuffles instead of its shared-memory staging, thresholds instead of its
// 16-way scan, a multiplication by 2^-exp instead of its division; a grid-stride
// loop over the blocks of the call.  HBM-bound: 4 bytes read and 17/32 byte written per
// element.
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "moe_internal.cuh"

namespace moe {

// Code of x (already divided by the block scale).  The reference scans the 16 table entries in order and
// keeps the first at the smallest distance (mxfp4.hpp:121-131).  That is: the nearest magnitude of
// {0, .5, 1, 1.5, 2, 3, 4, 6}, the smaller one at an exact midpoint (the distances there are exact in fp32,
// so thresholds decide exactly as the scan does), the sign bit only with a non-zero magnitude (+0 precedes
// -0 in the table), and code 0 for NaN and for infinities (no distance is smaller than the first, infinite one).
__device__ __forceinline__ uint32_t e2m1_first_nearest(float x) {
  const float a = fabsf(x);
  uint32_t idx = (a > 0.25f) + (a > 0.75f) + (a > 1.25f) + (a > 1.75f) + (a > 2.5f) + (a > 3.5f) + (a > 5.0f);
  if (!(a < __int_as_float(0x7f800000))) idx = 0;
  return (x < 0.f && idx != 0) ? (idx | 8u) : idx;
}

// Four lanes per 32-element block, eight consecutive elements per lane (two 16-byte loads in flight).
__global__ void __launch_bounds__(256)
mxfp4_quantize_kernel(const float *__restrict__ src, size_t n, uint8_t *__restrict__ codes,
                      uint8_t *__restrict__ scales, size_t n_blocks) {
  const int lane = threadIdx.x & 31;
  const size_t total = n_blocks * 4;  // 8-element groups, the last block padded with zeros
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  const bool vec_ok = (reinterpret_cast<uintptr_t>(src) & 15u) == 0;
  for (size_t base = static_cast<size_t>(blockIdx.x) * blockDim.x + (threadIdx.x & ~31); base < total; base += stride) {
    const size_t q = base + lane, g0 = q * 8;
    float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};  // elements past the end count as 0 (mxfp4.hpp:170-174)
    if (q < total) {
      if (vec_ok && g0 + 7 < n) {
        const float4 f0 = __ldg(reinterpret_cast<const float4 *>(src + g0));
        const float4 f1 = __ldg(reinterpret_cast<const float4 *>(src + g0) + 1);
        v[0] = f0.x; v[1] = f0.y; v[2] = f0.z; v[3] = f0.w;
        v[4] = f1.x; v[5] = f1.y; v[6] = f1.z; v[7] = f1.w;
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (g0 + j < n) v[j] = src[g0 + j];
      }
    }
    // largest |v| of the block; a NaN never wins a '>' in the reference's scan, fmaxf drops it the same way
    float maxabs = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) maxabs = fmaxf(maxabs, fabsf(v[j]));
    maxabs = fmaxf(maxabs, __shfl_xor_sync(0xffffffffu, maxabs, 1));
    maxabs = fmaxf(maxabs, __shfl_xor_sync(0xffffffffu, maxabs, 2));
    // exp = ilogb(maxabs) - 2 (the largest power of two among the E2M1 magnitudes is 2^2), 0 for a zero block
    const uint32_t mbits = __float_as_uint(maxabs);
    int exp_scale = 0;
    float x[8];
    if (mbits >= 0x01800000u && mbits < 0x7f800000u) {
      // maximum of at least 2^-124: the exponent field is ilogb, and 2^-exp is a normal float, so multiplying
      // by it rounds exactly as the reference's division by 2^exp does
      exp_scale = static_cast<int>(mbits >> 23) - 127 - 2;
      const float inv = __uint_as_float(static_cast<uint32_t>(127 - exp_scale) << 23);
#pragma unroll
      for (int j = 0; j < 8; ++j) x[j] = v[j] * inv;
    } else {
      if (maxabs > 0.f) {  // tiny or infinite maximum: the reference's own library calls
        int e;
        frexpf(maxabs, &e);
        exp_scale = (e - 1) - 2;
      }
      const float X = ldexpf(1.0f, exp_scale);
#pragma unroll
      for (int j = 0; j < 8; ++j) x[j] = v[j] / X;
    }
    uint32_t word = 0;  // low nibble = even element
#pragma unroll
    for (int j = 0; j < 8; ++j) word |= e2m1_first_nearest(x[j]) << (4 * j);
    if (q < total) {
      const size_t b = q >> 2;
      reinterpret_cast<uint32_t *>(codes + b * 16)[q & 3] = word;
      if ((q & 3) == 0) scales[b] = static_cast<uint8_t>(min(max(exp_scale + 127, 0), 255));
    }
  }
}

}  // namespace moe

using namespace moe;

namespace {

int qfail(moe_ctx *c, int code, const char *fmt, ...) {
  if (c) {
    char buf[400];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    c->err = buf;
  }
  return code;
}

uint16_t bf16_rn(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return static_cast<uint16_t>((u >> 16) | 0x40u);
  u += 0x7fffu + ((u >> 16) & 1u);
  return static_cast<uint16_t>(u >> 16);
}

void launch_quantize(const float *src, size_t n, uint8_t *codes, uint8_t *scales, cudaStream_t s) {
  const size_t n_blocks = (n + 31) / 32;
  const size_t want = (n_blocks * 4 + 255) / 256;  // four lanes per block, 256 threads per CTA
  const unsigned grid = static_cast<unsigned>(std::min<size_t>(want, 148 * 16));
  mxfp4_quantize_kernel<<<std::max(grid, 1u), 256, 0, s>>>(src, n, codes, scales, n_blocks);
}

// One fp32 tensor in host memory -> codes and scales in host memory, through the GPU in chunks with the copy
// of the next chunk overlapping the kernel on this one (the reference's double buffering, without its
// per-chunk host synchronisation).
int quantize_host_tensor(moe_ctx *c, const float *src, size_t n, std::vector<uint8_t> &codes, std::vector<uint8_t> &scales) {
  const size_t n_blocks = (n + 31) / 32;
  codes.resize(n_blocks * 16);
  scales.resize(n_blocks);
  const size_t chunk_blocks = std::min<size_t>(n_blocks, (64u << 20) / 128);  // 64 MiB of fp32 per chunk
  float *d_src[2] = {nullptr, nullptr};
  uint8_t *d_codes = nullptr, *d_scales = nullptr;
  cudaStream_t st[2] = {nullptr, nullptr};
  int rc = MOE_OK;
  auto cleanup = [&]() {
    for (int i = 0; i < 2; ++i) {
      if (st[i]) { cudaStreamSynchronize(st[i]); cudaStreamDestroy(st[i]); }
      cudaFree(d_src[i]);
    }
    cudaFree(d_codes);
    cudaFree(d_scales);
  };
  bool ok = cudaMalloc(reinterpret_cast<void **>(&d_codes), n_blocks * 16) == cudaSuccess &&
            cudaMalloc(reinterpret_cast<void **>(&d_scales), n_blocks) == cudaSuccess;
  for (int i = 0; ok && i < 2; ++i)
    ok = cudaMalloc(reinterpret_cast<void **>(&d_src[i]), chunk_blocks * 128) == cudaSuccess &&
         cudaStreamCreateWithFlags(&st[i], cudaStreamNonBlocking) == cudaSuccess;
  if (!ok) {
    cleanup();
    return qfail(c, MOE_ERR_CUDA, "quantise: device staging allocation failed: %s", cudaGetErrorString(cudaGetLastError()));
  }
  int ping = 0;
  for (size_t b0 = 0; b0 < n_blocks; b0 += chunk_blocks, ping ^= 1) {
    const size_t nb = std::min(chunk_blocks, n_blocks - b0);
    const size_t e0 = b0 * 32, ne = std::min(nb * 32, n - e0);
    // stream ping: copy in, quantise; the other stream is still busy with the previous chunk
    if (cudaMemcpyAsync(d_src[ping], src + e0, ne * sizeof(float), cudaMemcpyHostToDevice, st[ping]) != cudaSuccess) {
      rc = qfail(c, MOE_ERR_CUDA, "quantise: host-to-device copy failed");
      break;
    }
    launch_quantize(d_src[ping], ne, d_codes + b0 * 16, d_scales + b0, st[ping]);
  }
  for (int i = 0; i < 2; ++i)
    if (cudaStreamSynchronize(st[i]) != cudaSuccess && rc == MOE_OK)
      rc = qfail(c, MOE_ERR_CUDA, "quantise: %s", cudaGetErrorString(cudaGetLastError()));
  if (rc == MOE_OK &&
      (cudaMemcpy(codes.data(), d_codes, codes.size(), cudaMemcpyDeviceToHost) != cudaSuccess ||
       cudaMemcpy(scales.data(), d_scales, scales.size(), cudaMemcpyDeviceToHost) != cudaSuccess))
    rc = qfail(c, MOE_ERR_CUDA, "quantise: device-to-host copy failed");
  cleanup();
  return rc;
}

}  // namespace

extern "C" {

int moe_quantize_mxfp4(const float *src_dev, size_t n_elems, uint8_t *codes_dev, uint8_t *scales_dev, void *stream) {
  if (!src_dev || !codes_dev || !scales_dev) return MOE_ERR_INVALID;
  if (reinterpret_cast<uintptr_t>(codes_dev) & 3u) return MOE_ERR_INVALID;  // codes are written as 32-bit words
  if (n_elems == 0) return MOE_OK;
  launch_quantize(src_dev, n_elems, codes_dev, scales_dev, static_cast<cudaStream_t>(stream));
  return cudaGetLastError() == cudaSuccess ? MOE_OK : MOE_ERR_CUDA;
}

int moe_load_layer_f32(moe_handle c, int layer, const float *w1, const float *b1, const float *w2, const float *b2,
                       const float *router_w, const float *router_b) {
  if (!c) return MOE_ERR_INVALID;
  if (!w1 || !b1 || !w2 || !b2 || !router_w || !router_b) return qfail(c, MOE_ERR_INVALID, "moe_load_layer_f32: null tensor");
  if (cudaSetDevice(c->cfg.device) != cudaSuccess) return qfail(c, MOE_ERR_CUDA, "moe_load_layer_f32: cudaSetDevice failed");
  const size_t E = c->E, H = c->H, D = c->D;
  // rows of H (MLP1) and of D (MLP2) elements are whole numbers of 32-element blocks, so quantising the flat
  // tensor, as the reference does, gives per-row blocks
  std::vector<uint8_t> c1, s1, c2, s2;
  int rc = quantize_host_tensor(c, w1, E * 2 * D * H, c1, s1);
  if (rc == MOE_OK) rc = quantize_host_tensor(c, w2, E * H * D, c2, s2);
  if (rc != MOE_OK) return rc;
  std::vector<uint16_t> bb1(E * 2 * D), bb2(E * H);   // biases are kept in bf16 (convert_float_array_to_bfloat16, getp_run.cpp:1638-1658)
  for (size_t i = 0; i < bb1.size(); ++i) bb1[i] = bf16_rn(b1[i]);
  for (size_t i = 0; i < bb2.size(); ++i) bb2[i] = bf16_rn(b2[i]);
  return moe_load_layer(c, layer, c1.data(), s1.data(), bb1.data(), c2.data(), s2.data(), bb2.data(), router_w, router_b);
}

}  // extern "C"
