// Grouped expert GEMM for sm_100a: MXFP4 weights x fp16 activations on the
// tcgen05 tensor cores, for MLP1 (+bias, clamped SwiGLU) and MLP2 (+bias).
//
// Reference counterparts: grouped_mlp1_bf16_bias_kernel_tiled_optimized_outbf16
// and grouped_mlp2_... (getp-csrc/kernels/moe.hpp:2651, :2923, :3197) with
// swiglu_epilogue_kernel_bf16_mlp_in_bf16 (:1472) between them, fed by weights
// that the reference first expands to bf16 in a staging buffer
// (getp_run.cpp:1019-1086).  Here the packed 4-bit weights are the only copy in
// HBM and are decoded on the way to the tensor cores.
//
// Shape of the computation ("swap-AB"): per work item (expert e, 256 weight
// rows, <= 96 token rows) the kernel forms D[n, tok] = sum_k W[e][n][k] * X[tok][k]
// with the WEIGHT rows on the MMA M axis (two M = 128 tiles) and the tokens on
// the N axis, so a decode-sized token count (tens of rows per expert) fills the
// tensor core and every weight byte is read and decoded once per token tile.
//
// Data flow per 128-element slice of k (one shared-memory stage):
//   TMA  : packed codes  [256 rows x 64 B]  (64-byte swizzle)         -> smem
//          E8M0 scales   [256 rows x 4]     (pre-tiled at load time)   -> smem
//          activations   [<=96 rows x 128 fp16] as two 64-wide K-major
//                        tiles (128-byte swizzle)                      -> smem
//   dequant warps (8): one weight row per thread, cvt.e2m1x2 -> fp16 pairs,
//          times 2^scale, tcgen05.st into a tensor-memory A buffer (64 k wide)
//   MMA thread: tcgen05.mma kind::f16, A from tensor memory, B from smem,
//          fp32 accumulators in tensor memory (double buffered across items)
//   epilogue warps (4): tcgen05.ld, bias, SwiGLU (MLP1) and store.
//
// Tensor memory map (512 columns): [0,384) two accumulator buffers of
// 2 tiles x 96 columns; [384,512) two A buffers of 2 tiles x 32 columns.
// No cluster launch, no multicast: every CTA fetches its own tiles.
#include "moe_internal.cuh"
#include "sm100_ptx.cuh"
#include "swiglu.cuh"

namespace moe {

using namespace sm100;

constexpr int kStages = 5;
constexpr int kWBytes = kPairRows * (kChunkK / 2);        // 16384
constexpr int kXHalfBytes = kTokTile * 128;               // 12288: 96 rows x 64 fp16
constexpr int kXBytes = 2 * kXHalfBytes;                  // 24576
constexpr int kStageBytes = kWBytes + kXBytes + kScaleChunkBytes;  // 41984
constexpr int kXBoxBytes = kXBoxRows * 128;               // 4096
constexpr int kNumBars = 2 * kStages + 8;
constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers etc.*/;

constexpr int kEpiWarps = 4, kDqWarps = 8;
constexpr int kProducerWarp = kEpiWarps + kDqWarps;  // 12
constexpr int kMmaWarp = kProducerWarp + 1;          // 13
constexpr int kThreads = (kMmaWarp + 1) * 32;        // 448

constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kAccCol0 = 0, kAccBufCols = 2 * kTokTile /*192*/, kAccTileCols = kTokTile;
constexpr uint32_t kACol0 = 384, kABufCols = 64, kATileCols = 32;

static_assert(kStageBytes % 1024 == 0, "stages must keep 1024-byte alignment for the swizzled tiles");
static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");

template <int MODE>  // 1 = MLP1 (bias + SwiGLU -> fp16), 2 = MLP2 (bias -> fp32)
__global__ void __launch_bounds__(kThreads, 1)
expert_gemm_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
                   const GemmArgs p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bar_base = smem_base + kStages * kStageBytes;
  volatile uint32_t *abort_flag = reinterpret_cast<volatile uint32_t *>(smem_gen + kStages * kStageBytes + 8 * kNumBars);
  uint32_t *tmem_slot = const_cast<uint32_t *>(abort_flag) + 1;

  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
  auto aready_bar = [&](int a) { return bar_base + 8u * (2 * kStages + a); };
  auto afree_bar = [&](int a) { return bar_base + 8u * (2 * kStages + 2 + a); };
  auto dfull_bar = [&](int d) { return bar_base + 8u * (2 * kStages + 4 + d); };
  auto dempty_bar = [&](int d) { return bar_base + 8u * (2 * kStages + 6 + d); };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int a = 0; a < 2; ++a) {
      mbar_init(aready_bar(a), kDqWarps);
      mbar_init(afree_bar(a), 1);
      mbar_init(dfull_bar(a), 1);
      mbar_init(dempty_bar(a), kEpiWarps);
    }
    *abort_flag = 0u;
    fence_mbar_init();
    fence_proxy_async_smem();
  }
  if (warp == kMmaWarp) {
    tmem_alloc(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish();
  }
  if (warp == kProducerWarp && lane == 0) {
    prefetch_tensormap(&tm_w);
    prefetch_tensormap(&tm_x);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int n_work = *p.n_work;
  const int K = p.K;
  const int nkc = p.n_kchunks;

  if (warp == kProducerWarp) {
    // ------------------------------------------------------------- TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int wi = blockIdx.x; ok && wi < n_work; wi += gridDim.x) {
        const WorkItem w = p.work[wi];
        const int nbox = (w.ntok + kXBoxRows - 1) / kXBoxRows;
        const uint8_t *sc_src = p.scales + (static_cast<size_t>(w.expert) * p.n_pairs + w.pair) * nkc * kScaleChunkBytes;
        for (int kc = 0; kc < nkc; ++kc, ++it) {
          const int s = it % kStages;
          if (!mbar_wait(empty_bar(s), ((it / kStages) & 1u) ^ 1u, abort_flag, p.status, ST_WAIT_EMPTY)) { ok = false; break; }
          const int k0 = kc * kChunkK;
          const int nhalf = (K - k0 > kSubK) ? 2 : 1;
          const uint32_t stage = smem_base + s * kStageBytes;
          mbar_arrive_expect_tx(full_bar(s), kWBytes + kScaleChunkBytes + nhalf * nbox * kXBoxBytes);
          tma_load_3d(stage, &tm_w, k0 / 2, w.pair * kPairRows, w.expert, full_bar(s));
          bulk_load(stage + kWBytes + kXBytes, sc_src + static_cast<size_t>(kc) * kScaleChunkBytes, kScaleChunkBytes, full_bar(s));
          for (int h = 0; h < nhalf; ++h)
            for (int b = 0; b < nbox; ++b)
              tma_load_2d(stage + kWBytes + h * kXHalfBytes + b * kXBoxBytes, &tm_x, k0 + h * kSubK,
                          w.row0 + b * kXBoxRows, full_bar(s));
        }
      }
      if (!ok) {  // give copies in flight time to land before the CTA's shared memory is released
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
      }
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      uint32_t it = 0, item = 0;
      bool ok = true;
      for (int wi = blockIdx.x; ok && wi < n_work; wi += gridDim.x, ++item) {
        const WorkItem w = p.work[wi];
        const int nmma = (w.ntok + 15) & ~15;
        const int ntiles = (w.pair * kPairRows + kTileRows < p.R) ? 2 : 1;
        const uint32_t idesc = idesc_f16_m128(nmma);
        const uint32_t d = item & 1u;
        if (!mbar_wait(dempty_bar(d), ((item >> 1) & 1u) ^ 1u, abort_flag, p.status, ST_WAIT_DEMPTY)) { ok = false; break; }
        tc_fence_after();
        for (int kc = 0; ok && kc < nkc; ++kc, ++it) {
          const int s = it % kStages;
          if (!mbar_wait(full_bar(s), (it / kStages) & 1u, abort_flag, p.status, ST_WAIT_FULL)) { ok = false; break; }
          const uint32_t xbase = smem_base + s * kStageBytes + kWBytes;
          const int krem = K - kc * kChunkK;
          for (int h = 0; h < 2; ++h) {
            if (!mbar_wait(aready_bar(h), it & 1u, abort_flag, p.status, ST_WAIT_AREADY)) { ok = false; break; }
            tc_fence_after();
            const int ksteps = max(0, min(4, (krem - h * kSubK) / 16));
            for (int t = 0; t < ntiles; ++t) {
              const uint32_t d_addr = tmem_base + kAccCol0 + d * kAccBufCols + t * kAccTileCols;
              const uint32_t a_addr = tmem_base + kACol0 + h * kABufCols + t * kATileCols;
              for (int j = 0; j < ksteps; ++j) {
                const uint64_t bdesc = smem_desc_sw128(xbase + h * kXHalfBytes + j * 32);
                mma_f16_ts(d_addr, a_addr + j * 8, bdesc, idesc, (kc | h | j) != 0);
              }
            }
            mma_commit(afree_bar(h));
          }
          if (ok) mma_commit(empty_bar(s));
        }
        if (ok) mma_commit(dfull_bar(d));
      }
    }
  } else if (warp >= kEpiWarps) {
    // ------------------------------------------------------------- dequant warps
    const int dq = warp - kEpiWarps;
    const int tile = dq >> 2, quad = warp & 3;
    const int rb = tile * kTileRows + quad * 32 + lane;  // row inside the 256-row box
    const uint32_t sw = static_cast<uint32_t>((rb >> 1) & 3);
    const uint32_t lane_field = static_cast<uint32_t>(quad * 32) << 16;
    uint32_t it = 0;
    bool ok = true;
    for (int wi = blockIdx.x; ok && wi < n_work; wi += gridDim.x) {
      const WorkItem w = p.work[wi];
      const bool active = tile == 0 || (w.pair * kPairRows + kTileRows < p.R);
      for (int kc = 0; ok && kc < nkc; ++kc, ++it) {
        const int s = it % kStages;
        if (!mbar_wait(full_bar(s), (it / kStages) & 1u, abort_flag, p.status, ST_WAIT_FULL)) { ok = false; break; }
        const uint8_t *stage = smem_gen + s * kStageBytes;
        const uint32_t sc4 = *reinterpret_cast<const uint32_t *>(stage + kWBytes + kXBytes + rb * 4);
        const int krem = K - kc * kChunkK;
        for (int h = 0; h < 2; ++h) {
          if (!mbar_wait(afree_bar(h), (it & 1u) ^ 1u, abort_flag, p.status, ST_WAIT_AFREE)) { ok = false; break; }
          tc_fence_after();
          const int nblk = max(0, min(2, (krem - h * kSubK) / 32));
          if (active) {
            for (int c = 0; c < nblk; ++c) {
              const uint32_t c16 = 2u * h + c;
              const uint4 codes = *reinterpret_cast<const uint4 *>(stage + rb * 64 + ((c16 ^ sw) << 4));
              uint32_t regs[16];
              dequant_block32(codes, e8m0_to_f16x2((sc4 >> (8 * c16)) & 0xffu), regs);
              tmem_st16(tmem_base + lane_field + kACol0 + h * kABufCols + tile * kATileCols + c * 16, regs);
            }
            tmem_wait_st();
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(aready_bar(h));
        }
      }
    }
  } else {
    // ------------------------------------------------------------- epilogue warps
    const int quad = warp;  // warps 0..3 <-> TMEM lanes 32*warp..
    const uint32_t lane_field = static_cast<uint32_t>(quad * 32) << 16;
    uint32_t item = 0;
    bool ok = true;
    for (int wi = blockIdx.x; ok && wi < n_work; wi += gridDim.x, ++item) {
      const WorkItem w = p.work[wi];
      const int nmma = (w.ntok + 15) & ~15;
      const int ntiles = (w.pair * kPairRows + kTileRows < p.R) ? 2 : 1;
      const uint32_t d = item & 1u;
      if (!mbar_wait(dfull_bar(d), (item >> 1) & 1u, abort_flag, p.status, ST_WAIT_DFULL)) { ok = false; break; }
      tc_fence_after();
      for (int t = 0; t < ntiles; ++t) {
        const int n_loc = w.pair * kPairRows + t * kTileRows + quad * 32 + lane;
        const bool row_ok = n_loc < p.R;
        float bias = 0.f;
        if (row_ok && p.add_bias) bias = __bfloat162float(p.bias[static_cast<size_t>(w.expert) * p.R + n_loc]);
        for (int c0 = 0; c0 < nmma; c0 += 16) {
          uint32_t v[16];
          tmem_ld16(tmem_base + lane_field + kAccCol0 + d * kAccBufCols + t * kAccTileCols + c0, v);
          tmem_wait_ld();
          if (MODE == 1) {
            const int odd = lane & 1;
#pragma unroll
            for (int i = 0; i < 16; i += 2) {
              const float f0 = __uint_as_float(v[i]) + bias, f1 = __uint_as_float(v[i + 1]) + bias;
              const float send = odd ? f0 : f1;
              const float recv = __shfl_xor_sync(0xffffffffu, send, 1);
              const float gate = odd ? recv : f0;
              const float up = odd ? f1 : recv;
              const int tok = c0 + i + odd;
              const float hv = swiglu_clamped(gate, up, p.limit, p.alpha);
              if (row_ok && tok < w.ntok)
                p.h_out[static_cast<size_t>(w.row0 + tok) * p.ld_out + (n_loc >> 1)] = __float2half_rn(hv);
            }
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const int tok = c0 + i;
              if (row_ok && tok < w.ntok)
                p.y_out[static_cast<size_t>(w.row0 + tok) * p.ld_out + n_loc] = __uint_as_float(v[i]) + bias;
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(dempty_bar(d));
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

cudaError_t expert_gemm_init() {
  cudaError_t e = cudaFuncSetAttribute(expert_gemm_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
  if (e != cudaSuccess) return e;
  return cudaFuncSetAttribute(expert_gemm_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
}

void launch_expert_gemm_mlp1(const CUtensorMap &tm_w, const CUtensorMap &tm_x, const GemmArgs &a, int grid,
                             cudaStream_t s) {
  expert_gemm_kernel<1><<<grid, kThreads, kSmemBytes, s>>>(tm_w, tm_x, a);
}
void launch_expert_gemm_mlp2(const CUtensorMap &tm_w, const CUtensorMap &tm_x, const GemmArgs &a, int grid,
                             cudaStream_t s) {
  expert_gemm_kernel<2><<<grid, kThreads, kSmemBytes, s>>>(tm_w, tm_x, a);
}

}  // namespace moe
