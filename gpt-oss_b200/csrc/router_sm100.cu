// Router logits on the tcgen05 tensor cores: logits[t, e] = sum_k t[t, k] * Wr[e, k], fp32.
// Reference: matmul + bias of run.cpp:660-669 (double accumulation of float products); the
// reference GPU path rounds the logits to bf16 (getp_run.cpp:2612-2620), which this path
// deliberately does not.
//
// The fp32 router weight is split at load time into three bf16 planes (hi + mid + lo == w
// exactly, 8+8+8 significand bits), so every plane times a bf16 activation is an exact fp32
// product and only the additions round.  One CTA owns 128 tokens x up to 128 experts x one
// slice of k (split-k keeps the SMs busy: 1856 tokens are only 15 token tiles): a producer warp
// streams 64-wide k chunks of the activations and of the three planes into a three-stage
// shared-memory ring with TMA (128-byte swizzle), one thread issues twelve
// tcgen05.mma kind::f16 (bf16 x bf16, M128 x N x K16) per chunk into one fp32 accumulator in
// tensor memory.  What happens to the accumulator depends on the launch:
//  * fused (up to 128 experts, the usual case): the CTAs of one token tile, one per k slice, form
//    a thread-block cluster.  Each parks its accumulator in its own shared memory; after a cluster
//    barrier CTA r adds, for its share of the 128 tokens, the slices of all CTAs in slice order in
//    double precision (distributed shared memory loads), adds the bias, and runs the top-k
//    selection and softmax for those tokens: logits, selection, weights and expert histogram leave
//    the kernel, no partial sums touch HBM.
//  * partial sums: four warps write the accumulator out as this slice's partial sums and
//    topk_softmax_kernel adds the slices, again in slice order in double precision.
// Either way the result does not depend on scheduling.  Every mbarrier wait is bounded; the cluster
// barriers are reached by every thread on every path.
#include <cooperative_groups.h>

#include "moe_internal.cuh"
#include "route_select.cuh"
#include "sm100_ptx.cuh"

namespace moe {
using namespace sm100;
namespace cg = cooperative_groups;

namespace {
constexpr int kRtTok = 128;                      // token rows per CTA = M of the instruction
constexpr int kRtExp = 128;                      // experts per CTA (N of the instruction, at most)
constexpr int kRtK = 64;                         // bf16 per k chunk: one 128-byte swizzled row
constexpr int kRtStages = 3;
constexpr int kRtTile = kRtTok * kRtK * 2;       // 16384 bytes: activations, and one weight plane
constexpr int kRtStage = 4 * kRtTile;            // activations + three planes
constexpr int kRtBarBytes = 64;
constexpr int kRtSmem = kRtStages * kRtStage + kRtBarBytes + 1024;  // + slack to align the ring to 1024
constexpr int kRtThreads = 512;                  // warps 0-3 read the accumulator, 4 loads, 5 issues; all 16 select (fused form)
constexpr int kRtTmemCols = 128;
constexpr int kRtRedPitch = (kRtExp + 4) * 4;    // bytes per parked accumulator row: 16-byte stores of a warp spread over all banks
static_assert(kRtTok * kRtRedPitch <= kRtStages * kRtStage, "the parked accumulator reuses the ring");

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// kind::f16 with bf16 operands, fp32 accumulator, both operands K-major, M = 128.
__host__ __device__ constexpr uint32_t idesc_bf16_m128(uint32_t n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((128u >> 4) << 24);
}

__device__ __forceinline__ void mma_f16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// kFused: see the top of the file; gridDim.y CTAs of one blockIdx.x are one cluster and gridDim.z == 1.
// Otherwise partial[(split * T + tok) * E + e] is written.
template <bool kFused>
__global__ void __launch_bounds__(kRtThreads, 1)
router_kernel(const __grid_constant__ CUtensorMap tm_t, const __grid_constant__ CUtensorMap tm_w,
              float *__restrict__ partial, int T, int H, int E, int n_mma, int chunks_per_split,
              unsigned int *status, RouteOut ro) {
  extern __shared__ uint8_t rt_raw[];
  const uint32_t ring = (smem_u32(rt_raw) + 1023u) & ~1023u;
  const uint32_t bars = ring + kRtStages * kRtStage;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (kRtStages + s); };
  const uint32_t acc_bar = bars + 8u * (2 * kRtStages);
  __shared__ uint32_t tmem_base;
  __shared__ uint32_t abort_word;
  volatile uint32_t *abort_flag = &abort_word;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tok0 = blockIdx.x * kRtTok, e0 = blockIdx.z * kRtExp;
  const int n_chunks = (H + kRtK - 1) / kRtK;
  const int c_begin = blockIdx.y * chunks_per_split, c_end = min(n_chunks, c_begin + chunks_per_split);
  const int n = c_end - c_begin;  // can be <= 0 in a cluster (a power-of-two slice count): that CTA contributes zeros

  if (threadIdx.x == 0) {
    for (int s = 0; s < kRtStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(acc_bar, 1);
    abort_word = 0u;
    fence_mbar_init();
  }
  if (warp == 4 && lane == 0) {
    prefetch_tensormap(&tm_t);
    prefetch_tensormap(&tm_w);
  }
  if (warp == 5) {
    tmem_alloc(smem_u32(&tmem_base), kRtTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = tmem_base;

  if (warp == 4) {
    // ---- producer: one activation box and three weight boxes per chunk
    const uint32_t bytes = kRtTile + 3u * static_cast<uint32_t>(n_mma) * kRtK * 2u;
    for (int i = 0; i < n; ++i) {
      const int s = i % kRtStages;
      if (i >= kRtStages &&
          !mbar_wait_warp(empty_bar(s), ((i / kRtStages) & 1u) ^ 1u, abort_flag, status, ST_WAIT_EMPTY))
        break;
      if (elect_one()) {
        const uint32_t dst = ring + s * kRtStage;
        const int k = (c_begin + i) * kRtK;
        mbar_arrive_expect_tx(full_bar(s), bytes);
        tma_load_2d(dst, &tm_t, k, tok0, full_bar(s));
        for (int pl = 0; pl < 3; ++pl) tma_load_3d(dst + (1 + pl) * kRtTile, &tm_w, k, e0, pl, full_bar(s));
      }
      __syncwarp();
    }
  } else if (warp == 5) {
    // ---- issue: 3 planes x 4 k steps of 16 per chunk, all into the same accumulator
    const uint32_t idesc = idesc_bf16_m128(static_cast<uint32_t>(n_mma));
    for (int i = 0; i < n; ++i) {
      const int s = i % kRtStages;
      if (!mbar_wait_warp(full_bar(s), (i / kRtStages) & 1u, abort_flag, status, ST_WAIT_FULL)) break;
      tc_fence_after();
      if (elect_one()) {
        const uint32_t a_addr = ring + s * kRtStage;
        const uint64_t a_desc = smem_desc_sw128(a_addr);
#pragma unroll
        for (int pl = 0; pl < 3; ++pl) {
          const uint64_t b_desc = smem_desc_sw128(a_addr + (1 + pl) * kRtTile);
#pragma unroll
          for (int ks = 0; ks < kRtK / 16; ++ks)  // 16 bf16 = 32 bytes along k: +2 in the address field
            mma_f16_ss(tm, a_desc + 2u * ks, b_desc + 2u * ks, idesc, (i | pl | ks) != 0 ? 1u : 0u);
        }
        mma_commit(empty_bar(s));
        if (i == n - 1) mma_commit(acc_bar);
      }
      __syncwarp();
    }
  } else if (warp < 4) {
    // ---- result: warp w owns accumulator lanes 32 w .. 32 w + 31 = tokens tok0 + 32 w + lane
    const bool have = n > 0 && mbar_wait_warp(acc_bar, 0u, abort_flag, status, ST_WAIT_DFULL);
    tc_fence_after();
    const int row = tok0 + warp * 32 + lane;
    if constexpr (kFused) {
      const uint32_t dst = ring + static_cast<uint32_t>(warp * 32 + lane) * kRtRedPitch;
      for (int c0 = 0; c0 < kRtExp; c0 += 16) {
        uint32_t v[16];
        if (have && c0 < n_mma) {
          tmem_ld16(tm + (static_cast<uint32_t>(warp * 32) << 16) + c0, v);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = 0u;
        }
#pragma unroll
        for (int j = 0; j < 16; j += 4)
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst + (c0 + j) * 4), "r"(v[j]), "r"(v[j + 1]),
                       "r"(v[j + 2]), "r"(v[j + 3])
                       : "memory");
      }
    } else if (have) {
      float *out = partial + (static_cast<size_t>(blockIdx.y) * T + min(row, T - 1)) * E + e0;
      const bool vec = (E & 3) == 0;
      for (int c0 = 0; c0 < n_mma; c0 += 16) {
        uint32_t v[16];
        tmem_ld16(tm + (static_cast<uint32_t>(warp * 32) << 16) + c0, v);
        tmem_wait_ld();
        if (row < T) {
          if (vec && e0 + c0 + 16 <= E) {
#pragma unroll
            for (int j = 0; j < 16; j += 4)
              *reinterpret_cast<uint4 *>(out + c0 + j) = make_uint4(v[j], v[j + 1], v[j + 2], v[j + 3]);
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (e0 + c0 + j < E) out[c0 + j] = __uint_as_float(v[j]);
          }
        }
      }
    }
  }
  if constexpr (kFused) {
    // every CTA of the cluster has parked its slice; this CTA finishes its share of the 128 tokens
    cg::cluster_group cluster = cg::this_cluster();
    cluster_sync_all();
    const int n_slices = static_cast<int>(cluster.num_blocks());
    const int rows_per = kRtTok / n_slices, first = static_cast<int>(cluster.block_rank()) * rows_per;
    const uint32_t ring_off = ring - smem_u32(rt_raw);
    for (int lr = warp; lr < rows_per; lr += kRtThreads / 32) {
      const int r = first + lr, tok = tok0 + r;
      if (tok >= T) break;
      // lane l takes experts 4 l .. 4 l + 3: one 16-byte load per slice, all of them in flight together
      // (remote shared memory answers slowly, dependent loads would serialise)
      const float4 *mine = reinterpret_cast<const float4 *>(rt_raw + ring_off + static_cast<uint32_t>(r) * kRtRedPitch) + lane;
      float4 part[8];
#pragma unroll
      for (int sl = 0; sl < 8; ++sl)
        part[sl] = sl < n_slices ? *cluster.map_shared_rank(mine, sl) : make_float4(0.f, 0.f, 0.f, 0.f);
      double sum[4] = {0.0, 0.0, 0.0, 0.0};
#pragma unroll
      for (int sl = 0; sl < 8; ++sl)
        if (sl < n_slices) {
          sum[0] += static_cast<double>(part[sl].x);
          sum[1] += static_cast<double>(part[sl].y);
          sum[2] += static_cast<double>(part[sl].z);
          sum[3] += static_cast<double>(part[sl].w);
        }
      float v[kMaxExpPerLane];
      unsigned taken = 0;
#pragma unroll
      for (int i = 0; i < kMaxExpPerLane; ++i) {
        const int e = 4 * lane + i;
        if (i < 4 && e < E) {
          v[i] = __fadd_rn(static_cast<float>(sum[i & 3]), ro.bias[e]);
        } else {
          v[i] = 0.f;
          taken |= 1u << i;
        }
      }
      float *logit_row = ro.logits + static_cast<size_t>(ro.row_offset + tok) * E;
      if ((E & 3) == 0) {
        if (4 * lane < E) *reinterpret_cast<float4 *>(logit_row + 4 * lane) = make_float4(v[0], v[1], v[2], v[3]);
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i)
          if (4 * lane + i < E) logit_row[4 * lane + i] = v[i];
      }
      select_softmax_store<true>(v, taken, lane, ro.K, static_cast<size_t>(ro.row_offset + tok), ro.idx, ro.w, ro.counts,
                                 ro.tp, ro.peers);
    }
    cluster_sync_all();  // nobody leaves while a peer may still read its shared memory
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 5) tmem_dealloc(tm, kRtTmemCols);
}

bool encode_bf16_map(CUtensorMap *m, const void *base, int rank, const cuuint64_t *dims, const cuuint64_t *strides,
                     const cuuint32_t *box) {
  TensorMapEncodeFn fn = tensor_map_encoder();
  if (!fn) return false;
  const cuuint32_t es[3] = {1, 1, 1};
  return fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, const_cast<void *>(base), dims, strides, box, es,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// N of the instruction: the experts of one CTA rounded up to the 16 the M = 128 shapes allow.
int router_mma_n(int E) { return std::min(kRtExp, (E + 15) / 16 * 16); }
}  // namespace

int router_splits(int T, int H, int sm_count) {
  const int tiles = (T + kRtTok - 1) / kRtTok, n_chunks = (H + kRtK - 1) / kRtK;
  int splits = std::max(1, std::min(std::min(16, n_chunks), sm_count / tiles));
  const int cps = (n_chunks + splits - 1) / splits;
  return (n_chunks + cps - 1) / cps;  // every split gets at least one chunk
}

int router_chunks(int H) { return (H + kRtK - 1) / kRtK; }

// The kernel's shared-memory limit is a property of the (kernel, device) pair, so every device a handle is
// created on sets it for itself (moe_create calls this with that device current); a flag shared by the
// whole process would leave the launch rejected on every GPU but the first one a one-process,
// one-thread-per-GPU caller touches.  *max_cluster receives the largest cluster (8, 4, 2 or 1 CTAs of
// this kernel's footprint) the device can place, 0 if it cannot run the fused form at all.
cudaError_t router_init(int *max_cluster) {
  cudaError_t e = cudaFuncSetAttribute(router_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kRtSmem);
  if (e != cudaSuccess) return e;
  e = cudaFuncSetAttribute(router_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kRtSmem);
  if (e != cudaSuccess) return e;
  *max_cluster = 0;
  for (int size = 8; size >= 1 && *max_cluster == 0; size >>= 1) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1, size, 1);
    cfg.blockDim = dim3(kRtThreads, 1, 1);
    cfg.dynamicSmemBytes = kRtSmem;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = 1;
    at[0].val.clusterDim.y = size;
    at[0].val.clusterDim.z = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, router_kernel<true>, &cfg) == cudaSuccess && n > 0) *max_cluster = size;
    else (void)cudaGetLastError();
  }
  return cudaSuccess;
}

// Planes [3][E][H] of the split router weight as one box per (chunk, plane): rows past E read as zero.
bool make_router_weight_map(CUtensorMap *m, const __nv_bfloat16 *w3, int E, int H) {
  const cuuint64_t dims[3] = {static_cast<cuuint64_t>(H), static_cast<cuuint64_t>(E), 3};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(H) * 2, static_cast<cuuint64_t>(E) * H * 2};
  const cuuint32_t box[3] = {kRtK, static_cast<cuuint32_t>(router_mma_n(E)), 1};
  return encode_bf16_map(m, w3, 3, dims, strides, box);
}

namespace {
// `t` ([T, H] bf16, 16-byte aligned, H a multiple of 8) is the caller's buffer, so its tensor map is made on the
// host for every call (no device work, no allocation; under stream capture it is baked into the launch
// like any other kernel argument).
bool make_rows_map(CUtensorMap *m, const __nv_bfloat16 *t, int T, int H) {
  if ((H & 7) != 0 || (reinterpret_cast<uintptr_t>(t) & 15) != 0) return false;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(H), static_cast<cuuint64_t>(T)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(H) * 2};
  const cuuint32_t box[2] = {kRtK, kRtTok};
  return encode_bf16_map(m, t, 2, dims, strides, box);
}
}  // namespace

// Split-k partial sums for topk_softmax_kernel.  Returns false when the rows have no tensor map.
bool launch_router_partials(const __nv_bfloat16 *t, const CUtensorMap &tm_w, float *partial, int T, int H, int E,
                            int splits, unsigned int *status, cudaStream_t s) {
  CUtensorMap tm_t;
  if (!make_rows_map(&tm_t, t, T, H)) return false;
  const int n_chunks = router_chunks(H), cps = (n_chunks + splits - 1) / splits;
  dim3 grid((T + kRtTok - 1) / kRtTok, splits, (E + kRtExp - 1) / kRtExp);
  router_kernel<false><<<grid, kRtThreads, kRtSmem, s>>>(tm_t, tm_w, partial, T, H, E, router_mma_n(E), cps, status,
                                                          RouteOut{});
  return true;
}

// Slices of the fused form: a power of two (the 128 tokens of a tile are dealt out evenly), no more than
// the device places in one cluster, and no more than keeps one CTA per SM.  0: use the partial-sum form.
int router_fused_slices(int T, int H, int E, int sm_count, int max_cluster) {
  if (E > kRtExp || max_cluster < 1) return 0;
  const int tiles = (T + kRtTok - 1) / kRtTok;
  const int lim = std::min(std::min(8, max_cluster), std::min(router_chunks(H), std::max(1, sm_count / tiles)));
  int slices = 1;
  while (slices * 2 <= lim) slices *= 2;
  return slices;
}

// Router GEMM, bias, top-k, softmax and expert histogram in one launch (E <= 128).
bool launch_router_fused(const __nv_bfloat16 *t, const CUtensorMap &tm_w, int T, int H, int E, int slices,
                         const RouteOut &ro, unsigned int *status, cudaStream_t s) {
  CUtensorMap tm_t;
  if (!make_rows_map(&tm_t, t, T, H)) return false;
  const int n_chunks = router_chunks(H), cps = (n_chunks + slices - 1) / slices;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((T + kRtTok - 1) / kRtTok, slices, 1);
  cfg.blockDim = dim3(kRtThreads, 1, 1);
  cfg.dynamicSmemBytes = kRtSmem;
  cfg.stream = s;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = 1;
  at[0].val.clusterDim.y = slices;
  at[0].val.clusterDim.z = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, router_kernel<true>, tm_t, tm_w, static_cast<float *>(nullptr), T, H, E,
                            router_mma_n(E), cps, status, ro) == cudaSuccess;
}

}  // namespace moe
