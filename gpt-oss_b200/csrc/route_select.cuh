// Top-k selection and softmax of one token's router logits by one warp, shared by
// topk_softmax_kernel (route.cu) and the fused router kernel (router_sm100.cu).
// Reference: topk (run.cpp:387-420) then softmax (run.cpp:335-353, :674); GPU counterpart
// route_select_softmax_kernel_bf16io (kernels/moe.hpp:465-561) and
// count_tokens_per_expert_kernel (:744).  Selection is exact: plain fp32 comparisons, equal
// values resolved towards the lower index (kernels/moe.hpp:333-342).  Weights stay fp32.
#pragma once
#include "moe_internal.cuh"

namespace moe {

constexpr int kMaxExpPerLane = 8;  // E <= 256
constexpr int kMaxTopK = 8;

// Lane l holds in v[i] the logit of expert l + 32 i (kContig = false), or of expert 4 l + i, i < 4
// (kContig = true, at most 128 experts); bit i of `taken` is set where that expert does not exist.  The
// outcome depends on values and expert numbers only, not on which lane holds what.
// Writes the K selected experts and their softmax weights to row `out_row` of the top-k buffers (of every
// rank of a tensor-parallel group when tp > 0) and adds the selection to the expert histogram.
template <bool kContig = false>
__device__ __forceinline__ void select_softmax_store(const float (&v)[kMaxExpPerLane], unsigned taken, int lane, int K,
                                                     size_t out_row, int *__restrict__ idx, float *__restrict__ w,
                                                     int *__restrict__ counts, int tp, const TpPeers &peers) {
  float sel_v = 0.f;  // lane k keeps the k-th selected logit
  int sel_i = 0;
  for (int k = 0; k < K; ++k) {
    float bv = 0.f;
    int bi = -1;
#pragma unroll
    for (int i = 0; i < kMaxExpPerLane; ++i) {
      if (taken & (1u << i)) continue;
      if (kContig && i >= 4) continue;
      if (bi < 0 || v[i] > bv) { bv = v[i]; bi = kContig ? 4 * lane + i : lane + 32 * i; }  // ascending e: ties keep the lower index
    }
#pragma unroll
    for (int off = 16; off; off >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
      if (oi >= 0 && (bi < 0 || ov > bv || (ov == bv && oi < bi))) { bv = ov; bi = oi; }
    }
    if (bi >= 0 && (kContig ? (bi >> 2) : (bi & 31)) == lane) taken |= 1u << (kContig ? (bi & 3) : (bi >> 5));
    if (lane == k) { sel_v = bv; sel_i = bi; }
  }
  // softmax over the K selected values, double max/sum as in run.cpp:335-353
  double mx = -1e300;
  for (int k = 0; k < K; ++k) {
    const float vk = __shfl_sync(0xffffffffu, sel_v, k);
    mx = fmax(mx, static_cast<double>(vk));
  }
  float ex = 0.f;
  if (lane < K) ex = expf(static_cast<float>(static_cast<double>(sel_v) - mx));
  double sum = 0.0;
  for (int k = 0; k < K; ++k) sum += static_cast<double>(__shfl_sync(0xffffffffu, ex, k));
  if (lane < K) {
    const float wt = static_cast<float>(static_cast<double>(ex) / sum);
    const size_t o = out_row * K + lane;
    if (tp > 0) {
      for (int r = 0; r < tp; ++r) {
        static_cast<int *>(peers.topk_idx[r])[o] = sel_i;
        static_cast<float *>(peers.topk_w[r])[o] = wt;
      }
    } else {
      idx[o] = sel_i;
      w[o] = wt;
    }
    if (counts != nullptr && sel_i >= 0) atomicAdd(&counts[sel_i], 1);
  }
}

}  // namespace moe
