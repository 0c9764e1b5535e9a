// Routing side of the MoE block (the router GEMM itself is router_sm100.cu): top-k + softmax, expert
// histogram, stable token->expert permutation, work list of the grouped GEMM,
// row gather and the weighted un-permute.  Everything stays on the device: the
// reference's per-layer host round trip (expert counts copied to the host, tile
// maps built there, getp-csrc/getp_run.cpp:2648-2692 and :3019-3068) is replaced
// by build_index_kernel.
#include <cuda_fp8.h>

#include <algorithm>
#include <cstdio>
#include <mutex>

#include "moe_internal.cuh"
#include "route_select.cuh"

namespace moe {

// ---------------------------------------------------------------------------
// Top-k + softmax over the selected logits + expert histogram.  One warp per
// token; the selection itself is select_softmax_store (route_select.cuh).
// ---------------------------------------------------------------------------

// With `partial` set, the logits are first formed from the router's split-k partial sums: slices added
// in ascending order in double precision, rounded to float, then the bias added in float
// (run.cpp:662-669), and written to `logits`.  Otherwise `logits` is the input.
// With tp > 0 the call routes rows [row_offset, row_offset + T) of a tensor-parallel group's union batch:
// logits go to those rows of `logits`, and the selection is written into the top-k buffers of every rank
// of the group (peer stores), so that no rank repeats another rank's routing.
__global__ void topk_softmax_kernel(float *__restrict__ logits, const float *__restrict__ partial, int splits,
                                    const float *__restrict__ bias, int T, int E, int K, int *__restrict__ idx,
                                    float *__restrict__ w, int *__restrict__ counts, int tp, TpPeers peers,
                                    int row_offset) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= T) return;
  float *row = logits + static_cast<size_t>(row_offset + warp) * E;
  float v[kMaxExpPerLane];
  unsigned taken = 0;
#pragma unroll
  for (int i = 0; i < kMaxExpPerLane; ++i) {
    const int e = lane + 32 * i;
    if (e < E) {
      if (partial != nullptr) {
        // the first 16 slices (router_splits() never makes more) are loaded together, then added in order
        const float *col = partial + static_cast<size_t>(warp) * E + e;
        const size_t slice = static_cast<size_t>(T) * E;
        float p[16];
#pragma unroll
        for (int sp = 0; sp < 16; ++sp) p[sp] = sp < splits ? col[sp * slice] : 0.f;
        double sum = 0.0;
#pragma unroll
        for (int sp = 0; sp < 16; ++sp)
          if (sp < splits) sum += static_cast<double>(p[sp]);
        for (int sp = 16; sp < splits; ++sp) sum += static_cast<double>(col[sp * slice]);
        v[i] = __fadd_rn(static_cast<float>(sum), bias[e]);
        row[e] = v[i];
      } else {
        v[i] = row[e];
      }
    } else {
      v[i] = 0.f;
      taken |= 1u << i;
    }
  }
  select_softmax_store(v, taken, lane, K, static_cast<size_t>(row_offset + warp), idx, w, counts, tp, peers);
}

// Expert histogram over an already exchanged selection (count_tokens_per_expert_kernel,
// kernels/moe.hpp:744); block-local bins first, so global atomics are E per block.
__global__ void __launch_bounds__(256) count_experts_kernel(const int *__restrict__ idx, int n, int E,
                                                            int *__restrict__ counts) {
  __shared__ int bins[256];
  for (int i = threadIdx.x; i < E; i += blockDim.x) bins[i] = 0;
  __syncthreads();
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    const int e = idx[i];
    if (e >= 0 && e < E) atomicAdd(&bins[e], 1);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < E; i += blockDim.x)
    if (bins[i]) atomicAdd(&counts[i], bins[i]);
}

void launch_count_experts(const int *idx, int n, int E, int *counts, cudaStream_t s) {
  const int blocks = std::max(1, std::min(64, (n + 1023) / 1024));
  count_experts_kernel<<<blocks, 256, 0, s>>>(idx, n, E, counts);
}

void launch_topk_softmax(float *logits, const float *partial, int splits, const float *bias, int T, int E, int K,
                         int *idx, float *w, int *counts, cudaStream_t s, int tp, const TpPeers *peers, int row_offset) {
  const int threads = 128;
  const int blocks = (T * 32 + threads - 1) / threads;
  TpPeers pv = {};
  if (tp > 0 && peers != nullptr) pv = *peers;
  topk_softmax_kernel<<<blocks, threads, 0, s>>>(logits, partial, splits, bias, T, E, K, idx, w, counts, tp, pv,
                                                 row_offset);
}

// ---------------------------------------------------------------------------
// Offsets, stable compaction and the GEMM work lists.  One block per expert.
// Reference: host scan + tile maps (getp_run.cpp:2648-2692) and
// route_build_index_kernel_bf16wts (kernels/moe.hpp:1173-1270): rows of one
// expert are in ascending token order.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(1024)
build_index_kernel(const int *__restrict__ topk_idx, const int *__restrict__ counts, int T, int E, int K,
                   int n_ntiles1, int n_ntiles2, int *__restrict__ offsets, int *__restrict__ tile_base,
                   int *__restrict__ pair_row, int *__restrict__ row_token, int *__restrict__ pair_slot,
                   unsigned int *__restrict__ tile_done, int tile_done_total_slot, WorkItem *__restrict__ work1,
                   WorkItem *__restrict__ work2, int *__restrict__ n_work, int max_work1, int max_work2,
                   unsigned int *status) {
  __shared__ int s_red[2][32];
  __shared__ int s_warp[32];
  const int e = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_warps = blockDim.x >> 5;   // 8, or 32 for batches whose selections 8 warps cannot hold in registers

  // Stable compaction in ascending token order.  Warp w owns the contiguous token range [w*per, (w+1)*per):
  // a first walk counts the range's hits with ballots, the block's one barrier turns the warps' counts into
  // starting positions, a second walk writes the rows.
  const int per = ((T + n_warps - 1) / n_warps + 31) / 32 * 32;       // tokens per warp, whole ballot steps
  const int t_begin = warp * per, t_end = min(T, t_begin + per);
  auto hit_of = [&](int t) -> int {
    if (t >= t_end) return -1;
    if (K == 4) {                                      // the usual case: one 16-byte load
      const int4 v = __ldg(reinterpret_cast<const int4 *>(topk_idx) + t);
      return v.x == e ? 0 : v.y == e ? 1 : v.z == e ? 2 : v.w == e ? 3 : -1;
    }
    for (int k = 0; k < K; ++k)
      if (topk_idx[static_cast<size_t>(t) * K + k] == e) return k;
    return -1;
  };
  // the first kCached ballot steps of the range (all of it up to 256 tokens per warp) are loaded at once and kept
  constexpr int kCached = 8;
  int cached[kCached];
#pragma unroll
  for (int j = 0; j < kCached; ++j) cached[j] = hit_of(t_begin + 32 * j + lane);

  // exclusive prefix over experts below e: rows and token tiles (its loads travel with the ones above)
  int my_rows = 0, my_tiles = 0;
  for (int i = tid; i < e; i += blockDim.x) {
    const int c = counts[i];
    my_rows += c;
    my_tiles += (c + kTokTile - 1) / kTokTile;
  }
#pragma unroll
  for (int off = 16; off; off >>= 1) {
    my_rows += __shfl_xor_sync(0xffffffffu, my_rows, off);
    my_tiles += __shfl_xor_sync(0xffffffffu, my_tiles, off);
  }
  // first walk: this warp's hits
  const int t_rest = t_begin + 32 * kCached;
  int mine = 0;
#pragma unroll
  for (int j = 0; j < kCached; ++j) mine += __popc(__ballot_sync(0xffffffffu, cached[j] >= 0));
  for (int t0 = t_rest; t0 < t_end; t0 += 32) mine += __popc(__ballot_sync(0xffffffffu, hit_of(t0 + lane) >= 0));
  if (lane == 0) { s_red[0][warp] = my_rows; s_red[1][warp] = my_tiles; s_warp[warp] = mine; }
  __syncthreads();   // the only block-wide barrier: prefix partials and hit counts of all warps
  int off = 0, tiles_before = 0;
  for (int i = 0; i < n_warps; ++i) { off += s_red[0][i]; tiles_before += s_red[1][i]; }
  const int cnt = counts[e];
  const int ntt = (cnt + kTokTile - 1) / kTokTile;  // token tiles of this expert (rows e's tiles, in order)
  if (tid == 0) {
    offsets[e] = off;
    tile_base[e] = tiles_before;
    if (e == E - 1) { offsets[E] = off + cnt; tile_base[E] = tiles_before + ntt; }
  }
  // completion counters of the fused expert MLP launch: this expert's token tiles, and the total
  for (int i = tid; i < ntt; i += blockDim.x) tile_done[tiles_before + i] = 0u;
  if (e == E - 1 && tid == 0) tile_done[tile_done_total_slot] = 0u;

  int before = 0, total_hits = 0;
  for (int i = 0; i < n_warps; ++i) {
    before += i < warp ? s_warp[i] : 0;
    total_hits += s_warp[i];
  }
  auto place = [&](int t, int hit) {
    const unsigned m = __ballot_sync(0xffffffffu, hit >= 0);
    if (hit >= 0) {
      const int pos = before + __popc(m & ((1u << lane) - 1u));
      if (pos < cnt) {
        const int r = off + pos;
        row_token[r] = t;
        // where the row's high term goes in the quantised activations: token tile, then 2 rows per token
        pair_slot[static_cast<size_t>(t) * K + hit] = (tiles_before + pos / kTokTile) * kTileM + 2 * (pos % kTokTile);
        pair_row[static_cast<size_t>(t) * K + hit] = r;
      } else {
        atomicOr(status, ST_BAD_INDEX);
      }
    }
    before += __popc(m);
  };
#pragma unroll
  for (int j = 0; j < kCached; ++j) place(t_begin + 32 * j + lane, cached[j]);
  for (int t0 = t_rest; t0 < t_end; t0 += 32) place(t0 + lane, hit_of(t0 + lane));
  if (tid == 0 && total_hits != cnt) atomicOr(status, ST_BAD_INDEX);

  // work items: one per (token tile of kTokTile rows, block of kTileN weight rows); items that share a
  // weight block are adjacent so that block is fetched from HBM once and re-read from L2.  Single blocks
  // rather than pairs: the items of a launch are dealt round-robin to one CTA per SM, and the finer the
  // items, the smaller the idle share of the last round (930 pair items of MLP2 over 148 SMs lose 10 %,
  // 1860 single ones 3 %).
  for (int which = 0; which < 2; ++which) {
    const int nn = which ? n_ntiles2 : n_ntiles1;
    WorkItem *work = which ? work2 : work1;
    const int cap = which ? max_work2 : max_work1;
    const int start = tiles_before * nn;
    for (int i = tid; i < ntt * nn; i += blockDim.x) {
      const int nt = i / ntt, tt = i % ntt;
      WorkItem it;
      it.expert = e;
      it.ntile = nt;
      it.tile = tiles_before + tt;
      it.row0 = off + tt * kTokTile;
      it.ntok = min(kTokTile, cnt - tt * kTokTile);
      it.nblk = 1;
      it.pad[0] = it.pad[1] = 0;
      if (start + i < cap) work[start + i] = it;
      else atomicOr(status, ST_BAD_INDEX);
    }
    if (e == E - 1 && tid == 0) n_work[which] = min((tiles_before + ntt) * nn, cap);
  }
}

void launch_build_index(const int *topk_idx, const int *counts, int T, int E, int K, int n_ntiles1, int n_ntiles2,
                        int *offsets, int *tile_base, int *pair_row, int *row_token, int *pair_slot,
                        unsigned int *tile_done, int tile_done_total_slot, WorkItem *work1, WorkItem *work2, int *n_work, int max_work1, int max_work2,
                        unsigned int *status, cudaStream_t s) {
  build_index_kernel<<<E, T > 2048 ? 1024 : 256, 0, s>>>(topk_idx, counts, T, E, K, n_ntiles1, n_ntiles2, offsets, tile_base,
                                       pair_row, row_token, pair_slot, tile_done, tile_done_total_slot, work1, work2, n_work,
                                                          max_work1, max_work2, status);
}

// ---------------------------------------------------------------------------
// Row gather + quantisation for the tensor-core GEMM.  Reference:
// pack_rows_kernel_bf16_in (kernels/moe.hpp:983-1048) copies bf16 rows; here
// each gathered row becomes TWO e4m3 rows (the block-scaled MMA has no bf16
// operand): with s = 2^e chosen so that the row's largest |x|/s lies in
// [128, 256), high = e4m3(x/s) and low = e4m3((x/s - high) * 16).  A bf16 value
// has 8 significant bits, the high term keeps 4 of them and the residual fits the
// 4 of the low term, so high + low/16 == x/s exactly unless x is more than 2^13
// below the row maximum.  Row 2i of a 128-row token tile is the high term of the
// tile's token i, row 2i+1 the low term; their UE8M0 scales (127+e, 127+e-4) go
// into the tile's 512-byte scale atom, byte (r%32)*16 + (r/32)*4 + kb for row r
// and every k block kb (the scale is per row, so the four bytes are equal).
// ---------------------------------------------------------------------------
// The two rows depend on the token only, not on the expert, so a warp quantises one TOKEN (its row stays in
// the warp's registers: kQrVec x 32 bytes per lane) and stores the result once per selected expert, at the
// tile rows build_index_kernel assigned to the (token, expert) pairs.
constexpr int kQrWarps = 4;

template <int kQrVec>         // 6: rows of up to 3072 elements, 8: up to 4096
__global__ void __launch_bounds__(kQrWarps * 32)
quantize_rows_kernel(const __nv_bfloat16 *__restrict__ t, const int *__restrict__ pair_slot, int T, int K,
                     uint8_t *__restrict__ xq, uint8_t *__restrict__ sfa, int H) {
  const int lane = threadIdx.x & 31;
  const int tok = blockIdx.x * kQrWarps + (threadIdx.x >> 5);
  if (tok >= T) return;   // whole warps leave: no block-wide barrier below
  int slot[kMaxTopK];
#pragma unroll
  for (int k = 0; k < kMaxTopK; ++k) slot[k] = k < K ? pair_slot[static_cast<size_t>(tok) * K + k] : -1;
  const uint4 *src = reinterpret_cast<const uint4 *>(t + static_cast<size_t>(tok) * H);
  const int ngrp = H / 16;    // a lane takes groups of 16 elements: 32 bytes in, 16 + 16 bytes out
  uint4 v[kQrVec][2];
  float amax = 0.f;
#pragma unroll
  for (int u = 0; u < kQrVec; ++u) {
    const int g = lane + u * 32;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      v[u][h] = g < ngrp ? __ldg(src + 2 * g + h) : make_uint4(0u, 0u, 0u, 0u);
      const uint32_t in[4] = {v[u][h].x, v[u][h].y, v[u][h].z, v[u][h].w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        amax = fmaxf(amax, fabsf(__uint_as_float(in[j] << 16)));
        amax = fmaxf(amax, fabsf(__uint_as_float(in[j] & 0xffff0000u)));
      }
    }
  }
#pragma unroll
  for (int off = 16; off; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
  // e = floor(log2(amax)) - 7, kept where both scales stay valid UE8M0 bytes
  int e = static_cast<int>((__float_as_uint(amax) >> 23) & 0xffu) - 127 - 7;
  e = max(-120, min(e, 120));
  const float inv = __uint_as_float(static_cast<uint32_t>(127 - e) << 23);  // 2^-e
  // activation tiles: [tile][k slice][128 rows][128 bytes]; 16 elements never straddle a slice
  const int n_kc = (H + kChunkK - 1) / kChunkK;
#pragma unroll
  for (int u = 0; u < kQrVec; ++u) {
    const int g = lane + u * 32;
    if (g >= ngrp) break;
    uint32_t h8[4], l8[4];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const uint32_t in[4] = {v[u][h].x, v[u][h].y, v[u][h].z, v[u][h].w};
      float f[8];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        f[2 * j] = __uint_as_float(in[j] << 16) * inv;
        f[2 * j + 1] = __uint_as_float(in[j] & 0xffff0000u) * inv;
      }
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        const uint32_t a = __nv_cvt_float2_to_fp8x2(make_float2(f[4 * q], f[4 * q + 1]), __NV_SATFINITE, __NV_E4M3);
        const uint32_t b = __nv_cvt_float2_to_fp8x2(make_float2(f[4 * q + 2], f[4 * q + 3]), __NV_SATFINITE, __NV_E4M3);
        const uint32_t hi = a | (b << 16);
        h8[2 * h + q] = hi;
        float rs[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const __half_raw hr = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>((hi >> (8 * j)) & 0xffu), __NV_E4M3);
          rs[j] = (f[4 * q + j] - __half2float(*reinterpret_cast<const __half *>(&hr))) * 16.0f;
        }
        const uint32_t c2 = __nv_cvt_float2_to_fp8x2(make_float2(rs[0], rs[1]), __NV_SATFINITE, __NV_E4M3);
        const uint32_t d2 = __nv_cvt_float2_to_fp8x2(make_float2(rs[2], rs[3]), __NV_SATFINITE, __NV_E4M3);
        l8[2 * h + q] = c2 | (d2 << 16);
      }
    }
    const size_t in_tile = static_cast<size_t>(g >> 3) * (kTileM * kChunkK) + (g & 7) * 16;  // slice g/8, byte 16*(g%8)
#pragma unroll
    for (int k = 0; k < kMaxTopK; ++k) {
      if (slot[k] < 0) continue;
      const int tile = slot[k] / kTileM, i2 = slot[k] % kTileM;   // i2 = 2 * (token's place in the tile)
      uint8_t *dst = xq + (static_cast<size_t>(tile) * n_kc * kTileM + i2) * kChunkK + in_tile;
      *reinterpret_cast<uint4 *>(dst) = make_uint4(h8[0], h8[1], h8[2], h8[3]);
      *reinterpret_cast<uint4 *>(dst + kChunkK) = make_uint4(l8[0], l8[1], l8[2], l8[3]);   // the low row follows
    }
  }
  if (lane < 2) {
    const uint32_t byte = static_cast<uint32_t>(127 + e - 4 * lane);
#pragma unroll
    for (int k = 0; k < kMaxTopK; ++k) {
      if (slot[k] < 0) continue;
      const int tile = slot[k] / kTileM, rr = slot[k] % kTileM + lane;  // row inside the tile: even = high, odd = low
      uint8_t *atom = sfa + static_cast<size_t>(tile) * kSfAtomBytes;
      *reinterpret_cast<uint32_t *>(atom + (rr % 32) * 16 + (rr / 32) * 4) = byte * 0x01010101u;
    }
  }
}

int quantize_rows_max_hidden() { return 32 * 8 * 16; }

void launch_quantize_rows(const __nv_bfloat16 *t, const int *pair_slot, int T, int K, uint8_t *xq, uint8_t *sfa, int H,
                          cudaStream_t s) {
  const int blocks = (T + kQrWarps - 1) / kQrWarps;
  if (H <= 32 * 6 * 16)
    quantize_rows_kernel<6><<<blocks, kQrWarps * 32, 0, s>>>(t, pair_slot, T, K, xq, sfa, H);
  else
    quantize_rows_kernel<8><<<blocks, kQrWarps * 32, 0, s>>>(t, pair_slot, T, K, xq, sfa, H);
}

// ---------------------------------------------------------------------------
// Row gather: xperm[r, :] = fp16(t[row_token[r], :]).  Reference:
// pack_rows_kernel_bf16_in (kernels/moe.hpp:983-1048).  The GEMM operands are
// fp16 (the MXFP4 decode instruction produces fp16); every bf16 value of
// magnitude in [2^-14, 65504] converts exactly.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(128)
gather_rows_kernel(const __nv_bfloat16 *__restrict__ t, const int *__restrict__ row_token,
                   const int *__restrict__ offsets, int E, __half *__restrict__ xperm, int H) {
  const int r = blockIdx.x;
  if (r >= offsets[E]) return;
  const int tok = row_token[r];
  const uint4 *src = reinterpret_cast<const uint4 *>(t + static_cast<size_t>(tok) * H);
  uint4 *dst = reinterpret_cast<uint4 *>(xperm + static_cast<size_t>(r) * H);
  for (int i = threadIdx.x; i < H / 8; i += blockDim.x) {
    const uint4 v = __ldg(src + i);
    const uint32_t in[4] = {v.x, v.y, v.z, v.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float lo = __uint_as_float(in[j] << 16), hi = __uint_as_float(in[j] & 0xffff0000u);
      const __half2 h = __floats2half2_rn(lo, hi);
      o[j] = *reinterpret_cast<const uint32_t *>(&h);
    }
    dst[i] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

void launch_gather_rows(const __nv_bfloat16 *t, const int *row_token, const int *offsets, int E, __half *xperm,
                        int H, int max_pairs, cudaStream_t s) {
  gather_rows_kernel<<<max_pairs, 128, 0, s>>>(t, row_token, offsets, E, xperm, H);
}

// ---------------------------------------------------------------------------
// Weighted un-permute: out[t, :] = sum_k w[t, k] * y[pair_row[t, k], :], terms
// added in ascending expert index with separate multiply and add, which is the
// order and rounding of run.cpp:678 / :738-741.  GPU counterpart:
// reduce_tokenwise_expert_outputs_bf16_bf16wts (kernels/moe.hpp:700-730).
// ---------------------------------------------------------------------------
// The expert rows of one step are all requested before the first is used, and the next step's while this
// one is finished.  kK: experts per token known at compile time, 0: any K up to kMaxTopK (predicated).
template <int kK>
__global__ void __launch_bounds__(128)
combine_kernel(const __half *__restrict__ y, const int *__restrict__ topk_idx, const float *__restrict__ topk_w,
               const int *__restrict__ pair_row, int T, int H, int K, __nv_bfloat16 *__restrict__ out_bf16,
               float *__restrict__ out_f32, int tp, TpPeers peers, int rows_local, int rank,
               const __nv_bfloat16 *__restrict__ residual) {
  constexpr int kSlots = kK > 0 ? kK : kMaxTopK;
  if (kK > 0) K = kK;
  int t = blockIdx.x;
  // tensor-parallel call: the row's bf16 partial goes straight into slot `rank` of the landing buffer of the
  // rank that owns row t (a peer store over NVLink), which is the send half of the reduce-scatter.  Blocks
  // start with the rows of the next rank and end with this rank's own rows, so that the link is busy from the
  // first block on and the rows that need no link fill the tail.
  if (tp > 0) {
    t = (t + (rank + 1) * rows_local) % T;
    out_bf16 = static_cast<__nv_bfloat16 *>(peers.partial[t / rows_local]) +
               (static_cast<ptrdiff_t>(rank) * rows_local + (t % rows_local) - t) * static_cast<ptrdiff_t>(H);
  }
  int ex[kSlots], row[kSlots];
  float wt[kSlots];
#pragma unroll
  for (int k = 0; k < kSlots; ++k) {
    if (k < K) {
      ex[k] = topk_idx[static_cast<size_t>(t) * K + k];
      wt[k] = topk_w[static_cast<size_t>(t) * K + k];
      row[k] = pair_row[static_cast<size_t>(t) * K + k];
    } else {
      ex[k] = 0x7fffffff; wt[k] = 0.f; row[k] = 0;
    }
  }
#pragma unroll
  for (int i = 1; i < kSlots; ++i)  // sort by expert index (a fixed network of compare-exchanges: registers only)
#pragma unroll
    for (int j = kSlots - 1; j >= i; --j)
      if (ex[j] < ex[j - 1]) {
        int a = ex[j]; ex[j] = ex[j - 1]; ex[j - 1] = a;
        a = row[j]; row[j] = row[j - 1]; row[j - 1] = a;
        float f = wt[j]; wt[j] = wt[j - 1]; wt[j - 1] = f;
      }
  const uint4 *src[kSlots];
#pragma unroll
  for (int k = 0; k < kSlots; ++k) src[k] = reinterpret_cast<const uint4 *>(y + static_cast<size_t>(row[k]) * H);
  // 16 bytes (8 values) per thread and expert row
  const int n_vec = H / 8;
  uint4 raw[kSlots];
  auto fetch = [&](int i) {
#pragma unroll
    for (int k = 0; k < kSlots; ++k)
      if (k < K && i < n_vec) raw[k] = __ldg(src[k] + i);
  };
  fetch(threadIdx.x);
  for (int i = threadIdx.x; i < n_vec; i += blockDim.x) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll
    for (int k = 0; k < kSlots; ++k) {
      if (k < K) {
        const uint32_t w4[4] = {raw[k].x, raw[k].y, raw[k].z, raw[k].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 v = __half22float2(*reinterpret_cast<const __half2 *>(&w4[j]));
          acc[2 * j] = __fadd_rn(acc[2 * j], __fmul_rn(v.x, wt[k]));
          acc[2 * j + 1] = __fadd_rn(acc[2 * j + 1], __fmul_rn(v.y, wt[k]));
        }
      }
    }
    fetch(i + blockDim.x);   // the next step's rows are on their way while this one is finished and stored
    if (out_f32 != nullptr) {
      float4 *o = reinterpret_cast<float4 *>(out_f32 + static_cast<size_t>(t) * H) + 2 * i;
      o[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
      o[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
    }
    if (residual != nullptr) {  // x += block output (accumulate_kernel_bf16, kernels/other_kernels.hpp:18-37), one rounding
      const uint4 r = __ldg(reinterpret_cast<const uint4 *>(residual + static_cast<size_t>(t) * H) + i);
      const uint32_t r4[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        acc[2 * j] += __uint_as_float(r4[j] << 16);
        acc[2 * j + 1] += __uint_as_float(r4[j] & 0xffff0000u);
      }
    }
    if (out_bf16 != nullptr) {
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const __nv_bfloat162 b = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
        o[j] = *reinterpret_cast<const uint32_t *>(&b);
      }
      reinterpret_cast<uint4 *>(out_bf16 + static_cast<size_t>(t) * H)[i] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

void launch_combine(const __half *y, const int *topk_idx, const float *topk_w, const int *pair_row, int T, int H,
                    int K, __nv_bfloat16 *out_bf16, float *out_f32, cudaStream_t s, int tp, const TpPeers *peers,
                    int rows_local, int rank, const __nv_bfloat16 *residual) {
  TpPeers pv = {};
  if (tp > 0 && peers != nullptr) pv = *peers;
  auto kernel = K == 4 ? combine_kernel<4> : combine_kernel<0>;
  kernel<<<T, 128, 0, s>>>(y, topk_idx, topk_w, pair_row, T, H, K, out_bf16, out_f32, tp, pv, rows_local, rank, residual);
}

// ---------------------------------------------------------------------------
// Pre-MoE RMSNorm, step 0 of moe_gpu / moe_gpu_120b: t = w * (x / sqrt(mean(x^2) + 1e-5)), bf16 in
// and out, sum of squares in double.  Reference: rmsnorm_kernel_bf16_io (kernels/rmsnorm.hpp:115-164)
// and rmsnorm of the CPU path (run.cpp:320-333).
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
rmsnorm_rows_kernel(const __nv_bfloat16 *__restrict__ x, const __nv_bfloat16 *__restrict__ w,
                    __nv_bfloat16 *__restrict__ t, int H) {
  __shared__ double s_part[8];
  const uint4 *src = reinterpret_cast<const uint4 *>(x + static_cast<size_t>(blockIdx.x) * H);
  double ss = 0.0;
  for (int c = threadIdx.x; c < H / 8; c += blockDim.x) {
    const uint4 v = __ldg(src + c);
    const uint32_t in[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float a = __uint_as_float(in[j] << 16), b = __uint_as_float(in[j] & 0xffff0000u);
      ss += static_cast<double>(a) * a + static_cast<double>(b) * b;
    }
  }
#pragma unroll
  for (int off = 16; off; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
  if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = ss;
  __syncthreads();
  double tot = 0.0;
#pragma unroll
  for (int i = 0; i < 8; ++i) tot += s_part[i];
  const float inv = static_cast<float>(1.0 / sqrt(tot / H + 1e-5));
  const uint4 *wv = reinterpret_cast<const uint4 *>(w);
  uint4 *dst = reinterpret_cast<uint4 *>(t + static_cast<size_t>(blockIdx.x) * H);
  for (int c = threadIdx.x; c < H / 8; c += blockDim.x) {
    const uint4 v = __ldg(src + c), g = __ldg(wv + c);
    const uint32_t in[4] = {v.x, v.y, v.z, v.w}, gn[4] = {g.x, g.y, g.z, g.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float a = __uint_as_float(gn[j] << 16) * (inv * __uint_as_float(in[j] << 16));
      const float b = __uint_as_float(gn[j] & 0xffff0000u) * (inv * __uint_as_float(in[j] & 0xffff0000u));
      const __nv_bfloat162 q = __floats2bfloat162_rn(a, b);
      o[j] = *reinterpret_cast<const uint32_t *>(&q);
    }
    dst[c] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

void launch_rmsnorm_rows(const __nv_bfloat16 *x, const __nv_bfloat16 *w, __nv_bfloat16 *t, int rows, int H,
                         cudaStream_t s) {
  rmsnorm_rows_kernel<<<rows, 256, 0, s>>>(x, w, t, H);
}

// ---------------------------------------------------------------------------
// Routing without any allocation (no counterpart in the reference).
//
// Who this is for: a caller that is not allowed to reach the CUDA allocator at
// the moment it needs a routing decision.  Two examples: a serving loop that
// was given all of its device memory once, at start-up, by a pool that owns the
// rest of the GPU, so that a later cudaMalloc can fail or fragment that pool;
// and a latency-critical thread for which the device-wide synchronisation
// hidden inside cudaMalloc/cudaFree would stall work on other streams.
//
// The router needs scratch memory for its split-k partial sums.  Here that
// scratch is a fixed array in the library's own device image instead of a
// cudaMalloc'ed buffer: 8 MiB, which every GPU that loads this library holds
// until the process exits.  Host code cannot use the array's name as a device
// address; its address is looked up once per device, with that device current,
// by cudaGetSymbolAddress on the first call made on that device.  That first
// call should therefore be made during start-up, before any stream capture.
//
// All calls share the one array per device, so two calls whose kernels overlap
// on the GPU (different streams) race; serialise them.  Nothing in the array
// has to start at zero: every element a call reads was written by the same call
// (each k-slice writes its full rows x experts block), so stale contents of an
// earlier, larger call are never read.
// ---------------------------------------------------------------------------
constexpr size_t kStaticRouteFloats = static_cast<size_t>(2) << 20;  // 2 Mi floats = 8 MiB
static __device__ __align__(256) float g_route_scratch[kStaticRouteFloats];

namespace {
constexpr int kMaxDevices = 64;
float *g_route_scratch_ptr[kMaxDevices] = {};
std::mutex g_route_scratch_mu;

// Device address of g_route_scratch on `device`, which must be the current device.
cudaError_t route_scratch_for(int device, float **out) {
  std::lock_guard<std::mutex> lock(g_route_scratch_mu);
  if (g_route_scratch_ptr[device] == nullptr) {
    float *p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void **>(&p), g_route_scratch);
    if (e != cudaSuccess) return e;
    g_route_scratch_ptr[device] = p;
  }
  *out = g_route_scratch_ptr[device];
  return cudaSuccess;
}
}  // namespace

}  // namespace moe

extern "C" int moe_route_static(moe_handle c, int layer, const void *t_dev, int rows, float *logits_dev,
                                int *idx_dev, float *w_dev, void *stream) {
  using namespace moe;
  if (!c) return MOE_ERR_INVALID;
  auto fail = [&](int code, const char *msg) { c->err = msg; return code; };
  if (layer < 0 || layer >= c->L || !t_dev || !logits_dev || !idx_dev || !w_dev || rows <= 0)
    return fail(MOE_ERR_INVALID, "moe_route_static: bad layer index, null pointer or rows <= 0");
  if (c->cfg.device < 0 || c->cfg.device >= kMaxDevices) return fail(MOE_ERR_INVALID, "moe_route_static: device ordinal out of range");
  LayerWeights &w = c->layers[layer];
  if (!w.loaded) return fail(MOE_ERR_STATE, "moe_route_static: layer has no weights");
  const size_t per_slice = static_cast<size_t>(rows) * c->E;
  if (per_slice > kStaticRouteFloats) {
    char buf[200];
    snprintf(buf, sizeof(buf), "moe_route_static: rows * n_experts = %zu exceeds the fixed scratch of %zu floats (8 MiB)",
             per_slice, kStaticRouteFloats);
    return fail(MOE_ERR_INVALID, buf);
  }
  if (cudaSetDevice(c->cfg.device) != cudaSuccess) return fail(MOE_ERR_CUDA, "moe_route_static: cudaSetDevice failed");
  float *scratch = nullptr;
  if (route_scratch_for(c->cfg.device, &scratch) != cudaSuccess)
    return fail(MOE_ERR_CUDA, "moe_route_static: cudaGetSymbolAddress failed");
  // as many k-slices as the regular path would use, but no more than fit the fixed scratch
  int splits = router_splits(rows, c->H, c->sm_count);
  const int fit = static_cast<int>(kStaticRouteFloats / per_slice);
  if (splits > fit) {
    const int n_chunks = router_chunks(c->H), cps = (n_chunks + fit - 1) / fit;
    splits = (n_chunks + cps - 1) / cps;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (!launch_router_partials(static_cast<const __nv_bfloat16 *>(t_dev), w.tm_router, scratch, rows, c->H, c->E, splits,
                              c->status, s))
    return fail(MOE_ERR_INVALID, "moe_route_static: no tensor map for the rows (16-byte aligned, hidden_dim a multiple of 8?)");
  launch_topk_softmax(logits_dev, scratch, splits, w.router_b, rows, c->E, c->K, idx_dev, w_dev, nullptr, s);
  c->launches += 2;
  if (cudaGetLastError() != cudaSuccess) return fail(MOE_ERR_CUDA, "moe_route_static: kernel launch failed");
  return MOE_OK;
}
