// Tensor-parallel exchange of the MoE block over NVLink peer memory.
//
// Reference counterparts: ring_allgather_rows_bf16 (getp-csrc/tp_ring.hpp:70-118)
// or the direct pulls of moe_gpu (getp_run.cpp:2580-2607) before the MLPs; the
// pull-and-add reduce-scatter of moe_gpu_120b (getp_run.cpp:3206-3246, with
// vec_add_inplace_bf16, tp_ring.hpp:220-231) after them; and the host spin
// barrier tp_group_barrier (getp-csrc/nccl.hpp:116-137).  The reference drives
// hipMemcpyPeerAsync from the host and synchronises stream and host between
// ring steps.  Behind NVSwitch every peer is one hop away, so a ring buys
// nothing: each rank PUSHES its rows into every peer's gather buffer with plain
// 16-byte stores, and each row owner PULLS its slice of every peer's partial
// output and adds them in rank order (fp32 add, bf16 payloads, deterministic).
// The host barrier becomes per-peer epoch flags in device memory, written with
// st.release.sys and polled with a bounded ld.acquire.sys loop.
//
// Kernels of different ranks wait on one another, so every rank of a group must
// run on its own GPU.  No TMA, no multicast: ordinary loads/stores on peer
// pointers.
#include "moe_internal.cuh"

namespace moe {

constexpr int kPushBlocks = 32;

__device__ __forceinline__ void st_release_sys(uint32_t *p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Every rank's rows [rows_local, H] -> slot `rank` of the gather buffer of every rank of the group.
__global__ void __launch_bounds__(256)
tp_allgather_push_kernel(const uint4 *__restrict__ src, size_t n_vec, TpPeers peers, int tp, size_t slot_vec) {
  // four vectors per thread and step: the loads are in flight together, the stores are posted
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i0 = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i0 < n_vec; i0 += 4 * stride) {
    uint4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (i0 + u * stride < n_vec) v[u] = __ldg(src + i0 + u * stride);
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (i0 + u * stride < n_vec)
        for (int r = 0; r < tp; ++r) reinterpret_cast<uint4 *>(peers.gather[r])[slot_vec + i0 + u * stride] = v[u];
  }
}

// The same push with the pre-MoE RMSNorm inside (moe_block of a TP group): block per row of the residual
// stream; t = w * (x / sqrt(mean(x^2) + 1e-5)) with the arithmetic of rmsnorm_rows_kernel (sum of squares in
// double, products in float, one bf16 rounding), so every rank's copy of a row equals the owner's own t bit
// for bit; the row goes straight into slot `rank` of every peer's gather buffer.  The normalised rows are
// never written and re-read locally for the exchange, and the push does not wait for the owner's own
// normalisation kernel (rmsnorm_kernel_bf16_io, kernels/rmsnorm.hpp:115-164, then ring_allgather_rows_bf16).
__global__ void __launch_bounds__(256)
tp_rmsnorm_push_kernel(const __nv_bfloat16 *__restrict__ x, const __nv_bfloat16 *__restrict__ w, int H, TpPeers peers,
                       int tp, size_t slot_row) {
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
  const size_t row_vec = (slot_row + blockIdx.x) * static_cast<size_t>(H / 8);
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
    const uint4 out = make_uint4(o[0], o[1], o[2], o[3]);
    for (int r = 0; r < tp; ++r) reinterpret_cast<uint4 *>(peers.gather[r])[row_vec + c] = out;
  }
}

// Tells every peer "my data of this phase and epoch is in place" and waits until every peer has said
// the same.  flags layout on each rank: [phase][tp] words, word [phase][r] written by rank r.
// One warp; lane r handles peer r.  The wait is bounded (about a second).
__global__ void tp_signal_wait_kernel(TpPeers peers, uint32_t *my_flags, int tp, int rank, int phase, uint32_t epoch,
                                      unsigned int *status) {
  const int r = threadIdx.x;
  __threadfence_system();
  if (r < tp) st_release_sys(peers.flags[r] + phase * kMaxTp + rank, epoch);
  if (r < tp) {
    const uint32_t *f = my_flags + phase * kMaxTp + r;
    const long long t0 = clock64();
    bool ok = false;
    for (uint32_t spin = 0;; ++spin) {
      // epochs only grow; signed difference tolerates wrap-around
      if (static_cast<int32_t>(ld_acquire_sys(f) - epoch) >= 0) { ok = true; break; }
      if ((spin & 255u) == 255u && clock64() - t0 > 2000000000LL) break;
    }
    if (!ok) atomicOr(status, ST_WAIT_PEER);
  }
  __threadfence_system();
}

// out[i] = bf16( sum over ranks r = 0..tp-1 of peer_partial[r][slot + i] ), fp32 adds in rank order.
__global__ void __launch_bounds__(256)
tp_reduce_scatter_pull_kernel(TpPeers peers, int tp, size_t slot_vec, size_t n_vec, uint4 *__restrict__ out) {
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n_vec; i += stride) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int r = 0; r < tp; ++r) {
      const uint4 v = reinterpret_cast<const uint4 *>(peers.partial[r])[slot_vec + i];
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        acc[2 * j] += __uint_as_float(w[j] << 16);
        acc[2 * j + 1] += __uint_as_float(w[j] & 0xffff0000u);
      }
    }
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const __nv_bfloat162 b = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
      o[j] = *reinterpret_cast<const uint32_t *>(&b);
    }
    out[i] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// out[i] = bf16( sum over slots s = 0..tp-1 of landing[s][i] ): the receive half of the reduce-scatter when
// every rank has pushed its partial rows into this rank's landing buffer (fp32 adds in rank order).
__global__ void __launch_bounds__(256)
tp_sum_slots_kernel(const uint4 *__restrict__ landing, int tp, size_t n_vec, uint4 *__restrict__ out,
                    const uint4 *__restrict__ residual) {
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n_vec; i += stride) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    if (residual != nullptr) {  // x += block output, folded into the same pass
      const uint4 v = residual[i];
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        acc[2 * j] = __uint_as_float(w[j] << 16);
        acc[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
      }
    }
    for (int r = 0; r < tp; ++r) {
      const uint4 v = landing[static_cast<size_t>(r) * n_vec + i];
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        acc[2 * j] += __uint_as_float(w[j] << 16);
        acc[2 * j + 1] += __uint_as_float(w[j] & 0xffff0000u);
      }
    }
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const __nv_bfloat162 b = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
      o[j] = *reinterpret_cast<const uint32_t *>(&b);
    }
    out[i] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

void launch_tp_sum_slots(const __nv_bfloat16 *landing, int tp, int rows_local, int H, __nv_bfloat16 *out, int sm_count,
                         cudaStream_t s, const __nv_bfloat16 *residual) {
  const size_t n_vec = static_cast<size_t>(rows_local) * H / 8;
  const int blocks = static_cast<int>(std::min<size_t>((n_vec + 255) / 256, static_cast<size_t>(sm_count) * 4));
  tp_sum_slots_kernel<<<std::max(blocks, 1), 256, 0, s>>>(reinterpret_cast<const uint4 *>(landing), tp, n_vec,
                                                          reinterpret_cast<uint4 *>(out),
                                                          reinterpret_cast<const uint4 *>(residual));
}

void launch_tp_allgather_push(const __nv_bfloat16 *src, int rows_local, int H, const TpPeers &peers, int tp, int rank,
                              cudaStream_t s, int row0, int n_rows) {
  // A few dozen blocks keep the links full (the stores are posted); the rest of the GPU stays free for the
  // kernels of the other stream that run beside the push.
  if (n_rows < 0) n_rows = rows_local - row0;
  if (n_rows <= 0) return;
  const size_t row_vec = static_cast<size_t>(H) / 8, n_vec = static_cast<size_t>(n_rows) * row_vec;
  const int blocks = static_cast<int>(std::min<size_t>((n_vec + 1023) / 1024, static_cast<size_t>(kPushBlocks)));
  tp_allgather_push_kernel<<<std::max(blocks, 1), 256, 0, s>>>(
      reinterpret_cast<const uint4 *>(src) + static_cast<size_t>(row0) * row_vec, n_vec, peers, tp,
      (static_cast<size_t>(rank) * rows_local + row0) * row_vec);
}

void launch_tp_rmsnorm_push(const __nv_bfloat16 *x, const __nv_bfloat16 *w, int rows_local, int H, const TpPeers &peers,
                            int tp, int rank, cudaStream_t s, int row0, int n_rows) {
  if (n_rows < 0) n_rows = rows_local - row0;
  if (n_rows <= 0) return;
  tp_rmsnorm_push_kernel<<<n_rows, 256, 0, s>>>(x + static_cast<size_t>(row0) * H, w, H, peers, tp,
                                                static_cast<size_t>(rank) * rows_local + row0);
}

void launch_tp_signal_wait(const TpPeers &peers, uint32_t *my_flags, int tp, int rank, int phase, uint32_t epoch,
                           unsigned int *status, cudaStream_t s) {
  tp_signal_wait_kernel<<<1, 32, 0, s>>>(peers, my_flags, tp, rank, phase, epoch, status);
}

void launch_tp_reduce_scatter_pull(const TpPeers &peers, int tp, int rank, int rows_local, int H, __nv_bfloat16 *out,
                                   int sm_count, cudaStream_t s) {
  const size_t n_vec = static_cast<size_t>(rows_local) * H / 8;
  const int blocks = static_cast<int>(std::min<size_t>((n_vec + 255) / 256, static_cast<size_t>(sm_count) * 4));
  tp_reduce_scatter_pull_kernel<<<std::max(blocks, 1), 256, 0, s>>>(peers, tp, static_cast<size_t>(rank) * n_vec, n_vec,
                                                                    reinterpret_cast<uint4 *>(out));
}

// All-reduce read half: out[i] = bf16( sum over ranks of peer_partial[r][i] ) for the first n_elems elements.
void launch_tp_sum_all(const TpPeers &peers, int tp, size_t n_elems, __nv_bfloat16 *out, int sm_count, cudaStream_t s) {
  const size_t n_vec = n_elems / 8;
  const int blocks = static_cast<int>(std::min<size_t>((n_vec + 255) / 256, static_cast<size_t>(sm_count) * 4));
  tp_reduce_scatter_pull_kernel<<<std::max(blocks, 1), 256, 0, s>>>(peers, tp, 0, n_vec, reinterpret_cast<uint4 *>(out));
}

}  // namespace moe
