// Header-only C++ shim that gives libmoe_b200.so the names the reference runtime uses around its
// MoE block, so that forward_batch_gpu-style callers change types (hipStream_t -> cudaStream_t) and
// little else.  Each function cites the reference code it stands in for.  Single process, one host
// thread per GPU, as the reference runs (getp-csrc/getp_run.cpp:3514-3517).
#pragma once
#include <cuda_runtime.h>

#include <atomic>
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstdlib>

#include "moe_b200.h"

#ifndef MAX_TP
#define MAX_TP 8  // getp-csrc/nccl.hpp:6
#endif
#ifndef MAX_GPUS
#define MAX_GPUS 8  // getp-csrc/config.hpp:9
#endif

// getp-csrc/nccl.hpp:25-38, minus the helper stream (the library owns its streams).
struct TPGroup {
  int world_size{1};
  int tp_size{1};
  int world_rank{0};
  int group_id{0};
  int rank_in_group{0};
  int group_devs[MAX_TP]{};
};

// getp-csrc/nccl.hpp:73-90: contiguous partition of the devices into TP groups.
inline void tp_init(TPGroup &tp, int world_size, int world_rank, int tp_size) {
  tp.world_size = world_size;
  tp.world_rank = world_rank;
  tp.tp_size = tp_size <= 0 ? 1 : tp_size;
  tp.group_id = world_rank / tp.tp_size;
  tp.rank_in_group = world_rank % tp.tp_size;
  for (int i = 0; i < tp.tp_size; ++i) tp.group_devs[i] = tp.group_id * tp.tp_size + i;
}
inline void tp_free(TPGroup &) {}  // getp-csrc/nccl.hpp:92-98: nothing to release here

// getp-csrc/getp_run.cpp:2488-2501: the same even split.  The library never re-quantises a shard (the
// reference does): MLP2 keeps the whole scale blocks around its shard.
inline void mlp2_shard_input(int D, int tp_size, int r, int &i_start, int &i_len) {
  if (moe_shard_range(D, tp_size, r, &i_start, &i_len) != MOE_OK) { i_start = 0; i_len = 0; }
}
inline void mlp1_shard(int twoD, int tp_size, int r, int &o_start, int &o_len) {
  int s = 0, n = 0;
  mlp2_shard_input(twoD / 2, tp_size, r, s, n);
  o_start = 2 * s;  // gate/up rows stay adjacent
  o_len = 2 * n;
}

// The per-device handles the reference keeps in gpu_transformers[] (getp_run.cpp:215).
inline moe_handle *moe_b200_handles() {
  static moe_handle h[MAX_GPUS] = {};
  return h;
}

inline void moe_b200_die(moe_handle h, const char *what, int rc) {  // HIP_CHECK semantics, nccl.hpp:11-19
  fprintf(stderr, "%s: %s (%s)\n", what, moe_strerror(rc), h ? moe_last_error(h) : "");
  abort();
}

// After every device of a group has created its handle: what tp_enable_p2p (nccl.hpp:41-70) plus the
// reference's reads of gpu_transformers[peer]->state.* amount to.
inline void moe_b200_connect_group(const TPGroup &tp) {
  moe_handle *hs = moe_b200_handles();
  moe_handle me = hs[tp.world_rank];
  for (int r = 0; r < tp.tp_size; ++r) {
    if (r == tp.rank_in_group) continue;
    const int dev = tp.group_devs[r];
    for (int which = 0; which < MOE_TP_N_BUFS; ++which) {
      void *p = nullptr;
      int rc = moe_tp_buffer(hs[dev], which, &p);
      if (rc == MOE_OK) rc = moe_tp_attach_ptr(me, which, r, p, dev);
      if (rc != MOE_OK) moe_b200_die(me, "moe_b200_connect_group", rc);
    }
  }
}

// moe_gpu / moe_gpu_120b (getp_run.cpp:2540, :2896) from step 1 on: `t_rows` are this device's
// RMS-normalised rows (state.t + row_offset*H), `out_rows` receives the block output of the same rows
// (what the reference then adds into state.x, other_kernels.hpp:18-37).  Every device of the group
// calls it from its own host thread; nothing here blocks the host.
inline void moe_gpu_b200(const TPGroup &tp, int layer_idx, const void *t_rows, int batch_size, void *out_rows,
                         cudaStream_t sMoe) {
  if (batch_size <= 0) return;
  moe_handle h = moe_b200_handles()[tp.world_rank];
  const int rc = tp.tp_size > 1 ? moe_tp_forward(h, layer_idx, t_rows, batch_size, out_rows, 0, sMoe)
                                : moe_forward(h, layer_idx, t_rows, batch_size, out_rows, 0, sMoe);
  if (rc != MOE_OK) moe_b200_die(h, "moe_gpu_b200", rc);
}

// moe_gpu / moe_gpu_120b as a whole, steps 0-10: `x_rows` are this device's rows of the residual stream
// (state.x + row_offset*H), normalised with `rms_ffn_w` (the layer's gain, bf16 [H]), run through the block
// and the group's exchange, and updated in place.
inline void moe_gpu_b200_block(const TPGroup &tp, int layer_idx, void *x_rows, const void *rms_ffn_w, int batch_size,
                               cudaStream_t sMoe) {
  if (batch_size <= 0) return;
  moe_handle h = moe_b200_handles()[tp.world_rank];
  const int rc = moe_block(h, layer_idx, x_rows, rms_ffn_w, batch_size, 0, sMoe);
  if (rc != MOE_OK) moe_b200_die(h, "moe_gpu_b200_block", rc);
}

// ring_allgather_rows_bf16 (getp-csrc/tp_ring.hpp:70-118), the reference's full signature.  Every rank's
// [R_local, C] rows end up, in rank order, in `my_dst` ([TP*R_local, C]).  The library gathers by peer stores
// into the handle's own symmetric buffer (moe_tp_buffer(h, MOE_TP_BUF_GATHER)); when `my_dst` is another
// buffer the rows are copied there on the same stream.  `peer_dst_bases` is what the reference's ring writes
// into on the other ranks; here every rank fills its own destination, so the argument is accepted and not
// used.  C must be the hidden size the handle was created with.
inline void ring_allgather_rows_bf16(void *my_dst, const void *my_src, int R_local, int C, void *const peer_dst_bases[],
                                     const TPGroup &tp, cudaStream_t s) {
  (void)peer_dst_bases;
  if (R_local == 0 || C == 0 || tp.tp_size <= 0) return;
  moe_handle h = moe_b200_handles()[tp.world_rank];
  int rc = moe_tp_allgather(h, my_src, R_local, s);
  if (rc != MOE_OK) moe_b200_die(h, "ring_allgather_rows_bf16", rc);
  void *gathered = nullptr;
  rc = moe_tp_buffer(h, MOE_TP_BUF_GATHER, &gathered);
  if (rc != MOE_OK) moe_b200_die(h, "ring_allgather_rows_bf16", rc);
  if (my_dst != nullptr && my_dst != gathered &&
      cudaMemcpyAsync(my_dst, gathered, static_cast<size_t>(tp.tp_size) * R_local * C * 2, cudaMemcpyDeviceToDevice, s) != cudaSuccess)
    moe_b200_die(h, "ring_allgather_rows_bf16: copy to my_dst", MOE_ERR_CUDA);
}

// ring_allreduce_sum_bf16 (getp-csrc/tp_ring.hpp:253-331): after the call buf_local holds the element-wise
// sum over the ranks of the group.  peer_bases and d_recv (the reference's peer pointers and receive tile) are
// accepted and not used: the values travel through the handle's symmetric partial-output buffer.
inline void ring_allreduce_sum_bf16(void *buf_local, void *const peer_bases[], size_t N_elems, void *d_recv,
                                    const TPGroup &tp, cudaStream_t s) {
  (void)peer_bases;
  (void)d_recv;
  if (tp.tp_size <= 1 || N_elems == 0) return;
  moe_handle h = moe_b200_handles()[tp.world_rank];
  const int rc = moe_tp_allreduce(h, buf_local, N_elems, s);
  if (rc != MOE_OK) moe_b200_die(h, "ring_allreduce_sum_bf16", rc);
}

// tp_group_barrier (getp-csrc/nccl.hpp:100-137): host barrier of the threads that drive one TP group.  The
// library's own calls need none (peers meet through device-side epoch flags); it is kept for callers that
// synchronise their threads around other work.  Unlike the reference's, the wait is bounded: a group that does
// not complete within 30 s aborts with a message instead of spinning forever.
#ifndef MAX_TP_GROUPS
#define MAX_TP_GROUPS 8
#endif
struct TPBarrierState {
  std::atomic<int> count[MAX_TP_GROUPS];
  std::atomic<uint64_t> epoch[MAX_TP_GROUPS];
  TPBarrierState() {
    for (int i = 0; i < MAX_TP_GROUPS; ++i) { count[i].store(0); epoch[i].store(0); }
  }
};
inline TPBarrierState &tp_barrier_state() {
  static TPBarrierState st;
  return st;
}
inline void tp_group_barrier(const TPGroup &tp) {
  TPBarrierState &st = tp_barrier_state();
  const int gid = tp.group_id % MAX_TP_GROUPS;
  const uint64_t seen = st.epoch[gid].load(std::memory_order_acquire);
  if (st.count[gid].fetch_add(1, std::memory_order_acq_rel) + 1 == tp.tp_size) {
    st.count[gid].store(0, std::memory_order_release);
    st.epoch[gid].fetch_add(1, std::memory_order_acq_rel);
    return;
  }
  const auto t0 = std::chrono::steady_clock::now();
  for (unsigned spin = 0; st.epoch[gid].load(std::memory_order_acquire) == seen; ++spin) {
    if ((spin & 0xffffu) == 0xffffu && std::chrono::steady_clock::now() - t0 > std::chrono::seconds(30)) {
      fprintf(stderr, "tp_group_barrier: group %d did not complete within 30 s\n", tp.group_id);
      abort();
    }
  }
}

// The part of the reference's per-device model state that its MoE call reads (GPUTransformer,
// getp_run.cpp:206-212, with the same field names), so that forward_batch_gpu-style callers compile against
// moe_gpu / moe_gpu_120b unchanged.  A caller that keeps the reference's own, larger structs defines
// MOE_B200_SHIM_NO_TYPES and uses moe_gpu_b200_block() directly.
#ifndef MOE_B200_SHIM_NO_TYPES
struct Config {              // run.cpp:25-45 (the fields the MoE block reads)
  int hidden_dim;
  int intermediate_dim;
  int n_experts;
  int experts_per_token;
  int n_layers;
  float swiglu_limit;
};
struct GPUTransformerWeights {  // getp_run.cpp:48-81
  void *rms_ffn_w;              // bf16 [n_layers, hidden_dim]
};
struct GPURunState {            // getp_run.cpp:84-176
  void *x;                      // bf16 [batch, hidden_dim], the residual stream
  void *t;                      // bf16 [batch, hidden_dim], normalised rows (not written here: the library keeps its own)
};
struct GPUTransformer {         // getp_run.cpp:206-212
  Config config;
  GPUTransformerWeights weights;
  GPURunState state;
};
inline TPGroup *tp_groups() {   // getp_run.cpp:216
  static TPGroup g[MAX_GPUS];
  return g;
}

// moe_gpu_120b / moe_gpu (getp_run.cpp:2896, :2540) with the reference's signature and contract: reads the rows
// state.x[row_offset .. row_offset + batch_size) of the residual stream and weights.rms_ffn_w of the layer, and
// adds the MoE output into state.x in place; called by the host thread of the current device, concurrently by
// the threads of a TP group.  The per-device handle and group are found through moe_b200_handles() and
// tp_groups(), indexed by the current device as the reference indexes gpu_transformers[] and tp_groups[].
inline void moe_gpu_120b(GPUTransformer *gpu_t, int layer_idx, int batch_size, int row_offset, cudaStream_t sMoe) {
  if (batch_size <= 0) return;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) moe_b200_die(nullptr, "moe_gpu_120b: cudaGetDevice", MOE_ERR_CUDA);
  const size_t H = static_cast<size_t>(gpu_t->config.hidden_dim);
  char *x = static_cast<char *>(gpu_t->state.x) + static_cast<size_t>(row_offset) * H * 2;
  const char *gain = static_cast<const char *>(gpu_t->weights.rms_ffn_w) + static_cast<size_t>(layer_idx) * H * 2;
  moe_gpu_b200_block(tp_groups()[dev], layer_idx, x, gain, batch_size, sMoe);
}
inline void moe_gpu(GPUTransformer *gpu_t, int layer_idx, int batch_size, int row_offset, cudaStream_t sMoe) {
  moe_gpu_120b(gpu_t, layer_idx, batch_size, row_offset, sMoe);   // one code path serves both model sizes
}
#endif  // MOE_B200_SHIM_NO_TYPES
