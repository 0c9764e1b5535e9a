// Header-only C++ shim that gives libmoe_b200.so the names the reference runtime uses around its
// MoE block, so that forward_batch_gpu-style callers change types (hipStream_t -> cudaStream_t) and
// little else.  Each function cites the reference code it stands in for.  Single process, one host
// thread per GPU, as the reference runs (getp-csrc/getp_run.cpp:3514-3517).
#pragma once
#include <cuda_runtime.h>

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

// ring_allgather_rows_bf16 (getp-csrc/tp_ring.hpp:70-118): the gathered [TP*R_local, C] rows end up in
// the handle's gather buffer (moe_tp_buffer(h, MOE_TP_BUF_GATHER)); C must be the hidden size.
inline void ring_allgather_rows_bf16(const void *my_src, int R_local, const TPGroup &tp, cudaStream_t s) {
  moe_handle h = moe_b200_handles()[tp.world_rank];
  const int rc = moe_tp_allgather(h, my_src, R_local, s);
  if (rc != MOE_OK) moe_b200_die(h, "ring_allgather_rows_bf16", rc);
}
