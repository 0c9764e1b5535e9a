// Host side of the tensor-parallel entry points of include/moe_b200.h: symmetric buffer
// exchange (replaces tp_init / tp_enable_p2p, getp-csrc/nccl.hpp:41-98) and the launch
// sequence all-gather -> block -> reduce-scatter (moe_gpu_120b, getp_run.cpp:2958-3246).
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "moe_internal.cuh"

using namespace moe;

namespace {

int tp_fail(moe_ctx *c, int code, const char *fmt, ...) {
  char buf[400];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  c->err = buf;
  return code;
}

void **slot(moe_ctx *c, int which, int rank) {
  switch (which) {
    case MOE_TP_BUF_GATHER: return &c->peers.gather[rank];
    case MOE_TP_BUF_PARTIAL: return &c->peers.partial[rank];
    case MOE_TP_BUF_FLAGS: return reinterpret_cast<void **>(&c->peers.flags[rank]);
    case MOE_TP_BUF_TOPK_IDX: return &c->peers.topk_idx[rank];
    case MOE_TP_BUF_TOPK_W: return &c->peers.topk_w[rank];
    default: return nullptr;
  }
}

bool group_complete(const moe_ctx *c) {
  for (int r = 0; r < c->cfg.tp_size; ++r)
    for (int w = 0; w < kTpBufs; ++w)
      if (!(c->tp_attached & (1ull << (kTpBufs * r + w)))) return false;
  return true;
}

}  // namespace

namespace moe {
int check_tp_call(moe_ctx *c, int rows_local, const char *who) {
  if (c->cfg.tp_size > 1 && !group_complete(c))
    return tp_fail(c, MOE_ERR_STATE, "%s: not every peer buffer of the %d-rank group is attached", who, c->cfg.tp_size);
  if (rows_local <= 0 || static_cast<long long>(rows_local) * c->cfg.tp_size > c->max_rows)
    return tp_fail(c, MOE_ERR_INVALID, "%s: rows_local %d x tp %d exceeds max_rows %d", who, rows_local, c->cfg.tp_size,
                   c->max_rows);
  if (cudaSetDevice(c->cfg.device) != cudaSuccess) return tp_fail(c, MOE_ERR_CUDA, "%s: cudaSetDevice failed", who);
  return MOE_OK;
}
}  // namespace moe

extern "C" {

int moe_tp_buffer(moe_handle c, int which, void **dev_ptr) {
  if (!c || !dev_ptr) return MOE_ERR_INVALID;
  void **s = slot(c, which, c->cfg.tp_rank);
  if (!s) return tp_fail(c, MOE_ERR_INVALID, "moe_tp_buffer: unknown buffer %d", which);
  *dev_ptr = *s;
  return MOE_OK;
}

int moe_tp_export(moe_handle c, int which, void *handle_out) {
  if (!c || !handle_out) return MOE_ERR_INVALID;
  void **s = slot(c, which, c->cfg.tp_rank);
  if (!s) return tp_fail(c, MOE_ERR_INVALID, "moe_tp_export: unknown buffer %d", which);
  if (cudaSetDevice(c->cfg.device) != cudaSuccess) return tp_fail(c, MOE_ERR_CUDA, "moe_tp_export: cudaSetDevice failed");
  static_assert(sizeof(cudaIpcMemHandle_t) == MOE_TP_HANDLE_BYTES, "handle size");
  cudaError_t e = cudaIpcGetMemHandle(static_cast<cudaIpcMemHandle_t *>(handle_out), *s);
  if (e != cudaSuccess) return tp_fail(c, MOE_ERR_CUDA, "cudaIpcGetMemHandle: %s", cudaGetErrorString(e));
  return MOE_OK;
}

int moe_tp_attach_ipc(moe_handle c, int which, int rank, const void *handle_in) {
  if (!c || !handle_in) return MOE_ERR_INVALID;
  if (rank < 0 || rank >= c->cfg.tp_size || !slot(c, which, 0))
    return tp_fail(c, MOE_ERR_INVALID, "moe_tp_attach_ipc: rank %d / buffer %d out of range", rank, which);
  if (rank == c->cfg.tp_rank) return MOE_OK;  // own buffers are known since creation
  if (cudaSetDevice(c->cfg.device) != cudaSuccess) return tp_fail(c, MOE_ERR_CUDA, "moe_tp_attach_ipc: cudaSetDevice failed");
  void *p = nullptr;
  cudaIpcMemHandle_t hd;
  memcpy(&hd, handle_in, sizeof(hd));
  cudaError_t e = cudaIpcOpenMemHandle(&p, hd, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return tp_fail(c, MOE_ERR_CUDA, "cudaIpcOpenMemHandle(rank %d): %s", rank, cudaGetErrorString(e));
  c->ipc_opened.push_back(p);
  *slot(c, which, rank) = p;
  c->tp_attached |= 1ull << (kTpBufs * rank + which);
  return MOE_OK;
}

int moe_tp_attach_ptr(moe_handle c, int which, int rank, void *dev_ptr, int peer_device) {
  if (!c || !dev_ptr) return MOE_ERR_INVALID;
  if (rank < 0 || rank >= c->cfg.tp_size || !slot(c, which, 0))
    return tp_fail(c, MOE_ERR_INVALID, "moe_tp_attach_ptr: rank %d / buffer %d out of range", rank, which);
  if (rank == c->cfg.tp_rank) return MOE_OK;
  if (cudaSetDevice(c->cfg.device) != cudaSuccess) return tp_fail(c, MOE_ERR_CUDA, "moe_tp_attach_ptr: cudaSetDevice failed");
  if (peer_device != c->cfg.device) {
    int can = 0;
    cudaDeviceCanAccessPeer(&can, c->cfg.device, peer_device);
    if (!can) return tp_fail(c, MOE_ERR_CUDA, "device %d cannot access device %d", c->cfg.device, peer_device);
    cudaError_t e = cudaDeviceEnablePeerAccess(peer_device, 0);
    if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled)
      return tp_fail(c, MOE_ERR_CUDA, "cudaDeviceEnablePeerAccess(%d): %s", peer_device, cudaGetErrorString(e));
    cudaGetLastError();
  }
  *slot(c, which, rank) = dev_ptr;
  c->tp_attached |= 1ull << (kTpBufs * rank + which);
  return MOE_OK;
}

int moe_tp_allgather(moe_handle c, const void *src, int rows_local, void *stream) {
  if (!c || !src) return MOE_ERR_INVALID;
  int rc = check_tp_call(c, rows_local, "moe_tp_allgather");
  if (rc != MOE_OK) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int tp = c->cfg.tp_size, rank = c->cfg.tp_rank;
  ++c->tp_epoch;
  launch_tp_allgather_push(static_cast<const __nv_bfloat16 *>(src), rows_local, c->H, c->peers, tp, rank, s);
  launch_tp_signal_wait(c->peers, c->tp_flags, tp, rank, kTpPhaseGather, c->tp_epoch, c->status, s);
  c->launches += 2;
  if (cudaGetLastError() != cudaSuccess) return tp_fail(c, MOE_ERR_CUDA, "moe_tp_allgather: launch failed");
  return MOE_OK;
}

int moe_tp_reduce_scatter(moe_handle c, int rows_local, void *out_local, void *stream) {
  if (!c || !out_local) return MOE_ERR_INVALID;
  int rc = check_tp_call(c, rows_local, "moe_tp_reduce_scatter");
  if (rc != MOE_OK) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int tp = c->cfg.tp_size, rank = c->cfg.tp_rank;
  ++c->tp_epoch_rs;  // every rank calls in lock-step, so the counters agree across the group
  launch_tp_signal_wait(c->peers, c->tp_flags, tp, rank, kTpPhaseScatter, c->tp_epoch_rs, c->status, s);
  launch_tp_reduce_scatter_pull(c->peers, tp, rank, rows_local, c->H, static_cast<__nv_bfloat16 *>(out_local),
                                c->sm_count, s);
  c->launches += 2;
  if (cudaGetLastError() != cudaSuccess) return tp_fail(c, MOE_ERR_CUDA, "moe_tp_reduce_scatter: launch failed");
  return MOE_OK;
}

int moe_tp_allreduce(moe_handle c, void *buf_dev, size_t n_elems, void *stream) {
  if (!c || !buf_dev) return MOE_ERR_INVALID;
  if (n_elems == 0) return MOE_OK;
  if (n_elems % 8 != 0 || n_elems > static_cast<size_t>(c->max_rows) * c->H)
    return tp_fail(c, MOE_ERR_INVALID, "moe_tp_allreduce: %zu elements (must be a multiple of 8 and at most max_rows * H = %zu)",
                   n_elems, static_cast<size_t>(c->max_rows) * c->H);
  int rc = check_tp_call(c, 1, "moe_tp_allreduce");
  if (rc != MOE_OK) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int tp = c->cfg.tp_size, rank = c->cfg.tp_rank;
  // 1. every rank has finished reading the partial buffers of the previous collective; 2. this rank's values are
  // in its partial buffer; 3. every rank's values are in place; 4. sum all ranks' buffers in rank order.
  ++c->tp_epoch;
  launch_tp_signal_wait(c->peers, c->tp_flags, tp, rank, kTpPhaseGather, c->tp_epoch, c->status, s);
  if (cudaMemcpyAsync(c->tp_partial, buf_dev, n_elems * 2, cudaMemcpyDeviceToDevice, s) != cudaSuccess)
    return tp_fail(c, MOE_ERR_CUDA, "moe_tp_allreduce: staging copy failed");
  ++c->tp_epoch_rs;
  launch_tp_signal_wait(c->peers, c->tp_flags, tp, rank, kTpPhaseScatter, c->tp_epoch_rs, c->status, s);
  launch_tp_sum_all(c->peers, tp, n_elems, static_cast<__nv_bfloat16 *>(buf_dev), c->sm_count, s);
  c->launches += 3;
  if (cudaGetLastError() != cudaSuccess) return tp_fail(c, MOE_ERR_CUDA, "moe_tp_allreduce: launch failed");
  return MOE_OK;
}

int moe_tp_forward(moe_handle c, int layer, const void *t_local, int rows_local, void *out_local, unsigned flags,
                   void *stream) {
  if (!c || !t_local || !out_local) return MOE_ERR_INVALID;
  int rc = check_tp_call(c, rows_local, "moe_tp_forward");
  if (rc != MOE_OK) return rc;
  return forward_impl(c, layer, static_cast<const __nv_bfloat16 *>(c->peers.gather[c->cfg.tp_rank]),
                      rows_local * c->cfg.tp_size, static_cast<__nv_bfloat16 *>(out_local),
                      flags & ~MOE_FWD_PARTIAL_F32, static_cast<cudaStream_t>(stream),
                      static_cast<const __nv_bfloat16 *>(t_local), rows_local);
}

int moe_block(moe_handle c, int layer, void *x_dev, const void *rms_w_dev, int rows_local, unsigned flags, void *stream) {
  if (!c || !x_dev || !rms_w_dev) return MOE_ERR_INVALID;
  int rc = check_tp_call(c, rows_local, "moe_block");
  if (rc != MOE_OK) return rc;
  const int tp = c->cfg.tp_size;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  __nv_bfloat16 *x = static_cast<__nv_bfloat16 *>(x_dev);
  // step 0 (t = rmsnorm(x) * w) runs inside: on one GPU as a kernel of its own, in a TP group inside the
  // all-gather push; the last kernel of the block adds its result to x in place
  flags &= ~MOE_FWD_PARTIAL_F32;
  const __nv_bfloat16 *gain = static_cast<const __nv_bfloat16 *>(rms_w_dev);
  if (tp > 1)
    return forward_impl(c, layer, static_cast<const __nv_bfloat16 *>(c->peers.gather[c->cfg.tp_rank]), rows_local * tp, x,
                        flags, s, x, rows_local, x, nullptr, gain);
  return forward_impl(c, layer, x, rows_local, x, flags, s, nullptr, 0, x, nullptr, gain);
}

int moe_tp_forward_host(moe_handle c, int layer, const void *t_local_host, int rows_local, void *out_local_host,
                        unsigned flags) {
  if (!c || !t_local_host || !out_local_host) return MOE_ERR_INVALID;
  int rc = check_tp_call(c, rows_local, "moe_tp_forward_host");
  if (rc != MOE_OK) return rc;
  const size_t bytes = static_cast<size_t>(rows_local) * c->H * 2;
  // staging: the fp32 debug buffer is unused on this path and large enough ([max_rows, H] fp32)
  __nv_bfloat16 *in_dev = reinterpret_cast<__nv_bfloat16 *>(c->out_f32);
  __nv_bfloat16 *out_dev = c->out_bf16;
  if (cudaMemcpyAsync(in_dev, t_local_host, bytes, cudaMemcpyHostToDevice, c->stream) != cudaSuccess)
    return tp_fail(c, MOE_ERR_CUDA, "moe_tp_forward_host: host-to-device copy failed");
  rc = moe_tp_forward(c, layer, in_dev, rows_local, out_dev, flags & ~MOE_FWD_PARTIAL_F32, c->stream);
  if (rc != MOE_OK) return rc;
  if (cudaMemcpyAsync(out_local_host, out_dev, bytes, cudaMemcpyDeviceToHost, c->stream) != cudaSuccess ||
      cudaStreamSynchronize(c->stream) != cudaSuccess)
    return tp_fail(c, MOE_ERR_CUDA, "moe_tp_forward_host: device-to-host copy failed: %s", cudaGetErrorString(cudaGetLastError()));
  unsigned st = 0;
  cudaMemcpy(&st, c->status, sizeof(st), cudaMemcpyDeviceToHost);
  if (st) {
    cudaMemset(c->status, 0, sizeof(unsigned));
    return tp_fail(c, status_error(st), "device status word 0x%x", st);
  }
  return MOE_OK;
}

}  // extern "C"
