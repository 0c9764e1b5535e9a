/*
 * C ABI of the B200 (sm_100a) tensor-parallel MXFP4 MoE block.
 *
 * This is the drop-in boundary for the MoE path of the reference runtime
 * (getp-csrc/getp_run.cpp): the reference has no FFI layer, its boundary is the
 * C++ call moe_gpu()/moe_gpu_120b() plus the weight loaders and the TP helpers.
 * Each entry point below names the reference interface it replaces.  Plain
 * pointers and sizes only; every function returns a status code (the reference
 * prints and abort()s, getp-csrc/nccl.hpp:11-19) and never exits the process.
 *
 * Threading model as in the reference (getp_run.cpp:3514-3517): one host thread
 * (or one process) per GPU; a handle is bound to one device and is used by one
 * thread at a time.
 */
#ifndef MOE_B200_H
#define MOE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct moe_ctx *moe_handle;

enum {
  MOE_OK = 0,
  MOE_ERR_INVALID = 1,     /* bad argument or unsupported shape */
  MOE_ERR_CUDA = 2,        /* a CUDA call failed; see moe_last_error() */
  MOE_ERR_NOMEM = 3,
  MOE_ERR_TIMEOUT = 4,     /* a bounded device- or host-side wait ran out */
  MOE_ERR_SCALE_RANGE = 5, /* an E8M0 weight scale byte is 0xFF (NaN) */
  MOE_ERR_STATE = 6,       /* layer not loaded, peers not attached, ... */
  MOE_ERR_NO_SM100 = 7,    /* device is not compute capability 10.x */
  MOE_ERR_Y_RANGE = 8      /* an MLP2 output exceeded 65504 in magnitude (it is kept in fp16 until the combine) */
};

/* moe_config.flags */
#define MOE_CFG_KEEP_F32_OUT 1u /* also keep the fp32 block output for moe_get_debug() */

/* Replaces Config (run.cpp:25-45, the fields the MoE block reads) plus the
 * globals BATCH_SIZE / TENSOR_PARALLEL_SIZE (getp-csrc/config.hpp:3,11). */
typedef struct moe_config {
  int hidden_dim;        /* H, multiple of 32 */
  int intermediate_dim;  /* D, multiple of 32 */
  int n_experts;         /* E <= 256 */
  int experts_per_token; /* K <= 8 */
  int n_layers;
  float swiglu_limit;    /* 7.0 */
  float swiglu_alpha;    /* 1.702 */
  int max_rows;          /* most rows one forward sees (the TP group's union batch) */
  int tp_size;           /* ranks sharing the intermediate dimension; 1 = no TP */
  int tp_rank;           /* rank_in_group (getp-csrc/nccl.hpp:30) */
  int device;            /* CUDA ordinal this handle is bound to */
  unsigned flags;        /* MOE_CFG_* */
} moe_config;

/* Replaces malloc_gpu_run_state* and malloc_gpu_weights_{20b,120b}
 * (getp_run.cpp:588, :656): allocates every device buffer the block needs. */
int moe_create(const moe_config *cfg, moe_handle *out);
int moe_destroy(moe_handle h);

/* Replaces copy_weights_to_gpu_{20b,120b} for the MoE tensors
 * (getp_run.cpp:744, :1480).  HOST pointers to one layer's FULL tensors in the
 * reference layout (GPUTransformerWeights, getp_run.cpp:48-81):
 *   w1_codes  [E, 2D, H/2] u8, two e2m1 codes per byte, low nibble = even element
 *   w1_scales [E, 2D, H/32] u8 E8M0, one per 32 elements along H
 *   b1        [E, 2D] bf16            (rows 2j = gate_j, 2j+1 = up_j)
 *   w2_codes  [E, H, D/2], w2_scales [E, H, D/32], b2 [E, H] bf16
 *   router_w  [E, H] fp32, router_b [E] fp32
 * With tp_size > 1 the rank's shard (mlp1_shard / mlp2_shard_input,
 * getp_run.cpp:2488-2501) is cut out inside.  Nothing is re-quantised: where a
 * shard boundary falls inside a 32-element scale block, MLP2 keeps the whole
 * blocks around its shard and the activations outside the shard are zero. */
int moe_load_layer(moe_handle h, int layer, const uint8_t *w1_codes, const uint8_t *w1_scales,
                   const uint16_t *b1, const uint8_t *w2_codes, const uint8_t *w2_scales,
                   const uint16_t *b2, const float *router_w, const float *router_b);

/* The intermediate range [start, start+len) a rank owns: the even split of
 * mlp2_shard_input (getp_run.cpp:2495-2501) when D / tp_size is a whole multiple
 * of 8, otherwise whole 32-element blocks dealt out as evenly as possible. */
int moe_shard_range(int intermediate_dim, int tp_size, int tp_rank, int *start, int *len);

/* moe_forward.flags */
#define MOE_FWD_SIMT_GEMM 1u    /* run the plain CUDA-core validation GEMM (fp16 operands) instead of tcgen05 */
#define MOE_FWD_PARTIAL_F32 2u  /* TP: leave this rank's fp32 partial in the handle, write no output */
#define MOE_FWD_SPLIT_ROUTER 4u /* route with the two-launch form (split-k partial sums, then top-k) that layers of more
                                   than 128 experts always take, instead of the fused cluster kernel */
#define MOE_FWD_SPLIT_MLP 8u    /* MLP1 and MLP2 as two launches of the expert GEMM kernel instead of one */

/* Replaces moe_gpu()/moe_gpu_120b() steps 2-8 (getp_run.cpp:2540, :2896): router,
 * top-k + softmax, permutation, MLP1 + SwiGLU, MLP2, weighted combine, for `rows`
 * already-normalised bf16 rows [rows, H] in DEVICE memory; writes bf16 [rows, H].
 * Stream-ordered on `stream` (a cudaStream_t); no host synchronisation inside. */
int moe_forward(moe_handle h, int layer, const void *t_dev, int rows, void *out_dev, unsigned flags,
                void *stream);

/* fp32 -> MXFP4 on the device: replaces a launch of quantize_pack_mxfp4_block32_kernel
 * (getp-csrc/memory/mxfp4.hpp:139-217; launched at getp_run.cpp:1210, :1433).  Per 32 consecutive
 * elements one E8M0 byte (ilogb of the block maximum minus 2, plus 127) and 16 bytes of e2m1 codes
 * (low nibble = even element), bit-identical to the reference's.  codes_dev: ceil(n/32)*16 bytes,
 * scales_dev: ceil(n/32) bytes; elements past n count as 0; codes_dev must be 4-byte aligned.
 * Stream-ordered on the current device, no handle needed. */
int moe_quantize_mxfp4(const float *src_dev, size_t n_elems, uint8_t *codes_dev, uint8_t *scales_dev,
                       void *stream);

/* moe_load_layer for an fp32 checkpoint (layout of run.cpp:206-247: w_mlp1 [E, 2D, H], b_mlp1 [E, 2D],
 * w_mlp2 [E, H, D], b_mlp2 [E, H], all fp32, host pointers to the layer's tensors): replaces
 * streaming_quantize_copy_mxfp4_cpu_to_gpu (getp_run.cpp:1104-1245) and the MoE part of
 * copy_weights_to_gpu_120b (:1480-1718).  The expert weights are quantised on the GPU in chunks
 * and the biases rounded to bf16, then loaded as by moe_load_layer.  The whole tensors are
 * quantised before the TP shard is cut; the reference quantises each shard, which gives different
 * MXFP4 blocks where a shard of the intermediate dimension does not start on a multiple of 32. */
int moe_load_layer_f32(moe_handle h, int layer, const float *w1, const float *b1, const float *w2,
                       const float *b2, const float *router_w, const float *router_b);

/* moe_load_layer_f32 straight from a checkpoint file in the reference's flat fp32 layout: the Config header
 * (run.cpp:25-45) followed by the tensors in the order of memory_map_weights (run.cpp:206-247), as
 * export_model_bin/gpt-oss-120b/export_model_bin.py writes it and load_checkpoint (run.cpp:249-293) maps it.
 * The MoE tensors of layer `file_layer` of the file become layer `layer` of the handle; the header's hidden,
 * expert, intermediate and top-k sizes and swiglu_limit must be the handle's.  rms_ffn_w_out (fp32 [H], may be
 * NULL) receives the layer's pre-MoE RMSNorm gain, which moe_block() takes as bf16.  The file is mapped
 * read-only for the duration of the call. */
int moe_load_layer_from_bin(moe_handle h, int layer, const char *path, int file_layer, float *rms_ffn_w_out);
/* Where the MoE tensors of one layer start in such a file, in floats from the start of the file, from the
 * fifteen 4-byte header fields alone (host arithmetic, no device): the order of memory_map_weights. */
enum {
  MOE_BIN_RMS_FFN_W = 0, MOE_BIN_ROUTER_W = 1, MOE_BIN_ROUTER_B = 2, MOE_BIN_W_MLP1 = 3, MOE_BIN_B_MLP1 = 4,
  MOE_BIN_W_MLP2 = 5, MOE_BIN_B_MLP2 = 6, MOE_BIN_N_TENSORS = 7
};
int moe_bin_layer_offsets(const int32_t *header, int layer, long long offsets[MOE_BIN_N_TENSORS], long long *total_floats);

/* Replaces moe_gpu()/moe_gpu_120b() as a whole (getp_run.cpp:2540, :2896), steps 0-10: the residual
 * stream rows x_dev (bf16 [rows_local, H], this rank's rows) are RMS-normalised with the bf16 gain
 * rms_w_dev [H] (rmsnorm_kernel_bf16_io, kernels/rmsnorm.hpp:115-164), go through the block (through
 * the tensor-parallel exchange when tp_size > 1; every rank of the group calls), and receive the
 * result in place: x += MoE(rmsnorm(x)) (accumulate_kernel_bf16, kernels/other_kernels.hpp:18-37). */
int moe_block(moe_handle h, int layer, void *x_dev, const void *rms_w_dev, int rows_local, unsigned flags,
              void *stream);

/* Same call for HOST buffers (pinned memory from moe_host_alloc copies
 * asynchronously): host->device copy, the block, device->host copy, then waits
 * and returns the device status. */
int moe_forward_host(moe_handle h, int layer, const void *t_host, int rows, void *out_host, unsigned flags);

/* The same call split in two so that the copies of one batch overlap the block of another: submit
 * returns at once with a ticket; wait blocks until that batch's result is in out_host.  Up to three
 * batches may be in flight (a fourth submit fails with MOE_ERR_STATE until the oldest was waited for);
 * both host buffers must stay valid, and should be pinned (moe_host_alloc), until the wait returns.
 * With tp_size > 1 the rows are this rank's rows and every rank of the group submits its batches in
 * the same order (the call is then moe_tp_forward_host split in two).
 * The reference has no counterpart: its forward_batch_gpu (getp_run.cpp:3254) copies tokens in, runs
 * and copies logits out on one stream, blocking the host thread. */
int moe_forward_host_submit(moe_handle h, int layer, const void *t_host, int rows, void *out_host,
                            unsigned flags, long long *ticket);
int moe_forward_host_wait(moe_handle h, long long ticket);

/* Waits for the handle's stream work and reports MOE_ERR_TIMEOUT if any kernel
 * recorded a bounded wait that ran out. */
int moe_synchronize(moe_handle h);

void *moe_host_alloc(size_t bytes);
void moe_host_free(void *p);

/* Stand-alone top-k + softmax over caller-supplied fp32 logits [rows, E] (device
 * pointers).  Replaces run_route_select_softmax_fused (kernels/moe.hpp:565-599). */
int moe_route_topk(moe_handle h, const float *logits_dev, int rows, int *idx_dev, float *w_dev, void *stream);

/* ---- tensor-parallel group (replaces TPGroup / tp_init / tp_enable_p2p, getp-csrc/nccl.hpp:25-98, and
 * the raw peer pointers the reference reads through gpu_transformers[], getp_run.cpp:2594,:2965,:3221).
 * A handle created with tp_size > 1 owns MOE_TP_N_BUFS symmetric buffers; every rank must learn every peer's. */
enum {
  MOE_TP_BUF_GATHER = 0,  /* bf16 [max_rows, H]  all-gather destination        (gather_x_g) */
  MOE_TP_BUF_PARTIAL = 1, /* bf16 [max_rows, H]  this rank's partial output    (e_agg_g)    */
  MOE_TP_BUF_FLAGS = 2,   /* u32  [3][8]         arrival epochs written by the peers        */
  MOE_TP_BUF_TOPK_IDX = 3,/* i32  [max_rows, K]  expert choice of every row of the union    (topk_i_g)  */
  MOE_TP_BUF_TOPK_W = 4,  /* f32  [max_rows, K]  routing weights of every row of the union  (topk_v_g)  */
  MOE_TP_N_BUFS = 5
};
#define MOE_TP_HANDLE_BYTES 64 /* sizeof(cudaIpcMemHandle_t) */
/* Ranks in different processes: export, exchange the 64 bytes by any channel, attach. */
int moe_tp_export(moe_handle h, int which, void *handle_out);
int moe_tp_attach_ipc(moe_handle h, int which, int rank, const void *handle_in);
/* Ranks in one process (one host thread per GPU, as the reference runs): pass the raw pointer. */
int moe_tp_buffer(moe_handle h, int which, void **dev_ptr);
int moe_tp_attach_ptr(moe_handle h, int which, int rank, void *dev_ptr, int peer_device);

/* Replaces moe_gpu_120b steps 1-9 (getp_run.cpp:2958-3246): all-gather of every rank's `rows_local`
 * normalised bf16 rows, the block on the union of tp_size * rows_local rows with this rank's weight
 * shard, and the reduce-scatter that leaves the summed bf16 rows of THIS rank in out_local_dev.
 * Every rank of the group must call it with the same rows_local; each rank runs on its own GPU.
 * Device-side waits on peers are bounded; a wait that ran out shows as MOE_ERR_TIMEOUT from
 * moe_synchronize().  Stream-ordered, no host synchronisation (the reference synchronises stream and
 * host threads between steps, getp_run.cpp:2955-2956,:3203-3204). */
int moe_tp_forward(moe_handle h, int layer, const void *t_local_dev, int rows_local, void *out_local_dev,
                   unsigned flags, void *stream);
/* moe_tp_forward for HOST buffers of this rank's rows (copies inside, waits, returns the device status). */
int moe_tp_forward_host(moe_handle h, int layer, const void *t_local_host, int rows_local, void *out_local_host,
                        unsigned flags);
/* The two collectives alone: ring_allgather_rows_bf16 (tp_ring.hpp:70-118) into the gather buffer, and
 * the owner-slice reduce-scatter (getp_run.cpp:3206-3246) of the partial buffers into out_local_dev. */
int moe_tp_allgather(moe_handle h, const void *src_local_dev, int rows_local, void *stream);
int moe_tp_reduce_scatter(moe_handle h, int rows_local, void *out_local_dev, void *stream);

/* Replaces ring_allreduce_sum_bf16 (getp-csrc/tp_ring.hpp:253-331) and the token-wise all-reduce of moe_gpu
 * (getp_run.cpp:2834-2874): after the call buf_dev (bf16, n_elems elements, the same count on every rank of
 * the group) holds the element-wise sum over the ranks, added in fp32 in rank order and rounded once, so every
 * rank ends with the same bits.  n_elems must be a multiple of 8 and at most max_rows * hidden_dim (the values
 * travel through the handle's partial-output buffer).  Every rank calls; stream-ordered, peer waits bounded. */
int moe_tp_allreduce(moe_handle h, void *buf_dev, size_t n_elems, void *stream);

/* No counterpart in the reference.  Router + top-k + softmax for a caller that must not reach
 * the CUDA allocator when it needs a routing decision (its memory was handed out once by a pool
 * that owns the device, or it cannot afford the device-wide synchronisation inside cudaMalloc).
 * The split-k scratch of the router lives in a fixed 8 MiB array inside the library's device image
 * (held by every GPU that loads the library until the process exits); the call allocates nothing.
 * t_dev: bf16 [rows, H] normalised rows; outputs, all caller-owned device memory: logits_dev fp32
 * [rows, E], idx_dev i32 [rows, K], w_dev fp32 [rows, K].  Limit: rows * n_experts <= 2 097 152
 * (MOE_ERR_INVALID beyond it).  The first call on a device looks up the array's device address and
 * should be made at start-up, before any stream capture.  All calls on a device share the array:
 * calls whose kernels overlap on the GPU race.  Stream-ordered on `stream`. */
int moe_route_static(moe_handle h, int layer, const void *t_dev, int rows, float *logits_dev, int *idx_dev,
                     float *w_dev, void *stream);

/* Intermediate results of the last forward, copied to host memory. */
enum {
  MOE_DBG_LOGITS = 0,   /* f32 [rows, E]    router_score_g */
  MOE_DBG_TOPK_IDX = 1, /* i32 [rows, K]    topk_i_g */
  MOE_DBG_TOPK_W = 2,   /* f32 [rows, K]    topk_v_g */
  MOE_DBG_COUNTS = 3,   /* i32 [E]          d_expert_counts */
  MOE_DBG_OFFSETS = 4,  /* i32 [E+1]        d_expert_offsets */
  MOE_DBG_PAIR_ROW = 5, /* i32 [rows, K]    local_ids_g */
  MOE_DBG_ROW_TOKEN = 6,/* i32 [rows*K]     expert_row_token_g */
  MOE_DBG_OUT_F32 = 7,  /* f32 [rows, H]    block output before the bf16 rounding (MOE_CFG_KEEP_F32_OUT) */
  MOE_DBG_STATUS = 8,   /* u32 [4096]       device status word (first element) and diagnostics */
  MOE_DBG_YBUF = 10,    /* f16 [rows*K, H]  MLP2 output, permuted rows (expert_output_partial_g) */
  MOE_DBG_GATHER = 11,  /* bf16 [rows, H]   all-gather destination of the TP group (gather_x_g) */
  MOE_DBG_TNORM = 12,   /* bf16 [rows_local, H]  RMS-normalised rows of the last moe_block() (state.t) */
  MOE_DBG_TP_PARTIAL = 13 /* bf16 [rows, H]  this rank's partial-output buffer of the TP group (e_agg_g) */
};
int moe_get_debug(moe_handle h, int which, void *host_dst, size_t bytes);

/* Per-stage device timing (replaces the reference's TIMER_BLOCK / ProfileManager,
 * getp-csrc/utils.hpp:48-222, which brackets stages with hipDeviceSynchronize):
 * while enabled, every moe_forward records CUDA events between its kernels on
 * the caller's stream.  moe_profile_collect waits for them, adds the elapsed
 * milliseconds of each stage over all calls since the last collect into
 * ms[MOE_N_STAGES] and returns the number of calls in *n_calls. */
enum {
  MOE_STAGE_ROUTER = 0, MOE_STAGE_TOPK = 1, MOE_STAGE_INDEX = 2, MOE_STAGE_GATHER = 3,
  MOE_STAGE_MLP1 = 4, MOE_STAGE_MLP2 = 5, MOE_STAGE_COMBINE = 6, MOE_N_STAGES = 7
};
int moe_profile_enable(moe_handle h, int on);
int moe_profile_collect(moe_handle h, float *ms, int *n_calls);

const char *moe_last_error(moe_handle h);
const char *moe_strerror(int code);
/* Number of kernels of this library launched by the handle so far. */
long long moe_launch_count(moe_handle h);

#ifdef __cplusplus
}
#endif
#endif
