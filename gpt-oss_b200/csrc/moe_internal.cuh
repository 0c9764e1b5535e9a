// Internal structures shared by the host API and the kernels of the MoE block.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/moe_b200.h"

namespace moe {

// ---- tiling constants of the expert GEMM (expert_gemm_sm100.cu) -------------
constexpr int kTileN = 240;        // weight rows per work item (UMMA N); divides 5760 and 2880
constexpr int kTileNPad = 256;     // rows reserved per weight tile in shared memory / scale atoms
constexpr int kChunkK = 128;       // reduction elements per shared-memory stage (4 MMA k-steps of 32)
constexpr int kTokTile = 64;       // token rows per work item
constexpr int kTileM = 2 * kTokTile;  // UMMA M: each token contributes a high and a low e4m3 row
constexpr int kSfAtomBytes = 512;  // scale factors of 128 rows x 4 k-blocks, tensor-memory order
constexpr int kSfbChunkBytes = 2 * kSfAtomBytes;  // weight scales of one tile (240 rows in two atoms)
constexpr int kWTileCodes = kTileN * kChunkK / 2;  // 15360 bytes of packed codes per weight tile
constexpr int kWTileStride = kWTileCodes + kSfbChunkBytes;  // 16384: codes, then scales
static_assert(kWTileStride == 16384, "weight tiles are 16 KB");

// Device status bits (MOE_DBG_STATUS).
enum : unsigned {
  ST_WAIT_FULL = 1u,      // expert GEMM: TMA data never arrived
  ST_WAIT_EMPTY = 2u,     // expert GEMM: stage never released
  ST_WAIT_AREADY = 4u,    // expert GEMM: dequantised tile never published
  ST_WAIT_AFREE = 8u,     // expert GEMM: tensor-memory A buffer never released
  ST_WAIT_DFULL = 16u,    // expert GEMM: accumulator never completed
  ST_WAIT_DEMPTY = 32u,   // expert GEMM: accumulator never drained
  ST_BAD_INDEX = 64u,     // routing produced an out-of-range row
  ST_WAIT_PEER = 128u,    // TP collective: a peer's flag never arrived
  ST_Y_RANGE = 256u,      // expert GEMM: an MLP2 output does not fit fp16 (|y| > 65504)
};

// Error code for a non-zero device status word.
inline int status_error(unsigned st) {
  return (st & ST_BAD_INDEX) ? MOE_ERR_STATE : (st & ST_Y_RANGE) ? MOE_ERR_Y_RANGE : MOE_ERR_TIMEOUT;
}

constexpr int kMaxTp = 8;  // MAX_TP of getp-csrc/nccl.hpp:6
// Symmetric buffers of a tensor-parallel group as seen from one rank: entry r is rank r's buffer
// (a peer mapping, or this rank's own memory for r == rank).
struct TpPeers {
  void *gather[kMaxTp];       // bf16 [max_rows, H]: all-gather destination (gather_x_g)
  void *partial[kMaxTp];      // bf16 [max_rows, H]: this rank's partial block output (e_agg_g)
  uint32_t *flags[kMaxTp];    // [kTpPhases][kMaxTp] epoch words
  void *topk_idx[kMaxTp];     // i32 [max_rows, K]: every rank routes its own rows and writes them to all (topk_i_g)
  void *topk_w[kMaxTp];       // f32 [max_rows, K]                                                  (topk_v_g)
};
constexpr int kTpBufs = 5;
// Hand-shakes of a tensor-parallel call, each with its own row of epoch words: the gathered rows are in
// place, the partial outputs are in place, the expert selections are in place.
enum { kTpPhaseGather = 0, kTpPhaseScatter = 1, kTpPhaseSelection = 2, kTpPhases = 3 };

// One call in flight through moe_forward_host_submit: its own input and output staging, so that the copies of
// neighbouring calls overlap the block of this one.
constexpr int kHostSlots = 3;
struct HostSlot {
  __nv_bfloat16 *in = nullptr, *out = nullptr;   // [max_rows, H] each
  unsigned int *status_dev = nullptr;            // status word of the call that owns the slot (cleared in stream order)
  unsigned int *status_host = nullptr;           // pinned copy of it, taken after the block
  cudaEvent_t in_ready = nullptr, out_ready = nullptr, done = nullptr;
  long long ticket = -1;                         // call that owns the slot; -1: free
};

// One work item of the grouped GEMM: one token tile against nblk adjacent kTileN-row blocks of the expert's
// weight matrix, processed one after the other (the index kernel emits single blocks).
struct __align__(16) WorkItem {
  int expert;  // expert index
  int ntile;   // first kTileN-row block of that expert's weight matrix
  int tile;    // global token-tile index (rows tile*kTileM .. of the quantised activations)
  int row0;    // first permuted row of the token tile
  int ntok;    // valid token rows in the tile (1..kTokTile)
  int nblk;    // row blocks in this item
  int pad[2];
};

struct GemmArgs {
  const WorkItem *work;
  const int *n_work;
  int K;          // reduction length in elements (multiple of 32)
  int R;          // weight rows per expert on this rank
  int n_kchunks;  // ceil(K / kChunkK)
  int n_ntiles;   // ceil(R / kTileN)
  const uint8_t *w_tiles;     // weight tiles [E][n_ntiles][n_kchunks][kWTileStride], see LayerWeights::w1_tiles
  const uint8_t *sfa;         // activation scales, one 512-byte atom per token tile
  int sfa_tile_stride;        // bytes between token tiles' atoms (0: one atom shared by all tiles)
  const __nv_bfloat16 *bias;  // [E][R]
  int add_bias;               // MLP2 on TP ranks other than 0 leaves the bias out
  uint8_t *hq_out;            // MLP1: quantised SwiGLU output, e4m3 tiles [tile][hq_nkc][128 rows][128 bytes]
  int hq_joff, hq_nkc;        //       column of the shard's first output inside MLP2's k window; its k slices
  __half *y_out;              // MLP2: [P, ld_out] fp16
  int ld_out;
  int h_exp;                  // MLP1: SwiGLU outputs are stored as e4m3(h * 2^-h_exp)
  float limit, alpha;
  unsigned int *status;
};

// How one launch of the expert GEMM kernel runs: which phases (0 = MLP1, 1 = MLP2), and where the MLP1 items
// of a token tile are counted so that the tile's MLP2 items, in the same launch, know when its SwiGLU rows
// are complete.
struct MlpFuse {
  int phase_begin, phase_end;
  unsigned int *tile_done;   // [total_slot + 1], zeroed by build_index_kernel; nullptr: phases in separate launches
  int total_slot;            // the last word counts the MLP1 items of all tiles
  int done_per_tile;         // epilogue warps x MLP1 weight blocks
};

struct LayerWeights {
  bool loaded = false;
  // MLP1 weights as the GEMM streams them: one 16 KB tile per (expert, 240-row block, 128-wide slice of k),
  // tiles of a block in k order: [240 rows x 64 bytes of packed e2m1 codes][two 512-byte E8M0 scale atoms in
  // the order tcgen05.cp wants].  Rows or k beyond the matrix hold zero codes and scale 1 (byte 127).
  uint8_t *w1_tiles = nullptr;
  __nv_bfloat16 *b1 = nullptr;   // [E, R1]
  uint8_t *w2_tiles = nullptr;   // MLP2 weights [E, H, Kw], same tiling
  __nv_bfloat16 *b2 = nullptr;   // [E, H]
  // raw (row-major, unpadded) scales for the validation GEMM
  uint8_t *w1_scales_raw = nullptr;  // [E, R1, H/32]
  uint8_t *w2_scales_raw = nullptr;  // [E, H, Dl/32]
  __nv_bfloat16 *router_w3 = nullptr;  // [3][E][H] exact 3-way bf16 split of the fp32 router weight
  float *router_b = nullptr;           // [E]
  CUtensorMap tm_w1, tm_w2, tm_router;
};

}  // namespace moe

struct moe_ctx {
  moe_config cfg;
  int H, D, E, K, L;
  int d0, Dl;     // this rank's slice of the intermediate dimension
  int R1;         // 2*Dl
  int k0, Kw;     // MLP2 reads intermediate columns [k0, k0+Kw): the whole scale blocks around the shard
  int joff;       // d0 - k0: column of the shard's first SwiGLU output inside that window
  int max_rows, max_pairs;
  int sm_count;
  int router_cluster = 0;   // largest thread-block cluster the fused router kernel can use on this device (0: none)
  cudaStream_t stream = nullptr;  // used by moe_forward_host
  std::vector<moe::LayerWeights> layers;

  // run state (names of the reference's GPURunState fields in comments)
  __nv_bfloat16 *t_in = nullptr;    // gather_x_g          [max_rows, H]
  __nv_bfloat16 *t_norm = nullptr;  // t                   [max_rows, H]  RMS-normalised rows of moe_block()
  float *logits = nullptr;          // router_score_g      [max_rows, E]
  float *router_part = nullptr;     // split-k partial sums of the router [splits, rows, E]
  int *topk_idx = nullptr;          // topk_i_g            [max_rows, K]
  float *topk_w = nullptr;          // topk_v_g            [max_rows, K]
  int *counts = nullptr;            // d_expert_counts     [E]
  int *offsets = nullptr;           // d_expert_offsets    [E+1]
  int *pair_row = nullptr;          // local_ids_g         [max_rows, K]
  int *row_token = nullptr;         // expert_row_token_g  [max_pairs]
  int *pair_slot = nullptr;         // row of the high term of (token, k) in xq [max_rows, K]
  unsigned int *tile_done = nullptr;   // [max_tiles + 1] MlpFuse::tile_done
  __half *xperm = nullptr;          // expert_input_buffer [max_pairs, H]   fp16 (validation GEMM only)
  __half *hbuf = nullptr;           // gate_up             [max_pairs, Dl]  fp16 (validation GEMM only)
  uint8_t *xq = nullptr;            // expert_input_buffer as e4m3 high/low rows, [max_tiles][k slices][128 rows][128 B]
  uint8_t *hq = nullptr;            // gate_up as e4m3 high/low rows, same tiling over MLP2's k window
  uint8_t *sfa_x = nullptr;         // per-tile scale atoms of xq [max_tiles][512]
  uint8_t *sfa_h = nullptr;         // the one scale atom of hq   [512]
  int *tile_base = nullptr;         // first token tile of each expert [E+1]
  int max_tiles = 0;
  int h_exp = 0;                    // hq holds e4m3(h * 2^-h_exp)
  __half *ybuf = nullptr;           // expert_output_partial [max_pairs, H] fp16
  float *out_f32 = nullptr;         // fp32 block output   [max_rows, H] (debug / TP partial)
  __nv_bfloat16 *out_bf16 = nullptr;// e_agg_g             [max_rows, H]
  moe::WorkItem *work1 = nullptr, *work2 = nullptr;
  int *n_work = nullptr;            // [2]
  int max_work1 = 0, max_work2 = 0;
  unsigned int *status = nullptr;
  CUtensorMap tm_x1, tm_x2;
  int last_rows = 0;
  long long launches = 0;
  moe::TpPeers peers = {};          // TP group view; own entries are set at creation
  __nv_bfloat16 *tp_partial = nullptr;  // this rank's bf16 partial output [max_rows, H]
  uint32_t *tp_flags = nullptr;     // [kTpPhases][kMaxTp], written by the peers
  uint64_t tp_attached = 0;         // bit (kTpBufs*r + which) set once rank r's buffer `which` is known
  moe::HostSlot host_slots[moe::kHostSlots];
  cudaStream_t h2d_stream = nullptr, d2h_stream = nullptr;
  long long host_submitted = 0;
  cudaStream_t aux_stream = nullptr;  // the all-gather push runs beside the router
  cudaEvent_t ev_fork = nullptr, ev_fork2 = nullptr, ev_join = nullptr;
  uint32_t tp_epoch = 0, tp_epoch_rs = 0;  // all-gather / reduce-scatter call counters
  std::vector<void *> ipc_opened;   // mappings to close at destroy
  bool profiling = false;
  std::vector<cudaEvent_t> prof_events;  // MOE_N_STAGES + 1 per profiled call
  std::vector<cudaEvent_t> prof_pool;    // recycled events
  std::string err;
};

namespace moe {

// cuTensorMapEncodeTiled through the runtime's driver entry point table (no link against libcuda).
typedef CUresult (*TensorMapEncodeFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                      const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                      CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
inline TensorMapEncodeFn tensor_map_encoder() {
  static TensorMapEncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<TensorMapEncodeFn>(p);
  });
  return fn;
}

// What the fused router kernel writes: logits [rows, E], and the selection, weights and expert histogram
// exactly as topk_softmax_kernel does (to every rank's top-k buffers when tp > 0, at row_offset).
struct RouteOut {
  float *logits;
  const float *bias;
  int K;
  int *idx;
  float *w;
  int *counts;
  int tp;
  int row_offset;
  TpPeers peers;
};

// router_sm100.cu
cudaError_t router_init(int *max_cluster);   // per-device kernel attributes; call with the device current
int router_fused_slices(int T, int H, int E, int sm_count, int max_cluster);
bool launch_router_fused(const __nv_bfloat16 *t, const CUtensorMap &tm_w, int T, int H, int E, int slices,
                         const RouteOut &ro, unsigned int *status, cudaStream_t s);
int router_splits(int T, int H, int sm_count);
int router_chunks(int H);
bool make_router_weight_map(CUtensorMap *m, const __nv_bfloat16 *w3, int E, int H);
bool launch_router_partials(const __nv_bfloat16 *t, const CUtensorMap &tm_w, float *partial, int T, int H, int E,
                            int splits, unsigned int *status, cudaStream_t s);
// route.cu
void launch_topk_softmax(float *logits, const float *partial, int splits, const float *bias, int T, int E, int K,
                         int *idx, float *w, int *counts, cudaStream_t s, int tp = 0, const TpPeers *peers = nullptr,
                         int row_offset = 0);
void launch_count_experts(const int *idx, int n, int E, int *counts, cudaStream_t s);
void launch_build_index(const int *topk_idx, const int *counts, int T, int E, int K, int n_ntiles1, int n_ntiles2,
                        int *offsets, int *tile_base, int *pair_row, int *row_token, int *pair_slot, unsigned int *tile_done, int tile_done_total_slot, WorkItem *work1,
                        WorkItem *work2, int *n_work, int max_work1, int max_work2, unsigned int *status,
                        cudaStream_t s);
void launch_quantize_rows(const __nv_bfloat16 *t, const int *pair_slot, int T, int K, uint8_t *xq, uint8_t *sfa, int H,
                          cudaStream_t s);
int quantize_rows_max_hidden();
void launch_gather_rows(const __nv_bfloat16 *t, const int *row_token, const int *offsets, int E, __half *xperm,
                        int H, int max_pairs, cudaStream_t s);
void launch_combine(const __half *y, const int *topk_idx, const float *topk_w, const int *pair_row, int T, int H,
                    int K, __nv_bfloat16 *out_bf16, float *out_f32, cudaStream_t s, int tp = 0,
                    const TpPeers *peers = nullptr, int rows_local = 0, int rank = 0,
                    const __nv_bfloat16 *residual = nullptr);
void launch_rmsnorm_rows(const __nv_bfloat16 *x, const __nv_bfloat16 *w, __nv_bfloat16 *t, int rows, int H,
                         cudaStream_t s);

// expert_gemm_sm100.cu
cudaError_t expert_gemm_init();
void launch_expert_mlp(const CUtensorMap &tm_w1, const CUtensorMap &tm_x1, const GemmArgs &a, const CUtensorMap &tm_w2,
                       const CUtensorMap &tm_x2, const GemmArgs &b, const MlpFuse &f, int grid, cudaStream_t s);
int expert_mlp_done_per_tile(int n_ntiles1);

// tp_collectives.cu
// Both pushes send rows [row0, row0 + n_rows) of this rank's rows_local rows (n_rows < 0: all of them).
void launch_tp_allgather_push(const __nv_bfloat16 *src, int rows_local, int H, const TpPeers &peers, int tp, int rank,
                              cudaStream_t s, int row0 = 0, int n_rows = -1);
void launch_tp_rmsnorm_push(const __nv_bfloat16 *x, const __nv_bfloat16 *w, int rows_local, int H, const TpPeers &peers,
                            int tp, int rank, cudaStream_t s, int row0 = 0, int n_rows = -1);
void launch_tp_signal_wait(const TpPeers &peers, uint32_t *my_flags, int tp, int rank, int phase, uint32_t epoch,
                           unsigned int *status, cudaStream_t s);
void launch_tp_sum_slots(const __nv_bfloat16 *landing, int tp, int rows_local, int H, __nv_bfloat16 *out, int sm_count,
                         cudaStream_t s, const __nv_bfloat16 *residual = nullptr);
void launch_tp_reduce_scatter_pull(const TpPeers &peers, int tp, int rank, int rows_local, int H, __nv_bfloat16 *out,
                                   int sm_count, cudaStream_t s);
void launch_tp_sum_all(const TpPeers &peers, int tp, size_t n_elems, __nv_bfloat16 *out, int sm_count, cudaStream_t s);

// expert_gemm_simt.cu (validation path)
void launch_simt_mlp1(const uint8_t *w_tiles, const uint8_t *scales_raw, const __nv_bfloat16 *bias,
                      const __half *x, const int *offsets, int E, int H, int R1, __half *h_out, int ld_h,
                      float limit, float alpha, int n_rows, cudaStream_t s);
void launch_simt_mlp2(const uint8_t *w_tiles, const uint8_t *scales_raw, const __nv_bfloat16 *bias,
                      int add_bias, const __half *h, const int *offsets, int E, int Dl, int H, __half *y_out,
                      int n_rows, cudaStream_t s);

// moe_tp_api.cu: argument and group checks shared by the calls of a tensor-parallel group.
int check_tp_call(moe_ctx *c, int rows_local, const char *who);

// moe_api.cu: the block itself.  With tp_rows_local > 0 this is a call of a tensor-parallel group: t is the
// gather buffer, t_local this rank's rows; routing is computed for the local rows only and exchanged, the
// combine pushes each row's partial to the rank that owns it, and out_dev receives this rank's summed rows.
// With norm_gain set (moe_block) `residual` holds the rows of the residual stream and the call starts with
// their RMSNorm: into c->t_norm, which then replaces t (one GPU) or t_local (TP group; the all-gather push
// normalises on the fly).
int forward_impl(moe_ctx *c, int layer, const __nv_bfloat16 *t, int T, __nv_bfloat16 *out_dev, unsigned flags,
                 cudaStream_t s, const __nv_bfloat16 *t_local, int tp_rows_local,
                 const __nv_bfloat16 *residual = nullptr, unsigned int *status = nullptr,
                 const __nv_bfloat16 *norm_gain = nullptr);

}  // namespace moe
