// Host side of the C ABI (include/moe_b200.h): context, weight ingestion and
// the launch sequence of one MoE block.  It mirrors, call for call, what the
// reference runtime does around its MoE kernels (getp-csrc/getp_run.cpp:
// malloc_gpu_run_state*, copy_weights_to_gpu_*, moe_gpu / moe_gpu_120b), minus
// the host synchronisations: nothing in moe_forward() waits for the device.
#include <algorithm>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "moe_internal.cuh"

using namespace moe;

namespace {

int fail(moe_ctx *c, int code, const char *fmt, ...) {
  if (c) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    c->err = buf;
  }
  return code;
}

#define CU_TRY(c, expr)                                                                       \
  do {                                                                                        \
    cudaError_t e__ = (expr);                                                                 \
    if (e__ != cudaSuccess)                                                                   \
      return fail((c), e__ == cudaErrorMemoryAllocation ? MOE_ERR_NOMEM : MOE_ERR_CUDA,       \
                  "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e__), __FILE__, __LINE__); \
  } while (0)

// Weight tiles (LayerWeights::w1_tiles): every 16 KB tile starts with 240 rows x 64 bytes of packed e2m1 codes,
// declared to TMA as 4-bit elements that it expands to the 8-bit containers of the block-scaled MMA
// (16U4_ALIGN16B): dims {128 codes, 240 rows, tiles}, one box = the codes of one tile, a contiguous 15 KB read.
int make_weight_map(moe_ctx *c, CUtensorMap *m, const uint8_t *base, size_t n_tiles) {
  TensorMapEncodeFn fn = tensor_map_encoder();
  if (!fn) return fail(c, MOE_ERR_CUDA, "cuTensorMapEncodeTiled not available");
  const cuuint64_t dims[3] = {kChunkK, kTileN, static_cast<cuuint64_t>(n_tiles)};
  const cuuint64_t strides[2] = {kChunkK / 2, kWTileStride};
  const cuuint32_t box[3] = {kChunkK, kTileN, 1};
  const cuuint32_t es[3] = {1, 1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, 3, const_cast<uint8_t *>(base), dims, strides, box, es,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(c, MOE_ERR_CUDA, "cuTensorMapEncodeTiled(weights, %zu tiles) -> %d", n_tiles, (int)r);
  return MOE_OK;
}

// e4m3 activation tiles: [token tile][k slice][128 rows][128 bytes], so that the 16 KB a work item needs for one
// k slice are one contiguous run (rows of K bytes would make the box 128 separate 128-byte pieces).  To TMA
// this is a matrix of 128-byte rows; box = 128 x 128, 128-byte swizzle.
int make_act_map(moe_ctx *c, CUtensorMap *m, const uint8_t *base, size_t n_tiles, int n_kc) {
  TensorMapEncodeFn fn = tensor_map_encoder();
  if (!fn) return fail(c, MOE_ERR_CUDA, "cuTensorMapEncodeTiled not available");
  const cuuint64_t rows = static_cast<cuuint64_t>(n_tiles) * n_kc * kTileM;
  const cuuint64_t dims[2] = {kChunkK, rows};
  const cuuint64_t strides[1] = {kChunkK};
  const cuuint32_t box[2] = {kChunkK, kTileM};
  const cuuint32_t es[2] = {1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t *>(base), dims, strides, box, es,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(c, MOE_ERR_CUDA, "cuTensorMapEncodeTiled(activations, %zu tiles x %d slices) -> %d", n_tiles, n_kc, (int)r);
  return MOE_OK;
}

uint16_t f32_to_bf16_rn(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  u += 0x7FFFu + ((u >> 16) & 1u);
  return static_cast<uint16_t>(u >> 16);
}
float bf16_to_f32(uint16_t b) {
  uint32_t u = static_cast<uint32_t>(b) << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

template <class T>
int dev_alloc(moe_ctx *c, T **p, size_t n) {
  CU_TRY(c, cudaMalloc(reinterpret_cast<void **>(p), n * sizeof(T) + 256));
  return MOE_OK;
}

// One weight matrix -> the 16 KB tiles the GEMM streams (LayerWeights::w1_tiles).  codes: [E][R] rows of
// row_bytes packed bytes at `pitch`; raw: E8M0 scales [E][R][nblk].  In a tile the scale of row r (of the tile's
// 240), k block kb sits at byte (r%32)*16 + (r/32 %4)*4 + kb of atom r/128, the order tcgen05.cp puts them into
// tensor memory; 127 (scale 1) and zero codes where no row or no block exists.
void tile_weights(const uint8_t *codes, size_t pitch, size_t row_bytes, const uint8_t *raw, int E, int R, int nblk,
                  int n_ntiles, int n_kc, std::vector<uint8_t> &out) {
  out.assign(static_cast<size_t>(E) * n_ntiles * n_kc * kWTileStride, 0);
  for (size_t t = 0; t < static_cast<size_t>(E) * n_ntiles * n_kc; ++t)
    memset(&out[t * kWTileStride + kWTileCodes], 127, kSfbChunkBytes);
  for (int e = 0; e < E; ++e)
    for (int r = 0; r < R; ++r) {
      const uint8_t *src_c = codes + (static_cast<size_t>(e) * R + r) * pitch;
      const uint8_t *src_s = raw + (static_cast<size_t>(e) * R + r) * nblk;
      const int nt = r / kTileN, rr = r % kTileN, atom = rr / 128, ra = rr % 128;
      uint8_t *tile0 = &out[(static_cast<size_t>(e) * n_ntiles + nt) * n_kc * kWTileStride];
      for (int kc = 0; kc < n_kc; ++kc) {
        const size_t off = static_cast<size_t>(kc) * (kChunkK / 2);
        if (off < row_bytes)
          memcpy(tile0 + static_cast<size_t>(kc) * kWTileStride + rr * (kChunkK / 2), src_c + off,
                 std::min<size_t>(kChunkK / 2, row_bytes - off));
      }
      for (int b = 0; b < nblk; ++b) {
        const int kc = b / 4, kb = b % 4;
        tile0[static_cast<size_t>(kc) * kWTileStride + kWTileCodes + atom * kSfAtomBytes + (ra % 32) * 16 + (ra / 32) * 4 + kb] =
            src_s[b];
      }
    }
}

void free_layer(LayerWeights &w) {
  cudaFree(w.w1_tiles); cudaFree(w.b1);
  cudaFree(w.w2_tiles); cudaFree(w.b2);
  cudaFree(w.w1_scales_raw); cudaFree(w.w2_scales_raw);
  cudaFree(w.router_w3); cudaFree(w.router_b);
  w = LayerWeights();
}

}  // namespace

namespace moe {

int forward_impl(moe_ctx *c, int layer, const __nv_bfloat16 *t, int rows, __nv_bfloat16 *out_dev, unsigned flags,
                 cudaStream_t s, const __nv_bfloat16 *t_local, int tp_rows_local, const __nv_bfloat16 *residual,
                 unsigned int *status, const __nv_bfloat16 *norm_gain) {
  if (status == nullptr) status = c->status;
  if (layer < 0 || layer >= c->L || !t || rows <= 0 || rows > c->max_rows)
    return fail(c, MOE_ERR_INVALID, "moe_forward: layer %d rows %d (max %d)", layer, rows, c->max_rows);
  if (!out_dev && !(flags & MOE_FWD_PARTIAL_F32)) return fail(c, MOE_ERR_INVALID, "moe_forward: null output");
  LayerWeights &w = c->layers[layer];
  if (!w.loaded) return fail(c, MOE_ERR_STATE, "layer %d has no weights", layer);
  CU_TRY(c, cudaSetDevice(c->cfg.device));
  const bool tpcall = tp_rows_local > 0;
  const int tp = c->cfg.tp_size, rank = c->cfg.tp_rank;
  const int T = rows, P = rows * c->K, E = c->E, H = c->H, K = c->K;
  const int n_nt1 = (c->R1 + kTileN - 1) / kTileN, n_nt2 = (H + kTileN - 1) / kTileN;

  CU_TRY(c, cudaMemsetAsync(c->counts, 0, sizeof(int) * E, s));
  auto mark = [&]() {
    if (!c->profiling) return;
    cudaEvent_t ev;
    if (!c->prof_pool.empty()) { ev = c->prof_pool.back(); c->prof_pool.pop_back(); }
    else if (cudaEventCreate(&ev) != cudaSuccess) return;
    cudaEventRecord(ev, s);
    c->prof_events.push_back(ev);
  };
  // a stage that launches nothing (its work went into the previous launch) shares that launch's event:
  // recording another one would book the few microseconds an event costs as the stage's time
  auto mark_empty = [&]() {
    if (c->profiling) c->prof_events.push_back(nullptr);
  };
  mark();
  if (norm_gain != nullptr && !tpcall) {   // step 0 of moe_gpu on one GPU: t = rmsnorm(x) * gain
    launch_rmsnorm_rows(residual, norm_gain, c->t_norm, rows, H, s);
    t = c->t_norm;
    c->launches += 1;
  }
  // Routing of `n` rows at `src`: one fused launch (router GEMM, bias, top-k, softmax, histogram) when the
  // experts fit one CTA, else partial sums and topk_softmax_kernel.  In a TP call the selection goes to the
  // top-k buffers of every rank at this rank's row offset and the histogram is taken after the exchange.
  bool routed_in_one_launch = false;
  auto route_rows = [&](const __nv_bfloat16 *src, int n) -> int {
    const int slices = (flags & MOE_FWD_SPLIT_ROUTER) ? 0 : router_fused_slices(n, H, E, c->sm_count, c->router_cluster);
    RouteOut ro = {};
    ro.logits = c->logits; ro.bias = w.router_b; ro.K = K;
    if (tpcall) { ro.tp = tp; ro.peers = c->peers; ro.row_offset = rank * tp_rows_local; }
    else { ro.idx = c->topk_idx; ro.w = c->topk_w; ro.counts = c->counts; }
    bool ok;
    if (slices > 0) {
      ok = launch_router_fused(src, w.tm_router, n, H, E, slices, ro, status, s);
      routed_in_one_launch = true;
      mark();
      c->launches -= 1;   // one launch where the tally below counts two
    } else {
      const int splits = router_splits(n, H, c->sm_count);
      ok = launch_router_partials(src, w.tm_router, c->router_part, n, H, E, splits, status, s);
      mark();
      launch_topk_softmax(ro.logits, c->router_part, splits, ro.bias, n, E, K, ro.idx, ro.w, ro.counts, s, ro.tp,
                          &ro.peers, ro.row_offset);
    }
    if (!ok) return fail(c, MOE_ERR_INVALID, "router launch refused (input rows 16-byte aligned, hidden_dim a multiple of 8?)");
    return MOE_OK;
  };
  if (!tpcall) {
    if (int rc = route_rows(t, T)) return rc;
    if (routed_in_one_launch) mark_empty(); else mark();
  } else {
    // The all-gather push runs on the side stream in two parts.  The first starts at once, beside the
    // routing of the same rows; the router's few peer stores (the selections, written to every rank) queue
    // behind it on the links, which is why it is only a part.  Once the selections are exchanged the second
    // part goes out, while this stream builds histogram and index from them.
    ++c->tp_epoch;
    const int part_a = tp_rows_local >= 256 ? (tp_rows_local * 2 / 5 + 7) / 8 * 8 : tp_rows_local;
    auto push_rows = [&](int row0, int n) {
      if (norm_gain != nullptr) launch_tp_rmsnorm_push(residual, norm_gain, tp_rows_local, H, c->peers, tp, rank, c->aux_stream, row0, n);
      else launch_tp_allgather_push(t_local, tp_rows_local, H, c->peers, tp, rank, c->aux_stream, row0, n);
    };
    CU_TRY(c, cudaEventRecord(c->ev_fork, s));
    CU_TRY(c, cudaStreamWaitEvent(c->aux_stream, c->ev_fork, 0));
    push_rows(0, part_a);
    if (norm_gain != nullptr) {   // moe_block: the rows the router reads are normalised here, the push normalises on the fly
      launch_rmsnorm_rows(residual, norm_gain, c->t_norm, tp_rows_local, H, s);
      c->launches += 1;
    }
    if (int rc = route_rows(norm_gain != nullptr ? c->t_norm : t_local, tp_rows_local)) return rc;
    launch_tp_signal_wait(c->peers, c->tp_flags, tp, rank, kTpPhaseSelection, c->tp_epoch, status, s);
    if (part_a < tp_rows_local) {
      CU_TRY(c, cudaEventRecord(c->ev_fork2, s));
      CU_TRY(c, cudaStreamWaitEvent(c->aux_stream, c->ev_fork2, 0));
      push_rows(part_a, tp_rows_local - part_a);
      c->launches += 1;
    }
    CU_TRY(c, cudaEventRecord(c->ev_join, c->aux_stream));
    launch_count_experts(c->topk_idx, T * K, E, c->counts, s);
    mark();
    c->launches += 4;
  }
  launch_build_index(c->topk_idx, c->counts, T, E, K, n_nt1, n_nt2, c->offsets, c->tile_base, c->pair_row,
                     c->row_token, c->pair_slot, c->tile_done, c->max_tiles, c->work1, c->work2, c->n_work, c->max_work1,
                     c->max_work2, status, s);
  if (tpcall) {   // now the gathered rows: this rank's push is complete (side stream), then every peer's
    CU_TRY(c, cudaStreamWaitEvent(s, c->ev_join, 0));
    launch_tp_signal_wait(c->peers, c->tp_flags, tp, rank, kTpPhaseGather, c->tp_epoch, status, s);
  }
  mark();
  if (flags & MOE_FWD_SIMT_GEMM) launch_gather_rows(t, c->row_token, c->offsets, E, c->xperm, H, P, s);
  else launch_quantize_rows(t, c->pair_slot, T, K, c->xq, c->sfa_x, H, s);
  mark();
  const int add_b2 = c->cfg.tp_rank == 0 ? 1 : 0;
  bool mlp_in_one_launch = false;
  if (flags & MOE_FWD_SIMT_GEMM) {
    launch_simt_mlp1(w.w1_tiles, w.w1_scales_raw, w.b1, c->xperm, c->offsets, E, H, c->R1,
                     c->hbuf + c->joff, c->Kw, c->cfg.swiglu_limit, c->cfg.swiglu_alpha, P, s);
    mark();
    launch_simt_mlp2(w.w2_tiles, w.w2_scales_raw, w.b2, add_b2, c->hbuf, c->offsets, E, c->Kw, H,
                     c->ybuf, P, s);
  } else {
    GemmArgs a{};
    a.work = c->work1; a.n_work = c->n_work; a.K = H; a.R = c->R1;
    a.n_kchunks = (H + kChunkK - 1) / kChunkK; a.n_ntiles = n_nt1;
    a.w_tiles = w.w1_tiles; a.sfa = c->sfa_x; a.sfa_tile_stride = kSfAtomBytes; a.bias = w.b1; a.add_bias = 1;
    a.hq_out = c->hq; a.hq_joff = c->joff; a.hq_nkc = (c->Kw + kChunkK - 1) / kChunkK; a.y_out = nullptr; a.ld_out = c->Kw;
    a.h_exp = c->h_exp;
    a.limit = c->cfg.swiglu_limit; a.alpha = c->cfg.swiglu_alpha; a.status = status;
    GemmArgs b = a;
    b.work = c->work2; b.n_work = c->n_work + 1; b.K = c->Kw; b.R = H;
    b.n_kchunks = (c->Kw + kChunkK - 1) / kChunkK; b.n_ntiles = n_nt2;
    b.w_tiles = w.w2_tiles; b.sfa = c->sfa_h; b.sfa_tile_stride = 0; b.bias = w.b2; b.add_bias = add_b2;
    b.hq_out = nullptr; b.y_out = c->ybuf; b.ld_out = H;
    MlpFuse fuse{};
    fuse.total_slot = c->max_tiles;
    fuse.done_per_tile = expert_mlp_done_per_tile(n_nt1);
    if (flags & MOE_FWD_SPLIT_MLP) {   // MLP1 and MLP2 as two launches
      fuse.phase_begin = 0; fuse.phase_end = 1; fuse.tile_done = nullptr;
      launch_expert_mlp(w.tm_w1, c->tm_x1, a, w.tm_w2, c->tm_x2, b, fuse, c->sm_count, s);
      mark();
      fuse.phase_begin = 1; fuse.phase_end = 2;
      launch_expert_mlp(w.tm_w1, c->tm_x1, a, w.tm_w2, c->tm_x2, b, fuse, c->sm_count, s);
    } else {                           // one launch; the MLP2 stage of a profile is then empty
      fuse.phase_begin = 0; fuse.phase_end = 2; fuse.tile_done = c->tile_done;
      launch_expert_mlp(w.tm_w1, c->tm_x1, a, w.tm_w2, c->tm_x2, b, fuse, c->sm_count, s);
      mark();
      c->launches -= 1;
      mlp_in_one_launch = true;
    }
  }
  if (mlp_in_one_launch) mark_empty(); else mark();
  if (!tpcall) {
    const bool partial = (flags & MOE_FWD_PARTIAL_F32) != 0;
    const bool keep_f32 = partial || (c->cfg.flags & MOE_CFG_KEEP_F32_OUT);
    launch_combine(c->ybuf, c->topk_idx, c->topk_w, c->pair_row, T, H, K, partial ? nullptr : out_dev,
                   keep_f32 ? c->out_f32 : nullptr, s, 0, nullptr, 0, 0, residual);
    mark();
  } else {
    // send half of the reduce-scatter inside the combine; then wait for every peer's rows and add the slots
    launch_combine(c->ybuf, c->topk_idx, c->topk_w, c->pair_row, T, H, K, c->tp_partial,
                   (c->cfg.flags & MOE_CFG_KEEP_F32_OUT) ? c->out_f32 : nullptr, s, tp, &c->peers, tp_rows_local, rank);
    ++c->tp_epoch_rs;
    launch_tp_signal_wait(c->peers, c->tp_flags, tp, rank, kTpPhaseScatter, c->tp_epoch_rs, status, s);
    launch_tp_sum_slots(c->tp_partial, tp, tp_rows_local, H, out_dev, c->sm_count, s, residual);
    mark();
    c->launches += 2;
  }
  c->launches += 7;
  c->last_rows = rows;
  CU_TRY(c, cudaGetLastError());
  return MOE_OK;
}

}  // namespace moe

extern "C" {

const char *moe_strerror(int code) {
  switch (code) {
    case MOE_OK: return "ok";
    case MOE_ERR_INVALID: return "invalid argument";
    case MOE_ERR_CUDA: return "CUDA error";
    case MOE_ERR_NOMEM: return "out of memory";
    case MOE_ERR_TIMEOUT: return "a bounded wait ran out";
    case MOE_ERR_SCALE_RANGE: return "E8M0 scale byte is NaN";
    case MOE_ERR_Y_RANGE: return "an expert output does not fit fp16";
    case MOE_ERR_STATE: return "wrong state";
    case MOE_ERR_NO_SM100: return "device is not sm_100";
    default: return "unknown";
  }
}

const char *moe_last_error(moe_handle h) { return h ? h->err.c_str() : "null handle"; }
long long moe_launch_count(moe_handle h) { return h ? h->launches : 0; }

int moe_shard_range(int D, int tp_size, int tp_rank, int *start, int *len) {
  if (D <= 0 || D % 32 || tp_size <= 0 || tp_rank < 0 || tp_rank >= tp_size || D / 32 < tp_size) return MOE_ERR_INVALID;
  int s, l;
  if (D % tp_size == 0 && (D / tp_size) % 8 == 0) {
    // the reference's even split (mlp2_shard_input, getp_run.cpp:2495-2501)
    l = D / tp_size;
    s = tp_rank * l;
  } else {
    // uneven case: distribute whole 32-element scale blocks
    const int nblk = D / 32, base = nblk / tp_size, rem = nblk % tp_size;
    l = 32 * (base + (tp_rank < rem ? 1 : 0));
    s = 32 * (tp_rank * base + (tp_rank < rem ? tp_rank : rem));
  }
  if (start) *start = s;
  if (len) *len = l;
  return MOE_OK;
}

int moe_create(const moe_config *cfg, moe_handle *out) {
  if (!cfg || !out) return MOE_ERR_INVALID;
  *out = nullptr;
  if (cfg->hidden_dim <= 0 || cfg->hidden_dim % 32 || cfg->hidden_dim > quantize_rows_max_hidden() || cfg->intermediate_dim <= 0 || cfg->intermediate_dim % 32 ||
      cfg->n_experts <= 0 || cfg->n_experts > 256 || (cfg->n_experts & 1) || cfg->experts_per_token <= 0 || cfg->experts_per_token > 8 ||
      cfg->experts_per_token > cfg->n_experts || cfg->n_layers <= 0 || cfg->max_rows <= 0 || cfg->tp_size <= 0 ||
      cfg->tp_rank < 0 || cfg->tp_rank >= cfg->tp_size)
    return MOE_ERR_INVALID;
  moe_ctx *c = new (std::nothrow) moe_ctx();
  if (!c) return MOE_ERR_NOMEM;
  *out = c;  // returned even on failure so the caller can read moe_last_error(); moe_destroy() frees it
  c->cfg = *cfg;
  c->H = cfg->hidden_dim; c->D = cfg->intermediate_dim; c->E = cfg->n_experts;
  c->K = cfg->experts_per_token; c->L = cfg->n_layers;
  if (moe_shard_range(c->D, cfg->tp_size, cfg->tp_rank, &c->d0, &c->Dl) != MOE_OK)
    return fail(c, MOE_ERR_INVALID, "intermediate_dim %d cannot be split over %d ranks on 32-element boundaries", c->D, cfg->tp_size);
  c->R1 = 2 * c->Dl;
  // MLP2 reads the window of whole scale blocks that encloses the shard; the SwiGLU outputs outside the
  // shard inside that window are never written and stay zero
  c->k0 = c->d0 / 32 * 32;
  c->Kw = (c->d0 + c->Dl + 31) / 32 * 32 - c->k0;
  c->joff = c->d0 - c->k0;
  c->max_rows = cfg->max_rows;
  c->max_pairs = cfg->max_rows * c->K;
  c->layers.resize(c->L);

  CU_TRY(c, cudaSetDevice(cfg->device));
  cudaDeviceProp prop;
  CU_TRY(c, cudaGetDeviceProperties(&prop, cfg->device));
  if (prop.major != 10) return fail(c, MOE_ERR_NO_SM100, "device %d is sm_%d%d; this library is sm_100a only", cfg->device, prop.major, prop.minor);
  c->sm_count = prop.multiProcessorCount;
  CU_TRY(c, cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking));
  CU_TRY(c, expert_gemm_init());
  CU_TRY(c, router_init(&c->router_cluster));

  const size_t T = c->max_rows, P = c->max_pairs;
  int rc;
  if ((rc = dev_alloc(c, &c->t_in, T * c->H))) return rc;
  if ((rc = dev_alloc(c, &c->t_norm, T * c->H))) return rc;
  if ((rc = dev_alloc(c, &c->logits, T * c->E))) return rc;
  // splits * rows never exceeds (sm_count / tiles) * 128 * tiles = 128 * sm_count
  if ((rc = dev_alloc(c, &c->router_part, std::max<size_t>(T, 128 * static_cast<size_t>(c->sm_count) + 128) * c->E))) return rc;
  if ((rc = dev_alloc(c, &c->topk_idx, T * c->K))) return rc;
  if ((rc = dev_alloc(c, &c->topk_w, T * c->K))) return rc;
  if ((rc = dev_alloc(c, &c->counts, (size_t)c->E))) return rc;
  if ((rc = dev_alloc(c, &c->offsets, (size_t)c->E + 1))) return rc;
  if ((rc = dev_alloc(c, &c->pair_row, T * c->K))) return rc;
  if ((rc = dev_alloc(c, &c->row_token, P))) return rc;
  if ((rc = dev_alloc(c, &c->pair_slot, P))) return rc;
  if ((rc = dev_alloc(c, &c->xperm, P * c->H))) return rc;
  if ((rc = dev_alloc(c, &c->hbuf, P * c->Kw))) return rc;
  if ((rc = dev_alloc(c, &c->ybuf, P * c->H))) return rc;
  if ((rc = dev_alloc(c, &c->out_f32, T * c->H))) return rc;
  if ((rc = dev_alloc(c, &c->out_bf16, T * c->H))) return rc;
  // symmetric buffers of the TP group; this rank's own entries are known now
  if ((rc = dev_alloc(c, &c->tp_partial, T * c->H))) return rc;
  if ((rc = dev_alloc(c, &c->tp_flags, static_cast<size_t>(kTpPhases) * kMaxTp))) return rc;
  CU_TRY(c, cudaMemset(c->tp_flags, 0, kTpPhases * kMaxTp * sizeof(uint32_t)));
  if (cfg->tp_size > kMaxTp) return fail(c, MOE_ERR_INVALID, "tp_size %d above %d", cfg->tp_size, kMaxTp);
  c->peers.gather[cfg->tp_rank] = c->t_in;
  c->peers.partial[cfg->tp_rank] = c->tp_partial;
  c->peers.flags[cfg->tp_rank] = c->tp_flags;
  c->peers.topk_idx[cfg->tp_rank] = c->topk_idx;
  c->peers.topk_w[cfg->tp_rank] = c->topk_w;
  c->tp_attached |= ((1ull << kTpBufs) - 1) << (kTpBufs * cfg->tp_rank);
  CU_TRY(c, cudaStreamCreateWithFlags(&c->aux_stream, cudaStreamNonBlocking));
  CU_TRY(c, cudaEventCreateWithFlags(&c->ev_fork, cudaEventDisableTiming));
  CU_TRY(c, cudaEventCreateWithFlags(&c->ev_fork2, cudaEventDisableTiming));
  CU_TRY(c, cudaEventCreateWithFlags(&c->ev_join, cudaEventDisableTiming));
  const int n_nt1 = (c->R1 + kTileN - 1) / kTileN, n_nt2 = (c->H + kTileN - 1) / kTileN;
  c->max_tiles = c->max_pairs / kTokTile + c->E + 1;
  if ((rc = dev_alloc(c, &c->tile_done, static_cast<size_t>(c->max_tiles) + 1))) return rc;
  c->max_work1 = c->max_tiles * n_nt1;
  c->max_work2 = c->max_tiles * n_nt2;
  // SwiGLU outputs are bounded by limit*(limit+1); they are stored as e4m3(h * 2^-h_exp) with the
  // largest magnitude kept below 256 (e4m3 saturates at 448)
  {
    const float bound = fmaxf(c->cfg.swiglu_limit * (c->cfg.swiglu_limit + 1.0f), 1.0f);
    c->h_exp = static_cast<int>(ceilf(log2f(bound))) - 8;
  }
  const int n_kc1 = (c->H + kChunkK - 1) / kChunkK, n_kc2 = (c->Kw + kChunkK - 1) / kChunkK;
  const size_t act_tile = static_cast<size_t>(kTileM) * kChunkK;   // 16 KB per (token tile, k slice)
  const size_t xq_bytes = static_cast<size_t>(c->max_tiles) * n_kc1 * act_tile;
  const size_t hq_bytes = static_cast<size_t>(c->max_tiles) * n_kc2 * act_tile;
  if ((rc = dev_alloc(c, &c->xq, xq_bytes))) return rc;
  if ((rc = dev_alloc(c, &c->hq, hq_bytes))) return rc;
  if ((rc = dev_alloc(c, &c->sfa_x, static_cast<size_t>(c->max_tiles) * kSfAtomBytes))) return rc;
  if ((rc = dev_alloc(c, &c->sfa_h, static_cast<size_t>(kSfAtomBytes)))) return rc;
  if ((rc = dev_alloc(c, &c->tile_base, static_cast<size_t>(c->E) + 1))) return rc;
  CU_TRY(c, cudaMemset(c->xq, 0, xq_bytes));   // bytes past K in the last slice and never-written columns stay 0
  CU_TRY(c, cudaMemset(c->hq, 0, hq_bytes));
  CU_TRY(c, cudaMemset(c->sfa_x, 127, static_cast<size_t>(c->max_tiles) * kSfAtomBytes));
  {
    uint8_t atom[kSfAtomBytes];
    for (int r = 0; r < kTileM; ++r)
      for (int kb = 0; kb < 4; ++kb)
        atom[(r % 32) * 16 + (r / 32) * 4 + kb] = static_cast<uint8_t>(127 + c->h_exp - ((r & 1) ? 4 : 0));
    CU_TRY(c, cudaMemcpy(c->sfa_h, atom, kSfAtomBytes, cudaMemcpyHostToDevice));
  }
  if ((rc = dev_alloc(c, &c->work1, (size_t)c->max_work1))) return rc;
  if ((rc = dev_alloc(c, &c->work2, (size_t)c->max_work2))) return rc;
  if ((rc = dev_alloc(c, &c->n_work, (size_t)2))) return rc;
  if ((rc = dev_alloc(c, &c->status, (size_t)4096))) return rc;
  CU_TRY(c, cudaMemset(c->status, 0, 4096 * sizeof(unsigned)));
  CU_TRY(c, cudaMemset(c->n_work, 0, 2 * sizeof(int)));
  // Rows past the current batch are read (and discarded) by token tiles that overhang; keep them finite.
  CU_TRY(c, cudaMemset(c->xperm, 0, P * c->H * sizeof(__half)));
  CU_TRY(c, cudaMemset(c->hbuf, 0, P * c->Kw * sizeof(__half)));
  if ((rc = make_act_map(c, &c->tm_x1, c->xq, c->max_tiles, n_kc1))) return rc;
  if ((rc = make_act_map(c, &c->tm_x2, c->hq, c->max_tiles, n_kc2))) return rc;
  return MOE_OK;
}

int moe_destroy(moe_handle c) {
  if (!c) return MOE_ERR_INVALID;
  cudaSetDevice(c->cfg.device);
  if (c->stream) { cudaStreamSynchronize(c->stream); cudaStreamDestroy(c->stream); }
  for (void *p : c->ipc_opened) cudaIpcCloseMemHandle(p);
  if (c->aux_stream) { cudaStreamSynchronize(c->aux_stream); cudaStreamDestroy(c->aux_stream); }
  for (cudaStream_t st : {c->h2d_stream, c->d2h_stream})
    if (st) { cudaStreamSynchronize(st); cudaStreamDestroy(st); }
  for (HostSlot &hs : c->host_slots) {
    cudaFree(hs.in); cudaFree(hs.out); cudaFree(hs.status_dev);
    if (hs.status_host) cudaFreeHost(hs.status_host);
    for (cudaEvent_t e : {hs.in_ready, hs.out_ready, hs.done})
      if (e) cudaEventDestroy(e);
  }
  if (c->ev_fork) cudaEventDestroy(c->ev_fork);
  if (c->ev_fork2) cudaEventDestroy(c->ev_fork2);
  if (c->ev_join) cudaEventDestroy(c->ev_join);
  cudaFree(c->tp_partial); cudaFree(c->tp_flags);
  for (auto &w : c->layers) free_layer(w);
  for (cudaEvent_t e : c->prof_events) if (e) cudaEventDestroy(e);
  for (cudaEvent_t e : c->prof_pool) cudaEventDestroy(e);
  cudaFree(c->t_in); cudaFree(c->t_norm); cudaFree(c->logits); cudaFree(c->router_part); cudaFree(c->topk_idx); cudaFree(c->topk_w); cudaFree(c->counts);
  cudaFree(c->offsets); cudaFree(c->pair_row); cudaFree(c->row_token); cudaFree(c->pair_slot); cudaFree(c->tile_done); cudaFree(c->xperm); cudaFree(c->hbuf);
  cudaFree(c->ybuf); cudaFree(c->out_f32); cudaFree(c->out_bf16); cudaFree(c->work1); cudaFree(c->work2);
  cudaFree(c->n_work); cudaFree(c->status);
  cudaFree(c->xq); cudaFree(c->hq); cudaFree(c->sfa_x); cudaFree(c->sfa_h); cudaFree(c->tile_base);
  delete c;
  return MOE_OK;
}

int moe_load_layer(moe_handle c, int layer, const uint8_t *w1_codes, const uint8_t *w1_scales, const uint16_t *b1,
                   const uint8_t *w2_codes, const uint8_t *w2_scales, const uint16_t *b2, const float *router_w,
                   const float *router_b) {
  if (!c) return MOE_ERR_INVALID;
  if (layer < 0 || layer >= c->L || !w1_codes || !w1_scales || !b1 || !w2_codes || !w2_scales || !b2 || !router_w || !router_b)
    return fail(c, MOE_ERR_INVALID, "moe_load_layer: bad layer index or null tensor");
  CU_TRY(c, cudaSetDevice(c->cfg.device));
  const int E = c->E, H = c->H, D = c->D, d0 = c->d0, R1 = c->R1, k0 = c->k0, Kw = c->Kw;
  LayerWeights &w = c->layers[layer];
  free_layer(w);

  // ---- this rank's shard, still in the reference layout -------------------
  // MLP1: rows [2*d0, 2*(d0+Dl)) of every expert (gate/up pairs stay adjacent);
  // MLP2: columns [k0, k0+Kw), the whole scale blocks that enclose the shard [d0, d0+Dl).
  const size_t w1_row = H / 2, s1_row = H / 32, p1 = w1_row;
  std::vector<uint8_t> c1(static_cast<size_t>(E) * R1 * p1, 0), s1(static_cast<size_t>(E) * R1 * s1_row);
  std::vector<uint16_t> bb1(static_cast<size_t>(E) * R1);
  for (int e = 0; e < E; ++e) {
    const size_t src_row0 = static_cast<size_t>(e) * 2 * D + 2 * d0;
    for (int r = 0; r < R1; ++r)
      memcpy(&c1[(static_cast<size_t>(e) * R1 + r) * p1], w1_codes + (src_row0 + r) * w1_row, w1_row);
    memcpy(&s1[static_cast<size_t>(e) * R1 * s1_row], w1_scales + src_row0 * s1_row, static_cast<size_t>(R1) * s1_row);
    memcpy(&bb1[static_cast<size_t>(e) * R1], b1 + src_row0, static_cast<size_t>(R1) * 2);
  }
  const size_t w2_row = Kw / 2, s2_row = Kw / 32, p2 = w2_row;
  std::vector<uint8_t> c2(static_cast<size_t>(E) * H * p2, 0), s2(static_cast<size_t>(E) * H * s2_row);
  for (size_t r = 0; r < static_cast<size_t>(E) * H; ++r) {
    memcpy(&c2[r * p2], w2_codes + r * (D / 2) + k0 / 2, w2_row);
    memcpy(&s2[r * s2_row], w2_scales + r * (D / 32) + k0 / 32, s2_row);
  }
  // 0xFF is the NaN encoding of E8M0; every other byte is a valid power of two for the tensor core
  for (const std::vector<uint8_t> *sv : {&s1, &s2})
    for (uint8_t b : *sv)
      if (b == 0xFF) return fail(c, MOE_ERR_SCALE_RANGE, "layer %d: E8M0 scale byte 0xFF (NaN)", layer);

  const int n_nt1 = (R1 + kTileN - 1) / kTileN, n_kc1 = (H + kChunkK - 1) / kChunkK;
  const int n_nt2 = (H + kTileN - 1) / kTileN, n_kc2 = (Kw + kChunkK - 1) / kChunkK;
  std::vector<uint8_t> t1, t2;
  tile_weights(c1.data(), p1, w1_row, s1.data(), E, R1, H / 32, n_nt1, n_kc1, t1);
  tile_weights(c2.data(), p2, w2_row, s2.data(), E, H, Kw / 32, n_nt2, n_kc2, t2);
  std::vector<uint8_t>().swap(c1);
  std::vector<uint8_t>().swap(c2);

  // router weight as three bf16 planes whose sum is the fp32 value exactly
  std::vector<uint16_t> w3(static_cast<size_t>(3) * E * H);
  for (size_t i = 0; i < static_cast<size_t>(E) * H; ++i) {
    const float v = router_w[i];
    const uint16_t hi = f32_to_bf16_rn(v);
    const float r1 = v - bf16_to_f32(hi);
    const uint16_t mid = f32_to_bf16_rn(r1);
    const float r2 = r1 - bf16_to_f32(mid);
    const uint16_t lo = f32_to_bf16_rn(r2);
    w3[i] = hi;
    w3[static_cast<size_t>(E) * H + i] = mid;
    w3[static_cast<size_t>(2) * E * H + i] = lo;
  }

  int rc;
  if ((rc = dev_alloc(c, &w.w1_tiles, t1.size()))) return rc;
  if ((rc = dev_alloc(c, &w.w1_scales_raw, s1.size()))) return rc;
  if ((rc = dev_alloc(c, &w.b1, bb1.size()))) return rc;
  if ((rc = dev_alloc(c, &w.w2_tiles, t2.size()))) return rc;
  if ((rc = dev_alloc(c, &w.w2_scales_raw, s2.size()))) return rc;
  if ((rc = dev_alloc(c, &w.b2, static_cast<size_t>(E) * H))) return rc;
  if ((rc = dev_alloc(c, &w.router_w3, w3.size()))) return rc;
  if ((rc = dev_alloc(c, &w.router_b, static_cast<size_t>(E)))) return rc;
  CU_TRY(c, cudaMemcpy(w.w1_tiles, t1.data(), t1.size(), cudaMemcpyHostToDevice));
  CU_TRY(c, cudaMemcpy(w.w1_scales_raw, s1.data(), s1.size(), cudaMemcpyHostToDevice));
  CU_TRY(c, cudaMemcpy(w.b1, bb1.data(), bb1.size() * 2, cudaMemcpyHostToDevice));
  CU_TRY(c, cudaMemcpy(w.w2_tiles, t2.data(), t2.size(), cudaMemcpyHostToDevice));
  CU_TRY(c, cudaMemcpy(w.w2_scales_raw, s2.data(), s2.size(), cudaMemcpyHostToDevice));
  CU_TRY(c, cudaMemcpy(w.b2, b2, static_cast<size_t>(E) * H * 2, cudaMemcpyHostToDevice));
  CU_TRY(c, cudaMemcpy(w.router_w3, w3.data(), w3.size() * 2, cudaMemcpyHostToDevice));
  CU_TRY(c, cudaMemcpy(w.router_b, router_b, static_cast<size_t>(E) * 4, cudaMemcpyHostToDevice));
  if ((rc = make_weight_map(c, &w.tm_w1, w.w1_tiles, static_cast<size_t>(E) * n_nt1 * n_kc1))) return rc;
  if ((rc = make_weight_map(c, &w.tm_w2, w.w2_tiles, static_cast<size_t>(E) * n_nt2 * n_kc2))) return rc;
  if (!make_router_weight_map(&w.tm_router, w.router_w3, E, H))
    return fail(c, MOE_ERR_CUDA, "cuTensorMapEncodeTiled(router weight, %d x %d) failed", E, H);
  w.loaded = true;
  return MOE_OK;
}

int moe_route_topk(moe_handle c, const float *logits_dev, int rows, int *idx_dev, float *w_dev, void *stream) {
  if (!c || !logits_dev || !idx_dev || !w_dev || rows <= 0) return MOE_ERR_INVALID;
  CU_TRY(c, cudaSetDevice(c->cfg.device));
  launch_topk_softmax(const_cast<float *>(logits_dev), nullptr, 0, nullptr, rows, c->E, c->K, idx_dev, w_dev, nullptr,
                      static_cast<cudaStream_t>(stream));
  c->launches += 1;
  CU_TRY(c, cudaGetLastError());
  return MOE_OK;
}

int moe_forward(moe_handle c, int layer, const void *t_dev, int rows, void *out_dev, unsigned flags, void *stream) {
  if (!c) return MOE_ERR_INVALID;
  return forward_impl(c, layer, static_cast<const __nv_bfloat16 *>(t_dev), rows, static_cast<__nv_bfloat16 *>(out_dev),
                      flags, static_cast<cudaStream_t>(stream), nullptr, 0);
}

int moe_synchronize(moe_handle c) {
  if (!c) return MOE_ERR_INVALID;
  CU_TRY(c, cudaSetDevice(c->cfg.device));
  CU_TRY(c, cudaDeviceSynchronize());
  unsigned st = 0;
  CU_TRY(c, cudaMemcpy(&st, c->status, sizeof(st), cudaMemcpyDeviceToHost));
  if (st) {
    CU_TRY(c, cudaMemset(c->status, 0, sizeof(unsigned)));
    return fail(c, status_error(st), "device status word 0x%x", st);
  }
  return MOE_OK;
}

int moe_forward_host(moe_handle c, int layer, const void *t_host, int rows, void *out_host, unsigned flags) {
  if (!c) return MOE_ERR_INVALID;
  if (!t_host || !out_host || rows <= 0 || rows > c->max_rows) return fail(c, MOE_ERR_INVALID, "moe_forward_host: bad arguments");
  CU_TRY(c, cudaSetDevice(c->cfg.device));
  const size_t bytes = static_cast<size_t>(rows) * c->H * 2;
  CU_TRY(c, cudaMemcpyAsync(c->t_in, t_host, bytes, cudaMemcpyHostToDevice, c->stream));
  int rc = moe_forward(c, layer, c->t_in, rows, c->out_bf16, flags & ~MOE_FWD_PARTIAL_F32, c->stream);
  if (rc != MOE_OK) return rc;
  CU_TRY(c, cudaMemcpyAsync(out_host, c->out_bf16, bytes, cudaMemcpyDeviceToHost, c->stream));
  CU_TRY(c, cudaStreamSynchronize(c->stream));
  unsigned st = 0;
  CU_TRY(c, cudaMemcpy(&st, c->status, sizeof(st), cudaMemcpyDeviceToHost));
  if (st) {
    CU_TRY(c, cudaMemset(c->status, 0, sizeof(unsigned)));
    return fail(c, status_error(st), "device status word 0x%x", st);
  }
  return MOE_OK;
}

namespace {

// staging buffers, events and copy streams of the pipelined host entry points, made on first use
int host_pipeline_init(moe_ctx *c) {
  if (c->h2d_stream) return MOE_OK;
  CU_TRY(c, cudaStreamCreateWithFlags(&c->h2d_stream, cudaStreamNonBlocking));
  CU_TRY(c, cudaStreamCreateWithFlags(&c->d2h_stream, cudaStreamNonBlocking));
  const size_t n = static_cast<size_t>(c->max_rows) * c->H;
  for (HostSlot &hs : c->host_slots) {
    int rc;
    if ((rc = dev_alloc(c, &hs.in, n))) return rc;
    if ((rc = dev_alloc(c, &hs.out, n))) return rc;
    if ((rc = dev_alloc(c, &hs.status_dev, static_cast<size_t>(1)))) return rc;
    CU_TRY(c, cudaMemset(hs.status_dev, 0, sizeof(unsigned)));
    CU_TRY(c, cudaHostAlloc(reinterpret_cast<void **>(&hs.status_host), sizeof(unsigned), cudaHostAllocDefault));
    CU_TRY(c, cudaEventCreateWithFlags(&hs.in_ready, cudaEventDisableTiming));
    CU_TRY(c, cudaEventCreateWithFlags(&hs.out_ready, cudaEventDisableTiming));
    CU_TRY(c, cudaEventCreateWithFlags(&hs.done, cudaEventDisableTiming));
  }
  return MOE_OK;
}

int host_slot_finish(moe_ctx *c, HostSlot &hs) {
  CU_TRY(c, cudaEventSynchronize(hs.done));
  hs.ticket = -1;
  // the slot's own status word: what the kernels of THIS call recorded, whatever runs before or after it
  const unsigned st = *hs.status_host;
  if (st) return fail(c, status_error(st), "device status word 0x%x", st);
  return MOE_OK;
}

}  // namespace

int moe_forward_host_submit(moe_handle c, int layer, const void *t_host, int rows, void *out_host, unsigned flags,
                            long long *ticket) {
  if (!c) return MOE_ERR_INVALID;
  if (!t_host || !out_host || !ticket) return fail(c, MOE_ERR_INVALID, "moe_forward_host_submit: bad arguments");
  const int tp = c->cfg.tp_size;
  int rc = check_tp_call(c, rows, "moe_forward_host_submit");  // rows are this rank's rows
  if (rc != MOE_OK) return rc;
  if ((rc = host_pipeline_init(c)) != MOE_OK) return rc;
  HostSlot &hs = c->host_slots[c->host_submitted % kHostSlots];
  if (hs.ticket >= 0)
    return fail(c, MOE_ERR_STATE, "moe_forward_host_submit: %d calls in flight, wait for ticket %lld first", kHostSlots,
                hs.ticket);
  const size_t bytes = static_cast<size_t>(rows) * c->H * 2;
  // copy in | block | copy out, each on its own stream; the block of call n runs while call n+1 copies in and
  // call n-1 copies out
  CU_TRY(c, cudaMemcpyAsync(hs.in, t_host, bytes, cudaMemcpyHostToDevice, c->h2d_stream));
  CU_TRY(c, cudaEventRecord(hs.in_ready, c->h2d_stream));
  CU_TRY(c, cudaStreamWaitEvent(c->stream, hs.in_ready, 0));
  CU_TRY(c, cudaMemsetAsync(hs.status_dev, 0, sizeof(unsigned), c->stream));   // cleared in stream order, before the block
  if (tp > 1)
    rc = forward_impl(c, layer, static_cast<const __nv_bfloat16 *>(c->peers.gather[c->cfg.tp_rank]), rows * tp, hs.out,
                      flags & ~MOE_FWD_PARTIAL_F32, c->stream, hs.in, rows, nullptr, hs.status_dev);
  else
    rc = forward_impl(c, layer, hs.in, rows, hs.out, flags & ~MOE_FWD_PARTIAL_F32, c->stream, nullptr, 0, nullptr,
                      hs.status_dev);
  if (rc != MOE_OK) return rc;
  CU_TRY(c, cudaEventRecord(hs.out_ready, c->stream));
  CU_TRY(c, cudaStreamWaitEvent(c->d2h_stream, hs.out_ready, 0));
  CU_TRY(c, cudaMemcpyAsync(out_host, hs.out, bytes, cudaMemcpyDeviceToHost, c->d2h_stream));
  CU_TRY(c, cudaMemcpyAsync(hs.status_host, hs.status_dev, sizeof(unsigned), cudaMemcpyDeviceToHost, c->d2h_stream));
  CU_TRY(c, cudaEventRecord(hs.done, c->d2h_stream));
  hs.ticket = c->host_submitted;
  *ticket = c->host_submitted++;
  return MOE_OK;
}

int moe_forward_host_wait(moe_handle c, long long ticket) {
  if (!c) return MOE_ERR_INVALID;
  if (ticket < 0 || ticket >= c->host_submitted) return fail(c, MOE_ERR_INVALID, "moe_forward_host_wait: unknown ticket %lld", ticket);
  CU_TRY(c, cudaSetDevice(c->cfg.device));
  HostSlot &hs = c->host_slots[ticket % kHostSlots];
  if (hs.ticket != ticket) return MOE_OK;  // already waited for
  return host_slot_finish(c, hs);
}

int moe_profile_enable(moe_handle c, int on) {
  if (!c) return MOE_ERR_INVALID;
  c->profiling = on != 0;
  return MOE_OK;
}

int moe_profile_collect(moe_handle c, float *ms, int *n_calls) {
  if (!c || !ms || !n_calls) return MOE_ERR_INVALID;
  CU_TRY(c, cudaSetDevice(c->cfg.device));
  const size_t per = MOE_N_STAGES + 1;
  const size_t calls = c->prof_events.size() / per;
  for (int i = 0; i < MOE_N_STAGES; ++i) ms[i] = 0.f;
  for (size_t k = 0; k < calls; ++k) {
    CU_TRY(c, cudaEventSynchronize(c->prof_events[k * per + MOE_N_STAGES]));   // the last one is always recorded
    cudaEvent_t from = c->prof_events[k * per];
    for (int i = 0; i < MOE_N_STAGES; ++i) {
      cudaEvent_t to = c->prof_events[k * per + i + 1];
      if (to == nullptr) continue;   // an empty stage: 0 ms, the next stage starts where this one did
      float t = 0.f;
      CU_TRY(c, cudaEventElapsedTime(&t, from, to));
      ms[i] += t;
      from = to;
    }
  }
  for (cudaEvent_t e : c->prof_events)
    if (e != nullptr) c->prof_pool.push_back(e);
  c->prof_events.clear();
  *n_calls = static_cast<int>(calls);
  return MOE_OK;
}

void *moe_host_alloc(size_t bytes) {
  void *p = nullptr;
  if (cudaHostAlloc(&p, bytes, cudaHostAllocDefault) != cudaSuccess) return nullptr;
  return p;
}
void moe_host_free(void *p) {
  if (p) cudaFreeHost(p);
}

int moe_get_debug(moe_handle c, int which, void *dst, size_t bytes) {
  if (!c || !dst) return MOE_ERR_INVALID;
  CU_TRY(c, cudaSetDevice(c->cfg.device));
  const size_t T = c->last_rows;
  const void *src = nullptr;
  size_t have = 0;
  switch (which) {
    case MOE_DBG_LOGITS: src = c->logits; have = T * c->E * 4; break;
    case MOE_DBG_TOPK_IDX: src = c->topk_idx; have = T * c->K * 4; break;
    case MOE_DBG_TOPK_W: src = c->topk_w; have = T * c->K * 4; break;
    case MOE_DBG_COUNTS: src = c->counts; have = (size_t)c->E * 4; break;
    case MOE_DBG_OFFSETS: src = c->offsets; have = ((size_t)c->E + 1) * 4; break;
    case MOE_DBG_PAIR_ROW: src = c->pair_row; have = T * c->K * 4; break;
    case MOE_DBG_ROW_TOKEN: src = c->row_token; have = T * c->K * 4; break;
    case MOE_DBG_OUT_F32: src = c->out_f32; have = T * c->H * 4; break;
    case MOE_DBG_STATUS: src = c->status; have = 4096 * 4; break;
    case MOE_DBG_GATHER: src = c->t_in; have = static_cast<size_t>(c->max_rows) * c->H * 2; break;
    case MOE_DBG_TNORM: src = c->t_norm; have = static_cast<size_t>(c->max_rows) * c->H * 2; break;
    case MOE_DBG_YBUF: src = c->ybuf; have = T * c->K * c->H * 2; break;
    case MOE_DBG_TP_PARTIAL: src = c->tp_partial; have = static_cast<size_t>(c->max_rows) * c->H * 2; break;
    default: return fail(c, MOE_ERR_INVALID, "moe_get_debug: unknown item %d", which);
  }
  if (bytes > have) return fail(c, MOE_ERR_INVALID, "moe_get_debug: %zu bytes asked, %zu available", bytes, have);
  CU_TRY(c, cudaDeviceSynchronize());
  CU_TRY(c, cudaMemcpy(dst, src, bytes, cudaMemcpyDeviceToHost));
  return MOE_OK;
}

}  // extern "C"
