// Grouped expert GEMM for sm_100a: block-scaled tcgen05 MMA (kind::mxf8f6f4)
// that consumes the MXFP4 expert weights exactly as they lie in HBM, for MLP1
// (+bias, clamped SwiGLU) and MLP2 (+bias).
//
// Reference counterparts: grouped_mlp1_bf16_bias_kernel_tiled_optimized_outbf16
// and grouped_mlp2_... (getp-csrc/kernels/moe.hpp:2651, :2923, :3197) with
// swiglu_epilogue_kernel_bf16_mlp_in_bf16 (:1472) between them, fed by weights
// that the reference first expands to bf16 in a staging buffer
// (getp_run.cpp:1019-1086).  Here the packed 4-bit codes and their E8M0 scales
// go from HBM through TMA straight into the tensor core; no thread touches a
// weight.
//
// Why this shape.  Issuing a tcgen05.mma costs its thread ~47 cycles whatever its
// shape, a wait or a commit more than that, and the block-scaled kinds exist for
// M = 128 only, so what counts is MACs per instruction and per pipeline step:
// weights go on the N axis (240 rows per work item; 240 divides both 5760 and
// 2880 and leaves tensor memory for two accumulators) and the tokens of one
// expert on the M = 128 axis.  There is no
// bf16 x fp4 instruction, so every bf16 activation is split into two e4m3 terms
// (high + low, exact for bf16 inputs): a token tile is 64 tokens = 128 rows,
// row 2i the high term of token i, row 2i+1 its low term whose block scale
// carries the extra 2^-4.  The two partial sums land in adjacent lanes of the
// accumulator and are added in the epilogue.
//
// Per 128-element slice of k (one shared-memory stage) the producer warp
// issues: weight codes [240 rows x 128] (TMA, 16U4_ALIGN16B: 4-bit codes are
// expanded to the 8-bit containers the MMA reads, 128-byte swizzle), weight
// scales (two 512-byte atoms, pre-tiled at load time), activations [128 rows x
// 128] e4m3 (TMA, 128-byte swizzle).  The MMA warp copies the scale atoms to
// tensor memory (tcgen05.cp) and issues four K = 32 instructions.  Both warps
// stay converged and elect one lane per instruction group, so that descriptors
// and tensor-memory addresses live in uniform registers.  Sixteen epilogue
// warps drain the fp32 accumulator (double buffered: 2 x 240 columns).
// What bounds the kernel is the SM's shared-memory port (128 bytes per cycle,
// shared by the copy engine's writes and the tensor core's reads): an M128 N240
// K32 instruction moves 23.5 KB through it, 184 cycles against 120 of tensor pipe.
// No cluster launch, no multicast: every CTA fetches its own tiles.
#include <cuda_fp8.h>

#include "moe_internal.cuh"
#include "sm100_ptx.cuh"
#include "swiglu.cuh"

namespace moe {

using namespace sm100;

constexpr int kStages = 4;
constexpr int kABytes = kTileM * kChunkK;         // 16384: 128 rows x 128 e4m3
constexpr int kWBytes = kTileNPad * kChunkK;      // 32768: 256 rows x 128 containers (240 loaded)
// the transaction count of a 16U4_ALIGN16B copy is the PACKED size: 240 rows x 64 bytes
constexpr int kWLoadBytes = kTileN * kChunkK / 2; // 15360
constexpr int kStageBytes = kABytes + kWBytes + kSfbChunkBytes;  // 50176
constexpr int kSfaSlots = 4;                      // per-item activation scale atoms, a ring of their own
constexpr int kSfaOff = kStages * kStageBytes;
constexpr int kBarOff = kSfaOff + kSfaSlots * kSfAtomBytes;
constexpr int kNumBars = 2 * kStages + 4 + 2 * kSfaSlots;  // full, empty, d_full[2], d_empty[2], sfa_full, sfa_empty
constexpr int kSmemBytes = kBarOff + 8 * kNumBars + 16 + 1024 /*alignment slack*/;

constexpr int kEpiWarps = 16;             // four per tensor-memory lane quadrant
constexpr int kEpiChunks = 4;             // 16-column chunks per epilogue warp (15 in all)
constexpr int kProducerWarp = 16, kMmaWarp = 17;
constexpr int kThreads = 18 * 32;

constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kAccBufCols = kTileN;          // accumulator buffer d at columns d*240
constexpr uint32_t kSfaCol0 = 480;                // + 4*(item & 1)
constexpr uint32_t kSfbCol0 = 488;                // + 8*(chunk & 1)

static_assert(kStageBytes % 1024 == 0, "stages must keep 1024-byte alignment for the swizzled tiles");
static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");

__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float c, float d) {
  const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return lo | (hi << 16);
}
__device__ __forceinline__ float e4m3_to_float(uint32_t byte) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(byte), __NV_E4M3);
  return __half2float(*reinterpret_cast<const __half *>(&h));
}

__device__ __forceinline__ uint32_t ld_acquire_gpu(const unsigned int *p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// One launch runs the phases [f.phase_begin, f.phase_end): phase 0 = MLP1 (bias + SwiGLU -> e4m3 high/low
// rows, args pa), phase 1 = MLP2 (bias -> fp16, args pb).  Run together, the pipeline state (stage ring,
// accumulator buffers, scale slots) simply carries over from the last MLP1 item of a CTA to its first MLP2
// item: no drain, no second prologue, and CTAs that are out of MLP1 items start on MLP2 while the others
// finish.  An MLP2 item reads the SwiGLU rows of its token tile, which the MLP1 items of that tile (on any
// SM) have written: every epilogue warp counts a finished MLP1 item into tile_done[tile] behind a fence, and
// the producer waits (bounded) for the tile's count before it requests the tile's rows.  MLP1 items wait for
// nothing and every CTA is resident (one per SM), so the MLP2 waits always end.
__global__ void __launch_bounds__(kThreads, 1)
expert_gemm_kernel(const __grid_constant__ CUtensorMap tm_w1, const __grid_constant__ CUtensorMap tm_x1,
                   const __grid_constant__ CUtensorMap tm_w2, const __grid_constant__ CUtensorMap tm_x2,
                   const GemmArgs pa, const GemmArgs pb, const MlpFuse f) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bar_base = smem_base + kBarOff;
  volatile uint32_t *abort_flag = reinterpret_cast<volatile uint32_t *>(smem_gen + kBarOff + 8 * kNumBars);
  uint32_t *tmem_slot = const_cast<uint32_t *>(abort_flag) + 1;

  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
  auto dfull_bar = [&](int d) { return bar_base + 8u * (2 * kStages + d); };
  auto dempty_bar = [&](int d) { return bar_base + 8u * (2 * kStages + 2 + d); };
  auto sfa_full_bar = [&](int q) { return bar_base + 8u * (2 * kStages + 4 + q); };
  auto sfa_empty_bar = [&](int q) { return bar_base + 8u * (2 * kStages + 4 + kSfaSlots + q); };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int d = 0; d < 2; ++d) {
      mbar_init(dfull_bar(d), 1);
      mbar_init(dempty_bar(d), kEpiWarps);
    }
    for (int q = 0; q < kSfaSlots; ++q) { mbar_init(sfa_full_bar(q), 1); mbar_init(sfa_empty_bar(q), 1); }
    *abort_flag = 0u;
    fence_mbar_init();
    fence_proxy_async_smem();
  }
  if (warp == kMmaWarp) {
    tmem_alloc(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish();
  }
  if (warp == kProducerWarp && lane == 0) {
    if (f.phase_begin == 0) { prefetch_tensormap(&tm_w1); prefetch_tensormap(&tm_x1); }
    if (f.phase_end == 2) { prefetch_tensormap(&tm_w2); prefetch_tensormap(&tm_x2); }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // Items of a phase are dealt round-robin.  In a fused launch the MLP2 deal starts where the MLP1 deal
  // ended, so that the CTAs with one MLP1 item more are not also the ones with one MLP2 item more.
  const int n_work1 = *pa.n_work;
  auto first_item = [&](int phase) -> int {
    if (phase == 0 || f.phase_begin != 0) return static_cast<int>(blockIdx.x);
    const int g = static_cast<int>(gridDim.x);
    return (static_cast<int>(blockIdx.x) + g - n_work1 % g) % g;
  };
  unsigned int *status = pa.status;

  if (warp == kProducerWarp) {
    // ------------------------------------------------------------- TMA producer
    // The warp stays converged; one elected lane issues the copies.
    uint32_t item = 0, s = 0, e_par = 1u;   // a fresh stage passes the first wait
    bool ok = true;
    bool all_done = f.tile_done == nullptr;   // every MLP1 item of the launch is finished: no more checks
    const uint64_t w_policy = l2_policy_evict_first();
   for (int phase = f.phase_begin; ok && phase < f.phase_end; ++phase) {
    const bool second = phase != 0;
    const CUtensorMap *tm_w = second ? &tm_w2 : &tm_w1, *tm_x = second ? &tm_x2 : &tm_x1;
    const WorkItem *work = second ? pb.work : pa.work;
    const int n_work = second ? *pb.n_work : n_work1;
    const int nkc = second ? pb.n_kchunks : pa.n_kchunks, n_ntiles = second ? pb.n_ntiles : pa.n_ntiles;
    const uint8_t *sfa = second ? pb.sfa : pa.sfa, *w_tiles = second ? pb.w_tiles : pa.w_tiles;
    const int sfa_tile_stride = second ? pb.sfa_tile_stride : pa.sfa_tile_stride;
    const int first = first_item(phase);
    WorkItem w_next = {};
    if (first < n_work) w_next = work[first];
    for (int wi = first; ok && wi < n_work; wi += gridDim.x) {
      const WorkItem w = w_next;
      if (wi + static_cast<int>(gridDim.x) < n_work) w_next = work[wi + gridDim.x];
      for (int blk = 0; ok && blk < w.nblk; ++blk, ++item) {
        if (second && !all_done) {
          // the SwiGLU rows of this token tile: all MLP1 items of the tile (one per weight block; the index
          // kernel emits single-block items) must have been counted in by their 16 epilogue warps
          const long long t0 = clock64();
          for (uint32_t spin = 0;; ++spin) {
            const uint32_t total = __shfl_sync(0xffffffffu, ld_acquire_gpu(f.tile_done + f.total_slot), 0);
            if (total >= static_cast<uint32_t>(kEpiWarps) * static_cast<uint32_t>(n_work1)) { all_done = true; break; }
            const uint32_t mine = __shfl_sync(0xffffffffu, ld_acquire_gpu(f.tile_done + w.tile), 0);
            if (mine >= static_cast<uint32_t>(f.done_per_tile)) break;
            if ((spin & 15u) == 15u) {
              const bool late = __any_sync(0xffffffffu, clock64() - t0 > kWaitCycles);
              if (late || __any_sync(0xffffffffu, *abort_flag != 0u)) {
                if (late && lane == 0) { *abort_flag = 1u; atomicOr(status, ST_WAIT_AREADY); }
                ok = false;
                break;
              }
            }
          }
          if (!ok) break;
          // written with ordinary stores on other SMs, read by the copy engine here
          asm volatile("fence.proxy.async;" ::: "memory");
        }
        // activation scale atom of this token tile, through its own ring so that the producer never waits
        // for an epilogue; a slot is free once the MMAs of the item that used it are done
        const uint32_t q = item % kSfaSlots;
        if (!mbar_wait_warp(sfa_empty_bar(q), ((item / kSfaSlots) & 1u) ^ 1u, abort_flag, status, ST_WAIT_EMPTY)) { ok = false; break; }
        if (elect_one()) {
          mbar_arrive_expect_tx(sfa_full_bar(q), kSfAtomBytes);
          bulk_load(smem_base + kSfaOff + q * kSfAtomBytes, sfa + static_cast<size_t>(w.tile) * sfa_tile_stride,
                    kSfAtomBytes, sfa_full_bar(q));
        }
        const uint32_t tile0 = (static_cast<uint32_t>(w.expert) * n_ntiles + w.ntile + blk) * nkc;
        for (int kc = 0; kc < nkc; ++kc) {
          if (!mbar_wait_warp(empty_bar(s), e_par, abort_flag, status, ST_WAIT_EMPTY)) { ok = false; break; }
          const uint32_t stage = smem_base + s * kStageBytes;
          if (elect_one()) {
            mbar_arrive_expect_tx(full_bar(s), kABytes + kWLoadBytes + kSfbChunkBytes);
            // the weight tile first: it has the longer way (HBM; the activations come from L2).  Weights pass
            // through once per step: they must not push the activations and the results out of L2
            tma_load_3d_hint(stage + kABytes, tm_w, 0, 0, static_cast<int>(tile0 + kc), full_bar(s), w_policy);
            bulk_load_hint(stage + kABytes + kWBytes, w_tiles + static_cast<size_t>(tile0 + kc) * kWTileStride + kWTileCodes,
                           kSfbChunkBytes, full_bar(s), w_policy);
            tma_load_2d(stage, tm_x, 0, (w.tile * nkc + kc) * kTileM, full_bar(s));   // one contiguous 16 KB tile
          }
          if (++s == kStages) { s = 0; e_par ^= 1u; }
        }
      }
    }
   }
    if (!ok) {  // give copies in flight time to land before the CTA's shared memory is released
      for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------------------------------------- MMA issuer
    // The warp stays converged and one elected lane issues the tcgen05 instructions, so that their operands
    // live in uniform registers.  The weights and activations need no tcgen05 fence after their wait (copy
    // engine and tensor core meet through the mbarrier); the accumulator hand-over from the epilogue does.
    const uint32_t tm = __shfl_sync(0xffffffffu, tmem_base, 0);
    uint32_t item = 0, s = 0, f_par = 0, sfb_sel = 0;
    bool ok = true;
    const uint64_t desc_fixed = smem_desc_sw128(0);
   for (int phase = f.phase_begin; ok && phase < f.phase_end; ++phase) {
    const bool second = phase != 0;
    const WorkItem *work = second ? pb.work : pa.work;
    const int n_work = second ? *pb.n_work : n_work1;
    const int K = second ? pb.K : pa.K, nkc = second ? pb.n_kchunks : pa.n_kchunks;
    const int full_chunks = K / kChunkK, tail_steps = (K % kChunkK) / 32;
    const int first = first_item(phase);
    uint32_t nblk_next = 0;
    if (first < n_work) nblk_next = work[first].nblk;
    for (int wi = first; ok && wi < n_work; wi += gridDim.x) {
      const uint32_t nblk = nblk_next;
      if (wi + static_cast<int>(gridDim.x) < n_work) nblk_next = work[wi + gridDim.x].nblk;
      for (uint32_t blk = 0; ok && blk < nblk; ++blk, ++item) {
        const uint32_t d = item & 1u;
        if (!mbar_wait_warp(dempty_bar(d), ((item >> 1) & 1u) ^ 1u, abort_flag, status, ST_WAIT_DEMPTY)) { ok = false; break; }
        const uint32_t q = item % kSfaSlots;
        if (!mbar_wait_warp(sfa_full_bar(q), (item / kSfaSlots) & 1u, abort_flag, status, ST_WAIT_AREADY)) { ok = false; break; }
        tc_fence_after();
        const uint32_t sfa_t = tm + kSfaCol0 + 4 * d;
        if (elect_one()) tmem_cp_sf_atom(sfa_t, smem_base + kSfaOff + q * kSfAtomBytes);
        const uint32_t d_addr = tm + d * kAccBufCols;
        for (int kc = 0; kc < nkc; ++kc) {
          if (!mbar_wait_warp(full_bar(s), f_par, abort_flag, status, ST_WAIT_FULL)) { ok = false; break; }
          const uint32_t stage = smem_base + s * kStageBytes;
          const uint32_t sfb_t = tm + kSfbCol0 + 8 * sfb_sel;
          const uint64_t adesc = desc_fixed | (stage >> 4), bdesc = desc_fixed | ((stage + kABytes) >> 4);
          if (elect_one()) {
            tmem_cp_sf_atom(sfb_t, stage + kABytes + kWBytes);
            tmem_cp_sf_atom(sfb_t + 4, stage + kABytes + kWBytes + kSfAtomBytes);
            if (kc < full_chunks) {
              mma_mxf8f6f4_ss(d_addr, adesc, bdesc, idesc_mxf8f6f4_m128(kTileN, 0), kc != 0, sfa_t, sfb_t);
              mma_mxf8f6f4_ss(d_addr, adesc + 2, bdesc + 2, idesc_mxf8f6f4_m128(kTileN, 1), 1u, sfa_t, sfb_t);
              mma_mxf8f6f4_ss(d_addr, adesc + 4, bdesc + 4, idesc_mxf8f6f4_m128(kTileN, 2), 1u, sfa_t, sfb_t);
              mma_mxf8f6f4_ss(d_addr, adesc + 6, bdesc + 6, idesc_mxf8f6f4_m128(kTileN, 3), 1u, sfa_t, sfb_t);
            } else {
              for (int kb = 0; kb < tail_steps; ++kb)
                mma_mxf8f6f4_ss(d_addr, adesc + 2 * kb, bdesc + 2 * kb, idesc_mxf8f6f4_m128(kTileN, kb), (kc | kb) != 0,
                                sfa_t, sfb_t);
            }
            mma_commit(empty_bar(s));
          }
          if (++s == kStages) { s = 0; f_par ^= 1u; }
          sfb_sel ^= 1u;
        }
        if (ok && elect_one()) {
          mma_commit(dfull_bar(d));
          mma_commit(sfa_empty_bar(q));
        }
      }
    }
   }
  } else {
    // ------------------------------------------------------------- epilogue warps
    // Warp w reads tensor-memory lanes 32*(w%4).., i.e. accumulator rows 32q + l: token 16q + l/2, high
    // (even l) or low (odd l) term.  Warps 4g..4g+3 take the 16-column chunks 4g..4g+3 (15 chunks in all).
    // Loads are software pipelined: chunk c+1 is in flight while chunk c is processed.
    const int quad = warp & 3, half = warp >> 2;
    const uint32_t lane_field = static_cast<uint32_t>(quad * 32) << 16;
    const int odd = lane & 1;
    const int tok = quad * 16 + (lane >> 1);
    const float h_scale = exp2f(static_cast<float>(-pa.h_exp));
    uint32_t item = 0;
    bool ok = true;
   for (int phase = f.phase_begin; ok && phase < f.phase_end; ++phase) {
    const bool second = phase != 0;
    const WorkItem *work = second ? pb.work : pa.work;
    const int n_work = second ? *pb.n_work : n_work1;
    const int R = second ? pb.R : pa.R;
    const __nv_bfloat16 *bias = second ? pb.bias : pa.bias;
    const int first = first_item(phase);
    WorkItem w_next = {};
    if (first < n_work) w_next = work[first];
    for (int wi = first; ok && wi < n_work; wi += gridDim.x) {
     const WorkItem w = w_next;
     if (wi + static_cast<int>(gridDim.x) < n_work) w_next = work[wi + gridDim.x];  // in flight during the wait below
     for (int blk = 0; ok && blk < w.nblk; ++blk, ++item) {
      const uint32_t d = item & 1u;
      if (!mbar_wait(dfull_bar(d), (item >> 1) & 1u, abort_flag, status, ST_WAIT_DFULL)) { ok = false; break; }
      tc_fence_after();
      const int n0 = (w.ntile + blk) * kTileN;
      const bool tok_ok = tok < w.ntok;
      const __nv_bfloat16 *bias_row = bias + static_cast<size_t>(w.expert) * R;
      const uint32_t acc = tmem_base + lane_field + d * kAccBufCols;
      // chunks of this warp that hold rows of the matrix (rows past it are zero-filled and produce nothing)
      const int c_beg = half * kEpiChunks;
      const int c_end = min(min(c_beg + kEpiChunks, kTileN / 16), (R - n0 + 15) / 16);

      auto process = [&](const uint32_t (&v)[16], int c0) {
        // Sum of the high and low partial products of a token (adjacent lanes).  Each lane of the pair keeps 8
        // of the 16 columns: the even lane columns 0-7, the odd lane 8-15 (MLP1: whole gate/up pairs, 4 outputs
        // each; MLP2: 8 fp16 values, one 16-byte store, the pair's two stores fill one 32-byte sector).
        float tot[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int ce = i, co = i + 8;   // columns the even / the odd lane keeps
          const float fe = __uint_as_float(v[ce]), fo = __uint_as_float(v[co]);
          const float mine = odd ? fo : fe;
          const float give = odd ? fe : fo;
          tot[i] = mine + __shfl_xor_sync(0xffffffffu, give, 1);
        }
        if (!second) {
          const int nc = n0 + c0 + 8 * odd;  // first of this lane's 8 columns
          float b[8];
          if (nc < R) {
            const uint4 bv = __ldg(reinterpret_cast<const uint4 *>(bias_row + nc));
            const uint32_t bw[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              b[2 * i] = __uint_as_float(bw[i] << 16);
              b[2 * i + 1] = __uint_as_float(bw[i] & 0xffff0000u);
            }
          } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) b[i] = 0.f;
          }
          float hs[4];
#pragma unroll
          for (int i = 0; i < 4; ++i)
            hs[i] = swiglu_clamped(tot[2 * i] + b[2 * i], tot[2 * i + 1] + b[2 * i + 1], pa.limit, pa.alpha) * h_scale;
          const uint32_t hi4 = pack_e4m3x4(hs[0], hs[1], hs[2], hs[3]);
          float r[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) r[i] = (hs[i] - e4m3_to_float((hi4 >> (8 * i)) & 0xffu)) * 16.0f;
          const uint32_t lo4 = pack_e4m3x4(r[0], r[1], r[2], r[3]);
          const int j = pa.hq_joff + (nc >> 1);  // this lane's 4 intermediate features, as columns of MLP2's k window
          if (tok_ok && nc < R) {
            // MLP2's activation tiles: [tile][k slice][128 rows][128 bytes]
            uint8_t *dst = pa.hq_out + ((static_cast<size_t>(w.tile) * pa.hq_nkc + (j >> 7)) * kTileM + 2 * tok) * kChunkK + (j & 127);
            *reinterpret_cast<uint32_t *>(dst) = hi4;
            *reinterpret_cast<uint32_t *>(dst + kChunkK) = lo4;
          }
        } else {
          const int na = n0 + c0 + 8 * odd;  // first of this lane's 8 columns
          if (tok_ok && na < R) {          // R is a multiple of 32 here, so the whole chunk is inside
            float b[8];
            if (pb.add_bias) {
              const uint4 bv = __ldg(reinterpret_cast<const uint4 *>(bias_row + na));
              const uint32_t bw[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                b[2 * i] = __uint_as_float(bw[i] << 16);
                b[2 * i + 1] = __uint_as_float(bw[i] & 0xffff0000u);
              }
            } else {
#pragma unroll
              for (int i = 0; i < 8; ++i) b[i] = 0.f;
            }
            // fp16 keeps 11 significant bits of a value that the combine will round to 8; what it cannot hold
            // is a magnitude above 65504, which is reported, not stored silently as infinity
            uint32_t o[4];
            float big = 0.f;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float y0 = tot[2 * i] + b[2 * i], y1 = tot[2 * i + 1] + b[2 * i + 1];
              big = fmaxf(big, fmaxf(fabsf(y0), fabsf(y1)));
              const __half2 hh = __floats2half2_rn(y0, y1);
              o[i] = *reinterpret_cast<const uint32_t *>(&hh);
            }
            if (big > 65504.f) atomicOr(status, ST_Y_RANGE);
            __half *dst = pb.y_out + static_cast<size_t>(w.row0 + tok) * pb.ld_out + na;
            *reinterpret_cast<uint4 *>(dst) = make_uint4(o[0], o[1], o[2], o[3]);
          }
        }
      };

      uint32_t va[16], vb[16];
      int c = c_beg;
      if (c < c_end) tmem_ld16(acc + c * 16, va);
      while (c < c_end) {
        tmem_wait_ld();
        if (c + 1 < c_end) tmem_ld16(acc + (c + 1) * 16, vb);
        process(va, c * 16);
        if (++c >= c_end) break;
        tmem_wait_ld();
        if (c + 1 < c_end) tmem_ld16(acc + (c + 1) * 16, va);
        process(vb, c * 16);
        ++c;
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(dempty_bar(d));
      if (!second && f.tile_done != nullptr) {
        // this warp's SwiGLU rows of the item are written: fence by every lane, then one count per warp
        __threadfence();
        __syncwarp();
        if (lane == 0) {
          atomicAdd(f.tile_done + w.tile, 1u);
          atomicAdd(f.tile_done + f.total_slot, 1u);
        }
      }
     }
    }
   }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

cudaError_t expert_gemm_init() {
  return cudaFuncSetAttribute(expert_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
}

// Phases [f.phase_begin, f.phase_end) of the expert MLP in one launch: both in the usual call, one at a
// time (two launches, f.tile_done = nullptr) on request.
void launch_expert_mlp(const CUtensorMap &tm_w1, const CUtensorMap &tm_x1, const GemmArgs &a, const CUtensorMap &tm_w2,
                       const CUtensorMap &tm_x2, const GemmArgs &b, const MlpFuse &f, int grid, cudaStream_t s) {
  expert_gemm_kernel<<<grid, kThreads, kSmemBytes, s>>>(tm_w1, tm_x1, tm_w2, tm_x2, a, b, f);
}

int expert_mlp_done_per_tile(int n_ntiles1) { return kEpiWarps * n_ntiles1; }

}  // namespace moe
