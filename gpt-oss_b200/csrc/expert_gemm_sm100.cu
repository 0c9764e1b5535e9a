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
// Shape.  Weights go on the N axis (192 rows per work item; 192 divides both
// 5760 and 2880) and the tokens of one expert on the M = 128 axis.  There is no
// bf16 x fp4 instruction, so every bf16 activation is split into two e4m3 terms
// (high + low, exact for bf16 inputs): a token tile is 64 tokens = 128 rows,
// row 2i the high term of token i, row 2i+1 its low term whose block scale
// carries the extra 2^-4.  The two partial sums land in adjacent lanes of the
// accumulator and are added in the epilogue.
//
// What bounds this kernel is the shared-memory port of the SM (128 bytes per
// cycle): every operand byte that goes through shared memory is written once by
// the copy engine and read once by the tensor core, and the 4-bit weights occupy
// 8-bit containers there.  With both operands in shared memory an M128 N240 K32
// instruction moves 23.5 KB through that port (184 cycles) against 120 cycles of
// tensor pipe.  So only the weights use shared memory here.  The activations
// take the other road into the tensor core: four loader warps read the token
// tile's 128-byte k slices from global memory (L2) into registers and store them
// into TENSOR MEMORY (tcgen05.st), from where the MMA reads its A operand
// ([d], [a_tmem], b_desc form).  Tensor memory then holds two accumulators of 192
// columns (the epilogue of one work item overlaps the main loop of the next), a
// ring of three A slices of 32 columns, and the scale factors.
//
// Per 128-element slice of k the producer thread issues: weight codes [192 rows
// x 128] (TMA, 16U4_ALIGN16B: 4-bit codes are expanded to the 8-bit containers
// the MMA reads, 128-byte swizzle) and the tile's weight scales (two 512-byte
// atoms, pre-tiled at load time); eight stages of 25 KB.  The MMA thread copies
// the scale atoms to tensor memory (tcgen05.cp) and issues four K = 32
// instructions.  Twelve epilogue warps drain the fp32 accumulator.
//
// The issuing thread is the other scarce resource: measured on this part, four
// MMAs with their two scale copies and one commit cost it less than the 384
// cycles the tensor pipe needs for them, but every mbarrier wait adds ~150 cycles
// cycles the tensor pipe needs for them, but every mbarrier wait adds ~130 cycles
// and every scale copy or further commit ~45.  So a k slice costs it ONE wait,
// four MMAs and ONE commit: "slice i is ready" is a single barrier on which the
// four loader warps arrive once the slice's activations are in tensor memory, and
// on which a scale warp arrives (through a tcgen05.commit) once the slice's weight
// stage has landed and it has copied the stage's weight scales into tensor memory; the commit that frees weight stage i % 6 also frees A slot
// and scale slot i % 3 (loaders and scale warps wait on the weight ring's
// barriers).  Two scale warps take the even and the odd slices.
// No cluster launch, no multicast: every CTA fetches its own tiles.
#include <cuda_fp8.h>

#include "moe_internal.cuh"
#include "sm100_ptx.cuh"
#include "swiglu.cuh"

namespace moe {

using namespace sm100;

constexpr int kWStages = 8;                       // a multiple of kASlots: one barrier frees a stage and an A slot
constexpr int kWCodeBytes = kTileN * kChunkK;     // 20480: 160 rows x 128 containers
// the transaction count of a 16U4_ALIGN16B copy is the PACKED size: 160 rows x 64 bytes
constexpr int kWLoadBytes = kTileN * kChunkK / 2; // 10240
constexpr int kWStageBytes = kWCodeBytes + kSfbChunkBytes;  // 21504
constexpr int kASlots = 4;                        // k slices of the token tile in tensor memory
constexpr int kSfbSlots = 6;                      // weight-scale slots in tensor memory (8 columns each)
static_assert(kWStages % kASlots == 0 && kWStages >= 2 * kASlots, "slice it: weight stage it % kWStages, A slot it % kASlots");
static_assert(kSfbSlots <= kWStages, "a scale slot's previous user is found on the weight ring's barriers");
constexpr int kSfaSlots = 4;                      // per-item activation scale atoms, a ring of their own
constexpr int kSfaOff = kWStages * kWStageBytes;
constexpr int kBarOff = kSfaOff + kSfaSlots * kSfAtomBytes;
// w_full, w_empty (also "A slot free", "scale slot free"), ready, d_full[2], d_empty[2], sfa_full, sfa_empty
constexpr int kNumBars = 3 * kWStages + 4 + 2 * kSfaSlots;
constexpr int kSmemBytes = kBarOff + 8 * kNumBars + 16 + 1024 /*alignment slack*/;

constexpr int kEpiWarps = 8;              // two per tensor-memory lane quadrant
constexpr int kEpiChunks = 5;             // 16-column chunks per epilogue warp (10 in all)
constexpr int kLoaderWarp0 = 8;           // warps 8..15: lane quadrant = warp % 4, half of the slice's columns = (warp - 8) / 4
constexpr int kLoaderWarps = 8;
constexpr int kPrefetch = 4;              // k slices a loader thread has in flight (16 registers each)
constexpr int kProducerWarp = 16, kMmaWarp = 17;
constexpr int kScaleWarp0 = 18;           // warps 18, 19: weight scales of the even / the odd slices
constexpr int kThreads = 20 * 32;

constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kAccBufCols = kTileN;          // accumulator buffer d at columns d*160
constexpr uint32_t kACol0 = 2 * kTileN;           // 320: A slices, 32 columns (128 bytes per row) each
constexpr uint32_t kSfaCol0 = kACol0 + 32 * kASlots;  // 448, + 4*(item & 1)
constexpr uint32_t kSfbCol0 = kSfaCol0 + 8;       // 456, + 8*(slice % 6)

static_assert(kTileN % 16 == 0 && kTileN / 16 == (kEpiWarps / 4) * kEpiChunks, "epilogue warps cover the tile");
static_assert(kWStageBytes % 1024 == 0, "stages must keep 1024-byte alignment for the swizzled tiles");
static_assert(kSfbCol0 + 8 * kSfbSlots <= kTmemCols, "tensor memory budget");
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

#ifdef MOE_GEMM_TIMELINE
// one CTA's per-slice timestamps (timing experiments): int32 [180 slices][8] behind the cycle counters
#define TL_MARK(slice, which) \
  do { if (MODE == 1 && blockIdx.x == 0 && (slice) < 180u) \
         reinterpret_cast<int *>(p.status + 2624)[(slice) * 8 + (which)] = static_cast<int>(clock64()); } while (0)
#else
#define TL_MARK(slice, which)
#endif

template <int MODE>  // 1 = MLP1 (bias + SwiGLU -> e4m3 high/low rows), 2 = MLP2 (bias -> fp16)
__global__ void __launch_bounds__(kThreads, 1)
expert_gemm_kernel(const __grid_constant__ CUtensorMap tm_w, const GemmArgs p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bar_base = smem_base + kBarOff;
  volatile uint32_t *abort_flag = reinterpret_cast<volatile uint32_t *>(smem_gen + kBarOff + 8 * kNumBars);
  uint32_t *tmem_slot = const_cast<uint32_t *>(abort_flag) + 1;

  auto wfull_bar = [&](int s) { return bar_base + 8u * s; };
  auto wempty_bar = [&](int s) { return bar_base + 8u * (kWStages + s); };
  // "slice ready", one per weight stage (not per A slot): the scale warps run up to six slices ahead of the
  // loaders, and an early arrival for slice it + 4 must not be counted into the phase of slice it
  auto ready_bar = [&](int s) { return bar_base + 8u * (2 * kWStages + s); };
  constexpr int kB0 = 3 * kWStages;
  auto dfull_bar = [&](int d) { return bar_base + 8u * (kB0 + d); };
  auto dempty_bar = [&](int d) { return bar_base + 8u * (kB0 + 2 + d); };
  auto sfa_full_bar = [&](int q) { return bar_base + 8u * (kB0 + 4 + q); };
  auto sfa_empty_bar = [&](int q) { return bar_base + 8u * (kB0 + 4 + kSfaSlots + q); };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kWStages; ++s) { mbar_init(wfull_bar(s), 1); mbar_init(wempty_bar(s), 1); }
    for (int s = 0; s < kWStages; ++s) mbar_init(ready_bar(s), kLoaderWarps + 1);   // the loader warps + the scale copy
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
  if (warp == kProducerWarp && lane == 0) prefetch_tensormap(&tm_w);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int n_work = *p.n_work;
  const int K = p.K;
  const int nkc = p.n_kchunks;

  if (warp == kProducerWarp) {
    // ------------------------------------------------------------- TMA producer (weights, scales)
    // The warp stays converged; one elected lane issues the copies.
    uint32_t item = 0, s = 0, e_par = 1u;   // a fresh stage passes the first wait
    bool ok = true;
    const uint64_t w_policy = l2_policy_evict_first();
    WorkItem w_next = {};
    if (static_cast<int>(blockIdx.x) < n_work) w_next = p.work[blockIdx.x];
    for (int wi = blockIdx.x; ok && wi < n_work; wi += gridDim.x, ++item) {
      const WorkItem w = w_next;
      if (wi + static_cast<int>(gridDim.x) < n_work) w_next = p.work[wi + gridDim.x];
      // activation scale atom of this token tile, through its own ring so that the producer never waits
      // for an epilogue; a slot is free once the MMAs of the item that used it are done
      const uint32_t q = item % kSfaSlots;
      if (!mbar_wait_warp(sfa_empty_bar(q), ((item / kSfaSlots) & 1u) ^ 1u, abort_flag, p.status, ST_WAIT_EMPTY)) { ok = false; break; }
      if (elect_one()) {
        mbar_arrive_expect_tx(sfa_full_bar(q), kSfAtomBytes);
        bulk_load(smem_base + kSfaOff + q * kSfAtomBytes, p.sfa + static_cast<size_t>(w.tile) * p.sfa_tile_stride,
                  kSfAtomBytes, sfa_full_bar(q));
      }
      const uint32_t tile0 = (static_cast<uint32_t>(w.expert) * p.n_ntiles + w.ntile) * nkc;
      for (int kc = 0; kc < nkc; ++kc) {
        if (!mbar_wait_warp(wempty_bar(s), e_par, abort_flag, p.status, ST_WAIT_EMPTY)) { ok = false; break; }
        const uint32_t stage = smem_base + s * kWStageBytes;
        if (elect_one()) {
#ifdef MOE_GEMM_ABLATE_W_LOADS   // timing experiments only: the stage is declared full without any copy
          (void)stage; (void)w_policy; (void)tile0;
          mbar_arrive(wfull_bar(s));
#else
          mbar_arrive_expect_tx(wfull_bar(s), kWLoadBytes + kSfbChunkBytes);
          // Weights pass through once per step: they must not push the activations and the results out of L2
          tma_load_3d_hint(stage, &tm_w, 0, 0, static_cast<int>(tile0 + kc), wfull_bar(s), w_policy);
          bulk_load_hint(stage + kWCodeBytes, p.w_tiles + static_cast<size_t>(tile0 + kc) * kWTileStride + kWTileCodes,
                         kSfbChunkBytes, wfull_bar(s), w_policy);
#endif
        }
        if (++s == kWStages) { s = 0; e_par ^= 1u; }
      }
    }
    if (!ok) {  // give copies in flight time to land before the CTA's shared memory is released
      for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------------------------------------- MMA issuer
    // The warp stays converged and one elected lane issues the tcgen05 instructions, so that their operands
    // (descriptors, tensor-memory addresses) are computed once per warp in uniform registers.
    const uint32_t tm = __shfl_sync(0xffffffffu, tmem_base, 0);
    uint32_t item = 0;
    uint32_t s = 0, sl = 0, fsl = 0;   // ring positions, kept without divisions
    bool ok = true;
#ifdef MOE_GEMM_TRACE
    long long tr_total = clock64(), tr_afull = 0, tr_item = 0, tr_t;
#define TR_BEGIN() tr_t = clock64()
#define TR_END(acc) acc += clock64() - tr_t
#else
#define TR_BEGIN()
#define TR_END(acc)
#endif
    const uint64_t desc_fixed = smem_desc_sw128(0);
    const int full_chunks = K / kChunkK, tail_steps = (K % kChunkK) / 32;
    uint32_t r_par = 0;
#ifdef MOE_GEMM_TIMELINE
    uint32_t tl_it = 0;
#endif
    for (int wi = blockIdx.x; ok && wi < n_work; wi += gridDim.x, ++item) {
      const uint32_t d = item & 1u;
      TR_BEGIN();
      if (!mbar_wait_warp(dempty_bar(d), ((item >> 1) & 1u) ^ 1u, abort_flag, p.status, ST_WAIT_DEMPTY)) { ok = false; break; }
      const uint32_t q = item % kSfaSlots;
      if (!mbar_wait_warp(sfa_full_bar(q), (item / kSfaSlots) & 1u, abort_flag, p.status, ST_WAIT_AREADY)) { ok = false; break; }
      TR_END(tr_item);
      tc_fence_after();
      const uint32_t sfa_t = tm + kSfaCol0 + 4 * d;
      if (elect_one()) tmem_cp_sf_atom(sfa_t, smem_base + kSfaOff + q * kSfAtomBytes);
      const uint32_t d_addr = tm + d * kAccBufCols;
      for (int kc = 0; kc < nkc; ++kc) {
        // the slice's activations are in tensor memory, its weights in shared memory, its scales copied
        TR_BEGIN();
        if (!mbar_wait_warp(ready_bar(s), r_par, abort_flag, p.status, ST_WAIT_AREADY)) { ok = false; break; }
        TR_END(tr_afull);
#ifdef MOE_GEMM_TIMELINE
        if (lane == 0) TL_MARK(tl_it, 5);
#endif
        tc_fence_after();
        const uint32_t stage = smem_base + s * kWStageBytes;
        const uint32_t sfb_t = tm + kSfbCol0 + 8 * fsl;   // filled by a scale warp
        const uint64_t bdesc = desc_fixed | (stage >> 4);
        const uint32_t a_t = tm + kACol0 + 32 * sl;   // 8 columns (32 bytes per row) per k step
        if (elect_one()) {
          if (kc < full_chunks) {
            mma_mxf8f6f4_ts(d_addr, a_t, bdesc, idesc_mxf8f6f4_m128(kTileN, 0), kc != 0, sfa_t, sfb_t);
            mma_mxf8f6f4_ts(d_addr, a_t + 8, bdesc + 2, idesc_mxf8f6f4_m128(kTileN, 1), 1u, sfa_t, sfb_t);
            mma_mxf8f6f4_ts(d_addr, a_t + 16, bdesc + 4, idesc_mxf8f6f4_m128(kTileN, 2), 1u, sfa_t, sfb_t);
            mma_mxf8f6f4_ts(d_addr, a_t + 24, bdesc + 6, idesc_mxf8f6f4_m128(kTileN, 3), 1u, sfa_t, sfb_t);
          } else {
            for (int kb = 0; kb < tail_steps; ++kb)
              mma_mxf8f6f4_ts(d_addr, a_t + 8 * kb, bdesc + 2 * kb, idesc_mxf8f6f4_m128(kTileN, kb), (kc | kb) != 0,
                              sfa_t, sfb_t);
          }
          mma_commit(wempty_bar(s));   // frees weight stage s, A slot sl and (two slices later) the scale slot
        }
#ifdef MOE_GEMM_TIMELINE
        if (lane == 0) TL_MARK(tl_it, 6);
        ++tl_it;
#endif
        if (++s == kWStages) { s = 0; r_par ^= 1u; }
        if (++sl == kASlots) sl = 0;
        if (++fsl == kSfbSlots) fsl = 0;
      }
      if (ok && elect_one()) {
        mma_commit(dfull_bar(d));
        mma_commit(sfa_empty_bar(q));
      }
    }
#ifdef MOE_GEMM_TRACE
    if (lane == 0) {
      long long *tr = reinterpret_cast<long long *>(p.status + 64) + ((MODE - 1) * 160 + blockIdx.x) * 4;
      tr[0] = clock64() - tr_total; tr[1] = tr_afull; tr[2] = tr_item;
    }
#endif
  } else if (warp >= kScaleWarp0) {
    // ------------------------------------------------------------- weight-scale copies
    // Slice it (it = warp parity, +2, ...): once the scale slot's previous user (slice it - 6) is done and
    // the weight stage has landed, copy its two scale atoms into tensor-memory slot it % 6; the commit arrives
    // on the slice's "ready" barrier when the copies have completed.  Six slots let the copies run ahead of
    // the MMAs, off the critical path.
    // The warp stays converged (operands in uniform registers); one elected lane issues.
    {
      const uint32_t tm = __shfl_sync(0xffffffffu, tmem_base, 0);
      const int n_mine = static_cast<int>(blockIdx.x) < n_work ? (n_work - 1 - static_cast<int>(blockIdx.x)) / static_cast<int>(gridDim.x) + 1 : 0;
      const uint32_t total = static_cast<uint32_t>(n_mine) * static_cast<uint32_t>(nkc);
      for (uint32_t it = warp - kScaleWarp0; it < total; it += 2) {
        const uint32_t ws = it % kWStages;
        if (it >= kSfbSlots) {
          const uint32_t prev = it - kSfbSlots;
          if (!mbar_wait_warp(wempty_bar(prev % kWStages), (prev / kWStages) & 1u, abort_flag, p.status, ST_WAIT_AFREE)) break;
        }
        if (lane == 0) TL_MARK(it, 2);
        if (!mbar_wait_warp(wfull_bar(ws), (it / kWStages) & 1u, abort_flag, p.status, ST_WAIT_FULL)) break;
        if (lane == 0) TL_MARK(it, 3);
        tc_fence_after();
        const uint32_t sf_smem = smem_base + ws * kWStageBytes + kWCodeBytes;
        const uint32_t sfb_t = tm + kSfbCol0 + 8 * (it % kSfbSlots);
        if (elect_one()) {
          tmem_cp_sf_atom(sfb_t, sf_smem);
          tmem_cp_sf_atom(sfb_t + 4, sf_smem + kSfAtomBytes);
          mma_commit(ready_bar(ws));
        }
        if (lane == 0) TL_MARK(it, 4);
      }
    }
  } else if (warp >= kLoaderWarp0) {
    // ------------------------------------------------------------- activation loaders
    // Thread = half a row of the token tile: tensor-memory lane 32*(warp%4) + lane, columns 16*kh .. of the
    // slice's slot, kh = (warp - 8) / 4.  The activation tiles lie in global memory as [token tile][k slice]
    // [16-byte column c = 0..7][128 rows][16 bytes], so the four loads of a warp for one slice are four
    // contiguous 512-byte runs.  Four slices are in flight per thread (L2 answers in about a thousand cycles
    // under this load, a slice lasts a few hundred).
    const int q = warp & 3, kh = (warp - kLoaderWarp0) >> 2;
    const int row = q * 32 + lane;
    const uint32_t a_lane = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + kACol0 + 16 * kh;
    const int n_mine = static_cast<int>(blockIdx.x) < n_work ? (n_work - 1 - static_cast<int>(blockIdx.x)) / static_cast<int>(gridDim.x) + 1 : 0;
    const uint32_t total = static_cast<uint32_t>(n_mine) * static_cast<uint32_t>(nkc);
    const size_t slice_bytes = static_cast<size_t>(kTileM) * kChunkK;
    int l_wi = blockIdx.x, l_kc = 0;
    const uint8_t *l_base = nullptr;
    bool l_valid = false;
    auto l_open = [&]() {
      if (l_wi < n_work) {
        const WorkItem w = p.work[l_wi];
        l_base = p.act + static_cast<size_t>(w.tile) * nkc * slice_bytes + (4 * kh) * kActColBytes + row * 16;
        l_valid = row < 2 * w.ntok;   // rows past the tile's tokens are not read; their lanes get zeros
      } else {
        l_valid = false;
      }
    };
    auto l_fetch = [&](uint4 (&v)[4]) {
#ifdef MOE_GEMM_ABLATE_A_LOADS
      if (false) {
#else
      if (l_valid) {
#endif
        const uint8_t *src = l_base + static_cast<size_t>(l_kc) * slice_bytes;
#pragma unroll
        for (int c = 0; c < 4; ++c) v[c] = ld_nc_v4(src + c * kActColBytes);
      } else {
#pragma unroll
        for (int c = 0; c < 4; ++c) v[c] = make_uint4(0u, 0u, 0u, 0u);
      }
      if (++l_kc == nkc) {
        l_kc = 0;
        l_wi += gridDim.x;
        l_open();
      }
    };
    // Slice it: A slot it % 4, weight stage it % 8.  The slot is free once the MMAs of slice it - 4 are done,
    // which is the completion the MMA warp commits to the weight ring's barrier of stage (it - 4) % 8.
    uint32_t sl = 0, rs = 0;                        // A slot and "ready" barrier of the slice being stored
    uint32_t fs = kWStages - kASlots, f_par = 1u;   // stage whose "empty" barrier frees the slot; the first four pass
#ifdef MOE_GEMM_TRACE
    long long tr_lwait = 0, tr_t;
#endif
#ifdef MOE_GEMM_TIMELINE
    uint32_t tl_it = 0;
#endif
    auto a_step = [&](const uint4 (&v)[4]) -> bool {
      TR_BEGIN();
      const bool ok = mbar_wait_warp(wempty_bar(fs), f_par, abort_flag, p.status, ST_WAIT_AFREE);
      TR_END(tr_lwait);
      if (!ok) return false;   // a vote: tcgen05.st is warp-wide, the warp goes on or gives up together
#ifdef MOE_GEMM_TIMELINE
      if (threadIdx.x == kLoaderWarp0 * 32) TL_MARK(tl_it, 0);
#endif
      tc_fence_after();
#ifdef MOE_GEMM_ABLATE_A_USE   // timing experiments only: the loads are issued but zeros are stored
      {
        const uint4 z[4] = {make_uint4(0u, 0u, 0u, 0u), make_uint4(0u, 0u, 0u, 0u), make_uint4(0u, 0u, 0u, 0u), make_uint4(0u, 0u, 0u, 0u)};
        tmem_st16v(a_lane + 32 * sl, z);
      }
#else
      tmem_st16v(a_lane + 32 * sl, v);
#endif
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(ready_bar(rs));   // the scale warp's arrival on the same barrier vouches for the weights
#ifdef MOE_GEMM_TIMELINE
      if (threadIdx.x == kLoaderWarp0 * 32) TL_MARK(tl_it, 1);
      ++tl_it;
#endif
      if (++sl == kASlots) sl = 0;
      if (++rs == kWStages) rs = 0;
      if (++fs == kWStages) { fs = 0; f_par ^= 1u; }
      return true;
    };
    uint4 v0[4], v1[4], v2[4], v3[4];
    static_assert(kPrefetch == 4, "four register sets below");
    l_open();
    l_fetch(v0); l_fetch(v1); l_fetch(v2); l_fetch(v3);
    for (uint32_t it = 0; it < total; it += 4) {
      if (!a_step(v0)) break;
      l_fetch(v0);
      if (it + 1 >= total) break;
      if (!a_step(v1)) break;
      l_fetch(v1);
      if (it + 2 >= total) break;
      if (!a_step(v2)) break;
      l_fetch(v2);
      if (it + 3 >= total) break;
      if (!a_step(v3)) break;
      l_fetch(v3);
    }
#ifdef MOE_GEMM_TRACE
    if (threadIdx.x == kLoaderWarp0 * 32)
      (reinterpret_cast<long long *>(p.status + 64) + ((MODE - 1) * 160 + blockIdx.x) * 4)[3] = tr_lwait;
#endif
  } else {
    // ------------------------------------------------------------- epilogue warps
    // Warp w reads tensor-memory lanes 32*(w%4).., i.e. accumulator rows 32q + l: token 16q + l/2, high
    // (even l) or low (odd l) term.  Warps 4g..4g+3 take the 16-column chunks 5g..5g+4 (10 chunks in all).
    // Loads are software pipelined: chunk c+1 is in flight while chunk c is processed.
    const int quad = warp & 3, half = warp >> 2;
    const uint32_t lane_field = static_cast<uint32_t>(quad * 32) << 16;
    const int odd = lane & 1;
    const int tok = quad * 16 + (lane >> 1);
    const float h_scale = exp2f(static_cast<float>(-p.h_exp));
    uint32_t item = 0;
    bool ok = true;
    WorkItem w_next = {};
    if (static_cast<int>(blockIdx.x) < n_work) w_next = p.work[blockIdx.x];
    for (int wi = blockIdx.x; ok && wi < n_work; wi += gridDim.x, ++item) {
      const WorkItem w = w_next;
      if (wi + static_cast<int>(gridDim.x) < n_work) w_next = p.work[wi + gridDim.x];  // in flight during the wait below
      const uint32_t d = item & 1u;
      if (!mbar_wait(dfull_bar(d), (item >> 1) & 1u, abort_flag, p.status, ST_WAIT_DFULL)) { ok = false; break; }
      tc_fence_after();
      const int n0 = w.ntile * kTileN;
      const bool tok_ok = tok < w.ntok;
      const __nv_bfloat16 *bias_row = p.bias + static_cast<size_t>(w.expert) * p.R;
      const uint32_t acc = tmem_base + lane_field + d * kAccBufCols;
      // chunks of this warp that hold rows of the matrix (rows past it are zero-filled and produce nothing)
      const int c_beg = half * kEpiChunks;
      const int c_end = min(min(c_beg + kEpiChunks, kTileN / 16), (p.R - n0 + 15) / 16);

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
        if (MODE == 1) {
          const int nc = n0 + c0 + 8 * odd;  // first of this lane's 8 columns
          float b[8];
          if (nc < p.R) {
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
            hs[i] = swiglu_clamped(tot[2 * i] + b[2 * i], tot[2 * i + 1] + b[2 * i + 1], p.limit, p.alpha) * h_scale;
          const uint32_t hi4 = pack_e4m3x4(hs[0], hs[1], hs[2], hs[3]);
          float r[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) r[i] = (hs[i] - e4m3_to_float((hi4 >> (8 * i)) & 0xffu)) * 16.0f;
          const uint32_t lo4 = pack_e4m3x4(r[0], r[1], r[2], r[3]);
          const int j = p.hq_joff + (nc >> 1);  // this lane's 4 intermediate features, as columns of MLP2's k window
          if (tok_ok && nc < p.R) {
            // MLP2's activation tiles: [tile][k slice][16-byte column][128 rows][16 bytes]
            uint8_t *dst = p.hq_out + (static_cast<size_t>(w.tile) * p.hq_nkc + (j >> 7)) * (kTileM * kChunkK) +
                           ((j & 127) >> 4) * kActColBytes + (2 * tok) * 16 + (j & 15);
            *reinterpret_cast<uint32_t *>(dst) = hi4;
            *reinterpret_cast<uint32_t *>(dst + 16) = lo4;   // the low row follows
          }
        } else {
          const int na = n0 + c0 + 8 * odd;  // first of this lane's 8 columns
          if (tok_ok && na < p.R) {          // R is a multiple of 32 here, so the whole chunk is inside
            float b[8];
            if (p.add_bias) {
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
            if (big > 65504.f) atomicOr(p.status, ST_Y_RANGE);
            __half *dst = p.y_out + static_cast<size_t>(w.row0 + tok) * p.ld_out + na;
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
  cudaError_t e = cudaFuncSetAttribute(expert_gemm_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
  if (e != cudaSuccess) return e;
  return cudaFuncSetAttribute(expert_gemm_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
}

void launch_expert_gemm_mlp1(const CUtensorMap &tm_w, const GemmArgs &a, int grid, cudaStream_t s) {
  expert_gemm_kernel<1><<<grid, kThreads, kSmemBytes, s>>>(tm_w, a);
}
void launch_expert_gemm_mlp2(const CUtensorMap &tm_w, const GemmArgs &a, int grid, cudaStream_t s) {
  expert_gemm_kernel<2><<<grid, kThreads, kSmemBytes, s>>>(tm_w, a);
}

}  // namespace moe
