/*
 * TEST INFRASTRUCTURE ONLY: CPU restatement ("port") of the reference's MoE
 * block.  It is the checker for the CUDA path and the CPU baseline that
 * bench.py reports beside it; the product library never links, loads or calls
 * it.
 *
 * Pinning: tests/test_oracle.py compares this file, on seeded inputs, with
 * the reference's own forward() (run.cpp compiled unmodified into
 * oracle/_ref/libref_moe.so by oracle/Makefile), with the reference's own
 * quantiser source run on host threads (oracle/_ref/libref_mxfp4.so), and with
 * the committed outputs of those binaries under tests/golden/.
 *
 * Every function names the reference lines it restates (paths are relative to
 * the reference project root).  The arithmetic keeps the reference's exact
 * types and order: float products, double accumulators, float stores.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "mxfp4_codec.h"

#ifdef _OPENMP
#include <omp.h>
#endif

/* Weight decode: see mxfp4_codec.h for the reference lines. */
void oracle_mxfp4_dequant(const uint8_t *codes, const uint8_t *scales,
                          size_t n_elems, float *out) {
  const size_t nblk = n_elems / 32;
#pragma omp parallel for schedule(static)
  for (size_t b = 0; b < nblk; ++b)
    oracle_mxfp4_dequant_span(codes + b * 16, scales + b, 32, out + b * 32);
}

/* run.cpp:355-368 (matmul): W(out,in) @ x(in) with a double accumulator that
 * receives float products in ascending j. */
static inline float dot_f32_acc64(const float *w, const float *x, int n) {
  double val = 0.0f;
  for (int j = 0; j < n; ++j)
    val += w[j] * x[j];
  return (float)val;
}

/* run.cpp:320-333 (rmsnorm): double sum of float squares, eps 1e-5f,
 * 1/sqrtf, o = weight * (ss * x) evaluated in double, stored as float. */
void oracle_rmsnorm(const float *x, const float *weight, int T, int H,
                    float *out) {
  for (int t = 0; t < T; ++t) {
    const float *xr = x + (size_t)t * H;
    float *o = out + (size_t)t * H;
    double ss = 0.0f;
    for (int j = 0; j < H; ++j)
      ss += xr[j] * xr[j];
    ss /= H;
    ss += 1e-5f;
    ss = 1.0f / sqrtf(ss);
    for (int j = 0; j < H; ++j)
      o[j] = weight[j] * (ss * xr[j]);
  }
}

/* run.cpp:660-669: router_score = W_router @ t + b_router. */
void oracle_router_logits(const float *t, const float *wr, const float *br,
                          int T, int H, int E, float *logits) {
#pragma omp parallel for schedule(static)
  for (int tok = 0; tok < T; ++tok)
    for (int e = 0; e < E; ++e) {
      float v = dot_f32_acc64(wr + (size_t)e * H, t + (size_t)tok * H, H);
      v += br[e];
      logits[(size_t)tok * E + e] = v;
    }
}

/* run.cpp:387-420 (topk: sort descending by value, take the first K) followed
 * by run.cpp:335-353 (softmax) applied to the K selected values (run.cpp:674).
 * The reference's comparator returns 0 on equal values, which leaves the order
 * of exact ties to qsort; this restatement resolves them as the reference GPU
 * kernel does (getp-csrc/kernels/moe.hpp:333-342): the lower index wins. */
void oracle_topk_softmax(const float *logits, int T, int E, int K, int *idx,
                         float *w) {
#pragma omp parallel for schedule(static)
  for (int tok = 0; tok < T; ++tok) {
    const float *s = logits + (size_t)tok * E;
    int *ti = idx + (size_t)tok * K;
    float *tv = w + (size_t)tok * K;
    for (int k = 0; k < K; ++k) {
      int best = -1;
      for (int e = 0; e < E; ++e) {
        int taken = 0;
        for (int p = 0; p < k; ++p)
          taken |= (ti[p] == e);
        if (taken)
          continue;
        if (best < 0 || s[e] > s[best])
          best = e;
      }
      ti[k] = best;
      tv[k] = s[best];
    }
    /* softmax, run.cpp:335-353 */
    double max_val = tv[0];
    for (int i = 1; i < K; ++i)
      if (tv[i] > max_val)
        max_val = tv[i];
    double sum = 0.0f;
    for (int i = 0; i < K; ++i) {
      tv[i] = expf(tv[i] - max_val);
      sum += tv[i];
    }
    for (int i = 0; i < K; ++i)
      tv[i] /= sum;
  }
}

/* run.cpp:700-724: de-interleave (even row = gate, odd row = up), clamp the
 * gate from above only and the up value on both sides, then
 * gate * sigmoid(alpha*gate) * (up + 1), alpha = 1.702f. */
static inline float swiglu_ref(float val, float up_val, float limit) {
  const float alpha = 1.702f;
  if (val > limit)
    val = limit;
  if (up_val > limit)
    up_val = limit;
  if (up_val < -limit)
    up_val = -limit;
  val *= (1.0f / (1.0f + expf(-alpha * val)));
  val *= (up_val + 1.0f);
  return val;
}

/*
 * One MoE block for T tokens, run.cpp:657-748, from packed MXFP4 weights.
 *   t        [T,H]   normalised inputs (bf16 values widened to float)
 *   w1c/w1s  [E,2D,H/2] codes, [E,2D,H/32] scales;  b1 [E,2D]
 *   w2c/w2s  [E,H,D/2],        [E,H,D/32];          b2 [E,H]
 *   wr [E,H], br [E]
 * Outputs: logits [T,E], topk_i/topk_v [T,K], out [T,H] (= e_agg, the block
 * output before the residual add of run.cpp:744-747).
 *
 * The reference walks tokens one at a time and, inside a token, experts in
 * ascending index (run.cpp:678).  Here the loop nest is expert-major so each
 * weight row is decoded once, but every per-token value is produced by the
 * same operations in the same order: out[t] receives its experts' terms in
 * ascending expert index.
 * d0/d1 restrict the intermediate range to [d0,d1) (a tensor-parallel shard,
 * getp-csrc/getp_run.cpp:2488-2501; it need not fall on scale-block boundaries:
 * the enclosing whole blocks of an MLP2 row are decoded and the shard cut out); add_b2 = 0 leaves the MLP2 bias out so
 * that shard partials can be summed.  d0=0, d1=D, add_b2=1 is the full block.
 */
int oracle_moe_layer_shard(const float *t, int T, int H, int D, int E, int K,
                           float limit, const uint8_t *w1c, const uint8_t *w1s,
                           const float *b1, const uint8_t *w2c,
                           const uint8_t *w2s, const float *b2, const float *wr,
                           const float *br, int d0, int d1, int add_b2,
                           float *logits, int *topk_i, float *topk_v,
                           float *out) {
  if (H % 32 || D % 32 || d0 < 0 || d1 > D || d0 >= d1)
    return -1;
  oracle_router_logits(t, wr, br, T, H, E, logits);
  oracle_topk_softmax(logits, T, E, K, topk_i, topk_v);
  memset(out, 0, (size_t)T * H * sizeof(float));

  const int Dl = d1 - d0;
  int *tok = (int *)malloc((size_t)T * sizeof(int));
  float *wt = (float *)malloc((size_t)T * sizeof(float));
  float *mlp1 = (float *)malloc((size_t)T * 2 * Dl * sizeof(float));
  float *gu = (float *)malloc((size_t)T * Dl * sizeof(float));
  float *y = (float *)malloc((size_t)T * H * sizeof(float));
  if (!tok || !wt || !mlp1 || !gu || !y)
    return -2;

  for (int e = 0; e < E; ++e) {
    int n = 0;
    for (int tk = 0; tk < T; ++tk)
      for (int k = 0; k < K; ++k)
        if (topk_i[(size_t)tk * K + k] == e) {
          tok[n] = tk;
          wt[n] = topk_v[(size_t)tk * K + k];
          ++n;
          break;
        }
    if (!n)
      continue;
    const uint8_t *c1 = w1c + (size_t)e * 2 * D * (H / 2);
    const uint8_t *s1 = w1s + (size_t)e * 2 * D * (H / 32);
    const float *bb1 = b1 + (size_t)e * 2 * D;
    /* MLP1 + bias, run.cpp:691-699 (rows 2*d0 .. 2*d1) */
#pragma omp parallel
    {
      float *row = (float *)malloc((size_t)H * sizeof(float));
#pragma omp for schedule(static)
      for (int i = 0; i < 2 * Dl; ++i) {
        const int gi = 2 * d0 + i;
        oracle_mxfp4_dequant_span(c1 + (size_t)gi * (H / 2),
                                  s1 + (size_t)gi * (H / 32), H, row);
        for (int r = 0; r < n; ++r) {
          float v = dot_f32_acc64(row, t + (size_t)tok[r] * H, H);
          v += bb1[gi];
          mlp1[(size_t)r * 2 * Dl + i] = v;
        }
      }
      free(row);
    }
    /* SwiGLU, run.cpp:700-724 */
#pragma omp parallel for schedule(static)
    for (int r = 0; r < n; ++r)
      for (int j = 0; j < Dl; ++j)
        gu[(size_t)r * Dl + j] =
            swiglu_ref(mlp1[(size_t)r * 2 * Dl + 2 * j],
                       mlp1[(size_t)r * 2 * Dl + 2 * j + 1], limit);
    /* MLP2 + bias, run.cpp:726-736 (columns d0 .. d1) */
    const uint8_t *c2 = w2c + (size_t)e * H * (D / 2);
    const uint8_t *s2 = w2s + (size_t)e * H * (D / 32);
    const float *bb2 = b2 + (size_t)e * H;
#pragma omp parallel
    {
      const int k0 = d0 / 32 * 32, k1 = (d1 + 31) / 32 * 32;
      float *row = (float *)malloc((size_t)(k1 - k0) * sizeof(float));
#pragma omp for schedule(static)
      for (int i = 0; i < H; ++i) {
        oracle_mxfp4_dequant_span(c2 + (size_t)i * (D / 2) + k0 / 2,
                                  s2 + (size_t)i * (D / 32) + k0 / 32, k1 - k0, row);
        for (int r = 0; r < n; ++r) {
          float v = dot_f32_acc64(row + (d0 - k0), gu + (size_t)r * Dl, Dl);
          if (add_b2)
            v += bb2[i];
          y[(size_t)r * H + i] = v;
        }
      }
      free(row);
    }
    /* weighted aggregation, run.cpp:738-741 */
#pragma omp parallel for schedule(static)
    for (int r = 0; r < n; ++r) {
      float *o = out + (size_t)tok[r] * H;
      const float ew = wt[r];
      for (int i = 0; i < H; ++i)
        o[i] += y[(size_t)r * H + i] * ew;
    }
  }
  free(tok);
  free(wt);
  free(mlp1);
  free(gu);
  free(y);
  return 0;
}

int oracle_moe_layer(const float *t, int T, int H, int D, int E, int K,
                     float limit, const uint8_t *w1c, const uint8_t *w1s,
                     const float *b1, const uint8_t *w2c, const uint8_t *w2s,
                     const float *b2, const float *wr, const float *br,
                     float *logits, int *topk_i, float *topk_v, float *out) {
  return oracle_moe_layer_shard(t, T, H, D, E, K, limit, w1c, w1s, b1, w2c,
                                w2s, b2, wr, br, 0, D, 1, logits, topk_i,
                                topk_v, out);
}

/*
 * The reference's load-time quantiser, getp-csrc/memory/mxfp4.hpp:113-131
 * (encode helpers) and :139-217 (quantize_pack_mxfp4_block32_kernel): per 32
 * consecutive elements, exp = ilogb(max|v|) - 2 (0 for an all-zero block), the
 * scale byte is exp + 127 clamped to [0, 255], every element is divided by
 * 2^exp (the unclamped one) and takes the FIRST of the 16 table entries at the
 * smallest distance (strict '<' while scanning codes 0..15, so a value midway
 * between two magnitudes keeps the smaller one and -0.0 never wins over +0.0);
 * elements past n count as 0; low nibble = even element.
 * codes: ceil(n/32)*16 bytes, scales: ceil(n/32) bytes.
 */
void oracle_mxfp4_quantize(const float *src, size_t n, uint8_t *codes,
                           uint8_t *scales) {
  const size_t nblk = (n + 31) / 32;
#pragma omp parallel for schedule(static)
  for (size_t b = 0; b < nblk; ++b) {
    float v[32];
    float maxabs = 0.f;
    for (int i = 0; i < 32; ++i) {
      const size_t g = b * 32 + (size_t)i;
      v[i] = g < n ? src[g] : 0.0f;
      const float a = fabsf(v[i]);
      if (a > maxabs)
        maxabs = a;
    }
    int exp_scale = 0;
    if (maxabs > 0.f) {
      int e;
      frexpf(maxabs, &e);
      exp_scale = (e - 1) - 2;
    }
    int eb = exp_scale + 127;
    if (eb < 0)
      eb = 0;
    if (eb > 255)
      eb = 255;
    scales[b] = (uint8_t)eb;
    const float X = ldexpf(1.0f, exp_scale);
    uint8_t nib[32];
    for (int i = 0; i < 32; ++i) {
      const float x = v[i] / X;
      uint8_t best = 0;
      float best_diff = fabsf(x - ORACLE_E2M1_LUT[0]);
      for (uint8_t c = 1; c < 16; ++c) {
        const float d = fabsf(x - ORACLE_E2M1_LUT[c]);
        if (d < best_diff) {
          best_diff = d;
          best = c;
        }
      }
      nib[i] = best;
    }
    for (int i = 0; i < 16; ++i)
      codes[b * 16 + i] = (uint8_t)((nib[2 * i + 1] << 4) | (nib[2 * i] & 0xF));
  }
}

/* Round-to-nearest-even float -> bf16 -> float (finite inputs). */
static inline float round_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  u += 0x7fffu + ((u >> 16) & 1u);
  u &= 0xffff0000u;
  memcpy(&f, &u, 4);
  return f;
}

/*
 * The block as forward() wraps it, run.cpp:657-747: t = rmsnorm(x) * gain,
 * e_agg = MoE(t), x_out = x + e_agg (run.cpp:744-747).  With t_as_bf16 = 0 this
 * is the CPU reference to the bit.  The reference's GPU path keeps x and t in
 * bf16 (rmsnorm_kernel_bf16_io stores bf16, getp-csrc/kernels/rmsnorm.hpp:160;
 * accumulate_kernel_bf16, getp-csrc/kernels/other_kernels.hpp:18-37):
 * t_as_bf16 = 1 rounds t to bf16 before the router and the experts see it, and
 * the caller compares x_out within bf16 rounding.
 */
int oracle_moe_block(const float *x, const float *gain, int T, int H, int D,
                     int E, int K, float limit, const uint8_t *w1c,
                     const uint8_t *w1s, const float *b1, const uint8_t *w2c,
                     const uint8_t *w2s, const float *b2, const float *wr,
                     const float *br, int t_as_bf16, float *t_out,
                     float *logits, int *topk_i, float *topk_v, float *e_agg,
                     float *x_out) {
  oracle_rmsnorm(x, gain, T, H, t_out);
  if (t_as_bf16)
    for (size_t i = 0; i < (size_t)T * H; ++i)
      t_out[i] = round_bf16(t_out[i]);
  int rc = oracle_moe_layer(t_out, T, H, D, E, K, limit, w1c, w1s, b1, w2c, w2s,
                            b2, wr, br, logits, topk_i, topk_v, e_agg);
  if (rc)
    return rc;
  for (size_t i = 0; i < (size_t)T * H; ++i)
    x_out[i] = x[i] + e_agg[i];
  return 0;
}

int oracle_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* A launcher may export OMP_NUM_THREADS=1 to every child (torchrun does); the timed CPU baseline asks
 * for the host's cores explicitly. */
void oracle_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}
