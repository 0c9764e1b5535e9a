/*
 * TEST INFRASTRUCTURE ONLY.
 *
 * This text is NOT a translation unit of its own: oracle/Makefile pipes the
 * CPU part of the reference's run.cpp (everything above its tokenizer section,
 * read in place from the reference checkout, never copied into this
 * repository) into the compiler and appends this file, so that the code below
 * sees the reference's own Config / TransformerWeights / RunState /
 * Transformer types and calls its unmodified matmul(), topk() and forward()
 * (run.cpp:355-368, :387-420, :528-756).
 *
 * It builds, in memory, a one-layer model whose attention contributes exactly
 * zero (all attention weights and biases are 0, so run.cpp:646-655 adds 0 to
 * the residual stream), feeds the caller's already-normalised bf16 inputs
 * through the embedding table, and makes the FFN RMSNorm (run.cpp:657) an
 * identity for the row at hand (see pick_identity_norm below).
 * The MoE block of forward() (run.cpp:657-748) then runs as written, on fp32
 * expert weights that are the exact dequantisation of the packed MXFP4
 * tensors (what the reference's exporter produces,
 * export_model_bin/gpt-oss-120b/export_model_bin.py:100-137).
 */
#include <sys/mman.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#include <vector>

#include "mxfp4_codec.h"

namespace {

struct RefMoe {
  Transformer tr;
  int H, D, E, K;
  const uint8_t *w1c, *w1s, *w2c, *w2s;
  size_t w1_elems, w2_elems; /* per expert */
  std::vector<char> have;    /* expert already dequantised */
  std::vector<float> zeros_qkv_w, zeros_qkv_b, zeros_o_w, zeros_o_b, sinks,
      ones_h, gain, out_w, row_in;
  float *w1, *w2; /* mmap'ed, NORESERVE: untouched experts cost nothing */
  size_t w1_bytes, w2_bytes;
};

float *map_lazy(size_t bytes) {
  void *p = mmap(nullptr, bytes, PROT_READ | PROT_WRITE,
                 MAP_PRIVATE | MAP_ANONYMOUS | MAP_NORESERVE, -1, 0);
  return p == MAP_FAILED ? nullptr : reinterpret_cast<float *>(p);
}

void need_expert(RefMoe *m, int e) {
  if (m->have[e])
    return;
  const size_t n1 = m->w1_elems, n2 = m->w2_elems;
  const uint8_t *c1 = m->w1c + (size_t)e * n1 / 2, *s1 = m->w1s + (size_t)e * n1 / 32;
  const uint8_t *c2 = m->w2c + (size_t)e * n2 / 2, *s2 = m->w2s + (size_t)e * n2 / 32;
  float *o1 = m->w1 + (size_t)e * n1, *o2 = m->w2 + (size_t)e * n2;
#pragma omp parallel for schedule(static)
  for (size_t b = 0; b < n1 / 32; ++b)
    oracle_mxfp4_dequant_span(c1 + b * 16, s1 + b, 32, o1 + b * 32);
#pragma omp parallel for schedule(static)
  for (size_t b = 0; b < n2 / 32; ++b)
    oracle_mxfp4_dequant_span(c2 + b * 16, s2 + b, 32, o2 + b * 32);
  m->have[e] = 1;
}


/* Chooses an embedding row x' = x * 2^k (exact) and a constant RMSNorm gain g
 * such that the reference's rmsnorm (run.cpp:320-333) maps x' back onto x bit
 * for bit.  The float roundings inside rmsnorm make g*ss differ from 2^-k by
 * up to a few 2^-24, which can move an 8-bit-mantissa value by one float ulp,
 * so a handful of (k, g) candidates are tried against a prediction of what
 * rmsnorm will compute; ref_moe_forward() then verifies the real state.t. */
void pick_identity_norm(RefMoe *m, const float *row) {
  const int H = m->H;
  static const int ks[] = {0, 1, -1, 2, -2, 3, -3, 4, -4, 5, -5, 6, -6, 7, -7, 8, -8};
  float best_g = 1.0f; int best_k = 0; long best_bad = -1;
  for (int k : ks) {
    const float sc = ldexpf(1.0f, k);
    double ss = 0.0f;
    for (int j = 0; j < H; ++j) { float xs = row[j] * sc; ss += xs * xs; }
    ss /= H;
    ss += 1e-5f;
    ss = 1.0f / sqrtf(ss);
    const float g0 = (float)(ldexp(1.0, -k) / ss);
    float cands[5] = {g0, nextafterf(g0, 0.0f), nextafterf(g0, INFINITY), 0, 0};
    cands[3] = nextafterf(cands[1], 0.0f);
    cands[4] = nextafterf(cands[2], INFINITY);
    for (float g : cands) {
      long bad = 0;
      for (int j = 0; j < H; ++j) {
        float xs = row[j] * sc;
        float tj = g * (ss * xs);
        bad += (tj != row[j]);
      }
      if (best_bad < 0 || bad < best_bad) { best_bad = bad; best_g = g; best_k = k; }
      if (bad == 0) break;
    }
    if (best_bad == 0) break;
  }
  const float sc = ldexpf(1.0f, best_k);
  for (int j = 0; j < H; ++j) { m->row_in[j] = row[j] * sc; m->gain[j] = best_g; }
}

} // namespace

extern "C" {

/* Pointers are borrowed: the caller keeps the packed tensors, biases and
 * router arrays alive for the life of the handle. */
void *ref_moe_create(int H, int D, int E, int K, float swiglu_limit,
                     const uint8_t *w1c, const uint8_t *w1s, const float *b1,
                     const uint8_t *w2c, const uint8_t *w2s, const float *b2,
                     const float *wr, const float *br) {
  RefMoe *m = new RefMoe();
  m->H = H; m->D = D; m->E = E; m->K = K;
  m->w1c = w1c; m->w1s = w1s; m->w2c = w2c; m->w2s = w2s;
  m->w1_elems = (size_t)2 * D * H;
  m->w2_elems = (size_t)H * D;
  m->have.assign(E, 0);
  m->w1_bytes = (size_t)E * m->w1_elems * sizeof(float);
  m->w2_bytes = (size_t)E * m->w2_elems * sizeof(float);
  m->w1 = map_lazy(m->w1_bytes);
  m->w2 = map_lazy(m->w2_bytes);
  if (!m->w1 || !m->w2) { delete m; return nullptr; }

  Config &c = m->tr.config;
  memset(&c, 0, sizeof(c));
  c.vocab_size = 1;           /* logits matmul shrinks to one zero row */
  c.hidden_dim = H;
  c.n_experts = E;
  c.experts_per_token = K;
  c.intermediate_dim = D;
  c.n_layers = 1;
  c.head_dim = 2;
  c.n_attn_heads = 1;
  c.n_kv_heads = 1;
  c.seq_len = 2;
  c.initial_context_length = 4096;
  c.rope_theta = 150000.0f;
  c.rope_scaling_factor = 1.0f; /* plain RoPE branch, no YaRN assert */
  c.sliding_window = 0;
  c.swiglu_limit = swiglu_limit;

  const int qkv_rows = c.head_dim * (c.n_attn_heads + 2 * c.n_kv_heads);
  m->zeros_qkv_w.assign((size_t)qkv_rows * H, 0.0f);
  m->zeros_qkv_b.assign(qkv_rows, 0.0f);
  m->zeros_o_w.assign((size_t)H * c.head_dim * c.n_attn_heads, 0.0f);
  m->zeros_o_b.assign(H, 0.0f);
  m->sinks.assign(c.n_attn_heads, 0.0f);
  m->ones_h.assign(H, 1.0f);
  m->gain.assign(H, 1.0f);
  m->out_w.assign(H, 0.0f);
  m->row_in.assign(H, 0.0f);

  TransformerWeights &w = m->tr.weights;
  memset(&w, 0, sizeof(w));
  w.token_embedding_table = m->row_in.data();
  w.rms_attn_w = m->ones_h.data();
  w.rms_ffn_w = m->gain.data();
  w.w_qkv = m->zeros_qkv_w.data();
  w.w_o = m->zeros_o_w.data();
  w.b_qkv = m->zeros_qkv_b.data();
  w.b_o = m->zeros_o_b.data();
  w.attn_sinks = m->sinks.data();
  w.w_router = const_cast<float *>(wr);
  w.b_router = const_cast<float *>(br);
  w.w_mlp1 = m->w1;
  w.w_mlp2 = m->w2;
  w.b_mlp1 = const_cast<float *>(b1);
  w.b_mlp2 = const_cast<float *>(b2);
  w.rms_out_w = m->ones_h.data();
  w.out = m->out_w.data();
  m->tr.fd = -1;
  m->tr.data = nullptr;
  m->tr.file_size = 0;
  malloc_run_state(&m->tr.state, &c);
  return m;
}

void ref_moe_destroy(void *h) {
  RefMoe *m = reinterpret_cast<RefMoe *>(h);
  if (!m) return;
  free_run_state(&m->tr.state);
  munmap(m->w1, m->w1_bytes);
  munmap(m->w2, m->w2_bytes);
  delete m;
}

/* Dequantise (as the exporter would have) every expert that the reference's
 * own router + topk select for these rows, so that forward() can be timed
 * without the decode.  Returns the number of distinct experts touched. */
int ref_moe_prepare(void *h, const float *t_rows, int T) {
  RefMoe *m = reinterpret_cast<RefMoe *>(h);
  RunState *s = &m->tr.state;
  TransformerWeights *w = &m->tr.weights;
  for (int i = 0; i < T; ++i) {
    memcpy(s->t, t_rows + (size_t)i * m->H, (size_t)m->H * sizeof(float));
    matmul(s->router_score, s->t, w->w_router, m->H, m->E);
    for (int e = 0; e < m->E; ++e) s->router_score[e] += w->b_router[e];
    topk(s->topk_v, s->topk_i, s->router_score, m->E, m->K);
    for (int k = 0; k < m->K; ++k) need_expert(m, s->topk_i[k]);
  }
  int n = 0;
  for (int e = 0; e < m->E; ++e) n += m->have[e];
  return n;
}

/* Runs the reference forward() once per row.  Returns the number of elements
 * of state.t that differ from the injected input (must be 0 for the identity
 * RMSNorm trick to hold); a negative value is an error. */
long ref_moe_forward(void *h, const float *t_rows, int T, float *logits,
                     int *topk_i, float *topk_v, float *out) {
  RefMoe *m = reinterpret_cast<RefMoe *>(h);
  RunState *s = &m->tr.state;
  const int H = m->H;
  long mismatches = 0;
  for (int i = 0; i < T; ++i) {
    const float *row = t_rows + (size_t)i * H;
    pick_identity_norm(m, row);
    forward(&m->tr, /*token=*/0, /*pos=*/0);
    for (int j = 0; j < H; ++j) mismatches += (s->t[j] != row[j]);
    if (logits) memcpy(logits + (size_t)i * m->E, s->router_score, (size_t)m->E * sizeof(float));
    if (topk_i) memcpy(topk_i + (size_t)i * m->K, s->topk_i, (size_t)m->K * sizeof(int));
    if (topk_v) memcpy(topk_v + (size_t)i * m->K, s->topk_v, (size_t)m->K * sizeof(float));
    if (out) memcpy(out + (size_t)i * H, s->e_agg, (size_t)H * sizeof(float));
  }
  return mismatches;
}

/* The block with its real RMSNorm: row x and gain vector go in as they are
 * (no identity trick), forward() normalises (run.cpp:657), runs the MoE and
 * adds the residual.  state.t and state.e_agg are read back; state.x is not,
 * because the final rmsnorm (run.cpp:750) overwrites it in place. */
void ref_moe_forward_block(void *h, const float *x_rows, const float *gain, int T,
                           float *t_out, float *logits, int *topk_i, float *topk_v,
                           float *e_agg) {
  RefMoe *m = reinterpret_cast<RefMoe *>(h);
  RunState *s = &m->tr.state;
  const int H = m->H;
  memcpy(m->gain.data(), gain, (size_t)H * sizeof(float));
  for (int i = 0; i < T; ++i) {
    memcpy(m->row_in.data(), x_rows + (size_t)i * H, (size_t)H * sizeof(float));
    /* experts are dequantised on demand: route the row first, as forward() will */
    rmsnorm(s->t, m->row_in.data(), m->gain.data(), H);
    matmul(s->router_score, s->t, m->tr.weights.w_router, H, m->E);
    for (int e = 0; e < m->E; ++e) s->router_score[e] += m->tr.weights.b_router[e];
    topk(s->topk_v, s->topk_i, s->router_score, m->E, m->K);
    for (int k = 0; k < m->K; ++k) need_expert(m, s->topk_i[k]);
    forward(&m->tr, /*token=*/0, /*pos=*/0);
    memcpy(t_out + (size_t)i * H, s->t, (size_t)H * sizeof(float));
    if (logits) memcpy(logits + (size_t)i * m->E, s->router_score, (size_t)m->E * sizeof(float));
    if (topk_i) memcpy(topk_i + (size_t)i * m->K, s->topk_i, (size_t)m->K * sizeof(int));
    if (topk_v) memcpy(topk_v + (size_t)i * m->K, s->topk_v, (size_t)m->K * sizeof(float));
    memcpy(e_agg + (size_t)i * H, s->e_agg, (size_t)H * sizeof(float));
  }
}

int ref_moe_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* A launcher may export OMP_NUM_THREADS=1 to every child (torchrun does); the timed run asks for the
 * host's cores explicitly. */
void ref_moe_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

} // extern "C"
