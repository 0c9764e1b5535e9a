// Checkpoint ingest from the reference's flat fp32 file: a Config header (run.cpp:25-45, fifteen 4-byte fields)
// followed by the tensors in the order of memory_map_weights (run.cpp:206-247), as
// export_model_bin/gpt-oss-120b/export_model_bin.py writes them.  Only the MoE tensors of one layer are read
// (the file is mapped, not copied); they are quantised to MXFP4 on the GPU exactly as moe_load_layer_f32 does,
// which is what the reference runtime does with the same bytes (copy_weights_to_gpu_120b,
// getp_run.cpp:1480-1718).
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstdio>
#include <cstring>

#include "moe_internal.cuh"

namespace {
// field order of the reference's Config
enum { kVocab, kHidden, kExperts, kTopK, kInter, kLayers, kHeadDim, kAttnHeads, kKvHeads, kSeqLen, kInitCtx,
       kRopeTheta, kRopeScale, kWindow, kSwigluLimit, kHeaderFields };
}  // namespace

extern "C" {

int moe_bin_layer_offsets(const int32_t *hdr, int layer, long long off[MOE_BIN_N_TENSORS], long long *total_floats) {
  if (!hdr || !off) return MOE_ERR_INVALID;
  const long long V = hdr[kVocab], H = hdr[kHidden], E = hdr[kExperts], D = hdr[kInter], L = hdr[kLayers];
  const long long hd = hdr[kHeadDim], nq = hdr[kAttnHeads], nkv = hdr[kKvHeads];
  if (V <= 0 || H <= 0 || E <= 0 || D <= 0 || L <= 0 || hd <= 0 || nq <= 0 || nkv <= 0 || layer < 0 || layer >= L)
    return MOE_ERR_INVALID;
  long long p = kHeaderFields;                 // in floats from the start of the file
  p += V * H;                                  // token_embedding_table
  p += V * H;                                  // out
  p += L * H;                                  // rms_attn_w
  off[MOE_BIN_RMS_FFN_W] = p + layer * H;      // rms_ffn_w [L, H]
  p += L * H;
  p += H;                                      // rms_out_w
  const long long qkv = hd * nq + 2 * hd * nkv;
  p += L * H * qkv;                            // w_qkv
  p += L * qkv;                                // b_qkv
  p += L * (hd * nq) * H;                      // w_o
  p += L * H;                                  // b_o
  p += L * nq;                                 // attn_sinks
  off[MOE_BIN_ROUTER_W] = p + layer * H * E;   // w_router [L, E, H]
  p += L * H * E;
  off[MOE_BIN_ROUTER_B] = p + layer * E;       // b_router [L, E]
  p += L * E;
  off[MOE_BIN_W_MLP1] = p + layer * E * 2 * D * H;   // w_mlp1 [L, E, 2D, H], rows gate/up interleaved
  p += L * E * 2 * D * H;
  off[MOE_BIN_B_MLP1] = p + layer * E * 2 * D;
  p += L * E * 2 * D;
  off[MOE_BIN_W_MLP2] = p + layer * E * H * D;       // w_mlp2 [L, E, H, D]
  p += L * E * H * D;
  off[MOE_BIN_B_MLP2] = p + layer * E * H;
  p += L * E * H;
  if (total_floats) *total_floats = p;
  return MOE_OK;
}

int moe_load_layer_from_bin(moe_handle c, int layer, const char *path, int file_layer, float *rms_ffn_w_out) {
  if (!c || !path) return MOE_ERR_INVALID;
  auto fail = [&](int code, const char *what) {
    char buf[400];
    snprintf(buf, sizeof(buf), "moe_load_layer_from_bin(%s): %s", path, what);
    c->err = buf;
    return code;
  };
  const int fd = open(path, O_RDONLY);
  if (fd < 0) return fail(MOE_ERR_INVALID, "cannot open the file");
  struct stat st;
  if (fstat(fd, &st) != 0 || st.st_size < static_cast<off_t>(kHeaderFields * 4)) { close(fd); return fail(MOE_ERR_INVALID, "file shorter than its header"); }
  void *map = mmap(nullptr, static_cast<size_t>(st.st_size), PROT_READ, MAP_PRIVATE, fd, 0);
  close(fd);
  if (map == MAP_FAILED) return fail(MOE_ERR_NOMEM, "mmap failed");
  const int32_t *hdr = static_cast<const int32_t *>(map);
  const float *f = static_cast<const float *>(map);
  long long off[MOE_BIN_N_TENSORS], total = 0;
  int rc = moe_bin_layer_offsets(hdr, file_layer, off, &total);
  if (rc != MOE_OK) rc = fail(MOE_ERR_INVALID, "bad header or layer index");
  else if (hdr[kHidden] != c->H || hdr[kExperts] != c->E || hdr[kInter] != c->D || hdr[kTopK] != c->K)
    rc = fail(MOE_ERR_INVALID, "header dimensions differ from the handle's (hidden, experts, intermediate, top-k)");
  else if (total * 4 > static_cast<long long>(st.st_size))
    rc = fail(MOE_ERR_INVALID, "file shorter than its header promises");
  else {
    float limit;
    memcpy(&limit, &hdr[kSwigluLimit], 4);
    if (limit != c->cfg.swiglu_limit) rc = fail(MOE_ERR_INVALID, "swiglu_limit of the file differs from the handle's");
  }
  if (rc == MOE_OK) {
    if (rms_ffn_w_out) memcpy(rms_ffn_w_out, f + off[MOE_BIN_RMS_FFN_W], static_cast<size_t>(c->H) * 4);
    rc = moe_load_layer_f32(c, layer, f + off[MOE_BIN_W_MLP1], f + off[MOE_BIN_B_MLP1], f + off[MOE_BIN_W_MLP2],
                            f + off[MOE_BIN_B_MLP2], f + off[MOE_BIN_ROUTER_W], f + off[MOE_BIN_ROUTER_B]);
  }
  munmap(map, static_cast<size_t>(st.st_size));
  return rc;
}

}  // extern "C"
