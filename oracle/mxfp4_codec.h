/*
 * TEST INFRASTRUCTURE ONLY. Nothing in the product library includes this file.
 *
 * MXFP4 decode shared by the CPU oracle and by the driver that feeds the
 * reference's own CPU forward().  The reference CPU path (run.cpp) works on
 * fp32 weights; its checkpoints are produced by dequantising MXFP4 tensors
 * with exactly this rule:
 *   - value table {0,.5,1,1.5,2,3,4,6} with bit 3 as sign
 *       getp-csrc/memory/mxfp4.hpp:7-10,
 *       export_model_bin/gpt-oss-120b/export_model_bin.py:80-97
 *   - byte idx>>1 holds two codes, LOW nibble = even element
 *       getp-csrc/memory/mxfp4.hpp:47-49,
 *       export_model_bin/gpt-oss-120b/export_model_bin.py:124-131
 *   - one E8M0 byte per 32 consecutive elements, scale = 2^(byte-127)
 *       getp-csrc/memory/mxfp4.hpp:20-24, :51-53
 */
#ifndef ORACLE_MXFP4_CODEC_H
#define ORACLE_MXFP4_CODEC_H

#include <math.h>
#include <stddef.h>
#include <stdint.h>

static const float ORACLE_E2M1_LUT[16] = {
    0.0f,  0.5f,  1.0f,  1.5f,  2.0f,  3.0f,  4.0f,  6.0f,
    -0.0f, -0.5f, -1.0f, -1.5f, -2.0f, -3.0f, -4.0f, -6.0f};

/* Dequantise n_elems (multiple of 32) consecutive elements. */
static inline void oracle_mxfp4_dequant_span(const uint8_t *codes,
                                             const uint8_t *scales,
                                             size_t n_elems, float *out) {
  for (size_t b = 0; b < n_elems / 32; ++b) {
    const float scale = ldexpf(1.0f, (int)scales[b] - 127);
    const uint8_t *c = codes + b * 16;
    float *o = out + b * 32;
    for (int i = 0; i < 16; ++i) {
      o[2 * i] = ORACLE_E2M1_LUT[c[i] & 0xF] * scale;
      o[2 * i + 1] = ORACLE_E2M1_LUT[c[i] >> 4] * scale;
    }
  }
}

#endif
