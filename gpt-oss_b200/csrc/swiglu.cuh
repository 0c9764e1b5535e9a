// Clamped SwiGLU of the GPT-OSS expert MLP, in the reference CPU path's order of
// operations (run.cpp:706-722): the gate is clamped from above only, the up
// value on both sides, then gate * sigmoid(alpha * gate) * (up + 1).  (The
// reference GPU kernel also clamps the gate from below, kernels/moe.hpp:1489;
// parity is defined against the CPU path.)  Explicit round-to-nearest
// intrinsics keep the compiler from fusing the multiply-adds differently from
// the CPU code.
#pragma once
#include <cuda_runtime.h>

namespace moe {

__device__ __forceinline__ float swiglu_clamped(float gate, float up, float limit, float alpha) {
  gate = fminf(gate, limit);
  up = fminf(fmaxf(up, -limit), limit);
  const float sig = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(__fmul_rn(-alpha, gate))));
  return __fmul_rn(__fmul_rn(gate, sig), __fadd_rn(up, 1.0f));
}

}  // namespace moe
