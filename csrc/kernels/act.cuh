// Activation functions and their derivatives, shared by the GEMM epilogues and the standalone
// elementwise kernels. Semantics follow machine_learning/src/arch/layers/{relu,sigmoid,tanh}.rs of
// the reference: derivatives are expressed in terms of the stored *activation* a (not the
// pre-activation), except GELU (not in the reference) whose derivative needs the pre-activation z.
#pragma once
#include <cuda_runtime.h>

namespace ono {

enum ActKind : int { ACT_NONE = 0, ACT_RELU = 1, ACT_SIGMOID = 2, ACT_TANH = 3, ACT_GELU = 4 };

__host__ __device__ __forceinline__ float act_fwd(int kind, float param, float x) {
  switch (kind) {
    case ACT_RELU: {
      // relu.rs:30-32: max(x, slope*x)
      float sx = param * x;
      return x > sx ? x : sx;
    }
    case ACT_SIGMOID:
      return param / (1.0f + expf(-x));  // sigmoid.rs:28-36
    case ACT_TANH:
      return param * tanhf(x);  // tanh.rs:28-38
    case ACT_GELU:
      return 0.5f * x * (1.0f + erff(x * 0.70710678118654752f));
    default:
      return x;
  }
}

// d * act'(.) given the stored value s (activation a; for GELU the pre-activation z).
// relu_quirk reproduces relu.rs:41-45, which overwrites d with slope*a where a <= 0.
__host__ __device__ __forceinline__ float act_bwd(int kind, float param, int relu_quirk, float s,
                                                  float d) {
  switch (kind) {
    case ACT_RELU:
      if (s > 0.0f) return d;
      return relu_quirk ? param * s : param * d;
    case ACT_SIGMOID:
      return d * s * (1.0f - s / param);  // sigmoid.rs:38-49
    case ACT_TANH:
      return d * (param - s * s / param);  // tanh.rs:40-51
    case ACT_GELU: {
      float cdf = 0.5f * (1.0f + erff(s * 0.70710678118654752f));
      float pdf = 0.3989422804014327f * expf(-0.5f * s * s);
      return d * (cdf + s * pdf);
    }
    default:
      return d;
  }
}

}  // namespace ono
