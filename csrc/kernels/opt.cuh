// Optimizer update shared by every kernel that applies one: the flat-shard optimizer, the fused
// synchronisation kernels and the weight-gradient GEMM epilogue that updates its own tile.
// Semantics: machine_learning/src/optimization/{gradient_descent,gradient_descent_with_momentum,adam}.rs
// of the reference (Adam keeps epsilon outside the bias correction, adam.rs:75-91).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ono {

struct OptScal {
  int kind;            // 0 SGD, 1 momentum, 2 Adam
  float lr, mu, b1, b2, eps;
  float gs;            // the gradient is multiplied by this first (1 / workers)
  float adam_step;     // lr * sqrt(1 - b2^t) / (1 - b1^t)
};

__device__ __forceinline__ float opt_apply(const OptScal& s, float p, float g, float& m, float& v) {
  g *= s.gs;
  if (s.kind == 0) return p - s.lr * g;
  if (s.kind == 1) {
    m = s.mu * m + g;
    return p - s.lr * m;
  }
  m = s.b1 * m + (1.0f - s.b1) * g;
  v = s.b2 * v + (1.0f - s.b2) * g * g;
  return p - s.adam_step * m / (sqrtf(v) + s.eps);
}

__device__ __forceinline__ float4 opt_apply4(const OptScal& s, float4 p, float4 g, float4& m, float4& v) {
  p.x = opt_apply(s, p.x, g.x, m.x, v.x);
  p.y = opt_apply(s, p.y, g.y, m.y, v.y);
  p.z = opt_apply(s, p.z, g.z, m.z, v.z);
  p.w = opt_apply(s, p.w, g.w, m.w, v.w);
  return p;
}

// Two f32 values -> one 32-bit word of two 16-bit floats (bf16, or IEEE f16 when `f16` is set), round to nearest.
__device__ __forceinline__ uint32_t pack16x2(float a, float b, int f16) {
  if (f16) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  __nv_bfloat162 t = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&t);
}
__device__ __forceinline__ float2 unpack16x2(uint32_t w, int f16) {
  if (f16) return __half22float2(*reinterpret_cast<__half2*>(&w));
  return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&w));
}
__device__ __forceinline__ uint2 pack_bf16x4(float4 p) {
  return make_uint2(pack16x2(p.x, p.y, 0), pack16x2(p.z, p.w, 0));
}
__device__ __forceinline__ float4 unpack16x4(uint2 w, int f16) {
  const float2 lo = unpack16x2(w.x, f16), hi = unpack16x2(w.y, f16);
  return make_float4(lo.x, lo.y, hi.x, hi.y);
}

}  // namespace ono
