// Philox4x32-10 counter-based generator shared by the CUDA initialiser kernel and its CPU twin.
// Element i of a model's parameter vector is drawn from counter i under the run's seed, so a value
// does not depend on how the vector is sharded across ranks (the reference instead shares one
// seeded StdRng stream across chained generators: machine_learning/src/initialization/builder.rs:104-172).
#pragma once
#include <math.h>
#include <stdint.h>

#if defined(__CUDACC__)
#define ONO_HD __host__ __device__ __forceinline__
#else
#define ONO_HD inline
#endif

namespace ono {

struct Philox4 {
  uint32_t v[4];
};

ONO_HD void philox_mulhilo(uint32_t a, uint32_t b, uint32_t& hi, uint32_t& lo) {
  const uint64_t p = static_cast<uint64_t>(a) * static_cast<uint64_t>(b);
  hi = static_cast<uint32_t>(p >> 32);
  lo = static_cast<uint32_t>(p);
}

ONO_HD Philox4 philox4x32_10(uint64_t counter, uint64_t seed) {
  uint32_t c0 = static_cast<uint32_t>(counter), c1 = static_cast<uint32_t>(counter >> 32), c2 = 0, c3 = 0;
  uint32_t k0 = static_cast<uint32_t>(seed), k1 = static_cast<uint32_t>(seed >> 32);
  for (int r = 0; r < 10; ++r) {
    uint32_t hi0, lo0, hi1, lo1;
    philox_mulhilo(0xD2511F53u, c0, hi0, lo0);
    philox_mulhilo(0xCD9E8D57u, c2, hi1, lo1);
    const uint32_t n0 = hi1 ^ c1 ^ k0, n1 = lo1, n2 = hi0 ^ c3 ^ k1, n3 = lo0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  Philox4 out;
  out.v[0] = c0; out.v[1] = c1; out.v[2] = c2; out.v[3] = c3;
  return out;
}

// kind 0: U[a,b) ; 1: U[a,b] ; 2: N(mean=a, std=b) via Box-Muller.
ONO_HD float philox_sample(uint64_t index, uint64_t seed, int kind, float a, float b) {
  const Philox4 r = philox4x32_10(index, seed);
  if (kind == 2) {
    const float u1 = (static_cast<float>(r.v[0] >> 8) + 1.0f) * (1.0f / 16777216.0f);  // (0,1]
    const float u2 = static_cast<float>(r.v[1] >> 8) * (1.0f / 16777216.0f);           // [0,1)
    const float z = sqrtf(-2.0f * logf(u1)) * cosf(6.283185307179586f * u2);
    return a + b * z;
  }
  const float u = kind == 1 ? static_cast<float>(r.v[0] >> 8) * (1.0f / 16777215.0f)
                            : static_cast<float>(r.v[0] >> 8) * (1.0f / 16777216.0f);
  return a + u * (b - a);
}

}  // namespace ono
