// Bandwidth-bound kernels around the GEMMs: fused softmax + loss + first backward step, bias
// gradient, optimizers on flat shards, round-cadence local SGD, Philox initialisers and the
// gather / cast / transpose that feeds the tensor-core operands.
// Reference semantics: machine_learning/src/arch/loss/{mse,cross_entropy}.rs, arch/layers/softmax.rs,
// optimization/{gradient_descent,gradient_descent_with_momentum,adam}.rs, param_manager.rs:168-197.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <stdint.h>

#include "../core/philox.h"
#include "act.cuh"
#include "ono_kernels.h"
#include "opt.cuh"

namespace ono {
void set_error(const char* fmt, const char* a, long long b, long long c);

static int launch_ok(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("%s launch failed (%lld)", what, (long long)e, 0);
    return -7;
  }
  return 0;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// ------------------------------------------------------------------------------------------------
// Loss: one warp per row.
// ------------------------------------------------------------------------------------------------
__global__ void loss_kernel(const OnoLoss l) {
  const int warps_per_block = blockDim.x >> 5;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float inv_n = 1.0f / ((float)l.B * (float)l.C);
  double block_loss = 0.0;
  int block_correct = 0;
  for (int row = blockIdx.x * warps_per_block + warp; row < l.B; row += gridDim.x * warps_per_block) {
    const float* a = l.a + (size_t)row * l.ld;
    const float* y = l.y + (size_t)row * l.ldy;
    float mx = -INFINITY, inv_z = 1.0f;
    if (l.softmax) {
      for (int j = lane; j < l.C; j += 32) mx = fmaxf(mx, a[j]);
      mx = warp_max(mx);
      float z = 0.0f;
      for (int j = lane; j < l.C; j += 32) z += expf(a[j] - mx);
      inv_z = 1.0f / warp_sum(z);
    }
    // pass 1: loss, dot = sum_k p_k g_k, argmax bookkeeping
    float loss = 0.0f, dot = 0.0f;
    float best_p = -INFINITY, best_y = -INFINITY;
    int arg_p = 0, arg_y = 0;
    for (int j = lane; j < l.C; j += 32) {
      const float p = l.softmax ? expf(a[j] - mx) * inv_z : a[j];
      const float yt = y[j];
      float g;
      if (l.kind == 1) {
        const float ps = fmaxf(p, l.eps);
        loss -= yt * logf(ps);
        g = -(yt / ps) * inv_n;
      } else {
        const float diff = p - yt;
        loss += diff * diff;
        g = 2.0f * diff * inv_n;
      }
      dot += p * g;
      if (p > best_p) { best_p = p; arg_p = j; }
      if (yt > best_y) { best_y = yt; arg_y = j; }
    }
    loss = warp_sum(loss);
    dot = warp_sum(dot);
    if (l.correct) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        float op = __shfl_xor_sync(0xffffffffu, best_p, o);
        int oa = __shfl_xor_sync(0xffffffffu, arg_p, o);
        if (op > best_p || (op == best_p && oa < arg_p)) { best_p = op; arg_p = oa; }
        float oy = __shfl_xor_sync(0xffffffffu, best_y, o);
        int ob = __shfl_xor_sync(0xffffffffu, arg_y, o);
        if (oy > best_y || (oy == best_y && ob < arg_y)) { best_y = oy; arg_y = ob; }
      }
      if (lane == 0 && arg_p == arg_y) block_correct += 1;
    }
    if (lane == 0) block_loss += (double)loss;
    // pass 2: gradient wrt the last layer's pre-activation
    for (int j = lane; j < l.C; j += 32) {
      const float p = l.softmax ? expf(a[j] - mx) * inv_z : a[j];
      const float yt = y[j];
      float g = l.kind == 1 ? -(yt / fmaxf(p, l.eps)) * inv_n : 2.0f * (p - yt) * inv_n;
      float d;
      if (l.softmax) d = p * (g - dot);
      else if (l.dact != ACT_NONE) {
        const float s = l.aux ? l.aux[(size_t)row * l.ld + j] : p;
        d = act_bwd(l.dact, l.dact_param, l.relu_quirk, s, g);
      } else d = g;
      if (l.probs) l.probs[(size_t)row * l.ld + j] = p;
      if (l.d_f32) l.d_f32[(size_t)row * l.ld_d + j] = d;
      if (l.d_bf16) reinterpret_cast<__nv_bfloat16*>(l.d_bf16)[(size_t)row * l.ld_d + j] = __float2bfloat16_rn(d);
      if (l.dT_f32) l.dT_f32[(size_t)j * l.ld_dT + row] = d;
      if (l.dT_bf16) reinterpret_cast<__nv_bfloat16*>(l.dT_bf16)[(size_t)j * l.ld_dT + row] = __float2bfloat16_rn(d);
    }
  }
  __shared__ double s_loss[32];
  __shared__ int s_correct[32];
  if (lane == 0) { s_loss[warp] = block_loss; s_correct[warp] = block_correct; }
  __syncthreads();
  if (threadIdx.x == 0) {
    double t = 0.0;
    int c = 0;
    for (int w = 0; w < warps_per_block; ++w) { t += s_loss[w]; c += s_correct[w]; }
    if (l.loss_sum) atomicAdd(l.loss_sum, t * (double)inv_n);
    if (l.correct && c) atomicAdd(l.correct, c);
  }
}

// ------------------------------------------------------------------------------------------------
// Softmax layer (forward and Jacobian-vector product): one warp per row, three passes over the row.
// ------------------------------------------------------------------------------------------------
__global__ void softmax_kernel(const OnoSoftmax a) {
  const int wpb = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __nv_bfloat16* ob = reinterpret_cast<__nv_bfloat16*>(a.out_bf16);
  __nv_bfloat16* otb = reinterpret_cast<__nv_bfloat16*>(a.outT_bf16);
  const __nv_bfloat16* pb = reinterpret_cast<const __nv_bfloat16*>(a.p_bf16);
  for (int row = blockIdx.x * wpb + warp; row < a.B; row += gridDim.x * wpb) {
    const float* x = a.x + (size_t)row * a.ld_x;
    float mx = -INFINITY, inv_z = 1.0f, dot = 0.0f;
    if (!a.backward) {
      for (int j = lane; j < a.C; j += 32) mx = fmaxf(mx, x[j]);
      mx = warp_max(mx);
      float z = 0.0f;
      for (int j = lane; j < a.C; j += 32) z += expf(x[j] - mx);
      inv_z = 1.0f / warp_sum(z);
    } else {
      for (int j = lane; j < a.C; j += 32) {
        const float p = a.p_f32 ? a.p_f32[(size_t)row * a.ld_p + j] : __bfloat162float(pb[(size_t)row * a.ld_p + j]);
        dot += p * x[j];
      }
      dot = warp_sum(dot);
    }
    for (int j = lane; j < a.C; j += 32) {
      float v;
      if (!a.backward) v = expf(x[j] - mx) * inv_z;
      else {
        const float p = a.p_f32 ? a.p_f32[(size_t)row * a.ld_p + j] : __bfloat162float(pb[(size_t)row * a.ld_p + j]);
        v = p * (x[j] - dot);      // softmax.rs:44-64
      }
      if (a.out_f32) a.out_f32[(size_t)row * a.ld_out + j] = v;
      if (ob) ob[(size_t)row * a.ld_out + j] = __float2bfloat16_rn(v);
      if (a.outT_f32) a.outT_f32[(size_t)j * a.ld_outT + row] = v;
      if (otb) otb[(size_t)j * a.ld_outT + row] = __float2bfloat16_rn(v);
    }
  }
}

// ------------------------------------------------------------------------------------------------
// Column sums (bias gradient). Block = 32 columns x 8 row-lanes.
// ------------------------------------------------------------------------------------------------
// Rows are split into `nchunks` slabs (grid.y) so that a tall, narrow matrix (the bias gradient of a
// convolution: hundreds of thousands of rows, 32 columns) still fills the GPU. Every slab writes its
// partial column sums to a scratch array; the last slab to finish for a column block (counted with an
// atomic) adds the partials in slab order, so the result does not depend on the arrival order.
// The scratch is shared by all calls of a process: calls must not overlap on the device (they are
// issued on one stream by the engines).
constexpr int CS_MAX_PART = 1 << 21;    // floats
constexpr int CS_MAX_COLBLOCKS = 1024;
__device__ float g_cs_part[CS_MAX_PART];
__device__ unsigned int g_cs_count[CS_MAX_COLBLOCKS];

template <typename T>
__device__ __forceinline__ float cs_load(const T* p) {
  if constexpr (sizeof(T) == 4) return *p;
  else return __bfloat162float(*p);
}

template <typename T>
__global__ void colsum_kernel(const T* d, int M, int N, int ld, float* out, float beta, int rows_per, int nchunks) {
  __shared__ float s[8][33];
  __shared__ int s_last;
  const int col = blockIdx.x * 32 + threadIdx.x;
  const int m0 = blockIdx.y * rows_per, m1 = min(M, m0 + rows_per);
  float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
  if (col < N) {
    int m = m0 + threadIdx.y;
    for (; m + 24 < m1; m += 32) {   // four independent loads in flight per thread
      a0 += cs_load(d + (size_t)m * ld + col);
      a1 += cs_load(d + (size_t)(m + 8) * ld + col);
      a2 += cs_load(d + (size_t)(m + 16) * ld + col);
      a3 += cs_load(d + (size_t)(m + 24) * ld + col);
    }
    for (; m < m1; m += 8) a0 += cs_load(d + (size_t)m * ld + col);
  }
  s[threadIdx.y][threadIdx.x] = (a0 + a1) + (a2 + a3);
  __syncthreads();
  float t = 0.0f;
  if (threadIdx.y == 0) {
#pragma unroll
    for (int i = 0; i < 8; ++i) t += s[i][threadIdx.x];
  }
  if (nchunks == 1) {
    if (threadIdx.y == 0 && col < N) out[col] = beta != 0.0f ? beta * out[col] + t : t;
    return;
  }
  if (threadIdx.y == 0) g_cs_part[((size_t)blockIdx.y * gridDim.x + blockIdx.x) * 32 + threadIdx.x] = t;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0 && threadIdx.y == 0) s_last = atomicAdd(&g_cs_count[blockIdx.x], 1u) == (unsigned)nchunks - 1u;
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  if (threadIdx.y == 0 && col < N) {
    float sum = 0.0f;
    for (int c = 0; c < nchunks; ++c) sum += __ldcg(&g_cs_part[((size_t)c * gridDim.x + blockIdx.x) * 32 + threadIdx.x]);
    out[col] = beta != 0.0f ? beta * out[col] + sum : sum;
  }
  if (threadIdx.x == 0 && threadIdx.y == 0) g_cs_count[blockIdx.x] = 0u;
}

// ------------------------------------------------------------------------------------------------
// Optimizers (128-bit vectorised main body, scalar tail).
// ------------------------------------------------------------------------------------------------
struct OptimScalars {
  float lr, mu, b1, b2, eps, gs, adam_step;
};

__device__ __forceinline__ float optim_one(int kind, const OptimScalars& s, float p, float g, float* m, float* v) {
  g *= s.gs;
  if (kind == 0) return p - s.lr * g;  // gradient_descent.rs:45-47
  if (kind == 1) {                     // gradient_descent_with_momentum.rs:55-62
    const float vel = s.mu * (*m) + g;
    *m = vel;
    return p - s.lr * vel;
  }
  // adam.rs:75-91: step = lr*sqrt(1-b2^t)/(1-b1^t); p -= step * m / (sqrt(v) + eps)
  const float mm = s.b1 * (*m) + (1.0f - s.b1) * g;
  const float vv = s.b2 * (*v) + (1.0f - s.b2) * g * g;
  *m = mm;
  *v = vv;
  return p - s.adam_step * mm / (sqrtf(vv) + s.eps);
}

__global__ void optim_kernel(const OnoOptim o) {
  OptimScalars s{o.lr, o.mu, o.b1, o.b2, o.eps, o.grad_scale, 0.0f};
  if (o.kind == 2) {
    const float b1t = o.adam_pows[0], b2t = o.adam_pows[1];
    s.adam_step = o.lr * sqrtf(1.0f - b2t) / (1.0f - b1t);
  }
  const long long n4 = o.n >> 2;
  const long long stride = (long long)gridDim.x * blockDim.x;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  float4* p4 = reinterpret_cast<float4*>(o.p);
  const float4* g4 = reinterpret_cast<const float4*>(o.g);
  float4* m4 = reinterpret_cast<float4*>(o.m);
  float4* v4 = reinterpret_cast<float4*>(o.v);
  __nv_bfloat16* pb = reinterpret_cast<__nv_bfloat16*>(o.p_bf16);
  for (long long i = tid; i < n4; i += stride) {
    float4 p = p4[i];
    const float4 g = g4[i];
    float4 m = o.kind >= 1 ? m4[i] : make_float4(0, 0, 0, 0);
    float4 v = o.kind == 2 ? v4[i] : make_float4(0, 0, 0, 0);
    p.x = optim_one(o.kind, s, p.x, g.x, &m.x, &v.x);
    p.y = optim_one(o.kind, s, p.y, g.y, &m.y, &v.y);
    p.z = optim_one(o.kind, s, p.z, g.z, &m.z, &v.z);
    p.w = optim_one(o.kind, s, p.w, g.w, &m.w, &v.w);
    p4[i] = p;
    if (o.kind >= 1) m4[i] = m;
    if (o.kind == 2) v4[i] = v;
    if (pb) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(p.x, p.y), hi = __floats2bfloat162_rn(p.z, p.w);
      uint2 pk;
      pk.x = *reinterpret_cast<uint32_t*>(&lo);
      pk.y = *reinterpret_cast<uint32_t*>(&hi);
      *reinterpret_cast<uint2*>(pb + 4 * i) = pk;
    }
    if (o.zero_grad) reinterpret_cast<float4*>(const_cast<float*>(o.g))[i] = make_float4(0, 0, 0, 0);
  }
  for (long long i = (n4 << 2) + tid; i < o.n; i += stride) {
    float m = o.kind >= 1 ? o.m[i] : 0.0f, v = o.kind == 2 ? o.v[i] : 0.0f;
    const float p = optim_one(o.kind, s, o.p[i], o.g[i], &m, &v);
    o.p[i] = p;
    if (o.kind >= 1) o.m[i] = m;
    if (o.kind == 2) o.v[i] = v;
    if (pb) pb[i] = __float2bfloat16_rn(p);
    if (o.zero_grad) const_cast<float*>(o.g)[i] = 0.0f;
  }
}

__global__ void adam_tick_kernel(float* pows, float b1, float b2) {
  pows[0] *= b1;
  pows[1] *= b2;
}

__global__ void local_sgd_kernel(float* p, const float* g, float* r, long long n, float lr, __nv_bfloat16* pb) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const float gi = g[i];
    const float pi = p[i] - lr * gi;
    p[i] = pi;
    r[i] += gi;
    if (pb) pb[i] = __float2bfloat16_rn(pi);
  }
}

__global__ void sumsq_kernel(const float* x, long long n, double* out) {
  double acc = 0.0;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const float v = x[i];
    acc += (double)v * (double)v;
  }
  __shared__ double s[32];
  float dummy = 0.0f; (void)dummy;
  // warp reduce in double
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) s[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    double t = 0.0;
    for (int w = 0; w < (blockDim.x >> 5); ++w) t += s[w];
    atomicAdd(out, t);
  }
}

__global__ void init_kernel(float* out, long long n, unsigned long long off, unsigned long long seed, int kind,
                            float a, float b) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    out[i] = philox_sample(off + (unsigned long long)i, seed, kind, a, b);
}

// ------------------------------------------------------------------------------------------------
// Row gather + cast + transpose through a 32x33 shared tile.
// ------------------------------------------------------------------------------------------------
__global__ void rows_kernel(const OnoRows r) {
  __shared__ float tile[32][33];
  const int r0 = blockIdx.y * 32, c0 = blockIdx.x * 32;
  __nv_bfloat16* db = reinterpret_cast<__nv_bfloat16*>(r.dst_bf16);
  __nv_bfloat16* dtb = reinterpret_cast<__nv_bfloat16*>(r.dstT_bf16);
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int row = r0 + i, col = c0 + threadIdx.x;
    float v = 0.0f;
    if (row < r.R && col < r.W) {
      const int srow = r.idx ? r.idx[row] : row;
      v = r.src[(size_t)srow * r.ld_src + col];
      if (r.dst_f32) r.dst_f32[(size_t)row * r.ld_dst + col] = v;
      if (db) db[(size_t)row * r.ld_dst + col] = __float2bfloat16_rn(v);
    }
    tile[i][threadIdx.x] = v;
  }
  if (!r.dstT_f32 && !dtb) return;
  __syncthreads();
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int col = c0 + i, row = r0 + threadIdx.x;  // output row = source column
    if (col < r.W && row < r.R) {
      const float v = tile[threadIdx.x][i];
      if (r.dstT_f32) r.dstT_f32[(size_t)col * r.ld_dstT + row] = v;
      if (dtb) dtb[(size_t)col * r.ld_dstT + row] = __float2bfloat16_rn(v);
    }
  }
}

static int grid_for(long long n, int block, int per_thread = 4) {
  long long g = (n + (long long)block * per_thread - 1) / ((long long)block * per_thread);
  if (g < 1) g = 1;
  if (g > 148 * 16) g = 148 * 16;
  return (int)g;
}

}  // namespace ono

using namespace ono;

extern "C" int ono_loss(const OnoLoss* l, ono_stream_t st) {
  if (!l || !l->a || !l->y || l->B <= 0 || l->C <= 0) { set_error("bad loss args%s", "", 0, 0); return -1; }
  const int wpb = 8;
  int grid = (l->B + wpb - 1) / wpb;
  if (grid > 148 * 8) grid = 148 * 8;
  loss_kernel<<<grid, wpb * 32, 0, (cudaStream_t)st>>>(*l);
  return launch_ok("loss");
}

namespace ono {
__global__ void push_add_kernel(const float* src, float* dst, long long n) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    atomicAdd(dst + i, src[i]);   // result unused: compiled to a reduction that needs no reply
}
}  // namespace ono

extern "C" int ono_softmax(const OnoSoftmax* a, ono_stream_t st) {
  if (!a || !a->x || a->B <= 0 || a->C <= 0 || (a->backward && !a->p_f32 && !a->p_bf16)) {
    set_error("bad softmax args%s", "", 0, 0);
    return -1;
  }
  const int wpb = 8;
  int grid = (a->B + wpb - 1) / wpb;
  if (grid > 148 * 8) grid = 148 * 8;
  softmax_kernel<<<grid, wpb * 32, 0, (cudaStream_t)st>>>(*a);
  return launch_ok("softmax");
}

namespace ono {
__global__ void cast16_kernel(const float* src, uint16_t* dst, long long n, int f16, int vec) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long n4 = vec ? n >> 2 : 0;
  for (long long i = tid; i < n4; i += stride) {
    const float4 x = __ldcs(reinterpret_cast<const float4*>(src) + i);
    *(reinterpret_cast<uint2*>(dst) + i) = make_uint2(pack16x2(x.x, x.y, f16), pack16x2(x.z, x.w, f16));
  }
  for (long long i = (n4 << 2) + tid; i < n; i += stride) {
    const uint32_t w = pack16x2(src[i], 0.0f, f16);
    dst[i] = (uint16_t)(w & 0xffffu);
  }
}
}  // namespace ono

extern "C" int ono_copy_async(void* dst, const void* src, long long bytes, ono_stream_t st) {
  if (!dst || !src || bytes < 0) { set_error("bad copy args%s", "", 0, 0); return -1; }
  if (bytes == 0) return 0;
  const cudaError_t e = cudaMemcpyAsync(dst, src, (size_t)bytes, cudaMemcpyDefault, (cudaStream_t)st);
  if (e != cudaSuccess) { set_error("cudaMemcpyAsync failed: %s", cudaGetErrorString(e), 0, 0); return -7; }
  return 0;
}

extern "C" int ono_cast16(const float* src, void* dst, long long n, int f16, ono_stream_t st) {
  if (!src || !dst || n < 0) { set_error("bad cast16 args%s", "", 0, 0); return -1; }
  if (((uintptr_t)dst & 1) != 0) { set_error("cast16 destination must be 2-byte aligned%s", "", 0, 0); return -1; }
  if (n == 0) return 0;
  const int vec = (((uintptr_t)src & 15) == 0 && ((uintptr_t)dst & 7) == 0) ? 1 : 0;
  ono::cast16_kernel<<<grid_for(n, 256, 8), 256, 0, (cudaStream_t)st>>>(src, (uint16_t*)dst, n, f16 ? 1 : 0, vec);
  return launch_ok("cast16");
}

extern "C" int ono_push_add(const float* src, float* dst, long long n, ono_stream_t st) {
  if (!src || !dst || n < 0) { set_error("bad push_add args%s", "", 0, 0); return -1; }
  if (n == 0) return 0;
  ono::push_add_kernel<<<grid_for(n, 256), 256, 0, (cudaStream_t)st>>>(src, dst, n);
  return launch_ok("push_add");
}

extern "C" int ono_colsum(const void* d, int dtype, int M, int N, int ld, float* out, float beta, ono_stream_t st) {
  if (!d || !out || M <= 0 || N <= 0) { set_error("bad colsum args%s", "", 0, 0); return -1; }
  const int gx = (N + 31) / 32;
  int nchunks = 1;
  if (gx <= CS_MAX_COLBLOCKS) {
    nchunks = std::max(1, std::min({(M + 127) / 128, (4 * 148 + gx - 1) / gx, CS_MAX_PART / (gx * 32)}));
  }
  const int rows_per = (((M + nchunks - 1) / nchunks) + 7) / 8 * 8;
  nchunks = (M + rows_per - 1) / rows_per;
  dim3 block(32, 8), grid(gx, nchunks);
  if (dtype == 0) colsum_kernel<float><<<grid, block, 0, (cudaStream_t)st>>>((const float*)d, M, N, ld, out, beta, rows_per, nchunks);
  else colsum_kernel<__nv_bfloat16><<<grid, block, 0, (cudaStream_t)st>>>((const __nv_bfloat16*)d, M, N, ld, out, beta, rows_per, nchunks);
  return launch_ok("colsum");
}

extern "C" int ono_optim(const OnoOptim* o, ono_stream_t st) {
  if (!o || !o->p || !o->g || o->n < 0) { set_error("bad optim args%s", "", 0, 0); return -1; }
  if (o->kind >= 1 && !o->m) { set_error("optimizer state m missing%s", "", 0, 0); return -1; }
  if (o->kind == 2 && (!o->v || !o->adam_pows)) { set_error("adam state missing%s", "", 0, 0); return -1; }
  if (((uintptr_t)o->p | (uintptr_t)o->g | (uintptr_t)o->m | (uintptr_t)o->v) & 15) {
    set_error("optimizer buffers must be 16-byte aligned%s", "", 0, 0);
    return -1;
  }
  if (o->p_bf16 && ((uintptr_t)o->p_bf16 & 7)) { set_error("bf16 shadow must be 8-byte aligned%s", "", 0, 0); return -1; }
  if (o->n == 0) return 0;
  optim_kernel<<<grid_for(o->n, 256, 8), 256, 0, (cudaStream_t)st>>>(*o);
  return launch_ok("optim");
}

extern "C" int ono_adam_tick(float* pows, float b1, float b2, ono_stream_t st) {
  adam_tick_kernel<<<1, 1, 0, (cudaStream_t)st>>>(pows, b1, b2);
  return launch_ok("adam_tick");
}

extern "C" int ono_local_sgd(float* p, const float* g, float* r, long long n, float lr, void* pb, ono_stream_t st) {
  if (n <= 0) return 0;
  local_sgd_kernel<<<grid_for(n, 256), 256, 0, (cudaStream_t)st>>>(p, g, r, n, lr, (__nv_bfloat16*)pb);
  return launch_ok("local_sgd");
}

extern "C" int ono_sumsq(const float* x, long long n, double* out, ono_stream_t st) {
  if (n <= 0) return 0;
  sumsq_kernel<<<grid_for(n, 256, 8), 256, 0, (cudaStream_t)st>>>(x, n, out);
  return launch_ok("sumsq");
}

extern "C" int ono_init(float* out, long long n, unsigned long long off, unsigned long long seed, int kind, float a,
                        float b, ono_stream_t st) {
  if (n <= 0) return 0;
  init_kernel<<<grid_for(n, 256), 256, 0, (cudaStream_t)st>>>(out, n, off, seed, kind, a, b);
  return launch_ok("init");
}

// f32 copy and/or transpose of an aligned matrix with 16-byte accesses on both sides: 64 x 64 tiles, rows read as
// float4, the transpose written as float4 along the source's rows (R % 4 == 0, W % 4 == 0, 16-byte aligned rows).
__global__ void __launch_bounds__(256) rows_vec_kernel(const OnoRows r) {
  __shared__ float tile[64][65];
  const int r0 = blockIdx.y * 64, c0 = blockIdx.x * 64;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    const int row = r0 + ty + 16 * p, col = c0 + 4 * tx;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (row < r.R && col < r.W) {
      v = *reinterpret_cast<const float4*>(r.src + (size_t)row * r.ld_src + col);
      if (r.dst_f32) *reinterpret_cast<float4*>(r.dst_f32 + (size_t)row * r.ld_dst + col) = v;
    }
    float* t = &tile[ty + 16 * p][4 * tx];
    t[0] = v.x; t[1] = v.y; t[2] = v.z; t[3] = v.w;
  }
  if (!r.dstT_f32) return;
  __syncthreads();
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    const int col = c0 + ty + 16 * p, row = r0 + 4 * tx;   // output row = source column
    if (col < r.W && row < r.R) {
      const int cl = ty + 16 * p;
      *reinterpret_cast<float4*>(r.dstT_f32 + (size_t)col * r.ld_dstT + row) =
          make_float4(tile[4 * tx][cl], tile[4 * tx + 1][cl], tile[4 * tx + 2][cl], tile[4 * tx + 3][cl]);
    }
  }
}

// Row gather out of pinned host memory (the batch feeder's host-to-device path). The loads cross PCIe, so what counts is
// bytes in flight, not threads: a few blocks, each thread with four independent 16-byte loads outstanding (24 blocks x 256
// threads x 64 bytes = 384 KB in flight, several times the bandwidth-delay product of a Gen5 x16 link). Kept this small on
// purpose: the kernel runs on the copy stream beside the training step, and a grid of thousands of blocks stalled on PCIe
// would fill the SMs' thread slots and hold back the persistent GEMM CTAs of the step it is supposed to hide behind.
constexpr int ROWS_HOST_BLOCKS = 24;
__global__ void __launch_bounds__(256) rows_host_kernel(const OnoRows r) {
  const int w4 = r.W >> 2;
  const long long total = (long long)r.R * w4, stride = (long long)gridDim.x * blockDim.x;
  constexpr int U = 4;
  for (long long base = (long long)blockIdx.x * blockDim.x + threadIdx.x; base < total; base += stride * U) {
    float4 v[U];
    long long at[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long e = base + u * stride;
      at[u] = -1;
      if (e < total) {
        const int row = (int)(e / w4), c4 = (int)(e - (long long)row * w4);
        v[u] = *reinterpret_cast<const float4*>(r.src + (size_t)r.idx[row] * r.ld_src + 4 * c4);
        at[u] = (long long)row * r.ld_dst + 4 * c4;
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (at[u] >= 0) *reinterpret_cast<float4*>(r.dst_f32 + at[u]) = v[u];
  }
}

static bool is_host_memory(const void* p) {
  cudaPointerAttributes a;
  if (cudaPointerGetAttributes(&a, p) != cudaSuccess) { cudaGetLastError(); return false; }
  return a.type == cudaMemoryTypeHost;
}

extern "C" int ono_rows(const OnoRows* r, ono_stream_t st) {
  if (!r || !r->src || r->R <= 0 || r->W <= 0) { set_error("bad rows args%s", "", 0, 0); return -1; }
  if (r->idx && r->dst_f32 && !r->dst_bf16 && !r->dstT_f32 && !r->dstT_bf16 && r->W % 4 == 0 && r->ld_src % 4 == 0 &&
      r->ld_dst % 4 == 0 && (((uintptr_t)r->src | (uintptr_t)r->dst_f32) & 15) == 0 && is_host_memory(r->src)) {
    rows_host_kernel<<<ROWS_HOST_BLOCKS, 256, 0, (cudaStream_t)st>>>(*r);
    return launch_ok("rows");
  }
  const bool vec = !r->idx && !r->dst_bf16 && !r->dstT_bf16 && (r->dst_f32 || r->dstT_f32) && r->R % 4 == 0 && r->W % 4 == 0 &&
                   r->ld_src % 4 == 0 && (!r->dst_f32 || r->ld_dst % 4 == 0) && (!r->dstT_f32 || r->ld_dstT % 4 == 0) &&
                   (((uintptr_t)r->src | (uintptr_t)r->dst_f32 | (uintptr_t)r->dstT_f32) & 15) == 0 && (long long)r->R * r->W >= (1 << 16);
  if (vec) {
    dim3 grid((r->W + 63) / 64, (r->R + 63) / 64);
    rows_vec_kernel<<<grid, 256, 0, (cudaStream_t)st>>>(*r);
    return launch_ok("rows");
  }
  dim3 block(32, 8), grid((r->W + 31) / 32, (r->R + 31) / 32);
  rows_kernel<<<grid, block, 0, (cudaStream_t)st>>>(*r);
  return launch_ok("rows");
}
