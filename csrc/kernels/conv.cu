// Convolution and pooling around the tcgen05 GEMM: the gather / scatter halves of the reference's
// im2col convolution (machine_learning/src/arch/layers/conv/conv2d.rs:84-104,202-266) and its max
// pooling (arch/layers/max_pooling.rs:47-157), on pixel-major activations.
//
// Activations of image layers are 2-D matrices [B*H*W, ldc] (one row per pixel, channels contiguous),
// which is exactly what the GEMM epilogue writes for Y = cols * K^T; the column order of `cols` is
// (ky, kx, c) (channels fastest: coalesced gathers), so the reference's kernel layout K[F][C][k][k] is permuted
// into that order when parameters are refreshed.
// Semantics kept from the reference: zero padding, output size floor((H+2p-k)/s)+1 (trailing rows and
// columns the strided window never reaches are dropped), zero padding competes in the max, and a
// pooling gradient whose arg-max lies in the padding is dropped.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>

#include "act.cuh"
#include "ono_kernels.h"

namespace ono {
void set_error(const char* fmt, const char* a, long long b, long long c);

template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

// Column order of `cols` is q = (ky, kx, c): channels fastest, so that both the gather below and the GEMM
// operand rows are contiguous runs of the pixel-major input. The kernel tensor K[F][C][k][k] is permuted to
// that order once per parameter refresh (kperm_kernel), and the weight gradient is permuted back.
//
// cols[r, q] = x[(b, oy*s+ky-p, ox*s+kx-p), c]  with r = (b, oy, ox); optional transposed copy colsT[q, r].
// One block handles a 32 x 32 tile of (r, q): reads and the row-major write are coalesced along q, the
// transposed write goes through shared memory and is coalesced along r.
template <typename T>
__global__ void im2col_kernel(const OnoConvGeom g, const T* x, int ldx, T* cols, int ld_cols, T* colsT, int ld_colsT) {
  __shared__ float tile[32][33];
  __shared__ int s_iy0[32], s_ix0[32], s_img[32];   // per tile row: window origin and image index (divisions once per row)
  const int ckk = g.C * g.K * g.K;
  const long long rows = (long long)g.B * g.OH * g.OW;
  const int qtiles = (ckk + 31) / 32;
  const long long ntiles = ((rows + 31) / 32) * qtiles;
  for (long long t = blockIdx.x; t < ntiles; t += gridDim.x) {
    const long long r0 = (t / qtiles) * 32;
    const int q0 = (int)(t % qtiles) * 32;
    const int q = q0 + threadIdx.x;
    const int c = q % g.C, kx = (q / g.C) % g.K, ky = q / (g.C * g.K);
    if (threadIdx.y == 0) {
      const long long r = r0 + threadIdx.x;
      const int ox = (int)(r % g.OW), oy = (int)((r / g.OW) % g.OH);
      s_iy0[threadIdx.x] = oy * g.S - g.P;
      s_ix0[threadIdx.x] = ox * g.S - g.P;
      s_img[threadIdx.x] = (int)(r / ((long long)g.OW * g.OH));
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int rr = threadIdx.y + 8 * j;
      const long long r = r0 + rr;
      float v = 0.f;
      if (r < rows && q < ckk) {
        const int iy = s_iy0[rr] + ky, ix = s_ix0[rr] + kx;
        if (iy >= 0 && iy < g.H && ix >= 0 && ix < g.W)
          v = to_f32(x[((long long)(s_img[rr] * g.H + iy) * g.W + ix) * ldx + c]);
        cols[r * ld_cols + q] = from_f32<T>(v);
      }
      tile[rr][threadIdx.x] = v;
    }
    if (colsT) {
      __syncthreads();
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int qq = threadIdx.y + 8 * j;
        const long long r = r0 + threadIdx.x;
        if (r < rows && q0 + qq < ckk) colsT[(long long)(q0 + qq) * ld_colsT + r] = from_f32<T>(tile[threadIdx.x][qq]);
      }
      __syncthreads();
    } else {
      __syncthreads();   // s_* are rewritten by the next tile
    }
  }
}

// dx[(b,iy,ix), c] = act'(aux) * sum_{ky,kx} dcols[(b,oy,ox), (ky,kx,c)] over the windows covering the pixel
// (gather form: no atomics). One block handles 32 pixels x 32 channels; the optional transposed copy
// dxT[c, pix] goes through shared memory.
template <typename T>
__global__ void col2im_kernel(const OnoConvGeom g, const T* dcols, int ld_dcols, const T* aux, int ld_aux, int dact,
                              float dact_param, int relu_quirk, T* dx, int ld_dx, T* dxT, int ld_dxT) {
  __shared__ float tile[32][33];
  __shared__ int s_iy[32], s_ix[32], s_img[32];
  const long long npix = (long long)g.B * g.H * g.W;
  const int ctiles = (g.C + 31) / 32;
  const long long ntiles = ((npix + 31) / 32) * ctiles;
  const int shift = g.S == 1 ? 0 : g.S == 2 ? 1 : g.S == 4 ? 2 : -1;   // power-of-two strides avoid the divisions
  for (long long t = blockIdx.x; t < ntiles; t += gridDim.x) {
    const long long p0 = (t / ctiles) * 32;
    const int c0 = (int)(t % ctiles) * 32;
    const int c = c0 + threadIdx.x;
    if (threadIdx.y == 0) {
      const long long pix = p0 + threadIdx.x;
      s_ix[threadIdx.x] = (int)(pix % g.W) + g.P;
      s_iy[threadIdx.x] = (int)((pix / g.W) % g.H) + g.P;
      s_img[threadIdx.x] = (int)(pix / ((long long)g.W * g.H));
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int pp = threadIdx.y + 8 * j;
      const long long pix = p0 + pp;
      float acc = 0.f;
      if (pix < npix && c < g.C) {
        const int ixp = s_ix[pp], iyp = s_iy[pp];
        const long long img_row = (long long)s_img[pp] * g.OH;
        for (int ky = 0; ky < g.K; ++ky) {
          const int ty = iyp - ky;
          if (ty < 0) break;
          int oy;
          if (shift >= 0) { if (ty & (g.S - 1)) continue; oy = ty >> shift; }
          else { if (ty % g.S) continue; oy = ty / g.S; }
          if (oy >= g.OH) continue;
          const T* rowp = dcols + (img_row + oy) * g.OW * (long long)ld_dcols + (ky * g.K) * g.C + c;
          for (int kx = 0; kx < g.K; ++kx) {
            const int tx = ixp - kx;
            if (tx < 0) break;
            int ox;
            if (shift >= 0) { if (tx & (g.S - 1)) continue; ox = tx >> shift; }
            else { if (tx % g.S) continue; ox = tx / g.S; }
            if (ox >= g.OW) continue;
            acc += to_f32(rowp[(long long)ox * ld_dcols + kx * g.C]);
          }
        }
        if (dact != ACT_NONE) acc = act_bwd(dact, dact_param, relu_quirk, to_f32(aux[pix * ld_aux + c]), acc);
        dx[pix * ld_dx + c] = from_f32<T>(acc);
      }
      tile[pp][threadIdx.x] = acc;
    }
    if (dxT) {
      __syncthreads();
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int cc = threadIdx.y + 8 * j;
        const long long pix = p0 + threadIdx.x;
        if (pix < npix && c0 + cc < g.C) dxT[(long long)(c0 + cc) * ld_dxT + pix] = from_f32<T>(tile[threadIdx.x][cc]);
      }
      __syncthreads();
    } else {
      __syncthreads();
    }
  }
}

// Four consecutive channels at once (16-byte loads of f32, 8-byte loads of bf16).
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
  return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* p, float4 v) {
  const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 u;
  u.x = *reinterpret_cast<const uint32_t*>(&a);
  u.y = *reinterpret_cast<const uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = u;
}

// im2col, four channels per thread (C % 4 == 0, so four consecutive columns share one tap): a block takes a
// 32 x 32 tile of (r, q) in one pass; one vector load, one vector store, the transposed copy through shared memory.
template <typename T>
__global__ void __launch_bounds__(256) im2col_vec_kernel(const OnoConvGeom g, const T* x, int ldx, T* cols, int ld_cols, T* colsT,
                                                         int ld_colsT) {
  __shared__ float tile[32][33];
  const int ckk = g.C * g.K * g.K;
  const long long rows = (long long)g.B * g.OH * g.OW;
  const int qtiles = (ckk + 31) / 32;
  const long long ntiles = ((rows + 31) / 32) * qtiles;
  const int qd = threadIdx.x & 7, rr = threadIdx.x >> 3;
  for (long long t = blockIdx.x; t < ntiles; t += gridDim.x) {
    const long long r0 = (t / qtiles) * 32;
    const int q0 = (int)(t % qtiles) * 32;
    const int q = q0 + 4 * qd;
    const long long r = r0 + rr;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (r < rows && q < ckk) {
      // 32-bit coordinate arithmetic (the launcher checks that pixel counts fit): 64-bit divisions cost ~50 instructions each
      const unsigned ri = (unsigned)r;
      const int tap = q / g.C, c = q - tap * g.C;
      const int ky = tap / g.K, kx = tap - ky * g.K;
      const unsigned rest = ri / (unsigned)g.OW;
      const int ox = (int)(ri - rest * (unsigned)g.OW);
      const unsigned img = rest / (unsigned)g.OH;
      const int oy = (int)(rest - img * (unsigned)g.OH);
      const int iy = oy * g.S - g.P + ky, ix = ox * g.S - g.P + kx;
      if (iy >= 0 && iy < g.H && ix >= 0 && ix < g.W) v = load4(x + (long long)((img * g.H + iy) * g.W + ix) * ldx + c);
      store4(cols + r * ld_cols + q, v);
    }
    if (colsT) {
      tile[rr][4 * qd] = v.x; tile[rr][4 * qd + 1] = v.y; tile[rr][4 * qd + 2] = v.z; tile[rr][4 * qd + 3] = v.w;
      __syncthreads();
      const int lane = threadIdx.x & 31, wy = threadIdx.x >> 5;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int qq = wy + 8 * j;
        const long long rw = r0 + lane;
        if (rw < rows && q0 + qq < ckk) colsT[(long long)(q0 + qq) * ld_colsT + rw] = from_f32<T>(tile[lane][qq]);
      }
      __syncthreads();
    }
  }
}

// col2im with compile-time kernel size and stride, four channels per thread: a block takes 32 pixels x 32 channels
// (thread = pixel x channel quad), the K x K taps unroll into independent predicated vector loads, so a thread has all
// its loads in flight at once instead of walking data-dependent loops. Needs C % 4 == 0 and 4-element aligned rows.
template <typename T, int K, int S>
__global__ void __launch_bounds__(256) col2im_vec_kernel(const OnoConvGeom g, const T* dcols, int ld_dcols, const T* aux, int ld_aux,
                                                         int dact, float dact_param, int relu_quirk, T* dx, int ld_dx, T* dxT, int ld_dxT) {
  __shared__ float tile[32][33];
  const long long npix = (long long)g.B * g.H * g.W;
  const int ctiles = (g.C + 31) / 32;
  const long long ntiles = ((npix + 31) / 32) * ctiles;
  const int q = threadIdx.x & 7, pp = threadIdx.x >> 3;
  for (long long t = blockIdx.x; t < ntiles; t += gridDim.x) {
    const long long p0 = (t / ctiles) * 32;
    const int c0 = (int)(t % ctiles) * 32;
    const int c = c0 + 4 * q;
    const long long pix = p0 + pp;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (pix < npix && c < g.C) {
      const unsigned pi = (unsigned)pix;               // 32-bit coordinate arithmetic, see im2col_vec_kernel
      const unsigned rest = pi / (unsigned)g.W;
      const int ixp = (int)(pi - rest * (unsigned)g.W) + g.P;
      const unsigned img = rest / (unsigned)g.H;
      const int iyp = (int)(rest - img * (unsigned)g.H) + g.P;
      const long long img_row = (long long)img * g.OH;
#pragma unroll
      for (int ky = 0; ky < K; ++ky) {
        const int ty = iyp - ky;
        const int oy = ty / S;
        const bool oky = ty >= 0 && (ty % S) == 0 && oy < g.OH;
#pragma unroll
        for (int kx = 0; kx < K; ++kx) {
          const int tx = ixp - kx;
          const int ox = tx / S;
          if (oky && tx >= 0 && (tx % S) == 0 && ox < g.OW) {
            const float4 v = load4(dcols + ((img_row + oy) * g.OW + ox) * (long long)ld_dcols + (ky * K + kx) * g.C + c);
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
          }
        }
      }
      if (dact != ACT_NONE) {
        const float4 a = load4(aux + pix * ld_aux + c);
        acc.x = act_bwd(dact, dact_param, relu_quirk, a.x, acc.x);
        acc.y = act_bwd(dact, dact_param, relu_quirk, a.y, acc.y);
        acc.z = act_bwd(dact, dact_param, relu_quirk, a.z, acc.z);
        acc.w = act_bwd(dact, dact_param, relu_quirk, a.w, acc.w);
      }
      store4(dx + pix * ld_dx + c, acc);
    }
    if (dxT) {
      tile[pp][4 * q] = acc.x; tile[pp][4 * q + 1] = acc.y; tile[pp][4 * q + 2] = acc.z; tile[pp][4 * q + 3] = acc.w;
      __syncthreads();
      const int lane = threadIdx.x & 31, wy = threadIdx.x >> 5;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int cc = wy + 8 * j;
        const long long px = p0 + lane;
        if (px < npix && c0 + cc < g.C) dxT[(long long)(c0 + cc) * ld_dxT + px] = from_f32<T>(tile[lane][cc]);
      }
      __syncthreads();
    }
  }
}

// Kernel tensor between the parameter layout K[F][C][k][k] (f32, contiguous) and the operand layout
// [F][(ky,kx,c)] used by the GEMMs. dir 0: parameters -> operand (dst, dtype T, leading dimension ld_dst) and
// optionally its transpose dstT[(ky,kx,c)][F]; dir 1: f32 operand-ordered gradient (src, ld_src) -> parameter
// order, dst = beta * dst + src.
template <typename T>
__global__ void kperm_kernel(int F, int C, int K, int dir, const float* src, int ld_src, void* dst_, int ld_dst, T* dstT,
                             int ld_dstT, float beta) {
  const int ckk = C * K * K;
  const long long total = (long long)F * ckk;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int f = (int)(i / ckk), q = (int)(i % ckk);                   // q in operand order (ky, kx, c)
    const int c = q % C, kx = (q / C) % K, ky = q / (C * K);
    const long long pidx = ((long long)(f * C + c) * K + ky) * K + kx;    // parameter order
    if (dir == 0) {
      const float v = src[pidx];
      reinterpret_cast<T*>(dst_)[(long long)f * ld_dst + q] = from_f32<T>(v);
      if (dstT) dstT[(long long)q * ld_dstT + f] = from_f32<T>(v);
    } else {
      float* d = reinterpret_cast<float*>(dst_);
      const float v = src[(long long)f * ld_src + q];
      d[pidx] = beta != 0.f ? beta * d[pidx] + v : v;
    }
  }
}

// ------------------------------------------------------------------------------------------------
// Single-input-channel convolution (the first layer of every image model of the reference), computed
// directly on CUDA cores: with C = 1 the GEMM would have K = k*k <= 25, far too short for the tensor
// cores, and im2col would write k*k times the input. Thread x = filter, thread y strides over output
// pixels; the k*k taps of a pixel are broadcast loads, the filter's weights live in registers.
// ------------------------------------------------------------------------------------------------
constexpr int C1_MAXKK = 25;  // up to 5 x 5 kernels

template <typename T>
__global__ void conv1_fwd_kernel(const OnoConvGeom g, int F, const T* x, int ldx, const float* kparams, const float* bias,
                                 int act, float act_param, T* y, int ldy) {
  const int kk = g.K * g.K;
  const int f = blockIdx.y * 32 + threadIdx.x;
  float w[C1_MAXKK];
#pragma unroll
  for (int i = 0; i < C1_MAXKK; ++i) w[i] = (i < kk && f < F) ? kparams[(long long)f * kk + i] : 0.f;
  const float bv = (bias && f < F) ? bias[f] : 0.f;
  // A warp takes 32 consecutive output pixels: lane l works out the window origin of pixel r0 + l once (the
  // divisions), then the warp walks the 32 pixels with the coordinates broadcast by shuffles.
  const int rows = g.B * g.OH * g.OW;
  const int ohw = g.OH * g.OW;
  for (int r0 = (blockIdx.x * blockDim.y + threadIdx.y) * 32; r0 < rows; r0 += gridDim.x * blockDim.y * 32) {
    const int rl = min(r0 + (int)threadIdx.x, rows - 1);
    const int img_l = rl / ohw, rem = rl - img_l * ohw;
    const int oy_l = rem / g.OW, ox_l = rem - oy_l * g.OW;
    const int my_iy0 = oy_l * g.S - g.P, my_ix0 = ox_l * g.S - g.P, my_base = img_l * g.H;
    const int np = min(32, rows - r0);
    for (int pp = 0; pp < np; ++pp) {
      const int iy0 = __shfl_sync(0xffffffffu, my_iy0, pp), ix0 = __shfl_sync(0xffffffffu, my_ix0, pp);
      const int base = __shfl_sync(0xffffffffu, my_base, pp);
      float acc = bv;
#pragma unroll
      for (int i = 0; i < C1_MAXKK; ++i) {
        if (i >= kk) break;
        const int ky = i / g.K, kx = i - ky * g.K;
        const int iy = iy0 + ky, ix = ix0 + kx;
        if (iy >= 0 && iy < g.H && ix >= 0 && ix < g.W) acc += w[i] * to_f32(x[(long long)((base + iy) * g.W + ix) * ldx]);
      }
      if (f < F) y[(long long)(r0 + pp) * ldy + f] = from_f32<T>(act_fwd(act, act_param, acc));
    }
  }
}

// dK[f][ky][kx] = sum over output pixels dy[r][f] * x[tap], db[f] = sum dy[r][f]. Every block writes one row of
// partial sums to a scratch array; the last block to finish (atomic ticket) adds the rows in block order, so the
// result does not depend on scheduling. Calls must not overlap on the device (one training stream).
constexpr int C1_MAXBLOCKS = 592;
constexpr int C1_MAXF = 128;
__device__ float g_c1_part[C1_MAXBLOCKS * C1_MAXF * (C1_MAXKK + 1)];
__device__ unsigned int g_c1_ticket;

template <typename T>
__global__ void conv1_wgrad_kernel(const OnoConvGeom g, int F, const T* x, int ldx, const T* dy, int ld_dy, float* gk,
                                   float* gb, float beta) {
  __shared__ float red[8][32][C1_MAXKK + 2];
  __shared__ int s_last;
  const int kk = g.K * g.K;
  const int nfb = (F + 31) / 32;
  float acc[C1_MAXKK + 1];
  const int rows = g.B * g.OH * g.OW;
  const int ohw = g.OH * g.OW;
  for (int fb = 0; fb < nfb; ++fb) {
    const int f = fb * 32 + threadIdx.x;
#pragma unroll
    for (int i = 0; i <= C1_MAXKK; ++i) acc[i] = 0.f;
    for (int r0 = (blockIdx.x * blockDim.y + threadIdx.y) * 32; r0 < rows; r0 += gridDim.x * blockDim.y * 32) {
      const int rl = min(r0 + (int)threadIdx.x, rows - 1);
      const int img_l = rl / ohw, rem = rl - img_l * ohw;
      const int oy_l = rem / g.OW, ox_l = rem - oy_l * g.OW;
      const int my_iy0 = oy_l * g.S - g.P, my_ix0 = ox_l * g.S - g.P, my_base = img_l * g.H;
      const int np = min(32, rows - r0);
      for (int pp = 0; pp < np; ++pp) {
        const int iy0 = __shfl_sync(0xffffffffu, my_iy0, pp), ix0 = __shfl_sync(0xffffffffu, my_ix0, pp);
        const int base = __shfl_sync(0xffffffffu, my_base, pp);
        const float d = f < F ? to_f32(dy[(long long)(r0 + pp) * ld_dy + f]) : 0.f;
#pragma unroll
        for (int i = 0; i < C1_MAXKK; ++i) {
          if (i >= kk) break;
          const int ky = i / g.K, kx = i - ky * g.K;
          const int iy = iy0 + ky, ix = ix0 + kx;
          if (iy >= 0 && iy < g.H && ix >= 0 && ix < g.W) acc[i] += d * to_f32(x[(long long)((base + iy) * g.W + ix) * ldx]);
        }
        acc[C1_MAXKK] += d;
      }
    }
#pragma unroll
    for (int i = 0; i <= C1_MAXKK; ++i) red[threadIdx.y][threadIdx.x][i] = acc[i];
    __syncthreads();
    if (threadIdx.y == 0 && f < F) {
      float* out = g_c1_part + ((size_t)blockIdx.x * C1_MAXF + f) * (C1_MAXKK + 1);
      for (int i = 0; i <= C1_MAXKK; ++i) {
        if (i >= kk && i != C1_MAXKK) continue;
        float t = 0.f;
#pragma unroll
        for (int yy = 0; yy < 8; ++yy) t += red[yy][threadIdx.x][i];
        out[i] = t;
      }
    }
    __syncthreads();
  }
  __threadfence();
  if (threadIdx.x == 0 && threadIdx.y == 0) s_last = atomicAdd(&g_c1_ticket, 1u) == gridDim.x - 1;
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  const int per = kk + 1;
  for (int idx = threadIdx.y * 32 + threadIdx.x; idx < F * per; idx += 256) {
    const int f = idx / per, i = idx % per;
    const int slot = i < kk ? i : C1_MAXKK;
    float t = 0.f;
    for (unsigned b = 0; b < gridDim.x; ++b) t += __ldcg(&g_c1_part[((size_t)b * C1_MAXF + f) * (C1_MAXKK + 1) + slot]);
    float* dst = i < kk ? gk + (long long)f * kk + i : gb + f;
    *dst = beta != 0.f ? beta * (*dst) + t : t;
  }
  if (threadIdx.x == 0 && threadIdx.y == 0) g_c1_ticket = 0u;
}

// Image-tiled variants of the two kernels above for k = 3 and k = 5 (compile-time taps): a block keeps one
// zero-padded image in shared memory, lane = filter, a warp walks output rows; a tap is one broadcast shared-memory
// load and one FMA, with no bounds test and no division in the pixel loop. Output and dy rows are 128-byte coalesced.
template <typename T>
__device__ __forceinline__ void c1_stage_image(const OnoConvGeom& g, const T* x, int ldx, int img, float* tile, int TW, int TH) {
  for (int i = threadIdx.x; i < TH * TW; i += 256) {
    const int ty = i / TW, tx = i - ty * TW;
    const int iy = ty - g.P, ix = tx - g.P;
    tile[i] = (iy >= 0 && iy < g.H && ix >= 0 && ix < g.W) ? to_f32(x[(long long)((img * g.H + iy) * g.W + ix) * ldx]) : 0.f;
  }
}

template <typename T, int K>
__global__ void __launch_bounds__(256) conv1_fwd_img_kernel(const OnoConvGeom g, int F, const T* x, int ldx, const float* kparams,
                                                            const float* bias, int act, float act_param, T* y, int ldy) {
  extern __shared__ float c1_tile[];
  const int TW = g.W + 2 * g.P, TH = g.H + 2 * g.P;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int f = blockIdx.y * 32 + lane;
  float w[K * K];
#pragma unroll
  for (int i = 0; i < K * K; ++i) w[i] = f < F ? kparams[(long long)f * (K * K) + i] : 0.f;
  const float bv = (bias && f < F) ? bias[f] : 0.f;
  for (int img = blockIdx.x; img < g.B; img += gridDim.x) {
    __syncthreads();   // the previous image has been read by every warp
    c1_stage_image(g, x, ldx, img, c1_tile, TW, TH);
    __syncthreads();
    for (int oy = warp; oy < g.OH; oy += 8) {
      const float* trow = c1_tile + oy * g.S * TW;
      T* yrow = y + (long long)(img * g.OH + oy) * g.OW * ldy + f;
#pragma unroll 4
      for (int ox = 0; ox < g.OW; ++ox) {
        const float* t0 = trow + ox * g.S;
        float acc = bv;
#pragma unroll
        for (int ky = 0; ky < K; ++ky)
#pragma unroll
          for (int kx = 0; kx < K; ++kx) acc += w[ky * K + kx] * t0[ky * TW + kx];
        if (f < F) yrow[(long long)ox * ldy] = from_f32<T>(act_fwd(act, act_param, acc));
      }
    }
  }
}

// Forward with 16-byte stores (F % 4 == 0): a lane holds four consecutive filters of one of the four pixels the warp
// works on at a time.
template <typename T, int K>
__global__ void __launch_bounds__(256) conv1_fwd_img4_kernel(const OnoConvGeom g, int F, const T* x, int ldx, const float* kparams,
                                                             const float* bias, int act, float act_param, T* y, int ldy) {
  extern __shared__ float c1_tile[];
  constexpr int KK = K * K;
  const int TW = g.W + 2 * g.P, TH = g.H + 2 * g.P;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int fq = lane & 7, pg = lane >> 3;
  const int f4 = blockIdx.y * 32 + 4 * fq;
  const bool live = f4 < F;
  float w[KK][4], bv[4];
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    bv[c] = (bias && live) ? bias[f4 + c] : 0.f;
#pragma unroll
    for (int i = 0; i < KK; ++i) w[i][c] = live ? kparams[(long long)(f4 + c) * KK + i] : 0.f;
  }
  for (int img = blockIdx.x; img < g.B; img += gridDim.x) {
    __syncthreads();
    c1_stage_image(g, x, ldx, img, c1_tile, TW, TH);
    __syncthreads();
    for (int oy = warp; oy < g.OH; oy += 8) {
      const float* trow = c1_tile + oy * g.S * TW;
      T* yrow = y + (long long)(img * g.OH + oy) * g.OW * ldy + f4;
#pragma unroll 2
      for (int ox = pg; ox < g.OW; ox += 4) {
        const float* t0 = trow + ox * g.S;
        float a0 = bv[0], a1 = bv[1], a2 = bv[2], a3 = bv[3];
#pragma unroll
        for (int ky = 0; ky < K; ++ky)
#pragma unroll
          for (int kx = 0; kx < K; ++kx) {
            const float t = t0[ky * TW + kx];
            a0 += w[ky * K + kx][0] * t; a1 += w[ky * K + kx][1] * t; a2 += w[ky * K + kx][2] * t; a3 += w[ky * K + kx][3] * t;
          }
        if (live)
          store4(yrow + (long long)ox * ldy, make_float4(act_fwd(act, act_param, a0), act_fwd(act, act_param, a1),
                                                         act_fwd(act, act_param, a2), act_fwd(act, act_param, a3)));
      }
    }
  }
}

// Partial sums of block b for (filter f, slot i; slot K*K = bias) go to g_c1_part[(f * (K*K+1) + i) * gridDim.x + b];
// conv1_wgrad_reduce_kernel then adds a pair's partials with one warp in a fixed order.
template <typename T, int K>
__global__ void __launch_bounds__(256) conv1_wgrad_img_kernel(const OnoConvGeom g, int F, const T* x, int ldx, const T* dy, int ld_dy) {
  extern __shared__ float c1_tile[];   // the padded image; afterwards the cross-warp reduction scratch
  constexpr int KK = K * K;
  const int TW = g.W + 2 * g.P, TH = g.H + 2 * g.P;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nfb = (F + 31) / 32;
  for (int fb = 0; fb < nfb; ++fb) {
    const int f = fb * 32 + lane;
    float acc[KK + 1];
#pragma unroll
    for (int i = 0; i <= KK; ++i) acc[i] = 0.f;
    for (int img = blockIdx.x; img < g.B; img += gridDim.x) {
      __syncthreads();
      c1_stage_image(g, x, ldx, img, c1_tile, TW, TH);
      __syncthreads();
      for (int oy = warp; oy < g.OH; oy += 8) {
        const float* trow = c1_tile + oy * g.S * TW;
        const T* drow = dy + (long long)(img * g.OH + oy) * g.OW * ld_dy + f;
#pragma unroll 4
        for (int ox = 0; ox < g.OW; ++ox) {
          const float d = f < F ? to_f32(drow[(long long)ox * ld_dy]) : 0.f;
          const float* t0 = trow + ox * g.S;
#pragma unroll
          for (int ky = 0; ky < K; ++ky)
#pragma unroll
            for (int kx = 0; kx < K; ++kx) acc[ky * K + kx] += d * t0[ky * TW + kx];
          acc[KK] += d;
        }
      }
    }
    __syncthreads();   // the image is no longer needed: its space takes the warps' sums
#pragma unroll
    for (int i = 0; i <= KK; ++i) c1_tile[(warp * 32 + lane) * (KK + 1) + i] = acc[i];
    __syncthreads();
    if (warp == 0 && f < F) {
#pragma unroll
      for (int i = 0; i <= KK; ++i) {
        float t = 0.f;
#pragma unroll
        for (int wq = 0; wq < 8; ++wq) t += c1_tile[(wq * 32 + lane) * (KK + 1) + i];
        g_c1_part[((size_t)f * (KK + 1) + i) * gridDim.x + blockIdx.x] = t;
      }
    }
  }
}

// The same with 16-byte loads of dy (F % 4 == 0): a lane holds four consecutive filters of one of four pixels the warp
// works on at a time, so a warp instruction brings in 512 bytes and the pixel loop has a quarter of the load
// instructions; the four pixel groups are folded with shuffles before the cross-warp reduction.
template <typename T, int K>
__global__ void __launch_bounds__(256) conv1_wgrad_img4_kernel(const OnoConvGeom g, int F, const T* x, int ldx, const T* dy, int ld_dy) {
  extern __shared__ float c1_tile[];
  constexpr int KK = K * K;
  const int TW = g.W + 2 * g.P, TH = g.H + 2 * g.P;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int fq = lane & 7, pg = lane >> 3;
  const int nfb = (F + 31) / 32;
  for (int fb = 0; fb < nfb; ++fb) {
    const int f4 = fb * 32 + 4 * fq;          // first of this lane's four filters
    const bool live = f4 < F;
    float acc[KK + 1][4];
#pragma unroll
    for (int i = 0; i <= KK; ++i) { acc[i][0] = 0.f; acc[i][1] = 0.f; acc[i][2] = 0.f; acc[i][3] = 0.f; }
    for (int img = blockIdx.x; img < g.B; img += gridDim.x) {
      __syncthreads();
      c1_stage_image(g, x, ldx, img, c1_tile, TW, TH);
      __syncthreads();
      for (int oy = warp; oy < g.OH; oy += 8) {
        const float* trow = c1_tile + oy * g.S * TW;
        const T* drow = dy + (long long)(img * g.OH + oy) * g.OW * ld_dy + f4;
#pragma unroll 2
        for (int ox = pg; ox < g.OW; ox += 4) {
          const float4 d = live ? load4(drow + (long long)ox * ld_dy) : make_float4(0.f, 0.f, 0.f, 0.f);
          const float* t0 = trow + ox * g.S;
#pragma unroll
          for (int ky = 0; ky < K; ++ky)
#pragma unroll
            for (int kx = 0; kx < K; ++kx) {
              const float t = t0[ky * TW + kx];
              acc[ky * K + kx][0] += d.x * t; acc[ky * K + kx][1] += d.y * t;
              acc[ky * K + kx][2] += d.z * t; acc[ky * K + kx][3] += d.w * t;
            }
          acc[KK][0] += d.x; acc[KK][1] += d.y; acc[KK][2] += d.z; acc[KK][3] += d.w;
        }
      }
    }
#pragma unroll
    for (int i = 0; i <= KK; ++i)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        float v = acc[i][c];
        v += __shfl_xor_sync(0xffffffffu, v, 8);
        v += __shfl_xor_sync(0xffffffffu, v, 16);
        acc[i][c] = v;
      }
    __syncthreads();   // the image is no longer needed: its space takes the warps' sums, [warp][filter][slot]
    if (pg == 0) {
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int i = 0; i <= KK; ++i) c1_tile[(warp * 32 + 4 * fq + c) * (KK + 1) + i] = acc[i][c];
    }
    __syncthreads();
    const int f = fb * 32 + lane;
    if (warp == 0 && f < F) {
#pragma unroll
      for (int i = 0; i <= KK; ++i) {
        float t = 0.f;
#pragma unroll
        for (int wq = 0; wq < 8; ++wq) t += c1_tile[(wq * 32 + lane) * (KK + 1) + i];
        g_c1_part[((size_t)f * (KK + 1) + i) * gridDim.x + blockIdx.x] = t;
      }
    }
  }
}

__global__ void __launch_bounds__(256) conv1_wgrad_reduce_kernel(int F, int kk, int nblocks, float* gk, float* gb, float beta) {
  const int lane = threadIdx.x & 31;
  const int pair = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (pair >= F * (kk + 1)) return;
  const float* p = g_c1_part + (size_t)pair * nblocks;
  float t = 0.f;
  for (int b = lane; b < nblocks; b += 32) t += p[b];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  if (lane == 0) {
    const int f = pair / (kk + 1), i = pair - f * (kk + 1);
    float* dst = i < kk ? gk + (long long)f * kk + i : gb + f;
    *dst = beta != 0.f ? beta * (*dst) + t : t;
  }
}

// Shared memory of the image-tiled kernels, or 0 when the shape has to take the generic kernels.
static size_t c1_img_smem(const OnoConvGeom* g) {
  if (g->K != 3 && g->K != 5) return 0;
  const size_t tile = (size_t)(g->H + 2 * g->P) * (g->W + 2 * g->P);
  const size_t red = (size_t)256 * (g->K * g->K + 1);
  const size_t bytes = std::max(tile, red) * sizeof(float);
  return bytes <= 48 * 1024 ? bytes : 0;
}

// y[(b,oy,ox), c] = max over the window of the zero-padded input; arg[...] = input pixel (iy*W+ix) of the
// maximum or -1 when the maximum is a padding zero. Ties: the last element in scan order.
template <typename T>
__global__ void pool_fwd_kernel(const OnoConvGeom g, const T* x, int ldx, T* y, int ldy, T* yT, int ld_yT, int* arg,
                                int act, float act_param) {
  const long long total = (long long)g.B * g.OH * g.OW * g.C;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i % g.C);
    const long long r = i / g.C;
    const int ox = (int)(r % g.OW), oy = (int)((r / g.OW) % g.OH), b = (int)(r / ((long long)g.OW * g.OH));
    float best = -INFINITY;
    int where = -1;
    for (int ky = 0; ky < g.K; ++ky)
      for (int kx = 0; kx < g.K; ++kx) {
        const int iy = oy * g.S + ky - g.P, ix = ox * g.S + kx - g.P;
        const bool in = iy >= 0 && iy < g.H && ix >= 0 && ix < g.W;
        const float v = in ? to_f32(x[((long long)(b * g.H + iy) * g.W + ix) * ldx + c]) : 0.f;
        if (v >= best) { best = v; where = in ? iy * g.W + ix : -1; }
      }
    arg[r * g.C + c] = where;
    const float out = act_fwd(act, act_param, best);
    y[r * ldy + c] = from_f32<T>(out);
    if (yT) yT[(long long)c * ld_yT + r] = from_f32<T>(out);
  }
}

// dx must be zero on entry. d is first taken through the pooling layer's own activation (on y), then
// routed to the arg-max input pixel. Overlapping windows (stride < k) make several outputs hit one pixel.
template <typename T>
__global__ void pool_bwd_kernel(const OnoConvGeom g, const T* d, int ldd, const T* y, int ldy, const int* arg, int act,
                                float act_param, int relu_quirk, float* dx, int ld_dx) {
  const long long total = (long long)g.B * g.OH * g.OW * g.C;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i % g.C);
    const long long r = i / g.C;
    const int where = arg[r * g.C + c];
    if (where < 0) continue;
    const int b = (int)(r / ((long long)g.OW * g.OH));
    float v = to_f32(d[r * ldd + c]);
    if (act != ACT_NONE) v = act_bwd(act, act_param, relu_quirk, to_f32(y[r * ldy + c]), v);
    atomicAdd(&dx[((long long)b * g.H * g.W + where) * ld_dx + c], v);
  }
}

// Pixel-major [B*HW, ldc] <-> the reference's flattened NCHW rows [B, C*HW] used by dense layers.
// to_flat = 1: flat[b, c*HW + p] = img[(b*HW + p), c]         (optionally also flatT[c*HW+p, b])
// to_flat = 0: img[(b*HW + p), c] = act'(aux) * flat[b, c*HW + p] (optionally also imgT[c, b*HW+p])
template <typename T>
__global__ void nchw_flat_kernel(int B, int C, int HW, int to_flat, T* img, int ld_img, T* flat, int ld_flat, T* outT,
                                 int ld_outT, const T* aux, int ld_aux, int dact, float dact_param, int relu_quirk) {
  const long long total = (long long)B * C * HW;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i % C);
    const long long bp = i / C;
    const int p = (int)(bp % HW), b = (int)(bp / HW);
    const long long f = (long long)c * HW + p;
    if (to_flat) {
      const T v = img[bp * ld_img + c];
      flat[(long long)b * ld_flat + f] = v;
      if (outT) outT[f * ld_outT + b] = v;
    } else {
      float v = to_f32(flat[(long long)b * ld_flat + f]);
      if (dact != ACT_NONE) v = act_bwd(dact, dact_param, relu_quirk, to_f32(aux[bp * ld_aux + c]), v);
      img[bp * ld_img + c] = from_f32<T>(v);
      if (outT) outT[(long long)c * ld_outT + bp] = from_f32<T>(v);
    }
  }
}

// f32 -> T with an activation derivative (pooling backward accumulates in f32).
template <typename T>
__global__ void finish_delta_kernel(long long rows, int C, const float* src, int ld_src, const T* aux, int ld_aux, int dact,
                                    float dact_param, int relu_quirk, T* dst, int ld_dst, T* dstT, int ld_dstT) {
  const long long total = rows * C;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i % C);
    const long long r = i / C;
    float v = src[r * ld_src + c];
    if (dact != ACT_NONE) v = act_bwd(dact, dact_param, relu_quirk, to_f32(aux[r * ld_aux + c]), v);
    dst[r * ld_dst + c] = from_f32<T>(v);
    if (dstT) dstT[(long long)c * ld_dstT + r] = from_f32<T>(v);
  }
}

static int grid_of(long long n) {
  long long g = (n + 255) / 256;
  if (g < 1) g = 1;
  if (g > 148 * 32) g = 148 * 32;
  return (int)g;
}
static int done(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { set_error("%s launch failed (%lld)", what, (long long)e, 0); return -7; }
  return 0;
}

}  // namespace ono

using namespace ono;
typedef __nv_bfloat16 bf16;

#define ONO_DISPATCH(dtype, CALL_F32, CALL_BF16) \
  if ((dtype) == 0) { CALL_F32; } else { CALL_BF16; }

extern "C" int ono_im2col(const OnoConvGeom* g, int dtype, const void* x, int ldx, void* cols, int ld_cols, void* colsT,
                          int ld_colsT, ono_stream_t st) {
  const long long n = (long long)g->B * g->OH * g->OW * g->C * g->K * g->K;
  const dim3 blk(32, 8);
  const int grid = grid_of(n / 4);
  {
    const int esz = dtype == 0 ? 4 : 2;
    const bool vec = g->C % 4 == 0 && ldx % 4 == 0 && ld_cols % 4 == 0 && (long long)g->B * g->H * g->W < (1ll << 31) &&
                     (long long)g->B * g->OH * g->OW < (1ll << 31) &&
                     (((uintptr_t)x | (uintptr_t)cols) & (uintptr_t)(4 * esz - 1)) == 0;
    if (vec) {
      ONO_DISPATCH(dtype,
                   (im2col_vec_kernel<float><<<grid, 256, 0, (cudaStream_t)st>>>(*g, (const float*)x, ldx, (float*)cols, ld_cols, (float*)colsT, ld_colsT)),
                   (im2col_vec_kernel<bf16><<<grid, 256, 0, (cudaStream_t)st>>>(*g, (const bf16*)x, ldx, (bf16*)cols, ld_cols, (bf16*)colsT, ld_colsT)))
      return done("im2col");
    }
  }
  ONO_DISPATCH(dtype,
               (im2col_kernel<float><<<grid, blk, 0, (cudaStream_t)st>>>(*g, (const float*)x, ldx, (float*)cols, ld_cols, (float*)colsT, ld_colsT)),
               (im2col_kernel<bf16><<<grid, blk, 0, (cudaStream_t)st>>>(*g, (const bf16*)x, ldx, (bf16*)cols, ld_cols, (bf16*)colsT, ld_colsT)))
  return done("im2col");
}

extern "C" int ono_col2im(const OnoConvGeom* g, int dtype, const void* dcols, int ld_dcols, const void* aux, int ld_aux,
                          int dact, float dact_param, int relu_quirk, void* dx, int ld_dx, void* dxT, int ld_dxT, ono_stream_t st) {
  const long long n = (long long)g->B * g->H * g->W * ((g->C + 31) / 32 * 32);
  const dim3 blk(32, 8);
  const int grid = grid_of(n / 4);
  const int esz = dtype == 0 ? 4 : 2;
  const bool vec = g->C % 4 == 0 && ld_dcols % 4 == 0 && ld_dx % 4 == 0 && (!aux || ld_aux % 4 == 0) &&
                   (long long)g->B * g->H * g->W < (1ll << 31) && (long long)g->B * g->OH * g->OW < (1ll << 31) &&
                   (((uintptr_t)dcols | (uintptr_t)dx | (uintptr_t)aux) & (uintptr_t)(4 * esz - 1)) == 0 && (aux || dact == ACT_NONE);
#define ONO_COL2IM_VEC(KK, SS)                                                                                                   \
  if (vec && g->K == KK && g->S == SS) {                                                                                          \
    ONO_DISPATCH(dtype,                                                                                                           \
                 (col2im_vec_kernel<float, KK, SS><<<grid, 256, 0, (cudaStream_t)st>>>(*g, (const float*)dcols, ld_dcols, (const float*)aux, ld_aux, dact, dact_param, relu_quirk, (float*)dx, ld_dx, (float*)dxT, ld_dxT)), \
                 (col2im_vec_kernel<bf16, KK, SS><<<grid, 256, 0, (cudaStream_t)st>>>(*g, (const bf16*)dcols, ld_dcols, (const bf16*)aux, ld_aux, dact, dact_param, relu_quirk, (bf16*)dx, ld_dx, (bf16*)dxT, ld_dxT))) \
    return done("col2im");                                                                                                        \
  }
  ONO_COL2IM_VEC(3, 1)
  ONO_COL2IM_VEC(3, 2)
  ONO_COL2IM_VEC(5, 1)
  ONO_COL2IM_VEC(5, 2)
#undef ONO_COL2IM_VEC
  ONO_DISPATCH(dtype,
               (col2im_kernel<float><<<grid, blk, 0, (cudaStream_t)st>>>(*g, (const float*)dcols, ld_dcols, (const float*)aux, ld_aux, dact, dact_param, relu_quirk, (float*)dx, ld_dx, (float*)dxT, ld_dxT)),
               (col2im_kernel<bf16><<<grid, blk, 0, (cudaStream_t)st>>>(*g, (const bf16*)dcols, ld_dcols, (const bf16*)aux, ld_aux, dact, dact_param, relu_quirk, (bf16*)dx, ld_dx, (bf16*)dxT, ld_dxT)))
  return done("col2im");
}

extern "C" int ono_conv1_fwd(const OnoConvGeom* g, int F, int dtype, const void* x, int ldx, const float* kparams, const float* bias,
                             int act, float act_param, void* y, int ldy, ono_stream_t st) {
  if (!g || g->C != 1 || g->K * g->K > C1_MAXKK || F <= 0) { set_error("conv1_fwd: needs one input channel and k <= 5%s", "", 0, 0); return -1; }
  const long long rows = (long long)g->B * g->OH * g->OW;
  if (rows >= (1ll << 31)) { set_error("conv1_fwd: too many output pixels%s", "", 0, 0); return -1; }
  if (const size_t sm = c1_img_smem(g)) {
    const dim3 grid((unsigned)std::min(g->B, 148 * 8), (F + 31) / 32);
    cudaStream_t s = (cudaStream_t)st;
    const int esz = dtype == 0 ? 4 : 2;
    const bool v4 = F % 4 == 0 && ldy % 4 == 0 && ((uintptr_t)y & (uintptr_t)(4 * esz - 1)) == 0;
    if (v4 && g->K == 3) {
      ONO_DISPATCH(dtype,
                   (conv1_fwd_img4_kernel<float, 3><<<grid, 256, sm, s>>>(*g, F, (const float*)x, ldx, kparams, bias, act, act_param, (float*)y, ldy)),
                   (conv1_fwd_img4_kernel<bf16, 3><<<grid, 256, sm, s>>>(*g, F, (const bf16*)x, ldx, kparams, bias, act, act_param, (bf16*)y, ldy)))
    } else if (v4) {
      ONO_DISPATCH(dtype,
                   (conv1_fwd_img4_kernel<float, 5><<<grid, 256, sm, s>>>(*g, F, (const float*)x, ldx, kparams, bias, act, act_param, (float*)y, ldy)),
                   (conv1_fwd_img4_kernel<bf16, 5><<<grid, 256, sm, s>>>(*g, F, (const bf16*)x, ldx, kparams, bias, act, act_param, (bf16*)y, ldy)))
    } else if (g->K == 3) {
      ONO_DISPATCH(dtype,
                   (conv1_fwd_img_kernel<float, 3><<<grid, 256, sm, s>>>(*g, F, (const float*)x, ldx, kparams, bias, act, act_param, (float*)y, ldy)),
                   (conv1_fwd_img_kernel<bf16, 3><<<grid, 256, sm, s>>>(*g, F, (const bf16*)x, ldx, kparams, bias, act, act_param, (bf16*)y, ldy)))
    } else {
      ONO_DISPATCH(dtype,
                   (conv1_fwd_img_kernel<float, 5><<<grid, 256, sm, s>>>(*g, F, (const float*)x, ldx, kparams, bias, act, act_param, (float*)y, ldy)),
                   (conv1_fwd_img_kernel<bf16, 5><<<grid, 256, sm, s>>>(*g, F, (const bf16*)x, ldx, kparams, bias, act, act_param, (bf16*)y, ldy)))
    }
    return done("conv1_fwd");
  }
  const dim3 blk(32, 8), grid((unsigned)std::min<long long>((rows + 255) / 256, 148 * 8), (F + 31) / 32);
  ONO_DISPATCH(dtype,
               (conv1_fwd_kernel<float><<<grid, blk, 0, (cudaStream_t)st>>>(*g, F, (const float*)x, ldx, kparams, bias, act, act_param, (float*)y, ldy)),
               (conv1_fwd_kernel<bf16><<<grid, blk, 0, (cudaStream_t)st>>>(*g, F, (const bf16*)x, ldx, kparams, bias, act, act_param, (bf16*)y, ldy)))
  return done("conv1_fwd");
}

extern "C" int ono_conv1_wgrad(const OnoConvGeom* g, int F, int dtype, const void* x, int ldx, const void* dy, int ld_dy, float* gk,
                               float* gb, float beta, ono_stream_t st) {
  if (!g || g->C != 1 || g->K * g->K > C1_MAXKK || F <= 0 || F > C1_MAXF) { set_error("conv1_wgrad: needs one input channel, k <= 5, F <= 128%s", "", 0, 0); return -1; }
  const long long rows = (long long)g->B * g->OH * g->OW;
  const dim3 blk(32, 8);
  if (rows >= (1ll << 31)) { set_error("conv1_wgrad: too many output pixels%s", "", 0, 0); return -1; }
  if (const size_t sm = c1_img_smem(g)) {
    const int nb = std::min(g->B, C1_MAXBLOCKS);
    cudaStream_t s = (cudaStream_t)st;
    const int esz = dtype == 0 ? 4 : 2;
    const bool v4 = F % 4 == 0 && ld_dy % 4 == 0 && ((uintptr_t)dy & (uintptr_t)(4 * esz - 1)) == 0;
    if (v4 && g->K == 3) {
      ONO_DISPATCH(dtype,
                   (conv1_wgrad_img4_kernel<float, 3><<<nb, 256, sm, s>>>(*g, F, (const float*)x, ldx, (const float*)dy, ld_dy)),
                   (conv1_wgrad_img4_kernel<bf16, 3><<<nb, 256, sm, s>>>(*g, F, (const bf16*)x, ldx, (const bf16*)dy, ld_dy)))
    } else if (v4) {
      ONO_DISPATCH(dtype,
                   (conv1_wgrad_img4_kernel<float, 5><<<nb, 256, sm, s>>>(*g, F, (const float*)x, ldx, (const float*)dy, ld_dy)),
                   (conv1_wgrad_img4_kernel<bf16, 5><<<nb, 256, sm, s>>>(*g, F, (const bf16*)x, ldx, (const bf16*)dy, ld_dy)))
    } else if (g->K == 3) {
      ONO_DISPATCH(dtype,
                   (conv1_wgrad_img_kernel<float, 3><<<nb, 256, sm, s>>>(*g, F, (const float*)x, ldx, (const float*)dy, ld_dy)),
                   (conv1_wgrad_img_kernel<bf16, 3><<<nb, 256, sm, s>>>(*g, F, (const bf16*)x, ldx, (const bf16*)dy, ld_dy)))
    } else {
      ONO_DISPATCH(dtype,
                   (conv1_wgrad_img_kernel<float, 5><<<nb, 256, sm, s>>>(*g, F, (const float*)x, ldx, (const float*)dy, ld_dy)),
                   (conv1_wgrad_img_kernel<bf16, 5><<<nb, 256, sm, s>>>(*g, F, (const bf16*)x, ldx, (const bf16*)dy, ld_dy)))
    }
    const int pairs = F * (g->K * g->K + 1);
    conv1_wgrad_reduce_kernel<<<(pairs + 7) / 8, 256, 0, s>>>(F, g->K * g->K, nb, gk, gb, beta);
    return done("conv1_wgrad");
  }
  const int grid = (int)std::min<long long>((rows + 255) / 256, C1_MAXBLOCKS);
  ONO_DISPATCH(dtype,
               (conv1_wgrad_kernel<float><<<grid, blk, 0, (cudaStream_t)st>>>(*g, F, (const float*)x, ldx, (const float*)dy, ld_dy, gk, gb, beta)),
               (conv1_wgrad_kernel<bf16><<<grid, blk, 0, (cudaStream_t)st>>>(*g, F, (const bf16*)x, ldx, (const bf16*)dy, ld_dy, gk, gb, beta)))
  return done("conv1_wgrad");
}

extern "C" int ono_conv_kperm(int F, int C, int K, int dir, int dtype, const float* src, int ld_src, void* dst, int ld_dst,
                              void* dstT, int ld_dstT, float beta, ono_stream_t st) {
  if (F <= 0 || C <= 0 || K <= 0 || !src || !dst) { set_error("bad kperm args%s", "", 0, 0); return -1; }
  const long long n = (long long)F * C * K * K;
  ONO_DISPATCH(dtype,
               (kperm_kernel<float><<<grid_of(n), 256, 0, (cudaStream_t)st>>>(F, C, K, dir, src, ld_src, dst, ld_dst, (float*)dstT, ld_dstT, beta)),
               (kperm_kernel<bf16><<<grid_of(n), 256, 0, (cudaStream_t)st>>>(F, C, K, dir, src, ld_src, dst, ld_dst, (bf16*)dstT, ld_dstT, beta)))
  return done("conv_kperm");
}

extern "C" int ono_pool_fwd(const OnoConvGeom* g, int dtype, const void* x, int ldx, void* y, int ldy, void* yT, int ld_yT,
                            int* arg, int act, float act_param, ono_stream_t st) {
  const long long n = (long long)g->B * g->OH * g->OW * g->C;
  ONO_DISPATCH(dtype,
               (pool_fwd_kernel<float><<<grid_of(n), 256, 0, (cudaStream_t)st>>>(*g, (const float*)x, ldx, (float*)y, ldy, (float*)yT, ld_yT, arg, act, act_param)),
               (pool_fwd_kernel<bf16><<<grid_of(n), 256, 0, (cudaStream_t)st>>>(*g, (const bf16*)x, ldx, (bf16*)y, ldy, (bf16*)yT, ld_yT, arg, act, act_param)))
  return done("pool_fwd");
}

extern "C" int ono_pool_bwd(const OnoConvGeom* g, int dtype, const void* d, int ldd, const void* y, int ldy, const int* arg,
                            int act, float act_param, int relu_quirk, float* dx, int ld_dx, ono_stream_t st) {
  const long long n = (long long)g->B * g->OH * g->OW * g->C;
  ONO_DISPATCH(dtype,
               (pool_bwd_kernel<float><<<grid_of(n), 256, 0, (cudaStream_t)st>>>(*g, (const float*)d, ldd, (const float*)y, ldy, arg, act, act_param, relu_quirk, dx, ld_dx)),
               (pool_bwd_kernel<bf16><<<grid_of(n), 256, 0, (cudaStream_t)st>>>(*g, (const bf16*)d, ldd, (const bf16*)y, ldy, arg, act, act_param, relu_quirk, dx, ld_dx)))
  return done("pool_bwd");
}

extern "C" int ono_nchw_flat(int dtype, int B, int C, int HW, int to_flat, void* img, int ld_img, void* flat, int ld_flat,
                             void* outT, int ld_outT, const void* aux, int ld_aux, int dact, float dact_param, int relu_quirk,
                             ono_stream_t st) {
  const long long n = (long long)B * C * HW;
  ONO_DISPATCH(dtype,
               (nchw_flat_kernel<float><<<grid_of(n), 256, 0, (cudaStream_t)st>>>(B, C, HW, to_flat, (float*)img, ld_img, (float*)flat, ld_flat, (float*)outT, ld_outT, (const float*)aux, ld_aux, dact, dact_param, relu_quirk)),
               (nchw_flat_kernel<bf16><<<grid_of(n), 256, 0, (cudaStream_t)st>>>(B, C, HW, to_flat, (bf16*)img, ld_img, (bf16*)flat, ld_flat, (bf16*)outT, ld_outT, (const bf16*)aux, ld_aux, dact, dact_param, relu_quirk)))
  return done("nchw_flat");
}

extern "C" int ono_finish_delta(int dtype, long long rows, int C, const float* src, int ld_src, const void* aux, int ld_aux,
                                int dact, float dact_param, int relu_quirk, void* dst, int ld_dst, void* dstT, int ld_dstT,
                                ono_stream_t st) {
  const long long n = rows * C;
  ONO_DISPATCH(dtype,
               (finish_delta_kernel<float><<<grid_of(n), 256, 0, (cudaStream_t)st>>>(rows, C, src, ld_src, (const float*)aux, ld_aux, dact, dact_param, relu_quirk, (float*)dst, ld_dst, (float*)dstT, ld_dstT)),
               (finish_delta_kernel<bf16><<<grid_of(n), 256, 0, (cudaStream_t)st>>>(rows, C, src, ld_src, (const bf16*)aux, ld_aux, dact, dact_param, relu_quirk, (bf16*)dst, ld_dst, (bf16*)dstT, ld_dstT)))
  return done("finish_delta");
}
