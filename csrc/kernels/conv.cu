// Convolution and pooling around the tcgen05 GEMM: the gather / scatter halves of the reference's
// im2col convolution (machine_learning/src/arch/layers/conv/conv2d.rs:84-104,202-266) and its max
// pooling (arch/layers/max_pooling.rs:47-157), on pixel-major activations.
//
// Activations of image layers are 2-D matrices [B*H*W, ldc] (one row per pixel, channels contiguous),
// which is exactly what the GEMM epilogue writes for Y = cols * K^T; the column order of `cols` is
// (c, ky, kx), i.e. the reference's kernel layout K[F][C][k][k] is used as the GEMM operand in place.
// Semantics kept from the reference: zero padding, output size floor((H+2p-k)/s)+1 (trailing rows and
// columns the strided window never reaches are dropped), zero padding competes in the max, and a
// pooling gradient whose arg-max lies in the padding is dropped.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

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

// cols[r, q] = x[(b, oy*s+ky-p, ox*s+kx-p), c]  with r = (b, oy, ox), q = (c, ky, kx); optional colsT.
template <typename T>
__global__ void im2col_kernel(const OnoConvGeom g, const T* x, int ldx, T* cols, int ld_cols, T* colsT, int ld_colsT) {
  const int ckk = g.C * g.K * g.K;
  const long long total = (long long)g.B * g.OH * g.OW * ckk;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int q = (int)(i % ckk);
    const long long r = i / ckk;
    const int kx = q % g.K, ky = (q / g.K) % g.K, c = q / (g.K * g.K);
    const int ox = (int)(r % g.OW), oy = (int)((r / g.OW) % g.OH), b = (int)(r / ((long long)g.OW * g.OH));
    const int iy = oy * g.S + ky - g.P, ix = ox * g.S + kx - g.P;
    T v = from_f32<T>(0.f);
    if (iy >= 0 && iy < g.H && ix >= 0 && ix < g.W) v = x[((long long)(b * g.H + iy) * g.W + ix) * ldx + c];
    cols[r * ld_cols + q] = v;
    if (colsT) colsT[(long long)q * ld_colsT + r] = v;
  }
}

// dx[(b,iy,ix), c] = act'(aux) * sum_{ky,kx} dcols[(b,oy,ox), (c,ky,kx)] over the windows covering it.
template <typename T>
__global__ void col2im_kernel(const OnoConvGeom g, const T* dcols, int ld_dcols, const T* aux, int ld_aux, int dact,
                              float dact_param, int relu_quirk, T* dx, int ld_dx, T* dxT, int ld_dxT) {
  const long long total = (long long)g.B * g.H * g.W * g.C;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i % g.C);
    const long long pix = i / g.C;
    const int ix = (int)(pix % g.W), iy = (int)((pix / g.W) % g.H), b = (int)(pix / ((long long)g.W * g.H));
    float acc = 0.f;
    for (int ky = 0; ky < g.K; ++ky) {
      const int ty = iy + g.P - ky;
      if (ty < 0 || ty % g.S) continue;
      const int oy = ty / g.S;
      if (oy >= g.OH) continue;
      for (int kx = 0; kx < g.K; ++kx) {
        const int tx = ix + g.P - kx;
        if (tx < 0 || tx % g.S) continue;
        const int ox = tx / g.S;
        if (ox >= g.OW) continue;
        acc += to_f32(dcols[((long long)(b * g.OH + oy) * g.OW + ox) * ld_dcols + (c * g.K + ky) * g.K + kx]);
      }
    }
    if (dact != ACT_NONE) acc = act_bwd(dact, dact_param, relu_quirk, to_f32(aux[pix * ld_aux + c]), acc);
    dx[pix * ld_dx + c] = from_f32<T>(acc);
    if (dxT) dxT[(long long)c * ld_dxT + pix] = from_f32<T>(acc);
  }
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
  ONO_DISPATCH(dtype,
               (im2col_kernel<float><<<grid_of(n), 256, 0, (cudaStream_t)st>>>(*g, (const float*)x, ldx, (float*)cols, ld_cols, (float*)colsT, ld_colsT)),
               (im2col_kernel<bf16><<<grid_of(n), 256, 0, (cudaStream_t)st>>>(*g, (const bf16*)x, ldx, (bf16*)cols, ld_cols, (bf16*)colsT, ld_colsT)))
  return done("im2col");
}

extern "C" int ono_col2im(const OnoConvGeom* g, int dtype, const void* dcols, int ld_dcols, const void* aux, int ld_aux,
                          int dact, float dact_param, int relu_quirk, void* dx, int ld_dx, void* dxT, int ld_dxT, ono_stream_t st) {
  const long long n = (long long)g->B * g->H * g->W * g->C;
  ONO_DISPATCH(dtype,
               (col2im_kernel<float><<<grid_of(n), 256, 0, (cudaStream_t)st>>>(*g, (const float*)dcols, ld_dcols, (const float*)aux, ld_aux, dact, dact_param, relu_quirk, (float*)dx, ld_dx, (float*)dxT, ld_dxT)),
               (col2im_kernel<bf16><<<grid_of(n), 256, 0, (cudaStream_t)st>>>(*g, (const bf16*)dcols, ld_dcols, (const bf16*)aux, ld_aux, dact, dact_param, relu_quirk, (bf16*)dx, ld_dx, (bf16*)dxT, ld_dxT)))
  return done("col2im");
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
