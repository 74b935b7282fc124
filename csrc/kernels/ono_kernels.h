// C ABI of the sm_100a kernel library (libono_kernels.so). Everything takes raw device pointers and
// a cudaStream_t so that the library has no dependency on a tensor framework: PyTorch owns the
// allocations and streams and calls in through ctypes; the C++ engine calls in directly.
//
// Every launcher returns 0 on success or a negative value for an argument error (nothing is
// launched in that case). Kernels that wait on something (mbarriers, peer flags) report a timeout
// by writing a non-zero code to the `status` word the caller supplied; the context stays usable.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* ono_stream_t;

enum OnoDtype { ONO_TF32 = 0, ONO_BF16 = 1 };      // tile dtype of a GEMM (tf32 reads f32 storage)
enum OnoMajor { ONO_K_MAJOR = 0, ONO_MN_MAJOR = 1 };

// Epilogue of the tcgen05 GEMM. v = acc[m][n] (f32, from TMEM), then in order:
//   v *= alpha (if alpha != 1); v += bias[n]; pre[m][n] = v; v = act(v);
//   v = dact(aux[m][n]) applied to v (backward through the previous activation);
//   v += beta * out_f32[m][n]; stores to any of out_f32 / outT_f32 / out_bf16 / outT_bf16.
typedef struct OnoEpilogue {
  float* out_f32;            // [M, ld_out] row-major, optional
  float* outT_f32;           // [N, ld_outT] (transposed copy), optional
  void* out_bf16;            // [M, ld_out], optional
  void* outT_bf16;           // [N, ld_outT], optional
  float* pre_f32;            // [M, ld_out] pre-activation, optional
  void* pre_bf16;            // [M, ld_out] pre-activation, optional
  const float* bias;         // [N], optional
  const float* aux_f32;      // [M, ld_aux], optional (stored activation or pre-activation)
  const void* aux_bf16;      // same in bf16, optional
  int ld_out, ld_outT, ld_aux;
  int act;                   // ActKind applied forward
  float act_param;
  int dact;                  // ActKind whose derivative multiplies v
  float dact_param;
  int relu_quirk;            // reproduce the reference's leaky-ReLU backward
  float alpha, beta;
} OnoEpilogue;

// D[M,N] = A[M,K] * B[K,N] with f32 accumulation in TMEM.
//   A: a_major == K_MAJOR  -> memory is [M, lda] with K contiguous
//      a_major == MN_MAJOR -> memory is [K, lda] with M contiguous (bf16 only)
//   B: b_major == K_MAJOR  -> memory is [N, ldb] with K contiguous
//      b_major == MN_MAJOR -> memory is [K, ldb] with N contiguous (bf16 only)
// Leading dimensions are in elements and must make row strides a multiple of 16 bytes.
typedef struct OnoGemm {
  const void* A;
  const void* B;
  int M, N, K;
  int lda, ldb;
  int dtype;       // OnoDtype
  int a_major, b_major;
  int bn;          // tile N: 0 = auto, else 32 / 128 / 256
  int max_ctas;    // 0 = one per SM
  OnoEpilogue epi;
  int* status;     // device int, set non-zero on an in-kernel timeout; may be null
} OnoGemm;

int ono_gemm(const OnoGemm* g, ono_stream_t stream);
// Last error text of this thread (argument errors / CUDA errors), for diagnostics.
const char* ono_last_error(void);
int ono_num_sms(void);

#ifdef __cplusplus
}
#endif
