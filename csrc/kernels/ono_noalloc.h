// Allocation-free entry point of the fused optimizer/synchronisation step.
//
// This has no counterpart in the reference (which has no GPU code at all); it exists for callers of
// this library that must not allocate device memory: a plug-in inside a serving or training process
// whose framework has already handed the whole HBM to its own caching allocator, code that runs
// between another component's captured CUDA graphs, or a recovery path that must not take the
// allocator's lock. There cudaMalloc can fail, stall the whole device, or wait on a lock the caller's
// own thread already holds.
//
// ono_sync_step (ono_kernels.h) needs two pieces of scratch memory from its caller besides the
// tensors it works on: the epoch-stamped flag pad and the per-block epoch words of its barrier.
// ono_sync_step_noalloc keeps exactly that scratch in a fixed array inside the library's device image
// (ONO_NOALLOC_SCRATCH_BYTES bytes, held by every GPU that loads the library until the process
// exits), for the single-GPU form of the step: one rank that owns the whole vector, i.e. the fused
// "scale the gradient, apply SGD / momentum / Adam, refresh the bf16 shadow, accumulate the gradient
// norm" pass.
//
// Rules of use:
//   * The caller passes every input and output (p, g, m, v, p_bf16, adam_pows, sumsq, status); the
//     call launches one kernel on `stream` and calls no allocating routine.
//   * At most ONO_NOALLOC_MAX_BLOCKS thread blocks (nblocks = 0 picks a grid); a larger request is
//     rejected with an error and nothing is launched.
//   * The first call on each device looks up the device address of the scratch array (that device
//     must be current). Make that first call outside any stream capture.
//   * All calls on a device share the scratch array. Its words are monotonically increasing stamps
//     that carry over from one call to the next by design (nothing has to be cleared between calls),
//     but two calls that overlap on the GPU (different streams, no ordering) race on them: order the
//     calls, as a single stream does.
#pragma once
#include "ono_kernels.h"

#ifdef __cplusplus
extern "C" {
#endif

#define ONO_NOALLOC_MAX_BLOCKS 512
#define ONO_NOALLOC_SCRATCH_BYTES (ONO_NOALLOC_MAX_BLOCKS * (ONO_MAX_RANKS + 1) * 4)

typedef struct OnoNoAllocStep {
  float* p;                // [n] parameters, updated in place
  const float* g;          // [n] gradient
  float* m;                // [n] first-moment / velocity state (momentum, Adam), else null
  float* v;                // [n] second-moment state (Adam), else null
  void* p_bf16;            // optional [n] bf16 copy of the updated parameters, 8-byte aligned
  long long n;             // element count, a multiple of 4 (pad the buffers); p, g, m, v 16-byte aligned
  int kind;                // 0 SGD, 1 momentum, 2 Adam
  float lr, mu, b1, b2, eps;
  int n_workers;           // the gradient is divided by this first (values below 1 mean 1)
  const float* adam_pows;  // device float[2] = {b1^t, b2^t} for this step (Adam only)
  double* sumsq;           // optional device double (8-byte aligned), += sum of squares of the scaled gradient
  int* status;             // optional device int, set non-zero if an in-kernel wait gave up
  int nblocks;             // 0 = choose; at most ONO_NOALLOC_MAX_BLOCKS
} OnoNoAllocStep;

// Returns 0 on success, a negative value if the arguments are rejected or the launch failed
// (ono_last_error() has the text).
int ono_sync_step_noalloc(const OnoNoAllocStep* s, ono_stream_t stream);

#ifdef __cplusplus
}
#endif
