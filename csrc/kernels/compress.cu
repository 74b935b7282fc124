// Gradient compression on the device: the f16 wire and the sparse "gradient dropping" serializer of the
// reference (comms/src/handles/compressor.rs:71-118, comms/src/sparse/protocol.rs:33-144), as kernels.
//
//   threshold   k-th smallest |x| of a stratified Philox sample of at most 16 384 elements, k = floor(sample*(1-r)),
//               floored at the smallest positive normal f16: the same samples and the same order statistic as the
//               host codec (core/codec.cpp), so both give the same number.
//   mask        what a rank puts on the wire and what it keeps: wire[i] = f16(x[i]) where |x[i]| >= threshold, else 0;
//               the sent entries are zeroed in the residual, the rest stays for the next round
//               (worker/src/middlewares/server_cluster.rs:85-104). Without a threshold it is the plain f16 wire.
//               Peers then reduce the wire buffer over NVLink like any gradient buffer.
//   compact     the same selection as (index, f16 value) pairs in ascending index order plus their count
//               (three passes: per-block counts, scan of the counts, ordered write) and
//   lift        acc[index] += value, the receiver's side (protocol.rs:96-144).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>

#include "../core/philox.h"
#include "ono_kernels.h"

namespace ono {
void set_error(const char* fmt, const char* a, long long b, long long c);

constexpr int SPARSE_SAMPLE_MAX = 1 << 14;
constexpr float MIN_POSITIVE_F16 = 6.103515625e-05f;

__device__ __forceinline__ float f16_round(float x) { return __half2float(__float2half_rn(x)); }

// One block, 1024 threads; the sample lives in shared memory and is sorted with a bitonic network.
__global__ void __launch_bounds__(1024) sparse_threshold_kernel(const float* x, long long n, float keep, unsigned long long seed,
                                                                float* thr_out) {
  extern __shared__ float sm[];
  const int sample = (int)min((long long)SPARSE_SAMPLE_MAX, n);
  int padded = 1;
  while (padded < sample) padded <<= 1;
  const double stride = (double)n / (double)sample;
  for (int i = threadIdx.x; i < padded; i += blockDim.x) {
    float v = INFINITY;
    if (i < sample) {
      long long idx = i;
      if (sample != n) {
        const Philox4 rnd = philox4x32_10((uint64_t)i, seed);
        const double u = (double)(rnd.v[0] >> 8) * (1.0 / 16777216.0);
        idx = (long long)(((double)i + u) * stride);
        if (idx >= n) idx = n - 1;
      }
      v = fabsf(x[idx]);
    }
    sm[i] = v;
  }
  __syncthreads();
  for (int k = 2; k <= padded; k <<= 1)
    for (int j = k >> 1; j > 0; j >>= 1) {
      for (int i = threadIdx.x; i < padded; i += blockDim.x) {
        const int l = i ^ j;
        if (l > i) {
          const float a = sm[i], b = sm[l];
          const bool up = (i & k) == 0;
          if ((a > b) == up) { sm[i] = b; sm[l] = a; }
        }
      }
      __syncthreads();
    }
  if (threadIdx.x == 0) {
    int k = (int)((float)sample * (1.0f - keep));
    k = min(k, sample - 1);
    *thr_out = fmaxf(sm[k], MIN_POSITIVE_F16);
  }
}

// wire_f32 (optional): the selection as f32 values rounded through f16; wire16 (optional): the same as 16-bit values
// (f16, or bf16 when f16 == 0), which is what crosses NVLink. Entries that are not sent are zero on the wire.
__global__ void sparse_mask_kernel(float* residual, long long n, const float* thr, float* wire_f32, uint16_t* wire16, int f16,
                                   unsigned long long* sent) {
  const float t = thr ? *thr : -1.0f;   // no threshold: everything is sent (plain 16-bit wire)
  unsigned long long mine = 0;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float v = residual[i];
    const bool send = fabsf(v) >= t;
    if (wire_f32) wire_f32[i] = send ? f16_round(v) : 0.0f;
    if (wire16) {
      uint16_t w = 0;
      if (send) {
        if (f16) { const __half h = __float2half_rn(v); w = *reinterpret_cast<const uint16_t*>(&h); }
        else { const __nv_bfloat16 h = __float2bfloat16_rn(v); w = *reinterpret_cast<const uint16_t*>(&h); }
      }
      wire16[i] = w;
    }
    if (send) { residual[i] = 0.0f; ++mine; }
  }
  if (sent) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mine += __shfl_xor_sync(0xffffffffu, mine, o);
    if ((threadIdx.x & 31) == 0 && mine) atomicAdd(sent, mine);
  }
}

constexpr int CB = 1024;  // elements per block in the compaction passes

__global__ void __launch_bounds__(256) compact_count_kernel(const float* x, long long n, const float* thr, unsigned int* counts) {
  const float t = *thr;
  const long long base = (long long)blockIdx.x * CB;
  int c = 0;
  for (int j = threadIdx.x; j < CB; j += 256) {
    const long long i = base + j;
    if (i < n && fabsf(x[i]) >= t) ++c;
  }
  __shared__ int s[8];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
  if ((threadIdx.x & 31) == 0) s[threadIdx.x >> 5] = c;
  __syncthreads();
  if (threadIdx.x == 0) {
    int tot = 0;
    for (int w = 0; w < 8; ++w) tot += s[w];
    counts[blockIdx.x] = (unsigned)tot;
  }
}

// Exclusive scan of the block counts in place (one block; the number of blocks is n / 1024).
__global__ void __launch_bounds__(1024) compact_scan_kernel(unsigned int* counts, int nblocks, unsigned int* total) {
  __shared__ unsigned int s[1024];
  __shared__ unsigned int carry;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  for (int b0 = 0; b0 < nblocks; b0 += 1024) {
    const int i = b0 + threadIdx.x;
    const unsigned int v = i < nblocks ? counts[i] : 0u;
    s[threadIdx.x] = v;
    __syncthreads();
    for (int o = 1; o < 1024; o <<= 1) {
      const unsigned int add = threadIdx.x >= o ? s[threadIdx.x - o] : 0u;
      __syncthreads();
      s[threadIdx.x] += add;
      __syncthreads();
    }
    if (i < nblocks) counts[i] = carry + s[threadIdx.x] - v;
    __syncthreads();
    if (threadIdx.x == 0) carry += s[1023];
    __syncthreads();
  }
  if (threadIdx.x == 0) *total = carry;
}

__global__ void __launch_bounds__(256) compact_write_kernel(float* x, long long n, const float* thr, const unsigned int* offsets,
                                                            unsigned int* idx, __half* val, unsigned int capacity, int zero_sent) {
  const float t = *thr;
  const long long base = (long long)blockIdx.x * CB;
  __shared__ unsigned int warp_base[8];
  __shared__ unsigned int running;
  if (threadIdx.x == 0) running = offsets[blockIdx.x];
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int j0 = 0; j0 < CB; j0 += 256) {      // ascending order: chunk, then warp, then lane
    const long long i = base + j0 + threadIdx.x;
    const float v = i < n ? x[i] : 0.0f;
    const bool send = i < n && fabsf(v) >= t;
    const unsigned int bal = __ballot_sync(0xffffffffu, send);
    if (lane == 0) warp_base[warp] = __popc(bal);
    __syncthreads();
    unsigned int before = running;
    for (int w = 0; w < warp; ++w) before += warp_base[w];
    if (send) {
      const unsigned int at = before + __popc(bal & ((1u << lane) - 1u));
      if (at < capacity) { idx[at] = (unsigned int)i; val[at] = __float2half_rn(v); }
      if (zero_sent) x[i] = 0.0f;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      unsigned int tot = 0;
      for (int w = 0; w < 8; ++w) tot += warp_base[w];
      running += tot;
    }
    __syncthreads();
  }
}

__global__ void sparse_lift_kernel(float* acc, long long n, const unsigned int* idx, const __half* val, const unsigned int* count,
                                   unsigned int capacity) {
  const unsigned int c = min(*count, capacity);
  for (unsigned int i = blockIdx.x * blockDim.x + threadIdx.x; i < c; i += gridDim.x * blockDim.x) {
    const unsigned int at = idx[i];
    if ((long long)at < n) acc[at] += __half2float(val[i]);   // indices of one message are distinct
  }
}

// The receiving side of the sparse wire for one sender and one owned range [begin, end): if the sender's message fits its
// list (count <= capacity) the owner looks up the part of the ascending index list that falls into its range (two binary
// searches) and adds exactly those (index, f16) pairs; otherwise the sender fell back to the dense 16-bit wire
// (protocol.rs:57-86 falls back when the sparse encoding is the larger one) and the owner adds that range of it.
// idx / val / count / dense16 may live in the sender's window (peer memory). *bytes += what was read from the sender.
__global__ void sparse_lift_range_kernel(float* acc, long long begin, long long end, const unsigned int* idx, const __half* val,
                                         const unsigned int* count, unsigned int capacity, const uint16_t* dense16, int dense_f16,
                                         unsigned long long* bytes) {
  __shared__ unsigned int s_lo, s_hi, s_cnt;
  if (threadIdx.x == 0) {
    const unsigned int c = *reinterpret_cast<const volatile unsigned int*>(count);
    s_cnt = c;
    if (c <= capacity) {
      auto lower = [&](unsigned int key) {
        unsigned int lo = 0, hi = c;
        while (lo < hi) {
          const unsigned int mid = (lo + hi) >> 1;
          if (reinterpret_cast<const volatile unsigned int*>(idx)[mid] < key) lo = mid + 1; else hi = mid;
        }
        return lo;
      };
      s_lo = lower((unsigned int)begin);
      s_hi = lower((unsigned int)end);
    }
  }
  __syncthreads();
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, stride = (long long)gridDim.x * blockDim.x;
  if (s_cnt <= capacity) {
    // (volatile loads: the sender rewrote these buffers this round, nothing cached from an earlier round may be used)
    for (long long i = s_lo + tid; i < s_hi; i += stride) {
      const unsigned int at = __ldcv(idx + i);
      const unsigned short w = __ldcv(reinterpret_cast<const unsigned short*>(val) + i);
      acc[at] += __half2float(*reinterpret_cast<const __half*>(&w));            // the indices of one message are distinct
    }
    if (bytes && tid == 0) atomicAdd(bytes, (unsigned long long)(s_hi - s_lo) * 6ull + 4ull);
  } else {
    for (long long i = begin + tid; i < end; i += stride) {
      const uint16_t w = __ldcv(dense16 + i);
      acc[i] += dense_f16 ? __half2float(*reinterpret_cast<const __half*>(&w)) : __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(&w));
    }
    if (bytes && tid == 0) atomicAdd(bytes, (unsigned long long)(end - begin) * 2ull + 4ull);
  }
}

static int done(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { set_error("%s launch failed (%lld)", what, (long long)e, 0); return -7; }
  return 0;
}
static int grid_for(long long n) { return (int)std::max<long long>(1, std::min<long long>((n + 255) / 256, 148 * 16)); }

}  // namespace ono

using namespace ono;

extern "C" int ono_sparse_threshold(const float* x, long long n, float r, unsigned long long seed, float* thr_out, ono_stream_t st) {
  if (!x || n <= 0 || !thr_out || r < 0.f || r > 1.f) { set_error("bad sparse_threshold args%s", "", 0, 0); return -1; }
  static bool attr_dev[64] = {false};     // a function attribute belongs to the device it was set on
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { set_error("bad device%s", "", 0, 0); return -6; }
  if (!attr_dev[dev]) {
    cudaFuncSetAttribute(sparse_threshold_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SPARSE_SAMPLE_MAX * 4);
    attr_dev[dev] = true;
  }
  sparse_threshold_kernel<<<1, 1024, SPARSE_SAMPLE_MAX * 4, (cudaStream_t)st>>>(x, n, r, seed, thr_out);
  return done("sparse_threshold");
}

extern "C" int ono_sparse_mask(float* residual, long long n, const float* thr, float* wire_f32, void* wire16, int wire16_f16,
                               unsigned long long* sent, ono_stream_t st) {
  if (!residual || (!wire_f32 && !wire16) || n <= 0) { set_error("bad sparse_mask args%s", "", 0, 0); return -1; }
  sparse_mask_kernel<<<grid_for(n), 256, 0, (cudaStream_t)st>>>(residual, n, thr, wire_f32, (uint16_t*)wire16, wire16_f16, sent);
  return done("sparse_mask");
}

extern "C" int ono_sparse_lift_range(float* acc, long long begin, long long end, const unsigned int* idx, const void* val_f16,
                                     const unsigned int* count, unsigned int capacity, const void* dense16, int dense_f16,
                                     unsigned long long* bytes, ono_stream_t st) {
  if (!acc || !idx || !val_f16 || !count || !dense16 || begin < 0 || end < begin || end >= (1ll << 32)) {
    set_error("bad sparse_lift_range args%s", "", 0, 0);
    return -1;
  }
  if (end == begin) return 0;
  sparse_lift_range_kernel<<<grid_for(end - begin), 256, 0, (cudaStream_t)st>>>(acc, begin, end, idx, (const __half*)val_f16, count, capacity,
                                                                            (const uint16_t*)dense16, dense_f16, bytes);
  return done("sparse_lift_range");
}

// scratch: at least ceil(n / 1024) unsigned ints. count receives the number of selected elements (it may exceed
// `capacity`, in which case only the first `capacity` pairs were written: the caller falls back to the dense wire,
// as the reference does when the sparse encoding is larger than the dense one).
extern "C" int ono_sparse_compact(float* x, long long n, const float* thr, unsigned int* scratch, unsigned int* idx, void* val_f16,
                                  unsigned int capacity, unsigned int* count, int zero_sent, ono_stream_t st) {
  if (!x || !thr || !scratch || !idx || !val_f16 || !count || n <= 0 || n >= (1ll << 32)) { set_error("bad sparse_compact args%s", "", 0, 0); return -1; }
  const int nblocks = (int)((n + CB - 1) / CB);
  compact_count_kernel<<<nblocks, 256, 0, (cudaStream_t)st>>>(x, n, thr, scratch);
  compact_scan_kernel<<<1, 1024, 0, (cudaStream_t)st>>>(scratch, nblocks, count);
  compact_write_kernel<<<nblocks, 256, 0, (cudaStream_t)st>>>(x, n, thr, scratch, idx, (__half*)val_f16, capacity, zero_sent);
  return done("sparse_compact");
}

extern "C" int ono_sparse_lift(float* acc, long long n, const unsigned int* idx, const void* val_f16, const unsigned int* count,
                               unsigned int capacity, ono_stream_t st) {
  if (!acc || !idx || !val_f16 || !count || n <= 0) { set_error("bad sparse_lift args%s", "", 0, 0); return -1; }
  sparse_lift_kernel<<<grid_for(capacity), 256, 0, (cudaStream_t)st>>>(acc, n, idx, (const __half*)val_f16, count, capacity);
  return done("sparse_lift");
}
