// Gradient synchronisation kernels over NVLink peer memory / NVSwitch multicast, each fused with
// the averaging and the optimizer step. See ono_kernels.h for the contract of each entry point and
// the reference code they replace (worker_ring.rs, server_cluster.rs, blocking/shard.rs, barrier.rs,
// non_blocking.rs, wild/shard.rs, stat_service.rs).
//
// Synchronisation between ranks uses epoch-stamped flag words in each rank's signal pad, written
// with st.release.sys and polled with ld.acquire.sys. Every poll loop is bounded by a wall-clock
// budget; on expiry the block records an error code and skips the rest of its work.
// No TMA is used here; peer data moves with plain vector loads/stores or multimem instructions.
#include <cooperative_groups.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include "ono_kernels.h"
#include "opt.cuh"
#include "ptx.cuh"

namespace ono {
void set_error(const char* fmt, const char* a, long long b, long long c);

// Barrier between block `blk` of every member rank. Thread t (< nranks) talks to rank t.
__device__ __forceinline__ bool rank_barrier(unsigned int* const* flags, int nranks, int rank, int blk,
                                             unsigned int members, uint32_t epoch, uint64_t budget) {
  __syncthreads();
  int ok = 1;
  const int t = threadIdx.x;
  if (t < nranks && ((members >> t) & 1u) && ((members >> rank) & 1u)) {
    __threadfence_system();
    st_release_sys(flags[t] + (size_t)blk * ONO_MAX_RANKS + rank, epoch);
    ok = wait_flag_ge(flags[rank] + (size_t)blk * ONO_MAX_RANKS + t, epoch, budget) ? 1 : 0;
  }
  return __syncthreads_and(ok) != 0;
}

// ------------------------------------------------------------------------------------------------
// Fused reduce-scatter + optimizer + all-gather (two-shot / one-shot / parameter server / NVLS)
// ------------------------------------------------------------------------------------------------
__device__ void sync_body(const OnoSync& a, const int rank, const int blk) {
  const OnoSyncLocal& L = a.loc[rank];
  __shared__ uint32_t s_epoch;
  if (threadIdx.x == 0) s_epoch = L.epoch[blk];
  __syncthreads();
  const uint32_t e0 = s_epoch;
  const unsigned int members = a.live_mask ? *a.live_mask : a.member_mask;
  const unsigned int workers = a.worker_mask & members;
  const uint64_t budget = a.timeout_ns;

  // Every member has finished producing its gradients (its kernel has started) before anyone reads.
  bool ok = rank_barrier(a.flags, a.nranks, rank, blk, members, e0 + 1, budget);
  if (!ok && threadIdx.x == 0 && L.status) atomicCAS(L.status, 0, ONO_ERR_TIMEOUT_PEER_FLAG);

  OptScal s{a.kind, a.lr, a.mu, a.b1, a.b2, a.eps, a.divide ? 1.0f / (float)a.n_workers : 1.0f, 0.0f};
  if (a.kind == 2 && L.adam_pows) s.adam_step = a.lr * sqrtf(1.0f - L.adam_pows[1]) / (1.0f - L.adam_pows[0]);

  double sq = 0.0;
  // 16-bit gradient windows whose ranges are multiples of 8 elements (the staged push lays shares out that way): one
  // 16-byte load per worker and thread brings eight gradients, and the fresh bf16 parameters leave as one 16-byte store
  // per thread (a full 512-byte line per warp over NVLink, P2P or multicast) instead of two 8-byte ones.
  // Not when f32 parameters leave for other GPUs: a thread's two float4 would go out as two stores that each fill half a
  // 32-byte sector, twice the packets over NVLink (measured: the tf32 MLP on four GPUs lost 13 %); that case keeps the
  // 8-byte path, whose stores are contiguous across the warp.
  bool wide8 = a.g_dtype != 0 && a.algo != 1;
  if (!L.fwd) {
    if (a.algo != 0) wide8 = wide8 && !a.p_mc_f32;
    else
      for (int q = 0; q < ONO_MAX_RANKS; ++q)
        if (q < a.nranks && q != rank && a.p_out_f32[q] && a.p_out_f32[q] != L.p_master) wide8 = false;
  }
  for (int ri = 0; ri < L.n_ranges && wide8; ++ri) wide8 = ((L.ranges[ri].begin | L.ranges[ri].end) & 7) == 0;
  if (ok && wide8) {
    const int f16 = a.g_dtype == 2;
    const long long stride = (long long)a.nblocks * blockDim.x;
    for (int ri = 0; ri < L.n_ranges; ++ri) {
      const long long b8 = L.ranges[ri].begin >> 3, e8 = L.ranges[ri].end >> 3;
      for (long long i8 = b8 + (long long)blk * blockDim.x + threadIdx.x; i8 < e8; i8 += stride) {
        float4 g0 = make_float4(0.f, 0.f, 0.f, 0.f), g1 = g0;
#pragma unroll
        for (int q = 0; q < ONO_MAX_RANKS; ++q)      // fixed rank order
          if (q < a.nranks && ((workers >> q) & 1u)) {
            const uint4 w = ld_relaxed_sys_v4_b32(reinterpret_cast<const uint4*>(a.g[q]) + i8);
            const float4 x0 = unpack16x4(make_uint2(w.x, w.y), f16), x1 = unpack16x4(make_uint2(w.z, w.w), f16);
            g0.x += x0.x; g0.y += x0.y; g0.z += x0.z; g0.w += x0.w;
            g1.x += x1.x; g1.y += x1.y; g1.z += x1.z; g1.w += x1.w;
          }
        const long long i4 = i8 << 1;
        if (L.fwd) {      // pre-reduction for the owner: the f32 sums travel, the owner's second launch does the rest
          *(reinterpret_cast<float4*>(L.fwd) + i4) = g0;
          *(reinterpret_cast<float4*>(L.fwd) + i4 + 1) = g1;
          continue;
        }
        const long long si = (i8 << 3) - L.state_off;
        float4 p0 = __ldcs(reinterpret_cast<const float4*>(L.p_master) + i4), p1 = __ldcs(reinterpret_cast<const float4*>(L.p_master) + i4 + 1);
        float4 m0 = make_float4(0.f, 0.f, 0.f, 0.f), m1 = m0, v0 = m0, v1 = m0;
        if (a.kind >= 1) { m0 = __ldcs(reinterpret_cast<const float4*>(L.m + si)); m1 = __ldcs(reinterpret_cast<const float4*>(L.m + si) + 1); }
        if (a.kind == 2) { v0 = __ldcs(reinterpret_cast<const float4*>(L.v + si)); v1 = __ldcs(reinterpret_cast<const float4*>(L.v + si) + 1); }
        p0 = opt_apply4(s, p0, g0, m0, v0);
        p1 = opt_apply4(s, p1, g1, m1, v1);
        if (L.sumsq) {
          const float q0 = g0.x * g0.x + g0.y * g0.y + g0.z * g0.z + g0.w * g0.w, q1 = g1.x * g1.x + g1.y * g1.y + g1.z * g1.z + g1.w * g1.w;
          sq += (double)(q0 + q1) * (double)(s.gs * s.gs);
        }
        if (a.kind >= 1) { __stcs(reinterpret_cast<float4*>(L.m + si), m0); __stcs(reinterpret_cast<float4*>(L.m + si) + 1, m1); }
        if (a.kind == 2) { __stcs(reinterpret_cast<float4*>(L.v + si), v0); __stcs(reinterpret_cast<float4*>(L.v + si) + 1, v1); }
        __stcs(reinterpret_cast<float4*>(L.p_master) + i4, p0);
        __stcs(reinterpret_cast<float4*>(L.p_master) + i4 + 1, p1);
        if (a.algo != 0) {
          if (a.p_mc_f32) {
            multimem_st_v4(reinterpret_cast<float4*>(a.p_mc_f32) + i4, p0);
            multimem_st_v4(reinterpret_cast<float4*>(a.p_mc_f32) + i4 + 1, p1);
          }
        } else {
#pragma unroll
          for (int q = 0; q < ONO_MAX_RANKS; ++q)
            if (q < a.nranks && a.p_out_f32[q] && a.p_out_f32[q] != L.p_master) {
              *(reinterpret_cast<float4*>(a.p_out_f32[q]) + i4) = p0;
              *(reinterpret_cast<float4*>(a.p_out_f32[q]) + i4 + 1) = p1;
            }
        }
        const uint2 lo = pack_bf16x4(p0), hi = pack_bf16x4(p1);
        const uint4 pb = make_uint4(lo.x, lo.y, hi.x, hi.y);
        if (a.algo != 0 && a.p_mc_bf16) {
          multimem_st_bf16x8(reinterpret_cast<uint4*>(a.p_mc_bf16) + i8, pb);
        } else {
#pragma unroll
          for (int q = 0; q < ONO_MAX_RANKS; ++q)
            if (q < a.nranks && a.p_out_bf16[q]) *(reinterpret_cast<uint4*>(a.p_out_bf16[q]) + i8) = pb;
        }
        if (a.zero_grad && ((workers >> rank) & 1u))
          *(reinterpret_cast<uint4*>(const_cast<float*>(a.g[rank])) + i8) = make_uint4(0u, 0u, 0u, 0u);
      }
    }
  } else if (ok && L.fwd) {
    if (threadIdx.x == 0 && L.status) atomicCAS(L.status, 0, ONO_ERR_BAD_ARG);   // pre-reduction needs the 16-byte path
  } else if (ok) {
    // Two float4 per thread and iteration, all loads issued before the first use, so that enough
    // bytes are in flight per SM to cover HBM / NVLink latency.
    constexpr int U = 2;
    const long long stride = (long long)a.nblocks * blockDim.x * U;
    for (int ri = 0; ri < L.n_ranges; ++ri) {
      const long long b4 = L.ranges[ri].begin >> 2;
      const long long e4 = (L.ranges[ri].end + 3) >> 2;
      for (long long base = b4 + (long long)blk * blockDim.x * U + threadIdx.x; base < e4; base += stride) {
        float4 g[U], p[U], m[U], v[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const long long i4 = base + (long long)u * blockDim.x;
          g[u] = p[u] = m[u] = v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
          if (i4 >= e4) continue;
          if (a.g_dtype != 0) {
            // 16-bit gradient wire (bf16 or f16): four values per 8-byte load, summed in f32 in rank order
            if (a.algo == 1) {
              g[u] = unpack16x4(multimem_ld_reduce_add_16x4(reinterpret_cast<const uint2*>(a.g_mc) + i4, a.g_dtype == 2),
                                a.g_dtype == 2);
            } else {
#pragma unroll
              for (int q = 0; q < ONO_MAX_RANKS; ++q)
                if (q < a.nranks && ((workers >> q) & 1u)) {
                  const float4 x = unpack16x4(ld_relaxed_sys_v2(reinterpret_cast<const uint2*>(a.g[q]) + i4), a.g_dtype == 2);
                  g[u].x += x.x; g[u].y += x.y; g[u].z += x.z; g[u].w += x.w;
                }
            }
          } else if (a.algo == 1) {
            g[u] = multimem_ld_reduce_add_v4(reinterpret_cast<const float4*>(a.g_mc) + i4);
          } else {
#pragma unroll
            for (int q = 0; q < ONO_MAX_RANKS; ++q)  // fixed rank order: run-to-run deterministic
              if (q < a.nranks && ((workers >> q) & 1u)) {
                const float4 x = ld_global_v4_volatile(reinterpret_cast<const float4*>(a.g[q]) + i4);
                g[u].x += x.x; g[u].y += x.y; g[u].z += x.z; g[u].w += x.w;
              }
          }
          const long long si = (i4 << 2) - L.state_off;
          // parameters and optimizer state are touched once per step: streaming (evict-first) accesses keep them from
          // displacing the bf16 shadow and the activations the next forward reads
          p[u] = __ldcs(reinterpret_cast<const float4*>(L.p_master) + i4);
          if (a.kind >= 1) m[u] = __ldcs(reinterpret_cast<const float4*>(L.m + si));
          if (a.kind == 2) v[u] = __ldcs(reinterpret_cast<const float4*>(L.v + si));
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const long long i4 = base + (long long)u * blockDim.x;
          if (i4 >= e4) continue;
          const long long si = (i4 << 2) - L.state_off;
          float4 pp = p[u];
          pp.x = opt_apply(s, pp.x, g[u].x, m[u].x, v[u].x);
          pp.y = opt_apply(s, pp.y, g[u].y, m[u].y, v[u].y);
          pp.z = opt_apply(s, pp.z, g[u].z, m[u].z, v[u].z);
          pp.w = opt_apply(s, pp.w, g[u].w, m[u].w, v[u].w);
          if (L.sumsq) {
            const float gx = g[u].x * s.gs, gy = g[u].y * s.gs, gz = g[u].z * s.gs, gw = g[u].w * s.gs;
            sq += (double)(gx * gx + gy * gy) + (double)(gz * gz + gw * gw);
          }
          if (a.kind >= 1) __stcs(reinterpret_cast<float4*>(L.m + si), m[u]);
          if (a.kind == 2) __stcs(reinterpret_cast<float4*>(L.v + si), v[u]);
          __stcs(reinterpret_cast<float4*>(L.p_master) + i4, pp);
          if (a.algo != 0) {   // 1: in-switch reduction and multicast stores; 2: multicast stores only
            if (a.p_mc_f32) multimem_st_v4(reinterpret_cast<float4*>(a.p_mc_f32) + i4, pp);
          } else {
#pragma unroll
            for (int q = 0; q < ONO_MAX_RANKS; ++q)
              if (q < a.nranks && a.p_out_f32[q] && a.p_out_f32[q] != L.p_master)
                *(reinterpret_cast<float4*>(a.p_out_f32[q]) + i4) = pp;
          }
          const uint2 pb = pack_bf16x4(pp);
          if (a.algo != 0 && a.p_mc_bf16) {
            multimem_st_bf16x4(reinterpret_cast<uint2*>(a.p_mc_bf16) + i4, pb);
          } else {
#pragma unroll
            for (int q = 0; q < ONO_MAX_RANKS; ++q)
              if (q < a.nranks && a.p_out_bf16[q])
                *(reinterpret_cast<uint2*>(a.p_out_bf16[q]) + i4) = pb;
          }
          if (a.zero_grad && ((workers >> rank) & 1u)) {
            if (a.g_dtype != 0) *(reinterpret_cast<uint2*>(const_cast<float*>(a.g[rank])) + i4) = make_uint2(0u, 0u);
            else *(reinterpret_cast<float4*>(const_cast<float*>(a.g[rank])) + i4) = make_float4(0.f, 0.f, 0.f, 0.f);
          }
        }
      }
    }
  }
  if (L.sumsq) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
    if ((threadIdx.x & 31) == 0 && sq != 0.0) atomicAdd(L.sumsq, sq);
  }
  // Nobody leaves before every member has stopped reading gradients and writing parameters.
  // After a failed entry barrier the exit barrier only gets a token budget: the peer is already known absent.
  const bool ok2 = rank_barrier(a.flags, a.nranks, rank, blk, members, e0 + 2, ok ? budget : 1000000ull);
  if (!ok2 && ok && threadIdx.x == 0 && L.status) atomicCAS(L.status, 0, ONO_ERR_TIMEOUT_BARRIER);
  if (threadIdx.x == 0) L.epoch[blk] = e0 + 2;
}

__global__ void __launch_bounds__(512, 2) sync_kernel(const OnoSync a) { sync_body(a, a.rank, blockIdx.x); }
__global__ void __launch_bounds__(512, 2) sync_kernel_emulated(const OnoSync a) { sync_body(a, blockIdx.y, blockIdx.x); }

// ------------------------------------------------------------------------------------------------
// Asynchronous parameter server: worker-driven remote read-modify-write of the owners' shards.
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(512) ps_async_kernel(const OnoPsAsync a) {
  const int blk = blockIdx.x;
  OptScal s{a.kind, a.lr, a.mu, a.b1, a.b2, a.eps, a.divide ? 1.0f / (float)a.n_workers : 1.0f, 0.0f};
  if (a.kind == 2 && a.adam_pows) s.adam_step = a.lr * sqrtf(1.0f - a.adam_pows[1]) / (1.0f - a.adam_pows[0]);
  __shared__ int s_ok;
  for (int owner = 0; owner < a.nranks; ++owner) {
    for (int ri = 0; ri < a.n_ranges[owner]; ++ri) {
      const OnoRange rg = a.ranges[owner][ri];
      const long long b4 = rg.begin >> 2, e4 = (rg.end + 3) >> 2;
      const long long per = (e4 - b4 + a.nblocks - 1) / a.nblocks;
      const long long lo = b4 + per * blk, hi = min(e4, lo + per);
      if (lo >= hi) continue;  // uniform per block
      unsigned int* lock = a.locks[owner] ? a.locks[owner] + (size_t)ri * a.nblocks + blk : nullptr;
      if (lock) {
        if (threadIdx.x == 0) {
          int got = 0;
          const uint64_t t0 = globaltimer_ns();
          while (true) {
            if (atomicCAS_system(lock, 0u, 1u) == 0u) { got = 1; break; }
            if (globaltimer_ns() - t0 > a.timeout_ns) break;
            __nanosleep(200);
          }
          __threadfence_system();
          s_ok = got;
        }
        __syncthreads();
        if (!s_ok) {
          if (threadIdx.x == 0 && a.status) atomicCAS(a.status, 0, ONO_ERR_TIMEOUT_BARRIER);
          __syncthreads();
          continue;
        }
      }
      float* master = a.master[owner];
      for (long long i4 = lo + threadIdx.x; i4 < hi; i4 += blockDim.x) {
        const float4 g = *(reinterpret_cast<const float4*>(a.g) + i4);
        const long long si = (i4 << 2) - a.state_off[owner];
        float4 p = ld_global_v4_volatile(reinterpret_cast<const float4*>(master) + i4);
        float4 m = make_float4(0.f, 0.f, 0.f, 0.f), v = m;
        if (a.kind >= 1) m = ld_global_v4_volatile(reinterpret_cast<const float4*>(a.m[owner] + si));
        if (a.kind == 2) v = ld_global_v4_volatile(reinterpret_cast<const float4*>(a.v[owner] + si));
        p.x = opt_apply(s, p.x, g.x, m.x, v.x);
        p.y = opt_apply(s, p.y, g.y, m.y, v.y);
        p.z = opt_apply(s, p.z, g.z, m.z, v.z);
        p.w = opt_apply(s, p.w, g.w, m.w, v.w);
        *(reinterpret_cast<float4*>(master) + i4) = p;
        if (a.kind >= 1) *reinterpret_cast<float4*>(a.m[owner] + si) = m;
        if (a.kind == 2) *reinterpret_cast<float4*>(a.v[owner] + si) = v;
        if (a.p_local_f32 && a.p_local_f32 != master) *(reinterpret_cast<float4*>(a.p_local_f32) + i4) = p;
        if (a.p_local_bf16) *(reinterpret_cast<uint2*>(a.p_local_bf16) + i4) = pack_bf16x4(p);
      }
      if (lock) {
        __syncthreads();
        if (threadIdx.x == 0) {
          __threadfence_system();
          st_release_sys(lock, 0u);
        }
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------
// Ring all-reduce, pull formulation: at every step a rank reads one chunk from its predecessor's
// window. Block b of each rank forms an independent pipeline with block b of its neighbours.
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void chunk_bounds4(long long n4, int nranks, int c, long long& lo, long long& hi) {
  // near-equal split: the first (n4 % nranks) chunks get one extra element (middlewares/mod.rs:15-59)
  const long long base = n4 / nranks, rem = n4 % nranks;
  lo = base * c + (c < rem ? c : rem);
  hi = lo + base + (c < rem ? 1 : 0);
}

constexpr int RING_UNROLL = 4;

__device__ void ring_body(const OnoRing& a, const int blk) {
  const int N = a.nranks, r = a.rank;
  const int prev = (r + N - 1) % N, next = (r + 1) % N;
  __shared__ uint32_t s_epoch;
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_epoch = a.epoch[blk];
  __syncthreads();
  const uint32_t base = s_epoch;
  uint32_t tick = base;  // value I have published to `next` so far
  const long long n4 = (a.n + 3) >> 2;
  float4* mine = reinterpret_cast<float4*>(a.acc[r]);
  const float4* theirs = reinterpret_cast<const float4*>(a.acc[prev]);
  unsigned int* fwd_flag_at_next = a.flags[next] + blk;             // my progress, seen by next
  const unsigned int* fwd_flag_mine = a.flags[r] + blk;             // prev's progress, seen by me
  unsigned int* back_flag_at_prev = a.flags[prev] + a.nblocks + blk;  // "I finished reading you"
  const unsigned int* back_flag_mine = a.flags[r] + a.nblocks + blk;
  bool ok = true;

  auto publish = [&]() {
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence_system();
      st_release_sys(fwd_flag_at_next, ++tick);
    } else {
      ++tick;
    }
  };
  auto wait_prev = [&](uint32_t want) {
    if (threadIdx.x == 0) s_ok = wait_flag_ge(fwd_flag_mine, want, a.timeout_ns) ? 1 : 0;
    __syncthreads();
    const bool good = s_ok != 0;
    __syncthreads();
    return good;
  };
  auto slice = [&](int c, long long& lo, long long& hi) {
    long long clo, chi;
    chunk_bounds4(n4, N, c, clo, chi);
    const long long per = (chi - clo + a.nblocks - 1) / a.nblocks;
    lo = clo + per * blk;
    hi = min(chi, lo + per);
  };

  // step 0: acc <- g
  {
    const float4* g4 = reinterpret_cast<const float4*>(a.g);
    for (int c = 0; c < N; ++c) {
      long long lo, hi;
      slice(c, lo, hi);
      for (long long i = lo + threadIdx.x; i < hi; i += blockDim.x) mine[i] = g4[i];
    }
    publish();  // base+1
  }
  // reduce-scatter: N-1 steps
  for (int s = 0; s < N - 1 && ok; ++s) {
    const int c = ((r - s - 1) % N + N) % N;
    ok = wait_prev(base + 1 + s);
    if (!ok) break;
    long long lo, hi;
    slice(c, lo, hi);
    // four peer loads in flight per thread before the first use: one block per SM has to keep its share of the link busy
    for (long long i0 = lo + threadIdx.x; i0 < hi; i0 += (long long)blockDim.x * RING_UNROLL) {
      float4 x[RING_UNROLL];
#pragma unroll
      for (int u = 0; u < RING_UNROLL; ++u) {
        const long long i = i0 + (long long)u * blockDim.x;
        if (i < hi) x[u] = ld_global_v4_volatile(theirs + i);
      }
#pragma unroll
      for (int u = 0; u < RING_UNROLL; ++u) {
        const long long i = i0 + (long long)u * blockDim.x;
        if (i < hi) {
          float4 y = mine[i];
          y.x += x[u].x; y.y += x[u].y; y.z += x[u].z; y.w += x[u].w;
          mine[i] = y;
        }
      }
    }
    if (s < N - 2) publish();
  }
  // owned chunk: average + optimizer; the payload that circulates from here on is the new params
  OptScal sc{a.kind, a.lr, a.mu, a.b1, a.b2, a.eps, 1.0f / (float)N, 0.0f};
  if (a.kind == 2 && a.adam_pows) sc.adam_step = a.lr * sqrtf(1.0f - a.adam_pows[1]) / (1.0f - a.adam_pows[0]);
  __nv_bfloat16* pb = reinterpret_cast<__nv_bfloat16*>(a.p_bf16);
  if (ok) {
    const int c = (r + 1) % N;
    long long lo, hi;
    slice(c, lo, hi);
    for (long long i = lo + threadIdx.x; i < hi; i += blockDim.x) {
      const float4 g = mine[i];
      float4 p = *(reinterpret_cast<float4*>(a.p) + i);
      float4 m = make_float4(0.f, 0.f, 0.f, 0.f), v = m;
      if (a.kind >= 1) m = *(reinterpret_cast<float4*>(a.m) + i);
      if (a.kind == 2) v = *(reinterpret_cast<float4*>(a.v) + i);
      p.x = opt_apply(sc, p.x, g.x, m.x, v.x);
      p.y = opt_apply(sc, p.y, g.y, m.y, v.y);
      p.z = opt_apply(sc, p.z, g.z, m.z, v.z);
      p.w = opt_apply(sc, p.w, g.w, m.w, v.w);
      if (a.kind >= 1) *(reinterpret_cast<float4*>(a.m) + i) = m;
      if (a.kind == 2) *(reinterpret_cast<float4*>(a.v) + i) = v;
      *(reinterpret_cast<float4*>(a.p) + i) = p;
      if (pb) *(reinterpret_cast<uint2*>(pb) + i) = pack_bf16x4(p);
      mine[i] = p;
    }
    publish();  // base+N  (N-2 publishes in the loop + the copy + this one)
  }
  // all-gather of the updated parameters: N-1 steps
  for (int s = 0; s < N - 1 && ok; ++s) {
    const int c = ((r - s) % N + N) % N;
    ok = wait_prev(base + N + s);
    if (!ok) break;
    long long lo, hi;
    slice(c, lo, hi);
    for (long long i0 = lo + threadIdx.x; i0 < hi; i0 += (long long)blockDim.x * RING_UNROLL) {
      float4 x[RING_UNROLL];
#pragma unroll
      for (int u = 0; u < RING_UNROLL; ++u) {
        const long long i = i0 + (long long)u * blockDim.x;
        if (i < hi) x[u] = ld_global_v4_volatile(theirs + i);
      }
#pragma unroll
      for (int u = 0; u < RING_UNROLL; ++u) {
        const long long i = i0 + (long long)u * blockDim.x;
        if (i < hi) {
          mine[i] = x[u];
          *(reinterpret_cast<float4*>(a.p) + i) = x[u];
          if (pb) *(reinterpret_cast<uint2*>(pb) + i) = pack_bf16x4(x[u]);
        }
      }
    }
    if (s < N - 2) publish();
  }
  // Tell prev that its window is no longer read, and wait for the same from next, so that the next
  // call may overwrite the windows.
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    st_release_sys(back_flag_at_prev, base + 2u * N);
    const bool fin = wait_flag_ge(back_flag_mine, base + 2u * N, ok ? a.timeout_ns : 1000000ull);
    if ((!ok || !fin) && a.status) atomicCAS(a.status, 0, ONO_ERR_TIMEOUT_PEER_FLAG);
    a.epoch[blk] = base + 2u * N;
  }
}

__global__ void __launch_bounds__(512) ring_kernel(const OnoRing a) { ring_body(a, blockIdx.x); }

// Every rank of the ring as one cooperative launch on one GPU (grid.y = rank): the blocks really wait on one another
// through the same flags, only the wires are missing. For single-GPU tests of the ring protocol.
__global__ void __launch_bounds__(512) ring_kernel_emulated(const OnoRingEmu e) {
  OnoRing a;
  const int r = blockIdx.y;
  a.nranks = e.nranks; a.rank = r; a.nblocks = e.nblocks; a.n = e.n;
  a.g = e.g[r];
  for (int q = 0; q < ONO_MAX_RANKS; ++q) { a.acc[q] = e.acc[q]; a.flags[q] = e.flags[q]; }
  a.epoch = e.epoch[r];
  a.p = e.p[r]; a.m = e.m[r]; a.v = e.v[r]; a.adam_pows = e.adam_pows; a.p_bf16 = e.p_bf16[r];
  a.kind = e.kind; a.lr = e.lr; a.mu = e.mu; a.b1 = e.b1; a.b2 = e.b2; a.eps = e.eps;
  a.status = e.status; a.timeout_ns = e.timeout_ns;
  ring_body(a, blockIdx.x);
}

// ------------------------------------------------------------------------------------------------
// Ping-pong latency probe
// ------------------------------------------------------------------------------------------------
__global__ void pingpong_kernel(int role, unsigned int* my_flag, unsigned int* peer_flag, int rounds,
                                unsigned int base, unsigned long long* rtt, int* status) {
  for (int i = 0; i < rounds; ++i) {
    const uint32_t e = base + 1 + i;
    if (role == 0) {
      const uint64_t t0 = globaltimer_ns();
      st_release_sys(peer_flag, e);
      if (!wait_flag_ge(my_flag, e, 1000000000ull)) {
        if (status) atomicCAS(status, 0, ONO_ERR_TIMEOUT_PEER_FLAG);
        return;
      }
      if (rtt) rtt[i] = globaltimer_ns() - t0;
    } else {
      if (!wait_flag_ge(my_flag, e, 1000000000ull)) {
        if (status) atomicCAS(status, 0, ONO_ERR_TIMEOUT_PEER_FLAG);
        return;
      }
      st_release_sys(peer_flag, e);
    }
  }
}

static int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("%s launch failed: %lld", what, (long long)e, 0);
    return -7;
  }
  return 0;
}

static int validate_sync(const OnoSync* s) {
  if (!s || s->nranks < 1 || s->nranks > ONO_MAX_RANKS || s->nblocks < 1 || s->n <= 0) {
    set_error("bad sync args%s", "", 0, 0);
    return -1;
  }
  if (s->algo == 1 && !s->g_mc) { set_error("NVLS needs multicast addresses%s", "", 0, 0); return -1; }
  if (s->g_dtype < 0 || s->g_dtype > 2) { set_error("g_dtype must be 0 (f32), 1 (bf16) or 2 (f16)%s", "", 0, 0); return -1; }
  for (int r = 0; r < s->nranks; ++r) {
    const OnoSyncLocal& L = s->loc[r];
    if (!L.fwd) continue;
    bool ok = s->g_dtype != 0 && s->algo != 1 && (((uintptr_t)L.fwd) & 15) == 0;
    for (int i = 0; i < L.n_ranges && ok; ++i) ok = ((L.ranges[i].begin | L.ranges[i].end) & 7) == 0;
    if (!ok) { set_error("pre-reduction needs 16-bit windows, peer loads and ranges cut at multiples of 8%s", "", 0, 0); return -1; }
  }
  return 0;
}

}  // namespace ono

using namespace ono;

extern "C" int ono_sync_step(const OnoSync* s, ono_stream_t st) {
  if (int rc = validate_sync(s)) return rc;
  if (s->rank < 0 || s->rank >= s->nranks) { set_error("bad rank%s", "", 0, 0); return -1; }
  sync_kernel<<<s->nblocks, 512, 0, (cudaStream_t)st>>>(*s);
  return check_launch("sync_step");
}

extern "C" int ono_sync_step_emulated(const OnoSync* s, ono_stream_t st) {
  if (int rc = validate_sync(s)) return rc;
  if (s->algo != 0) { set_error("emulation supports algo 0 only%s", "", 0, 0); return -1; }
  // All rank-blocks wait on one another, so they must be co-resident: cooperative launch, which
  // fails cleanly if the grid does not fit.
  OnoSync copy = *s;
  void* args[] = {&copy};
  dim3 grid(s->nblocks, s->nranks);
  cudaError_t e = cudaLaunchCooperativeKernel((void*)sync_kernel_emulated, grid, dim3(512), args, 0, (cudaStream_t)st);
  if (e != cudaSuccess) {
    set_error("cooperative launch failed: %s", cudaGetErrorString(e), 0, 0);
    return -7;
  }
  return 0;
}

extern "C" int ono_ps_async_step(const OnoPsAsync* s, ono_stream_t st) {
  if (!s || s->nranks < 1 || s->nranks > ONO_MAX_RANKS || s->nblocks < 1 || !s->g) {
    set_error("bad ps_async args%s", "", 0, 0);
    return -1;
  }
  ps_async_kernel<<<s->nblocks, 512, 0, (cudaStream_t)st>>>(*s);
  return check_launch("ps_async_step");
}

// ------------------------------------------------------------------------------------------------
// Staged reduce-scatter (see OnoStagePull). One thread per block drives a ring of shared-memory slots:
// bulk load peer -> slot (completion on an mbarrier), bulk store slot -> local staging buffer.
// ------------------------------------------------------------------------------------------------
namespace ono {
constexpr uint32_t PULL_CHUNK = 32768;   // bytes per bulk copy
constexpr int PULL_SLOTS = 6;            // 192 KB of shared memory in flight per block

__global__ void __launch_bounds__(32) stage_pull_kernel(const OnoStagePull a) {
  extern __shared__ uint8_t pull_raw[];
  uint8_t* slots = pull_raw + ((128u - (smem_u32(pull_raw) & 127u)) & 127u);
  __shared__ __align__(8) uint64_t bar[PULL_SLOTS];
  __shared__ int abort_flag;
  if (threadIdx.x != 0) return;
  for (int s = 0; s < PULL_SLOTS; ++s) mbar_init(&bar[s], 1);
  abort_flag = 0;
  mbar_fence_init();
  const uint32_t want = *a.step;
  // every source rank must have announced this bucket for this step before its window is read
  for (int q = 0; q < a.nranks; ++q) {
    if (!a.src[q] || q == a.rank) continue;
    if (!wait_flag_ge(a.ready + q * ONO_STAGE_BUCKETS + a.bucket, want, a.timeout_ns)) {
      if (a.status) atomicCAS(a.status, 0, ONO_ERR_TIMEOUT_PEER_FLAG);
      return;
    }
  }
  asm volatile("fence.proxy.async;" ::: "memory");   // the copies below run in the async proxy, after the acquires above
  // my work items: chunk g of the enumeration (source, range, offset) with g % nblocks == blockIdx.x
  struct Item { const uint8_t* src; uint8_t* dst; uint32_t bytes; };
  auto item = [&](long long want_idx, Item& out) -> bool {   // want_idx-th item of this block, in enumeration order
    long long g = 0, mine = 0;
    for (int q = 0; q < a.nranks; ++q) {
      if (!a.src[q] || q == a.rank) continue;
      for (int r = 0; r < a.n_ranges; ++r) {
        const long long b0 = a.ranges[r].begin * 4ll, b1 = ((a.ranges[r].end + 3) / 4 * 4) * 4ll;
        const long long nch = (b1 - b0 + PULL_CHUNK - 1) / PULL_CHUNK;
        // chunks of this (q, r) that belong to this block: g + c with (g + c) % nblocks == blk
        long long first = ((long long)blockIdx.x - g % a.nblocks + a.nblocks) % a.nblocks;
        const long long cnt = first < nch ? (nch - first + a.nblocks - 1) / a.nblocks : 0;
        if (want_idx < mine + cnt) {
          const long long c = first + (want_idx - mine) * a.nblocks;
          const long long off = b0 + c * PULL_CHUNK;
          out.src = reinterpret_cast<const uint8_t*>(a.src[q]) + off;
          out.dst = reinterpret_cast<uint8_t*>(a.dst[q]) + off;
          out.bytes = (uint32_t)min((long long)PULL_CHUNK, b1 - off);
          return true;
        }
        mine += cnt;
        g += nch;
      }
    }
    return false;
  };
  volatile int* abortp = &abort_flag;
  Item it;
  long long issued = 0;
  for (; issued < PULL_SLOTS && item(issued, it); ++issued) {
    mbar_expect_tx(&bar[issued], it.bytes);
    bulk_load_1d(slots + (size_t)issued * PULL_CHUNK, it.src, it.bytes, &bar[issued]);
  }
  // A slot is refilled PULL_LAG items after its store was issued, so the wait for that store to have read the slot
  // almost never blocks and PULL_SLOTS - PULL_LAG loads stay in flight.
  constexpr int PULL_LAG = 2;
  for (long long j = 0; item(j, it); ++j) {
    const int s = (int)(j % PULL_SLOTS);
    if (!mbar_wait_bounded(&bar[s], (uint32_t)((j / PULL_SLOTS) & 1), abortp, a.timeout_ns)) {
      if (a.status) atomicCAS(a.status, 0, ONO_ERR_TIMEOUT_FULL);
      break;
    }
    bulk_store_1d(it.dst, slots + (size_t)s * PULL_CHUNK, it.bytes);
    tma_store_commit();
    const long long jr = j - PULL_LAG;              // the store of item jr has had PULL_LAG items to drain
    Item nx;
    if (jr >= 0 && item(jr + PULL_SLOTS, nx)) {
      tma_store_wait_read<PULL_LAG>();
      const int sr = (int)(jr % PULL_SLOTS);
      mbar_expect_tx(&bar[sr], nx.bytes);
      bulk_load_1d(slots + (size_t)sr * PULL_CHUNK, nx.src, nx.bytes, &bar[sr]);
    }
  }
  tma_store_wait_all<0>();   // staged data is in memory before the kernel ends
}

struct FlagPtrs { unsigned int* p[ONO_MAX_RANKS]; };
__global__ void stage_signal_kernel2(FlagPtrs f, int nranks, int rank, int bucket, const unsigned int* step) {
  const int q = threadIdx.x;
  if (q < nranks && f.p[q]) {
    __threadfence_system();
    st_release_sys(f.p[q] + rank * ONO_STAGE_BUCKETS + bucket, *step);
  }
}
__global__ void stage_tick_kernel(unsigned int* step) { *step += 1u; }
}  // namespace ono

extern "C" int ono_stage_pull(const OnoStagePull* s, ono_stream_t st) {
  if (!s || s->nranks < 1 || s->nranks > ONO_MAX_RANKS || s->nblocks < 1 || s->bucket < 0 || s->bucket >= ONO_STAGE_BUCKETS ||
      !s->ready || !s->step || s->n_ranges < 0 || s->n_ranges > ONO_MAX_RANGES) {
    set_error("bad stage_pull args%s", "", 0, 0);
    return -1;
  }
  for (int r = 0; r < s->n_ranges; ++r)
    if (s->ranges[r].begin % 4) { set_error("stage_pull ranges must begin at multiples of 4 elements%s", "", 0, 0); return -1; }
  static bool attr_dev[64] = {false};     // a function attribute belongs to the device it was set on
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { set_error("bad device%s", "", 0, 0); return -6; }
  const int smem = PULL_SLOTS * PULL_CHUNK + 128;
  if (!attr_dev[dev]) {
    cudaError_t e = cudaFuncSetAttribute(stage_pull_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) { set_error("cudaFuncSetAttribute(stage_pull): %s", cudaGetErrorString(e), 0, 0); return -6; }
    attr_dev[dev] = true;
  }
  stage_pull_kernel<<<s->nblocks, 32, smem, (cudaStream_t)st>>>(*s);
  return check_launch("stage_pull");
}

extern "C" int ono_stage_signal(unsigned int* const* flags, int nranks, int rank, int bucket, const unsigned int* step,
                                ono_stream_t st) {
  if (!flags || nranks < 1 || nranks > ONO_MAX_RANKS || !step) { set_error("bad stage_signal args%s", "", 0, 0); return -1; }
  FlagPtrs f;
  for (int q = 0; q < ONO_MAX_RANKS; ++q) f.p[q] = q < nranks ? flags[q] : nullptr;
  stage_signal_kernel2<<<1, 32, 0, (cudaStream_t)st>>>(f, nranks, rank, bucket, step);
  return check_launch("stage_signal");
}

extern "C" int ono_stage_tick(unsigned int* step, ono_stream_t st) {
  if (!step) return -1;
  stage_tick_kernel<<<1, 1, 0, (cudaStream_t)st>>>(step);
  return check_launch("stage_tick");
}

extern "C" int ono_ring_allreduce(const OnoRing* r, ono_stream_t st) {
  if (!r || r->nranks < 1 || r->nranks > ONO_MAX_RANKS || r->nblocks < 1 || r->n <= 0) {
    set_error("bad ring args%s", "", 0, 0);
    return -1;
  }
  ring_kernel<<<r->nblocks, 512, 0, (cudaStream_t)st>>>(*r);
  return check_launch("ring_allreduce");
}

extern "C" int ono_ring_allreduce_emulated(const OnoRingEmu* r, ono_stream_t st) {
  if (!r || r->nranks < 1 || r->nranks > ONO_MAX_RANKS || r->nblocks < 1 || r->n <= 0) {
    set_error("bad ring args%s", "", 0, 0);
    return -1;
  }
  OnoRingEmu copy = *r;
  void* args[] = {&copy};
  cudaError_t e = cudaLaunchCooperativeKernel((void*)ring_kernel_emulated, dim3(r->nblocks, r->nranks), dim3(512), args, 0, (cudaStream_t)st);
  if (e != cudaSuccess) { set_error("cooperative launch failed: %s", cudaGetErrorString(e), 0, 0); return -7; }
  return 0;
}

extern "C" int ono_pingpong(int role, unsigned int* my_flag, unsigned int* peer_flag, int rounds, unsigned int base,
                            unsigned long long* rtt, int* status, ono_stream_t st) {
  pingpong_kernel<<<1, 1, 0, (cudaStream_t)st>>>(role, my_flag, peer_flag, rounds, base, rtt, status);
  return check_launch("pingpong");
}

// Size of each ABI structure, so that a binding can check its own layout at load time.
extern "C" int ono_sizeof(int which) {
  switch (which) {
    case 0: return (int)sizeof(OnoGemm);
    case 1: return (int)sizeof(OnoLoss);
    case 2: return (int)sizeof(OnoOptim);
    case 3: return (int)sizeof(OnoRows);
    case 4: return (int)sizeof(OnoSync);
    case 5: return (int)sizeof(OnoPsAsync);
    case 6: return (int)sizeof(OnoRing);
    case 7: return (int)sizeof(OnoStagePull);
    case 8: return (int)sizeof(OnoRingEmu);
    default: return -1;
  }
}

// ------------------------------------------------------------------------------------------------
// Allocation-free single-GPU form of the fused step (see ono_noalloc.h).
// ------------------------------------------------------------------------------------------------
#include "ono_noalloc.h"

namespace ono {
// Flag pad [ONO_NOALLOC_MAX_BLOCKS][ONO_MAX_RANKS] followed by the epoch words [ONO_NOALLOC_MAX_BLOCKS].
// Zero at load time; afterwards the stamps only grow.
static __device__ __align__(256) unsigned int g_noalloc_scratch[ONO_NOALLOC_SCRATCH_BYTES / 4];

// Device address of the scratch array, looked up once per device. In host code the array's name is
// only a handle for the runtime, never an address a kernel may be given.
static unsigned int* noalloc_scratch_ptr() {
  constexpr int kMaxDevices = 64;
  static unsigned int* cache[kMaxDevices] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    set_error("no current CUDA device%s", "", 0, 0);
    return nullptr;
  }
  if (!cache[dev]) {
    void* ptr = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
    if (e != cudaSuccess || !ptr) {
      set_error("cudaGetSymbolAddress failed: %s", cudaGetErrorString(e), 0, 0);
      return nullptr;
    }
    cache[dev] = static_cast<unsigned int*>(ptr);
  }
  return cache[dev];
}
}  // namespace ono

extern "C" int ono_sync_step_noalloc(const OnoNoAllocStep* s, ono_stream_t st) {
  if (!s || !s->p || !s->g || s->n <= 0) { set_error("bad no-alloc step args%s", "", 0, 0); return -1; }
  if (s->kind < 0 || s->kind > 2) { set_error("unknown optimizer kind%s", "", 0, 0); return -1; }
  if (s->kind >= 1 && !s->m) { set_error("optimizer state m missing%s", "", 0, 0); return -1; }
  if (s->kind == 2 && (!s->v || !s->adam_pows)) { set_error("adam state missing%s", "", 0, 0); return -1; }
  if (((uintptr_t)s->p | (uintptr_t)s->g | (uintptr_t)s->m | (uintptr_t)s->v) & 15) {
    set_error("buffers must be 16-byte aligned%s", "", 0, 0);
    return -1;
  }
  if (((uintptr_t)s->p_bf16 & 7) || ((uintptr_t)s->sumsq & 7) || ((uintptr_t)s->adam_pows & 3) || ((uintptr_t)s->status & 3)) {
    set_error("p_bf16 and sumsq must be 8-byte aligned, adam_pows and status 4-byte aligned%s", "", 0, 0);
    return -1;
  }
  if (s->n % 4 != 0) { set_error("n must be padded to a multiple of 4 elements%s", "", 0, 0); return -1; }
  if (s->nblocks > ONO_NOALLOC_MAX_BLOCKS) {
    set_error("nblocks %s%lld exceeds the built-in scratch (max %lld blocks)", "", (long long)s->nblocks,
              (long long)ONO_NOALLOC_MAX_BLOCKS);
    return -2;
  }
  unsigned int* scratch = noalloc_scratch_ptr();
  if (!scratch) return -3;
  int nblocks = s->nblocks;
  if (nblocks <= 0) {
    const long long n4 = (s->n + 3) >> 2;
    long long want = (n4 + 1023) / 1024;
    const long long cap = 2LL * ono_num_sms();
    if (want > cap) want = cap;
    if (want > ONO_NOALLOC_MAX_BLOCKS) want = ONO_NOALLOC_MAX_BLOCKS;
    nblocks = want < 1 ? 1 : (int)want;
  }
  OnoSync a;
  memset(&a, 0, sizeof(a));
  a.nranks = 1;
  a.rank = 0;
  a.algo = 0;
  a.nblocks = nblocks;
  a.n = s->n;
  a.g[0] = s->g;
  a.p_out_f32[0] = s->p;
  a.p_out_bf16[0] = s->p_bf16;
  a.flags[0] = scratch;
  a.worker_mask = a.member_mask = 1u;
  a.n_workers = s->n_workers < 1 ? 1 : s->n_workers;
  a.kind = s->kind;
  a.lr = s->lr; a.mu = s->mu; a.b1 = s->b1; a.b2 = s->b2; a.eps = s->eps;
  a.divide = a.n_workers > 1 ? 1 : 0;
  a.timeout_ns = 2000000000ull;
  OnoSyncLocal& L = a.loc[0];
  L.p_master = s->p;
  L.m = s->m;
  L.v = s->v;
  L.state_off = 0;
  L.adam_pows = s->adam_pows;
  L.epoch = scratch + (size_t)ONO_NOALLOC_MAX_BLOCKS * ONO_MAX_RANKS;
  L.sumsq = s->sumsq;
  L.status = s->status;
  L.n_ranges = 1;
  L.ranges[0].begin = 0;
  L.ranges[0].end = s->n;
  sync_kernel<<<nblocks, 512, 0, (cudaStream_t)st>>>(a);
  return check_launch("sync_step_noalloc");
}
