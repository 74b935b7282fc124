// Persistent, warp-specialised tcgen05 GEMM for sm_100a: the dense forward / dgrad / wgrad work of
// the reference's Dense layer (machine_learning/src/arch/layers/dense.rs:36-64) and the GEMM half
// of its im2col convolution (arch/layers/conv/conv2d.rs:119-125), rebuilt for Blackwell.
//
//   warp 4 (one elected lane)  TMA producer: cp.async.bulk.tensor tiles -> 128B-swizzled smem ring
//   warp 5 (one elected lane)  MMA issuer:   tcgen05.mma (kind::tf32 | kind::f16/bf16), f32
//                                            accumulators in TMEM, double buffered (2 x BN columns)
//   warps 0-3 and 6-9          epilogue:     two groups taking alternate 32-column chunks: tcgen05.ld
//                                            TMEM -> registers, bias / activation / activation-
//                                            derivative / accumulate, stores (row-major through a
//                                            swizzled staging tile + TMA store, transposed, f32, bf16)
//
// Operands may be K-major or MN-major (bf16 and tf32); the difference is confined to the TMA box
// pattern and three descriptor fields computed on the host (see make_operand()).
// All mbarrier waits are bounded; on a timeout the kernel records a code in *status, every role
// leaves its loop, TMEM is freed and the kernel returns normally.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdio.h>
#include <string.h>

#include <algorithm>
#include <mutex>

#include "act.cuh"
#include "ono_kernels.h"
#include "opt.cuh"
#include "ptx.cuh"

namespace ono {

// Predicated, fully unrolled tail loop: keeps v[] in registers (no dynamic indexing).
#define ONO_TAIL_LOOP(j) _Pragma("unroll") for (int j = 0; j < 32; ++j) if (j < ncols)

struct OperandDev {
  int mn_major;       // 0: K contiguous in global memory, 1: MN contiguous
  int n_box;          // TMA boxes per stage
  int box_mn;         // MN extent covered by one box
  uint32_t box_stride_bytes;
  uint32_t lbo_bytes, sbo_bytes, kstep_bytes;
  uint32_t layout_type;  // shared-memory descriptor layout: 2 = 128B swizzle, 1 = 128B swizzle on 32B units
};

struct GemmDev {
  int M, N, K;
  OperandDev a, b;
  uint32_t idesc;
  OnoEpilogue epi;
  int* status;
  unsigned long long timeout_ns;
  int split_k;  // > 1: K is split over that many work items per tile; split s writes its partial product to slab s of `slabs`
  int tma_out;  // 0: thread stores only; 1: out_f32 leaves through a TMA store; 2: out_bf16 does; 3: out_f32 += through TMA reduce-add
  float* slabs;            // split-K partial products: [split_k][M][slab_ld] f32
  long long slab_elems;    // M * slab_ld
  int slab_ld;
  OnoApply apply;          // optimizer applied to the result tile in the epilogue (apply.p != nullptr)
  const unsigned int* gate;          // flags that must reach *gate_target before the first operand load (nullptr: none)
  const unsigned int* gate_target;
  int gate_stride;
  unsigned int gate_mask;
};

template <int BN>
struct TileCfg {
  static constexpr int STAGES = BN == 256 ? 4 : (BN == 128 ? 6 : 8);
  static constexpr uint32_t TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;
};

__device__ __forceinline__ void fail(const GemmDev& p, volatile int* abort_flag, int code) {
  if (p.status) atomicCAS(p.status, 0, code);
  *abort_flag = 1;
}

// Processes 32 consecutive columns [n0, n0+32) of row m held in v[].
__device__ __forceinline__ void epilogue_chunk(const OnoEpilogue& e, float (&v)[32], int m, int n0,
                                               int M, int N, int tma_out) {
  const bool row_ok = m < M;
  const int ncols = min(32, N - n0);
  const bool full = ncols == 32;
  if (e.alpha != 1.0f) {
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] *= e.alpha;
  }
  if (e.bias) {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j < ncols) v[j] += __ldg(e.bias + n0 + j);
  } else if (e.bias_bf16) {
    const __nv_bfloat16* bb = reinterpret_cast<const __nv_bfloat16*>(e.bias_bf16) + n0;
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j < ncols) v[j] += __bfloat162float(bb[j]);
  }
  const size_t row_off = (size_t)m * e.ld_out + n0;
  if (row_ok && e.pre_f32) {
    if (full) {
#pragma unroll
      for (int j = 0; j < 32; j += 4)
        *reinterpret_cast<float4*>(e.pre_f32 + row_off + j) =
            make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
    } else {
      ONO_TAIL_LOOP(j) e.pre_f32[row_off + j] = v[j];
    }
  }
  if (row_ok && e.pre_bf16) {
    __nv_bfloat16* pb = reinterpret_cast<__nv_bfloat16*>(e.pre_bf16) + row_off;
    if (full) {
#pragma unroll
      for (int j = 0; j < 32; j += 8) {
        uint4 pk;
        __nv_bfloat162 t0 = __floats2bfloat162_rn(v[j], v[j + 1]);
        __nv_bfloat162 t1 = __floats2bfloat162_rn(v[j + 2], v[j + 3]);
        __nv_bfloat162 t2 = __floats2bfloat162_rn(v[j + 4], v[j + 5]);
        __nv_bfloat162 t3 = __floats2bfloat162_rn(v[j + 6], v[j + 7]);
        pk.x = *reinterpret_cast<uint32_t*>(&t0);
        pk.y = *reinterpret_cast<uint32_t*>(&t1);
        pk.z = *reinterpret_cast<uint32_t*>(&t2);
        pk.w = *reinterpret_cast<uint32_t*>(&t3);
        *reinterpret_cast<uint4*>(pb + j) = pk;
      }
    } else {
      ONO_TAIL_LOOP(j) pb[j] = __float2bfloat16_rn(v[j]);
    }
  }
  if (e.act != ACT_NONE) {
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = act_fwd(e.act, e.act_param, v[j]);
  }
  if (e.dact != ACT_NONE && row_ok) {
    const size_t aoff = (size_t)m * e.ld_aux + n0;
    if (e.aux_f32) {
      if (full) {
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
          float4 a = *reinterpret_cast<const float4*>(e.aux_f32 + aoff + j);
          v[j] = act_bwd(e.dact, e.dact_param, e.relu_quirk, a.x, v[j]);
          v[j + 1] = act_bwd(e.dact, e.dact_param, e.relu_quirk, a.y, v[j + 1]);
          v[j + 2] = act_bwd(e.dact, e.dact_param, e.relu_quirk, a.z, v[j + 2]);
          v[j + 3] = act_bwd(e.dact, e.dact_param, e.relu_quirk, a.w, v[j + 3]);
        }
      } else {
        ONO_TAIL_LOOP(j)
          v[j] = act_bwd(e.dact, e.dact_param, e.relu_quirk, e.aux_f32[aoff + j], v[j]);
      }
    } else if (e.aux_bf16) {
      const __nv_bfloat16* ab = reinterpret_cast<const __nv_bfloat16*>(e.aux_bf16) + aoff;
      if (full) {
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
          uint4 pk = *reinterpret_cast<const uint4*>(ab + j);
          const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&pk);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            float2 f = __bfloat1622float2(h[q]);
            v[j + 2 * q] = act_bwd(e.dact, e.dact_param, e.relu_quirk, f.x, v[j + 2 * q]);
            v[j + 2 * q + 1] = act_bwd(e.dact, e.dact_param, e.relu_quirk, f.y, v[j + 2 * q + 1]);
          }
        }
      } else {
        ONO_TAIL_LOOP(j)
          v[j] = act_bwd(e.dact, e.dact_param, e.relu_quirk, __bfloat162float(ab[j]), v[j]);
      }
    }
  }
  if (row_ok && e.out_f32 && tma_out != 1 && tma_out != 3) {
    float* o = e.out_f32 + row_off;
    if (full) {
#pragma unroll
      for (int j = 0; j < 32; j += 4) {
        float4 r = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
        if (e.beta != 0.0f) {
          float4 old = *reinterpret_cast<const float4*>(o + j);
          r.x += e.beta * old.x; r.y += e.beta * old.y; r.z += e.beta * old.z; r.w += e.beta * old.w;
          v[j] = r.x; v[j + 1] = r.y; v[j + 2] = r.z; v[j + 3] = r.w;
        }
        *reinterpret_cast<float4*>(o + j) = r;
      }
    } else {
      ONO_TAIL_LOOP(j) {
        if (e.beta != 0.0f) v[j] += e.beta * o[j];
        o[j] = v[j];
      }
    }
  }
  if (row_ok && e.out_bf16 && tma_out != 2) {
    __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(e.out_bf16) + row_off;
    if (full) {
#pragma unroll
      for (int j = 0; j < 32; j += 8) {
        uint4 pk;
        pk.x = pack16x2(v[j], v[j + 1], e.out16_f16);
        pk.y = pack16x2(v[j + 2], v[j + 3], e.out16_f16);
        pk.z = pack16x2(v[j + 4], v[j + 5], e.out16_f16);
        pk.w = pack16x2(v[j + 6], v[j + 7], e.out16_f16);
        *reinterpret_cast<uint4*>(o + j) = pk;
      }
    } else if (e.out16_f16) {
      __half* oh = reinterpret_cast<__half*>(o);
      ONO_TAIL_LOOP(j) oh[j] = __float2half_rn(v[j]);
    } else {
      ONO_TAIL_LOOP(j) o[j] = __float2bfloat16_rn(v[j]);
    }
  }
  // Transposed copies: for a fixed column the 32 lanes of a warp hold 32 consecutive rows, so each
  // store instruction writes one contiguous 128-byte (f32) or 64-byte (bf16) run.
  if (row_ok && e.outT_f32) {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j < ncols) e.outT_f32[(size_t)(n0 + j) * e.ld_outT + m] = v[j];
  }
  if (row_ok && e.outT_bf16) {
    __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(e.outT_bf16);
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j < ncols) o[(size_t)(n0 + j) * e.ld_outT + m] = __float2bfloat16_rn(v[j]);
  }
}

// PAIR = true: two CTAs of a cluster work on one 256 x BN tile (tcgen05 cta_group::2). Each CTA stages its own
// 128 rows of A and its own BN/2 rows of B, so every byte of B crosses L2 -> SM once per pair instead of
// once per CTA; the leader CTA (cluster rank 0) issues the MMAs for both, each CTA drains its own TMEM.
// APPLY = true: the instantiation whose epilogue applies the optimizer through TMA: the operand ring shrinks to two
// stages and every epilogue warp gets APPLY_WARP_BYTES of shared memory for the tiles of the master, the optimizer state
// and the bf16 shadow that belong to the 32 x 32 accumulator chunk it is working on (see the epilogue below).
struct ApplyMaps { CUtensorMap p, m, v, s; };
constexpr uint32_t APPLY_WARP_BYTES = 20480;

template <int ESIZE, int BN, bool PAIR, bool APPLY>
__global__ void __launch_bounds__(320, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ CUtensorMap tmC, const __grid_constant__ ApplyMaps am, const GemmDev p) {
  constexpr int BM = 128;              // rows per CTA
  constexpr int TILE_M = PAIR ? 256 : 128;
  constexpr int BK = 128 / ESIZE;      // one 128-byte swizzle row of K per stage
  constexpr int UMMA_K = 32 / ESIZE;   // 8 for tf32, 16 for bf16
  constexpr int KSTEPS = BK / UMMA_K;  // 4
  constexpr int BN_CTA = PAIR ? BN / 2 : BN;   // rows of B staged by one CTA
  constexpr uint32_t A_BYTES = BM * 128, B_BYTES = BN_CTA * 128, STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr int STAGES = APPLY ? 2 : TileCfg<BN_CTA>::STAGES;
  constexpr uint32_t TMEM_COLS = TileCfg<BN>::TMEM_COLS;
  const uint32_t crank = PAIR ? cluster_ctarank() : 0u;
  const bool leader = crank == 0u;
  const int unit = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;      // CTA or CTA pair
  const int units = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  // eight 4 KB output staging tiles (one per epilogue warp: 32 rows x 128 B) behind the operand ring, for TMA stores
  uint8_t* cstage = smem + (size_t)STAGES * STAGE_BYTES;

  __shared__ __align__(8) uint64_t full_bar[STAGES];
  __shared__ __align__(8) uint64_t empty_bar[STAGES];
  __shared__ __align__(8) uint64_t tmem_full_bar[2];
  __shared__ __align__(8) uint64_t tmem_empty_bar[2];
  __shared__ __align__(8) uint64_t drain_bar;
  __shared__ __align__(8) uint64_t apply_bar[APPLY ? 16 : 1];   // [epilogue warp][buffer]: tiles of a chunk have landed
  __shared__ uint32_t tmem_base_smem;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  volatile int* abortp = &abort_flag;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tmem_full_bar[b], 1);
      mbar_init(&tmem_empty_bar[b], PAIR ? 512 : 256);   // 8 epilogue warps; a pair's leader counts both CTAs'
    }
    mbar_init(&drain_bar, 1);
    if (APPLY)
      for (int b = 0; b < 16; ++b) mbar_init(&apply_bar[b], 1);
    abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 4 && lane == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    if (p.tma_out) tma_prefetch_desc(&tmC);
    if (APPLY) { tma_prefetch_desc(&am.p); tma_prefetch_desc(&am.m); tma_prefetch_desc(&am.v); tma_prefetch_desc(&am.s); }
  }
  if (warp == 5) {
    if (PAIR) { tmem_alloc_pair(&tmem_base_smem, TMEM_COLS); tmem_relinquish_pair(); }
    else { tmem_alloc(&tmem_base_smem, TMEM_COLS); tmem_relinquish(); }
  }
  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();   // the peer's barriers exist before anything is signalled across CTAs
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_smem;

  const int num_m = (p.M + TILE_M - 1) / TILE_M;
  const int num_n = (p.N + BN - 1) / BN;
  const int total_tiles = num_m * num_n;
  const int KB = (p.K + BK - 1) / BK;
  const uint64_t budget = p.timeout_ns;
  // with a gate the producer may legitimately spend its whole budget before the first load: the roles behind it wait longer,
  // so that a gate that never opens is reported as such and not as a stalled pipeline
  const uint64_t cbudget = p.gate ? 2 * budget + 1000000ull : budget;
  // split-K: a work item is (tile, split); split s reduces k-blocks [s*KB_PER, min(KB, (s+1)*KB_PER))
  // and adds its partial product to the output with atomics (the host guarantees no split is empty).
  const int SPLITS = p.split_k > 1 ? p.split_k : 1;
  const int KB_PER = (KB + SPLITS - 1) / SPLITS;
  const int total_work = total_tiles * SPLITS;

  if (warp == 4) {
    if (lane == 0) {
      // ---------------- TMA producer ----------------
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      if (p.gate) {
        // the operands are still being delivered (e.g. fresh weights arriving from their owners): wait, bounded, for every
        // selected flag, then order the TMA (async proxy) reads behind the acquire
        const uint32_t want = *p.gate_target;
        for (int i = 0; i < 32 && ok; ++i)
          if (((p.gate_mask >> i) & 1u) && !wait_flag_ge(p.gate + (size_t)i * p.gate_stride, want, budget)) {
            fail(p, abortp, ONO_ERR_TIMEOUT_PEER_FLAG);
            ok = false;
          }
        asm volatile("fence.proxy.async;" ::: "memory");
      }
      for (int work = unit; work < total_work && ok; work += units) {
        const int tile = work / SPLITS, split = work % SPLITS;
        const int m0 = (tile % num_m) * TILE_M + (int)crank * BM;
        const int n0 = (tile / num_m) * BN + (int)crank * (PAIR ? BN_CTA : 0);
        const int kb0 = split * KB_PER, kb1 = min(KB, kb0 + KB_PER);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1u, abortp, budget)) {
            fail(p, abortp, ONO_ERR_TIMEOUT_EMPTY);
            ok = false;
            break;
          }
          // pair: both CTAs' copies complete on the leader's barrier, which expects the bytes of both
          if (!PAIR) mbar_expect_tx(&full_bar[stage], STAGE_BYTES);
          else if (leader) mbar_expect_tx(&full_bar[stage], 2u * STAGE_BYTES);
          const uint32_t full_remote = PAIR ? mapa_shared(smem_u32(&full_bar[stage]), 0u) : 0u;
          uint8_t* sa = smem + (size_t)stage * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          const int k0 = kb * BK;
          for (int i = 0; i < p.a.n_box; ++i) {
            const int mn = m0 + i * p.a.box_mn;
            if (PAIR) tma_load_2d_pair(sa + i * p.a.box_stride_bytes, &tmA, full_remote,
                                       p.a.mn_major ? mn : k0, p.a.mn_major ? k0 : mn);
            else tma_load_2d(sa + i * p.a.box_stride_bytes, &tmA, &full_bar[stage],
                             p.a.mn_major ? mn : k0, p.a.mn_major ? k0 : mn);
          }
          for (int i = 0; i < p.b.n_box; ++i) {
            const int mn = n0 + i * p.b.box_mn;
            if (PAIR) tma_load_2d_pair(sb + i * p.b.box_stride_bytes, &tmB, full_remote,
                                       p.b.mn_major ? mn : k0, p.b.mn_major ? k0 : mn);
            else tma_load_2d(sb + i * p.b.box_stride_bytes, &tmB, &full_bar[stage],
                             p.b.mn_major ? mn : k0, p.b.mn_major ? k0 : mn);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) {
        // Give copies already in flight time to land before the CTA retires its shared memory.
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) { __nanosleep(1000); }
      }
    }
  } else if (warp == 5) {
    if (lane == 0 && leader) {
      // ---------------- MMA issuer (the pair's leader issues for both CTAs) ----------------
      int stage = 0;
      uint32_t phase = 0;
      int t = 0;
      bool ok = true;
      for (int work = unit; work < total_work && ok; work += units, ++t) {
        const int split = work % SPLITS;
        const int kb0 = split * KB_PER, kb1 = min(KB, kb0 + KB_PER);
        const int buf = t & 1;
        const uint32_t acc_phase = (t >> 1) & 1;
        if (!mbar_wait_bounded(&tmem_empty_bar[buf], acc_phase ^ 1u, abortp, cbudget)) {
          fail(p, abortp, ONO_ERR_TIMEOUT_TMEM_EMPTY);
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(buf * BN);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait_bounded(&full_bar[stage], phase, abortp, cbudget)) {
            fail(p, abortp, ONO_ERR_TIMEOUT_FULL);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + (size_t)stage * STAGE_BYTES);
          const uint32_t b_addr = a_addr + A_BYTES;
#pragma unroll
          for (int k = 0; k < KSTEPS; ++k) {
            const uint64_t adesc =
                make_smem_desc_sw128(a_addr + k * p.a.kstep_bytes, p.a.lbo_bytes, p.a.sbo_bytes, p.a.layout_type);
            const uint64_t bdesc =
                make_smem_desc_sw128(b_addr + k * p.b.kstep_bytes, p.b.lbo_bytes, p.b.sbo_bytes, p.b.layout_type);
            const uint32_t acc = (kb != kb0) || (k != 0);
            if (PAIR) {
              if (ESIZE == 4) umma_tf32_pair(d_tmem, adesc, bdesc, p.idesc, acc);
              else umma_f16_pair(d_tmem, adesc, bdesc, p.idesc, acc);
            } else {
              if (ESIZE == 4) umma_tf32(d_tmem, adesc, bdesc, p.idesc, acc);
              else umma_f16(d_tmem, adesc, bdesc, p.idesc, acc);
            }
          }
          // the stage is free (in both CTAs of a pair) once these MMAs have read it
          if (PAIR) umma_commit_pair_mc(&empty_bar[stage], 3);
          else umma_commit(&empty_bar[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) {
          if (PAIR) umma_commit_pair_mc(&tmem_full_bar[buf], 3);
          else umma_commit(&tmem_full_bar[buf]);
        }
      }
      // Make sure no MMA is still running before TMEM is released.
      if (PAIR) umma_commit_pair(&drain_bar);
      else umma_commit(&drain_bar);
      mbar_wait_bounded(&drain_bar, 0, abortp, ok ? cbudget : 1000000ull);
    }
  } else {
    // ---------------- epilogue warps 0..3 (TMEM lanes 32*warp .. 32*warp+31) ----------------
    int t = 0;
    bool ok = true;
    // Two groups of four warps (warps 0-3 and 6-9) take alternate 32-column chunks of the accumulator, each
    // group. Every warp owns a 4 KB staging tile (its 32 rows x 32 columns) and its own TMA-store queue, so eight
    // stores are in flight per CTA and no warp waits for another.
    const int grp = warp >= 6 ? 1 : 0;
    const int quad = warp & 3;                 // TMEM lane quadrant this warp may read
    uint8_t* const wstage = cstage + (size_t)(grp * 4 + quad) * 4096u;
    const uint32_t tmem_empty_remote[2] = {PAIR ? mapa_shared(smem_u32(&tmem_empty_bar[0]), 0u) : 0u,
                                           PAIR ? mapa_shared(smem_u32(&tmem_empty_bar[1]), 0u) : 0u};
    if constexpr (APPLY) {
      // ---------------- optimizer in the epilogue, tiles moved by TMA ----------------
      // For every 32 x 32 chunk of dW the warp brings the matching tiles of the f32 master and of the optimizer state
      // into shared memory with TMA loads (issued one chunk ahead when two buffers fit, also across output tiles, since
      // they do not depend on the MMAs), updates them in place with the gradient values it reads from TMEM (a lane
      // holds one row in both), writes the bf16 shadow tile next to them and sends everything back with TMA stores.
      // Out-of-range rows and columns are zero-filled by the loads and clipped by the stores.
      const OnoApply& ap = p.apply;
      const int narr = 1 + (ap.kind >= 1 ? 1 : 0) + (ap.kind == 2 ? 1 : 0);
      const uint32_t slot_bytes = (uint32_t)narr * 4096u + 2048u;
      const int nbuf = APPLY_WARP_BYTES / slot_bytes >= 2 ? 2 : 1;
      const int ew = grp * 4 + quad;                                   // epilogue warp index 0..7
      uint8_t* const wbase = cstage + (size_t)ew * APPLY_WARP_BYTES;
      uint64_t* const bars = &apply_bar[ew * 2];
      OptScal os{ap.kind, ap.lr, ap.mu, ap.b1, ap.b2, ap.eps, ap.grad_scale, 0.0f};
      if (ap.kind == 2) os.adam_step = ap.lr * sqrtf(1.0f - __ldg(ap.adam_pows + 1)) / (1.0f - __ldg(ap.adam_pows));
      // chunk iterator over this warp's (work item, column chunk) sequence
      // (each group of four warps walks its own contiguous half of the tile's columns, so that a warp's successive
      // chunks continue the same rows in memory)
      constexpr int CPG = BN / 64;                 // chunks per group and tile
      auto first_chunk = [&](int& w, int& c) {
        c = grp * CPG;
        while (w < total_work && (w / num_m) * BN + c * 32 >= p.N) w += units;
      };
      auto next_chunk = [&](int& w, int& c) {
        c += 1;
        if (c >= (grp + 1) * CPG || (w / num_m) * BN + c * 32 >= p.N) { w += units; first_chunk(w, c); }
      };
      auto issue = [&](int w, int c, int b) {      // lane 0: loads of chunk (w, c) into buffer b
        const int y = (w % num_m) * TILE_M + (int)crank * BM + quad * 32;
        const int x = (w / num_m) * BN + c * 32;
        uint8_t* dst = wbase + (size_t)b * slot_bytes;
        mbar_expect_tx(&bars[b], (uint32_t)narr * 4096u);
        tma_load_2d(dst, &am.p, &bars[b], x, y);
        if (ap.kind >= 1) tma_load_2d(dst + 4096, &am.m, &bars[b], x, y);
        if (ap.kind == 2) tma_load_2d(dst + 8192, &am.v, &bars[b], x, y);
      };
      int pw = unit, pc = 0;                       // next chunk to prefetch
      first_chunk(pw, pc);
      long long issued = 0, done = 0;
      if (lane == 0)
        for (; issued < nbuf && pw < total_work; ++issued) { issue(pw, pc, (int)issued); next_chunk(pw, pc); }
      for (int work = unit; work < total_work && ok; work += units, ++t) {
        const int m0 = (work % num_m) * TILE_M + (int)crank * BM;
        const int n0 = (work / num_m) * BN;
        const int buf = t & 1;
        const uint32_t acc_phase = (t >> 1) & 1;
        const bool got = mbar_wait_bounded(&tmem_full_bar[buf], acc_phase, abortp, cbudget);
        if (!__all_sync(0xffffffffu, got)) {
          if (lane == 0) fail(p, abortp, ONO_ERR_TIMEOUT_TMEM_FULL);
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(buf * BN);
#pragma unroll 1
        for (int c = grp * CPG; c < (grp + 1) * CPG; ++c) {
          const int nc = n0 + c * 32;
          if (nc >= p.N) break;
          const int b = (int)(done % nbuf);
          const bool landed = mbar_wait_bounded(&bars[b], (uint32_t)((done / nbuf) & 1), abortp, cbudget);
          if (!__all_sync(0xffffffffu, landed)) {
            if (lane == 0) fail(p, abortp, ONO_ERR_TIMEOUT_FULL);
            ok = false;
            break;
          }
          uint32_t r[32];
          tmem_ld_x32(t_row + (uint32_t)(c * 32), r);
          tmem_ld_wait();
          uint8_t* const tp = wbase + (size_t)b * slot_bytes + lane * 128;      // this lane's row of the master tile
          uint8_t* const ts = wbase + (size_t)b * slot_bytes + (size_t)narr * 4096u + lane * 64;   // and of the shadow tile
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) {
            float4 out[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const int j = 2 * jj + h;
              const uint32_t o = (uint32_t)((j ^ (lane & 7)) << 4);
              const float4 g = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                           __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
              float4 P = *reinterpret_cast<const float4*>(tp + o);
              float4 Mo = make_float4(0.f, 0.f, 0.f, 0.f), Vo = Mo;
              if (ap.kind >= 1) Mo = *reinterpret_cast<const float4*>(tp + 4096 + o);
              if (ap.kind == 2) Vo = *reinterpret_cast<const float4*>(tp + 8192 + o);
              P = opt_apply4(os, P, g, Mo, Vo);
              *reinterpret_cast<float4*>(tp + o) = P;
              if (ap.kind >= 1) *reinterpret_cast<float4*>(tp + 4096 + o) = Mo;
              if (ap.kind == 2) *reinterpret_cast<float4*>(tp + 8192 + o) = Vo;
              out[h] = P;
            }
            if (ap.p_bf16) {
              const uint2 lo = pack_bf16x4(out[0]), hi = pack_bf16x4(out[1]);
              *reinterpret_cast<uint4*>(ts + ((jj ^ ((lane >> 1) & 3)) << 4)) = make_uint4(lo.x, lo.y, hi.x, hi.y);
            }
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            const int y = m0 + quad * 32;
            uint8_t* src = wbase + (size_t)b * slot_bytes;
            tma_store_2d(&am.p, src, nc, y);
            if (ap.kind >= 1) tma_store_2d(&am.m, src + 4096, nc, y);
            if (ap.kind == 2) tma_store_2d(&am.v, src + 8192, nc, y);
            if (ap.p_bf16) tma_store_2d(&am.s, src + (size_t)narr * 4096u, nc, y);
            tma_store_commit();
            if (pw < total_work) {                  // refill this buffer once its stores have read it
              tma_store_wait_read<0>();
              issue(pw, pc, b);
              next_chunk(pw, pc);
              ++issued;
            }
          }
          __syncwarp();
          ++done;
        }
        tc_fence_before();
        if (PAIR) mbar_arrive_cluster(tmem_empty_remote[buf]);
        else mbar_arrive(&tmem_empty_bar[buf]);
      }
      if (lane == 0) {
        tma_store_wait_all<0>();
        if (!ok) {      // loads already issued into this warp's buffers must land before the CTA retires its shared memory
          const uint64_t t0 = globaltimer_ns();
          while (globaltimer_ns() - t0 < 200000ull) { __nanosleep(1000); }
        }
      }
    } else
    for (int work = unit; work < total_work && ok; work += units, ++t) {
      const int tile = work / SPLITS;
      const int m0 = (tile % num_m) * TILE_M + (int)crank * BM;
      const int n0 = (tile / num_m) * BN;
      const int buf = t & 1;
      const uint32_t acc_phase = (t >> 1) & 1;
      const bool got = mbar_wait_bounded(&tmem_full_bar[buf], acc_phase, abortp, cbudget);
      if (!__all_sync(0xffffffffu, got)) {
        if (lane == 0) fail(p, abortp, ONO_ERR_TIMEOUT_TMEM_FULL);
        ok = false;
        break;
      }
      tc_fence_after();
      const int row = quad * 32 + lane;
      const int m = m0 + row;
      const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(buf * BN);
#pragma unroll 1
      for (int c = grp; c < BN / 32; c += 2) {
        const int nc = n0 + c * 32;
        if (nc >= p.N) break;  // uniform across the CTA
        uint32_t r[32];
        tmem_ld_x32(t_row + (uint32_t)(c * 32), r);
        tmem_ld_wait();
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
        if (SPLITS > 1) {
          // partial product of one K range: plain stores into this split's own slab; the finishing pass adds the
          // slabs in split order, so the sum does not depend on which CTA finished first
          if (m < p.M) {
            float* o = p.slabs + (size_t)(work % SPLITS) * p.slab_elems + (size_t)m * p.slab_ld + nc;
#pragma unroll
            for (int j = 0; j < 32; j += 4)
              if (nc + j < p.slab_ld) *reinterpret_cast<float4*>(o + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
          }
          continue;
        }
        if (p.apply.p) {
          // Optimizer in the epilogue. The warp stages its 32 x 32 tile of dW, then walks the tile so that eight
          // lanes cover one 128-byte row segment: every access to the master, the state and the shadow is a full line.
          __syncwarp();                       // the previous chunk's reads of the staging tile are done
          {
            uint8_t* rp = wstage + lane * 128;
#pragma unroll
            for (int j = 0; j < 8; ++j)
              *reinterpret_cast<float4*>(rp + ((j ^ (lane & 7)) << 4)) =
                  make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
          }
          __syncwarp();
          const OnoApply& ap = p.apply;
          OptScal os{ap.kind, ap.lr, ap.mu, ap.b1, ap.b2, ap.eps, ap.grad_scale, 0.0f};
          if (ap.kind == 2) os.adam_step = ap.lr * sqrtf(1.0f - __ldg(ap.adam_pows + 1)) / (1.0f - __ldg(ap.adam_pows));
          const int c4 = lane & 7, rsub = lane >> 3;
          const int col = nc + c4 * 4;
          const int mbase = m0 + quad * 32 + rsub;
          float4 P[8], Mo[8], Vo[8];
#pragma unroll
          for (int it = 0; it < 8; ++it) {
            const int mr = mbase + it * 4;
            P[it] = Mo[it] = Vo[it] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (col < p.N && mr < p.M) {
              const size_t off = (size_t)mr * ap.ld + col;
              P[it] = __ldcs(reinterpret_cast<const float4*>(ap.p + off));
              if (ap.kind >= 1) Mo[it] = __ldcs(reinterpret_cast<const float4*>(ap.m + off));
              if (ap.kind == 2) Vo[it] = __ldcs(reinterpret_cast<const float4*>(ap.v + off));
            }
          }
#pragma unroll
          for (int it = 0; it < 8; ++it) {
            const int r = it * 4 + rsub;
            const int mr = mbase + it * 4;
            if (col < p.N && mr < p.M) {
              const size_t off = (size_t)mr * ap.ld + col;
              const float4 g = *reinterpret_cast<const float4*>(wstage + r * 128 + ((c4 ^ (r & 7)) << 4));
              const float4 pp = opt_apply4(os, P[it], g, Mo[it], Vo[it]);
              __stcs(reinterpret_cast<float4*>(ap.p + off), pp);
              if (ap.kind >= 1) __stcs(reinterpret_cast<float4*>(ap.m + off), Mo[it]);
              if (ap.kind == 2) __stcs(reinterpret_cast<float4*>(ap.v + off), Vo[it]);
              if (ap.p_bf16) *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(ap.p_bf16) + off) = pack_bf16x4(pp);
            }
          }
          continue;
        }
        epilogue_chunk(p.epi, v, m, nc, p.M, p.N, p.tma_out);
        if (p.tma_out) {
          // registers -> swizzled staging tile -> one TMA store per warp and 32 x 32 chunk; the TMA unit
          // clips rows >= M and columns >= N
          if (lane == 0) tma_store_wait_read<0>();  // this warp's previous store has read the tile
          __syncwarp();
          if (p.tma_out != 2) {
            uint8_t* rp = wstage + lane * 128;
#pragma unroll
            for (int j = 0; j < 8; ++j)
              *reinterpret_cast<float4*>(rp + ((j ^ (row & 7)) << 4)) =
                  make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
          } else {
            uint8_t* rp = wstage + lane * 64;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint4 pk;
              pk.x = pack16x2(v[8 * j], v[8 * j + 1], p.epi.out16_f16);
              pk.y = pack16x2(v[8 * j + 2], v[8 * j + 3], p.epi.out16_f16);
              pk.z = pack16x2(v[8 * j + 4], v[8 * j + 5], p.epi.out16_f16);
              pk.w = pack16x2(v[8 * j + 6], v[8 * j + 7], p.epi.out16_f16);
              *reinterpret_cast<uint4*>(rp + ((j ^ ((row >> 1) & 3)) << 4)) = pk;
            }
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            if (p.tma_out == 3) tma_reduce_add_2d(&tmC, wstage, nc, m0 + quad * 32);
            else tma_store_2d(&tmC, wstage, nc, m0 + quad * 32);
            tma_store_commit();
          }
        }
      }
      tc_fence_before();
      if (PAIR) mbar_arrive_cluster(tmem_empty_remote[buf]);
      else mbar_arrive(&tmem_empty_bar[buf]);
    }
    if (!APPLY && p.tma_out && lane == 0) tma_store_wait_all<0>();  // global writes done before exit
  }

  tc_fence_before();
  __syncthreads();
  // pair: neither CTA retires its shared memory, barriers or TMEM while the other may still touch them
  if (PAIR) cluster_sync_all();
  if (warp == 5) {
    tc_fence_after();
    if (PAIR) tmem_dealloc_pair(tmem_base, TMEM_COLS);
    else tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// Two-pass form (split-K). Used for problems with a handful of output tiles and a long reduction (e.g. 342 x 128 x 3136:
// three tiles, i.e. three SMs streaming 98 k-blocks each) and whenever the caller asks for a split: the reduction is
// split over the SMs, split s stores its partial product into slab s of a workspace, and this pass adds the slabs in
// split order and runs the regular epilogue (bias, activation, derivative, every output form) on the sums. The result
// is the same to the bit from run to run. The workspace comes from the caller (OnoGemm::workspace, e.g. one per
// stream); without one a static buffer is used, and such GEMMs must then not overlap on the device.
constexpr long long SPLIT_SCRATCH_ELEMS = 4ll << 20;
__device__ float g_split_scratch[SPLIT_SCRATCH_ELEMS];

// One block per 32 x 32 tile of the result, eight warps: warp w adds the slabs w, w + 8, w + 16, ... (a lane owns one row of
// the tile, eight 16-byte loads per slab), the eight partial sums are then added in warp order through shared memory, and
// warp 0 runs the epilogue. The order of every addition is fixed, so the result does not depend on timing.
__global__ void __launch_bounds__(256) gemm_finish_kernel(const float* slabs, long long slab_elems, int nslabs, int ld, int M,
                                                          int N, const OnoEpilogue e) {
  __shared__ float part[7][32][33];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m = blockIdx.x * 32 + lane;
  const int n0 = blockIdx.y * 32;
  float v[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) v[j] = 0.f;
  if (m < M) {
    for (int sidx = warp; sidx < nslabs; sidx += 8) {
      const float* src = slabs + (size_t)sidx * slab_elems + (size_t)m * ld + n0;
#pragma unroll
      for (int j = 0; j < 32; j += 4)
        if (n0 + j < ld) {
          const float4 q = __ldcs(reinterpret_cast<const float4*>(src + j));
          v[j] += q.x; v[j + 1] += q.y; v[j + 2] += q.z; v[j + 3] += q.w;
        }
    }
  }
  if (warp > 0) {
#pragma unroll
    for (int j = 0; j < 32; ++j) part[warp - 1][lane][j] = v[j];
  }
  __syncthreads();
  if (warp != 0) return;
#pragma unroll 1
  for (int w = 0; w < 7; ++w) {
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] += part[w][lane][j];
  }
  epilogue_chunk(e, v, m, n0, M, N, 0);
}

// ------------------------------------------------------------------------------------------------
// Host side
// ------------------------------------------------------------------------------------------------
static thread_local char g_err[512] = "";
void set_error(const char* fmt, const char* a = "", long long b = 0, long long c = 0) {
  snprintf(g_err, sizeof(g_err), fmt, a, b, c);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(f);
  });
  return fn;
}

// 2-D row-major global matrix [rows, cols] with leading dimension ld (elements); box = {box_cols
// (innermost, 128 bytes), box_rows}; 128-byte swizzle.
int encode_map_2d(CUtensorMap* map, const void* base, int esize, long long rows, long long cols,
                  long long ld, int box_cols, int box_rows, bool swizzle_32b_units = false) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) { set_error("cuTensorMapEncodeTiled unavailable%s", ""); return -2; }
  if (((uintptr_t)base & 15) != 0) { set_error("TMA base not 16-byte aligned%s", ""); return -3; }
  if ((ld * esize) % 16 != 0) { set_error("TMA row stride %s%lld bytes not a multiple of 16", "", ld * esize); return -3; }
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)(ld * esize)};
  cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMapDataType dt = esize == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUresult r = fn(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle_32b_units ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled failed (%s%lld)", "", (long long)r); return -4; }
  return 0;
}

// Output tile map for the TMA-store epilogue: box = {32 columns, 32 rows}; the 128-byte (f32) or
// 64-byte (bf16) rows use the matching swizzle so that the staging writes are bank-conflict free.
static int encode_out_map(CUtensorMap* map, const void* base, int esize, long long rows, long long cols, long long ld) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) { set_error("cuTensorMapEncodeTiled unavailable%s", ""); return -2; }
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)(ld * esize)};
  cuuint32_t box[2] = {32u, 32u};   // one epilogue warp's rows
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, esize == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                  const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  esize == 4 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled (output) failed (%s%lld)", "", (long long)r); return -4; }
  return 0;
}

// Fills the device-side operand description and encodes the operand's tensor map.
static int make_operand(OperandDev* od, CUtensorMap* map, const void* ptr, int esize, int major,
                        int MN, int K, int ld, int tile_mn) {
  const int BK = 128 / esize;
  if (major == ONO_K_MAJOR) {
    od->mn_major = 0;
    od->n_box = 1;
    od->box_mn = tile_mn;
    od->box_stride_bytes = 0;
    od->lbo_bytes = 16;      // unused for a single swizzle atom along K
    od->sbo_bytes = 1024;    // 8 rows x 128 bytes
    od->kstep_bytes = 32;    // one UMMA_K slice inside the 128-byte row
    od->layout_type = 2;
    return encode_map_2d(map, ptr, esize, MN, K, ld, BK, tile_mn);
  }
  if (esize == 4) {
    // 32-bit MN-major operands: rows of 32 elements (128 bytes) of MN, swizzled on 32-byte units in atoms of 4 K-rows
    // (the layout tcgen05 defines for tf32 operands whose MN dimension is contiguous); one MMA (UMMA_K = 8) reads two atoms.
    const int chunk4 = 32;
    od->mn_major = 1;
    od->n_box = tile_mn / chunk4;
    if (od->n_box < 1) { set_error("MN-major tile too narrow%s", ""); return -5; }
    od->box_mn = chunk4;
    od->box_stride_bytes = (uint32_t)BK * 128u;
    od->lbo_bytes = od->box_stride_bytes;   // between 32-wide MN atoms
    od->sbo_bytes = 512;                    // between groups of 4 K-rows
    od->kstep_bytes = 8u * 128u;            // UMMA_K rows of K
    od->layout_type = 1;
    return encode_map_2d(map, ptr, esize, K, MN, ld, chunk4, BK, true);
  }
  const int chunk = 128 / esize;  // 64 elements of MN per 128-byte row
  od->mn_major = 1;
  od->n_box = tile_mn / chunk;
  if (od->n_box < 1) { set_error("MN-major tile too narrow%s", ""); return -5; }
  od->box_mn = chunk;
  od->box_stride_bytes = (uint32_t)BK * 128u;  // BK rows of K, 128 bytes each
  od->lbo_bytes = od->box_stride_bytes;        // between 64-wide MN atoms
  od->sbo_bytes = 1024;                        // between groups of 8 K-rows
  od->kstep_bytes = (32 / esize) * 128u;       // UMMA_K rows of K
  od->layout_type = 2;
  return encode_map_2d(map, ptr, esize, K, MN, ld, chunk, BK);
}

// cudaFuncSetAttribute, symbol addresses and SM counts belong to a device: caches are kept per device.
constexpr int kMaxDevices = 64;
static int current_device() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 0;
  return dev;
}
static int num_sms() {
  static int sms[kMaxDevices] = {0};
  const int dev = current_device();
  if (sms[dev] == 0) {
    cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev);
    if (sms[dev] <= 0) sms[dev] = 148;
  }
  return sms[dev];
}

static ApplyMaps g_no_apply_maps;   // zero-filled: instantiations without the TMA optimizer epilogue never touch it

template <int ESIZE, int BN, bool PAIR, bool APPLY = false>
static int launch(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const GemmDev& p, int max_ctas,
                  cudaStream_t stream, const ApplyMaps& am = g_no_apply_maps) {
  constexpr int BN_CTA = PAIR ? BN / 2 : BN;
  constexpr int STAGES = APPLY ? 2 : TileCfg<BN_CTA>::STAGES;
  constexpr size_t smem = (size_t)STAGES * (128 * 128 + BN_CTA * 128) + (APPLY ? 8 * APPLY_WARP_BYTES : 2 * 16384) + 1024;
  static bool attr_done[kMaxDevices] = {false};
  static int max_pairs_dev[kMaxDevices] = {0};
  const int dev = current_device();
  bool& attr_set = attr_done[dev];
  int& max_pairs = max_pairs_dev[dev];
  auto kern = gemm_tcgen05_kernel<ESIZE, BN, PAIR, APPLY>;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) { set_error("cudaFuncSetAttribute: %s", cudaGetErrorString(e)); return -6; }
    if (PAIR) {
      // how many 2-CTA clusters the device can hold at once (an SM count that is odd inside a GPC loses one)
      cudaLaunchConfig_t q = {};
      q.gridDim = dim3(2 * num_sms());
      q.blockDim = dim3(320);
      q.dynamicSmemBytes = smem;
      cudaLaunchAttribute at[1];
      at[0].id = cudaLaunchAttributeClusterDimension;
      at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
      q.attrs = at;
      q.numAttrs = 1;
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, kern, &q) != cudaSuccess || n <= 0) { cudaGetLastError(); n = num_sms() / 2; }
      max_pairs = n;
    }
    attr_set = true;
  }
  const int tile_m = PAIR ? 256 : 128;
  const int tiles = ((p.M + tile_m - 1) / tile_m) * ((p.N + BN - 1) / BN) * (p.split_k > 1 ? p.split_k : 1);
  if (!PAIR) {
    int grid = max_ctas > 0 ? max_ctas : num_sms();
    if (grid > tiles) grid = tiles;
    kern<<<grid, 320, smem, stream>>>(ta, tb, tc, am, p);
  } else {
    int pairs = max_ctas > 0 ? std::max(1, max_ctas / 2) : max_pairs;
    if (pairs > max_pairs) pairs = max_pairs;
    if (pairs > tiles) pairs = tiles;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs);
    cfg.blockDim = dim3(320);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    cudaError_t le = cudaLaunchKernelEx(&cfg, kern, ta, tb, tc, am, p);
    if (le != cudaSuccess) { set_error("gemm pair launch: %s", cudaGetErrorString(le)); return -7; }
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { set_error("gemm launch: %s", cudaGetErrorString(e)); return -7; }
  return 0;
}

}  // namespace ono

extern "C" const char* ono_last_error(void) { return ono::g_err; }
extern "C" int ono_num_sms(void) { return ono::num_sms(); }

extern "C" int ono_gemm(const OnoGemm* g, ono_stream_t stream_) {
  using namespace ono;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (!g || !g->A || !g->B || g->M <= 0 || g->N <= 0 || g->K <= 0) { set_error("bad gemm args%s", ""); return -1; }
  const int esize = g->dtype == ONO_TF32 ? 4 : 2;
  int bn = g->bn;
  if (bn == 0) {
    if (g->N <= 32) bn = 32;
    else if (g->N <= 128) bn = 128;
    else {
      // Prefer 256-wide tiles unless they leave most SMs idle.
      const long long t256 = (long long)((g->M + 127) / 128) * ((g->N + 255) / 256);
      bn = t256 >= (long long)num_sms() * 3 / 4 ? 256 : 128;
    }
  }
  if (bn != 32 && bn != 128 && bn != 256) { set_error("bn must be 32, 128 or 256%s", ""); return -1; }
  if (g->b_major == ONO_MN_MAJOR && bn < 64) bn = 128;
  const OnoEpilogue& e = g->epi;
  if ((e.out_f32 || e.out_bf16 || e.pre_f32 || e.pre_bf16) && e.ld_out < g->N) { set_error("ld_out < N%s", ""); return -1; }
  if ((e.outT_f32 || e.outT_bf16) && e.ld_outT < g->M) { set_error("ld_outT < M%s", ""); return -1; }
  // The vectorised epilogue paths need 16-byte aligned rows.
  if ((e.out_f32 || e.pre_f32) && (e.ld_out % 4 != 0)) { set_error("ld_out must be a multiple of 4 for f32 outputs%s", ""); return -1; }
  if ((e.out_bf16 || e.pre_bf16) && (e.ld_out % 8 != 0)) { set_error("ld_out must be a multiple of 8 for bf16 outputs%s", ""); return -1; }
  if (e.dact != ACT_NONE) {
    if (!e.aux_f32 && !e.aux_bf16) { set_error("dact needs aux%s", ""); return -1; }
    if (e.aux_f32 && e.ld_aux % 4 != 0) { set_error("ld_aux must be a multiple of 4%s", ""); return -1; }
    if (e.aux_bf16 && e.ld_aux % 8 != 0) { set_error("ld_aux must be a multiple of 8%s", ""); return -1; }
  }

  GemmDev p;
  memset(&p, 0, sizeof(p));
  p.M = g->M; p.N = g->N; p.K = g->K;
  p.epi = g->epi;
  p.status = g->status;
  p.timeout_ns = g->timeout_ns ? g->timeout_ns : 2000000000ull;
  if (g->gate) {
    if (!g->gate_target || !g->gate_mask || g->gate_stride < 0) { set_error("gate needs a target word and a flag mask%s", ""); return -1; }
    p.gate = g->gate; p.gate_target = g->gate_target; p.gate_stride = g->gate_stride; p.gate_mask = g->gate_mask;
  }
  CUtensorMap ta, tb;
  int rc = make_operand(&p.a, &ta, g->A, esize, g->a_major, g->M, g->K, g->lda, 128);
  if (rc) return rc;
  // CTA pairs: on request only for now (M must span more than one 128-row block to be worth a pair)
  const bool pair = g->pair > 0 && bn >= 128 && g->M > 128;
  rc = make_operand(&p.b, &tb, g->B, esize, g->b_major, g->N, g->K, g->ldb, pair ? bn / 2 : bn);
  if (rc) return rc;
  // Optimizer in the epilogue: the result tile updates the master / state tiles and is not stored.
  const OnoApply& ap = g->apply;
  if (ap.p) {
    if (e.out_f32 || e.out_bf16 || e.outT_f32 || e.outT_bf16 || e.pre_f32 || e.pre_bf16 || e.bias || e.bias_bf16 ||
        e.act != ACT_NONE || e.dact != ACT_NONE || e.reduce_out) {
      set_error("apply: the epilogue optimizer excludes every other output%s", "");
      return -1;
    }
    if (ap.kind < 0 || ap.kind > 2 || (ap.kind >= 1 && !ap.m) || (ap.kind == 2 && (!ap.v || !ap.adam_pows))) {
      set_error("apply: optimizer kind or state missing%s", "");
      return -1;
    }
    if (g->N % 4 != 0 || ap.ld % 4 != 0 || ap.ld < g->N || (((uintptr_t)ap.p | (uintptr_t)ap.m | (uintptr_t)ap.v) & 15) ||
        ((uintptr_t)ap.p_bf16 & 7)) {
      set_error("apply: N and ld must be multiples of 4 and the matrices 16-byte aligned%s", "");
      return -1;
    }
    if (g->split_k > 1) { set_error("apply: split-K is not supported%s", ""); return -1; }
    p.apply = ap;
  }
  // split-K (g->split_k > 1, or 0 = automatic for long-K problems with few output tiles): see gemm_finish_kernel.
  bool two_pass = false;
  {
    const int BKe = 128 / esize;
    const int KBh = (g->K + BKe - 1) / BKe;
    const long long tiles0 = (long long)((g->M + (pair ? 255 : 127)) / (pair ? 256 : 128)) * ((g->N + bn - 1) / bn);
    const long long ldn = ((long long)g->N + 3) / 4 * 4;
    int want = g->split_k > 1 ? g->split_k : 0;
    if (g->split_k == 0 && !ap.p && !e.reduce_out && !pair && tiles0 * 8 <= num_sms() && KBh >= 16)
      want = (int)std::min<long long>(KBh / 4, num_sms() / tiles0);
    if (want > KBh) want = KBh;
    if (want >= 2) {
      if (e.reduce_out) { set_error("split-K cannot be combined with reduce_out%s", ""); return -1; }
      float* ws = g->workspace;
      long long ws_elems = g->workspace_elems;
      if (!ws) {
        static float* scratch_dev[kMaxDevices] = {nullptr};
        float*& sp = scratch_dev[current_device()];
        if (!sp && cudaGetSymbolAddress((void**)&sp, g_split_scratch) != cudaSuccess) {
          set_error("split scratch address unavailable%s", "");
          return -6;
        }
        ws = sp;
        ws_elems = SPLIT_SCRATCH_ELEMS;
      } else if (((uintptr_t)ws & 15) != 0) {
        set_error("split-K workspace must be 16-byte aligned%s", "");
        return -1;
      }
      const long long slab = (long long)g->M * ldn;
      if (want > ws_elems / slab) want = (int)(ws_elems / slab);   // as many slabs as the workspace holds
      if (want >= 2) {
        const int per = (KBh + want - 1) / want;
        p.split_k = (KBh + per - 1) / per;                         // no empty split
        p.slabs = ws;
        p.slab_elems = slab;
        p.slab_ld = (int)ldn;
        two_pass = p.split_k > 1;
      } else if (g->split_k > 1 && slab > ws_elems) {
        set_error("split-K workspace too small for one slab (%s%lld elements needed)", "", slab);
        return -1;
      }
    }
    if (!two_pass) p.split_k = 1;
  }
  // One row-major output may leave through TMA stores (coalesced, off the LSU path): the f32 output
  // when it is not accumulated into, else the 16-bit output.
  CUtensorMap tc;
  memset(&tc, 0, sizeof(tc));
  p.tma_out = 0;
  if (two_pass || ap.p) {
    // plain stores into the slabs / updates in place, no TMA store
  } else if (e.reduce_out) {
    if (!e.out_f32 || e.out_bf16 || e.outT_f32 || e.outT_bf16 || e.pre_f32 || e.pre_bf16 || ((uintptr_t)e.out_f32 & 15)) {
      set_error("reduce_out supports a plain, 16-byte aligned f32 output only%s", "");
      return -1;
    }
    rc = encode_out_map(&tc, e.out_f32, 4, g->M, g->N, e.ld_out);
    if (rc) return rc;
    p.tma_out = 3;
  } else if (e.out_f32 && e.beta == 0.0f && ((uintptr_t)e.out_f32 & 15) == 0 && g->N % 4 == 0) {
    if (encode_out_map(&tc, e.out_f32, 4, g->M, g->N, e.ld_out) == 0) p.tma_out = 1;
  } else if (e.out_bf16 && ((uintptr_t)e.out_bf16 & 15) == 0 && g->N % 8 == 0) {
    if (encode_out_map(&tc, e.out_bf16, 2, g->M, g->N, e.ld_out) == 0) p.tma_out = 2;
  }
  // (A TMA store writes whole 16-byte units: with a row of N elements that ends inside a unit it would put the
  // zero-filled rest of the unit into the columns after N, which belong to the caller when the output is a view of a
  // wider matrix. Such shapes leave through thread stores. The reduce-add form adds those zeros, which changes nothing.)
  const uint32_t fmt = g->dtype == ONO_TF32 ? 2u : 1u;  // TF32 / BF16
  p.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)p.a.mn_major << 15) |
            ((uint32_t)p.b.mn_major << 16) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)((pair ? 256 : 128) >> 4) << 24);

  // The TMA form of the optimizer epilogue: bf16 CTA pairs with 256-column tiles (the weight gradients of wide layers),
  // a reduction short enough for the two-stage operand ring, shadow rows that a bf16 tensor map can address.
  ApplyMaps am;
  // Momentum and SGD fit two chunk buffers per warp (loads run one chunk ahead); Adam's three state tiles fit only one,
  // which measured slower than reading them from registers (8192 x 8192 x 512: 0.48 ms against 0.44 ms), so Adam stays
  // on the register form. A TMA store writes whole 16-byte units, hence the shadow needs N % 8 == 0 here.
  const bool apply_tma = ap.p && pair && esize == 2 && bn == 256 && g->K <= 2048 && ap.kind <= 1 &&
                         (!ap.p_bf16 || (g->N % 8 == 0 && ap.ld % 8 == 0 && ((uintptr_t)ap.p_bf16 & 15) == 0));
  if (apply_tma) {
    memset(&am, 0, sizeof(am));
    if ((rc = encode_out_map(&am.p, ap.p, 4, g->M, g->N, ap.ld))) return rc;
    if (ap.kind >= 1 && (rc = encode_out_map(&am.m, ap.m, 4, g->M, g->N, ap.ld))) return rc;
    if (ap.kind == 2 && (rc = encode_out_map(&am.v, ap.v, 4, g->M, g->N, ap.ld))) return rc;
    if (ap.p_bf16 && (rc = encode_out_map(&am.s, ap.p_bf16, 2, g->M, g->N, ap.ld))) return rc;
    // unused maps still get prefetched by the kernel: point them at the master's map
    if (ap.kind < 1) am.m = am.p;
    if (ap.kind < 2) am.v = am.p;
    if (!ap.p_bf16) am.s = am.p;
  }
  auto run = [&]() -> int {
    if (apply_tma) return launch<2, 256, true, true>(ta, tb, tc, p, g->max_ctas, stream, am);
    if (pair) {
      if (esize == 4) return bn == 128 ? launch<4, 128, true>(ta, tb, tc, p, g->max_ctas, stream)
                                       : launch<4, 256, true>(ta, tb, tc, p, g->max_ctas, stream);
      return bn == 128 ? launch<2, 128, true>(ta, tb, tc, p, g->max_ctas, stream)
                       : launch<2, 256, true>(ta, tb, tc, p, g->max_ctas, stream);
    }
    if (esize == 4) {
      if (bn == 32) return launch<4, 32, false>(ta, tb, tc, p, g->max_ctas, stream);
      if (bn == 128) return launch<4, 128, false>(ta, tb, tc, p, g->max_ctas, stream);
      return launch<4, 256, false>(ta, tb, tc, p, g->max_ctas, stream);
    }
    if (bn == 32) return launch<2, 32, false>(ta, tb, tc, p, g->max_ctas, stream);
    if (bn == 128) return launch<2, 128, false>(ta, tb, tc, p, g->max_ctas, stream);
    return launch<2, 256, false>(ta, tb, tc, p, g->max_ctas, stream);
  };
  rc = run();
  if (rc || !two_pass) return rc;
  const dim3 fgrid((g->M + 31) / 32, (g->N + 31) / 32);
  gemm_finish_kernel<<<fgrid, 256, 0, stream>>>(p.slabs, p.slab_elems, p.split_k, p.slab_ld, g->M, g->N, g->epi);
  if (cudaGetLastError() != cudaSuccess) { set_error("gemm_finish launch failed%s", ""); return -7; }
  return 0;
}
