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
  const void* bias_bf16;     // [N] bias in bf16, optional (used when bias is null)
  const float* aux_f32;      // [M, ld_aux], optional (stored activation or pre-activation)
  const void* aux_bf16;      // same in bf16, optional
  int ld_out, ld_outT, ld_aux;
  int act;                   // ActKind applied forward
  float act_param;
  int dact;                  // ActKind whose derivative multiplies v
  float dact_param;
  int relu_quirk;            // reproduce the reference's leaky-ReLU backward
  float alpha, beta;
  int reduce_out;            // out_f32 += result through TMA reduce-add (out_f32 may be a peer GPU's memory: the GEMM pushes its
                             // tiles into the owner's accumulator over NVLink); plain f32 output only, beta ignored
  int out16_f16;             // 1: out_bf16 receives IEEE f16 values instead of bf16 (a 16-bit gradient wire in either format);
                             //    out_bf16 may be a peer GPU's memory: the tiles leave through TMA stores over NVLink
} OnoEpilogue;

// Optimizer step applied by the weight-gradient GEMM's own epilogue, for a layer that one rank owns outright: the
// tile of dW is never written to memory. The epilogue reads the matching tile of the f32 master and of the optimizer
// state, updates them in place and writes the bf16 shadow (optional). p, m, v and p_bf16 are [M, ld] matrices with the
// geometry of the GEMM result; ld and N must be multiples of 4 and the pointers 16-byte aligned (p_bf16: 8).
// p == NULL switches it off. No other output and no bias / activation may be requested together with it.
typedef struct OnoApply {
  float* p; float* m; float* v; void* p_bf16;
  int ld;
  int kind;                  // OnoOptim kinds: 0 SGD, 1 momentum, 2 Adam
  float lr, mu, b1, b2, eps;
  float grad_scale;          // the gradient is multiplied by this first
  const float* adam_pows;    // device float[2] = {b1^t, b2^t} after this step's tick (Adam)
} OnoApply;

// D[M,N] = A[M,K] * B[K,N] with f32 accumulation in TMEM.
//   A: a_major == K_MAJOR  -> memory is [M, lda] with K contiguous
//      a_major == MN_MAJOR -> memory is [K, lda] with M contiguous
//   B: b_major == K_MAJOR  -> memory is [N, ldb] with K contiguous
//      b_major == MN_MAJOR -> memory is [K, ldb] with N contiguous
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
  int split_k;     // > 1: split K over (at most) that many work items per tile, each storing its partial product into its
                   //      own slab of the workspace; a finishing pass adds the slabs in order and runs the whole epilogue
                   //      (run-to-run deterministic). 0 = the library decides, 1 = never split
  int pair;        // CTA pairs (256-row tiles, tcgen05 cta_group::2): 0 = automatic, 1 = on, -1 = off
  OnoEpilogue epi;
  int* status;     // device int, set non-zero on an in-kernel timeout; may be null
  OnoApply apply;  // optimizer fused into the epilogue (apply.p == NULL: off)
  // Gate on the operands: the TMA producer does not load anything before every selected flag word has reached the target
  // (gate[i * gate_stride] >= *gate_target for every i with bit i of gate_mask set; a bounded acquire wait: on a timeout the
  // kernel records an error in *status and returns without having loaded). Lets a GEMM be queued before another GPU has
  // finished delivering its weights (the parameter pull of a layer hides behind the layers before it). gate == NULL: off.
  const unsigned int* gate;
  const unsigned int* gate_target;
  int gate_stride;
  unsigned int gate_mask;
  unsigned long long timeout_ns;   // budget of every wait inside the kernel (0 = 2 s)
  float* workspace;           // split-K slabs, 16-byte aligned; NULL = a static buffer of the library, which GEMMs that overlap
  long long workspace_elems;  // on the device would share: give each stream its own workspace. Size in floats.
} OnoGemm;

int ono_gemm(const OnoGemm* g, ono_stream_t stream);
// Last error text of this thread (argument errors / CUDA errors), for diagnostics.
const char* ono_last_error(void);
int ono_num_sms(void);

// ---------------------------------------------------------------------------------------------
// Loss (+ fused softmax) : reference arch/loss/{mse,cross_entropy}.rs and arch/layers/softmax.rs.
// n = B*C normalises both the loss and the gradient (the reference's convention).
//   kind 0 (MSE):  L = sum (p-y)^2 / n          g = 2 (p-y) / n
//   kind 1 (CE):   L = -sum y ln max(p,eps) / n g = -(y / max(p,eps)) / n
//   softmax = 1:   p = softmax(a) and d = p * (g - sum_k p_k g_k)   (softmax.rs:44-64)
//   softmax = 0:   p = a and d = g * act'(aux)                     (last layer's activation)
// ---------------------------------------------------------------------------------------------
typedef struct OnoLoss {
  const float* a;        // [B, ld]
  const float* y;        // [B, ldy]
  const float* aux;      // [B, ld] value act' is evaluated on (null -> a)
  int B, C, ld, ldy;
  int kind, softmax;
  int dact; float dact_param; int relu_quirk;
  float eps;
  float* probs;          // optional [B, ld]
  float* d_f32;          // optional [B, ld_d]
  float* dT_f32;         // optional [C, ld_dT]
  void* d_bf16;          // optional [B, ld_d]
  void* dT_bf16;         // optional [C, ld_dT]
  int ld_d, ld_dT;
  double* loss_sum;      // += L (atomic)
  int* correct;          // optional, += #rows whose argmax(p) == argmax(y)
} OnoLoss;
int ono_loss(const OnoLoss* l, ono_stream_t stream);

// Softmax as a layer's activation anywhere in a network (arch/layers/softmax.rs:24-64), one warp per row.
//   backward == 0: out = softmax(x) row-wise (x: pre-activations)
//   backward == 1: out = p * (x - sum_k p_k x_k) (x: gradient w.r.t. the softmax output, p: the stored output, f32 or bf16)
// Any of the four output forms may be requested (row-major / transposed, f32 / bf16).
typedef struct OnoSoftmax {
  const float* x; int ld_x;
  const float* p_f32; const void* p_bf16; int ld_p;
  int B, C, backward;
  float* out_f32; void* out_bf16; float* outT_f32; void* outT_bf16;
  int ld_out, ld_outT;
} OnoSoftmax;
int ono_softmax(const OnoSoftmax* s, ono_stream_t stream);

// out[n] = beta*out[n] + sum_m d[m][n]   (bias gradient, dense.rs:58). dtype: 0 f32, 1 bf16.
int ono_colsum(const void* d, int dtype, int M, int N, int ld, float* out, float beta, ono_stream_t stream);

// Optimizers on a flat f32 shard (optimization/{gradient_descent,gradient_descent_with_momentum,adam}.rs).
typedef struct OnoOptim {
  float* p; const float* g; float* m; float* v;
  long long n;
  int kind;              // 0 SGD, 1 momentum, 2 Adam
  float lr, mu, b1, b2, eps;
  float grad_scale;      // g is multiplied by this first (1/N averaging)
  const float* adam_pows;// device float[2] = {b1^t, b2^t} after this step's tick
  void* p_bf16;          // optional bf16 shadow of p
  int zero_grad;         // 1: g is zeroed after use (g must be writable)
} OnoOptim;
int ono_optim(const OnoOptim* o, ono_stream_t stream);
int ono_adam_tick(float* pows, float b1, float b2, ono_stream_t stream);  // pows *= {b1, b2}
// Round cadence (sequential.rs:129-141): p -= lr*g ; r += g ; optional bf16 shadow of p.
int ono_local_sgd(float* p, const float* g, float* r, long long n, float lr, void* p_bf16, ono_stream_t stream);
// sum of squares of x accumulated into *out (double); used for the gradient-norm switch metric.
int ono_sumsq(const float* x, long long n, double* out, ono_stream_t stream);

// Counter-based initialisers (Philox4x32-10 keyed by seed, counter = global element index) so that
// any shard owner can generate exactly its slice. kind 0: U[lo,hi) ; 1: U[lo,hi] ; 2: N(a,b).
int ono_init(float* out, long long n, unsigned long long index_offset, unsigned long long seed,
             int kind, float a, float b, ono_stream_t stream);

// Row gather / cast / transpose: for r in [0,R): src row = idx ? idx[r] : r.
// Writes any of dst_f32 [R,ld_dst], dstT_f32 [W,ld_dstT], dst_bf16, dstT_bf16.
typedef struct OnoRows {
  const float* src; int ld_src;
  const int* idx;        // optional
  int R, W;
  float* dst_f32; float* dstT_f32; void* dst_bf16; void* dstT_bf16;
  int ld_dst, ld_dstT;
} OnoRows;
int ono_rows(const OnoRows* r, ono_stream_t stream);

// ---------------------------------------------------------------------------------------------
// Convolution / pooling helpers around the GEMM (conv.cu). Image activations are pixel-major
// matrices [B*H*W, ld]; dtype 0 = f32, 1 = bf16. K is the square kernel (conv) or filter (pool) size.
// ---------------------------------------------------------------------------------------------
typedef struct OnoConvGeom { int B, C, H, W, K, S, P, OH, OW; } OnoConvGeom;
int ono_im2col(const OnoConvGeom* g, int dtype, const void* x, int ldx, void* cols, int ld_cols, void* colsT,
               int ld_colsT, ono_stream_t stream);
int ono_col2im(const OnoConvGeom* g, int dtype, const void* dcols, int ld_dcols, const void* aux, int ld_aux, int dact,
               float dact_param, int relu_quirk, void* dx, int ld_dx, void* dxT, int ld_dxT, ono_stream_t stream);
// Direct convolution for a single input channel (k <= 5, at most 128 filters for the gradient): forward with bias + activation, and the weight + bias gradient
// (deterministic two-stage reduction; gk = beta*gk + dK in parameter order [F][k][k], gb likewise).
int ono_conv1_fwd(const OnoConvGeom* g, int F, int dtype, const void* x, int ldx, const float* kparams, const float* bias, int act,
                  float act_param, void* y, int ldy, ono_stream_t st);
int ono_conv1_wgrad(const OnoConvGeom* g, int F, int dtype, const void* x, int ldx, const void* dy, int ld_dy, float* gk, float* gb,
                    float beta, ono_stream_t st);
// Kernel tensor K[F][C][k][k] (f32) <-> GEMM operand order [F][(ky,kx,c)]: dir 0 parameters -> operand (dtype of dst and
// dstT: 0 f32, 1 bf16; dstT optional, [(ky,kx,c)][F]); dir 1 operand-ordered f32 gradient -> parameter order, dst = beta*dst + src.
int ono_conv_kperm(int F, int C, int K, int dir, int dtype, const float* src, int ld_src, void* dst, int ld_dst, void* dstT,
                   int ld_dstT, float beta, ono_stream_t st);
int ono_pool_fwd(const OnoConvGeom* g, int dtype, const void* x, int ldx, void* y, int ldy, void* yT, int ld_yT, int* arg,
                 int act, float act_param, ono_stream_t stream);
int ono_pool_bwd(const OnoConvGeom* g, int dtype, const void* d, int ldd, const void* y, int ldy, const int* arg, int act,
                 float act_param, int relu_quirk, float* dx, int ld_dx, ono_stream_t stream);
int ono_nchw_flat(int dtype, int B, int C, int HW, int to_flat, void* img, int ld_img, void* flat, int ld_flat, void* outT,
                  int ld_outT, const void* aux, int ld_aux, int dact, float dact_param, int relu_quirk, ono_stream_t stream);
int ono_finish_delta(int dtype, long long rows, int C, const float* src, int ld_src, const void* aux, int ld_aux, int dact,
                     float dact_param, int relu_quirk, void* dst, int ld_dst, void* dstT, int ld_dstT, ono_stream_t stream);

// ---------------------------------------------------------------------------------------------
// Fused gradient synchronisation over NVLink peer memory ("symmetric windows": the same buffer
// allocated on every rank, every rank holding a mapped pointer to every peer's copy).
//
// One kernel = reduce-scatter of the workers' gradients into the owner of each parameter range
// + averaging + the owner's optimizer step + all-gather of the fresh parameters to every rank
// that consumes them. It expresses the reference's three exchanges:
//   * ring all-reduce + local optimizer (worker/src/middlewares/worker_ring.rs:82-204,
//     worker/src/workers/all_reduce.rs:114-133): every rank owns 1/N of the vector ("two-shot"),
//     or every rank owns all of it and writes only to itself ("one-shot", small vectors);
//   * parameter-server push + BlockingStore/BarrierSync update + pull
//     (parameter_server/src/storage/blocking/shard.rs:56-92, synchronization/barrier.rs:41-50,
//     comms/src/clusters/parameter_server.rs:50-81): only server ranks own ranges;
//   * the switch between the two is a change of the ownership table only.
// algo 0 = P2P loads/stores, algo 1 = NVLS (multimem.ld_reduce / multimem.st through NVSwitch).
// Cross-rank waits are bounded; a timeout sets *status and the kernel returns.
// ---------------------------------------------------------------------------------------------
#define ONO_MAX_RANKS 8
#define ONO_MAX_RANGES 16
typedef struct OnoRange { long long begin, end; } OnoRange;   // element indices, begin % 4 == 0

typedef struct OnoSyncLocal {
  float* p_master;        // f32 master copy of the parameters this rank owns (indexed globally)
  float* m; float* v;     // optimizer state of the owned ranges, indexed (global index - state_off)
  long long state_off;
  const float* adam_pows; // {b1^t, b2^t}
  unsigned int* epoch;    // [nblocks] barrier epochs of this rank (device, zero-initialised)
  double* sumsq;          // optional: += sum of squares of the averaged gradient over owned ranges
  int* status;            // optional error word
  // Pre-reduction for another owner (16-bit gradient windows only, ranges cut at multiples of 8): when set, this rank
  // does not own its ranges; it sums the workers' 16-bit slabs over them in f32, in rank order, and stores the sums here
  // (an f32 vector indexed globally: this rank's own, from where a copy engine carries them to the owner, or the
  // owner's over NVLink). No optimizer, no parameter stores. The owner then finishes those ranges from its own f32
  // vector in a second launch. Halves (or better) the bytes that
  // converge on an owner when there are fewer owners than workers.
  float* fwd;
  int n_ranges;
  OnoRange ranges[ONO_MAX_RANGES];
} OnoSyncLocal;

typedef struct OnoSync {
  int nranks, rank, algo, nblocks;
  long long n;                               // vector length (elements)
  const float* g[ONO_MAX_RANKS];             // every rank's gradient window
  float* p_out_f32[ONO_MAX_RANKS];           // every rank's f32 parameter window (null = not wanted)
  void* p_out_bf16[ONO_MAX_RANKS];           // every rank's bf16 parameter window (null = not wanted)
  unsigned int* flags[ONO_MAX_RANKS];        // every rank's signal pad [nblocks][ONO_MAX_RANKS]
  const float* g_mc; float* p_mc_f32; void* p_mc_bf16;   // multicast addresses (algo 1); null = per-peer stores
  unsigned int worker_mask;                  // ranks whose gradients are summed
  unsigned int member_mask;                  // ranks taking part in the barriers
  const unsigned int* live_mask;             // optional device word overriding member_mask (shrink)
  int n_workers;                             // divisor of the average (reference: nworkers)
  int kind; float lr, mu, b1, b2, eps;       // optimizer (OnoOptim kinds)
  int divide;                                // 1: scale by 1/n_workers (0 reproduces WildStore)
  int zero_grad;                             // 1: owners zero the summed gradient ranges afterwards
  int g_dtype;                               // element type of the g windows: 0 f32, 1 bf16, 2 f16 (16-bit gradient wire:
                                             // g[q] and g_mc then address 2-byte elements with the same indices)
  unsigned long long timeout_ns;
  OnoSyncLocal loc[ONO_MAX_RANKS];           // a real launch reads loc[rank] only
} OnoSync;

int ono_sync_step(const OnoSync* s, ono_stream_t stream);
// All ranks of the struct as one cooperative launch on ONE GPU (grid.y = rank). For single-GPU tests
// of the multi-rank logic; algo must be 0.
int ono_sync_step_emulated(const OnoSync* s, ono_stream_t stream);

// Asynchronous parameter server (synchronization/non_blocking.rs:20-31 with BlockingStore or
// storage/wild/shard.rs:43-58): the calling worker applies its own gradient to the owners' masters
// over NVLink (optionally under a per-range lock) and keeps the fresh values as its pulled params.
typedef struct OnoPsAsync {
  int nranks, rank, nblocks;
  const float* g;                            // this worker's gradient (local)
  float* p_local_f32; void* p_local_bf16;    // this worker's parameter buffers (pull destination)
  float* master[ONO_MAX_RANKS];              // owners' f32 masters (peer pointers), indexed globally
  float* m[ONO_MAX_RANKS]; float* v[ONO_MAX_RANKS]; long long state_off[ONO_MAX_RANKS];
  unsigned int* locks[ONO_MAX_RANKS];        // owners' lock words [ONO_MAX_RANGES] (null = wild)
  int n_ranges[ONO_MAX_RANKS]; OnoRange ranges[ONO_MAX_RANKS][ONO_MAX_RANGES];
  int n_workers; int divide;
  int kind; float lr, mu, b1, b2, eps; const float* adam_pows;
  int* status; unsigned long long timeout_ns;
} OnoPsAsync;
int ono_ps_async_step(const OnoPsAsync* s, ono_stream_t stream);

// Ring all-reduce (reduce-scatter + all-gather, N-1 steps each, chunked like
// worker/src/middlewares/mod.rs:15-59) with the average and SGD/momentum/Adam fused into the last
// hop. `acc` is a symmetric scratch window of n floats per rank.
typedef struct OnoRing {
  int nranks, rank, nblocks;
  long long n;
  const float* g;                            // local gradient
  float* acc[ONO_MAX_RANKS];                 // every rank's accumulation window
  unsigned int* flags[ONO_MAX_RANKS];        // every rank's step flags [nblocks]
  unsigned int* epoch;                       // [nblocks] local
  float* p; float* m; float* v; const float* adam_pows; void* p_bf16;
  int kind; float lr, mu, b1, b2, eps;
  int* status; unsigned long long timeout_ns;
} OnoRing;
int ono_ring_allreduce(const OnoRing* r, ono_stream_t stream);
// All ranks of the ring as one cooperative launch on ONE GPU (grid.y = rank), every rank with its own buffers: for
// single-GPU tests of the ring protocol (the flags are the same; the launch fails cleanly if the grid is not co-resident).
typedef struct OnoRingEmu {
  int nranks, nblocks;
  long long n;
  const float* g[ONO_MAX_RANKS];
  float* acc[ONO_MAX_RANKS]; unsigned int* flags[ONO_MAX_RANKS]; unsigned int* epoch[ONO_MAX_RANKS];
  float* p[ONO_MAX_RANKS]; float* m[ONO_MAX_RANKS]; float* v[ONO_MAX_RANKS]; void* p_bf16[ONO_MAX_RANKS];
  const float* adam_pows;
  int kind; float lr, mu, b1, b2, eps;
  int* status; unsigned long long timeout_ns;
} OnoRingEmu;
int ono_ring_allreduce_emulated(const OnoRingEmu* r, ono_stream_t stream);

// Staged reduce-scatter: while backward is still running, a few SMs copy the peers' finished gradient ranges (those this
// rank owns) from their windows into local staging buffers with bulk async copies through shared memory; the fused
// optimizer kernel then reads every worker's gradient from local HBM. `ready` are this rank's flag words
// [source rank * ONO_STAGE_BUCKETS + bucket], written by ono_stage_signal on the source once its gradients of that bucket exist.
#define ONO_STAGE_BUCKETS 64
typedef struct OnoStagePull {
  int nranks, rank, nblocks, bucket;
  const float* src[ONO_MAX_RANKS];           // every rank's gradient window (null = not a worker / self)
  float* dst[ONO_MAX_RANKS];                 // local staging buffer of each source rank
  int n_ranges;
  OnoRange ranges[ONO_MAX_RANGES];           // owned ranges of this bucket (multiples of 4 elements)
  const unsigned int* ready;                 // local flag words
  const unsigned int* step;                  // device word holding the current step number
  int* status; unsigned long long timeout_ns;
} OnoStagePull;
int ono_stage_pull(const OnoStagePull* s, ono_stream_t stream);
// writes *step into flags[q][rank * ONO_STAGE_BUCKETS + bucket] of every rank q (release at system scope)
int ono_stage_signal(unsigned int* const* flags, int nranks, int rank, int bucket, const unsigned int* step, ono_stream_t stream);
int ono_stage_tick(unsigned int* step, ono_stream_t stream);
// dst[i] += src[i] with reductions that need no reply (dst may be a peer GPU's memory).
int ono_push_add(const float* src, float* dst, long long n, ono_stream_t stream);
// cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDefault, stream): a copy-engine transfer (no SM involved); dst or src may be a
// peer GPU's window. One call per copy.
int ono_copy_async(void* dst, const void* src, long long bytes, ono_stream_t stream);
// dst[i] = 16-bit float of src[i] (bf16, or f16 when f16 != 0); dst may be a peer GPU's memory (the 16-bit gradient
// wire for values that do not leave through a GEMM epilogue: bias gradients, unaligned layers, convolution kernels).
int ono_cast16(const float* src, void* dst, long long n, int f16, ono_stream_t stream);
// Flag ping-pong between two GPUs (node/src/stat_service.rs:107-152 rebuilt as a device probe).
// role 0 pings, role 1 answers; rtt_ns[rounds] is written by role 0.
int ono_pingpong(int role, unsigned int* my_flag, unsigned int* peer_flag, int rounds, unsigned int base_epoch,
                 unsigned long long* rtt_ns, int* status, ono_stream_t stream);

// ---------------------------------------------------------------------------------------------
// Gradient compression (comms/src/handles/compressor.rs, comms/src/sparse/protocol.rs), see compress.cu.
// ---------------------------------------------------------------------------------------------
// threshold = k-th smallest |x| of a seeded sample of <= 16384 elements, k = floor(sample * (1 - r)), >= min positive f16
int ono_sparse_threshold(const float* x, long long n, float r, unsigned long long seed, float* thr_out, ono_stream_t st);
// What a rank puts on the wire and what it keeps: entries with |x[i]| >= *thr are sent and zeroed in x, the rest stays as the
// residual; thr == NULL sends everything (plain 16-bit wire). The sent values (0 elsewhere) are written as f32 rounded through
// f16 to wire_f32 and / or as 16-bit values (f16, or bf16 when wire16_f16 == 0) to wire16, the buffer peers read over NVLink;
// *sent (optional) is incremented by the number of entries sent
int ono_sparse_mask(float* x, long long n, const float* thr, float* wire_f32, void* wire16, int wire16_f16, unsigned long long* sent,
                    ono_stream_t st);
// (index, f16) pairs of the selected entries in ascending index order; scratch holds ceil(n/1024) unsigned ints
int ono_sparse_compact(float* x, long long n, const float* thr, unsigned int* scratch, unsigned int* idx, void* val_f16,
                       unsigned int capacity, unsigned int* count, int zero_sent, ono_stream_t st);
int ono_sparse_lift(float* acc, long long n, const unsigned int* idx, const void* val_f16, const unsigned int* count,
                    unsigned int capacity, ono_stream_t st);
// One sender's contribution to the range [begin, end) an owner holds: the pairs of the sender's ascending (index, f16) list that
// fall into the range (found by binary search, so only those cross NVLink), or, if the sender's selection did not fit its list
// (*count > capacity), that range of its dense 16-bit wire. acc is local; the other pointers may be the sender's window.
// *bytes (optional) += the bytes read from the sender.
int ono_sparse_lift_range(float* acc, long long begin, long long end, const unsigned int* idx, const void* val_f16,
                          const unsigned int* count, unsigned int capacity, const void* dense16, int dense_f16,
                          unsigned long long* bytes, ono_stream_t st);

#ifdef __cplusplus
}
#endif
