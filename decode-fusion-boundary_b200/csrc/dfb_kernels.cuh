// Device code of the Qwen3 decode step for sm_100a.
//
// Two kernel families:
//   * stream_gemv_kernel<LOADS, DEPTH, MODE>: a weight-streaming skinny GEMM
//     out[rows<=8, N] = x[rows, K] @ W[N, K]^T with a fused prologue (residual
//     add + RMSNorm, or the embedding gather) and a fused epilogue (bf16 store,
//     SwiGLU, or bf16-rounded logits + greedy argmax).
//   * paged_attention_kernel: q/k RMSNorm + RoPE + KV-cache write + split-KV
//     paged GQA decode attention with an in-kernel merge of the splits.
//
// Every kernel is an ordinary (non-cooperative) launch.  Inside a step they are
// chained with programmatic dependent launch: each kernel first lets its
// successor start (griddepcontrol.launch_dependents), issues the loads that do
// not depend on its predecessor (its weights / the old KV entries), and only
// then waits for the predecessor (griddepcontrol.wait).  No kernel spins on a
// flag: the two cross-CTA reductions use the "last CTA to arrive finishes the
// job" pattern (one atomic ticket per CTA), so there is no unbounded wait.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace dfb {

constexpr int kMaxRows = 8;
constexpr int kMaxRanks = 8;          // tensor-parallel ranks
constexpr int kTileRows = 8;          // weight rows per tile = N of mma.m16n8k16
constexpr int kAttnThreads = 128;
constexpr int kAttnChunk = 64;        // context positions per attention CTA
constexpr int kHeadDim = 128;
constexpr int kMaxSplits = 32;        // 2048 / kAttnChunk

enum GemvMode : int {
  kModeStore = 0,      // plain x, bf16 store            (o_proj, down_proj)
  kModeNormStore = 1,  // add+RMSNorm prologue, bf16 store (qkv_proj)
  kModeNormSwiglu = 2, // add+RMSNorm prologue, SwiGLU epilogue (gate_up_proj)
  kModeNormArgmax = 3, // add+RMSNorm prologue, logits + argmax (lm_head)
};

struct __align__(8) ArgmaxPart {
  float value;
  int index;
};

struct GemvArgs {
  const __nv_bfloat16* w;        // [N, K] row-major
  int n_tiles;                   // tiles of 8 output rows (SwiGLU: 4 gate + 4 up rows)
  int rows;                      // batch rows, 1..8
  int k;                         // K (= LOADS * 256)
  // prologue
  const __nv_bfloat16* x;        // [rows, K] input (norm modes: hidden state or embedding table)
  const int* ids;                // norm modes: if non-null, x row r = x[ids[r]]
  const __nv_bfloat16* res_in;   // norm modes: residual or null
  __nv_bfloat16* res_out;        // norm modes: new residual or null
  const __nv_bfloat16* norm_w;   // [K]
  float eps;
  // epilogue
  __nv_bfloat16* out;            // [rows, out_stride]
  int out_stride;
  int gate_rows;                 // SwiGLU: intermediate size (up rows start here)
  float* logits_out;             // argmax: optional [rows, vocab] fp32
  int vocab;
  ArgmaxPart* parts;             // argmax: [gridDim.x, 8]
  unsigned int* ticket;          // argmax: arrival counter (self-resetting)
  int* tokens;                   // argmax: [rows] result (feedback buffer)
  int* tokens_out;               // argmax: optional second copy
  ArgmaxPart* best_out;          // argmax: optional [rows] (value, index) of the winner (tensor-parallel merge)
  unsigned long long* trace;     // optional timeline slot of this launch (8 words) or null
  int* status;                   // [4] device status word or null
  int late_trigger;              // 1: let the successor start only after this kernel has read its inputs
  int bulk_x;                    // 1: FP32 kernels fetch x and the residual of the fused norm with bulk copies
  // tensor-parallel exchange fused into this kernel (dfb_exchange.cuh); 0 = none
  int tp_mode;                   // 1: push the [rows, 1024] result into every peer's window as tagged words
                                 // 2: the fused norm adds the peers' partial results found in this rank's window
  int tp_size, tp_rank, tp_slot; // ranks, this rank, index of the exchange in the step
  const unsigned int* tp_step;   // device step counter behind the tags
  unsigned char* tp_window[kMaxRanks];   // every rank's window as mapped here
  unsigned long long tp_wait_ns; // how long a pull waits for a peer before it records kStatusPeerTimeout
  // look-ahead: weights of a kernel further down the chain, requested into L2 (no registers, no
  // shared memory, nothing waits for them) so that the kernel that needs them finds them on chip
  const void* ahead_ptr;
  unsigned long long ahead_bytes;  // multiple of 16; 0 = none
  int ahead_late;                // 1: issue the request after this kernel's own work, 0: before its dependency wait
  int embed_rows;                // rows of the embedding table behind `ids` (ids are clamped into it)
  // sampling (argmax mode): rows with temps[r] > 1e-10 pick argmax(logit / T + Gumbel noise), i.e. a draw from
  // softmax(logits / T); the others stay greedy
  const float* temps;            // [rows] device, or null = every row greedy
  unsigned int* sample_ctr;      // device counter of sampled LM-head launches: the noise stream's step index
  unsigned long long sample_seed;
  int sample_idx_offset;         // first vocabulary row of this rank's shard (noise is a function of the global index)
};

// ---------------------------------------------------------------------------
// small helpers
// ---------------------------------------------------------------------------
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Streaming 128-bit weight load: read-only path, no L1 allocation.
__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
// Coherent 128-bit load served from L2: for data written by the previous kernel.
__device__ __forceinline__ uint4 ldg_cg(const void* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ float bf_lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf_hi(uint32_t u) { return __uint_as_float(u & 0xffff0000u); }
__device__ __forceinline__ float round_bf16(float f) { return __bfloat162float(__float2bfloat16_rn(f)); }
// a * b - c * d and a * b + c * d with every product and the sum rounded to fp32 on its own, as the elementwise
// torch expressions of the reference's rotary embedding do (layers/rotary_embedding.py:6-16); a fused
// multiply-add here moves results near zero by one bf16 step
__device__ __forceinline__ float mul_sub_unfused(float a, float b, float c, float d) {
  return __fsub_rn(__fmul_rn(a, b), __fmul_rn(c, d));
}
__device__ __forceinline__ float mul_add_unfused(float a, float b, float c, float d) {
  return __fadd_rn(__fmul_rn(a, b), __fmul_rn(c, d));
}

// ---------------------------------------------------------------------------
// Sampling fused after the LM head (layers/sampler.py:7-16 of the reference:
// argmax(softmax(logits / T) / E) with E ~ Exp(1), clamped at 1e-10).  Since the
// softmax's normalisation is one positive factor per row, the same draw is
// argmax(logit / T - log E): no softmax pass, no second look at the logits.
// E comes from a counter-based generator, a function of (seed, step, row, global
// vocabulary index) only, so that every CTA, every kernel variant and every
// tensor-parallel rank sees the same noise: the splitmix64 finaliser over
// seed + counter * 0x9E3779B97F4A7C15, its top 23 bits as a uniform in (0, 1).
// ---------------------------------------------------------------------------
struct SampleRow {
  float temp;       // <= 1e-10: greedy
  unsigned step;
};
// The per-row state lives in shared memory and the key function is not inlined, so that the greedy path of
// the LM-head kernels keeps its registers: a step that samples nothing pays one uniform branch per logit.
__device__ __forceinline__ void sample_rows_load(const GemvArgs& a, SampleRow* rows_smem, int tid) {
  if (a.temps && tid < kMaxRows) {
    SampleRow s{0.f, 0u};
    if (tid < a.rows) {
      s.temp = a.temps[tid];
      if (s.temp > 1e-10f) s.step = *(volatile unsigned int*)a.sample_ctr;
    }
    rows_smem[tid] = s;
  }
}
__device__ __noinline__ float sample_key(unsigned long long seed, int idx_offset, const SampleRow* rows_smem, int row,
                                         int idx, float logit) {
  const SampleRow s = rows_smem[row];
  if (!(s.temp > 1e-10f)) return logit;
  const unsigned long long ctr =
      ((unsigned long long)(s.step * 8u + (unsigned)row) << 32) | (unsigned)(idx + idx_offset);
  unsigned long long z = seed + ctr * 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  z ^= z >> 31;
  const float u = ((float)(unsigned)(z >> 41) + 0.5f) * 1.1920928955078125e-07f;   // 2^-23: u in (0, 1)
  const float e = fmaxf(-logf(u), 1e-10f);
  return __fdiv_rn(logit, s.temp) - logf(e);
}
// called by the one thread that publishes the step's tokens
__device__ __forceinline__ void sample_advance(const GemvArgs& a) {
  if (a.temps) *a.sample_ctr += 1u;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
  f[0] = bf_lo(v.x); f[1] = bf_hi(v.x); f[2] = bf_lo(v.y); f[3] = bf_hi(v.y);
  f[4] = bf_lo(v.z); f[5] = bf_hi(v.z); f[6] = bf_lo(v.w); f[7] = bf_hi(v.w);
}
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
  // A rows 8..15 (a1, a3) are always zero: the batch has at most 8 rows.
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
}

// The full m16n8k16 (all 16 rows of A in use).
__device__ __forceinline__ void mma_bf16_16816_full(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                    uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Asks the memory system to bring [p, p + bytes) into L2 (bulk prefetch: no
// destination, nothing to wait for).  p 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void l2_prefetch(const void* p, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}
// The whole grid covers [base, base + bytes) in 4 KB pieces; called by warp 0 of every CTA.
__device__ __forceinline__ void l2_prefetch_slice(const void* base, unsigned long long bytes, int cta, int ctas) {
  if (base == nullptr || bytes == 0) return;
  constexpr unsigned long long kPiece = 4096;
  const unsigned long long pieces = (bytes + kPiece - 1) / kPiece;
  const unsigned char* b = static_cast<const unsigned char*>(base);
  for (unsigned long long c = (unsigned long long)cta * 32 + (threadIdx.x & 31); c < pieces;
       c += (unsigned long long)ctas * 32) {
    const unsigned long long off = c * kPiece;
    const unsigned long long left = bytes - off;
    l2_prefetch(b + off, (uint32_t)(left < kPiece ? left : kPiece));
  }
}

// Optional timeline: per kernel {earliest CTA start, latest return from the
// dependency wait, latest CTA end, earliest wait return} in globaltimer ns.
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void trace_min(unsigned long long* slot, int i) {
  if (slot) atomicMin(slot + i, global_ns());
}
__device__ __forceinline__ void trace_max(unsigned long long* slot, int i) {
  if (slot) atomicMax(slot + i, global_ns());
}

// Device-side error reporting: the first error of a step wins; the kernel goes
// on with a safe substitute value and the host reads the word after the step.
constexpr int kStatusBadPosition = 1;
constexpr int kStatusBadBlock = 2;
constexpr int kStatusBadToken = 5;       // a token id outside the embedding table (clamped, never dereferenced)
constexpr int kStatusBadGrid = 6;        // the attention grid has fewer splits than a row's context needs
constexpr int kKernelAttention = 2;
constexpr int kKernelStage = 4;
__device__ __forceinline__ void report_status(int* status, int code, int kernel, int index, int value) {
  if (status && atomicCAS(status, 0, code) == 0) {
    status[1] = kernel;
    status[2] = index;
    status[3] = value;
  }
}

// A token id as an embedding row: ids outside [0, embed_rows) are recorded and
// replaced by row 0 (embed_rows <= 0: the caller vouches for the ids).
constexpr int kKernelGemvIds = 5;
__device__ __forceinline__ int clamp_token(int id, int embed_rows, int* status, int row) {
  if (embed_rows > 0 && (id < 0 || id >= embed_rows)) {
    report_status(status, kStatusBadToken, kKernelGemvIds, row, id);
    return 0;
  }
  return id;
}

// ---------------------------------------------------------------------------
// mbarrier + bulk-copy (TMA, untiled) helpers
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// global -> shared bulk copy; 16-byte aligned addresses, size a multiple of 16
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait: gives up after kMbarSpinLimit polls (each poll may itself block
// for a short hardware-defined time) and lets the caller report the failure.
constexpr int kMbarSpinLimit = 400000;
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
  for (int i = 0; i < kMbarSpinLimit; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}
constexpr int kStatusCopyTimeout = 3;
constexpr int kKernelGemv = 1;

// ---------------------------------------------------------------------------
// Weight-streaming skinny GEMM, weights staged through shared memory by TMA.
//
// One tile = 8 weight rows x K.  A CTA owns tiles blockIdx.x, +gridDim.x, ...
// Each tile is fetched by 8 bulk copies (one per row) into a shared-memory stage
// whose rows are padded by 64 bytes, which makes the fragment reads below free
// of bank conflicts.  The first STAGES tiles are requested BEFORE the dependency
// wait: the copies run in the async proxy, so they neither hold registers nor
// queue in front of the latency-critical activation loads that follow the wait.
//
// The WARPS warps split K: warp w owns columns [w*K/WARPS, (w+1)*K/WARPS) =
// LOADS blocks of 32.  In block j, lane (g = lane/4, t = lane%4) reads the 16
// bytes W[row g][32j + 8t .. +7] from the stage and holds the matching 16 bytes
// of x[batch g] in registers; word pairs (0,1) and (2,3) feed two m16n8k16 MMAs
// with the batch on M and the weight rows on N.  The k order inside an MMA is a
// fixed permutation applied to both operands, which a dot product ignores.
// ---------------------------------------------------------------------------
template <int LOADS, int WARPS>
struct GemvSmem {
  static constexpr int kK = LOADS * 32 * WARPS;
  static constexpr int kRowStride = 2 * kK + 64;      // bytes
  static constexpr int kStageBytes = kTileRows * kRowStride;
  static constexpr int bytes(int stages) { return stages * kStageBytes + 8 * stages + 16; }
};

template <int LOADS, int WARPS, int STAGES, int MODE>
__global__ void __launch_bounds__(WARPS * 32, LOADS <= 4 ? 3 : 2)
stream_gemv_kernel(const GemvArgs a) {
  constexpr bool kNorm = MODE != kModeStore;
  constexpr int kWarps = WARPS;
  using SM = GemvSmem<LOADS, WARPS>;
  constexpr int K = SM::kK;
  if (!a.late_trigger) pdl_launch_dependents();
  if (threadIdx.x == 0) trace_min(a.trace, 0);

  extern __shared__ __align__(128) unsigned char dyn_smem[];
  unsigned char* stage_base = dyn_smem;
  uint64_t* full = reinterpret_cast<uint64_t*>(dyn_smem + STAGES * SM::kStageBytes);
  __shared__ float red[2][kWarps][64];
  __shared__ float ssq[kWarps][kMaxRows];
  __shared__ int last_flag;

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int kbase = warp * (LOADS * 32) + 8 * t;  // this lane's first column
  const int stride = gridDim.x;

  // row `r` of tile `tile` in global memory
  auto weight_row = [&](int tile, int r) -> const __nv_bfloat16* {
    int row;
    if (MODE == kModeNormSwiglu) row = ((r & 1) ? a.gate_rows : 0) + tile * 4 + (r >> 1);
    else row = tile * kTileRows + r;
    return a.w + (size_t)row * K;
  };
  // warp 0: request tile `tile` into stage `s`
  auto request_tile = [&](int tile, int s) {
    if (lane == 0) mbar_expect_tx(&full[s], kTileRows * 2 * K);
    __syncwarp();
    if (lane < kTileRows)
      bulk_g2s(stage_base + s * SM::kStageBytes + lane * SM::kRowStride, weight_row(tile, lane), 2 * K, &full[s]);
  };

  // ---- weight prefetch, independent of the previous kernel ----
  if (warp == 0) {
    if (lane == 0) {
#pragma unroll
      for (int s = 0; s < STAGES; ++s) mbar_init(&full[s], 1);
      fence_mbar_init();
    }
    __syncwarp();
#pragma unroll
    for (int s = 0; s < STAGES; ++s) {
      const int tl = blockIdx.x + s * stride;
      if (tl < a.n_tiles) request_tile(tl, s);
    }
  }
  uint4 nw[kNorm ? LOADS : 1];
  if (kNorm) {
#pragma unroll
    for (int j = 0; j < LOADS; ++j) nw[j] = ldg_stream(a.norm_w + kbase + 32 * j);
  }
  if (warp == 1) l2_prefetch_slice(a.ahead_ptr, a.ahead_bytes, blockIdx.x, gridDim.x);
  __syncthreads();  // the barriers are initialised before anyone polls them

  pdl_wait();
  if (threadIdx.x == 0) { trace_max(a.trace, 1); trace_min(a.trace, 3); }

  // ---- prologue: this lane's fragments of x[batch g] ----
  uint4 xa[LOADS];
  const bool live = g < a.rows;
  if (!kNorm) {
#pragma unroll
    for (int j = 0; j < LOADS; ++j)
      xa[j] = live ? ldg_cg(a.x + (size_t)g * K + kbase + 32 * j) : make_uint4(0, 0, 0, 0);
  } else {
    float xs[LOADS][8];
    float ss = 0.f;
    if (live) {
      const size_t xrow = a.ids ? (size_t)clamp_token(a.ids[g], a.embed_rows, a.status, g) : (size_t)g;
      uint4 hv[LOADS], rv[LOADS];
#pragma unroll
      for (int j = 0; j < LOADS; ++j) {
        hv[j] = ldg_cg(a.x + xrow * K + kbase + 32 * j);
        rv[j] = a.res_in ? ldg_cg(a.res_in + (size_t)g * K + kbase + 32 * j) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int j = 0; j < LOADS; ++j) {
        float hf[8], rf[8];
        unpack8(hv[j], hf);
        unpack8(rv[j], rf);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          xs[j][e] = hf[e] + rf[e];
          ss += xs[j][e] * xs[j][e];
        }
        if (a.res_out && blockIdx.x == 0) {
          uint4 o;
          o.x = pack_bf16(xs[j][0], xs[j][1]); o.y = pack_bf16(xs[j][2], xs[j][3]);
          o.z = pack_bf16(xs[j][4], xs[j][5]); o.w = pack_bf16(xs[j][6], xs[j][7]);
          *reinterpret_cast<uint4*>(a.res_out + (size_t)g * K + kbase + 32 * j) = o;
        }
      }
    }
    ss += __shfl_xor_sync(0xffffffffu, ss, 1);
    ss += __shfl_xor_sync(0xffffffffu, ss, 2);
    if (t == 0) ssq[warp][g] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) tot += ssq[w][g];
    const float rstd = 1.0f / sqrtf(tot / (float)K + a.eps);
#pragma unroll
    for (int j = 0; j < LOADS; ++j) {
      float wf[8], y[8];
      unpack8(nw[j], wf);
#pragma unroll
      for (int e = 0; e < 8; ++e) y[e] = live ? round_bf16(xs[j][e] * rstd) * wf[e] : 0.f;
      xa[j].x = pack_bf16(y[0], y[1]); xa[j].y = pack_bf16(y[2], y[3]);
      xa[j].z = pack_bf16(y[4], y[5]); xa[j].w = pack_bf16(y[6], y[7]);
    }
  }

  if (a.late_trigger) pdl_launch_dependents();
  if (threadIdx.x == 0) trace_max(a.trace, 4);
  // ---- main loop over this CTA's tiles ----
  const int eb = tid >> 3, er = tid & 7;  // epilogue thread -> (batch row, tile row)
  float best_v = -INFINITY;
  int best_i = 0x7fffffff;
  __shared__ SampleRow srows[kMaxRows];
  if (MODE == kModeNormArgmax) sample_rows_load(a, srows, tid);   // a CTA barrier follows before the first epilogue
  int it = 0;
  bool copy_ok = true;
  for (int tile = blockIdx.x; tile < a.n_tiles; tile += stride, ++it) {
    const int s = it % STAGES;
    if (!mbar_wait_bounded(&full[s], (it / STAGES) & 1)) { copy_ok = false; break; }
    const unsigned char* wrow = stage_base + s * SM::kStageBytes + g * SM::kRowStride + 2 * kbase;
    float c[4][4];
#pragma unroll
    for (int q = 0; q < 4; ++q) { c[q][0] = 0.f; c[q][1] = 0.f; c[q][2] = 0.f; c[q][3] = 0.f; }
#pragma unroll
    for (int j = 0; j < LOADS; ++j) {
      const uint4 wv = *reinterpret_cast<const uint4*>(wrow + 64 * j);
      mma_bf16_16816(c[(2 * j) & 3], xa[j].x, xa[j].y, wv.x, wv.y);
      mma_bf16_16816(c[(2 * j + 1) & 3], xa[j].z, xa[j].w, wv.z, wv.w);
    }
    if (threadIdx.x == 0 && it == 0) trace_max(a.trace, 5);
    float* r = red[it & 1][warp];
    *reinterpret_cast<float2*>(r + 2 * lane) =
        make_float2((c[0][0] + c[1][0]) + (c[2][0] + c[3][0]), (c[0][1] + c[1][1]) + (c[2][1] + c[3][1]));
    __syncthreads();  // every warp is done with stage s
    if (warp == 0) {
      const int nxt = tile + STAGES * stride;
      if (nxt < a.n_tiles) request_tile(nxt, s);
    }
    if (tid < 64) {
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < kWarps; ++w) v += red[it & 1][w][tid];
      v = round_bf16(v);
      if (MODE == kModeStore || MODE == kModeNormStore) {
        if (eb < a.rows) a.out[(size_t)eb * a.out_stride + tile * kTileRows + er] = __float2bfloat16_rn(v);
      } else if (MODE == kModeNormSwiglu) {
        const float up = __shfl_xor_sync(0xffffffffu, v, 1);
        if (!(er & 1) && eb < a.rows) {
          const float act = v / (1.0f + expf(-v)) * up;
          a.out[(size_t)eb * a.out_stride + tile * 4 + (er >> 1)] = __float2bfloat16_rn(act);
        }
      } else {
        const int idx = tile * kTileRows + er;
        if (eb < a.rows) {
          if (a.logits_out) a.logits_out[(size_t)eb * a.vocab + idx] = v;
          const float key = a.temps ? sample_key(a.sample_seed, a.sample_idx_offset, srows, eb, idx, v) : v;
          if (key > best_v || (key == best_v && idx < best_i)) { best_v = key; best_i = idx; }
        }
      }
    }
    if (threadIdx.x == 0 && it == 0) trace_max(a.trace, 6);
  }
  if (!copy_ok) {
    // A bulk copy never completed: record it, give the copies in flight one more
    // bounded chance to land, and leave without touching the outputs further.
    report_status(a.status, kStatusCopyTimeout, kKernelGemv, blockIdx.x, it);
#pragma unroll 1
    for (int s = 0; s < STAGES; ++s) mbar_wait_bounded(&full[s], 0);
  }

  if (MODE == kModeNormArgmax) {
    // reduce over the 8 tile-row threads of each batch row, then over CTAs
    if (tid < 64) {
#pragma unroll
      for (int m = 1; m < 8; m <<= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best_v, m);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, m);
        if (ov > best_v || (ov == best_v && oi < best_i)) { best_v = ov; best_i = oi; }
      }
      if (er == 0) a.parts[blockIdx.x * kMaxRows + eb] = ArgmaxPart{best_v, best_i};
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) last_flag = (atomicAdd(a.ticket, 1u) == gridDim.x - 1) ? 1 : 0;
    __syncthreads();
    if (last_flag) {
      __threadfence();
      for (int b = warp; b < a.rows; b += kWarps) {  // one warp per batch row
        float v = -INFINITY;
        int i = 0x7fffffff;
        for (int c2 = lane; c2 < (int)gridDim.x; c2 += 32) {
          const int2 raw = __ldcg(reinterpret_cast<const int2*>(a.parts + c2 * kMaxRows + b));
          const ArgmaxPart p{__int_as_float(raw.x), raw.y};
          if (p.value > v || (p.value == v && p.index < i)) { v = p.value; i = p.index; }
        }
#pragma unroll
        for (int m = 16; m >= 1; m >>= 1) {
          const float ov = __shfl_xor_sync(0xffffffffu, v, m);
          const int oi = __shfl_xor_sync(0xffffffffu, i, m);
          if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
        }
        if (lane == 0) {
          a.tokens[b] = i;
          if (a.tokens_out) a.tokens_out[b] = i;
          if (a.best_out) a.best_out[b] = ArgmaxPart{v, i};
        }
      }
      if (tid == 0) { *a.ticket = 0u; sample_advance(a); }
    }
  }
  if (threadIdx.x == 0) trace_max(a.trace, 2);
}

// ---------------------------------------------------------------------------
// Paged GQA decode attention with fused q/k RMSNorm + RoPE + KV-cache write.
// grid = (splits, kv_heads, rows), 128 threads.  CTA (s, h, r) covers context
// positions [64 s, 64 s + 64) of row r for KV head h and its two query heads.
// ---------------------------------------------------------------------------
struct AttnArgs {
  const __nv_bfloat16* qkv;     // [rows, qkv_stride]: q | k | v of the new token (pre-norm)
  int qkv_stride;
  int q_size, kv_size;          // 2048, 1024
  const int* positions;         // [rows]
  const int* block_tables;      // [rows, bt_stride]
  int bt_stride;
  int bt_cols;                  // valid columns of a row of block_tables (0 = not known)
  const int* row_active;        // [rows] or null
  const __nv_bfloat16* q_norm;  // [128]
  const __nv_bfloat16* k_norm;  // [128]
  const float* cos_sin;         // [max_pos, 128]
  float eps;
  float scale;
  __nv_bfloat16* k_cache;       // this layer: [blocks, block_size, kv_heads, 128]
  __nv_bfloat16* v_cache;
  int block_size;
  int kv_heads;
  int num_blocks;
  int max_pos;
  int* status;                  // [4]: code, kernel id, index, observed value
  __nv_bfloat16* out;           // [rows, q_size]
  float* part_o;                // [rows, kv_heads, kMaxSplits, 2, 128]
  float2* part_ml;              // [rows, kv_heads, kMaxSplits, 2] (max, sum)
  unsigned int* tickets;        // [rows, kv_heads]
  unsigned long long* trace;    // optional timeline slot of this launch or null
  int late_trigger;             // 1: let the successor start only after this kernel has read its inputs
  const void* ahead_ptr;        // look-ahead prefetch into L2 (see GemvArgs)
  unsigned long long ahead_bytes;
};

// CHAIN only separates instantiations: a function's preferred shared-memory split is
// a property of the function, and the two kernel chains prefer different ones.
// Thread-block cluster helpers for the cluster variant of the attention kernel: the CTAs of one (row, KV head)
// form a cluster along x and merge their partial results through distributed shared memory.
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float ld_dsmem_f32(const float* local, unsigned cta_rank) {
  unsigned la = (unsigned)__cvta_generic_to_shared(local), ra;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(la), "r"(cta_rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(ra) : "memory");
  return v;
}
__device__ __forceinline__ float2 ld_dsmem_f32x2(const float2* local, unsigned cta_rank) {
  unsigned la = (unsigned)__cvta_generic_to_shared(local), ra;
  float2 v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(la), "r"(cta_rank));
  asm volatile("ld.shared::cluster.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(ra) : "memory");
  return v;
}
constexpr int kAttnClusterMax = 16;   // chunks of one (row, KV head) that one cluster can merge

// CLUSTER: the grid's x dimension is one thread-block cluster (2..16 CTAs, launched with that cluster
// dimension).  The chunks' partial results then stay in shared memory: one cluster barrier, CTA 0 reads its
// peers' partials through distributed shared memory and writes the row, a second barrier keeps the peers'
// shared memory alive until it has.  No global partials, no fence, no ticket.  Every CTA of a cluster whose
// row has more than one chunk passes both barriers, also those without a chunk; a row with a single chunk
// uses neither (all CTAs of a cluster see the same row, hence the same count).
// CHUNK: positions per CTA, 64 or (256 threads only) 128: short contexts of small batches then need no split at
// all up to 128 tokens, and half as many partial results beyond.
template <int THREADS, int CHAIN, bool CLUSTER = false, int CHUNK = kAttnChunk>
__global__ void __launch_bounds__(THREADS) paged_attention_kernel(const AttnArgs a) {
  constexpr int PG = THREADS / 16;           // position groups: 16 threads share one position
  constexpr int ITER = CHUNK / PG;      // positions per thread
  constexpr int J = 2 * kHeadDim / THREADS;  // output elements per thread in the reduction and the merge
  static_assert(THREADS == 128 || THREADS == 256, "128 or 256 threads");
  static_assert(CHUNK == kAttnChunk || (CHUNK == 2 * kAttnChunk && THREADS == 256), "64 positions, or 128 with 256 threads");
  if (!a.late_trigger) pdl_launch_dependents();
  const int split = blockIdx.x, kvh = blockIdx.y, row = blockIdx.z;
  const int tid = threadIdx.x;
  if (tid == 0) { trace_min(a.trace, 0); trace_max(a.trace, 4); }
  int pos = a.positions[row];
  bool write_ok = true;   // false once any input of this row had to be replaced: its KV slot is then left alone
  if (pos < 0 || pos >= a.max_pos) {
    // A position outside the RoPE table / block table: record it and carry on
    // with a clamped value so that no address is formed from it.
    report_status(a.status, kStatusBadPosition, kKernelAttention, row, pos);
    pos = pos < 0 ? 0 : a.max_pos - 1;
    write_ok = false;
  }
  if (tid < 32)
    l2_prefetch_slice(a.ahead_ptr, a.ahead_bytes, (int)((blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x),
                      (int)(gridDim.x * gridDim.y * gridDim.z));
  int ctx = pos + 1;
  int nsplits = (ctx + CHUNK - 1) / CHUNK;
  if (nsplits > (int)gridDim.x) {
    // The host sized the grid from a context bound smaller than this row's position: the chunk holding
    // the new token has no CTA.  Record it and attend to what the grid covers, so that the tickets
    // still balance and nothing is written outside the covered range.
    if (split == 0) report_status(a.status, kStatusBadGrid, kKernelAttention, row, pos);
    nsplits = (int)gridDim.x;
    ctx = nsplits * CHUNK;
    pos = ctx - 1;
    write_ok = false;
  }
  if (split >= nsplits) {  // split 0 always stays and orders the grid after its predecessor
    if (CLUSTER && nsplits > 1) {
      cluster_sync_all();
      cluster_sync_all();
    }
    return;
  }

  __shared__ float qs[2][kHeadDim];
  __shared__ __align__(16) float cpo[CLUSTER ? 2 * kHeadDim : 4];   // cluster variant: this chunk's partial output
  __shared__ float2 cml[2];                                         // ... and its (max, sum) per head
  __shared__ __align__(16) __nv_bfloat16 ks[kHeadDim];
  __shared__ __align__(16) __nv_bfloat16 vs[kHeadDim];
  __shared__ float mred[PG][2];
  __shared__ float lred[PG / 2][2];            // per warp: its two position groups are added by shuffle
  __shared__ __align__(16) float ored[PG / 2][2][kHeadDim];
  __shared__ int last_flag;

  const int start = split * CHUNK;
  const int end = min(ctx, start + CHUNK);
  const bool owner = split == nsplits - 1;  // the chunk holding the new token
  const int pg = tid >> 4, l16 = tid & 15;  // position group, 16-byte slice of the head
  int bt_col = start / a.block_size;
  if (a.bt_cols > 0 && bt_col >= a.bt_cols) {
    // the position lies beyond the columns the caller filled in: never read a stale table entry
    report_status(a.status, kStatusBadBlock, kKernelAttention, row, -1 - bt_col);
    bt_col = a.bt_cols - 1;
    write_ok = false;
  }
  int block = a.block_tables[row * a.bt_stride + bt_col];
  if (block < 0 || block >= a.num_blocks) {
    report_status(a.status, kStatusBadBlock, kKernelAttention, row, block);
    block = 0;
    write_ok = false;
  }
  const size_t tok_stride = (size_t)a.kv_heads * kHeadDim;
  const size_t base = ((size_t)block * a.block_size + (start % a.block_size)) * tok_stride + (size_t)kvh * kHeadDim + 8 * l16;

  // ---- old KV entries: independent of the previous kernel ----
  // Iteration i covers positions start + PG i .. start + PG i + PG - 1; when
  // none of them exists the whole CTA skips the iteration.
  uint4 kreg[ITER], vreg[ITER];
#pragma unroll
  for (int i = 0; i < ITER; ++i) {
    const int p = start + pg + PG * i;
    if (start + PG * i < end && p < end && p != pos) {
      kreg[i] = ldg_stream(a.k_cache + base + (size_t)(pg + PG * i) * tok_stride);
      vreg[i] = ldg_stream(a.v_cache + base + (size_t)(pg + PG * i) * tok_stride);
    } else {
      kreg[i] = make_uint4(0, 0, 0, 0);
      vreg[i] = make_uint4(0, 0, 0, 0);
    }
  }

  // constants of the new token's norm and rotation: also independent of the predecessor
  const int warp = tid >> 5, lane = tid & 31;
  uint32_t wlo = 0, whi = 0;
  float2 rc = make_float2(0.f, 0.f), rs = make_float2(0.f, 0.f);
  if (warp < 3) {
    const __nv_bfloat16* nw = warp < 2 ? a.q_norm : a.k_norm;
    const float* cs = a.cos_sin + (size_t)pos * kHeadDim;
    wlo = *reinterpret_cast<const uint32_t*>(nw + 2 * lane);
    whi = *reinterpret_cast<const uint32_t*>(nw + 2 * lane + 64);
    rc = *reinterpret_cast<const float2*>(cs + 2 * lane);
    rs = *reinterpret_cast<const float2*>(cs + 64 + 2 * lane);
  }

  pdl_wait();
  if (tid == 0) { trace_max(a.trace, 1); trace_min(a.trace, 3); }

  // ---- new token: q (2 heads) and k get RMSNorm + RoPE, v is copied ----
  {
    const __nv_bfloat16* src = a.qkv + (size_t)row * a.qkv_stride;
    if (warp < 3) {
      const __nv_bfloat16* vec = warp < 2 ? src + (2 * kvh + warp) * kHeadDim : src + a.q_size + kvh * kHeadDim;
      const int d = 2 * lane;  // handles d, d+1 and their RoPE partners d+64, d+65
      const uint32_t lo = __ldcg(reinterpret_cast<const uint32_t*>(vec + d));
      const uint32_t hi = __ldcg(reinterpret_cast<const uint32_t*>(vec + d + 64));
      float x[4] = {bf_lo(lo), bf_hi(lo), bf_lo(hi), bf_hi(hi)};
      float ss = x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3];
#pragma unroll
      for (int m = 16; m >= 1; m >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, m);
      const float rstd = 1.0f / sqrtf(ss / (float)kHeadDim + a.eps);
      const float w[4] = {bf_lo(wlo), bf_hi(wlo), bf_lo(whi), bf_hi(whi)};
#pragma unroll
      for (int e = 0; e < 4; ++e) x[e] = round_bf16(round_bf16(x[e] * rstd) * w[e]);
      const float2 c = rc, s = rs;
      const float y0 = round_bf16(mul_sub_unfused(x[0], c.x, x[2], s.x)), y1 = round_bf16(mul_sub_unfused(x[1], c.y, x[3], s.y));
      const float y2 = round_bf16(mul_add_unfused(x[2], c.x, x[0], s.x)), y3 = round_bf16(mul_add_unfused(x[3], c.y, x[1], s.y));
      if (warp < 2) {
        qs[warp][d] = y0; qs[warp][d + 1] = y1; qs[warp][d + 64] = y2; qs[warp][d + 65] = y3;
      } else {
        *reinterpret_cast<uint32_t*>(ks + d) = pack_bf16(y0, y1);
        *reinterpret_cast<uint32_t*>(ks + d + 64) = pack_bf16(y2, y3);
      }
    } else if (warp == 3) {
      const __nv_bfloat16* vec = src + a.q_size + a.kv_size + kvh * kHeadDim;
      reinterpret_cast<uint2*>(vs)[lane] = __ldcg(reinterpret_cast<const uint2*>(vec) + lane);
    }
  }
  __syncthreads();
  if (a.late_trigger) pdl_launch_dependents();

  if (owner) {
    const int pi = pos - start;  // 0..63
    if ((pi % PG) == pg) {
      const int i = pi / PG;
      const uint4 kn = reinterpret_cast<const uint4*>(ks)[l16];
      const uint4 vn = reinterpret_cast<const uint4*>(vs)[l16];
#pragma unroll
      for (int u = 0; u < ITER; ++u)
        if (u == i) { kreg[u] = kn; vreg[u] = vn; }
      if (write_ok && (a.row_active == nullptr || a.row_active[row] != 0)) {
        const size_t off = base + (size_t)pi * tok_stride;
        *reinterpret_cast<uint4*>(a.k_cache + off) = kn;
        *reinterpret_cast<uint4*>(a.v_cache + off) = vn;
      }
    }
  }

  // ---- scores ----
  float q0[8], q1[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) { q0[e] = qs[0][8 * l16 + e]; q1[e] = qs[1][8 * l16 + e]; }
  float s0[ITER], s1[ITER];
  float m0 = -INFINITY, m1 = -INFINITY;
#pragma unroll
  for (int i = 0; i < ITER; ++i) {
    if (start + PG * i >= end) {   // no position of this iteration exists (same for every thread of the CTA)
      s0[i] = -INFINITY;
      s1[i] = -INFINITY;
      continue;
    }
    float kf[8];
    unpack8(kreg[i], kf);
    float d0 = 0.f, d1 = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) { d0 += kf[e] * q0[e]; d1 += kf[e] * q1[e]; }
#pragma unroll
    for (int m = 8; m >= 1; m >>= 1) {
      d0 += __shfl_xor_sync(0xffffffffu, d0, m);
      d1 += __shfl_xor_sync(0xffffffffu, d1, m);
    }
    const bool valid = start + pg + PG * i < end;
    s0[i] = valid ? d0 * a.scale : -INFINITY;
    s1[i] = valid ? d1 * a.scale : -INFINITY;
    m0 = fmaxf(m0, s0[i]);
    m1 = fmaxf(m1, s1[i]);
  }
  if (l16 == 0) { mred[pg][0] = m0; mred[pg][1] = m1; }
  __syncthreads();
  if (tid == 0) trace_max(a.trace, 5);
#pragma unroll
  for (int p = 0; p < PG; ++p) { m0 = fmaxf(m0, mred[p][0]); m1 = fmaxf(m1, mred[p][1]); }

  // ---- softmax numerators and P.V for this thread's positions ----
  constexpr float kLog2e = 1.4426950408889634f;
  float o0[8], o1[8], l0 = 0.f, l1 = 0.f;
#pragma unroll
  for (int e = 0; e < 8; ++e) { o0[e] = 0.f; o1[e] = 0.f; }
#pragma unroll
  for (int i = 0; i < ITER; ++i) {
    if (start + PG * i >= end) continue;
    const float p0 = exp2f((s0[i] - m0) * kLog2e);  // -inf -> 0
    const float p1 = exp2f((s1[i] - m1) * kLog2e);
    l0 += p0;
    l1 += p1;
    float vf[8];
    unpack8(vreg[i], vf);
#pragma unroll
    for (int e = 0; e < 8; ++e) { o0[e] += p0 * vf[e]; o1[e] += p1 * vf[e]; }
  }
  // a warp holds two position groups (lanes 0-15 and 16-31): add them here
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    o0[e] += __shfl_xor_sync(0xffffffffu, o0[e], 16);
    o1[e] += __shfl_xor_sync(0xffffffffu, o1[e], 16);
  }
  l0 += __shfl_xor_sync(0xffffffffu, l0, 16);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 16);
  if (lane < 16) {
    float4* r0 = reinterpret_cast<float4*>(&ored[warp][0][8 * l16]);
    float4* r1 = reinterpret_cast<float4*>(&ored[warp][1][8 * l16]);
    r0[0] = make_float4(o0[0], o0[1], o0[2], o0[3]);
    r0[1] = make_float4(o0[4], o0[5], o0[6], o0[7]);
    r1[0] = make_float4(o1[0], o1[1], o1[2], o1[3]);
    r1[1] = make_float4(o1[4], o1[5], o1[6], o1[7]);
    if (l16 == 0) { lred[warp][0] = l0; lred[warp][1] = l1; }
  }
  __syncthreads();

  // ---- sum over the position groups: element idx = head * 128 + dim ----
  float O[J], L[J];
#pragma unroll
  for (int j = 0; j < J; ++j) {
    const int idx = tid + j * THREADS, h = idx >> 7, d = idx & (kHeadDim - 1);
    O[j] = 0.f;
    L[j] = 0.f;
#pragma unroll
    for (int p = 0; p < PG / 2; ++p) { O[j] += ored[p][h][d]; L[j] += lred[p][h]; }
  }

  // the two query heads of this KV head are adjacent in the output row
  __nv_bfloat16* out = a.out + (size_t)row * a.q_size + (size_t)(2 * kvh) * kHeadDim;
  if (nsplits == 1) {
#pragma unroll
    for (int j = 0; j < J; ++j) out[tid + j * THREADS] = __float2bfloat16_rn(O[j] / L[j]);
    if (tid == 0) trace_max(a.trace, 2);
    return;
  }

  // ---- several splits: publish the partial, one CTA merges ----
  constexpr int MS = CLUSTER ? kAttnClusterMax : kMaxSplits;
  const size_t pidx = ((size_t)row * a.kv_heads + kvh) * kMaxSplits;
  if (CLUSTER) {
#pragma unroll
    for (int j = 0; j < J; ++j) {
      const int idx = tid + j * THREADS;
      cpo[idx] = O[j];
      if ((idx & (kHeadDim - 1)) == 0) cml[idx >> 7] = make_float2((idx >> 7) ? m1 : m0, L[j]);
    }
    cluster_sync_all();   // every chunk's partial is in its CTA's shared memory
    if (tid == 0) trace_max(a.trace, 6);
    if (split != 0) {
      cluster_sync_all(); // CTA 0 has read this CTA's partial
      if (tid == 0) trace_max(a.trace, 2);
      return;
    }
  } else {
    float* po = a.part_o + (pidx + split) * 2 * kHeadDim;
#pragma unroll
    for (int j = 0; j < J; ++j) {
      const int idx = tid + j * THREADS;
      po[idx] = O[j];
      if ((idx & (kHeadDim - 1)) == 0)  // one thread per head publishes (max, sum)
        a.part_ml[(pidx + split) * 2 + (idx >> 7)] = make_float2((idx >> 7) ? m1 : m0, L[j]);
    }
    __syncthreads();
    if (tid == 0) {
      // One acquire-release atomic at GPU scope instead of fence + atomic + fence: the release covers the whole
      // CTA's partials (they happen before it through the barrier above), the acquire the other CTAs' partials
      // that the last arrival reads below (through the barrier that follows).
      unsigned int prev;
      asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;"
                   : "=r"(prev) : "l"(a.tickets + row * a.kv_heads + kvh) : "memory");
      last_flag = prev == (unsigned)(nsplits - 1) ? 1 : 0;
      trace_max(a.trace, 6);
    }
    __syncthreads();
    if (!last_flag) {
      if (tid == 0) trace_max(a.trace, 2);
      return;
    }
  }
  // Every load of the merge is issued before anything is computed, so that the
  // merge costs one trip (to L2, or to the peers' shared memory) whatever the number of splits.
  float pv[J][MS];
  const float* ps = a.part_o + pidx * 2 * kHeadDim;
#pragma unroll
  for (int j = 0; j < J; ++j)
#pragma unroll
    for (int s = 0; s < MS; ++s) {
      if (CLUSTER) pv[j][s] = s < nsplits ? ld_dsmem_f32(&cpo[tid + j * THREADS], (unsigned)s) : 0.f;
      else pv[j][s] = s < nsplits ? __ldcg(ps + (size_t)s * 2 * kHeadDim + tid + j * THREADS) : 0.f;
    }
  // `ored` is free again (every thread passed two barriers after reading it).
  float* msm = &ored[0][0][0];        // [2 * MS] partial maxima, index 2 s + head
  float* lsm = msm + 2 * kMaxSplits;  // [2 * MS] weighted partial sums
  float* wsm = lsm + 2 * kMaxSplits;  // [2 * MS] weights
  if (tid < 2 * nsplits) {
    const float2 ml = CLUSTER ? ld_dsmem_f32x2(&cml[tid & 1], (unsigned)(tid >> 1)) : __ldcg(&a.part_ml[pidx * 2 + tid]);
    msm[tid] = ml.x;
    lsm[tid] = ml.y;
  }
  __syncthreads();
  if (tid == 0) trace_max(a.trace, 7);
  if (tid < 2 * nsplits) {
    float M = -INFINITY;
    for (int s = 0; s < nsplits; ++s) M = fmaxf(M, msm[2 * s + (tid & 1)]);
    const float w = exp2f((msm[tid] - M) * kLog2e);
    lsm[tid] = w * lsm[tid];  // only this thread touches this entry before the barrier
    wsm[tid] = w;
  }
  __syncthreads();
#pragma unroll
  for (int j = 0; j < J; ++j) {
    const int idx = tid + j * THREADS, h = idx >> 7;
    float A = 0.f, S = 0.f;
#pragma unroll
    for (int s = 0; s < MS; ++s) {
      if (s < nsplits) {
        A += wsm[2 * s + h] * pv[j][s];
        S += lsm[2 * s + h];
      }
    }
    out[idx] = __float2bfloat16_rn(A / S);
  }
  if (CLUSTER) {
    cluster_sync_all();   // the peers may leave: their partials have been read (pv, msm, lsm are local copies)
    if (tid == 0) trace_max(a.trace, 2);
  } else if (tid == 0) {
    a.tickets[row * a.kv_heads + kvh] = 0u;
    trace_max(a.trace, 2);
  }
}

// Tensor parallel: every rank holds the winners of all ranks' vocabulary shards
// ([ranks][kMaxRows] pairs with shard-local indices); the greedy token of a row
// is the largest value, the lowest global index among equals.
__global__ void merge_shard_argmax_kernel(const ArgmaxPart* all, int ranks, int rows, int shard_rows, int* tokens,
                                          int* tokens_out) {
  const int b = threadIdx.x;
  if (b >= rows) return;
  float v = -INFINITY;
  int idx = 0x7fffffff;
  for (int r = 0; r < ranks; ++r) {
    const ArgmaxPart p = all[r * kMaxRows + b];
    const int gi = p.index + r * shard_rows;
    if (p.value > v || (p.value == v && gi < idx)) { v = p.value; idx = gi; }
  }
  tokens[b] = idx;
  if (tokens_out) tokens_out[b] = idx;
}

// Copies one step's inputs into the decoder's fixed staging buffers (so a
// captured graph can read them from constant addresses), converting the
// engine's int64 ids / positions to int32.  Token ids index the embedding
// table in the first kernel of the step, so an id outside [0, embed_rows) is
// recorded in the status word and replaced by 0 here: no address is ever
// formed from it.  Without `ids` the previous step's tokens (`prev_tokens`)
// are fed back, with the same check (an all-NaN row of logits has no winner).
struct StageArgs {
  const int64_t* ids;        // null: feed back prev_tokens
  const int* prev_tokens;    // [rows] tokens of the previous step (device)
  const int64_t* positions;
  const int* block_tables;
  int bt_cols, bt_stride_in, bt_stride_out;
  const int* row_active;     // null: all active
  const float* temps;        // null: greedy step (temps_out is then left alone)
  float* temps_out;
  int rows;
  int embed_rows;
  int* ids_out;
  int* positions_out;
  int* bt_out;
  int* row_active_out;
  int* status;
};
__global__ void stage_inputs_kernel(const StageArgs a) {
  const int tid = threadIdx.x;
  if (tid < a.rows) {
    long long id = a.ids ? (long long)a.ids[tid] : (long long)a.prev_tokens[tid];
    if (id < 0 || id >= a.embed_rows) {
      report_status(a.status, kStatusBadToken, kKernelStage, tid, (int)id);
      id = 0;
    }
    a.ids_out[tid] = (int)id;
    a.positions_out[tid] = (int)a.positions[tid];
    a.row_active_out[tid] = a.row_active ? a.row_active[tid] : 1;
    if (a.temps) {
      const float t = a.temps[tid];
      a.temps_out[tid] = t >= 0.f ? t : 0.f;   // negative or NaN: greedy
    }
  }
  for (int i = tid; i < a.rows * a.bt_cols; i += blockDim.x) {
    const int r = i / a.bt_cols, c = i % a.bt_cols;
    a.bt_out[r * a.bt_stride_out + c] = a.block_tables[r * a.bt_stride_in + c];
  }
}


// Prefill side of the shared paged cache: the K / V rows of N prompt tokens go to their slots
// (layers/attention.py:10-40 of the reference, a Triton kernel there).  One token row is row_bytes of K and as
// many of V; a CTA walks tokens with stride gridDim.x, its first half copies K, its second half V, 16 bytes per
// thread and trip.  slot -1 means "no slot" (padding of a captured batch) and is skipped like there; any other
// slot outside [0, num_slots) is never turned into an address: it is skipped and recorded in `status`.
constexpr int kStatusBadSlot = 7;
constexpr int kKernelStoreKv = 8;
__global__ void __launch_bounds__(256) store_kvcache_kernel(const unsigned char* __restrict__ key, const unsigned char* __restrict__ value,
                                                            long long key_stride_bytes, long long value_stride_bytes,
                                                            unsigned char* __restrict__ k_cache, unsigned char* __restrict__ v_cache,
                                                            const int* __restrict__ slot_mapping, int n_tokens, int row_bytes,
                                                            long long num_slots, int* status) {
  const int half = threadIdx.x >> 7, t = threadIdx.x & 127;
  const unsigned char* src = half ? value : key;
  unsigned char* dst = half ? v_cache : k_cache;
  const long long src_stride = half ? value_stride_bytes : key_stride_bytes;
  // four tokens per trip: their loads are all in flight before the first store (one load per thread and trip
  // leaves too few requests in flight: 4.2 TB/s against 6.0 TB/s at 65,536 tokens)
  constexpr int U = 4;
  const int pieces = row_bytes / 16;
  for (int i0 = blockIdx.x; i0 < n_tokens; i0 += U * gridDim.x) {
    long long slot[U];
    uint4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int i = i0 + u * gridDim.x;
      slot[u] = i < n_tokens ? (long long)slot_mapping[i] : -1;
      if (slot[u] != -1 && (slot[u] < 0 || slot[u] >= num_slots)) {
        if (threadIdx.x == 0) report_status(status, kStatusBadSlot, kKernelStoreKv, i, (int)slot[u]);
        slot[u] = -1;
      }
    }
    for (int c = t; c < pieces; c += 128) {
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (slot[u] != -1)
          v[u] = ldg_stream(reinterpret_cast<const uint4*>(src + (long long)(i0 + u * gridDim.x) * src_stride) + c);
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (slot[u] != -1) reinterpret_cast<uint4*>(dst + slot[u] * row_bytes)[c] = v[u];
    }
  }
}

// Host-buffer steps without copy nodes: the packed inputs are read straight from pinned host memory into the
// staging area, and the tokens plus the status word are written straight into pinned host memory (both
// mappings are the host allocations themselves under unified addressing).  A copy node of a CUDA graph costs
// more than a one-warp kernel for these few hundred bytes.
__global__ void copy_ints_kernel(const int* __restrict__ src, int* __restrict__ dst, int n) {
  for (int i = threadIdx.x; i < n; i += blockDim.x) dst[i] = src[i];
}
// `seq` (device) counts the steps published; its new value follows the data into host_out[n], after a
// system-scope fence, so that a host thread polling that word sees complete data once it changes.
__global__ void publish_result_kernel(const int* tokens_and_status, int* host_out, int n, unsigned int* seq) {
  pdl_wait();   // launched with a programmatic dependency on the LM head: everything before it has completed
  if ((int)threadIdx.x < n) host_out[threadIdx.x] = tokens_and_status[threadIdx.x];
  __threadfence_system();
  __syncwarp();
  if (threadIdx.x == 0) {
    const unsigned int next = *seq + 1u;
    *seq = next;
    *reinterpret_cast<volatile int*>(host_out + n) = (int)next;
  }
}

// Between the steps of a burst (several decode steps enqueued at once, dfb_decode_burst_enqueue): publishes
// the step's tokens in a ring in pinned host memory that the kernel writes directly (no copy node, the host
// can read finished steps while later ones run), then turns them into the next step's inputs on the device:
// ids = tokens (clamped as in stage_inputs_kernel), positions + 1.
struct PublishArgs {
  const int* tokens;        // [rows] this step's result
  int* status;              // [4] device status word
  int* ids_out;             // staged inputs of the next step
  int* positions_out;
  int rows, embed_rows;
  unsigned int* slot;       // device: steps published so far in this burst
  int* ring;                // pinned host memory, mapped: [capacity][8] tokens
  int* ring_status;         // pinned: [4] copy of the status word
  volatile int* ring_done;  // pinned: steps whose tokens are visible to the host
};
__global__ void publish_tokens_kernel(const PublishArgs a) {
  const int tid = threadIdx.x;
  const unsigned slot = *a.slot;
  if (tid < a.rows) {
    const int tok = a.tokens[tid];
    a.ring[slot * kMaxRows + tid] = tok;
    long long id = tok;
    if (id < 0 || id >= a.embed_rows) {
      report_status(a.status, kStatusBadToken, kKernelStage, tid, tok);
      id = 0;
    }
    a.ids_out[tid] = (int)id;
    a.positions_out[tid] += 1;
  }
  __syncwarp();
  if (tid < 4) a.ring_status[tid] = a.status[tid];
  __threadfence_system();
  __syncwarp();
  if (tid == 0) {
    *a.ring_done = (int)slot + 1;
    *a.slot = slot + 1;
  }
}

}  // namespace dfb
