// Weight-streaming skinny GEMM for 3..8 batch rows on the 5th-generation tensor
// cores (tcgen05.mma, accumulators in tensor memory), K = 1024:
//   out[rows <= 8, N] = x[rows, 1024] @ W[N, 1024]^T
// with the fused prologue (residual add + RMSNorm, or the embedding gather) and
// the fused epilogues (bf16 store, SwiGLU, bf16-rounded logits + greedy argmax)
// of the other GEMV kernels.
//
// Shape of one MMA tile.  The weights are the A operand (M side), the batch is
// the B operand (N = 16).  A tile of R weight rows is laid out as an M = 2R
// operand: rows [0, R) hold W[tile rows, k-block of the FIRST half of K] and
// rows [R, 2R) hold W[the same rows, the matching k-block of the SECOND half];
// the B operand holds x[batch b, first half] in its rows 0-7 and x[b, second
// half] in rows 8-15.  The accumulator D[m][n] then carries the first-half dot
// products in its block (m < R, n < 8) and the second-half ones in (m >= R,
// n >= 8); the two off-diagonal blocks are never read.  A batch of at most 8
// would leave half of N = 16 empty anyway; this way every byte the tensor core
// reads from shared memory is a weight byte that was needed, and a tile needs
// half as many MMAs.
//
// Data movement.  One elected thread requests the weight boxes with TMA
// (cp.async.bulk.tensor.2d, 128-byte swizzle, completion on an mbarrier) into a
// ring of eight shared-memory stages = one tile; the requests of the first tile
// are issued BEFORE the dependency wait (the weights do not depend on the
// previous kernel), so for the per-layer projections, whose CTAs own one tile,
// the whole tile is on its way before the activations exist.  Four issuer warps
// (one elected thread each) take every fourth stage: 4 MMAs per stage (K = 16
// each) into the issuer's own accumulator, a commit to the stage's "empty"
// barrier and, after the issuer's last stage of the tile, to the accumulators'
// "full" barrier.  Eight prologue warps build the B operand: the rows of h and
// of the residual arrive by bulk copies (TMA), then add + RMSNorm, bf16,
// written in the swizzled K-major layout.  Four of them go on as the epilogue:
// they read the accumulators with tcgen05.ld, add the issuers' accumulators and
// the two diagonal blocks (the latter through shared memory), round once to
// bf16 and run the epilogue.  Two accumulator buffers let the MMAs of the next
// tile run under the epilogue of the current one (LM head).  There is no
// CTA-wide barrier inside the loop.
//
// Every wait is bounded: on expiry the waiting thread records status 3 in the
// decoder's status word, raises the CTA's abort flag, every role drains, the
// copies in flight are given a bounded chance to land and the tensor memory is
// released before the CTA returns.
#pragma once

#include <cuda.h>   // CUtensorMap (type only; the encoder is looked up through the runtime)

#include "dfb_exchange.cuh"
#include "dfb_kernels.cuh"

namespace dfb {

struct TcArgs {
  GemvArgs g;
  int n_rows;                       // rows of W; tiles may run past it (TMA fills with zeros, the epilogue masks)
  alignas(64) CUtensorMap wmap;     // W as [n_rows, 1024] bf16, box {64 columns, BOX rows}, 128-byte swizzle
};

constexpr int kTcIssuers = 4;       // MMA-issuing warps; each owns every kTcIssuers-th k-block and its own accumulator
constexpr int kTcProWarps = 8;      // warps building the B operand; the first four of them also run the epilogue
constexpr int kTcProThreads = 32 * kTcProWarps;
constexpr int kTcFirstPro = 1 + kTcIssuers;             // warp 0: TMA, warps 1-4: MMA, warps 5-12: prologue (5-8: epilogue)
constexpr int kTcThreads = 32 * (kTcFirstPro + kTcProWarps);
constexpr int kTcK = 1024;
constexpr int kTcKbPairs = kTcK / 128;   // stages per tile: 64 columns of each half of K
constexpr int kTcAccCols = 16 * kTcIssuers;   // tensor-memory columns of one accumulator buffer
constexpr int kKernelTcGemv = 6;

template <int MT>
struct TcSmem {
  static constexpr int kStages = kTcKbPairs;                     // the ring holds exactly one tile
  static constexpr int kStageBytes = MT * 128;
  static constexpr int kXBytes = kTcKbPairs * 2048;              // B operand: 8 x [16 rows x 128 B]
  static constexpr int kResBytes = kMaxRows * kTcK * 2;          // residual rows as fetched by the bulk copies
  static constexpr int kRedBytes = 2 * 2 * kMaxRows * (MT / 2) * 4;   // [buffer][half][batch][row] fp32
  static constexpr int kBarBytes = 8 * (2 * kStages + 6) + 64;
  static constexpr int bytes() { return 1024 + kStages * kStageBytes + kXBytes + kResBytes + kRedBytes + kBarBytes + 256; }
};

// ---- small PTX wrappers ----------------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void named_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
// Barrier over `threads` threads that also ANDs a predicate: every participant gets the same answer, so
// a decision to give up is taken by all of them or by none (a thread that left alone would strand the rest).
__device__ __forceinline__ bool named_sync_and(int id, int threads, bool mine) {
  uint32_t out;
  asm volatile(
      "{\n.reg .pred p, q;\nsetp.ne.b32 q, %1, 0;\nbar.red.and.pred p, %2, %3, q;\nselp.u32 %0, 1, 0, p;\n}"
      : "=r"(out) : "r"((uint32_t)mine), "r"(id), "r"(threads) : "memory");
  return out != 0;
}
// shared-memory matrix descriptor: K-major, 128-byte swizzle, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t tc_smem_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);   // start address
  d |= (uint64_t)1 << 16;                     // leading-dimension byte offset (not used by swizzled K-major operands)
  d |= (uint64_t)(1024 >> 4) << 32;           // stride-dimension byte offset: next 8-row group
  d |= (uint64_t)1 << 46;                     // descriptor version of this architecture
  d |= (uint64_t)2 << 61;                     // 128-byte swizzle
  return d;
}
// instruction descriptor of kind::f16: bf16 x bf16 -> fp32, both operands K-major, M x N
__device__ __forceinline__ constexpr uint32_t tc_idesc(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate));
}
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
               ::"r"(smem_u32(bar)) : "memory");
}
// 16 consecutive accumulator columns of this thread's lane (the warp reads its own 32-lane quarter)
__device__ __forceinline__ void tc_ld16(uint32_t taddr, float (&v)[16]) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr) : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// 8 consecutive accumulator columns of this thread's lane
__device__ __forceinline__ void tc_ld8(uint32_t taddr, float (&v)[8]) {
  uint32_t r[8];
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr) : "memory");
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Bounded mbarrier wait that also gives up when another role of the CTA has failed.
__device__ __forceinline__ bool tc_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  for (int i = 0; i < kMbarSpinLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 255) == 255 && *abort_flag) return false;
  }
  return false;
}

// MT = 2 x (weight rows per tile): 64 for QKV (32 rows per tile), 128 for gate/up (32 gate + 32 up rows)
// and for the LM head (64 rows per tile, persistent CTAs).
//
// Issue rate.  One thread issues a tcgen05.mma of this size (N = 16) about every 51 cycles at best,
// whatever M is, while the tensor core needs only 8-16; several issuing warps multiply the rate until the
// operand reads from shared memory (about 110 bytes per cycle) become the limit.  So the k-blocks of a
// tile are dealt to four issuer warps, each with its own accumulator, the issue loops are fully unrolled
// with the descriptors advanced by additions only, and the epilogue adds the four accumulators.
template <int MODE, int MT>
__global__ void __launch_bounds__(kTcThreads, 1) tc_gemv_kernel(const __grid_constant__ TcArgs args) {
  const GemvArgs& a = args.g;
  constexpr int R = MT / 2;
  constexpr bool kSwiglu = MODE == kModeNormSwiglu;
  constexpr int BOX = kSwiglu ? R / 2 : R;             // rows of one TMA box
  using SM = TcSmem<MT>;
  constexpr int STAGES = SM::kStages;
  static_assert(MODE != kModeStore, "the plain projections (K = 2048 / 3072) have their own kernels");
  static_assert(MT == 64 || MT == 128, "M of the MMA");
  if (!a.late_trigger) pdl_launch_dependents();
  if (threadIdx.x == 0) trace_min(a.trace, 0);

  extern __shared__ unsigned char tc_dyn_raw[];
  const uint32_t raw = smem_u32(tc_dyn_raw);
  unsigned char* dyn = tc_dyn_raw + (((raw + 1023u) & ~1023u) - raw);    // the swizzle pattern repeats every 1024 bytes
  unsigned char* stages = dyn;
  unsigned char* xs = dyn + STAGES * SM::kStageBytes;                    // h rows as fetched, then the B operand
  unsigned char* rstage = xs + SM::kXBytes;                              // residual rows as fetched
  float* red = reinterpret_cast<float*>(rstage + SM::kResBytes);         // [2][2][8][R]
  uint64_t* full = reinterpret_cast<uint64_t*>(rstage + SM::kResBytes + SM::kRedBytes);
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint64_t* x_ready = acc_empty + 2;
  uint64_t* x_in = x_ready + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(x_in + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* last_flag = const_cast<int*>(abort_flag) + 1;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_tiles = a.n_tiles, stride = gridDim.x;

  if (tid == 0) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    mbar_init(&acc_full[0], kTcIssuers); mbar_init(&acc_full[1], kTcIssuers);
    mbar_init(&acc_empty[0], 128); mbar_init(&acc_empty[1], 128);
    mbar_init(x_ready, kTcProThreads);
    mbar_init(x_in, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {   // tensor memory: two accumulator buffers of one 16-column accumulator per issuer
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(tmem_slot)), "n"(2 * kTcAccCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer: never waits for the previous kernel ----------------
    if (lane == 0) {
      const uint32_t stage0 = smem_u32(stages), full0 = smem_u32(&full[0]);
      int armed = 0, it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += stride, ++it) {
#pragma unroll
        for (int kb = 0; kb < kTcKbPairs; ++kb) {
          if (!tc_wait(&empty[kb], (it & 1) ^ 1, abort_flag)) { ok = false; break; }
          mbar_expect_tx(&full[kb], SM::kStageBytes);
          const uint32_t dst = stage0 + kb * SM::kStageBytes;
          const uint32_t bar = full0 + 8 * kb;
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            const int x = kb * 64 + half * (kTcK / 2);
            if (kSwiglu) {
              tma_load_2d(dst + (half * R) * 128, &args.wmap, x, tile * BOX, bar);                      // gate rows
              tma_load_2d(dst + (half * R + BOX) * 128, &args.wmap, x, a.gate_rows + tile * BOX, bar);  // up rows
            } else {
              tma_load_2d(dst + (half * R) * 128, &args.wmap, x, tile * R, bar);
            }
          }
          ++armed;
        }
      }
      if (!ok) {
        if (!*abort_flag) report_status(a.status, kStatusCopyTimeout, kKernelTcGemv, blockIdx.x, 1);
        *abort_flag = 1;
      }
      if (*abort_flag) {   // give the copies in flight a bounded chance to land before the CTA goes away
        for (int s = 0; s < STAGES && s < armed; ++s) mbar_wait_bounded(&full[s], 0);
      }
    }
    __syncwarp();
  } else if (warp <= kTcIssuers) {
    // ---------------- MMA issuers: issuer i takes the k-blocks i, i + 4 ----------------
    if (lane == 0) {
      const int issuer = warp - 1;
      constexpr uint32_t idesc = tc_idesc(MT, 16);
      const uint64_t a_desc = tc_smem_desc(smem_u32(stages)), b_desc = tc_smem_desc(smem_u32(xs));
      bool ok = tc_wait(x_ready, 0, abort_flag);
      tc_fence_after();
      int it = 0;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += stride, ++it) {
        const int buf = it & 1;
        if (!tc_wait(&acc_empty[buf], ((it >> 1) & 1) ^ 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * kTcAccCols + issuer * 16;
#pragma unroll
        for (int j = 0; j < kTcKbPairs / kTcIssuers; ++j) {
          const int kb = j * kTcIssuers + issuer;
          if (!tc_wait(&full[kb], it & 1, abort_flag)) { ok = false; break; }
          tc_fence_after();
          // descriptor address fields count 16-byte units: a stage is kStageBytes / 16 of them, a B tile 128,
          // one K = 16 step inside the 128-byte swizzle atom 2
          const uint64_t ad = a_desc + (uint64_t)(kb * (SM::kStageBytes / 16));
          const uint64_t bd = b_desc + (uint64_t)(kb * (2048 / 16));
#pragma unroll
          for (int k = 0; k < 4; ++k) tc_mma(d_tmem, ad + 2 * k, bd + 2 * k, idesc, (j | k) ? 1u : 0u);
          tc_commit(&empty[kb]);
        }
        if (!ok) break;
        tc_commit(&acc_full[buf]);
      }
      if (!ok) {
        if (!*abort_flag) report_status(a.status, kStatusCopyTimeout, kKernelTcGemv, blockIdx.x, 2);
        *abort_flag = 1;
      }
    }
    __syncwarp();
  } else {
    // ---------------- prologue: 8 warps, one per batch row; epilogue: the first four of them ----------------
    const int pt = tid - 32 * kTcFirstPro, pwarp = warp - kTcFirstPro;
    uint4 nw4[4];   // the norm weights of this lane's four 16-byte pieces (pieces lane, lane + 32, + 64, + 96 of a row)
#pragma unroll
    for (int c = 0; c < 4; ++c) nw4[c] = ldg_stream(a.norm_w + 8 * (32 * c + lane));
    // The rows of h and of the residual come in by bulk copies (TMA): ordinary loads issued here would
    // queue in the load/store unit behind the loads of the successor kernel that was let in early.
    const bool bulk_x = a.ids == nullptr && a.res_in != nullptr;
    if (bulk_x && pt == 0) mbar_expect_tx(x_in, (uint32_t)(a.rows * 2 * kTcK * 2));
    named_sync(1, kTcProThreads);      // the byte count is posted before any copy can complete
    pdl_wait();
    if (pt == 0) { trace_max(a.trace, 1); trace_min(a.trace, 3); }
    if (bulk_x && pt < 16) {
      // sixteen threads issue one row copy each (one thread issuing all of them is slower than the copies)
      const int b = pt & 7;
      if (b < a.rows) {
        if (pt < 8) bulk_g2s(xs + b * 2 * kTcK, a.x + (size_t)b * kTcK, 2 * kTcK, x_in);
        else bulk_g2s(rstage + b * 2 * kTcK, a.res_in + (size_t)b * kTcK, 2 * kTcK, x_in);
      }
    }

    // x = h (+ residual), bf16 residual out, RMSNorm, bf16 y in the swizzled layout of the B operand.
    // Warp b owns batch row b: a lane holds four 16-byte pieces of the row, the sum of squares needs one
    // butterfly and no cross-warp step, every lane computes one root; the eight rows proceed in parallel.
    {
      const int b = pwarp;
      uint4 hv[4], rv[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) { hv[c] = make_uint4(0, 0, 0, 0); rv[c] = make_uint4(0, 0, 0, 0); }
      if (bulk_x) {
        if (!named_sync_and(1, kTcProThreads, tc_wait(x_in, 0, abort_flag))) {
          if (pt == 0 && !*abort_flag) report_status(a.status, kStatusCopyTimeout, kKernelTcGemv, blockIdx.x, 4);
          *abort_flag = 1;
        }
        if (b < a.rows) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            hv[c] = *reinterpret_cast<const uint4*>(xs + b * 2 * kTcK + 16 * (32 * c + lane));
            rv[c] = *reinterpret_cast<const uint4*>(rstage + b * 2 * kTcK + 16 * (32 * c + lane));
          }
        }
      } else if (b < a.rows) {
        const size_t xrow = a.ids ? (size_t)clamp_token(a.ids[b], a.embed_rows, a.status, b) : (size_t)b;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          hv[c] = ldg_cg(a.x + xrow * kTcK + 8 * (32 * c + lane));
          if (a.res_in) rv[c] = ldg_cg(a.res_in + (size_t)b * kTcK + 8 * (32 * c + lane));
        }
      }
      if (a.late_trigger) pdl_launch_dependents();   // the successor's prefetch traffic starts after x is here
      named_sync(1, kTcProThreads);    // every row has been read before any y is written over the staging bytes
      float x[4][8];
      float ss = 0.f;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        float hf[8], rf[8];
        unpack8(hv[c], hf);
        unpack8(rv[c], rf);
#pragma unroll
        for (int e = 0; e < 8; ++e) { x[c][e] = hf[e] + rf[e]; ss = fmaf(x[c][e], x[c][e], ss); }
      }
      if (a.res_out && blockIdx.x == 0 && b < a.rows) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint4 o;
          o.x = pack_bf16(x[c][0], x[c][1]); o.y = pack_bf16(x[c][2], x[c][3]);
          o.z = pack_bf16(x[c][4], x[c][5]); o.w = pack_bf16(x[c][6], x[c][7]);
          *reinterpret_cast<uint4*>(a.res_out + (size_t)b * kTcK + 8 * (32 * c + lane)) = o;
        }
      }
#pragma unroll
      for (int m = 16; m >= 1; m >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, m);
      const float rstd = 1.0f / sqrtf(ss / (float)kTcK + a.eps);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        float wf[8], y[8];
        unpack8(nw4[c], wf);
#pragma unroll
        for (int e = 0; e < 8; ++e) y[e] = round_bf16(x[c][e] * rstd) * wf[e];   // rows beyond the batch are zero
        uint4 o;
        o.x = pack_bf16(y[0], y[1]); o.y = pack_bf16(y[2], y[3]); o.z = pack_bf16(y[4], y[5]); o.w = pack_bf16(y[6], y[7]);
        // piece q of the row -> half of K, k-block, 16-byte chunk inside the 128-byte swizzle atom
        const int q = 32 * c + lane, half = q >> 6, kb = (q & 63) >> 3, cc = q & 7, n = b + 8 * half;
        *reinterpret_cast<uint4*>(xs + kb * 2048 + n * 128 + ((cc ^ (n & 7)) << 4)) = o;
      }
    }
    fence_async_smem();      // the MMAs read shared memory through the async proxy
    tc_mbar_arrive(x_ready);
    if (pt == 0) trace_max(a.trace, 4);
    if (pwarp < 4) {
    const int et = pt, ewarp = pwarp;

    // epilogue thread -> batch row eb and rows er, er + 16, ... of the tile
    const int eb = et >> 4, er = et & 15;
    const int q = warp & 3;                       // the quarter of the tensor memory lanes this warp may read
    const int h = q >> 1;                         // which half of K those lanes accumulated
    const int lrow = (q & 1) * (R / 2) + lane;    // tile row of this thread's lane
    const bool lvalid = lane < R / 2;             // M = 64 keeps 16 rows in each quarter, M = 128 all 32
    float best_v = -INFINITY;
    int best_i = 0x7fffffff;
    __shared__ SampleRow srows[kMaxRows];
    if (MODE == kModeNormArgmax) {
      sample_rows_load(a, srows, et);
      named_sync(2, 128);
    }
    int it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < n_tiles; tile += stride, ++it) {
      const int buf = it & 1;
      if (!named_sync_and(2, 128, tc_wait(&acc_full[buf], (it >> 1) & 1, abort_flag))) { ok = false; break; }
      tc_fence_after();
      // this lane's 8 useful columns (its half of K) of every issuer's accumulator
      float v[kTcIssuers][8];
      const uint32_t taddr = tmem_base + ((uint32_t)(32 * q) << 16) + buf * kTcAccCols + 8 * h;
#pragma unroll
      for (int u = 0; u < kTcIssuers; ++u) tc_ld8(taddr + 16 * u, v[u]);
      tc_wait_ld();
      tc_fence_before();
      tc_mbar_arrive(&acc_empty[buf]);            // the accumulators may be overwritten by the tile after next
      float* rb = red + (size_t)buf * 2 * kMaxRows * R;
      if (lvalid) {
#pragma unroll
        for (int b = 0; b < kMaxRows; ++b) rb[(h * kMaxRows + b) * R + lrow] = (v[0][b] + v[1][b]) + (v[2][b] + v[3][b]);
      }
      named_sync(2, 128);
      if (et == 0 && it == 0) trace_max(a.trace, 5);
      if (kSwiglu) {
        // tile rows [0, R/2) are gate rows, [R/2, R) the matching up rows
#pragma unroll
        for (int i = 0; i < R / 32; ++i) {
          const int r = er + 16 * i;
          float gv = rb[eb * R + r] + rb[(kMaxRows + eb) * R + r];
          float uv = rb[eb * R + r + R / 2] + rb[(kMaxRows + eb) * R + r + R / 2];
          gv = round_bf16(gv);
          uv = round_bf16(uv);
          if (eb < a.rows)
            a.out[(size_t)eb * a.out_stride + tile * (R / 2) + r] = __float2bfloat16_rn(gv / (1.0f + expf(-gv)) * uv);
        }
      } else {
#pragma unroll
        for (int i = 0; i < R / 16; ++i) {
          const int r = er + 16 * i;
          const float val = round_bf16(rb[eb * R + r] + rb[(kMaxRows + eb) * R + r]);
          const int row = tile * R + r;
          if (eb < a.rows && row < args.n_rows) {
            if (MODE == kModeNormArgmax) {
              if (a.logits_out) a.logits_out[(size_t)eb * a.vocab + row] = val;
              const float key = a.temps ? sample_key(a.sample_seed, a.sample_idx_offset, srows, eb, row, val) : val;
              if (key > best_v || (key == best_v && row < best_i)) { best_v = key; best_i = row; }
            } else {
              a.out[(size_t)eb * a.out_stride + row] = __float2bfloat16_rn(val);
            }
          }
        }
      }
      if (et == 0 && it == 0) trace_max(a.trace, 6);
    }
    if (!ok) {
      if (!*abort_flag) report_status(a.status, kStatusCopyTimeout, kKernelTcGemv, blockIdx.x, 3);
      *abort_flag = 1;
    }

    if (MODE == kModeNormArgmax) {
      // the 16 threads of a batch row -> one partial per CTA -> the last CTA to arrive merges the grid's
#pragma unroll
      for (int m = 8; m >= 1; m >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best_v, m);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, m);
        if (ov > best_v || (ov == best_v && oi < best_i)) { best_v = ov; best_i = oi; }
      }
      if (er == 0) a.parts[blockIdx.x * kMaxRows + eb] = ArgmaxPart{best_v, best_i};
      __threadfence();
      named_sync(2, 128);
      if (et == 0) *last_flag = (atomicAdd(a.ticket, 1u) == gridDim.x - 1) ? 1 : 0;
      named_sync(2, 128);
      if (*last_flag) {
        __threadfence();
        for (int b = ewarp; b < a.rows; b += 4) {
          float bv = -INFINITY;
          int bi = 0x7fffffff;
          for (int c2 = lane; c2 < (int)gridDim.x; c2 += 32) {
            const int2 rawp = __ldcg(reinterpret_cast<const int2*>(a.parts + c2 * kMaxRows + b));
            const float pv = __int_as_float(rawp.x);
            if (pv > bv || (pv == bv && rawp.y < bi)) { bv = pv; bi = rawp.y; }
          }
#pragma unroll
          for (int m = 16; m >= 1; m >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, m);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, m);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
          }
          if (lane == 0) {
            a.tokens[b] = bi;
            if (a.tokens_out) a.tokens_out[b] = bi;
            if (a.best_out) a.best_out[b] = ArgmaxPart{bv, bi};
          }
        }
        if (et == 0) { *a.ticket = 0u; sample_advance(a); }
      }
    }
    if (et == 0) trace_max(a.trace, 2);
    }   // epilogue warps
  }

  // every MMA has completed (the epilogue waited for the last accumulator) or the CTA has given up
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "n"(2 * kTcAccCols) : "memory");
  }
}

}  // namespace dfb
