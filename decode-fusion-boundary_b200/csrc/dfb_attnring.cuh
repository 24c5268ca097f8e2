// Paged GQA decode attention for long contexts and full batches: the same
// computation as paged_attention_kernel (q/k RMSNorm + RoPE + KV-cache write +
// split-KV attention with an in-kernel merge), organised for streaming.
//
// A CTA owns one batch row and one chunk of 64 context positions for ALL eight
// KV heads.  In the cache ([block][position][kv_head][128]) the eight heads of a
// position are one contiguous 2 KB run for K and one for V, and consecutive
// positions of a block follow one another, so a stage of 8 positions is ONE
// bulk copy (TMA, completion on an mbarrier) of 16 KB for K and one for V into
// a ring of three shared-memory stages; the next stages are in flight while
// the current one is scored, and the first three are requested before the
// dependency wait (the old entries do not depend on the previous kernel).  A
// stage is always fetched whole: slots of the block beyond the row's context,
// and the new token's own slot, are allocated memory whose contents are
// ignored (masked, respectively replaced from shared memory).  The warp that
// finishes a stage last requests the next one into it, so nobody waits to
// refill.
//
// Warp w owns KV head w and its two query heads.  Scores: lane (p, quarter)
// takes position p of the stage and four 16-byte pieces of its K row against q
// values held in registers as packed bf16; the pieces are dealt so that the
// eight lanes of a quarter warp read eight different 16-byte bank groups (piece
// (4 quarter + i + p) mod 16 in step i), which keeps the dense rows free of
// bank conflicts; two shuffles add the quarters; the online softmax needs one
// warp reduction per stage, not one per position.  P.V: lane l owns output dimensions [4 l, 4 l + 4) and walks
// the positions of the stage (8-byte reads of V, the probabilities by shuffle).
// Per context position this is about a third of the instructions of the
// register-resident kernel, whose CTAs load, then compute with nothing in
// flight.
//
// The partial results of the chunks of a row go through the same buffers and
// the same "last to arrive merges" tickets, here one ticket per (row, KV head)
// taken by the head's warp.  Every wait is bounded and reports status 3.
#pragma once

#include "dfb_kernels.cuh"

namespace dfb {

constexpr int kRingPos = 8;                          // positions per stage
constexpr int kRingStages = 3;
constexpr int kRingHeads = 8;                        // KV heads = warps
constexpr int kRingRowBytes = kRingHeads * kHeadDim * 2;         // one position: 2 KB, dense
constexpr int kRingStageBytes = 2 * kRingPos * kRingRowBytes;    // K rows, then V rows
constexpr int kRingSubs = kAttnChunk / kRingPos;     // stages a full chunk goes through
constexpr int kRingThreads = 32 * kRingHeads;
constexpr int kRingSmemBytes = kRingStages * kRingStageBytes + 128;
constexpr int kKernelAttnRing = 7;

// Packed FP32 multiply-add (two IEEE fused multiply-adds in one instruction slot): the kernel is bound by
// instruction issue, not by the FP32 pipe, and every result is bit-identical to two fmaf().
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
  unsigned long long ra, rb, rc, rd;
  asm("mov.b64 %0, {%1, %2};" : "=l"(ra) : "f"(a.x), "f"(a.y));
  asm("mov.b64 %0, {%1, %2};" : "=l"(rb) : "f"(b.x), "f"(b.y));
  asm("mov.b64 %0, {%1, %2};" : "=l"(rc) : "f"(c.x), "f"(c.y));
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(rd) : "l"(ra), "l"(rb), "l"(rc));
  float2 d;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(d.x), "=f"(d.y) : "l"(rd));
  return d;
}
__device__ __forceinline__ float2 fmul2(float2 a, float2 b) {
  unsigned long long ra, rb, rd;
  asm("mov.b64 %0, {%1, %2};" : "=l"(ra) : "f"(a.x), "f"(a.y));
  asm("mov.b64 %0, {%1, %2};" : "=l"(rb) : "f"(b.x), "f"(b.y));
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(rd) : "l"(ra), "l"(rb));
  float2 d;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(d.x), "=f"(d.y) : "l"(rd));
  return d;
}
// the two bf16 values of a packed word as fp32
__device__ __forceinline__ float2 bf2(uint32_t w) { return make_float2(bf_lo(w), bf_hi(w)); }

__device__ __forceinline__ void fence_async_smem_ring() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
// reductions over the 8 positions of a stage: lanes that differ only in bits 3-4 (the quarters) hold equal values
__device__ __forceinline__ float pos_max(float v) {
#pragma unroll
  for (int m = 4; m >= 1; m >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, m));
  return v;
}
__device__ __forceinline__ float pos_sum(float v) {
#pragma unroll
  for (int m = 4; m >= 1; m >>= 1) v += __shfl_xor_sync(0xffffffffu, v, m);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int m = 16; m >= 1; m >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, m));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int m = 16; m >= 1; m >>= 1) v += __shfl_xor_sync(0xffffffffu, v, m);
  return v;
}

// CH: context positions per CTA, 64 or 32 (half as many stages per CTA and twice the CTAs: mid-size grids then
// cover every SM, and three of a CTA's four stages are in flight before the dependency resolves).
template <int CH>
__global__ void __launch_bounds__(kRingThreads, 2) paged_attention_ring_kernel(const AttnArgs a) {
  static_assert(CH == kAttnChunk || 2 * CH == kAttnChunk, "64 or 32 positions per CTA");
  if (!a.late_trigger) pdl_launch_dependents();
  const int split = blockIdx.x, row = blockIdx.y;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) { trace_min(a.trace, 0); trace_max(a.trace, 4); }
  int pos = a.positions[row];
  bool write_ok = true;
  if (pos < 0 || pos >= a.max_pos) {
    report_status(a.status, kStatusBadPosition, kKernelAttention, row, pos);
    pos = pos < 0 ? 0 : a.max_pos - 1;
    write_ok = false;
  }
  int ctx = pos + 1;
  int nsplits = (ctx + CH - 1) / CH;
  if (nsplits > (int)gridDim.x) {   // the host's context bound was too small (see paged_attention_kernel)
    if (split == 0) report_status(a.status, kStatusBadGrid, kKernelAttention, row, pos);
    nsplits = (int)gridDim.x;
    ctx = nsplits * CH;
    pos = ctx - 1;
    write_ok = false;
  }
  if (split >= nsplits) return;

  extern __shared__ __align__(128) unsigned char ring_smem[];
  __shared__ uint64_t full[kRingStages];
  __shared__ unsigned int done[kRingStages];    // warps that have finished the stage's current contents
  __shared__ __align__(16) __nv_bfloat16 qsm[kRingHeads][2][kHeadDim];   // q after norm + RoPE (bf16 values)
  __shared__ __align__(16) __nv_bfloat16 knew[kRingHeads][kHeadDim];
  __shared__ __align__(16) __nv_bfloat16 vnew[kRingHeads][kHeadDim];

  const int start = split * CH;
  const int end = min(ctx, start + CH);
  const bool owner = split == nsplits - 1;
  const int nsub = (end - start + kRingPos - 1) / kRingPos;
  int bt_col = start / a.block_size;
  if (a.bt_cols > 0 && bt_col >= a.bt_cols) {
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
  const size_t tok_stride = (size_t)kRingHeads * kHeadDim;
  const size_t chunk_base = ((size_t)block * a.block_size + (start % a.block_size)) * tok_stride;

  if (tid == 0) {
#pragma unroll
    for (int s = 0; s < kRingStages; ++s) { mbar_init(&full[s], 1); done[s] = 0u; }
    fence_mbar_init();
  }
  __syncthreads();

  // one elected lane requests stage j: the 8 positions' K rows as one copy, their V rows as another
  auto issue_stage = [&](int j) {
    const int s = j % kRingStages;
    mbar_expect_tx(&full[s], (uint32_t)kRingStageBytes);
    const size_t off = chunk_base + (size_t)(j * kRingPos) * tok_stride;
    bulk_g2s(ring_smem + s * kRingStageBytes, a.k_cache + off, kRingPos * kRingRowBytes, &full[s]);
    bulk_g2s(ring_smem + s * kRingStageBytes + kRingPos * kRingRowBytes, a.v_cache + off, kRingPos * kRingRowBytes, &full[s]);
  };
  if (tid == 0) {
    for (int j = 0; j < kRingStages && j < nsub; ++j) issue_stage(j);
  }
  if (tid >= 32 && tid < 64)
    l2_prefetch_slice(a.ahead_ptr, a.ahead_bytes, (int)(blockIdx.y * gridDim.x + blockIdx.x), (int)(gridDim.x * gridDim.y));

  // constants of the new token's norm and rotation: independent of the predecessor
  const uint32_t qw_lo = *reinterpret_cast<const uint32_t*>(a.q_norm + 2 * lane);
  const uint32_t qw_hi = *reinterpret_cast<const uint32_t*>(a.q_norm + 2 * lane + 64);
  const uint32_t kw_lo = *reinterpret_cast<const uint32_t*>(a.k_norm + 2 * lane);
  const uint32_t kw_hi = *reinterpret_cast<const uint32_t*>(a.k_norm + 2 * lane + 64);
  const float* cs = a.cos_sin + (size_t)pos * kHeadDim;
  const float2 rc = *reinterpret_cast<const float2*>(cs + 2 * lane);
  const float2 rs = *reinterpret_cast<const float2*>(cs + 64 + 2 * lane);

  pdl_wait();
  if (tid == 0) { trace_max(a.trace, 1); trace_min(a.trace, 3); }

  // ---- new token: this warp's two query heads and its K head get RMSNorm + RoPE (in lockstep), V is copied ----
  {
    const __nv_bfloat16* src = a.qkv + (size_t)row * a.qkv_stride;
    const __nv_bfloat16* vec[3] = {src + (2 * warp) * kHeadDim, src + (2 * warp + 1) * kHeadDim,
                                   src + a.q_size + warp * kHeadDim};
    const int d = 2 * lane;   // handles d, d+1 and their RoPE partners d+64, d+65
    uint32_t lo[3], hi[3];
#pragma unroll
    for (int i = 0; i < 3; ++i) {
      lo[i] = __ldcg(reinterpret_cast<const uint32_t*>(vec[i] + d));
      hi[i] = __ldcg(reinterpret_cast<const uint32_t*>(vec[i] + d + 64));
    }
    const uint2 vv = __ldcg(reinterpret_cast<const uint2*>(src + a.q_size + a.kv_size + warp * kHeadDim) + lane);
    float x[3][4], ss[3];
#pragma unroll
    for (int i = 0; i < 3; ++i) {
      x[i][0] = bf_lo(lo[i]); x[i][1] = bf_hi(lo[i]); x[i][2] = bf_lo(hi[i]); x[i][3] = bf_hi(hi[i]);
      ss[i] = x[i][0] * x[i][0] + x[i][1] * x[i][1] + x[i][2] * x[i][2] + x[i][3] * x[i][3];
    }
#pragma unroll
    for (int m = 16; m >= 1; m >>= 1) {
#pragma unroll
      for (int i = 0; i < 3; ++i) ss[i] += __shfl_xor_sync(0xffffffffu, ss[i], m);
    }
#pragma unroll
    for (int i = 0; i < 3; ++i) {
      const float rstd = 1.0f / sqrtf(ss[i] / (float)kHeadDim + a.eps);
      const uint32_t wl = i < 2 ? qw_lo : kw_lo, wh = i < 2 ? qw_hi : kw_hi;
      const float w[4] = {bf_lo(wl), bf_hi(wl), bf_lo(wh), bf_hi(wh)};
      float y[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) y[e] = round_bf16(round_bf16(x[i][e] * rstd) * w[e]);
      const uint32_t r_lo = pack_bf16(round_bf16(mul_sub_unfused(y[0], rc.x, y[2], rs.x)), round_bf16(mul_sub_unfused(y[1], rc.y, y[3], rs.y)));
      const uint32_t r_hi = pack_bf16(round_bf16(mul_add_unfused(y[2], rc.x, y[0], rs.x)), round_bf16(mul_add_unfused(y[3], rc.y, y[1], rs.y)));
      __nv_bfloat16* dst = i < 2 ? qsm[warp][i] : knew[warp];
      *reinterpret_cast<uint32_t*>(dst + d) = r_lo;
      *reinterpret_cast<uint32_t*>(dst + d + 64) = r_hi;
    }
    reinterpret_cast<uint2*>(vnew[warp])[lane] = vv;
  }
  __syncwarp();
  if (a.late_trigger) pdl_launch_dependents();

  if (owner && write_ok && (a.row_active == nullptr || a.row_active[row] != 0)) {
    // the new token's K / V of this head into the cache: lanes 0-15 the 16-byte pieces of K, lanes 16-31 of V
    const size_t off = chunk_base + (size_t)(pos - start) * tok_stride + (size_t)warp * kHeadDim + 8 * (lane & 15);
    const uint4 piece = reinterpret_cast<const uint4*>(lane < 16 ? knew[warp] : vnew[warp])[lane & 15];
    *reinterpret_cast<uint4*>((lane < 16 ? a.k_cache : a.v_cache) + off) = piece;
  }

  // this lane's four 16-byte pieces (8 dimensions each) of the two query heads, packed bf16: piece
  // (4 quarter + i + p) mod 16 in step i, the same pieces it reads of its position's K row
  const int qp = lane & (kRingPos - 1), quarter = lane >> 3;
  uint4 q0r[4], q1r[4];
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const int piece = (4 * quarter + c + qp) & 15;
    q0r[c] = reinterpret_cast<const uint4*>(qsm[warp][0])[piece];
    q1r[c] = reinterpret_cast<const uint4*>(qsm[warp][1])[piece];
  }

  constexpr float kLog2e = 1.4426950408889634f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  float o0[4] = {0.f, 0.f, 0.f, 0.f}, o1[4] = {0.f, 0.f, 0.f, 0.f};
  bool ok = true;
  for (int j = 0; j < nsub; ++j) {
    const int s = j % kRingStages;
    // the whole warp takes the same decision (a lane that left alone would strand the shuffles below)
    if (!__all_sync(0xffffffffu, mbar_wait_bounded(&full[s], (j / kRingStages) & 1))) { ok = false; break; }
    unsigned char* kst = ring_smem + s * kRingStageBytes;
    unsigned char* vst = kst + kRingPos * kRingRowBytes;
    const int p0 = start + j * kRingPos;
    const int npos = min(kRingPos, end - p0);
    if (owner && pos >= p0 && pos < p0 + kRingPos) {
      // the new token's row of this head comes from shared memory
      const int pr = pos - p0;
      unsigned char* dst = (lane < 16 ? kst : vst) + pr * kRingRowBytes + warp * (kHeadDim * 2) + 16 * (lane & 15);
      *reinterpret_cast<uint4*>(dst) = reinterpret_cast<const uint4*>(lane < 16 ? knew[warp] : vnew[warp])[lane & 15];
      __syncwarp();
    }
    // ---- scores of position qp: this lane's 32 dimensions, then the four quarters are added ----
    float d0 = 0.f, d1 = 0.f;
    {
      const unsigned char* krow = kst + qp * kRingRowBytes + warp * (kHeadDim * 2);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const uint4 kv = *reinterpret_cast<const uint4*>(krow + 16 * ((4 * quarter + c + qp) & 15));
        // (even, odd) dimension pairs of the piece: the products of a pair go through one packed FMA, the
        // accumulators (t, u) = (sum over even dimensions, sum over odd dimensions) per query head as before
        const uint32_t kw[4] = {kv.x, kv.y, kv.z, kv.w};
        const uint32_t aw[4] = {q0r[c].x, q0r[c].y, q0r[c].z, q0r[c].w};
        const uint32_t bw[4] = {q1r[c].x, q1r[c].y, q1r[c].z, q1r[c].w};
        float2 tu0 = fmul2(bf2(kw[0]), bf2(aw[0])), tu1 = fmul2(bf2(kw[0]), bf2(bw[0]));
#pragma unroll
        for (int e = 1; e < 4; ++e) {
          const float2 kf = bf2(kw[e]);
          tu0 = ffma2(kf, bf2(aw[e]), tu0);
          tu1 = ffma2(kf, bf2(bw[e]), tu1);
        }
        d0 += tu0.x + tu0.y;
        d1 += tu1.x + tu1.y;
      }
    }
    d0 += __shfl_xor_sync(0xffffffffu, d0, 8);  d1 += __shfl_xor_sync(0xffffffffu, d1, 8);
    d0 += __shfl_xor_sync(0xffffffffu, d0, 16); d1 += __shfl_xor_sync(0xffffffffu, d1, 16);
    const bool valid = qp < npos;
    const float s0 = valid ? d0 * a.scale : -INFINITY, s1 = valid ? d1 * a.scale : -INFINITY;
    // ---- online softmax over the stages (every lane holds the same running maximum and sum) ----
    const float n0 = fmaxf(m0, pos_max(s0)), n1 = fmaxf(m1, pos_max(s1));   // a stage has at least one position
    const float c0 = exp2f((m0 - n0) * kLog2e), c1 = exp2f((m1 - n1) * kLog2e);   // first stage: exp2(-inf) = 0
    const float p0v = exp2f((s0 - n0) * kLog2e), p1v = exp2f((s1 - n1) * kLog2e); // invalid positions: 0
    l0 = l0 * c0 + pos_sum(p0v);
    l1 = l1 * c1 + pos_sum(p1v);
    m0 = n0; m1 = n1;
#pragma unroll
    for (int e = 0; e < 4; ++e) { o0[e] *= c0; o1[e] *= c1; }
    // ---- P.V: this lane's 4 output dimensions over the positions of the stage ----
    const unsigned char* vcol = vst + warp * (kHeadDim * 2) + 8 * lane;
#pragma unroll
    for (int p = 0; p < kRingPos; ++p) {
      const float w0 = __shfl_sync(0xffffffffu, p0v, p), w1 = __shfl_sync(0xffffffffu, p1v, p);
      if (p < npos) {   // same for the whole warp; rows beyond npos were never loaded
        const uint2 v2 = *reinterpret_cast<const uint2*>(vcol + p * kRingRowBytes);
        const float2 va = bf2(v2.x), vb = bf2(v2.y), ww0 = make_float2(w0, w0), ww1 = make_float2(w1, w1);
        float2 r;
        r = ffma2(ww0, va, make_float2(o0[0], o0[1])); o0[0] = r.x; o0[1] = r.y;
        r = ffma2(ww0, vb, make_float2(o0[2], o0[3])); o0[2] = r.x; o0[3] = r.y;
        r = ffma2(ww1, va, make_float2(o1[0], o1[1])); o1[0] = r.x; o1[1] = r.y;
        r = ffma2(ww1, vb, make_float2(o1[2], o1[3])); o1[2] = r.x; o1[3] = r.y;
      }
    }
    __syncwarp();
    if (j + kRingStages < nsub && lane == 0) {
      // the warp that finishes the stage last requests the positions three stages ahead into it
      __threadfence_block();
      if (atomicAdd(&done[s], 1u) == kRingHeads - 1) {
        done[s] = 0u;
        __threadfence_block();
        fence_async_smem_ring();
        issue_stage(j + kRingStages);
      }
    }
  }
  if (!ok) {
    report_status(a.status, kStatusCopyTimeout, kKernelAttnRing, blockIdx.x, row);
    // give the copies in flight a bounded chance to land before the CTA goes away
    if (warp == 0) for (int s = 0; s < kRingStages; ++s) { mbar_wait_bounded(&full[s], 0); mbar_wait_bounded(&full[s], 1); }
  }
  if (tid == 0) trace_max(a.trace, 5);

  // ---- this head's result: direct when the row has a single chunk, else partial + merge by the last to arrive ----
  __nv_bfloat16* out = a.out + (size_t)row * a.q_size + (size_t)(2 * warp) * kHeadDim + 4 * lane;
  if (nsplits == 1) {
    *reinterpret_cast<uint2*>(out) = make_uint2(pack_bf16(o0[0] / l0, o0[1] / l0), pack_bf16(o0[2] / l0, o0[3] / l0));
    *reinterpret_cast<uint2*>(out + kHeadDim) = make_uint2(pack_bf16(o1[0] / l1, o1[1] / l1), pack_bf16(o1[2] / l1, o1[3] / l1));
  } else {
    const size_t pidx = ((size_t)row * a.kv_heads + warp) * kMaxSplits;
    float* po = a.part_o + (pidx + split) * 2 * kHeadDim + 4 * lane;
    *reinterpret_cast<float4*>(po) = make_float4(o0[0], o0[1], o0[2], o0[3]);
    *reinterpret_cast<float4*>(po + kHeadDim) = make_float4(o1[0], o1[1], o1[2], o1[3]);
    if (lane < 2) a.part_ml[(pidx + split) * 2 + lane] = make_float2(lane ? m1 : m0, lane ? l1 : l0);
    __syncwarp();
    int last = 0;
    if (lane == 0) {
      // acquire-release at GPU scope: publishes this warp's partial (ordered before it by the warp barrier
      // above) and makes the other chunks' partials visible to the last arrival
      unsigned int prev;
      asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;"
                   : "=r"(prev) : "l"(a.tickets + row * a.kv_heads + warp) : "memory");
      last = prev == (unsigned)(nsplits - 1) ? 1 : 0;
    }
    last = __shfl_sync(0xffffffffu, last, 0);
    if (last) {
      // lane s holds (max, sum) of chunk s for both heads; weights by shuffle, partial outputs 8 chunks at a time
      float2 ml0 = make_float2(-INFINITY, 0.f), ml1 = make_float2(-INFINITY, 0.f);
      if (lane < nsplits) {
        ml0 = __ldcg(&a.part_ml[(pidx + lane) * 2]);
        ml1 = __ldcg(&a.part_ml[(pidx + lane) * 2 + 1]);
      }
      const float M0 = warp_max(ml0.x), M1 = warp_max(ml1.x);
      const float w0 = lane < nsplits ? exp2f((ml0.x - M0) * kLog2e) : 0.f;
      const float w1 = lane < nsplits ? exp2f((ml1.x - M1) * kLog2e) : 0.f;
      const float S0 = warp_sum(w0 * ml0.y), S1 = warp_sum(w1 * ml1.y);
      float A0[4] = {0.f, 0.f, 0.f, 0.f}, A1[4] = {0.f, 0.f, 0.f, 0.f};
      const float* ps = a.part_o + pidx * 2 * kHeadDim + 4 * lane;
      for (int sb = 0; sb < nsplits; sb += 8) {
        float4 pa[8], pb[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          if (sb + u < nsplits) {
            pa[u] = __ldcg(reinterpret_cast<const float4*>(ps + (size_t)(sb + u) * 2 * kHeadDim));
            pb[u] = __ldcg(reinterpret_cast<const float4*>(ps + (size_t)(sb + u) * 2 * kHeadDim + kHeadDim));
          } else {
            pa[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            pb[u] = make_float4(0.f, 0.f, 0.f, 0.f);
          }
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const float x0 = __shfl_sync(0xffffffffu, w0, (sb + u) & 31), x1 = __shfl_sync(0xffffffffu, w1, (sb + u) & 31);
          A0[0] = fmaf(x0, pa[u].x, A0[0]); A0[1] = fmaf(x0, pa[u].y, A0[1]); A0[2] = fmaf(x0, pa[u].z, A0[2]); A0[3] = fmaf(x0, pa[u].w, A0[3]);
          A1[0] = fmaf(x1, pb[u].x, A1[0]); A1[1] = fmaf(x1, pb[u].y, A1[1]); A1[2] = fmaf(x1, pb[u].z, A1[2]); A1[3] = fmaf(x1, pb[u].w, A1[3]);
        }
      }
      *reinterpret_cast<uint2*>(out) = make_uint2(pack_bf16(A0[0] / S0, A0[1] / S0), pack_bf16(A0[2] / S0, A0[3] / S0));
      *reinterpret_cast<uint2*>(out + kHeadDim) = make_uint2(pack_bf16(A1[0] / S1, A1[1] / S1), pack_bf16(A1[2] / S1, A1[3] / S1));
      if (lane == 0) a.tickets[row * a.kv_heads + warp] = 0u;
    }
  }
  if (tid == 0) trace_max(a.trace, 2);
}

}  // namespace dfb
