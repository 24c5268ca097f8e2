// Weight-streaming GEMV for one or two batch rows on the FP32 pipe.
//
// mma.sync issues only about one m16n8k16 per 38 cycles per SM sub-partition on
// this part, and a batch of one or two rows wastes most of each MMA anyway, so
// for rows <= 2 every projection is a classic row-parallel GEMV:
//   * a warp owns whole weight rows (RPW = 2: one row per half-warp, K = 1024;
//     RPW = 1: one row per warp, K = 2048 / 3072), lanes interleave 16-byte
//     chunks of the row, so global loads are fully coalesced 128-bit loads;
//   * the row's weights are requested into registers BEFORE the dependency wait
//     (programmatic dependent launch), so they stream while the previous kernel
//     is still running;
//   * x (after the fused residual add + RMSNorm, done by all 256 threads, 4
//     elements each) is kept in shared memory as fp32;
//   * products are accumulated in fp32, reduced with shuffles, rounded once to
//     bf16, and the epilogue (store / SwiGLU / logits + greedy argmax) runs in the
//     lane that holds the sum.  No shared-memory reduction, no tensor cores.
// Registers stay low (about 64), so three CTAs of 8 warps share an SM: the
// occupancy hides the instruction latency that dominates these tiny kernels.
#pragma once

#include "dfb_kernels.cuh"

namespace dfb {

constexpr int kRowThreads = 256;
constexpr int kRowWarps = 8;

template <int K, int RPW, int NB, int MODE>
__global__ void __launch_bounds__(kRowThreads, 3) row_gemv_kernel(const GemvArgs a) {
  constexpr bool kNorm = MODE != kModeStore;
  constexpr int LPR = 32 / RPW;            // lanes per row
  constexpr int NL = K / LPR / 8;          // 16-byte weight chunks per lane
  constexpr int RPC = kRowWarps * RPW;     // rows (or gate/up pairs * 2) per CTA and group
  static_assert(!kNorm || K == 1024, "the fused norm covers the hidden size only");
  pdl_launch_dependents();
  if (threadIdx.x == 0) trace_min(a.trace, 0);

  __shared__ __align__(16) float xs[NB][K];
  __shared__ float ssq[kRowWarps][NB];
  __shared__ float cta_v[kRowWarps][NB];
  __shared__ int cta_i[kRowWarps][NB];
  __shared__ int last_flag;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int half = lane / LPR, lr = lane % LPR;   // row slot inside the warp, lane inside the row
  const int n_groups = a.n_tiles;

  // weights of group `grp` for this lane: row r, chunks lr + LPR * j
  auto weight_row = [&](int grp) -> const __nv_bfloat16* {
    if (MODE == kModeNormSwiglu) {
      const int i = grp * kRowWarps + warp;                       // gate / up pair index
      return a.w + (size_t)(half ? a.gate_rows + i : i) * K;
    }
    return a.w + (size_t)(grp * RPC + warp * RPW + half) * K;
  };
  uint4 wreg[NL];
  int grp = blockIdx.x;
  if (grp < n_groups) {
    const __nv_bfloat16* p = weight_row(grp) + 8 * lr;
#pragma unroll
    for (int j = 0; j < NL; ++j) wreg[j] = ldg_stream(p + 8 * LPR * j);
  }
  uint2 nwv = make_uint2(0, 0);
  if (kNorm) nwv = *reinterpret_cast<const uint2*>(a.norm_w + 4 * tid);

  pdl_wait();
  if (threadIdx.x == 0) { trace_max(a.trace, 1); trace_min(a.trace, 3); }
  const bool probe = a.trace && blockIdx.x == 0 && threadIdx.x == 0;   // cycle counts of CTA 0 in words 5-7
  long long c0 = 0, c1 = 0, c2 = 0;
  if (probe) c0 = clock64();

  // ---- x into shared memory as fp32 (with the fused residual add + RMSNorm) ----
  if (kNorm) {
    float x[NB][4];
#pragma unroll
    for (int b = 0; b < NB; ++b) {
      if (b < a.rows) {
        const size_t xrow = a.ids ? (size_t)a.ids[b] : (size_t)b;
        const uint2 hv = __ldcg(reinterpret_cast<const uint2*>(a.x + xrow * K) + tid);
        uint2 rv = make_uint2(0, 0);
        if (a.res_in) rv = __ldcg(reinterpret_cast<const uint2*>(a.res_in + (size_t)b * K) + tid);
        x[b][0] = bf_lo(hv.x) + bf_lo(rv.x); x[b][1] = bf_hi(hv.x) + bf_hi(rv.x);
        x[b][2] = bf_lo(hv.y) + bf_lo(rv.y); x[b][3] = bf_hi(hv.y) + bf_hi(rv.y);
        if (a.res_out && blockIdx.x == 0)
          reinterpret_cast<uint2*>(a.res_out + (size_t)b * K)[tid] =
              make_uint2(pack_bf16(x[b][0], x[b][1]), pack_bf16(x[b][2], x[b][3]));
      } else {
        x[b][0] = 0.f; x[b][1] = 0.f; x[b][2] = 0.f; x[b][3] = 0.f;
      }
      float ss = x[b][0] * x[b][0] + x[b][1] * x[b][1] + x[b][2] * x[b][2] + x[b][3] * x[b][3];
#pragma unroll
      for (int m = 16; m >= 1; m >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, m);
      if (lane == 0) ssq[warp][b] = ss;
    }
    __syncthreads();
    const float w0 = bf_lo(nwv.x), w1 = bf_hi(nwv.x), w2 = bf_lo(nwv.y), w3 = bf_hi(nwv.y);
#pragma unroll
    for (int b = 0; b < NB; ++b) {
      float tot = 0.f;
#pragma unroll
      for (int w = 0; w < kRowWarps; ++w) tot += ssq[w][b];
      const float rstd = 1.0f / sqrtf(tot / (float)K + a.eps);
      float4 y;
      y.x = round_bf16(round_bf16(x[b][0] * rstd) * w0); y.y = round_bf16(round_bf16(x[b][1] * rstd) * w1);
      y.z = round_bf16(round_bf16(x[b][2] * rstd) * w2); y.w = round_bf16(round_bf16(x[b][3] * rstd) * w3);
      reinterpret_cast<float4*>(xs[b])[tid] = y;
    }
  } else {
#pragma unroll
    for (int b = 0; b < NB; ++b)
      for (int c = tid; c < K / 8; c += kRowThreads) {
        float f[8];
        if (b < a.rows) {
          const uint4 v = ldg_cg(a.x + (size_t)b * K + 8 * c);
          unpack8(v, f);
        } else {
#pragma unroll
          for (int e = 0; e < 8; ++e) f[e] = 0.f;
        }
        reinterpret_cast<float4*>(xs[b])[2 * c] = make_float4(f[0], f[1], f[2], f[3]);
        reinterpret_cast<float4*>(xs[b])[2 * c + 1] = make_float4(f[4], f[5], f[6], f[7]);
      }
  }
  __syncthreads();
  if (threadIdx.x == 0) trace_max(a.trace, 4);
  if (probe) { c1 = clock64(); a.trace[5] = (unsigned long long)(c1 - c0); }
  float best_v[NB];
  int best_i[NB];
#pragma unroll
  for (int b = 0; b < NB; ++b) { best_v[b] = -INFINITY; best_i[b] = 0x7fffffff; }

  // ---- row groups of this CTA ----
  for (; grp < n_groups; grp += gridDim.x) {
    float acc[NB][4];
#pragma unroll
    for (int b = 0; b < NB; ++b) { acc[b][0] = 0.f; acc[b][1] = 0.f; acc[b][2] = 0.f; acc[b][3] = 0.f; }
#pragma unroll
    for (int j = 0; j < NL; ++j) {
      float wf[8];
      unpack8(wreg[j], wf);
      const int col = 8 * (lr + LPR * j);
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        const float4 x0 = *reinterpret_cast<const float4*>(&xs[b][col]);
        const float4 x1 = *reinterpret_cast<const float4*>(&xs[b][col + 4]);
        acc[b][0] = fmaf(wf[0], x0.x, acc[b][0]); acc[b][1] = fmaf(wf[1], x0.y, acc[b][1]);
        acc[b][2] = fmaf(wf[2], x0.z, acc[b][2]); acc[b][3] = fmaf(wf[3], x0.w, acc[b][3]);
        acc[b][0] = fmaf(wf[4], x1.x, acc[b][0]); acc[b][1] = fmaf(wf[5], x1.y, acc[b][1]);
        acc[b][2] = fmaf(wf[6], x1.z, acc[b][2]); acc[b][3] = fmaf(wf[7], x1.w, acc[b][3]);
      }
    }
    // request the next group's weights as soon as the registers are free
    const int nxt = grp + gridDim.x;
    if (nxt < n_groups) {
      const __nv_bfloat16* p = weight_row(nxt) + 8 * lr;
#pragma unroll
      for (int j = 0; j < NL; ++j) wreg[j] = ldg_stream(p + 8 * LPR * j);
    }
    float v[NB];
#pragma unroll
    for (int b = 0; b < NB; ++b) {
      float s = (acc[b][0] + acc[b][1]) + (acc[b][2] + acc[b][3]);
#pragma unroll
      for (int m = LPR / 2; m >= 1; m >>= 1) s += __shfl_xor_sync(0xffffffffu, s, m);
      v[b] = round_bf16(s);
    }
    if (probe && grp == (int)blockIdx.x) { c2 = clock64(); a.trace[6] = (unsigned long long)(c2 - c1); }
    if (MODE == kModeNormSwiglu) {
      // lanes 0-15 hold gate_i, lanes 16-31 hold up_i
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        const float up = __shfl_xor_sync(0xffffffffu, v[b], 16);
        if (lane == 0 && b < a.rows)
          a.out[(size_t)b * a.out_stride + grp * kRowWarps + warp] = __float2bfloat16_rn(v[b] / (1.0f + expf(-v[b])) * up);
      }
    } else {
      const int row = grp * RPC + warp * RPW + half;
      if (lr == 0) {
#pragma unroll
        for (int b = 0; b < NB; ++b) {
          if (b < a.rows) {
            if (MODE == kModeNormArgmax) {
              if (a.logits_out) a.logits_out[(size_t)b * a.vocab + row] = v[b];
              if (v[b] > best_v[b] || (v[b] == best_v[b] && row < best_i[b])) { best_v[b] = v[b]; best_i[b] = row; }
            } else {
              a.out[(size_t)b * a.out_stride + row] = __float2bfloat16_rn(v[b]);
            }
          }
        }
      }
    }
  }

  if (MODE == kModeNormArgmax) {
    // half-warp leaders -> warp -> CTA -> grid (the last CTA to arrive finishes)
#pragma unroll
    for (int b = 0; b < NB; ++b) {
      if (RPW == 2) {
        const float ov = __shfl_xor_sync(0xffffffffu, best_v[b], 16);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i[b], 16);
        if (ov > best_v[b] || (ov == best_v[b] && oi < best_i[b])) { best_v[b] = ov; best_i[b] = oi; }
      }
      if (lane == 0) { cta_v[warp][b] = best_v[b]; cta_i[warp][b] = best_i[b]; }
    }
    __syncthreads();
    if (tid < NB) {
      float v = cta_v[0][tid];
      int i = cta_i[0][tid];
      for (int w = 1; w < kRowWarps; ++w)
        if (cta_v[w][tid] > v || (cta_v[w][tid] == v && cta_i[w][tid] < i)) { v = cta_v[w][tid]; i = cta_i[w][tid]; }
      a.parts[blockIdx.x * kMaxRows + tid] = ArgmaxPart{v, i};
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) last_flag = (atomicAdd(a.ticket, 1u) == gridDim.x - 1) ? 1 : 0;
    __syncthreads();
    if (last_flag) {
      __threadfence();
      for (int b = warp; b < a.rows; b += kRowWarps) {
        float v = -INFINITY;
        int i = 0x7fffffff;
        for (int c2 = lane; c2 < (int)gridDim.x; c2 += 32) {
          const int2 raw = __ldcg(reinterpret_cast<const int2*>(a.parts + c2 * kMaxRows + b));
          const float pv = __int_as_float(raw.x);
          if (pv > v || (pv == v && raw.y < i)) { v = pv; i = raw.y; }
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
        }
      }
      if (tid == 0) *a.ticket = 0u;
    }
  }
  if (threadIdx.x == 0) trace_max(a.trace, 2);
  if (probe) a.trace[7] = (unsigned long long)(clock64() - c2);
}

}  // namespace dfb
