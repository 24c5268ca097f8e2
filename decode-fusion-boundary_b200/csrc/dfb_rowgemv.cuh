// Weight-streaming GEMV for up to eight batch rows on the FP32 pipe.
//
// mma.sync issues only about one m16n8k16 per 38 cycles per SM sub-partition on
// this part, and a small batch wastes most of each MMA anyway, so the
// projections run on the FP32 pipe:
//   * a CTA owns RC consecutive weight rows (16 at K = 1024, 8 at K = 2048 and
//     3072) and its warps split K: warp w owns columns [w*S, (w+1)*S) with
//     S = 128 or 256, so a lane needs only 8 values of x per batch row, kept in
//     registers, and multiplies them with the same 16-byte chunk of 8 rows;
//   * the weight chunks (8 x 16 bytes per lane, fully coalesced) are requested
//     BEFORE the dependency wait (programmatic dependent launch), so they stream
//     while the previous kernel is still running;
//   * the residual add + RMSNorm is done by the whole CTA, 4 elements per thread;
//   * per-row partial sums are reduced with a halving butterfly of shuffles, then
//     across warps through shared memory, rounded once to bf16; the epilogue
//     (store / SwiGLU / logits + greedy argmax) is done by one thread per row.
#pragma once

#include "dfb_exchange.cuh"
#include "dfb_kernels.cuh"

namespace dfb {

template <int K>
struct RowCfg {
  // K <= 1536: one warp per 128 columns (also the tensor-parallel shards 256 ... 1536);
  // K = 2048 / 3072: 8 / 12 warps of 256 columns
  static constexpr int kWarps = K <= 1536 ? K / 128 : (K == 3072 ? 12 : 8);
  static constexpr int kSlice = K / kWarps;            // columns per warp: 128 or 256
  static constexpr int kLanesPerRow = kSlice / 8;      // 16 or 32 lanes cover the slice
  static constexpr int kHalves = 32 / kLanesPerRow;    // row halves handled side by side: 2 or 1
  static constexpr int kRows = 8 * kHalves;            // rows per CTA and group: 16 or 8
  static constexpr int kThreads = kWarps * 32;
};

template <int K, int NB>
constexpr int row_smem_bytes() { return NB * K * 4; }   // fp32 copy of x, dynamic shared memory

template <int K, int NB, int MODE>
__global__ void __launch_bounds__(RowCfg<K>::kThreads, (K == 3072 || K == 1536 || NB > 2) ? 2 : 3)
row_gemv_kernel(const GemvArgs a) {
  using C = RowCfg<K>;
  constexpr bool kNorm = MODE != kModeStore;
  constexpr int W = C::kWarps, LPR = C::kLanesPerRow, RC = C::kRows;
  static_assert(!kNorm || K == 1024, "the fused norm covers the hidden size only");
  if (!a.late_trigger) pdl_launch_dependents();
  if (threadIdx.x == 0) trace_min(a.trace, 0);

  extern __shared__ __align__(16) float xs_dyn[];
  float (*xs)[K] = reinterpret_cast<float (*)[K]>(xs_dyn);
  __shared__ float ssq[W][NB];
  __shared__ float red[W][NB][RC];
  __shared__ int last_flag;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int hr = lane / LPR, lc = lane % LPR;      // row half, 16-byte chunk inside the warp's slice
  const int col = warp * C::kSlice + 8 * lc;       // this lane's 8 columns
  const int n_groups = a.n_tiles;

  // weight row i (0..7) of this lane's half in group `grp`
  auto weight_ptr = [&](int grp, int i) -> const __nv_bfloat16* {
    int row;
    if (MODE == kModeNormSwiglu) row = (hr ? a.gate_rows : 0) + grp * 8 + i;   // half 0: gate rows, half 1: up rows
    else row = grp * RC + hr * 8 + i;
    return a.w + (size_t)row * K + col;
  };
  uint4 wreg[8];
  int grp = blockIdx.x;
  if (grp < n_groups) {
#pragma unroll
    for (int i = 0; i < 8; ++i) wreg[i] = ldg_stream(weight_ptr(grp, i));
  }
  uint2 nwv = make_uint2(0, 0);
  if (kNorm) nwv = *reinterpret_cast<const uint2*>(a.norm_w + 4 * tid);
  if (warp == 0 && !a.ahead_late) l2_prefetch_slice(a.ahead_ptr, a.ahead_bytes, blockIdx.x, gridDim.x);
  // Norm modes fetch x and the residual with two bulk copies per batch row (TMA) into
  // the bytes that later hold the fp32 copy of x: ordinary loads would queue in the
  // load/store unit behind the weight requests of the kernels that were let in early
  // (measured: 3,600 instead of 1,600 cycles until x is in shared memory).
  __shared__ uint64_t xbar;
  const bool bulk_x = kNorm && a.bulk_x && a.ids == nullptr && a.res_in != nullptr;
  if (bulk_x) {
    if (tid == 0) { mbar_init(&xbar, 1); fence_mbar_init(); }
    __syncthreads();
  }

  pdl_wait();
  if (bulk_x && tid == 0) {
    mbar_expect_tx(&xbar, (uint32_t)(a.rows * 4 * K));
    for (int b = 0; b < a.rows; ++b) {
      bulk_g2s(xs[b], a.x + (size_t)b * K, 2 * K, &xbar);                                  // bytes [0, 2K) of row b
      bulk_g2s(reinterpret_cast<unsigned char*>(xs[b]) + 2 * K, a.res_in + (size_t)b * K, 2 * K, &xbar);
    }
  }
  if (threadIdx.x == 0) { trace_max(a.trace, 1); trace_min(a.trace, 3); }

  // ---- x into shared memory as fp32 (with the fused residual add + RMSNorm) ----
  if (kNorm) {
    float x[NB][4];
#pragma unroll
    for (int b = 0; b < NB; ++b) {
      if (b < a.rows) {
        uint2 hv, rv = make_uint2(0, 0);
        if (bulk_x) {
          if (b == 0 && !mbar_wait_bounded(&xbar, 0))
            report_status(a.status, kStatusCopyTimeout, kKernelGemv, blockIdx.x, 0);
          hv = reinterpret_cast<const uint2*>(xs[b])[tid];
          rv = reinterpret_cast<const uint2*>(reinterpret_cast<const unsigned char*>(xs[b]) + 2 * K)[tid];
        } else {
          const size_t xrow = a.ids ? (size_t)clamp_token(a.ids[b], a.embed_rows, a.status, b) : (size_t)b;
          hv = __ldcg(reinterpret_cast<const uint2*>(a.x + xrow * K) + tid);
          if (a.res_in) rv = __ldcg(reinterpret_cast<const uint2*>(a.res_in + (size_t)b * K) + tid);
        }
        x[b][0] = bf_lo(hv.x); x[b][1] = bf_hi(hv.x); x[b][2] = bf_lo(hv.y); x[b][3] = bf_hi(hv.y);
        if (a.tp_mode == 2) {
          // tensor parallel: hv is this rank's partial projection; add the peers' (pushed into this rank's
          // window by their projection kernels) in rank order and round once, like the unfused exchange
          const unsigned int tag = exchange_tag(a.tp_step, a.tp_slot);
          float acc[4] = {0.f, 0.f, 0.f, 0.f};
          for (int r = 0; r < a.tp_size; ++r) {
            if (r == a.tp_rank) {
#pragma unroll
              for (int e = 0; e < 4; ++e) acc[e] += x[b][e];
            } else {
              uint32_t d[1][2];
              pull_words<1>(a.tp_window[a.tp_rank], a.tp_slot & 1, r, b * 512 + 2 * tid, 1, tag, a.status,
                            a.tp_wait_ns, d);
              acc[0] += bf_lo(d[0][0]); acc[1] += bf_hi(d[0][0]); acc[2] += bf_lo(d[0][1]); acc[3] += bf_hi(d[0][1]);
            }
          }
#pragma unroll
          for (int e = 0; e < 4; ++e) x[b][e] = round_bf16(acc[e]);
        }
        x[b][0] += bf_lo(rv.x); x[b][1] += bf_hi(rv.x); x[b][2] += bf_lo(rv.y); x[b][3] += bf_hi(rv.y);
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
      for (int w = 0; w < W; ++w) tot += ssq[w][b];
      const float rstd = 1.0f / sqrtf(tot / (float)K + a.eps);
      float4 y;
      y.x = round_bf16(round_bf16(x[b][0] * rstd) * w0); y.y = round_bf16(round_bf16(x[b][1] * rstd) * w1);
      y.z = round_bf16(round_bf16(x[b][2] * rstd) * w2); y.w = round_bf16(round_bf16(x[b][3] * rstd) * w3);
      reinterpret_cast<float4*>(xs[b])[tid] = y;
    }
  } else if (NB > 2) {
#pragma unroll
    for (int b = 0; b < NB; ++b)
      for (int c = tid; c < K / 8; c += C::kThreads) {
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
  constexpr bool kDirectX = !kNorm && NB <= 2;   // plain x, one or two rows: each lane loads its 8 values itself
  if (!kDirectX) __syncthreads();
  if (a.late_trigger) pdl_launch_dependents();
  if (threadIdx.x == 0) trace_max(a.trace, 4);

  // this lane's 8 values of x per batch row (kept in registers for one or two rows)
  float xr[NB <= 2 ? NB : 1][8];
#pragma unroll
  for (int b = 0; b < (NB <= 2 ? NB : 0); ++b) {
    if (kDirectX) {
      if (b < a.rows) unpack8(ldg_cg(a.x + (size_t)b * K + col), xr[b]);
      else {
#pragma unroll
        for (int e = 0; e < 8; ++e) xr[b][e] = 0.f;
      }
      continue;
    }
    const float4 x0 = *reinterpret_cast<const float4*>(&xs[b][col]);
    const float4 x1 = *reinterpret_cast<const float4*>(&xs[b][col + 4]);
    xr[b][0] = x0.x; xr[b][1] = x0.y; xr[b][2] = x0.z; xr[b][3] = x0.w;
    xr[b][4] = x1.x; xr[b][5] = x1.y; xr[b][6] = x1.z; xr[b][7] = x1.w;
  }

  float best_v = -INFINITY;   // epilogue thread (b, r): running argmax of its rows
  int best_i = 0x7fffffff;
  const int eb = tid / RC, er = tid % RC;   // epilogue thread -> (batch row, row of the group), tid < RC * NB
  __shared__ SampleRow srows[kMaxRows];
  if (MODE == kModeNormArgmax) sample_rows_load(a, srows, tid);   // a CTA barrier follows before the first epilogue

  // ---- row groups of this CTA ----
  for (int it = 0; grp < n_groups; grp += gridDim.x, ++it) {
    // 8 rows x 8 columns per lane, two batch rows at a time: partial dot products
    // p[b][i], then a halving butterfly over the lanes of a row half, after which
    // lane lc holds the sum over the warp's slice for row (lc & 7)
    constexpr int BP = NB < 2 ? 1 : 2;
    const int nxt = grp + gridDim.x;
#pragma unroll
    for (int b0 = 0; b0 < NB; b0 += BP) {
      float xv[BP][8];
#pragma unroll
      for (int bb = 0; bb < BP; ++bb) {
        if (NB <= 2) {
#pragma unroll
          for (int e = 0; e < 8; ++e) xv[bb][e] = xr[NB <= 2 ? b0 + bb : 0][e];
        } else {   // larger batches re-read x from shared memory instead of holding 8 x NB registers
          const float4 x0 = *reinterpret_cast<const float4*>(&xs[b0 + bb][col]);
          const float4 x1 = *reinterpret_cast<const float4*>(&xs[b0 + bb][col + 4]);
          xv[bb][0] = x0.x; xv[bb][1] = x0.y; xv[bb][2] = x0.z; xv[bb][3] = x0.w;
          xv[bb][4] = x1.x; xv[bb][5] = x1.y; xv[bb][6] = x1.z; xv[bb][7] = x1.w;
        }
      }
      float p[BP][8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float wf[8];
        unpack8(wreg[i], wf);
#pragma unroll
        for (int bb = 0; bb < BP; ++bb) {
          float s0 = wf[0] * xv[bb][0], s1 = wf[1] * xv[bb][1];
          s0 = fmaf(wf[2], xv[bb][2], s0); s1 = fmaf(wf[3], xv[bb][3], s1);
          s0 = fmaf(wf[4], xv[bb][4], s0); s1 = fmaf(wf[5], xv[bb][5], s1);
          s0 = fmaf(wf[6], xv[bb][6], s0); s1 = fmaf(wf[7], xv[bb][7], s1);
          p[bb][i] = s0 + s1;
        }
      }
      if (b0 + BP >= NB && nxt < n_groups) {   // the weight registers are free: request the next group's
#pragma unroll
        for (int i = 0; i < 8; ++i) wreg[i] = ldg_stream(weight_ptr(nxt, i));
      }
#pragma unroll
      for (int bb = 0; bb < BP; ++bb) {
        float q4[4], q2[2], q1;
        const bool k4 = lc & 4, k2 = lc & 2, k1 = lc & 1;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float mine = k4 ? p[bb][4 + k] : p[bb][k], other = k4 ? p[bb][k] : p[bb][4 + k];
          q4[k] = mine + __shfl_xor_sync(0xffffffffu, other, 4);
        }
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          const float mine = k2 ? q4[2 + k] : q4[k], other = k2 ? q4[k] : q4[2 + k];
          q2[k] = mine + __shfl_xor_sync(0xffffffffu, other, 2);
        }
        {
          const float mine = k1 ? q2[1] : q2[0], other = k1 ? q2[0] : q2[1];
          q1 = mine + __shfl_xor_sync(0xffffffffu, other, 1);
        }
        q1 += __shfl_xor_sync(0xffffffffu, q1, 8);
        if (LPR == 32) q1 += __shfl_xor_sync(0xffffffffu, q1, 16);
        if (lc < 8) red[warp][b0 + bb][hr * 8 + lc] = q1;
      }
    }
    if (threadIdx.x == 0 && it == 0) trace_max(a.trace, 5);
    __syncthreads();
    if (MODE == kModeStore) {
      // narrow shards have fewer threads than outputs of a group: loop (same trip count for every thread)
      const bool push = a.tp_mode == 1;
      const unsigned int tag = push ? exchange_tag(a.tp_step, a.tp_slot) : 0u;
      for (int t0 = 0; t0 < RC * NB; t0 += C::kThreads) {
        const int t = t0 + tid;
        const bool act = t < RC * NB;
        const int b = act ? t / RC : 0, r = act ? t % RC : 0;
        float v = 0.f;
        if (act) {
#pragma unroll
          for (int w = 0; w < W; ++w) v += red[w][b][r];
        }
        v = round_bf16(v);
        const float vn = __shfl_down_sync(0xffffffffu, v, 1);   // the next row's value (same batch row: RC is even)
        if (act && b < a.rows) {
          a.out[(size_t)b * a.out_stride + grp * RC + r] = __float2bfloat16_rn(v);
          if (push && !(r & 1)) {
            // tensor parallel: the same two values as one tagged word into every peer's window
            const uint2 word = make_uint2(pack_bf16(v, vn), tag);
            const size_t wi = (size_t)b * 512 + (size_t)(grp * RC + r) / 2;
            for (int p = 0; p < a.tp_size; ++p)
              if (p != a.tp_rank) inbox_words(a.tp_window[p], a.tp_slot & 1, a.tp_rank)[wi] = word;
          }
        }
      }
    } else {
      float v = 0.f;
      if (tid < RC * NB) {
#pragma unroll
        for (int w = 0; w < W; ++w) v += red[w][eb][er];
        v = round_bf16(v);
      }
      if (MODE == kModeNormSwiglu) {
        // rows 0-7 of the group are gate rows, rows 8-15 the matching up rows
        const float up = __shfl_down_sync(0xffffffffu, v, 8);
        if (tid < RC * NB && er < 8 && eb < a.rows)
          a.out[(size_t)eb * a.out_stride + grp * 8 + er] = __float2bfloat16_rn(v / (1.0f + expf(-v)) * up);
      } else if (tid < RC * NB && eb < a.rows) {
        const int row = grp * RC + er;
        if (MODE == kModeNormArgmax) {
          if (a.logits_out) a.logits_out[(size_t)eb * a.vocab + row] = v;
          const float key = a.temps ? sample_key(a.sample_seed, a.sample_idx_offset, srows, eb, row, v) : v;
          if (key > best_v || (key == best_v && row < best_i)) { best_v = key; best_i = row; }
        } else {
          a.out[(size_t)eb * a.out_stride + row] = __float2bfloat16_rn(v);
        }
      }
    }
    if (nxt < n_groups) __syncthreads();   // `red` is reused by the next group
  }

  if (warp == 0 && a.ahead_late) l2_prefetch_slice(a.ahead_ptr, a.ahead_bytes, blockIdx.x, gridDim.x);
  if (MODE == kModeNormArgmax) {
    // threads (b, r) -> one partial per batch row and CTA -> grid (the last CTA to arrive finishes)
    if (tid < 128) {
#pragma unroll
      for (int m = RC / 2; m >= 1; m >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best_v, m);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, m);
        if (ov > best_v || (ov == best_v && oi < best_i)) { best_v = ov; best_i = oi; }
      }
      if (tid < RC * NB && er == 0) a.parts[blockIdx.x * kMaxRows + eb] = ArgmaxPart{best_v, best_i};
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) last_flag = (atomicAdd(a.ticket, 1u) == gridDim.x - 1) ? 1 : 0;
    __syncthreads();
    if (last_flag) {
      __threadfence();
      for (int b = warp; b < a.rows; b += W) {
        float v = -INFINITY;
        int i = 0x7fffffff;
        for (int c3 = lane; c3 < (int)gridDim.x; c3 += 32) {
          const int2 raw = __ldcg(reinterpret_cast<const int2*>(a.parts + c3 * kMaxRows + b));
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
          if (a.best_out) a.best_out[b] = ArgmaxPart{v, i};
        }
      }
      if (tid == 0) { *a.ticket = 0u; sample_advance(a); }
    }
  }
  if (threadIdx.x == 0) trace_max(a.trace, 2);
}

}  // namespace dfb
