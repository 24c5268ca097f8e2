// Weight-streaming skinny GEMM for 3..8 batch rows at K = 1024 with the WEIGHTS
// on the M side of mma.sync.m16n8k16 (16 weight rows x 8 batch rows per MMA).
//
// stream_gemv_kernel puts the batch on M, where rows 8..15 of every MMA are
// zero padding; mma.sync issues only about once per 38 cycles per SM
// sub-partition on this part, so half of that scarce issue rate is wasted.
// Here one MMA covers 16 weight rows, which halves the MMAs per weight byte.
//
//   * a tile is 16 weight rows x K (SwiGLU: 8 gate rows + the 8 matching up
//     rows), fetched by 16 bulk copies (TMA, untiled) into a shared-memory
//     stage with rows padded by 64 bytes; the first PSTAGES tiles are requested
//     before the dependency wait;
//   * the 8 warps split K (128 columns each); lane (g = lane/4, t = lane%4)
//     reads 16 bytes of rows g and g+8 per 32-column block (A fragments of two
//     MMAs, conflict-free thanks to the padding) and the matching 16 bytes of
//     x[batch g] (B fragments) from a bf16 copy of x in shared memory;
//   * the residual add + RMSNorm is done ONE WARP PER BATCH ROW: the rows of h
//     and of the residual arrive by bulk copies (TMA), a lane owns four 16-byte
//     pieces of its row, the sum of squares needs one butterfly and no
//     cross-warp step, every lane computes one root, and the normalised row is
//     written in place; the eight rows proceed in parallel without a barrier
//     between them (with every thread handling all rows, the cross-warp
//     reduction and eight roots per thread made this prologue the longest part
//     of the kernel after its dependency);
//   * cross-warp reduction in shared memory, one thread per output for the
//     epilogue (store / SwiGLU / logits + greedy argmax);
//   * PSTAGES = 0 keeps the weights in REGISTERS instead of shared-memory
//     stages: lane (g, t) loads the 16-byte pieces of rows g and g + 8 it would
//     have read from the stage straight from global memory (eight 128-bit
//     loads per tile, requested before the dependency wait; the next tile's
//     once the MMAs have consumed them).  The CTA then holds 33 KB of shared
//     memory instead of 101-135 KB, so that it fits on an SM beside its
//     predecessor's CTAs and its weights stream while that kernel still runs,
//     as in the FP32 chain.
#pragma once

#include "dfb_exchange.cuh"
#include "dfb_kernels.cuh"

namespace dfb {

struct PairSmem {
  static constexpr int kK = 1024;
  static constexpr int kRowStride = 2 * kK + 64;       // bytes
  static constexpr int kStageBytes = 16 * kRowStride;  // 33,792
  static constexpr int kXBytes = kMaxRows * kRowStride; // bf16 copy of x, same padding
  static constexpr int kResBytes = kMaxRows * 2 * kK;   // residual rows as fetched by the bulk copies
  static constexpr int bytes(int stages) { return stages * kStageBytes + kXBytes + kResBytes + 8 * (stages + 1) + 16; }
};

template <int PSTAGES, int MODE>
__global__ void __launch_bounds__(256, 2) pair_gemv_kernel(const GemvArgs a) {
  constexpr bool kNorm = MODE != kModeStore;
  constexpr bool kReg = PSTAGES == 0;     // weights in registers, no shared-memory stages
  constexpr int kStagesOr1 = kReg ? 1 : PSTAGES;
  constexpr int K = PairSmem::kK, kWarps = 8;
  using SM = PairSmem;
  if (!a.late_trigger) pdl_launch_dependents();
  if (threadIdx.x == 0) trace_min(a.trace, 0);

  extern __shared__ __align__(128) unsigned char dyn_smem[];
  unsigned char* stage_base = dyn_smem;
  unsigned char* xsb = dyn_smem + PSTAGES * SM::kStageBytes;                 // [8][kRowStride] bf16 x
  unsigned char* rstage = xsb + SM::kXBytes;                                 // [8][2 K] residual rows
  uint64_t* full = reinterpret_cast<uint64_t*>(rstage + SM::kResBytes);
  uint64_t* x_in = full + PSTAGES;
  __shared__ float red[2][kWarps][128];
  __shared__ float ssq[kWarps][kMaxRows];
  __shared__ ArgmaxPart wpart[4][kMaxRows];
  __shared__ int last_flag;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int kbase = warp * 128 + 8 * t;   // this lane's first column
  const int stride = gridDim.x;

  // row r (0..15) of tile `tile`
  auto weight_row = [&](int tile, int r) -> const __nv_bfloat16* {
    int row;
    if (MODE == kModeNormSwiglu) row = (r >= 8 ? a.gate_rows : 0) + tile * 8 + (r & 7);
    else row = tile * 16 + r;
    return a.w + (size_t)row * K;
  };
  auto request_tile = [&](int tile, int s) {
    if (lane == 0) mbar_expect_tx(&full[s], 16 * 2 * K);
    __syncwarp();
    if (lane < 16)
      bulk_g2s(stage_base + s * SM::kStageBytes + lane * SM::kRowStride, weight_row(tile, lane), 2 * K, &full[s]);
  };

  // ---- weight prefetch, independent of the previous kernel ----
  uint4 wu[4], wv[4];   // kReg: rows g and g + 8 of the current tile, this lane's piece of each 32-column block
  if (kReg) {
    if (blockIdx.x < a.n_tiles) {
      const __nv_bfloat16* r0 = weight_row(blockIdx.x, g) + kbase;
      const __nv_bfloat16* r1 = weight_row(blockIdx.x, g + 8) + kbase;
#pragma unroll
      for (int j = 0; j < 4; ++j) { wu[j] = ldg_stream(r0 + 32 * j); wv[j] = ldg_stream(r1 + 32 * j); }
    }
  }
  if (warp == 0) {
    if (lane == 0) {
#pragma unroll
      for (int s = 0; s < PSTAGES; ++s) mbar_init(&full[s], 1);
      mbar_init(x_in, 1);
      fence_mbar_init();
      // the activation rows' byte count is posted here, long before any of their copies can complete
      if (kNorm && a.ids == nullptr && a.res_in != nullptr && a.tp_mode != 2) mbar_expect_tx(x_in, (uint32_t)(a.rows * 4 * K));
    }
    __syncwarp();
#pragma unroll
    for (int s = 0; s < PSTAGES; ++s) {
      const int tl = blockIdx.x + s * stride;
      if (tl < a.n_tiles) request_tile(tl, s);
    }
  }
  uint2 nwv = make_uint2(0, 0);
  if (kNorm) nwv = *reinterpret_cast<const uint2*>(a.norm_w + 4 * tid);
  uint4 nw4[4];   // row-per-warp prologue: the norm weights of this lane's four 16-byte pieces
#pragma unroll
  for (int c = 0; c < 4; ++c) nw4[c] = kNorm ? ldg_stream(a.norm_w + 8 * (32 * c + lane)) : make_uint4(0, 0, 0, 0);
  if (warp == 1) l2_prefetch_slice(a.ahead_ptr, a.ahead_bytes, blockIdx.x, gridDim.x);
  __syncthreads();  // the barriers are initialised before anyone polls them

  pdl_wait();
  if (threadIdx.x == 0) { trace_max(a.trace, 1); trace_min(a.trace, 3); }

  // ---- x (bf16) into shared memory, with the fused residual add + RMSNorm ----
  const bool bulk_x = kNorm && a.ids == nullptr && a.res_in != nullptr && a.tp_mode != 2;
  if (kNorm && bulk_x) {
    // warp b owns batch row b; lane l owns the 16-byte pieces l, l + 32, l + 64, l + 96 of the row
    if (tid < 16) {                       // sixteen threads issue one row copy each
      const int b = tid & 7;
      if (b < a.rows) {
        if (tid < 8) bulk_g2s(xsb + b * SM::kRowStride, a.x + (size_t)b * K, 2 * K, x_in);
        else bulk_g2s(rstage + b * 2 * K, a.res_in + (size_t)b * K, 2 * K, x_in);
      }
    }
    if (!__syncthreads_and(mbar_wait_bounded(x_in, 0) ? 1 : 0))
      report_status(a.status, kStatusCopyTimeout, kKernelGemv, blockIdx.x, -1);
    if (a.late_trigger) pdl_launch_dependents();
    const int b = warp;
    unsigned char* xrow = xsb + b * SM::kRowStride;
    if (b < a.rows) {
      float x[4][8];
      float ss = 0.f;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const uint4 hv = *reinterpret_cast<const uint4*>(xrow + 16 * (32 * c + lane));
        const uint4 rv = *reinterpret_cast<const uint4*>(rstage + b * 2 * K + 16 * (32 * c + lane));
        float hf[8], rf[8];
        unpack8(hv, hf);
        unpack8(rv, rf);
#pragma unroll
        for (int e = 0; e < 8; ++e) { x[c][e] = hf[e] + rf[e]; ss = fmaf(x[c][e], x[c][e], ss); }
      }
      if (a.res_out && blockIdx.x == 0) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint4 o;
          o.x = pack_bf16(x[c][0], x[c][1]); o.y = pack_bf16(x[c][2], x[c][3]);
          o.z = pack_bf16(x[c][4], x[c][5]); o.w = pack_bf16(x[c][6], x[c][7]);
          *reinterpret_cast<uint4*>(a.res_out + (size_t)b * K + 8 * (32 * c + lane)) = o;
        }
      }
#pragma unroll
      for (int m = 16; m >= 1; m >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, m);
      const float rstd = 1.0f / sqrtf(ss / (float)K + a.eps);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        float wf[8], y[8];
        unpack8(nw4[c], wf);
#pragma unroll
        for (int e = 0; e < 8; ++e) y[e] = round_bf16(x[c][e] * rstd) * wf[e];
        uint4 o;
        o.x = pack_bf16(y[0], y[1]); o.y = pack_bf16(y[2], y[3]); o.z = pack_bf16(y[4], y[5]); o.w = pack_bf16(y[6], y[7]);
        *reinterpret_cast<uint4*>(xrow + 16 * (32 * c + lane)) = o;    // in place: this lane read exactly these bytes
      }
    } else {
#pragma unroll
      for (int c = 0; c < 4; ++c) *reinterpret_cast<uint4*>(xrow + 16 * (32 * c + lane)) = make_uint4(0, 0, 0, 0);
    }
  } else if (kNorm) {
    float x[kMaxRows][4];
    uint2 hv[kMaxRows], rv[kMaxRows];
#pragma unroll
    for (int b = 0; b < kMaxRows; ++b) {
      hv[b] = make_uint2(0, 0);
      rv[b] = make_uint2(0, 0);
      if (b < a.rows) {
        const size_t xrow = a.ids ? (size_t)clamp_token(a.ids[b], a.embed_rows, a.status, b) : (size_t)b;
        hv[b] = __ldcg(reinterpret_cast<const uint2*>(a.x + xrow * K) + tid);
        if (a.res_in) rv[b] = __ldcg(reinterpret_cast<const uint2*>(a.res_in + (size_t)b * K) + tid);
      }
    }
#pragma unroll
    for (int b = 0; b < kMaxRows; ++b) {
      x[b][0] = bf_lo(hv[b].x); x[b][1] = bf_hi(hv[b].x); x[b][2] = bf_lo(hv[b].y); x[b][3] = bf_hi(hv[b].y);
    }
    if (a.tp_mode == 2) {
      // tensor parallel: hv holds this rank's partial projection; add the peers' (pushed into this rank's
      // window by their projection kernels) in rank order and round once, like the unfused exchange
      const unsigned int tag = exchange_tag(a.tp_step, a.tp_slot);
      float acc[kMaxRows][4];
#pragma unroll
      for (int b = 0; b < kMaxRows; ++b)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[b][e] = 0.f;
      for (int r = 0; r < a.tp_size; ++r) {
        if (r == a.tp_rank) {
#pragma unroll
          for (int b = 0; b < kMaxRows; ++b)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[b][e] += x[b][e];
        } else {
          uint32_t d[kMaxRows][2];
          pull_words<kMaxRows>(a.tp_window[a.tp_rank], a.tp_slot & 1, r, 2 * tid, a.rows, tag, a.status,
                               a.tp_wait_ns, d);
#pragma unroll
          for (int b = 0; b < kMaxRows; ++b) {
            acc[b][0] += bf_lo(d[b][0]); acc[b][1] += bf_hi(d[b][0]);
            acc[b][2] += bf_lo(d[b][1]); acc[b][3] += bf_hi(d[b][1]);
          }
        }
      }
#pragma unroll
      for (int b = 0; b < kMaxRows; ++b)
#pragma unroll
        for (int e = 0; e < 4; ++e) x[b][e] = round_bf16(acc[b][e]);
    }
#pragma unroll
    for (int b = 0; b < kMaxRows; ++b) {
      x[b][0] += bf_lo(rv[b].x); x[b][1] += bf_hi(rv[b].x);
      x[b][2] += bf_lo(rv[b].y); x[b][3] += bf_hi(rv[b].y);
      if (a.res_out && blockIdx.x == 0 && b < a.rows)
        reinterpret_cast<uint2*>(a.res_out + (size_t)b * K)[tid] =
            make_uint2(pack_bf16(x[b][0], x[b][1]), pack_bf16(x[b][2], x[b][3]));
      float ss = x[b][0] * x[b][0] + x[b][1] * x[b][1] + x[b][2] * x[b][2] + x[b][3] * x[b][3];
#pragma unroll
      for (int m = 16; m >= 1; m >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, m);
      if (lane == 0) ssq[warp][b] = ss;
    }
    __syncthreads();
    const float w0 = bf_lo(nwv.x), w1 = bf_hi(nwv.x), w2 = bf_lo(nwv.y), w3 = bf_hi(nwv.y);
#pragma unroll
    for (int b = 0; b < kMaxRows; ++b) {
      float tot = 0.f;
#pragma unroll
      for (int w = 0; w < kWarps; ++w) tot += ssq[w][b];
      const float rstd = 1.0f / sqrtf(tot / (float)K + a.eps);
      // rows beyond the batch are zero (x is zero there)
      const uint2 y = make_uint2(pack_bf16(round_bf16(x[b][0] * rstd) * w0, round_bf16(x[b][1] * rstd) * w1),
                                 pack_bf16(round_bf16(x[b][2] * rstd) * w2, round_bf16(x[b][3] * rstd) * w3));
      *reinterpret_cast<uint2*>(xsb + b * SM::kRowStride + 8 * tid) = y;
    }
  } else {
#pragma unroll
    for (int b = 0; b < kMaxRows; ++b)
      if (tid < K / 8) {
        const uint4 v = b < a.rows ? ldg_cg(a.x + (size_t)b * K + 8 * tid) : make_uint4(0, 0, 0, 0);
        *reinterpret_cast<uint4*>(xsb + b * SM::kRowStride + 16 * tid) = v;
      }
  }
  __syncthreads();
  uint4 xa[4];   // B fragments: x[batch g], this lane's 8 columns of each 32-column block
#pragma unroll
  for (int j = 0; j < 4; ++j) xa[j] = *reinterpret_cast<const uint4*>(xsb + g * SM::kRowStride + 2 * (kbase + 32 * j));
  if (a.late_trigger) pdl_launch_dependents();
  if (threadIdx.x == 0) trace_max(a.trace, 4);

  // ---- main loop over this CTA's tiles ----
  const int er = tid >> 3, eb = tid & 7;  // epilogue thread (tid < 128) -> (tile row, batch row)
  float best_v = -INFINITY;
  int best_i = 0x7fffffff;
  __shared__ SampleRow srows[kMaxRows];
  if (MODE == kModeNormArgmax) sample_rows_load(a, srows, tid);   // a CTA barrier follows before the first epilogue
  int it = 0;
  bool copy_ok = true;
  for (int tile = blockIdx.x; tile < a.n_tiles; tile += stride, ++it) {
    const int s = it % kStagesOr1;
    if (!kReg && !mbar_wait_bounded(&full[s], (it / kStagesOr1) & 1)) { copy_ok = false; break; }
    const unsigned char* w0p = stage_base + s * SM::kStageBytes + g * SM::kRowStride + 2 * kbase;
    const unsigned char* w1p = w0p + 8 * SM::kRowStride;
    float c[4][4];
#pragma unroll
    for (int q = 0; q < 4; ++q) { c[q][0] = 0.f; c[q][1] = 0.f; c[q][2] = 0.f; c[q][3] = 0.f; }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint4 u = kReg ? wu[j] : *reinterpret_cast<const uint4*>(w0p + 64 * j);   // row g
      const uint4 v = kReg ? wv[j] : *reinterpret_cast<const uint4*>(w1p + 64 * j);   // row g + 8
      mma_bf16_16816_full(c[(2 * j) & 3], u.x, v.x, u.y, v.y, xa[j].x, xa[j].y);
      mma_bf16_16816_full(c[(2 * j + 1) & 3], u.z, v.z, u.w, v.w, xa[j].z, xa[j].w);
    }
    if (kReg) {   // the weight registers are free: request the next tile's
      const int nxt = tile + stride;
      if (nxt < a.n_tiles) {
        const __nv_bfloat16* r0 = weight_row(nxt, g) + kbase;
        const __nv_bfloat16* r1 = weight_row(nxt, g + 8) + kbase;
#pragma unroll
        for (int j = 0; j < 4; ++j) { wu[j] = ldg_stream(r0 + 32 * j); wv[j] = ldg_stream(r1 + 32 * j); }
      }
    }
    if (threadIdx.x == 0 && it == 0) trace_max(a.trace, 5);
    // C: (row g, batch 2t, 2t+1) in [0],[1]; (row g+8, ...) in [2],[3]; red index = row * 8 + batch
    float* r = red[it & 1][warp];
    *reinterpret_cast<float2*>(r + g * 8 + 2 * t) =
        make_float2((c[0][0] + c[1][0]) + (c[2][0] + c[3][0]), (c[0][1] + c[1][1]) + (c[2][1] + c[3][1]));
    *reinterpret_cast<float2*>(r + (g + 8) * 8 + 2 * t) =
        make_float2((c[0][2] + c[1][2]) + (c[2][2] + c[3][2]), (c[0][3] + c[1][3]) + (c[2][3] + c[3][3]));
    __syncthreads();  // every warp is done with stage s
    if (!kReg && warp == 0) {
      const int nxt = tile + PSTAGES * stride;
      if (nxt < a.n_tiles) request_tile(nxt, s);
    }
    if (MODE == kModeNormSwiglu) {
      if (tid < 64) {   // (gate row er, batch eb); the matching up row is 8 rows further
        float gv = 0.f, uv = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) { gv += red[it & 1][w][tid]; uv += red[it & 1][w][tid + 64]; }
        gv = round_bf16(gv);
        uv = round_bf16(uv);
        if (eb < a.rows)
          a.out[(size_t)eb * a.out_stride + tile * 8 + er] = __float2bfloat16_rn(gv / (1.0f + expf(-gv)) * uv);
      }
    } else if (tid < 128) {
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < kWarps; ++w) v += red[it & 1][w][tid];
      v = round_bf16(v);
      const int idx = tile * 16 + er;
      if (eb < a.rows) {
        if (MODE == kModeNormArgmax) {
          if (a.logits_out) a.logits_out[(size_t)eb * a.vocab + idx] = v;
          const float key = a.temps ? sample_key(a.sample_seed, a.sample_idx_offset, srows, eb, idx, v) : v;
          if (key > best_v || (key == best_v && idx < best_i)) { best_v = key; best_i = idx; }
        } else {
          a.out[(size_t)eb * a.out_stride + idx] = __float2bfloat16_rn(v);
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
    for (int s = 0; s < PSTAGES; ++s) mbar_wait_bounded(&full[s], 0);
  }

  if (MODE == kModeNormArgmax) {
    // threads (er, eb), tid = er * 8 + eb: over er within the warp (lane bits 3, 4), over the 4 warps, over CTAs
    if (tid < 128) {
#pragma unroll
      for (int m = 8; m <= 16; m <<= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best_v, m);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, m);
        if (ov > best_v || (ov == best_v && oi < best_i)) { best_v = ov; best_i = oi; }
      }
      if (lane < 8) wpart[warp][lane] = ArgmaxPart{best_v, best_i};
    }
    __syncthreads();
    if (tid < kMaxRows) {
      ArgmaxPart p = wpart[0][tid];
#pragma unroll
      for (int w = 1; w < 4; ++w) {
        const ArgmaxPart q = wpart[w][tid];
        if (q.value > p.value || (q.value == p.value && q.index < p.index)) p = q;
      }
      a.parts[blockIdx.x * kMaxRows + tid] = p;
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

// o_proj / down_proj (K = 2048 / 3072, plain store) for 2..8 batch rows with the weights in registers, the
// companion of pair_gemv_kernel<0, ...>: a CTA owns tiles of 8 weight rows, its 8 or 12 warps split K (256
// columns each), lane (g, t) holds the 16-byte pieces of row g for the warp's eight 32-column blocks (eight
// 128-bit loads per tile, requested before the dependency wait) and, once the dependency has resolved, the
// matching pieces of x[batch g] straight from global memory; rows 8..15 of each MMA are zero.  No shared-memory
// staging at all (2-3 KB for the cross-warp reduction), so the CTA is resident beside its predecessor.
template <int K>
__global__ void __launch_bounds__(K / 256 * 32, 2) reg_store_gemv_kernel(const GemvArgs a) {
  constexpr int W = K / 256;
  static_assert(K == 2048 || K == 3072, "o_proj and down_proj widths");
  if (!a.late_trigger) pdl_launch_dependents();
  if (threadIdx.x == 0) trace_min(a.trace, 0);
  __shared__ float red[2][W][64];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int kbase = warp * 256 + 8 * t;
  const int stride = gridDim.x;

  uint4 wu[8];
  int tile = blockIdx.x;
  if (tile < a.n_tiles) {
    const __nv_bfloat16* r0 = a.w + (size_t)(tile * 8 + g) * K + kbase;
#pragma unroll
    for (int j = 0; j < 8; ++j) wu[j] = ldg_stream(r0 + 32 * j);
  }
  if (warp == 1) l2_prefetch_slice(a.ahead_ptr, a.ahead_bytes, blockIdx.x, gridDim.x);

  pdl_wait();
  if (threadIdx.x == 0) { trace_max(a.trace, 1); trace_min(a.trace, 3); }
  uint4 xa[8];   // B fragments: x[batch g], this lane's 8 columns of each 32-column block
#pragma unroll
  for (int j = 0; j < 8; ++j)
    xa[j] = g < a.rows ? ldg_cg(a.x + (size_t)g * K + kbase + 32 * j) : make_uint4(0, 0, 0, 0);
  if (a.late_trigger) pdl_launch_dependents();
  if (threadIdx.x == 0) trace_max(a.trace, 4);

  for (int it = 0; tile < a.n_tiles; tile += stride, ++it) {
    float c[4][4];
#pragma unroll
    for (int q = 0; q < 4; ++q) { c[q][0] = 0.f; c[q][1] = 0.f; c[q][2] = 0.f; c[q][3] = 0.f; }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      mma_bf16_16816_full(c[(2 * j) & 3], wu[j].x, 0u, wu[j].y, 0u, xa[j].x, xa[j].y);
      mma_bf16_16816_full(c[(2 * j + 1) & 3], wu[j].z, 0u, wu[j].w, 0u, xa[j].z, xa[j].w);
    }
    const int nxt = tile + stride;
    if (nxt < a.n_tiles) {
      const __nv_bfloat16* r0 = a.w + (size_t)(nxt * 8 + g) * K + kbase;
#pragma unroll
      for (int j = 0; j < 8; ++j) wu[j] = ldg_stream(r0 + 32 * j);
    }
    if (threadIdx.x == 0 && it == 0) trace_max(a.trace, 5);
    // C: (row g, batch 2t, 2t+1) in [0], [1]; red index = row * 8 + batch
    *reinterpret_cast<float2*>(&red[it & 1][warp][g * 8 + 2 * t]) =
        make_float2((c[0][0] + c[1][0]) + (c[2][0] + c[3][0]), (c[0][1] + c[1][1]) + (c[2][1] + c[3][1]));
    __syncthreads();
    if (tid < 64) {
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < W; ++w) v += red[it & 1][w][tid];
      const int er = tid >> 3, eb = tid & 7;
      if (eb < a.rows) a.out[(size_t)eb * a.out_stride + tile * 8 + er] = __float2bfloat16_rn(v);
    }
    if (threadIdx.x == 0 && it == 0) trace_max(a.trace, 6);
  }
  if (threadIdx.x == 0) trace_max(a.trace, 2);
}

}  // namespace dfb
