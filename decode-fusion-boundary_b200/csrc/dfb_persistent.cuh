// The whole decode step as ONE persistent kernel (ordinary launch, one CTA per
// SM, no cooperative groups, no grid-wide barrier).
//
//   * Warp 8 of every CTA is a TMA producer: it walks the CTA's static list of
//     weight "units" (8 rows x 1024 columns = 16 KB) for all layers and streams
//     them with bulk copies into a 12-slot shared-memory ring, throttled only by
//     the ring.  The HBM stream therefore never stops at an op boundary and is
//     never burstier than 12 units per SM.
//   * Warps 0-7 are consumers.  For every op (qkv, attention, o_proj, gate/up,
//     down per layer, then the LM head) they obtain the op's input vector, run
//     m16n8k16 MMAs on the units that have landed, and publish their outputs.
//   * Activations cross CTAs in 8-byte words {two bf16 values, 32-bit tag}
//     written with one store and polled with plain volatile loads: the tag
//     (step epoch, layer, op) says whether the data is there, so the dependency
//     between ops costs one store -> L2 -> load round trip and nothing is ever
//     zeroed.  Every poll is bounded: on expiry the CTA records a status word and
//     the whole grid fast-forwards to the end instead of hanging.
//   * The residual stream never leaves the SM: every CTA keeps the fragments it
//     needs in registers.
#pragma once

#include "dfb_kernels.cuh"

namespace dfb {

constexpr int kPConsumerWarps = 8;
constexpr int kPConsumers = kPConsumerWarps * 32;     // 256
constexpr int kPThreads = kPConsumers + 32;           // + the producer warp
constexpr int kUnitCols = 1024;
constexpr int kUnitBytes = kTileRows * kUnitCols * 2; // 16 KB: one bulk copy (two for a gate/up tile)
constexpr int kPSlots = 12;
constexpr int kRound = 4;                             // tiles reduced behind one barrier
template <int N> struct IntC { static constexpr int value = N; };
constexpr int kPDynSmem = kPSlots * kUnitBytes + 2 * kPSlots * 8 + 64;
constexpr int kHidden = 1024;

enum POp : int { kOpQkv = 0, kOpAttn = 1, kOpO = 2, kOpGateUp = 3, kOpDown = 4, kOpLmHead = 5 };
constexpr int kKernelPersistent = 3;
constexpr int kStatusPollTimeout = 4;
constexpr int kPollSpinLimit = 1 << 19;   // volatile-load round trips before giving up (~0.3 s)

struct PLayerWeights {   // same layout as DfbLayerWeights
  const __nv_bfloat16 *ln_in, *wqkv, *q_norm, *k_norm, *wo, *ln_post, *wgu, *wd;
};

struct PersistArgs {
  const PLayerWeights* layers;   // device array [n_layers]
  int n_layers;
  int rows;
  int q_heads, kv_heads;         // 16, 8
  int intermediate;              // 3072
  int vocab;
  float eps, scale;
  const __nv_bfloat16* embed;
  const __nv_bfloat16* final_norm;
  const float* cos_sin;
  // step inputs (decoder staging buffers)
  const int* ids;
  const int* positions;
  const int* block_tables;
  int bt_stride;
  const int* row_active;
  // paged KV cache
  __nv_bfloat16* k_cache;
  __nv_bfloat16* v_cache;
  size_t kv_layer_elems;
  int block_size, num_blocks, max_pos;
  // tagged exchange buffers, [8 rows][values / 2] words each
  uint2* x_qkv;
  uint2* x_attn;
  uint2* x_hattn;
  uint2* x_act;
  uint2* x_hmlp;
  // split-KV partials, argmax partials, results
  float* part_o;
  float2* part_ml;
  unsigned int* tickets;         // [8 * kv_heads] attention, [8 * kv_heads] LM head
  ArgmaxPart* parts;             // [gridDim.x, 8]
  int* tokens;
  float* logits_out;
  unsigned int* epoch;           // step counter, advanced by the kernel itself
  int* status;
  unsigned long long* trace;     // [ops, 8] or null
};

__device__ __forceinline__ uint32_t p_tag(unsigned epoch, int layer, int op) {
  return (epoch << 12) | ((uint32_t)(layer + 1) << 3) | (uint32_t)op;
}
// Tile t of an op belongs to CTA (t + rot) mod G; rot differs per op and per
// layer so that the uneven remainders do not always hit the same CTAs.
__device__ __forceinline__ int p_rot(int layer, int op, int G) {
  // qkv 0, attention 100, o_proj 68, gate/up 48, down 20, LM head 0
  const int base = op == kOpAttn ? 100 : op == kOpO ? 68 : op == kOpGateUp ? 48 : op == kOpDown ? 20 : 0;
  return (base + layer * 53) % G;
}
__device__ __forceinline__ int p_first(int cta, int rot, int G) {
  int t = (cta - rot) % G;
  return t < 0 ? t + G : t;
}
__device__ __forceinline__ uint4 ld_volatile_v4(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint2 ld_volatile_v2(const void* p) {
  uint2 v;
  asm volatile("ld.volatile.global.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ int ld_volatile_s32(const int* p) {
  int v;
  asm volatile("ld.volatile.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_ll(uint2* p, uint32_t data, uint32_t tag) {
  asm volatile("st.global.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(data), "r"(tag) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void bar_consumers() { asm volatile("bar.sync 1, 256;" ::: "memory"); }
__device__ __forceinline__ void bar_attn() { asm volatile("bar.sync 2, 128;" ::: "memory"); }

// One bounded-wait step: true when the caller must stop waiting, either because
// some CTA already reported an error or because this wait ran out of patience.
__device__ __forceinline__ bool p_give_up(int& spins, int* status, int what, int index) {
  if ((++spins & 255) != 0) return false;
  if (ld_volatile_s32(status) != 0) return true;
  if (spins >= kPollSpinLimit) {
    report_status(status, kStatusPollTimeout, kKernelPersistent, what, index);
    return true;
  }
  return false;
}
__device__ __forceinline__ void p_wait_mbar(uint64_t* bar, uint32_t parity, int* status, int what) {
  int spins = 0;
  while (!mbar_try_wait(bar, parity))
    if (p_give_up(spins, status, what, (int)parity)) return;
}

// Poll NF fragments of 8 bf16 (= 4 tagged words = 32 bytes each) of one row.
// Fragment j covers columns first_col + 32 j .. + 7.
template <int NF>
__device__ __forceinline__ void ll_load_frags(const uint2* row_words, int first_col, uint32_t tag, uint4 (&out)[NF],
                                              int* status, int what) {
  int spins = 0;
  while (true) {
    uint4 lo[NF], hi[NF];
#pragma unroll
    for (int j = 0; j < NF; ++j) {
      const uint2* p = row_words + ((first_col + 32 * j) >> 1);
      lo[j] = ld_volatile_v4(p);
      hi[j] = ld_volatile_v4(p + 2);
    }
    bool ok = true;
#pragma unroll
    for (int j = 0; j < NF; ++j) {
      ok = ok && lo[j].y == tag && lo[j].w == tag && hi[j].y == tag && hi[j].w == tag;
      out[j] = make_uint4(lo[j].x, lo[j].z, hi[j].x, hi[j].z);
    }
    if (ok || p_give_up(spins, status, what, first_col)) return;
  }
}

struct PAttnSmem {
  float qs[2][kHeadDim];
  __align__(16) __nv_bfloat16 ks[kHeadDim];
  __align__(16) __nv_bfloat16 vs[kHeadDim];
  float mred[8][2];
  float lred[8][2];
  float ored[8][2][kHeadDim];
  int last_flag;
};

// ---- one attention work item: (row, kv head, 64-position split) --------------
__device__ __forceinline__ void p_attention_item(const PersistArgs& a, PAttnSmem& sm, int layer, int row, int kvh,
                                                 int split, int nsplits, int pos, uint32_t tag_in, uint32_t tag_out) {
  const int tid = threadIdx.x;  // 0..127
  const int warp = tid >> 5, lane = tid & 31;
  const int ctx = pos + 1;
  const int start = split * kAttnChunk;
  const int end = min(ctx, start + kAttnChunk);
  const bool owner = split == nsplits - 1;
  const int pg = tid >> 4, l16 = tid & 15;
  __nv_bfloat16* kc = a.k_cache + (size_t)layer * a.kv_layer_elems;
  __nv_bfloat16* vc = a.v_cache + (size_t)layer * a.kv_layer_elems;
  int block = a.block_tables[row * a.bt_stride + start / a.block_size];
  if (block < 0 || block >= a.num_blocks) {
    report_status(a.status, kStatusBadBlock, kKernelAttention, row, block);
    block = 0;
  }
  const size_t tok_stride = (size_t)a.kv_heads * kHeadDim;
  const size_t base = ((size_t)block * a.block_size + (start % a.block_size)) * tok_stride + (size_t)kvh * kHeadDim + 8 * l16;

  // old KV entries first: they do not depend on this layer's qkv
  uint4 kreg[8], vreg[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int p = start + pg + 8 * i;
    if (p < end && p != pos) {
      kreg[i] = ldg_stream(kc + base + (size_t)(pg + 8 * i) * tok_stride);
      vreg[i] = ldg_stream(vc + base + (size_t)(pg + 8 * i) * tok_stride);
    } else {
      kreg[i] = make_uint4(0, 0, 0, 0);
      vreg[i] = make_uint4(0, 0, 0, 0);
    }
  }

  // new token: q (2 heads) and k get RMSNorm + RoPE, v is copied
  const int q_size = a.q_heads * kHeadDim, kv_size = a.kv_heads * kHeadDim;
  const uint2* xrow = a.x_qkv + (size_t)row * ((q_size + 2 * kv_size) / 2);
  const PLayerWeights& lw = a.layers[layer];
  if (warp < 3) {
    const int col = warp < 2 ? (2 * kvh + warp) * kHeadDim : q_size + kvh * kHeadDim;
    const __nv_bfloat16* nw = warp < 2 ? lw.q_norm : lw.k_norm;
    const int d = 2 * lane;
    const uint32_t wlo = *reinterpret_cast<const uint32_t*>(nw + d);
    const uint32_t whi = *reinterpret_cast<const uint32_t*>(nw + d + 64);
    const float* cs = a.cos_sin + (size_t)pos * kHeadDim;
    const float2 c = *reinterpret_cast<const float2*>(cs + d);
    const float2 s = *reinterpret_cast<const float2*>(cs + 64 + d);
    uint2 lo, hi;
    int spins = 0;
    do {
      lo = ld_volatile_v2(xrow + ((col + d) >> 1));
      hi = ld_volatile_v2(xrow + ((col + d + 64) >> 1));
    } while ((lo.y != tag_in || hi.y != tag_in) && !p_give_up(spins, a.status, kOpAttn, col));
    float x[4] = {bf_lo(lo.x), bf_hi(lo.x), bf_lo(hi.x), bf_hi(hi.x)};
    float ss = x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3];
#pragma unroll
    for (int m = 16; m >= 1; m >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, m);
    const float rstd = 1.0f / sqrtf(ss / (float)kHeadDim + a.eps);
    const float w[4] = {bf_lo(wlo), bf_hi(wlo), bf_lo(whi), bf_hi(whi)};
#pragma unroll
    for (int e = 0; e < 4; ++e) x[e] = round_bf16(round_bf16(x[e] * rstd) * w[e]);
    const float y0 = round_bf16(mul_sub_unfused(x[0], c.x, x[2], s.x)), y1 = round_bf16(mul_sub_unfused(x[1], c.y, x[3], s.y));
    const float y2 = round_bf16(mul_add_unfused(x[2], c.x, x[0], s.x)), y3 = round_bf16(mul_add_unfused(x[3], c.y, x[1], s.y));
    if (warp < 2) {
      sm.qs[warp][d] = y0; sm.qs[warp][d + 1] = y1; sm.qs[warp][d + 64] = y2; sm.qs[warp][d + 65] = y3;
    } else {
      *reinterpret_cast<uint32_t*>(sm.ks + d) = pack_bf16(y0, y1);
      *reinterpret_cast<uint32_t*>(sm.ks + d + 64) = pack_bf16(y2, y3);
    }
  } else {
    const int col = q_size + kv_size + kvh * kHeadDim + 4 * lane;
    uint4 v;
    int spins = 0;
    do {
      v = ld_volatile_v4(xrow + (col >> 1));
    } while ((v.y != tag_in || v.w != tag_in) && !p_give_up(spins, a.status, kOpAttn, col));
    reinterpret_cast<uint2*>(sm.vs)[lane] = make_uint2(v.x, v.z);
  }
  bar_attn();

  if (owner) {
    const int pi = pos - start;
    if ((pi & 7) == pg) {
      const int i = pi >> 3;
      const uint4 kn = reinterpret_cast<const uint4*>(sm.ks)[l16];
      const uint4 vn = reinterpret_cast<const uint4*>(sm.vs)[l16];
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (u == i) { kreg[u] = kn; vreg[u] = vn; }
      if (a.row_active == nullptr || a.row_active[row] != 0) {
        const size_t off = base + (size_t)pi * tok_stride;
        *reinterpret_cast<uint4*>(kc + off) = kn;
        *reinterpret_cast<uint4*>(vc + off) = vn;
      }
    }
  }

  float q0[8], q1[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) { q0[e] = sm.qs[0][8 * l16 + e]; q1[e] = sm.qs[1][8 * l16 + e]; }
  float s0[8], s1[8];
  float m0 = -INFINITY, m1 = -INFINITY;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
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
    const bool valid = start + pg + 8 * i < end;
    s0[i] = valid ? d0 * a.scale : -INFINITY;
    s1[i] = valid ? d1 * a.scale : -INFINITY;
    m0 = fmaxf(m0, s0[i]);
    m1 = fmaxf(m1, s1[i]);
  }
  if (l16 == 0) { sm.mred[pg][0] = m0; sm.mred[pg][1] = m1; }
  bar_attn();
#pragma unroll
  for (int p = 0; p < 8; ++p) { m0 = fmaxf(m0, sm.mred[p][0]); m1 = fmaxf(m1, sm.mred[p][1]); }

  constexpr float kLog2e = 1.4426950408889634f;
  float o0[8], o1[8], l0 = 0.f, l1 = 0.f;
#pragma unroll
  for (int e = 0; e < 8; ++e) { o0[e] = 0.f; o1[e] = 0.f; }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float p0 = exp2f((s0[i] - m0) * kLog2e);
    const float p1 = exp2f((s1[i] - m1) * kLog2e);
    l0 += p0;
    l1 += p1;
    float vf[8];
    unpack8(vreg[i], vf);
#pragma unroll
    for (int e = 0; e < 8; ++e) { o0[e] += p0 * vf[e]; o1[e] += p1 * vf[e]; }
  }
#pragma unroll
  for (int e = 0; e < 8; ++e) { sm.ored[pg][0][8 * l16 + e] = o0[e]; sm.ored[pg][1][8 * l16 + e] = o1[e]; }
  if (l16 == 0) { sm.lred[pg][0] = l0; sm.lred[pg][1] = l1; }
  bar_attn();

  const int d = tid;
  float O0 = 0.f, O1 = 0.f, L0 = 0.f, L1 = 0.f;
#pragma unroll
  for (int p = 0; p < 8; ++p) { O0 += sm.ored[p][0][d]; O1 += sm.ored[p][1][d]; L0 += sm.lred[p][0]; L1 += sm.lred[p][1]; }

  uint2* orow = a.x_attn + (size_t)row * (q_size / 2);
  auto publish = [&](float r0, float r1) {
    // thread d holds element d of both query heads; even d stores the (d, d+1) pair
    const float n0 = __shfl_xor_sync(0xffffffffu, r0, 1), n1 = __shfl_xor_sync(0xffffffffu, r1, 1);
    if (!(d & 1)) {
      st_ll(orow + (2 * kvh) * 64 + (d >> 1), pack_bf16(r0, n0), tag_out);
      st_ll(orow + (2 * kvh + 1) * 64 + (d >> 1), pack_bf16(r1, n1), tag_out);
    }
  };
  if (nsplits == 1) {
    publish(O0 / L0, O1 / L1);
    return;
  }
  // several splits: publish the partial; the last CTA to arrive merges (no waiting)
  const size_t pidx = ((size_t)row * a.kv_heads + kvh) * kMaxSplits;
  float* po = a.part_o + (pidx + split) * 2 * kHeadDim;
  po[d] = O0;
  po[kHeadDim + d] = O1;
  if (tid == 0) { a.part_ml[(pidx + split) * 2] = make_float2(m0, L0); a.part_ml[(pidx + split) * 2 + 1] = make_float2(m1, L1); }
  __threadfence();
  bar_attn();
  if (tid == 0) sm.last_flag = (atomicAdd(a.tickets + row * a.kv_heads + kvh, 1u) == (unsigned)(nsplits - 1)) ? 1 : 0;
  bar_attn();
  if (!sm.last_flag) return;
  __threadfence();
  float M0 = -INFINITY, M1 = -INFINITY;
  for (int s = 0; s < nsplits; ++s) {
    M0 = fmaxf(M0, __ldcg(&a.part_ml[(pidx + s) * 2]).x);
    M1 = fmaxf(M1, __ldcg(&a.part_ml[(pidx + s) * 2 + 1]).x);
  }
  float A0 = 0.f, A1 = 0.f, S0 = 0.f, S1 = 0.f;
  for (int s = 0; s < nsplits; ++s) {
    const float2 ml0 = __ldcg(&a.part_ml[(pidx + s) * 2]);
    const float2 ml1 = __ldcg(&a.part_ml[(pidx + s) * 2 + 1]);
    const float w0 = exp2f((ml0.x - M0) * kLog2e), w1 = exp2f((ml1.x - M1) * kLog2e);
    const float* ps = a.part_o + (pidx + s) * 2 * kHeadDim;
    A0 += w0 * __ldcg(ps + d);
    A1 += w1 * __ldcg(ps + kHeadDim + d);
    S0 += w0 * ml0.y;
    S1 += w1 * ml1.y;
  }
  publish(A0 / S0, A1 / S1);
  if (tid == 0) a.tickets[row * a.kv_heads + kvh] = 0u;
}

// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(kPThreads, 1) decode_step_persistent_kernel(const PersistArgs a) {
  extern __shared__ __align__(128) unsigned char dyn_smem[];
  unsigned char* ring = dyn_smem;
  uint64_t* full = reinterpret_cast<uint64_t*>(dyn_smem + kPSlots * kUnitBytes);
  uint64_t* empty = full + kPSlots;
  __shared__ float red[2][kRound][kPConsumerWarps][64];
  __shared__ float arg_v[kRound][kMaxRows];
  __shared__ int arg_i[kRound][kMaxRows];
  __shared__ float ssq[2][kPConsumerWarps][kMaxRows];
  __shared__ PAttnSmem attn_sm;
  __shared__ int pos_s[kMaxRows];
  __shared__ int last_flag;

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int G = gridDim.x, cta = blockIdx.x;
  const int L = a.n_layers;
  const int q_size = a.q_heads * kHeadDim, kv_size = a.kv_heads * kHeadDim;
  const int qkv_rows = q_size + 2 * kv_size;
  const int t_qkv = qkv_rows / kTileRows, t_o = kHidden / kTileRows, t_gu = a.intermediate / 4,
            t_down = kHidden / kTileRows, t_lm = a.vocab / kTileRows;
  const int ch_o = q_size / kUnitCols, ch_down = a.intermediate / kUnitCols;

  if (tid == 0) {
    for (int s = 0; s < kPSlots; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], kPConsumerWarps); }
    fence_mbar_init();
  }
  if (tid < kMaxRows) {
    int p = tid < a.rows ? a.positions[tid] : 0;
    if (p < 0 || p >= a.max_pos) {
      report_status(a.status, kStatusBadPosition, kKernelAttention, tid, p);
      p = p < 0 ? 0 : a.max_pos - 1;
    }
    pos_s[tid] = p;
  }
  const unsigned epoch = *reinterpret_cast<volatile unsigned*>(a.epoch);
  __syncthreads();

  // =========================== producer warp ===============================
  if (warp == kPConsumerWarps) {
    int n = 0;
    // A tile is 8 consecutive weight rows = 8 * K * 2 contiguous bytes (K = 1024 *
    // chunks), fetched as `chunks` bulk copies of 16 KB into consecutive ring
    // slots.  A gate/up tile is 4 gate rows followed by 4 up rows (two 8 KB copies).
    auto produce = [&](const __nv_bfloat16* w, int tiles, int chunks, bool swiglu, int rot) {
      for (int t = p_first(cta, rot, G); t < tiles; t += G)
        for (int ch = 0; ch < chunks; ++ch, ++n) {
          const int slot = n % kPSlots;
          if (n >= kPSlots) p_wait_mbar(&empty[slot], ((n / kPSlots) - 1) & 1, a.status, 100 + slot);
          if (lane == 0) {
            mbar_expect_tx(&full[slot], kUnitBytes);
            unsigned char* dst = ring + slot * kUnitBytes;
            if (swiglu) {
              bulk_g2s(dst, w + (size_t)(t * 4) * kHidden, kUnitBytes / 2, &full[slot]);
              bulk_g2s(dst + kUnitBytes / 2, w + (size_t)(a.intermediate + t * 4) * kHidden, kUnitBytes / 2, &full[slot]);
            } else {
              bulk_g2s(dst, w + ((size_t)t * chunks + ch) * (kUnitBytes / 2), kUnitBytes, &full[slot]);
            }
          }
          __syncwarp();
        }
    };
    for (int l = 0; l < L; ++l) {
      const PLayerWeights lw = a.layers[l];
      produce(lw.wqkv, t_qkv, 1, false, p_rot(l, kOpQkv, G));
      produce(lw.wo, t_o, ch_o, false, p_rot(l, kOpO, G));
      produce(lw.wgu, t_gu, 1, true, p_rot(l, kOpGateUp, G));
      produce(lw.wd, t_down, ch_down, false, p_rot(l, kOpDown, G));
    }
    produce(a.embed, t_lm, 1, false, p_rot(L, kOpLmHead, G));
    return;
  }

  // =========================== consumer warps ==============================
  const int g = lane >> 2, t4 = lane & 3;
  const int kbase = warp * 128 + 8 * t4;   // this lane's first column inside a 1024-column unit
  const bool live = g < a.rows;
  const int rr = tid >> 6;                 // epilogue thread -> tile of the round,
  const int eb = (tid & 63) >> 3, er = tid & 7;   //   batch row, tile row
  int n_cons = 0;                          // units consumed (ring position)
  int n_round = 0;                         // rounds finished (parity of `red`)
  int n_norm = 0;                          // norms done (parity of `ssq`)
  uint4 res[4];                            // residual fragments of row g, packed bf16
#pragma unroll
  for (int j = 0; j < 4; ++j) res[j] = make_uint4(0, 0, 0, 0);

  auto trace_op = [&](int op_index, int word, bool is_min) {
    if (a.trace && tid == 0) {
      if (is_min) trace_min(a.trace + 8 * op_index, word);
      else trace_max(a.trace + 8 * op_index, word);
    }
  };

  // x = h (+ residual); residual = bf16(x); returns RMSNorm(x) * w as MMA fragments
  auto add_norm = [&](const uint4 (&hv)[4], const uint4 (&nw)[4], uint4 (&xa)[4]) {
    float xs[4][8];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float hf[8], rf[8];
      unpack8(hv[j], hf);
      unpack8(res[j], rf);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        xs[j][e] = live ? hf[e] + rf[e] : 0.f;
        ss += xs[j][e] * xs[j][e];
      }
      res[j].x = pack_bf16(xs[j][0], xs[j][1]); res[j].y = pack_bf16(xs[j][2], xs[j][3]);
      res[j].z = pack_bf16(xs[j][4], xs[j][5]); res[j].w = pack_bf16(xs[j][6], xs[j][7]);
    }
    ss += __shfl_xor_sync(0xffffffffu, ss, 1);
    ss += __shfl_xor_sync(0xffffffffu, ss, 2);
    float (*sq)[kMaxRows] = ssq[n_norm & 1];
    ++n_norm;
    if (t4 == 0) sq[warp][g] = ss;
    bar_consumers();
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < kPConsumerWarps; ++w) tot += sq[w][g];
    const float rstd = 1.0f / sqrtf(tot / (float)kHidden + a.eps);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float wf[8], y[8];
      unpack8(nw[j], wf);
#pragma unroll
      for (int e = 0; e < 8; ++e) y[e] = round_bf16(xs[j][e] * rstd) * wf[e];
      xa[j].x = pack_bf16(y[0], y[1]); xa[j].y = pack_bf16(y[2], y[3]);
      xa[j].z = pack_bf16(y[4], y[5]); xa[j].w = pack_bf16(y[6], y[7]);
    }
  };
  auto load_norm_w = [&](const __nv_bfloat16* norm_w, uint4 (&nw)[4]) {
#pragma unroll
    for (int j = 0; j < 4; ++j) nw[j] = ldg_stream(norm_w + kbase + 32 * j);
  };

  // One ROUND: up to kRound tiles (each `chunks` units of 8 rows x 1024 columns)
  // are multiplied back to back, every warp on its own K slice; then ONE
  // barrier, after which 64 threads per tile add the 8 warps' partial sums.
  // Thread (rr, eb, er) gets the bf16-rounded value of tile rr, batch row eb,
  // tile row er (meaningful when rr < nr).
  auto run_round = [&](int nr, auto chunks_tag, bool swiglu, const auto& xa) -> float {
    constexpr int CH = decltype(chunks_tag)::value;     // 16 KB units per tile; K = 1024 * CH
    constexpr int K = kUnitCols * CH;
    float c[kRound][2][4];
#pragma unroll
    for (int r = 0; r < kRound; ++r)
#pragma unroll
      for (int q = 0; q < 2; ++q) { c[r][q][0] = 0.f; c[r][q][1] = 0.f; c[r][q][2] = 0.f; c[r][q][3] = 0.f; }
    // row of the tile this lane multiplies (MMA column n = g); gate/up tiles hold
    // gate rows 0-3 then up rows 0-3 and present them interleaved
    const int srow = swiglu ? ((g & 1) ? 4 + (g >> 1) : (g >> 1)) : g;
    const int col0 = warp * (K / kPConsumerWarps) + 8 * t4;
#pragma unroll
    for (int r = 0; r < kRound; ++r) {
      if (r < nr) {
#pragma unroll
        for (int u = 0; u < CH; ++u) {
          const int nu = n_cons + u;
          p_wait_mbar(&full[nu % kPSlots], (nu / kPSlots) & 1, a.status, 200 + u);
        }
#pragma unroll
        for (int j = 0; j < 4 * CH; ++j) {
          const int off = (srow * K + col0 + 32 * j) * 2;           // byte offset inside the tile
          const int slot = (n_cons + (off >> 14)) % kPSlots;
          const uint4 wv = *reinterpret_cast<const uint4*>(ring + slot * kUnitBytes + (off & (kUnitBytes - 1)));
          mma_bf16_16816(c[r][0], xa[j].x, xa[j].y, wv.x, wv.y);
          mma_bf16_16816(c[r][1], xa[j].z, xa[j].w, wv.z, wv.w);
        }
        __syncwarp();
        if (lane == 0) {
#pragma unroll
          for (int u = 0; u < CH; ++u) mbar_arrive(&empty[(n_cons + u) % kPSlots]);
        }
        n_cons += CH;
      }
    }
    float (*rd)[kPConsumerWarps][64] = red[n_round & 1];
    ++n_round;
#pragma unroll
    for (int r = 0; r < kRound; ++r)
      if (r < nr)
        *reinterpret_cast<float2*>(&rd[r][warp][2 * lane]) = make_float2(c[r][0][0] + c[r][1][0], c[r][0][1] + c[r][1][1]);
    bar_consumers();
    float v = 0.f;
    if (rr < nr) {
#pragma unroll
      for (int w = 0; w < kPConsumerWarps; ++w) v += rd[rr][w][tid & 63];
      v = round_bf16(v);
    }
    return v;
  };
  // tiles of one round: first tile t, then every G-th, at most kRound, below T
  auto round_size = [&](int t, int T) -> int {
    const int left = (T - t + G - 1) / G;
    return left < kRound ? left : kRound;
  };
  // publish values (eb, n0 + er) of this thread's tile as tagged words
  auto store_pairs = [&](float v, bool valid, uint2* out, int row_words, int n0, uint32_t tag) {
    const float hi = __shfl_xor_sync(0xffffffffu, v, 1);
    if (valid && !(er & 1) && eb < a.rows) st_ll(out + (size_t)eb * row_words + ((n0 + er) >> 1), pack_bf16(v, hi), tag);
  };

  for (int l = 0; l < L; ++l) {
    const PLayerWeights lw = a.layers[l];
    const int oi = 5 * l;
    // ------------------------------ qkv ------------------------------------
    {
      trace_op(oi + kOpQkv, 0, true);
      uint4 hv[4], nw[4], xa[4];
      load_norm_w(lw.ln_in, nw);
      if (live) {
        if (l == 0) {
          const __nv_bfloat16* e = a.embed + (size_t)a.ids[g] * kHidden + kbase;
#pragma unroll
          for (int j = 0; j < 4; ++j) hv[j] = ldg_stream(e + 32 * j);
        } else {
          ll_load_frags<4>(a.x_hmlp + (size_t)g * (kHidden / 2), kbase, p_tag(epoch, l - 1, kOpDown), hv, a.status, kOpQkv);
        }
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) hv[j] = make_uint4(0, 0, 0, 0);
      }
      trace_op(oi + kOpQkv, 1, false);
      add_norm(hv, nw, xa);
      const uint32_t tag = p_tag(epoch, l, kOpQkv);
      for (int t = p_first(cta, p_rot(l, kOpQkv, G), G); t < t_qkv; t += kRound * G) {
        const int nr = round_size(t, t_qkv);
        const float v = run_round(nr, IntC<1>{}, false, xa);
        store_pairs(v, rr < nr, a.x_qkv, qkv_rows / 2, (t + rr * G) * kTileRows, tag);
      }
      trace_op(oi + kOpQkv, 2, false);
    }
    // ---------------------------- attention --------------------------------
    if (warp < 4) {
      trace_op(oi + kOpAttn, 0, true);
      const uint32_t tag_in = p_tag(epoch, l, kOpQkv), tag_out = p_tag(epoch, l, kOpAttn);
      int total = 0;
      for (int r = 0; r < a.rows; ++r) total += a.kv_heads * ((pos_s[r] + kAttnChunk) / kAttnChunk);
      for (int item = p_first(cta, p_rot(l, kOpAttn, G), G); item < total; item += G) {
        int i = item, row = 0, ns = 1;
        for (row = 0; row < a.rows; ++row) {
          ns = (pos_s[row] + kAttnChunk) / kAttnChunk;
          if (i < a.kv_heads * ns) break;
          i -= a.kv_heads * ns;
        }
        bar_attn();  // the previous item is done with the shared scratch
        p_attention_item(a, attn_sm, l, row, i / ns, i % ns, ns, pos_s[row], tag_in, tag_out);
      }
      trace_op(oi + kOpAttn, 2, false);
    }
    // ------------------------------ o_proj ---------------------------------
    {
      const int t0 = p_first(cta, p_rot(l, kOpO, G), G);
      if (t0 < t_o) {
        trace_op(oi + kOpO, 0, true);
        uint4 xa[8];   // this lane's K slice: columns warp * 256 + 32 j + 8 t4
        if (live)
          ll_load_frags<8>(a.x_attn + (size_t)g * (q_size / 2), warp * 256 + 8 * t4, p_tag(epoch, l, kOpAttn), xa,
                           a.status, kOpO);
        else
#pragma unroll
          for (int j = 0; j < 8; ++j) xa[j] = make_uint4(0, 0, 0, 0);
        trace_op(oi + kOpO, 1, false);
        const uint32_t tag = p_tag(epoch, l, kOpO);
        for (int t = t0; t < t_o; t += kRound * G) {
          const int nr = round_size(t, t_o);
          const float v = run_round(nr, IntC<2>{}, false, xa);
          store_pairs(v, rr < nr, a.x_hattn, kHidden / 2, (t + rr * G) * kTileRows, tag);
        }
        trace_op(oi + kOpO, 2, false);
      }
    }
    // ----------------------------- gate / up -------------------------------
    {
      trace_op(oi + kOpGateUp, 0, true);
      uint4 hv[4], nw[4], xa[4];
      load_norm_w(lw.ln_post, nw);
      if (live)
        ll_load_frags<4>(a.x_hattn + (size_t)g * (kHidden / 2), kbase, p_tag(epoch, l, kOpO), hv, a.status, kOpGateUp);
      else
#pragma unroll
        for (int j = 0; j < 4; ++j) hv[j] = make_uint4(0, 0, 0, 0);
      trace_op(oi + kOpGateUp, 1, false);
      add_norm(hv, nw, xa);
      const uint32_t tag = p_tag(epoch, l, kOpGateUp);
      for (int t = p_first(cta, p_rot(l, kOpGateUp, G), G); t < t_gu; t += kRound * G) {
        const int nr = round_size(t, t_gu);
        const float v = run_round(nr, IntC<1>{}, true, xa);
        // tile rows alternate gate, up: even er holds gate, er + 1 holds up
        const float up = __shfl_xor_sync(0xffffffffu, v, 1);
        const float act = round_bf16(v / (1.0f + expf(-v)) * up);
        const float nxt = __shfl_xor_sync(0xffffffffu, act, 2);
        if (rr < nr && (er & 3) == 0 && eb < a.rows)
          st_ll(a.x_act + (size_t)eb * (a.intermediate / 2) + (t + rr * G) * 2 + (er >> 2), pack_bf16(act, nxt), tag);
      }
      trace_op(oi + kOpGateUp, 2, false);
    }
    // ------------------------------- down ----------------------------------
    {
      const int t0 = p_first(cta, p_rot(l, kOpDown, G), G);
      if (t0 < t_down) {
        trace_op(oi + kOpDown, 0, true);
        uint4 xa[12];  // this lane's K slice: columns warp * 384 + 32 j + 8 t4
        if (live)
          ll_load_frags<12>(a.x_act + (size_t)g * (a.intermediate / 2), warp * 384 + 8 * t4, p_tag(epoch, l, kOpGateUp), xa,
                            a.status, kOpDown);
        else
#pragma unroll
          for (int j = 0; j < 12; ++j) xa[j] = make_uint4(0, 0, 0, 0);
        trace_op(oi + kOpDown, 1, false);
        const uint32_t tag = p_tag(epoch, l, kOpDown);
        for (int t = t0; t < t_down; t += kRound * G) {
          const int nr = round_size(t, t_down);
          const float v = run_round(nr, IntC<3>{}, false, xa);
          store_pairs(v, rr < nr, a.x_hmlp, kHidden / 2, (t + rr * G) * kTileRows, tag);
        }
        trace_op(oi + kOpDown, 2, false);
      }
    }
  }

  // ------------------------------- LM head ---------------------------------
  {
    const int oi = 5 * L;
    trace_op(oi, 0, true);
    uint4 hv[4], nw[4], xa[4];
    load_norm_w(a.final_norm, nw);
    if (live)
      ll_load_frags<4>(a.x_hmlp + (size_t)g * (kHidden / 2), kbase, p_tag(epoch, L - 1, kOpDown), hv, a.status, kOpLmHead);
    else
#pragma unroll
      for (int j = 0; j < 4; ++j) hv[j] = make_uint4(0, 0, 0, 0);
    trace_op(oi, 1, false);
    add_norm(hv, nw, xa);
    float best_v = -INFINITY;
    int best_i = 0x7fffffff;
    for (int t = p_first(cta, p_rot(L, kOpLmHead, G), G); t < t_lm; t += kRound * G) {
      const int nr = round_size(t, t_lm);
      const float v = run_round(nr, IntC<1>{}, false, xa);
      if (rr < nr && eb < a.rows) {
        const int idx = (t + rr * G) * kTileRows + er;
        if (a.logits_out) a.logits_out[(size_t)eb * a.vocab + idx] = v;
        if (v > best_v || (v == best_v && idx < best_i)) { best_v = v; best_i = idx; }
      }
    }
    // reduce over the 8 tile rows (lanes), then over the kRound tile slots (smem)
#pragma unroll
    for (int m = 1; m < 8; m <<= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best_v, m);
      const int oi2 = __shfl_xor_sync(0xffffffffu, best_i, m);
      if (ov > best_v || (ov == best_v && oi2 < best_i)) { best_v = ov; best_i = oi2; }
    }
    if (er == 0) { arg_v[rr][eb] = best_v; arg_i[rr][eb] = best_i; }
    bar_consumers();
    if (tid < kMaxRows) {
      float v = arg_v[0][tid];
      int i = arg_i[0][tid];
      for (int r = 1; r < kRound; ++r)
        if (arg_v[r][tid] > v || (arg_v[r][tid] == v && arg_i[r][tid] < i)) { v = arg_v[r][tid]; i = arg_i[r][tid]; }
      a.parts[cta * kMaxRows + tid] = ArgmaxPart{v, i};
    }
    __threadfence();
    bar_consumers();
    unsigned int* ticket = a.tickets + kMaxRows * a.kv_heads;
    if (tid == 0) last_flag = (atomicAdd(ticket, 1u) == (unsigned)(G - 1)) ? 1 : 0;
    bar_consumers();
    if (last_flag) {
      __threadfence();
      for (int b = warp; b < a.rows; b += kPConsumerWarps) {
        float v = -INFINITY;
        int i = 0x7fffffff;
        for (int c2 = lane; c2 < G; c2 += 32) {
          const int2 raw = __ldcg(reinterpret_cast<const int2*>(a.parts + c2 * kMaxRows + b));
          const float pv = __int_as_float(raw.x);
          if (pv > v || (pv == v && raw.y < i)) { v = pv; i = raw.y; }
        }
#pragma unroll
        for (int m = 16; m >= 1; m >>= 1) {
          const float ov = __shfl_xor_sync(0xffffffffu, v, m);
          const int oi2 = __shfl_xor_sync(0xffffffffu, i, m);
          if (ov > v || (ov == v && oi2 < i)) { v = ov; i = oi2; }
        }
        if (lane == 0) a.tokens[b] = i;
      }
      if (tid == 0) {
        *ticket = 0u;
        *a.epoch = epoch + 1u;   // every CTA has read this step's epoch long ago
      }
    }
    trace_op(oi, 2, false);
  }
}

}  // namespace dfb
