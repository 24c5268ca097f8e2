// Causal prefill attention over the prompt tokens of a batch of sequences: the step on the other side of the
// shared paged cache.  The reference calls FlashAttention for it (flash_attn_varlen_func with causal = True,
// layers/attention.py:64-70); this is the same computation, written against the tensor cores with mma.sync, for
// both of its cases: without a prefix cache K / V are the fresh projections of the same tokens; with one they
// are read back from the paged cache through the block tables, the sequence's keys outnumber its queries, and
// query i attends to keys 0 .. i + (keys - queries) (the causal mask aligned to the last key, as FlashAttention):
//
//   * q [N, q_heads, 128], k / v [N, kv_heads, 128] bf16, tokens of all sequences back to back, sequence b =
//     rows [cu_seqlens[b], cu_seqlens[b + 1]); grouped-query attention (q head h reads KV head
//     h / (q_heads / kv_heads)); out [N, q_heads, 128] bf16;
//   * a CTA of four warps owns 64 query rows of one (sequence, q head), a warp 16 of them; the Q fragments (A
//     operand, 16 rows x 128 dims) stay in registers; K / V tiles of 64 positions are brought into shared memory
//     (rows padded by 16 bytes, so that the fragment reads below are free of bank conflicts), two tiles in
//     flight (cp.async double buffer);
//   * S = Q K^T: K rows are the B operand directly (ldmatrix, two position tiles per instruction); the causal mask is
//     applied on the diagonal tiles; online softmax in fp32 with one running (max, sum) per row, held by the four
//     lanes that share the row;
//   * O += P V: the S accumulators, rounded to bf16, ARE the A fragments of the second product (no trip through
//     shared memory); V fragments by ldmatrix.trans; O in fp32 registers, divided by the row sum at the end.
//
// P is rounded to bf16 before it multiplies V, as FlashAttention does.  mma.sync issues about once per 38 cycles
// per SM sub-partition on this part, which bounds this kernel far below the tcgen05 peak: it is the functional
// counterpart of the reference's prefill attention on the shared cache layout, not a roofline kernel.
#pragma once

#include "dfb_kernels.cuh"

namespace dfb {

constexpr int kPfTile = 64;                      // query rows per CTA and KV positions per tile
constexpr int kPfRowBytes = kHeadDim * 2 + 16;   // padded shared-memory row of a K / V tile
constexpr int kPfTileBytes = kPfTile * kPfRowBytes;
constexpr int kPfSmemBytes = 4 * kPfTileBytes;   // K and V, two buffers each
constexpr int kKernelPrefill = 9;

struct PrefillArgs {
  const __nv_bfloat16* q;
  const __nv_bfloat16* k;
  const __nv_bfloat16* v;
  __nv_bfloat16* out;
  const int* cu_seqlens;        // [batch + 1] query rows
  const int* cu_seqlens_k;      // [batch + 1] keys; equal to cu_seqlens without a prefix cache
  const int* block_tables;      // null: k / v hold the keys of sequence b at rows cu_seqlens_k[b] ...; else
                                // [batch, bt_stride] physical blocks and k / v are one layer's cache
                                // [num_blocks, block_size] rows
  int bt_stride, block_size, block_shift, num_blocks;   // block_size = 1 << block_shift
  long long q_stride, k_stride, v_stride, out_stride;   // elements between token rows (cache: between slots)
  int q_heads, kv_heads;
  float scale;
  int* status;                  // optional device status word (a block id outside the cache)
};

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s) : "memory");
}

// PAGED: keys come from the paged cache through the block tables (block_size a power of two: the position's
// block and offset are a shift and a mask); else they are rows of k / v, and the copy loop has no table walk.
template <bool PAGED>
__global__ void __launch_bounds__(128) prefill_attention_kernel(const PrefillArgs a) {
  extern __shared__ __align__(128) unsigned char pf_smem[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int seq = blockIdx.z, head = blockIdx.y;
  const int kvh = head / (a.q_heads / a.kv_heads);
  const int seq_start = a.cu_seqlens[seq], seq_len = a.cu_seqlens[seq + 1] - seq_start;
  const int k_start = a.cu_seqlens_k[seq], k_len = a.cu_seqlens_k[seq + 1] - k_start;
  const int shift = max(k_len - seq_len, 0);      // keys before the first query (the cached prefix)
  const int q0 = blockIdx.x * kPfTile;            // first query row of this CTA inside the sequence
  if (q0 >= seq_len || k_len < 1) return;
  const int q_hi = min(q0 + kPfTile, seq_len);    // one past the CTA's last query row
  const int n_tiles = (shift + q_hi + kPfTile - 1) / kPfTile;   // causal: key positions [0, shift + q_hi)

  auto k_tile = [&](int buf) { return pf_smem + buf * kPfTileBytes; };
  auto v_tile = [&](int buf) { return pf_smem + (2 + buf) * kPfTileBytes; };
  // every thread copies 8 + 8 pieces of 16 bytes per tile (64 rows x 16 pieces for K, the same for V); rows
  // beyond the sequence are filled with zeros so that no stale bits (a NaN pattern) ever meet a zero probability
  auto load_tile = [&](int tile, int buf) {
    const int p0 = tile * kPfTile;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int idx = tid + 128 * i, row = idx >> 4, piece = idx & 15;
      unsigned char* kd = k_tile(buf) + row * kPfRowBytes + 16 * piece;
      unsigned char* vd = v_tile(buf) + row * kPfRowBytes + 16 * piece;
      const int p = p0 + row;
      long long tok = -1;                          // row of k / v that holds key p, or none
      if (p < k_len) {
        if (PAGED) {
          const int block = a.block_tables[(size_t)seq * a.bt_stride + (p >> a.block_shift)];
          if (block >= 0 && block < a.num_blocks) tok = ((long long)block << a.block_shift) + (p & (a.block_size - 1));
          else if (piece == 0) report_status(a.status, kStatusBadBlock, kKernelPrefill, seq, block);   // row read as zeros
        } else {
          tok = k_start + p;
        }
      }
      if (tok >= 0) {
        cp_async16(kd, a.k + (size_t)tok * a.k_stride + (size_t)kvh * kHeadDim + 8 * piece);
        cp_async16(vd, a.v + (size_t)tok * a.v_stride + (size_t)kvh * kHeadDim + 8 * piece);
      } else {
        *reinterpret_cast<uint4*>(kd) = make_uint4(0, 0, 0, 0);
        *reinterpret_cast<uint4*>(vd) = make_uint4(0, 0, 0, 0);
      }
    }
    cp_async_commit();
  };
  load_tile(0, 0);

  // ---- Q fragments: rows r0 = q0 + 16 warp + g and r0 + 8, eight k-steps of 16 dims ----
  const int r_lo = q0 + 16 * warp + g, r_hi = r_lo + 8;
  uint32_t qf[8][4];
  {
    const __nv_bfloat16* ql = a.q + (size_t)(seq_start + min(r_lo, seq_len - 1)) * a.q_stride + (size_t)head * kHeadDim;
    const __nv_bfloat16* qh = a.q + (size_t)(seq_start + min(r_hi, seq_len - 1)) * a.q_stride + (size_t)head * kHeadDim;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      qf[ks][0] = *reinterpret_cast<const uint32_t*>(ql + 16 * ks + 2 * t);
      qf[ks][1] = *reinterpret_cast<const uint32_t*>(qh + 16 * ks + 2 * t);
      qf[ks][2] = *reinterpret_cast<const uint32_t*>(ql + 16 * ks + 8 + 2 * t);
      qf[ks][3] = *reinterpret_cast<const uint32_t*>(qh + 16 * ks + 8 + 2 * t);
    }
  }

  constexpr float kLog2e = 1.4426950408889634f;
  const float sl2 = a.scale * kLog2e;             // scores are kept in units of log2 e
  float o[16][4];                                 // 16 n-tiles of 8 dims: (row lo, 2t), (lo, 2t+1), (hi, 2t), (hi, 2t+1)
#pragma unroll
  for (int n = 0; n < 16; ++n) { o[n][0] = 0.f; o[n][1] = 0.f; o[n][2] = 0.f; o[n][3] = 0.f; }
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;

  for (int tile = 0; tile < n_tiles; ++tile) {
    const int buf = tile & 1;
    if (tile + 1 < n_tiles) { load_tile(tile + 1, buf ^ 1); cp_async_wait<1>(); }
    else cp_async_wait<0>();
    __syncthreads();
    const int p0 = tile * kPfTile;
    const unsigned char* kt = k_tile(buf);
    const unsigned char* vt = v_tile(buf);

    // ---- S = Q K^T for this warp's 16 rows x 64 positions ----
    float s[8][4];
#pragma unroll
    for (int n = 0; n < 8; ++n) { s[n][0] = 0.f; s[n][1] = 0.f; s[n][2] = 0.f; s[n][3] = 0.f; }
    // one ldmatrix.x4 brings the B fragments of two position tiles for one k-step: matrices (positions 16 np ..
    // + 7, dims 16 ks .. + 7), (same positions, dims + 8), (positions + 8 .. + 15, dims 16 ks ..), (those, dims + 8)
#pragma unroll
    for (int np = 0; np < 4; ++np) {
      const unsigned char* kaddr = kt + (16 * np + (lane & 7) + (lane >> 4) * 8) * kPfRowBytes + ((lane >> 3) & 1) * 16;
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        uint32_t kb[4];
        ldmatrix_x4(kb, kaddr + 32 * ks);
        mma_bf16_16816_full(s[2 * np], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], kb[0], kb[1]);
        mma_bf16_16816_full(s[2 * np + 1], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], kb[2], kb[3]);
      }
    }
    // ---- scale, causal mask (and the tail of the sequence), online softmax ----
    float t_lo = -INFINITY, t_hi = -INFINITY;
#pragma unroll
    for (int n = 0; n < 8; ++n) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int pos = p0 + 8 * n + 2 * t + e;
        const bool in = pos < k_len;
        s[n][e] = (in && pos <= shift + r_lo) ? s[n][e] * sl2 : -INFINITY;
        s[n][2 + e] = (in && pos <= shift + r_hi) ? s[n][2 + e] * sl2 : -INFINITY;
        t_lo = fmaxf(t_lo, s[n][e]);
        t_hi = fmaxf(t_hi, s[n][2 + e]);
      }
    }
    t_lo = fmaxf(t_lo, __shfl_xor_sync(0xffffffffu, t_lo, 1)); t_lo = fmaxf(t_lo, __shfl_xor_sync(0xffffffffu, t_lo, 2));
    t_hi = fmaxf(t_hi, __shfl_xor_sync(0xffffffffu, t_hi, 1)); t_hi = fmaxf(t_hi, __shfl_xor_sync(0xffffffffu, t_hi, 2));
    // position 0 is visible to every row, so after the first tile the maxima are finite; rows beyond the
    // sequence (clamped duplicates of its last row) behave like that row and are never stored
    const float n_lo = fmaxf(m_lo, t_lo), n_hi = fmaxf(m_hi, t_hi);
    const float c_lo = exp2f(m_lo - n_lo), c_hi = exp2f(m_hi - n_hi);
    m_lo = n_lo; m_hi = n_hi;
    float sum_lo = 0.f, sum_hi = 0.f;
    uint32_t pf[8][2];                            // P as bf16 pairs: [n][0] = row lo, [n][1] = row hi
#pragma unroll
    for (int n = 0; n < 8; ++n) {
      const float p0v = exp2f(s[n][0] - n_lo), p1v = exp2f(s[n][1] - n_lo);
      const float p2v = exp2f(s[n][2] - n_hi), p3v = exp2f(s[n][3] - n_hi);
      pf[n][0] = pack_bf16(p0v, p1v);
      pf[n][1] = pack_bf16(p2v, p3v);
      // the row sums use the rounded probabilities, the values that actually multiply V
      sum_lo += bf_lo(pf[n][0]) + bf_hi(pf[n][0]);
      sum_hi += bf_lo(pf[n][1]) + bf_hi(pf[n][1]);
    }
    sum_lo += __shfl_xor_sync(0xffffffffu, sum_lo, 1); sum_lo += __shfl_xor_sync(0xffffffffu, sum_lo, 2);
    sum_hi += __shfl_xor_sync(0xffffffffu, sum_hi, 1); sum_hi += __shfl_xor_sync(0xffffffffu, sum_hi, 2);
    l_lo = l_lo * c_lo + sum_lo;
    l_hi = l_hi * c_hi + sum_hi;
#pragma unroll
    for (int n = 0; n < 16; ++n) { o[n][0] *= c_lo; o[n][1] *= c_lo; o[n][2] *= c_hi; o[n][3] *= c_hi; }

    // ---- O += P V: k-step kk covers positions 16 kk .. 16 kk + 15 (score tiles 2 kk and 2 kk + 1) ----
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      const uint32_t a0 = pf[2 * kk][0], a1 = pf[2 * kk][1], a2 = pf[2 * kk + 1][0], a3 = pf[2 * kk + 1][1];
#pragma unroll
      for (int nn = 0; nn < 8; ++nn) {            // two dim-tiles (16 dims) per ldmatrix.x4
        // matrices: (positions 16kk..+7, dims 16nn..+7), (positions +8..+15, same dims),
        //           (positions 16kk..+7, dims 16nn+8..+15), (positions +8..+15, those dims)
        const int mrow = 16 * kk + (lane & 7) + ((lane >> 3) & 1) * 8;
        const int mcol = 16 * nn + (lane >> 4) * 8;
        uint32_t vb[4];
        ldmatrix_x4_trans(vb, vt + mrow * kPfRowBytes + 2 * mcol);
        mma_bf16_16816_full(o[2 * nn], a0, a1, a2, a3, vb[0], vb[1]);
        mma_bf16_16816_full(o[2 * nn + 1], a0, a1, a2, a3, vb[2], vb[3]);
      }
    }
    __syncthreads();   // everyone is done with this buffer before the tile after next lands in it
  }

  // ---- normalise and store this warp's rows ----
  const float inv_lo = 1.0f / l_lo, inv_hi = 1.0f / l_hi;
  if (r_lo < seq_len) {
    __nv_bfloat16* dst = a.out + (size_t)(seq_start + r_lo) * a.out_stride + (size_t)head * kHeadDim + 2 * t;
#pragma unroll
    for (int n = 0; n < 16; ++n) *reinterpret_cast<uint32_t*>(dst + 8 * n) = pack_bf16(o[n][0] * inv_lo, o[n][1] * inv_lo);
  }
  if (r_hi < seq_len) {
    __nv_bfloat16* dst = a.out + (size_t)(seq_start + r_hi) * a.out_stride + (size_t)head * kHeadDim + 2 * t;
#pragma unroll
    for (int n = 0; n < 16; ++n) *reinterpret_cast<uint32_t*>(dst + 8 * n) = pack_bf16(o[n][2] * inv_hi, o[n][3] * inv_hi);
  }
}

}  // namespace dfb
