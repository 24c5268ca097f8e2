// Tensor-parallel exchange over peer-mapped memory (NVLink), one rank per GPU.
//
// Every rank owns a "window": for each of two buffers an inbox with one slot per
// source rank, plus an inbox and flags for the greedy winners of the LM-head
// shards.  The peers' windows are mapped into this process, so a rank PUSHES
// its partial result into its slot of every peer's inbox, then waits for the
// peers' data in its own window (local reads) and adds the partials in rank
// order, which makes the sum bit-identical on every rank.
//
// The partial sums travel as 8-byte words {two bf16 values, tag}, each written
// by one 8-byte store, so data and "it has arrived" flag cannot be seen apart:
// the receiver polls the word until its tag is the expected one.  That costs one
// NVLink crossing per exchange instead of data + fence + flag.  Tags grow with
// every exchange (step counter * 64 + index of the exchange in the step + 1) and
// are never reset, so there is no reset race.  The two projections of a layer
// alternate between the two buffers: a rank can only reach its next use of a
// buffer after every peer has consumed the current one (each exchange needs
// every rank's contribution).
//
// Every wait is bounded (kPeerWaitNs of globaltimer): on expiry the kernel
// records kStatusPeerTimeout in the status word, stops waiting and finishes, so
// a missing peer can never hang the GPU; later waits of the same step return at
// once when they see the status word set.
#pragma once

#include "dfb_kernels.cuh"

namespace dfb {

constexpr int kExchangeSlots = 64;                     // exchanges per step fit in 6 bits
constexpr unsigned long long kPeerWaitNs = 2000000000ull;  // default limit of a wait for a peer: 2 s
constexpr int kStatusPeerTimeout = 4;
constexpr int kKernelExchange = 3;

// layout of one rank's window (bytes from its base)
struct Window {
  static constexpr size_t kSlotWords = (size_t)kMaxRows * 1024 / 2;              // one partial: {2 bf16, tag} words
  static constexpr size_t kInboxBytes = 2 * kMaxRanks * kSlotWords * 8;          // [2][8][4096] uint2
  static constexpr size_t kPairsOff = kInboxBytes;                               // [8][8] ArgmaxPart
  static constexpr size_t kPairFlagsOff = kPairsOff + kMaxRanks * kMaxRows * 8;  // [8] u32
  static constexpr size_t kBytes = kPairFlagsOff + kMaxRanks * 4 + 192;
};

struct ExchangeArgs {
  unsigned char* window[kMaxRanks];   // base of every rank's window as mapped here; window[rank] is local
  int size, rank;
  int rows;
  int buf;                            // 0 / 1: which inbox
  int slot;                           // index of this exchange in the step, 0 .. kExchangeSlots-2
  const unsigned int* step_counter;   // device counter, the same on every rank
  __nv_bfloat16* local;               // [rows, 1024]: partial in, sum out
  int* status;
  unsigned long long* trace;
  unsigned long long wait_ns;         // limit of each wait for a peer
};

__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Waits until *flag has reached `tag` (wrap-safe).  Returns false after kPeerWaitNs
// or when another wait of this step has already failed.
__device__ __forceinline__ bool wait_flag(const unsigned int* flag, unsigned int tag, int* status, int who,
                                          unsigned long long limit_ns) {
  const unsigned long long t0 = global_ns();
  int polls = 0;
  while ((int)(ld_acquire_sys(flag) - tag) < 0) {
    if ((++polls & 63) == 0) {
      if (*reinterpret_cast<volatile int*>(status) != 0) return false;
      if (global_ns() - t0 > limit_ns) {
        report_status(status, kStatusPeerTimeout, kKernelExchange, who, (int)tag);
        return false;
      }
    }
  }
  return true;
}

// Polls one {data, tag} word until the tag arrives; bounded like wait_flag.
__device__ __forceinline__ bool wait_word(const uint2* p, unsigned int tag, int* status, int who, uint32_t& data,
                                          unsigned long long limit_ns) {
  const unsigned long long t0 = global_ns();
  int polls = 0;
  for (;;) {
    uint2 v;
    asm volatile("ld.relaxed.sys.global.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    if (v.y == tag) { data = v.x; return true; }
    if ((++polls & 63) == 0) {
      if (*reinterpret_cast<volatile int*>(status) != 0) break;
      if (global_ns() - t0 > limit_ns) {
        report_status(status, kStatusPeerTimeout, kKernelExchange, who, (int)tag);
        break;
      }
    }
  }
  data = 0u;
  return false;
}

__device__ __forceinline__ unsigned int exchange_tag(const unsigned int* step_counter, int slot) {
  return *step_counter * kExchangeSlots + (unsigned)slot + 1u;
}
// words of source rank `src` in inbox `buf` of the window at `window`
__device__ __forceinline__ uint2* inbox_words(unsigned char* window, int buf, int src) {
  return reinterpret_cast<uint2*>(window) + ((size_t)buf * kMaxRanks + src) * Window::kSlotWords;
}
__device__ __forceinline__ uint4 ld_relaxed_sys_v4(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

// Fused consumer side: the two words (4 values) starting at word `first` of each of
// NR batch rows from peer `src`, all loads in flight together, re-read until both
// tags are there (bounded like wait_flag).  Returns the data words in d[b][0..1].
template <int NR>
__device__ __forceinline__ void pull_words(unsigned char* window, int buf, int src, int first, int rows,
                                           unsigned int tag, int* status, unsigned long long limit_ns,
                                           uint32_t (&d)[NR][2]) {
  const uint2* base = inbox_words(window, buf, src) + first;
  uint4 w[NR];
#pragma unroll
  for (int b = 0; b < NR; ++b)
    w[b] = b < rows ? ld_relaxed_sys_v4(base + (size_t)b * 512) : make_uint4(0, tag, 0, tag);
  const unsigned long long t0 = global_ns();
  int polls = 0;
  for (;;) {
    bool all = true;
#pragma unroll
    for (int b = 0; b < NR; ++b)
      if (w[b].y != tag || w[b].w != tag) {
        all = false;
        w[b] = ld_relaxed_sys_v4(base + (size_t)b * 512);
      }
    if (all) break;
    if ((++polls & 63) == 0) {
      if (*reinterpret_cast<volatile int*>(status) != 0) break;
      if (global_ns() - t0 > limit_ns) {
        report_status(status, kStatusPeerTimeout, kKernelExchange, src, (int)tag);
        break;
      }
    }
  }
#pragma unroll
  for (int b = 0; b < NR; ++b) { d[b][0] = w[b].x; d[b][1] = w[b].z; }
}

// Sum of the ranks' partial [rows, 1024] results, in place.  One CTA of 1024
// threads; thread t owns the 8 values t*8 .. t*8+7 = 4 words.
__global__ void __launch_bounds__(1024) exchange_sum_kernel(const ExchangeArgs a) {
  pdl_launch_dependents();
  const int tid = threadIdx.x;
  if (tid == 0) trace_min(a.trace, 0);
  const unsigned int tag = *a.step_counter * kExchangeSlots + (unsigned)a.slot + 1u;
  const bool live = tid * 8 < a.rows * 1024;
  pdl_wait();
  if (tid == 0) { trace_max(a.trace, 1); trace_min(a.trace, 3); }
  if (!live) return;

  const uint4 mine = ldg_cg(a.local + tid * 8);
  const uint32_t mw[4] = {mine.x, mine.y, mine.z, mine.w};
  const size_t word0 = (size_t)a.buf * kMaxRanks * Window::kSlotWords + (size_t)tid * 4;
  for (int r = 0; r < a.size; ++r) {
    if (r == a.rank) continue;
    uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint2*>(a.window[r]) + word0 + (size_t)a.rank * Window::kSlotWords);
    // two 16-byte stores of two words each; a word is never torn (8-byte aligned halves of one store)
    dst[0] = make_uint4(mw[0], tag, mw[1], tag);
    dst[1] = make_uint4(mw[2], tag, mw[3], tag);
  }
  float acc[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) acc[e] = 0.f;
  const uint2* inbox = reinterpret_cast<const uint2*>(a.window[a.rank]) + word0;
  for (int r = 0; r < a.size; ++r) {   // the same order on every rank: identical sums
    uint32_t w[4];
    if (r == a.rank) {
#pragma unroll
      for (int k = 0; k < 4; ++k) w[k] = mw[k];
    } else {
#pragma unroll
      for (int k = 0; k < 4; ++k) wait_word(inbox + (size_t)r * Window::kSlotWords + k, tag, a.status, r, w[k], a.wait_ns);
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) { acc[2 * k] += bf_lo(w[k]); acc[2 * k + 1] += bf_hi(w[k]); }
  }
  uint4 out;
  out.x = pack_bf16(acc[0], acc[1]); out.y = pack_bf16(acc[2], acc[3]);
  out.z = pack_bf16(acc[4], acc[5]); out.w = pack_bf16(acc[6], acc[7]);
  *reinterpret_cast<uint4*>(a.local + tid * 8) = out;
  if (tid == 0) trace_max(a.trace, 2);
}

// The ranks' greedy winners -> the step's tokens; also advances the step counter
// (the last exchange of a step).
struct ExchangeArgmaxArgs {
  unsigned char* window[kMaxRanks];
  int size, rank, rows;
  int shard_rows;
  unsigned int* step_counter;
  const ArgmaxPart* best_local;   // [kMaxRows]
  int* tokens;
  int* tokens_out;
  int* status;
  unsigned long long wait_ns;     // limit of each wait for a peer
};
__global__ void exchange_argmax_kernel(const ExchangeArgmaxArgs a) {
  const int tid = threadIdx.x;   // 32 threads
  const unsigned int tag = *a.step_counter * kExchangeSlots + kExchangeSlots;   // the last tag of this step
  ArgmaxPart mine = ArgmaxPart{-INFINITY, 0};
  if (tid < a.rows) {
    mine = a.best_local[tid];
    for (int r = 0; r < a.size; ++r)
      if (r != a.rank)
        reinterpret_cast<ArgmaxPart*>(a.window[r] + Window::kPairsOff)[a.rank * kMaxRows + tid] = mine;
  }
  __threadfence_system();
  __syncwarp();
  if (tid < a.size && tid != a.rank) {
    st_release_sys(reinterpret_cast<unsigned int*>(a.window[tid] + Window::kPairFlagsOff) + a.rank, tag);
    wait_flag(reinterpret_cast<const unsigned int*>(a.window[a.rank] + Window::kPairFlagsOff) + tid, tag, a.status, tid,
              a.wait_ns);
  }
  __syncwarp();
  if (tid < a.rows) {
    const ArgmaxPart* all = reinterpret_cast<const ArgmaxPart*>(a.window[a.rank] + Window::kPairsOff);
    float v = -INFINITY;
    int idx = 0x7fffffff;
    for (int r = 0; r < a.size; ++r) {
      ArgmaxPart p = mine;
      if (r != a.rank) {
        const int2 raw = __ldcg(reinterpret_cast<const int2*>(all + r * kMaxRows + tid));
        p.value = __int_as_float(raw.x);
        p.index = raw.y;
      }
      const int gi = p.index + r * a.shard_rows;
      if (p.value > v || (p.value == v && gi < idx)) { v = p.value; idx = gi; }
    }
    a.tokens[tid] = idx;
    if (a.tokens_out) a.tokens_out[tid] = idx;
  }
  __syncwarp();
  if (tid == 0) *a.step_counter += 1u;
}

}  // namespace dfb
