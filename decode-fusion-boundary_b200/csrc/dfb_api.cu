// Host side of the C ABI declared in include/dfb_decode.h: decoder object,
// per-step kernel chain (programmatic dependent launch), CUDA-graph cache,
// host-buffer step, standalone launchers.
#include "dfb_kernels.cuh"
#include "dfb_persistent.cuh"
#include "dfb_rowgemv.cuh"
#include "dfb_exchange.cuh"
#include "dfb_pairgemv.cuh"
#include "dfb_tcgemv.cuh"
#include "dfb_attnring.cuh"
#include "dfb_prefill.cuh"

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <new>
#include <tuple>
#include <utility>
#include <vector>

#include "../../include/dfb_decode.h"

using namespace dfb;

// With DFB_DEBUG set in the environment every failing CUDA call is reported on
// stderr with its source line.
static bool dfb_debug() {
  static int on = -1;
  if (on < 0) on = getenv("DFB_DEBUG") ? 1 : 0;
  return on == 1;
}
#define DFB_CUDA(expr)                                                                          \
  do {                                                                                          \
    cudaError_t e_ = (expr);                                                                    \
    if (e_ != cudaSuccess) {                                                                    \
      if (dfb_debug()) fprintf(stderr, "dfb: %s -> %s (line %d)\n", #expr, cudaGetErrorString(e_), __LINE__); \
      return (int)e_;                                                                           \
    }                                                                                           \
  } while (0)

namespace {

typedef __nv_bfloat16 bf16;

// Kernels of one chain overlap on an SM (a dependent kernel's CTAs become
// resident while its predecessor still runs).  An SM changes its split between
// L1 and shared memory only when it is idle, so every kernel of a chain asks
// for the same split; otherwise a kernel that prefers another one starts late.
// `percent` is the share of the SM's 228 KB that goes to shared memory (-1:
// leave the choice to the driver).
int env_int(const char* name, int fallback) {
  const char* v = getenv(name);
  return v && *v ? atoi(v) : fallback;
}

// Tuning knobs of the kernel chain.  Every decoder owns a copy (dfb_set_option
// changes that decoder only); the standalone dfb_launch_* entry points use the
// defaults.
struct ChainOptions {
  int row_max_rows = 1;        // largest batch that takes the FP32 GEMV kernels (0 = never); measured: two rows run
                               // 1-2 % faster on the tensor-core kernels, one row 18 % slower
  int attn_wide_ctas = 2 * 148;// attention grids up to this many CTAs use 256-thread CTAs
  int carve_fp32 = 12;         // chain of FP32 GEMV kernels: little shared memory, L1 helps
  int carve_mma = 50;          // chain of tensor-core GEMV kernels: room for the weight stages, the rest stays L1
  int late_trigger = 0;        // FP32 chain: 1 = a kernel lets its successor start only after it has read its inputs
  int pair_gemv = 1;           // tensor-core chain, K = 1024: 16 weight rows per MMA; 0: stream_gemv_kernel
  int bulk_x = 1;              // FP32 chain: the fused norm fetches its inputs with bulk copies (TMA) instead of loads
  // L2 look-ahead (bulk prefetches issued by kernels with many CTAs for a kernel at least two places down the
  // chain): 1 = gate/up requests the next layer's Wqkv, 2 = down_proj the next layer's Wo, 4 = QKV this layer's
  // Wgu, 8 = o_proj this layer's Wd, 16 = the last layer's gate/up and down_proj request the head of the LM head,
  // 32 = requests are issued after the kernel's own work instead of before its dependency wait (FP32 chain).
  // Off by default: measured neutral to slightly negative at every batch size (the chain is bound by the
  // latency of its dependent hops, not by how early the weights reach the chip).
  int look_ahead = 0;
  int lmhead_ahead_mb = 32;    // MB of the LM head requested by the last layer
  unsigned long long peer_wait_ns = kPeerWaitNs;   // tensor parallel: limit of a wait for a peer
  // batches above row_max_rows: K = 1024 projections on tcgen05.mma (dfb_tcgemv.cuh).  DFB_TCGEN05=<mask> in the
  // environment changes the initial value (a diagnostic switch for the handle-less standalone launchers).
  // Bit mask: 1 = QKV, 2 = gate/up, 4 = LM head.  Default: the LM head only (equal to the mma.sync kernel in time);
  // the two per-layer projections are parity-tested but measured slower inside the chain than their mma.sync
  // counterparts (their longer post-dependency path: bulk copies of x, two issue loops, accumulator read).
  int tcgen05 = env_int("DFB_TCGEN05", 4);
  int carve_tc = 100;          // ... whose chain asks for all of an SM's L1/shared memory as shared memory
  int attn_cluster = env_int("DFB_ATTN_CLUSTER", 148);  // attention grids of at most this many CTAs (and 2..16 chunks
                               // per row) launch the chunks of one (row, KV head) as a thread-block cluster that
                               // merges its partial results through distributed shared memory instead of global
                               // memory and a ticket; 0 = never.  Larger grids lose more to the co-scheduling of
                               // 16-CTA clusters than the merge saves (batch 8 / context 512: 1,009 against 709 us)
  int attn_chunk128 = env_int("DFB_ATTN_CHUNK128", 1);    // 1: context bounds of 65..128 tokens run ONE 128-position chunk
                               // per row and KV head (256 threads, twice the K/V per thread) instead of two merged
                               // 64-position chunks (batch 1: 461 against 474 us per step); N > 1: also every grid
                               // that 128-position chunks bring to at most N CTAs (measured 2-5 % slower than
                               // 64-position chunks with a cluster merge); 0: never
  int attn_ring32_min = env_int("DFB_ATTN_RING32", 0);   // steps with context bound <= 1024 whose rows x 32-position
                               // chunks reach this value (and that the rule below does not take) run the streaming
                               // kernel with 32 positions per CTA; 0 = never.  Off: the streaming kernel's fixed
                               // cost per CTA (q/k norm and rotation for all eight heads, ring start-up) loses to
                               // the register-resident kernel at these sizes (batch 8 / context 512: 811 against
                               // 709 us per step, batch 4: 769 against 636)
  int reg_weights = env_int("DFB_REG_WEIGHTS", 0);   // batches above row_max_rows, a bit mask: 1 = QKV and gate/up,
                               // 2 = o_proj and down_proj, 4 = LM head keep their weights in registers (loaded straight
                               // from global memory in MMA fragment order, pair_gemv_kernel<0, ...> and
                               // reg_store_gemv_kernel) instead of shared-memory stages, so that a kernel's CTAs fit
                               // beside its predecessor's; 8 = those kernels launch up to two CTAs per SM.  Off:
                               // measured slower at every batch (batch 8 / context 512: 758 us with bit 1, 719 with
                               // bit 2, 786 with both, against 709): at 2-8 rows a successor that streams its
                               // weights beside the running kernel takes bandwidth from that kernel's own stream
  int host_io = env_int("DFB_HOST_IO", 6);   // steps from host buffers: 1 = the inputs reach the staging area by a one-warp
                               // kernel that reads pinned host memory, 2 = tokens and status are written to pinned
                               // host memory by a one-warp kernel, instead of copy nodes in the step's graph; 4 = the
                               // host then polls the sequence word that follows the tokens into pinned memory
                               // instead of synchronising the stream
  int attn_ring_min = 200;     // steps whose rows x 64-position chunks of the context bound reach this many take the
                               // streaming attention kernel (dfb_attnring.cuh), which needs about two CTAs per SM
                               // to pay; smaller ones stay on the register-resident kernel; 0 = never
};
const ChainOptions kDefaultOptions;

// Function attributes are per device: remember what was set for (device, function).
std::mutex g_attr_mu;
void prefer_carveout(const void* fn, int percent) {
  if (percent < 0) return;
  static std::map<std::pair<int, const void*>, int> last;
  int dev = 0;
  cudaGetDevice(&dev);
  std::lock_guard<std::mutex> lock(g_attr_mu);
  auto key = std::make_pair(dev, fn);
  auto it = last.find(key);
  if (it != last.end() && it->second == percent) return;
  last[key] = percent;
  cudaFuncSetAttribute(fn, cudaFuncAttributePreferredSharedMemoryCarveout, percent);
}
// Dynamic shared memory beyond 48 KB needs a one-time opt-in per device and function.
cudaError_t ensure_dynamic_smem(const void* fn, int bytes) {
  static std::map<std::pair<int, const void*>, int> done;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  std::lock_guard<std::mutex> lock(g_attr_mu);
  auto key = std::make_pair(dev, fn);
  auto it = done.find(key);
  if (it != done.end() && it->second >= bytes) return cudaSuccess;
  e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e == cudaSuccess) done[key] = bytes;
  return e;
}

// Clusters of more than 8 CTAs need a one-time opt-in per device and function.
cudaError_t ensure_large_clusters(const void* fn) {
  static std::map<std::pair<int, const void*>, int> done;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  std::lock_guard<std::mutex> lock(g_attr_mu);
  auto key = std::make_pair(dev, fn);
  if (done.count(key)) return cudaSuccess;
  e = cudaFuncSetAttribute(fn, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
  if (e == cudaSuccess) done[key] = 1;
  return e;
}

// Largest cluster of the attention kernel that this device can co-schedule (16 needs the non-portable opt-in
// and enough SMs in one GPC; 8 is guaranteed): asked once per device from the occupancy calculator, for the
// heaviest cluster instantiation.  A partitioned or smaller part then merges wider rows through the ticket path.
template <typename Kernel>
int max_attention_cluster(Kernel kernel, int threads) {
  static std::map<int, int> best;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 8;
  {
    std::lock_guard<std::mutex> lock(g_attr_mu);
    auto it = best.find(dev);
    if (it != best.end()) return it->second;
  }
  int result = 8;
  if (ensure_large_clusters((const void*)kernel) == cudaSuccess) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(16, 8, 1);
    cfg.blockDim = dim3(threads);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 16; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) == cudaSuccess && n >= 1) result = 16;
    else (void)cudaGetLastError();
  }
  std::lock_guard<std::mutex> lock(g_attr_mu);
  best[dev] = result;
  return result;
}

struct Launcher {
  cudaStream_t stream;
  bool pdl;
  unsigned long long* trace = nullptr;  // base of the timeline buffer or null
  int count = 0;
  int err = 0;
  int carve = -1;  // preferred shared-memory share of every kernel this launcher launches
  int exchanges = 0;        // tensor-parallel exchanges launched so far in this step
  int push_slot = -1;       // >= 0: the next projection pushes its result to the peers as exchange `push_slot`
  int pull_slot = -1;       // >= 0: the next fused norm adds the peers' partial results of exchange `pull_slot`
  const DfbHandle* tp = nullptr;  // set by a tensor-parallel step
  const ChainOptions* opt = &kDefaultOptions;
  const void* ahead_ptr = nullptr;        // look-ahead request the next launched kernel carries (cleared by it)
  unsigned long long ahead_bytes = 0;
  bool ahead_late = false;
  int embed_rows = 0;                     // rows of the embedding table when a kernel gathers by token id
  bool plain_next = false;  // the next launch follows a foreign kernel (a collective): no programmatic dependency
  unsigned long long* next_trace() const { return trace ? trace + 8 * count : nullptr; }
  // what every GEMV launch of a step carries: the pending look-ahead request and the embedding row count
  void fill_common(GemvArgs& a) {
    a.ahead_ptr = ahead_ptr; a.ahead_bytes = ahead_bytes; a.ahead_late = ahead_late ? 1 : 0; a.embed_rows = embed_rows;
    a.late_trigger = opt->late_trigger;
    ahead_ptr = nullptr; ahead_bytes = 0;
  }
  template <typename Args>
  void launch(void (*kernel)(Args), dim3 grid, dim3 block, const Args& args, bool allow_pdl = true,
              size_t smem = 0, int cluster_x = 0) {
    if (err) return;
    prefer_carveout((const void*)kernel, carve);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n_attr = 0;
    if (pdl && allow_pdl && !plain_next) {
      attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
      ++n_attr;
    }
    if (cluster_x > 1) {   // the grid's x dimension is made of thread-block clusters of this many CTAs
      attr[n_attr].id = cudaLaunchAttributeClusterDimension;
      attr[n_attr].val.clusterDim.x = (unsigned)cluster_x;
      attr[n_attr].val.clusterDim.y = 1;
      attr[n_attr].val.clusterDim.z = 1;
      ++n_attr;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n_attr;
    plain_next = false;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, args);
    if (e != cudaSuccess) {
      err = (int)e;
      if (dfb_debug())
      {
        cudaFuncAttributes fa = {};
        cudaFuncGetAttributes(&fa, (const void*)kernel);
        int occ = -1;
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, (const void*)kernel, (int)block.x, smem);
        fprintf(stderr, "dfb: launch %d failed: %s (grid %u, block %u, smem %zu; regs %d, static smem %zu, "
                "max threads %d, max dyn smem %d, occupancy %d)\n", count, cudaGetErrorString(e), grid.x, block.x, smem,
                fa.numRegs, fa.sharedSizeBytes, fa.maxThreadsPerBlock, fa.maxDynamicSharedSizeBytes, occ);
      }
    }
    ++count;
  }
};

}  // namespace

constexpr int kMaxBurst = 1024;   // steps of one burst (capacity of the pinned token ring)

struct DfbHandle {
  DfbModelDesc m;
  std::vector<DfbLayerWeights> layers;
  int device = 0;
  int sm_count = 148;
  int max_pages = 0;
  size_t kv_layer_elems = 0;
  // options
  bool use_graph = true;
  bool use_pdl = true;
  int lmhead_ctas = 0;
  bool trace_on = false;
  ChainOptions opt;              // tuning knobs of this decoder's kernel chain
  int step_mode = 0;             // 0: chain of per-op kernels (default); 1: one persistent kernel per step
  int persist_ctas = 0;          // grid of the persistent kernel (0 = one CTA per SM)
  int trace_entries = 0;         // timeline entries written by the last traced step
  PLayerWeights* d_layers = nullptr;
  uint2 *x_qkv = nullptr, *x_attn = nullptr, *x_hattn = nullptr, *x_act = nullptr, *x_hmlp = nullptr;
  unsigned int* epoch = nullptr;
  unsigned long long* trace = nullptr;  // [kMaxTraceKernels, 4] globaltimer ns
  // device scratch (one slab)
  void* slab = nullptr;
  int* stage = nullptr;          // ids[8] | positions[8] | row_active[8] | block_tables[8, max_pages]
  bf16* hbuf = nullptr;          // [8, hidden]   output of o_proj / down_proj
  bf16* res[2] = {nullptr, nullptr};
  bf16* qkv = nullptr;           // [8, qkv_rows]
  bf16* attn = nullptr;          // [8, q_size]
  bf16* act = nullptr;           // [8, intermediate]
  float* part_o = nullptr;
  float2* part_ml = nullptr;
  unsigned int* tickets = nullptr;  // [8*kv_heads] attention + [1] lm head
  ArgmaxPart* parts = nullptr;
  int* tokens = nullptr;         // [8]
  int* status = nullptr;         // [4]
  // pinned host staging
  int* host_stage = nullptr;
  int* host_tokens = nullptr;
  unsigned long long sample_seed = 0;   // dfb_set_seed
  unsigned int* sample_ctr = nullptr;   // device: sampled LM-head launches so far (position in the noise stream)
  const float* lm_temps = nullptr;      // temperatures the LM head being enqueued samples with (null = greedy)
  // burst: several steps enqueued at once, tokens published in a pinned ring written by the device
  int* burst_ring = nullptr;            // pinned: [kMaxBurst][8] tokens | [4] status | [1] steps done
  unsigned int* burst_slot = nullptr;   // device
  unsigned int* publish_seq = nullptr;  // device: host-buffer steps published so far (follows the tokens to the host)
  unsigned int published = 0;           // host: the value the next published step will carry
  cudaEvent_t burst_event = nullptr;
  int burst_rows = 0, burst_steps = 0;  // of the burst in flight (0 = none)
  // fixed-slot runtime (dfb_slot_* / dfb_slots_*): host-side state of every slot
  struct Slot {
    bool active = false;
    long long token = 0;        // input of the slot's next step
    long long position = 0;     // pre-decode length of the slot's next step
    float temperature = 0.f;
    std::vector<int> table;     // the slot's block table (physical block ids)
  };
  std::vector<Slot> slots;
  int* burst_status() const { return burst_ring + kMaxBurst * kMaxRows; }
  volatile int* burst_done() const { return burst_ring + kMaxBurst * kMaxRows + 4; }
  cudaStream_t capture_stream = nullptr;
  // One captured step: the input staging (a kernel for device inputs, a host-to-device copy for host inputs),
  // the kernel chain and the copy-out of tokens + status, so that a step is ONE graph launch with no
  // stream-level gaps between its parts.  The staging kernel's arguments and the copy-out's destination follow
  // the caller's pointers: they are patched into the instantiated graph when they change.
  struct StepGraph {
    cudaGraphExec_t exec = nullptr;
    cudaGraph_t graph = nullptr;            // kept: the node handles below belong to it
    cudaGraphNode_t stage_node = nullptr;   // stage_inputs_kernel (device-input steps)
    cudaGraphNode_t out_node = nullptr;     // device-to-device copy of tokens + status (device-input steps with out_tokens)
    StageArgs stage_args = {};
    void* out_ptr = nullptr;
  };
  std::map<long long, StepGraph> graphs;
  int64_t steps = 0;
  int kernels_per_step = 0;
  int last_status[4] = {0, 0, 0, 0};  // last non-zero status word seen by a host-buffer step
  // tensor parallel
  DfbTensorParallel tp = {};     // size 0 or 1: single GPU
  ArgmaxPart* best_local = nullptr;  // [8] this rank's LM-head winners
  ArgmaxPart* best_all = nullptr;    // [ranks, 8]
  bool full_geometry = true;     // unsharded Qwen3-0.6B shapes (what the persistent kernel is built for)
  bool sharded() const { return tp.size > 1; }
  unsigned char* window_local = nullptr;          // this rank's exchange window (its own allocation)
  unsigned char* windows[kMaxRanks] = {};          // every rank's window as mapped into this process
  bool direct = false;                             // exchanges go through the windows instead of the collectives
  bool fused = true;                               // ... and inside the projection / norm kernels, not in a kernel of their own
  unsigned int* tp_step = nullptr;                 // device step counter behind the exchange tags
  unsigned char* loopback[kMaxRanks] = {};         // stand-ins for the peers' windows (dfb_tp_open_loopback)
  int embed_rows() const { return m.vocab * (tp.size > 1 ? tp.size : 1); }   // the embedding table is never sharded
  const bf16* lm_head() const { return (const bf16*)m.embed + (size_t)tp.vocab_offset * m.hidden; }
  int qkv_rows() const { return (m.q_heads + 2 * m.kv_heads) * m.head_dim; }
  int q_size() const { return m.q_heads * m.head_dim; }
  int kv_size() const { return m.kv_heads * m.head_dim; }
  int* st_ids() const { return stage; }
  int* st_pos() const { return stage + 8; }
  int* st_active() const { return stage + 16; }
  int* st_bt() const { return stage + 24; }
  float* st_temps() const { return reinterpret_cast<float*>(stage + 24 + 8 * max_pages); }   // [8] sampling temperatures
  int stage_ints() const { return 32 + 8 * max_pages; }
};

namespace {

constexpr int kMaxTraceKernels = 1024;

// Tensor parallel, fused exchange: a projection that pushes (producer) or a fused norm that pulls.
void tp_fill(Launcher& L, const DfbHandle* h, GemvArgs& a, bool producer) {
  const int slot = producer ? L.push_slot : L.pull_slot;
  if (!h || slot < 0) return;
  a.tp_mode = producer ? 1 : 2;
  a.tp_size = h->tp.size; a.tp_rank = h->tp.rank; a.tp_slot = slot; a.tp_step = h->tp_step;
  a.tp_wait_ns = h->opt.peer_wait_ns;
  for (int r = 0; r < h->tp.size; ++r) a.tp_window[r] = h->windows[r];
  if (producer) L.push_slot = -1; else L.pull_slot = -1;
}

int loads_for_k(int k) { return (k % 256 == 0) ? k / 256 : 0; }

// One CTA per SM at most, and at most half of an SM's registers per CTA, so
// that the CTAs of two consecutive kernels are resident together: the
// successor prefetches its weights while the predecessor computes.
int sm_count_cached() {
  static int count[64] = {};   // per device
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (count[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    count[dev] = n;
  }
  return count[dev];
}
int grid_for(int n_tiles) { const int sms = sm_count_cached(); return n_tiles < sms ? n_tiles : sms; }
// grid of the kernels that keep their weights in registers: one CTA per SM, or (option bit 8) up to two
int reg_grid(const Launcher& L, int n_tiles) {
  const int cap = ((L.opt->reg_weights & 8) ? 2 : 1) * sm_count_cached();
  return n_tiles < cap ? n_tiles : cap;
}

constexpr int kRingFlag = 256;   // bit of the split-bucket value that selects the streaming attention kernel
constexpr int kRing32Flag = 1024;    // ... with kRingFlag: the streaming kernel with 32 positions per CTA
constexpr int kChunk128Flag = 512;   // ... that selects 128-position chunks in the register-resident kernel

// ---- kernel launch wrappers -------------------------------------------------
// Launch one instantiation of the GEMV kernel; its dynamic shared memory (the
// weight stages) exceeds 48 KB, which needs a one-time opt-in per function.
template <int LOADS, int WARPS, int STAGES, int MODE>
void launch_gemv(Launcher& L, GemvArgs& a, int grid, bool allow_pdl = true) {
  constexpr int smem = GemvSmem<LOADS, WARPS>::bytes(STAGES);
  auto kernel = stream_gemv_kernel<LOADS, WARPS, STAGES, MODE>;
  cudaError_t e = ensure_dynamic_smem((const void*)kernel, smem);
  if (e != cudaSuccess) { L.err = (int)e; return; }
  a.trace = L.next_trace();
  L.fill_common(a);
  L.launch(kernel, dim3(grid), dim3(WARPS * 32), a, allow_pdl, smem);
}

// Tensor-core GEMV with 16 weight rows per MMA (dfb_pairgemv.cuh), K = 1024, 3..8 batch rows.
template <int PSTAGES, int MODE>
void launch_pair(Launcher& L, GemvArgs& a, int grid, bool allow_pdl = true, int carve = -2) {
  constexpr int smem = PairSmem::bytes(PSTAGES);
  auto kernel = pair_gemv_kernel<PSTAGES, MODE>;
  cudaError_t e = ensure_dynamic_smem((const void*)kernel, smem);
  if (e != cudaSuccess) { L.err = (int)e; return; }
  a.trace = L.next_trace();
  L.fill_common(a);
  const int chain_carve = L.carve;
  if (carve != -2) L.carve = carve;   // this kernel wants another L1/shared split than the rest of its chain
  L.launch(kernel, dim3(grid), dim3(256), a, allow_pdl, smem);
  L.carve = chain_carve;
}

// ---- tcgen05 GEMV (dfb_tcgemv.cuh) ------------------------------------------------------------------------
// The TMA descriptor of a weight matrix [rows, 1024] bf16 with boxes of {64 columns, box_rows rows} and the
// 128-byte swizzle the MMA's shared-memory descriptors expect.  cuTensorMapEncodeTiled is a driver entry
// point; it is looked up through the runtime so that the library links against no driver stub.  Encoded
// maps are kept per (address, rows, box rows): weights do not move while a decoder lives.
typedef CUresult (*TensorMapEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                           const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                           CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                           CUtensorMapFloatOOBfill);
int tc_weight_map(const void* w, int rows, int box_rows, CUtensorMap* out) {
  static std::mutex mu;
  static TensorMapEncodeTiledFn encode = nullptr;
  static std::map<std::tuple<const void*, int, int>, CUtensorMap> cache;
  std::lock_guard<std::mutex> lock(mu);
  auto key = std::make_tuple(w, rows, box_rows);
  auto it = cache.find(key);
  if (it != cache.end()) { *out = it->second; return 0; }
  if (!encode) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
    if (e != cudaSuccess) return (int)e;
    if (!fn || qres != cudaDriverEntryPointSuccess) return (int)cudaErrorNotSupported;
    encode = (TensorMapEncodeTiledFn)fn;
  }
  if ((uintptr_t)w % 16) return DFB_E_BAD_ARG;
  const cuuint64_t dims[2] = {(cuuint64_t)kTcK, (cuuint64_t)rows};       // innermost first
  const cuuint64_t strides[1] = {(cuuint64_t)kTcK * sizeof(bf16)};       // bytes between rows
  const cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
  const cuuint32_t elem[2] = {1u, 1u};
  CUtensorMap m;
  CUresult r = encode(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(w), dims, strides, box, elem,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    if (dfb_debug()) fprintf(stderr, "dfb: cuTensorMapEncodeTiled failed with %d\n", (int)r);
    return (int)cudaErrorInvalidValue;
  }
  if (cache.size() > 4096) cache.clear();
  cache[key] = m;
  *out = m;
  return 0;
}

template <int MODE, int MT>
void launch_tc(Launcher& L, GemvArgs& a, int n_rows, int box_rows, int grid, bool allow_pdl = true, int carve = -2) {
  using SM = TcSmem<MT>;
  auto kernel = tc_gemv_kernel<MODE, MT>;
  cudaError_t e = ensure_dynamic_smem((const void*)kernel, SM::bytes());
  if (e != cudaSuccess) { L.err = (int)e; return; }
  a.trace = L.next_trace();
  L.fill_common(a);
  TcArgs t;
  memset(&t, 0, sizeof(t));
  t.g = a;
  t.n_rows = n_rows;
  const int rc = tc_weight_map(a.w, n_rows, box_rows, &t.wmap);
  if (rc) { L.err = rc; return; }
  const int chain_carve = L.carve;
  if (carve != -2) L.carve = carve;   // this kernel wants another L1/shared split than the rest of its chain
  L.launch(kernel, dim3(grid), dim3(kTcThreads), t, allow_pdl, SM::bytes());
  L.carve = chain_carve;
}
// whether this launch takes the tcgen05 kernels: a batch above the FP32 kernels' range, no fused tensor-parallel pull
bool use_tc(const Launcher& L, int rows, int which) {
  return (L.opt->tcgen05 & which) && rows > L.opt->row_max_rows && L.pull_slot < 0;
}

// FP32 row-parallel GEMV (dfb_rowgemv.cuh), used for one or two batch rows.
template <int K, int NB, int MODE>
void launch_row_nb(Launcher& L, GemvArgs& a, int grid, bool allow_pdl) {
  constexpr int smem = row_smem_bytes<K, NB>();
  auto kernel = row_gemv_kernel<K, NB, MODE>;
  if (smem > 32 * 1024) {   // static + dynamic shared memory beyond 48 KB needs the opt-in
    cudaError_t e = ensure_dynamic_smem((const void*)kernel, smem);
    if (e != cudaSuccess) { L.err = (int)e; return; }
  }
  a.late_trigger = L.opt->late_trigger;
  a.bulk_x = L.opt->bulk_x;
  L.fill_common(a);
  // The down projection has one CTA per SM's worth of work (128 CTAs): asking for at
  // least 16 KB keeps two of them off one SM (with the 32 KB split of this chain),
  // which measured 25 us per step faster at batch 1 than letting them pair up.
  constexpr int launch_smem = (MODE == kModeStore && K == 3072 && smem < 16 * 1024) ? 16 * 1024 : smem;
  L.launch(kernel, dim3(grid), dim3(RowCfg<K>::kThreads), a, allow_pdl, launch_smem);
}
template <int K, int MODE>
void launch_row(Launcher& L, GemvArgs& a, int rows, int grid, bool allow_pdl = true) {
  a.trace = L.next_trace();
  if (rows == 1) launch_row_nb<K, 1, MODE>(L, a, grid, allow_pdl);
  else if (rows == 2) launch_row_nb<K, 2, MODE>(L, a, grid, allow_pdl);
  else if (rows <= 4) launch_row_nb<K, 4, MODE>(L, a, grid, allow_pdl);
  else launch_row_nb<K, 8, MODE>(L, a, grid, allow_pdl);
}

int launch_norm_qkv(Launcher& L, const bf16* x, const int* ids, const bf16* res_in, bf16* res_out, const bf16* ln_w,
                    const bf16* w, bf16* out, int rows, int hidden, int n, float eps, int* status, bool allow_pdl) {
  if (hidden != 1024 || n % kTileRows) return DFB_E_GEOMETRY;
  GemvArgs a = {};
  a.w = w; a.n_tiles = n / kTileRows; a.rows = rows; a.k = hidden;
  a.x = x; a.ids = ids; a.res_in = res_in; a.res_out = res_out; a.norm_w = ln_w; a.eps = eps;
  a.out = out; a.out_stride = n; a.status = status;
  if (rows <= L.opt->row_max_rows && n % 16 == 0) {
    a.n_tiles = n / 16;
    tp_fill(L, L.tp, a, false);
    launch_row<1024, kModeNormStore>(L, a, rows, a.n_tiles, allow_pdl);
    return L.err;
  }
  if (use_tc(L, rows, 1) && n % 32 == 0) {
    a.n_tiles = n / 32;
    launch_tc<kModeNormStore, 64>(L, a, n, 32, a.n_tiles, allow_pdl);
    return L.err;
  }
  if (L.opt->pair_gemv && n % 16 == 0) {
    a.n_tiles = n / 16;
    tp_fill(L, L.tp, a, false);
    if (L.opt->reg_weights & 1) launch_pair<0, kModeNormStore>(L, a, reg_grid(L, a.n_tiles), allow_pdl);
    else launch_pair<2, kModeNormStore>(L, a, grid_for(a.n_tiles), allow_pdl);
    return L.err;
  }
  launch_gemv<4, 8, 4, kModeNormStore>(L, a, grid_for(a.n_tiles), allow_pdl);
  return L.err;
}

// rows of a row group of the FP32 kernel for input width k (RowCfg<K>::kRows)
int RowRowsFor(int k) { return k <= 1536 ? 16 : 8; }

int launch_linear(Launcher& L, const bf16* x, const bf16* w, bf16* out, int rows, int n, int k, int* status) {
  if (n % kTileRows) return DFB_E_GEOMETRY;
  GemvArgs a = {};
  a.w = w; a.n_tiles = n / kTileRows; a.rows = rows; a.k = k; a.x = x; a.out = out; a.out_stride = n;
  a.status = status;
  // The FP32 kernels cover every input width (the full model's 2048 / 3072 and the
  // tensor-parallel shards 256 ... 1536); the tensor-core kernels 1024, 2048 and 3072.
  const int mma_loads = (k == 1024 || k == 2048 || k == 3072) ? loads_for_k(k) : 0;
  if (rows <= L.opt->row_max_rows || mma_loads == 0 || L.push_slot >= 0) {
    a.n_tiles = n / RowRowsFor(k);
    tp_fill(L, L.tp, a, true);
    switch (k) {
      case 256: launch_row<256, kModeStore>(L, a, rows, a.n_tiles); break;
      case 384: launch_row<384, kModeStore>(L, a, rows, a.n_tiles); break;
      case 512: launch_row<512, kModeStore>(L, a, rows, a.n_tiles); break;
      case 768: launch_row<768, kModeStore>(L, a, rows, a.n_tiles); break;
      case 1024: launch_row<1024, kModeStore>(L, a, rows, a.n_tiles); break;
      case 1536: launch_row<1536, kModeStore>(L, a, rows, a.n_tiles); break;
      case 2048: launch_row<2048, kModeStore>(L, a, rows, a.n_tiles); break;
      case 3072: launch_row<3072, kModeStore>(L, a, rows, a.n_tiles); break;
      default: return DFB_E_GEOMETRY;
    }
    return L.err;
  }
  if ((L.opt->reg_weights & 2) && (k == 2048 || k == 3072)) {
    a.trace = L.next_trace();
    L.fill_common(a);
    const int grid = reg_grid(L, a.n_tiles);
    if (k == 2048) L.launch(reg_store_gemv_kernel<2048>, dim3(grid), dim3(256), a);
    else L.launch(reg_store_gemv_kernel<3072>, dim3(grid), dim3(384), a);
    return L.err;
  }
  const int grid = grid_for(a.n_tiles);
  switch (mma_loads) {
    case 4: launch_gemv<4, 8, 4, kModeStore>(L, a, grid); break;
    case 8: launch_gemv<8, 8, 2, kModeStore>(L, a, grid); break;
    case 12: launch_gemv<12, 8, 2, kModeStore>(L, a, grid); break;
    default: return DFB_E_GEOMETRY;
  }
  return L.err;
}

int launch_gateup(Launcher& L, const bf16* h, const bf16* res_in, bf16* res_out, const bf16* ln_w, const bf16* wgu,
                  bf16* act, int rows, int hidden, int inter, float eps, int* status) {
  if (hidden != 1024 || inter % 4) return DFB_E_GEOMETRY;
  GemvArgs a = {};
  a.w = wgu; a.n_tiles = inter / 4; a.rows = rows; a.k = hidden;
  a.x = h; a.res_in = res_in; a.res_out = res_out; a.norm_w = ln_w; a.eps = eps;
  a.out = act; a.out_stride = inter; a.gate_rows = inter; a.status = status;
  if (rows <= L.opt->row_max_rows && inter % 8 == 0) {
    a.n_tiles = inter / 8;
    tp_fill(L, L.tp, a, false);
    launch_row<1024, kModeNormSwiglu>(L, a, rows, a.n_tiles);
    return L.err;
  }
  if (use_tc(L, rows, 2) && inter % 32 == 0) {
    a.n_tiles = inter / 32;   // a tile = 32 gate rows + the 32 matching up rows
    launch_tc<kModeNormSwiglu, 128>(L, a, 2 * inter, 32, a.n_tiles);
    return L.err;
  }
  if (L.opt->pair_gemv && inter % 8 == 0) {
    a.n_tiles = inter / 8;
    tp_fill(L, L.tp, a, false);
    if (L.opt->reg_weights & 1) launch_pair<0, kModeNormSwiglu>(L, a, reg_grid(L, a.n_tiles));
    else launch_pair<3, kModeNormSwiglu>(L, a, grid_for(a.n_tiles));
    return L.err;
  }
  launch_gemv<4, 8, 6, kModeNormSwiglu>(L, a, grid_for(a.n_tiles));
  return L.err;
}

int launch_lmhead(Launcher& L, DfbHandle* h, const bf16* hid, const bf16* res_in, int rows, int* tokens_out,
                  float* logits_out) {
  const DfbModelDesc& m = h->m;
  GemvArgs a = {};
  a.w = h->lm_head(); a.n_tiles = m.vocab / kTileRows; a.rows = rows; a.k = m.hidden;
  a.x = hid; a.res_in = res_in; a.norm_w = (const bf16*)m.final_norm; a.eps = m.eps;
  a.logits_out = logits_out; a.vocab = m.vocab; a.status = h->status;
  a.parts = h->parts; a.ticket = h->tickets + kMaxRows * m.kv_heads; a.tokens = h->tokens;
  a.tokens_out = h->sharded() ? nullptr : tokens_out;
  a.best_out = h->sharded() ? h->best_local : nullptr;
  a.temps = h->lm_temps; a.sample_ctr = h->sample_ctr; a.sample_seed = h->sample_seed;
  a.sample_idx_offset = h->sharded() ? h->tp.vocab_offset : 0;
  if (rows <= L.opt->row_max_rows && m.vocab % 16 == 0) {
    a.n_tiles = m.vocab / 16;
    int grid = h->lmhead_ctas > 0 ? h->lmhead_ctas : 3 * h->sm_count;
    if (grid > a.n_tiles) grid = a.n_tiles;
    tp_fill(L, L.tp, a, false);
    launch_row<1024, kModeNormArgmax>(L, a, rows, grid);
  } else if (use_tc(L, rows, 4) && !h->sharded()) {
    // persistent CTAs, 64 vocabulary rows per tile, the weight ring never drains between tiles
    a.n_tiles = (m.vocab + 63) / 64;
    int grid = h->lmhead_ctas > 0 ? h->lmhead_ctas : h->sm_count;
    if (grid > a.n_tiles) grid = a.n_tiles;
    launch_tc<kModeNormArgmax, 128>(L, a, m.vocab, 64, grid, true, 100);
  } else if (L.opt->pair_gemv && m.vocab % 16 == 0) {
    // The LM head is long enough to be bound by its per-tile CTA barrier with one CTA per SM: two CTAs of two
    // stages each (93 KB) overlap one another's barriers; that needs more shared memory than the chain's split.
    a.n_tiles = m.vocab / 16;
    int grid = h->lmhead_ctas > 0 ? h->lmhead_ctas : 2 * h->sm_count;
    if (grid > a.n_tiles) grid = a.n_tiles;
    tp_fill(L, L.tp, a, false);
    if (L.opt->reg_weights & 4) launch_pair<0, kModeNormArgmax>(L, a, grid, true);
    else launch_pair<2, kModeNormArgmax>(L, a, grid, true, 100);
  } else {
    int grid = h->lmhead_ctas > 0 ? h->lmhead_ctas : h->sm_count;
    if (grid > a.n_tiles) grid = a.n_tiles;
    launch_gemv<4, 8, 6, kModeNormArgmax>(L, a, grid);
  }
  if (h->sharded() && !L.err && h->direct) {
    ExchangeArgmaxArgs e = {};
    for (int r = 0; r < h->tp.size; ++r) e.window[r] = h->windows[r];
    e.size = h->tp.size; e.rank = h->tp.rank; e.rows = rows; e.shard_rows = m.vocab; e.step_counter = h->tp_step;
    e.best_local = h->best_local; e.tokens = h->tokens; e.tokens_out = tokens_out; e.status = h->status;
    e.wait_ns = h->opt.peer_wait_ns;
    exchange_argmax_kernel<<<1, 32, 0, L.stream>>>(e);
    ++L.count;
    L.plain_next = true;
  } else if (h->sharded() && !L.err) {
    // every rank collects the winners of all vocabulary shards and picks the same token
    if (!h->tp.all_gather) return DFB_E_COMM;
    if (h->tp.all_gather(h->best_local, h->best_all, sizeof(ArgmaxPart) * kMaxRows, h->tp.dtype_int8, h->tp.comm,
                         (dfb_stream_t)L.stream))
      return DFB_E_COMM;
    merge_shard_argmax_kernel<<<1, 32, 0, L.stream>>>(h->best_all, h->tp.size, rows, m.vocab, h->tokens, tokens_out);
    ++L.count;
    L.plain_next = true;
  }
  return L.err;
}

// Tensor parallel: sum the ranks' partial results of a row-parallel projection in place.
int tp_sum(Launcher& L, DfbHandle* h, bf16* buf, int rows) {
  if (!h->sharded() || L.err) return L.err;
  if (h->direct) {
    ExchangeArgs a = {};
    for (int r = 0; r < h->tp.size; ++r) a.window[r] = h->windows[r];
    a.size = h->tp.size; a.rank = h->tp.rank; a.rows = rows; a.slot = L.exchanges; a.buf = L.exchanges & 1;
    a.step_counter = h->tp_step; a.local = buf; a.status = h->status; a.wait_ns = h->opt.peer_wait_ns;
    if (++L.exchanges >= kExchangeSlots - 1) return DFB_E_TOO_LARGE;
    a.trace = L.next_trace();
    L.launch(exchange_sum_kernel, dim3(1), dim3(1024), a);
    return L.err;
  }
  if (!h->tp.all_reduce) return DFB_E_COMM;
  if (h->tp.all_reduce(buf, buf, (size_t)rows * h->m.hidden, h->tp.dtype_bf16, h->tp.op_sum, h->tp.comm,
                       (dfb_stream_t)L.stream))
    return DFB_E_COMM;
  L.plain_next = true;
  return 0;
}

int launch_attention(Launcher& L, DfbHandle* h, int layer, const bf16* qkv, const int* positions, const int* bt,
                     int bt_stride, int bt_cols, const int* row_active, bf16* out, int rows, int nsplit_arg) {
  const bool ring = (nsplit_arg & kRingFlag) != 0;   // set by split_bucket for long contexts
  const bool chunk128 = (nsplit_arg & kChunk128Flag) != 0;   // ... and for small grids
  const int nsplit = nsplit_arg & (kRingFlag - 1);
  const DfbModelDesc& m = h->m;
  AttnArgs a = {};
  a.qkv = qkv; a.qkv_stride = h->qkv_rows(); a.q_size = h->q_size(); a.kv_size = h->kv_size();
  a.positions = positions; a.block_tables = bt; a.bt_stride = bt_stride; a.bt_cols = bt_cols; a.row_active = row_active;
  a.ahead_ptr = L.ahead_ptr; a.ahead_bytes = L.ahead_bytes;
  L.ahead_ptr = nullptr; L.ahead_bytes = 0;
  a.q_norm = (const bf16*)h->layers[layer].q_norm; a.k_norm = (const bf16*)h->layers[layer].k_norm;
  a.cos_sin = m.rope_cos_sin; a.eps = m.eps; a.scale = 1.0f / sqrtf((float)m.head_dim);
  a.k_cache = (bf16*)m.k_cache + (size_t)layer * h->kv_layer_elems;
  a.v_cache = (bf16*)m.v_cache + (size_t)layer * h->kv_layer_elems;
  a.block_size = m.block_size; a.kv_heads = m.kv_heads; a.num_blocks = m.num_blocks; a.max_pos = m.max_model_len;
  a.out = out; a.part_o = h->part_o; a.part_ml = h->part_ml; a.tickets = h->tickets; a.status = h->status;
  a.trace = L.next_trace();
  // The two chains (FP32 / tensor-core GEMV kernels) prefer different shared-memory
  // splits, so each has its own instantiation of the attention kernel.  With few
  // CTAs most SMs are idle during attention: 256 threads then halve each thread's
  // share of the chunk and with it the latency of the CTA.
  const int ctas = nsplit * m.kv_heads * rows;
  a.late_trigger = L.opt->late_trigger;
  if (ring && m.kv_heads == kRingHeads) {
    // long contexts / full batches: one CTA per (row, chunk) for all KV heads, K/V streamed through shared memory
    const bool ring32 = (nsplit_arg & kRing32Flag) != 0;
    auto kernel = ring32 ? paged_attention_ring_kernel<kAttnChunk / 2> : paged_attention_ring_kernel<kAttnChunk>;
    cudaError_t e = ensure_dynamic_smem((const void*)kernel, kRingSmemBytes);
    if (e != cudaSuccess) { L.err = (int)e; return L.err; }
    const int chain_carve = L.carve;
    L.carve = 100;   // two CTAs of about 104 KB per SM
    L.launch(kernel, dim3(nsplit, rows), dim3(kRingThreads), a, true, kRingSmemBytes);
    L.carve = chain_carve;
    return L.err;
  }
  // 2..16 chunks: the chunks of one (row, KV head) form a thread-block cluster and merge in shared memory
  int cluster = (nsplit >= 2 && nsplit <= kAttnClusterMax && ctas <= L.opt->attn_cluster) ? nsplit : 0;
  if (cluster > 8 && cluster > max_attention_cluster(paged_attention_kernel<256, 1, true, 2 * kAttnChunk>, 256)) cluster = 0;
  const bool wide = ctas <= L.opt->attn_wide_ctas;
  const dim3 grid(nsplit, m.kv_heads, rows);
  auto go = [&](auto kernel, int threads) {
    if (cluster > 8) {
      cudaError_t e = ensure_large_clusters((const void*)kernel);
      if (e != cudaSuccess) { L.err = (int)e; return; }
    }
    L.launch(kernel, grid, dim3(threads), a, true, 0, cluster);
  };
  if (chunk128) {
    if (rows <= L.opt->row_max_rows) {
      if (cluster) go(paged_attention_kernel<256, 0, true, 2 * kAttnChunk>, 256);
      else go(paged_attention_kernel<256, 0, false, 2 * kAttnChunk>, 256);
    } else {
      if (cluster) go(paged_attention_kernel<256, 1, true, 2 * kAttnChunk>, 256);
      else go(paged_attention_kernel<256, 1, false, 2 * kAttnChunk>, 256);
    }
  } else if (rows <= L.opt->row_max_rows) {
    if (cluster) { if (wide) go(paged_attention_kernel<256, 0, true>, 256); else go(paged_attention_kernel<128, 0, true>, 128); }
    else if (wide) go(paged_attention_kernel<256, 0, false>, 256);
    else go(paged_attention_kernel<128, 0, false>, 128);
  } else {
    if (cluster) { if (wide) go(paged_attention_kernel<256, 1, true>, 256); else go(paged_attention_kernel<128, 1, true>, 128); }
    else if (wide) go(paged_attention_kernel<256, 1, false>, 256);
    else go(paged_attention_kernel<128, 1, false>, 128);
  }
  return L.err;
}

// Grid of the attention kernel for a context bound: the number of 64-position chunks rounded up to a power
// of two (one captured graph per bucket), plus kRingFlag when rows x chunks is large enough for the streaming
// kernel to keep about two CTAs per SM busy.
int split_bucket(const DfbHandle* h, int max_context, int rows) {
  if (max_context < 1) max_context = 1;
  if (max_context > h->m.max_model_len) max_context = h->m.max_model_len;
  int need = (max_context + kAttnChunk - 1) / kAttnChunk;
  const bool ring64 = h->m.kv_heads == kRingHeads && h->opt.attn_ring_min > 0 && rows * need >= h->opt.attn_ring_min;
  // mid-size steps: the streaming kernel with 32 positions per CTA (its partial results fit the 32 slots up to 1024 tokens)
  const int need32 = (max_context + kAttnChunk / 2 - 1) / (kAttnChunk / 2);
  const bool ring32 = !ring64 && h->m.kv_heads == kRingHeads && h->opt.attn_ring32_min > 0 && need32 <= kMaxSplits &&
                      h->m.block_size % (kAttnChunk / 2) == 0 && rows * need32 >= h->opt.attn_ring32_min;
  const bool ring = ring64 || ring32;
  if (ring32) need = need32;
  // small grids: 128 positions per CTA halve the number of partial results (none up to 128 tokens)
  const int need128 = (max_context + 2 * kAttnChunk - 1) / (2 * kAttnChunk);
  const bool chunk128 = !ring && h->m.block_size % (2 * kAttnChunk) == 0 && h->opt.attn_chunk128 > 0 &&
                        ((need128 == 1 && need == 2) || rows * h->m.kv_heads * need128 <= h->opt.attn_chunk128);
  if (chunk128) need = need128;
  int b = 1;
  while (b < need) b <<= 1;
  if (b > kMaxSplits) b = kMaxSplits;
  return b | (ring ? kRingFlag : 0) | (ring32 ? kRing32Flag : 0) | (chunk128 ? kChunk128Flag : 0);
}

// The whole step as one chain of 5 kernels per layer + the LM head.
//
// Look-ahead: kernel i of the chain also asks for the weights of kernel i + 2 to
// be brought into L2 (a bulk prefetch: no registers, no shared memory, nothing
// waits for it).  Kernel i + 1 requests its own weights into registers / shared
// memory as soon as it is resident, i.e. while kernel i runs; its CTAs that only
// fit on the SMs after kernel i has ended, and everything its first tiles do not
// cover, would otherwise start their HBM round trip after the dependency.
int enqueue_step(DfbHandle* h, int rows, int nsplit, int bt_cols, cudaStream_t stream, float* logits_out) {
  const DfbModelDesc& m = h->m;
  Launcher L{stream, h->use_pdl, h->trace_on ? h->trace : nullptr};
  L.opt = &h->opt;
  L.carve = rows <= h->opt.row_max_rows ? h->opt.carve_fp32
            : ((h->opt.tcgen05 & 3) && !h->sharded()) ? h->opt.carve_tc : h->opt.carve_mma;
  L.tp = h;
  L.embed_rows = h->embed_rows();
  // Tensor parallel over the windows: the projections push their partial results and the next fused norm
  // pulls them, when every consumer of this step runs on a kernel that can (all Qwen3 shards do).
  const bool pair_ok = h->opt.pair_gemv && h->qkv_rows() % 16 == 0 && m.intermediate % 8 == 0 && m.vocab % 16 == 0;
  const bool row_ok = h->qkv_rows() % 16 == 0 && m.intermediate % 8 == 0 && m.vocab % 16 == 0;
  const bool fused = h->sharded() && h->direct && h->fused && (rows <= h->opt.row_max_rows ? row_ok : pair_ok);
  auto exchange = [&](int rc_in) -> int {   // after a row-parallel projection into h->hbuf
    if (rc_in || !h->sharded()) return rc_in;
    if (!fused) return tp_sum(L, h, h->hbuf, rows);
    L.pull_slot = L.exchanges;
    return ++L.exchanges >= kExchangeSlots - 1 ? DFB_E_TOO_LARGE : 0;
  };
  const int ahead = h->opt.look_ahead;
  const size_t b_qkv = sizeof(bf16) * (size_t)h->qkv_rows() * m.hidden, b_o = sizeof(bf16) * (size_t)m.hidden * h->q_size();
  const size_t b_gu = sizeof(bf16) * 2 * (size_t)m.intermediate * m.hidden, b_d = sizeof(bf16) * (size_t)m.hidden * m.intermediate;
  size_t b_lm = (size_t)h->opt.lmhead_ahead_mb << 20;
  if (b_lm > sizeof(bf16) * (size_t)m.vocab * m.hidden) b_lm = sizeof(bf16) * (size_t)m.vocab * m.hidden;
  auto want = [&](int bit, const void* p, size_t bytes) {
    if (ahead & bit) { L.ahead_ptr = p; L.ahead_bytes = bytes; L.ahead_late = (ahead & 32) != 0; }
  };
  int rc = 0;
  int cur = 0;  // index of the residual buffer holding the current residual
  for (int l = 0; l < m.layers && !rc; ++l) {
    const DfbLayerWeights& w = h->layers[l];
    const bool last = l + 1 == m.layers;
    want(4, w.wgu, b_gu);
    if (l == 0) {
      // embedding rows are gathered by token id; the residual starts as the embedding itself.
      // No PDL on the first kernel: it must observe the staged inputs of this step.
      rc = launch_norm_qkv(L, (const bf16*)m.embed, h->st_ids(), nullptr, h->res[cur], (const bf16*)w.ln_in,
                           (const bf16*)w.wqkv, h->qkv, rows, m.hidden, h->qkv_rows(), m.eps, h->status, false);
    } else {
      rc = launch_norm_qkv(L, h->hbuf, nullptr, h->res[cur], h->res[cur ^ 1], (const bf16*)w.ln_in,
                           (const bf16*)w.wqkv, h->qkv, rows, m.hidden, h->qkv_rows(), m.eps, h->status, true);
      cur ^= 1;
    }
    if (rc) break;
    // attention requests nothing: at short contexts its grid is a handful of CTAs, far too few to issue from
    rc = launch_attention(L, h, l, h->qkv, h->st_pos(), h->st_bt(), h->max_pages, bt_cols, h->st_active(), h->attn, rows,
                          nsplit);
    if (rc) break;
    if (fused) L.push_slot = L.exchanges;
    want(8, w.wd, b_d);
    rc = exchange(launch_linear(L, h->attn, (const bf16*)w.wo, h->hbuf, rows, m.hidden, h->q_size(), h->status));
    if (rc) break;
    if (last) want(16, h->lm_head(), b_lm / 2);
    else want(1, h->layers[l + 1].wqkv, b_qkv);
    rc = launch_gateup(L, h->hbuf, h->res[cur], h->res[cur ^ 1], (const bf16*)w.ln_post, (const bf16*)w.wgu, h->act,
                       rows, m.hidden, m.intermediate, m.eps, h->status);
    cur ^= 1;
    if (rc) break;
    if (fused) L.push_slot = L.exchanges;
    if (last) want(16, (const char*)h->lm_head() + b_lm / 2, b_lm - b_lm / 2);
    else want(2, h->layers[l + 1].wo, b_o);
    rc = exchange(launch_linear(L, h->act, (const bf16*)w.wd, h->hbuf, rows, m.hidden, m.intermediate, h->status));
  }
  if (!rc) rc = launch_lmhead(L, h, h->hbuf, h->res[cur], rows, nullptr, logits_out);
  h->kernels_per_step = L.count;
  h->trace_entries = L.count;
  return rc ? rc : L.err;
}

// The whole step as one persistent kernel (dfb_persistent.cuh).
int enqueue_persistent(DfbHandle* h, int rows, cudaStream_t stream, float* logits_out) {
  const DfbModelDesc& m = h->m;
  PersistArgs a = {};
  a.layers = h->d_layers; a.n_layers = m.layers; a.rows = rows; a.q_heads = m.q_heads; a.kv_heads = m.kv_heads;
  a.intermediate = m.intermediate; a.vocab = m.vocab; a.eps = m.eps; a.scale = 1.0f / sqrtf((float)m.head_dim);
  a.embed = (const bf16*)m.embed; a.final_norm = (const bf16*)m.final_norm; a.cos_sin = m.rope_cos_sin;
  a.ids = h->st_ids(); a.positions = h->st_pos(); a.block_tables = h->st_bt(); a.bt_stride = h->max_pages;
  a.row_active = h->st_active();
  a.k_cache = (bf16*)m.k_cache; a.v_cache = (bf16*)m.v_cache; a.kv_layer_elems = h->kv_layer_elems;
  a.block_size = m.block_size; a.num_blocks = m.num_blocks; a.max_pos = m.max_model_len;
  a.x_qkv = h->x_qkv; a.x_attn = h->x_attn; a.x_hattn = h->x_hattn; a.x_act = h->x_act; a.x_hmlp = h->x_hmlp;
  a.part_o = h->part_o; a.part_ml = h->part_ml; a.tickets = h->tickets; a.parts = h->parts; a.tokens = h->tokens;
  a.logits_out = logits_out; a.epoch = h->epoch; a.status = h->status;
  a.trace = h->trace_on ? h->trace : nullptr;
  int grid = h->persist_ctas > 0 ? h->persist_ctas : h->sm_count;
  if (grid > h->sm_count) grid = h->sm_count;   // every CTA must be resident at once
  Launcher L{stream, false};
  L.launch(decode_step_persistent_kernel, dim3(grid), dim3(kPThreads), a, false, kPDynSmem);
  h->kernels_per_step = 1;
  h->trace_entries = 5 * m.layers + 1;
  return L.err;
}

// What surrounds the kernel chain of one step.
struct StepIo {
  const StageArgs* stage = nullptr;   // device inputs: arguments of stage_inputs_kernel
  bool host = false;                  // host inputs: h->host_stage -> h->stage before, h->tokens -> h->host_tokens after
  int* out_tokens = nullptr;          // device inputs: optional copy of tokens + status
  bool sampling = false;              // the staged temperatures are live: the LM head samples rows with T > 1e-10
  bool burst = false;                 // inputs are already staged on the device; publish_tokens_kernel follows the chain
};

int enqueue_whole_step(DfbHandle* h, int rows, int nsplit, int bt_cols, const StepIo& io, cudaStream_t stream,
                       float* logits_out) {
  if (io.burst) {
    // staged by the burst's one host-to-device copy, advanced on the device from step to step
  } else if (io.host && (h->opt.host_io & 1)) {
    copy_ints_kernel<<<1, 128, 0, stream>>>(h->host_stage, h->stage, h->stage_ints());
    DFB_CUDA(cudaGetLastError());
  } else if (io.host) {
    DFB_CUDA(cudaMemcpyAsync(h->stage, h->host_stage, sizeof(int) * h->stage_ints(), cudaMemcpyHostToDevice, stream));
  } else if (io.stage) {
    stage_inputs_kernel<<<1, 128, 0, stream>>>(*io.stage);
    DFB_CUDA(cudaGetLastError());
  }
  if (io.sampling && h->step_mode == 1) return DFB_E_BAD_ARG;   // the persistent kernel's LM head is greedy only
  h->lm_temps = io.sampling ? h->st_temps() : nullptr;
  int rc = h->step_mode == 1 ? enqueue_persistent(h, rows, stream, logits_out)
                             : enqueue_step(h, rows, nsplit, bt_cols, stream, logits_out);
  h->lm_temps = nullptr;
  if (rc) return rc;
  if (io.burst) {
    PublishArgs p = {};
    p.tokens = h->tokens; p.status = h->status; p.ids_out = h->st_ids(); p.positions_out = h->st_pos();
    p.rows = rows; p.embed_rows = h->embed_rows(); p.slot = h->burst_slot;
    p.ring = h->burst_ring; p.ring_status = h->burst_status(); p.ring_done = h->burst_done();
    publish_tokens_kernel<<<1, 32, 0, stream>>>(p);
    DFB_CUDA(cudaGetLastError());
  } else if (io.host && (h->opt.host_io & 2)) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1); cfg.blockDim = dim3(32); cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (h->use_pdl && !h->sharded()) ? 1 : 0;   // after a collective: an ordinary dependency
    DFB_CUDA(cudaLaunchKernelEx(&cfg, publish_result_kernel, (const int*)h->tokens, h->host_tokens, kMaxRows + 4,
                                h->publish_seq));
  } else if (io.host) {
    DFB_CUDA(cudaMemcpyAsync(h->host_tokens, h->tokens, sizeof(int) * (kMaxRows + 4), cudaMemcpyDeviceToHost, stream));
  } else if (io.out_tokens) {
    DFB_CUDA(cudaMemcpyAsync(io.out_tokens, h->tokens, sizeof(int) * (kMaxRows + 4), cudaMemcpyDeviceToDevice, stream));
  }
  return 0;
}

// The captured graph of a step geometry: one per (rows, split bucket, filled block-table columns, kind of
// inputs / outputs); captured and instantiated on first use (or ahead of time by dfb_warm).
int get_step_graph(DfbHandle* h, int rows, int nsplit, int bt_cols, const StepIo& io, DfbHandle::StepGraph** out) {
  const bool persistent = h->step_mode == 1;
  const int io_kind = (io.burst ? 0 : io.host ? 3 : (io.out_tokens ? 2 : 1)) + (io.sampling ? 4 : 0);
  const long long key = ((persistent ? (1ll << 40) : 0ll) + (((long long)bt_cols * 16 + rows) * 4096 + nsplit) * 2 +
                         (h->use_pdl ? 1 : 0)) * 8 + io_kind;
  auto it = h->graphs.find(key);
  if (it == h->graphs.end()) {
    cudaGraph_t graph = nullptr;
    DFB_CUDA(cudaStreamBeginCapture(h->capture_stream, cudaStreamCaptureModeThreadLocal));
    int rc = enqueue_whole_step(h, rows, nsplit, bt_cols, io, h->capture_stream, nullptr);
    cudaError_t e = cudaStreamEndCapture(h->capture_stream, &graph);
    if (rc) { if (graph) cudaGraphDestroy(graph); return rc; }
    if (e != cudaSuccess) return (int)e;
    DfbHandle::StepGraph g;
    if (!io.host && !io.burst) {
      // find the two nodes whose parameters follow the caller's pointers
      size_t n = 0;
      e = cudaGraphGetNodes(graph, nullptr, &n);
      std::vector<cudaGraphNode_t> nodes(n);
      if (e == cudaSuccess && n) e = cudaGraphGetNodes(graph, nodes.data(), &n);
      for (size_t i = 0; e == cudaSuccess && i < n; ++i) {
        cudaGraphNodeType type;
        e = cudaGraphNodeGetType(nodes[i], &type);
        if (e != cudaSuccess) break;
        if (type == cudaGraphNodeTypeKernel && !g.stage_node) {
          cudaKernelNodeParams kp = {};
          e = cudaGraphKernelNodeGetParams(nodes[i], &kp);
          if (e == cudaSuccess && kp.func == (void*)stage_inputs_kernel) g.stage_node = nodes[i];
        } else if (type == cudaGraphNodeTypeMemcpy && io.out_tokens) {
          g.out_node = nodes[i];
        }
      }
      if (e == cudaSuccess && (!g.stage_node || (io.out_tokens && !g.out_node))) e = cudaErrorInvalidValue;
      if (e != cudaSuccess) { cudaGraphDestroy(graph); return (int)e; }
      g.stage_args = *io.stage;
      g.out_ptr = io.out_tokens;
    }
    e = cudaGraphInstantiate(&g.exec, graph, 0);
    if (e != cudaSuccess) { cudaGraphDestroy(graph); return (int)e; }
    g.graph = graph;
    it = h->graphs.emplace(key, g).first;
  }
  *out = &it->second;
  return 0;
}

int run_step(DfbHandle* h, int rows, int nsplit, int bt_cols, const StepIo& io, cudaStream_t stream, float* logits_out) {
  if (!h->use_graph || logits_out) return enqueue_whole_step(h, rows, nsplit, bt_cols, io, stream, logits_out);
  DfbHandle::StepGraph* gp = nullptr;
  int rc = get_step_graph(h, rows, nsplit, bt_cols, io, &gp);
  if (rc) return rc;
  DfbHandle::StepGraph& g = *gp;
  if (!io.host && !io.burst) {
    if (memcmp(&g.stage_args, io.stage, sizeof(StageArgs)) != 0) {
      StageArgs args = *io.stage;
      void* params[1] = {&args};
      cudaKernelNodeParams kp = {};
      kp.func = (void*)stage_inputs_kernel;
      kp.gridDim = dim3(1); kp.blockDim = dim3(128); kp.sharedMemBytes = 0; kp.kernelParams = params; kp.extra = nullptr;
      DFB_CUDA(cudaGraphExecKernelNodeSetParams(g.exec, g.stage_node, &kp));
      g.stage_args = args;
    }
    if (io.out_tokens && g.out_ptr != io.out_tokens) {
      DFB_CUDA(cudaGraphExecMemcpyNodeSetParams1D(g.exec, g.out_node, io.out_tokens, h->tokens, sizeof(int) * (kMaxRows + 4),
                                                  cudaMemcpyDeviceToDevice));
      g.out_ptr = io.out_tokens;
    }
  }
  DFB_CUDA(cudaGraphLaunch(g.exec, stream));
  return 0;
}

}  // namespace

extern "C" {

const char* dfb_error_string(int code) {
  switch (code) {
    case 0: return "success";
    case DFB_E_BAD_ARG: return "dfb: bad argument";
    case DFB_E_GEOMETRY: return "dfb: unsupported model geometry";
    case DFB_E_ABI: return "dfb: ABI version mismatch";
    case DFB_E_DEVICE_STATUS: return "dfb: a kernel reported an error (see dfb_read_status)";
    case DFB_E_TOO_LARGE: return "dfb: request exceeds a fixed capacity";
    case DFB_E_COMM: return "dfb: a tensor-parallel collective failed";
    default: return code > 0 ? cudaGetErrorString((cudaError_t)code) : "dfb: unknown error";
  }
}

int dfb_create(const DfbModelDesc* d, DfbHandle** out) {
  if (!d || !out) return DFB_E_BAD_ARG;
  *out = nullptr;
  if (d->abi_version != DFB_ABI_VERSION) return DFB_E_ABI;
  // full model: q_size 2048, intermediate 3072; tensor-parallel shards: 1/2, 1/4, 1/8 of both
  const int q_size = d->q_heads * d->head_dim, inter = d->intermediate;
  const bool q_ok = q_size == 2048 || q_size == 1024 || q_size == 512 || q_size == 256;
  const bool i_ok = inter == 3072 || inter == 1536 || inter == 768 || inter == 384;
  if (d->hidden != 1024 || d->head_dim != kHeadDim || d->q_heads != 2 * d->kv_heads || d->kv_heads < 1 ||
      d->kv_heads > 8 || d->layers < 1 || d->vocab % kTileRows || d->vocab < kTileRows || !q_ok || !i_ok ||
      d->max_model_len < 1 || d->max_model_len > kMaxSplits * kAttnChunk || d->block_size < kAttnChunk ||
      d->block_size % kAttnChunk || d->num_blocks < 1)
    return DFB_E_GEOMETRY;
  if (!d->embed || !d->final_norm || !d->rope_cos_sin || !d->layer_weights || !d->k_cache || !d->v_cache)
    return DFB_E_BAD_ARG;
  DfbHandle* h = new (std::nothrow) DfbHandle();
  if (!h) return (int)cudaErrorMemoryAllocation;
  h->m = *d;
  h->full_geometry = q_size == 2048 && inter == 3072;
  h->layers.assign(d->layer_weights, d->layer_weights + d->layers);
  h->m.layer_weights = nullptr;
  for (const DfbLayerWeights& w : h->layers)
    if (!w.ln_in || !w.wqkv || !w.q_norm || !w.k_norm || !w.wo || !w.ln_post || !w.wgu || !w.wd) {
      delete h;
      return DFB_E_BAD_ARG;
    }
  cudaError_t e = cudaGetDevice(&h->device);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&h->sm_count, cudaDevAttrMultiProcessorCount, h->device);
  if (e != cudaSuccess) { delete h; return (int)e; }
  h->max_pages = (d->max_model_len + d->block_size - 1) / d->block_size;
  h->kv_layer_elems = (size_t)d->num_blocks * d->block_size * d->kv_heads * d->head_dim;

  // one slab, 256-byte aligned pieces
  size_t off = 0;
  auto carve = [&](size_t bytes) { size_t o = off; off += (bytes + 255) & ~(size_t)255; return o; };
  const size_t o_stage = carve(sizeof(int) * h->stage_ints());
  const size_t o_h = carve(sizeof(bf16) * kMaxRows * d->hidden);
  const size_t o_r0 = carve(sizeof(bf16) * kMaxRows * d->hidden);
  const size_t o_r1 = carve(sizeof(bf16) * kMaxRows * d->hidden);
  const size_t o_qkv = carve(sizeof(bf16) * kMaxRows * h->qkv_rows());
  const size_t o_attn = carve(sizeof(bf16) * kMaxRows * h->q_size());
  const size_t o_act = carve(sizeof(bf16) * kMaxRows * d->intermediate);
  const size_t o_po = carve(sizeof(float) * kMaxRows * d->kv_heads * kMaxSplits * 2 * kHeadDim);
  const size_t o_pml = carve(sizeof(float2) * kMaxRows * d->kv_heads * kMaxSplits * 2);
  const size_t o_tk = carve(sizeof(unsigned) * (2 * kMaxRows * d->kv_heads + 1));
  const size_t o_layers = carve(sizeof(PLayerWeights) * d->layers);
  const size_t o_xqkv = carve(sizeof(uint2) * kMaxRows * h->qkv_rows() / 2);
  const size_t o_xattn = carve(sizeof(uint2) * kMaxRows * h->q_size() / 2);
  const size_t o_xhattn = carve(sizeof(uint2) * kMaxRows * d->hidden / 2);
  const size_t o_xact = carve(sizeof(uint2) * kMaxRows * d->intermediate / 2);
  const size_t o_xhmlp = carve(sizeof(uint2) * kMaxRows * d->hidden / 2);
  const size_t o_epoch = carve(sizeof(unsigned) * 4);
  const size_t o_parts = carve(sizeof(ArgmaxPart) * kMaxRows * 4096);
  const size_t o_trace = carve(sizeof(unsigned long long) * 8 * kMaxTraceKernels);
  const size_t o_tok = carve(sizeof(int) * (kMaxRows + 4));  // tokens[8] | status[4], contiguous
  const size_t o_best = carve(sizeof(ArgmaxPart) * kMaxRows * 9);  // this rank's winners | all ranks' (up to 8)
  const size_t o_tpstep = carve(sizeof(unsigned) * 4);
  const size_t o_sctr = carve(sizeof(unsigned) * 4);
  const size_t o_bslot = carve(sizeof(unsigned) * 4);
  const size_t o_pseq = carve(sizeof(unsigned) * 4);
  e = cudaMalloc(&h->slab, off);
  if (e == cudaSuccess) e = cudaMemset(h->slab, 0, off);
  if (e == cudaSuccess) e = cudaMallocHost((void**)&h->host_stage, sizeof(int) * h->stage_ints());
  if (e == cudaSuccess) e = cudaMallocHost((void**)&h->host_tokens, sizeof(int) * (kMaxRows + 8));
  if (e == cudaSuccess) h->host_tokens[kMaxRows + 4] = 0;
  if (e == cudaSuccess) e = cudaMallocHost((void**)&h->burst_ring, sizeof(int) * (kMaxBurst * kMaxRows + 8));
  if (e == cudaSuccess) e = cudaEventCreateWithFlags(&h->burst_event, cudaEventDisableTiming);
  if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&h->capture_stream, cudaStreamNonBlocking);
  if (e != cudaSuccess) { dfb_destroy(h); return (int)e; }
  char* s = (char*)h->slab;
  h->stage = (int*)(s + o_stage); h->hbuf = (bf16*)(s + o_h);
  h->res[0] = (bf16*)(s + o_r0); h->res[1] = (bf16*)(s + o_r1);
  h->qkv = (bf16*)(s + o_qkv); h->attn = (bf16*)(s + o_attn); h->act = (bf16*)(s + o_act);
  h->part_o = (float*)(s + o_po); h->part_ml = (float2*)(s + o_pml); h->tickets = (unsigned*)(s + o_tk);
  h->parts = (ArgmaxPart*)(s + o_parts); h->trace = (unsigned long long*)(s + o_trace);
  h->d_layers = (PLayerWeights*)(s + o_layers);
  h->x_qkv = (uint2*)(s + o_xqkv); h->x_attn = (uint2*)(s + o_xattn); h->x_hattn = (uint2*)(s + o_xhattn);
  h->x_act = (uint2*)(s + o_xact); h->x_hmlp = (uint2*)(s + o_xhmlp); h->epoch = (unsigned int*)(s + o_epoch);
  {
    static_assert(sizeof(PLayerWeights) == sizeof(DfbLayerWeights), "layer pointer tables must have one layout");
    const unsigned one = 1u;   // tags are built from the epoch and must never be zero
    e = cudaMemcpy(h->d_layers, h->layers.data(), sizeof(PLayerWeights) * d->layers, cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMemcpy(h->epoch, &one, sizeof(one), cudaMemcpyHostToDevice);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(decode_step_persistent_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPDynSmem);
    if (e != cudaSuccess) { dfb_destroy(h); return (int)e; }
  }
  h->tokens = (int*)(s + o_tok); h->status = h->tokens + kMaxRows;
  h->best_local = (ArgmaxPart*)(s + o_best); h->best_all = h->best_local + kMaxRows;
  h->tp_step = (unsigned int*)(s + o_tpstep);
  h->sample_ctr = (unsigned int*)(s + o_sctr);
  h->burst_slot = (unsigned int*)(s + o_bslot);
  h->publish_seq = (unsigned int*)(s + o_pseq);
  *out = h;
  return 0;
}

void dfb_destroy(DfbHandle* h) {
  if (!h) return;
  // a burst in flight still writes the pinned token ring: let it finish before anything is freed
  if (h->burst_steps && h->burst_event) cudaEventSynchronize(h->burst_event);
  for (auto& kv : h->graphs) { cudaGraphExecDestroy(kv.second.exec); cudaGraphDestroy(kv.second.graph); }
  if (h->capture_stream) cudaStreamDestroy(h->capture_stream);
  for (int r = 0; r < kMaxRanks; ++r) {
    if (h->loopback[r]) cudaFree(h->loopback[r]);
    else if (h->windows[r] && h->windows[r] != h->window_local) cudaIpcCloseMemHandle(h->windows[r]);
  }
  if (h->window_local) cudaFree(h->window_local);
  if (h->host_stage) cudaFreeHost(h->host_stage);
  if (h->host_tokens) cudaFreeHost(h->host_tokens);
  if (h->burst_ring) cudaFreeHost(h->burst_ring);
  if (h->burst_event) cudaEventDestroy(h->burst_event);
  if (h->slab) cudaFree(h->slab);
  delete h;
}

int dfb_set_tensor_parallel(DfbHandle* h, const DfbTensorParallel* tp) {
  if (!h || !tp) return DFB_E_BAD_ARG;
  if ((tp->size != 2 && tp->size != 4 && tp->size != 8) || tp->rank < 0 || tp->rank >= tp->size ||
      tp->vocab_offset < 0)
    return DFB_E_BAD_ARG;
  if (h->step_mode != 0 || h->steps != 0) return DFB_E_BAD_ARG;  // before the first step, kernel chain only
  h->tp = *tp;
  // the narrow o_proj / down_proj shards run on the FP32 kernels at every batch; two rows stay there as a whole
  if (h->opt.row_max_rows == 1) h->opt.row_max_rows = 2;
  for (auto& kv : h->graphs) { cudaGraphExecDestroy(kv.second.exec); cudaGraphDestroy(kv.second.graph); }
  h->graphs.clear();
  return 0;
}

int dfb_tp_window_handle(DfbHandle* h, void* handle_out) {
  if (!h || !handle_out || !h->sharded()) return DFB_E_BAD_ARG;
  if (!h->window_local) {
    DFB_CUDA(cudaMalloc((void**)&h->window_local, Window::kBytes));
    DFB_CUDA(cudaMemset(h->window_local, 0, Window::kBytes));
  }
  cudaIpcMemHandle_t ipc;
  DFB_CUDA(cudaIpcGetMemHandle(&ipc, h->window_local));
  static_assert(sizeof(ipc) == DFB_TP_HANDLE_BYTES, "IPC handle size");
  memcpy(handle_out, &ipc, sizeof(ipc));
  return 0;
}

int dfb_tp_open_peers(DfbHandle* h, const void* handles) {
  if (!h || !handles || !h->sharded() || !h->window_local || h->direct || h->steps != 0) return DFB_E_BAD_ARG;
  const char* p = (const char*)handles;
  for (int r = 0; r < h->tp.size; ++r) {
    if (r == h->tp.rank) { h->windows[r] = h->window_local; continue; }
    cudaIpcMemHandle_t ipc;
    memcpy(&ipc, p + (size_t)r * DFB_TP_HANDLE_BYTES, sizeof(ipc));
    void* mapped = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&mapped, ipc, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
      for (int q = 0; q < r; ++q)
        if (q != h->tp.rank && h->windows[q]) { cudaIpcCloseMemHandle(h->windows[q]); h->windows[q] = nullptr; }
      return (int)e;
    }
    h->windows[r] = (unsigned char*)mapped;
  }
  h->direct = true;
  for (auto& kv : h->graphs) { cudaGraphExecDestroy(kv.second.exec); cudaGraphDestroy(kv.second.graph); }
  h->graphs.clear();
  return 0;
}

int dfb_tp_open_loopback(DfbHandle* h) {
  if (!h || !h->sharded() || h->direct || h->steps != 0) return DFB_E_BAD_ARG;
  if (!h->window_local) {
    DFB_CUDA(cudaMalloc((void**)&h->window_local, Window::kBytes));
    DFB_CUDA(cudaMemset(h->window_local, 0, Window::kBytes));
  }
  for (int r = 0; r < h->tp.size; ++r) {
    if (r == h->tp.rank) { h->windows[r] = h->window_local; continue; }
    DFB_CUDA(cudaMalloc((void**)&h->loopback[r], Window::kBytes));
    DFB_CUDA(cudaMemset(h->loopback[r], 0, Window::kBytes));
    h->windows[r] = h->loopback[r];
  }
  h->direct = true;
  for (auto& kv : h->graphs) { cudaGraphExecDestroy(kv.second.exec); cudaGraphDestroy(kv.second.graph); }
  h->graphs.clear();
  return 0;
}

int dfb_set_option(DfbHandle* h, int option, int value) {
  if (!h) return DFB_E_BAD_ARG;
  // every option below may change which kernels a captured step holds
  auto drop_graphs = [&]() {
    for (auto& kv : h->graphs) { cudaGraphExecDestroy(kv.second.exec); cudaGraphDestroy(kv.second.graph); }
    h->graphs.clear();
  };
  switch (option) {
    case DFB_OPT_USE_GRAPH: h->use_graph = value != 0; return 0;
    case DFB_OPT_USE_PDL: h->use_pdl = value != 0; return 0;
    case DFB_OPT_ROW_GEMV:
      if (value < 0 || value > kMaxRows) return DFB_E_BAD_ARG;
      h->opt.row_max_rows = value;
      break;
    case DFB_OPT_SMEM_CARVEOUT:
      if (value < -1 || value > 100) return DFB_E_BAD_ARG;
      h->opt.carve_fp32 = value;
      break;
    case DFB_OPT_SMEM_CARVEOUT_MMA:
      if (value < -1 || value > 100) return DFB_E_BAD_ARG;
      h->opt.carve_mma = value;
      h->opt.carve_tc = value;
      break;
    case DFB_OPT_TP_FUSED:
      if (value != 0 && value != 1) return DFB_E_BAD_ARG;
      h->fused = value != 0;
      break;
    case DFB_OPT_BULK_X:
      if (value != 0 && value != 1) return DFB_E_BAD_ARG;
      h->opt.bulk_x = value;
      break;
    case DFB_OPT_PAIR_GEMV:
      if (value != 0 && value != 1) return DFB_E_BAD_ARG;
      h->opt.pair_gemv = value;
      break;
    case DFB_OPT_LATE_TRIGGER:
      if (value != 0 && value != 1) return DFB_E_BAD_ARG;
      h->opt.late_trigger = value;
      break;
    case DFB_OPT_ATTN_WIDE:
      if (value < 0) return DFB_E_BAD_ARG;
      h->opt.attn_wide_ctas = value;
      break;
    case DFB_OPT_LOOK_AHEAD:
      if (value < 0 || value > 63) return DFB_E_BAD_ARG;
      h->opt.look_ahead = value;
      break;
    case DFB_OPT_LMHEAD_AHEAD_MB:
      if (value < 0 || value > 100) return DFB_E_BAD_ARG;
      h->opt.lmhead_ahead_mb = value;
      break;
    case DFB_OPT_ATTN_RING:
      if (value < 0) return DFB_E_BAD_ARG;
      h->opt.attn_ring_min = value;
      break;
    case DFB_OPT_HOST_IO:
      if (value < 0 || value > 7) return DFB_E_BAD_ARG;
      h->opt.host_io = value;
      break;
    case DFB_OPT_REG_WEIGHTS:
      if (value < 0 || value > 15) return DFB_E_BAD_ARG;
      h->opt.reg_weights = value;
      break;
    case DFB_OPT_ATTN_RING32:
      if (value < 0) return DFB_E_BAD_ARG;
      h->opt.attn_ring32_min = value;
      break;
    case DFB_OPT_ATTN_CHUNK128:
      if (value < 0) return DFB_E_BAD_ARG;
      h->opt.attn_chunk128 = value;
      break;
    case DFB_OPT_ATTN_CLUSTER:
      if (value < 0) return DFB_E_BAD_ARG;
      h->opt.attn_cluster = value;
      break;
    case DFB_OPT_TCGEN05:
      if (value < 0 || value > 7) return DFB_E_BAD_ARG;
      h->opt.tcgen05 = value;
      break;
    case DFB_OPT_PEER_WAIT_US:
      if (value < 1) return DFB_E_BAD_ARG;
      h->opt.peer_wait_ns = 1000ull * (unsigned long long)value;
      break;
    case DFB_OPT_STEP_MODE:
      if (value != 0 && value != 1) return DFB_E_BAD_ARG;
      if (value == 1 && (!h->full_geometry || h->sharded())) return DFB_E_GEOMETRY;  // built for the whole model only
      h->step_mode = value;
      return 0;
    case DFB_OPT_PERSIST_CTAS:
      if (value < 0 || value > 4096) return DFB_E_BAD_ARG;
      h->persist_ctas = value;
      break;
    case DFB_OPT_TRACE:
      h->trace_on = value != 0;
      break;
    case DFB_OPT_LMHEAD_CTAS:
      if (value < 0 || value > 4096) return DFB_E_BAD_ARG;
      h->lmhead_ctas = value;
      break;
    default: return DFB_E_BAD_ARG;
  }
  drop_graphs();
  return 0;
}

int dfb_warm(DfbHandle* h, int32_t max_rows, int32_t max_context, int32_t kinds, int32_t* graphs_out) {
  if (graphs_out) *graphs_out = h ? (int32_t)h->graphs.size() : 0;
  if (!h || max_rows < 1 || max_rows > kMaxRows || max_context < 1 || kinds < 1 || kinds > 31) return DFB_E_BAD_ARG;
  if (max_context > h->m.max_model_len) max_context = h->m.max_model_len;
  if (!h->use_graph) return 0;
  // dummy arguments of the input staging kernel for the device-pointer kinds: a launch patches them anyway
  StageArgs a = {};
  a.prev_tokens = h->tokens; a.positions = reinterpret_cast<const int64_t*>(h->stage);
  a.block_tables = h->st_bt(); a.bt_stride_in = h->max_pages; a.bt_stride_out = h->max_pages;
  a.embed_rows = h->embed_rows(); a.status = h->status;
  a.ids_out = h->st_ids(); a.positions_out = h->st_pos(); a.bt_out = h->st_bt(); a.row_active_out = h->st_active();
  a.temps_out = h->st_temps();
  const int bs = h->m.block_size;
  for (int rows = 1; rows <= max_rows; ++rows) {
    a.rows = rows;
    for (int ctx = 1;; ctx += kAttnChunk) {
      if (ctx > max_context) ctx = max_context;
      const int cols = (ctx + bs - 1) / bs;
      a.bt_cols = cols;
      // context bounds a step of this many columns can come with: the exact one, and the full last column
      // (what dfb_decode_step assumes without a max_context hint)
      const int bounds[2] = {ctx, cols * bs};
      for (int bi = 0; bi < 2; ++bi) {
        const int nsplit = split_bucket(h, bounds[bi], rows);
        for (int sampling = 0; sampling < 2; ++sampling) {
          if (sampling && !(kinds & 16)) continue;
          if (sampling && h->step_mode == 1) continue;
          a.temps = sampling ? h->st_temps() : nullptr;
          for (int kind = 0; kind < 4; ++kind) {
            if (!(kinds & (1 << kind))) continue;
            if (kind == 0 && h->step_mode == 1) continue;   // bursts run on the kernel chain only
            StepIo io;
            io.sampling = sampling != 0;
            if (kind == 0) io.burst = true;
            else if (kind == 3) io.host = true;
            else { io.stage = &a; io.out_tokens = kind == 2 ? h->tokens : nullptr; }
            DfbHandle::StepGraph* g = nullptr;
            int rc = get_step_graph(h, rows, nsplit, cols, io, &g);
            if (rc) return rc;
          }
        }
      }
      if (ctx >= max_context) break;
    }
  }
  if (graphs_out) *graphs_out = (int32_t)h->graphs.size();
  return 0;
}

int dfb_store_kvcache(const void* key, const void* value, int64_t key_stride, int64_t value_stride, void* k_cache,
                      void* v_cache, const int32_t* slot_mapping, int32_t n_tokens, int32_t row_elems,
                      int64_t num_slots, int32_t* status, dfb_stream_t stream) {
  if (!key || !value || !k_cache || !v_cache || !slot_mapping || n_tokens < 0 || num_slots < 1) return DFB_E_BAD_ARG;
  // rows are moved in 16-byte pieces: bf16 rows of a multiple of 8 elements, 16-byte aligned bases and strides
  if (row_elems < 8 || row_elems % 8 || key_stride < row_elems || value_stride < row_elems || key_stride % 8 ||
      value_stride % 8)
    return DFB_E_BAD_ARG;
  if (((uintptr_t)key | (uintptr_t)value | (uintptr_t)k_cache | (uintptr_t)v_cache) & 15) return DFB_E_BAD_ARG;
  if (n_tokens == 0) return 0;
  int grid = 8 * sm_count_cached();
  if (grid > n_tokens) grid = n_tokens;
  store_kvcache_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(
      (const unsigned char*)key, (const unsigned char*)value, 2 * key_stride, 2 * value_stride, (unsigned char*)k_cache,
      (unsigned char*)v_cache, slot_mapping, n_tokens, 2 * row_elems, num_slots, status);
  DFB_CUDA(cudaGetLastError());
  return 0;
}

int dfb_prefill_attention(const void* q, const void* k, const void* v, void* out, const int32_t* cu_seqlens_q,
                          const int32_t* cu_seqlens_k, int32_t batch, int32_t max_seqlen_q, int64_t q_stride,
                          int64_t k_stride, int64_t v_stride, int64_t out_stride, int32_t q_heads, int32_t kv_heads,
                          int32_t head_dim, float scale, const int32_t* block_tables, int32_t block_table_stride,
                          int32_t block_size, int32_t num_blocks, int32_t* status, dfb_stream_t stream) {
  if (!q || !k || !v || !out || !cu_seqlens_q || batch < 1 || max_seqlen_q < 1) return DFB_E_BAD_ARG;
  if (head_dim != kHeadDim || q_heads < 1 || kv_heads < 1 || q_heads % kv_heads) return DFB_E_GEOMETRY;
  // 16-byte pieces of K / V rows and 4-byte pieces of Q / out rows: aligned bases, strides in multiples of 8
  if (q_stride < (int64_t)q_heads * head_dim || out_stride < (int64_t)q_heads * head_dim ||
      k_stride < (int64_t)kv_heads * head_dim || v_stride < (int64_t)kv_heads * head_dim)
    return DFB_E_BAD_ARG;
  if ((q_stride | k_stride | v_stride | out_stride) % 8) return DFB_E_BAD_ARG;
  if (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)out) & 15) return DFB_E_BAD_ARG;
  int block_shift = 0;
  if (block_tables) {
    if (block_table_stride < 1 || block_size < 1 || num_blocks < 1 || !cu_seqlens_k) return DFB_E_BAD_ARG;
    if (block_size & (block_size - 1)) return DFB_E_GEOMETRY;   // blocks of a power of two tokens (the reference's are 256)
    while ((1 << block_shift) < block_size) ++block_shift;
  }
  const void* fn = block_tables ? (const void*)prefill_attention_kernel<true> : (const void*)prefill_attention_kernel<false>;
  cudaError_t e = ensure_dynamic_smem(fn, kPfSmemBytes);
  if (e != cudaSuccess) return (int)e;
  prefer_carveout(fn, 100);   // two CTAs of 68 KB per SM (registers allow no more)
  PrefillArgs a = {};
  a.q = (const bf16*)q; a.k = (const bf16*)k; a.v = (const bf16*)v; a.out = (bf16*)out;
  a.cu_seqlens = cu_seqlens_q; a.cu_seqlens_k = cu_seqlens_k ? cu_seqlens_k : cu_seqlens_q;
  a.block_tables = block_tables; a.bt_stride = block_table_stride; a.block_size = block_size; a.num_blocks = num_blocks;
  a.block_shift = block_shift;
  a.q_stride = q_stride; a.k_stride = k_stride; a.v_stride = v_stride; a.out_stride = out_stride;
  a.q_heads = q_heads; a.kv_heads = kv_heads; a.scale = scale; a.status = status;
  const dim3 grid((max_seqlen_q + kPfTile - 1) / kPfTile, q_heads, batch);
  if (block_tables) prefill_attention_kernel<true><<<grid, 128, kPfSmemBytes, (cudaStream_t)stream>>>(a);
  else prefill_attention_kernel<false><<<grid, 128, kPfSmemBytes, (cudaStream_t)stream>>>(a);
  DFB_CUDA(cudaGetLastError());
  return 0;
}

int dfb_set_seed(DfbHandle* h, uint64_t seed) {
  if (!h) return DFB_E_BAD_ARG;
  // the seed is a kernel argument of every captured LM head; the noise stream restarts at step 0
  for (auto& kv : h->graphs) { cudaGraphExecDestroy(kv.second.exec); cudaGraphDestroy(kv.second.graph); }
  h->graphs.clear();
  h->sample_seed = seed;
  DFB_CUDA(cudaMemset(h->sample_ctr, 0, sizeof(unsigned)));
  return 0;
}

int dfb_decode_step(DfbHandle* h, const DfbStepDesc* s, dfb_stream_t stream_) {
  if (!h || !s) return DFB_E_BAD_ARG;
  cudaStream_t stream = (cudaStream_t)stream_;
  if (s->rows < 1 || s->rows > kMaxRows || !s->positions || !s->block_tables) return DFB_E_BAD_ARG;
  if (s->block_table_cols < 1 || s->block_table_stride < s->block_table_cols) return DFB_E_BAD_ARG;
  if (s->block_table_cols > h->max_pages) return DFB_E_TOO_LARGE;
  StageArgs a = {};
  a.ids = s->input_ids; a.positions = s->positions; a.block_tables = s->block_tables;
  a.bt_cols = s->block_table_cols; a.bt_stride_in = s->block_table_stride; a.bt_stride_out = h->max_pages;
  a.row_active = s->row_active; a.rows = s->rows;
  a.prev_tokens = h->tokens;   // input_ids == NULL: the previous step's tokens become this step's input ids
  a.embed_rows = h->embed_rows(); a.status = h->status;
  a.ids_out = h->st_ids(); a.positions_out = h->st_pos(); a.bt_out = h->st_bt();
  a.row_active_out = h->st_active();
  a.temps = s->temperatures; a.temps_out = h->st_temps();
  // The attention grid is sized from the caller's bound; a bound that does not cover the filled
  // block-table columns would only be caught on the device (status 6), so never go below one column.
  int bound = s->block_table_cols * h->m.block_size;
  if (s->max_context > 0 && s->max_context < bound) {
    bound = s->max_context;
    const int lowest = (s->block_table_cols - 1) * h->m.block_size + 1;   // the last column holds at least one token
    if (bound < lowest) bound = lowest;
  }
  StepIo io;
  io.stage = &a;
  io.out_tokens = s->out_tokens;
  io.sampling = s->temperatures != nullptr;
  if (io.sampling && s->out_logits && h->step_mode == 1) return DFB_E_BAD_ARG;
  int rc = run_step(h, s->rows, split_bucket(h, bound, s->rows), s->block_table_cols, io, stream, s->out_logits);
  if (rc) return rc;
  ++h->steps;
  return 0;
}

int dfb_decode_step_host(DfbHandle* h, int32_t rows, const int64_t* input_ids, const int64_t* positions,
                         const int32_t* block_tables, int32_t cols, const int32_t* row_active, int32_t* out_tokens,
                         dfb_stream_t stream_) {
  return dfb_decode_step_host_sampled(h, rows, input_ids, positions, block_tables, cols, row_active, nullptr,
                                      out_tokens, stream_);
}

// Validates one step's host inputs (for a burst: of all its steps) and packs them into the pinned staging
// buffer: ids | positions | row_active | block tables | temperatures.  Returns 0 and the largest context.
static int pack_host_inputs(DfbHandle* h, int rows, const int64_t* input_ids, const int64_t* positions,
                            const int32_t* block_tables, int cols, const int32_t* row_active,
                            const float* temperatures, int steps, int* max_ctx_out) {
  if (!h || !input_ids || !positions || !block_tables) return DFB_E_BAD_ARG;
  if (rows < 1 || rows > kMaxRows || cols < 1 || steps < 1) return DFB_E_BAD_ARG;
  if (cols > h->max_pages) return DFB_E_TOO_LARGE;
  if (h->burst_steps) return DFB_E_BAD_ARG;   // a burst is in flight: collect it first (it owns the staging buffers)
  int* hs = h->host_stage;
  int max_ctx = 1;
  for (int r = 0; r < rows; ++r) {
    const int64_t last = positions[r] + steps - 1;                              // position of the row's last step
    if (positions[r] < 0 || last >= h->m.max_model_len) return DFB_E_BAD_ARG;
    if (last >= (int64_t)cols * h->m.block_size) return DFB_E_BAD_ARG;         // beyond the block table given
    // ids index the whole (replicated) embedding table, also on a tensor-parallel shard
    if (input_ids[r] < 0 || input_ids[r] >= h->embed_rows()) return DFB_E_BAD_ARG;
    hs[r] = (int)input_ids[r];
    hs[8 + r] = (int)positions[r];
    hs[16 + r] = row_active ? row_active[r] : 1;
    if (positions[r] + 1 > max_ctx) max_ctx = (int)positions[r] + 1;
    for (int c = 0; c < cols; ++c) hs[24 + r * h->max_pages + c] = block_tables[r * cols + c];
    if (temperatures) {
      if (!(temperatures[r] >= 0.f)) return DFB_E_BAD_ARG;   // negative or NaN (sampling_params.py:14-15)
      memcpy(&hs[24 + 8 * h->max_pages + r], &temperatures[r], sizeof(float));
    }
  }
  *max_ctx_out = max_ctx;
  return 0;
}

int dfb_decode_step_host_sampled(DfbHandle* h, int32_t rows, const int64_t* input_ids, const int64_t* positions,
                                 const int32_t* block_tables, int32_t cols, const int32_t* row_active,
                                 const float* temperatures, int32_t* out_tokens, dfb_stream_t stream_) {
  if (!out_tokens) return DFB_E_BAD_ARG;
  int max_ctx = 1;
  int rc = pack_host_inputs(h, rows, input_ids, positions, block_tables, cols, row_active, temperatures, 1, &max_ctx);
  if (rc) return rc;
  cudaStream_t stream = (cudaStream_t)stream_;
  StepIo io;
  io.sampling = temperatures != nullptr;
  io.host = true;      // the two copies between the pinned staging buffers and the device are part of the step's graph
  rc = run_step(h, rows, split_bucket(h, max_ctx, rows), cols, io, stream, nullptr);
  if (rc) return rc;
  bool arrived = false;
  if ((h->opt.host_io & 2) && (h->opt.host_io & 4) && h->use_graph) {
    // The publishing kernel is the step's last node: once its sequence word has changed in pinned memory the
    // tokens and the status are there.  Polling it saves the driver's stream synchronisation; after about a
    // tenth of a second without it (an error, a debugger) the ordinary synchronisation takes over.
    const int want = (int)++h->published;
    volatile int* word = h->host_tokens + kMaxRows + 4;
    for (long spin = 0; spin < 40000000l; ++spin)
      if (*word == want) { arrived = true; break; }
  } else if (h->opt.host_io & 2) {
    ++h->published;
  }
  if (!arrived) DFB_CUDA(cudaStreamSynchronize(stream));
  for (int r = 0; r < rows; ++r) out_tokens[r] = h->host_tokens[r];
  ++h->steps;
  if (h->host_tokens[kMaxRows]) {
    h->last_status[0] = h->host_tokens[kMaxRows]; h->last_status[1] = h->host_tokens[kMaxRows + 1];
    h->last_status[2] = h->host_tokens[kMaxRows + 2]; h->last_status[3] = h->host_tokens[kMaxRows + 3];
    DFB_CUDA(cudaMemsetAsync(h->status, 0, sizeof(int) * 4, stream));
    return DFB_E_DEVICE_STATUS;
  }
  return 0;
}

// ---- fixed-slot runtime --------------------------------------------------------------------------------
// The decode side of a continuous-batching engine: DFB_MAX_SLOTS fixed slots whose sequences come and go
// between steps; a step packs the live slots, in slot order, into launches of at most DFB_MAX_ROWS rows (every
// geometry is a cached graph, so a change of the live set never captures once dfb_warm has run), advances
// tokens and positions on the host side of the slots, and reports which slots emitted.
int dfb_slot_set(DfbHandle* h, int32_t slot, int32_t active, int64_t token, int64_t position,
                 const int32_t* block_table, int32_t cols, float temperature) {
  if (!h || slot < 0 || slot >= DFB_MAX_SLOTS) return DFB_E_BAD_ARG;
  if (h->slots.empty()) h->slots.resize(DFB_MAX_SLOTS);
  DfbHandle::Slot& s = h->slots[slot];
  if (!active) { s = DfbHandle::Slot(); return 0; }   // retired: the scheduler may hand its blocks to someone else
  if (!block_table || cols < 1) return DFB_E_BAD_ARG;
  if (cols > h->max_pages) return DFB_E_TOO_LARGE;
  if (token < 0 || token >= h->embed_rows() || position < 0 || position >= h->m.max_model_len) return DFB_E_BAD_ARG;
  if (!(temperature >= 0.f)) return DFB_E_BAD_ARG;
  for (int c = 0; c < cols; ++c)
    if (block_table[c] < 0 || block_table[c] >= h->m.num_blocks) return DFB_E_BAD_ARG;
  s.active = true; s.token = token; s.position = position; s.temperature = temperature;
  s.table.assign(block_table, block_table + cols);
  return 0;
}

int dfb_slot_get(DfbHandle* h, int32_t slot, int32_t* active, int64_t* token, int64_t* position) {
  if (!h || slot < 0 || slot >= DFB_MAX_SLOTS) return DFB_E_BAD_ARG;
  const bool known = !h->slots.empty();
  if (active) *active = known && h->slots[slot].active ? 1 : 0;
  if (token) *token = known ? h->slots[slot].token : 0;
  if (position) *position = known ? h->slots[slot].position : 0;
  return 0;
}

int dfb_slots_step(DfbHandle* h, long long* sampled_tokens, int32_t* emitted, dfb_stream_t stream) {
  if (!h || !sampled_tokens || !emitted) return DFB_E_BAD_ARG;
  for (int i = 0; i < DFB_MAX_SLOTS; ++i) { sampled_tokens[i] = 0; emitted[i] = 0; }
  if (h->slots.empty()) return 0;
  // live slots that have room for their next token: a slot whose position ran past its block table (the
  // scheduler has to append a block first) or past the model length sits the step out and emits nothing
  int live[DFB_MAX_SLOTS], n_live = 0;
  for (int i = 0; i < DFB_MAX_SLOTS; ++i) {
    const DfbHandle::Slot& s = h->slots[i];
    if (!s.active) continue;
    if (s.position >= h->m.max_model_len || s.position >= (long long)s.table.size() * h->m.block_size) continue;
    live[n_live++] = i;
  }
  int first_error = 0;
  for (int g0 = 0; g0 < n_live; g0 += kMaxRows) {
    const int rows = n_live - g0 < kMaxRows ? n_live - g0 : kMaxRows;
    int64_t ids[kMaxRows], pos[kMaxRows];
    float temps[kMaxRows];
    int32_t out[kMaxRows];
    int cols = 1;
    bool sampled = false;
    for (int r = 0; r < rows; ++r) {
      const DfbHandle::Slot& s = h->slots[live[g0 + r]];
      ids[r] = s.token; pos[r] = s.position; temps[r] = s.temperature;
      sampled = sampled || s.temperature > 1e-10f;
      // columns the launch needs: those that hold this row's context (the tables may be longer)
      const int need = (int)(s.position / h->m.block_size) + 1;
      if (need > cols) cols = need;
    }
    std::vector<int32_t> bt((size_t)rows * cols, 0);   // right-padded with block 0, as the engine pads its tables
    for (int r = 0; r < rows; ++r) {
      const DfbHandle::Slot& s = h->slots[live[g0 + r]];
      for (int c = 0; c < cols && c < (int)s.table.size(); ++c) bt[(size_t)r * cols + c] = s.table[c];
    }
    const int rc = dfb_decode_step_host_sampled(h, rows, ids, pos, bt.data(), cols, nullptr, sampled ? temps : nullptr,
                                                out, stream);
    if (rc && rc != DFB_E_DEVICE_STATUS) return rc;
    if (rc && !first_error) first_error = rc;
    for (int r = 0; r < rows; ++r) {
      DfbHandle::Slot& s = h->slots[live[g0 + r]];
      s.token = out[r];
      s.position += 1;
      sampled_tokens[live[g0 + r]] = out[r];
      emitted[live[g0 + r]] = 1;
    }
  }
  return first_error;
}

int dfb_slots_run(DfbHandle* h, int32_t max_steps, dfb_token_callback callback, void* context, dfb_stream_t stream) {
  if (!h || !callback || max_steps < 1) return DFB_E_BAD_ARG;
  long long tokens[DFB_MAX_SLOTS];
  int32_t emitted[DFB_MAX_SLOTS];
  for (int step = 0; step < max_steps; ++step) {
    const int rc = dfb_slots_step(h, tokens, emitted, stream);
    if (rc) return rc;
    int any = 0;
    for (int i = 0; i < DFB_MAX_SLOTS; ++i) any |= emitted[i];
    if (!any) return 0;                       // nothing is live, or every live slot waits for a block
    // the callback may retire, admit or re-point slots (dfb_slot_set) before the next step
    if (callback(context, tokens, emitted, DFB_MAX_SLOTS)) return 0;
  }
  return 0;
}

int dfb_decode_burst_enqueue(DfbHandle* h, int32_t rows, int32_t steps, const int64_t* input_ids,
                             const int64_t* positions, const int32_t* block_tables, int32_t cols,
                             const int32_t* row_active, const float* temperatures, dfb_stream_t stream_) {
  if (steps > kMaxBurst) return DFB_E_TOO_LARGE;
  int max_ctx = 1;
  int rc = pack_host_inputs(h, rows, input_ids, positions, block_tables, cols, row_active, temperatures, steps, &max_ctx);
  if (rc) return rc;
  if (h->step_mode == 1) return DFB_E_BAD_ARG;   // the persistent kernel takes its inputs per launch
  cudaStream_t stream = (cudaStream_t)stream_;
  *h->burst_done() = 0;
  DFB_CUDA(cudaMemsetAsync(h->burst_slot, 0, sizeof(unsigned), stream));
  DFB_CUDA(cudaMemcpyAsync(h->stage, h->host_stage, sizeof(int) * h->stage_ints(), cudaMemcpyHostToDevice, stream));
  StepIo io;
  io.sampling = temperatures != nullptr;
  io.burst = true;
  for (int s = 0; s < steps; ++s) {
    // the attention grid follows the growing context; everything else of the step is the same graph
    rc = run_step(h, rows, split_bucket(h, max_ctx + s, rows), cols, io, stream, nullptr);
    if (rc) return rc;
    ++h->steps;
  }
  DFB_CUDA(cudaEventRecord(h->burst_event, stream));
  h->burst_rows = rows;
  h->burst_steps = steps;
  return 0;
}

int dfb_decode_burst_collect(DfbHandle* h, int32_t wait, int32_t* out_tokens, int32_t* steps_done) {
  if (!h || !out_tokens || !steps_done) return DFB_E_BAD_ARG;
  *steps_done = 0;
  if (!h->burst_steps) return DFB_E_BAD_ARG;
  if (wait) DFB_CUDA(cudaEventSynchronize(h->burst_event));
  int done = *h->burst_done();   // written by the device after the tokens of that step (system-wide fence between)
  if (done > h->burst_steps) done = h->burst_steps;
  for (int s = 0; s < done; ++s)
    for (int r = 0; r < h->burst_rows; ++r) out_tokens[s * h->burst_rows + r] = h->burst_ring[s * kMaxRows + r];
  *steps_done = done;
  if (done < h->burst_steps) return 0;     // still running (wait == 0): call again
  h->burst_steps = 0;
  const int* st = h->burst_status();
  if (st[0]) {
    h->last_status[0] = st[0]; h->last_status[1] = st[1]; h->last_status[2] = st[2]; h->last_status[3] = st[3];
    DFB_CUDA(cudaMemset(h->status, 0, sizeof(int) * 4));
    return DFB_E_DEVICE_STATUS;
  }
  return 0;
}

int dfb_decode_burst_host(DfbHandle* h, int32_t rows, int32_t steps, const int64_t* input_ids,
                          const int64_t* positions, const int32_t* block_tables, int32_t cols,
                          const int32_t* row_active, const float* temperatures, int32_t* out_tokens,
                          dfb_stream_t stream) {
  if (!out_tokens) return DFB_E_BAD_ARG;
  int rc = dfb_decode_burst_enqueue(h, rows, steps, input_ids, positions, block_tables, cols, row_active,
                                    temperatures, stream);
  if (rc) return rc;
  int done = 0;
  return dfb_decode_burst_collect(h, 1, out_tokens, &done);
}

int dfb_read_status(DfbHandle* h, DfbStatus* out) {
  if (!h || !out) return DFB_E_BAD_ARG;
  int st[4];
  DFB_CUDA(cudaMemcpy(st, h->status, sizeof(st), cudaMemcpyDeviceToHost));
  if (!st[0] && h->last_status[0]) {
    memcpy(st, h->last_status, sizeof(st));
    memset(h->last_status, 0, sizeof(h->last_status));
    out->device_status = st[0];
    out->detail[0] = st[1]; out->detail[1] = st[2]; out->detail[2] = st[3];
    out->steps = h->steps;
    out->kernels_per_step = h->kernels_per_step;
    return DFB_E_DEVICE_STATUS;
  }
  out->device_status = st[0];
  out->detail[0] = st[1]; out->detail[1] = st[2]; out->detail[2] = st[3];
  out->steps = h->steps;
  out->kernels_per_step = h->kernels_per_step;
  if (st[0]) DFB_CUDA(cudaMemset(h->status, 0, sizeof(st)));
  return st[0] ? DFB_E_DEVICE_STATUS : 0;
}

int dfb_read_trace(DfbHandle* h, uint64_t* out, int32_t max_kernels) {
  if (!h || !out || max_kernels < 1) return DFB_E_BAD_ARG;
  int n = max_kernels > kMaxTraceKernels ? kMaxTraceKernels : max_kernels;
  DFB_CUDA(cudaMemcpy(out, h->trace, sizeof(uint64_t) * 8 * n, cudaMemcpyDeviceToHost));
  if (h->trace_entries < n) n = h->trace_entries;
  // re-arm: minima (words 0 and 3) start at the largest value, maxima at zero
  std::vector<unsigned long long> init(8 * kMaxTraceKernels, 0ull);
  for (int i = 0; i < kMaxTraceKernels; ++i) { init[8 * i] = ~0ull; init[8 * i + 3] = ~0ull; }
  DFB_CUDA(cudaMemcpy(h->trace, init.data(), sizeof(unsigned long long) * init.size(), cudaMemcpyHostToDevice));
  return n;
}

// ---- standalone launchers ----------------------------------------------------
int dfb_launch_rmsnorm_qkv(const void* hh, const int32_t* ids, const void* residual, void* residual_out,
                           const void* ln_w, const void* wqkv, void* qkv_out, int32_t rows, int32_t hidden,
                           int32_t qkv_rows, float eps, dfb_stream_t stream) {
  if (!hh || !ln_w || !wqkv || !qkv_out || rows < 1 || rows > kMaxRows) return DFB_E_BAD_ARG;
  if (ids && residual) return DFB_E_BAD_ARG;
  Launcher L{(cudaStream_t)stream, false};
  return launch_norm_qkv(L, (const bf16*)hh, ids, (const bf16*)residual, (bf16*)residual_out, (const bf16*)ln_w,
                         (const bf16*)wqkv, (bf16*)qkv_out, rows, hidden, qkv_rows, eps, nullptr, false);
}

int dfb_launch_attention(DfbHandle* h, int32_t layer, const void* qkv, const int32_t* positions,
                         const int32_t* block_tables, int32_t block_table_stride, const int32_t* row_active,
                         void* attn_out, int32_t rows, int32_t max_context, dfb_stream_t stream) {
  if (!h || !qkv || !positions || !block_tables || !attn_out) return DFB_E_BAD_ARG;
  if (rows < 1 || rows > kMaxRows || layer < 0 || layer >= h->m.layers) return DFB_E_BAD_ARG;
  Launcher L{(cudaStream_t)stream, false};
  L.opt = &h->opt;
  return launch_attention(L, h, layer, (const bf16*)qkv, positions, block_tables, block_table_stride, 0, row_active,
                          (bf16*)attn_out, rows, split_bucket(h, max_context > 0 ? max_context : h->m.max_model_len, rows));
}

int dfb_launch_linear(const void* x, const void* w, void* out, int32_t rows, int32_t n, int32_t k,
                      dfb_stream_t stream) {
  if (!x || !w || !out || rows < 1 || rows > kMaxRows) return DFB_E_BAD_ARG;
  Launcher L{(cudaStream_t)stream, false};
  return launch_linear(L, (const bf16*)x, (const bf16*)w, (bf16*)out, rows, n, k, nullptr);
}

int dfb_launch_rmsnorm_gateup_swiglu(const void* hh, const void* residual, void* residual_out, const void* ln_w,
                                     const void* wgu, void* act_out, int32_t rows, int32_t hidden,
                                     int32_t intermediate, float eps, dfb_stream_t stream) {
  if (!hh || !residual || !ln_w || !wgu || !act_out || rows < 1 || rows > kMaxRows) return DFB_E_BAD_ARG;
  Launcher L{(cudaStream_t)stream, false};
  return launch_gateup(L, (const bf16*)hh, (const bf16*)residual, (bf16*)residual_out, (const bf16*)ln_w,
                       (const bf16*)wgu, (bf16*)act_out, rows, hidden, intermediate, eps, nullptr);
}

int dfb_launch_lmhead_argmax(DfbHandle* h, const void* hidden_in, const void* residual, int32_t* out_tokens,
                             float* out_logits, int32_t rows, dfb_stream_t stream) {
  return dfb_launch_lmhead_sample(h, hidden_in, residual, nullptr, out_tokens, out_logits, rows, stream);
}

int dfb_launch_lmhead_sample(DfbHandle* h, const void* hidden_in, const void* residual, const float* temperatures,
                             int32_t* out_tokens, float* out_logits, int32_t rows, dfb_stream_t stream) {
  if (!h || !hidden_in || !residual || rows < 1 || rows > kMaxRows) return DFB_E_BAD_ARG;
  Launcher L{(cudaStream_t)stream, false};
  L.opt = &h->opt;
  h->lm_temps = temperatures;
  const int rc = launch_lmhead(L, h, (const bf16*)hidden_in, (const bf16*)residual, rows, out_tokens, out_logits);
  h->lm_temps = nullptr;
  return rc;
}

// ---- LM head + argmax without any allocation -----------------------------------
// The per-CTA argmax partials, the arrival ticket and the result live in this
// fixed array instead of a decoder's cudaMalloc'ed slab.  Every device that loads
// the library holds it (about 66 KB) until the process exits.
constexpr int kNoAllocMaxCtas = 1024;
constexpr int kNoAllocMaxVocab = 262144;
constexpr size_t kNoAllocPartsBytes = sizeof(ArgmaxPart) * kMaxRows * kNoAllocMaxCtas;
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocPartsBytes + 256];

int dfb_lmhead_argmax_noalloc(const void* embed, const void* final_norm, const void* hidden_in, const void* residual,
                              int32_t rows, int32_t hidden, int32_t vocab, float eps, int32_t* out_tokens,
                              float* out_logits, dfb_stream_t stream_) {
  if (!embed || !final_norm || !hidden_in || !residual || !out_tokens) return DFB_E_BAD_ARG;
  if (rows < 1 || rows > kMaxRows) return DFB_E_BAD_ARG;
  if (hidden != 1024 || vocab < 16 || vocab % 16) return DFB_E_GEOMETRY;
  if (vocab > kNoAllocMaxVocab) return DFB_E_TOO_LARGE;
  // One-time set-up per device, with that device current: in host code the array's
  // name is only a stand-in, the kernel needs the address the runtime reports.
  static unsigned char* scratch_of_device[64] = {};
  int dev = 0;
  DFB_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return DFB_E_TOO_LARGE;
  if (!scratch_of_device[dev]) {
    void* p = nullptr;
    DFB_CUDA(cudaGetSymbolAddress(&p, g_noalloc_scratch));
    if (!p) return (int)cudaErrorInvalidSymbol;
    scratch_of_device[dev] = (unsigned char*)p;
  }
  unsigned char* scratch = scratch_of_device[dev];
  cudaStream_t stream = (cudaStream_t)stream_;
  unsigned int* ticket = (unsigned int*)(scratch + kNoAllocPartsBytes);
  int* tokens = (int*)(scratch + kNoAllocPartsBytes + 64);
  // the array keeps the previous call's contents: the ticket must start at zero
  DFB_CUDA(cudaMemsetAsync(ticket, 0, sizeof(unsigned int), stream));
  GemvArgs a = {};
  a.w = (const bf16*)embed; a.rows = rows; a.k = hidden;
  a.x = (const bf16*)hidden_in; a.res_in = (const bf16*)residual; a.norm_w = (const bf16*)final_norm; a.eps = eps;
  a.logits_out = out_logits; a.vocab = vocab;
  a.parts = (ArgmaxPart*)scratch; a.ticket = ticket; a.tokens = tokens; a.tokens_out = out_tokens;
  Launcher L{stream, false};
  if (rows <= 2) {
    a.n_tiles = vocab / 16;
    int grid = 3 * sm_count_cached();
    if (grid > a.n_tiles) grid = a.n_tiles;
    if (grid > kNoAllocMaxCtas) grid = kNoAllocMaxCtas;
    launch_row<1024, kModeNormArgmax>(L, a, rows, grid, false);
  } else {
    a.n_tiles = vocab / kTileRows;
    int grid = sm_count_cached();
    if (grid > a.n_tiles) grid = a.n_tiles;
    if (grid > kNoAllocMaxCtas) grid = kNoAllocMaxCtas;
    launch_gemv<4, 8, 6, kModeNormArgmax>(L, a, grid, false);
  }
  return L.err;
}

}  // extern "C"
