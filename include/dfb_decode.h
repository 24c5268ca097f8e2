/*
 * dfb_decode.h -- C ABI of the B200 (sm_100a) Qwen3 greedy decode step.
 *
 * This is the native boundary behind nano-vLLM's decode_backend="megakernel"
 * switch.  It replaces the reference project's native entry points
 *
 *   extern "C" cudaError_t tg_launch_decode(const tg::TgLaunchDesc*, cudaStream_t)
 *       src/nanovllm/backends/megakernel/csrc/torch_bindings.cpp:27-31
 *       src/nanovllm/backends/megakernel/csrc/taskgraph_kernel.cu:1927-1987
 *   extern "C" void tg_launch_zero_regions(const TgZeroRegion*, int, int, cudaStream_t)
 *       src/nanovllm/backends/megakernel/csrc/taskgraph_kernel.cu:2015-2023
 *
 * and the POD launch descriptor src/nanovllm/backends/megakernel/csrc/tg_abi.h:97-174.
 * Like that header it compiles without CUDA headers: device addresses are plain
 * pointers, the stream is an opaque pointer, there are no torch types, no
 * exceptions, and every call returns an int status (0 = success, a positive
 * value = the cudaError_t that failed, a negative value = a DFB_E_* code).
 *
 * The library has no CPU fallback: every entry point either runs the CUDA path
 * or returns an error.
 */
#ifndef DFB_DECODE_H_
#define DFB_DECODE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DFB_ABI_VERSION 2
#define DFB_MAX_ROWS 8          /* TG_MAX_BATCH, backends/megakernel/taskgraph.py:33 */
#define DFB_ATTN_CHUNK 64       /* context positions handled by one attention CTA */

/* negative status codes */
#define DFB_E_BAD_ARG (-1)      /* null pointer, rows out of range, bad stride ... */
#define DFB_E_GEOMETRY (-2)     /* model shape the kernels are not built for */
#define DFB_E_ABI (-3)          /* abi_version mismatch */
#define DFB_E_DEVICE_STATUS (-4)/* a kernel reported an error in the status word */
#define DFB_E_TOO_LARGE (-5)    /* request exceeds a fixed capacity */
#define DFB_E_COMM (-6)         /* a tensor-parallel collective returned an error */

typedef void* dfb_stream_t;     /* a cudaStream_t */
typedef struct DfbHandle DfbHandle;

/* Per-layer weight pointers (device, bf16, [out, in] row-major).  Replaces the
 * 11-pointer-per-layer blob of backends/megakernel/weights.py:172-183, keeping
 * nano-vLLM's fused qkv_proj / gate_up_proj tensors instead of splitting them. */
typedef struct DfbLayerWeights {
  const void* ln_in;    /* [hidden]                          input_layernorm.weight */
  const void* wqkv;     /* [q_size + 2*kv_size, hidden]      self_attn.qkv_proj.weight (q|k|v rows) */
  const void* q_norm;   /* [head_dim] */
  const void* k_norm;   /* [head_dim] */
  const void* wo;       /* [hidden, q_size]                  self_attn.o_proj.weight */
  const void* ln_post;  /* [hidden]                          post_attention_layernorm.weight */
  const void* wgu;      /* [2*intermediate, hidden]          mlp.gate_up_proj.weight (gate|up rows) */
  const void* wd;       /* [hidden, intermediate]            mlp.down_proj.weight */
} DfbLayerWeights;

/* Model + paged KV cache description (cf. tg_abi.h:97-174 geometry fields and
 * backends/megakernel/cache.py:16-119 for the cache layout). */
typedef struct DfbModelDesc {
  int32_t abi_version;      /* DFB_ABI_VERSION */
  int32_t hidden;           /* 1024 */
  int32_t layers;           /* 28 (any value >= 1 is accepted) */
  int32_t q_heads;          /* 16 */
  int32_t kv_heads;         /* 8 */
  int32_t head_dim;         /* 128 */
  int32_t intermediate;     /* 3072 */
  int32_t vocab;            /* 151936 (any multiple of 8) */
  int32_t max_model_len;    /* rows of rope_cos_sin; <= 2048 */
  int32_t block_size;       /* tokens per KV block; multiple of DFB_ATTN_CHUNK */
  int32_t num_blocks;       /* physical blocks in the cache */
  float eps;                /* RMSNorm epsilon */
  const void* embed;        /* bf16 [vocab, hidden]; also the tied LM head */
  const void* final_norm;   /* bf16 [hidden] */
  const float* rope_cos_sin;/* fp32 [max_model_len, head_dim]: cos | sin halves */
  const DfbLayerWeights* layer_weights; /* HOST array of `layers` entries (copied) */
  void* k_cache;            /* bf16 [layers, num_blocks, block_size, kv_heads, head_dim] */
  void* v_cache;            /* same shape; engine-owned, shared with prefill */
} DfbModelDesc;

/* One decode step; all pointers are DEVICE pointers.  Mirrors the per-step
 * inputs of TaskGraphDecoder.decode_rows (backends/megakernel/taskgraph.py:354-445). */
typedef struct DfbStepDesc {
  int32_t rows;               /* 1..DFB_MAX_ROWS */
  int32_t block_table_cols;   /* valid columns of block_tables */
  int32_t block_table_stride; /* elements between rows of block_tables */
  int32_t max_context;        /* upper bound of positions[r]+1 if the host knows it, else 0
                                 (then block_table_cols*block_size is used) */
  const int64_t* input_ids;   /* [rows]; NULL = feed back the previous step's tokens */
  const int64_t* positions;   /* [rows] pre-decode length of each row (= RoPE position) */
  const int32_t* block_tables;/* [rows, stride] physical block ids, right-padded with 0 */
  const int32_t* row_active;  /* [rows] or NULL (= all active); 0 skips the KV write only */
  int32_t* out_tokens;        /* NULL, or int32[DFB_MAX_ROWS + 4]: greedy token ids in [0, rows) and the
                                 decoder's status word (see DfbStatus) in [DFB_MAX_ROWS, DFB_MAX_ROWS + 4),
                                 so one device-to-host read returns both */
  float* out_logits;          /* [rows, vocab] or NULL; bf16-rounded logits as fp32 (parity checks) */
  const float* temperatures;  /* NULL = greedy step, or [rows] sampling temperatures (device): rows with a
                                 temperature above 1e-10 draw from softmax(logits / T), the others stay greedy
                                 (layers/sampler.py:7-16; see dfb_set_seed) */
} DfbStepDesc;

/* Tensor-parallel shard of the step.  The reference's megakernel backend runs
 * on one GPU only (it answers tensor_parallel_size != 1 with an explicit
 * fallback reason, backends/megakernel/taskgraph.py:119-122); the partitioning
 * here is the one of the reference's torch path: KV heads and their query
 * heads, o_proj columns, gate/up rows, down_proj columns and LM-head rows are
 * split evenly over the ranks (layers/linear.py:54-153, layers/embed_head.py,
 * engine/model_runner.py:188), with a sum over the ranks after o_proj and
 * after down_proj.
 *
 * A sharded decoder is created with the LOCAL sizes in DfbModelDesc (q_heads,
 * kv_heads, intermediate, vocab = rows of this rank's LM-head shard; KV cache
 * with the local kv_heads) and the rank's slices of the weights; `embed`
 * still points to the whole embedding table (replicated), of which rows
 * [vocab_offset, vocab_offset + vocab) are this rank's LM head.  The two
 * collectives are called through function pointers with the signatures of
 * ncclAllReduce / ncclAllGather, so that the library links against no
 * communication library; `comm` is the caller's communicator. */
typedef int (*dfb_all_reduce_fn)(const void* send, void* recv, size_t count, int dtype, int op, void* comm,
                                 dfb_stream_t stream);
typedef int (*dfb_all_gather_fn)(const void* send, void* recv, size_t send_count, int dtype, void* comm,
                                 dfb_stream_t stream);
typedef struct DfbTensorParallel {
  int32_t size;               /* ranks: 2, 4 or 8 */
  int32_t rank;
  int32_t vocab_offset;       /* first embedding row of this rank's LM-head shard */
  int32_t dtype_bf16;         /* the communication library's code for bf16 (ncclBfloat16 = 9) */
  int32_t dtype_int8;         /* ... for bytes (ncclInt8 = 0) */
  int32_t op_sum;             /* ... for a sum (ncclSum = 0) */
  dfb_all_reduce_fn all_reduce;
  dfb_all_gather_fn all_gather;
  void* comm;
} DfbTensorParallel;

/* Device status codes (DfbStatus.device_status); detail = {kernel id, index, observed value}.  A kernel that
 * meets one of these records the first of a step, substitutes a safe value (no address is formed from the bad
 * input, the row's KV slot is left unwritten) and finishes; the step's result for that row is then invalid. */
#define DFB_STATUS_BAD_POSITION 1  /* positions[index] outside [0, max_model_len) */
#define DFB_STATUS_BAD_BLOCK 2     /* block id of row `index` outside [0, num_blocks), or (value < 0) a position
                                      beyond the block-table columns given: value = -1 - column */
#define DFB_STATUS_COPY_TIMEOUT 3  /* a bulk copy into shared memory did not complete within its bounded wait */
#define DFB_STATUS_PEER_TIMEOUT 4  /* tensor parallel: peer `index` did not deliver tag `value` in time */
#define DFB_STATUS_BAD_TOKEN 5     /* token id of row `index` outside the embedding table (row 0 used instead) */
#define DFB_STATUS_BAD_SLOT 7      /* dfb_store_kvcache: slot_mapping[index] outside [-1, num_slots): the row was skipped */
#define DFB_STATUS_BAD_GRID 6      /* max_context smaller than positions[index] + 1: the attention grid is too small */

typedef struct DfbStatus {
  int32_t device_status;      /* 0 = ok; otherwise the first DFB_STATUS_* code a kernel recorded */
  int32_t detail[3];          /* kernel id, index, observed value */
  int64_t steps;              /* decode steps enqueued so far */
  int64_t kernels_per_step;   /* kernels of this library launched by one step */
} DfbStatus;

/* options for dfb_set_option */
#define DFB_OPT_USE_GRAPH 1   /* 1 (default): replay a captured CUDA graph per (rows, split bucket) */
#define DFB_OPT_USE_PDL 2     /* 1 (default): chain kernels with programmatic dependent launch */
#define DFB_OPT_LMHEAD_CTAS 3 /* grid of the LM-head kernel (default 2 x SM count) */
#define DFB_OPT_STEP_MODE 5   /* 0 (default): the step is a chain of per-op kernels; 1: one persistent kernel */
#define DFB_OPT_PERSIST_CTAS 6/* grid of the persistent kernel, 1..SM count (0 = SM count, the default) */
/* Options 7-17 belong to the decoder they are set on (no process-wide state). */
#define DFB_OPT_ROW_GEMV 7    /* largest batch (0..8) that runs the projections on the FP32 GEMV kernels in the
                                 kernel chain; larger batches use the tensor-core kernels (default 1; 2 on a
                                 tensor-parallel shard) */
#define DFB_OPT_ATTN_WIDE 8   /* attention grids of at most this many CTAs run 256-thread CTAs
                                 instead of 128-thread ones (default 296 = two per SM) */
#define DFB_OPT_SMEM_CARVEOUT 9      /* share (percent, -1 = driver's choice) of an SM's L1/shared memory that the
                                        kernels of the FP32 chain ask for as shared memory (default 12) */
#define DFB_OPT_SMEM_CARVEOUT_MMA 10 /* the same for the tensor-core chains (default 50; 100 when a per-layer
                                        projection runs on tcgen05) */
#define DFB_OPT_LATE_TRIGGER 11 /* FP32 chain: 0 (default) = a kernel lets its successor start (and request its
                                  weights) at once, 1 = only after it has read its own inputs */
#define DFB_OPT_PAIR_GEMV 12    /* mma.sync chain, K = 1024: 1 (default) = 16 weight rows per MMA (pair_gemv_kernel),
                                  0 = 8 weight rows per MMA (stream_gemv_kernel) */
#define DFB_OPT_BULK_X 13       /* FP32 chain: 1 (default) = the fused norm fetches x and the residual with bulk
                                  copies (TMA), 0 = with ordinary loads */
#define DFB_OPT_TP_FUSED 14     /* tensor parallel over peer windows: 1 (default) = the projections push and the next
                                  fused norm pulls the partial results, 0 = a separate exchange kernel */
#define DFB_OPT_LOOK_AHEAD 15   /* L2 look-ahead, a bit mask (default 0 = none; measured neutral): kernels with many CTAs also request
                                  weights of a kernel at least two places further down the chain into L2 (bulk
                                  prefetch): 1 = gate/up asks for the next layer's Wqkv, 2 = down_proj for the next
                                  layer's Wo, 4 = QKV for this layer's Wgu, 8 = o_proj for this layer's Wd, 16 = the
                                  last layer asks for the head of the LM head, 32 = ask after the kernel's own work
                                  instead of before its dependency wait */
#define DFB_OPT_LMHEAD_AHEAD_MB 16 /* MB of the LM head that the last layer's kernels request into L2 (default 32) */
#define DFB_OPT_PEER_WAIT_US 17 /* tensor parallel over peer windows: how long (microseconds) a kernel waits for a
                                  peer's data before it records status 4 and goes on (default 2,000,000) */
#define DFB_OPT_TCGEN05 18      /* batches above DFB_OPT_ROW_GEMV: which K = 1024 projections run on tcgen05.mma with
                                  TMA-fed shared-memory stages and accumulators in tensor memory instead of the
                                  mma.sync kernels; a bit mask: 1 = QKV, 2 = gate/up, 4 = LM head (default 4) */
#define DFB_OPT_ATTN_RING 19    /* steps whose rows x ceil(context bound / 64) reach this value run the streaming attention
                                  kernel (one CTA per row and 64-position chunk for all KV heads, K/V through a
                                  shared-memory ring fed by bulk copies) instead of the register-resident one;
                                  0 = never (default 200) */
#define DFB_OPT_ATTN_CLUSTER 20 /* register-resident attention kernel: grids of at most this many CTAs with 2..16
                                  chunks per row launch the chunks of one (row, KV head) as a thread-block cluster
                                  that merges its partial results through distributed shared memory (no global
                                  partials, no ticket); 0 = never (default 148: one row up to context 1024) */
#define DFB_OPT_ATTN_CHUNK128 21 /* register-resident attention kernel: 1 (default) = a step whose context bound is
                                  65..128 tokens runs one 128-position chunk per row and KV head instead of two
                                  merged 64-position chunks; N > 1 = also every grid that 128-position chunks
                                  bring to at most N CTAs; 0 = never.  Rows of launches with different bounds may
                                  then differ in the last bit of the attention output (another summation order) */
#define DFB_OPT_ATTN_RING32 22  /* steps with a context bound of at most 1024 tokens whose rows x ceil(bound / 32) reach
                                  this value, and that DFB_OPT_ATTN_RING does not take, run the streaming attention
                                  kernel with 32 positions per CTA; 0 = never (the default: measured slower) */
#define DFB_OPT_REG_WEIGHTS 23  /* batches above DFB_OPT_ROW_GEMV, a bit mask: 1 = QKV and gate/up, 2 = o_proj and
                                  down_proj, 4 = LM head run the mma.sync kernels that keep their weights in
                                  registers (loaded from global memory in MMA fragment order before the dependency
                                  wait) instead of shared-memory stages: their CTAs need 3-33 KB of shared memory
                                  and are resident beside their predecessor's; 8 = up to two CTAs per SM
                                  (default 0: measured slower than the staged kernels at every batch) */
#define DFB_OPT_HOST_IO 24      /* steps from host buffers, a bit mask: 1 = the packed inputs are read from pinned host
                                  memory by a one-warp kernel, 2 = tokens and status are written to pinned host
                                  memory by a one-warp kernel, instead of copy nodes in the step's graph; 4 = with 2:
                                  the call returns when the sequence word that the kernel writes after the tokens
                                  has arrived (polled in pinned memory) instead of synchronising the stream
                                  (default 6) */
#define DFB_OPT_TRACE 4       /* 1: every kernel records its timeline (see dfb_read_trace); default 0 */

/* Build a decoder for one model on the current device: validates the geometry,
 * copies the pointer tables, allocates the activation scratch (a few MB).
 * Replaces TaskGraphDecoder.__init__ (taskgraph.py:150-305). */
int dfb_create(const DfbModelDesc* desc, DfbHandle** out);
/* Make `h` one rank of a tensor-parallel group (see DfbTensorParallel); call once,
 * before the first step.  Every rank must then enqueue the same steps in the same order. */
int dfb_set_tensor_parallel(DfbHandle* h, const DfbTensorParallel* tp);
/* Exchanges over peer-mapped memory instead of the two collectives (NVLink, all ranks on one node, one
 * process per GPU).  Each rank calls dfb_tp_window_handle, which allocates its exchange window (about 260 KB)
 * and writes a DFB_TP_HANDLE_BYTES-byte inter-process handle (a cudaIpcMemHandle_t); the caller gathers the
 * handles of all ranks, in rank order, and passes them to dfb_tp_open_peers on every rank, after which the
 * sums after o_proj / down_proj and the merge of the greedy winners are done by the library's own kernels
 * (a push into every peer's window, a flag, a bounded wait; all_reduce / all_gather may then be NULL).  A
 * peer that does not arrive within the wait limit (DFB_OPT_PEER_WAIT_US, 2 s by default) makes the waiting
 * kernel record status 4 and finish; the step's result is then invalid and dfb_read_status reports it. */
#define DFB_TP_HANDLE_BYTES 64
int dfb_tp_window_handle(DfbHandle* h, void* handle_out);
int dfb_tp_open_peers(DfbHandle* h, const void* handles);
/* Diagnostic stand-in for dfb_tp_open_peers on ONE GPU in one process: the "peers'" windows are plain local
 * allocations that nobody fills, so every wait for a peer runs into its limit (DFB_OPT_PEER_WAIT_US).  It
 * exists to exercise the timeout path (status 4, the step still completes, the context stays usable) without
 * a second rank and without leaving anything waiting; the tokens of such a step mean nothing. */
int dfb_tp_open_loopback(DfbHandle* h);
void dfb_destroy(DfbHandle* h);
int dfb_set_option(DfbHandle* h, int option, int value);

/* Capture ahead of time the graphs of every step geometry up to `max_rows` rows and `max_context` tokens, so
 * that no step of a serving run pays a capture (a few milliseconds) when the batch size changes or a row's
 * context crosses a chunk or block boundary: the counterpart of ModelRunner.capture_cudagraph
 * (engine/model_runner.py:379-416), which captures the torch path's graphs for its batch sizes at start-up.
 * `kinds` is a bit mask of the entry points to prepare: 1 = bursts, 2 = dfb_decode_step without out_tokens,
 * 4 = dfb_decode_step with out_tokens, 8 = the host-buffer steps, 16 = also the sampling variants of those.
 * `graphs_out` (may be NULL) receives the number of graphs the decoder holds afterwards.  Options set later
 * drop the graphs again. */
int dfb_warm(DfbHandle* h, int32_t max_rows, int32_t max_context, int32_t kinds, int32_t* graphs_out);

/* Enqueue one decode step on `stream` (no host synchronisation, no allocation
 * after the first call for a given (rows, bucket)).  Replaces tg_launch_decode +
 * tg_launch_zero_regions + the three staging copies of taskgraph.py:395-413. */
int dfb_decode_step(DfbHandle* h, const DfbStepDesc* step, dfb_stream_t stream);

/* Same step with HOST buffers: copies ids / positions / block tables to the
 * device, runs the step, copies the token ids back and synchronises `stream`.
 * This is the call behind MegakernelBackend.decode (backend.py:240-258): one
 * H2D, one D2H, one sync per step.  block_tables is [rows, cols] row-major.
 * Returns DFB_E_DEVICE_STATUS if a kernel recorded an error during the step. */
int dfb_decode_step_host(DfbHandle* h, int32_t rows, const int64_t* input_ids, const int64_t* positions,
                         const int32_t* block_tables, int32_t cols, const int32_t* row_active,
                         int32_t* out_tokens, dfb_stream_t stream);

/* dfb_decode_step_host with one sampling temperature per row (host array, NULL = greedy for every row; a
 * negative or NaN temperature is DFB_E_BAD_ARG, as sampling_params.py:14-15 rejects it).  The temperatures
 * travel in the same host-to-device copy as the other inputs.  Replaces prepare_sample + Sampler.forward
 * (engine/model_runner.py:286-289,374, layers/sampler.py:7-16) for the rows the backend would otherwise hand
 * back with "greedy sampling only" (backends/megakernel/taskgraph.py:123-130). */
int dfb_decode_step_host_sampled(DfbHandle* h, int32_t rows, const int64_t* input_ids, const int64_t* positions,
                                 const int32_t* block_tables, int32_t cols, const int32_t* row_active,
                                 const float* temperatures, int32_t* out_tokens, dfb_stream_t stream);

/* A burst: `steps` consecutive decode steps of the same rows enqueued at once, the whole loop resident on the
 * device.  One host-to-device copy stages the inputs; after every step a one-warp kernel writes the step's
 * tokens into a ring in pinned host memory (no copy node; the host may read finished steps while later ones
 * run) and turns them into the next step's inputs on the device (ids = tokens, positions + 1).  Step s of row
 * r runs at position positions[r] + s, so the block tables must already hold the blocks of positions[r] +
 * steps - 1 (DFB_E_BAD_ARG otherwise); steps <= DFB_MAX_BURST.  Rows run on past an end-of-sequence token:
 * the caller cuts the stream.  This is the step loop of LLMEngine.generate / ModelRunner.run
 * (engine/llm_engine.py, engine/model_runner.py:264-284,315-376) without its per-step pinned tensor builds,
 * small host-to-device copies and .tolist() synchronisation.
 *   dfb_decode_burst_enqueue  returns once everything is enqueued on `stream` (no synchronisation);
 *   dfb_decode_burst_collect  copies the tokens of the finished steps into out_tokens[steps_done][rows];
 *                             wait = 1 blocks until the burst is complete, wait = 0 returns at once
 *                             (steps_done < steps: call again).  The call that sees the last step ends the
 *                             burst and returns DFB_E_DEVICE_STATUS if a kernel recorded an error;
 *   dfb_decode_burst_host     = enqueue + collect(wait = 1).
 * While a burst is in flight the decoder accepts no other step from host buffers. */
#define DFB_MAX_BURST 1024
int dfb_decode_burst_enqueue(DfbHandle* h, int32_t rows, int32_t steps, const int64_t* input_ids,
                             const int64_t* positions, const int32_t* block_tables, int32_t cols,
                             const int32_t* row_active, const float* temperatures, dfb_stream_t stream);
int dfb_decode_burst_collect(DfbHandle* h, int32_t wait, int32_t* out_tokens, int32_t* steps_done);
int dfb_decode_burst_host(DfbHandle* h, int32_t rows, int32_t steps, const int64_t* input_ids,
                          const int64_t* positions, const int32_t* block_tables, int32_t cols,
                          const int32_t* row_active, const float* temperatures, int32_t* out_tokens,
                          dfb_stream_t stream);

/* Fixed-slot runtime: the decode side of a continuous-batching engine as the reference designed it (fixed rows
 * whose sequences come and go, `set_slot(row, active, start_pos, ...)`, a token callback after every step:
 * backends/megakernel/row_contract.py:1-24, csrc/tg_abi.h:185-199) and never built.  DFB_MAX_SLOTS slots live in
 * the decoder; a step packs the live ones, in slot order, into launches of at most DFB_MAX_ROWS rows — more live
 * slots than that become several launches per step — runs them from host state (one packed copy each), and then
 * holds each slot's new token and position.  A slot whose next position lies beyond its block table (the
 * scheduler has to append a block and call dfb_slot_set again) or beyond the model length sits the step out.
 * A retired slot (active = 0) is simply no longer launched, so its freed blocks are never written again; every
 * geometry is a cached graph (dfb_warm), so a change of the live set captures nothing.
 *   dfb_slot_set   admit (active = 1: next input token, pre-decode length, block table, temperature; 0 = greedy)
 *                  or retire (active = 0) a slot; also the way to give a live slot a longer block table;
 *   dfb_slot_get   the slot's state as the runtime holds it;
 *   dfb_slots_step one step of all live slots: sampled_tokens[DFB_MAX_SLOTS], emitted[DFB_MAX_SLOTS] (1 = this
 *                  slot produced sampled_tokens[slot]); synchronises `stream`;
 *   dfb_slots_run  steps until max_steps, until no slot emits, or until the callback returns non-zero; the
 *                  callback (the reference's TgTokenCallback signature) runs on the calling thread after each
 *                  step and may call dfb_slot_set.  Scheduling, preemption and prefill stay with the engine. */
#define DFB_MAX_SLOTS 32
typedef int (*dfb_token_callback)(void* context, const long long* sampled_tokens, const int32_t* emitted_rows,
                                  int32_t batch_size);
int dfb_slot_set(DfbHandle* h, int32_t slot, int32_t active, int64_t token, int64_t position,
                 const int32_t* block_table, int32_t cols, float temperature);
int dfb_slot_get(DfbHandle* h, int32_t slot, int32_t* active, int64_t* token, int64_t* position);
int dfb_slots_step(DfbHandle* h, long long* sampled_tokens, int32_t* emitted, dfb_stream_t stream);
int dfb_slots_run(DfbHandle* h, int32_t max_steps, dfb_token_callback callback, void* context, dfb_stream_t stream);

/* Seed of the sampling noise (default 0) and restart of its stream.  A sampled row takes
 * argmax_i(logit_i / T - log E_i), E_i ~ Exp(1) clamped at 1e-10, which is the reference's
 * argmax(softmax(logits / T) / E) without the softmax pass.  E_i = -log(u_i), u_i = (top 23 bits of
 * splitmix64_finalise(seed + c * 0x9E3779B97F4A7C15) + 0.5) / 2^23 with the 64-bit counter
 * c = ((n * 8 + row) << 32) | i, n = the number of sampled LM-head launches of this decoder since the seed was
 * set (greedy steps do not advance it), i = the token's index in the whole vocabulary: the draw is a
 * function of (seed, n, row, i) alone, identical on every tensor-parallel rank and reproducible on the host.
 * torch's own generator stream is not reproduced: parity with the reference's sampler is in distribution.
 * Call it between steps (it synchronises nothing): a step in flight may see either stream position. */
int dfb_set_seed(DfbHandle* h, uint64_t seed);

/* Read (and clear) the device status word; synchronises nothing by itself, so
 * call it after the stream has been synchronised. */
int dfb_read_status(DfbHandle* h, DfbStatus* out);
const char* dfb_error_string(int code);

/* Timeline of the last traced step (DFB_OPT_TRACE): for each of its kernels, in
 * launch order, eight uint64 words of globaltimer ns: {earliest CTA start,
 * latest return from the dependency wait, latest CTA end, earliest return from
 * the wait, latest end of the prologue, latest end of the first tile's math,
 * latest end of the first tile, 0} (`out` holds 8 * max_kernels words).  Returns the number of kernels written (<= max_kernels) or a negative
 * code, and re-arms the buffer; call it once before the traced step to arm it.
 * This is the per-task-time-versus-CTA-count diagnostic the reference ran as an
 * SM-count sweep (TG_NUM_SMS, backends/megakernel/taskgraph.py:68-83). */
int dfb_read_trace(DfbHandle* h, uint64_t* out, int32_t max_kernels);

/* ---- standalone, non-cooperative launches of each kernel -------------------
 * One plain launch per call, so each kernel can be profiled or checked alone.
 * All pointers are device pointers; `rows` <= DFB_MAX_ROWS.  They compute what
 * the same-named step of the reference torch path computes (file:line in
 * src/nanovllm/). */

/* models/qwen3.py:153-156 + :79.  x = h (+ residual); residual_out = bf16(x);
 * qkv = RMSNorm(x; ln_w) @ wqkv^T.  If `ids` is non-NULL, h is gathered from the
 * rows ids[r] of `h` (an embedding table) and `residual` must be NULL. */
int dfb_launch_rmsnorm_qkv(const void* h, const int32_t* ids, const void* residual, void* residual_out,
                           const void* ln_w, const void* wqkv, void* qkv_out, int32_t rows, int32_t hidden,
                           int32_t qkv_rows, float eps, dfb_stream_t stream);
/* models/qwen3.py:84-88 + layers/attention.py:33-40,72-74: q/k RMSNorm, RoPE,
 * KV write at positions[r], paged GQA decode attention over [0, positions[r]]. */
int dfb_launch_attention(DfbHandle* h, int32_t layer, const void* qkv, const int32_t* positions,
                         const int32_t* block_tables, int32_t block_table_stride, const int32_t* row_active,
                         void* attn_out, int32_t rows, int32_t max_context, dfb_stream_t stream);
/* layers/linear.py:152-153: out[rows, n] = x[rows, k] @ w[n, k]^T (o_proj, down_proj). */
int dfb_launch_linear(const void* x, const void* w, void* out, int32_t rows, int32_t n, int32_t k,
                      dfb_stream_t stream);
/* models/qwen3.py:158 + :115-117: add+RMSNorm, gate/up projection, SiLU(gate)*up. */
int dfb_launch_rmsnorm_gateup_swiglu(const void* h, const void* residual, void* residual_out, const void* ln_w,
                                     const void* wgu, void* act_out, int32_t rows, int32_t hidden,
                                     int32_t intermediate, float eps, dfb_stream_t stream);
/* models/qwen3.py:186,216-220 + layers/sampler.py:9,15: final add+RMSNorm, tied
 * LM head, bf16-rounded logits, greedy argmax (lowest index wins ties). */
int dfb_launch_lmhead_argmax(DfbHandle* h, const void* hidden_in, const void* residual, int32_t* out_tokens,
                             float* out_logits, int32_t rows, dfb_stream_t stream);
/* The same with sampling: `temperatures` is a DEVICE array [rows] (NULL = greedy); layers/sampler.py:7-16. */
int dfb_launch_lmhead_sample(DfbHandle* h, const void* hidden_in, const void* residual, const float* temperatures,
                             int32_t* out_tokens, float* out_logits, int32_t rows, dfb_stream_t stream);

/* The prefill side of the shared paged cache (layers/attention.py:10-40, `store_kvcache` and its Triton kernel):
 * the K / V rows of `n_tokens` prompt tokens, bf16 [n_tokens, row_elems] with row strides key_stride /
 * value_stride (elements), go to rows slot_mapping[i] of k_cache / v_cache viewed as [num_slots, row_elems]
 * (num_slots = num_blocks * block_size of one layer; row_elems = kv_heads * head_dim).  slot -1 is skipped as in
 * the reference; any other slot outside [0, num_slots) is skipped too and recorded in `status` (NULL, or a device
 * int32[4] that receives {DFB_STATUS_BAD_SLOT, kernel id, token index, slot}).  All pointers are device pointers;
 * nothing is allocated and nothing synchronised.  Prefill ATTENTION itself stays on the engine's torch path. */
int dfb_store_kvcache(const void* key, const void* value, int64_t key_stride, int64_t value_stride, void* k_cache,
                      void* v_cache, const int32_t* slot_mapping, int32_t n_tokens, int32_t row_elems,
                      int64_t num_slots, int32_t* status, dfb_stream_t stream);

/* Causal prefill attention over the prompt tokens of `batch` sequences laid back to back: the reference's
 * flash_attn_varlen_func(..., causal=True[, block_table=...]) call of layers/attention.py:64-70, both cases.
 * q [N, q_heads, head_dim] and out [N, q_heads, head_dim] hold the query tokens, sequence b = rows
 * [cu_seqlens_q[b], cu_seqlens_q[b + 1]) (device int32 [batch + 1]); max_seqlen_q bounds the grid (a longer
 * sequence would lose its tail rows).
 *   without a prefix cache (block_tables = NULL): k / v [N, kv_heads, head_dim] are the projections of the same
 *     tokens and cu_seqlens_k may be NULL (= cu_seqlens_q);
 *   with one: k / v are ONE LAYER of the paged cache, [num_blocks * block_size, kv_heads, head_dim] rows with
 *     k_stride / v_stride elements between slots, sequence b's keys 0 .. cu_seqlens_k[b + 1] - cu_seqlens_k[b] - 1
 *     are found through block_tables[b, position / block_size] (device int32 [batch, block_table_stride]), and
 *     query i attends to keys 0 .. i + (keys - queries) (the mask aligned to the last key, as FlashAttention).
 * All tensors bf16, row strides in elements; head_dim 128, grouped-query attention with q_heads a multiple of
 * kv_heads.  fp32 accumulation and softmax, probabilities rounded to bf16 before they multiply V (as
 * FlashAttention does).  A block id outside [0, num_blocks) is never followed: the key row is read as zeros and
 * `status` (NULL, or a device int32[4]) receives {DFB_STATUS_BAD_BLOCK, kernel id, sequence, block id}.
 * Allocates nothing, synchronises nothing. */
int dfb_prefill_attention(const void* q, const void* k, const void* v, void* out, const int32_t* cu_seqlens_q,
                          const int32_t* cu_seqlens_k, int32_t batch, int32_t max_seqlen_q, int64_t q_stride,
                          int64_t k_stride, int64_t v_stride, int64_t out_stride, int32_t q_heads, int32_t kv_heads,
                          int32_t head_dim, float scale, const int32_t* block_tables, int32_t block_table_stride,
                          int32_t block_size, int32_t num_blocks, int32_t* status, dfb_stream_t stream);

/* Final add+RMSNorm, tied LM head and greedy argmax WITHOUT any allocation.
 * (No counterpart in the reference: its LM head always runs inside a decoder
 * that allocated its scratch at start-up.)
 *
 * Who needs it: a caller that may not call cudaMalloc at the point where it wants
 * the next token -- an engine that handed almost all free device memory to its
 * KV cache at start-up (nano-vLLM sizes the cache from gpu_memory_utilization),
 * so a later allocation can fail; a caller inside a region where its own policy
 * forbids allocation after warm-up; or one that has no DfbHandle at all.  The
 * scratch this kernel needs (one argmax partial per CTA and batch row, an arrival
 * ticket, the result) lives in a fixed array inside the library instead: about
 * 66 KB on every device that loads the library, held until the process exits.
 *
 * Limits: rows 1..DFB_MAX_ROWS, hidden 1024, vocab a multiple of 16 and at most
 * 262,144 (DFB_E_TOO_LARGE beyond that), at most 1024 CTAs.  `out_logits` may be
 * NULL.  The first call on a device looks up the array's device address (once per
 * device, with that device current); make that first call before any stream
 * capture.  All calls share the one array and it keeps the last call's contents
 * (the ticket is cleared on `stream` at every call), so two calls whose kernels
 * overlap on the GPU race: keep them on one stream or order them yourself.
 * Calls no cudaMalloc / cudaFree and no allocating library routine. */
int dfb_lmhead_argmax_noalloc(const void* embed, const void* final_norm, const void* hidden_in, const void* residual,
                              int32_t rows, int32_t hidden, int32_t vocab, float eps, int32_t* out_tokens,
                              float* out_logits, dfb_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* DFB_DECODE_H_ */
