/*
 * ypk.h - C ABI of the B200 persistent-kernel decode runtime.
 *
 * This is the boundary a host binding links against.  It replaces the
 * three-function CPython launcher the reference JIT-compiles per model
 * (python/yirage/persistent_kernel.py:16-94: init_func / launch_func /
 * finalize_func) and the extern "C" entry points those forward to
 * (include/yirage/persistent_kernel/persistent_kernel.cuh:1036
 * init_persistent_kernel, :1253 launch_persistent_kernel, :1320
 * finalize_persistent_kernel).  The reference entry points take a
 * std::vector by value and keep one process-global RuntimeConfig; here every
 * call takes plain pointers and sizes and works on an explicit handle.
 *
 * All functions return 0 on success or a negative ypk_error.  A message for
 * the last failure on a handle is available from ypk_last_error().
 * A handle is not thread-safe; several handles may coexist in a process.
 * The caller owns every tensor it binds and must keep it alive and unmoved
 * while the handle exists (same convention as the reference, which bakes the
 * pointers into generated code, src/kernel/runtime.cc:763).  Buffers created
 * with ypk_alloc_tensor / ypk_shuffle_tensor belong to the handle and are
 * released by ypk_destroy (the reference leaks them, runtime.cc:778-790).
 */
#ifndef YPK_H_
#define YPK_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define YPK_ABI_VERSION 1

typedef struct ypk_handle ypk_handle;

enum ypk_error {
  YPK_OK = 0,
  YPK_ERR_INVALID = -1,    /* bad argument / malformed graph            */
  YPK_ERR_CUDA = -2,       /* a CUDA runtime call failed                 */
  YPK_ERR_TIMEOUT = -3,    /* a bounded device-side wait ran out         */
  YPK_ERR_STATE = -4,      /* call made in the wrong order               */
  YPK_ERR_UNSUPPORTED = -5 /* shape or option outside what is built      */
};

/* Element types; numeric values follow the reference's task-graph JSON
 * (include/yirage/type.h:84-119). */
enum ypk_dtype {
  YPK_F16 = 940,
  YPK_BF16 = 941,
  YPK_F32 = 942,
  YPK_I32 = 955,
  YPK_I64 = 965
};

/* Task kinds executed by the worker CTAs.  These are the fused forms of the
 * reference's TaskType list (persistent_kernel/runtime_header.h:62-124). */
enum ypk_task_type {
  YPK_TASK_NOP = 0,
  YPK_TASK_EMBED = 1,         /* embedding.cuh:42-70                      */
  YPK_TASK_LINEAR = 2,        /* [rmsnorm+] x.W^T [+residual | silu*mul]  */
  YPK_TASK_ATTENTION = 3,     /* paged GQA decode, RoPE, append, split-KV */
  YPK_TASK_ARGMAX_PARTIAL = 4,
  YPK_TASK_ARGMAX_REDUCE = 5,
  YPK_TASK_RMSNORM = 6,       /* stand-alone norm (unfused graphs)        */
  YPK_TASK_SILU_MUL = 7,      /* stand-alone silu(g)*u                    */
  YPK_TASK_ALLREDUCE = 8,     /* push partial to peers + local reduce     */
  YPK_TASK_NGRAM_PARTIAL = 9, /* prompt lookup: earliest match per slice  */
  YPK_TASK_NGRAM_GLOBAL = 10, /* prompt lookup: drafts into the input ids */
  YPK_TASK_VERIFY = 11,       /* greedy verification of the drafts        */
  YPK_TASK_MOE_TOPK = 12,     /* router: softmax, top-k, active experts   */
  YPK_TASK_MOE_SILU_MUL = 13, /* silu(gate)*up per active expert slot     */
  YPK_TASK_MOE_COMBINE = 14,  /* residual + sum_j weight_j * expert out_j */
  YPK_TASK_TYPE_COUNT
};

/* ypk_task.flags */
#define YPK_F_NORM 0x1u        /* LINEAR: fold RMSNorm(x)*norm_w in front  */
#define YPK_F_RESIDUAL 0x2u    /* LINEAR: add residual[b, n]               */
#define YPK_F_SILU_MUL 0x4u    /* LINEAR: rows come as 2 gate + 2 up       */
#define YPK_F_F16 0x8u         /* operands are fp16 instead of bf16        */
#define YPK_F_ROPE 0x10u       /* ATTENTION: rotate new q/k                */
#define YPK_F_QK_NORM 0x20u    /* ATTENTION: RMSNorm of every new q head and of the new k over
                                  the head dimension, before the rotation (Qwen3)          */
#define YPK_F_QTILES 0x80u     /* ATTENTION: iarg[0] names an entry of the iteration's query-tile
                                  list instead of a request slot: a request that brings more
                                  new tokens than one task takes (8, or 32 / q-heads-per-kv-
                                  head) is spread over several tasks, each of which also
                                  stages the k / v of the request's earlier new tokens.  All
                                  ATTENTION tasks of a graph carry it or none; with it a
                                  request may take up to 64 new tokens per iteration.
                                  iarg[14] = entries of the list the graph has tasks for (the
                                  most an iteration can need: n + (max_tokens - n) / tile
                                  tokens with n = min(max_requests, max_tokens)) */
#define YPK_F_NORM_NOWEIGHT 0x40u /* LINEAR: RMSNorm without a weight      */
/* Flagged-word hand-off between tasks (no event, no fence): a [tokens][ld] tensor of 16-bit
 * values travels as [max_tokens][ld / 2] 8-byte words {two values, 32-bit tag}; the tag
 * names the iteration and the producing operator, a reader polls until it sees it. */
#define YPK_F_LL_IN 0x100u     /* LINEAR: x comes as flagged words (ptr[5]);
                                  ALLREDUCE: the ranks' partials do (buf);
                                  ATTENTION: the packed q/k/v do (ptr[0])    */
#define YPK_F_LL_RES 0x200u    /* LINEAR: residual as flagged words (ptr[6]) */
#define YPK_F_LL_OUT 0x400u    /* result also leaves as flagged words (ptr[7]);
                                  ATTENTION: only as flagged words (ptr[3])  */
#define YPK_F_LL_PUSH 0x800u   /* LINEAR: partial sum: flagged words only, into slot `rank`
                                  of ptr[7] = [world][max_tokens][ld / 2] on every rank;
                                  ARGMAX_REDUCE: exchange the slice winners (ptr[3]) */

#define YPK_F_LL_OPT 0x1000u   /* LINEAR with YPK_F_LL_IN: take x as flagged words only in
                                  iterations of one or two tokens; otherwise wait for
                                  dep_event and read the plain tensor (ptr[0])             */

#define YPK_F_MOE 0x4000u      /* LINEAR over the weights of an expert chosen at run time: ptr[5] =
                                  active-expert list int32 [E + 1] (count at [E]) as MOE_TOPK
                                  leaves it, iarg[10] = slot of that list the task serves,
                                  iarg[11] = E, iarg[12] = weight rows per expert; the task is
                                  skipped when the slot is beyond the count.  Plain 16-bit rows
                                  in and out (no flagged words, no norm, no split along K) */
#define YPK_F_NORM_OUT 0x8000u  /* LINEAR of a graph of more than 8 tokens whose result feeds an
                                  RMSNorm: besides its rows out[b, n] the task writes them
                                  multiplied by that norm's weight, xg[b, n] = out[b, n] * g[n]
                                  (ptr_aux = xg, same pitch as out; ptr[3] = g), and the sum of
                                  out[b, n]^2 over its rows into ptr[6] = fp32
                                  [row blocks][pitch] at block iarg[12] & 0xffff (pitch =
                                  iarg[12] >> 16 tokens).  Tensor-core path only.             */
#define YPK_F_NORM_PRE 0x10000u /* LINEAR that reads such an xg: the RMS factor of token b,
                                  rsqrt(sum over the iarg[12] & 0xffff blocks of ptr[3] =
                                  fp32 [blocks][pitch] / K + eps), is applied to the dot
                                  products.  Together the two flags replace a RMSNORM operator
                                  between two LINEAR operators.  Tensor-core path only.       */
#define YPK_F_TRIG_WIDE 0x2000u /* publish trig_event only in iterations of more than two tokens:
                                  its only waiters carry YPK_F_LL_OPT (they count those
                                  iterations, not all, towards the event's value)          */

#define YPK_TASK_NPTR 8
#define YPK_TASK_NINT 16
#define YPK_TASK_NFLT 4

/* A pointer operand of a task, as passed to ypk_load_graph: tensor slot + 1 in
 * the top 16 bits, byte offset in the low 48.  0 means "no tensor". */
#define YPK_REF(slot, byte_off) \
  ((((uint64_t)(slot) + 1u) << 48) | ((uint64_t)(byte_off) & 0xFFFFFFFFFFFFull))

/* One unit of work for a worker CTA.  Mirrors the role of TaskDesc
 * (persistent_kernel/runtime_header.h:136-269) with run-time shapes instead
 * of template arguments.  176 bytes, 16-byte aligned.
 *
 * LINEAR:  ptr = {x, W, out, norm_w, residual, ll_x, ll_residual, ll_out}
 *          iarg = {K, row0, nrows, ldx, ldw, ldout, ldres, out_col0}; iarg[9] is filled in
 *                  by ypk_load_graph (TMA tensor map of W, or -1); iarg[10..12] = tag ids
 *                  of the producers of x and of the residual, and this operator's own
 *          farg = {eps}
 *          Split along K (graphs of more than 8 tokens only; no flagged words there):
 *          iarg[13] = first column k0 and iarg[14] = number of columns of the task's K range
 *          (0: up to K), iarg[15] = split | nsplit << 8 | workspace tokens << 16, iarg[8] =
 *          row pitch of the workspace, iarg[10] = index of the row block's arrival counter;
 *          ptr[5] = workspace fp32 [nsplit][tokens][pitch], ptr[6] = partial sums of squares
 *          fp32 [blocks][nsplit][tokens], ptr[7] = counters uint32 [blocks][ceil(tokens / 16)].
 *          Every split of a row block leaves its partial sums there; the last to arrive adds
 *          them in split order and writes the rows.
 * EMBED:   ptr = {ids(int64), table, out}; iarg = {hidden, col0, ncols,
 *                  ldtable, ldout, rows of the table}; an id outside [0, rows) gives zeros
 * ATTENTION: ptr = {qkv, k_cache, v_cache, out, cos, sin, split scratch, qk-norm weights};
 *          with YPK_F_QK_NORM ptr[7] = [2][128] 16-bit weights (q heads, then k) and
 *          farg = {eps}
 *          iarg = {request, kv_head, split, nsplit, q_per_kv, num_kv_heads,
 *                  ld_qkv, ld_out, max_rows}; iarg[9], iarg[10] are filled in by
 *                  ypk_load_graph (TMA tensor maps of the two caches); with YPK_F_LL_IN
 *                  qkv is the flagged-word form and iarg[11] its producer's tag id, with
 *                  YPK_F_LL_OUT out is written as flagged words under tag id iarg[12]
 * ARGMAX_PARTIAL: ptr = {logits, part_val, part_idx}; iarg = {col0, ncols,
 *                  ldlogits, part, nparts, valid}; valid != 0: only columns [0, valid) of a
 *                  logits row can be sampled (the rest pads the lm_head; negative: none)
 * NGRAM_PARTIAL / NGRAM_GLOBAL / VERIFY: speculative decoding by prompt lookup (serving mode;
 *          the reference's find_ngram_partial / find_ngram_global / target_verify_greedy,
 *          tasks/speculative_decoding/prompt_lookup.cuh, target_verify.cuh).  With a VERIFY task
 *          in the graph (iarg = {draft tokens S, 1..7}) a request that is past its prompt
 *          brings its last token plus S draft slots per iteration when the token budget
 *          allows.  NGRAM_PARTIAL: ptr = {partial int32 [max_requests][nparts]}, iarg = {part,
 *          nparts, n-gram length}: lowest position in its share of every slot's history where
 *          the history's last n-gram occurs earlier.  NGRAM_GLOBAL: ptr = {partial, ids int64
 *          [max_tokens]}, iarg = {nparts, n-gram length}: ids = the iteration's input tokens
 *          with the draft slots filled by the tokens that followed the earliest match (-1:
 *          none); the embedding reads ids.  VERIFY: ptr = {ids, model outputs int64
 *          [max_tokens]}: num_new_tokens[request] = accepted drafts + 1; the batcher advances
 *          the request by that many tokens.
 * Mixture of experts (tasks/blackwell/topk_softmax_sm100.cuh, moe_linear_sm100.cuh,
 *          mul_sum_add_sm100.cuh of the reference).  Expert work is laid out by *active slot*:
 *          slot a of an iteration is the a-th expert (ascending id) that some token selected.
 *          MOE_TOPK: ptr = {router logits 16-bit [tokens][E], weights fp32 [max_tokens][k],
 *          routing int32 [E][max_tokens] (k index + 1 of the token at that expert, 0: none),
 *          active list int32 [E + 1], slot of (token, k index) int32 [max_tokens][k]};
 *          iarg = {E, k, ld of the logits}: softmax over the experts in fp32, the k largest in
 *          order (lowest id on ties), weights divided by their sum.
 *          LINEAR with YPK_F_MOE: the expert projections, one task per (slot, row slab), x and
 *          out being the slot's [max_tokens][width] block.  MOE_SILU_MUL: ptr = {in 16-bit
 *          [slots][max_tokens][2 I], out [slots][max_tokens][I], active list}; iarg = {I, E,
 *          slot0, nslots}.  MOE_COMBINE: ptr = {expert outputs [slots][max_tokens][H], weights,
 *          slot of (token, k index), residual [tokens][H], out [tokens][H]}; iarg = {H, k,
 *          col0, ncols, ld residual, ld out}: fp32 sum in k order on top of the residual, one
 *          rounding.
 * ARGMAX_REDUCE: ptr = {part_val, part_idx, out(int64)}; iarg = {nparts}, iarg[4] = row pitch
 *          of the partial buffers (0: nparts); with
 *          YPK_F_LL_PUSH (vocabulary split over the ranks) ptr[3] = exchange buffer
 *          [world][max_tokens][2] flagged words in the symmetric arena, iarg = {nparts,
 *          first vocabulary row of this rank's slice, world, rank}, iarg[12] = tag id
 * ALLREDUCE: ptr = {in, buf, out, signals} (buf, signals from the symmetric arena;
 *          buf = [2][world][max_tokens][hidden] 16-bit, signals uint64[])
 *          iarg = {col0, ncols, ld_in, ld_out, hidden, max_tokens, index of this all-reduce
 *                  among those of the iteration, signal index, world, rank, all-reduces per
 *                  iteration} (the half of buf is the parity of the running all-reduce
 *                  number); with YPK_F_LL_IN | YPK_F_LL_OUT: buf = [world][max_tokens]
 *                  [hidden / 2] flagged words pushed by the producing LINEAR tasks,
 *                  ptr[7] = flagged-word copy of out, iarg[10] / iarg[12] = tag ids of the
 *                  producer / of this operator, no signals
 * RMSNORM: ptr = {x, w, out}; iarg = {K, row0, nrows, ldx, ldout}; farg = {eps}
 * SILU_MUL: ptr = {in, out}; iarg = {col0, ncols, group, ldin, ldout}
 * The number of batch rows is the active-token count of the iteration (mode 1) or the
 * `batch` argument of ypk_launch (mode 0).
 */
typedef struct ypk_task {
  int32_t type;
  uint32_t flags;
  int32_t dep_event;   /* -1: none.  Run when counter[dep] >= dep_count*iter */
  int32_t dep_count;
  int32_t trig_event;  /* -1: none.  counter[trig] += 1 when done           */
  int32_t op_id;       /* index of the graph operator this task came from   */
  uint64_t ptr[YPK_TASK_NPTR];
  int32_t iarg[YPK_TASK_NINT];
  float farg[YPK_TASK_NFLT];
  uint64_t ptr_aux;    /* ninth pointer operand (YPK_F_NORM_OUT), else 0       */
} ypk_task;

/* Serving parameters; the meta pointers are the ten caller-owned tensors the
 * reference passes to init_func (persistent_kernel.py:1291-1316), same order. */
typedef struct ypk_config {
  int32_t abi_version;        /* YPK_ABI_VERSION                           */
  int32_t device;             /* CUDA ordinal                              */
  int32_t world_size, rank;   /* tensor-parallel group                     */
  int32_t num_workers;        /* worker CTAs; 0 = one per SM               */
  int32_t mode;               /* 0: one pass per launch (operator graphs)
                                 1: offline serving, batching on device    */
  int32_t max_seq_length;
  int32_t max_num_batched_requests;
  int32_t max_num_batched_tokens;
  int32_t max_num_pages;
  int32_t page_size;
  int32_t total_num_requests;
  int64_t eos_token_id;
  uint64_t wait_budget_ns;    /* bound of every device-side wait; 0 = 2 s  */
  void *step;                 /* int32 [total_num_requests]                */
  void *tokens;               /* int64 [total_num_requests, max_seq_length]*/
  void *input_tokens;         /* int64 [max_num_batched_tokens]            */
  void *output_tokens;        /* int64 [max_num_batched_tokens]            */
  void *num_new_tokens;       /* int32 [total_num_requests]                */
  void *prompt_lengths;       /* int32 [total_num_requests]                */
  void *qo_indptr;            /* int32 [max_num_batched_requests + 1]      */
  void *paged_kv_indptr;      /* int32 [max_num_batched_requests + 1]      */
  void *paged_kv_indices;     /* int32 [max_num_pages]                     */
  void *paged_kv_last_page_len; /* int32 [max_num_batched_requests]        */
  void *profiler_buffer;      /* optional device buffer, may be NULL: 8 uint64 per
                                 (worker, queue position), rewritten every iteration:
                                 {iteration<<32 | task, t_fetch, t_dependency_met,
                                 t_done, t_inputs_staged, t_last_stage, 0, 0} in
                                 globaltimer ns; needs workers * longest queue * 64
                                 bytes                                */
  uint64_t profiler_bytes;
} ypk_config;

typedef struct ypk_status {
  int32_t error;          /* 0 or a ypk_error raised on the device          */
  int32_t fail_worker;    /* CTA that gave up                               */
  int32_t fail_task;      /* task index it was on (-1 if none)              */
  int32_t fail_event;     /* event it waited for (-1 if none); negative codes:
                             -2 shared-memory ring barrier, -3 iteration word,
                             -5 all-reduce arrivals, -6 flagged word,
                             -7 (error YPK_ERR_STATE) the KV page pool ran out */
  int64_t iterations;     /* iterations completed since create/reset        */
  int32_t finished;       /* 1 when every request has retired               */
  int32_t active_tokens;  /* tokens in the batch that is pending            */
  int64_t tasks_executed; /* worker-side task executions, last launch       */
  int64_t tensor_core_tasks; /* of those, LINEAR tasks run on tcgen05 / TMEM */
} ypk_status;

/* Library / build information. */
int ypk_abi_version(void);
const char *ypk_last_error(const ypk_handle *h);

/* Lifetime (init_persistent_kernel / finalize_persistent_kernel).
 * Environment, read by ypk_create: YPK_TENSOR_CORE = "auto" (default: a LINEAR task with
 * 9..64 tokens takes the tcgen05 path when its estimated time beats the GEMV path),
 * "always" (whenever the task is eligible) or "never". */
int ypk_create(const ypk_config *cfg, ypk_handle **out);
int ypk_destroy(ypk_handle *h);

/* Tensor registry: IODesc TorchTensor / CUDAMallocTensor / ShuffledTorchTensor
 * (src/kernel/graph.cc:338-437). */
int ypk_bind_tensor(ypk_handle *h, int32_t slot, const char *name, void *dev_ptr,
                    uint64_t bytes);
int ypk_alloc_tensor(ypk_handle *h, int32_t slot, const char *name, uint64_t bytes);
/* dst = row-interleave of n_src row-major matrices with the same row length:
 * the destination is a sequence of blocks, block g holding rows
 * [g*gran[i], (g+1)*gran[i]) of source i for i = 0..n_src-1
 * (materialisation of shuffle_tensors, src/kernel/runtime.cc:804-842). */
int ypk_shuffle_tensor(ypk_handle *h, int32_t dst_slot, const char *name, int32_t n_src,
                       const int32_t *src_slots, const int32_t *rows, const int32_t *gran,
                       uint64_t row_bytes);
int ypk_tensor_ptr(ypk_handle *h, int32_t slot, void **dev_ptr, uint64_t *bytes);

/* Tensor parallelism.  Every rank owns one "symmetric arena" of device memory; tensors
 * allocated from it sit at the same offset on every rank (allocate them in the same order
 * everywhere), so a kernel reaches a peer's copy as peer_arena_base + own offset.  Replaces
 * the NVSHMEM symmetric heap of the reference (nvshmem_malloc for io_category
 * "nvshmem_tensor", src/kernel/runtime.cc:797; bootstrap persistent_kernel.cuh:1072-1085).
 * ypk_comm_export writes a 64-byte CUDA IPC handle of the own arena; the caller moves the
 * handles between the ranks' processes (any transport) and gives each peer's handle to
 * ypk_comm_import, which maps that peer's arena.  All of this before the first launch. */
#define YPK_IPC_HANDLE_BYTES 64
int ypk_comm_init(ypk_handle *h, uint64_t arena_bytes);
int ypk_alloc_symmetric(ypk_handle *h, int32_t slot, const char *name, uint64_t bytes);
int ypk_comm_export(ypk_handle *h, void *handle_out);
int ypk_comm_import(ypk_handle *h, int32_t peer_rank, const void *handle);
/* Device-to-device copy of `bytes` bytes of a registered tensor, starting at byte_off,
 * into caller memory on the same device (inspection of runtime-owned intermediates;
 * the reference has no counterpart, its intermediates are unreachable from Python). */
int ypk_read_tensor(ypk_handle *h, int32_t slot, uint64_t byte_off, void *dst_dev_ptr,
                    uint64_t bytes);

/* Task graph: tasks in execution order, events as (trigger count) per event,
 * and the per-worker queues: worker w runs tasks
 * queue[queue_off[w] .. queue_off[w+1]) in that order every iteration. */
int ypk_load_graph(ypk_handle *h, const ypk_task *tasks, int32_t num_tasks,
                   int32_t num_events, const int32_t *queue, const int32_t *queue_off,
                   int32_t num_queues);

/* init_kernel (persistent_kernel.cuh:107-132): zero step[], request slots,
 * refill the free-page queue.  Also clears a device error (ypk_status.error) of a
 * single-GPU handle; a tensor-parallel handle that has seen a device error cannot be
 * reset (YPK_ERR_STATE): destroy the handles of all ranks and create them again.
 * Extension: a caller may write step[r] = s0 > 0 after the reset and before the first
 * launch; request r then enters with its first s0 tokens taken as already cached (it is
 * given the pages for them, in free-queue order, and starts at position s0).  What those
 * pages hold is up to the caller (a benchmark that wants a long context without running the
 * prefill leaves them as they are). */
int ypk_reset(ypk_handle *h);

/* launch_persistent_kernel: run the megakernel on `stream` (a cudaStream_t,
 * may be NULL for the default stream).  mode 1 runs until every request has
 * retired or max_iterations (>0) iterations have completed, whichever comes
 * first; mode 0 runs the graph once for `batch` rows.  Returns after the
 * kernel has finished (the reference call is synchronous too). */
int ypk_launch(ypk_handle *h, void *stream, int32_t max_iterations, int32_t batch);
/* Same, but returns right after enqueueing; pair with ypk_wait. */
int ypk_launch_async(ypk_handle *h, void *stream, int32_t max_iterations, int32_t batch);
int ypk_wait(ypk_handle *h);

int ypk_get_status(ypk_handle *h, ypk_status *out);

/* Two graphs over one set of requests: a graph built for many tokens per iteration runs the
 * prompts, a graph built for a few tokens the decoding (the reference builds one graph for
 * max_num_batched_tokens and runs everything on it, persistent_kernel.cuh:231-239; here the
 * task kernels for at most 8 tokens and those for up to 64 differ).
 * ypk_set_pause_below(h, n): launches of h return, with the batch left waiting, as soon as
 * the batcher forms a batch of at most n tokens (0 switches this off).
 * ypk_adopt_batch(dst, src): dst takes over the requests of src where src stopped: the
 * request slots, the free-page queue and the waiting batch.  Both handles must have been
 * created over the same meta tensors, page pool and limits except max_num_batched_tokens,
 * and the K/V caches of their graphs must be the same memory.  dst must be able to run the
 * waiting batch (YPK_ERR_STATE otherwise); src is finished afterwards until it is reset. */
int ypk_set_pause_below(ypk_handle *h, int32_t tokens);
int ypk_adopt_batch(ypk_handle *dst, ypk_handle *src);

/* dst[c, r] = src[r, c] for a row-major [rows, cols] matrix of 16-bit elements (device
 * pointers on the current device, 16-byte aligned, rows and cols multiples of 8; enqueued on
 * `stream`, no handle needed).  The kernel-graph surface stores a matmul weight as [K, N]
 * (src/kernel/matmul.cc), the LINEAR task streams [N, K]: the weight is turned once, the
 * first time it is seen. */
int ypk_transpose_16bit(const void *src, void *dst, int32_t rows, int32_t cols, void *stream);

/* Greedy sampling for callers that cannot let a library allocate device memory (a host
 * whose own allocator owns the whole GPU, or a path where the device-wide synchronisation
 * of cudaMalloc / cudaFree is not acceptable).  No counterpart in the reference: there the
 * chunk buffers of the two arg-max tasks are cudaMalloc'ed by generated code.
 *
 * out_tokens[b] = index of the largest of logits[b, 0:vocab] (bf16, row stride ld
 * elements), lowest index on ties, for b < batch.  All pointers are device pointers on the
 * current device; the kernel is enqueued on `stream` and the call does not wait for it.
 * Needs no handle.  The per-chunk partial results go to a fixed array inside the library
 * (about 100 KB per GPU, held until the process exits), which is why batch is limited to
 * 64 rows; larger batches are refused with YPK_ERR_UNSUPPORTED.  The call makes no
 * cudaMalloc / cudaFree and calls no allocating library routine.
 * The first call on each device looks up the array's device address
 * (cudaGetSymbolAddress); make that first call outside any stream capture.
 * All calls share the one array: two calls whose kernels can overlap on the GPU (different
 * streams, no dependency) race on it - serialise them. */
int ypk_argmax_noalloc(const void *logits_bf16, int32_t batch, int32_t vocab, int64_t ld,
                       int64_t *out_tokens, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* YPK_H_ */
