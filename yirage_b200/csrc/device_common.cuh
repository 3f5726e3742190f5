// Device-side plumbing shared by every task of the persistent megakernel:
// the run-time descriptor handed to the kernel, shared-memory map, mbarrier /
// bulk-copy (TMA engine) wrappers, acquire/release helpers and bounded waits.
//
// Structure of one worker CTA (one per SM, 288 threads):
//   warps 0..7  consumers: wait for the task's dependency event, stage the
//               activations, do the arithmetic, publish the trigger event;
//   warp  8     producer: walks the same per-worker task queue on its own and
//               streams the bytes that do not depend on activations (weight
//               rows, cached K/V tiles) into a 5-stage shared-memory ring with
//               cp.async.bulk + mbarrier, so HBM stays busy while the consumers
//               sit on an event.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stddef.h>
#include <stdint.h>
#include "../../include/ypk.h"

namespace ypk {

constexpr int kConsumerWarps = 8;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kBlockThreads = kConsumerThreads + 32;  // + producer warp
constexpr int kProducerWarp = kConsumerWarps;

constexpr int kStages = 5;
constexpr int kStageBytes = 34816;               // 34 KB
// GEMV: a stage is 16 weight rows x 1024 columns, 2 KB per row
constexpr int kStageCols = 1024;                 // weight columns per ring stage
constexpr int kRowPitch = kStageCols * 2 + 16;   // 2064 B: 8 rows -> 8 distinct 16-byte bank groups
constexpr int kRowBlock = 16;                    // weight rows per ring stage (M of the MMA)
constexpr int kWarpCols = kStageCols / kConsumerWarps;  // 128 columns of every stage per warp
constexpr int kMaxBatch = 8;                     // tokens per pass (N of the MMA)
constexpr int kMaxAccRows = 256;                 // rows of one LINEAR task when K is chunked

constexpr int kKvTile = 64;                      // cached tokens per ring stage
constexpr int kHeadDim = 128;
constexpr int kKPitch = kHeadDim * 2 + 16;       // 272 B per row of the q / new-token tiles
// A cached K/V stage is four TMA boxes of 64 tokens x 64 dims (128 B rows, 128-byte
// swizzle): K dims 0..63, K dims 64..127, V dims 0..63, V dims 64..127.
constexpr int kKvBoxBytes = kKvTile * 128;       // 8192
constexpr int kVOffset = 2 * kKvBoxBytes;        // V boxes follow the K boxes
constexpr int kMaxNewTokens = 8;                 // new tokens one ATTENTION task takes (a query tile)
constexpr int kMaxNewKeys = 64;                  // new tokens of one request per iteration when its
                                                 // queries are spread over several tasks (YPK_F_QTILES)
constexpr int kMaxAttnRows = 32;                 // new tokens x q heads per kv head, per task
// Cached tiles one attention split should hold.  A warp needs ~2.8 us per tile, so a CTA
// with more tiles than it can overlap runs in rounds; measured on Llama-3-8B at ~600 tokens
// of context, 2..5 tiles per split all beat one CTA per head by ~4 us per layer.
constexpr int kAttnTilesPerSplit = 4;
constexpr int kSiluGran = 2;                     // fused gate/up rows come as 2 gate + 2 up

// Tensor-core LINEAR path (more than 16 tokens): weights arrive as TMA boxes of 64 rows x one
// k-block (a k-block is 64 columns = one 128-byte swizzled row), tokens sit in a ring of 8 KB
// units (one k-block of up to 64 tokens).
constexpr int kUmmaKBlock = 64;
constexpr int kUmmaBoxRows = 64;                 // weight rows per TMA box
constexpr int kUmmaBoxBytes = kUmmaBoxRows * 128;   // 8192
constexpr int kUmmaMaxBatch = 64;                // tokens per pass (M of the MMA)
constexpr int kUmmaUnits = 7;                    // token ring: 7 x 8 KB
constexpr int kUmmaUnitBytes = 8192;
constexpr int kUmmaTmemCols = 512;               // all of the SM's tensor memory (a task uses <= 256 columns)

// Shared-memory map (dynamic shared memory, bytes).
constexpr int kOffRing = 0;
constexpr int kOffXs = kOffRing + kStages * kStageBytes;   // 174080
constexpr int kXsBytes = 36864;                            // activations of a pass, 16-bit
constexpr int kOffPart = kOffXs + kXsBytes;                // 210944
constexpr int kPartBytes = 2 * kConsumerWarps * kRowBlock * kMaxBatch * 4;  // 8192
constexpr int kOffRes = kOffPart + kPartBytes;             // 219136
constexpr int kResBytes = kMaxAccRows * kMaxBatch * 2;     // 4096: residual slice of a task
constexpr int kOffAcc = kOffRes + kResBytes;               // 223232
constexpr int kAccBytes = kMaxAccRows * kMaxBatch * 4;     // 8192
constexpr int kOffMisc = kOffAcc + kAccBytes;              // 231424
constexpr int kMiscBytes = 1024;
constexpr int kSmemBytes = kOffMisc + kMiscBytes;          // 232448 = 227 KB, the per-CTA maximum
constexpr int kScratchSmemBytes = kXsBytes + kPartBytes + kResBytes + kAccBytes;  // 57344 from kOffXs
static_assert(kUmmaUnits * kUmmaUnitBytes <= kScratchSmemBytes, "token ring does not fit");
static_assert(4 * kUmmaBoxBytes <= kStageBytes, "a 256-row k-block does not fit a ring stage");

// Layout of the misc area.
struct __align__(16) Misc {
  unsigned long long full_bar[kStages];
  unsigned long long empty_bar[kStages];
  float rnorm[kMaxBatch];
  unsigned long long ctrl_word;  // broadcast of the published control word
  int flag;                      // generic broadcast slot for the consumers
  unsigned long long *prof_rec;  // timeline record of the current task (thread 0), or null
  int abort_flag;                // set when this CTA has seen an abort
  uint32_t tmem_base;            // tensor-memory address of the CTA's accumulator columns
  unsigned long long xfull_bar[kUmmaUnits];   // token ring of the tensor-core LINEAR path
  unsigned long long xempty_bar[kUmmaUnits];
  unsigned long long acc_bar;    // every MMA of the current task has completed
  float rnorm_umma[kUmmaMaxBatch];
  // arguments of the MMA issuer of the tensor-core LINEAR path (umma_issue), which is a
  // function of its own and takes them from here rather than through the call stack
  int is_nrows, is_nkb, is_task, is_failed;
  uint32_t is_slot, is_phase, is_xslot, is_xphase;
  alignas(16) ypk_task ctask;    // consumer copy of the current task (copied 16 bytes at a time)
  alignas(16) ypk_task ptask;                // producer copy of the current task
};
static_assert(sizeof(Misc) <= kMiscBytes, "misc area too small");
static_assert(offsetof(Misc, ctask) % 16 == 0 && offsetof(Misc, ptask) % 16 == 0, "task copies");
static_assert(sizeof(ypk_task) == 176, "ypk_task layout changed");

// Control block in global memory (unsigned long long words).
enum CtrlWord {
  kCtrlPublished = 0,  // iteration << 32 | state << 16 | active tokens
  kCtrlAbort = 1,      // 0 or error code
  kCtrlFailInfo = 2,   // worker << 40 | (task & 0xfffff) << 20 | (event & 0xfffff)
  kCtrlTasksDone = 3,
  kCtrlFinished = 4,
  kCtrlUmmaTasks = 5,  // LINEAR tasks that took the tensor-core path
  kCtrlWideIters = 6,  // iterations of more than two tokens since the last reset
  kCtrlWords = 8
};
constexpr unsigned kStateRun = 0, kStateStop = 1;

struct Runtime {
  const ypk_task *tasks;
  const int *queue;
  const int *queue_off;
  unsigned long long *events;
  unsigned long long *ctrl;
  // continuous batching state (caller-owned meta tensors + library-owned slots)
  int *step;
  long long *tokens;
  long long *input_tokens;
  long long *output_tokens;
  int *prompt_len;
  int *num_new;       // [total_req] tokens the last iteration gave each request (VERIFY task)
  int *qo_indptr;
  int *kv_indptr;
  int *kv_indices;
  int *kv_last_len;
  int *request_ids;   // [max_req]
  int *page_queue;    // [max_pages]
  int *kv_tmp;        // [max_pages] scratch copy of kv_indices for the batcher
  // Query tiles of the iteration (YPK_F_QTILES): entry i = request slot | first new token of
  // the tile << 12 | tokens of the tile << 20, or -1.  A request with more new tokens than one
  // ATTENTION task takes contributes one tile per rt.attn_chunk tokens.
  int *qtiles;        // [max_tok]
  int *bstate;        // [0] next request id, [1] page queue head, [2] tail
  long long eos;
  long long base_iter;
  long long base_wide;   // iterations of more than two tokens before this launch (see YPK_F_TRIG_WIDE)
  unsigned long long budget_ns;
  int mode, max_seq, max_req, max_tok, max_pages, page_size, total_req;
  int max_iters, fixed_batch, resume_pending, rank, world;
  int max_new_tokens;  // prefill chunk of one request per iteration (<= kMaxNewTokens, or
                       // <= kMaxNewKeys when every ATTENTION task reads the query-tile list)
  int spec_len;        // draft tokens per decoding request and iteration (0: no speculation)
  int attn_chunk;      // new tokens per query tile
  int pause_below;     // > 0: stop (batch pending) once the next batch has at most this many
                       // tokens: the caller continues with a graph built for small batches
  int end_event, end_count;  // event every task of the last operator triggers
  // optional per-task timeline: 8 words per (worker, queue position), overwritten every
  // iteration: {iteration << 32 | task, t_fetch, t_dependency_met, t_done, t_inputs_staged,
  // t_last_stage_consumed, 0, 0} (globaltimer ns; the last two only for LINEAR tasks)
  const void *tmaps;   // array of 128-byte TMA tensor maps (K/V caches, LINEAR weights), or null
  int num_tmaps;       // their number
  int use_tmem;        // allocate tensor memory: some LINEAR task can take the tcgen05 path
  int umma_policy;     // 0 / 1 = whenever eligible, 2 = never
  int umma_depth;      // token units the stagers keep in flight (YPK_UMMA_DEPTH, default 4)
  // iterations run before the last reset: flagged-word tags and all-reduce arrival counts
  // keep growing across resets (ll_epoch also steps over an aborted iteration)
  unsigned long long ll_epoch, ar_epoch;
  int ll_push_fence;   // diagnostic (YPK_LL_PUSH_FENCE=1): system-scope fence after a task's pushes
  char *arena[8];      // symmetric arena of every tensor-parallel rank as mapped here (own at [rank])
  unsigned long long *prof;
  int prof_stride;  // records per worker
};

// ---------------------------------------------------------------- PTX helpers
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ unsigned long long globaltimer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ unsigned long long ld_acquire_u64(const unsigned long long *p) {
  unsigned long long v;
  asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long ld_relaxed_u64(const unsigned long long *p) {
  unsigned long long v;
  asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long ld_acquire_sys_u64(const unsigned long long *p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_sys_add_u64(unsigned long long *p, unsigned long long v) {
  asm volatile("red.release.sys.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void st_release_u64(unsigned long long *p, unsigned long long v) {
  asm volatile("st.release.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void red_release_add_u64(unsigned long long *p, unsigned long long v) {
  asm volatile("red.release.gpu.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

__device__ __forceinline__ void mbar_init(unsigned long long *bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(unsigned long long *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned long long *bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Global -> shared bulk copy through the TMA engine; completion is counted in
// bytes on `bar`.  dst, src 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, uint32_t bytes,
                                         unsigned long long *bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
          "r"(smem_u32(dst)),
      "l"(src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void bulk_g2s_hint(void *dst, const void *src, uint32_t bytes,
                                              unsigned long long *bar, unsigned long long policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint "
      "[%0], [%1], %2, [%3], %4;" ::"r"(smem_u32(dst)),
      "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
      : "memory");
}
// Tiled TMA load of one box of a rank-3 tensor map into shared memory; (x, y, z) are element
// coordinates from the innermost dimension outwards, x * element size a multiple of 16 B.
__device__ __forceinline__ void tma_load_3d(void *dst, const void *tmap, int x, int y, int z,
                                            unsigned long long *bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3, %4}], [%5];" ::"r"(smem_u32(dst)),
      "l"(tmap), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ unsigned long long policy_evict_first() {
  unsigned long long p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ void consumer_bar() {
  asm volatile("bar.sync 1, %0;" ::"n"(kConsumerThreads) : "memory");
}

// Packed fp32x2 arithmetic (two FMAs per issue slot on sm_100).
__device__ __forceinline__ unsigned long long fma2(unsigned long long a, unsigned long long b,
                                                   unsigned long long c) {
  unsigned long long d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ unsigned long long pack2(float lo, float hi) {
  unsigned long long d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "f"(lo), "f"(hi));
  return d;
}
__device__ __forceinline__ float2 unpack2(unsigned long long v) {
  float2 r;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(r.x), "=f"(r.y) : "l"(v));
  return r;
}
// Two packed 16-bit floats -> fp32x2.
template <bool F16>
__device__ __forceinline__ unsigned long long cvt_pair(uint32_t p) {
  if constexpr (F16) {
    float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&p));
    return pack2(f.x, f.y);
  } else {
    unsigned long long d;
    uint32_t lo = p << 16, hi = p & 0xffff0000u;
    asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(hi));
    return d;
  }
}
template <bool F16>
__device__ __forceinline__ float cvt_one(uint16_t v) {
  if constexpr (F16) {
    return __half2float(__ushort_as_half(v));
  } else {
    return __uint_as_float(static_cast<uint32_t>(v) << 16);
  }
}
template <bool F16>
__device__ __forceinline__ uint16_t cvt_out(float v) {
  if constexpr (F16) {
    return __half_as_ushort(__float2half_rn(v));
  } else {
    return __bfloat16_as_ushort(__float2bfloat16_rn(v));
  }
}
__device__ __forceinline__ float bf16_round(float v) {
  return __bfloat162float(__float2bfloat16_rn(v));
}

// ------------------------------------------------------------ bounded waiting
// Every wait in the kernel goes through one of these.  When the budget runs
// out the waiter records who gave up, raises the global abort word and
// returns false; every other waiter sees the abort word and returns false too,
// so the grid drains instead of hanging.
struct WaitCtx {
  const Runtime *rt;
  Misc *misc;
  int worker;
  int task;
  bool failed;  // sticky: once a wait of this warp has given up, later waits return at once
};

__device__ __forceinline__ bool abort_seen(const WaitCtx &w) {
  return ld_relaxed_u64(w.rt->ctrl + kCtrlAbort) != 0ull;
}
static __device__ __noinline__ void raise_abort(const WaitCtx &w, int code, int event) {
  unsigned long long info = (static_cast<unsigned long long>(w.worker) << 40) |
                            ((static_cast<unsigned long long>(w.task) & 0xfffffull) << 20) |
                            (static_cast<unsigned long long>(event) & 0xfffffull);
  unsigned long long old = atomicCAS(w.rt->ctrl + kCtrlAbort, 0ull,
                                     static_cast<unsigned long long>(static_cast<unsigned>(-code)));
  if (old == 0ull) {
    w.rt->ctrl[kCtrlFailInfo] = info;
    __threadfence();
  }
}

// Wait until *ctr >= need (acquire).  One thread calls this.
__device__ __forceinline__ bool wait_counter(const WaitCtx &w, const unsigned long long *ctr,
                                             unsigned long long need, int event) {
  if (ld_acquire_u64(ctr) >= need) return true;
  unsigned long long t0 = globaltimer();
  for (uint32_t it = 1;; ++it) {
    if (ld_acquire_u64(ctr) >= need) return true;
    __nanosleep(20);
    if ((it & 63u) == 0u) {
      if (abort_seen(w)) return false;
      if (globaltimer() - t0 > w.rt->budget_ns) {
        raise_abort(w, YPK_ERR_TIMEOUT, event);
        return false;
      }
    }
  }
}

// Same for a counter that peer GPUs bump over NVLink (system scope).
__device__ __forceinline__ bool wait_counter_sys(const WaitCtx &w, const unsigned long long *ctr,
                                                 unsigned long long need, int event) {
  if (ld_acquire_sys_u64(ctr) >= need) return true;
  unsigned long long t0 = globaltimer();
  for (uint32_t it = 1;; ++it) {
    if (ld_acquire_sys_u64(ctr) >= need) return true;
    __nanosleep(20);
    if ((it & 63u) == 0u) {
      if (abort_seen(w)) return false;
      if (globaltimer() - t0 > w.rt->budget_ns) {
        raise_abort(w, YPK_ERR_TIMEOUT, event);
        return false;
      }
    }
  }
}

// Wait for a phase of an mbarrier.  Called by all 32 lanes of a warp together; the
// outcome is the same for every lane, so control flow stays warp-uniform.  After a
// failure the caller keeps walking its loops (skipping the work) so that CTA-level
// barriers still line up; every later wait returns false immediately.
__device__ __forceinline__ bool wait_mbar(WaitCtx &w, unsigned long long *bar, uint32_t parity) {
  if (w.failed) return false;
  if (__all_sync(0xffffffffu, mbar_try_wait(bar, parity))) return true;
  const unsigned long long t0 = globaltimer();
  for (uint32_t it = 1;; ++it) {
    if (__all_sync(0xffffffffu, mbar_try_wait(bar, parity))) return true;
    if ((it & 127u) == 0u) {
      const bool seen = abort_seen(w);
      const bool late = globaltimer() - t0 > w.rt->budget_ns;
      if (__any_sync(0xffffffffu, seen || late)) {
        if ((threadIdx.x & 31) == 0 && !seen) raise_abort(w, YPK_ERR_TIMEOUT, -2);
        w.failed = true;
        return false;
      }
    }
  }
}

// Position in the shared-memory ring; producer and consumers each keep one and
// advance it identically.
struct RingPos {
  uint32_t slot = 0;
  uint32_t phase = 0;
  uint32_t count = 0;  // stages passed so far
  __device__ __forceinline__ void advance() {
    ++count;
    if (++slot == kStages) {
      slot = 0;
      phase ^= 1u;
    }
  }
};

// Per-thread position in the token ring and phase of the accumulator barrier; every
// consumer thread keeps one and advances it identically.
struct UmmaState {
  uint32_t xslot = 0, xphase = 0, acc_phase = 0;
  __device__ __forceinline__ void advance() {
    if (++xslot == uint32_t(kUmmaUnits)) {
      xslot = 0;
      xphase ^= 1u;
    }
  }
};

// Columns of K staged per pass for a batch of `b` tokens: b rows of 16-bit activations
// (row pitch = columns + 8) have to fit the x area; multiple of kStageCols.
__device__ __forceinline__ int chunk_cols(int b, int K) {
  const int kc = (kXsBytes / 2 / b - 8) / kStageCols * kStageCols;
  return kc < K ? kc : K;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

}  // namespace ypk
