// Host side of the C ABI declared in include/ypk.h: handle, tensor registry, graph
// loading/validation, launch and status.  The device code lives in megakernel.cuh.
//
// A handle created with cfg.device == -1 is a host-only handle: it validates and
// resolves graphs exactly like a real one but owns no device memory and cannot launch.
// It exists so that graph validation can be exercised on a machine without a GPU.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdlib.h>
#include <stdio.h>
#include <string.h>

#include <algorithm>
#include <string>
#include <vector>

#include "../../include/ypk.h"
#include "argmax_noalloc.cuh"
#include "megakernel.cuh"
#include "task_attention.cuh"   // kAttnRowFloats

using namespace ypk;

namespace {

// dst[c][r] = src[r][c], 16-bit elements, 32 x 32 tiles through shared memory
__global__ void transpose16_kernel(const uint16_t *src, uint16_t *dst, int rows, int cols) {
  __shared__ uint16_t tile[32][33];
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int r = r0 + i, c = c0 + threadIdx.x;
    if (r < rows && c < cols) tile[i][threadIdx.x] = src[size_t(r) * cols + c];
  }
  __syncthreads();
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int c = c0 + i, r = r0 + threadIdx.x;
    if (r < rows && c < cols) dst[size_t(c) * rows + r] = tile[threadIdx.x][i];
  }
}

struct Slot {
  void *ptr = nullptr;
  uint64_t bytes = 0;
  bool owned = false;
  bool used = false;
  std::string name;
};

}  // namespace

struct ypk_handle {
  ypk_config cfg;
  bool host_only = false;
  int num_workers = 0;
  int sm_count = 0;
  std::vector<Slot> slots;
  std::vector<ypk_task> tasks;  // resolved copies
  std::vector<int32_t> queue, queue_off;
  int num_events = 0;
  int end_event = -1, end_count = 0;
  int max_new_tokens = kMaxNewTokens;  // prefill chunk per request the attention tasks allow
  int attn_chunk = kMaxNewTokens;      // new tokens per query tile (YPK_F_QTILES)
  bool attn_plain = false, attn_qtiles = false;   // kinds of ATTENTION task in the graph
  int pause_below = 0;
  int spec_len = 0;                    // draft tokens per decoding request (a VERIFY task sets it)
  bool has_moe = false;                // some LINEAR task picks its expert at run time
  bool graph_loaded = false;
  // device state
  ypk_task *d_tasks = nullptr;
  int *d_queue = nullptr, *d_queue_off = nullptr;
  unsigned long long *d_events = nullptr, *d_ctrl = nullptr;
  char *arena = nullptr;         // symmetric arena (tensor parallelism)
  uint64_t arena_bytes = 0, arena_used = 0;
  char *peer_arena[8] = {nullptr};   // peers' arenas mapped through CUDA IPC (own at [rank])
  void *d_tmaps = nullptr;       // CUtensorMap[], one per distinct K / V cache tensor
  int num_tmaps = 0;
  std::vector<uint64_t> tmap_keys;  // device address of the cache each map describes
  bool use_tmem = false;            // some LINEAR task has a weight tensor map
  int umma_policy = 0;              // YPK_TENSOR_CORE: auto (by estimated cost) / always / never
  int *d_request_ids = nullptr, *d_page_queue = nullptr, *d_kv_tmp = nullptr, *d_bstate = nullptr;
  int *d_qtiles = nullptr;
  // progress
  long long base_iter = 0;
  // iterations of earlier runs (see Runtime::ll_epoch / ar_epoch)
  unsigned long long ll_epoch = 0, ar_epoch = 0;
  long long abort_iters = 0;   // last iteration an aborted launch had published
  long long wide_iters = 0;    // iterations of more than two tokens since the last reset
  int pending_tokens = 0;
  bool resume_pending = false;
  bool finished = false;
  bool in_flight = false;
  cudaStream_t stream = nullptr;
  ypk_status status;
  std::string err;
};

namespace {

thread_local std::string g_err;

int fail(ypk_handle *h, int code, const char *fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  if (h) h->err = buf;
  g_err = buf;
  return code;
}

#define CUDA_TRY(h, call)                                                              \
  do {                                                                                 \
    cudaError_t e_ = (call);                                                           \
    if (e_ != cudaSuccess)                                                             \
      return fail(h, YPK_ERR_CUDA, "%s failed: %s", #call, cudaGetErrorString(e_));    \
  } while (0)

Slot *get_slot(ypk_handle *h, int32_t slot, bool create) {
  if (slot < 0 || slot >= 65534) return nullptr;
  if (size_t(slot) >= h->slots.size()) {
    if (!create) return nullptr;
    h->slots.resize(size_t(slot) + 1);
  }
  return &h->slots[size_t(slot)];
}

void release_slot(ypk_handle *h, Slot &s) {
  if (s.owned && s.ptr && !h->host_only) cudaFree(s.ptr);
  s = Slot();
}

// Resolve one encoded operand; checks that [offset, offset+need) lies inside the tensor.
int resolve(ypk_handle *h, int ti, int pi, uint64_t ref, uint64_t need, uint64_t align,
            uint64_t *out) {
  if (ref == 0) {
    *out = 0;
    return need == 0 ? YPK_OK
                     : fail(h, YPK_ERR_INVALID, "task %d: operand %d is required", ti, pi);
  }
  const int slot = int(ref >> 48) - 1;
  const uint64_t off = ref & 0xFFFFFFFFFFFFull;
  Slot *s = get_slot(h, slot, false);
  if (!s || !s->used)
    return fail(h, YPK_ERR_INVALID, "task %d: operand %d names unbound tensor slot %d", ti, pi,
                slot);
  if (off + need > s->bytes)
    return fail(h, YPK_ERR_INVALID,
                "task %d: operand %d reaches byte %llu of tensor '%s' (%llu bytes)", ti, pi,
                (unsigned long long)(off + need), s->name.c_str(), (unsigned long long)s->bytes);
  const uint64_t addr = reinterpret_cast<uint64_t>(s->ptr) + off;
  if (align && addr % align)
    return fail(h, YPK_ERR_INVALID, "task %d: operand %d of tensor '%s' is not %llu-byte aligned",
                ti, pi, s->name.c_str(), (unsigned long long)align);
  *out = addr;
  return YPK_OK;
}

// Shape checks + pointer resolution for one task.  `mb` = largest batch the graph can see.
int check_task(ypk_handle *h, int ti, const ypk_task &in, ypk_task *out) {
  *out = in;
  const int mb = h->cfg.max_num_batched_tokens > 0 ? h->cfg.max_num_batched_tokens : 1;
  const int32_t *a = in.iarg;
  uint64_t need[YPK_TASK_NPTR] = {0}, align[YPK_TASK_NPTR] = {0};
  bool required[YPK_TASK_NPTR] = {false};
  uint64_t need_aux = 0, align_aux = 0;   // the ninth operand (ptr_aux)
  auto rows = [](int ld, int n, int cols) -> uint64_t {  // bytes spanned by n rows of 16-bit
    return n <= 0 ? 0 : (uint64_t(n - 1) * ld + cols) * 2u;
  };
  switch (in.type) {
    case YPK_TASK_NOP: break;
    case YPK_TASK_LINEAR: {
      const int K = a[0], row0 = a[1], nrows = a[2], ldx = a[3], ldw = a[4], ldo = a[5],
                ldr = a[6], oc0 = a[7];
      if (K <= 0 || K % 64 || nrows <= 0 || nrows > kMaxAccRows || row0 < 0)
        return fail(h, YPK_ERR_UNSUPPORTED,
                    "task %d: LINEAR needs K %% 64 == 0 and 1..%d rows (K=%d rows=%d)", ti,
                    kMaxAccRows, K, nrows);
      if (ldx % 8 || ldw % 8 || ldx < K || ldw < K)
        return fail(h, YPK_ERR_INVALID, "task %d: LINEAR strides (ldx=%d ldw=%d K=%d)", ti, ldx,
                    ldw, K);
      const bool silu = in.flags & YPK_F_SILU_MUL;
      if (silu && (row0 % (2 * kSiluGran) || nrows % (2 * kSiluGran)))
        return fail(h, YPK_ERR_INVALID, "task %d: SILU_MUL rows must come in %d-row granules", ti,
                    2 * kSiluGran);
      if ((in.flags & YPK_F_NORM) && (in.flags & YPK_F_NORM_NOWEIGHT))
        return fail(h, YPK_ERR_INVALID, "task %d: NORM and NORM_NOWEIGHT together", ti);
      const int ocols0 = silu ? oc0 + row0 / 2 : oc0 + row0;
      const int ocols = silu ? nrows / 2 : nrows;
      need[0] = rows(ldx, mb, K); align[0] = 16; required[0] = true;
      need[1] = rows(ldw, row0 + nrows, K); align[1] = 16; required[1] = true;
      need[2] = rows(ldo, mb, ocols0 + ocols); align[2] = 2; required[2] = true;
      if (in.flags & YPK_F_MOE) {
        // the weights of one of E experts, picked at run time from the active list
        const int E = a[11], per = a[12], slot = a[10];
        if (in.flags & (YPK_F_NORM | YPK_F_NORM_NOWEIGHT | YPK_F_RESIDUAL | YPK_F_SILU_MUL | YPK_F_LL_IN |
                        YPK_F_LL_RES | YPK_F_LL_OUT | YPK_F_LL_PUSH | YPK_F_LL_OPT) || a[13] || a[14] || a[15])
          return fail(h, YPK_ERR_UNSUPPORTED, "task %d: an expert LINEAR task is a plain projection", ti);
        if (E < 1 || slot < 0 || slot >= E || per < row0 + nrows)
          return fail(h, YPK_ERR_INVALID, "task %d: expert LINEAR slot %d of %d experts, %d rows each", ti,
                      slot, E, per);
        if (h->cfg.world_size != 1)
          return fail(h, YPK_ERR_UNSUPPORTED, "task %d: mixture-of-experts graphs are built for one GPU", ti);
        need[1] = rows(ldw, (E - 1) * per + row0 + nrows, K);
        need[5] = uint64_t(E + 1) * 4; align[5] = 4; required[5] = true;
        h->has_moe = true;
      }
      if (in.flags & YPK_F_NORM) { need[3] = uint64_t(K) * 2; align[3] = 16; required[3] = true; }
      if (in.flags & YPK_F_RESIDUAL) {
        need[4] = rows(ldr, mb, ocols0 + ocols); align[4] = 2; required[4] = true;
      }
      // K range / split along K (graphs of more than 8 tokens)
      const int k0 = a[13], klen = a[14] > 0 ? a[14] : K - a[13];
      const int split = a[15] & 0xff, nsplit = (a[15] >> 8) & 0xff, ws_tok = a[15] >> 16;
      if (k0 < 0 || k0 % 64 || klen <= 0 || klen % 64 || k0 + klen > K)
        return fail(h, YPK_ERR_INVALID, "task %d: LINEAR K range [%d, %d) of %d", ti, k0, k0 + klen, K);
      if (nsplit > 1) {
        const int ws_ld = a[8], cnt = a[10];
        if (mb <= kMaxBatch || (in.flags & (YPK_F_LL_IN | YPK_F_LL_RES | YPK_F_LL_OUT | YPK_F_LL_PUSH)))
          return fail(h, YPK_ERR_UNSUPPORTED,
                      "task %d: the split along K is built for graphs of more than %d tokens", ti, kMaxBatch);
        if (split >= nsplit || ws_tok < mb || ws_ld < row0 + nrows || cnt < 0)
          return fail(h, YPK_ERR_INVALID, "task %d: split %d of %d, workspace [%d tokens][%d rows]", ti,
                      split, nsplit, ws_tok, ws_ld);
        need[5] = uint64_t(nsplit) * ws_tok * ws_ld * 4; align[5] = 16; required[5] = true;
        need[6] = uint64_t(cnt + 1) * nsplit * ws_tok * 4; align[6] = 4; required[6] = true;
        need[7] = uint64_t(cnt + 1) * ((ws_tok + 15) / 16) * 4; align[7] = 4; required[7] = true;
      } else if (klen != K) {
        return fail(h, YPK_ERR_INVALID, "task %d: a K range needs a split count", ti);
      }
      // RMSNorm carried across two operators (graphs of more than 8 tokens, tensor-core path)
      if (in.flags & (YPK_F_NORM_OUT | YPK_F_NORM_PRE)) {
        const int blk = a[12] & 0xffff, pitch = a[12] >> 16;
        if (mb <= kMaxBatch || (in.flags & (YPK_F_NORM | YPK_F_NORM_NOWEIGHT | YPK_F_MOE | YPK_F_LL_IN |
                                            YPK_F_LL_RES | YPK_F_LL_OUT | YPK_F_LL_PUSH | YPK_F_LL_OPT)))
          return fail(h, YPK_ERR_UNSUPPORTED,
                      "task %d: a norm carried across operators needs a graph of more than %d tokens and "
                      "plain 16-bit rows", ti, kMaxBatch);
        if (pitch < mb)
          return fail(h, YPK_ERR_INVALID, "task %d: sums of squares for %d tokens, the graph has %d", ti,
                      pitch, mb);
        if (in.flags & YPK_F_NORM_OUT) {
          if (silu || row0 % 4 || nrows % 4 || oc0 % 4 || ldo % 4)
            return fail(h, YPK_ERR_INVALID, "task %d: NORM_OUT needs rows and columns in fours, no SILU_MUL", ti);
          need[3] = uint64_t(ocols0 + ocols) * 2; align[3] = 2; required[3] = true;
          need[6] = uint64_t(blk + 1) * pitch * 4; align[6] = 4; required[6] = true;
          need_aux = rows(ldo, mb, ocols0 + ocols); align_aux = 8;
        }
        if (in.flags & YPK_F_NORM_PRE) {
          if (in.flags & YPK_F_NORM_OUT)
            return fail(h, YPK_ERR_UNSUPPORTED, "task %d: NORM_PRE and NORM_OUT on one task", ti);
          if (blk < 1) return fail(h, YPK_ERR_INVALID, "task %d: NORM_PRE over no row blocks", ti);
          need[3] = uint64_t(blk) * pitch * 4; align[3] = 4; required[3] = true;
        }
      }
      // flagged-word copies: 4 bytes per value ([max_tokens][ld / 2] 8-byte words)
      const uint32_t ll = in.flags & (YPK_F_LL_IN | YPK_F_LL_RES | YPK_F_LL_OUT | YPK_F_LL_PUSH);
      if (ll) {
        if (mb > kMaxBatch)
          return fail(h, YPK_ERR_UNSUPPORTED,
                      "task %d: flagged-word hand-off is built for at most %d tokens", ti, kMaxBatch);
        if ((in.flags & YPK_F_LL_PUSH) && !(in.flags & YPK_F_LL_OUT))
          return fail(h, YPK_ERR_INVALID, "task %d: LL_PUSH without LL_OUT", ti);
        if ((in.flags & YPK_F_LL_RES) && !(in.flags & YPK_F_RESIDUAL))
          return fail(h, YPK_ERR_INVALID, "task %d: LL_RES without RESIDUAL", ti);
        if (in.flags & YPK_F_LL_IN) {
          if (ldx % 4) return fail(h, YPK_ERR_INVALID, "task %d: LL_IN needs ldx %% 4 == 0", ti);
          need[5] = uint64_t(mb) * ldx * 4; align[5] = 16; required[5] = true;
        }
        if (in.flags & YPK_F_LL_RES) {
          if (ldr % 2 || (oc0 + row0) % 2 || nrows % 2)
            return fail(h, YPK_ERR_INVALID, "task %d: LL_RES needs even rows and columns", ti);
          need[6] = uint64_t(mb) * ldr * 4; align[6] = 8; required[6] = true;
        }
        if (in.flags & YPK_F_LL_OUT) {
          const int gran = silu ? 2 * kSiluGran : 2;
          if (ldo % 2 || oc0 % 2 || row0 % gran || nrows % gran)
            return fail(h, YPK_ERR_INVALID, "task %d: LL_OUT needs rows in granules of %d", ti, gran);
          const uint64_t copies = (in.flags & YPK_F_LL_PUSH) ? uint64_t(h->cfg.world_size) : 1u;
          need[7] = copies * mb * ldo * 4; align[7] = 8; required[7] = true;
        }
      }
      break;
    }
    case YPK_TASK_EMBED: {
      const int col0 = a[1], ncols = a[2], ldt = a[3], ldo = a[4];
      if (ncols <= 0 || ncols % 8 || col0 % 8 || ldt % 8 || ldo % 8)
        return fail(h, YPK_ERR_INVALID, "task %d: EMBED columns must be multiples of 8", ti);
      need[0] = uint64_t(mb) * 8; align[0] = 8; required[0] = true;
      if (a[5] <= 0)
        return fail(h, YPK_ERR_INVALID, "task %d: EMBED needs the row count of its table (iarg[5])", ti);
      need[1] = rows(ldt, a[5], col0 + ncols); align[1] = 16; required[1] = true;
      need[2] = rows(ldo, mb, col0 + ncols); align[2] = 16; required[2] = true;
      break;
    }
    case YPK_TASK_ATTENTION: {
      const int r = a[0], kvh = a[1], split = a[2], nsplit = a[3], G = a[4], hkv = a[5],
                ldq = a[6], ldo = a[7], max_rows = a[8];
      const bool qtiles = (in.flags & YPK_F_QTILES) != 0;
      // iarg[0] is a request slot, or with YPK_F_QTILES an entry of the query-tile list
      // (iarg[14] = length of that list as the graph was built for it)
      const int nslots = qtiles ? a[14] : h->cfg.max_num_batched_requests;
      if (qtiles && (a[14] < 1 || a[14] > h->cfg.max_num_batched_tokens))
        return fail(h, YPK_ERR_INVALID, "task %d: ATTENTION over %d query tiles, the graph has %d token slots",
                    ti, a[14], h->cfg.max_num_batched_tokens);
      if (qtiles && ((in.flags & (YPK_F_LL_IN | YPK_F_LL_OUT)) ||
                     h->cfg.max_num_batched_requests > 4096))
        return fail(h, YPK_ERR_UNSUPPORTED,
                    "task %d: ATTENTION over query tiles needs plain 16-bit rows on both sides "
                    "and at most 4096 request slots", ti);
      if (G < 1 || G > 8 || hkv < 1 || kvh < 0 || kvh >= hkv || nsplit < 1 || split < 0 ||
          split >= nsplit || r < 0 || r >= nslots)
        return fail(h, YPK_ERR_UNSUPPORTED,
                    "task %d: ATTENTION needs 1..8 q heads per kv head (got %d), head_dim 128", ti,
                    G);
      if (h->cfg.page_size <= 0 || h->cfg.page_size % kKvTile)
        return fail(h, YPK_ERR_UNSUPPORTED, "ATTENTION needs page_size %% %d == 0 (got %d)",
                    kKvTile, h->cfg.page_size);
      if (max_rows < std::min(G * kMaxNewTokens, kMaxAttnRows))
        return fail(h, YPK_ERR_INVALID, "task %d: ATTENTION scratch rows %d < %d", ti, max_rows,
                    std::min(G * kMaxNewTokens, kMaxAttnRows));
      h->attn_chunk = std::min(h->attn_chunk, kMaxAttnRows / G);
      (qtiles ? h->attn_qtiles : h->attn_plain) = true;
      if (!h->cfg.qo_indptr || !h->cfg.paged_kv_indptr || !h->cfg.paged_kv_indices ||
          !h->cfg.paged_kv_last_page_len)
        return fail(h, YPK_ERR_INVALID, "ATTENTION needs the paged-KV meta tensors in ypk_config");
      const uint64_t cache_bytes =
          uint64_t(h->cfg.max_num_pages) * h->cfg.page_size * hkv * kHeadDim * 2u;
      need[0] = rows(ldq, mb, hkv * (G + 2) * kHeadDim); align[0] = 16; required[0] = true;
      need[1] = cache_bytes; align[1] = 16; required[1] = true;
      need[2] = cache_bytes; align[2] = 16; required[2] = true;
      need[3] = rows(ldo, mb, hkv * G * kHeadDim); align[3] = 4; required[3] = true;
      // flagged-word forms of the packed q/k/v and of the result: 4 bytes per value
      if (in.flags & YPK_F_LL_IN) { need[0] = uint64_t(mb) * ldq * 4; align[0] = 16; }
      if (in.flags & YPK_F_LL_OUT) { need[3] = uint64_t(mb) * ldo * 4; align[3] = 8; }
      if ((in.flags & (YPK_F_LL_IN | YPK_F_LL_OUT)) && (mb > kMaxBatch || ldq % 4 || ldo % 2))
        return fail(h, YPK_ERR_UNSUPPORTED, "task %d: flagged-word ATTENTION shape", ti);
      if (in.flags & YPK_F_ROPE) {
        need[4] = need[5] = uint64_t(kHeadDim) * 2; align[4] = align[5] = 2;
        required[4] = required[5] = true;
      }
      if (nsplit > 1) {
        need[6] = uint64_t(nslots) * hkv * nsplit * max_rows *
                  kAttnRowFloats * 8u;   // flagged words {fp32 bits, tag}
        align[6] = 16; required[6] = true;
      }
      if (in.flags & YPK_F_QK_NORM) {
        need[7] = 2u * kHeadDim * 2u; align[7] = 16; required[7] = true;
      }
      break;
    }
    case YPK_TASK_ARGMAX_PARTIAL: {
      const int col0 = a[0], ncols = a[1], ld = a[2], part = a[3], nparts = a[4];
      if (ncols <= 0 || part < 0 || part >= nparts)
        return fail(h, YPK_ERR_INVALID, "task %d: ARGMAX_PARTIAL part %d of %d", ti, part, nparts);
      need[0] = rows(ld, mb, col0 + ncols); align[0] = 2; required[0] = true;
      need[1] = uint64_t(mb) * nparts * 2; align[1] = 2; required[1] = true;
      need[2] = uint64_t(mb) * nparts * 8; align[2] = 8; required[2] = true;
      break;
    }
    case YPK_TASK_ARGMAX_REDUCE: {
      const int nparts = a[0], ldp = a[4] > 0 ? a[4] : a[0];
      if (nparts <= 0 || ldp < nparts) return fail(h, YPK_ERR_INVALID, "task %d: ARGMAX_REDUCE nparts", ti);
      need[0] = uint64_t(mb) * ldp * 2; align[0] = 2; required[0] = true;
      need[1] = uint64_t(mb) * ldp * 8; align[1] = 8; required[1] = true;
      need[2] = uint64_t(mb) * 8; align[2] = 8; required[2] = true;
      if (in.flags & YPK_F_LL_PUSH) {   // vocabulary split over the ranks: winners are exchanged
        if (a[2] != h->cfg.world_size || a[3] != h->cfg.rank || a[2] < 2 || a[2] > 8 || a[1] < 0)
          return fail(h, YPK_ERR_INVALID, "task %d: ARGMAX_REDUCE exchange for rank %d of %d", ti, a[3], a[2]);
        need[3] = uint64_t(a[2]) * mb * 16; align[3] = 16; required[3] = true;
      }
      break;
    }
    case YPK_TASK_MOE_TOPK: {
      const int E = a[0], K = a[1], ld = a[2];
      if (E < 1 || E > 1024 || K < 1 || K > 32 || K > E || ld < E)
        return fail(h, YPK_ERR_UNSUPPORTED, "task %d: MOE_TOPK over %d experts, top %d (up to 1024 / 32)", ti, E, K);
      need[0] = rows(ld, mb, E); align[0] = 2; required[0] = true;
      need[1] = uint64_t(mb) * K * 4; align[1] = 4; required[1] = true;
      need[2] = uint64_t(E) * mb * 4; align[2] = 4; required[2] = true;
      need[3] = uint64_t(E + 1) * 4; align[3] = 4; required[3] = true;
      need[4] = uint64_t(mb) * K * 4; align[4] = 4; required[4] = true;
      break;
    }
    case YPK_TASK_MOE_SILU_MUL: {
      const int I = a[0], E = a[1], slot0 = a[2], nslots = a[3];
      if (I < 1 || E < 1 || slot0 < 0 || nslots < 1)
        return fail(h, YPK_ERR_INVALID, "task %d: MOE_SILU_MUL shape", ti);
      need[0] = uint64_t(slot0 + nslots) * mb * 2 * I * 2; align[0] = 2; required[0] = true;
      need[1] = uint64_t(slot0 + nslots) * mb * I * 2; align[1] = 2; required[1] = true;
      need[2] = uint64_t(E + 1) * 4; align[2] = 4; required[2] = true;
      break;
    }
    case YPK_TASK_MOE_COMBINE: {
      const int H = a[0], K = a[1], col0 = a[2], ncols = a[3], ldr = a[4], ldo = a[5];
      if (H < 1 || K < 1 || col0 < 0 || ncols < 1 || col0 + ncols > H || ldr < H || ldo < H)
        return fail(h, YPK_ERR_INVALID, "task %d: MOE_COMBINE shape", ti);
      // the expert outputs are [slots][max_tokens][H]; a token's slots are below the count
      need[0] = uint64_t(mb) * H * 2; align[0] = 2; required[0] = true;
      need[1] = uint64_t(mb) * K * 4; align[1] = 4; required[1] = true;
      need[2] = uint64_t(mb) * K * 4; align[2] = 4; required[2] = true;
      need[3] = rows(ldr, mb, H); align[3] = 2; required[3] = true;
      need[4] = rows(ldo, mb, H); align[4] = 2; required[4] = true;
      break;
    }
    case YPK_TASK_NGRAM_PARTIAL: {
      const int part = a[0], nparts = a[1], ngram = a[2];
      if (h->cfg.mode != 1 || !h->cfg.num_new_tokens)
        return fail(h, YPK_ERR_INVALID, "task %d: prompt lookup needs the serving mode and num_new_tokens", ti);
      if (nparts < 1 || part < 0 || part >= nparts || ngram < 1 || ngram > 8)
        return fail(h, YPK_ERR_INVALID, "task %d: NGRAM_PARTIAL part %d of %d, n-gram of %d", ti, part, nparts, ngram);
      need[0] = uint64_t(h->cfg.max_num_batched_requests) * nparts * 4; align[0] = 4; required[0] = true;
      break;
    }
    case YPK_TASK_NGRAM_GLOBAL: {
      const int nparts = a[0], ngram = a[1];
      if (h->cfg.mode != 1 || !h->cfg.num_new_tokens)
        return fail(h, YPK_ERR_INVALID, "task %d: prompt lookup needs the serving mode and num_new_tokens", ti);
      if (nparts < 1 || ngram < 1 || ngram > 8)
        return fail(h, YPK_ERR_INVALID, "task %d: NGRAM_GLOBAL over %d parts, n-gram of %d", ti, nparts, ngram);
      need[0] = uint64_t(h->cfg.max_num_batched_requests) * nparts * 4; align[0] = 4; required[0] = true;
      need[1] = uint64_t(mb) * 8; align[1] = 8; required[1] = true;
      break;
    }
    case YPK_TASK_VERIFY: {
      if (h->cfg.mode != 1 || !h->cfg.num_new_tokens)
        return fail(h, YPK_ERR_INVALID, "task %d: VERIFY needs the serving mode and num_new_tokens", ti);
      if (a[0] < 1 || a[0] + 1 > kMaxNewTokens)
        return fail(h, YPK_ERR_UNSUPPORTED, "task %d: %d draft tokens (1..%d)", ti, a[0], kMaxNewTokens - 1);
      if (h->spec_len && h->spec_len != a[0])
        return fail(h, YPK_ERR_INVALID, "task %d: two VERIFY tasks with different draft lengths", ti);
      h->spec_len = a[0];
      need[0] = uint64_t(mb) * 8; align[0] = 8; required[0] = true;
      need[1] = uint64_t(mb) * 8; align[1] = 8; required[1] = true;
      break;
    }
    case YPK_TASK_ALLREDUCE: {
      const int col0 = a[0], ncols = a[1], ldi = a[2], ldo = a[3], hidden = a[4], mt = a[5],
                sidx = a[7], world = a[8], rank = a[9];
      if (world != h->cfg.world_size || rank != h->cfg.rank || world < 2 || world > 8)
        return fail(h, YPK_ERR_INVALID, "task %d: ALLREDUCE for rank %d of %d on a handle of rank %d of %d",
                    ti, rank, world, h->cfg.rank, h->cfg.world_size);
      if (ncols <= 0 || ncols % 8 || col0 % 8 || col0 + ncols > hidden || ldi % 8 || ldo % 8 ||
          hidden % 8 || mt < mb || sidx < 0)
        return fail(h, YPK_ERR_INVALID, "task %d: ALLREDUCE shape", ti);
      if (!h->arena) return fail(h, YPK_ERR_STATE, "ALLREDUCE needs ypk_comm_init first");
      need[2] = rows(ldo, mb, col0 + ncols); align[2] = 16; required[2] = true;
      if (in.flags & YPK_F_LL_IN) {
        // partials arrive as flagged words pushed by the producing LINEAR tasks
        if (!(in.flags & YPK_F_LL_OUT) || mt != h->cfg.max_num_batched_tokens || ldo != hidden)
          return fail(h, YPK_ERR_INVALID, "task %d: flagged-word ALLREDUCE shape", ti);
        need[1] = uint64_t(world) * mt * hidden * 4; align[1] = 16; required[1] = true;
        need[7] = uint64_t(mt) * ldo * 4; align[7] = 8; required[7] = true;
        break;
      }
      if (a[10] < 1 || a[6] < 0 || a[6] >= a[10])
        return fail(h, YPK_ERR_INVALID, "task %d: ALLREDUCE is number %d of %d in the iteration", ti,
                    a[6], a[10]);
      need[0] = rows(ldi, mb, col0 + ncols); align[0] = 16; required[0] = true;
      need[1] = uint64_t(2) * world * mt * hidden * 2; align[1] = 16; required[1] = true;
      need[3] = uint64_t(sidx + 1) * 8; align[3] = 8; required[3] = true;
      break;
    }
    case YPK_TASK_RMSNORM: {
      const int K = a[0], ldx = a[3], ldo = a[4];
      if (K <= 0) return fail(h, YPK_ERR_INVALID, "task %d: RMSNORM K", ti);
      need[0] = rows(ldx, mb, K); align[0] = 2; required[0] = true;
      if (in.ptr[1]) { need[1] = uint64_t(K) * 2; align[1] = 2; }
      need[2] = rows(ldo, mb, K); align[2] = 2; required[2] = true;
      break;
    }
    case YPK_TASK_SILU_MUL: {
      const int col0 = a[0], ncols = a[1], gs = a[2], ldi = a[3], ldo = a[4];
      if (gs <= 0 || ncols <= 0) return fail(h, YPK_ERR_INVALID, "task %d: SILU_MUL shape", ti);
      need[0] = rows(ldi, mb, 2 * (col0 + ncols)); align[0] = 2; required[0] = true;
      need[1] = rows(ldo, mb, col0 + ncols); align[1] = 2; required[1] = true;
      break;
    }
    default:
      return fail(h, YPK_ERR_UNSUPPORTED, "task %d: task type %d is not built", ti, in.type);
  }
  for (int p = 0; p < YPK_TASK_NPTR; ++p) {
    if (!required[p] && in.ptr[p] == 0) {
      out->ptr[p] = 0;
      continue;
    }
    if (required[p] && in.ptr[p] == 0)
      return fail(h, YPK_ERR_INVALID, "task %d (type %d): operand %d is required", ti, in.type, p);
    int rc = resolve(h, ti, p, in.ptr[p], need[p], align[p], &out->ptr[p]);
    if (rc) return rc;
  }
  out->ptr_aux = 0;
  if (need_aux) {
    if (in.ptr_aux == 0)
      return fail(h, YPK_ERR_INVALID, "task %d (type %d): operand 8 is required", ti, in.type);
    int rc = resolve(h, ti, 8, in.ptr_aux, need_aux, align_aux, &out->ptr_aux);
    if (rc) return rc;
  } else if (in.ptr_aux != 0) {
    return fail(h, YPK_ERR_INVALID, "task %d (type %d): takes no ninth operand", ti, in.type);
  }
  if ((in.type == YPK_TASK_LINEAR && (in.flags & YPK_F_LL_PUSH)) ||
      (in.type == YPK_TASK_ARGMAX_REDUCE && (in.flags & YPK_F_LL_PUSH)) ||
      (in.type == YPK_TASK_ALLREDUCE && (in.flags & YPK_F_LL_IN))) {
    const int p = in.type == YPK_TASK_LINEAR ? 7 : in.type == YPK_TASK_ARGMAX_REDUCE ? 3 : 1;
    const uint64_t a0 = reinterpret_cast<uint64_t>(h->arena);
    if (!h->arena || out->ptr[p] < a0 || out->ptr[p] + need[p] > a0 + h->arena_bytes)
      return fail(h, YPK_ERR_INVALID, "task %d: the pushed flagged-word buffer is not in the symmetric arena",
                  ti);
  } else if (in.type == YPK_TASK_ALLREDUCE) {
    for (int p : {1, 3}) {
      const uint64_t a0 = reinterpret_cast<uint64_t>(h->arena);
      if (out->ptr[p] < a0 || out->ptr[p] + need[p] > a0 + h->arena_bytes)
        return fail(h, YPK_ERR_INVALID, "task %d: ALLREDUCE operand %d is not in the symmetric arena",
                    ti, p);
    }
  }
  if (in.dep_event >= h->num_events || in.trig_event >= h->num_events)
    return fail(h, YPK_ERR_INVALID, "task %d: event index out of range", ti);
  if (in.dep_event >= 0 && in.dep_count <= 0)
    return fail(h, YPK_ERR_INVALID, "task %d: dependency without a trigger count", ti);
  return YPK_OK;
}

// Rank-3 tiled tensor map over a KV cache [pages*page_size tokens][kv heads][128] bf16:
// box = 64 dims x 1 head x 64 tokens, 128-byte swizzle.
int encode_kv_tmap(ypk_handle *h, void *base, int hkv, CUtensorMap *out) {
  typedef CUresult (*EncodeFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                               const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                               const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static EncodeFn fn = nullptr;
  if (!fn) {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !p)
      return fail(h, YPK_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    fn = reinterpret_cast<EncodeFn>(p);
  }
  const cuuint64_t tokens = cuuint64_t(h->cfg.max_num_pages) * h->cfg.page_size;
  const cuuint64_t dims[3] = {cuuint64_t(kHeadDim), cuuint64_t(hkv), tokens};
  const cuuint64_t strides[2] = {cuuint64_t(kHeadDim) * 2, cuuint64_t(hkv) * kHeadDim * 2};
  const cuuint32_t box[3] = {64, 1, cuuint32_t(kKvTile)};
  const cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, base, dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(h, YPK_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d)", int(r));
  return YPK_OK;
}

// Rank-3 view {64 columns, rows, K / 64} of a row-major 16-bit weight [rows][ldw] for the
// tensor-core LINEAR path: box = one 128-byte k-block x 64 rows, 128-byte swizzle, so that a
// box lands in shared memory as [row][128 B] (eight 8-row core-matrix groups).
int encode_weight_tmap(ypk_handle *h, void *base, int rows, int K, int ldw, CUtensorMap *out) {
  typedef CUresult (*EncodeFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                               const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                               const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static EncodeFn fn = nullptr;
  if (!fn) {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !p)
      return fail(h, YPK_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    fn = reinterpret_cast<EncodeFn>(p);
  }
  const cuuint64_t dims[3] = {cuuint64_t(kUmmaKBlock), cuuint64_t(rows), cuuint64_t(K / kUmmaKBlock)};
  const cuuint64_t strides[2] = {cuuint64_t(ldw) * 2, cuuint64_t(kUmmaKBlock) * 2};
  const cuuint32_t box[3] = {cuuint32_t(kUmmaKBlock), cuuint32_t(kUmmaBoxRows), 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, base, dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(h, YPK_ERR_CUDA, "cuTensorMapEncodeTiled failed for a weight (%d)", int(r));
  return YPK_OK;
}

void free_graph(ypk_handle *h) {
  if (!h->host_only && h->d_tmaps) cudaFree(h->d_tmaps);
  h->d_tmaps = nullptr;
  h->num_tmaps = 0;
  h->tmap_keys.clear();
  if (!h->host_only) {
    if (h->d_tasks) cudaFree(h->d_tasks);
    if (h->d_queue) cudaFree(h->d_queue);
    if (h->d_queue_off) cudaFree(h->d_queue_off);
    if (h->d_events) cudaFree(h->d_events);
  }
  h->d_tasks = nullptr;
  h->d_queue = h->d_queue_off = nullptr;
  h->d_events = nullptr;
  h->graph_loaded = false;
}

}  // namespace

extern "C" {

int ypk_abi_version(void) { return YPK_ABI_VERSION; }

const char *ypk_last_error(const ypk_handle *h) { return h ? h->err.c_str() : g_err.c_str(); }

int ypk_create(const ypk_config *cfg, ypk_handle **out) {
  if (!cfg || !out) return fail(nullptr, YPK_ERR_INVALID, "ypk_create: null argument");
  if (cfg->abi_version != YPK_ABI_VERSION)
    return fail(nullptr, YPK_ERR_INVALID, "ypk_create: ABI version %d, library has %d",
                cfg->abi_version, YPK_ABI_VERSION);
  if (cfg->mode != 0 && cfg->mode != 1)
    return fail(nullptr, YPK_ERR_INVALID, "ypk_create: mode must be 0 or 1");
  if (cfg->world_size < 1 || cfg->rank < 0 || cfg->rank >= cfg->world_size)
    return fail(nullptr, YPK_ERR_INVALID, "ypk_create: rank %d of world %d", cfg->rank,
                cfg->world_size);
  if (cfg->mode == 1) {
    if (!cfg->step || !cfg->tokens || !cfg->input_tokens || !cfg->output_tokens ||
        !cfg->prompt_lengths || !cfg->qo_indptr || !cfg->paged_kv_indptr ||
        !cfg->paged_kv_indices || !cfg->paged_kv_last_page_len)
      return fail(nullptr, YPK_ERR_INVALID, "ypk_create: serving mode needs every meta tensor");
    if (cfg->max_seq_length <= 0 || cfg->max_num_batched_requests <= 0 ||
        cfg->max_num_batched_tokens <= 0 || cfg->max_num_batched_tokens > 0xffff ||
        cfg->max_num_pages <= 0 || cfg->page_size <= 0 || cfg->total_num_requests <= 0)
      return fail(nullptr, YPK_ERR_INVALID, "ypk_create: serving sizes must be positive");
  }
  ypk_handle *h = new ypk_handle();
  h->cfg = *cfg;
  if (const char *pol = getenv("YPK_TENSOR_CORE")) {
    h->umma_policy = !strcmp(pol, "always") ? 1 : !strcmp(pol, "never") ? 2 : 0;
  }
  if (h->cfg.wait_budget_ns == 0) h->cfg.wait_budget_ns = 2000000000ull;
  memset(&h->status, 0, sizeof h->status);
  h->status.fail_task = h->status.fail_event = h->status.fail_worker = -1;
  h->host_only = cfg->device < 0;
  if (h->host_only) {
    h->sm_count = 148;
    h->num_workers = cfg->num_workers > 0 ? cfg->num_workers : h->sm_count;
    *out = h;
    return YPK_OK;
  }
  cudaError_t e = cudaSetDevice(cfg->device);
  if (e != cudaSuccess) {
    int rc = fail(nullptr, YPK_ERR_CUDA, "cudaSetDevice(%d): %s", cfg->device,
                  cudaGetErrorString(e));
    delete h;
    return rc;
  }
  cudaDeviceProp prop;
  e = cudaGetDeviceProperties(&prop, cfg->device);
  if (e == cudaSuccess && prop.major != 10) {
    int rc = fail(nullptr, YPK_ERR_UNSUPPORTED,
                  "device %d is sm_%d%d; this library is built for sm_100a only", cfg->device,
                  prop.major, prop.minor);
    delete h;
    return rc;
  }
  const void *variants[4] = {(const void *)ypk_megakernel_decode,
                             (const void *)ypk_megakernel_decode_tp,
                             (const void *)ypk_megakernel_wide,
                             (const void *)ypk_megakernel_moe};
  int per_sm = 1 << 30;
  for (const void *k : variants) {
    int n = 0;
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e == cudaSuccess)
      e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, k, kBlockThreads, kSmemBytes);
    per_sm = std::min(per_sm, n);
  }
  if (e != cudaSuccess || per_sm < 1) {
    int rc = fail(nullptr, YPK_ERR_CUDA, "megakernel cannot be made resident: %s",
                  e != cudaSuccess ? cudaGetErrorString(e) : "0 blocks per SM");
    delete h;
    return rc;
  }
  h->sm_count = prop.multiProcessorCount;
  h->num_workers = cfg->num_workers > 0 ? cfg->num_workers : h->sm_count;
  if (h->num_workers > h->sm_count * per_sm) h->num_workers = h->sm_count * per_sm;
  if (cudaMalloc(&h->d_ctrl, kCtrlWords * 8) != cudaSuccess ||
      cudaMemset(h->d_ctrl, 0, kCtrlWords * 8) != cudaSuccess) {
    int rc = fail(nullptr, YPK_ERR_CUDA, "control block allocation failed");
    delete h;
    return rc;
  }
  if (cudaMalloc(&h->d_qtiles, std::max(1, cfg->max_num_batched_tokens) * 4) != cudaSuccess) {
    int rc = fail(nullptr, YPK_ERR_CUDA, "query-tile list allocation failed");
    ypk_destroy(h);
    return rc;
  }
  if (cfg->mode == 1) {
    const int MR = cfg->max_num_batched_requests, MP = cfg->max_num_pages;
    if (cudaMalloc(&h->d_request_ids, MR * 4) != cudaSuccess ||
        cudaMalloc(&h->d_page_queue, MP * 4) != cudaSuccess ||
        cudaMalloc(&h->d_kv_tmp, MP * 4) != cudaSuccess ||

        cudaMalloc(&h->d_bstate, 16) != cudaSuccess) {
      int rc = fail(nullptr, YPK_ERR_CUDA, "batcher state allocation failed");
      ypk_destroy(h);
      return rc;
    }
    int rc = ypk_reset(h);
    if (rc) {
      g_err = h->err;
      ypk_destroy(h);
      return rc;
    }
  }
  *out = h;
  return YPK_OK;
}

int ypk_destroy(ypk_handle *h) {
  if (!h) return YPK_OK;
  if (!h->host_only) {
    cudaSetDevice(h->cfg.device);
    if (h->in_flight) cudaStreamSynchronize(h->stream);
  }
  free_graph(h);
  for (auto &s : h->slots) release_slot(h, s);
  if (!h->host_only) {
    for (int p = 0; p < 8; ++p)
      if (h->peer_arena[p] && p != h->cfg.rank) cudaIpcCloseMemHandle(h->peer_arena[p]);
    if (h->arena) cudaFree(h->arena);
    if (h->d_ctrl) cudaFree(h->d_ctrl);
    if (h->d_request_ids) cudaFree(h->d_request_ids);
    if (h->d_page_queue) cudaFree(h->d_page_queue);
    if (h->d_kv_tmp) cudaFree(h->d_kv_tmp);
    if (h->d_qtiles) cudaFree(h->d_qtiles);
    if (h->d_bstate) cudaFree(h->d_bstate);
  }
  delete h;
  return YPK_OK;
}

int ypk_bind_tensor(ypk_handle *h, int32_t slot, const char *name, void *dev_ptr,
                    uint64_t bytes) {
  if (!h) return fail(nullptr, YPK_ERR_INVALID, "null handle");
  if (!dev_ptr || bytes == 0) return fail(h, YPK_ERR_INVALID, "bind_tensor: empty tensor");
  Slot *s = get_slot(h, slot, true);
  if (!s) return fail(h, YPK_ERR_INVALID, "bind_tensor: bad slot %d", slot);
  release_slot(h, *s);
  s->ptr = dev_ptr;
  s->bytes = bytes;
  s->used = true;
  s->name = name ? name : "";
  return YPK_OK;
}

int ypk_alloc_tensor(ypk_handle *h, int32_t slot, const char *name, uint64_t bytes) {
  if (!h) return fail(nullptr, YPK_ERR_INVALID, "null handle");
  if (bytes == 0) return fail(h, YPK_ERR_INVALID, "alloc_tensor: zero bytes");
  Slot *s = get_slot(h, slot, true);
  if (!s) return fail(h, YPK_ERR_INVALID, "alloc_tensor: bad slot %d", slot);
  release_slot(h, *s);
  if (h->host_only) {
    // distinct, 256-byte aligned fake addresses so that alignment checks still mean something
    static uint64_t next_fake = 0x100000000ull;
    s->ptr = reinterpret_cast<void *>(next_fake);
    next_fake += (bytes + 255) / 256 * 256;
  } else {
    CUDA_TRY(h, cudaSetDevice(h->cfg.device));
    CUDA_TRY(h, cudaMalloc(&s->ptr, bytes));
    CUDA_TRY(h, cudaMemset(s->ptr, 0, bytes));
    s->owned = true;
  }
  s->bytes = bytes;
  s->used = true;
  s->name = name ? name : "";
  return YPK_OK;
}

int ypk_shuffle_tensor(ypk_handle *h, int32_t dst_slot, const char *name, int32_t n_src,
                       const int32_t *src_slots, const int32_t *rows, const int32_t *gran,
                       uint64_t row_bytes) {
  if (!h) return fail(nullptr, YPK_ERR_INVALID, "null handle");
  if (n_src < 1 || n_src > 8 || !src_slots || !rows || !gran || row_bytes == 0)
    return fail(h, YPK_ERR_INVALID, "shuffle_tensor: bad arguments");
  int64_t total_rows = 0, block_rows = 0, groups = -1;
  for (int i = 0; i < n_src; ++i) {
    Slot *s = get_slot(h, src_slots[i], false);
    if (!s || !s->used) return fail(h, YPK_ERR_INVALID, "shuffle_tensor: source %d unbound", i);
    if (rows[i] <= 0 || gran[i] <= 0 || rows[i] % gran[i])
      return fail(h, YPK_ERR_INVALID, "shuffle_tensor: rows %d not a multiple of granule %d",
                  rows[i], gran[i]);
    if (uint64_t(rows[i]) * row_bytes > s->bytes)
      return fail(h, YPK_ERR_INVALID, "shuffle_tensor: source %d smaller than rows*row_bytes", i);
    const int64_t g = rows[i] / gran[i];
    if (groups >= 0 && g != groups)
      return fail(h, YPK_ERR_INVALID, "shuffle_tensor: sources disagree on the group count");
    groups = g;
    total_rows += rows[i];
    block_rows += gran[i];
  }
  int rc = ypk_alloc_tensor(h, dst_slot, name, uint64_t(total_rows) * row_bytes);
  if (rc) return rc;
  if (h->host_only) return YPK_OK;
  Slot *d = get_slot(h, dst_slot, false);
  int64_t row_in_block = 0;
  for (int i = 0; i < n_src; ++i) {
    Slot *s = get_slot(h, src_slots[i], false);
    // block g of the destination, rows [row_in_block, row_in_block+gran[i]) <- source rows
    // [g*gran[i], (g+1)*gran[i]): one strided 2-D copy per source.
    CUDA_TRY(h, cudaMemcpy2D(static_cast<char *>(d->ptr) + row_in_block * row_bytes,
                             size_t(block_rows) * row_bytes, s->ptr, size_t(gran[i]) * row_bytes,
                             size_t(gran[i]) * row_bytes, size_t(groups),
                             cudaMemcpyDeviceToDevice));
    row_in_block += gran[i];
  }
  return YPK_OK;
}

int ypk_comm_init(ypk_handle *h, uint64_t arena_bytes) {
  if (!h) return fail(nullptr, YPK_ERR_INVALID, "null handle");
  if (h->arena) return fail(h, YPK_ERR_STATE, "comm_init called twice");
  if (h->cfg.world_size < 2 || h->cfg.world_size > 8)
    return fail(h, YPK_ERR_UNSUPPORTED, "tensor parallelism is built for 2..8 ranks (got %d)",
                h->cfg.world_size);
  if (arena_bytes == 0) return fail(h, YPK_ERR_INVALID, "comm_init: empty arena");
  arena_bytes = (arena_bytes + 255) / 256 * 256;
  if (h->host_only) {
    h->arena = reinterpret_cast<char *>(0x7000000000ull);
  } else {
    CUDA_TRY(h, cudaSetDevice(h->cfg.device));
    CUDA_TRY(h, cudaMalloc(&h->arena, arena_bytes));
    CUDA_TRY(h, cudaMemset(h->arena, 0, arena_bytes));   // counters start at zero
  }
  h->arena_bytes = arena_bytes;
  h->arena_used = 0;
  h->peer_arena[h->cfg.rank] = h->arena;
  return YPK_OK;
}

int ypk_alloc_symmetric(ypk_handle *h, int32_t slot, const char *name, uint64_t bytes) {
  if (!h) return fail(nullptr, YPK_ERR_INVALID, "null handle");
  if (!h->arena) return fail(h, YPK_ERR_STATE, "alloc_symmetric before comm_init");
  if (bytes == 0) return fail(h, YPK_ERR_INVALID, "alloc_symmetric: zero bytes");
  const uint64_t off = (h->arena_used + 255) / 256 * 256;
  if (off + bytes > h->arena_bytes)
    return fail(h, YPK_ERR_INVALID, "alloc_symmetric: arena of %llu bytes is full",
                (unsigned long long)h->arena_bytes);
  Slot *s = get_slot(h, slot, true);
  if (!s) return fail(h, YPK_ERR_INVALID, "alloc_symmetric: bad slot %d", slot);
  release_slot(h, *s);
  s->ptr = h->arena + off;
  s->bytes = bytes;
  s->used = true;
  s->owned = false;   // lives and dies with the arena
  s->name = name ? name : "";
  h->arena_used = off + bytes;
  return YPK_OK;
}

int ypk_comm_export(ypk_handle *h, void *handle_out) {
  if (!h || !handle_out) return fail(h, YPK_ERR_INVALID, "comm_export: null argument");
  if (!h->arena) return fail(h, YPK_ERR_STATE, "comm_export before comm_init");
  static_assert(sizeof(cudaIpcMemHandle_t) == YPK_IPC_HANDLE_BYTES, "IPC handle size");
  memset(handle_out, 0, YPK_IPC_HANDLE_BYTES);
  if (h->host_only) return YPK_OK;
  CUDA_TRY(h, cudaSetDevice(h->cfg.device));
  cudaIpcMemHandle_t ipc;
  CUDA_TRY(h, cudaIpcGetMemHandle(&ipc, h->arena));
  memcpy(handle_out, &ipc, sizeof ipc);
  return YPK_OK;
}

int ypk_comm_import(ypk_handle *h, int32_t peer_rank, const void *handle) {
  if (!h || !handle) return fail(h, YPK_ERR_INVALID, "comm_import: null argument");
  if (!h->arena) return fail(h, YPK_ERR_STATE, "comm_import before comm_init");
  if (peer_rank < 0 || peer_rank >= h->cfg.world_size || peer_rank == h->cfg.rank)
    return fail(h, YPK_ERR_INVALID, "comm_import: peer %d of world %d (own rank %d)", peer_rank,
                h->cfg.world_size, h->cfg.rank);
  if (h->peer_arena[peer_rank]) return fail(h, YPK_ERR_STATE, "peer %d imported twice", peer_rank);
  if (h->host_only) {
    h->peer_arena[peer_rank] = reinterpret_cast<char *>(0x7100000000ull + (uint64_t(peer_rank) << 32));
    return YPK_OK;
  }
  CUDA_TRY(h, cudaSetDevice(h->cfg.device));
  cudaIpcMemHandle_t ipc;
  memcpy(&ipc, handle, sizeof ipc);
  void *p = nullptr;
  CUDA_TRY(h, cudaIpcOpenMemHandle(&p, ipc, cudaIpcMemLazyEnablePeerAccess));
  h->peer_arena[peer_rank] = static_cast<char *>(p);
  return YPK_OK;
}

int ypk_tensor_ptr(ypk_handle *h, int32_t slot, void **dev_ptr, uint64_t *bytes) {
  if (!h) return fail(nullptr, YPK_ERR_INVALID, "null handle");
  Slot *s = get_slot(h, slot, false);
  if (!s || !s->used) return fail(h, YPK_ERR_INVALID, "tensor_ptr: slot %d unbound", slot);
  if (dev_ptr) *dev_ptr = s->ptr;
  if (bytes) *bytes = s->bytes;
  return YPK_OK;
}

int ypk_read_tensor(ypk_handle *h, int32_t slot, uint64_t byte_off, void *dst_dev_ptr,
                    uint64_t bytes) {
  if (!h) return fail(nullptr, YPK_ERR_INVALID, "null handle");
  if (h->host_only) return fail(h, YPK_ERR_STATE, "host-only handle has no device memory");
  Slot *s = get_slot(h, slot, false);
  if (!s || !s->used) return fail(h, YPK_ERR_INVALID, "read_tensor: slot %d unbound", slot);
  if (!dst_dev_ptr || byte_off + bytes > s->bytes)
    return fail(h, YPK_ERR_INVALID, "read_tensor: range outside tensor '%s'", s->name.c_str());
  CUDA_TRY(h, cudaSetDevice(h->cfg.device));
  CUDA_TRY(h, cudaMemcpy(dst_dev_ptr, static_cast<char *>(s->ptr) + byte_off, bytes,
                         cudaMemcpyDeviceToDevice));
  return YPK_OK;
}

int ypk_load_graph(ypk_handle *h, const ypk_task *tasks, int32_t num_tasks, int32_t num_events,
                   const int32_t *queue, const int32_t *queue_off, int32_t num_queues) {
  if (!h) return fail(nullptr, YPK_ERR_INVALID, "null handle");
  if (h->in_flight) return fail(h, YPK_ERR_STATE, "load_graph while a launch is in flight");
  if (!tasks || num_tasks <= 0 || num_events < 0 || !queue || !queue_off || num_queues <= 0)
    return fail(h, YPK_ERR_INVALID, "load_graph: bad arguments");
  if (num_queues > h->num_workers)
    return fail(h, YPK_ERR_INVALID, "load_graph: %d queues for %d workers", num_queues,
                h->num_workers);
  if (num_tasks > 0xfffff) return fail(h, YPK_ERR_UNSUPPORTED, "load_graph: too many tasks");
  h->num_events = num_events;
  if (queue_off[0] != 0 || queue_off[num_queues] != num_tasks)
    return fail(h, YPK_ERR_INVALID, "load_graph: queues must cover every task exactly once");
  std::vector<char> seen(size_t(num_tasks), 0);
  for (int w = 0; w < num_queues; ++w) {
    if (queue_off[w + 1] < queue_off[w])
      return fail(h, YPK_ERR_INVALID, "load_graph: queue offsets must not decrease");
    int prev = -1;
    for (int q = queue_off[w]; q < queue_off[w + 1]; ++q) {
      const int ti = queue[q];
      if (ti < 0 || ti >= num_tasks || seen[size_t(ti)])
        return fail(h, YPK_ERR_INVALID, "load_graph: task %d queued twice or out of range", ti);
      // Tasks are numbered in dependency order; a queue that runs them out of order
      // can wait on an event that its own later task has to produce.
      if (ti < prev)
        return fail(h, YPK_ERR_INVALID, "load_graph: queue %d is not in task order", w);
      prev = ti;
      seen[size_t(ti)] = 1;
    }
  }
  h->max_new_tokens = h->attn_chunk = kMaxNewTokens;
  h->attn_plain = h->attn_qtiles = false;
  h->spec_len = 0;
  h->has_moe = false;
  std::vector<ypk_task> resolved(static_cast<size_t>(num_tasks));
  std::vector<int> trig_count(size_t(num_events), 0), last_trig(size_t(num_events), -1);
  for (int i = 0; i < num_tasks; ++i) {
    int rc = check_task(h, i, tasks[i], &resolved[size_t(i)]);
    if (rc) return rc;
    if (tasks[i].trig_event >= 0) {
      trig_count[size_t(tasks[i].trig_event)]++;
      last_trig[size_t(tasks[i].trig_event)] = i;
    }
  }
  if (h->attn_plain && h->attn_qtiles)
    return fail(h, YPK_ERR_INVALID,
                "ATTENTION tasks over request slots and over query tiles in one graph");
  // A request may bring more new tokens than one ATTENTION task takes only if every such task
  // reads the query-tile list.
  h->max_new_tokens = h->attn_qtiles ? std::min(kMaxNewKeys, h->cfg.max_num_batched_tokens)
                                     : h->attn_chunk;
  for (int i = 0; i < num_tasks; ++i) {
    const ypk_task &t = tasks[i];
    if (t.dep_event < 0) continue;
    if (trig_count[size_t(t.dep_event)] != t.dep_count)
      return fail(h, YPK_ERR_INVALID,
                  "task %d waits for %d triggers of event %d but %d tasks trigger it", i,
                  t.dep_count, t.dep_event, trig_count[size_t(t.dep_event)]);
    // every producer of the awaited event must come earlier in task order
    if (last_trig[size_t(t.dep_event)] >= i)
      return fail(h, YPK_ERR_INVALID, "task %d waits for event %d that task %d triggers", i,
                  t.dep_event, last_trig[size_t(t.dep_event)]);
  }
  // tensor maps for the K / V caches the attention tasks read (one per distinct tensor)
  std::vector<uint64_t> keys;
  std::vector<int> key_hkv;
  for (int i = 0; i < num_tasks; ++i) {
    ypk_task &t = resolved[size_t(i)];
    if (t.type != YPK_TASK_ATTENTION) continue;
    for (int which = 0; which < 2; ++which) {
      const uint64_t addr = t.ptr[1 + which];
      size_t k = 0;
      while (k < keys.size() && keys[k] != addr) ++k;
      if (k == keys.size()) {
        keys.push_back(addr);
        key_hkv.push_back(t.iarg[5]);
      } else if (key_hkv[k] != t.iarg[5]) {
        return fail(h, YPK_ERR_INVALID, "task %d: cache tensor used with two head counts", i);
      }
      t.iarg[9 + which] = int(k);
    }
  }
  // tensor maps for the weights of LINEAR tasks that can take the tensor-core path (more
  // than 8 tokens in flight): one per distinct (weight, K, row pitch)
  struct WeightKey { uint64_t addr; int K, ldw, rows; };
  std::vector<WeightKey> wkeys;
  const bool umma_possible = h->cfg.max_num_batched_tokens > kMaxBatch;
  for (int i = 0; i < num_tasks; ++i) {
    ypk_task &t = resolved[size_t(i)];
    if (t.type != YPK_TASK_LINEAR) continue;
    t.iarg[9] = -1;
    if (t.flags & YPK_F_MOE) continue;   // the expert's rows are picked at run time: GEMV paths only
    const int K = t.iarg[0], nrows = t.iarg[2], ldw = t.iarg[4];
    const bool silu_ok = !(t.flags & YPK_F_SILU_MUL) || (t.iarg[1] % (2 * kSiluGran) == 0);
    if (!umma_possible || K % kUmmaKBlock != 0 || nrows > kMaxAccRows || ldw % 8 != 0 ||
        (t.ptr[1] & 15u) != 0 || t.iarg[3] % 8 != 0 || (t.ptr[0] & 15u) != 0 || !silu_ok)
      continue;
    size_t k = 0;
    while (k < wkeys.size() &&
           !(wkeys[k].addr == t.ptr[1] && wkeys[k].K == K && wkeys[k].ldw == ldw))
      ++k;
    if (k == wkeys.size()) wkeys.push_back({t.ptr[1], K, ldw, 0});
    wkeys[k].rows = std::max(wkeys[k].rows, t.iarg[1] + nrows);
    t.iarg[9] = int(keys.size() + k);
  }
  // ... and for their activations (same kind of view; every row the graph can see).  The
  // index goes where narrow graphs keep a flagged-word tag, which wide graphs do not have.
  std::vector<WeightKey> xkeys;
  for (int i = 0; i < num_tasks && umma_possible; ++i) {
    ypk_task &t = resolved[size_t(i)];
    if (t.type != YPK_TASK_LINEAR || (t.flags & YPK_F_MOE)) continue;
    t.iarg[11] = -1;
    if (t.iarg[9] < 0 || (t.flags & (YPK_F_NORM | YPK_F_NORM_NOWEIGHT))) continue;
    const int K = t.iarg[0], ldx = t.iarg[3];
    size_t k = 0;
    while (k < xkeys.size() && !(xkeys[k].addr == t.ptr[0] && xkeys[k].K == K && xkeys[k].ldw == ldx))
      ++k;
    if (k == xkeys.size()) xkeys.push_back({t.ptr[0], K, ldx, h->cfg.max_num_batched_tokens});
    t.iarg[11] = int(keys.size() + wkeys.size() + k);
  }
  for (int i = 0; i < num_tasks; ++i) {
    const ypk_task &t = resolved[size_t(i)];
    if (t.type == YPK_TASK_LINEAR && (t.flags & (YPK_F_NORM_OUT | YPK_F_NORM_PRE)) &&
        (!umma_possible || t.iarg[9] < 0 || t.iarg[11] < 0))
      return fail(h, YPK_ERR_UNSUPPORTED,
                  "task %d: a norm carried across operators exists on the tensor-core path only, "
                  "which this task's shape or alignment rules out", i);
  }
  h->end_event = tasks[num_tasks - 1].trig_event;
  h->end_count = h->end_event >= 0 ? trig_count[size_t(h->end_event)] : 0;

  free_graph(h);
  h->use_tmem = !wkeys.empty();
  if (!(keys.empty() && wkeys.empty()) && !h->host_only) {
    std::vector<CUtensorMap> maps(keys.size() + wkeys.size() + xkeys.size());
    for (size_t k = 0; k < keys.size(); ++k) {
      int rc = encode_kv_tmap(h, reinterpret_cast<void *>(keys[k]), key_hkv[k], &maps[k]);
      if (rc) return rc;
    }
    for (size_t k = 0; k < wkeys.size(); ++k) {
      int rc = encode_weight_tmap(h, reinterpret_cast<void *>(wkeys[k].addr), wkeys[k].rows,
                                  wkeys[k].K, wkeys[k].ldw, &maps[keys.size() + k]);
      if (rc) return rc;
    }
    for (size_t k = 0; k < xkeys.size(); ++k) {
      int rc = encode_weight_tmap(h, reinterpret_cast<void *>(xkeys[k].addr), xkeys[k].rows, xkeys[k].K,
                                  xkeys[k].ldw, &maps[keys.size() + wkeys.size() + k]);
      if (rc) return rc;
    }
    CUDA_TRY(h, cudaSetDevice(h->cfg.device));
    CUDA_TRY(h, cudaMalloc(&h->d_tmaps, sizeof(CUtensorMap) * maps.size()));
    CUDA_TRY(h, cudaMemcpy(h->d_tmaps, maps.data(), sizeof(CUtensorMap) * maps.size(),
                           cudaMemcpyHostToDevice));
    h->num_tmaps = int(maps.size());
  }
  h->tmap_keys = keys;
  h->tasks.swap(resolved);
  h->queue.assign(queue, queue + num_tasks);
  h->queue_off.assign(queue_off, queue_off + num_queues + 1);
  // workers beyond num_queues get empty queues
  while (int(h->queue_off.size()) < h->num_workers + 1) h->queue_off.push_back(num_tasks);
  if (!h->host_only) {
    CUDA_TRY(h, cudaSetDevice(h->cfg.device));
    CUDA_TRY(h, cudaMalloc(&h->d_tasks, sizeof(ypk_task) * size_t(num_tasks)));
    CUDA_TRY(h, cudaMalloc(&h->d_queue, 4 * size_t(num_tasks)));
    CUDA_TRY(h, cudaMalloc(&h->d_queue_off, 4 * h->queue_off.size()));
    CUDA_TRY(h, cudaMalloc(&h->d_events, 8 * size_t(num_events + 1)));
    CUDA_TRY(h, cudaMemcpy(h->d_tasks, h->tasks.data(), sizeof(ypk_task) * size_t(num_tasks),
                           cudaMemcpyHostToDevice));
    CUDA_TRY(h, cudaMemcpy(h->d_queue, h->queue.data(), 4 * size_t(num_tasks),
                           cudaMemcpyHostToDevice));
    CUDA_TRY(h, cudaMemcpy(h->d_queue_off, h->queue_off.data(), 4 * h->queue_off.size(),
                           cudaMemcpyHostToDevice));
    CUDA_TRY(h, cudaMemset(h->d_events, 0, 8 * size_t(num_events + 1)));
  }
  h->ar_epoch += static_cast<unsigned long long>(h->base_iter);
  h->ll_epoch += static_cast<unsigned long long>(h->base_iter) + 1;
  h->base_iter = 0;
  h->wide_iters = 0;
  h->resume_pending = false;
  h->pending_tokens = 0;
  h->graph_loaded = true;
  return YPK_OK;
}

int ypk_reset(ypk_handle *h) {
  if (!h) return fail(nullptr, YPK_ERR_INVALID, "null handle");
  if (h->in_flight) return fail(h, YPK_ERR_STATE, "reset while a launch is in flight");
  if (h->status.error && h->arena)
    // After an abort the ranks have stopped in different places: arrival counters in the
    // peers' arenas hold part of the aborted iteration and the ranks' tag epochs no longer
    // agree.  Nothing on one rank can repair that.
    return fail(h, YPK_ERR_STATE,
                "a tensor-parallel handle cannot be reset after a device error: destroy the "
                "handles of all ranks and create them again");
  h->ar_epoch += static_cast<unsigned long long>(h->base_iter);
  // step over every iteration an aborted launch may have written tags for
  h->ll_epoch += static_cast<unsigned long long>(std::max(h->base_iter, h->abort_iters)) + 1;
  h->abort_iters = 0;
  h->base_iter = 0;
  h->wide_iters = 0;
  h->resume_pending = false;
  h->pending_tokens = 0;
  h->finished = false;
  memset(&h->status, 0, sizeof h->status);
  h->status.fail_task = h->status.fail_event = h->status.fail_worker = -1;
  if (h->host_only) return YPK_OK;
  CUDA_TRY(h, cudaSetDevice(h->cfg.device));
  CUDA_TRY(h, cudaMemset(h->d_ctrl, 0, kCtrlWords * 8));
  if (h->d_events) CUDA_TRY(h, cudaMemset(h->d_events, 0, 8 * size_t(h->num_events + 1)));
  if (h->cfg.mode == 1) {
    const ypk_config &c = h->cfg;
    const int MR = c.max_num_batched_requests, MP = c.max_num_pages;
    CUDA_TRY(h, cudaMemset(c.step, 0, 4 * size_t(c.total_num_requests)));
    CUDA_TRY(h, cudaMemset(c.qo_indptr, 0, 4 * size_t(MR + 1)));
    CUDA_TRY(h, cudaMemset(c.paged_kv_indptr, 0, 4 * size_t(MR + 1)));
    CUDA_TRY(h, cudaMemset(h->d_request_ids, 0xff, 4 * size_t(MR)));
    std::vector<int> pages(static_cast<size_t>(MP));
    for (int i = 0; i < MP; ++i) pages[size_t(i)] = i;
    CUDA_TRY(h, cudaMemcpy(h->d_page_queue, pages.data(), 4 * size_t(MP), cudaMemcpyHostToDevice));
    const int bstate[4] = {0, 0, MP, 0};
    CUDA_TRY(h, cudaMemcpy(h->d_bstate, bstate, 16, cudaMemcpyHostToDevice));
  }
  return YPK_OK;
}

int ypk_launch_async(ypk_handle *h, void *stream, int32_t max_iterations, int32_t batch) {
  if (!h) return fail(nullptr, YPK_ERR_INVALID, "null handle");
  if (h->host_only) return fail(h, YPK_ERR_STATE, "host-only handle cannot launch");
  if (!h->graph_loaded) return fail(h, YPK_ERR_STATE, "launch before load_graph");
  if (h->in_flight) return fail(h, YPK_ERR_STATE, "a launch is already in flight");
  if (h->status.error) return fail(h, YPK_ERR_STATE, "handle is in a failed state; reset it");
  const ypk_config &c = h->cfg;
  if (c.mode == 0 && (batch < 1 || batch > (c.max_num_batched_tokens > 0 ? c.max_num_batched_tokens : 1)))
    return fail(h, YPK_ERR_INVALID, "launch: batch %d outside 1..max_num_batched_tokens", batch);
  if (c.mode == 1 && h->finished) return YPK_OK;  // nothing left to do
  CUDA_TRY(h, cudaSetDevice(c.device));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  Runtime rt;
  memset(&rt, 0, sizeof rt);
  rt.tasks = h->d_tasks;
  rt.queue = h->d_queue;
  rt.queue_off = h->d_queue_off;
  rt.events = h->d_events;
  rt.ctrl = h->d_ctrl;
  rt.step = static_cast<int *>(c.step);
  rt.tokens = static_cast<long long *>(c.tokens);
  rt.input_tokens = static_cast<long long *>(c.input_tokens);
  rt.output_tokens = static_cast<long long *>(c.output_tokens);
  rt.prompt_len = static_cast<int *>(c.prompt_lengths);
  rt.num_new = static_cast<int *>(c.num_new_tokens);
  rt.spec_len = h->spec_len;
  rt.qo_indptr = static_cast<int *>(c.qo_indptr);
  rt.kv_indptr = static_cast<int *>(c.paged_kv_indptr);
  rt.kv_indices = static_cast<int *>(c.paged_kv_indices);
  rt.kv_last_len = static_cast<int *>(c.paged_kv_last_page_len);
  rt.request_ids = h->d_request_ids;
  rt.page_queue = h->d_page_queue;
  rt.kv_tmp = h->d_kv_tmp;
  rt.qtiles = h->attn_qtiles ? h->d_qtiles : nullptr;
  rt.attn_chunk = h->attn_chunk;
  rt.pause_below = h->pause_below;
  rt.bstate = h->d_bstate;
  rt.eos = c.eos_token_id;
  rt.base_iter = h->base_iter;
  rt.base_wide = h->wide_iters;
  rt.budget_ns = c.wait_budget_ns;
  rt.mode = c.mode;
  rt.max_seq = c.max_seq_length;
  rt.max_req = c.max_num_batched_requests;
  rt.max_tok = c.max_num_batched_tokens;
  rt.max_pages = c.max_num_pages;
  rt.page_size = c.page_size;
  rt.total_req = c.total_num_requests;
  rt.max_iters = max_iterations;
  rt.fixed_batch = batch;
  rt.resume_pending = h->resume_pending ? 1 : 0;
  rt.rank = c.rank;
  rt.world = c.world_size;
  rt.max_new_tokens = h->max_new_tokens;
  rt.end_event = h->end_event;
  rt.end_count = h->end_count;
  rt.tmaps = h->d_tmaps;
  rt.num_tmaps = h->d_tmaps ? h->num_tmaps : 0;
  rt.use_tmem = h->use_tmem ? 1 : 0;
  rt.umma_policy = h->umma_policy;
  { const char *d = getenv("YPK_UMMA_DEPTH"); rt.umma_depth = d ? std::min(5, std::max(1, atoi(d))) : 4; }
  rt.ll_epoch = h->ll_epoch;
  { const char *pf = getenv("YPK_LL_PUSH_FENCE"); rt.ll_push_fence = (pf && pf[0] == '1') ? 1 : 0; }
  rt.ar_epoch = h->ar_epoch;
  for (int p = 0; p < 8; ++p) rt.arena[p] = h->peer_arena[p];
  if (h->arena)
    for (int p = 0; p < c.world_size; ++p)
      if (!h->peer_arena[p]) return fail(h, YPK_ERR_STATE, "launch before peer %d was imported", p);
  rt.prof = nullptr;
  rt.prof_stride = 0;
  if (c.profiler_buffer) {
    int longest = 0;
    for (size_t w = 0; w + 1 < h->queue_off.size(); ++w)
      longest = std::max(longest, h->queue_off[w + 1] - h->queue_off[w]);
    const uint64_t need = uint64_t(h->num_workers) * longest * 64u;
    if (need > c.profiler_bytes)
      return fail(h, YPK_ERR_INVALID, "profiler buffer has %llu bytes, the graph needs %llu",
                  (unsigned long long)c.profiler_bytes, (unsigned long long)need);
    rt.prof = static_cast<unsigned long long *>(c.profiler_buffer);
    rt.prof_stride = longest;
  }
  if (c.mode == 0 && h->attn_qtiles) {
    // One-pass graphs have no batcher: the query-tile list is made here from the caller's
    // qo_indptr (a blocking read of max_requests + 1 integers; serving launches never do this).
    const int MR = c.max_num_batched_requests, MT = c.max_num_batched_tokens;
    std::vector<int> qo(size_t(MR) + 1), tiles(size_t(std::max(1, MT)), -1);
    CUDA_TRY(h, cudaStreamSynchronize(st));
    CUDA_TRY(h, cudaMemcpy(qo.data(), c.qo_indptr, 4 * qo.size(), cudaMemcpyDeviceToHost));
    int n = 0;
    for (int i = 0; i < MR && n < MT; ++i)
      for (int t0 = 0, T = qo[size_t(i) + 1] - qo[size_t(i)]; t0 < T && n < MT; t0 += h->attn_chunk)
        tiles[size_t(n++)] = i | (t0 << 12) | (std::min(h->attn_chunk, T - t0) << 20);
    CUDA_TRY(h, cudaMemcpy(h->d_qtiles, tiles.data(), 4 * tiles.size(), cudaMemcpyHostToDevice));
  }
  // The control word a new launch starts from: last completed iteration, stopped, and
  // the size of the batch that is waiting (if any).
  const unsigned long long words[kCtrlWords] = {
      (static_cast<unsigned long long>(h->base_iter) << 32) |
          (static_cast<unsigned long long>(kStateStop) << 16) |
          static_cast<unsigned long long>(h->pending_tokens),
      0ull, 0ull, 0ull, 0ull, 0ull, 0ull, 0ull};
  CUDA_TRY(h, cudaMemcpyAsync(h->d_ctrl, words, sizeof words, cudaMemcpyHostToDevice, st));
  void *args[] = {&rt};
  // Workers wait on each other, so they must all be resident: a cooperative launch
  // refuses to start otherwise instead of deadlocking.
  // The variant that carries no code this configuration cannot run (see ypk_megakernel).
  const bool wide = c.max_num_batched_tokens > kMaxBatch, tp = c.world_size > 1;
  const void *kernel = h->has_moe ? (const void *)ypk_megakernel_moe
                       : wide     ? (const void *)ypk_megakernel_wide
                       : tp       ? (const void *)ypk_megakernel_decode_tp
                                  : (const void *)ypk_megakernel_decode;
  CUDA_TRY(h, cudaLaunchCooperativeKernel(kernel, dim3(h->num_workers),
                                          dim3(kBlockThreads), args, kSmemBytes, st));
  h->stream = st;
  h->in_flight = true;
  return YPK_OK;
}

int ypk_wait(ypk_handle *h) {
  if (!h) return fail(nullptr, YPK_ERR_INVALID, "null handle");
  if (!h->in_flight) return YPK_OK;
  CUDA_TRY(h, cudaSetDevice(h->cfg.device));
  cudaError_t e = cudaStreamSynchronize(h->stream);
  h->in_flight = false;
  if (e != cudaSuccess) {
    h->status.error = YPK_ERR_CUDA;
    return fail(h, YPK_ERR_CUDA, "megakernel failed: %s", cudaGetErrorString(e));
  }
  unsigned long long words[kCtrlWords];
  CUDA_TRY(h, cudaMemcpy(words, h->d_ctrl, sizeof words, cudaMemcpyDeviceToHost));
  h->status.tasks_executed = (int64_t)words[kCtrlTasksDone];
  h->wide_iters = (long long)words[kCtrlWideIters];
  h->status.tensor_core_tasks = (int64_t)words[kCtrlUmmaTasks];
  if (words[kCtrlAbort]) {
    const unsigned long long info = words[kCtrlFailInfo];
    h->status.error = -int(words[kCtrlAbort]);
    h->status.fail_worker = int(info >> 40);
    h->status.fail_task = int((info >> 20) & 0xfffff);
    int ev = int(info & 0xfffff);
    if (ev & 0x80000) ev |= ~0xfffff;  // sign-extend the 20-bit field
    h->status.fail_event = ev;
    // how far the aborted launch got: tags of flagged words up to there may sit in buffers
    h->abort_iters = (long long)(words[kCtrlPublished] >> 32);
    if (ev == -7)
      return fail(h, h->status.error,
                  "the KV page pool ran out: a running request needs a page and none of the %d "
                  "is free (max_num_pages is too small for max_num_batched_requests x "
                  "max_seq_length)", h->cfg.max_num_pages);
    return fail(h, h->status.error,
                "device wait timed out: worker %d, task %d, event %d (negative: -2 ring "
                "barrier, -3 iteration word, -5 all-reduce arrivals, -6 flagged word)",
                h->status.fail_worker, h->status.fail_task, h->status.fail_event);
  }
  if (h->cfg.mode == 0) {
    h->base_iter += 1;
    h->status.iterations = h->base_iter;
    return YPK_OK;
  }
  const unsigned long long w = words[kCtrlPublished];
  const long long pub_iter = (long long)(w >> 32);
  const int ntok = int(w & 0xffffull);
  h->base_iter = pub_iter - 1;  // the published iteration itself did not run
  h->pending_tokens = ntok;
  h->resume_pending = ntok > 0;
  h->finished = words[kCtrlFinished] != 0 || ntok == 0;
  h->status.iterations = h->base_iter;
  h->status.finished = h->finished ? 1 : 0;
  h->status.active_tokens = ntok;
  return YPK_OK;
}

int ypk_set_pause_below(ypk_handle *h, int32_t tokens) {
  if (!h) return fail(nullptr, YPK_ERR_INVALID, "null handle");
  if (h->in_flight) return fail(h, YPK_ERR_STATE, "set_pause_below while a launch is in flight");
  if (tokens < 0) return fail(h, YPK_ERR_INVALID, "set_pause_below: negative token count");
  h->pause_below = tokens;
  return YPK_OK;
}

int ypk_adopt_batch(ypk_handle *dst, ypk_handle *src) {
  if (!dst || !src) return fail(nullptr, YPK_ERR_INVALID, "null handle");
  if (dst == src) return fail(dst, YPK_ERR_INVALID, "adopt_batch: source and destination are one handle");
  if (dst->host_only || src->host_only) return fail(dst, YPK_ERR_STATE, "adopt_batch on a host-only handle");
  if (dst->in_flight || src->in_flight) return fail(dst, YPK_ERR_STATE, "adopt_batch while a launch is in flight");
  if (dst->status.error || src->status.error)
    return fail(dst, YPK_ERR_STATE, "adopt_batch: a handle is in a failed state");
  if (!dst->graph_loaded) return fail(dst, YPK_ERR_STATE, "adopt_batch before load_graph");
  const ypk_config &a = dst->cfg, &b = src->cfg;
  if (a.mode != 1 || b.mode != 1 || a.device != b.device ||
      a.max_num_batched_requests != b.max_num_batched_requests ||
      a.max_num_pages != b.max_num_pages || a.page_size != b.page_size ||
      a.max_seq_length != b.max_seq_length || a.total_num_requests != b.total_num_requests ||
      a.eos_token_id != b.eos_token_id || a.step != b.step || a.tokens != b.tokens ||
      a.input_tokens != b.input_tokens || a.output_tokens != b.output_tokens ||
      a.prompt_lengths != b.prompt_lengths || a.qo_indptr != b.qo_indptr ||
      a.paged_kv_indptr != b.paged_kv_indptr || a.paged_kv_indices != b.paged_kv_indices ||
      a.paged_kv_last_page_len != b.paged_kv_last_page_len)
    return fail(dst, YPK_ERR_INVALID,
                "adopt_batch: the two handles must serve the same requests through the same "
                "meta tensors, page pool and request slots");
  if (src->finished || !src->resume_pending) {
    // nothing is waiting: every request has retired
    dst->finished = true;
    dst->resume_pending = false;
    dst->pending_tokens = 0;
    dst->status.finished = 1;
    dst->status.active_tokens = 0;
    return YPK_OK;
  }
  // The waiting batch was formed under the source's limits; the destination's tasks must be
  // able to take it.  The token count bounds every request's share too.
  if (src->pending_tokens > a.max_num_batched_tokens ||
      (src->pending_tokens > dst->max_new_tokens && src->max_new_tokens > dst->max_new_tokens))
    return fail(dst, YPK_ERR_STATE,
                "adopt_batch: the waiting batch has %d tokens, this graph takes %d per "
                "iteration and %d per request", src->pending_tokens, a.max_num_batched_tokens,
                dst->max_new_tokens);
  CUDA_TRY(dst, cudaSetDevice(a.device));
  const size_t MR = size_t(a.max_num_batched_requests), MP = size_t(a.max_num_pages);
  CUDA_TRY(dst, cudaMemcpy(dst->d_request_ids, src->d_request_ids, 4 * MR, cudaMemcpyDeviceToDevice));
  CUDA_TRY(dst, cudaMemcpy(dst->d_page_queue, src->d_page_queue, 4 * MP, cudaMemcpyDeviceToDevice));
  CUDA_TRY(dst, cudaMemcpy(dst->d_bstate, src->d_bstate, 16, cudaMemcpyDeviceToDevice));
  dst->pending_tokens = src->pending_tokens;
  dst->resume_pending = true;
  dst->finished = false;
  dst->status.finished = 0;
  dst->status.active_tokens = src->pending_tokens;
  // the source has given its batch away: it runs again only after a reset
  src->resume_pending = false;
  src->pending_tokens = 0;
  src->finished = true;
  src->status.finished = 1;
  return YPK_OK;
}

int ypk_launch(ypk_handle *h, void *stream, int32_t max_iterations, int32_t batch) {
  int rc = ypk_launch_async(h, stream, max_iterations, batch);
  if (rc) return rc;
  return ypk_wait(h);
}

int ypk_argmax_noalloc(const void *logits_bf16, int32_t batch, int32_t vocab, int64_t ld,
                       int64_t *out_tokens, void *stream) {
  if (!logits_bf16 || !out_tokens)
    return fail(nullptr, YPK_ERR_INVALID, "argmax_noalloc: null logits or output");
  if (batch < 1 || batch > kNoAllocMaxBatch)
    return fail(nullptr, YPK_ERR_UNSUPPORTED,
                "argmax_noalloc: batch %d is outside 1..%d (the built-in scratch is fixed)", batch,
                kNoAllocMaxBatch);
  if (vocab < 1 || ld < vocab || ld > 0x7fffffff)
    return fail(nullptr, YPK_ERR_INVALID, "argmax_noalloc: vocab %d / row stride %lld", vocab,
                (long long)ld);
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64)
    return fail(nullptr, YPK_ERR_CUDA, "argmax_noalloc: no current device (%s)",
                cudaGetErrorString(e));
  // Set-up, once per device, with that device current: the device address of the array.
  static unsigned char *scratch_of[64] = {nullptr};
  if (!scratch_of[dev]) {
    void *p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess || !p)
      return fail(nullptr, YPK_ERR_CUDA, "argmax_noalloc: cudaGetSymbolAddress: %s",
                  cudaGetErrorString(e));
    scratch_of[dev] = static_cast<unsigned char *>(p);
  }
  unsigned char *scratch = scratch_of[dev];
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // the arrival counter has to start at zero even if an earlier call was cut short
  e = cudaMemsetAsync(scratch + kNoAllocCtrOff, 0, 256, st);
  if (e != cudaSuccess)
    return fail(nullptr, YPK_ERR_CUDA, "argmax_noalloc: clearing the counter: %s",
                cudaGetErrorString(e));
  argmax_noalloc_kernel<<<kNoAllocParts, kConsumerThreads, 0, st>>>(
      static_cast<const uint16_t *>(logits_bf16), batch, vocab, (long long)ld,
      reinterpret_cast<long long *>(out_tokens), scratch);
  e = cudaGetLastError();
  if (e != cudaSuccess)
    return fail(nullptr, YPK_ERR_CUDA, "argmax_noalloc: launch: %s", cudaGetErrorString(e));
  return YPK_OK;
}

int ypk_transpose_16bit(const void *src, void *dst, int32_t rows, int32_t cols, void *stream) {
  if (!src || !dst || rows <= 0 || cols <= 0 || rows % 8 || cols % 8)
    return fail(nullptr, YPK_ERR_INVALID, "transpose: %d x %d (multiples of 8, non-null)", rows, cols);
  dim3 grid((cols + 31) / 32, (rows + 31) / 32), block(32, 8);
  transpose16_kernel<<<grid, block, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint16_t *>(src), static_cast<uint16_t *>(dst), rows, cols);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(nullptr, YPK_ERR_CUDA, "transpose: %s", cudaGetErrorString(e));
  return YPK_OK;
}

int ypk_get_status(ypk_handle *h, ypk_status *out) {
  if (!h || !out) return fail(h, YPK_ERR_INVALID, "get_status: null argument");
  *out = h->status;
  return YPK_OK;
}

}  // extern "C"
