// Small tasks of the decode graph: embedding gather, arg-max sampling, stand-alone
// RMSNorm and SiLU*mul (used when a graph does not match the fused LINEAR forms), and the
// on-device continuous batcher that runs between iterations.
#pragma once
#include "device_common.cuh"
#include "ll_handoff.cuh"

namespace ypk {

// out[b, col0:col0+ncols] = table[ids[b], col0:col0+ncols]; an id outside [0, rows) gives
// zeros (tasks/ampere/embedding.cuh:42-70 reads whatever row the id names; a sampled id can
// lie in the zero-padded tail of the lm_head, beyond the embedding table).
__device__ __forceinline__ void embed_task(const ypk_task &t, int batch) {
  const long long *ids = reinterpret_cast<const long long *>(t.ptr[0]);
  const uint16_t *table = reinterpret_cast<const uint16_t *>(t.ptr[1]);
  uint16_t *out = reinterpret_cast<uint16_t *>(t.ptr[2]);
  const int col0 = t.iarg[1], ncols = t.iarg[2], ldt = t.iarg[3], ldo = t.iarg[4];
  const long long rows = t.iarg[5];
  const int vec = ncols / 8;
  for (int idx = threadIdx.x; idx < batch * vec; idx += kConsumerThreads) {
    const int b = idx / vec, c = (idx - b * vec) * 8 + col0;
    const long long id = __ldcg(ids + b);
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (id >= 0 && id < rows) v = __ldg(reinterpret_cast<const uint4 *>(table + size_t(id) * ldt + c));
    *reinterpret_cast<uint4 *>(out + size_t(b) * ldo + c) = v;
  }
}

// Per-chunk (max, first index) of bf16 logits (tasks/blackwell/argmax_sm100.cuh:78-114;
// ties resolve to the lowest index here, which is what torch.argmax does).
__device__ __forceinline__ void argmax_partial_task(const ypk_task &t, int batch) {
  const uint16_t *logits = reinterpret_cast<const uint16_t *>(t.ptr[0]);
  uint16_t *pval = reinterpret_cast<uint16_t *>(t.ptr[1]);
  long long *pidx = reinterpret_cast<long long *>(t.ptr[2]);
  const int col0 = t.iarg[0], ld = t.iarg[2], part = t.iarg[3], nparts = t.iarg[4];
  // iarg[5] != 0: only the first iarg[5] columns of a logits row are real vocabulary (the
  // rest is padding of the lm_head and must not be sampled); negative = none of them
  const int ncols = t.iarg[5] != 0 ? max(0, min(t.iarg[1], t.iarg[5] - col0)) : t.iarg[1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int b = warp; b < batch; b += kConsumerWarps) {
    const uint16_t *row = logits + size_t(b) * ld + col0;
    float best = -INFINITY;
    int bidx = 0x7fffffff;
    for (int c = lane; c < ncols; c += 32) {
      const float v = cvt_one<false>(__ldcg(row + c));
      if (v > best) {  // strict: the first (lowest) index of a lane wins
        best = v;
        bidx = c;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bidx, o);
      if (ov > best || (ov == best && oi < bidx)) {
        best = ov;
        bidx = oi;
      }
    }
    if (lane == 0) {
      pval[size_t(b) * nparts + part] = __bfloat16_as_ushort(__float2bfloat16_rn(best));
      pidx[size_t(b) * nparts + part] = bidx == 0x7fffffff ? col0 : col0 + bidx;
    }
  }
}

// Final reduction over the chunks (argmax_sm100.cuh:116-167), token id as int64.
// With YPK_F_LL_PUSH the logits are one rank's slice of a vocabulary split over the
// tensor-parallel ranks (iarg = {nparts, first vocabulary row of the slice, world, rank}):
// the slice's winner goes to every rank as two flagged words {value bits, tag}, {index, tag}
// into slot `rank` of ptr[3] = [world][max_tokens][2] words (symmetric arena), and every rank
// takes the best of the world slots, lowest index on ties, so all ranks sample the same token.
template <bool TP>
__device__ __forceinline__ bool argmax_reduce_task(WaitCtx &wc, const Runtime *rt, const ypk_task &t,
                                                   int batch, long long iter) {
  const uint16_t *pval = reinterpret_cast<const uint16_t *>(t.ptr[0]);
  const long long *pidx = reinterpret_cast<const long long *>(t.ptr[1]);
  long long *out = reinterpret_cast<long long *>(t.ptr[2]);
  const int nparts = t.iarg[0];
  const int ldp = t.iarg[4] > 0 ? t.iarg[4] : nparts;   // row pitch of the partial buffers
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  LLPoll poll;
  for (int b = warp; b < batch; b += kConsumerWarps) {
    float best = -INFINITY;
    long long bidx = 0x7fffffffffffffffll;
    for (int p = lane; p < nparts; p += 32) {
      const float v = cvt_one<false>(__ldcg(pval + size_t(b) * ldp + p));
      const long long i = __ldcg(pidx + size_t(b) * ldp + p);
      if (v > best || (v == best && i < bidx)) {
        best = v;
        bidx = i;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const long long oi = __shfl_xor_sync(0xffffffffu, bidx, o);
      if (ov > best || (ov == best && oi < bidx)) {
        best = ov;
        bidx = oi;
      }
    }
    if (TP && (t.flags & YPK_F_LL_PUSH)) {
      const int world = t.iarg[2], rank = t.iarg[3];
      const uint32_t tag = ll_tag(*rt, iter, t.iarg[12]);
      const size_t off = size_t(reinterpret_cast<char *>(t.ptr[3]) - rt->arena[rank]);
      bidx += t.iarg[1];
      if (lane < world) {   // lane p tells rank p
        unsigned long long *dst = reinterpret_cast<unsigned long long *>(rt->arena[lane] + off) +
                                  (size_t(rank) * rt->max_tok + b) * 2;
        ll_store_sys(dst, ll_word(__float_as_uint(best), tag));
        ll_store_sys(dst + 1, ll_word(static_cast<uint32_t>(bidx), tag));
      }
      best = -INFINITY;
      bidx = 0x7fffffffffffffffll;
      if (lane < world) {   // and reads what rank p found
        const unsigned long long *src =
            reinterpret_cast<const unsigned long long *>(t.ptr[3]) + (size_t(lane) * rt->max_tok + b) * 2;
        unsigned long long wv, wi;
        ll_load2(src, wv, wi);
        while (!(ll_ok(wv, tag) && ll_ok(wi, tag)) && poll.again(wc)) ll_load2(src, wv, wi);
        best = __uint_as_float(static_cast<uint32_t>(wv));
        bidx = static_cast<long long>(static_cast<uint32_t>(wi));
      }
#pragma unroll
      for (int o = 4; o > 0; o >>= 1) {   // world <= 8
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const long long oi = __shfl_xor_sync(0xffffffffu, bidx, o);
        if (ov > best || (ov == best && oi < bidx)) {
          best = ov;
          bidx = oi;
        }
      }
    }
    if (lane == 0) out[b] = bidx;
  }
  return !__any_sync(0xffffffffu, poll.failed);
}

// out[b, :] = bf16(x * rsqrt(mean(x^2) + eps) * w) for rows [row0, row0+nrows) of the batch
// (tasks/hopper/rmsnorm_hopper.cuh:20-155).  ptr = {x, w, out}; iarg = {K, row0, nrows, ldx, ldout}.
// The CTA takes the rows one after the other: 16-byte loads, the row kept in registers
// between the two passes (K <= 16384), statistics summed across the 8 warps through `red`
// ([8] floats of shared memory).
template <bool F16>
__device__ __forceinline__ void rmsnorm_rows(const ypk_task &t, int batch, float *red) {
  const uint16_t *x = reinterpret_cast<const uint16_t *>(t.ptr[0]);
  const uint16_t *w = reinterpret_cast<const uint16_t *>(t.ptr[1]);
  uint16_t *out = reinterpret_cast<uint16_t *>(t.ptr[2]);
  const int K = t.iarg[0], row0 = t.iarg[1], ldx = t.iarg[3], ldo = t.iarg[4];
  const int row1 = min(batch, row0 + t.iarg[2]);
  const float eps = t.farg[0];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  constexpr int kV = 8;   // 16-byte chunks per thread: 8 x 8 x 256 = 16384 columns
  const bool vec = (K % 8) == 0 && K <= kV * 8 * kConsumerThreads && (ldx % 8) == 0 && (ldo % 8) == 0;
  for (int b = row0; b < row1; ++b) {
    const uint16_t *xr = x + size_t(b) * ldx;
    uint16_t *orow = out + size_t(b) * ldo;
    float ss = 0.f;
    uint4 xv[kV];
    if (vec) {
#pragma unroll
      for (int u = 0; u < kV; ++u) {
        const int k = (u * kConsumerThreads + tid) * 8;
        xv[u] = make_uint4(0u, 0u, 0u, 0u);
        if (k < K) xv[u] = __ldcg(reinterpret_cast<const uint4 *>(xr + k));
      }
#pragma unroll
      for (int u = 0; u < kV; ++u) {
        const uint32_t p[4] = {xv[u].x, xv[u].y, xv[u].z, xv[u].w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = unpack2(cvt_pair<F16>(p[i]));
          ss += f.x * f.x + f.y * f.y;
        }
      }
    } else {
      for (int k = tid; k < K; k += kConsumerThreads) {
        const float f = cvt_one<F16>(__ldcg(xr + k));
        ss += f * f;
      }
    }
    ss = warp_sum(ss);
    consumer_bar();               // the previous row is done with `red`
    if (lane == 0) red[warp] = ss;
    consumer_bar();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < kConsumerWarps; ++i) tot += red[i];
    const float rn = rsqrtf(tot / float(K) + eps);
    if (vec) {
#pragma unroll
      for (int u = 0; u < kV; ++u) {
        const int k = (u * kConsumerThreads + tid) * 8;
        if (k < K) {
          uint4 wv = make_uint4(0u, 0u, 0u, 0u);
          if (w) wv = __ldg(reinterpret_cast<const uint4 *>(w + k));
          const uint32_t p[4] = {xv[u].x, xv[u].y, xv[u].z, xv[u].w};
          const uint32_t q[4] = {wv.x, wv.y, wv.z, wv.w};
          uint32_t o[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 f = unpack2(cvt_pair<F16>(p[i]));
            float2 g = make_float2(1.f, 1.f);
            if (w) g = unpack2(cvt_pair<F16>(q[i]));
            o[i] = uint32_t(cvt_out<F16>(f.x * rn * g.x)) | (uint32_t(cvt_out<F16>(f.y * rn * g.y)) << 16);
          }
          *reinterpret_cast<uint4 *>(orow + k) = make_uint4(o[0], o[1], o[2], o[3]);
        }
      }
    } else {
      for (int k = tid; k < K; k += kConsumerThreads) {
        const float f = cvt_one<F16>(__ldcg(xr + k));
        const float wf = w ? cvt_one<F16>(__ldg(w + k)) : 1.f;
        orow[k] = cvt_out<F16>(f * rn * wf);
      }
    }
  }
}
__device__ __forceinline__ void rmsnorm_task(const ypk_task &t, int batch, float *red) {
  if (t.flags & YPK_F_F16) {
    rmsnorm_rows<true>(t, batch, red);
  } else {
    rmsnorm_rows<false>(t, batch, red);
  }
}

// out[b, j] = bf16(silu(gate)) * up for output columns [col0, col0+ncols); the input row
// holds groups of (gs gate | gs up) columns (tasks/ampere/silu_mul.cuh:19-42).
// ptr = {in, out}; iarg = {col0, ncols, gs, ldin, ldout}.
__device__ __forceinline__ void silu_mul_task(const ypk_task &t, int batch) {
  const uint16_t *in = reinterpret_cast<const uint16_t *>(t.ptr[0]);
  uint16_t *out = reinterpret_cast<uint16_t *>(t.ptr[1]);
  const int col0 = t.iarg[0], ncols = t.iarg[1], gs = t.iarg[2], ldi = t.iarg[3], ldo = t.iarg[4];
  for (int idx = threadIdx.x; idx < batch * ncols; idx += kConsumerThreads) {
    const int b = idx / ncols, j = col0 + (idx - b * ncols);
    const int grp = j / gs, within = j - grp * gs;
    const float g = cvt_one<false>(__ldcg(in + size_t(b) * ldi + size_t(grp) * 2 * gs + within));
    const float u = cvt_one<false>(__ldcg(in + size_t(b) * ldi + size_t(grp) * 2 * gs + gs + within));
    const float s = bf16_round(g / (1.0f + __expf(-g)));
    out[size_t(b) * ldo + j] = cvt_out<false>(s * u);
  }
}

// ------------------------------------------------------------ mixture of experts
// MOE_TOPK (one task): router of a mixture-of-experts layer (topk_softmax_task_impl,
// tasks/blackwell/topk_softmax_sm100.cuh:63-303, renormalize = true): a warp per token.
__device__ __forceinline__ void moe_topk_task(const Runtime &rt, const ypk_task &t, int batch) {
  const uint16_t *logits = reinterpret_cast<const uint16_t *>(t.ptr[0]);
  float *weights = reinterpret_cast<float *>(t.ptr[1]);
  int *routing = reinterpret_cast<int *>(t.ptr[2]);
  int *active = reinterpret_cast<int *>(t.ptr[3]);
  int *tok_slot = reinterpret_cast<int *>(t.ptr[4]);
  const int E = t.iarg[0], K = t.iarg[1], ld = t.iarg[2], MT = rt.max_tok;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  constexpr int kPerLane = 32;            // up to 1024 experts
  for (int i = tid; i < E * MT; i += kConsumerThreads) routing[i] = 0;
  consumer_bar();
  for (int b = warp; b < batch; b += kConsumerWarps) {
    float p[kPerLane];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) {
      const int e = lane + i * 32;
      p[i] = e < E ? cvt_one<false>(__ldcg(logits + size_t(b) * ld + e)) : -INFINITY;
      mx = fmaxf(mx, p[i]);
    }
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) {
      p[i] = lane + i * 32 < E ? expf(p[i] - mx) : -1.f;
      sum += fmaxf(p[i], 0.f);
    }
    sum = warp_sum(sum);
    const float inv = 1.f / sum;
#pragma unroll
    for (int i = 0; i < kPerLane; ++i)
      if (p[i] >= 0.f) p[i] *= inv;
    float wsum = 0.f, mine = 0.f;
    int mine_e = -1;
    for (int j = 0; j < K; ++j) {
      float best = -1.f;
      int be = 0x7fffffff;
#pragma unroll
      for (int i = 0; i < kPerLane; ++i) {
        if (p[i] > best) {       // ascending ids within a lane: the first of equals stays
          best = p[i];
          be = lane + i * 32;
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oe = __shfl_xor_sync(0xffffffffu, be, o);
        if (ov > best || (ov == best && oe < be)) {
          best = ov;
          be = oe;
        }
      }
      wsum += best;
      if (lane == j) {
        mine = best;
        mine_e = be;
      }
#pragma unroll
      for (int i = 0; i < kPerLane; ++i)
        if (lane + i * 32 == be) p[i] = -1.f;      // taken
    }
    if (lane < K) {
      weights[size_t(b) * K + lane] = mine / wsum;
      routing[size_t(mine_e) * MT + b] = lane + 1;
      tok_slot[size_t(b) * K + lane] = mine_e;     // expert id for now, slot below
    }
  }
  consumer_bar();
  // active experts in ascending order (the reference appends them in atomic order)
  if (warp == 0) {
    int count = 0;
    for (int e0 = 0; e0 < E; e0 += 32) {
      const int e = e0 + lane;
      bool used = false;
      if (e < E)
        for (int b = 0; b < batch && !used; ++b) used = routing[size_t(e) * MT + b] != 0;
      const unsigned m = __ballot_sync(0xffffffffu, used);
      if (used) active[count + __popc(m & ((1u << lane) - 1u))] = e;
      count += __popc(m);
    }
    if (lane == 0) active[E] = count;
  }
  consumer_bar();
  for (int i = tid; i < batch * K; i += kConsumerThreads) {
    const int e = tok_slot[i];
    int lo = 0, hi = active[E] - 1;               // position of e in the ascending list
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (active[mid] < e) lo = mid + 1; else hi = mid;
    }
    tok_slot[i] = lo;
  }
}

// LINEAR with YPK_F_MOE: called by one thread on the shared-memory copy of the task before
// the task runs.  Points the weight operand at the rows of the expert in active slot
// iarg[10]; a slot beyond the iteration's count turns the copy into a NOP.  The producer warp
// (`wait` true) first waits for the event the task depends on: the router runs earlier in the
// same iteration.  Returns 1: run, 0: skip, -1: the wait gave up.
static __device__ __noinline__ int moe_resolve(WaitCtx &wc, const Runtime &rt, ypk_task *t,
                                               long long iter, bool wait) {
  if (wait && t->dep_event >= 0) {
    const unsigned long long need =
        static_cast<unsigned long long>(t->dep_count) * static_cast<unsigned long long>(iter);
    if (!wait_counter(wc, rt.events + t->dep_event, need, t->dep_event)) return -1;
  }
  const int *active = reinterpret_cast<const int *>(t->ptr[5]);
  const int slot = t->iarg[10], E = t->iarg[11];
  if (slot >= __ldcg(active + E)) {
    t->type = YPK_TASK_NOP;
    return 0;
  }
  const long long expert = __ldcg(active + slot);
  t->ptr[1] += static_cast<unsigned long long>(expert) * static_cast<unsigned long long>(t->iarg[12]) *
               static_cast<unsigned long long>(t->iarg[4]) * 2ull;
  return 1;
}

// MOE_SILU_MUL: out[slot][b][i] = silu(in[slot][b][i]) * in[slot][b][I + i] for the active
// slots this task owns, with the rounding points of silu_mul_task.
__device__ __forceinline__ void moe_silu_mul_task(const Runtime &rt, const ypk_task &t, int batch) {
  const uint16_t *in = reinterpret_cast<const uint16_t *>(t.ptr[0]);
  uint16_t *out = reinterpret_cast<uint16_t *>(t.ptr[1]);
  const int *active = reinterpret_cast<const int *>(t.ptr[2]);
  const int I = t.iarg[0], E = t.iarg[1], slot0 = t.iarg[2], nslots = t.iarg[3], MT = rt.max_tok;
  const int count = __ldcg(active + E);
  for (int s = slot0; s < min(slot0 + nslots, count); ++s) {
    for (int i = threadIdx.x; i < batch * I; i += kConsumerThreads) {
      const int b = i / I, c = i - b * I;
      const uint16_t *row = in + (size_t(s) * MT + b) * 2 * I;
      const float g = cvt_one<false>(__ldcg(row + c)), u = cvt_one<false>(__ldcg(row + I + c));
      const float sg = bf16_round(g / (1.0f + __expf(-g)));
      out[(size_t(s) * MT + b) * I + c] = cvt_out<false>(sg * u);
    }
  }
}

// MOE_COMBINE: out[b][c] = round(residual[b][c] + sum_j weight[b][j] * expert_out[slot(b, j)][b][c])
// (mul_sum_add_sm100_task_impl, tasks/blackwell/mul_sum_add_sm100.cuh:24-47).
__device__ __forceinline__ void moe_combine_task(const Runtime &rt, const ypk_task &t, int batch) {
  const uint16_t *eo = reinterpret_cast<const uint16_t *>(t.ptr[0]);
  const float *weights = reinterpret_cast<const float *>(t.ptr[1]);
  const int *tok_slot = reinterpret_cast<const int *>(t.ptr[2]);
  const uint16_t *res = reinterpret_cast<const uint16_t *>(t.ptr[3]);
  uint16_t *out = reinterpret_cast<uint16_t *>(t.ptr[4]);
  const int H = t.iarg[0], K = t.iarg[1], col0 = t.iarg[2], ncols = t.iarg[3], ldr = t.iarg[4],
            ldo = t.iarg[5], MT = rt.max_tok;
  for (int i = threadIdx.x; i < batch * ncols; i += kConsumerThreads) {
    const int b = i / ncols, c = col0 + (i - b * ncols);
    float acc = cvt_one<false>(__ldcg(res + size_t(b) * ldr + c));
    for (int j = 0; j < K; ++j) {
      const int s = __ldcg(tok_slot + size_t(b) * K + j);
      acc += cvt_one<false>(__ldcg(eo + (size_t(s) * MT + b) * H + c)) * __ldcg(weights + size_t(b) * K + j);
    }
    out[size_t(b) * ldo + c] = cvt_out<false>(acc);
  }
}

// ------------------------------------------------------------ prompt-lookup drafts
// Speculative decoding by prompt lookup (the reference's find_ngram_partial / find_ngram_global
// / target_verify_greedy tasks, tasks/speculative_decoding/prompt_lookup.cuh:22-132 and
// target_verify.cuh:20-60, which serve one request; here every request slot of the batch).
// A request that is past its prompt brings its last token plus draft slots (the batcher
// leaves -1 in them).  The drafts are the tokens that followed the earliest earlier
// occurrence of the history's last `ngram` tokens.
//
// NGRAM_PARTIAL: ptr = {partial int32 [max_requests][nparts]}; iarg = {part, nparts, ngram}.
// Part p looks at its share of the candidate positions of every slot and leaves the lowest
// matching position (or INT_MAX).
__device__ __forceinline__ void ngram_partial_task(const Runtime &rt, const ypk_task &t, int *red) {
  int *partial = reinterpret_cast<int *>(t.ptr[0]);
  const int part = t.iarg[0], nparts = t.iarg[1], N = t.iarg[2];
  const int tid = threadIdx.x;
  for (int i = 0; i < rt.max_req; ++i) {
    const int req = __ldcg(rt.request_ids + i);
    int best = 0x7fffffff;
    if (req >= 0) {
      const int T = __ldcg(rt.qo_indptr + i + 1) - __ldcg(rt.qo_indptr + i);
      const int step = __ldcg(rt.step + req);
      const int total = step + 1 - N;          // candidate positions: 0 .. total - 1
      if (T > 1 && step >= __ldcg(rt.prompt_len + req) && total > 0) {
        const long long *row = rt.tokens + size_t(req) * rt.max_seq;
        const int per = (total + nparts - 1) / nparts;
        const int lo = part * per, hi = min(total, lo + per);
        for (int idx = lo + tid; idx < hi && best == 0x7fffffff; idx += kConsumerThreads) {
          bool same = true;
          for (int k = 0; k < N && same; ++k)
            same = __ldcg(row + idx + k) == __ldcg(row + total + k);
          if (same) best = idx;
        }
      }
    }
    if (tid == 0) *red = 0x7fffffff;
    consumer_bar();
    if (best != 0x7fffffff) atomicMin(red, best);
    consumer_bar();
    if (tid == 0) partial[size_t(i) * nparts + part] = *red;
    consumer_bar();
  }
}

// NGRAM_GLOBAL: ptr = {partial, ids out int64 [max_tokens]}; iarg = {nparts, ngram}.  Copies
// the iteration's input tokens to `ids` (what the embedding reads) and fills the draft slots.
__device__ __forceinline__ void ngram_global_task(const Runtime &rt, const ypk_task &t, int batch) {
  const int *partial = reinterpret_cast<const int *>(t.ptr[0]);
  long long *ids = reinterpret_cast<long long *>(t.ptr[1]);
  const int nparts = t.iarg[0], N = t.iarg[1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = warp; i < rt.max_req; i += kConsumerWarps) {
    const int req = __ldcg(rt.request_ids + i);
    if (req < 0) continue;
    const int qo = __ldcg(rt.qo_indptr + i), T = __ldcg(rt.qo_indptr + i + 1) - qo;
    const int step = __ldcg(rt.step + req);
    const bool drafts = T > 1 && step >= __ldcg(rt.prompt_len + req);
    int m = 0x7fffffff;
    if (drafts) {
      for (int p = lane; p < nparts; p += 32) m = min(m, __ldcg(partial + size_t(i) * nparts + p));
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) m = min(m, __shfl_xor_sync(0xffffffffu, m, o));
    }
    const long long *row = rt.tokens + size_t(req) * rt.max_seq;
    for (int j = lane; j < T; j += 32) {
      long long v = __ldcg(rt.input_tokens + qo + j);
      if (drafts && j > 0) {
        const long long src = static_cast<long long>(m) + N + (j - 1);
        v = (m != 0x7fffffff && src <= step) ? __ldcg(row + src) : -1ll;
      }
      ids[qo + j] = v;
    }
  }
  (void)batch;
}

// VERIFY: ptr = {ids (with the drafts), model outputs int64 [max_tokens]}; iarg = {spec length}.
// num_new_tokens[request] = accepted drafts + 1 (the model's own next token), or the number
// of tokens the slot brought when it carried no drafts.  The batcher reads it.
__device__ __forceinline__ void verify_greedy_task(const Runtime &rt, const ypk_task &t) {
  const long long *ids = reinterpret_cast<const long long *>(t.ptr[0]);
  const long long *target = reinterpret_cast<const long long *>(t.ptr[1]);
  for (int i = threadIdx.x; i < rt.max_req; i += kConsumerThreads) {
    const int req = __ldcg(rt.request_ids + i);
    if (req < 0) continue;
    const int qo = __ldcg(rt.qo_indptr + i), T = __ldcg(rt.qo_indptr + i + 1) - qo;
    int n = T;
    if (T > 1 && __ldcg(rt.step + req) >= __ldcg(rt.prompt_len + req)) {
      int acc = T - 1;
      for (int k = 0; k < T - 1; ++k) {
        if (__ldcg(ids + qo + k + 1) != __ldcg(target + qo + k)) {
          acc = k;
          break;
        }
      }
      n = acc + 1;
    }
    rt.num_new[req] = n;
  }
}

// ------------------------------------------------------------ batcher
// Continuous batching between iterations, one thread (the reference runs the same
// logic in scheduler 0: persistent_kernel.cuh:169-322).  Retires finished requests and
// frees their pages, compacts the active ones, admits new requests, chunks prefill to
// the token budget (and to rt.max_new_tokens per request), copies the iteration's input
// tokens and rebuilds qo_indptr / paged_kv_indptr / paged_kv_indices.
// paged_kv_last_page_len is written in [1, page_size].
// `first` skips the finalisation of a previous batch.  Returns the number of active
// tokens of the next iteration (0 = everything retired), or -1 when a request that is
// already running needs a page and the pool has none left (the reference hands out pages
// without looking, persistent_kernel.cuh:262-270, and two requests then share one).
// The query-tile list of the batch in qo_indptr (see Runtime::qtiles).
static __device__ __noinline__ void build_query_tiles(const Runtime &rt) {
  if (rt.qtiles == nullptr) return;
  const int ch = max(1, rt.attn_chunk);
  int n = 0;
  for (int i = 0; i < rt.max_req && n < rt.max_tok; ++i) {
    if (rt.request_ids[i] < 0) continue;
    const int T = rt.qo_indptr[i + 1] - rt.qo_indptr[i];
    for (int t0 = 0; t0 < T && n < rt.max_tok; t0 += ch)
      rt.qtiles[n++] = i | (t0 << 12) | (min(ch, T - t0) << 20);
  }
  for (; n < rt.max_tok; ++n) rt.qtiles[n] = -1;
}

static __device__ __noinline__ int prepare_next_batch_impl(const Runtime &rt, bool first);
static __device__ __forceinline__ int prepare_next_batch(const Runtime &rt, bool first) {
  const int ntok = prepare_next_batch_impl(rt, first);
  if (ntok > 0) build_query_tiles(rt);
  return ntok;
}
static __device__ __noinline__ int prepare_next_batch_impl(const Runtime &rt, bool first) {
  const int MR = rt.max_req, MT = rt.max_tok, MP = rt.max_pages, PS = rt.page_size;
  int head = rt.bstate[1], tail = rt.bstate[2];
  if (!first) {
    for (int i = 0; i < MR; ++i) {
      const int req = rt.request_ids[i];
      if (req < 0) continue;
      const int step = rt.step[req];
      const int qo = rt.qo_indptr[i];
      int ntok = rt.qo_indptr[i + 1] - qo;
      const int plen = rt.prompt_len[req];
      // drafts were verified: only the accepted outputs count
      if (rt.spec_len > 0 && step >= plen && ntok > 1) ntok = max(1, min(ntok, __ldcg(rt.num_new + req)));
      for (int j = 0; j < ntok; ++j) {
        if (step + j + 1 >= plen && step + j + 1 < rt.max_seq) {
          rt.tokens[size_t(req) * rt.max_seq + step + j + 1] = __ldcg(rt.output_tokens + qo + j);
        }
      }
      rt.step[req] = step + ntok;
      const bool full = step + ntok + 1 >= rt.max_seq;
      const bool eos = step + ntok >= plen && step + ntok < rt.max_seq &&
                       rt.tokens[size_t(req) * rt.max_seq + step + ntok] == rt.eos;
      if (full || eos) {
        rt.request_ids[i] = -1;
        const int kv = rt.kv_indptr[i];
        const int np = rt.kv_indptr[i + 1] - kv;
        for (int j = 0; j < np; ++j) {
          rt.page_queue[tail % MP] = rt.kv_indices[kv + j];
          ++tail;
        }
      }
    }
  }
  int nreq = 0, ntok = 0, npages = 0;
  // Surviving requests keep their pages.  A request that grows can push the compacted
  // list past the old position of a later request, so rebuild from a copy.
  {
    const int nold_total = rt.kv_indptr[MR];
    for (int j = 0; j < nold_total; ++j) rt.kv_tmp[j] = rt.kv_indices[j];
  }
  for (int i = 0; i < MR; ++i) {
    const int req = rt.request_ids[i];
    if (req < 0) continue;
    const int kv = rt.kv_indptr[i];
    const int nold = rt.kv_indptr[i + 1] - kv;
    const int step = rt.step[req];
    int nnew = rt.prompt_len[req] - step;
    const bool past_prompt = nnew <= 0;
    nnew = nnew > 0 ? min(min(nnew, MT - ntok), rt.max_new_tokens) : min(1, MT - ntok);
    if (past_prompt && rt.spec_len > 0) {
      // the last token and the draft slots (filled by the NGRAM_GLOBAL task)
      const int want = 1 + rt.spec_len;
      if (MT - ntok >= want && want <= rt.max_new_tokens && step + want < rt.max_seq) nnew = want;
    }
    // nreq <= i, so the indptr entries overwritten below have been consumed already.
    for (int j = 0; j < nold; ++j) rt.kv_indices[npages + j] = rt.kv_tmp[kv + j];
    rt.request_ids[nreq] = req;
    rt.qo_indptr[nreq] = ntok;
    rt.kv_indptr[nreq] = npages;
    for (int j = 0; j < nnew; ++j)
      rt.input_tokens[ntok + j] =
          (past_prompt && j > 0) ? -1ll : rt.tokens[size_t(req) * rt.max_seq + step + j];
    const int total = step + nnew;
    const int need = (total + PS - 1) / PS;
    if (need > nold && (tail - head < need - nold || npages + need > MP)) return -1;
    for (int j = nold; j < need; ++j) {
      rt.kv_indices[npages + j] = rt.page_queue[head % MP];
      ++head;
    }
    const int have = max(need, nold);
    rt.kv_last_len[nreq] = total > 0 ? (total - 1) % PS + 1 : 0;
    npages += have;
    ntok += nnew;
    ++nreq;
  }
  while (nreq < MR && ntok < MT) {
    const int req = rt.bstate[0];
    if (req >= rt.total_req) break;
    // A request normally enters at step 0.  If the caller set step[req] = s0 after the reset,
    // its first s0 tokens count as already cached: the request gets the pages for them and
    // starts at position s0 (what those pages hold is the caller's business).
    const int s0 = max(0, min(rt.step[req], rt.max_seq - 2));
    const int left = rt.prompt_len[req] - s0;
    int nnew = left > 0 ? min(min(left, MT - ntok), rt.max_new_tokens) : min(1, MT - ntok);
    const int need = (s0 + nnew + PS - 1) / PS;
    if (npages + need > MP || (tail - head) < need) break;  // no page budget yet
    rt.request_ids[nreq] = req;
    rt.qo_indptr[nreq] = ntok;
    rt.kv_indptr[nreq] = npages;
    for (int j = 0; j < nnew; ++j)
      rt.input_tokens[ntok + j] = rt.tokens[size_t(req) * rt.max_seq + s0 + j];
    for (int j = 0; j < need; ++j) {
      rt.kv_indices[npages + j] = rt.page_queue[head % MP];
      ++head;
    }
    rt.kv_last_len[nreq] = s0 + nnew > 0 ? (s0 + nnew - 1) % PS + 1 : 0;
    npages += need;
    ntok += nnew;
    ++nreq;
    rt.bstate[0] = req + 1;
  }
  for (int i = nreq; i < MR; ++i) rt.request_ids[i] = -1;
  for (int i = nreq; i <= MR; ++i) {
    rt.qo_indptr[i] = ntok;
    rt.kv_indptr[i] = npages;
  }
  rt.bstate[1] = head;
  rt.bstate[2] = tail;
  return ntok;
}

}  // namespace ypk
