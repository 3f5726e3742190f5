// ALLREDUCE task: sum over the tensor-parallel ranks of a [batch, hidden] partial result, for
// one slice of columns.  Semantics of the reference's allreduce expansion
// (src/kernel/runtime.cc:215-363: every rank puts its tile into slot `rank` of every peer's
// buffer and signals the peer's counter, then a reduce task sums the slots,
// tasks/ampere/reduction.cuh:139-166: fp32 accumulation in rank order, own slice read from
// the input, one rounding).  The reference does the put with NVSHMEM
// (task_register.cc:669-686); here the peers' buffers are plain peer-mapped device memory
// (CUDA IPC over NVLink / NVSwitch) inside one symmetric arena per rank:
//
//   1. push: 16-byte stores of this rank's slice into slot `rank` of each peer's buffer;
//   2. CTA barrier, then one thread per peer does fence.acq_rel.sys + red.relaxed.sys.add on
//      that peer's counter (the fence is cumulative over the other threads' stores);
//   3. bounded wait until the own counter has world-1 arrivals for this iteration
//      (ld.acquire.sys), so the remote tiles are in this GPU's memory before they are read;
//   4. reduce from local memory only.
//
// The buffer has two halves used by alternate all-reduces: a fast rank writing all-reduce
// k+1 cannot touch what a slow rank still reads for k, and it cannot reach k+2 before the
// slow rank has pushed k+1, i.e. finished reading k.  "Alternate" counts across iteration
// boundaries, so the half is the parity of the running all-reduce number
// (iterations so far * all-reduces per iteration + index in the iteration): a graph with an
// odd number of all-reduces still never uses one half twice in a row.  No TMA and no
// multicast are involved.
//
// ptr  = {in, buf, out, signals};  buf = [2][world][max_tokens][hidden] 16-bit, symmetric
// iarg = {col0, ncols, ld_in, ld_out, hidden, max_tokens, index of this all-reduce in the
//         iteration, signal index, world, rank, all-reduces per iteration}
#pragma once
#include "device_common.cuh"
#include "ll_handoff.cuh"

namespace ypk {

__device__ __forceinline__ bool allreduce_task(WaitCtx &wc, Misc *misc, const Runtime &rt,
                                               const ypk_task &t, int batch, long long iter) {
  const int tid = threadIdx.x;
  const uint16_t *in = reinterpret_cast<const uint16_t *>(t.ptr[0]);
  char *buf = reinterpret_cast<char *>(t.ptr[1]);
  uint16_t *out = reinterpret_cast<uint16_t *>(t.ptr[2]);
  char *sig = reinterpret_cast<char *>(t.ptr[3]);
  const int col0 = t.iarg[0], ncols = t.iarg[1], ld_in = t.iarg[2], ld_out = t.iarg[3];
  const int hidden = t.iarg[4], max_tok = t.iarg[5], sidx = t.iarg[7];
  const int world = t.iarg[8], rank = t.iarg[9];
  const int half = int(((rt.ar_epoch + static_cast<unsigned long long>(iter)) *
                            static_cast<unsigned long long>(t.iarg[10]) +
                        static_cast<unsigned long long>(t.iarg[6])) & 1ull);
  const size_t buf_off = size_t(buf - rt.arena[rank]), sig_off = size_t(sig - rt.arena[rank]);
  const int nvec = ncols / 8;
  auto slot = [&](int r, int b) -> size_t {   // byte offset of row b of rank r's slot in the half
    return ((size_t(half) * world + r) * max_tok + b) * size_t(hidden) * 2 + size_t(col0) * 2;
  };
  for (int idx = tid; idx < batch * nvec; idx += kConsumerThreads) {
    const int b = idx / nvec, c = idx - b * nvec;
    const uint4 v = __ldcg(reinterpret_cast<const uint4 *>(in + size_t(b) * ld_in + col0 + c * 8));
    for (int p = 0; p < world; ++p) {
      if (p == rank) continue;
      *reinterpret_cast<uint4 *>(rt.arena[p] + buf_off + slot(rank, b) + c * 16) = v;
    }
  }
  consumer_bar();
  // One signalling thread per peer, side by side: each orders the CTA's stores (known to it
  // through the barrier) with a system-scope fence and bumps its peer's counter.  A single
  // thread doing the peers in turn would pay one NVLink round trip per peer.
  if (tid < world && tid != rank) {
    asm volatile("fence.acq_rel.sys;" ::: "memory");
    asm volatile("red.relaxed.sys.global.add.u64 [%0], %1;" ::"l"(
                     reinterpret_cast<unsigned long long *>(rt.arena[tid] + sig_off) + sidx),
                 "l"(1ull)
                 : "memory");
  }
  if (tid == 0) {
    // arrivals are never reset: count the iterations of earlier runs too
    const unsigned long long need = static_cast<unsigned long long>(world - 1) *
                                    (rt.ar_epoch + static_cast<unsigned long long>(iter));
    misc->flag = wait_counter_sys(wc, reinterpret_cast<unsigned long long *>(sig) + sidx, need,
                                  -5) ? 1 : 0;
  }
  consumer_bar();
  if (misc->flag == 0) return false;
  for (int idx = tid; idx < batch * nvec; idx += kConsumerThreads) {
    const int b = idx / nvec, c = idx - b * nvec;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    for (int r = 0; r < world; ++r) {
      const uint4 v = r == rank
          ? __ldcg(reinterpret_cast<const uint4 *>(in + size_t(b) * ld_in + col0 + c * 8))
          : __ldcg(reinterpret_cast<const uint4 *>(buf + slot(r, b) + c * 16));
      const uint32_t p[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = unpack2(cvt_pair<false>(p[i]));
        acc[2 * i] += f.x;
        acc[2 * i + 1] += f.y;
      }
    }
    uint32_t o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      o[i] = uint32_t(cvt_out<false>(acc[2 * i])) | (uint32_t(cvt_out<false>(acc[2 * i + 1])) << 16);
    }
    *reinterpret_cast<uint4 *>(out + size_t(b) * ld_out + col0 + c * 8) = make_uint4(o[0], o[1], o[2], o[3]);
  }
  return true;
}

// Flagged-word form (YPK_F_LL_IN | YPK_F_LL_OUT): the LINEAR tasks that produce the partial
// sums have already pushed them, as {two values, tag} words, into slot `rank` of `buf` on
// every rank (buf = [world][max_tokens][hidden / 2] words, single-buffered: a rank cannot
// push the next partial of this buffer before it has consumed this one's sum on every rank).
// This task only polls the world slots of its column slice, adds them in rank order in fp32,
// rounds once and hands the sum on, again as flagged words (ptr[7]) plus the plain tensor.
// No signal counters, no fences, no event in or out.
static __device__ __noinline__ bool allreduce_ll_task(WaitCtx &wc, const Runtime &rt, const ypk_task &t,
                                                  int batch, long long iter) {
  const int tid = threadIdx.x;
  const unsigned long long *buf = reinterpret_cast<const unsigned long long *>(t.ptr[1]);
  uint16_t *out = reinterpret_cast<uint16_t *>(t.ptr[2]);
  unsigned long long *ll_out = reinterpret_cast<unsigned long long *>(t.ptr[7]);
  const int col0 = t.iarg[0], ncols = t.iarg[1], ld_out = t.iarg[3];
  const int hidden = t.iarg[4], max_tok = t.iarg[5], world = t.iarg[8];
  const uint32_t tag_in = ll_tag(rt, iter, t.iarg[10]), tag_out = ll_tag(rt, iter, t.iarg[12]);
  const int nword = ncols >> 1;
  const size_t slot_words = size_t(max_tok) * size_t(hidden >> 1);
  LLPoll poll;
  for (int idx = tid; idx < batch * nword; idx += kConsumerThreads) {
    const int b = idx / nword, c = idx - b * nword;
    const unsigned long long *src = buf + size_t(b) * size_t(hidden >> 1) + size_t(col0 >> 1) + c;
    // every rank's word in flight at once; the late ones are asked for again together, so a
    // round costs one trip to L2 however many ranks are late
    unsigned long long w[8];
    bool late[8];
#pragma unroll
    for (int r = 0; r < 8; ++r) late[r] = r < world;
    for (;;) {
#pragma unroll
      for (int r = 0; r < 8; ++r)
        if (late[r]) w[r] = ll_load(src + r * slot_words);
      bool any = false;
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        if (late[r]) late[r] = !ll_ok(w[r], tag_in);
        any |= late[r];
      }
      if (!any || !poll.again(wc)) break;
    }
    float s0 = 0.f, s1 = 0.f;
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      if (r < world) {
        const float2 f = unpack2(cvt_pair<false>(static_cast<uint32_t>(w[r])));
        s0 += f.x;
        s1 += f.y;
      }
    }
    const uint32_t packed = uint32_t(cvt_out<false>(s0)) | (uint32_t(cvt_out<false>(s1)) << 16);
    *reinterpret_cast<uint32_t *>(out + size_t(b) * ld_out + col0 + 2 * c) = packed;
    ll_store(ll_out + size_t(b) * size_t(ld_out >> 1) + size_t(col0 >> 1) + c, ll_word(packed, tag_out));
  }
  return !poll.failed;
}

}  // namespace ypk
