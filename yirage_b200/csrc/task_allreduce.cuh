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
// slow rank has pushed k+1, i.e. finished reading k.  No TMA and no multicast are involved.
//
// ptr  = {in, buf, out, signals};  buf = [2][world][max_tokens][hidden] 16-bit, symmetric
// iarg = {col0, ncols, ld_in, ld_out, hidden, max_tokens, half, signal index, world, rank}
#pragma once
#include "device_common.cuh"

namespace ypk {

__device__ __forceinline__ bool allreduce_task(WaitCtx &wc, Misc *misc, const Runtime &rt,
                                               const ypk_task &t, int batch, long long iter) {
  const int tid = threadIdx.x;
  const uint16_t *in = reinterpret_cast<const uint16_t *>(t.ptr[0]);
  char *buf = reinterpret_cast<char *>(t.ptr[1]);
  uint16_t *out = reinterpret_cast<uint16_t *>(t.ptr[2]);
  char *sig = reinterpret_cast<char *>(t.ptr[3]);
  const int col0 = t.iarg[0], ncols = t.iarg[1], ld_in = t.iarg[2], ld_out = t.iarg[3];
  const int hidden = t.iarg[4], max_tok = t.iarg[5], half = t.iarg[6], sidx = t.iarg[7];
  const int world = t.iarg[8], rank = t.iarg[9];
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
    const unsigned long long need =
        static_cast<unsigned long long>(world - 1) * static_cast<unsigned long long>(iter);
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

}  // namespace ypk
