// Arg-max sampling without any allocation.
//
// The graph path samples with two tasks (ARGMAX_PARTIAL into per-chunk (value, index)
// buffers that the runtime allocates, then ARGMAX_REDUCE).  Some hosts cannot let a
// library allocate: a serving process that has handed the whole device to its own pool
// allocator (a cudaMalloc from a plugin then fails or fragments the pool), or a latency
// path where the implicit device synchronisation of cudaMalloc/cudaFree is not acceptable.
// For them the same two steps run as one kernel whose chunk buffers live in a fixed
// __device__ array of this library: 64 batch rows x 128 chunks at most.  Every GPU that
// loads the library carries the array (about 100 KB) until the process exits.
#pragma once
#include "task_misc.cuh"

namespace ypk {

constexpr int kNoAllocMaxBatch = 64;
constexpr int kNoAllocParts = 128;
constexpr size_t kNoAllocValBytes = size_t(kNoAllocMaxBatch) * kNoAllocParts * 2;   // bf16
constexpr size_t kNoAllocIdxBytes = size_t(kNoAllocMaxBatch) * kNoAllocParts * 8;   // int64
constexpr size_t kNoAllocIdxOff = (kNoAllocValBytes + 255) / 256 * 256;
constexpr size_t kNoAllocCtrOff = kNoAllocIdxOff + kNoAllocIdxBytes;
constexpr size_t kNoAllocBytes = kNoAllocCtrOff + 256;

// In device code this name is the array itself.  In host code it is only a handle for
// cudaGetSymbolAddress: passing it to a kernel as a pointer would hand the kernel a host
// address.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocBytes];

// One CTA per chunk of the vocabulary; the CTA that arrives last reduces the chunks.
// `scratch` is the device address of g_noalloc_scratch obtained on the host.
__global__ void __launch_bounds__(kConsumerThreads) argmax_noalloc_kernel(
    const uint16_t *logits, int batch, int vocab, long long ld, long long *out,
    unsigned char *scratch) {
  __shared__ int is_last;
  uint16_t *pval = reinterpret_cast<uint16_t *>(scratch);
  long long *pidx = reinterpret_cast<long long *>(scratch + kNoAllocIdxOff);
  unsigned int *counter = reinterpret_cast<unsigned int *>(scratch + kNoAllocCtrOff);
  const int per = (vocab + kNoAllocParts - 1) / kNoAllocParts;
  const int col0 = blockIdx.x * per;
  const int ncols = max(0, min(per, vocab - col0));
  ypk_task t;
  t.ptr[0] = reinterpret_cast<uint64_t>(logits);
  t.ptr[1] = reinterpret_cast<uint64_t>(pval);
  t.ptr[2] = reinterpret_cast<uint64_t>(pidx);
  t.iarg[0] = col0;
  t.iarg[1] = ncols;
  t.iarg[2] = int(ld);
  t.iarg[3] = blockIdx.x;
  t.iarg[4] = kNoAllocParts;
  t.iarg[5] = 0;   // every column of [0, vocab) is real vocabulary
  argmax_partial_task(t, batch);   // an empty chunk yields (-inf, col0) and never wins
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned old = atomicAdd(counter, 1u);
    is_last = old == gridDim.x - 1;
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  ypk_task r;
  r.ptr[0] = reinterpret_cast<uint64_t>(pval);
  r.ptr[1] = reinterpret_cast<uint64_t>(pidx);
  r.ptr[2] = reinterpret_cast<uint64_t>(out);
  r.iarg[0] = kNoAllocParts;
  r.iarg[4] = 0;   // partial rows are exactly that wide
  r.flags = 0;   // no cross-rank exchange: the wait context and the runtime are never touched
  WaitCtx none{nullptr, nullptr, 0, -1, false};
  argmax_reduce_task<false>(none, nullptr, r, batch, 0);
  if (threadIdx.x == 0) *counter = 0u;   // the next call starts from zero again
}

}  // namespace ypk
