// The task runners of the persistent megakernel: one out-of-line device function per task
// kind and variant (each gets its own register allocation, and the worker loop keeps its
// state in registers).  They have internal linkage: every kernel's translation unit
// (megakernel_*.cu) includes this header and compiles its own copies of the runners that
// kernel calls, as relocatable device code under the plain function-call ABI.  Measured on
// B200: compiled as one unit together with all kernels, the hot one-GPU decode path moved by
// up to 12 % when an unrelated task kind was edited; called across translation units it
// lost 7 %; as a unit's own functions it is both the fastest and independent of the other
// kernels' code.
//
// Convention: the ring position and the failure state go in and come back by value;
// `failed` true = a bounded wait inside the task gave up.
//
// A call is not free here (about a microsecond per task: what is saved around it or passed on
// the stack lives in local memory and comes back from L2, the L1 beside the 227 KB ring being
// too small to hold it), so the worker loop inlines the bodies of its hottest tasks instead of
// calling their runners: see megakernel_body.cuh.
#pragma once
#include "device_common.cuh"
#include "task_allreduce.cuh"
#include "task_attention.cuh"
#include "task_linear.cuh"
#include "task_linear_umma.cuh"
#include "task_misc.cuh"

namespace ypk {

struct TaskRet {
  RingPos pos;
  bool failed;
};
struct TaskRetU {
  RingPos pos;
  UmmaState us;
  bool failed;
};
struct ProdRet {
  RingPos pos;
  bool ok;   // false = a wait gave up
};

namespace {   // internal linkage: one copy per including unit

// LINEAR, at most 8 tokens per pass.  LL: some operand travels as flagged words; TP: can push
// partial sums to peer GPUs; MANY: 3..8 tokens (activation rows of all tokens requested
// together) instead of 1..2.
template <bool LL, bool TP, bool MANY>
__device__ __noinline__ TaskRet run_linear(const Runtime *rt, Misc *misc, char *smem, int worker,
                                           int task, bool failed, int batch, long long iter,
                                           RingPos pos) {
  WaitCtx wc{rt, misc, worker, task, failed};
  linear_consume_groups<LL, TP, MANY>(wc, smem, misc, *rt, misc->ctask, batch, iter, pos);
  return TaskRet{pos, wc.failed};
}
// LINEAR, more than 8 tokens: 16 per pass on mma.sync ...
__device__ __noinline__ TaskRet run_linear16(const Runtime *rt, Misc *misc, char *smem, int worker,
                                             int task, bool failed, int batch, RingPos pos) {
  WaitCtx wc{rt, misc, worker, task, failed};
  linear_consume_groups16(wc, smem, misc, misc->ctask, batch, pos);
  return TaskRet{pos, wc.failed};
}
// ... or on tcgen05 / TMEM
__device__ __noinline__ TaskRetU run_linear_umma(const Runtime *rt, Misc *misc, char *smem,
                                                 int worker, int task, bool failed, int batch,
                                                 RingPos pos, UmmaState us) {
  WaitCtx wc{rt, misc, worker, task, failed};
  linear_consume_umma(wc, smem, misc, misc->ctask, batch, pos, us);
  return TaskRetU{pos, us, wc.failed};
}
__device__ __noinline__ TaskRet run_attention(const Runtime *rt, Misc *misc, char *smem, int worker,
                                              int task, bool failed, long long iter, RingPos pos) {
  WaitCtx wc{rt, misc, worker, task, failed};
  attention_consume(wc, smem, misc, *rt, misc->ctask, iter, pos);
  return TaskRet{pos, wc.failed};
}
// EMBED, ARGMAX_*, RMSNORM, SILU_MUL (and ALLREDUCE with TP); returns `failed`.
template <bool TP>
__device__ __noinline__ bool run_small(const Runtime *rt, Misc *misc, int worker, int task,
                                       bool failed, int batch, long long iter) {
  WaitCtx wc{rt, misc, worker, task, failed};
  const ypk_task &t = misc->ctask;
  switch (t.type) {
    case YPK_TASK_EMBED: embed_task(t, batch); break;
    case YPK_TASK_ARGMAX_PARTIAL: argmax_partial_task(t, batch); break;
    case YPK_TASK_ARGMAX_REDUCE:
      if (!argmax_reduce_task<TP>(wc, rt, t, batch, iter)) wc.failed = true;
      break;
    case YPK_TASK_RMSNORM: rmsnorm_task(t, batch, misc->rnorm); break;
    case YPK_TASK_SILU_MUL: silu_mul_task(t, batch); break;
    case YPK_TASK_NGRAM_PARTIAL: ngram_partial_task(*rt, t, &misc->flag); break;
    case YPK_TASK_NGRAM_GLOBAL: ngram_global_task(*rt, t, batch); break;
    case YPK_TASK_VERIFY: verify_greedy_task(*rt, t); break;
    case YPK_TASK_MOE_TOPK: moe_topk_task(*rt, t, batch); break;
    case YPK_TASK_MOE_SILU_MUL: moe_silu_mul_task(*rt, t, batch); break;
    case YPK_TASK_MOE_COMBINE: moe_combine_task(*rt, t, batch); break;
    case YPK_TASK_ALLREDUCE:
      if constexpr (!TP) {
        wc.failed = true;   // single-GPU kernels have no all-reduce (the host never picks them then)
      } else if (t.flags & YPK_F_LL_IN) {
        if (!allreduce_ll_task(wc, *rt, t, batch, iter)) wc.failed = true;
      } else if (!allreduce_task(wc, misc, *rt, t, batch, iter)) {
        wc.failed = true;
      }
      break;
    default: break;
  }
  return wc.failed;
}
// Producer warp: streams the weights / cached K,V of the task in misc->ptask into the ring.
// WIDE: the graph can see more than 8 tokens (16-token and tcgen05 traversals).
template <bool WIDE>
__device__ __noinline__ ProdRet run_produce(const Runtime *rt, Misc *misc, char *smem, int worker,
                                            int task, int batch, RingPos pos,
                                            unsigned long long policy) {
  WaitCtx wc{rt, misc, worker, task, false};
  const ypk_task &t = misc->ptask;
  bool ok = true;
  if (t.type == YPK_TASK_LINEAR) {
    if constexpr (WIDE) {
      ok = linear_uses_umma(*rt, t, batch) ? linear_produce_umma(wc, smem, misc, *rt, t, batch, pos, policy)
           : (batch > kMaxBatch || t.iarg[15] != 0)
               ? linear_produce16(wc, smem, misc, t, batch, pos, policy)
               : linear_produce(wc, smem, misc, t, batch, pos, policy);
    } else {
      ok = linear_produce(wc, smem, misc, t, batch, pos, policy);
    }
  } else if (t.type == YPK_TASK_ATTENTION) {
    ok = attention_produce(wc, smem, misc, *rt, t, pos);
  }
  return ProdRet{pos, ok};
}

}  // namespace
}  // namespace ypk
