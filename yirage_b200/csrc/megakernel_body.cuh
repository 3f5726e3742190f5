// The persistent megakernel: one CTA per SM, each walking its own queue of tasks every
// iteration; dependencies are monotonic event counters in global memory
// (counter >= triggers_per_iteration * iteration), so nothing is reset between
// iterations or launches.  Plays the role of the reference's worker_kernel +
// scheduler_kernel pair (persistent_kernel.cuh:454-974) with the scheduling done ahead of
// time on the host (static assignment, as the reference's schedulers do round-robin at run
// time) and every SM used as a worker.
#pragma once
#include "megakernel.cuh"
#include "runners.cuh"

namespace ypk {

// 176 bytes = 11 x 16
__device__ __forceinline__ void copy_task(ypk_task *dst, const ypk_task *src, int idx, int stride) {
  const uint4 *s = reinterpret_cast<const uint4 *>(src);
  uint4 *d = reinterpret_cast<uint4 *>(dst);
  for (int i = idx; i < int(sizeof(ypk_task) / 16); i += stride) d[i] = __ldg(s + i);
}

// Spin (bounded) until the control word carries iteration `iter`.  One thread.
__device__ __forceinline__ bool wait_iteration(const WaitCtx &wc, long long iter,
                                               unsigned long long *word_out) {
  const unsigned long long *p = wc.rt->ctrl + kCtrlPublished;
  unsigned long long t0 = 0;
  for (uint32_t it = 0;; ++it) {
    const unsigned long long w = ld_acquire_u64(p);
    if ((long long)(w >> 32) >= iter) {
      *word_out = w;
      return true;
    }
    __nanosleep(40);
    if ((it & 63u) == 63u) {
      if (t0 == 0) t0 = globaltimer();
      if (abort_seen(wc)) return false;
      if (globaltimer() - t0 > wc.rt->budget_ns) {
        raise_abort(wc, YPK_ERR_TIMEOUT, -3);
        return false;
      }
    }
  }
}

__device__ __forceinline__ unsigned long long make_word(long long iter, unsigned state, int ntok) {
  return (static_cast<unsigned long long>(iter) << 32) |
         (static_cast<unsigned long long>(state) << 16) | static_cast<unsigned long long>(ntok);
}

// Kernel variants.  TP: tensor-parallel code (all-reduce tasks, arg-max exchange, pushes of
// partial sums to peers).  WIDE: more than 8 tokens per iteration (16-token and tcgen05
// LINEAR paths, TMEM).  What a configuration cannot run is not called from its variant:
// <false, false> one GPU decode, <true, false> tensor-parallel decode, <true, true> the rest.
template <bool TP, bool WIDE, bool MOE = false>
__device__ __forceinline__ void megakernel_body(const Runtime &rt) {
  extern __shared__ __align__(1024) char smem[];
  Misc *misc = reinterpret_cast<Misc *>(smem + kOffMisc);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int worker = blockIdx.x;
  const bool is_producer = warp == kProducerWarp;

  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&misc->full_bar[s], 1);
      mbar_init(&misc->empty_bar[s], kConsumerWarps);
    }
    for (int s = 0; s < kUmmaUnits; ++s) {
      mbar_init(&misc->xfull_bar[s], 1);
      mbar_init(&misc->xempty_bar[s], 1);
    }
    mbar_init(&misc->acc_bar, 1);
    misc->flag = 0;
    misc->abort_flag = 0;
    misc->tmem_base = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  // The tensor maps live in global memory and were written by the host (a copy before the
  // launch): a thread has to acquire each of them through the tensor-map proxy before it hands
  // it to the TMA unit, or the unit may still hold an older map that lived at the same address
  // (a graph loaded earlier into memory the allocator has since handed out again).  Every
  // thread does it for every map once, here.
  for (int m = 0; m < rt.num_tmaps; ++m) {
    asm volatile("fence.proxy.tensormap::generic.acquire.sys [%0], 128;" ::"l"(
                     static_cast<const char *>(rt.tmaps) + size_t(m) * 128)
                 : "memory");
  }
  // Accumulator columns of the tensor-core LINEAR path: taken once, for the kernel's lifetime.
  if (WIDE && rt.use_tmem) {
    if (warp == 0) tmem_alloc(misc);
    tcgen05_before_sync();
    __syncthreads();
    tcgen05_after_sync();
  }

  const int q0 = __ldg(rt.queue_off + worker), q1 = __ldg(rt.queue_off + worker + 1);
  WaitCtx wc{&rt, misc, worker, -1, false};
  // swizzled TMA boxes assume ring stages on 1 KB boundaries
  if (tid == 0 && (smem_u32(smem) & 1023u) != 0u) raise_abort(wc, YPK_ERR_STATE, -4);
  RingPos pos;
  UmmaState ustate;
  long long iter = rt.base_iter;
  long long wide_iter = rt.base_wide;   // iterations of more than two tokens so far
  long long tasks_done = 0, umma_done = 0;
  unsigned long long policy = 0;
  if (is_producer) policy = policy_evict_first();

  // Worker 0 opens the first iteration: either a batch is pending from a paused launch
  // (its token count sits in the low bits of the control word) or the batcher forms one.
  if (rt.mode == 1 && worker == 0 && tid == 0) {
    int ntok;
    if (rt.resume_pending) {
      ntok = int(rt.ctrl[kCtrlPublished] & 0xffffull);
      build_query_tiles(rt);   // the batch may have been formed by a launch of another graph
    } else {
      ntok = prepare_next_batch(rt, false);
    }
    if (ntok < 0) {
      raise_abort(wc, YPK_ERR_STATE, -7);   // KV page pool exhausted
    } else {
      if (ntok == 0) rt.ctrl[kCtrlFinished] = 1ull;
      __threadfence();
      st_release_u64(rt.ctrl + kCtrlPublished,
                     make_word(iter + 1, ntok > 0 ? kStateRun : kStateStop, ntok));
    }
  }

  bool ok = true;
  int iters_here = 0;
  while (ok) {
    ++iter;
    int batch = rt.fixed_batch;
    if (rt.mode == 1) {
      unsigned long long word = 0;
      if (is_producer) {
        int good = 1;
        if (lane == 0) good = wait_iteration(wc, iter, &word) ? 1 : 0;
        ok = __shfl_sync(0xffffffffu, good, 0) != 0;
        word = __shfl_sync(0xffffffffu, word, 0);
        // K/V written with ordinary stores in earlier iterations is read by bulk copies
        asm volatile("fence.proxy.async;" ::: "memory");
      } else {
        if (tid == 0) {
          const bool good = wait_iteration(wc, iter, &word);
          misc->ctrl_word = word;
          misc->flag = good ? 1 : 0;
        }
        consumer_bar();
        word = misc->ctrl_word;
        ok = misc->flag != 0;
        consumer_bar();
      }
      if (!ok) break;
      if (((word >> 16) & 0xffffull) == kStateStop) break;
      batch = int(word & 0xffffull);
    }

    if (batch > 2) ++wide_iter;
    if (is_producer) {
      // ---------------------------------------------------------------- producer
      for (int q = q0; q < q1 && ok; ++q) {
        const int ti = __ldg(rt.queue + q);
        copy_task(&misc->ptask, rt.tasks + ti, lane, 32);
        __syncwarp();
        wc.task = ti;
        const ypk_task &t = misc->ptask;
        if (MOE && t.type == YPK_TASK_LINEAR && (t.flags & YPK_F_MOE)) {
          // the expert whose rows are streamed is known once the router has run
          int go = 1;
          if (lane == 0) go = moe_resolve(wc, rt, &misc->ptask, iter, true);
          go = __shfl_sync(0xffffffffu, go, 0);
          __syncwarp();   // lane 0 rewrote the task copy
          if (go < 0) ok = false;
          if (go <= 0) continue;
        }
        if (t.type == YPK_TASK_LINEAR || t.type == YPK_TASK_ATTENTION) {
          const ProdRet r = run_produce<WIDE>(&rt, misc, smem, worker, ti, batch, pos, policy);
          pos = r.pos;
          ok = r.ok;
        }
        __syncwarp();
      }
    } else {
      // ---------------------------------------------------------------- consumers
      for (int q = q0; q < q1 && ok; ++q) {
        const int ti = __ldg(rt.queue + q);
        if (tid < int(sizeof(ypk_task) / 16)) copy_task(&misc->ctask, rt.tasks + ti, tid, 11);
        wc.task = ti;
        consumer_bar();
        const ypk_task &t = misc->ctask;
        unsigned long long *prec = nullptr;
        if (rt.prof != nullptr && tid == 0 && q - q0 < rt.prof_stride) {
          prec = rt.prof + (size_t(worker) * rt.prof_stride + (q - q0)) * 8;
          prec[0] = (static_cast<unsigned long long>(iter) << 32) | unsigned(ti);
          prec[1] = globaltimer();
          prec[4] = prec[5] = prec[6] = prec[7] = 0ull;
        }
        if (tid == 0) misc->prof_rec = prec;
        // (a LINEAR task whose flagged input is optional polls it instead in small iterations)
        if (t.dep_event >= 0 && !((t.flags & YPK_F_LL_OPT) && batch <= 2)) {
          if (tid == 0) {
            // an event that is published in iterations of more than two tokens only
            // (YPK_F_TRIG_WIDE on its producers) is counted in those iterations
            const unsigned long long need =
                static_cast<unsigned long long>(t.dep_count) *
                static_cast<unsigned long long>((t.flags & YPK_F_LL_OPT) ? wide_iter : iter);
            misc->flag = wait_counter(wc, rt.events + t.dep_event, need, t.dep_event) ? 1 : 0;
          }
          consumer_bar();
          ok = misc->flag != 0;
        }
        if (prec) prec[2] = globaltimer();
        if (MOE && ok && t.type == YPK_TASK_LINEAR && (t.flags & YPK_F_MOE)) {
          if (tid == 0) moe_resolve(wc, rt, &misc->ctask, iter, false);   // may turn the task into a NOP
          consumer_bar();
        }
        if (ok) {
          if (t.type == YPK_TASK_LINEAR) {
            if (WIDE && linear_uses_umma(rt, t, batch)) {
              linear_consume_umma(wc, smem, misc, misc->ctask, batch, pos, ustate);
              ++umma_done;
            } else if (t.flags & (YPK_F_LL_IN | YPK_F_LL_RES | YPK_F_LL_OUT)) {
              if (!WIDE && batch <= 2) {
                // the one- and two-token form of the flagged-word path is part of this loop:
                // a call costs about a microsecond per task (registers saved and restored
                // through local memory, which misses the small L1 left beside the ring)
                linear_consume_groups<true, TP, false>(wc, smem, misc, rt, misc->ctask, batch, iter, pos);
              } else {
                const TaskRet r =
                    batch > 2 ? run_linear<true, TP, true>(&rt, misc, smem, worker, ti, wc.failed, batch, iter, pos)
                              : run_linear<true, TP, false>(&rt, misc, smem, worker, ti, wc.failed, batch, iter, pos);
                pos = r.pos;
                wc.failed = r.failed;
              }
            } else if (WIDE && (batch > kMaxBatch || t.iarg[15] != 0)) {
              // more than 8 tokens, or a task that covers a K range only (the 16-token pass
              // is the GEMV path that can leave partial sums for the split along K)
              const TaskRet r = run_linear16(&rt, misc, smem, worker, ti, wc.failed, batch, pos);
              pos = r.pos;
              wc.failed = r.failed;
            } else {
              const TaskRet r =
                  batch > 2 ? run_linear<false, false, true>(&rt, misc, smem, worker, ti, wc.failed, batch, iter, pos)
                            : run_linear<false, false, false>(&rt, misc, smem, worker, ti, wc.failed, batch, iter, pos);
              pos = r.pos;
              wc.failed = r.failed;
            }
          } else if (t.type == YPK_TASK_ATTENTION) {
            if (!WIDE) {
              // (one call level less: the two forms of the task are functions of their own)
              attention_consume(wc, smem, misc, rt, misc->ctask, iter, pos);
            } else {
              const TaskRet r = run_attention(&rt, misc, smem, worker, ti, wc.failed, iter, pos);
              pos = r.pos;
              wc.failed = r.failed;
            }
          } else {
            wc.failed = run_small<TP>(&rt, misc, worker, ti, wc.failed, batch, iter);
          }
          // a wait that gave up inside the task is known to one warp only: agree on it.
          if (wc.failed) misc->abort_flag = 1;
          consumer_bar();
          ok = misc->abort_flag == 0;
          // The barrier orders every thread's global writes before thread 0; its gpu-scope
          // release on the counter is cumulative over them, so a waiter that acquires the
          // counter sees the task's output.
          if (ok && t.trig_event >= 0 && tid == 0 && !((t.flags & YPK_F_TRIG_WIDE) && batch <= 2)) {
            red_release_add_u64(rt.events + t.trig_event, 1ull);
          }
        }
        if (prec) prec[3] = globaltimer();
        consumer_bar();  // ctask may be overwritten from here on
        ++tasks_done;
      }
    }

    ++iters_here;
    if (rt.mode == 0) break;

    // ------------------------------------------------------------ iteration boundary
    // Worker 0 waits until every task of the last operator has triggered, runs the
    // batcher and publishes the next iteration (or the stop word).
    if (worker == 0 && !is_producer && ok && tid == 0) {
      bool good = true;
      if (rt.end_event >= 0) {
        good = wait_counter(wc, rt.events + rt.end_event,
                            static_cast<unsigned long long>(rt.end_count) *
                                static_cast<unsigned long long>(iter),
                            rt.end_event);
      }
      if (good) {
        const int ntok = prepare_next_batch(rt, false);
        const bool pause = (rt.max_iters > 0 && iters_here >= rt.max_iters) ||
                           (rt.pause_below > 0 && ntok <= rt.pause_below);
        if (ntok < 0) {
          raise_abort(wc, YPK_ERR_STATE, -7);   // KV page pool exhausted: every waiter leaves
        } else {
          if (ntok == 0) rt.ctrl[kCtrlFinished] = 1ull;
          __threadfence();
          st_release_u64(rt.ctrl + kCtrlPublished,
                         make_word(iter + 1, (ntok == 0 || pause) ? kStateStop : kStateRun, ntok));
        }
      }
    }
  }

  // ------------------------------------------------------------------ drain
  // After an abort the producer can leave with bulk copies in flight: wait (bounded) for
  // the last fill of every stage, so that no copy lands after the CTA has exited.  On
  // the normal path these waits return at once.
  if (is_producer) {
    for (uint32_t s = 0; s < uint32_t(kStages); ++s) {
      if (pos.count <= s) continue;  // never filled
      const uint32_t last_phase = s < pos.slot ? pos.phase : (pos.phase ^ 1u);
      const unsigned long long t0 = globaltimer();
      for (uint32_t it = 0; !mbar_try_wait(&misc->full_bar[s], last_phase); ++it) {
        if ((it & 255u) == 255u && globaltimer() - t0 > rt.budget_ns) break;
      }
    }
  }
  if (tid == 0 && worker == 0 && !is_producer) rt.ctrl[kCtrlWideIters] = (unsigned long long)wide_iter;
  if (tid == 0 && tasks_done) atomicAdd(rt.ctrl + kCtrlTasksDone, (unsigned long long)tasks_done);
  if (tid == 0 && umma_done) atomicAdd(rt.ctrl + kCtrlUmmaTasks, (unsigned long long)umma_done);
  if (WIDE && rt.use_tmem) {
    // After an abort the issuing thread can leave with MMAs in flight: wait (bounded) for
    // them before the columns are handed back.  On the normal path every task has waited.
    if (tid == 0 && ld_relaxed_u64(rt.ctrl + kCtrlAbort) != 0ull) {
      umma_commit(&misc->acc_bar);
      const unsigned long long t0 = globaltimer();
      for (uint32_t it = 0; !mbar_try_wait(&misc->acc_bar, ustate.acc_phase); ++it) {
        if ((it & 255u) == 255u && globaltimer() - t0 > 1000000ull) break;
      }
    }
    tcgen05_before_sync();
    __syncthreads();
    if (warp == 0) tmem_free(misc->tmem_base);
  }
  __syncthreads();
}

}  // namespace ypk
