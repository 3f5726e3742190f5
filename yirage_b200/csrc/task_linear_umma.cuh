// LINEAR task for more than 16 tokens on the 5th-generation tensor cores (tcgen05.mma with
// accumulators in tensor memory).  out[tokens, rows] = x[tokens, K] . W[rows, K]^T for the
// row block and K range of the task, up to 64 tokens per pass.
//
// Operand roles.  The tokens are the M side of the MMA (padded to 64) and the WEIGHT ROWS are
// the N side, up to 256 of them per instruction.  A tcgen05.mma occupies the tensor pipe for
// about 78 ns whatever its shape on this part, so what an instruction consumes decides
// whether the task can follow HBM: with the weights on M (as in the reference's Blackwell
// linear task, tasks/blackwell/linear_sm100_mpk.cuh:31-707: M = 128 weight rows, N = 16
// tokens) an instruction covers at most 4 KB of weights, about what 78 ns of one SM's share of
// HBM delivers, and in practice less; with 128..256 weight rows on N it covers 4..8 KB at
// M = 64.  Operators whose row slab per worker would be narrow (o_proj, down_proj, qkv) are
// cut by the host into row blocks x K ranges instead (split along K, see
// linear_splitk_finish), which also cuts the token bytes each CTA has to fetch.
//
//   B (weights)   tiled TMA through a rank-3 view {64 columns, rows, K / 64} of the weight
//                 with the 128-byte swizzle: one box is 64 rows x one 64-column k-block (8 KB)
//                 and lands as [row][128 B], i.e. as eight 8-row core-matrix groups of the
//                 K-major UMMA layout, 1024 bytes apart.  A ring stage holds `kbs` k-blocks
//                 of the task's whole row block: [k-block][box][64 rows][128 B].  Rows past
//                 the task's block belong to a neighbour (their columns of the accumulator
//                 are never read); rows past the end of the tensor arrive as zeros.
//   A (tokens)    tiled TMA as well, through the same kind of view of the activation tensor:
//                 one box of 64 token rows x one k-block per unit of a second ring of seven
//                 8 KB units, issued by lane 0 of consumer warp 1.  The task must not carry a
//                 fused RMSNorm: graphs of more than 8 tokens keep the norm as an operator of
//                 its own (as the reference does), so the tokens need no arithmetic on their
//                 way in.  (A first version staged them with cp.async and multiplied the norm
//                 weight in place: the generic-to-async proxy fence that every unit then
//                 needs cost about 0.4 us per unit, more than the MMAs of the unit.)
//   D             fp32 in tensor memory: 64 rows (tokens) x Npad columns (weight rows of the
//                 block, padded to 8).  Lane 0 of consumer warp 0 issues four
//                 tcgen05.mma.cta_group::1.kind::f16 (M = 64, N = Npad, K = 16) per k-block;
//                 tcgen05.commit hands weight stages and token units back to their producers
//                 and signals the end.
//   epilogue      tcgen05.ld 32x32b: with M = 64, token t sits in TMEM lane 32 * (t / 16) + t % 16,
//                 so a thread holds one token and reads 8 neighbouring weight rows at a time:
//                 RMS factor, residual or SiLU(gate) * up (the 2 + 2 granules lie inside the
//                 8), stores.  A task that covers only a K range leaves its partial sums in
//                 the workspace instead and the last split finishes the rows.
//
// The TMEM columns are allocated once per CTA when the kernel starts and freed when it ends
// (the reference allocates and frees them inside every task, linear_sm100_mpk.cuh:561,704).
#pragma once
#include "device_common.cuh"
#include "task_linear.cuh"

namespace ypk {

__device__ __forceinline__ int umma_npad(int nrows) { return (nrows + 7) & ~7; }
// 64-row TMA boxes per k-block of the task's row block, and k-blocks per ring stage
__device__ __forceinline__ int umma_nbox(int nrows) { return (nrows + kUmmaBoxRows - 1) / kUmmaBoxRows; }
__device__ __forceinline__ int umma_stage_kblocks(int nrows) {
  return kStageBytes / (umma_nbox(nrows) * kUmmaBoxBytes);
}

// Order in which a worker walks the stages of its K range.  Every task of an operator reads
// the same token rows; if all workers walked K in the same order they would all ask L2 for the
// same 8 KB of tokens at the same moment (measured: the token ring then delivers a k-block per
// microsecond, the tensor pipe could take three).  Each worker therefore starts at its own
// stage and wraps around; the fp32 sum over K is taken in that rotated order.
struct UmmaWalk {
  int nkb, kbs, stages, rot;
  __device__ __forceinline__ UmmaWalk(int nkb_, int kbs_, int worker) : nkb(nkb_), kbs(kbs_) {
    stages = (nkb + kbs - 1) / kbs;
    rot = int((unsigned(worker) * 37u) % unsigned(stages));
  }
  // stage visited at position si: its first k-block and its number of k-blocks
  __device__ __forceinline__ void stage(int si, int &kb, int &nk) const {
    int s = si + rot;
    if (s >= stages) s -= stages;
    kb = s * kbs;
    nk = min(kbs, nkb - kb);
  }
};

// Does this task take the tensor-core path at this batch?  Producer and consumers evaluate
// this identically.  In a graph of more than 8 tokens every eligible task with more than 2
// tokens does (measured on the gated MLP of Llama-3-8B: 16 tokens 0.52 ms against 0.64 ms for
// one 16-token GEMV pass, 64 tokens 0.67 ms against 2.36 ms for four passes);
// YPK_TENSOR_CORE=never keeps the GEMV passes.
__device__ __forceinline__ bool linear_uses_umma(const Runtime &rt, const ypk_task &t, int batch) {
  // a norm carried across two operators exists on this path only (the host has checked the maps)
  if (t.flags & (YPK_F_NORM_OUT | YPK_F_NORM_PRE)) return true;
  if (batch <= 2 || t.iarg[9] < 0 || t.iarg[11] < 0 || rt.umma_policy == 2) return false;
  return (t.flags & (YPK_F_NORM | YPK_F_NORM_NOWEIGHT)) == 0;
}

__device__ __forceinline__ void tma_load_3d_hint(void *dst, const void *tmap, int x, int y, int z,
                                                 unsigned long long *bar, unsigned long long policy) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      ".L2::cache_hint [%0], [%1, {%2, %3, %4}], [%5], %6;" ::"r"(smem_u32(dst)),
      "l"(tmap), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar)), "l"(policy)
      : "memory");
}

// ------------------------------------------------------------------ producer
// Traversal (must match the issuer in linear_consume_umma_group): groups of 64 tokens ->
// stages of `kbs` k-blocks over the task's K range.
__device__ __forceinline__ bool linear_produce_umma(WaitCtx &wc, char *smem, Misc *misc,
                                                    const Runtime &rt, const ypk_task &t, int batch,
                                                    RingPos &pos, unsigned long long policy) {
  const int lane = threadIdx.x & 31;
  const LinearArgs a = linear_args(t);
  const char *tmap = static_cast<const char *>(rt.tmaps) + size_t(t.iarg[9]) * 128;
  const int nbox = umma_nbox(a.nrows), kbs = umma_stage_kblocks(a.nrows);
  const int kb0 = a.k0 / kUmmaKBlock, nkb = a.klen / kUmmaKBlock;
  const int ngroups = (batch + kUmmaMaxBatch - 1) / kUmmaMaxBatch;
  const UmmaWalk walk(nkb, kbs, wc.worker);
  for (int grp = 0; grp < ngroups; ++grp) {
    for (int si = 0; si < walk.stages; ++si) {
      int kb, nk;
      walk.stage(si, kb, nk);
      if (!wait_mbar(wc, &misc->empty_bar[pos.slot], pos.phase ^ 1u)) return false;
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      char *stage = smem + kOffRing + pos.slot * kStageBytes;
      if (lane == 0) mbar_expect_tx(&misc->full_bar[pos.slot], uint32_t(nk * nbox) * kUmmaBoxBytes);
      __syncwarp();
      if (lane < nk * nbox) {
        const int j = lane / nbox, bx = lane - j * nbox;
        tma_load_3d_hint(stage + lane * kUmmaBoxBytes, tmap, 0, a.row0 + bx * kUmmaBoxRows, kb0 + kb + j,
                         &misc->full_bar[pos.slot], policy);
      }
      pos.advance();
    }
  }
  return true;
}

// ------------------------------------------------------------------ tcgen05 wrappers
// Shared-memory matrix descriptor of a K-major operand with 128-byte rows and 128-byte
// swizzle (8 rows x 128 B core groups, 1024-byte aligned); `sbo` is the byte distance
// between consecutive 8-row groups.
__device__ __forceinline__ unsigned long long umma_smem_desc(const void *tile, uint32_t sbo) {
  unsigned long long d = 0;
  d |= static_cast<unsigned long long>((smem_u32(tile) & 0x3ffffu) >> 4);  // start address
  d |= 1ull << 16;                                  // leading byte offset: unused with a swizzle
  d |= static_cast<unsigned long long>(sbo >> 4) << 32;
  d |= 1ull << 46;                                  // descriptor version of sm_100
  d |= 2ull << 61;                                  // SWIZZLE_128B
  return d;
}
// Instruction descriptor of kind::f16: fp32 accumulate, A and B K-major, dense.
__device__ __forceinline__ uint32_t umma_instr_desc(int M, int N, bool f16) {
  uint32_t d = 0;
  d |= 1u << 4;                   // D: fp32
  d |= (f16 ? 0u : 1u) << 7;      // A: fp16 / bf16
  d |= (f16 ? 0u : 1u) << 10;     // B
  d |= uint32_t(N >> 3) << 17;
  d |= uint32_t(M >> 4) << 24;
  return d;
}
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, unsigned long long adesc,
                                         unsigned long long bdesc, uint32_t idesc, bool accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate ? 1u : 0u)
      : "memory");
}
// Arrives on `bar` once every tcgen05.mma this thread has issued so far has completed.
__device__ __forceinline__ void umma_commit(unsigned long long *bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, float (&v)[8]) {
  uint32_t r[8];
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
                 "=r"(r[7])
               : "r"(taddr)
               : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, "
      "%13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
        "=r"(r[15])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
// 32 columns per thread in one instruction (one wait for four 8-column groups)
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, "
      "%13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
        "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]),
        "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]),
        "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tcgen05_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

// Called by warp 0 of the CTA, all lanes.  Writes the base address to misc->tmem_base.
__device__ __forceinline__ void tmem_alloc(Misc *misc) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(&misc->tmem_base)),
               "r"(uint32_t(kUmmaTmemCols))
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_free(uint32_t base) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base),
               "r"(uint32_t(kUmmaTmemCols))
               : "memory");
}

// cp.async.wait_group with a run-time count (the instruction takes an immediate).
__device__ __forceinline__ void cp_async_wait_pending(int n) {
  switch (n) {
    case 0: asm volatile("cp.async.wait_group 0;" ::: "memory"); break;
    case 1: asm volatile("cp.async.wait_group 1;" ::: "memory"); break;
    case 2: asm volatile("cp.async.wait_group 2;" ::: "memory"); break;
    case 3: asm volatile("cp.async.wait_group 3;" ::: "memory"); break;
    case 4: asm volatile("cp.async.wait_group 4;" ::: "memory"); break;
    default: asm volatile("cp.async.wait_group 5;" ::: "memory"); break;
  }
}

// ------------------------------------------------------------------ MMA issuer
// Warp 0 of the consumers, all lanes; lane 0 issues.  Walks the weight stages of the task
// from ring position (is_slot, is_phase) and the token units from (is_xslot, is_xphase) of
// the misc area; leaves the warp's failure state in is_failed.
template <bool F16>
static __device__ __noinline__ void umma_issue(const Runtime *rt, Misc *misc, char *smem) {
  const int lane = threadIdx.x & 31;
  const int nrows = misc->is_nrows, nkb = misc->is_nkb;
  uint32_t slot = misc->is_slot, phase = misc->is_phase, xslot = misc->is_xslot, xphase = misc->is_xphase;
  WaitCtx wc{rt, misc, int(blockIdx.x), misc->is_task, misc->is_failed != 0};
  if (nrows <= 0 || nrows > kMaxAccRows || nkb <= 0 || slot >= uint32_t(kStages) ||
      xslot >= uint32_t(kUmmaUnits)) {
    // arguments that cannot be: give up (recorded as event -9) instead of walking them
    if (lane == 0) {
      raise_abort(wc, YPK_ERR_STATE, -9);
      misc->is_failed = 1;
    }
    __syncwarp();
    return;
  }
  char *xring = smem + kOffXs;
  const int nbox = umma_nbox(nrows), kbs = umma_stage_kblocks(nrows);
  const UmmaWalk walk(nkb, kbs, wc.worker);
  const uint32_t tmem = misc->tmem_base;
  const uint32_t idesc = umma_instr_desc(kUmmaMaxBatch, umma_npad(nrows), F16);
  // timeline (lane 0): [4] first stage in hand, [5] last MMA issued, [6] / [7] ns spent
  // waiting for weight stages / token units
  unsigned long long *prec = lane == 0 ? misc->prof_rec : nullptr;
  unsigned long long wait_w = 0, wait_x = 0;
  for (int si = 0; si < walk.stages; ++si) {
    int kb, nk;
    walk.stage(si, kb, nk);
    unsigned long long tw = prec ? globaltimer() : 0ull;
    const bool got = wait_mbar(wc, &misc->full_bar[slot], phase);
    if (prec) {
      const unsigned long long now = globaltimer();
      wait_w += now - tw;
      if (si == 0) prec[4] = now;
    }
    const char *stage = smem + kOffRing + slot * kStageBytes;
    for (int j = 0; j < nk; ++j) {
      tw = prec ? globaltimer() : 0ull;
      const bool xok = wait_mbar(wc, &misc->xfull_bar[xslot], xphase);
      if (prec) wait_x += globaltimer() - tw;
      if (got && xok && lane == 0) {
        tcgen05_after_sync();
        const unsigned long long ad = umma_smem_desc(xring + xslot * kUmmaUnitBytes, 1024);
        const unsigned long long bd = umma_smem_desc(stage + j * nbox * kUmmaBoxBytes, 1024);
#pragma unroll
        for (int kk = 0; kk < kUmmaKBlock / 16; ++kk) {
          // 32 bytes per 16-wide K step inside the swizzle atom: +2 in the address field
          umma_f16(tmem, ad + 2ull * kk, bd + 2ull * kk, idesc, si + j > 0 || kk > 0);
        }
        umma_commit(&misc->xempty_bar[xslot]);   // the unit is free once these have run
      }
      if (++xslot == uint32_t(kUmmaUnits)) {
        xslot = 0;
        xphase ^= 1u;
      }
    }
    if (got && !wc.failed) {
      if (lane == 0) {
        umma_commit(&misc->empty_bar[slot]);   // one of the 8 arrivals, when the MMAs are done
      } else if (lane < kConsumerWarps) {
        mbar_arrive(&misc->empty_bar[slot]);   // the other 7: nothing else reads the stage
      }
    }
    __syncwarp();
    if (++slot == uint32_t(kStages)) {
      slot = 0;
      phase ^= 1u;
    }
  }
  if (lane == 0) {
    umma_commit(&misc->acc_bar);
    misc->is_failed = wc.failed ? 1 : 0;
  }
  if (prec) {
    prec[5] = globaltimer();
    prec[6] = wait_w;
    prec[7] = wait_x;
  }
  __syncwarp();
}

// ------------------------------------------------------------------ consumer
// One group of B <= 64 tokens starting at token b0.
template <bool F16>
__device__ __forceinline__ void linear_consume_umma_group(WaitCtx &wc, char *smem, Misc *misc,
                                                          const LinearArgs &a, int b0, int B,
                                                          RingPos &pos, UmmaState &us) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  char *xring = smem + kOffXs;                       // kUmmaUnits x 8 KB
  constexpr bool norm = false;   // a fused norm keeps the task on the GEMV path (linear_uses_umma)
  const bool silu = (a.flags & YPK_F_SILU_MUL) != 0;
  const int Npad = umma_npad(a.nrows);
  const int nbox = umma_nbox(a.nrows), kbs = umma_stage_kblocks(a.nrows);
  const int nkb = a.klen / kUmmaKBlock;              // k-blocks of the task = token units
  const UmmaWalk walk(nkb, kbs, wc.worker);
  const uint32_t tmem = misc->tmem_base;
  // sums of squares over this task's K range, turned into the RMS factors in place
  float *ssum = misc->rnorm_umma;
  // a norm carried over from the producing operator (YPK_F_NORM_PRE) / on to the next one
  // (YPK_F_NORM_OUT); their scratch is the part of the GEMV area this path does not use
  const bool norm_pre = (a.flags & YPK_F_NORM_PRE) != 0;
  static_assert(kUmmaMaxBatch == 64 && 32 * (kMaxAccRows / 4) * 4 <= kPartBytes, "norm scratch");

  if (warp == 0) {
    // ------------------------------------------------------------ MMA issuer
    // A function of its own, so that its registers are allocated for the issue loop alone
    // (as part of this function the loop ran up to 12 % slower, depending on what the
    // epilogues below happened to need), with its arguments in shared memory: passed on the
    // call stack they cost about a microsecond per task.
    if (lane == 0) {
      misc->is_nrows = a.nrows;
      misc->is_nkb = nkb;
      misc->is_task = wc.task;
      misc->is_failed = wc.failed ? 1 : 0;
      misc->is_slot = pos.slot;
      misc->is_phase = pos.phase;
      misc->is_xslot = us.xslot;
      misc->is_xphase = us.xphase;
    }
    __syncwarp();
    umma_issue<F16>(wc.rt, misc, smem);
    __syncwarp();
    wc.failed = misc->is_failed != 0;
    for (int si = 0; si < walk.stages; ++si) pos.advance();
  } else if (warp == 1) {
    // ------------------------------------------------------------ token loader
    // One tiled-TMA box of 64 token rows x one k-block per unit, in the issuer's order.  The
    // bytes arrive through the async proxy, as the tensor core reads them: no fence, no
    // thread touches them.  (Rows past the batch are rows of the activation buffer that this
    // iteration did not write, or zero fill past its end: they only reach accumulator rows
    // that nobody reads.)
    const char *xmap = static_cast<const char *>(wc.rt->tmaps) + size_t(a.x_tmap) * 128;
    UmmaState xi = us;
    for (int si = 0; si < walk.stages; ++si) {
      int kb, nk;
      walk.stage(si, kb, nk);
      for (int j = 0; j < nk; ++j) {
        const bool free_ok = wait_mbar(wc, &misc->xempty_bar[xi.xslot], xi.xphase ^ 1u);
        if (free_ok && lane == 0) {
          mbar_expect_tx(&misc->xfull_bar[xi.xslot], kUmmaUnitBytes);
          tma_load_3d(xring + xi.xslot * kUmmaUnitBytes, xmap, 0, b0, a.k0 / kUmmaKBlock + kb + j,
                      &misc->xfull_bar[xi.xslot]);
        }
        __syncwarp();
        xi.advance();
      }
      pos.advance();   // keep the weight-ring position in step with the issuer
    }
  } else {
    if (warp == 2 && norm_pre) {
      // RMS factors of the group's tokens from the sums of squares the producing operator
      // left per row block (this warp has nothing else to do while the MMAs run).
      // (misc->rnorm_umma has a slot per token of the group; nothing else uses it in a task
      // with a carried norm until the epilogue, which reads the slots of its 32 tokens at 0..31)
      for (int t = lane; t < B; t += 32) {
        float ssum_t = 0.f;
        for (int blk = 0; blk < a.ss_blk; ++blk)
          ssum_t += __ldcg(a.ss_io + size_t(blk) * a.ss_pitch + b0 + t);
        misc->rnorm_umma[t] = rsqrtf(ssum_t / float(a.K) + a.eps);
      }
    }
    for (int si = 0; si < walk.stages; ++si) pos.advance();
  }
  for (int u = 0; u < nkb; ++u) us.advance();

  wait_mbar(wc, &misc->acc_bar, us.acc_phase);
  us.acc_phase ^= 1u;
  consumer_bar();   // statistics published, every MMA of the group complete
  tcgen05_after_sync();
  if (norm && a.nsplit == 1) {
    if (tid < B) ssum[tid] = rsqrtf(ssum[tid] / float(a.K) + a.eps);
    consumer_bar();
  }

  // Epilogue.  With M = 64, token t is TMEM lane 32 * (t / 16) + t % 16: warp w reads the lane
  // quarter w % 4, whose lower 16 lanes hold tokens 16 * (w % 4) .. + 15, and half of the
  // 8-column groups (8 neighbouring weight rows).
  const int lq = warp & 3, chalf = warp >> 2;
  const int tok = lq * 16 + lane;                 // token of this thread (lanes < 16)
  const bool live = lane < 16 && tok < B;
  const int ncol8 = Npad >> 3;
  const int gmid = (ncol8 + 1) >> 1;
  const int g0 = chalf == 0 ? 0 : gmid, g1 = chalf == 0 ? gmid : ncol8;
  // The accumulator goes to shared memory (the token ring is idle by now), 32 tokens at a time:
  // a warp reads its own quarter of the TMEM lanes, whose lower 16 lanes hold 16 tokens, so
  // the two quarters of a half are read by four warps of 16 live threads; all 256 threads
  // then run the epilogue (or leave the partial sums of a K range) from there.
  const int pitch = Npad + 4;                   // floats; rows stay 16-byte aligned
  float *acc_s = reinterpret_cast<float *>(smem + kOffXs);   // [32][pitch] <= 32 x 260 x 4 B
  for (int half = 0; half * 32 < B && !wc.failed; ++half) {
    if ((lq >> 1) == half && lq * 16 < B) {     // warp-uniform
      float *dst_row = acc_s + ((lq & 1) * 16 + lane) * pitch;
      int g = g0;
      for (; g + 4 <= g1; g += 4) {
        float v[32];
        tmem_ld32(tmem + (uint32_t(lq * 32) << 16) + uint32_t(g * 8), v);
        if (live) {
          float4 *dst = reinterpret_cast<float4 *>(dst_row + g * 8);
#pragma unroll
          for (int i = 0; i < 8; ++i) dst[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
        }
      }
      for (; g < g1; ++g) {
        float v[8];
        tmem_ld8(tmem + (uint32_t(lq * 32) << 16) + uint32_t(g * 8), v);
        if (live) {
          float4 *dst = reinterpret_cast<float4 *>(dst_row + g * 8);
          dst[0] = make_float4(v[0], v[1], v[2], v[3]);
          dst[1] = make_float4(v[4], v[5], v[6], v[7]);
        }
      }
    }
    tcgen05_before_sync();
    consumer_bar();
    const int bh = b0 + half * 32, Bh = min(32, B - half * 32);
    auto acc = [&](int r, int b) { return acc_s[b * pitch + r]; };
    // scratch of a norm carried on (behind the accumulator staging area; the token ring, which
    // covers it, is idle by now)
    float *sq_s = reinterpret_cast<float *>(smem + kOffPart);     // [32 tokens][rows / 4]
    if (norm_pre && half == 1 && tid < Bh) misc->rnorm_umma[tid] = misc->rnorm_umma[32 + tid];   // read after a barrier
    if (a.nsplit > 1) {
      linear_splitk_finish<F16, true>(a, misc, bh, Bh, ssum, acc, sq_s);
    } else {
      if (norm_pre) consumer_bar();
      linear_epilogue_quads<F16>(a, misc, bh, Bh, norm_pre, acc, sq_s);
    }
    consumer_bar();   // the staging area is reused by the next half (and by the next task)
  }
  (void)silu;
  (void)ncol8;
  // the next group's first MMA overwrites the accumulators: order these reads before it
  tcgen05_before_sync();
}

__device__ __forceinline__ void linear_consume_umma(WaitCtx &wc, char *smem, Misc *misc,
                                                    const ypk_task &t, int batch, RingPos &pos,
                                                    UmmaState &us) {
  const LinearArgs a = linear_args(t);
  for (int b0 = 0; b0 < batch; b0 += kUmmaMaxBatch) {
    const int B = min(kUmmaMaxBatch, batch - b0);
    if (a.flags & YPK_F_F16) {
      linear_consume_umma_group<true>(wc, smem, misc, a, b0, B, pos, us);
    } else {
      linear_consume_umma_group<false>(wc, smem, misc, a, b0, B, pos, us);
    }
    consumer_bar();   // the group's shared-memory scratch is dead before the next one starts
  }
}

}  // namespace ypk
