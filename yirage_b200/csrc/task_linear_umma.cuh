// LINEAR task for 9..64 tokens: the fused operator of task_linear.cuh on the 5th-generation
// tensor cores.  With more than 8 tokens the projection is a real dense contraction,
// out^T[rows, batch] = W[rows, K] . x^T[K, batch].  As in the reference's Blackwell linear
// task (tasks/blackwell/linear_sm100_mpk.cuh:31-707) the weights are the M side of the MMA
// and the batch, padded to a multiple of 16, is N.
//
//   A (weights)   tiled TMA through a rank-3 view {64 columns, rows, K / 64} of the weight:
//                 one box is 8 rows x 4 k-blocks (4 KB) and lands as [k-block][row][128 B]
//                 with the 128-byte swizzle, i.e. as four 8-row core-matrix groups of the
//                 K-major UMMA layout.  A ring stage holds one "super-step" of one row
//                 block: up to 8 such boxes (64 rows) x 4 k-blocks, or, for a task of at
//                 most 32 rows, 4 boxes x 8 k-blocks.  Rows past the task's slab are never
//                 read back; rows past the end of the tensor arrive as zeros.
//   B (tokens)    staged by consumer warps 1..7 with 16-byte cp.async into a second ring of
//                 seven 8 KB units (64 / N k-blocks each), same swizzled K-major layout, then
//                 multiplied in place by the norm weight while the RMS statistics are
//                 taken; several units are in flight so that the L2 latency is hidden.
//   D             fp32 accumulators in tensor memory, N columns per 64-row block (at most
//                 four blocks per task) and per partial sum (up to four, see below).  Lane 0 of consumer warp 0 issues tcgen05.mma
//                 (cta_group::1, kind::f16, M = 64, so that a block reads only its own 64
//                 rows of shared memory); tcgen05.commit hands weight stages and token units
//                 back to their producers and signals the end.
//   epilogue      tcgen05.ld 32x32b: with M = 64 row r of a block sits in TMEM lane
//                 32 * (r / 16) + r % 16, i.e. in the lower 16 lanes of warp r / 16 -> RMS
//                 factor, residual or SiLU(gate) * up -> 16-bit stores.
//
// The TMEM columns are allocated once per CTA when the kernel starts and freed when it ends
// (the reference allocates and frees them inside every task, linear_sm100_mpk.cuh:561,704).
#pragma once
#include "device_common.cuh"
#include "task_linear.cuh"

namespace ypk {

__device__ __forceinline__ int umma_n(int batch) { return (batch + 15) / 16 * 16; }
// k-blocks per token-ring unit (8 KB): 4, 2, 1, 1 for N = 16, 32, 48, 64
__device__ __forceinline__ int umma_unit_kblocks(int N) { return kUmmaMaxBatch / N; }

// k-blocks per ring stage: 8 for a task of at most 32 rows (one block, <= 4 boxes per
// k-half), else 4.
__device__ __forceinline__ int umma_step_kblocks(const LinearArgs &a) {
  return (a.nrows <= 32 && (a.K / kUmmaKBlock) % (2 * kUmmaStepKBlocks) == 0) ? 2 * kUmmaStepKBlocks
                                                                             : kUmmaStepKBlocks;
}

// Does this task take the tensor-core path at this batch?  Producer and consumers evaluate
// this identically.  A tcgen05.mma occupies the SM's tensor pipe for about 78 ns whatever M
// and N (measured back to back: 64x16x16 and 128x256x16 alike; about 130 ns each inside this
// task, with its waits and commits), and a task issues K / 16 of them per 64-row block; the
// GEMV path instead streams the weights once per 16 tokens at about 3/4 of the SM's share of
// HBM (44 bytes / ns).  Take whichever is estimated to finish first: with the slabs of an 8B
// model that is the GEMV path up to 32 tokens and, for the wider slabs, the tensor-core path
// beyond.
__device__ __forceinline__ bool linear_uses_umma(const Runtime &rt, const ypk_task &t, int batch) {
  if (batch <= kMaxBatch || batch > kUmmaMaxBatch || t.iarg[9] < 0 || rt.umma_policy == 2 ||
      (t.flags & (YPK_F_LL_IN | YPK_F_LL_RES | YPK_F_LL_OUT)))
    return false;
  if (rt.umma_policy == 1) return true;
  const long long K = t.iarg[0], nrows = t.iarg[2];
  const long long wbytes = nrows * K * 2;
  const long long nblocks = (nrows + kUmmaBlockRows - 1) / kUmmaBlockRows;
  const long long mma_ns = nblocks * (K / 16) * 130;
  const long long umma_ns = max(wbytes / 44, mma_ns);
  const long long gemv_ns = ((batch + kWideBatch - 1) / kWideBatch) * (wbytes / 33);
  return umma_ns < gemv_ns;
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
// Traversal (must match the issuer in linear_consume_umma): super-steps of 4 k-blocks ->
// row blocks of <= 64 rows; one ring stage each.
__device__ __forceinline__ bool linear_produce_umma(WaitCtx &wc, char *smem, Misc *misc,
                                                    const Runtime &rt, const ypk_task &t,
                                                    RingPos &pos, unsigned long long policy) {
  const int lane = threadIdx.x & 31;
  const LinearArgs a = linear_args(t);
  const char *tmap = static_cast<const char *>(rt.tmaps) + size_t(t.iarg[9]) * 128;
  const int KS = umma_step_kblocks(a);
  const int halves = KS / kUmmaStepKBlocks;            // TMA boxes per 8-row group
  const int nss = a.K / (kUmmaKBlock * KS);
  for (int ss = 0; ss < nss; ++ss) {
    for (int r0 = 0; r0 < a.nrows; r0 += kUmmaBlockRows) {
      const int groups = (min(kUmmaBlockRows, a.nrows - r0) + 7) / 8;
      if (!wait_mbar(wc, &misc->empty_bar[pos.slot], pos.phase ^ 1u)) return false;
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      char *stage = smem + kOffRing + pos.slot * kStageBytes;
      if (lane == 0)
        mbar_expect_tx(&misc->full_bar[pos.slot], uint32_t(groups * halves) * kUmmaBoxBytes);
      __syncwarp();
      if (lane < groups * halves) {
        const int g = lane / halves, hf = lane - g * halves;
        tma_load_3d_hint(stage + lane * kUmmaBoxBytes, tmap, 0, a.row0 + r0 + g * 8,
                         ss * KS + hf * kUmmaStepKBlocks, &misc->full_bar[pos.slot], policy);
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

__device__ __forceinline__ void cp_async16_zfill(void *dst, const void *src, bool real) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src),
               "r"(real ? 16u : 0u)
               : "memory");
}

// ------------------------------------------------------------------ consumer
template <bool F16>
__device__ __forceinline__ void linear_consume_umma_t(WaitCtx &wc, char *smem, Misc *misc,
                                                      const LinearArgs &a, int B, RingPos &pos,
                                                      UmmaState &us) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  char *xring = smem + kOffXs;                       // kUmmaUnits x 8 KB
  const uint16_t *x = reinterpret_cast<const uint16_t *>(a.x);
  const uint16_t *nw = reinterpret_cast<const uint16_t *>(a.norm_w);
  const bool norm = (a.flags & (YPK_F_NORM | YPK_F_NORM_NOWEIGHT)) != 0;
  const bool has_nw = (a.flags & YPK_F_NORM) != 0;
  const bool silu = (a.flags & YPK_F_SILU_MUL) != 0;
  const int N = umma_n(B);
  const int XB = umma_unit_kblocks(N);               // k-blocks per unit
  const int nkb = a.K / kUmmaKBlock;                 // multiple of kUmmaStepKBlocks
  const int nunits = nkb / XB;
  const int KS = umma_step_kblocks(a);               // k-blocks per weight stage
  const int nsteps = nkb / KS;
  const int nblocks = (a.nrows + kUmmaBlockRows - 1) / kUmmaBlockRows;
  // Back-to-back MMAs into one accumulator serialise on its read-modify-write (about 100 ns
  // each, whatever M and N), so the four 16-wide K steps of a k-block go to up to four
  // accumulators, summed in the epilogue.
  const int nacc = min(kUmmaKBlock / 16, kUmmaTmemCols / (nblocks * N));
  const uint32_t tmem = misc->tmem_base;

  if (warp == 0) {
    // ------------------------------------------------------------ MMA issuer
    const uint32_t idesc = umma_instr_desc(kUmmaBlockRows, N, F16);
    UmmaState xbase = us;   // unit holding the first k-block of the current step
    // timeline (lane 0): [4] first stage in hand, [5] last MMA issued, [6] / [7] ns spent
    // waiting for weight stages / token units
    unsigned long long *prec = lane == 0 ? misc->prof_rec : nullptr;
    unsigned long long wait_w = 0, wait_x = 0;
    for (int ss = 0; ss < nsteps; ++ss) {
      for (int blk = 0; blk < nblocks; ++blk) {
        unsigned long long tw = prec ? globaltimer() : 0ull;
        const bool got = wait_mbar(wc, &misc->full_bar[pos.slot], pos.phase);
        if (prec) {
          const unsigned long long now = globaltimer();
          wait_w += now - tw;
          if (ss == 0 && blk == 0) prec[4] = now;
        }
        const char *stage = smem + kOffRing + pos.slot * kStageBytes;
        if (got && lane == 0) tcgen05_after_sync();
        UmmaState xu = xbase;
        for (int j = 0; j < KS; ++j) {
          const int ju = j % XB;
          // a token unit is awaited when the first block first touches it ...
          bool xok = true;
          if (blk == 0 && ju == 0) {
            tw = prec ? globaltimer() : 0ull;
            xok = wait_mbar(wc, &misc->xfull_bar[xu.xslot], xu.xphase);
            if (prec) wait_x += globaltimer() - tw;
          }
          if (got && xok && lane == 0) {
            if (blk == 0 && ju == 0) tcgen05_after_sync();
            const unsigned long long ad = umma_smem_desc(stage + j * 1024, uint32_t(KS) * 1024u);
            const unsigned long long bd =
                umma_smem_desc(xring + xu.xslot * kUmmaUnitBytes + ju * N * 128, 1024);
#pragma unroll
            for (int kk = 0; kk < kUmmaKBlock / 16; ++kk) {
              // 32 bytes per 16-wide K step inside the swizzle atom: +2 in the address field
              const int acc = kk % nacc;
              umma_f16(tmem + uint32_t((blk * nacc + acc) * N), ad + 2ull * kk, bd + 2ull * kk,
                       idesc, ss > 0 || j > 0 || kk >= nacc);
            }
            // ... and handed back when the last block is done with it
            if (blk == nblocks - 1 && ju == XB - 1) umma_commit(&misc->xempty_bar[xu.xslot]);
          }
          if (ju == XB - 1) xu.advance();
        }
        if (got && !wc.failed) {
          if (lane == 0) {
            umma_commit(&misc->empty_bar[pos.slot]);   // one of the 8 arrivals, when the MMAs are done
          } else if (lane < kConsumerWarps) {
            mbar_arrive(&misc->empty_bar[pos.slot]);   // the other 7: nothing else reads the stage
          }
        }
        __syncwarp();
        pos.advance();
        if (blk == nblocks - 1) xbase = xu;
      }
    }
    if (lane == 0) umma_commit(&misc->acc_bar);
    if (prec) {
      prec[5] = globaltimer();
      prec[6] = wait_w;
      prec[7] = wait_x;
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ token stagers (7 warps)
    // Thread -> (16-byte chunk c, row b): a warp covers 4 rows x 8 chunks per pass and the
    // 7 warps 28 rows, so a thread sees the same <= 3 rows in every unit.
    const int c = lane & 7, rb = (warp - 1) * 4 + (lane >> 3);
    constexpr int kRowsPerPass = (kConsumerWarps - 1) * 4;                         // 28
    constexpr int kMaxPasses = (kUmmaMaxBatch + kRowsPerPass - 1) / kRowsPerPass;  // 3
    // Units in flight.  The first block of a multi-block task holds every unit of a step
    // (KS / XB of the 7) until the last block has used them, so the copies can only run
    // 7 - KS / XB units ahead of the oldest unit still needed; a one-block task hands its
    // units back as it goes.
    const int kDepth = nblocks == 1 ? 5 : min(5, kUmmaUnits - KS / XB);
    float ssq[kMaxPasses] = {0.f, 0.f, 0.f};
    UmmaState xi = us, xf = us;   // issue / finish positions
    for (int u = 0; u < nunits + kDepth; ++u) {
      if (u < nunits) {
        const bool free_ok = wait_mbar(wc, &misc->xempty_bar[xi.xslot], xi.xphase ^ 1u);
        char *unit = xring + xi.xslot * kUmmaUnitBytes;
        if (free_ok) {
          for (int j = 0; j < XB; ++j) {
            const int k = (u * XB + j) * kUmmaKBlock + c * 8;
            // the norm weights of this unit are wanted a few units from now: bring them to L1
            if (has_nw && rb < B) asm volatile("prefetch.global.L1 [%0];" ::"l"(nw + k));
#pragma unroll
            for (int p = 0; p < kMaxPasses; ++p) {
              const int b = rb + p * kRowsPerPass;
              if (b < N) {
                const int bs = b < B ? b : 0;
                cp_async16_zfill(unit + j * N * 128 + b * 128 + ((c ^ (b & 7)) << 4),
                                 x + size_t(bs) * a.ldx + k, b < B);
              }
            }
          }
        }
        xi.advance();
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
      if (u >= kDepth) {
        const int uf = u - kDepth;
        cp_async_wait_pending(kDepth);
        char *unit = xring + xf.xslot * kUmmaUnitBytes;
        if (norm) {
          for (int j = 0; j < XB; ++j) {
            const int k = (uf * XB + j) * kUmmaKBlock + c * 8;
            uint4 wv = make_uint4(0u, 0u, 0u, 0u);
            if (has_nw) wv = __ldg(reinterpret_cast<const uint4 *>(nw + k));
            const uint32_t q[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
            for (int p = 0; p < kMaxPasses; ++p) {
              const int b = rb + p * kRowsPerPass;
              if (b < B) {
                uint4 *cell = reinterpret_cast<uint4 *>(unit + j * N * 128 + b * 128 +
                                                        ((c ^ (b & 7)) << 4));
                const uint4 v = *cell;
                const uint32_t pv[4] = {v.x, v.y, v.z, v.w};
                uint32_t o[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  const float2 f = unpack2(cvt_pair<F16>(pv[i]));
                  ssq[p] += f.x * f.x + f.y * f.y;
                  if (has_nw) {
                    const float2 g = unpack2(cvt_pair<F16>(q[i]));
                    o[i] = uint32_t(cvt_out<F16>(f.x * g.x)) |
                           (uint32_t(cvt_out<F16>(f.y * g.y)) << 16);
                  } else {
                    o[i] = pv[i];
                  }
                }
                if (has_nw) *cell = make_uint4(o[0], o[1], o[2], o[3]);
              }
            }
          }
        }
        // generic-proxy writes (cp.async, the fix-up) -> visible to the tensor core
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0 && !wc.failed) mbar_arrive(&misc->xfull_bar[xf.xslot]);
        xf.advance();
      }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    if (norm) {
#pragma unroll
      for (int p = 0; p < kMaxPasses; ++p) {
        float s = ssq[p];
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        s += __shfl_xor_sync(0xffffffffu, s, 2);
        s += __shfl_xor_sync(0xffffffffu, s, 4);
        const int b = rb + p * kRowsPerPass;
        if (c == 0 && b < B) misc->rnorm_umma[b] = rsqrtf(s / float(a.K) + a.eps);
      }
    }
    // keep the weight-ring position in step with the issuer
    for (int i = 0; i < nsteps * nblocks; ++i) pos.advance();
  }
  for (int u = 0; u < nunits; ++u) us.advance();

  wait_mbar(wc, &misc->acc_bar, us.acc_phase);
  us.acc_phase ^= 1u;
  consumer_bar();   // RMS factors published, every MMA of the task complete
  tcgen05_after_sync();

  // Epilogue.  With M = 64 row r of a block is TMEM lane 32 * (r / 16) + r % 16: warp w reads
  // the lane quarter w % 4, whose lower 16 lanes hold rows 16 * (w % 4) .. + 15, and half of
  // the token columns.
  const int lq = warp & 3, chalf = warp >> 2;
  if (!wc.failed) {
    for (int blk = 0; blk < nblocks; ++blk) {
      const int r = blk * kUmmaBlockRows + lq * 16 + lane;   // row of the task (lanes < 16)
      const bool live = lane < 16 && r < a.nrows;
      const int p = a.row0 + r;                               // row of the weight
      for (int c0 = chalf * (N / 2); c0 < (chalf + 1) * (N / 2); c0 += 8) {
        float v[8];
        tmem_ld8(tmem + (uint32_t(lq * 32) << 16) + uint32_t(blk * nacc * N + c0), v);
        for (int acc = 1; acc < nacc; ++acc) {
          float v2[8];
          tmem_ld8(tmem + (uint32_t(lq * 32) << 16) + uint32_t((blk * nacc + acc) * N + c0), v2);
#pragma unroll
          for (int i = 0; i < 8; ++i) v[i] += v2[i];
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int b = c0 + i;
          float val = v[i];
          if (norm) val *= misc->rnorm_umma[b < B ? b : 0];
          if (silu) {
            // granules of kSiluGran gate rows then kSiluGran up rows: the partner is 2 lanes on
            const float up = __shfl_down_sync(0xffffffffu, val, kSiluGran);
            if (live && b < B && (p % (2 * kSiluGran)) < kSiluGran) {
              const int col = a.out_col0 + (p / (2 * kSiluGran)) * kSiluGran + p % kSiluGran;
              reinterpret_cast<uint16_t *>(a.out)[size_t(b) * a.ldout + col] =
                  cvt_out<F16>(silu_mul_ref(val, up));
            }
          } else if (live && b < B) {
            const int col = a.out_col0 + p;
            if (a.flags & YPK_F_RESIDUAL) {
              val += cvt_one<F16>(
                  __ldcg(reinterpret_cast<const uint16_t *>(a.res) + size_t(b) * a.ldres + col));
            }
            reinterpret_cast<uint16_t *>(a.out)[size_t(b) * a.ldout + col] = cvt_out<F16>(val);
          }
        }
      }
    }
  }
  // the next task's first MMA overwrites the accumulators: order these reads before it
  tcgen05_before_sync();
}

__device__ __forceinline__ void linear_consume_umma(WaitCtx &wc, char *smem, Misc *misc,
                                                    const ypk_task &t, int batch, RingPos &pos,
                                                    UmmaState &us) {
  const LinearArgs a = linear_args(t);
  if (a.flags & YPK_F_F16) {
    linear_consume_umma_t<true>(wc, smem, misc, a, batch, pos, us);
  } else {
    linear_consume_umma_t<false>(wc, smem, misc, a, batch, pos, us);
  }
}

}  // namespace ypk
