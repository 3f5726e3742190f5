// ATTENTION task: GQA incremental-decode / chunked-prefill attention over a paged bf16
// KV cache for one (request, kv head, KV split).
//
// Semantics follow the reference's paged attention task
// (tasks/blackwell/attention_sm100.cuh:33-660): packed QKV rows laid out per kv head as
// [q_per_kv q heads | k | v], rotate-half RoPE on the new q and k with bf16 cos/sin rows
// (tasks/blackwell/rotary_embedding_sm100.cuh:56-73), the rotated k and v of the new
// tokens are written into their page slots, causal softmax with scale 1/sqrt(128) in
// fp32, P rounded to bf16 before P.V (as the reference's mma does), bf16 output.
// Differences by design: the sequence is split across CTAs (split-KV) and, inside a CTA,
// across warps; partial results are merged in shared memory and, across CTAs, by whichever
// split finishes last; the K/V tiles arrive through the producer warp's bulk copies
// instead of cp.async; and the sequence length is (pages-1)*page_size + last_page_len with
// last_page_len in [1, page_size] (the reference's 0-when-full convention under-counts by
// a page, attention_sm100.cuh:101-102).
//
// Mapping: a ring stage holds 64 cached tokens of one kv head, fetched as four tiled-TMA
// boxes (K / V x low / high 64 dims) with the 128-byte swizzle that keeps ldmatrix conflict
// free.  The query rows (new tokens x q heads of the
// group, <= 32) form one or two 16-row MMA tiles.  Every 64-token stage is owned by ONE
// warp, which runs the whole flash-attention step on it with m16n8k16 MMAs: S = Q.K^T
// (K as the col-major operand straight from its rows), online softmax in the log2 domain
// on the accumulator fragments (row max/sum by quad shuffles), P.V with V through
// ldmatrix.trans.  Warps own stages round-robin, so up to five tiles are in flight.
#pragma once
#include "device_common.cuh"
#include <type_traits>
#include "ll_handoff.cuh"
#include "task_linear.cuh"  // ldmatrix_x4, mma_16816

namespace ypk {

struct AttnShape {
  int T;         // new tokens this task takes (all of the request's, or one query tile of them)
  int pre;       // new tokens of the request in this iteration that come before those
  int qo0;       // row of the task's first token in the packed qkv / output
  int kv0;       // first entry of the request in kv_indices
  int seq_len;   // tokens up to and including the task's own
  int cached;    // tokens the pages held before this iteration = seq_len - pre - T
  int tile0, tile1;  // cached 64-token tiles of this split
  int nact;      // active splits of this (request, head)
  bool active, handles_new;
};

__device__ __forceinline__ AttnShape attn_shape(const Runtime &rt, const ypk_task &t) {
  AttnShape s;
  int r = t.iarg[0];
  const int split = t.iarg[2], nsplit = t.iarg[3];
  int tile = 0;
  if (t.flags & YPK_F_QTILES) {
    // iarg[0] names an entry of the iteration's query-tile list instead of a request slot
    tile = __ldcg(rt.qtiles + r);
    r = tile < 0 ? 0 : (tile & 0xfff);
  }
  const int qo = __ldcg(rt.qo_indptr + r);
  const int treq = __ldcg(rt.qo_indptr + r + 1) - qo;
  s.pre = (t.flags & YPK_F_QTILES) ? ((tile >> 12) & 0xff) : 0;
  s.T = (t.flags & YPK_F_QTILES) ? (tile < 0 ? 0 : (tile >> 20)) : treq;
  s.qo0 = qo + s.pre;
  s.kv0 = __ldcg(rt.kv_indptr + r);
  const int npages = __ldcg(rt.kv_indptr + r + 1) - s.kv0;
  s.cached = (npages - 1) * rt.page_size + __ldcg(rt.kv_last_len + r) - treq;
  s.seq_len = s.cached + s.pre + s.T;
  const int tiles = (s.cached + kKvTile - 1) / kKvTile;
  const int want = min(nsplit, (tiles + kAttnTilesPerSplit - 1) / kAttnTilesPerSplit);
  const int tps = max(1, (tiles + max(want, 1) - 1) / max(want, 1));
  s.nact = tiles > 0 ? (tiles + tps - 1) / tps : 1;
  s.active = s.T > 0 && s.T <= kMaxNewTokens && s.T * t.iarg[4] <= kMaxAttnRows &&
             s.pre + s.T <= kMaxNewKeys && npages > 0 && split < s.nact;
  s.tile0 = min(tiles, split * tps);
  s.tile1 = min(tiles, s.tile0 + tps);
  s.handles_new = split == s.nact - 1;
  return s;
}

// ------------------------------------------------------------------ producer
__device__ __forceinline__ bool attention_produce(WaitCtx &wc, char *smem, Misc *misc,
                                                  const Runtime &rt, const ypk_task &t,
                                                  RingPos &pos) {
  const int lane = threadIdx.x & 31;
  const AttnShape s = attn_shape(rt, t);
  if (!s.active) return true;
  const int h = t.iarg[1];
  const char *ktm = static_cast<const char *>(rt.tmaps) + size_t(t.iarg[9]) * 128;
  const char *vtm = static_cast<const char *>(rt.tmaps) + size_t(t.iarg[10]) * 128;
  for (int tile = s.tile0; tile < s.tile1; ++tile) {
    const int tok0 = tile * kKvTile;
    const int page = __ldcg(rt.kv_indices + s.kv0 + tok0 / rt.page_size);
    const size_t row0 = size_t(page) * rt.page_size + (tok0 % rt.page_size);
    if (!wait_mbar(wc, &misc->empty_bar[pos.slot], pos.phase ^ 1u)) return false;
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // consumers may have zero-padded
    char *stage = smem + kOffRing + pos.slot * kStageBytes;
    // One K or V row of a kv head is only 256 contiguous bytes; as separate bulk copies they
    // are limited by the TMA engine's per-copy cost and as cp.async by one warp's loads in
    // flight.  The tiled TMA path moves a 64-token x 64-dim box (8 KB) per instruction.  The
    // box is always 64 tokens: a tile never crosses a page (page_size % 64 == 0), rows past
    // the sequence end are masked by the consumer.
    if (lane == 0) {
      mbar_expect_tx(&misc->full_bar[pos.slot], 4u * kKvBoxBytes);
      const int z = int(row0);
      tma_load_3d(stage, ktm, 0, h, z, &misc->full_bar[pos.slot]);
      tma_load_3d(stage + kKvBoxBytes, ktm, 64, h, z, &misc->full_bar[pos.slot]);
      tma_load_3d(stage + kVOffset, vtm, 0, h, z, &misc->full_bar[pos.slot]);
      tma_load_3d(stage + kVOffset + kKvBoxBytes, vtm, 64, h, z, &misc->full_bar[pos.slot]);
    }
    __syncwarp();
    pos.advance();
  }
  return true;
}

// ------------------------------------------------------------------ consumer
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void *smem_row) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(smem_row)));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  return uint32_t(__bfloat16_as_ushort(__float2bfloat16_rn(lo))) |
         (uint32_t(__bfloat16_as_ushort(__float2bfloat16_rn(hi))) << 16);
}

// Flash-attention state of one warp for a 16-row query tile.  A lane holds rows
// lane/4 ("lo") and lane/4 + 8 ("hi"); per 8-wide block of head dims the four values are
// {lo[d], lo[d+1], hi[d], hi[d+1]} with d = (lane % 4) * 2.
struct AttnAcc {
  float o[kHeadDim / 8][4];
  float m[2];   // running max (log2 domain), rows lo / hi
  float l[2];   // this lane's share of the running sum
};

// One 64-token tile (or the new-token mini tile): S = Q K^T, online softmax, O += P V.
// ksm / vsm: rows of 128 bf16 at kKPitch.  `ntok` valid tokens; when `causal`, token j is
// visible to query row (t, g) only if j <= t + pre (rows are numbered t * G + g; `pre` new
// tokens of the same request precede the query rows' own).
// SWZ: ksm / vsm are TMA stages (two 64x128-byte boxes each, 128-byte swizzle: the 16-byte
// chunk c of row r sits at chunk c ^ (r & 7)); otherwise plain rows at kKPitch.
template <bool SWZ>
__device__ __forceinline__ void attn_tile_mma(const char *qsm, const char *ksm, char *vsm,
                                              int ntok, bool causal, int G, int row_base,
                                              int lane, AttnAcc &acc, int pre = 0) {
  // 1/sqrt(128) * log2(e): scores live in the log2 domain so exp2f can be used
  const float qscale = 0.08838834764831845f * 1.4426950408889634f;
  const int nblk = (ntok + 7) >> 3;        // 8-token blocks with at least one valid token
  const int nk16 = (ntok + 15) >> 4;       // 16-token steps of P.V
  if (ntok < nk16 * 16) {
    // P is zero for the padding tokens of the last 16-token step, but 0 * (stale bytes that
    // happen to be Inf/NaN) would poison the row: clear those V rows.  The generic-proxy
    // stores are fenced against the bulk copy that refills the stage later.
    for (int i = lane; i < (nk16 * 16 - ntok) * (kHeadDim / 8); i += 32) {
      const int row = ntok + i / (kHeadDim / 8), c = i % (kHeadDim / 8);
      char *dst = SWZ ? vsm + (c >> 3) * kKvBoxBytes + row * 128 + (c & 7) * 16  // whole row: any order
                      : vsm + row * kKPitch + c * 16;
      *reinterpret_cast<uint4 *>(dst) = make_uint4(0u, 0u, 0u, 0u);
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncwarp();
  }
  float s[kKvTile / 8][4];
#pragma unroll
  for (int nb = 0; nb < kKvTile / 8; ++nb) s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.f;

  // lane-constant address parts
  const char *qrow = qsm + (row_base + ((lane >> 3) & 1) * 8 + (lane & 7)) * kKPitch +
                     ((lane >> 4) & 1) * 16;
  const char *krow = ksm + (lane & 7) * kKPitch + (lane >> 3) * 16;   // plain layout
  const int sw = lane & 7;  // row & 7 of every ldmatrix row this lane addresses
  // The asm statements keep program order and a warp issues in order, so fragment loads are
  // grouped four at a time ahead of the MMAs that use them: their latencies overlap.
#pragma unroll
  for (int kp = 0; kp < kHeadDim / 32; ++kp) {   // pairs of 16-wide steps over the head dim
    uint32_t q0[4], q1[4];
    ldmatrix_x4(q0, qrow + kp * 64);
    ldmatrix_x4(q1, qrow + kp * 64 + 32);
#pragma unroll
    for (int nq = 0; nq < kKvTile / 32; ++nq) {   // groups of four 8-token blocks
      if (nq * 4 < nblk) {
        uint32_t kf[4][4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int nb = nq * 4 + j;
          if constexpr (SWZ) {
            const int cg = kp * 4 + (lane >> 3);  // 16-byte chunk of the 256-byte row
            ldmatrix_x4(kf[j], ksm + (cg >> 3) * kKvBoxBytes + (nb * 8 + sw) * 128 +
                                   (((cg & 7) ^ sw) << 4));
          } else {
            ldmatrix_x4(kf[j], krow + nb * 8 * kKPitch + kp * 64);
          }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          mma_16816<false>(s[nq * 4 + j], q0, kf[j][0], kf[j][1]);
          mma_16816<false>(s[nq * 4 + j], q1, kf[j][2], kf[j][3]);
        }
      }
    }
  }
  // scale, mask, row max
  const int r_lo = row_base + (lane >> 2), r_hi = r_lo + 8;
  const int t_lo = r_lo / G, t_hi = r_hi / G;
  float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
  for (int nb = 0; nb < kKvTile / 8; ++nb) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int tok = nb * 8 + (lane & 3) * 2 + (e & 1);
      const int tq = (e & 2) ? t_hi : t_lo;
      const bool vis = nb < nblk && tok < ntok && (!causal || tok <= tq + pre);
      s[nb][e] = vis ? s[nb][e] * qscale : -INFINITY;
      mx[e >> 1] = fmaxf(mx[e >> 1], s[nb][e]);
    }
  }
  float corr[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
    mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
    const float m_new = fmaxf(acc.m[h], mx[h]);
    // a row that has seen nothing yet keeps m = -inf; use 0 as the exponent base then
    const float base = m_new == -INFINITY ? 0.f : m_new;
    corr[h] = exp2f(acc.m[h] - base);   // exp2f(-inf) = 0
    acc.m[h] = m_new;
    mx[h] = base;
    acc.l[h] *= corr[h];
  }
  // p = exp2(s - m), packed to bf16 A fragments of the P.V product
  uint32_t pf[kKvTile / 16][4];
#pragma unroll
  for (int kk = 0; kk < kKvTile / 16; ++kk) {
    float p[8];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      p[e] = exp2f(s[2 * kk][e] - mx[e >> 1]);
      p[4 + e] = exp2f(s[2 * kk + 1][e] - mx[e >> 1]);
    }
    acc.l[0] += (p[0] + p[1]) + (p[4] + p[5]);
    acc.l[1] += (p[2] + p[3]) + (p[6] + p[7]);
    pf[kk][0] = pack_bf16(p[0], p[1]);
    pf[kk][1] = pack_bf16(p[2], p[3]);
    pf[kk][2] = pack_bf16(p[4], p[5]);
    pf[kk][3] = pack_bf16(p[6], p[7]);
  }
#pragma unroll
  for (int nb = 0; nb < kHeadDim / 8; ++nb) {
    acc.o[nb][0] *= corr[0];
    acc.o[nb][1] *= corr[0];
    acc.o[nb][2] *= corr[1];
    acc.o[nb][3] *= corr[1];
  }
  // O += P V: V rows are the k dimension, so its fragments come transposed
  const char *vrow = vsm + ((lane & 7) + ((lane >> 3) & 1) * 8) * kKPitch + (lane >> 4) * 16;
#pragma unroll
  for (int kk = 0; kk < kKvTile / 16; ++kk) {
    if (kk < nk16) {
#pragma unroll
      for (int nq = 0; nq < kHeadDim / 64; ++nq) {   // groups of four 16-dim pairs
        uint32_t vf[4][4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int np = nq * 4 + j;
          if constexpr (SWZ) {
            const int cg = np * 2 + (lane >> 4);
            const int row = kk * 16 + sw + ((lane >> 3) & 1) * 8;
            ldmatrix_x4_trans(vf[j], vsm + (cg >> 3) * kKvBoxBytes + row * 128 + (((cg & 7) ^ sw) << 4));
          } else {
            ldmatrix_x4_trans(vf[j], vrow + kk * 16 * kKPitch + np * 32);
          }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          mma_16816<false>(acc.o[2 * (nq * 4 + j)], pf[kk], vf[j][0], vf[j][1]);
          mma_16816<false>(acc.o[2 * (nq * 4 + j) + 1], pf[kk], vf[j][2], vf[j][3]);
        }
      }
    }
  }
}

// Layout of one merged/partial row in shared or global scratch: 128 outputs, m, l, and two
// floats of padding so that every row starts on a 16-byte boundary.
constexpr int kAttnRowFloats = kHeadDim + 4;

// A warp's state for its 16-row tile -> shared memory [16][kAttnRowFloats].
// `hi` = false skips rows 8..15 (a decode step has at most 8 query rows).
__device__ __forceinline__ void attn_store_state(float *dst, const AttnAcc &acc, int lane,
                                                 bool hi = true) {
  const int r = lane >> 2, c = (lane & 3) * 2;
  float l0 = acc.l[0], l1 = acc.l[1];
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
#pragma unroll
  for (int nb = 0; nb < kHeadDim / 8; ++nb) {
    *reinterpret_cast<float2 *>(dst + r * kAttnRowFloats + nb * 8 + c) =
        make_float2(acc.o[nb][0], acc.o[nb][1]);
    if (hi)
      *reinterpret_cast<float2 *>(dst + (r + 8) * kAttnRowFloats + nb * 8 + c) =
          make_float2(acc.o[nb][2], acc.o[nb][3]);
  }
  if ((lane & 3) == 0) {
    dst[r * kAttnRowFloats + kHeadDim] = acc.m[0];
    dst[r * kAttnRowFloats + kHeadDim + 1] = l0;
    if (hi) {
      dst[(r + 8) * kAttnRowFloats + kHeadDim] = acc.m[1];
      dst[(r + 8) * kAttnRowFloats + kHeadDim + 1] = l1;
    }
  }
}

// ---- decode form: at most 8 query rows --------------------------------------------------
// With one new token per request the query tile has G <= 8 rows, and a 16-row MMA tile of
// queries is half empty.  The products are taken transposed instead: S^T = K Q^T (the 64
// cached tokens are the M side, the 8 query rows the N side) and O^T = V^T P^T (head dims on
// the M side), 32 + 32 MMAs per tile instead of 64 + 64, and a third of the accumulator
// registers.  P^T leaves the first product in the accumulator layout and enters the second
// as a B operand, which is that layout transposed: movmatrix does it in registers.
//
// A lane holds, for query rows q0 = (lane % 4) * 2 and q0 + 1: their running max and its
// share of their running sum, and for each 16-dim block of the head the outputs
// {[d][q0], [d][q0 + 1], [d + 8][q0], [d + 8][q0 + 1]} with d = lane / 4.
struct AttnAccT {
  float o[kHeadDim / 16][4];
  float m[2];
  float l[2];
};

__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t v) {
  uint32_t r;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(r) : "r"(v));
  return r;
}

// [mt0, mt1): the 16-token blocks of the tile this warp takes (several warps can share a tile).
// The blocks are taken one at a time in a loop that is NOT unrolled, each with its own step of
// the running softmax: a task runs this code once, from a cold instruction cache, and the
// time of the 64-token form unrolled was fetching instructions, not executing them.
template <bool SWZ>
__device__ __forceinline__ void attn_tile_mma_t(const char *qsm, const char *ksm, char *vsm,
                                                int ntok, bool causal, int G, int lane,
                                                AttnAccT &acc, int mt0 = 0, int mt1 = kKvTile / 16) {
  const float qscale = 0.08838834764831845f * 1.4426950408889634f;   // 1/sqrt(128) * log2(e)
  const int nk16 = min(mt1, (ntok + 15) >> 4);   // end of the blocks with at least one valid token
  if (ntok < nk16 * 16) {
    // P is zero for the padding tokens of the last block, but 0 * (stale Inf/NaN) would
    // poison the output: clear those V rows (see attn_tile_mma).  (Only the warp that takes
    // the tile's last valid block gets here.)
    for (int i = lane; i < (nk16 * 16 - ntok) * (kHeadDim / 8); i += 32) {
      const int row = ntok + i / (kHeadDim / 8), c = i % (kHeadDim / 8);
      char *dst = SWZ ? vsm + (c >> 3) * kKvBoxBytes + row * 128 + (c & 7) * 16
                      : vsm + row * kKPitch + c * 16;
      *reinterpret_cast<uint4 *>(dst) = make_uint4(0u, 0u, 0u, 0u);
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncwarp();
  }
  const int sw = lane & 7;
  // Q^T as the B operand: the 8 query rows, 32 head dims per ldmatrix.x4
  uint32_t qf[kHeadDim / 32][4];
#pragma unroll
  for (int p = 0; p < kHeadDim / 32; ++p)
    ldmatrix_x4(qf[p], qsm + sw * kKPitch + (p * 32 + (lane >> 3) * 8) * 2);
  const int q0 = (lane & 3) * 2;

#pragma unroll 1
  for (int mt = mt0; mt < nk16; ++mt) {
    // S^T block = K[16 tokens] Q^T
    float st[4] = {0.f, 0.f, 0.f, 0.f};
    {
      const int row = mt * 16 + ((lane >> 3) & 1) * 8 + sw;   // token of this lane's ldmatrix row
#pragma unroll
      for (int half = 0; half < 2; ++half) {                   // 64 head dims at a time
        uint32_t kf[4][4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int cg = (half * 4 + j) * 2 + (lane >> 4);     // 16-byte chunk of the 256-byte row
          if constexpr (SWZ) {
            ldmatrix_x4(kf[j], ksm + (cg >> 3) * kKvBoxBytes + row * 128 + (((cg & 7) ^ sw) << 4));
          } else {
            ldmatrix_x4(kf[j], ksm + row * kKPitch + cg * 16);
          }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int ks = half * 4 + j;                         // 16-dim step
          mma_16816<false>(st, kf[j], qf[ks >> 1][(ks & 1) * 2], qf[ks >> 1][(ks & 1) * 2 + 1]);
        }
      }
    }
    // scale, mask, column max (a column = one query row)
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int tok = mt * 16 + (lane >> 2) + ((e & 2) ? 8 : 0);
      const int tq = (q0 + (e & 1)) / G;
      const bool vis = tok < ntok && (!causal || tok <= tq);
      st[e] = vis ? st[e] * qscale : -INFINITY;
      mx[e & 1] = fmaxf(mx[e & 1], st[e]);
    }
    float corr[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      mx[j] = fmaxf(mx[j], __shfl_xor_sync(0xffffffffu, mx[j], 4));
      mx[j] = fmaxf(mx[j], __shfl_xor_sync(0xffffffffu, mx[j], 8));
      mx[j] = fmaxf(mx[j], __shfl_xor_sync(0xffffffffu, mx[j], 16));
      const float m_new = fmaxf(acc.m[j], mx[j]);
      const float base = m_new == -INFINITY ? 0.f : m_new;   // nothing seen yet: exponent base 0
      corr[j] = exp2f(acc.m[j] - base);
      acc.m[j] = m_new;
      mx[j] = base;
      acc.l[j] *= corr[j];
    }
    // p = exp2(s - m), rounded to bf16, transposed into the B fragment of the second product
    float pv[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) pv[e] = exp2f(st[e] - mx[e & 1]);
    acc.l[0] += pv[0] + pv[2];
    acc.l[1] += pv[1] + pv[3];
    const uint32_t pb0 = movmatrix_trans(pack_bf16(pv[0], pv[1]));   // tokens mt*16 + 0..7
    const uint32_t pb1 = movmatrix_trans(pack_bf16(pv[2], pv[3]));   // tokens mt*16 + 8..15
#pragma unroll
    for (int md = 0; md < kHeadDim / 16; ++md) {
      acc.o[md][0] *= corr[0];
      acc.o[md][1] *= corr[1];
      acc.o[md][2] *= corr[0];
      acc.o[md][3] *= corr[1];
    }
    // O^T += V^T P^T: V rows are the k dimension of an A operand, so they come transposed
    {
      const int row = mt * 16 + sw + ((lane >> 4) & 1) * 8;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t vf[4][4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int cg = (half * 4 + j) * 2 + ((lane >> 3) & 1);
          if constexpr (SWZ) {
            ldmatrix_x4_trans(vf[j], vsm + (cg >> 3) * kKvBoxBytes + row * 128 + (((cg & 7) ^ sw) << 4));
          } else {
            ldmatrix_x4_trans(vf[j], vsm + row * kKPitch + cg * 16);
          }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) mma_16816<false>(acc.o[half * 4 + j], vf[j], pb0, pb1);
      }
    }
  }
}

// A warp's transposed state -> shared memory [8 rows][kAttnRowFloats].
__device__ __forceinline__ void attn_store_state_t(float *dst, const AttnAccT &acc, int lane) {
  const int q0 = (lane & 3) * 2, d0 = lane >> 2;
  float l0 = acc.l[0], l1 = acc.l[1];
#pragma unroll
  for (int o = 4; o <= 16; o <<= 1) {
    l0 += __shfl_xor_sync(0xffffffffu, l0, o);
    l1 += __shfl_xor_sync(0xffffffffu, l1, o);
  }
#pragma unroll
  for (int md = 0; md < kHeadDim / 16; ++md) {
    dst[q0 * kAttnRowFloats + md * 16 + d0] = acc.o[md][0];
    dst[(q0 + 1) * kAttnRowFloats + md * 16 + d0] = acc.o[md][1];
    dst[q0 * kAttnRowFloats + md * 16 + d0 + 8] = acc.o[md][2];
    dst[(q0 + 1) * kAttnRowFloats + md * 16 + d0 + 8] = acc.o[md][3];
  }
  if (lane < 4) {
    dst[q0 * kAttnRowFloats + kHeadDim] = acc.m[0];
    dst[q0 * kAttnRowFloats + kHeadDim + 1] = l0;
    dst[(q0 + 1) * kAttnRowFloats + kHeadDim] = acc.m[1];
    dst[(q0 + 1) * kAttnRowFloats + kHeadDim + 1] = l1;
  }
}

// q/k RMSNorm inside attention (YPK_F_QK_NORM; Qwen3: attention_sm100.cuh:349-379,
// norm_sm100.cuh): every new q head and the new k are normalised over the 128 head dims and
// scaled by a weight before the rotation, the result rounded to bf16 as an operator output
// would be.  Called by the 16 neighbouring lanes that hold the 16 8-dim chunks of one
// (token, head); `pk` are the lane's own 8 values, `ov` their rotate-half partners (the
// chunk 64 dims away, same head, hence the same RMS), w the 128 weights of the head kind.
struct QkPair {
  uint4 pk, ov;
};
static __device__ __noinline__ QkPair qk_norm_chunk(uint4 pk, uint4 ov, const uint16_t *w, int d0,
                                             float eps, bool partner, unsigned lanes) {
  const uint32_t pv[4] = {pk.x, pk.y, pk.z, pk.w}, po[4] = {ov.x, ov.y, ov.z, ov.w};
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = unpack2(cvt_pair<false>(pv[i]));
    ss += f.x * f.x + f.y * f.y;
  }
#pragma unroll
  for (int o = 1; o < 16; o <<= 1) ss += __shfl_xor_sync(lanes, ss, o);
  const float rn = rsqrtf(ss * (1.0f / kHeadDim) + eps);
  const uint4 wv = __ldg(reinterpret_cast<const uint4 *>(w + d0));
  const uint32_t pw[4] = {wv.x, wv.y, wv.z, wv.w};
  uint32_t o1[4], o2[4] = {0u, 0u, 0u, 0u};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = unpack2(cvt_pair<false>(pv[i])), g = unpack2(cvt_pair<false>(pw[i]));
    o1[i] = pack_bf16((f.x * rn) * g.x, (f.y * rn) * g.y);
  }
  if (partner) {
    const uint4 wo = __ldg(reinterpret_cast<const uint4 *>(w + (d0 ^ 64)));
    const uint32_t qw[4] = {wo.x, wo.y, wo.z, wo.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = unpack2(cvt_pair<false>(po[i])), g = unpack2(cvt_pair<false>(qw[i]));
      o2[i] = pack_bf16((f.x * rn) * g.x, (f.y * rn) * g.y);
    }
  }
  return QkPair{make_uint4(o1[0], o1[1], o1[2], o1[3]), make_uint4(o2[0], o2[1], o2[2], o2[3])};
}

// Rotate-half RoPE of 8 neighbouring head dims: `pk` the values at dims d0.., `ov` their
// partners 64 dims away, cos / sin rows of [positions][128] 16-bit values.
__device__ __forceinline__ uint4 rope_chunk(uint4 pk, uint4 ov, uint4 cv, uint4 sv, int d0) {
  const uint32_t pv[4] = {pk.x, pk.y, pk.z, pk.w}, po[4] = {ov.x, ov.y, ov.z, ov.w},
                 pc[4] = {cv.x, cv.y, cv.z, cv.w}, ps[4] = {sv.x, sv.y, sv.z, sv.w};
  uint32_t o[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 v2 = unpack2(cvt_pair<false>(pv[i])), o2 = unpack2(cvt_pair<false>(po[i])),
                 c2 = unpack2(cvt_pair<false>(pc[i])), s2 = unpack2(cvt_pair<false>(ps[i]));
    const float sgn = d0 < 64 ? -1.f : 1.f;
    // two products and a sum, each rounded to fp32 (no fused multiply-add): the rounding
    // points of x * cos + rotate_half(x) * sin evaluated in fp32
    o[i] = pack_bf16(__fadd_rn(__fmul_rn(v2.x, c2.x), sgn * __fmul_rn(o2.x, s2.x)),
                     __fadd_rn(__fmul_rn(v2.y, c2.y), sgn * __fmul_rn(o2.y, s2.y)));
  }
  return make_uint4(o[0], o[1], o[2], o[3]);
}

// DECODE: the request has at most 8 query rows this iteration (transposed products).
template <bool DECODE>
__device__ __forceinline__ void attention_consume_impl(WaitCtx &wc, char *smem, Misc *misc,
                                                       const Runtime &rt, const ypk_task &t,
                                                       const AttnShape &s, long long iter,
                                                       RingPos &pos) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int h = t.iarg[1], split = t.iarg[2], nsplit = t.iarg[3];
  const int G = t.iarg[4], hkv = t.iarg[5], ld_qkv = t.iarg[6], ld_out = t.iarg[7];
  const int max_rows = t.iarg[8];
  const uint16_t *qkv = reinterpret_cast<const uint16_t *>(t.ptr[0]);
  uint16_t *kcache = reinterpret_cast<uint16_t *>(t.ptr[1]);
  uint16_t *vcache = reinterpret_cast<uint16_t *>(t.ptr[2]);
  uint16_t *out = reinterpret_cast<uint16_t *>(t.ptr[3]);
  const uint16_t *cosp = reinterpret_cast<const uint16_t *>(t.ptr[4]);
  const uint16_t *sinp = reinterpret_cast<const uint16_t *>(t.ptr[5]);
  float *scratch = reinterpret_cast<float *>(t.ptr[6]);
  const bool rope = (t.flags & YPK_F_ROPE) != 0;
  // q/k RMSNorm: ptr[7] = [2][128] weights (q heads, then k), farg[0] = epsilon
  const bool qk_norm = (t.flags & YPK_F_QK_NORM) != 0;
  const uint16_t *qk_w = reinterpret_cast<const uint16_t *>(t.ptr[7]);
  // flagged-word hand-off: with YPK_F_LL_IN ptr[0] holds the packed q/k/v as {two values,
  // tag} words ([max_tokens][ld_qkv / 2]), with YPK_F_LL_OUT ptr[3] takes the result that way
  const bool ll_in = (t.flags & YPK_F_LL_IN) != 0, ll_out = (t.flags & YPK_F_LL_OUT) != 0;
  const uint32_t tag_in = ll_tag(rt, iter, t.iarg[11]), tag_out = ll_tag(rt, iter, t.iarg[12]);
  const unsigned long long *qkv_ll = reinterpret_cast<const unsigned long long *>(t.ptr[0]);
  unsigned long long *out_ll = reinterpret_cast<unsigned long long *>(t.ptr[3]);
  LLPoll poll;
  const int T = s.T, rows = T * G;
  const int nm = (rows + 15) >> 4;            // 16-row query tiles: 1 or 2
  const int nslots = kConsumerWarps / nm;     // warps that share the tiles of one query tile
  const int mt = warp / nslots, slot = warp - mt * nslots;

  // shared-memory scratch of the task (everything from kOffXs up to the misc area)
  char *qsm = smem + kOffXs;                                    // [32][272 B] bf16 q rows
  // the new tokens' k and v: 16 rows, or kMaxNewKeys when earlier query tiles of the same
  // request precede this one (never in the decode form)
  constexpr int kNewRows = DECODE ? 16 : kMaxNewKeys;
  char *knew = qsm + kMaxAttnRows * kKPitch;                    // [kNewRows][272 B]
  char *vnew = knew + kNewRows * kKPitch;                       // [kNewRows][272 B]
  static_assert(kMaxAttnRows * kKPitch + 2 * kMaxNewKeys * kKPitch <= kScratchSmemBytes, "attention scratch");
  const int pre = DECODE ? 0 : s.pre;
  float *mrg = reinterpret_cast<float *>(smem + kOffXs);        // merge: [4 warps][16][132] fp32

  // Stage q (rotated, rounded to bf16) and, in the split that owns the new tokens, the
  // rotated k and v; append those to the cache page.  One thread handles 8 consecutive dims
  // with 16-byte loads of the values, their rotate-half partners and the cos/sin row.
  if (s.handles_new) {
    for (int i = tid; i < 16 * (kHeadDim / 8); i += kConsumerThreads) {   // clear rows T..15 of v
      const int row = i >> 4;
      if (row >= pre + T) *reinterpret_cast<uint4 *>(vnew + row * kKPitch + (i & 15) * 16) = make_uint4(0u, 0u, 0u, 0u);
    }
  }
  const int heads_to_stage = G + (s.handles_new ? 2 : 0);
  for (int idx = tid; idx < T * heads_to_stage * (kHeadDim / 8); idx += kConsumerThreads) {
    const int c = idx & 15;                       // 8-dim chunk of the head
    const int hh = (idx >> 4) % heads_to_stage;
    const int tk = idx / (heads_to_stage * 16);
    const int d0 = c * 8;
    const int pos_t = s.seq_len - T + tk;
    const size_t col = size_t(h) * (G + 2) * kHeadDim + hh * kHeadDim;
    const uint16_t *src = qkv + size_t(s.qo0 + tk) * ld_qkv + col;
    const bool rot = rope && hh <= G;   // q heads and k, not v
    // the page of the new token (k and v only): asked for ahead of the values it goes with
    int page = 0;
    if (hh >= G) page = __ldcg(rt.kv_indices + s.kv0 + pos_t / rt.page_size);
    // the cos / sin row of the position is asked for ahead of the values as well: it is a
    // new row every iteration (a trip to HBM for the first task that touches it)
    uint4 cv = make_uint4(0u, 0u, 0u, 0u), sv = cv;
    if (rot) {
      cv = __ldcg(reinterpret_cast<const uint4 *>(cosp + size_t(pos_t) * kHeadDim + d0));
      sv = __ldcg(reinterpret_cast<const uint4 *>(sinp + size_t(pos_t) * kHeadDim + d0));
    }
    uint4 pk, ov = make_uint4(0u, 0u, 0u, 0u);
    if (ll_in) {
      // 8 dims = four words; the rotate-half partner's four with them, polled together
      const unsigned long long *wsrc = qkv_ll + size_t(s.qo0 + tk) * size_t(ld_qkv >> 1) + (col >> 1);
      unsigned long long w[8];
      for (;;) {
        ll_load2(wsrc + (d0 >> 1), w[0], w[1]);
        ll_load2(wsrc + (d0 >> 1) + 2, w[2], w[3]);
        bool ok = true;
        if (rot) {
          ll_load2(wsrc + ((d0 ^ 64) >> 1), w[4], w[5]);
          ll_load2(wsrc + ((d0 ^ 64) >> 1) + 2, w[6], w[7]);
#pragma unroll
          for (int i = 4; i < 8; ++i) ok = ok && ll_ok(w[i], tag_in);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) ok = ok && ll_ok(w[i], tag_in);
        if (ok || !poll.again(wc)) break;
      }
      pk = make_uint4(uint32_t(w[0]), uint32_t(w[1]), uint32_t(w[2]), uint32_t(w[3]));
      if (rot) ov = make_uint4(uint32_t(w[4]), uint32_t(w[5]), uint32_t(w[6]), uint32_t(w[7]));
    } else {
      pk = __ldcg(reinterpret_cast<const uint4 *>(src + d0));
      if (rot) ov = __ldcg(reinterpret_cast<const uint4 *>(src + (d0 ^ 64)));
    }
    if (qk_norm && hh <= G) {
      // the 16 chunks of a (token, head) sit in 16 neighbouring lanes (idx & 15 = chunk)
      const QkPair n = qk_norm_chunk(pk, ov, qk_w + (hh == G ? kHeadDim : 0), d0, t.farg[0], rot,
                                     (lane & 16) ? 0xffff0000u : 0x0000ffffu);
      pk = n.pk;
      ov = n.ov;
    }
    if (rot) pk = rope_chunk(pk, ov, cv, sv, d0);
    if (hh < G) {
      *reinterpret_cast<uint4 *>(qsm + (tk * G + hh) * kKPitch + d0 * 2) = pk;
    } else {
      const size_t off =
          ((size_t(page) * rt.page_size + (pos_t % rt.page_size)) * hkv + h) * kHeadDim + d0;
      if (hh == G) {
        *reinterpret_cast<uint4 *>(knew + (pre + tk) * kKPitch + d0 * 2) = pk;
        *reinterpret_cast<uint4 *>(kcache + off) = pk;
      } else {
        *reinterpret_cast<uint4 *>(vnew + (pre + tk) * kKPitch + d0 * 2) = pk;
        *reinterpret_cast<uint4 *>(vcache + off) = pk;
      }
    }
  }
  if constexpr (!DECODE) {
    // The request's new tokens ahead of this query tile: their k (normalised, rotated) and v
    // are staged from the packed rows as well: the tasks of one iteration do not wait for one
    // another's appends.  The append itself is left to the task that owns those tokens.
    if (s.handles_new && pre > 0) {
      for (int idx = tid; idx < pre * 2 * (kHeadDim / 8); idx += kConsumerThreads) {
        const int c = idx & 15, hh = G + ((idx >> 4) & 1), tk = idx >> 5;
        const int d0 = c * 8;
        const int pos_t = s.cached + tk;
        const uint16_t *src = qkv + size_t(s.qo0 - pre + tk) * ld_qkv +
                              size_t(h) * (G + 2) * kHeadDim + hh * kHeadDim;
        const bool rot = rope && hh == G;
        uint4 pk = __ldcg(reinterpret_cast<const uint4 *>(src + d0));
        uint4 ov = make_uint4(0u, 0u, 0u, 0u);
        if (rot) ov = __ldcg(reinterpret_cast<const uint4 *>(src + (d0 ^ 64)));
        if (qk_norm && hh == G) {
          const QkPair n = qk_norm_chunk(pk, ov, qk_w + kHeadDim, d0, t.farg[0], rot,
                                         (lane & 16) ? 0xffff0000u : 0x0000ffffu);
          pk = n.pk;
          ov = n.ov;
        }
        if (rot) {
          pk = rope_chunk(pk, ov, __ldcg(reinterpret_cast<const uint4 *>(cosp + size_t(pos_t) * kHeadDim + d0)),
                          __ldcg(reinterpret_cast<const uint4 *>(sinp + size_t(pos_t) * kHeadDim + d0)), d0);
        }
        *reinterpret_cast<uint4 *>((hh == G ? knew : vnew) + tk * kKPitch + d0 * 2) = pk;
      }
    }
  }
  // a poll that gave up is known to one thread; the mbarrier waits need a warp-uniform state
  if (ll_in) wc.failed = __any_sync(0xffffffffu, poll.failed || wc.failed);
  consumer_bar();
  if (tid == 0 && misc->prof_rec) misc->prof_rec[4] = globaltimer();

  using Acc = typename std::conditional<DECODE, AttnAccT, AttnAcc>::type;
  Acc acc;
#pragma unroll
  for (int i = 0; i < int(sizeof(acc.o) / sizeof(acc.o[0])); ++i) acc.o[i][0] = acc.o[i][1] = acc.o[i][2] = acc.o[i][3] = 0.f;
  acc.m[0] = acc.m[1] = -INFINITY;
  acc.l[0] = acc.l[1] = 0.f;

  // Every warp passes every stage (so that ring positions stay in step) but computes only
  // on the tiles it owns; the others are released as soon as they have landed.
  // Decode form: a split of few tiles lets 2 or 4 warps share a tile, 32 or 16 tokens each (a
  // tile costs a warp about 2 us, and the states of all eight warps are merged anyway); the
  // last warp stays free for the new tokens.
  int parts = 1;
  if constexpr (DECODE) {
    const int free_slots = nslots - (s.handles_new ? 1 : 0), ntile = s.tile1 - s.tile0;
    parts = ntile * 4 <= free_slots ? 4 : (ntile * 2 <= free_slots ? 2 : 1);
  }
  for (int tile = s.tile0; tile < s.tile1; ++tile) {
    const int ntok = min(kKvTile, s.cached - tile * kKvTile);
    const bool got = wait_mbar(wc, &misc->full_bar[pos.slot], pos.phase);
    char *stage = smem + kOffRing + pos.slot * kStageBytes;
    if constexpr (DECODE) {
      const int u0 = (tile - s.tile0) * parts;       // parts > 1: every unit has a warp of its own
      const bool mine = parts > 1 ? (slot >= u0 && slot < u0 + parts) : (u0 % nslots == slot);
      const int per = (kKvTile / 16) / parts, b0 = parts > 1 ? (slot - u0) * per : 0;
      if (got && mine && b0 * 16 < ntok)
        attn_tile_mma_t<true>(qsm, stage, stage + kVOffset, ntok, false, G, lane, acc, b0, b0 + per);
    } else {
      if (got && (tile - s.tile0) % nslots == slot)
        attn_tile_mma<true>(qsm, stage, stage + kVOffset, ntok, false, G, mt * 16, lane, acc);
    }
    __syncwarp();
    if (lane == 0 && got) mbar_arrive(&misc->empty_bar[pos.slot]);
    pos.advance();
  }
  // the new tokens: causal among themselves; the last slot of the group is the one with
  // the fewest cached tiles
  if (s.handles_new && slot == nslots - 1) {
    if constexpr (DECODE) {
      attn_tile_mma_t<false>(qsm, knew, vnew, T, true, G, lane, acc);
    } else {
      attn_tile_mma<false>(qsm, knew, vnew, pre + T, true, G, mt * 16, lane, acc, pre);
    }
  }
  consumer_bar();  // q / knew / vnew are dead from here on; the area becomes the merge buffer
  if (tid == 0 && misc->prof_rec) misc->prof_rec[5] = globaltimer();

  // Split-KV partials travel as flagged words {fp32 bits, tag}: the split that owns the new
  // tokens (the last one) folds the others' rows into its own as they show up, the others
  // just write.  No arrival counter, no fence, no second pass.
  const bool single = s.nact == 1;
  const bool combiner = s.handles_new;
  const uint32_t tag_sp = ll_tag(rt, iter, t.iarg[13]);
  unsigned long long *scr_w = reinterpret_cast<unsigned long long *>(scratch);
  const size_t split_words = size_t(max_rows) * kAttnRowFloats;
  unsigned long long *head_scr = scr_w + (size_t(t.iarg[0]) * hkv + h) * nsplit * split_words;
  unsigned long long *my_scr = head_scr + size_t(split) * split_words;
  // merge states are [16 rows][132] per warp, [8 rows][132] in the decode form
  constexpr int kStateFloats = (DECODE ? 8 : 16) * kAttnRowFloats;
  // Merge the warps of a query tile, four states at a time, then finish rows [mt*16, ..).
  // Two neighbouring head dims of a finished query row: plain bf16, or one flagged word.
  auto emit = [&](int row, int d, float v0, float v1) {
    const int tk = row / G, g = row - tk * G;
    const size_t col = size_t(h * G + g) * kHeadDim + d;
    const uint32_t packed = pack_bf16(v0, v1);
    if (ll_out) {
      ll_store(out_ll + size_t(s.qo0 + tk) * size_t(ld_out >> 1) + (col >> 1), ll_word(packed, tag_out));
    } else {
      *reinterpret_cast<uint32_t *>(out + size_t(s.qo0 + tk) * ld_out + col) = packed;
    }
  };
  auto finalize = [&](int mtile, int nstates) {
    const int row_lo = mtile * 16, nrow = min(16, rows - row_lo);
    for (int idx = tid; idx < nrow * (kHeadDim / 2); idx += kConsumerThreads) {
      const int d = (idx & (kHeadDim / 2 - 1)) * 2, rr = idx >> 6;
      float m = -INFINITY;
      for (int w = 0; w < nstates; ++w)
        m = fmaxf(m, mrg[w * kStateFloats + rr * kAttnRowFloats + kHeadDim]);
      float l = 0.f, o0 = 0.f, o1 = 0.f;
      for (int w = 0; w < nstates; ++w) {
        const float *pr = mrg + w * kStateFloats + rr * kAttnRowFloats;
        const float c = pr[kHeadDim] == -INFINITY ? 0.f : exp2f(pr[kHeadDim] - m);
        const float2 po = *reinterpret_cast<const float2 *>(pr + d);
        l += pr[kHeadDim + 1] * c;
        o0 += po.x * c;
        o1 += po.y * c;
      }
      const int row = row_lo + rr;
      if (single) {
        emit(row, d, o0 / l, o1 / l);
      } else if (!combiner) {
        unsigned long long *dst = my_scr + row * kAttnRowFloats;
        ll_store(dst + d, ll_word(__float_as_uint(o0), tag_sp));
        ll_store(dst + d + 1, ll_word(__float_as_uint(o1), tag_sp));
        if (d == 0) {
          ll_store(dst + kHeadDim, ll_word(__float_as_uint(m), tag_sp));
          ll_store(dst + kHeadDim + 1, ll_word(__float_as_uint(l), tag_sp));
        }
      } else {
        // fold in the other splits in split order, this split's own row last
        float mr = -INFINITY, lr = 0.f, a0 = 0.f, a1 = 0.f;
        auto fold = [&](float ms, float ls, float x0, float x1) {
          if (ms == -INFINITY) return;
          const float m_new = fmaxf(mr, ms);
          const float c_old = exp2f(mr - m_new), c_new = exp2f(ms - m_new);   // exp2f(-inf) = 0
          lr = lr * c_old + ls * c_new;
          a0 = a0 * c_old + x0 * c_new;
          a1 = a1 * c_old + x1 * c_new;
          mr = m_new;
        };
        for (int sp = 0; sp < s.nact - 1; ++sp) {
          const unsigned long long *pr = head_scr + size_t(sp) * split_words + row * kAttnRowFloats;
          unsigned long long w0, w1, w2, w3;
          for (;;) {
            ll_load2(pr + d, w0, w1);
            ll_load2(pr + kHeadDim, w2, w3);
            if ((ll_ok(w0, tag_sp) && ll_ok(w1, tag_sp) && ll_ok(w2, tag_sp) && ll_ok(w3, tag_sp)) ||
                !poll.again(wc))
              break;
          }
          fold(__uint_as_float(uint32_t(w2)), __uint_as_float(uint32_t(w3)),
               __uint_as_float(uint32_t(w0)), __uint_as_float(uint32_t(w1)));
        }
        fold(m, l, o0, o1);
        emit(row, d, a0 / lr, a1 / lr);
      }
    }
  };
  if constexpr (DECODE) {
    // decode: eight 8-row states fit the buffer at once
    attn_store_state_t(mrg + warp * kStateFloats, acc, lane);
    consumer_bar();
    finalize(0, kConsumerWarps);
  } else if (nm == 1) {
    // eight states: warps 4..7 hand theirs to warps 0..3, which fold them in
    if (warp >= 4) attn_store_state(mrg + (warp - 4) * kStateFloats, acc, lane);
    consumer_bar();
    if (warp < 4) {
      const float *ps = mrg + warp * kStateFloats;
      const int rr = lane >> 2, c = (lane & 3) * 2;
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        const float *pr = ps + (rr + hh * 8) * kAttnRowFloats;
        const float mo = pr[kHeadDim], lo = pr[kHeadDim + 1];
        const float m_new = fmaxf(acc.m[hh], mo);
        const float base = m_new == -INFINITY ? 0.f : m_new;
        const float ca = exp2f(acc.m[hh] - base), cb = exp2f(mo - base);
        // acc.l is a per-lane share; the partner's l is the full row sum: add it on one lane
        acc.l[hh] = acc.l[hh] * ca + ((lane & 3) == 0 ? lo * cb : 0.f);
        acc.m[hh] = m_new;
#pragma unroll
        for (int nb = 0; nb < kHeadDim / 8; ++nb) {
          const float2 po = *reinterpret_cast<const float2 *>(pr + nb * 8 + c);
          acc.o[nb][2 * hh] = acc.o[nb][2 * hh] * ca + po.x * cb;
          acc.o[nb][2 * hh + 1] = acc.o[nb][2 * hh + 1] * ca + po.y * cb;
        }
      }
    }
    consumer_bar();
    if (warp < 4) attn_store_state(mrg + warp * kStateFloats, acc, lane);
    consumer_bar();
    finalize(0, 4);
  } else {
    if (warp < 4) attn_store_state(mrg + warp * kStateFloats, acc, lane);
    consumer_bar();
    finalize(0, 4);
    consumer_bar();
    if (warp >= 4) attn_store_state(mrg + (warp - 4) * kStateFloats, acc, lane);
    consumer_bar();
    finalize(1, 4);
  }
  if (poll.failed) wc.failed = true;
}

// The two forms are separate out-of-line functions: the 16-row form needs twice the
// accumulator registers and must not weigh on the decode form's allocation.
struct AttnRet {
  RingPos pos;
  bool failed;
};
template <bool DECODE>
__device__ __noinline__ AttnRet attention_consume_out(const Runtime *rt, Misc *misc, char *smem,
                                                      int worker, int task, bool failed,
                                                      AttnShape s, long long iter, RingPos pos) {
  WaitCtx wc{rt, misc, worker, task, failed};
  attention_consume_impl<DECODE>(wc, smem, misc, *rt, misc->ctask, s, iter, pos);
  return AttnRet{pos, wc.failed};
}

__device__ __forceinline__ void attention_consume(WaitCtx &wc, char *smem, Misc *misc,
                                                  const Runtime &rt, const ypk_task &t,
                                                  long long iter, RingPos &pos) {
  const AttnShape s = attn_shape(rt, t);
  if (!s.active) return;
  const AttnRet r = s.T * t.iarg[4] <= 8 && s.pre == 0
      ? attention_consume_out<true>(&rt, misc, smem, wc.worker, wc.task, wc.failed, s, iter, pos)
      : attention_consume_out<false>(&rt, misc, smem, wc.worker, wc.task, wc.failed, s, iter, pos);
  pos = r.pos;
  wc.failed = r.failed;
}

}  // namespace ypk
