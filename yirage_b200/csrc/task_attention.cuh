// ATTENTION task: GQA incremental-decode / chunked-prefill attention over a paged bf16
// KV cache for one (request, kv head, KV split).
//
// Semantics follow the reference's paged attention task
// (tasks/blackwell/attention_sm100.cuh:33-660): packed QKV rows laid out per kv head as
// [q_per_kv q heads | k | v], rotate-half RoPE on the new q and k with bf16 cos/sin rows
// (tasks/blackwell/rotary_embedding_sm100.cuh:56-73), the rotated k and v of the new
// tokens are written into their page slots, causal softmax with scale 1/sqrt(128) in
// fp32, bf16 output.  Differences by design: the sequence is split across CTAs
// (split-KV) and the partial results are merged by whichever split finishes last, the
// K/V tiles arrive through the producer warp's bulk copies instead of cp.async, and the
// sequence length is (pages-1)*page_size + last_page_len with last_page_len in
// [1, page_size] (the reference's 0-when-full convention under-counts by a page,
// attention_sm100.cuh:101-102).
//
// Mapping: a ring stage holds 64 cached tokens (K rows at 272-byte pitch, then V rows).
// A warp owns (q head g, token half th) units; lane <-> token for Q.K (16-byte K reads,
// q read as shared-memory broadcasts), warp-shuffle max/sum for the online softmax, then
// lane <-> 4 head dims for P.V with p broadcast by shuffle.
#pragma once
#include "device_common.cuh"

namespace ypk {

struct AttnShape {
  int T;         // new tokens of this request in this iteration
  int qo0;       // first row of the request in the packed qkv / output
  int kv0;       // first entry of the request in kv_indices
  int seq_len;   // tokens including the new ones
  int cached;    // seq_len - T
  int tile0, tile1;  // cached 64-token tiles of this split
  int nact;      // active splits of this (request, head)
  bool active, handles_new;
};

__device__ __forceinline__ AttnShape attn_shape(const Runtime &rt, const ypk_task &t) {
  AttnShape s;
  const int r = t.iarg[0], split = t.iarg[2], nsplit = t.iarg[3];
  s.qo0 = __ldcg(rt.qo_indptr + r);
  s.T = __ldcg(rt.qo_indptr + r + 1) - s.qo0;
  s.kv0 = __ldcg(rt.kv_indptr + r);
  const int npages = __ldcg(rt.kv_indptr + r + 1) - s.kv0;
  s.seq_len = (npages - 1) * rt.page_size + __ldcg(rt.kv_last_len + r);
  s.cached = s.seq_len - s.T;
  const int tiles = (s.cached + kKvTile - 1) / kKvTile;
  const int tps = max(1, (tiles + nsplit - 1) / nsplit);
  s.nact = tiles > 0 ? (tiles + tps - 1) / tps : 1;
  s.active = s.T > 0 && s.T <= kMaxNewTokens && npages > 0 && split < s.nact;
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
  const int h = t.iarg[1], hkv = t.iarg[5];
  const char *kc = reinterpret_cast<const char *>(t.ptr[1]);
  const char *vc = reinterpret_cast<const char *>(t.ptr[2]);
  for (int tile = s.tile0; tile < s.tile1; ++tile) {
    const int tok0 = tile * kKvTile;
    const int ntok = min(kKvTile, s.cached - tok0);
    const int page = __ldcg(rt.kv_indices + s.kv0 + tok0 / rt.page_size);
    const size_t row0 = size_t(page) * rt.page_size + (tok0 % rt.page_size);
    if (!wait_mbar(wc, &misc->empty_bar[pos.slot], pos.phase ^ 1u)) return false;
    char *stage = smem + kOffRing + pos.slot * kStageBytes;
    if (lane == 0) mbar_expect_tx(&misc->full_bar[pos.slot], uint32_t(ntok) * kHeadDim * 4u);
    __syncwarp();
    for (int i = lane; i < ntok; i += 32) {
      const size_t off = ((row0 + i) * hkv + h) * (kHeadDim * 2);
      bulk_g2s(stage + i * kKPitch, kc + off, kHeadDim * 2, &misc->full_bar[pos.slot]);
      bulk_g2s(stage + kVOffset + i * (kHeadDim * 2), vc + off, kHeadDim * 2,
               &misc->full_bar[pos.slot]);
    }
    pos.advance();
  }
  return true;
}

// ------------------------------------------------------------------ consumer
// Online-softmax state of one (unit, q row): running max (log2 domain), running sum,
// and 4 output dims per lane.
template <int TM>
struct AttnState {
  float m[2][TM], l[2][TM], o[2][TM][4];
};

template <int TM>
__device__ __forceinline__ void attn_tile(const char *ksm, const char *vsm, const float *qs,
                                          int ntok, bool causal, int T, int G, int warp, int lane,
                                          AttnState<TM> &st) {
#pragma unroll
  for (int uu = 0; uu < 2; ++uu) {
    const int u = warp + kConsumerWarps * uu;
    if (u >= 2 * G) break;
    const int g = u >> 1, th = u & 1;
    const int tok = th * 32 + lane;
    const bool valid = tok < ntok;
    const int nhalf = min(32, ntok - th * 32);
    if (nhalf <= 0) continue;
    unsigned long long sacc[TM];
#pragma unroll
    for (int t = 0; t < TM; ++t) sacc[t] = 0ull;
    const uint4 *kp = reinterpret_cast<const uint4 *>(ksm + tok * kKPitch);
#pragma unroll 2
    for (int s8 = 0; s8 < kHeadDim / 8; ++s8) {
      uint4 kv = make_uint4(0u, 0u, 0u, 0u);
      if (valid) kv = kp[s8];
      const unsigned long long k0 = cvt_pair<false>(kv.x), k1 = cvt_pair<false>(kv.y),
                               k2 = cvt_pair<false>(kv.z), k3 = cvt_pair<false>(kv.w);
#pragma unroll
      for (int t = 0; t < TM; ++t) {
        if (t < T) {
          const ulonglong2 *qp =
              reinterpret_cast<const ulonglong2 *>(qs + (t * G + g) * kHeadDim + s8 * 8);
          const ulonglong2 qa = qp[0], qb = qp[1];
          sacc[t] = fma2(k0, qa.x, sacc[t]);
          sacc[t] = fma2(k1, qa.y, sacc[t]);
          sacc[t] = fma2(k2, qb.x, sacc[t]);
          sacc[t] = fma2(k3, qb.y, sacc[t]);
        }
      }
    }
    float p[TM];
#pragma unroll
    for (int t = 0; t < TM; ++t) {
      p[t] = 0.f;
      if (t < T) {
        const float2 f = unpack2(sacc[t]);
        const bool vis = valid && (!causal || tok <= t);
        const float sc = vis ? f.x + f.y : -INFINITY;
        const float mx = warp_max(sc);
        const float m_new = fmaxf(st.m[uu][t], mx);
        if (m_new != -INFINITY) {
          const float corr = exp2f(st.m[uu][t] - m_new);  // exp2f(-inf) = 0 on first use
          p[t] = vis ? exp2f(sc - m_new) : 0.f;
          st.l[uu][t] = st.l[uu][t] * corr + warp_sum(p[t]);
#pragma unroll
          for (int d = 0; d < 4; ++d) st.o[uu][t][d] *= corr;
          st.m[uu][t] = m_new;
        }
      }
    }
    const char *vp = vsm + (th * 32) * (kHeadDim * 2) + lane * 8;
    for (int j = 0; j < nhalf; ++j) {
      const uint2 vv = *reinterpret_cast<const uint2 *>(vp + j * (kHeadDim * 2));
      const float2 v01 = unpack2(cvt_pair<false>(vv.x)), v23 = unpack2(cvt_pair<false>(vv.y));
#pragma unroll
      for (int t = 0; t < TM; ++t) {
        if (t < T) {
          const float pj = __shfl_sync(0xffffffffu, p[t], j);
          st.o[uu][t][0] += pj * v01.x;
          st.o[uu][t][1] += pj * v01.y;
          st.o[uu][t][2] += pj * v23.x;
          st.o[uu][t][3] += pj * v23.y;
        }
      }
    }
  }
}

// Layout of one merged/partial row in shared or global scratch: 128 outputs, m, l, and two
// floats of padding so that every row starts on a 16-byte boundary (float4 stores).
constexpr int kAttnRowFloats = kHeadDim + 4;

template <int TM>
__device__ __forceinline__ void attention_consume_t(WaitCtx &wc, char *smem, Misc *misc,
                                                    const Runtime &rt, const ypk_task &t,
                                                    const AttnShape &s, RingPos &pos) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int r = t.iarg[0], h = t.iarg[1], split = t.iarg[2], nsplit = t.iarg[3];
  const int G = t.iarg[4], hkv = t.iarg[5], ld_qkv = t.iarg[6], ld_out = t.iarg[7];
  const int max_rows = t.iarg[8];
  const uint16_t *qkv = reinterpret_cast<const uint16_t *>(t.ptr[0]);
  uint16_t *kcache = reinterpret_cast<uint16_t *>(t.ptr[1]);
  uint16_t *vcache = reinterpret_cast<uint16_t *>(t.ptr[2]);
  uint16_t *out = reinterpret_cast<uint16_t *>(t.ptr[3]);
  const uint16_t *cosp = reinterpret_cast<const uint16_t *>(t.ptr[4]);
  const uint16_t *sinp = reinterpret_cast<const uint16_t *>(t.ptr[5]);
  float *scratch = reinterpret_cast<float *>(t.ptr[6]);
  unsigned int *counters = reinterpret_cast<unsigned int *>(t.ptr[7]);
  const bool rope = (t.flags & YPK_F_ROPE) != 0;
  const int T = s.T, rows = T * G;

  float *qs = reinterpret_cast<float *>(smem + kOffXs);                  // [rows][128] fp32
  char *knew = smem + kOffXs + 64 * kHeadDim * 4;                         // [T] rows, K pitch
  char *vnew = knew + kMaxNewTokens * kKPitch;                            // [T][256 B]
  // 1/sqrt(128) * log2(e): scores live in the log2 domain so exp2f can be used
  const float qscale = 0.08838834764831845f * 1.4426950408889634f;

  // Stage q (rotated, rounded to bf16 like the reference's shared-memory copy, scaled)
  // and, in the split that owns the new tokens, the rotated k and v; append those to the
  // cache page.
  const int heads_to_stage = G + (s.handles_new ? 2 : 0);
  for (int idx = tid; idx < T * heads_to_stage * kHeadDim; idx += kConsumerThreads) {
    const int d = idx & (kHeadDim - 1);
    const int hh = (idx >> 7) % heads_to_stage;
    const int tk = idx / (heads_to_stage * kHeadDim);
    const int pos_t = s.seq_len - T + tk;
    const uint16_t *src = qkv + size_t(s.qo0 + tk) * ld_qkv + size_t(h) * (G + 2) * kHeadDim +
                          hh * kHeadDim;
    float v = cvt_one<false>(__ldcg(src + d));
    if (rope && hh <= G) {  // q heads and k, not v
      const float other = cvt_one<false>(__ldcg(src + (d ^ 64)));
      const float c = cvt_one<false>(__ldcg(cosp + size_t(pos_t) * kHeadDim + d));
      const float sn = cvt_one<false>(__ldcg(sinp + size_t(pos_t) * kHeadDim + d));
      v = d < 64 ? v * c - other * sn : v * c + other * sn;
    }
    v = bf16_round(v);
    if (hh < G) {
      qs[(tk * G + hh) * kHeadDim + d] = v * qscale;
    } else {
      const uint16_t bits = __bfloat16_as_ushort(__float2bfloat16_rn(v));
      const int page = __ldcg(rt.kv_indices + s.kv0 + pos_t / rt.page_size);
      const size_t off =
          ((size_t(page) * rt.page_size + (pos_t % rt.page_size)) * hkv + h) * kHeadDim + d;
      if (hh == G) {
        reinterpret_cast<uint16_t *>(knew + tk * kKPitch)[d] = bits;
        kcache[off] = bits;
      } else {
        reinterpret_cast<uint16_t *>(vnew + tk * (kHeadDim * 2))[d] = bits;
        vcache[off] = bits;
      }
    }
  }
  consumer_bar();

  AttnState<TM> st;
#pragma unroll
  for (int uu = 0; uu < 2; ++uu)
#pragma unroll
    for (int tt = 0; tt < TM; ++tt) {
      st.m[uu][tt] = -INFINITY;
      st.l[uu][tt] = 0.f;
#pragma unroll
      for (int d = 0; d < 4; ++d) st.o[uu][tt][d] = 0.f;
    }

  for (int tile = s.tile0; tile < s.tile1; ++tile) {
    const int ntok = min(kKvTile, s.cached - tile * kKvTile);
    const bool got = wait_mbar(wc, &misc->full_bar[pos.slot], pos.phase);
    const char *stage = smem + kOffRing + pos.slot * kStageBytes;
    if (got) attn_tile<TM>(stage, stage + kVOffset, qs, ntok, false, T, G, warp, lane, st);
    __syncwarp();
    if (lane == 0 && got) mbar_arrive(&misc->empty_bar[pos.slot]);
    pos.advance();
  }
  if (s.handles_new) attn_tile<TM>(knew, vnew, qs, T, true, T, G, warp, lane, st);
  consumer_bar();  // q / knew / vnew are dead from here on; reuse the area for the merge

  // Per-unit partials -> shared memory: [unit][t] rows of (o[128], m, l).
  float *pm = reinterpret_cast<float *>(smem + kOffXs);
#pragma unroll
  for (int uu = 0; uu < 2; ++uu) {
    const int u = warp + kConsumerWarps * uu;
    if (u < 2 * G) {
#pragma unroll
      for (int tt = 0; tt < TM; ++tt) {
        if (tt < T) {
          float *row = pm + (u * T + tt) * kAttnRowFloats;
          *reinterpret_cast<float4 *>(row + lane * 4) =
              make_float4(st.o[uu][tt][0], st.o[uu][tt][1], st.o[uu][tt][2], st.o[uu][tt][3]);
          if (lane == 0) {
            row[kHeadDim] = st.m[uu][tt];
            row[kHeadDim + 1] = st.l[uu][tt];
          }
        }
      }
    }
  }
  consumer_bar();

  // Merge the two token halves of every (t, g) row; either finish here (single split)
  // or park the partial in global scratch for the last-arriving split to combine.
  const bool single = s.nact == 1;
  float *my_scr =
      scratch + ((size_t(r) * hkv + h) * nsplit + split) * size_t(max_rows) * kAttnRowFloats;
  for (int idx = tid; idx < rows * kHeadDim; idx += kConsumerThreads) {
    const int d = idx & (kHeadDim - 1);
    const int row = idx >> 7;          // t * G + g
    const int tk = row / G, g = row - tk * G;
    const float *a = pm + ((2 * g) * T + tk) * kAttnRowFloats;
    const float *b = pm + ((2 * g + 1) * T + tk) * kAttnRowFloats;
    const float ma = a[kHeadDim], mb = b[kHeadDim];
    const float m = fmaxf(ma, mb);
    const float ca = ma == -INFINITY ? 0.f : exp2f(ma - m);
    const float cb = mb == -INFINITY ? 0.f : exp2f(mb - m);
    const float l = a[kHeadDim + 1] * ca + b[kHeadDim + 1] * cb;
    const float o = a[d] * ca + b[d] * cb;
    if (single) {
      out[size_t(s.qo0 + tk) * ld_out + size_t(h * G + g) * kHeadDim + d] =
          __bfloat16_as_ushort(__float2bfloat16_rn(o / l));
    } else {
      float *dst = my_scr + row * kAttnRowFloats;
      dst[d] = o;
      if (d == 0) {
        dst[kHeadDim] = m;
        dst[kHeadDim + 1] = l;
      }
    }
  }
  if (single) return;

  __threadfence();
  consumer_bar();
  if (tid == 0) {
    const unsigned old = atomicAdd(counters + r * hkv + h, 1u);
    misc->flag = (old == unsigned(s.nact - 1)) ? 1 : 0;
  }
  consumer_bar();
  if (misc->flag) {
    __threadfence();
    const float *base = scratch + (size_t(r) * hkv + h) * nsplit * size_t(max_rows) * kAttnRowFloats;
    for (int idx = tid; idx < rows * kHeadDim; idx += kConsumerThreads) {
      const int d = idx & (kHeadDim - 1);
      const int row = idx >> 7;
      const int tk = row / G, g = row - tk * G;
      float m = -INFINITY;
      for (int sp = 0; sp < s.nact; ++sp)
        m = fmaxf(m, __ldcg(base + (size_t(sp) * max_rows + row) * kAttnRowFloats + kHeadDim));
      float l = 0.f, o = 0.f;
      for (int sp = 0; sp < s.nact; ++sp) {
        const float *pr = base + (size_t(sp) * max_rows + row) * kAttnRowFloats;
        const float ms = __ldcg(pr + kHeadDim);
        const float c = ms == -INFINITY ? 0.f : exp2f(ms - m);
        l += __ldcg(pr + kHeadDim + 1) * c;
        o += __ldcg(pr + d) * c;
      }
      out[size_t(s.qo0 + tk) * ld_out + size_t(h * G + g) * kHeadDim + d] =
          __bfloat16_as_ushort(__float2bfloat16_rn(o / l));
    }
    if (tid == 0) counters[r * hkv + h] = 0u;
  }
}

__device__ __forceinline__ void attention_consume(WaitCtx &wc, char *smem, Misc *misc,
                                                  const Runtime &rt, const ypk_task &t,
                                                  RingPos &pos) {
  const AttnShape s = attn_shape(rt, t);
  if (!s.active) return;
  if (s.T == 1) {
    attention_consume_t<1>(wc, smem, misc, rt, t, s, pos);
  } else {
    attention_consume_t<kMaxNewTokens>(wc, smem, misc, rt, t, s, pos);
  }
}

}  // namespace ypk
