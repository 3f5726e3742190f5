// LINEAR task: out[b, n] = epilogue( rnorm[b] * sum_k W[n, k] * x[b, k] * norm_w[k] )
// for the weight rows [row0, row0 + nrows) owned by this worker, batch <= 8 per pass.
//
// Fused form of the reference's rmsnorm task + linear task (+ residual) + silu_mul task
// (tasks/hopper/rmsnorm_hopper.cuh:20-155, tasks/blackwell/linear_sm100_mpk.cuh:31-707,
// tasks/ampere/silu_mul.cuh:19-42; fused semantics as in tasks/ampere/norm_linear.cuh:412-427,
// where the division by the RMS happens after the matmul).
//
// Data movement: W is [N, K] row-major (torch nn.Linear.weight), so the rows of a
// worker are contiguous in HBM.  The producer warp streams them in stages of
// 32 rows x 512 columns (one 1 KB cp.async.bulk per row, issued by 32 lanes at once)
// into the ring; row pitch 1040 B keeps the consumers' 16-byte reads conflict free.
// Consumers: lane <-> weight row, warp <-> 64-column slice of the stage, activations
// pre-scaled and held in shared memory as fp32 and read as warp-wide broadcasts,
// packed fp32x2 FMAs, fp32 accumulation, one fixed-order cross-warp sum per row block.
#pragma once
#include "device_common.cuh"

namespace ypk {

struct LinearArgs {
  const char *x;
  const char *w;
  char *out;
  const char *norm_w;
  const char *res;
  int K, row0, nrows, ldx, ldw, ldout, ldres, out_col0;
  float eps;
  uint32_t flags;
};

__device__ __forceinline__ LinearArgs linear_args(const ypk_task &t) {
  LinearArgs a;
  a.x = reinterpret_cast<const char *>(t.ptr[0]);
  a.w = reinterpret_cast<const char *>(t.ptr[1]);
  a.out = reinterpret_cast<char *>(t.ptr[2]);
  a.norm_w = reinterpret_cast<const char *>(t.ptr[3]);
  a.res = reinterpret_cast<const char *>(t.ptr[4]);
  a.K = t.iarg[0];
  a.row0 = t.iarg[1];
  a.nrows = t.iarg[2];
  a.ldx = t.iarg[3];
  a.ldw = t.iarg[4];
  a.ldout = t.iarg[5];
  a.ldres = t.iarg[6];
  a.out_col0 = t.iarg[7];
  a.eps = t.farg[0];
  a.flags = t.flags;
  return a;
}

// ------------------------------------------------------------------ producer
// Traversal (must match linear_consume): batch groups -> K chunks -> row blocks
// -> 512-column stages.
__device__ __forceinline__ bool linear_produce(WaitCtx &wc, char *smem, Misc *misc,
                                               const ypk_task &t, int batch, RingPos &pos,
                                               unsigned long long policy) {
  const int lane = threadIdx.x & 31;
  const LinearArgs a = linear_args(t);
  const int nbg = (batch + kMaxBatch - 1) / kMaxBatch;
  for (int bg = 0; bg < nbg; ++bg) {
    const int bc = min(kMaxBatch, batch - bg * kMaxBatch);
    const int KC = chunk_cols(bc, a.K);
    for (int k0 = 0; k0 < a.K; k0 += KC) {
      const int klen = min(KC, a.K - k0);
      for (int r0 = 0; r0 < a.nrows; r0 += kRowBlock) {
        const int nr = min(kRowBlock, a.nrows - r0);
        for (int ks = 0; ks < klen; ks += kStageCols) {
          const int ncols = min(kStageCols, klen - ks);
          if (!wait_mbar(wc, &misc->empty_bar[pos.slot], pos.phase ^ 1u)) return false;
          char *stage = smem + kOffRing + pos.slot * kStageBytes;
          if (lane == 0) mbar_expect_tx(&misc->full_bar[pos.slot], uint32_t(nr) * ncols * 2u);
          __syncwarp();
          if (lane < nr) {
            const char *src =
                a.w + (size_t(a.row0 + r0 + lane) * a.ldw + size_t(k0 + ks)) * 2u;
            bulk_g2s_hint(stage + lane * kRowPitch, src, uint32_t(ncols) * 2u,
                          &misc->full_bar[pos.slot], policy);
          }
          pos.advance();
        }
      }
    }
  }
  return true;
}

// ------------------------------------------------------------------ consumer
template <int B, bool F16>
__device__ __forceinline__ void linear_stage_math(const char *stage, const float *xs, int xs_ld,
                                                  int kofs, int ncols, int nr, int warp, int lane,
                                                  unsigned long long (&acc)[B]) {
  const int c0 = warp * 64;
  if (c0 >= ncols || lane >= nr) return;
  const uint4 *wp = reinterpret_cast<const uint4 *>(stage + lane * kRowPitch + c0 * 2);
  const float *xb = xs + kofs + c0;
#pragma unroll 4
  for (int s = 0; s < 8; ++s) {
    const uint4 wv = wp[s];
    const unsigned long long w0 = cvt_pair<F16>(wv.x), w1 = cvt_pair<F16>(wv.y),
                             w2 = cvt_pair<F16>(wv.z), w3 = cvt_pair<F16>(wv.w);
#pragma unroll
    for (int b = 0; b < B; ++b) {
      const ulonglong2 *xp = reinterpret_cast<const ulonglong2 *>(xb + b * xs_ld + s * 8);
      const ulonglong2 xa = xp[0], xc = xp[1];
      acc[b] = fma2(w0, xa.x, acc[b]);
      acc[b] = fma2(w1, xa.y, acc[b]);
      acc[b] = fma2(w2, xc.x, acc[b]);
      acc[b] = fma2(w3, xc.y, acc[b]);
    }
  }
}

__device__ __forceinline__ float silu_mul_ref(float g, float u) {
  // Rounding points of the unfused reference: linear output in bf16, silu in fp32
  // rounded to bf16, product in bf16 (tasks/ampere/silu_mul.cuh:33-40).
  const float gr = bf16_round(g), ur = bf16_round(u);
  const float s = bf16_round(gr / (1.0f + __expf(-gr)));
  return s * ur;
}

// Writes the finished values of `nr` rows starting at task row r0.
// val(r, b) returns the fp32 dot product (before the RMS scale).
template <bool F16, typename ValFn>
__device__ __forceinline__ void linear_epilogue(const LinearArgs &a, const Misc *misc, int r0,
                                                int nr, int b0, int bc, int tid, ValFn val) {
  const bool norm = (a.flags & (YPK_F_NORM | YPK_F_NORM_NOWEIGHT)) != 0;
  if (a.flags & YPK_F_SILU_MUL) {
    const int nout = nr >> 1;  // 16-row granules: 8 gate rows then 8 up rows
    for (int idx = tid; idx < nout * bc; idx += kConsumerThreads) {
      const int b = idx / nout, o = idx - b * nout;
      const int rg = (o >> 3) * 16 + (o & 7);
      float g = val(rg, b), u = val(rg + 8, b);
      if (norm) {
        g *= misc->rnorm[b];
        u *= misc->rnorm[b];
      }
      const int col = a.out_col0 + ((a.row0 + r0) >> 1) + o;
      reinterpret_cast<uint16_t *>(a.out)[size_t(b0 + b) * a.ldout + col] =
          cvt_out<F16>(silu_mul_ref(g, u));
    }
  } else {
    for (int idx = tid; idx < nr * bc; idx += kConsumerThreads) {
      const int b = idx / nr, r = idx - b * nr;
      float v = val(r, b);
      if (norm) v *= misc->rnorm[b];
      const int col = a.out_col0 + a.row0 + r0 + r;
      if (a.flags & YPK_F_RESIDUAL) {
        const uint16_t rv = __ldcg(reinterpret_cast<const uint16_t *>(a.res) +
                                   size_t(b0 + b) * a.ldres + col);
        // fp32 add, one rounding
        v += cvt_one<F16>(rv);
      }
      reinterpret_cast<uint16_t *>(a.out)[size_t(b0 + b) * a.ldout + col] = cvt_out<F16>(v);
    }
  }
}

template <int B, bool F16>
__device__ __forceinline__ void linear_consume_group(WaitCtx &wc, char *smem, Misc *misc,
                                                     const LinearArgs &a, int b0, RingPos &pos) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  float *xs = reinterpret_cast<float *>(smem + kOffXs);
  float *part = reinterpret_cast<float *>(smem + kOffPart);
  float *accs = reinterpret_cast<float *>(smem + kOffAcc);
  const uint16_t *x = reinterpret_cast<const uint16_t *>(a.x) + size_t(b0) * a.ldx;
  const uint16_t *nw = reinterpret_cast<const uint16_t *>(a.norm_w);
  const bool norm = (a.flags & (YPK_F_NORM | YPK_F_NORM_NOWEIGHT)) != 0;
  const bool has_nw = (a.flags & YPK_F_NORM) != 0;

  // RMS statistics over the full K (fp32, as rmsnorm_hopper.cuh accumulates).
  if (norm) {
    float ss[B];
#pragma unroll
    for (int b = 0; b < B; ++b) ss[b] = 0.f;
    for (int k = tid * 8; k < a.K; k += kConsumerThreads * 8) {
#pragma unroll
      for (int b = 0; b < B; ++b) {
        const uint4 v = __ldcg(reinterpret_cast<const uint4 *>(x + size_t(b) * a.ldx + k));
        const uint32_t p[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = unpack2(cvt_pair<F16>(p[i]));
          ss[b] += f.x * f.x + f.y * f.y;
        }
      }
    }
    float *red = part;  // [warp][B]
#pragma unroll
    for (int b = 0; b < B; ++b) {
      const float s = warp_sum(ss[b]);
      if (lane == 0) red[warp * B + b] = s;
    }
    consumer_bar();
    if (tid < B) {
      float s = 0.f;
      for (int w = 0; w < kConsumerWarps; ++w) s += red[w * B + tid];
      misc->rnorm[tid] = rsqrtf(s / float(a.K) + a.eps);
    }
    // rnorm and `red` are separated from their next use by the barriers below
  }

  const int KC = chunk_cols(B, a.K);
  const bool chunked = KC < a.K;
  if (chunked) {
    for (int i = tid; i < a.nrows * B; i += kConsumerThreads) accs[i] = 0.f;
  }
  int pb = 0;
  for (int k0 = 0; k0 < a.K; k0 += KC) {
    const int klen = min(KC, a.K - k0);
    consumer_bar();  // everyone is done with the previous contents of xs / red
    // stage x[b, k0 : k0+klen] * norm_w as fp32
    for (int k = tid * 8; k < klen; k += kConsumerThreads * 8) {
      float wn[8];
      if (has_nw) {
        const uint4 v = __ldcg(reinterpret_cast<const uint4 *>(nw + k0 + k));
        const uint32_t p[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = unpack2(cvt_pair<F16>(p[i]));
          wn[2 * i] = f.x;
          wn[2 * i + 1] = f.y;
        }
      }
#pragma unroll
      for (int b = 0; b < B; ++b) {
        const uint4 v = __ldcg(reinterpret_cast<const uint4 *>(x + size_t(b) * a.ldx + k0 + k));
        const uint32_t p[4] = {v.x, v.y, v.z, v.w};
        float f[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 t2 = unpack2(cvt_pair<F16>(p[i]));
          f[2 * i] = t2.x;
          f[2 * i + 1] = t2.y;
        }
        if (has_nw) {
#pragma unroll
          for (int i = 0; i < 8; ++i) f[i] *= wn[i];
        }
        float4 *dst = reinterpret_cast<float4 *>(xs + b * KC + k);
        dst[0] = make_float4(f[0], f[1], f[2], f[3]);
        dst[1] = make_float4(f[4], f[5], f[6], f[7]);
      }
    }
    consumer_bar();

    for (int r0 = 0; r0 < a.nrows; r0 += kRowBlock) {
      const int nr = min(kRowBlock, a.nrows - r0);
      unsigned long long acc[B];
#pragma unroll
      for (int b = 0; b < B; ++b) acc[b] = 0ull;
      for (int ks = 0; ks < klen; ks += kStageCols) {
        const int ncols = min(kStageCols, klen - ks);
        const bool got = wait_mbar(wc, &misc->full_bar[pos.slot], pos.phase);
        if (got) {
          linear_stage_math<B, F16>(smem + kOffRing + pos.slot * kStageBytes, xs, KC, ks, ncols,
                                    nr, warp, lane, acc);
        }
        __syncwarp();
        if (lane == 0 && got) mbar_arrive(&misc->empty_bar[pos.slot]);
        pos.advance();
      }
      float *pp = part + pb * (kConsumerWarps * kRowBlock * kMaxBatch);
#pragma unroll
      for (int b = 0; b < B; ++b) {
        const float2 f = unpack2(acc[b]);
        pp[(warp * kRowBlock + lane) * B + b] = f.x + f.y;
      }
      consumer_bar();
      auto summed = [&](int r, int b) {
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < kConsumerWarps; ++w) s += pp[(w * kRowBlock + r) * B + b];
        return s;
      };
      if (!chunked) {
        linear_epilogue<F16>(a, misc, r0, nr, b0, B, tid, summed);
      } else {
        for (int idx = tid; idx < nr * B; idx += kConsumerThreads) {
          const int b = idx / nr, r = idx - b * nr;
          accs[(r0 + r) * B + b] += summed(r, b);
        }
      }
      pb ^= 1;
    }
  }
  if (chunked) {
    consumer_bar();
    auto fromacc = [&](int r, int b) { return accs[r * B + b]; };
    linear_epilogue<F16>(a, misc, 0, a.nrows, b0, B, tid, fromacc);
  }
}

template <bool F16>
__device__ __forceinline__ void linear_consume_dispatch(WaitCtx &wc, char *smem, Misc *misc,
                                                        const LinearArgs &a, int b0, int bc,
                                                        RingPos &pos) {
  switch (bc) {
    case 1: linear_consume_group<1, F16>(wc, smem, misc, a, b0, pos); break;
    case 2: linear_consume_group<2, F16>(wc, smem, misc, a, b0, pos); break;
    case 3: linear_consume_group<3, F16>(wc, smem, misc, a, b0, pos); break;
    case 4: linear_consume_group<4, F16>(wc, smem, misc, a, b0, pos); break;
    case 5: linear_consume_group<5, F16>(wc, smem, misc, a, b0, pos); break;
    case 6: linear_consume_group<6, F16>(wc, smem, misc, a, b0, pos); break;
    case 7: linear_consume_group<7, F16>(wc, smem, misc, a, b0, pos); break;
    default: linear_consume_group<8, F16>(wc, smem, misc, a, b0, pos); break;
  }
}

__device__ __forceinline__ void linear_consume(WaitCtx &wc, char *smem, Misc *misc,
                                               const ypk_task &t, int batch, RingPos &pos) {
  const LinearArgs a = linear_args(t);
  const int nbg = (batch + kMaxBatch - 1) / kMaxBatch;
  for (int bg = 0; bg < nbg; ++bg) {
    const int b0 = bg * kMaxBatch;
    const int bc = min(kMaxBatch, batch - b0);
    if (a.flags & YPK_F_F16) {
      linear_consume_dispatch<true>(wc, smem, misc, a, b0, bc, pos);
    } else {
      linear_consume_dispatch<false>(wc, smem, misc, a, b0, bc, pos);
    }
  }
}

}  // namespace ypk
