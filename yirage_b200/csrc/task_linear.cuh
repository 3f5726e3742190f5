// LINEAR task: out[b, n] = epilogue( rnorm[b] * sum_k W[n, k] * x[b, k] * norm_w[k] )
// for the weight rows [row0, row0 + nrows) owned by this worker, batch <= 8 per pass.
//
// Fused form of the reference's rmsnorm task + linear task (+ residual) + silu_mul task
// (tasks/hopper/rmsnorm_hopper.cuh:20-155, tasks/blackwell/linear_sm100_mpk.cuh:31-707,
// tasks/ampere/silu_mul.cuh:19-42; fused semantics as in tasks/ampere/norm_linear.cuh:412-427,
// where the division by the RMS happens after the matmul).
//
// This is the decode-time GEMV: 2 bytes of weight per 2*batch flops, i.e. bound by HBM.
// Data movement: W is [N, K] row-major (torch nn.Linear.weight), so the rows of a worker are
// contiguous in HBM.  The producer warp streams them through the shared-memory ring in
// stages of 16 rows x 1024 columns, one 2 KB cp.async.bulk per row (row pitch 2064 B so that
// 8 rows hit 8 different 16-byte bank groups).  Arithmetic: the batch is padded to the 8
// columns of a warp-level m16n8k16 MMA (bf16/fp16 in, fp32 accumulate) and the 16 weight
// rows of the stage are its M side, so one ldmatrix + one mma handle 512 bytes of weights
// whatever the batch; warp w owns the 128-column slice w of every stage and the eight
// partial 16x8 tiles are summed in a fixed order once per row block.  The activations of the
// pass sit in shared memory as 16-bit values already multiplied by the norm weight; batch
// rows beyond the real batch alias the last real row (their MMA columns are never stored).
#pragma once
#include "device_common.cuh"
#include "ll_handoff.cuh"

namespace ypk {

__device__ __forceinline__ float silu_mul_ref(float g, float u) {
  // Rounding points of the unfused reference: linear output in bf16, silu in fp32
  // rounded to bf16, product in bf16 (tasks/ampere/silu_mul.cuh:33-40).
  const float gr = bf16_round(g), ur = bf16_round(u);
  const float s = bf16_round(gr / (1.0f + __expf(-gr)));
  return s * ur;
}

struct LinearArgs {
  const char *x;
  const char *w;
  char *out;
  const char *norm_w;
  const char *res;
  int K, row0, nrows, ldx, ldw, ldout, ldres, out_col0;
  float eps;
  uint32_t flags;
  // flagged-word hand-off (YPK_F_LL_*): x, residual and result as 8-byte words, and the
  // tags to expect / to write this iteration
  const unsigned long long *ll_x, *ll_res;
  unsigned long long *ll_out;
  uint32_t tag_x, tag_res, tag_out;
  // K range of the task (graphs of more than 8 tokens may split an operator along K): the
  // task covers columns [k0, k0 + klen) of K; with nsplit > 1 it is split `split` of
  // `nsplit` of its row block, whose partial sums meet in the workspace `ws`
  int k0, klen, split, nsplit, ws_ld, ws_tok, cnt_idx;
  int x_tmap;   // tensor map of x for the tensor-core path (graphs of more than 8 tokens), or -1
  float *ws, *ws_ss;
  unsigned int *ws_cnt;
  // RMSNorm carried across two operators (YPK_F_NORM_OUT / YPK_F_NORM_PRE): the scaled copy
  // of the result, the sums of squares per (row block, token) and their layout
  char *xg;
  float *ss_io;
  int ss_blk, ss_pitch;   // producer: its block; consumer: the number of blocks
};

__device__ __forceinline__ LinearArgs linear_args(const ypk_task &t, const Runtime *rt = nullptr,
                                                  long long iter = 0) {
  LinearArgs a;
  a.ll_x = reinterpret_cast<const unsigned long long *>(t.ptr[5]);
  a.ll_res = reinterpret_cast<const unsigned long long *>(t.ptr[6]);
  a.ll_out = reinterpret_cast<unsigned long long *>(t.ptr[7]);
  a.tag_x = a.tag_res = a.tag_out = 0;
  if (rt != nullptr) {
    a.tag_x = ll_tag(*rt, iter, t.iarg[10]);
    a.tag_res = ll_tag(*rt, iter, t.iarg[11]);
    a.tag_out = ll_tag(*rt, iter, t.iarg[12]);
  }
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
  a.k0 = t.iarg[13];
  a.klen = t.iarg[14] > 0 ? t.iarg[14] : a.K - a.k0;
  a.split = t.iarg[15] & 0xff;
  a.nsplit = max(1, (t.iarg[15] >> 8) & 0xff);
  a.ws_tok = t.iarg[15] >> 16;      // tokens per split slot of the workspace
  a.ws_ld = t.iarg[8];              // its row pitch (weight rows of the operator)
  a.x_tmap = t.iarg[11];
  a.cnt_idx = t.iarg[10];           // row block's counter (the tag fields are free in wide graphs)
  a.ws = a.ws_ss = nullptr;
  a.ws_cnt = nullptr;
  a.xg = reinterpret_cast<char *>(t.ptr_aux);
  a.ss_io = reinterpret_cast<float *>((t.flags & YPK_F_NORM_OUT) ? t.ptr[6] : t.ptr[3]);
  a.ss_blk = t.iarg[12] & 0xffff;
  a.ss_pitch = t.iarg[12] >> 16;
  if (a.nsplit > 1) {
    a.ws = reinterpret_cast<float *>(t.ptr[5]);
    a.ws_ss = reinterpret_cast<float *>(t.ptr[6]);
    a.ws_cnt = reinterpret_cast<unsigned int *>(t.ptr[7]);
  }
  return a;
}

// ---- RMSNorm carried across two operators ---------------------------------------------------
// YPK_F_NORM_OUT: up to four neighbouring finished values (before rounding) of a token row at
// output column `col`: stores them times the following norm's weight `g` into the row `xrow`
// of the scaled copy and returns the sum of their squares, both from the values as rounded
// for `out`.
// (Out of line and with plain arguments: taking the LinearArgs by reference would give the
// struct an address, i.e. a home in local memory, for every LINEAR task.)
template <bool F16>
static __device__ __noinline__ float norm_out_quad(const uint16_t *g, uint16_t *xrow, int col, float v0,
                                                   float v1, float v2, float v3, int n, bool vec) {
  const float v[4] = {v0, v1, v2, v3};
  float sq = 0.f;
  uint16_t o[4] = {0, 0, 0, 0};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (i < n) {
      const float r = cvt_one<F16>(cvt_out<F16>(v[i]));
      sq += r * r;
      o[i] = cvt_out<F16>(r * cvt_one<F16>(__ldg(g + col + i)));
    }
  }
  if (vec && n == 4) {
    *reinterpret_cast<uint2 *>(xrow + col) =
        make_uint2(uint32_t(o[0]) | (uint32_t(o[1]) << 16), uint32_t(o[2]) | (uint32_t(o[3]) << 16));
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i)
      if (i < n) xrow[col + i] = o[i];
  }
  return sq;
}
// ... and the sums of squares of the task's rows per token: sq_s[b * nq + q] holds the share
// of quad q; added in quad order, so the result does not depend on the thread schedule.
// `dst` = the block's row of the sums-of-squares buffer at the first token.
static __device__ __noinline__ void norm_out_sums(float *dst, const float *sq_s, int nq, int B) {
  consumer_bar();
  const int tid = threadIdx.x;
  if (tid < B) {
    float s = 0.f;
    for (int q = 0; q < nq; ++q) s += sq_s[tid * nq + q];
    __stcg(dst + tid, s);
  }
}

// ---- split along K ------------------------------------------------------------------------
// An operator whose rows per worker would be too few for the tensor cores (o_proj, down_proj,
// qkv of a wide graph) is cut into row blocks x K ranges.  Each task leaves the fp32 partial
// dot products of its range, [tokens][rows of the block], in its slot of the workspace
// (ws[split][token][row], L2 resident) together with its partial sums of squares, then
// arrives on the block's counter; the task that arrives last adds the slots in split order
// (so the result does not depend on who was last) and runs the epilogue.  The counter is
// never reset: the nsplit-th, 2*nsplit-th, ... arrival is the last of its iteration.
// `accs(r, b)` = this task's own partial for row r of the block and token b.
// STORE_OWN false: the caller has written its partials to its slot already.
// `sq_s`: shared scratch of B * nrows / 4 floats for YPK_F_NORM_OUT (nullptr: a path that such
// tasks never take).  With YPK_F_NORM_PRE the caller has put the RMS factors of tokens
// b0 .. b0 + B into misc->rnorm_umma.
template <bool F16, bool STORE_OWN, typename AccFn>
__device__ __forceinline__ void linear_splitk_finish(const LinearArgs &a, Misc *misc, int b0, int B,
                                                     const float *ss_part, AccFn accs,
                                                     float *sq_s = nullptr) {
  const int tid = threadIdx.x;
  const bool norm = (a.flags & (YPK_F_NORM | YPK_F_NORM_NOWEIGHT)) != 0;
  const bool pre = (a.flags & YPK_F_NORM_PRE) != 0;
  const bool nout = (a.flags & YPK_F_NORM_OUT) != 0 && sq_s != nullptr;
  const size_t slot = size_t(a.ws_tok) * size_t(a.ws_ld);
  // four neighbouring rows at a time where the workspace rows allow 16-byte accesses
  const bool vec = ((a.nrows | a.ws_ld | a.row0) & 3) == 0;
  if constexpr (STORE_OWN) {
    float *mine = a.ws + size_t(a.split) * slot;
    if (vec) {
      const int nq = a.nrows >> 2;
      for (int idx = tid; idx < nq * B; idx += kConsumerThreads) {
        const int b = idx / nq, r = (idx - b * nq) * 4;
        __stcg(reinterpret_cast<float4 *>(mine + size_t(b0 + b) * a.ws_ld + a.row0 + r),
               make_float4(accs(r, b), accs(r + 1, b), accs(r + 2, b), accs(r + 3, b)));
      }
    } else {
      for (int idx = tid; idx < a.nrows * B; idx += kConsumerThreads) {
        const int b = idx / a.nrows, r = idx - b * a.nrows;
        __stcg(mine + size_t(b0 + b) * a.ws_ld + a.row0 + r, accs(r, b));
      }
    }
  }
  // partial sums of squares: [block][split][token]
  float *ssb = a.ws_ss + (size_t(a.cnt_idx) * a.nsplit) * a.ws_tok;
  if (norm && tid < B) __stcg(ssb + size_t(a.split) * a.ws_tok + b0 + tid, ss_part[tid]);
  // The barrier orders every thread's stores before thread 0, whose gpu-scope release on the
  // counter is cumulative over them; the last arriver's acquire, passed on by the next
  // barrier, lets its threads read the other splits' slots.  (A __threadfence() by all 256
  // threads here cost about a microsecond per task.)
  consumer_bar();
  if (tid == 0) {
    // one counter per (row block, group of 16 tokens): a task passes here once per group
    unsigned int *ctr = a.ws_cnt + size_t(a.cnt_idx) * size_t((a.ws_tok + 15) >> 4) + (b0 >> 4);
    unsigned old;
    asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(old) : "l"(ctr) : "memory");
    misc->flag = ((old + 1u) % unsigned(a.nsplit)) == 0u ? 1 : 0;
  }
  consumer_bar();
  const bool last = misc->flag != 0;
  consumer_bar();   // flag is read by everybody before anyone can rewrite it
  if (!last) return;
  if (norm && tid < B) {
    float s = 0.f;
    for (int sp = 0; sp < a.nsplit; ++sp) s += __ldcg(ssb + size_t(sp) * a.ws_tok + b0 + tid);
    misc->rnorm_umma[tid] = rsqrtf(s / float(a.K) + a.eps);
  }
  consumer_bar();
  auto total = [&](int r, int b) {
    float s = 0.f;
    for (int sp = 0; sp < a.nsplit; ++sp)
      s += __ldcg(a.ws + size_t(sp) * slot + size_t(b0 + b) * a.ws_ld + a.row0 + r);
    return s;
  };
  uint16_t *out = reinterpret_cast<uint16_t *>(a.out);
  if (vec) {
    // sums of four neighbouring rows: one 16-byte load per split
    const int nq = a.nrows >> 2;
    const bool silu = (a.flags & YPK_F_SILU_MUL) != 0, res = (a.flags & YPK_F_RESIDUAL) != 0;
    for (int idx = tid; idx < nq * B; idx += kConsumerThreads) {
      const int b = idx / nq, r = (idx - b * nq) * 4;
      float4 t4 = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int sp = 0; sp < a.nsplit; ++sp) {
        const float4 p = __ldcg(reinterpret_cast<const float4 *>(
            a.ws + size_t(sp) * slot + size_t(b0 + b) * a.ws_ld + a.row0 + r));
        t4.x += p.x; t4.y += p.y; t4.z += p.z; t4.w += p.w;
      }
      float v[4] = {t4.x, t4.y, t4.z, t4.w};
      if (norm || pre) {
        const float rn = misc->rnorm_umma[b];
#pragma unroll
        for (int i = 0; i < 4; ++i) v[i] *= rn;
      }
      uint16_t *orow = out + size_t(b0 + b) * a.ldout;
      if (silu) {
        // a granule of 2 gate + 2 up rows -> 2 outputs
        const int col = a.out_col0 + ((a.row0 + r) >> 1);
        const uint32_t o = uint32_t(cvt_out<F16>(silu_mul_ref(v[0], v[2]))) |
                           (uint32_t(cvt_out<F16>(silu_mul_ref(v[1], v[3]))) << 16);
        if ((col & 1) == 0) {
          *reinterpret_cast<uint32_t *>(orow + col) = o;
        } else {
          orow[col] = uint16_t(o);
          orow[col + 1] = uint16_t(o >> 16);
        }
      } else {
        const int col = a.out_col0 + a.row0 + r;
        const uint16_t *rrow = reinterpret_cast<const uint16_t *>(a.res) + size_t(b0 + b) * a.ldres;
        if ((col & 3) == 0 && (!res || (a.ldres & 3) == 0) && (a.ldout & 3) == 0) {
          if (res) {
            const uint2 rv = __ldcg(reinterpret_cast<const uint2 *>(rrow + col));
            const float2 f0 = unpack2(cvt_pair<F16>(rv.x)), f1 = unpack2(cvt_pair<F16>(rv.y));
            v[0] += f0.x; v[1] += f0.y; v[2] += f1.x; v[3] += f1.y;
          }
          *reinterpret_cast<uint2 *>(orow + col) =
              make_uint2(uint32_t(cvt_out<F16>(v[0])) | (uint32_t(cvt_out<F16>(v[1])) << 16),
                         uint32_t(cvt_out<F16>(v[2])) | (uint32_t(cvt_out<F16>(v[3])) << 16));
        } else {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            if (res) v[i] += cvt_one<F16>(__ldcg(rrow + col + i));
            orow[col + i] = cvt_out<F16>(v[i]);
          }
        }
        if (nout)
          sq_s[idx] = norm_out_quad<F16>(reinterpret_cast<const uint16_t *>(a.norm_w),
                                         reinterpret_cast<uint16_t *>(a.xg) + size_t(b0 + b) * a.ldout, col,
                                         v[0], v[1], v[2], v[3], 4, (col & 3) == 0 && (a.ldout & 3) == 0);
      }
    }
    if (nout) norm_out_sums(a.ss_io + size_t(a.ss_blk) * a.ss_pitch + b0, sq_s, nq, B);
  } else if (a.flags & YPK_F_SILU_MUL) {
    const int ngr = a.nrows >> 2;   // granules of 2 gate + 2 up rows -> 2 outputs
    for (int idx = tid; idx < ngr * B; idx += kConsumerThreads) {
      const int b = idx / ngr, g = idx - b * ngr;
      float v[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) v[i] = total(g * 4 + i, b) * ((norm || pre) ? misc->rnorm_umma[b] : 1.f);
      const int col = a.out_col0 + ((a.row0 + g * 4) >> 1);
      uint16_t *orow = out + size_t(b0 + b) * a.ldout;
      orow[col] = cvt_out<F16>(silu_mul_ref(v[0], v[2]));
      orow[col + 1] = cvt_out<F16>(silu_mul_ref(v[1], v[3]));
    }
  } else {
    for (int idx = tid; idx < a.nrows * B; idx += kConsumerThreads) {
      const int b = idx / a.nrows, r = idx - b * a.nrows;
      float v = total(r, b);
      if (norm || pre) v *= misc->rnorm_umma[b];
      const int col = a.out_col0 + a.row0 + r;
      if (a.flags & YPK_F_RESIDUAL)
        v += cvt_one<F16>(__ldcg(reinterpret_cast<const uint16_t *>(a.res) + size_t(b0 + b) * a.ldres + col));
      out[size_t(b0 + b) * a.ldout + col] = cvt_out<F16>(v);
    }
  }
}

// Tokens per pass over the weights: 8 (one n-tile of the MMA) up to batch 8, else 16 (two
// n-tiles per weight fragment, see linear_consume_group16).
constexpr int kWideBatch = 16;
__device__ __forceinline__ int linear_group_size(int batch) {
  return batch > kMaxBatch ? kWideBatch : kMaxBatch;
}

// ------------------------------------------------------------------ producer
// Traversal (must match linear_consume): batch groups -> K chunks -> 16-row blocks
// -> 1024-column stages.
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
          // the slot may last have been written through the generic proxy (attention tiles
          // arrive by cp.async, partial tiles are zero-padded by the consumers)
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
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

__device__ __forceinline__ bool linear_produce16(WaitCtx &wc, char *smem, Misc *misc,
                                               const ypk_task &t, int batch, RingPos &pos,
                                               unsigned long long policy) {
  const int lane = threadIdx.x & 31;
  const LinearArgs a = linear_args(t);
  // groups of 16 tokens, K in chunks of one stage (see linear_consume_group16)
  const int nbg = (batch + kWideBatch - 1) / kWideBatch;
  for (int bg = 0; bg < nbg; ++bg) {
    const int KC = min(a.klen, kStageCols);
    for (int k0 = a.k0; k0 < a.k0 + a.klen; k0 += KC) {
      const int klen = min(KC, a.k0 + a.klen - k0);
      for (int r0 = 0; r0 < a.nrows; r0 += kRowBlock) {
        const int nr = min(kRowBlock, a.nrows - r0);
        for (int ks = 0; ks < klen; ks += kStageCols) {
          const int ncols = min(kStageCols, klen - ks);
          if (!wait_mbar(wc, &misc->empty_bar[pos.slot], pos.phase ^ 1u)) return false;
          // the slot may last have been written through the generic proxy (attention tiles
          // arrive by cp.async, partial tiles are zero-padded by the consumers)
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
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
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void *smem_row) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(smem_row)));
}
template <bool F16>
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                          uint32_t b1) {
  if constexpr (F16) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  } else {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
}

// Writes the finished values of `nr` rows starting at task row r0.  val(r, b) returns the
// fp32 dot product (before the RMS scale); res_s holds the residual slice of the task,
// [batch][nrows] 16-bit, staged in shared memory when the task started.
// Result pair (columns col, col + 1 of token b) in flagged-word form: into this GPU's copy
// (and the plain tensor), or, for a partial sum (YPK_F_LL_PUSH), into slot `rank` of the copy
// on rank `peer`.  The copies for the different peers are made by different threads (the
// epilogue loops run over peer x pair): one thread storing to the peers in turn pays the
// address translation of each peer's mapping one after the other, about a microsecond each,
// and the last peer in everybody's loop then runs that far behind the first.
template <bool F16, bool TP>
__device__ __forceinline__ void ll_emit(const LinearArgs &a, const Runtime &rt, int b, int col,
                                        float v0, float v1, int peer) {
  const uint32_t packed = uint32_t(cvt_out<F16>(v0)) | (uint32_t(cvt_out<F16>(v1)) << 16);
  const size_t widx = size_t(b) * size_t(a.ldout >> 1) + size_t(col >> 1);
  const unsigned long long w = ll_word(packed, a.tag_out);
  if (TP && (a.flags & YPK_F_LL_PUSH)) {
    const size_t off = size_t(reinterpret_cast<char *>(a.ll_out) - rt.arena[rt.rank]) +
                       (size_t(rt.rank) * rt.max_tok * size_t(a.ldout >> 1) + widx) * 8;
    ll_store_sys(reinterpret_cast<unsigned long long *>(rt.arena[peer] + off), w);
  } else {
    *reinterpret_cast<uint32_t *>(reinterpret_cast<uint16_t *>(a.out) + size_t(b) * a.ldout + col) =
        packed;
    ll_store(a.ll_out + widx, w);
  }
}

// Flagged-word epilogue (YPK_F_LL_OUT).  Values come from the per-warp partial tiles
// (`pall` = [8 warps][16 rows][8 tokens]) or, for a K-chunked task, from `accs`
// ([rows][8 tokens]); two neighbouring result columns per thread.
template <bool F16, bool TP>
__device__ __forceinline__ void linear_epilogue_ll(const LinearArgs &a, const Runtime &rt,
                                                const Misc *misc, const uint16_t *res_s, int r0,
                                                int nr, int b0, int bc, const float *pall,
                                                const float *accs) {
  const int tid = threadIdx.x;
  const bool norm = (a.flags & (YPK_F_NORM | YPK_F_NORM_NOWEIGHT)) != 0;
  auto val = [&](int r, int b) {
    if (pall == nullptr) return accs[r * kMaxBatch + b];
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < kConsumerWarps; ++w) s += pall[(w * kRowBlock + r) * kMaxBatch + b];
    return s;
  };
  const int ncopy = (TP && (a.flags & YPK_F_LL_PUSH)) ? rt.world : 1;
  if (a.flags & YPK_F_SILU_MUL) {
    const int npair = nr >> 2;   // one 2 gate + 2 up granule = one pair of outputs
    for (int idx0 = tid; idx0 < npair * bc * ncopy; idx0 += kConsumerThreads) {
      const int peer = idx0 / (npair * bc), idx = idx0 - peer * (npair * bc);
      const int b = idx / npair, g = idx - b * npair;
      const int rg = g * (2 * kSiluGran);
      float g0 = val(rg, b), g1 = val(rg + 1, b), u0 = val(rg + 2, b), u1 = val(rg + 3, b);
      if (norm) {
        const float rn = misc->rnorm[b];
        g0 *= rn; g1 *= rn; u0 *= rn; u1 *= rn;
      }
      const int col = a.out_col0 + ((a.row0 + r0) >> 1) + g * kSiluGran;
      ll_emit<F16, TP>(a, rt, b0 + b, col, silu_mul_ref(g0, u0), silu_mul_ref(g1, u1), peer);
    }
  } else {
    const int npair = nr >> 1;
    for (int idx0 = tid; idx0 < npair * bc * ncopy; idx0 += kConsumerThreads) {
      const int peer = idx0 / (npair * bc), idx = idx0 - peer * (npair * bc);
      const int b = idx / npair, r = (idx - b * npair) * 2;
      float v0 = val(r, b), v1 = val(r + 1, b);
      if (norm) {
        v0 *= misc->rnorm[b];
        v1 *= misc->rnorm[b];
      }
      if (a.flags & YPK_F_RESIDUAL) {
        v0 += cvt_one<F16>(res_s[b * a.nrows + r0 + r]);
        v1 += cvt_one<F16>(res_s[b * a.nrows + r0 + r + 1]);
      }
      ll_emit<F16, TP>(a, rt, b0 + b, a.out_col0 + a.row0 + r0 + r, v0, v1, peer);
    }
  }
  if (TP && rt.ll_push_fence && (a.flags & YPK_F_LL_PUSH)) asm volatile("fence.acq_rel.sys;" ::: "memory");
}

template <bool F16, typename ValFn>
__device__ __forceinline__ void linear_epilogue(const LinearArgs &a, const Misc *misc,
                                                const uint16_t *res_s, int r0, int nr, int b0,
                                                int bc, int tid, ValFn val) {
  const bool norm = (a.flags & (YPK_F_NORM | YPK_F_NORM_NOWEIGHT)) != 0;
  if (a.flags & YPK_F_SILU_MUL) {
    const int nout = nr >> 1;  // granules of kSiluGran gate rows followed by kSiluGran up rows
    for (int idx = tid; idx < nout * bc; idx += kConsumerThreads) {
      const int b = idx / nout, o = idx - b * nout;
      const int rg = (o / kSiluGran) * (2 * kSiluGran) + (o % kSiluGran);
      float g = val(rg, b), u = val(rg + kSiluGran, b);
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
      if (a.flags & YPK_F_RESIDUAL) v += cvt_one<F16>(res_s[b * a.nrows + r0 + r]);  // fp32 add
      reinterpret_cast<uint16_t *>(a.out)[size_t(b0 + b) * a.ldout + col] = cvt_out<F16>(v);
    }
  }
}

// Sum of the per-warp statistics -> misc->rnorm.  `red` is [8 warps][8] floats of scratch.
__device__ __forceinline__ void publish_rnorm(const LinearArgs &a, Misc *misc, float *red,
                                              const float (&ss)[kMaxBatch], int B, int tid) {
  const int warp = tid >> 5, lane = tid & 31;
#pragma unroll
  for (int b = 0; b < kMaxBatch; ++b) {
    const float s = warp_sum(ss[b]);
    if (lane == 0) red[warp * kMaxBatch + b] = s;
  }
  consumer_bar();
  if (tid < B) {
    float s = 0.f;
    for (int w = 0; w < kConsumerWarps; ++w) s += red[w * kMaxBatch + tid];
    misc->rnorm[tid] = rsqrtf(s / float(a.K) + a.eps);
  }
  consumer_bar();
}

// Residual slice of a task from flagged words (YPK_F_LL_RES): pairs of columns, polled until
// this iteration's producer has written them.  Returns true if a poll gave up.
__device__ __forceinline__ bool linear_stage_residual_ll(WaitCtx &wc, const LinearArgs &a,
                                                      uint16_t *res_s, int b0, int B) {
  LLPoll poll;
  const int npair = a.nrows >> 1;
  for (int i = threadIdx.x; i < npair * B; i += kConsumerThreads) {
    const int b = i / npair, rp = i - b * npair;
    const unsigned long long *src = a.ll_res + size_t(b0 + b) * size_t(a.ldres >> 1) +
                                    size_t((a.out_col0 + a.row0) >> 1) + rp;
    unsigned long long w = ll_load(src);
    while (!ll_ok(w, a.tag_res) && poll.again(wc)) w = ll_load(src);
    *reinterpret_cast<uint32_t *>(res_s + b * a.nrows + 2 * rp) = static_cast<uint32_t>(w);
  }
  return poll.failed;
}

// x[b0 .. b0 + B, k0 .. k0 + klen) from flagged words (YPK_F_LL_IN) into xs, multiplied by the
// norm weight, with the sums of squares added to ss[].  A thread takes 4 columns (two words,
// one 16-byte load) per step and has the loads of four steps in flight; words that are not
// there yet are polled again, all stragglers of the four steps in one round, so that a round
// costs one trip to L2 however many words are late.  Returns true if a poll gave up.
template <bool F16>
__device__ __forceinline__ bool linear_stage_x_ll(WaitCtx &wc, const LinearArgs &a, uint16_t *xs,
                                               int xpitch, int b0, int B, int k0, int klen,
                                               float *ss) {
  const int tid = threadIdx.x;
  const uint16_t *nw = reinterpret_cast<const uint16_t *>(a.norm_w);
  const bool has_nw = (a.flags & YPK_F_NORM) != 0;
  LLPoll poll;
  constexpr int kU = 4;
  for (int kb = tid * 4; kb < klen; kb += kConsumerThreads * 4 * kU) {
    uint2 wnv[kU];
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const int k = kb + u * kConsumerThreads * 4;
      wnv[u] = make_uint2(0u, 0u);
      if (has_nw && k < klen) wnv[u] = __ldg(reinterpret_cast<const uint2 *>(nw + k0 + k));
    }
    for (int b = 0; b < B; ++b) {
      const unsigned long long *row = a.ll_x + size_t(b0 + b) * size_t(a.ldx >> 1);
      unsigned long long w0[kU], w1[kU];
      bool late[kU];
#pragma unroll
      for (int u = 0; u < kU; ++u) late[u] = kb + u * kConsumerThreads * 4 < klen;
      for (;;) {
#pragma unroll
        for (int u = 0; u < kU; ++u)
          if (late[u]) ll_load2(row + ((k0 + kb + u * kConsumerThreads * 4) >> 1), w0[u], w1[u]);
        bool any = false;
#pragma unroll
        for (int u = 0; u < kU; ++u) {
          if (late[u]) late[u] = !(ll_ok(w0[u], a.tag_x) && ll_ok(w1[u], a.tag_x));
          any |= late[u];
        }
        if (!any || !poll.again(wc)) break;
      }
      float s = 0.f;
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        const int k = kb + u * kConsumerThreads * 4;
        if (k < klen) {
          const uint32_t p[2] = {static_cast<uint32_t>(w0[u]), static_cast<uint32_t>(w1[u])};
          const uint32_t q[2] = {wnv[u].x, wnv[u].y};
          uint32_t o[2];
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            const float2 f = unpack2(cvt_pair<F16>(p[i]));
            s += f.x * f.x + f.y * f.y;
            if (has_nw) {
              const float2 g = unpack2(cvt_pair<F16>(q[i]));
              o[i] = uint32_t(cvt_out<F16>(f.x * g.x)) | (uint32_t(cvt_out<F16>(f.y * g.y)) << 16);
            } else {
              o[i] = p[i];
            }
          }
          *reinterpret_cast<uint2 *>(xs + b * xpitch + k) = make_uint2(o[0], o[1]);
        }
      }
      ss[b] += s;
    }
  }
  return poll.failed;
}

// ---- staging for more than two tokens ---------------------------------------------------
// The loops above keep the loads of several K steps of ONE token in flight, which is right
// for one or two tokens.  With more tokens they would take the tokens one after the other,
// one trip to L2 each (8 tokens: 8 trips, ~4.5 us per 2048-column chunk against ~5 us of
// weight streaming for the whole task).  Here a token row belongs to one warp (to two warps
// for up to 4 tokens), which keeps 8 loads of its row in flight and needs no per-token
// register arrays: one running sum of squares, added to the slot of the warp's token.
// Compiled only into the MANY instantiation of the consumer (3..8 tokens), so the one- and
// two-token path keeps its code and register allocation.
template <bool F16>
__device__ __forceinline__ void stage_x_norm_rows(const uint16_t *x, int ldx, const uint16_t *nw,
                                                  bool has_nw, uint16_t *xs, int xpitch, int B,
                                                  int k0, int klen, float (&ss)[kMaxBatch]) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int wpr = B <= 4 ? 2 : 1;               // warps per token row
  const int b = warp / wpr, ph = warp - b * wpr;
  constexpr int KU = 8;
  const int step = 32 * wpr * 8;                // columns one pass of the row's warps covers
  float s = 0.f;
  if (b < B) {
    const uint16_t *row = x + size_t(b) * ldx + k0;
    for (int kb = (ph * 32 + lane) * 8; kb < klen; kb += step * KU) {
      uint4 xv[KU], wv[KU];
#pragma unroll
      for (int u = 0; u < KU; ++u) {
        const int k = kb + u * step;
        xv[u] = wv[u] = make_uint4(0u, 0u, 0u, 0u);
        if (k < klen) {
          xv[u] = __ldcg(reinterpret_cast<const uint4 *>(row + k));
          if (has_nw) wv[u] = __ldg(reinterpret_cast<const uint4 *>(nw + k0 + k));
        }
      }
#pragma unroll
      for (int u = 0; u < KU; ++u) {
        const int k = kb + u * step;
        if (k < klen) {
          const uint32_t p[4] = {xv[u].x, xv[u].y, xv[u].z, xv[u].w};
          const uint32_t q[4] = {wv[u].x, wv[u].y, wv[u].z, wv[u].w};
          uint32_t o[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 f = unpack2(cvt_pair<F16>(p[i]));
            s += f.x * f.x + f.y * f.y;
            if (has_nw) {
              const float2 g = unpack2(cvt_pair<F16>(q[i]));
              o[i] = uint32_t(cvt_out<F16>(f.x * g.x)) | (uint32_t(cvt_out<F16>(f.y * g.y)) << 16);
            } else {
              o[i] = p[i];
            }
          }
          *reinterpret_cast<uint4 *>(xs + b * xpitch + k) = make_uint4(o[0], o[1], o[2], o[3]);
        }
      }
    }
  }
#pragma unroll
  for (int bb = 0; bb < kMaxBatch; ++bb)
    if (bb == b) ss[bb] += s;
}

// The same from flagged words: 4 columns (two words, one 16-byte load) per step; words that
// are not there yet are asked for again, all stragglers of the 8 steps in one round.
template <bool F16>
__device__ __forceinline__ void stage_x_ll_rows(const WaitCtx &wc, LLPoll &poll,
                                                const unsigned long long *ll_x, int ldx, uint32_t tag,
                                                const uint16_t *nw, bool has_nw, uint16_t *xs,
                                                int xpitch, int b0, int B, int k0, int klen,
                                                float (&ss)[kMaxBatch]) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int wpr = B <= 4 ? 2 : 1;
  const int b = warp / wpr, ph = warp - b * wpr;
  constexpr int KU = 8;
  const int step = 32 * wpr * 4;
  float s = 0.f;
  if (b < B) {
    const unsigned long long *row = ll_x + size_t(b0 + b) * size_t(ldx >> 1) + (k0 >> 1);
    for (int kb = (ph * 32 + lane) * 4; kb < klen; kb += step * KU) {
      unsigned long long w0[KU], w1[KU];
      bool late[KU];
#pragma unroll
      for (int u = 0; u < KU; ++u) late[u] = kb + u * step < klen;
      for (;;) {
#pragma unroll
        for (int u = 0; u < KU; ++u)
          if (late[u]) ll_load2(row + ((kb + u * step) >> 1), w0[u], w1[u]);
        bool any = false;
#pragma unroll
        for (int u = 0; u < KU; ++u) {
          if (late[u]) late[u] = !(ll_ok(w0[u], tag) && ll_ok(w1[u], tag));
          any |= late[u];
        }
        if (!any || !poll.again(wc)) break;
      }
#pragma unroll
      for (int u = 0; u < KU; ++u) {
        const int k = kb + u * step;
        if (k < klen) {
          const uint32_t p[2] = {static_cast<uint32_t>(w0[u]), static_cast<uint32_t>(w1[u])};
          // the norm weights (a few KB, hot in L1) are fetched here rather than before the
          // poll: held across it they cost 16 registers that this function does not have
          uint2 wn = make_uint2(0u, 0u);
          if (has_nw) wn = __ldg(reinterpret_cast<const uint2 *>(nw + k0 + k));
          const uint32_t q[2] = {wn.x, wn.y};
          uint32_t o[2];
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            const float2 f = unpack2(cvt_pair<F16>(p[i]));
            s += f.x * f.x + f.y * f.y;
            if (has_nw) {
              const float2 g = unpack2(cvt_pair<F16>(q[i]));
              o[i] = uint32_t(cvt_out<F16>(f.x * g.x)) | (uint32_t(cvt_out<F16>(f.y * g.y)) << 16);
            } else {
              o[i] = p[i];
            }
          }
          *reinterpret_cast<uint2 *>(xs + b * xpitch + k) = make_uint2(o[0], o[1]);
        }
      }
    }
  }
#pragma unroll
  for (int bb = 0; bb < kMaxBatch; ++bb)
    if (bb == b) ss[bb] += s;
}

// LL = the task uses the flagged-word hand-off somewhere (YPK_F_LL_*); the two instantiations
// are separate out-of-line functions, so the event path compiles as if the other did not exist.
// TP = the kernel variant that can push partial sums to peer GPUs (YPK_F_LL_PUSH).
// MANY = the instantiation for 3..8 tokens (batched staging, see above).
template <bool F16, bool LL, bool TP, bool MANY>
__device__ __forceinline__ void linear_consume_group(WaitCtx &wc, char *smem, Misc *misc,
                                                     const Runtime &rt, const LinearArgs &a,
                                                     int b0, int B, RingPos &pos) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  uint16_t *xs = reinterpret_cast<uint16_t *>(smem + kOffXs);
  float *part = reinterpret_cast<float *>(smem + kOffPart);          // [2][8 warps][16][8]
  uint16_t *res_s = reinterpret_cast<uint16_t *>(smem + kOffRes);    // [B][nrows]
  float *accs = reinterpret_cast<float *>(smem + kOffAcc);           // [nrows][8] when chunked
  const uint16_t *x = reinterpret_cast<const uint16_t *>(a.x) + size_t(b0) * a.ldx;
  const uint16_t *nw = reinterpret_cast<const uint16_t *>(a.norm_w);
  const bool norm = (a.flags & (YPK_F_NORM | YPK_F_NORM_NOWEIGHT)) != 0;
  const bool has_nw = (a.flags & YPK_F_NORM) != 0;
  constexpr int kPartHalf = kConsumerWarps * kRowBlock * kMaxBatch;

  const int KC = chunk_cols(B, a.K);
  const bool chunked = KC < a.K;
  const int xpitch = KC + 8;  // elements; +16 bytes keeps the batch rows on distinct banks
  if (chunked) {
    for (int i = tid; i < a.nrows * kMaxBatch; i += kConsumerThreads) accs[i] = 0.f;
  }
  bool poll_failed = false;
  if (LL && (a.flags & YPK_F_RESIDUAL) && (a.flags & YPK_F_LL_RES)) {
    if constexpr (LL) poll_failed = linear_stage_residual_ll(wc, a, res_s, b0, B);
  } else if (a.flags & YPK_F_RESIDUAL) {
    for (int i = tid; i < a.nrows * B; i += kConsumerThreads) {
      const int b = i / a.nrows, r = i - b * a.nrows;
      res_s[i] = __ldcg(reinterpret_cast<const uint16_t *>(a.res) + size_t(b0 + b) * a.ldres +
                        a.out_col0 + a.row0 + r);
    }
  }
  float ss[kMaxBatch];
#pragma unroll
  for (int b = 0; b < kMaxBatch; ++b) ss[b] = 0.f;

  // lane-constant parts of the ldmatrix addresses
  const int a_row = ((lane >> 3) & 1) * 8 + (lane & 7);      // row of the 16-row block
  const int a_kof = ((lane >> 4) & 1) * 8;                   // k offset inside a 16-wide step
  const int b_row = min(lane & 7, B - 1);                    // batch row (aliased beyond B)
  const int b_kof = (lane >> 3) * 8;                         // k offset inside a 32-wide pair

  int pb = 0;
  bool rnorm_ready = !norm;
  for (int k0 = 0; k0 < a.K; k0 += KC) {
    const int klen = min(KC, a.K - k0);
    consumer_bar();  // the previous pass is done with xs
    // Stage x[b, k0:k0+klen] into shared memory as 16-bit values.  Without a norm this is a
    // plain copy and goes global -> shared with 16-byte cp.async (one round trip whatever
    // K).  With a norm the values pass through registers: multiplied by the norm weight and
    // squared into the RMS statistics (fp32, as rmsnorm_hopper.cuh); the loads of four
    // iterations are issued before the first is used.
    if (LL && (a.flags & YPK_F_LL_IN) && !(MANY && (a.flags & YPK_F_LL_OPT))) {
      if constexpr (LL && MANY) {
        LLPoll poll;
        stage_x_ll_rows<F16>(wc, poll, a.ll_x, a.ldx, a.tag_x, nw, has_nw, xs, xpitch, b0, B, k0, klen, ss);
        poll_failed |= poll.failed;
      } else if constexpr (LL) {
        poll_failed |= linear_stage_x_ll<F16>(wc, a, xs, xpitch, b0, B, k0, klen, ss);
      }
    } else if (!norm) {
      for (int k = tid * 8; k < klen; k += kConsumerThreads * 8) {
#pragma unroll
        for (int b = 0; b < kMaxBatch; ++b) {
          if (b < B) {
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(
                             smem_u32(xs + b * xpitch + k)),
                         "l"(x + size_t(b) * a.ldx + k0 + k)
                         : "memory");
          }
        }
      }
      asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
    } else if constexpr (MANY) {
      stage_x_norm_rows<F16>(x, a.ldx, nw, has_nw, xs, xpitch, B, k0, klen, ss);
    } else {
      constexpr int kU = 4;
      for (int kb = tid * 8; kb < klen; kb += kConsumerThreads * 8 * kU) {
        uint4 wnv[kU];
#pragma unroll
        for (int u = 0; u < kU; ++u) {
          const int k = kb + u * kConsumerThreads * 8;
          wnv[u] = make_uint4(0u, 0u, 0u, 0u);
          if (has_nw && k < klen) wnv[u] = __ldcg(reinterpret_cast<const uint4 *>(nw + k0 + k));
        }
#pragma unroll
        for (int b = 0; b < kMaxBatch; ++b) {
          if (b < B) {
            uint4 xv[kU];
#pragma unroll
            for (int u = 0; u < kU; ++u) {
              const int k = kb + u * kConsumerThreads * 8;
              xv[u] = make_uint4(0u, 0u, 0u, 0u);
              if (k < klen)
                xv[u] = __ldcg(reinterpret_cast<const uint4 *>(x + size_t(b) * a.ldx + k0 + k));
            }
#pragma unroll
            for (int u = 0; u < kU; ++u) {
              const int k = kb + u * kConsumerThreads * 8;
              if (k < klen) {
                const uint32_t p[4] = {xv[u].x, xv[u].y, xv[u].z, xv[u].w};
                const uint32_t q[4] = {wnv[u].x, wnv[u].y, wnv[u].z, wnv[u].w};
                uint32_t o[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  const float2 f = unpack2(cvt_pair<F16>(p[i]));
                  ss[b] += f.x * f.x + f.y * f.y;
                  if (has_nw) {
                    const float2 g = unpack2(cvt_pair<F16>(q[i]));
                    o[i] = uint32_t(cvt_out<F16>(f.x * g.x)) |
                           (uint32_t(cvt_out<F16>(f.y * g.y)) << 16);
                  } else {
                    o[i] = p[i];
                  }
                }
                *reinterpret_cast<uint4 *>(xs + b * xpitch + k) = make_uint4(o[0], o[1], o[2], o[3]);
              }
            }
          }
        }
      }
    }
    // a poll that gave up is known to one thread: the mbarrier waits below need the
    // failure state to be the same across the warp
    if constexpr (LL) wc.failed = __any_sync(0xffffffffu, poll_failed || wc.failed);
    consumer_bar();
    if (tid == 0 && misc->prof_rec && k0 == 0) misc->prof_rec[4] = globaltimer();

    for (int r0 = 0; r0 < a.nrows; r0 += kRowBlock) {
      const int nr = min(kRowBlock, a.nrows - r0);
      float d[4] = {0.f, 0.f, 0.f, 0.f};
      for (int ks = 0; ks < klen; ks += kStageCols) {
        const int ncols = min(kStageCols, klen - ks);
        const bool got = wait_mbar(wc, &misc->full_bar[pos.slot], pos.phase);
        const int c0 = warp * kWarpCols;
        if (got && c0 < ncols) {
          const char *stage = smem + kOffRing + pos.slot * kStageBytes;
          const char *ap = stage + a_row * kRowPitch + (c0 + a_kof) * 2;
          const uint16_t *bp = xs + b_row * xpitch + ks + c0 + b_kof;
          const int nsteps = min(kWarpCols, ncols - c0) / 32;  // pairs of 16-wide k steps
          if (nsteps == kWarpCols / 32) {
            // full slice: all twelve fragment loads first (the asm statements keep program
            // order and a warp issues in order), then the eight MMAs on two accumulators
            uint32_t bf[4][4], a0[4][4], a1[4][4];
#pragma unroll
            for (int s = 0; s < 4; ++s) {
              ldmatrix_x4(bf[s], bp + s * 32);
              ldmatrix_x4(a0[s], ap + s * 64);
              ldmatrix_x4(a1[s], ap + s * 64 + 32);
            }
            float e[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int s = 0; s < 4; ++s) {
              mma_16816<F16>(d, a0[s], bf[s][0], bf[s][1]);
              mma_16816<F16>(e, a1[s], bf[s][2], bf[s][3]);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) d[i] += e[i];
          } else {
            for (int s = 0; s < nsteps; ++s) {
              uint32_t bf[4], a0[4], a1[4];
              ldmatrix_x4(bf, bp + s * 32);
              ldmatrix_x4(a0, ap + s * 64);
              ldmatrix_x4(a1, ap + s * 64 + 32);
              mma_16816<F16>(d, a0, bf[0], bf[1]);
              mma_16816<F16>(d, a1, bf[2], bf[3]);
            }
          }
        }
        __syncwarp();
        if (lane == 0 && got) mbar_arrive(&misc->empty_bar[pos.slot]);
        pos.advance();
      }
      if (tid == 0 && misc->prof_rec && r0 + kRowBlock >= a.nrows) misc->prof_rec[5] = globaltimer();
      // this warp's partial tile: rows lane/4 and lane/4+8, batch columns (lane%4)*2, +1
      float *pp = part + pb * kPartHalf + warp * (kRowBlock * kMaxBatch);
      const int pr = lane >> 2, pc = (lane & 3) * 2;
      *reinterpret_cast<float2 *>(pp + pr * kMaxBatch + pc) = make_float2(d[0], d[1]);
      *reinterpret_cast<float2 *>(pp + (pr + 8) * kMaxBatch + pc) = make_float2(d[2], d[3]);
      if (!rnorm_ready && !chunked) {
        // statistics are complete after the single staging pass; accs is idle here
        publish_rnorm(a, misc, accs, ss, B, tid);
        rnorm_ready = true;
      } else {
        consumer_bar();
      }
      const float *pall = part + pb * kPartHalf;
      auto summed = [&](int r, int b) {
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < kConsumerWarps; ++w) s += pall[(w * kRowBlock + r) * kMaxBatch + b];
        return s;
      };
      if (!chunked) {
        if (LL && (a.flags & YPK_F_LL_OUT)) {
          if constexpr (LL) linear_epilogue_ll<F16, TP>(a, rt, misc, res_s, r0, nr, b0, B, pall, nullptr);
        } else {
          linear_epilogue<F16>(a, misc, res_s, r0, nr, b0, B, tid, summed);
        }
      } else {
        for (int idx = tid; idx < nr * B; idx += kConsumerThreads) {
          const int b = idx / nr, r = idx - b * nr;
          accs[(r0 + r) * kMaxBatch + b] += summed(r, b);
        }
      }
      pb ^= 1;
    }
  }
  if (chunked) {
    // statistics cover the whole K only now; the idle half of part is the scratch
    if (norm) {
      consumer_bar();
      publish_rnorm(a, misc, part + pb * kPartHalf, ss, B, tid);
    } else {
      consumer_bar();
    }
    auto fromacc = [&](int r, int b) { return accs[r * kMaxBatch + b]; };
    if (LL && (a.flags & YPK_F_LL_OUT)) {
      if constexpr (LL) linear_epilogue_ll<F16, TP>(a, rt, misc, res_s, 0, a.nrows, b0, B, nullptr, accs);
    } else {
      linear_epilogue<F16>(a, misc, res_s, 0, a.nrows, b0, B, tid, fromacc);
    }
  }
}

// Epilogue from fp32 sums held somewhere addressable (shared memory): acc(r, b) = sum for row r
// of the task and token b of the group; four consecutive rows per thread and step.  RMS
// factors, if any, are in misc->rnorm_umma.
template <bool F16, typename AccFn>
__device__ __forceinline__ void linear_epilogue_quads(const LinearArgs &a, const Misc *misc, int b0,
                                                      int B, bool norm, AccFn acc, float *sq_s = nullptr) {
  const bool silu = (a.flags & YPK_F_SILU_MUL) != 0;
  const bool nout = (a.flags & YPK_F_NORM_OUT) != 0 && sq_s != nullptr && !silu;
  const int nquads = (a.nrows + 3) >> 2;
  for (int it = threadIdx.x; it < nquads * B; it += kConsumerThreads) {
    const int b = it / nquads, r = (it - b * nquads) * 4;
    float v[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = r + i < a.nrows ? acc(r + i, b) : 0.f;
    if (norm) {
      const float rn = misc->rnorm_umma[b];
#pragma unroll
      for (int i = 0; i < 4; ++i) v[i] *= rn;
    }
    uint16_t *orow = reinterpret_cast<uint16_t *>(a.out) + size_t(b0 + b) * a.ldout;
    if (silu) {
      const int col = a.out_col0 + ((a.row0 + r) >> 1);
      *reinterpret_cast<uint32_t *>(orow + col) =
          uint32_t(cvt_out<F16>(silu_mul_ref(v[0], v[2]))) | (uint32_t(cvt_out<F16>(silu_mul_ref(v[1], v[3]))) << 16);
    } else {
      const int col = a.out_col0 + a.row0 + r;
      const uint16_t *rrow = reinterpret_cast<const uint16_t *>(a.res) + size_t(b0 + b) * a.ldres;
      const bool res = (a.flags & YPK_F_RESIDUAL) != 0;
      if (r + 4 <= a.nrows && (col & 3) == 0 && (a.ldout & 3) == 0 && (!res || (a.ldres & 3) == 0)) {
        if (res) {
          const uint2 rv = __ldcg(reinterpret_cast<const uint2 *>(rrow + col));
          const float2 f0 = unpack2(cvt_pair<F16>(rv.x)), f1 = unpack2(cvt_pair<F16>(rv.y));
          v[0] += f0.x; v[1] += f0.y; v[2] += f1.x; v[3] += f1.y;
        }
        *reinterpret_cast<uint2 *>(orow + col) =
            make_uint2(uint32_t(cvt_out<F16>(v[0])) | (uint32_t(cvt_out<F16>(v[1])) << 16),
                       uint32_t(cvt_out<F16>(v[2])) | (uint32_t(cvt_out<F16>(v[3])) << 16));
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          if (r + i < a.nrows) {
            if (res) v[i] += cvt_one<F16>(__ldcg(rrow + col + i));
            orow[col + i] = cvt_out<F16>(v[i]);
          }
        }
      }
      if (nout)
        sq_s[it] = norm_out_quad<F16>(reinterpret_cast<const uint16_t *>(a.norm_w),
                                      reinterpret_cast<uint16_t *>(a.xg) + size_t(b0 + b) * a.ldout, col,
                                      v[0], v[1], v[2], v[3], min(4, a.nrows - r),
                                      (col & 3) == 0 && (a.ldout & 3) == 0);
    }
  }
  if (nout) norm_out_sums(a.ss_io + size_t(a.ss_blk) * a.ss_pitch + b0, sq_s, nquads, B);
}

// ------------------------------------------------------------------ 16 tokens per pass
// More than 8 tokens: the weights are streamed once per 16 tokens.  Every weight fragment
// (ldmatrix of 16 rows x 16 columns) feeds two m16n8k16 MMAs, tokens 0..7 and 8..15, so
// the extra tokens cost tensor-pipe issue slots (a few per cent in use) and no HBM bytes.
// The activations of 16 tokens do not fit shared memory for a whole K, so K goes in chunks
// of one ring stage (1024 columns), one stage per (chunk, 16-row block).  A barrier and a
// cross-warp sum after every stage would cost as much as the stage's HBM time, so each warp
// adds its partial tile straight into a shared fp32 accumulator [rows][16] with
// red.shared.add.f32 and the warps only meet at chunk boundaries.  (The order of those eight
// additions is not fixed: results of this path can differ in the last fp32 bit between runs,
// unlike the 8-token path.)  The residual is read in the epilogue.
template <bool F16>
__device__ __forceinline__ void linear_consume_group16(WaitCtx &wc, char *smem, Misc *misc,
                                                       const LinearArgs &a, int b0, int B,
                                                       RingPos &pos) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  constexpr int kTok = kWideBatch;
  constexpr int kXs16Bytes = kTok * (kStageCols + 8) * 2;                  // 33024
  static_assert(kXs16Bytes + kMaxAccRows * kTok * 4 <= kScratchSmemBytes, "accumulators do not fit");
  uint16_t *xs = reinterpret_cast<uint16_t *>(smem + kOffXs);
  float *accs = reinterpret_cast<float *>(smem + kOffXs + kXs16Bytes);     // [nrows][16]
  const uint16_t *x = reinterpret_cast<const uint16_t *>(a.x) + size_t(b0) * a.ldx;
  const uint16_t *nw = reinterpret_cast<const uint16_t *>(a.norm_w);
  const bool norm = (a.flags & (YPK_F_NORM | YPK_F_NORM_NOWEIGHT)) != 0;
  const bool has_nw = (a.flags & YPK_F_NORM) != 0;
  const int KC = min(a.klen, kStageCols);
  const int xpitch = KC + 8;

  for (int i = tid; i < a.nrows * kTok; i += kConsumerThreads) accs[i] = 0.f;
  float ss[kTok / 2];
#pragma unroll
  for (int i = 0; i < kTok / 2; ++i) ss[i] = 0.f;

  const int a_row = ((lane >> 3) & 1) * 8 + (lane & 7);
  const int a_kof = ((lane >> 4) & 1) * 8;
  const int b_row0 = min(lane & 7, B - 1), b_row1 = min(8 + (lane & 7), B - 1);
  const int b_kof = (lane >> 3) * 8;

  for (int k0 = a.k0; k0 < a.k0 + a.klen; k0 += KC) {
    const int klen = min(KC, a.k0 + a.klen - k0);
    consumer_bar();  // the previous chunk is done with xs (and the accumulators are zeroed)
    if (!norm) {
      for (int k = tid * 8; k < klen; k += kConsumerThreads * 8) {
#pragma unroll
        for (int b = 0; b < kTok; ++b) {
          if (b < B) {
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(xs + b * xpitch + k)),
                         "l"(x + size_t(b) * a.ldx + k0 + k)
                         : "memory");
          }
        }
      }
      asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
    } else {
      // a chunk is at most 1024 columns: 128 threads x 8 columns; each half of the block takes
      // the tokens of one parity
      const int par = tid >> 7, k = (tid & 127) * 8;
      if (k < klen) {
        uint4 wnv = make_uint4(0u, 0u, 0u, 0u);
        if (has_nw) wnv = __ldcg(reinterpret_cast<const uint4 *>(nw + k0 + k));
        const uint32_t q[4] = {wnv.x, wnv.y, wnv.z, wnv.w};
        uint4 xv[kTok / 2];
#pragma unroll
        for (int i = 0; i < kTok / 2; ++i) {
          const int b = par + 2 * i;
          xv[i] = make_uint4(0u, 0u, 0u, 0u);
          if (b < B) xv[i] = __ldcg(reinterpret_cast<const uint4 *>(x + size_t(b) * a.ldx + k0 + k));
        }
#pragma unroll
        for (int i = 0; i < kTok / 2; ++i) {
          const int b = par + 2 * i;
          if (b < B) {
            const uint32_t p[4] = {xv[i].x, xv[i].y, xv[i].z, xv[i].w};
            uint32_t o[4];
            float s2 = 0.f;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 f = unpack2(cvt_pair<F16>(p[e]));
              s2 += f.x * f.x + f.y * f.y;
              if (has_nw) {
                const float2 g = unpack2(cvt_pair<F16>(q[e]));
                o[e] = uint32_t(cvt_out<F16>(f.x * g.x)) | (uint32_t(cvt_out<F16>(f.y * g.y)) << 16);
              } else {
                o[e] = p[e];
              }
            }
            ss[i] += s2;   // token par + 2 * i
            *reinterpret_cast<uint4 *>(xs + b * xpitch + k) = make_uint4(o[0], o[1], o[2], o[3]);
          }
        }
      }
    }
    consumer_bar();

    for (int r0 = 0; r0 < a.nrows; r0 += kRowBlock) {
      float d0[4] = {0.f, 0.f, 0.f, 0.f}, d1[4] = {0.f, 0.f, 0.f, 0.f};
      const bool got = wait_mbar(wc, &misc->full_bar[pos.slot], pos.phase);
      const int c0 = warp * kWarpCols;
      const bool mine = got && c0 < klen;
      if (mine) {
        const char *stage = smem + kOffRing + pos.slot * kStageBytes;
        const char *ap = stage + a_row * kRowPitch + (c0 + a_kof) * 2;
        const uint16_t *bp0 = xs + b_row0 * xpitch + c0 + b_kof;
        const uint16_t *bp1 = xs + b_row1 * xpitch + c0 + b_kof;
        const int nsteps = min(kWarpCols, klen - c0) / 32;
        if (nsteps == kWarpCols / 32) {
          // full slice: the sixteen fragment loads first (the asm statements keep program
          // order and a warp issues in order), then the sixteen MMAs on four accumulators
          uint32_t f0[4][4], f1[4][4], a0[4][4], a1[4][4];
#pragma unroll
          for (int s = 0; s < 4; ++s) {
            ldmatrix_x4(f0[s], bp0 + s * 32);
            ldmatrix_x4(f1[s], bp1 + s * 32);
            ldmatrix_x4(a0[s], ap + s * 64);
            ldmatrix_x4(a1[s], ap + s * 64 + 32);
          }
          float e0[4] = {0.f, 0.f, 0.f, 0.f}, e1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int s = 0; s < 4; ++s) {
            mma_16816<F16>(d0, a0[s], f0[s][0], f0[s][1]);
            mma_16816<F16>(d1, a0[s], f1[s][0], f1[s][1]);
            mma_16816<F16>(e0, a1[s], f0[s][2], f0[s][3]);
            mma_16816<F16>(e1, a1[s], f1[s][2], f1[s][3]);
          }
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            d0[i] += e0[i];
            d1[i] += e1[i];
          }
        } else {
          for (int s = 0; s < nsteps; ++s) {
            uint32_t f0[4], f1[4], a0[4], a1[4];
            ldmatrix_x4(f0, bp0 + s * 32);
            ldmatrix_x4(f1, bp1 + s * 32);
            ldmatrix_x4(a0, ap + s * 64);
            ldmatrix_x4(a1, ap + s * 64 + 32);
            mma_16816<F16>(d0, a0, f0[0], f0[1]);
            mma_16816<F16>(d1, a0, f1[0], f1[1]);
            mma_16816<F16>(d0, a1, f0[2], f0[3]);
            mma_16816<F16>(d1, a1, f1[2], f1[3]);
          }
        }
      }
      __syncwarp();
      if (lane == 0 && got) mbar_arrive(&misc->empty_bar[pos.slot]);
      pos.advance();
      if (mine) {
        // this warp's partial tile: rows lane/4 and +8, tokens (lane%4)*2, +1 and those + 8
        const int pr = r0 + (lane >> 2), pc = (lane & 3) * 2;
        if (pr < a.nrows) {
          atomicAdd(accs + pr * kTok + pc, d0[0]);
          atomicAdd(accs + pr * kTok + pc + 1, d0[1]);
          atomicAdd(accs + pr * kTok + 8 + pc, d1[0]);
          atomicAdd(accs + pr * kTok + 8 + pc + 1, d1[1]);
        }
        if (pr + 8 < a.nrows) {
          atomicAdd(accs + (pr + 8) * kTok + pc, d0[2]);
          atomicAdd(accs + (pr + 8) * kTok + pc + 1, d0[3]);
          atomicAdd(accs + (pr + 8) * kTok + 8 + pc, d1[2]);
          atomicAdd(accs + (pr + 8) * kTok + 8 + pc + 1, d1[3]);
        }
      }
    }
  }
  consumer_bar();   // every warp's last additions are in
  if (a.nsplit > 1) {
    // this task covered a K range only: its partial sums (and partial statistics) go to the
    // block's workspace, the last split to arrive finishes the rows
    float *mred = reinterpret_cast<float *>(xs);   // [8 warps][8]; the activations are dead by now
    float *sstok = mred + kConsumerWarps * (kTok / 2);   // [16] per-token partial sums of squares
    if (norm) {
#pragma unroll
      for (int i = 0; i < kTok / 2; ++i) {
        const float r = warp_sum(ss[i]);
        if (lane == 0) mred[warp * (kTok / 2) + i] = r;
      }
      consumer_bar();
      if (tid < kTok) {
        const int half = tid & 1, i = tid >> 1;
        float sred = 0.f;
        for (int w = half * 4; w < half * 4 + 4; ++w) sred += mred[w * (kTok / 2) + i];
        sstok[tid] = sred;
      }
      consumer_bar();
    }
    linear_splitk_finish<F16, true>(a, misc, b0, B, sstok, [&](int r, int b) { return accs[r * kTok + b]; });
    return;
  }
  // RMS factors: each half of the block holds the statistics of the tokens of its parity
  if (norm) {
    float rs[kTok / 2];
#pragma unroll
    for (int i = 0; i < kTok / 2; ++i) rs[i] = warp_sum(ss[i]);
    float *mred = reinterpret_cast<float *>(xs);   // [8 warps][8]; the activations are dead by now
    if (lane == 0) {
#pragma unroll
      for (int i = 0; i < kTok / 2; ++i) mred[warp * (kTok / 2) + i] = rs[i];
    }
    consumer_bar();
    if (tid < B) {
      const int half = tid & 1, i = tid >> 1;   // warps 0..3 hold the even tokens, 4..7 the odd ones
      float sred = 0.f;
      for (int w = half * 4; w < half * 4 + 4; ++w) sred += mred[w * (kTok / 2) + i];
      misc->rnorm_umma[tid] = rsqrtf(sred / float(a.K) + a.eps);
    }
    consumer_bar();
  }
  linear_epilogue_quads<F16>(a, misc, b0, B, norm, [&](int r, int b) { return accs[r * kTok + b]; });
}

// More than 8 tokens on the GEMV path: groups of 16.
__device__ __forceinline__ void linear_consume_groups16(WaitCtx &wc, char *smem, Misc *misc,
                                                        const ypk_task &t, int batch, RingPos &pos) {
  const LinearArgs a = linear_args(t);
  const int nbg = (batch + kWideBatch - 1) / kWideBatch;
  for (int bg = 0; bg < nbg; ++bg) {
    const int b0 = bg * kWideBatch;
    const int bc = min(kWideBatch, batch - b0);
    if (a.flags & YPK_F_F16) {
      linear_consume_group16<true>(wc, smem, misc, a, b0, bc, pos);
    } else {
      linear_consume_group16<false>(wc, smem, misc, a, b0, bc, pos);
    }
    if (bg + 1 < nbg) consumer_bar();  // smem of this group is dead before the next one starts
  }
}

template <bool LL, bool TP, bool MANY>
__device__ __forceinline__ void linear_consume_groups(WaitCtx &wc, char *smem, Misc *misc,
                                                      const Runtime &rt, const ypk_task &t,
                                                      int batch, long long iter, RingPos &pos) {
  const LinearArgs a = linear_args(t, LL ? &rt : nullptr, iter);
  const int nbg = (batch + kMaxBatch - 1) / kMaxBatch;
  for (int bg = 0; bg < nbg; ++bg) {
    const int b0 = bg * kMaxBatch;
    const int bc = min(kMaxBatch, batch - b0);
    if (a.flags & YPK_F_F16) {
      linear_consume_group<true, LL, TP, MANY>(wc, smem, misc, rt, a, b0, bc, pos);
    } else {
      linear_consume_group<false, LL, TP, MANY>(wc, smem, misc, rt, a, b0, bc, pos);
    }
    if (bg + 1 < nbg) consumer_bar();  // smem of this group is dead before the next one starts
  }
}

}  // namespace ypk
