// Latent attention over a paged cache that stores ONE latent row c_j per token (no per-head keys
// or values): every query head attends to the same rows, keys and values are both c_j.  The
// per-head key expansion is folded into the query beforehand (q'_h = W_uk,h^T q_h) and the value
// expansion is applied to the result afterwards (o_h = W_uv,h sum_j p_j c_j), so the cache traffic
// per token is R numbers instead of H * (dim + vdim).
//   softmax with a sink: the running (max, sum) pair starts at (sink_h, 1) instead of (-inf, 0),
//   which puts exp(sink_h) into the denominator exactly once, with no key and no value.
// Scores, softmax and accumulation are fp32.  Two kernels:
//   latent_attn_tile_kernel   up to 16 consecutive rows of one sequence per CTA (prompt portions), or,
//                             for decoded tokens, up to 16 heads of one token per CTA (kHeadRows)
//   latent_attn_decode_kernel one (token, head) per CTA, all 256 threads spread over keys (decoded
//                             tokens of models with fewer than 4 heads)
//   both decode forms deal the key blocks of a row to nsplit CTAs; latent_attn_merge_kernel merges them
//   window > 0: a query sees the last `window` keys up to itself only (mask + a later start of the key loop)
// A decoupled rotary part rides in the same rows: the cache row is latent | ONE rotated key part shared by all
// heads, the folded query of head h is (W_uk,h^T q_h | rotated q part), so the dot product over the row is the
// sum of both score terms; the columns of the weighted sum that belong to the rotary part are simply not used by
// the value expansion.  latent_rope_kernel writes those rows and query parts.
#include "../../include/vila_b200.h"
#include "common.cuh"
#include "kernels.h"
#include "dtype_any.cuh"

namespace vb {
namespace {

constexpr int kThreads = 256;
constexpr int BQ = 16;   // query rows per tile
constexpr int BKEY = 32; // keys per iteration
constexpr float kNegBig = -1e30f;

__device__ __forceinline__ size_t cache_row(const int32_t* pt, int page, int j) {
  return static_cast<size_t>(pt[j / page]) * page + (j % page);
}

// Shared-memory rows are R4 = ceil(R / 4) * 4 wide (zero padded) with a stride of R4 + 4 floats:
// rows start 16-byte aligned and float4 reads of 8 consecutive rows hit 8 different bank groups.
__host__ __device__ __forceinline__ int round4(int r) { return (r + 3) & ~3; }

// One warp per latent row: the page-table lookup happens once per row, the row is read with 16-byte
// loads when its width allows and widened to fp32.  Rows past nkeys and the pad columns are zero.
// Source row of key j: through a page table (pt != nullptr: pool row, elements row * ld + col0) or
// contiguous from first_row.
__device__ __forceinline__ void load_rows_block(float* Cs, int RS, int R4, const void* src, int dt,
                                                const int32_t* pt, int page, size_t first_row, int64_t ld,
                                                size_t col0, int j0, int nkeys, int R) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const bool al8 = (R & 7) == 0 && (ld & 7) == 0 && (col0 & 7) == 0;
  for (int jj = warp; jj < BKEY; jj += nw) {
    float* dst = Cs + jj * RS;
    const int j = j0 + jj;
    if (j >= nkeys) {
      for (int k = lane; k < R4; k += 32) dst[k] = 0.f;
      continue;
    }
    const size_t row = pt ? cache_row(pt, page, j) : first_row + j;
    const size_t off = row * ld + col0;
    if (dt == VILA_DT_BF16 && al8) {
      const uint4* s4 = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(src) + off);
      for (int v = lane; v < (R >> 3); v += 32) {
        const uint4 u = __ldg(s4 + v);
        float4 a, b;
        a.x = __uint_as_float(u.x << 16); a.y = __uint_as_float(u.x & 0xffff0000u);
        a.z = __uint_as_float(u.y << 16); a.w = __uint_as_float(u.y & 0xffff0000u);
        b.x = __uint_as_float(u.z << 16); b.y = __uint_as_float(u.z & 0xffff0000u);
        b.z = __uint_as_float(u.w << 16); b.w = __uint_as_float(u.w & 0xffff0000u);
        *reinterpret_cast<float4*>(dst + 8 * v) = a;
        *reinterpret_cast<float4*>(dst + 8 * v + 4) = b;
      }
    } else if (dt == VILA_DT_F32 && al8) {
      const float4* s4 = reinterpret_cast<const float4*>(static_cast<const float*>(src) + off);
      for (int v = lane; v < (R >> 2); v += 32) *reinterpret_cast<float4*>(dst + 4 * v) = __ldg(s4 + v);
    } else {
      for (int k = lane; k < R4; k += 32) dst[k] = k < R ? ld_any(src, dt, off + k) : 0.f;
    }
  }
}

// One warp per latent row: the page-table lookup happens once per row, the row is read with 16-byte
// loads when its width allows and widened to fp32.  Rows past nkeys and the pad columns are zero.
__device__ __forceinline__ void load_latent_block(float* Cs, int RS, int R4, const void* cache, int dt,
                                                  const int32_t* pt, int page, int j0, int nkeys, int R) {
  load_rows_block(Cs, RS, R4, cache, dt, pt, page, 0, R, 0, j0, nkeys, R);
}

// thread (i = tid / 16, l = tid % 16): scores of query i for keys l and l + 16 of the block (float4
// dot products), then the accumulator columns 4l .. 4l+3 (+ 64, + 128, ...) of query i.
template <int KK4, bool kHeadRows>
__global__ void __launch_bounds__(kThreads) latent_attn_tile_kernel(const vila_latent_attn_params p) {
  extern __shared__ __align__(16) float sm[];
  const int R = p.R, R4 = round4(R), RS = R4 + 4;
  float* Qs = sm;                  // [BQ][R4]
  float* Cs = Qs + BQ * R4;        // [BKEY][RS]
  float* Ps = Cs + BKEY * RS;      // [BQ][BKEY]
  const int tid = threadIdx.x, i = tid >> 4, l = tid & 15;
  const int* tile = p.tiles + 4 * blockIdx.x;
  // kHeadRows (decoded tokens): the 16 rows of the tile are 16 HEADS of one token, which all attend to
  // the same latent rows, so a block of keys is loaded once for all of them; the keys are dealt to
  // gridDim.z CTAs and merged afterwards.  Otherwise: 16 consecutive tokens of one sequence, one head.
  const int h0 = kHeadRows ? blockIdx.y * BQ : blockIdx.y;
  const int h = kHeadRows ? h0 + i : h0;
  const int row0 = tile[0], pos0 = tile[2], slot = tile[3];
  const int n = kHeadRows ? min(BQ, p.H - h0) : tile[1];
  const int split = kHeadRows ? blockIdx.z : 0, nsplit = kHeadRows ? p.nsplit : 1;
  const int32_t* pt = p.page_tables + static_cast<size_t>(slot) * p.pt_stride;
  const size_t ldq = static_cast<size_t>(p.H) * R;
  for (int idx = tid; idx < BQ * R4; idx += kThreads) {
    const int qi = idx / R4, k = idx % R4;
    const size_t src = kHeadRows ? row0 * ldq + static_cast<size_t>(h0 + qi) * R + k
                                 : (row0 + qi) * ldq + static_cast<size_t>(h0) * R + k;
    Qs[idx] = (qi < n && k < R) ? p.q[src] * p.scale : 0.f;
  }
  const bool has_sink = p.sink != nullptr && split == 0 && i < n;   // the sink belongs to split 0
  float m = has_sink ? p.sink[h] : kNegBig;
  float lsum = has_sink ? 1.0f : 0.0f;
  float4 acc[KK4];
#pragma unroll
  for (int kk = 0; kk < KK4; ++kk) acc[kk] = make_float4(0.f, 0.f, 0.f, 0.f);
  const int nkeys = kHeadRows ? pos0 + 1 : pos0 + n;
  const int my_last = kHeadRows ? pos0 : pos0 + i;  // last visible key of query i
  // sliding window: the first visible key of query i; the key loop starts at the block of the tile's first row
  const int my_first = p.window > 0 ? max(my_last - p.window + 1, 0) : 0;
  const int j_begin = p.window > 0 ? (max(pos0 - p.window + 1, 0) / BKEY) * BKEY : 0;
  for (int j0 = j_begin + split * BKEY; j0 < nkeys; j0 += nsplit * BKEY) {
    __syncthreads();  // Qs ready (first pass) / previous block consumed
    load_latent_block(Cs, RS, R4, p.cache, p.cache_dtype, pt, p.page, j0, nkeys, R);
    __syncthreads();
    float s0 = 0.f, s1 = 0.f;
    const float4* qr = reinterpret_cast<const float4*>(Qs + i * R4);
    const float4* c0 = reinterpret_cast<const float4*>(Cs + l * RS);
    const float4* c1 = reinterpret_cast<const float4*>(Cs + (l + 16) * RS);
#pragma unroll 4
    for (int k = 0; k < (R4 >> 2); ++k) {
      const float4 qv = qr[k], a = c0[k], b = c1[k];
      s0 = fmaf(qv.x, a.x, s0); s0 = fmaf(qv.y, a.y, s0); s0 = fmaf(qv.z, a.z, s0); s0 = fmaf(qv.w, a.w, s0);
      s1 = fmaf(qv.x, b.x, s1); s1 = fmaf(qv.y, b.y, s1); s1 = fmaf(qv.z, b.z, s1); s1 = fmaf(qv.w, b.w, s1);
    }
    const bool v0 = i < n && j0 + l <= my_last && j0 + l >= my_first;
    const bool v1 = i < n && j0 + l + 16 <= my_last && j0 + l + 16 >= my_first;
    s0 = v0 ? s0 : kNegBig;
    s1 = v1 ? s1 : kNegBig;
    float bm = fmaxf(s0, s1);
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, o));
    const float m_new = fmaxf(m, bm);
    const float alpha = expf(m - m_new);
    const float p0 = v0 ? expf(s0 - m_new) : 0.f, p1 = v1 ? expf(s1 - m_new) : 0.f;
    float ps = p0 + p1;
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
    lsum = lsum * alpha + ps;
    m = m_new;
    Ps[i * BKEY + l] = p0;
    Ps[i * BKEY + l + 16] = p1;
    __syncthreads();
    const float* pr = Ps + i * BKEY;
#pragma unroll
    for (int kk = 0; kk < KK4; ++kk) {
      acc[kk].x *= alpha; acc[kk].y *= alpha; acc[kk].z *= alpha; acc[kk].w *= alpha;
    }
#pragma unroll 4
    for (int jj = 0; jj < BKEY; ++jj) {
      const float pj = pr[jj];
      const float* cr = Cs + jj * RS + 4 * l;
#pragma unroll
      for (int kk = 0; kk < KK4; ++kk) {
        if (4 * l + 64 * kk < R4) {
          const float4 c = *reinterpret_cast<const float4*>(cr + 64 * kk);
          acc[kk].x = fmaf(pj, c.x, acc[kk].x); acc[kk].y = fmaf(pj, c.y, acc[kk].y);
          acc[kk].z = fmaf(pj, c.z, acc[kk].z); acc[kk].w = fmaf(pj, c.w, acc[kk].w);
        }
      }
    }
  }
  if (kHeadRows && nsplit > 1) {
    if (i < n) {   // un-normalised partial of this split: R sums, then the running max and sum
      float* part = p.partial + ((static_cast<size_t>(row0) * p.H + h) * nsplit + split) * (R + 2);
#pragma unroll
      for (int kk = 0; kk < KK4; ++kk) {
        const int k = 4 * l + 64 * kk;
        const float v[4] = {acc[kk].x, acc[kk].y, acc[kk].z, acc[kk].w};
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (k + e < R) part[k + e] = v[e];
      }
      if (l == 0) {
        part[R] = m;
        part[R + 1] = lsum;
      }
    }
    return;
  }
  if (i < n) {
    const size_t row = kHeadRows ? row0 : row0 + i;
    float g = 1.0f / lsum;
    if (p.gate) g *= sigmoid_f(ld_any(p.gate, p.gate_dtype, row * p.ldg + h));
    const size_t ob = row * ldq + static_cast<size_t>(h) * R;
#pragma unroll
    for (int kk = 0; kk < KK4; ++kk) {
      const int k = 4 * l + 64 * kk;
      const float v[4] = {acc[kk].x, acc[kk].y, acc[kk].z, acc[kk].w};
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (k + e < R) st_any(p.out, p.out_dtype, ob + k + e, v[e] * g);
    }
  }
}

// One query row per CTA.  Per block of 32 keys: 8 threads share a key's dot product, warp 0 updates
// the running softmax, then thread (k = tid % RP, jg = tid / RP) adds the keys jj = jg (mod G) into
// column k.  The G partial accumulators of a column are summed in a fixed order at the end.
template <int KK>
__global__ void __launch_bounds__(kThreads) latent_attn_decode_kernel(const vila_latent_attn_params p, int RP) {
  extern __shared__ __align__(16) float sm[];
  const int R = p.R, R4 = round4(R), RS = R4 + 4;
  float* Qs = sm;               // [R4]
  float* Cs = Qs + R4;          // [BKEY][RS]
  float* Ps = Cs + BKEY * RS;   // [BKEY] + alpha + sum + max
  const int tid = threadIdx.x;
  const int h = blockIdx.y;
  const int* tile = p.tiles + 4 * blockIdx.x;
  const int row0 = tile[0], pos0 = tile[2], slot = tile[3];
  const int32_t* pt = p.page_tables + static_cast<size_t>(slot) * p.pt_stride;
  const size_t ldq = static_cast<size_t>(p.H) * R;
  for (int k = tid; k < R4; k += kThreads)
    Qs[k] = k < R ? p.q[row0 * ldq + static_cast<size_t>(h) * R + k] * p.scale : 0.f;
  // key groups per column; at most BKEY so that the final [G][R] exchange fits into Cs
  const int G = RP >= kThreads ? 1 : (kThreads / RP < BKEY ? kThreads / RP : BKEY);
  const int jg = RP >= kThreads ? 0 : tid / RP;
  const int kcol = RP >= kThreads ? tid : (jg < G ? tid % RP : R);  // R: this thread owns no column
  float acc[KK];
#pragma unroll
  for (int kk = 0; kk < KK; ++kk) acc[kk] = 0.f;
  // split s of nsplit takes the key blocks s, s + nsplit, ...; the sink belongs to split 0
  const int split = blockIdx.z, nsplit = p.nsplit;
  const bool has_sink = p.sink != nullptr && split == 0;
  float m = has_sink ? p.sink[h] : kNegBig;   // meaningful in warp 0 only
  float lsum = has_sink ? 1.0f : 0.0f;
  const int nkeys = pos0 + 1;
  const int first = p.window > 0 ? max(pos0 - p.window + 1, 0) : 0;   // sliding window: the first visible key
  const int jj_s = tid >> 3, sub = tid & 7;
  for (int j0 = (first / BKEY + split) * BKEY; j0 < nkeys; j0 += nsplit * BKEY) {
    __syncthreads();
    load_latent_block(Cs, RS, R4, p.cache, p.cache_dtype, pt, p.page, j0, nkeys, R);
    __syncthreads();
    float s = 0.f;
    {
      const float4* q4 = reinterpret_cast<const float4*>(Qs);
      const float4* c4 = reinterpret_cast<const float4*>(Cs + jj_s * RS);
      for (int k = sub; k < (R4 >> 2); k += 8) {
        const float4 qv = q4[k], c = c4[k];
        s = fmaf(qv.x, c.x, s); s = fmaf(qv.y, c.y, s); s = fmaf(qv.z, c.z, s); s = fmaf(qv.w, c.w, s);
      }
    }
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (sub == 0) Ps[jj_s] = (j0 + jj_s < nkeys && j0 + jj_s >= first) ? s : kNegBig;
    __syncthreads();
    if (tid < 32) {
      const float sc = Ps[tid];
      const float m_new = fmaxf(m, warp_max(sc));
      const float alpha = expf(m - m_new);
      const float pv = sc > 0.5f * kNegBig ? expf(sc - m_new) : 0.f;
      lsum = lsum * alpha + warp_sum(pv);
      m = m_new;
      Ps[tid] = pv;
      if (tid == 0) Ps[BKEY] = alpha;
    }
    __syncthreads();
    const float alpha = Ps[BKEY];
#pragma unroll
    for (int kk = 0; kk < KK; ++kk) {
      const int k = kcol + kThreads * kk;
      if (k < R && (RP >= kThreads || kcol < R)) {
        float a = acc[kk] * alpha;
        for (int jj = jg; jj < BKEY; jj += G) a = fmaf(Ps[jj], Cs[jj * RS + k], a);
        acc[kk] = a;
      }
    }
  }
  __syncthreads();
  if (tid == 0) {
    Ps[BKEY + 1] = lsum;
    Ps[BKEY + 2] = m;
  }
  // cross-group reduction through Cs (reused): [G][R]
  if (G > 1) {
    if (kcol < R) Cs[jg * R + kcol] = acc[0];
    __syncthreads();
    if (jg == 0 && kcol < R) {
      float a = 0.f;
      for (int g2 = 0; g2 < G; ++g2) a += Cs[g2 * R + kcol];
      acc[0] = a;
    }
  } else {
    __syncthreads();
  }
  if (nsplit > 1) {
    // un-normalised partial result of this split: R sums, then the running max and sum
    float* part = p.partial + ((static_cast<size_t>(row0) * p.H + h) * nsplit + split) * (R + 2);
    if (jg == 0) {
#pragma unroll
      for (int kk = 0; kk < KK; ++kk) {
        const int k = kcol + kThreads * kk;
        if (k < R && (RP >= kThreads || kcol < R)) part[k] = acc[kk];
      }
    }
    if (tid == 0) {
      part[R] = Ps[BKEY + 2];
      part[R + 1] = Ps[BKEY + 1];
    }
    return;
  }
  if (jg == 0) {
    float g = 1.0f / Ps[BKEY + 1];
    if (p.gate) g *= sigmoid_f(ld_any(p.gate, p.gate_dtype, static_cast<size_t>(row0) * p.ldg + h));
#pragma unroll
    for (int kk = 0; kk < KK; ++kk) {
      const int k = kcol + kThreads * kk;
      if (k < R && (RP >= kThreads || kcol < R))
        st_any(p.out, p.out_dtype, row0 * ldq + static_cast<size_t>(h) * R + k, acc[kk] * g);
    }
  }
}

// Merge of the nsplit partial results of a (row, head): weights exp(m_s - max m), fixed order.
__global__ void __launch_bounds__(kThreads) latent_attn_merge_kernel(const vila_latent_attn_params p) {
  const int h = blockIdx.y, R = p.R, ns = p.nsplit;
  const int row0 = p.tiles[4 * blockIdx.x];
  const float* part = p.partial + (static_cast<size_t>(row0) * p.H + h) * ns * (R + 2);
  float mx = kNegBig;
  for (int s = 0; s < ns; ++s) mx = fmaxf(mx, part[s * (R + 2) + R]);
  float den = 0.f;
  for (int s = 0; s < ns; ++s) den += expf(part[s * (R + 2) + R] - mx) * part[s * (R + 2) + R + 1];
  float g = 1.0f / den;
  if (p.gate) g *= sigmoid_f(ld_any(p.gate, p.gate_dtype, static_cast<size_t>(row0) * p.ldg + h));
  for (int k = threadIdx.x; k < R; k += kThreads) {
    float a = 0.f;
    for (int s = 0; s < ns; ++s) a += expf(part[s * (R + 2) + R] - mx) * part[s * (R + 2) + k];
    st_any(p.out, p.out_dtype, (static_cast<size_t>(row0) * p.H + h) * R + k, a * g);
  }
}

// Separate keys and values (the un-folded form, for prompt portions that are a large part of their
// context): same thread layout and online softmax as latent_attn_tile_kernel, K rows of width dim for
// the scores, V rows of width vdim for the weighted sum, both contiguous per sequence.
template <int KK4>
__global__ void __launch_bounds__(kThreads) sink_attn_tile_kernel(const vila_sink_attn_params p) {
  extern __shared__ __align__(16) float sm[];
  const int D = p.dim, D4 = round4(D), DS = D4 + 4, V = p.vdim, V4 = round4(V), VS = V4 + 4;
  float* Qs = sm;                  // [BQ][D4]
  float* Ks = Qs + BQ * D4;        // [BKEY][DS]
  float* Vs = Ks + BKEY * DS;      // [BKEY][VS]
  float* Ps = Vs + BKEY * VS;      // [BQ][BKEY]
  const int tid = threadIdx.x, i = tid >> 4, l = tid & 15;
  const int h = blockIdx.y;
  const int* tile = p.tiles + 4 * blockIdx.x;
  const int row0 = tile[0], n = tile[1], pos0 = tile[2];
  const size_t kv0 = static_cast<size_t>(tile[3]);
  for (int idx = tid; idx < BQ * D4; idx += kThreads) {
    const int qi = idx / D4, k = idx % D4;
    Qs[idx] = (qi < n && k < D)
                  ? ld_any(p.q, p.q_dtype, static_cast<size_t>(row0 + qi) * p.ldq + static_cast<size_t>(h) * D + k) * p.scale
                  : 0.f;
  }
  float m = p.sink ? p.sink[h] : kNegBig;
  float lsum = p.sink ? 1.0f : 0.0f;
  float4 acc[KK4];
#pragma unroll
  for (int kk = 0; kk < KK4; ++kk) acc[kk] = make_float4(0.f, 0.f, 0.f, 0.f);
  const int nkeys = pos0 + n;
  const int my_last = pos0 + i;
  for (int j0 = 0; j0 < nkeys; j0 += BKEY) {
    __syncthreads();
    load_rows_block(Ks, DS, D4, p.k, p.kv_dtype, nullptr, 1, kv0, p.ldk, static_cast<size_t>(h) * D, j0, nkeys, D);
    load_rows_block(Vs, VS, V4, p.v, p.kv_dtype, nullptr, 1, kv0, p.ldv, static_cast<size_t>(h) * V, j0, nkeys, V);
    __syncthreads();
    float s0 = 0.f, s1 = 0.f;
    const float4* qr = reinterpret_cast<const float4*>(Qs + i * D4);
    const float4* c0 = reinterpret_cast<const float4*>(Ks + l * DS);
    const float4* c1 = reinterpret_cast<const float4*>(Ks + (l + 16) * DS);
#pragma unroll 4
    for (int k = 0; k < (D4 >> 2); ++k) {
      const float4 qv = qr[k], a = c0[k], b = c1[k];
      s0 = fmaf(qv.x, a.x, s0); s0 = fmaf(qv.y, a.y, s0); s0 = fmaf(qv.z, a.z, s0); s0 = fmaf(qv.w, a.w, s0);
      s1 = fmaf(qv.x, b.x, s1); s1 = fmaf(qv.y, b.y, s1); s1 = fmaf(qv.z, b.z, s1); s1 = fmaf(qv.w, b.w, s1);
    }
    const bool v0 = i < n && j0 + l <= my_last, v1 = i < n && j0 + l + 16 <= my_last;
    s0 = v0 ? s0 : kNegBig;
    s1 = v1 ? s1 : kNegBig;
    float bm = fmaxf(s0, s1);
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, o));
    const float m_new = fmaxf(m, bm);
    const float alpha = expf(m - m_new);
    const float p0 = v0 ? expf(s0 - m_new) : 0.f, p1 = v1 ? expf(s1 - m_new) : 0.f;
    float ps = p0 + p1;
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
    lsum = lsum * alpha + ps;
    m = m_new;
    Ps[i * BKEY + l] = p0;
    Ps[i * BKEY + l + 16] = p1;
    __syncthreads();
    const float* pr = Ps + i * BKEY;
#pragma unroll
    for (int kk = 0; kk < KK4; ++kk) {
      acc[kk].x *= alpha; acc[kk].y *= alpha; acc[kk].z *= alpha; acc[kk].w *= alpha;
    }
#pragma unroll 4
    for (int jj = 0; jj < BKEY; ++jj) {
      const float pj = pr[jj];
      const float* cr = Vs + jj * VS + 4 * l;
#pragma unroll
      for (int kk = 0; kk < KK4; ++kk) {
        if (4 * l + 64 * kk < V4) {
          const float4 c = *reinterpret_cast<const float4*>(cr + 64 * kk);
          acc[kk].x = fmaf(pj, c.x, acc[kk].x); acc[kk].y = fmaf(pj, c.y, acc[kk].y);
          acc[kk].z = fmaf(pj, c.z, acc[kk].z); acc[kk].w = fmaf(pj, c.w, acc[kk].w);
        }
      }
    }
  }
  if (i < n) {
    const size_t row = row0 + i;
    float g = 1.0f / lsum;
    if (p.gate) g *= sigmoid_f(ld_any(p.gate, p.gate_dtype, row * p.ldg + h));
    const size_t ob = row * p.ldo + static_cast<size_t>(h) * V;
#pragma unroll
    for (int kk = 0; kk < KK4; ++kk) {
      const int k = 4 * l + 64 * kk;
      const float v[4] = {acc[kk].x, acc[kk].y, acc[kk].z, acc[kk].w};
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (k + e < V) st_any(p.out, p.out_dtype, ob + k + e, v[e] * g);
    }
  }
}

// One CTA per token.  Warp 0: RMS norm of the first R columns of the token's kv row -> pool row, all warps: the
// rotary part of the kv row -> pool row columns R.., and the rotary part of every query head -> qa columns R..
// of that head.  Angles in double, everything else fp32.
__global__ void __launch_bounds__(kThreads) latent_rope_kernel(const vila_latent_rope_params p) {
  extern __shared__ float cs[];   // cos [rot / 2] | sin [rot / 2]
  const int t = blockIdx.x, tid = threadIdx.x, half = p.rot >> 1, RW = p.R + p.rot;
  const double pos = static_cast<double>(p.positions[t]);
  const float mag = p.mscale != 0.f ? p.mscale : 1.0f;
  for (int i = tid; i < half; i += kThreads) {
    double s, c;
    sincos(pos * p.inv_freq[i], &s, &c);
    cs[i] = static_cast<float>(c) * mag;
    cs[half + i] = static_cast<float>(s) * mag;
  }
  __syncthreads();
  const bool halves = p.layout == 1;
  // rotated value of column c (0 .. rot - 1) of the vector that starts at element `base` of src
  auto turned = [&](const void* src, int dt, size_t base, int c) {
    const int o = halves ? (c < half ? c + half : c - half) : (c ^ 1);
    const int i = halves ? (c < half ? c : c - half) : (c >> 1);
    const bool second = halves ? c >= half : (c & 1) != 0;
    const float v = ld_any(src, dt, base + c), w = ld_any(src, dt, base + o);
    return second ? fmaf(v, cs[i], w * cs[half + i]) : fmaf(v, cs[i], -(w * cs[half + i]));
  };
  if (p.kv != nullptr) {
    const size_t src = static_cast<size_t>(t) * p.ld_kv, dst = static_cast<size_t>(p.cache_rows[t]) * RW;
    if (tid < 32) {
      float ss = 0.f;
      for (int c = tid; c < p.R; c += 32) {
        const float v = ld_any(p.kv, p.kv_dtype, src + c);
        ss = fmaf(v, v, ss);
      }
      ss = warp_sum(ss);
      const float r = 1.0f / sqrtf(ss / static_cast<float>(p.R) + p.eps);
      for (int c = tid; c < p.R; c += 32)
        st_any(p.pool, p.pool_dtype, dst + c, ld_any(p.kv, p.kv_dtype, src + c) * r * (p.norm_w ? p.norm_w[c] : 1.0f));
    }
    for (int c = tid; c < p.rot; c += kThreads) st_any(p.pool, p.pool_dtype, dst + p.R + c, turned(p.kv, p.kv_dtype, src + p.R, c));
  }
  if (p.q != nullptr) {
    for (int idx = tid; idx < p.H * p.rot; idx += kThreads) {
      const int h = idx / p.rot, c = idx - h * p.rot;
      p.qa[(static_cast<size_t>(t) * p.H + h) * RW + p.R + c] =
          turned(p.q, p.q_dtype, static_cast<size_t>(t) * p.ld_q + static_cast<size_t>(h) * p.q_head + p.q_off, c);
    }
  }
}

// dst[i] = src[rows[i]]: one warp per row, 16-byte pieces when everything is 16-byte aligned
__global__ void __launch_bounds__(kThreads) gather_rows_kernel(const unsigned char* __restrict__ src,
                                                               const int32_t* __restrict__ rows,
                                                               unsigned char* __restrict__ dst, int n_rows,
                                                               int row_bytes, int vec) {
  const int r = blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (r >= n_rows) return;
  const unsigned char* s = src + static_cast<size_t>(rows[r]) * row_bytes;
  unsigned char* d = dst + static_cast<size_t>(r) * row_bytes;
  if (vec) {
    for (int b = lane; b < (row_bytes >> 4); b += 32)
      reinterpret_cast<uint4*>(d)[b] = __ldg(reinterpret_cast<const uint4*>(s) + b);
  } else {
    for (int b = lane; b < row_bytes; b += 32) d[b] = s[b];
  }
}

template <typename K>
int set_smem(K kern, size_t bytes) {
  if (bytes > 48 * 1024)
    VB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes)));
  return 0;
}

}  // namespace

int latent_attention(const vila_latent_attn_params& p, cudaStream_t stream) {
  if (p.ntiles <= 0) return 0;
  VB_CHECK(p.R >= 1 && p.R <= 1024, "latent_attention: latent width %d not in [1, 1024]", p.R);
  VB_CHECK(p.H >= 1 && p.H <= 65535 && p.page >= 1 && p.window >= 0, "latent_attention: H=%d page=%d window=%d", p.H,
           p.page, p.window);
  const dim3 grid(p.ntiles, p.H), block(kThreads);
  if (p.decode && p.H >= 4) {
    // decoded tokens, several heads: the heads of a token are the rows of a tile (one latent load for all)
    VB_CHECK(p.nsplit >= 1 && p.nsplit <= 64 && (p.nsplit == 1 || p.partial != nullptr),
             "latent_attention: nsplit=%d needs 1..64 and a partial buffer", p.nsplit);
    const int r4 = round4(p.R);
    const size_t smem = sizeof(float) * (BQ * r4 + BKEY * (r4 + 4) + BQ * BKEY);
    const dim3 hgrid(p.ntiles, (p.H + BQ - 1) / BQ, p.nsplit), block(kThreads);
#define VB_LAT_HEADS(KK)                                                                       \
  do {                                                                                         \
    if (set_smem(latent_attn_tile_kernel<KK, true>, smem)) return 2;                           \
    VB_CUDA(launch_serial(latent_attn_tile_kernel<KK, true>, hgrid, block, smem, stream, p));  \
  } while (0)
    if (p.R <= 64) VB_LAT_HEADS(1);
    else if (p.R <= 128) VB_LAT_HEADS(2);
    else if (p.R <= 256) VB_LAT_HEADS(4);
    else if (p.R <= 512) VB_LAT_HEADS(8);
    else VB_LAT_HEADS(16);
#undef VB_LAT_HEADS
    if (p.nsplit > 1)
      VB_CUDA(launch_serial(latent_attn_merge_kernel, dim3(p.ntiles, p.H), block, 0, stream, p));
    return 0;
  }
  if (p.decode) {
    int rp = 1;
    while (rp < p.R) rp <<= 1;
    const int r4 = round4(p.R);
    const size_t smem = sizeof(float) * (r4 + BKEY * (r4 + 4) + BKEY + 4);
    VB_CHECK(p.nsplit >= 1 && p.nsplit <= 64 && (p.nsplit == 1 || p.partial != nullptr),
             "latent_attention: nsplit=%d needs 1..64 and a partial buffer", p.nsplit);
    const dim3 dgrid(p.ntiles, p.H, p.nsplit);
    if (p.R <= 256) {
      if (set_smem(latent_attn_decode_kernel<1>, smem)) return 2;
      VB_CUDA(launch_serial(latent_attn_decode_kernel<1>, dgrid, block, smem, stream, p, rp));
    } else if (p.R <= 512) {
      if (set_smem(latent_attn_decode_kernel<2>, smem)) return 2;
      VB_CUDA(launch_serial(latent_attn_decode_kernel<2>, dgrid, block, smem, stream, p, rp));
    } else {
      if (set_smem(latent_attn_decode_kernel<4>, smem)) return 2;
      VB_CUDA(launch_serial(latent_attn_decode_kernel<4>, dgrid, block, smem, stream, p, rp));
    }
    if (p.nsplit > 1) VB_CUDA(launch_serial(latent_attn_merge_kernel, grid, block, 0, stream, p));
    return 0;
  }
  const int r4 = round4(p.R);
  const size_t smem = sizeof(float) * (BQ * r4 + BKEY * (r4 + 4) + BQ * BKEY);
#define VB_LAT_TILE(KK)                                                                    \
  do {                                                                                     \
    if (set_smem(latent_attn_tile_kernel<KK, false>, smem)) return 2;                      \
    VB_CUDA(launch_serial(latent_attn_tile_kernel<KK, false>, grid, block, smem, stream, p)); \
  } while (0)
  if (p.R <= 64) VB_LAT_TILE(1);
  else if (p.R <= 128) VB_LAT_TILE(2);
  else if (p.R <= 256) VB_LAT_TILE(4);
  else if (p.R <= 512) VB_LAT_TILE(8);
  else VB_LAT_TILE(16);
#undef VB_LAT_TILE
  return 0;
}

int latent_rope_append(const vila_latent_rope_params& p, cudaStream_t stream) {
  if (p.T <= 0) return 0;
  VB_CHECK(p.R >= 1 && p.rot >= 0 && p.rot % 2 == 0 && (p.rot == 0 || p.inv_freq != nullptr) && p.positions != nullptr &&
               (p.layout == 0 || p.layout == 1),
           "latent_rope_append: R=%d rot=%d layout=%d", p.R, p.rot, p.layout);
  VB_CHECK(p.kv == nullptr || (p.pool != nullptr && p.cache_rows != nullptr), "latent_rope_append: kv rows need a pool");
  VB_CHECK(p.q == nullptr || (p.qa != nullptr && p.H >= 1 && p.q_off >= 0 && p.q_off + p.rot <= p.q_head),
           "latent_rope_append: H=%d q_head=%d q_off=%d rot=%d", p.H, p.q_head, p.q_off, p.rot);
  VB_CUDA(launch_serial(latent_rope_kernel, dim3(p.T), dim3(kThreads), sizeof(float) * (p.rot + 2), stream, p));
  return 0;
}

int sink_attention(const vila_sink_attn_params& p, cudaStream_t stream) {
  if (p.ntiles <= 0) return 0;
  VB_CHECK(p.dim >= 1 && p.dim <= 512 && p.vdim >= 1 && p.vdim <= 512 && p.H >= 1 && p.H <= 65535,
           "sink_attention: H=%d dim=%d vdim=%d (dims <= 512)", p.H, p.dim, p.vdim);
  const int d4 = round4(p.dim), v4 = round4(p.vdim);
  const size_t smem = sizeof(float) * (BQ * d4 + BKEY * (d4 + 4) + BKEY * (v4 + 4) + BQ * BKEY);
  const dim3 grid(p.ntiles, p.H), block(kThreads);
#define VB_SINK_TILE(KK)                                                                 \
  do {                                                                                   \
    if (set_smem(sink_attn_tile_kernel<KK>, smem)) return 2;                             \
    VB_CUDA(launch_serial(sink_attn_tile_kernel<KK>, grid, block, smem, stream, p));     \
  } while (0)
  if (p.vdim <= 64) VB_SINK_TILE(1);
  else if (p.vdim <= 128) VB_SINK_TILE(2);
  else if (p.vdim <= 256) VB_SINK_TILE(4);
  else VB_SINK_TILE(8);
#undef VB_SINK_TILE
  return 0;
}

int gather_rows(const void* src, const int32_t* rows, void* dst, int n_rows, int row_bytes, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  VB_CHECK(row_bytes > 0, "gather_rows: row_bytes=%d", row_bytes);
  const int vec = row_bytes % 16 == 0 && reinterpret_cast<uintptr_t>(src) % 16 == 0 &&
                  reinterpret_cast<uintptr_t>(dst) % 16 == 0;
  VB_CUDA(launch_serial(gather_rows_kernel, dim3((n_rows + 7) / 8), dim3(kThreads), 0, stream,
                        static_cast<const unsigned char*>(src), rows, static_cast<unsigned char*>(dst), n_rows,
                        row_bytes, vec));
  return 0;
}

}  // namespace vb
