// vila_glinear: any-shape (grouped) linear layer on the CUDA cores, fp32 accumulation.
// It serves (a) every linear layer of the true-fp32 path, (b) shapes the tcgen05 GEMM does not
// take (N or K not a multiple of 8), (c) per-head batched projections (latent attention: the key /
// value expansions folded into queries and outputs) and (d) routed experts, where the rows of a
// group are a segment of a sorted (token, choice) list read through an index and written back
// through an index with the routing weight applied.
// Tile: BM x 64 x 16 with 256 threads, each thread a (BM/16) x 4 block of outputs.  The summation
// order over K is fixed and the same for every row, wherever the row sits in a tile or a batch.
#include "../../include/vila_b200.h"
#include "common.cuh"
#include "kernels.h"
#include "dtype_any.cuh"

#include <mma.h>

namespace vb {
namespace {

constexpr int BN = 64, BK = 16, kThreads = 256;

// clamped gated unit: g = min(zg, limit), u = clamp(zu, +-limit), g * sigmoid(alpha * g) * (u + 1)
__device__ __forceinline__ float glu_clamp_f(float zg, float zu, const vila_glinear_ext& x) {
  const float g = fminf(zg, x.act_limit), u = fminf(fmaxf(zu, -x.act_limit), x.act_limit);
  return g * sigmoid_f(x.act_alpha * g) * (u + 1.0f);
}

// scale of the INPUT row behind sorted position i (= output row: in_scale is only taken without o_rows)
__device__ __forceinline__ float in_scale_of(const vila_glinear_params& p, const vila_glinear_ext& x, int i) {
  return x.in_scale ? x.in_scale[p.a_rows ? p.a_rows[i] : i] : 1.0f;
}

// Epilogue of a thread's TM x 4 block: bias, activation (or SwiGLU over column pairs), routing weight,
// scatter through the output row index.
template <int TM>
__device__ __forceinline__ void store_block(const vila_glinear_params& p, const vila_glinear_ext& x, int g, int n0,
                                            int tx, const int* orows, float (&acc)[TM][4]) {
  const size_t o_col0 = p.mode == 0 ? static_cast<size_t>(g) * p.o_group_off : 0;
  const bool swiglu = (p.flags & VILA_FLAG_SWIGLU) != 0;
  const bool glu_clamp = (p.flags & VILA_FLAG_GLU_CLAMP) != 0;
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int orow = orows[i];
    if (orow < 0) continue;
    const float rs = p.row_scale ? p.row_scale[orow] : 1.0f;
    const float is = in_scale_of(p, x, orow);
    float v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      float z = acc[i][j] * is;
      if (p.bias && n < p.N) z += ld_any(p.bias, p.w_dtype, static_cast<size_t>(g) * p.bias_group_stride + n);
      if (p.act == VILA_ACT_SILU) z = silu_exact_f(z);
      else if (p.act == VILA_ACT_RELU2) { z = fmaxf(z, 0.f); z = z * z; }
      else if (p.act == VILA_ACT_GELU_TANH) {
        z = 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
      } else if (p.act == VILA_ACT_XIELU) z = xielu_f(z, x.act_pos, x.act_neg);
      v[j] = z;
    }
    const size_t ob = static_cast<size_t>(orow) * p.ldo + o_col0;
    if (glu_clamp) {
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int n = n0 + tx * 4 + 2 * j;
        if (n + 1 < p.N) st_any(p.out, p.out_dtype, ob + n / 2, glu_clamp_f(v[2 * j], v[2 * j + 1], x) * rs);
      }
    } else if (swiglu) {
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int n = n0 + tx * 4 + 2 * j;
        if (n + 1 < p.N) st_any(p.out, p.out_dtype, ob + n / 2, silu_exact_f(v[2 * j]) * v[2 * j + 1] * rs);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int n = n0 + tx * 4 + j;
        if (n < p.N) st_any(p.out, p.out_dtype, ob + n, v[j] * rs);
      }
    }
  }
}

// Which rows does this CTA own?  mode 0: tile blockIdx.y of group blockIdx.z; mode 1: blockIdx.y counts
// the BM-row tiles of all groups in order.  Fills the A-row / output-row tables; false: no work.
template <int BM>
__device__ __forceinline__ bool tile_rows(const vila_glinear_params& p, int* arow_s, int* orow_s, int* grp_s,
                                          int& g) {
  const int tid = threadIdx.x;
  int m0, m_end;
  if (p.mode == 0) {
    g = blockIdx.z;
    m0 = blockIdx.y * BM;
    m_end = p.M;
  } else {
    if (tid == 0) {
      int t = blockIdx.y, found = -1, start = 0;
      for (int e = 0; e < p.groups; ++e) {
        const int b = p.seg[e], n = p.seg[e + 1] - b, nt = (n + BM - 1) / BM;
        if (t < nt) { found = e; start = b + t * BM; break; }
        t -= nt;
      }
      grp_s[0] = found;
      grp_s[1] = start;
    }
    __syncthreads();
    g = grp_s[0];
    if (g < 0) return false;
    m0 = grp_s[1];
    m_end = p.seg[g + 1];
  }
  for (int m = tid; m < BM; m += blockDim.x) {
    const int i = m0 + m;
    int ar = -1, orow = -1;
    if (i < m_end) {
      ar = p.a_rows ? p.a_rows[i] / p.a_row_div : i;
      orow = p.o_rows ? p.o_rows[i] : i;
    }
    arow_s[m] = ar;
    orow_s[m] = orow;
  }
  __syncthreads();
  return true;
}

template <int BM>
__global__ void __launch_bounds__(kThreads) glinear_kernel(const vila_glinear_params p, const vila_glinear_ext x) {
  constexpr int TM = BM / 16;
  __shared__ float As[BK][BM + 1];
  __shared__ __align__(16) float Ws[BK][BN];
  __shared__ int arow_s[BM], orow_s[BM];
  __shared__ int grp_s[2];
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  int g;
  if (!tile_rows<BM>(p, arow_s, orow_s, grp_s, g)) return;
  const int n0 = blockIdx.x * BN;
  const size_t a_col0 = p.mode == 0 ? static_cast<size_t>(g) * p.a_group_off : 0;
  const size_t w_base = static_cast<size_t>(g) * p.w_group_stride;

  float acc[TM][4];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < p.K; k0 += BK) {
    for (int idx = tid; idx < BM * BK; idx += kThreads) {
      const int m = idx / BK, k = idx % BK;
      const int ar = arow_s[m];
      float v = 0.f;
      if (ar >= 0 && k0 + k < p.K) v = ld_any(p.a, p.a_dtype, static_cast<size_t>(ar) * p.lda + a_col0 + k0 + k);
      As[k][m] = v;
    }
    for (int idx = tid; idx < BN * BK; idx += kThreads) {
      const int n = idx / BK, k = idx % BK;
      float v = 0.f;
      if (n0 + n < p.N && k0 + k < p.K)
        v = ld_any(p.w, p.w_dtype, w_base + static_cast<size_t>(n0 + n) * p.ldw + k0 + k);
      Ws[k][n] = v;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      const float4 wv = *reinterpret_cast<const float4*>(&Ws[k][tx * 4]);
#pragma unroll
      for (int i = 0; i < TM; ++i) {
        const float a = As[k][ty * TM + i];
        acc[i][0] = fmaf(a, wv.x, acc[i][0]);
        acc[i][1] = fmaf(a, wv.y, acc[i][1]);
        acc[i][2] = fmaf(a, wv.z, acc[i][2]);
        acc[i][3] = fmaf(a, wv.w, acc[i][3]);
      }
    }
    __syncthreads();
  }

  store_block<TM>(p, x, g, n0, tx, orow_s + ty * TM, acc);
}

// ---- bf16 operands, many rows: warp-level tensor-core tiles (wmma, fp32 accumulators) ---------------
// Same tiling as glinear_kernel<64> (64 x 64 outputs per CTA, groups, row gather / scatter,
// epilogues); 8 warps as 4 x 2, each 16 x 32 outputs; K in steps of 32 through shared memory.  The
// accumulators go through shared memory once so that the epilogue is the shared one.
constexpr int WK = 32, WLD = WK + 8;

__device__ __forceinline__ uint4 load8_bf16(const __nv_bfloat16* base, size_t off, int k, int K, bool row_ok,
                                            bool vec) {
  uint4 v = make_uint4(0u, 0u, 0u, 0u);
  if (!row_ok || k >= K) return v;
  if (vec) return __ldg(reinterpret_cast<const uint4*>(base + off + k));
  __nv_bfloat16 t[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) t[e] = k + e < K ? base[off + k + e] : __float2bfloat16_rn(0.f);
  return *reinterpret_cast<uint4*>(t);
}

__global__ void __launch_bounds__(kThreads) glinear_wmma_kernel(const vila_glinear_params p, const vila_glinear_ext x, int vec) {
  using namespace nvcuda;
  constexpr int BM = 64;
  __shared__ __align__(32) __nv_bfloat16 As[BM][WLD];
  __shared__ __align__(32) __nv_bfloat16 Ws[BN][WLD];
  __shared__ __align__(32) float Cs[BM][BN + 4];
  __shared__ int arow_s[BM], orow_s[BM];
  __shared__ int grp_s[2];
  const int tid = threadIdx.x, warp = tid >> 5;
  int g;
  if (!tile_rows<BM>(p, arow_s, orow_s, grp_s, g)) return;
  const int n0 = blockIdx.x * BN;
  const size_t a_col0 = p.mode == 0 ? static_cast<size_t>(g) * p.a_group_off : 0;
  const size_t w_base = static_cast<size_t>(g) * p.w_group_stride;
  const __nv_bfloat16* A = static_cast<const __nv_bfloat16*>(p.a);
  const __nv_bfloat16* W = static_cast<const __nv_bfloat16*>(p.w);
  const int wm = warp & 3, wn = warp >> 2;
  wmma::fragment<wmma::accumulator, 16, 16, 16, float> c[2];
  wmma::fill_fragment(c[0], 0.f);
  wmma::fill_fragment(c[1], 0.f);
  const int lr = tid >> 2, lk = (tid & 3) * 8;   // this thread stages 8 elements of row lr
  const int ar = arow_s[lr];
  const bool w_ok = n0 + lr < p.N;
  const size_t a_off = static_cast<size_t>(ar < 0 ? 0 : ar) * p.lda + a_col0;
  const size_t w_off = w_base + static_cast<size_t>(n0 + lr) * p.ldw;
  for (int k0 = 0; k0 < p.K; k0 += WK) {
    *reinterpret_cast<uint4*>(&As[lr][lk]) = load8_bf16(A, a_off, k0 + lk, p.K, ar >= 0, vec);
    *reinterpret_cast<uint4*>(&Ws[lr][lk]) = load8_bf16(W, w_off, k0 + lk, p.K, w_ok, vec);
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < WK; kk += 16) {
      wmma::fragment<wmma::matrix_a, 16, 16, 16, __nv_bfloat16, wmma::row_major> fa;
      wmma::load_matrix_sync(fa, &As[wm * 16][kk], WLD);
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        wmma::fragment<wmma::matrix_b, 16, 16, 16, __nv_bfloat16, wmma::col_major> fb;
        wmma::load_matrix_sync(fb, &Ws[wn * 32 + j * 16][kk], WLD);
        wmma::mma_sync(c[j], fa, fb, c[j]);
      }
    }
    __syncthreads();
  }
  wmma::store_matrix_sync(&Cs[wm * 16][wn * 32], c[0], BN + 4, wmma::mem_row_major);
  wmma::store_matrix_sync(&Cs[wm * 16][wn * 32 + 16], c[1], BN + 4, wmma::mem_row_major);
  __syncthreads();
  const int tx = tid & 15, ty = tid >> 4;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = Cs[ty * 4 + i][tx * 4 + j];
  store_block<4>(p, x, g, n0, tx, orow_s + ty * 4, acc);
}

// ---- few rows per group (decoded tokens): weight-streaming kernel ---------------------------------
// One warp per PAIR of output columns; the lanes split K in 8-element pieces (16-byte loads of bf16
// weights, 32-byte of fp32), every weight byte is read once per pass, the rows of A
// come from L1 / L2 (a pass covers up to 8 rows; more rows of a group mean more passes).  Serves the routed experts, the per-head folded projections and the output head
// of decode steps, all of which are bound by the weight stream.
constexpr int kSmallRows = 8, kSmallWarps = 8;   // rows per pass over the weights

__device__ __forceinline__ void load8(const void* p, int dt, size_t i, float (&v)[8]) {
  if (dt) {
    const float4 a = __ldg(reinterpret_cast<const float4*>(static_cast<const float*>(p) + i));
    const float4 b = __ldg(reinterpret_cast<const float4*>(static_cast<const float*>(p) + i + 4));
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  } else {
    const uint4 u = __ldg(reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(p) + i));
    v[0] = __uint_as_float(u.x << 16); v[1] = __uint_as_float(u.x & 0xffff0000u);
    v[2] = __uint_as_float(u.y << 16); v[3] = __uint_as_float(u.y & 0xffff0000u);
    v[4] = __uint_as_float(u.z << 16); v[5] = __uint_as_float(u.z & 0xffff0000u);
    v[6] = __uint_as_float(u.w << 16); v[7] = __uint_as_float(u.w & 0xffff0000u);
  }
}

__device__ __forceinline__ float finish(const vila_glinear_params& p, const vila_glinear_ext& x, float z, int g, int n) {
  if (p.bias) z += ld_any(p.bias, p.w_dtype, static_cast<size_t>(g) * p.bias_group_stride + n);
  if (p.act == VILA_ACT_SILU) z = silu_exact_f(z);
  else if (p.act == VILA_ACT_RELU2) { z = fmaxf(z, 0.f); z = z * z; }
  else if (p.act == VILA_ACT_GELU_TANH)
    z = 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
  else if (p.act == VILA_ACT_XIELU) z = xielu_f(z, x.act_pos, x.act_neg);
  return z;
}

// vec: K % 8 == 0 and every row of A and W starts on an 8-element boundary (16 B bf16, 32 B fp32)
__global__ void __launch_bounds__(kSmallWarps * 32) glinear_small_kernel(const vila_glinear_params p, const vila_glinear_ext x, int vec) {
  __shared__ int arow_s[kSmallRows], orow_s[kSmallRows];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = blockIdx.y;
  const int n_a = (blockIdx.x * kSmallWarps + warp) * 2, n_b = n_a + 1;
  const int m_begin = p.mode == 0 ? 0 : p.seg[g], m_end = p.mode == 0 ? p.M : p.seg[g + 1];
  const size_t a_col0 = p.mode == 0 ? static_cast<size_t>(g) * p.a_group_off : 0;
  const size_t o_col0 = p.mode == 0 ? static_cast<size_t>(g) * p.o_group_off : 0;
  const size_t wa = static_cast<size_t>(g) * p.w_group_stride + static_cast<size_t>(n_a) * p.ldw;
  const size_t wb = wa + p.ldw;
  const bool has_a = n_a < p.N, has_b = n_b < p.N;
  const bool swiglu = (p.flags & VILA_FLAG_SWIGLU) != 0;
  const bool glu_clamp = (p.flags & VILA_FLAG_GLU_CLAMP) != 0;
  for (int m0 = m_begin; m0 < m_end; m0 += kSmallRows) {
    const int nr = min(kSmallRows, m_end - m0);
    __syncthreads();
    if (threadIdx.x < kSmallRows) {
      const int i = m0 + threadIdx.x;
      const bool ok = threadIdx.x < nr;
      arow_s[threadIdx.x] = ok ? (p.a_rows ? p.a_rows[i] / p.a_row_div : i) : 0;
      orow_s[threadIdx.x] = ok ? (p.o_rows ? p.o_rows[i] : i) : -1;
    }
    __syncthreads();
    float acc_a[kSmallRows], acc_b[kSmallRows];
#pragma unroll
    for (int r = 0; r < kSmallRows; ++r) acc_a[r] = acc_b[r] = 0.f;
    if (has_a) {
      if (vec) {
#pragma unroll 2
        for (int k = lane * 8; k < p.K; k += 256) {
          float w0[8], w1[8], a[8];
          load8(p.w, p.w_dtype, wa + k, w0);
          if (has_b) load8(p.w, p.w_dtype, wb + k, w1);
          else {
#pragma unroll
            for (int e = 0; e < 8; ++e) w1[e] = 0.f;
          }
#pragma unroll
          for (int r = 0; r < kSmallRows; ++r) {
            if (r < nr) {
              load8(p.a, p.a_dtype, static_cast<size_t>(arow_s[r]) * p.lda + a_col0 + k, a);
#pragma unroll
              for (int e = 0; e < 8; ++e) {
                acc_a[r] = fmaf(a[e], w0[e], acc_a[r]);
                acc_b[r] = fmaf(a[e], w1[e], acc_b[r]);
              }
            }
          }
        }
      } else {
        for (int k = lane; k < p.K; k += 32) {
          const float w0 = ld_any(p.w, p.w_dtype, wa + k);
          const float w1 = has_b ? ld_any(p.w, p.w_dtype, wb + k) : 0.f;
#pragma unroll
          for (int r = 0; r < kSmallRows; ++r) {
            if (r < nr) {
              const float a = ld_any(p.a, p.a_dtype, static_cast<size_t>(arow_s[r]) * p.lda + a_col0 + k);
              acc_a[r] = fmaf(a, w0, acc_a[r]);
              acc_b[r] = fmaf(a, w1, acc_b[r]);
            }
          }
        }
      }
    }
#pragma unroll
    for (int r = 0; r < kSmallRows; ++r) {
      if (r < nr) {   // nr is uniform over the CTA
        const int orow = orow_s[r];
        const float is = in_scale_of(p, x, orow);
        const float za = warp_sum(acc_a[r]) * is, zb = warp_sum(acc_b[r]) * is;
        if (lane == 0 && has_a) {
          const float rs = p.row_scale ? p.row_scale[orow] : 1.0f;
          const size_t ob = static_cast<size_t>(orow) * p.ldo + o_col0;
          if (glu_clamp) {
            if (has_b) st_any(p.out, p.out_dtype, ob + n_a / 2, glu_clamp_f(finish(p, x, za, g, n_a), finish(p, x, zb, g, n_b), x) * rs);
          } else if (swiglu) {
            if (has_b) st_any(p.out, p.out_dtype, ob + n_a / 2, silu_exact_f(finish(p, x, za, g, n_a)) * finish(p, x, zb, g, n_b) * rs);
          } else {
            st_any(p.out, p.out_dtype, ob + n_a, finish(p, x, za, g, n_a) * rs);
            if (has_b) st_any(p.out, p.out_dtype, ob + n_b, finish(p, x, zb, g, n_b) * rs);
          }
        }
      }
    }
  }
}

}  // namespace

int glinear(const vila_glinear_params& p, cudaStream_t stream, const vila_glinear_ext* ext) {
  vila_glinear_ext x = {1.0f, INFINITY, 0.f, 0.f, nullptr};
  if (ext) x = *ext;
  VB_CHECK(x.in_scale == nullptr || p.o_rows == nullptr, "glinear: in_scale is indexed through a_rows; o_rows must be NULL");
  if (p.M <= 0 || p.N <= 0) return 0;
  VB_CHECK(p.K > 0 && p.groups >= 1, "glinear: K=%d groups=%d", p.K, p.groups);
  VB_CHECK(p.mode == 0 || (p.mode == 1 && p.seg != nullptr), "glinear: mode %d needs seg", p.mode);
  VB_CHECK(!(p.flags & (VILA_FLAG_SWIGLU | VILA_FLAG_GLU_CLAMP)) || (p.N % 2 == 0 && p.act == VILA_ACT_NONE),
           "glinear: the SwiGLU epilogue needs an even N and no other activation");
  VB_CHECK(p.a_rows == nullptr || p.a_row_div >= 1, "glinear: a_row_div=%d", p.a_row_div);
  const bool small = p.M <= 16;
  // few rows: stream the weights once per 16-row chunk instead of tiling
  if ((p.mode == 0 && p.M <= 2 * kSmallRows) || (p.mode == 1 && p.M <= 8 * kSmallRows)) {
    const size_t ea = p.a_dtype ? 4 : 2, ew = p.w_dtype ? 4 : 2;
    const bool vec = p.K % 8 == 0 && p.lda % 8 == 0 && p.ldw % 8 == 0 && p.w_group_stride % 8 == 0 &&
                     p.a_group_off % 8 == 0 && reinterpret_cast<uintptr_t>(p.a) % (8 * ea) == 0 &&
                     reinterpret_cast<uintptr_t>(p.w) % (8 * ew) == 0;
    const dim3 grid((p.N + 2 * kSmallWarps - 1) / (2 * kSmallWarps), p.groups);
    VB_CHECK(grid.y <= 65535, "glinear: too many groups (%d)", p.groups);
    VB_CUDA(launch_serial(glinear_small_kernel, grid, dim3(kSmallWarps * 32), 0, stream, p, x, vec ? 1 : 0));
    return 0;
  }
  const int bm = small ? 16 : 64;
  dim3 grid((p.N + BN - 1) / BN, 1, 1);
  if (p.mode == 0) {
    grid.y = (p.M + bm - 1) / bm;
    grid.z = p.groups;
  } else {
    grid.y = (p.M + bm - 1) / bm + p.groups;  // upper bound of sum_g ceil(rows_g / bm)
  }
  VB_CHECK(grid.y <= 65535 && grid.z <= 65535, "glinear: too many tiles (M=%d groups=%d)", p.M, p.groups);
  if (!small && p.a_dtype == VILA_DT_BF16 && p.w_dtype == VILA_DT_BF16) {
    // bf16 operands: tensor-core tiles.  16-byte loads need every row of A and W to start on an
    // 8-element boundary; otherwise the same kernel stages element by element.
    const bool vec = p.K % 8 == 0 && p.lda % 8 == 0 && p.ldw % 8 == 0 && p.w_group_stride % 8 == 0 &&
                     p.a_group_off % 8 == 0 && reinterpret_cast<uintptr_t>(p.a) % 16 == 0 &&
                     reinterpret_cast<uintptr_t>(p.w) % 16 == 0;
    VB_CUDA(launch_serial(glinear_wmma_kernel, grid, dim3(kThreads), 0, stream, p, x, vec ? 1 : 0));
    return 0;
  }
  if (small) VB_CUDA(launch_serial(glinear_kernel<16>, grid, dim3(kThreads), 0, stream, p, x));
  else VB_CUDA(launch_serial(glinear_kernel<64>, grid, dim3(kThreads), 0, stream, p, x));
  return 0;
}

}  // namespace vb
