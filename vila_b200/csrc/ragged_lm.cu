// Row-wise building blocks of ragged-batch language-model steps with an fp32 residual stream:
// embedding gather, RMS norm (plain or zero-centred weights, optional scatter into a paged pool),
// the gated + normed residual update, and the router / grouping kernels of routed experts.
// All arithmetic is fp32; tensors are read and written in the dtype their code names.
// These kernels (and the other ragged-batch kernels: glinear, latent_attn, hgrn2) are launched
// stream-serialised (launch_serial), not with programmatic dependent launch: overlapping them with the
// persistent GEMMs deadlocked in one measured configuration, so they neither start early nor release
// their successor early.
#include "../../include/vila_b200.h"
#include "common.cuh"
#include "kernels.h"
#include "dtype_any.cuh"

namespace vb {
namespace {

constexpr int kRowThreads = 256;
constexpr int kRowsPerCta = kRowThreads / 32;
constexpr int kWideCols = 512;  // rows at least this wide get a whole CTA, narrower ones a warp

// TPR threads share a row: 32 = one warp (8 rows per CTA), 256 = the whole CTA.
template <int TPR>
__device__ __forceinline__ float row_sum(float v, float* red) {
  v = warp_sum(v);
  if (TPR == 32) return v;
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = l < kRowsPerCta ? red[l] : 0.f;
  return warp_sum(t);
}
template <int TPR>
__device__ __forceinline__ int row_of() {
  return TPR == 32 ? blockIdx.x * kRowsPerCta + (threadIdx.x >> 5) : blockIdx.x;
}
template <int TPR>
__device__ __forceinline__ int col0_of() { return TPR == 32 ? (threadIdx.x & 31) : threadIdx.x; }

__global__ void __launch_bounds__(kRowThreads)
embed_rows_kernel(const void* __restrict__ table, int dt, const int32_t* __restrict__ ids,
                  float* __restrict__ out, int rows, int cols) {
  const int row = blockIdx.x * kRowsPerCta + (threadIdx.x >> 5);
  if (row >= rows) return;
  const size_t src = static_cast<size_t>(ids[row]) * cols;
  float* o = out + static_cast<size_t>(row) * cols;
  for (int c = lane_id(); c < cols; c += 32) o[c] = ld_any(table, dt, src + c);
}

template <int TPR>
__global__ void __launch_bounds__(kRowThreads)
rmsnorm_rows_kernel(const void* __restrict__ x, int x_dt, int64_t ldx, const void* __restrict__ w,
                    int w_dt, float w_off, float eps, void* __restrict__ out, int o_dt, int64_t ldo,
                    const int32_t* __restrict__ out_rows, int rows, int cols, int groups) {
  // groups > 1: `rows` counts (row, piece) pairs, `cols` is the width of a piece; piece g of row r
  // starts at column g * cols and uses the weights [g * cols, (g + 1) * cols)
  __shared__ float red[kRowsPerCta];
  const int vrow = row_of<TPR>();
  if (vrow >= rows) return;   // TPR == 256: uniform over the CTA
  const int row = vrow / groups, piece = vrow - row * groups;
  const size_t xb = static_cast<size_t>(row) * ldx + static_cast<size_t>(piece) * cols;
  if (w) w = static_cast<const char*>(w) + static_cast<size_t>(piece) * cols * (w_dt ? 4 : 2);
  float ss = 0.f;
  for (int c = col0_of<TPR>(); c < cols; c += TPR) {
    const float v = ld_any(x, x_dt, xb + c);
    ss += v * v;
  }
  ss = row_sum<TPR>(ss, red);
  const float r = 1.0f / sqrtf(ss / static_cast<float>(cols) + eps);
  const size_t ob = static_cast<size_t>(out_rows ? out_rows[row] : row) * ldo + static_cast<size_t>(piece) * cols;
  for (int c = col0_of<TPR>(); c < cols; c += TPR) {
    const float g = w ? ld_any(w, w_dt, c) + w_off : 1.0f;
    st_any(out, o_dt, ob + c, ld_any(x, x_dt, xb + c) * r * g);
  }
}

// Pre-norm residual step in one pass: x += a + sum_j part_j (a first, then the partials by index), then
// out = x / sqrt(mean(x^2) + eps) * w: the operand of the sublayer that reads x next.
template <int TPR>
__global__ void __launch_bounds__(kRowThreads)
residual_norm_rows_kernel(float* __restrict__ x, const void* __restrict__ a, int a_dt, int64_t lda,
                          const void* __restrict__ part, int p_dt, int64_t ldp, int np, const void* __restrict__ w,
                          int w_dt, float eps, void* __restrict__ out, int o_dt, int rows, int cols) {
  __shared__ float red[kRowsPerCta];
  const int row = row_of<TPR>();
  if (row >= rows) return;
  float* xr = x + static_cast<size_t>(row) * cols;
  float ss = 0.f;
  for (int c = col0_of<TPR>(); c < cols; c += TPR) {
    float y = a ? ld_any(a, a_dt, static_cast<size_t>(row) * lda + c) : 0.f;
    if (part)
      for (int j = 0; j < np; ++j) y += ld_any(part, p_dt, (static_cast<size_t>(row) * np + j) * ldp + c);
    const float v = xr[c] + y;
    xr[c] = v;
    ss += v * v;
  }
  ss = row_sum<TPR>(ss, red);
  const float r = 1.0f / sqrtf(ss / static_cast<float>(cols) + eps);
  for (int c = col0_of<TPR>(); c < cols; c += TPR)   // every thread re-reads the columns it wrote itself
    st_any(out, o_dt, static_cast<size_t>(row) * cols + c, xr[c] * r * (w ? ld_any(w, w_dt, c) : 1.0f));
}

__device__ __forceinline__ float gated_value(const void* part, int p_dt, int64_t ldp, int np,
                                             const void* gate, int g_dt, int64_t ldg,
                                             const void* gb, int b_dt, int row, int c) {
  float y = 0.f;
  for (int j = 0; j < np; ++j)
    y += ld_any(part, p_dt, (static_cast<size_t>(row) * np + j) * ldp + c);
  if (gate) {
    float z = ld_any(gate, g_dt, static_cast<size_t>(row) * ldg + c);
    if (gb) z += ld_any(gb, b_dt, c);
    y *= sigmoid_f(z);
  }
  return y;
}

template <int TPR>
__global__ void __launch_bounds__(kRowThreads)
gated_norm_residual_kernel(float* __restrict__ x, const void* __restrict__ part, int p_dt, int64_t ldp,
                           int np, const void* __restrict__ gate, int g_dt, int64_t ldg,
                           const void* __restrict__ gb, int b_dt, const void* __restrict__ w, int w_dt,
                           float w_off, float eps, float mult, int rows, int cols) {
  __shared__ float red[kRowsPerCta];
  const int row = row_of<TPR>();
  if (row >= rows) return;
  float ss = 0.f;
  for (int c = col0_of<TPR>(); c < cols; c += TPR) {
    const float y = gated_value(part, p_dt, ldp, np, gate, g_dt, ldg, gb, b_dt, row, c);
    ss += y * y;
  }
  ss = row_sum<TPR>(ss, red);
  const float r = 1.0f / sqrtf(ss / static_cast<float>(cols) + eps);
  float* xr = x + static_cast<size_t>(row) * cols;
  for (int c = col0_of<TPR>(); c < cols; c += TPR) {
    const float y = gated_value(part, p_dt, ldp, np, gate, g_dt, ldg, gb, b_dt, row, c);
    const float g = w ? ld_any(w, w_dt, c) + w_off : 1.0f;
    xr[c] += mult * (y * r * g);
  }
}

// ---- routed experts ------------------------------------------------------------------------------
// E logits per token (fp32 dot products over the row), then `top` rounds of arg-max.  TPR == 32: one
// warp per token; TPR == 256 (few tokens): the 8 warps of a CTA split the experts of ONE token.
template <int TPR>
__global__ void __launch_bounds__(kRowThreads)
moe_route_kernel(const void* __restrict__ x, int x_dt, int64_t ldx, const float* __restrict__ wr,
                 const float* __restrict__ bias, int32_t* __restrict__ idx, float* __restrict__ weight,
                 int rows, int cols, int experts, int top) {
  extern __shared__ float z_s[];  // TPR == 32: [kRowsPerCta][experts]; 256: [experts]
  const int wid = threadIdx.x >> 5, lane = lane_id();
  const int row = row_of<TPR>();
  if (row >= rows) return;
  float* z = TPR == 32 ? z_s + wid * experts : z_s;
  const size_t xb = static_cast<size_t>(row) * ldx;
  for (int e = (TPR == 32 ? 0 : wid); e < experts; e += (TPR == 32 ? 1 : kRowsPerCta)) {
    const float* we = wr + static_cast<size_t>(e) * cols;
    float s = 0.f;
    for (int c = lane; c < cols; c += 32) s += ld_any(x, x_dt, xb + c) * we[c];
    s = warp_sum(s);
    if (lane == 0) z[e] = s + (bias ? bias[e] : 0.f);
  }
  if (TPR == 32) __syncwarp();
  else {
    __syncthreads();
    if (wid != 0) return;
  }
  float first = 0.f, denom = 0.f;
  for (int j = 0; j < top; ++j) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int e = lane; e < experts; e += 32) {
      const float v = z[e];
      if (v > best) { best = v; bi = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (j == 0) first = best;
    const float e_j = expf(best - first);
    denom += e_j;
    if (lane == 0) {
      idx[static_cast<size_t>(row) * top + j] = bi;
      weight[static_cast<size_t>(row) * top + j] = e_j;
      z[bi] = -INFINITY;
    }
    __syncwarp();
  }
  if (lane == 0)
    for (int j = 0; j < top; ++j) weight[static_cast<size_t>(row) * top + j] /= denom;
}

// Single CTA: per-expert counts, exclusive prefix, then a stable placement (pair ids stay ascending
// inside every expert's segment) with warp ballots.
__global__ void __launch_bounds__(1024)
moe_group_kernel(const int32_t* __restrict__ idx, int32_t* __restrict__ seg, int32_t* __restrict__ sorted,
                 int pairs, int experts) {
  extern __shared__ int cnt_s[];  // [experts + 1]
  const int wid = threadIdx.x >> 5, lane = lane_id(), nw = blockDim.x >> 5;
  for (int e = wid; e < experts; e += nw) {
    int n = 0;
    for (int p0 = 0; p0 < pairs; p0 += 32) {
      const int p = p0 + lane;
      n += __popc(__ballot_sync(0xffffffffu, p < pairs && idx[p] == e));
    }
    if (lane == 0) cnt_s[e + 1] = n;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    cnt_s[0] = 0;
    for (int e = 0; e < experts; ++e) cnt_s[e + 1] += cnt_s[e];
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= experts; e += blockDim.x) seg[e] = cnt_s[e];
  for (int e = wid; e < experts; e += nw) {
    int at = cnt_s[e];
    for (int p0 = 0; p0 < pairs; p0 += 32) {
      const int p = p0 + lane;
      const bool mine = p < pairs && idx[p] == e;
      const unsigned m = __ballot_sync(0xffffffffu, mine);
      if (mine) sorted[at + __popc(m & ((1u << lane) - 1u))] = p;
      at += __popc(m);
    }
  }
}

inline int row_grid(int rows) { return (rows + kRowsPerCta - 1) / kRowsPerCta; }

// ---- word row + hashed (previous, current) pair row ------------------------------------------------
__global__ void __launch_bounds__(kRowThreads)
embed_pair_rows_kernel(const void* __restrict__ table, int dt, const void* __restrict__ pair, int pdt,
                       const int32_t* __restrict__ ids, const int32_t* __restrict__ prev, long long mul_prev,
                       long long mul_cur, long long buckets, float* __restrict__ out, int rows, int cols) {
  const int row = blockIdx.x * kRowsPerCta + (threadIdx.x >> 5);
  if (row >= rows) return;
  const long long id = ids[row], pv = prev[row];
  long long r = buckets;
  if (pv >= 0) {
    r = (pv * mul_prev + id * mul_cur) % buckets;
    if (r < 0) r += buckets;
  }
  const size_t src = static_cast<size_t>(id) * cols, psrc = static_cast<size_t>(r) * cols;
  float* o = out + static_cast<size_t>(row) * cols;
  for (int c = lane_id(); c < cols; c += 32) o[c] = ld_any(table, dt, src + c) + ld_any(pair, pdt, psrc + c);
}

__global__ void __launch_bounds__(kRowThreads)
add_row_vector_kernel(float* __restrict__ x, const void* __restrict__ vec, int dt, size_t total, int cols) {
  for (size_t i = blockIdx.x * static_cast<size_t>(kRowThreads) + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * kRowThreads)
    x[i] += ld_any(vec, dt, i % cols);
}

// x += mult * (a + sum_j part_j): the sum runs in a fixed order (a first, then the partials by index)
__global__ void __launch_bounds__(kRowThreads)
residual_add_rows_kernel(float* __restrict__ x, const void* __restrict__ a, int a_dt, int64_t lda,
                         const void* __restrict__ part, int p_dt, int64_t ldp, int np, float mult,
                         void* __restrict__ copy, int c_dt, int rows, int cols) {
  const size_t total = static_cast<size_t>(rows) * cols;
  for (size_t i = blockIdx.x * static_cast<size_t>(kRowThreads) + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * kRowThreads) {
    const size_t r = i / cols, c = i % cols;
    float y = a ? ld_any(a, a_dt, r * lda + c) : 0.f;
    if (part)
      for (int j = 0; j < np; ++j) y += ld_any(part, p_dt, (r * np + j) * ldp + c);
    const float v = x[i] + mult * y;
    x[i] = v;
    if (copy) st_any(copy, c_dt, i, v);
  }
}

__global__ void __launch_bounds__(kRowThreads)
gelu_mul_gather_kernel(const void* __restrict__ z, int z_dt, const void* __restrict__ table, int dt, int64_t ldt,
                       const int32_t* __restrict__ ids, int col0, void* __restrict__ out, int o_dt, int rows,
                       int cols) {
  const size_t total = static_cast<size_t>(rows) * cols;
  for (size_t i = blockIdx.x * static_cast<size_t>(kRowThreads) + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * kRowThreads) {
    const size_t r = i / cols, c = i % cols;
    const float v = ld_any(z, z_dt, i);
    const float g = 0.5f * v * (1.0f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
    st_any(out, o_dt, i, g * ld_any(table, dt, static_cast<size_t>(ids[r]) * ldt + col0 + c));
  }
}

// ---- sigmoid router with group-limited choice -------------------------------------------------------
// Logits as in moe_route_kernel (fp32 dot products over the row).  Then one warp per token: scores
// s = sigmoid(z); choice c = s + correction; group score = sum of the two largest c of the group; the
// `keep` best groups stay, the others' c become -inf; `top` rounds of arg-max over c (ties: lower index);
// the weight of a chosen expert is its s.
__device__ __forceinline__ void warp_argmax(float& best, int& bi) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
}

template <int TPR>
__global__ void __launch_bounds__(kRowThreads)
moe_route_sigmoid_kernel(const void* __restrict__ x, int x_dt, int64_t ldx, const float* __restrict__ wr,
                         const float* __restrict__ corr, int32_t* __restrict__ idx, float* __restrict__ weight,
                         int rows, int cols, int experts, int top, int groups, int keep) {
  extern __shared__ float z_s[];  // per token: s [experts] | c [experts] | group score [groups]
  const int wid = threadIdx.x >> 5, lane = lane_id();
  const int row = row_of<TPR>();
  if (row >= rows) return;
  const int per_tok = 2 * experts + groups;
  float* s = TPR == 32 ? z_s + wid * per_tok : z_s;
  float* c = s + experts;
  float* gs = c + experts;
  const size_t xb = static_cast<size_t>(row) * ldx;
  for (int e = (TPR == 32 ? 0 : wid); e < experts; e += (TPR == 32 ? 1 : kRowsPerCta)) {
    const float* we = wr + static_cast<size_t>(e) * cols;
    float a = 0.f;
    for (int k = lane; k < cols; k += 32) a += ld_any(x, x_dt, xb + k) * we[k];
    a = warp_sum(a);
    if (lane == 0) {
      const float sv = sigmoid_f(a);
      s[e] = sv;
      c[e] = sv + (corr ? corr[e] : 0.f);
    }
  }
  if (TPR == 32) __syncwarp();
  else {
    __syncthreads();
    if (wid != 0) return;
  }
  const int gsize = experts / groups;
  if (keep < groups) {
    for (int g = lane; g < groups; g += 32) {
      float a = -INFINITY, b = -INFINITY;   // largest, second largest
      for (int e = g * gsize; e < (g + 1) * gsize; ++e) {
        const float v = c[e];
        if (v > a) { b = a; a = v; }
        else if (v > b) b = v;
      }
      gs[g] = gsize >= 2 ? a + b : a;
    }
    __syncwarp();
    // `keep` rounds of arg-max over the groups; a kept group is marked by +inf
    for (int j = 0; j < keep; ++j) {
      float best = -INFINITY;
      int bi = 0x7fffffff;
      for (int g = lane; g < groups; g += 32) {
        const float v = gs[g];
        if (v != INFINITY && v > best) { best = v; bi = g; }
      }
      warp_argmax(best, bi);
      if (lane == 0 && bi != 0x7fffffff) gs[bi] = INFINITY;
      __syncwarp();
    }
    for (int e = lane; e < experts; e += 32)
      if (gs[e / gsize] != INFINITY) c[e] = -INFINITY;
    __syncwarp();
  }
  for (int j = 0; j < top; ++j) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int e = lane; e < experts; e += 32) {
      const float v = c[e];
      if (v > best) { best = v; bi = e; }
    }
    warp_argmax(best, bi);
    if (bi == 0x7fffffff) bi = 0;   // fewer selectable experts than `top` (refused by the launcher's callers)
    if (lane == 0) {
      idx[static_cast<size_t>(row) * top + j] = bi;
      weight[static_cast<size_t>(row) * top + j] = s[bi];
      c[bi] = -INFINITY;
    }
    __syncwarp();
  }
}

inline int flat_grid(size_t total) {
  const size_t g = (total + kRowThreads - 1) / kRowThreads;
  return static_cast<int>(g < 1 ? 1 : (g > 148 * 16 ? 148 * 16 : g));
}

// ---- scaled embedding + sinusoidal positions ---------------------------------------------------------
// A warp (narrow rows) or a CTA (wide rows) per row; a thread takes column pairs (2i, 2i + 1) = (sin, cos) of ONE
// angle position * inv_freq[i].
// The angle is formed and brought into [-pi, pi] in double, so that far positions keep their phase (an fp32
// product loses it); sine and cosine of the reduced angle are evaluated in fp32.
template <int TPR>
__global__ void __launch_bounds__(kRowThreads)
embed_sincos_rows_kernel(const void* __restrict__ table, int dt, const int32_t* __restrict__ ids,
                         const int32_t* __restrict__ positions, const double* __restrict__ inv_freq, float scale,
                         float* __restrict__ out, void* __restrict__ copy, int c_dt, int rows, int cols) {
  const int row = row_of<TPR>();
  if (row >= rows) return;
  const size_t src = static_cast<size_t>(ids[row]) * cols, dst = static_cast<size_t>(row) * cols;
  const double pos = static_cast<double>(positions[row]);
  for (int i = col0_of<TPR>(); 2 * i < cols; i += TPR) {
    const double ang = pos * inv_freq[i];
    const float red = static_cast<float>(fma(-6.283185307179586476925, rint(ang * 0.15915494309189533577), ang));
    float sn, cs;
    sincosf(red, &sn, &cs);
    const float v0 = fmaf(ld_any(table, dt, src + 2 * i), scale, sn);
    out[dst + 2 * i] = v0;
    if (copy) st_any(copy, c_dt, dst + 2 * i, v0);
    if (2 * i + 1 < cols) {
      const float v1 = fmaf(ld_any(table, dt, src + 2 * i + 1), scale, cs);
      out[dst + 2 * i + 1] = v1;
      if (copy) st_any(copy, c_dt, dst + 2 * i + 1, v1);
    }
  }
}

// ---- post-normed residual update of one or two scaled branches ---------------------------------------
// x += rms(sa * a + sb * b) * w  (the norm sits on the sublayer's OUTPUT); optionally the updated row is
// also written in the dtype of the next projection's operand.
template <int TPR>
__global__ void __launch_bounds__(kRowThreads)
branch_norm_residual_kernel(float* __restrict__ x, const void* __restrict__ a, int a_dt, int64_t lda, float sa,
                            const void* __restrict__ b, int b_dt, int64_t ldb, float sb,
                            const void* __restrict__ w, int w_dt, float eps, void* __restrict__ copy, int c_dt,
                            int rows, int cols) {
  __shared__ float red[kRowsPerCta];
  const int row = row_of<TPR>();
  if (row >= rows) return;
  const size_t ab = static_cast<size_t>(row) * lda, bb = static_cast<size_t>(row) * ldb;
  float ss = 0.f;
  for (int c = col0_of<TPR>(); c < cols; c += TPR) {
    float y = sa * ld_any(a, a_dt, ab + c);
    if (b) y = fmaf(sb, ld_any(b, b_dt, bb + c), y);
    ss = fmaf(y, y, ss);
  }
  ss = row_sum<TPR>(ss, red);
  const float r = 1.0f / sqrtf(ss / static_cast<float>(cols) + eps);
  const size_t xb = static_cast<size_t>(row) * cols;
  for (int c = col0_of<TPR>(); c < cols; c += TPR) {
    float y = sa * ld_any(a, a_dt, ab + c);
    if (b) y = fmaf(sb, ld_any(b, b_dt, bb + c), y);
    const float v = x[xb + c] + y * r * (w ? ld_any(w, w_dt, c) : 1.0f);
    x[xb + c] = v;
    if (copy) st_any(copy, c_dt, xb + c, v);
  }
}

}  // namespace

int embed_rows(const void* table, int dt, const int32_t* ids, float* out, int rows, int cols,
               cudaStream_t stream) {
  if (rows <= 0) return 0;
  VB_CUDA(launch_serial(embed_rows_kernel, dim3(row_grid(rows)), dim3(kRowThreads), 0, stream, table, dt,
                     ids, out, rows, cols));
  return 0;
}

int rmsnorm_rows(const void* x, int x_dt, int64_t ldx, const void* w, int w_dt, float w_off, float eps,
                 void* out, int o_dt, int64_t ldo, const int32_t* out_rows, int rows, int cols,
                 cudaStream_t stream, int groups) {
  if (rows <= 0) return 0;
  VB_CHECK(cols > 0 && groups >= 1 && cols % groups == 0, "rmsnorm_rows: cols=%d groups=%d", cols, groups);
  const int vrows = rows * groups, vcols = cols / groups;
  if (vcols >= kWideCols)
    VB_CUDA(launch_serial(rmsnorm_rows_kernel<256>, dim3(vrows), dim3(kRowThreads), 0, stream, x, x_dt, ldx, w,
                       w_dt, w_off, eps, out, o_dt, ldo, out_rows, vrows, vcols, groups));
  else
    VB_CUDA(launch_serial(rmsnorm_rows_kernel<32>, dim3(row_grid(vrows)), dim3(kRowThreads), 0, stream, x, x_dt,
                       ldx, w, w_dt, w_off, eps, out, o_dt, ldo, out_rows, vrows, vcols, groups));
  return 0;
}

int residual_norm_rows(float* x, const void* a, int a_dt, int64_t lda, const void* part, int p_dt, int64_t ldp, int np,
                       const void* w, int w_dt, float eps, void* out, int o_dt, int rows, int cols, cudaStream_t stream) {
  if (rows <= 0) return 0;
  VB_CHECK(cols > 0 && out != nullptr && (part == nullptr || np >= 1), "residual_norm_rows: cols=%d n_partials=%d", cols, np);
  if (cols >= kWideCols)
    VB_CUDA(launch_serial(residual_norm_rows_kernel<256>, dim3(rows), dim3(kRowThreads), 0, stream, x, a, a_dt, lda,
                          part, p_dt, ldp, np, w, w_dt, eps, out, o_dt, rows, cols));
  else
    VB_CUDA(launch_serial(residual_norm_rows_kernel<32>, dim3(row_grid(rows)), dim3(kRowThreads), 0, stream, x, a,
                          a_dt, lda, part, p_dt, ldp, np, w, w_dt, eps, out, o_dt, rows, cols));
  return 0;
}

int gated_norm_residual(float* x, const void* part, int p_dt, int64_t ldp, int np, const void* gate,
                        int g_dt, int64_t ldg, const void* gb, int b_dt, const void* w, int w_dt,
                        float w_off, float eps, int rows, int cols, cudaStream_t stream, float mult) {
  if (rows <= 0) return 0;
  VB_CHECK(np >= 1 && cols > 0, "gated_norm_residual: n_partials=%d cols=%d", np, cols);
  if (cols >= kWideCols)
    VB_CUDA(launch_serial(gated_norm_residual_kernel<256>, dim3(rows), dim3(kRowThreads), 0, stream, x, part,
                       p_dt, ldp, np, gate, g_dt, ldg, gb, b_dt, w, w_dt, w_off, eps, mult, rows, cols));
  else
    VB_CUDA(launch_serial(gated_norm_residual_kernel<32>, dim3(row_grid(rows)), dim3(kRowThreads), 0, stream, x,
                       part, p_dt, ldp, np, gate, g_dt, ldg, gb, b_dt, w, w_dt, w_off, eps, mult, rows, cols));
  return 0;
}

int moe_route(const void* x, int x_dt, int64_t ldx, const float* wr, const float* bias, int32_t* idx,
              float* weight, int rows, int cols, int experts, int top, cudaStream_t stream) {
  if (rows <= 0) return 0;
  VB_CHECK(experts >= 1 && top >= 1 && top <= experts && experts <= 1024,
           "moe_route: experts=%d top=%d", experts, top);
  if (rows <= 1024)   // few tokens: a CTA per token, its warps split the experts
    VB_CUDA(launch_serial(moe_route_kernel<256>, dim3(rows), dim3(kRowThreads), sizeof(float) * experts, stream,
                       x, x_dt, ldx, wr, bias, idx, weight, rows, cols, experts, top));
  else
    VB_CUDA(launch_serial(moe_route_kernel<32>, dim3(row_grid(rows)), dim3(kRowThreads),
                       sizeof(float) * kRowsPerCta * experts, stream, x, x_dt, ldx, wr, bias, idx, weight, rows,
                       cols, experts, top));
  return 0;
}


int embed_pair_rows(const void* table, int dt, const void* pair, int pdt, const int32_t* ids,
                    const int32_t* prev, long long mul_prev, long long mul_cur, long long buckets, float* out,
                    int rows, int cols, cudaStream_t stream) {
  if (rows <= 0) return 0;
  VB_CHECK(buckets >= 1 && cols > 0, "embed_pair_rows: buckets=%lld cols=%d", buckets, cols);
  VB_CUDA(launch_serial(embed_pair_rows_kernel, dim3(row_grid(rows)), dim3(kRowThreads), 0, stream, table, dt,
                        pair, pdt, ids, prev, mul_prev, mul_cur, buckets, out, rows, cols));
  return 0;
}

int add_row_vector(float* x, const void* vec, int dt, int rows, int cols, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return 0;
  const size_t total = static_cast<size_t>(rows) * cols;
  VB_CUDA(launch_serial(add_row_vector_kernel, dim3(flat_grid(total)), dim3(kRowThreads), 0, stream, x, vec, dt,
                        total, cols));
  return 0;
}

int residual_add_rows(float* x, const void* a, int a_dt, int64_t lda, const void* part, int p_dt, int64_t ldp,
                      int np, float mult, void* copy, int c_dt, int rows, int cols, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return 0;
  VB_CHECK(part == nullptr || np >= 1, "residual_add_rows: n_partials=%d", np);
  VB_CUDA(launch_serial(residual_add_rows_kernel, dim3(flat_grid(static_cast<size_t>(rows) * cols)),
                        dim3(kRowThreads), 0, stream, x, a, a_dt, lda, part, p_dt, ldp, np, mult, copy, c_dt, rows, cols));
  return 0;
}

int gelu_mul_gather(const void* z, int z_dt, const void* table, int dt, int64_t ldt, const int32_t* ids, int col0,
                    void* out, int o_dt, int rows, int cols, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return 0;
  VB_CUDA(launch_serial(gelu_mul_gather_kernel, dim3(flat_grid(static_cast<size_t>(rows) * cols)),
                        dim3(kRowThreads), 0, stream, z, z_dt, table, dt, ldt, ids, col0, out, o_dt, rows, cols));
  return 0;
}

int moe_route_sigmoid(const void* x, int x_dt, int64_t ldx, const float* wr, const float* corr, int32_t* idx,
                      float* weight, int rows, int cols, int experts, int top, int groups, int keep,
                      cudaStream_t stream) {
  if (rows <= 0) return 0;
  VB_CHECK(experts >= 1 && experts <= 1024 && groups >= 1 && experts % groups == 0 && keep >= 1 && keep <= groups &&
               top >= 1 && top <= keep * (experts / groups),
           "moe_route_sigmoid: experts=%d top=%d groups=%d keep=%d", experts, top, groups, keep);
  const size_t per_tok = sizeof(float) * (2 * experts + groups);
  if (rows <= 1024 || per_tok * kRowsPerCta > 48 * 1024)   // few tokens, or too many experts for a warp's share
    VB_CUDA(launch_serial(moe_route_sigmoid_kernel<256>, dim3(rows), dim3(kRowThreads), per_tok, stream, x, x_dt,
                          ldx, wr, corr, idx, weight, rows, cols, experts, top, groups, keep));
  else
    VB_CUDA(launch_serial(moe_route_sigmoid_kernel<32>, dim3(row_grid(rows)), dim3(kRowThreads),
                          per_tok * kRowsPerCta, stream, x, x_dt, ldx, wr, corr, idx, weight, rows, cols, experts,
                          top, groups, keep));
  return 0;
}

int moe_group(const int32_t* idx, int32_t* seg, int32_t* sorted, int pairs, int experts,
              cudaStream_t stream) {
  VB_CHECK(experts >= 1 && experts <= 8192 && pairs >= 0, "moe_group: experts=%d pairs=%d", experts, pairs);
  VB_CUDA(launch_serial(moe_group_kernel, dim3(1), dim3(1024), sizeof(int) * (experts + 1), stream, idx, seg,
                     sorted, pairs, experts));
  return 0;
}

int embed_sincos_rows(const void* table, int dt, const int32_t* ids, const int32_t* positions, const double* inv_freq,
                      float scale, float* out, void* copy, int c_dt, int rows, int cols, cudaStream_t stream) {
  if (rows <= 0) return 0;
  VB_CHECK(cols >= 1 && inv_freq != nullptr && positions != nullptr, "embed_sincos_rows: cols=%d", cols);
  if (cols >= kWideCols)
    VB_CUDA(launch_serial(embed_sincos_rows_kernel<256>, dim3(rows), dim3(kRowThreads), 0, stream, table, dt, ids,
                          positions, inv_freq, scale, out, copy, c_dt, rows, cols));
  else
    VB_CUDA(launch_serial(embed_sincos_rows_kernel<32>, dim3(row_grid(rows)), dim3(kRowThreads), 0, stream, table, dt,
                          ids, positions, inv_freq, scale, out, copy, c_dt, rows, cols));
  return 0;
}

int branch_norm_residual(float* x, const void* a, int a_dt, int64_t lda, float sa, const void* b, int b_dt,
                         int64_t ldb, float sb, const void* w, int w_dt, float eps, void* copy, int c_dt, int rows,
                         int cols, cudaStream_t stream) {
  if (rows <= 0) return 0;
  VB_CHECK(cols > 0 && a != nullptr, "branch_norm_residual: cols=%d", cols);
  if (cols >= kWideCols)
    VB_CUDA(launch_serial(branch_norm_residual_kernel<256>, dim3(rows), dim3(kRowThreads), 0, stream, x, a, a_dt, lda,
                          sa, b, b_dt, ldb, sb, w, w_dt, eps, copy, c_dt, rows, cols));
  else
    VB_CUDA(launch_serial(branch_norm_residual_kernel<32>, dim3(row_grid(rows)), dim3(kRowThreads), 0, stream, x, a,
                          a_dt, lda, sa, b, b_dt, ldb, sb, w, w_dt, eps, copy, c_dt, rows, cols));
  return 0;
}

}  // namespace vb
