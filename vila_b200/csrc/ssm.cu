// State-space mixers on ragged batches.  Every sequence of a step brings a portion of any length (a
// prompt piece or one decoded token); what it needs from the past lives in its state slot of a
// caller-owned fp32 pool and is advanced by the rows the step brings.  A sequence at position 0 never
// reads its slot (a reused slot's stale contents are not seen).
//
//   causal_conv_rows    out[t, c] = act(bias[c] + sum_j w[c, j] in[t - (taps - 1) + j, c]); a thread owns a
//                       channel and walks kConvRows consecutive rows with the last taps inputs in
//                       registers (taps + rows - 1 loads for `rows` outputs); rows before the portion come
//                       from the state [slots, taps - 1, cols], rows before position 0 are zero
//   causal_conv_state   the last taps - 1 inputs of every sequence, after the convolution
//   ssd_scan            S_t = a_t S_{t-1} + dt_t B_t x_t^T,  y_t = S_t^T C_t + D x_t  with one decay
//                       a_t = exp(-exp(A_log) dt_t) per head.  Grid (sequence, head, 32 columns of P);
//                       thread (column c = tid / 8, r = tid % 8) keeps the state entries n = r * KPT .. of
//                       its column in registers (state layout [.., P, N]: a thread's entries are
//                       contiguous, 8 lanes cover a column's N), the sum over n ends with three shuffles.
//                       16 tokens at a time are staged in shared memory with softplus / exp evaluated once,
//                       the next 16 are fetched into registers meanwhile, outputs leave through shared memory
//   selective_scan      S_t[c, n] = exp(dt_t,c A[c, n]) S_{t-1}[c, n] + dt_t,c x_t,c B_t,n,  y = S C + D x; grid
//                       (sequence, 32 channels); thread (channel, r) as above, A[c, n] in registers
// softplus, exponentials, decays, step sizes, states and sums are fp32 whatever the tensors' dtype; time
// runs in order, so a row's result does not depend on how the sequence was cut into steps.
#include <algorithm>
#include "../../include/vila_b200.h"
#include "common.cuh"
#include "kernels.h"
#include "dtype_any.cuh"

namespace vb {
namespace {

constexpr int kThreads = 256;
constexpr int kMaxTaps = 16;
constexpr int kConvRows = 8;
constexpr int kChunk = 16;      // tokens staged per stage of a scan
constexpr int kLanes = 8;       // threads that share a state column / channel
constexpr int kCols = kThreads / kLanes;

__device__ __forceinline__ float softplus_f(float z) { return z > 20.0f ? z : log1pf(expf(z)); }

// ---- causal depthwise convolution ------------------------------------------------------------------------
template <int TAPS>   // 0: run-time tap count (<= kMaxTaps)
__global__ void __launch_bounds__(kThreads) causal_conv_rows_kernel(const vila_causal_conv_params p) {
  constexpr int WN = TAPS ? TAPS : kMaxTaps;
  const int taps = TAPS ? TAPS : p.taps, back = taps - 1;
  const int c = blockIdx.y * kThreads + threadIdx.x;
  if (c >= p.cols) return;
  float w[WN], win[WN];   // win[j]: input `back - j` positions before the current row (win[back] = current)
#pragma unroll
  for (int j = 0; j < WN; ++j) {
    w[j] = j < taps ? ld_any(p.w, p.w_dtype, static_cast<size_t>(c) * taps + j) : 0.f;
    win[j] = 0.f;
  }
  const float bias = p.bias ? ld_any(p.bias, p.w_dtype, c) : 0.f;
  const int t0 = blockIdx.x * kConvRows, t1 = min(p.rows, t0 + kConvRows);
  for (int t = t0; t < t1; ++t) {
    const int* sq = p.seqs + 4 * p.row_seq[t];
    const int row0 = sq[0], pos = sq[2] + (t - row0);
    const float cur = ld_any(p.in, p.in_dtype, static_cast<size_t>(t) * p.ld_in + c);
    if (t == t0 || t == row0) {
      // (re)fill the window: earlier rows of the portion, the sequence's state, or zero before position 0
      const float* st = p.state + static_cast<size_t>(sq[3]) * back * p.cols;
#pragma unroll
      for (int j = 0; j < WN; ++j) {
        if (j >= back) continue;
        const int d = back - j;
        float v = 0.f;
        if (pos - d >= 0) {
          if (t - d >= row0) v = ld_any(p.in, p.in_dtype, static_cast<size_t>(t - d) * p.ld_in + c);
          else v = st[static_cast<size_t>(back - (row0 - (t - d))) * p.cols + c];
        }
        win[j] = v;
      }
    } else {
#pragma unroll
      for (int j = 0; j + 1 < WN; ++j)
        if (j + 1 < taps) win[j] = win[j + 1];
    }
    float acc = bias;
#pragma unroll
    for (int j = 0; j < WN; ++j) {
      if (j == back) win[j] = cur;
      if (j < taps) acc = fmaf(w[j], win[j], acc);
    }
    if (p.act == VILA_CONV_SILU) acc = silu_exact_f(acc);
    st_any(p.out, p.out_dtype, static_cast<size_t>(t) * p.ld_out + c, acc);
  }
}

// New state row j holds position end - back + j (end = first position after the portion): a row of the
// portion, an older state row (at an index above the one being written: j runs upwards, one thread per
// channel, nothing is overwritten before it is read), or zero before position 0.
__global__ void __launch_bounds__(kThreads) causal_conv_state_kernel(const vila_causal_conv_params p) {
  const int* sq = p.seqs + 4 * blockIdx.x;
  const int row0 = sq[0], n = sq[1], pos0 = sq[2], slot = sq[3];
  const int back = p.taps - 1;
  float* st = p.state + static_cast<size_t>(slot) * back * p.cols;
  for (int c = blockIdx.y * kThreads + threadIdx.x; c < p.cols; c += gridDim.y * kThreads) {
    for (int j = 0; j < back; ++j) {
      const int q = pos0 + n - back + j;
      float v = 0.f;
      if (q >= pos0) v = ld_any(p.in, p.in_dtype, static_cast<size_t>(row0 + (q - pos0)) * p.ld_in + c);
      else if (q >= 0) v = st[static_cast<size_t>(j + n) * p.cols + c];
      st[static_cast<size_t>(j) * p.cols + c] = v;
    }
  }
}

// ---- scalar-decay recurrence (state-space duality form) ----------------------------------------------
// Both scans keep global memory out of the time loop: the inputs of 16 tokens are fetched into registers
// while the previous 16 are being processed, go to shared memory with softplus / exp / silu evaluated once,
// and the outputs of the 16 tokens leave through shared memory after the loop.
template <int KPT>   // state entries per thread: N <= 8 * KPT, KPT a multiple of 4
__global__ void __launch_bounds__(kThreads) ssd_scan_kernel(const vila_ssd_scan_params p) {
  extern __shared__ __align__(16) float sm[];
  constexpr int NP = kLanes * KPT;               // state entries the 8 owners cover
  constexpr int NS = kLanes * (KPT + 4);         // padded floats per token for B or C: 4 per owner, so that the
                                                 // owners' float4 reads fall into different banks
  constexpr int BCN = kChunk * NP / kThreads;    // B (or C) entries a thread brings in per stage
  constexpr int XN = kChunk * kCols / kThreads;  // x (or z) entries a thread brings in per stage
  float* B_s = sm;                               // [kChunk][NS]
  float* C_s = B_s + kChunk * NS;                // [kChunk][NS]
  float* x_s = C_s + kChunk * NS;                // [kChunk][kCols]
  float* z_s = x_s + kChunk * kCols;             // [kChunk][kCols] silu(z), or 1
  float* y_s = z_s + kChunk * kCols;             // [kChunk][kCols]
  float* dt_s = y_s + kChunk * kCols;            // [kChunk]
  float* a_s = dt_s + kChunk;                    // [kChunk]
  const int tid = threadIdx.x, r = tid & (kLanes - 1), c = tid >> 3;
  const int* sq = p.seqs + 4 * blockIdx.x;
  const int row0 = sq[0], n = sq[1], pos0 = sq[2], slot = sq[3];
  const int h = blockIdx.y, P = p.P, N = p.N, g = h / (p.H / p.G);
  const int col0 = blockIdx.z * kCols, col = col0 + c;
  const bool col_ok = col < P;
  const int n0 = r * KPT;                        // first state index of this thread
  float* st = p.state + ((static_cast<size_t>(slot) * p.H + h) * P + (col_ok ? col : 0)) * N;
  float S[KPT];
#pragma unroll
  for (int k = 0; k < KPT; ++k) S[k] = (pos0 > 0 && col_ok && n0 + k < N) ? st[n0 + k] : 0.f;
  const float neg_a = -expf(p.A_log[h]), bias = p.dt_bias[h], Dh = p.D[h];
  const size_t xoff = static_cast<size_t>(h) * P, boff = static_cast<size_t>(p.H) * P + static_cast<size_t>(g) * N;
  const size_t coff = boff + static_cast<size_t>(p.G) * N;
  uint32_t rb[BCN], rc[BCN], rx[XN], rz[XN], rdt = 0u;   // raw bits: converted when they go to shared memory
  const int dt_in = p.in_dtype;
  auto fetch = [&](int t0) {
    const int nt = min(kChunk, n - t0);
#pragma unroll
    for (int k = 0; k < BCN; ++k) {
      const int idx = tid + k * kThreads, t = idx / NP, i = idx - t * NP;
      const bool ok = t < nt && i < N;
      const size_t base = static_cast<size_t>(row0 + t0 + t) * p.ld_xbc;
      rb[k] = ok ? ld_raw(p.xbc, dt_in, base + boff + i) : 0u;
      rc[k] = ok ? ld_raw(p.xbc, dt_in, base + coff + i) : 0u;
    }
#pragma unroll
    for (int k = 0; k < XN; ++k) {
      const int idx = tid + k * kThreads, t = idx / kCols, gc = col0 + (idx - t * kCols);
      const bool ok = t < nt && gc < P;
      const size_t row = static_cast<size_t>(row0 + t0 + t);
      rx[k] = ok ? ld_raw(p.xbc, dt_in, row * p.ld_xbc + xoff + gc) : 0u;
      rz[k] = (ok && p.z) ? ld_raw(p.z, dt_in, row * p.ld_z + xoff + gc) : 0u;
    }
    if (tid < kChunk) rdt = tid < nt ? ld_raw(p.dt, dt_in, static_cast<size_t>(row0 + t0 + tid) * p.ld_dt + h) : 0u;
  };
  fetch(0);
  for (int t0 = 0; t0 < n; t0 += kChunk) {
    const int nt = min(kChunk, n - t0);
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BCN; ++k) {
      const int idx = tid + k * kThreads, t = idx / NP, i = idx - t * NP;
      const int at = t * NS + i + (i / KPT) * 4;
      B_s[at] = raw_to_float(rb[k], dt_in);
      C_s[at] = raw_to_float(rc[k], dt_in);
    }
#pragma unroll
    for (int k = 0; k < XN; ++k) {
      const int idx = tid + k * kThreads;
      x_s[idx] = raw_to_float(rx[k], dt_in);
      z_s[idx] = p.z ? silu_exact_f(raw_to_float(rz[k], dt_in)) : 1.0f;
    }
    if (tid < kChunk) {
      const float dt = softplus_f(raw_to_float(rdt, dt_in) + bias);
      dt_s[tid] = dt;
      a_s[tid] = expf(neg_a * dt);
    }
    __syncthreads();
    if (t0 + kChunk < n) fetch(t0 + kChunk);     // in flight while this stage is processed
    for (int t = 0; t < nt; ++t) {
      const float x = x_s[t * kCols + c], dt = dt_s[t], a = a_s[t];
      const float xdt = dt * x;
      const float4* Bt = reinterpret_cast<const float4*>(B_s + t * NS + r * (KPT + 4));
      const float4* Ct = reinterpret_cast<const float4*>(C_s + t * NS + r * (KPT + 4));
      float y0 = 0.f, y1 = 0.f;
#pragma unroll
      for (int k4 = 0; k4 < KPT / 4; ++k4) {
        const float4 b = Bt[k4], cv = Ct[k4];
        S[4 * k4 + 0] = fmaf(a, S[4 * k4 + 0], b.x * xdt);
        S[4 * k4 + 1] = fmaf(a, S[4 * k4 + 1], b.y * xdt);
        S[4 * k4 + 2] = fmaf(a, S[4 * k4 + 2], b.z * xdt);
        S[4 * k4 + 3] = fmaf(a, S[4 * k4 + 3], b.w * xdt);
        y0 = fmaf(S[4 * k4 + 0], cv.x, y0);
        y1 = fmaf(S[4 * k4 + 1], cv.y, y1);
        y0 = fmaf(S[4 * k4 + 2], cv.z, y0);
        y1 = fmaf(S[4 * k4 + 3], cv.w, y1);
      }
      float y = y0 + y1;
      y += __shfl_xor_sync(0xffffffffu, y, 1);
      y += __shfl_xor_sync(0xffffffffu, y, 2);
      y += __shfl_xor_sync(0xffffffffu, y, 4);
      if (r == 0) y_s[t * kCols + c] = fmaf(Dh, x, y) * z_s[t * kCols + c];
    }
    __syncthreads();
    for (int idx = tid; idx < nt * kCols; idx += kThreads) {
      const int t = idx / kCols, gc = col0 + (idx - t * kCols);
      if (gc < P) st_any(p.out, p.out_dtype, static_cast<size_t>(row0 + t0 + t) * p.ld_out + xoff + gc, y_s[idx]);
    }
  }
  if (col_ok) {
#pragma unroll
    for (int k = 0; k < KPT; ++k)
      if (n0 + k < N) st[n0 + k] = S[k];
  }
}

// ---- per-channel selective recurrence ------------------------------------------------------------------
template <int KPT>   // state entries per thread: N <= 8 * KPT
__global__ void __launch_bounds__(kThreads) selective_scan_kernel(const vila_selective_scan_params p) {
  extern __shared__ __align__(16) float sm[];
  constexpr int NP = kLanes * KPT;
  constexpr int KP = KPT >= 4 ? KPT + 4 : KPT;   // padded entries per owner
  constexpr int NS = kLanes * KP;
  constexpr int BCN = (kChunk * NP + kThreads - 1) / kThreads;
  constexpr int XN = kChunk * kCols / kThreads;
  float* B_s = sm;                               // [kChunk][NS]
  float* C_s = B_s + kChunk * NS;                // [kChunk][NS]
  float* x_s = C_s + kChunk * NS;                // [kChunk][kCols]
  float* dt_s = x_s + kChunk * kCols;            // [kChunk][kCols]
  float* z_s = dt_s + kChunk * kCols;            // [kChunk][kCols] silu(z), or 1
  float* y_s = z_s + kChunk * kCols;             // [kChunk][kCols]
  const int tid = threadIdx.x, r = tid & (kLanes - 1), c = tid >> 3;
  const int* sq = p.seqs + 4 * blockIdx.x;
  const int row0 = sq[0], n = sq[1], pos0 = sq[2], slot = sq[3];
  const int N = p.N, ch0 = blockIdx.y * kCols, ch = ch0 + c;
  const bool ch_ok = ch < p.C;
  const int n0 = r * KPT;
  float* st = p.state + (static_cast<size_t>(slot) * p.C + (ch_ok ? ch : 0)) * N;
  float S[KPT], A[KPT];
#pragma unroll
  for (int k = 0; k < KPT; ++k) {
    const bool ok = ch_ok && n0 + k < N;
    S[k] = (pos0 > 0 && ok) ? st[n0 + k] : 0.f;
    A[k] = ok ? -expf(p.A_log[static_cast<size_t>(ch) * N + n0 + k]) : 0.f;
  }
  const float Dc = ch_ok ? p.D[ch] : 0.f;
  uint32_t rb[BCN], rc[BCN], rx[XN], rd[XN], rz[XN];     // raw bits: converted when they go to shared memory
  const int dt_in = p.in_dtype;
  float dbias[XN];                                       // a thread stages the same channels in every stage
#pragma unroll
  for (int k = 0; k < XN; ++k) {
    const int gc = ch0 + (tid + k * kThreads) % kCols;
    dbias[k] = gc < p.C ? p.dt_bias[gc] : 0.f;
  }
  auto fetch = [&](int t0) {
    const int nt = min(kChunk, n - t0);
#pragma unroll
    for (int k = 0; k < BCN; ++k) {
      const int idx = tid + k * kThreads, t = idx / NP, i = idx - t * NP;
      const bool ok = t < nt && i < N;              // t < nt <= kChunk also bounds idx
      const size_t base = static_cast<size_t>(row0 + t0 + t) * p.ld_bc;
      rb[k] = ok ? ld_raw(p.bc, dt_in, base + i) : 0u;
      rc[k] = ok ? ld_raw(p.bc, dt_in, base + N + i) : 0u;
    }
#pragma unroll
    for (int k = 0; k < XN; ++k) {
      const int idx = tid + k * kThreads, t = idx / kCols, gc = ch0 + (idx - t * kCols);
      const bool ok = t < nt && gc < p.C;
      const size_t row = static_cast<size_t>(row0 + t0 + t);
      rx[k] = ok ? ld_raw(p.x, dt_in, row * p.ld_x + gc) : 0u;
      rd[k] = ok ? ld_raw(p.dt, dt_in, row * p.ld_dt + gc) : 0u;
      rz[k] = (ok && p.z) ? ld_raw(p.z, dt_in, row * p.ld_z + gc) : 0u;
    }
  };
  fetch(0);
  for (int t0 = 0; t0 < n; t0 += kChunk) {
    const int nt = min(kChunk, n - t0);
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BCN; ++k) {
      const int idx = tid + k * kThreads, t = idx / NP, i = idx - t * NP;
      if (idx < kChunk * NP) {
        const int at = t * NS + (i / KPT) * KP + (i % KPT);
        B_s[at] = raw_to_float(rb[k], dt_in);
        C_s[at] = raw_to_float(rc[k], dt_in);
      }
    }
#pragma unroll
    for (int k = 0; k < XN; ++k) {
      const int idx = tid + k * kThreads;
      x_s[idx] = raw_to_float(rx[k], dt_in);
      dt_s[idx] = softplus_f(raw_to_float(rd[k], dt_in) + dbias[k]);
      z_s[idx] = p.z ? silu_exact_f(raw_to_float(rz[k], dt_in)) : 1.0f;
    }
    __syncthreads();
    if (t0 + kChunk < n) fetch(t0 + kChunk);     // in flight while this stage is processed
    for (int t = 0; t < nt; ++t) {
      const float x = x_s[t * kCols + c], dt = dt_s[t * kCols + c];
      const float xdt = dt * x;
      const float* Bt = B_s + t * NS + r * KP;
      const float* Ct = C_s + t * NS + r * KP;
      float y0 = 0.f, y1 = 0.f;
#pragma unroll
      for (int k = 0; k < KPT; ++k) {
        S[k] = fmaf(expf(dt * A[k]), S[k], Bt[k] * xdt);
        if (k & 1) y1 = fmaf(S[k], Ct[k], y1);
        else y0 = fmaf(S[k], Ct[k], y0);
      }
      float y = y0 + y1;
      y += __shfl_xor_sync(0xffffffffu, y, 1);
      y += __shfl_xor_sync(0xffffffffu, y, 2);
      y += __shfl_xor_sync(0xffffffffu, y, 4);
      if (r == 0) y_s[t * kCols + c] = fmaf(Dc, x, y) * z_s[t * kCols + c];
    }
    __syncthreads();
    for (int idx = tid; idx < nt * kCols; idx += kThreads) {
      const int t = idx / kCols, gc = ch0 + (idx - t * kCols);
      if (gc < p.C) st_any(p.out, p.out_dtype, static_cast<size_t>(row0 + t0 + t) * p.ld_out + gc, y_s[idx]);
    }
  }
  if (ch_ok) {
#pragma unroll
    for (int k = 0; k < KPT; ++k)
      if (n0 + k < N) st[n0 + k] = S[k];
  }
}

}  // namespace

int causal_conv_rows(const vila_causal_conv_params& p, cudaStream_t stream) {
  if (p.rows <= 0 || p.cols <= 0) return 0;
  VB_CHECK(p.taps >= 1 && p.taps <= kMaxTaps && (p.taps == 1 || p.state != nullptr), "causal_conv_rows: taps=%d",
           p.taps);
  const dim3 grid((p.rows + kConvRows - 1) / kConvRows, (p.cols + kThreads - 1) / kThreads);
  VB_CHECK(grid.y <= 65535, "causal_conv_rows: cols=%d", p.cols);
#define VB_CONV(T) VB_CUDA(launch_serial(causal_conv_rows_kernel<T>, grid, dim3(kThreads), 0, stream, p))
  switch (p.taps) {
    case 2: VB_CONV(2); break;
    case 3: VB_CONV(3); break;
    case 4: VB_CONV(4); break;
    default: VB_CONV(0); break;
  }
#undef VB_CONV
  return 0;
}

int causal_conv_state(const vila_causal_conv_params& p, cudaStream_t stream) {
  if (p.nseq <= 0 || p.cols <= 0 || p.taps <= 1) return 0;
  VB_CHECK(p.taps <= kMaxTaps && p.state != nullptr, "causal_conv_state: taps=%d", p.taps);
  const dim3 grid(p.nseq, std::min(64, (p.cols + kThreads - 1) / kThreads));
  VB_CUDA(launch_serial(causal_conv_state_kernel, grid, dim3(kThreads), 0, stream, p));
  return 0;
}

int ssd_scan(const vila_ssd_scan_params& p, cudaStream_t stream) {
  if (p.nseq <= 0) return 0;
  VB_CHECK(p.H >= 1 && p.G >= 1 && p.H % p.G == 0 && p.P >= 1 && p.N >= 1 && p.N <= 256,
           "ssd_scan: H=%d G=%d P=%d N=%d (<= 256)", p.H, p.G, p.P, p.N);
  const dim3 grid(p.nseq, p.H, (p.P + kCols - 1) / kCols);
  VB_CHECK(grid.y <= 65535 && grid.z <= 65535, "ssd_scan: grid too large");
#define VB_SSD(KPT)                                                                                         \
  VB_CUDA(launch_serial(ssd_scan_kernel<KPT>, grid, dim3(kThreads),                                         \
                        sizeof(float) * (2 * kChunk * kLanes * (KPT + 4) + 3 * kChunk * kCols + 2 * kChunk), stream, p))
  if (p.N <= 32) VB_SSD(4);
  else if (p.N <= 64) VB_SSD(8);
  else if (p.N <= 128) VB_SSD(16);
  else VB_SSD(32);
#undef VB_SSD
  return 0;
}

int selective_scan(const vila_selective_scan_params& p, cudaStream_t stream) {
  if (p.nseq <= 0) return 0;
  VB_CHECK(p.C >= 1 && p.N >= 1 && p.N <= 256, "selective_scan: C=%d N=%d (<= 256)", p.C, p.N);
  const dim3 grid(p.nseq, (p.C + kCols - 1) / kCols);
  VB_CHECK(grid.y <= 65535, "selective_scan: C=%d", p.C);
#define VB_SEL(KPT)                                                                                          \
  VB_CUDA(launch_serial(selective_scan_kernel<KPT>, grid, dim3(kThreads),                                    \
                        sizeof(float) * (2 * kChunk * kLanes * (KPT >= 4 ? KPT + 4 : KPT) + 4 * kChunk * kCols), \
                        stream, p))
  if (p.N <= 8) VB_SEL(1);
  else if (p.N <= 16) VB_SEL(2);
  else if (p.N <= 32) VB_SEL(4);
  else if (p.N <= 64) VB_SEL(8);
  else if (p.N <= 128) VB_SEL(16);
  else VB_SEL(32);
#undef VB_SEL
  return 0;
}

}  // namespace vb
